#!/usr/bin/env python
"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|rmsnorm|rope] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: for the default workload (C2) one
`flash_attention_decode` call over a ragged batch of 16 sequences (32 q / 8 kv heads, head size 128, lengths
uniform in [1024, 2048], cache padded to 2048, bf16).  The metric is the reference's own
(benchmark_kernel.py:48-49): bytes of K and V that belong to valid tokens, 2*2*Hkv*D*sum(len), per second,
in decimal GB/s.

Printed JSON line (rank 0):
  value          GB/s over all GPUs with inputs resident in HBM; K steps timed as one region with CUDA events
                 on the launching stream, barrier + synchronize on both sides, max over ranks
  e2e            the same metric through the extension module with HOST inputs: every step copies q, k, v
                 (and seq_lens) from pinned host memory, runs the kernel and reads the output back
  roofline       achieved algorithmic GB/s of the flash-decode kernel against the measured HBM copy bandwidth
  cpu_baseline   the reference's PyTorch attention path (scaled_dot_product_attention, bf16, on the CPU tensors)
                 timed on this box's host cores over a bounded number of passes
  clocks         SM clock and throttle reasons sampled through NVML while the GPU was busy

L2 hygiene: every step reads a different one of 8 KV caches (1.07 GB in total, L2 is 126 MB), so a cache is
cold again when its turn comes.  With --impl reference the CPU baseline alone is run and reported.
Multi-GPU (launched by torch.distributed.run, one rank per GPU): C2 is weak-scaled, every rank owns a batch
of 16 sequences and no data crosses GPUs; C3 (--workload c3) shards the KV sequence across ranks and merges
the per-rank (o, lse) pairs after one all-gather.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
from __graft_entry__ import load_package  # noqa: E402

N_ROTATE = 8
FALLBACK_PEAK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one flash_decode_small_kernel launch on the C2 workload (seed 42),
# from the ncu capture summarised in profiles/flash_decode_c2_full.md: 102.10 MB read + 4.05 MB written.
C2_TRAFFIC_BYTES = 106_150_000
C3_TRAFFIC_BYTES = 540_310_000  # flash_decode_small_kernel, profiles/flash_decode_c3_full.md: 536.91 MB read + 3.40 MB written


def hbm_peak():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_GBS, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML every ~5 ms in a thread."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
        0x10: "sync_boost",
    }

    def __init__(self, index: int):
        self.samples = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._marks = {}
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and all(v.strip().isdigit() for v in vis.split(",")) else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report that, never fail the bench
            self.nv = None
            self.err = repr(e)

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, rs))
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def mark(self, name):
        self._marks[name] = time.perf_counter()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.nv:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + self.err}
        t0, t1 = self._marks.get("t0"), self._marks.get("t1")
        timed = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1]
        window = "timed region"
        if len(timed) < 3:  # region shorter than the sampling period: use every sample taken under load
            w0 = self._marks.get("w0", 0)
            timed = [s for s in self.samples if s[0] >= w0]
            window = "warm-up + timed region"
        if not timed:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "no samples"}
        mhz = sorted(s[1] for s in timed)
        bits = 0
        for s in timed:
            bits |= s[2]
        reasons = [n for b, n in self.REASONS.items() if bits & b]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(timed), "window": window}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def make_decode_workload(name: str, rank: int, world: int, seq_len: int = 131072):
    """Returns (case on CPU, description).  Values are seeded N(0,1) in bf16 (synthetic data)."""
    from oracle import inputs

    if name == "c2":
        case = inputs.config2(seed=42 + rank)
        desc = "C2 batched decode attention: B=16/GPU, Hq=32, Hkv=8, D=128, len~U[1024,2048], cache padded to 2048, bf16"
    elif name == "c1":
        case = inputs.config1(seed=42 + rank)
        desc = "C1 single decode step: B=1, Hq=32, Hkv=8, D=64, S=256, bf16"
    elif name == "c3":
        case = inputs.config3(seed=42, S=seq_len)
        desc = f"C3 long-context decode: B=1, Hq=32, Hkv=8, D=128, S={seq_len}, bf16, KV sequence sharded over the GPUs"
    else:
        raise ValueError(name)
    return case, desc


def kv_bytes(case) -> int:
    """2 (K,V) * 2 bytes * Hkv * D * sum(len): benchmark_kernel.py:48."""
    B, Hkv, S, D = case.k.shape
    tokens = int(case.seq_lens.clamp(0, S).sum()) if case.seq_lens is not None else B * S
    return 2 * 2 * Hkv * D * tokens


def cpu_attention_pass(case):
    from oracle import attention

    return attention.sdpa_reference(case.q, case.k, case.v, case.seq_lens, dtype=torch.bfloat16)


def time_cpu_baseline(case, budget_s: float = 12.0, max_passes: int = 20):
    """Times the reference's CPU attention call on a bounded number of passes over the same batch."""
    cpu_attention_pass(case)  # warm-up (thread pool, allocator)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max_passes and (time.perf_counter() < t_end or len(times) < 2):
        t = time.perf_counter()
        cpu_attention_pass(case)
        times.append(time.perf_counter() - t)
    best = sorted(times)[len(times) // 2]
    return kv_bytes(case) / best / 1e9, len(times), best


# ------------------------------------------------------------------------------------------------
def run_reference_arm(args, rank, world):
    """The reference's own CPU implementation of the path, timed on the host cores (rank 0 only)."""
    if rank != 0:
        return
    case, desc = make_decode_workload(args.workload if args.workload in ("c1", "c2", "c3") else "c2", 0, 1, args.seq_len)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_attention_pass(case)
    steps = max(1, min(args.steps, 10))
    t = time.perf_counter()
    for _ in range(steps):
        cpu_attention_pass(case)
    dt = (time.perf_counter() - t) / steps
    val = kv_bytes(case) / dt / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "flash-decode HBM GB/s", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc.replace("/GPU", ""), "note": "F.scaled_dot_product_attention(enable_gqa=True) with a "
                   "length mask on the bf16 CPU tensors: the reference's PyTorch attention path (model.py:115-116)"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "reference",
                         "sample": f"mean of {steps} full passes over one batch; os.cpu_count()={os.cpu_count()}"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "rmsnorm", "rope", "c5", "prefill"])
    ap.add_argument("--gen-len", type=int, default=2048, help="c5: tokens generated per sequence")
    ap.add_argument("--batch", type=int, default=64, help="c5: sequences per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--head-dim", type=int, default=64, choices=[64, 128], help="prefill: head size")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-comparator", action="store_true", help="c1-c3: skip the torch SDPA timing on the GPU")
    ap.add_argument("--no-graph", action="store_true", help="c1-c3: launch every step through the extension call "
                    "instead of replaying a captured launch")
    ap.add_argument("--seq-len", type=int, default=131072, help="c3: cached tokens (a shard of C3 on one GPU: 131072 / N)")
    ap.add_argument("--max-ctas", type=int, default=0)
    ap.add_argument("--nccl-merge", action="store_true", help="c3 on >1 GPU: all_gather + merge kernel instead of the fused exchange")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    pkg = load_package()
    ext = pkg.extension()  # no fallback: raises if the CUDA extension is not built

    if args.workload == "c5":
        line = bench_end_to_end(args, ext, pkg, dev, rank, world)
    elif args.workload == "prefill":
        line = bench_prefill(args, ext, pkg, dev, rank, world)
    elif args.workload in ("rmsnorm", "rope"):
        line = bench_pre_attention(args, ext, pkg, dev, rank, world)
    else:
        line = bench_decode(args, ext, pkg, dev, rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sync_all(world):
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int, dev) -> float:
    import torch.distributed as dist

    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int, dev) -> float:
    import torch.distributed as dist

    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def bench_decode(args, ext, pkg, dev, rank, world):
    case, desc = make_decode_workload(args.workload, rank, world, args.seq_len)
    sharded_seq = args.workload == "c3" and world > 1
    if sharded_seq:
        lo, hi = pkg.sharding.kv_shard_bounds(case.k.shape[2], world)[rank]
        from oracle.inputs import DecodeCase

        full_bytes = kv_bytes(case)
        case = DecodeCase(case.q, case.k[:, :, lo:hi], case.v[:, :, lo:hi], None)
    my_bytes = kv_bytes(case)

    # ---- device-resident inputs: N_ROTATE distinct KV caches so that each step finds L2 cold ----
    q = case.q.to(dev)
    lens = case.seq_lens.to(dev) if case.seq_lens is not None else None
    n_rot = N_ROTATE if args.workload != "c3" else 2
    ks, vs = [], []
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    for i in range(n_rot):
        if i == 0:
            ks.append(case.k.to(dev))
            vs.append(case.v.to(dev))
        else:  # same shape, strides and distribution, different values
            B, Hkv, S, D = case.k.shape
            ks.append(torch.randn(B, S, Hkv, D, generator=g, device=dev, dtype=torch.float32).bfloat16().transpose(1, 2))
            vs.append(torch.randn(B, S, Hkv, D, generator=g, device=dev, dtype=torch.float32).bfloat16().transpose(1, 2))
    rot_bytes = sum(k.numel() * 2 * 2 for k in ks)
    out = torch.empty_like(q)

    xchg = None
    if sharded_seq and not args.nccl_merge:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        xchg = pkg.sharding.KvShardExchange(ext, q.shape[0], q.shape[1], q.shape[3], dev)

    def step(i):
        j = i % n_rot
        if sharded_seq and xchg is not None:
            return pkg.sharding.decode_kv_sharded_fused(ext, q, ks[j], vs[j], xchg, device_epoch=True)
        if sharded_seq:
            return pkg.sharding.decode_kv_sharded(ext, q, ks[j], vs[j], None)
        return ext.flash_attention_decode(q, ks[j], vs[j], seq_lens=lens, out=out, max_ctas=args.max_ctas)

    # The launches of the rotating caches are captured back to back in one CUDA graph: the timed loop then
    # costs the host one graph launch per n_rot steps instead of the extension's argument checks and
    # tensor-map encoding per step, which take as long as a short kernel.  (The fused exchange numbers its
    # calls on the device, so its two launches per step are captured too; the NCCL variant stays eager.)
    use_graph = not args.no_graph and (not sharded_seq or xchg is not None)
    n_graph = max(n_rot, 8)  # launches per graph: a graph launch costs the host about as much as an eager call
    run_steps = graph_runner(step, n_graph, dev) if use_graph else eager_runner(step)
    run_steps.prepare(args.warmup)
    run_steps.prepare(args.steps)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    sampler.mark("w0")
    run_steps(args.warmup)
    sync_all(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark("t0")
    start.record()
    run_steps(args.steps)
    end.record()
    torch.cuda.synchronize()
    sampler.mark("t1")
    sync_all(world)
    sampler.stop()
    ms_total = start.elapsed_time(end)
    ms_max = max_over_ranks(ms_total, world, dev)
    status = ext.flash_decode_status(q)
    if status != 0:
        raise RuntimeError(f"device-side wait ran out (status {status})")
    total_bytes = full_bytes if sharded_seq else sum_over_ranks(float(my_bytes), world, dev)
    value = total_bytes * args.steps / (ms_max * 1e-3) / 1e9
    ms_per_step = ms_max / args.steps

    # ---- roofline of the flash-decode kernel: algorithmic bytes of one launch / its average duration ----
    peak, peak_kind = hbm_peak()
    launch_ms = ms_total / args.steps
    achieved = my_bytes / (launch_ms * 1e-3) / 1e9
    # which of the library's two decode kernels these sizes run (0 = persistent grid, else the static deal's split)
    if args.max_ctas > 0:
        choice = 0
    elif args.max_ctas < 0:
        choice = -args.max_ctas
    else:
        choice = pkg.capi.load().l3ci_flash_decode_kernel_choice(q.shape[0], q.shape[1], ks[0].shape[1], q.shape[-1],
                                                                 ks[0].shape[2], int(lens is not None))
    kernel = "flash_decode_kernel" if choice == 0 else "flash_decode_small_kernel"
    traffic = None
    if world == 1 and args.workload == "c2" and kernel == "flash_decode_small_kernel":
        traffic = C2_TRAFFIC_BYTES
    if world == 1 and args.workload == "c3" and kernel == "flash_decode_small_kernel" and args.seq_len == 131072:
        traffic = C3_TRAFFIC_BYTES
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_kind": peak_kind,
                "kernel": kernel, "kernel_split": (None if choice in (0, 1) else {"ctas_per_unit": choice // 16, "warps_per_unit": choice % 16}),
                "algorithmic_bytes_per_launch": my_bytes,
                "frac_of_8TBs_nominal": achieved / 8000.0}
    if sharded_seq:
        roofline["note"] = "per-rank shard; the step also holds the exchange of shard results and their merge"
    if xchg is not None and xchg.check() != 0:
        raise RuntimeError("exchange wait ran out")

    # ---- comparator on the same GPU: torch's own attention (the call the reference checks itself against,
    # benchmark_kernel.py:27-28), same rotating caches, same timing; informational ----
    comparators = None
    if world == 1 and not args.no_comparator:
        import torch.nn.functional as F

        mask = None
        if lens is not None:
            mask = (torch.arange(case.k.shape[2], device=dev)[None, :] < lens[:, None])[:, None, None, :]
        try:
            sd_step = lambda i: F.scaled_dot_product_attention(q, ks[i % n_rot], vs[i % n_rot], attn_mask=mask,  # noqa: E731
                                                               enable_gqa=True)
            sd_run = graph_runner(sd_step, n_graph, dev) if use_graph else eager_runner(sd_step)
            n_sd = max(n_rot, min(args.steps, 200))
            sd_run.prepare(n_sd)
            sd_run.prepare(n_graph)
            sd_run(n_graph)
            torch.cuda.synchronize()
            start.record()
            sd_run(n_sd)
            end.record()
            torch.cuda.synchronize()
            sd_ms = start.elapsed_time(end) / n_sd
            comparators = {"torch_sdpa_gpu": {"ms_per_step": sd_ms, "GB/s": my_bytes / (sd_ms * 1e-3) / 1e9, "steps": n_sd,
                                              "call": "F.scaled_dot_product_attention(q, k, v, enable_gqa=True" +
                                                      (", attn_mask=lengths)" if mask is not None else ")")}}
        except Exception as exc:  # the comparator is optional evidence, never a reason to lose the bench line
            comparators = {"torch_sdpa_gpu": {"error": str(exc)[:200]}}

    # ---- end to end through the extension with host buffers (pinned), copies inside the timed region ----
    # Host side: q [B,1,Hq,D], K and V as the cache holds them, [B,S,Hkv,D], all pinned.  Only the cached tokens
    # of a sequence are input (rows beyond seq_lens[b] are padding that the kernel never reads), so a step copies
    # rows [0, len_b) of every sequence into a device cache that stays allocated.
    hq = case.q.transpose(1, 2).contiguous().pin_memory()
    hk = case.k.transpose(1, 2).contiguous().pin_memory()
    hv = case.v.transpose(1, 2).contiguous().pin_memory()
    hl = case.seq_lens.pin_memory() if case.seq_lens is not None else None
    host_lens = [int(x) for x in case.seq_lens.tolist()] if case.seq_lens is not None else [case.k.shape[2]] * case.k.shape[0]
    hout = torch.empty_like(hq).pin_memory()
    dk_cache, dv_cache = torch.empty_like(hk, device=dev), torch.empty_like(hv, device=dev)
    row_bytes = hk.shape[2] * hk.shape[3] * 2
    h2d = hq.numel() * 2 + 2 * sum(host_lens) * row_bytes + (hl.numel() * 4 if hl is not None else 0)
    d2h = hout.numel() * 2

    def e2e_step():
        dq = hq.to(dev, non_blocking=True).transpose(1, 2)
        for b, n in enumerate(host_lens):
            dk_cache[b, :n].copy_(hk[b, :n], non_blocking=True)
            dv_cache[b, :n].copy_(hv[b, :n], non_blocking=True)
        dk, dv = dk_cache.transpose(1, 2), dv_cache.transpose(1, 2)
        dl = hl.to(dev, non_blocking=True) if hl is not None else None
        if sharded_seq and xchg is not None:
            o = pkg.sharding.decode_kv_sharded_fused(ext, dq, dk, dv, xchg, device_epoch=True)
        elif sharded_seq:
            o = pkg.sharding.decode_kv_sharded(ext, dq, dk, dv, None)
        else:
            o = ext.flash_attention_decode(dq, dk, dv, seq_lens=dl)
        hout.copy_(o.transpose(1, 2), non_blocking=True)

    for _ in range(3):
        e2e_step()
    sync_all(world)
    e_steps = max(1, args.e2e_steps)
    start.record()
    for _ in range(e_steps):
        e2e_step()
    end.record()
    torch.cuda.synchronize()
    sync_all(world)
    e_ms = max_over_ranks(start.elapsed_time(end), world, dev)
    e2e_val = total_bytes * e_steps / (e_ms * 1e-3) / 1e9
    e2e = {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "steps": e_steps, "ms_per_step": e_ms / e_steps}

    # ---- CPU baseline on this box's host cores (rank 0, N=1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, passes, sec = time_cpu_baseline(case)
        cpu = {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "reference",
               "sample": f"median of {passes} full passes of F.scaled_dot_product_attention (bf16, enable_gqa, length "
                         f"mask) over the same batch, {sec * 1e3:.1f} ms each; os.cpu_count()={os.cpu_count()}"}

    B, Hkv, S, D = case.k.shape
    line = {
        "metric": "flash-decode HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if sharded_seq else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "global_batch": B * (1 if sharded_seq else world), "kv_bytes_per_step": int(total_bytes),
                   "l2": f"{n_rot} rotating KV caches per GPU, {rot_bytes / 1e6:.0f} MB > 126 MB L2: each step reads a cold cache",
                   "launch": f"steps are replayed from a CUDA graph of {n_graph} steps back to back" if use_graph
                             else "each step is an eager extension call",
                   "parallelism": ("kv-sequence sharded x%d + %s" % (world, "NCCL all_gather + lse merge" if xchg is None else
                                                                  "fused NVLink exchange/merge kernel")) if sharded_seq else
                                  ("data-parallel x%d, no collective" % world),
                   "pct_of_8TBs_nominal_per_gpu": 100.0 * achieved / 8000.0},
        "roofline": roofline, "e2e": e2e, "gpu_launches": args.steps * (2 if sharded_seq else 1),
        "clocks": sampler.summary(),
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if comparators is not None:
        line["comparators"] = comparators
    return line


def graph_runner(step, n_rot, dev):
    """Returns run_steps(K): K steps as replays of a CUDA graph that holds the n_rot launches step(0..n_rot-1)
    back to back (plus one graph of K % n_rot launches), so that consecutive launches follow each other on the
    device without waiting for the host."""
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step(0)  # per-stream workspaces are allocated outside the capture
    torch.cuda.current_stream(dev).wait_stream(side)
    graphs = {}
    keep = []  # results of the captured calls stay alive, so every step of a graph writes its own buffer

    def graph_of(n):
        if n not in graphs:
            side.wait_stream(torch.cuda.current_stream(dev))
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(gr, stream=side):
                    for j in range(n):
                        keep.append(step(j))
            torch.cuda.current_stream(dev).wait_stream(side)
            graphs[n] = gr
        return graphs[n]

    def prepare(K):
        graph_of(n_rot)
        if K % n_rot:
            graph_of(K % n_rot)

    def run_steps(K):
        for _ in range(K // n_rot):
            graphs[n_rot].replay()
        if K % n_rot:
            graphs[K % n_rot].replay()

    run_steps.prepare = prepare
    return run_steps


def eager_runner(step):
    def run_steps(K):
        for i in range(K):
            step(i)

    run_steps.prepare = lambda K: None
    return run_steps


def bench_prefill(args, ext, pkg, dev, rank, world):
    """Causal GQA prefill attention at the 1B shape with 2048-token prompts (the long-prompt scenarios of the
    reference's README tables; there the call is torch's SDPA, model.py:114-116): B=4, Hq=32, Hkv=8, D=64, T=2048.
    Compute-bound: the figure is TFLOP/s over the causal half, 4 * B * Hq * D * T * (T + 1) / 2 flops."""
    import torch.nn.functional as F

    B, Hq, Hkv, D, T = 4, 32, 8, args.head_dim, 2048
    g = torch.Generator(device=dev).manual_seed(42 + rank)
    n_rot = 4
    qs = [torch.randn(B, T, Hq, D, generator=g, device=dev).bfloat16().transpose(1, 2) for _ in range(n_rot)]
    ks = [torch.randn(B, T, Hkv, D, generator=g, device=dev).bfloat16().transpose(1, 2) for _ in range(n_rot)]
    vs = [torch.randn(B, T, Hkv, D, generator=g, device=dev).bfloat16().transpose(1, 2) for _ in range(n_rot)]
    flops = 4.0 * B * Hq * D * T * (T + 1) / 2
    steps = min(args.steps, 400)

    def timed(step):
        run_steps = eager_runner(step) if args.no_graph else graph_runner(step, n_rot, dev)
        run_steps.prepare(args.warmup)
        run_steps.prepare(steps)
        run_steps(args.warmup)
        sync_all(world)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run_steps(steps)
        end.record()
        torch.cuda.synchronize()
        sync_all(world)
        return start.elapsed_time(end)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    sampler.mark("t0")
    ms_total = timed(lambda i: ext.prefill_attention(qs[i % n_rot], ks[i % n_rot], vs[i % n_rot]))
    sampler.mark("t1")
    sampler.stop()
    ms_max = max_over_ranks(ms_total, world, dev)
    sd_ms = timed(lambda i: F.scaled_dot_product_attention(qs[i % n_rot], ks[i % n_rot], vs[i % n_rot], is_causal=True,
                                                           enable_gqa=True)) / steps
    got = ext.prefill_attention(qs[0], ks[0], vs[0]).float()
    ref = F.scaled_dot_product_attention(qs[0], ks[0], vs[0], is_causal=True, enable_gqa=True).float()
    peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json"))) \
        if os.path.exists(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    achieved = flops / (ms_total / steps * 1e-3) / 1e12
    return {
        "metric": "prefill attention TFLOP/s", "value": flops * world * steps / (ms_max * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "warmup": args.warmup, "ms_per_step": ms_max / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"causal GQA prefill B={B} Hq={Hq} Hkv={Hkv} D={D} T={T}", "flops_per_step": flops,
                   "l2": f"{n_rot} rotating q/k/v sets", "max_abs_diff_vs_torch_sdpa_gpu": float((got - ref).abs().max())},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": "measured" if peaks else "fallback", "kernel": "prefill_attention_kernel",
                     "note": "mma.sync path; its own ceiling is about a quarter of the tcgen05 peak the denominator was measured with"},
        "comparators": {"torch_sdpa_gpu": {"ms_per_step": sd_ms, "TFLOP/s": flops / (sd_ms * 1e-3) / 1e12,
                                           "call": "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"}},
        "gpu_launches": steps, "clocks": sampler.summary(),
    }


def bench_pre_attention(args, ext, pkg, dev, rank, world):
    """C4: RMSNorm over [4096, 2048] tokens, or fused RoPE + KV-cache write of q (32x64) and k, v (8x64)."""
    from oracle import inputs

    x, w, eps, qkv = inputs.config4(seed=42 + rank)
    Hq, Hkv, D, B, S = 32, 8, 64, 2, 2048
    freq = pkg.rope_table.precompute_freqs_cis(D, S, **{k: v for k, v in inputs.ROPE_CONFIG4.items()}).to(dev)
    n_rot = 12  # 12 x (33.5 | 50 MB) > 126 MB L2
    if args.workload == "rmsnorm":
        xs = [x.to(dev) if i == 0 else torch.randn_like(x.float(), device=dev).bfloat16() for i in range(n_rot)]
        dw = w.to(dev)
        nbytes = 2 * x.numel() * 2 + w.numel() * 2
        step = lambda i: ext.rms_norm(xs[i % n_rot], dw, eps)
        kernel = "rms_norm_kernel"
        desc = "C4 RMSNorm: tokens 4096 x hidden 2048 bf16, eps 1e-5"
    else:
        qs = [qkv.to(dev) if i == 0 else torch.randn_like(qkv.float(), device=dev).bfloat16() for i in range(n_rot)]
        cks = [torch.zeros(B, S, Hkv, D, dtype=torch.bfloat16, device=dev) for _ in range(n_rot)]
        cvs = [torch.zeros_like(cks[0]) for _ in range(n_rot)]
        nbytes = 2 * qkv.numel() * 2 + freq.numel() * 4
        step = lambda i: ext.rot_embed_kv_cache(qs[i % n_rot], freq, cks[i % n_rot], cvs[i % n_rot], 0, Hq, Hkv)
        kernel = "rot_embed_kv_cache_kernel"
        desc = "C4 fused RoPE + KV-cache write: tokens 4096, q 32x64, k/v 8x64 bf16, Llama-3 scaling factor 32"
    run_steps = eager_runner(step) if args.no_graph else graph_runner(step, n_rot, dev)
    run_steps.prepare(args.warmup)
    run_steps.prepare(args.steps)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    sampler.mark("w0")
    run_steps(args.warmup)
    sync_all(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark("t0")
    start.record()
    run_steps(args.steps)
    end.record()
    torch.cuda.synchronize()
    sampler.mark("t1")
    sync_all(world)
    sampler.stop()
    ms_total = start.elapsed_time(end)
    ms_max = max_over_ranks(ms_total, world, dev)
    value = nbytes * world * args.steps / (ms_max * 1e-3) / 1e9
    peak, peak_kind = hbm_peak()
    achieved = nbytes / (ms_total / args.steps * 1e-3) / 1e9
    return {
        "metric": "pre-attention HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "l2": f"{n_rot} rotating inputs and outputs > 126 MB L2", "bytes_per_step": nbytes,
                   "launch": "each step is an eager extension call (with its output allocation)" if args.no_graph else
                             f"steps are replayed from a CUDA graph of {n_rot} extension calls back to back"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": kernel},
        "gpu_launches": args.steps, "clocks": sampler.summary(),
    }


def bench_end_to_end(args, ext, pkg, dev, rank, world):
    """C5: random-init Llama-3.2-1B architecture, batch 64 per GPU, 128-token prompts, greedy decoding of
    --gen-len tokens; tokens/s = generated tokens / (prefill + decode) time, the reference's formula
    (benchmark_model.py:82).  One step = one whole generation; replicas only across GPUs."""
    dl = pkg.decode_loop
    cfg = dl.DecoderConfig()
    B, P, G = args.batch, 128, args.gen_len
    steps = min(args.steps, 3) if args.steps != 2000 else 1
    model = dl.Llama3Decoder(ext, cfg, dev, max_batch=B, max_len=P + G, seed=42 + rank)
    g = torch.Generator().manual_seed(1000 + rank)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).to(dev)
    model.generate(prompts, min(G, 8))  # warm-up: allocations, cuBLAS heuristics, graph capture path
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    sampler.mark("w0")
    sync_all(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark("t0")
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        toks = model.generate(prompts, G)
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    sampler.mark("t1")
    sync_all(world)
    sampler.stop()
    ms = max_over_ranks(max(start.elapsed_time(end), wall * 1e3), world, dev)
    if ext.flash_decode_status(toks) != 0:
        raise RuntimeError("device-side wait ran out")
    value = G * B * world * steps / (ms * 1e-3)
    # end to end through the public call with host inputs: prompts from pinned host memory, tokens read back
    hp = prompts.cpu().pin_memory()
    hout = torch.empty(B, G, dtype=torch.int64).pin_memory()
    sync_all(world)
    t0 = time.perf_counter()
    toks = model.generate(hp.to(dev, non_blocking=True), G)
    hout.copy_(toks, non_blocking=True)
    torch.cuda.synchronize()
    e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world, dev)
    e2e = {"value": G * B * world / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": hp.numel() * 8,
           "d2h_bytes_per_step": hout.numel() * 8, "steps": 1, "ms_per_step": e_ms}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_end_to_end(cfg, dl, B, P, G)
    decode_steps = (G - 1) * steps
    line = {
        "metric": "Llama-3.2-1B decode tokens/sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": 1, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        # the reference's README publishes 2041.67 tokens/s for this configuration (on an RTX 4060)
        "vs_baseline": value / 2041.67 if (G == 2048 and B == 64) else None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"C5 random-init Llama-3.2-1B architecture, batch {B}/GPU, prompt {P}, {G} greedy tokens",
                   "global_batch": B * world, "parallelism": "replicas x%d" % world,
                   "l2": "working set per decode step (2.5 GB weights + KV cache) >> 126 MB L2",
                   "note": "GEMMs are cuBLAS via torch; RMSNorm (+ residual add), SiLU*mul, RoPE + cache write, decode attention and the greedy step are this "
                           "repository's kernels; the decode step is replayed from a CUDA graph",
                   "reference_published_rtx4060_tokens_per_s": 2041.67},
        "e2e": e2e,
        # per decode step: 33 RMSNorm (32 with the residual add) + 16 SiLU*mul + 16 fused RoPE/cache + 16
        # flash-decode + 1 greedy-step launches of this library; the prefill pass has no flash-decode
        "gpu_launches": decode_steps * 82 + steps * 65, "clocks": sampler.summary(),
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    return line


def cpu_baseline_end_to_end(cfg, dl, B, P, G):
    """The same architecture through the CPU restatement on a bounded sample, extrapolated: prefill of 4 of
    the B prompts (scaled by B/4) plus 2 decode steps of the full batch at the start of generation (scaled by
    G; later steps attend to longer caches, so this favours the CPU)."""
    from oracle.decode_loop import CpuDecoder

    weights = dl.init_weights(cfg, 42)
    cpu = CpuDecoder(cfg, weights, B, P + 8)
    g = torch.Generator().manual_seed(1000)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    t = time.perf_counter()
    cpu.forward(prompts[:4], 0)
    t_prefill = (time.perf_counter() - t) * (B / 4)
    tok = torch.zeros(B, 1, dtype=torch.int64)
    cpu.forward(tok, P)  # warm-up of the decode path
    t = time.perf_counter()
    for i in range(2):
        cpu.forward(tok, P + 1 + i)
    t_step = (time.perf_counter() - t) / 2
    total = t_prefill + t_step * (G - 1)
    return {"value": G * B / total, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"prefill of 4/{B} prompts ({t_prefill:.1f} s when scaled) + 2 decode steps of the full batch "
                      f"({t_step * 1e3:.0f} ms each) extrapolated to {G} tokens; os.cpu_count()={os.cpu_count()}"}


if __name__ == "__main__":
    main()
