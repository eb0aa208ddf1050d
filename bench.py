#!/usr/bin/env python
"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|rmsnorm|rope|c5|prefill]
                    [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: for the default workload (C2) one
`flash_attention_decode` call over a ragged batch of 16 sequences (32 q / 8 kv heads, head size 128, lengths
uniform in [1024, 2048], cache padded to 2048, bf16).  The metric is the reference's own
(benchmark_kernel.py:48-49): bytes of K and V that belong to valid tokens, 2*2*Hkv*D*sum(len), per second,
in decimal GB/s.

Printed JSON line (rank 0):
  value          GB/s over all GPUs with inputs resident in HBM; K steps timed as one region with CUDA events
                 on the launching stream, barrier + synchronize on both sides, max over ranks.  A region
                 shorter than 50 ms is repeated (each repeat bracketed the same way) and the median region is
                 reported, with the minimum and maximum beside it (`regions`)
  e2e            the same metric through the extension module with HOST inputs: every step copies q, k, v
                 (and seq_lens) from pinned host memory, runs the kernel and reads the output back
  roofline       achieved algorithmic GB/s of the flash-decode kernel against the measured HBM copy bandwidth
  cpu_baseline   the reference's PyTorch attention path (scaled_dot_product_attention, bf16, on the CPU tensors)
                 timed on this box's host cores over a bounded number of passes (rank 0)
  clocks         SM clock and throttle reasons sampled through NVML while the GPU was busy
  c3             (default workload only, every N) the long-context step: 131072 cached tokens of one sequence,
                 KV sequence sharded over the N ranks, per-rank decode kernel + fused NVLink exchange/merge;
                 rank 0's merged output is checked against the CPU oracle BEFORE timing and the process
                 exits non-zero on a mismatch; strong scaling
  c1, c4_rmsnorm, c4_rope, c5
                 (default workload, N = 1) the other configurations, each with its own roofline; prefill_d64 and
                 prefill_d128: causal prefill attention (the step before the path) against torch's SDPA
  comparators    torch's SDPA on the same GPU tensors; and, at N = 1, the reference's own CUDA kernels rebuilt
                 for sm_100 (oracle/_ref, when present), timed beside this library's calls

L2 hygiene: every step reads a different one of 8 KV caches (1.07 GB in total, L2 is 126 MB), so a cache is
cold again when its turn comes.  With --impl reference the CPU baseline alone is run and reported.
Multi-GPU (launched by torch.distributed.run, one rank per GPU): C2 is weak-scaled, every rank owns a batch
of 16 sequences and no data crosses GPUs; C3 shards the KV sequence across ranks and merges the per-rank
(o, lse) pairs over NVLink.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from ncu captures of these kernels on these workloads
# (seed 42); reported only when the kernel and the shape of the run are the captured ones.
TRAFFIC = {
    ("c2", "flash_decode_small_kernel"): (106_150_000, "ncu capture of flash_decode_small_kernel on C2: 102.10 MB read + 4.05 MB written"),
    ("c3", "flash_decode_small_kernel"): (540_310_000, "ncu capture of flash_decode_small_kernel on C3: 536.91 MB read + 3.40 MB written"),
}
MIN_REGION_MS = 50.0   # a K-step region shorter than this is repeated until this much has been timed
MAX_REGIONS = 400


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


def use_all_host_cores() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; the CPU baseline is meant to use the host
    cores the box has, as a plain `python bench.py` run does."""
    n = os.cpu_count() or 1
    if torch.get_num_threads() < n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def time_cpu_baseline(case, budget_s: float = 12.0, max_passes: int = 20):
    """Times the reference's CPU attention call on a bounded number of passes over the same batch."""
    use_all_host_cores()
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
    """The reference's own CPU implementation of the path, timed on the host cores (rank 0 only): the same
    workload, metric and unit as the GPU arm at this N.  A step is one pass of
    F.scaled_dot_product_attention over the global batch (the N per-GPU batches of the GPU arm, one after the
    other); W warm-up steps, then K timed steps, as asked for."""
    if rank != 0:
        return
    cores = use_all_host_cores()
    name = args.workload if args.workload in ("c1", "c2", "c3") else "c2"
    n_batches = world if name != "c3" else 1   # C3 is one sequence whatever N is (strong scaling)
    cases, desc = [], None
    for r in range(n_batches):
        case, desc = make_decode_workload(name, r, world, args.seq_len)
        cases.append(case)
    total_bytes = sum(kv_bytes(c) for c in cases)
    for _ in range(args.warmup):
        for c in cases:
            cpu_attention_pass(c)
    t = time.perf_counter()
    for _ in range(args.steps):
        for c in cases:
            cpu_attention_pass(c)
    dt = (time.perf_counter() - t) / args.steps
    val = total_bytes / dt / 1e9
    line = {
        "impl": "reference", "metric": "flash-decode HBM GB/s", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if name == "c3" else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "global_batch": sum(c.k.shape[0] for c in cases), "kv_bytes_per_step": int(total_bytes),
                   "note": "F.scaled_dot_product_attention(enable_gqa=True) with a length mask on the bf16 CPU tensors: the "
                           "reference's PyTorch attention path (model.py:115-116), no GPU involved"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "reference",
                         "sample": f"mean of {args.steps} passes over the global batch of {n_batches} x the per-GPU batch; "
                                   f"os.cpu_count()={os.cpu_count()}"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def launch_kind(args) -> str:
    """What config.launch says about programmatic dependent launch."""
    return ("; plain launches (--plain-launch)" if args.plain_launch else
            "; kernels launched with programmatic stream serialization (each waits with griddepcontrol.wait for "
            "the previous step's kernel before its first global access)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--workload", default=None, choices=["c1", "c2", "c3", "rmsnorm", "rope", "c5", "prefill"],
                    help="default: c2 as the headline plus the sub-records of the other configurations")
    ap.add_argument("--gen-len", type=int, default=2048, help="c5: tokens generated per sequence")
    ap.add_argument("--batch", type=int, default=64, help="c5: sequences per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--head-dim", type=int, default=64, choices=[64, 128], help="prefill: head size")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-comparator", action="store_true", help="skip the torch SDPA and reference-CUDA timings on the GPU")
    ap.add_argument("--no-subrecords", action="store_true", help="default workload: only the C2 headline")
    ap.add_argument("--no-graph", action="store_true", help="c1-c3: launch every step through the extension call "
                    "instead of replaying a captured launch")
    ap.add_argument("--seq-len", type=int, default=131072, help="c3: cached tokens (a shard of C3 on one GPU: 131072 / N)")
    ap.add_argument("--max-ctas", type=int, default=0)
    ap.add_argument("--plain-launch", action="store_true", help="launch kernels without programmatic dependent launch "
                    "(l3ci_set_programmatic_launch(0)); for A/B runs")
    ap.add_argument("--nccl-merge", action="store_true", help="c3 on >1 GPU: all_gather + merge kernel instead of the fused exchange")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)
    full_line = args.workload is None and not args.no_subrecords
    if args.workload is None:
        args.workload = "c2"

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
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev)

    pkg = load_package()
    if args.plain_launch:
        pkg.capi.load().l3ci_set_programmatic_launch(0)
    ext = pkg.extension()  # no fallback: raises if the CUDA extension is not built

    if args.workload == "c5":
        line = bench_end_to_end(args, ext, pkg, dev, rank, world)
    elif args.workload == "prefill":
        line = bench_prefill(args, ext, pkg, dev, rank, world)
    elif args.workload in ("rmsnorm", "rope"):
        line = bench_pre_attention(args, ext, pkg, dev, rank, world, args.workload)
    else:
        line = bench_decode(args, ext, pkg, dev, rank, world, args.workload)
    if full_line:
        add_sub_records(line, args, ext, pkg, dev, rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def add_sub_records(line, args, ext, pkg, dev, rank, world):
    """The configurations beside the headline, measured in the same process: C3 at every N (sharded over the
    ranks, checked against the oracle before it is timed), and at N = 1 also C1, the two C4 kernels, C5 and the
    reference's own CUDA kernels as a comparator."""
    def brief(rec, keep=("metric", "value", "unit", "ms_per_step", "steps", "regions", "scaling", "config", "roofline",
                         "parity", "comparators", "gpu_launches", "e2e", "clocks")):
        return {k: rec[k] for k in keep if k in rec}

    torch.cuda.empty_cache()
    line["c3"] = brief(bench_decode(args, ext, pkg, dev, rank, world, "c3", lean=True))
    if world > 1:
        return
    torch.cuda.empty_cache()
    line["c1"] = brief(bench_decode(args, ext, pkg, dev, rank, world, "c1", lean=True))
    torch.cuda.empty_cache()
    line["c4_rmsnorm"] = brief(bench_pre_attention(args, ext, pkg, dev, rank, world, "rmsnorm"))
    torch.cuda.empty_cache()
    line["c4_rope"] = brief(bench_pre_attention(args, ext, pkg, dev, rank, world, "rope"))
    torch.cuda.empty_cache()
    if not args.no_comparator:
        try:
            line.setdefault("comparators", {})["reference_cuda_sm100"] = time_reference_cuda(ext, pkg, dev)
        except Exception as exc:   # optional evidence, never a reason to lose the bench line
            line.setdefault("comparators", {})["reference_cuda_sm100"] = {"error": str(exc)[:300]}
        torch.cuda.empty_cache()
    for hd in (64, 128):
        pf_args = argparse.Namespace(**vars(args))
        pf_args.head_dim = hd
        line[f"prefill_d{hd}"] = brief(bench_prefill(pf_args, ext, pkg, dev, rank, world))
        torch.cuda.empty_cache()
    c5_args = argparse.Namespace(**vars(args))
    c5_args.no_cpu_baseline = True
    c5_args.steps = 1
    line["c5"] = brief(bench_end_to_end(c5_args, ext, pkg, dev, rank, world))
    torch.cuda.empty_cache()


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


def timed_regions(run_steps, steps: int, world: int, dev, sampler=None):
    """Times `steps` steps as ONE region (CUDA events on the launching stream, barrier + synchronize on both
    sides) and repeats the region while less than MIN_REGION_MS has been timed in total.  Returns
    (this rank's ms of the median region, max-over-ranks ms of the median region, summary dict).  The repeat
    decision uses the max over ranks, so every rank makes the same number of repeats."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    regions, total = [], 0.0
    if sampler is not None:
        sampler.mark("t0")
    while True:
        sync_all(world)
        start.record()
        run_steps(steps)
        end.record()
        torch.cuda.synchronize()
        sync_all(world)
        mine = start.elapsed_time(end)
        worst = max_over_ranks(mine, world, dev)
        regions.append((worst, mine))
        total += worst
        if total >= MIN_REGION_MS or len(regions) >= MAX_REGIONS:
            break
    if sampler is not None:
        sampler.mark("t1")
    regions.sort()
    worst, mine = regions[len(regions) // 2]
    summary = {"n": len(regions), "steps_each": steps, "ms_median": worst, "ms_min": regions[0][0], "ms_max": regions[-1][0],
               "reported": "median region"}
    return mine, worst, summary


def attention_parity(out, case_full, rank, world, dev, what):
    """Rank 0 compares `out` (bf16 [B,Hq,1,D] on the device) with the CPU oracle under the attention tolerance
    (2e-2 absolute + 1e-2 relative against fp32) and a relative-L2 bound of 1e-2; every rank learns the verdict
    and the process group leaves with a non-zero exit code on a mismatch."""
    import torch.distributed as dist

    rec = {"checked": what, "oracle": "F.scaled_dot_product_attention in fp32 on the CPU (oracle.attention.sdpa_reference)",
           "tolerance": "|err| <= 2e-2 + 1e-2*|ref| and relative L2 <= 1e-2"}
    ok = torch.ones(1, dtype=torch.int32, device=dev)
    if rank == 0:
        from oracle import attention

        use_all_host_cores()
        want = attention.sdpa_reference(case_full.q, case_full.k, case_full.v, case_full.seq_lens)
        got = out.detach().float().cpu()
        err = (got - want).abs()
        rel_l2 = float((got - want).norm() / want.norm().clamp_min(1e-30))
        fine = bool(torch.isfinite(got).all()) and bool((err <= 2e-2 + 1e-2 * want.abs()).all()) and rel_l2 <= 1e-2
        rec.update({"ok": fine, "max_abs_err": float(err.max()), "rel_l2_err": rel_l2, "max_abs_ref": float(want.abs().max())})
        ok[0] = 1 if fine else 0
    if world > 1:
        dist.broadcast(ok, 0)
    if int(ok.item()) != 1:
        if rank == 0:
            print(json.dumps({"error": "parity check failed before timing", "parity": rec}), flush=True)
        raise SystemExit(3)
    return rec


def bench_decode(args, ext, pkg, dev, rank, world, workload, lean=False):
    """C1 / C2 / C3.  `lean`: a sub-record (no end-to-end leg, no CPU baseline)."""
    case, desc = make_decode_workload(workload, rank, world, args.seq_len)
    sharded_seq = workload == "c3" and world > 1
    case_full = case
    full_bytes = kv_bytes(case)
    if sharded_seq:
        lo, hi = pkg.sharding.kv_shard_bounds(case.k.shape[2], world)[rank]
        from oracle.inputs import DecodeCase

        case = DecodeCase(case.q, case.k[:, :, lo:hi], case.v[:, :, lo:hi], None)
    my_bytes = kv_bytes(case)

    # ---- device-resident inputs: N_ROTATE distinct KV caches so that each step finds L2 cold ----
    q = case.q.to(dev)
    lens = case.seq_lens.to(dev) if case.seq_lens is not None else None
    n_rot = N_ROTATE if workload != "c3" else 2
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
        xchg = pkg.sharding.KvShardExchange(ext, q.shape[0], q.shape[1], q.shape[3], dev)

    def step(i):
        j = i % n_rot
        if sharded_seq and xchg is not None:
            return pkg.sharding.decode_kv_sharded_fused(ext, q, ks[j], vs[j], xchg, device_epoch=True)
        if sharded_seq:
            return pkg.sharding.decode_kv_sharded(ext, q, ks[j], vs[j], None)
        return ext.flash_attention_decode(q, ks[j], vs[j], seq_lens=lens, out=out, max_ctas=args.max_ctas)

    # ---- parity before timing: the step on the seeded inputs (cache 0) against the CPU oracle ----
    parity = None
    if workload == "c3" or lean:
        got = step(0)
        torch.cuda.synchronize()
        parity = attention_parity(got, case_full, rank, world, dev,
                                  f"{workload} step output of rank 0" + (f" (KV sharded over {world} ranks, merged)" if sharded_seq else ""))

    # The launches of the rotating caches are captured back to back in one CUDA graph: the timed loop then
    # costs the host one graph launch per n_rot steps instead of the extension's argument checks and
    # tensor-map encoding per step, which take as long as a short kernel.  (The fused exchange numbers its
    # calls on the device, so its launches are captured too; the NCCL variant stays eager.)
    use_graph = not args.no_graph and (not sharded_seq or xchg is not None)
    n_graph = max(n_rot, 8)  # launches per graph: a graph launch costs the host about as much as an eager call
    run_steps = graph_runner(step, n_graph, dev) if use_graph else eager_runner(step)
    run_steps.prepare(args.warmup)
    run_steps.prepare(args.steps)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    sampler.mark("w0")
    run_steps(args.warmup)
    ms_total, ms_max, regions = timed_regions(run_steps, args.steps, world, dev, sampler)
    sampler.stop()
    status = ext.flash_decode_status(q)
    if status != 0:
        raise RuntimeError(f"device-side wait ran out (status {status})")
    one_launch = bool(xchg is not None and xchg.one_launch)
    total_bytes = full_bytes if sharded_seq else sum_over_ranks(float(my_bytes), world, dev)
    value = total_bytes * args.steps / (ms_max * 1e-3) / 1e9
    ms_per_step = ms_max / args.steps

    # ---- roofline of the flash-decode kernel: algorithmic bytes of one launch / its average duration ----
    peak, peak_kind = hbm_peak()
    launch_ms = ms_total / args.steps
    achieved = my_bytes / (launch_ms * 1e-3) / 1e9
    # which of the library's decode kernels these sizes run (0 = persistent grid, else the static deal's split)
    if args.max_ctas > 0:
        choice = 0
    elif args.max_ctas < 0:
        choice = -args.max_ctas
    else:
        choice = pkg.capi.load().l3ci_flash_decode_kernel_choice(q.shape[0], q.shape[1], ks[0].shape[1], q.shape[-1],
                                                                 ks[0].shape[2], int(lens is not None))
    kernel = "flash_decode_kernel" if choice == 0 else "flash_decode_small_kernel"
    traffic, traffic_source = None, None
    if world == 1 and (workload != "c3" or args.seq_len == 131072) and (workload, kernel) in TRAFFIC:
        traffic, traffic_source = TRAFFIC[(workload, kernel)]
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_source, "peak_kind": peak_kind,
                "kernel": kernel, "kernel_split": (None if choice in (0, 1) else {"ctas_per_unit": choice // 16, "warps_per_unit": choice % 16}),
                "algorithmic_bytes_per_launch": my_bytes,
                "frac_of_8TBs_nominal": achieved / 8000.0}
    if sharded_seq:
        roofline["note"] = ("per-rank shard of %d tokens; the step also holds the exchange of shard results and their merge, so this "
                            "is the whole step against the HBM time of the shard" % case.k.shape[2])
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
            _, sd_total, _ = timed_regions(sd_run, n_sd, 1, dev)
            sd_ms = sd_total / n_sd
            comparators = {"torch_sdpa_gpu": {"ms_per_step": sd_ms, "GB/s": my_bytes / (sd_ms * 1e-3) / 1e9, "steps": n_sd,
                                              "call": "F.scaled_dot_product_attention(q, k, v, enable_gqa=True" +
                                                      (", attn_mask=lengths)" if mask is not None else ")")}}
        except Exception as exc:  # the comparator is optional evidence, never a reason to lose the bench line
            comparators = {"torch_sdpa_gpu": {"error": str(exc)[:200]}}

    B, Hkv, S, D = case.k.shape
    line = {
        "metric": "flash-decode HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if workload == "c3" else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "global_batch": B * (1 if sharded_seq else world), "kv_bytes_per_step": int(total_bytes),
                   "l2": f"{n_rot} rotating KV caches per GPU, {rot_bytes / 1e6:.0f} MB > 126 MB L2: each step reads a cold cache",
                   "launch": (f"steps are replayed from a CUDA graph of {n_graph} steps back to back" if use_graph
                              else "each step is an eager extension call") + launch_kind(args),
                   "parallelism": ("kv-sequence sharded x%d + %s" % (world, "NCCL all_gather + lse merge" if xchg is None else
                                                                  ("exchange over NVLink (peer stores, no collective) and merge in the decode "
                                                                   "kernel's tail: one launch per rank and step" if one_launch else
                                                                   "decode kernel + one exchange/merge kernel over NVLink (peer stores, no collective)"))) if sharded_seq else
                                  ("data-parallel x%d, no collective" % world),
                   "pct_of_8TBs_nominal_per_gpu": 100.0 * achieved / 8000.0},
        "regions": regions, "roofline": roofline,
        "gpu_launches": args.steps * (2 if sharded_seq and not one_launch else 1),
        "clocks": sampler.summary(),
    }
    if parity is not None:
        line["parity"] = parity
    if comparators is not None:
        line["comparators"] = comparators
    if lean:
        return line

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
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(e_steps):
        e2e_step()
    end.record()
    torch.cuda.synchronize()
    sync_all(world)
    e_ms = max_over_ranks(start.elapsed_time(end), world, dev)
    e2e_val = total_bytes * e_steps / (e_ms * 1e-3) / 1e9
    line["e2e"] = {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "steps": e_steps, "ms_per_step": e_ms / e_steps}

    # ---- CPU baseline on this box's host cores (rank 0, at every N; the other ranks wait at the next barrier) ----
    if rank == 0 and not args.no_cpu_baseline:
        v, passes, sec = time_cpu_baseline(case_full if workload == "c3" else case)
        line["cpu_baseline"] = {
            "value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "reference",
            "sample": f"median of {passes} full passes of F.scaled_dot_product_attention (bf16, enable_gqa, length "
                      f"mask) over one GPU's batch, {sec * 1e3:.1f} ms each; os.cpu_count()={os.cpu_count()}"}
    sync_all(world)
    return line


def time_reference_cuda(ext, pkg, dev):
    """The reference's own CUDA kernels (custom_kernels/custom_kernels.cu, unmodified, rebuilt for sm_100 into
    oracle/_ref) beside this library's calls on the same GPU and tensors: its three functions on C1, on a
    uniform-length C2 (its interface has one length for the batch) and on C4.  Both sides are timed the same way:
    eager calls back to back with CUDA events (the reference launches on the legacy default stream and allocates
    its outputs and scratch inside every call, so it cannot be captured in a graph), and the device time of the
    kernels alone from the profiler's kernel records.  Its attention output is not a correctness reference."""
    from oracle import build_ref, inputs

    ref = build_ref.load()
    if ref is None:
        return {"unavailable": "oracle/_ref/reference_kernels_sm100.so is not built (needs the reference checkout at build time)"}

    def timed(fn, n_inputs, calls=48):
        for i in range(4):
            fn(i % n_inputs)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(calls):
            fn(i % n_inputs)
        end.record()
        torch.cuda.synchronize()
        eager_us = start.elapsed_time(end) * 1e3 / calls
        kernel_us = None
        try:
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for i in range(n_inputs):
                    fn(i)
                torch.cuda.synchronize()
            total = sum(e.device_time_total for e in prof.key_averages() if e.device_type.name == "CUDA" or e.device_time_total > 0)
            kernel_us = total / n_inputs
        except Exception:
            pass
        return eager_us, kernel_us

    res = {"source": "the reference's custom_kernels.cu + main.cpp, unmodified, compiled for sm_100 (oracle/build_ref.py)",
           "timing": "eager_us: CUDA events around 48 back-to-back calls on rotating inputs larger than L2; kernel_us: device "
                     "time of the kernels of one call (profiler kernel records), mean over the rotating inputs"}

    def pair(name, nbytes, ref_fn, our_fn, n_inputs):
        r_eager, r_kernel = timed(ref_fn, n_inputs)
        o_eager, o_kernel = timed(our_fn, n_inputs)
        rec = {"bytes": nbytes, "reference": {"eager_us": r_eager, "kernel_us": r_kernel},
               "this_library": {"eager_us": o_eager, "kernel_us": o_kernel}}
        if r_kernel and o_kernel:
            rec["kernel_time_ratio"] = r_kernel / o_kernel
            rec["reference"]["GB/s"] = nbytes / r_kernel / 1e3
            rec["this_library"]["GB/s"] = nbytes / o_kernel / 1e3
        res[name] = rec

    g = torch.Generator(device=dev).manual_seed(7)

    def caches(B, S, Hkv, D, n):
        return [torch.randn(B, S, Hkv, D, generator=g, device=dev).bfloat16().transpose(1, 2) for _ in range(n)]

    # C1 (the cache is 0.5 MB: 8 caches do not leave L2; reported as it is, the call is latency-bound)
    c1 = inputs.config1()
    q1 = c1.q.to(dev)
    k1, v1 = caches(1, 256, 8, 64, 8), caches(1, 256, 8, 64, 8)
    pair("c1_attention", kv_bytes(c1), lambda i: ref.flash_attention_decode(q1, k1[i], v1[i]),
         lambda i: ext.flash_attention_decode(q1, k1[i], v1[i]), 8)
    # C2 with one length for the whole batch: B=16, 2048 cached tokens each
    q2 = torch.randn(16, 1, 32, 128, generator=g, device=dev).bfloat16().transpose(1, 2)
    k2, v2 = caches(16, 2048, 8, 128, 4), caches(16, 2048, 8, 128, 4)
    pair("c2_uniform_attention", 2 * 2 * 8 * 128 * 16 * 2048, lambda i: ref.flash_attention_decode(q2, k2[i], v2[i]),
         lambda i: ext.flash_attention_decode(q2, k2[i], v2[i]), 4)
    del k2, v2
    # C4: RMSNorm and the rotation of q and k (two calls, as model.py:100-101 makes them)
    x, w, eps, qkv = inputs.config4(seed=42)
    xs = [x.to(dev)] + [torch.randn(x.shape, generator=g, device=dev).bfloat16() for _ in range(7)]
    dw = w.to(dev)
    pair("c4_rms_norm", 2 * x.numel() * 2 + w.numel() * 2, lambda i: ref.rms_norm(xs[i], dw, eps), lambda i: ext.rms_norm(xs[i], dw, eps), 8)
    del xs
    Hq, Hkv, D = 32, 8, 64
    B, S = qkv.shape[:2]
    freq = pkg.rope_table.precompute_freqs_cis(D, S, **inputs.ROPE_CONFIG4).to(dev)
    qs = [qkv.to(dev)] + [torch.randn(qkv.shape, generator=g, device=dev).bfloat16() for _ in range(5)]

    def views(t):
        return t[..., : Hq * D].view(B, S, Hq, D), t[..., Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)

    def rope_ref(i):
        a, b = views(qs[i])
        return ref.rot_embed(a, freq), ref.rot_embed(b, freq)

    def rope_ours(i):
        a, b = views(qs[i])
        return ext.rot_embed(a, freq), ext.rot_embed(b, freq)

    pair("c4_rot_embed_q_and_k", 2 * B * S * (Hq + Hkv) * D * 2 + freq.numel() * 4, rope_ref, rope_ours, 6)
    return res


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
                     "traffic": None, "peak_kind": "measured" if peaks else "fallback",
                     "kernel": "prefill_tc_persist_kernel (tcgen05 + tensor memory, two query heads of a KV head per item, persistent grid)"},
        "comparators": {"torch_sdpa_gpu": {"ms_per_step": sd_ms, "TFLOP/s": flops / (sd_ms * 1e-3) / 1e12,
                                           "call": "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"}},
        "gpu_launches": steps, "clocks": sampler.summary(),
    }


def bench_pre_attention(args, ext, pkg, dev, rank, world, workload):
    """C4: RMSNorm over [4096, 2048] tokens, or fused RoPE + KV-cache write of q (32x64) and k, v (8x64)."""
    from oracle import inputs

    x, w, eps, qkv = inputs.config4(seed=42 + rank)
    Hq, Hkv, D, B, S = 32, 8, 64, 2, 2048
    freq = pkg.rope_table.precompute_freqs_cis(D, S, **{k: v for k, v in inputs.ROPE_CONFIG4.items()}).to(dev)
    n_rot = 12  # 12 x (33.5 | 50 MB) > 126 MB L2
    if workload == "rmsnorm":
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
    ms_total, ms_max, regions = timed_regions(run_steps, args.steps, world, dev, sampler)
    sampler.stop()
    value = nbytes * world * args.steps / (ms_max * 1e-3) / 1e9
    peak, peak_kind = hbm_peak()
    achieved = nbytes / (ms_total / args.steps * 1e-3) / 1e9
    # What a plain pass over the SAME number of bytes reaches when it is timed the same way (torch's elementwise
    # kernel over rotating buffers, replayed from a graph): the measured peak is a 2 GB copy, and a launch of a few tens of MB
    # spends a fifth of its time ramping up and draining whatever it does.
    comparators = None
    if world == 1 and not args.no_comparator:
        half = nbytes // 4   # bf16 elements read (and as many written)
        src = [torch.empty(half, dtype=torch.bfloat16, device=dev).normal_() for _ in range(n_rot)]
        dst = [torch.empty_like(src[0]) for _ in range(n_rot)]
        # (an elementwise kernel: copy_ of same-dtype contiguous tensors becomes a driver memcpy, timed quite differently)
        cp_step = lambda i: torch.neg(src[i % n_rot], out=dst[i % n_rot])  # noqa: E731
        cp_run = eager_runner(cp_step) if args.no_graph else graph_runner(cp_step, n_rot, dev)
        cp_run.prepare(args.steps)
        cp_run(n_rot)
        _, cp_total, _ = timed_regions(cp_run, args.steps, 1, dev)
        cp_gbs = 4 * half / (cp_total / args.steps * 1e-3) / 1e9
        comparators = {"torch_elementwise_same_bytes": {"ms_per_step": cp_total / args.steps, "GB/s": cp_gbs,
                                                 "kernel_frac_of_this_copy": achieved / cp_gbs,
                                                 "call": "torch.neg(src, out=dst), bf16, read + write = the kernel's algorithmic bytes"}}
        del src, dst
    line = {
        "metric": "pre-attention HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "l2": f"{n_rot} rotating inputs and outputs > 126 MB L2", "bytes_per_step": nbytes,
                   "launch": ("each step is an eager extension call (with its output allocation)" if args.no_graph else
                              f"steps are replayed from a CUDA graph of {n_rot} extension calls back to back") + launch_kind(args)},
        "regions": regions,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": kernel, "algorithmic_bytes_per_launch": nbytes,
                     "frac_of_8TBs_nominal": achieved / 8000.0},
        "gpu_launches": args.steps, "clocks": sampler.summary(),
    }
    if comparators is not None:
        line["comparators"] = comparators
    return line


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
    ref_loop = None
    if world == 1 and not args.no_comparator:
        del model
        torch.cuda.empty_cache()
        try:
            ref_loop = time_reference_model_loop(pkg, dev, B, P, min(G, 512), prompts)
        except Exception as exc:   # optional evidence, never a reason to lose the bench line
            ref_loop = {"error": str(exc)[:300]}
    decode_steps = (G - 1) * steps
    # HBM bytes a generation cannot avoid: every decode step streams the weights once (16 layers + the tied head)
    # and the cached K and V of all sequences and layers; prefill, activations and the logits are left out
    D = cfg.head_dim
    weight_bytes = 2 * (cfg.n_layer * ((cfg.n_head + 2 * cfg.n_kv_head) * D * cfg.n_embd + cfg.n_embd * cfg.n_embd +
                                       3 * cfg.hidden_dim * cfg.n_embd) + cfg.vocab_size * cfg.n_embd)
    kv_bytes_per_token = 2 * 2 * cfg.n_kv_head * D * cfg.n_layer * B
    gen_bytes = (G - 1) * weight_bytes + kv_bytes_per_token * sum(P + t for t in range(1, G))
    peak, peak_kind = hbm_peak()
    achieved = gen_bytes * steps / (ms * 1e-3) / 1e9
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
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_kind": peak_kind, "kernel": "whole decode step (cuBLAS GEMMs + this library's kernels)",
                     "algorithmic_bytes_per_launch": gen_bytes // max(1, G - 1),
                     "note": "weights once per decode step + cached K/V of the step, averaged over the generation; the time "
                             "includes the prefill pass"},
        "launches_per_decode_step": {"this_library": 82, "detail": "33 RMSNorm (32 fused with the residual add), 16 SiLU*mul, 16 fused "
                                     "RoPE + cache write, 16 flash-decode, 1 greedy step; plus 81 cuBLAS GEMMs and the embedding lookup"},
        "e2e": e2e,
        # per decode step: 33 RMSNorm (32 with the residual add) + 16 SiLU*mul + 16 fused RoPE/cache + 16
        # flash-decode + 1 greedy-step launches of this library; the prefill pass has no flash-decode
        "gpu_launches": decode_steps * 82 + steps * 65, "clocks": sampler.summary(),
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if ref_loop is not None:
        line["comparators"] = {"reference_model_loop": ref_loop}
        try:
            line["comparators"]["sampling_step"] = time_sampling_step(ext, dev, B, cfg.vocab_size)
        except Exception as exc:
            line["comparators"]["sampling_step"] = {"error": str(exc)[:300]}
    return line


def time_sampling_step(ext, dev, B, vocab):
    """The token choice of one decode step over logits [B, vocab]: this library's greedy and nucleus-sampling kernels,
    and the reference's sampling branch as torch runs it (model.py:367-369 + sample_top_p, model.py:400-423:
    softmax, full sort, cumsum, mask, renormalise, multinomial, gather), each as eager calls with CUDA events."""
    logits = torch.randn(B, vocab, device=dev).bfloat16()
    out = torch.zeros(B, 4, dtype=torch.int64, device=dev)
    steps = torch.zeros(B, dtype=torch.int64, device=dev)
    cur = torch.zeros(B, dtype=torch.int64, device=dev)
    pos = torch.zeros(B, dtype=torch.int32, device=dev)
    lens = torch.zeros(B, dtype=torch.int32, device=dev)

    def reference_sampling():
        probs = torch.softmax(logits.float() / 0.6, dim=-1)
        ps, pi = torch.sort(probs, dim=-1, descending=True)
        mask = torch.cumsum(ps, dim=-1) - ps > 0.9
        ps[mask] = 0.0
        ps.div_(ps.sum(dim=-1, keepdim=True))
        return torch.gather(pi, -1, torch.multinomial(ps, num_samples=1))

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / n

    def reset_then(fn):
        def run():
            steps.zero_()
            fn()
        return run

    return {"batch": B, "vocab": vocab, "temperature": 0.6, "top_p": 0.9,
            "top_p_step_us": timed(reset_then(lambda: ext.top_p_step(logits, out, steps, cur, pos, lens, 0.6, 0.9, 1)), 50),
            "greedy_step_us": timed(reset_then(lambda: ext.greedy_step(logits, out, steps, cur, pos, lens)), 50),
            "torch_sample_top_p_us": timed(reference_sampling, 10)}


def time_reference_model_loop(pkg, dev, B, P, G, prompts):
    """The reference's own generation loop — its unmodified model.py (`LLaMA3.generate`, model.py:314-396; taken
    from baseline/_ref/, where build() puts it when the reference checkout is present) — running on THIS build of
    `custom_kernels_extension`, at the same architecture, batch and prompt length with random-init weights, greedy,
    ignore_eos.  Same kernels underneath; what differs is the loop around them: eager launches, two rot_embed calls
    and two cache copies per layer, unfused residual adds and SiLU, a host sync per token.  tokens/s by the
    reference's formula (benchmark_model.py:82) over a generation of G tokens."""
    import importlib.util
    import types

    ref_dir = Path(os.environ.get("L3CI_REFERENCE_DIR", REPO / "baseline" / "_ref"))
    if not (ref_dir / "model.py").exists():
        return {"unavailable": f"{ref_dir / 'model.py'} is absent (the reference checkout was not there at build time)"}
    pkg.extension()
    saved = sys.modules.get("transformers")
    stub = types.ModuleType("transformers")
    stub.AutoModelForCausalLM = stub.AutoTokenizer = None
    sys.modules["transformers"] = stub   # imported at model.py:21 for the checkpoint loader only
    try:
        spec = importlib.util.spec_from_file_location("l3ci_reference_model", ref_dir / "model.py")
        model_py = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(model_py)
    finally:
        if saved is not None:
            sys.modules["transformers"] = saved
        else:
            del sys.modules["transformers"]
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)   # as from_pretrained_llama3_hf builds it (model.py:282, 298-300)
    try:
        with torch.device(dev):
            m = model_py.LLaMA3(model_py.LlamaConfig(max_model_len=P + G, max_gen_batch_size=B)).eval()
    finally:
        torch.set_default_dtype(old)
    m.tokenizer = types.SimpleNamespace(pad_id=-1, stop_tokens=[128001, 128009])
    plist = prompts.tolist()
    m.generate(plist, 4, temperature=0, ignore_eos=True)   # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = m.generate(plist, G, temperature=0, ignore_eos=True)
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    del m
    torch.cuda.empty_cache()
    return {"tokens_per_s": G * B / sec, "seconds": sec, "generated_tokens_per_sequence": G, "batch": B, "prompt": P,
            "what": "unmodified reference model.py (LLaMA3.generate, temperature 0, ignore_eos) on this build of the extension; "
                    "shorter generation than the headline (shorter caches on average, which favours it)"}


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
