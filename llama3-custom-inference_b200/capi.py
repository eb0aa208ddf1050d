"""ctypes binding of the C ABI declared in include/l3ci_b200.h.

torch is used only to own device memory and to name the stream; every compute call below goes
`tensor.data_ptr()` -> `extern "C"` entry point of lib/libl3ci_b200.so.  The helpers mirror the
argument meaning of the reference's three extension functions (custom_kernels/main.cpp:2-8) so that
a test written against the reference reads the same here.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libl3ci_b200.so"

# l3ci_status
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_SCRATCH, ERR_CUDA, ERR_DEVICE_WAIT = range(7)

# Every symbol include/l3ci_b200.h declares.
EXPORTS = (
    "l3ci_status_string", "l3ci_last_error", "l3ci_version", "l3ci_set_device_wait_limit_ns", "l3ci_set_programmatic_launch",
    "l3ci_rms_norm", "l3ci_add_rms_norm", "l3ci_silu_mul", "l3ci_greedy_step", "l3ci_top_p_step", "l3ci_rot_embed", "l3ci_rot_embed_kv_cache", "l3ci_rot_embed_kv_cache_at",
    "l3ci_flash_decode_scratch_bytes", "l3ci_flash_decode", "l3ci_flash_decode_static", "l3ci_flash_decode_poll",
    "l3ci_flash_decode_kernel_choice",
    "l3ci_lse_merge", "l3ci_lse_exchange_bytes", "l3ci_lse_exchange_merge", "l3ci_prefill_attention",
    "l3ci_flash_decode_exchange_bytes", "l3ci_flash_decode_exchange",
)


class FlashDecodeArgs(C.Structure):
    """struct l3ci_flash_decode_args"""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("o_partial", C.c_void_p), ("lse", C.c_void_p), ("seq_lens", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("n_seq", C.c_int32),
        ("q_sb", C.c_int64), ("q_sh", C.c_int64),
        ("k_sb", C.c_int64), ("k_sh", C.c_int64), ("k_st", C.c_int64),
        ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("v_st", C.c_int64),
        ("o_sb", C.c_int64), ("o_sh", C.c_int64),
        ("scale", C.c_float), ("max_ctas", C.c_int32), ("stream", C.c_void_p),
    ]


class PrefillArgs(C.Structure):
    """struct l3ci_prefill_args"""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("T", C.c_int32), ("n_keys", C.c_int32), ("start_pos", C.c_int32),
        ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("q_st", C.c_int64),
        ("k_sb", C.c_int64), ("k_sh", C.c_int64), ("k_st", C.c_int64),
        ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("v_st", C.c_int64),
        ("o_sb", C.c_int64), ("o_sh", C.c_int64), ("o_st", C.c_int64),
        ("scale", C.c_float), ("variant", C.c_int32), ("stream", C.c_void_p),
    ]


class L3ciError(RuntimeError):
    """A C-ABI call returned a status other than L3CI_OK."""

    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"{what}: status {status} ({detail})")
        self.status = status


_lib = None


def load() -> C.CDLL:
    """Loads lib/libl3ci_b200.so once and declares the prototypes.  Raises OSError if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise OSError(f"{LIB_PATH} is missing: run build.py in this directory; there is no fallback")
    lib = C.CDLL(str(LIB_PATH))
    i64, i32, vp, f32 = C.c_int64, C.c_int32, C.c_void_p, C.c_float
    lib.l3ci_status_string.restype = C.c_char_p
    lib.l3ci_status_string.argtypes = [C.c_int]
    lib.l3ci_last_error.restype = C.c_char_p
    lib.l3ci_last_error.argtypes = []
    lib.l3ci_version.restype = C.c_char_p
    lib.l3ci_version.argtypes = []
    lib.l3ci_set_programmatic_launch.restype = C.c_int
    lib.l3ci_set_programmatic_launch.argtypes = [C.c_int]
    lib.l3ci_set_device_wait_limit_ns.restype = C.c_uint64
    lib.l3ci_set_device_wait_limit_ns.argtypes = [C.c_uint64]
    lib.l3ci_rms_norm.restype = C.c_int
    lib.l3ci_rms_norm.argtypes = [vp, vp, vp, i64, i64, i64, i64, f32, vp]
    lib.l3ci_add_rms_norm.restype = C.c_int
    lib.l3ci_add_rms_norm.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, vp]
    lib.l3ci_silu_mul.restype = C.c_int
    lib.l3ci_silu_mul.argtypes = [vp, vp, vp, i64, i64, i64, i64, vp]
    lib.l3ci_prefill_attention.restype = C.c_int
    lib.l3ci_prefill_attention.argtypes = [C.POINTER(PrefillArgs)]
    lib.l3ci_greedy_step.restype = C.c_int
    lib.l3ci_greedy_step.argtypes = [vp, i64, i64, i64, vp, i64, i64, vp, vp, vp, vp, vp]
    lib.l3ci_top_p_step.restype = C.c_int
    lib.l3ci_top_p_step.argtypes = [vp, i64, i64, i64, f32, f32, C.c_uint64, vp, i64, i64, vp, vp, vp, vp, vp, vp, vp]
    lib.l3ci_rot_embed.restype = C.c_int
    lib.l3ci_rot_embed.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp]
    lib.l3ci_rot_embed_kv_cache.restype = C.c_int
    lib.l3ci_rot_embed_kv_cache.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64, vp]
    lib.l3ci_rot_embed_kv_cache_at.restype = C.c_int
    lib.l3ci_rot_embed_kv_cache_at.argtypes = [vp, vp, i64, vp, vp, vp, vp] + [i64] * 10 + [vp]
    lib.l3ci_flash_decode_scratch_bytes.restype = C.c_size_t
    lib.l3ci_flash_decode_scratch_bytes.argtypes = [i32, i32, i32, i32]
    lib.l3ci_flash_decode_kernel_choice.restype = C.c_int
    lib.l3ci_flash_decode_kernel_choice.argtypes = [i32, i32, i32, i32, i32, i32]
    lib.l3ci_flash_decode.restype = C.c_int
    lib.l3ci_flash_decode.argtypes = [C.POINTER(FlashDecodeArgs)]
    lib.l3ci_flash_decode_static.restype = C.c_int
    lib.l3ci_flash_decode_static.argtypes = [C.POINTER(FlashDecodeArgs)]
    lib.l3ci_flash_decode_poll.restype = C.c_int
    lib.l3ci_flash_decode_poll.argtypes = [vp, C.c_size_t, vp]
    lib.l3ci_lse_merge.restype = C.c_int
    lib.l3ci_lse_merge.argtypes = [vp, vp, vp, i32, i32, i32, i32, i64, i64, vp]
    lib.l3ci_lse_exchange_bytes.restype = C.c_size_t
    lib.l3ci_lse_exchange_bytes.argtypes = [i32, i32, i32, i32]
    lib.l3ci_lse_exchange_merge.restype = C.c_int
    lib.l3ci_lse_exchange_merge.argtypes = [vp, i32, i32, C.c_uint32, vp, i32, i32, i32, i64, i64, vp, vp]
    lib.l3ci_flash_decode_exchange_bytes.restype = C.c_size_t
    lib.l3ci_flash_decode_exchange_bytes.argtypes = [i32, i32, i32, i32]
    lib.l3ci_flash_decode_exchange.restype = C.c_int
    lib.l3ci_flash_decode_exchange.argtypes = [C.POINTER(FlashDecodeArgs), vp, i32, i32, C.c_uint32, vp]
    _lib = lib
    return lib


def _check(status: int, what: str) -> None:
    if status != OK:
        raise L3ciError(status, what, load().l3ci_last_error().decode())


def _stream(t) -> int:
    import torch

    return torch.cuda.current_stream(t.device).cuda_stream


def _on(t):
    import torch

    return torch.cuda.device(t.device)


# ---- reference-shaped helpers over torch CUDA tensors -------------------------------------------------


def rms_norm(x, weight, eps: float):
    """`rms_norm(input, weight, eps)` (custom_kernels/custom_kernels.cu:369-389): input [..., E] contiguous."""
    import torch

    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    out = torch.empty_like(x)
    E = x.shape[-1]
    rows = x.numel() // E if E else 0
    with _on(x):
        _check(load().l3ci_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, E, E, E, eps, _stream(x)),
               "l3ci_rms_norm")
    return out


def add_rms_norm(x, residual, weight, eps: float):
    """Returns (bf16(x + residual), rmsnorm of that sum * weight); dense [..., E] tensors."""
    import torch

    assert x.is_contiguous() and residual.is_contiguous() and x.shape == residual.shape
    s, out = torch.empty_like(x), torch.empty_like(x)
    E = x.shape[-1]
    with _on(x):
        _check(load().l3ci_add_rms_norm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), s.data_ptr(),
                                        out.data_ptr(), x.numel() // E, E, eps, _stream(x)), "l3ci_add_rms_norm")
    return s, out


def silu_mul(gate, up):
    """bf16(bf16(silu(gate)) * up) for 2-D tensors of equal shape whose rows are contiguous."""
    import torch

    assert gate.dim() == 2 and gate.shape == up.shape and gate.stride(1) == 1 and up.stride(1) == 1
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    with _on(gate):
        _check(load().l3ci_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.shape[0], gate.shape[1],
                                    gate.stride(0), up.stride(0), _stream(gate)), "l3ci_silu_mul")
    return out


def greedy_step(logits, out_tokens=None, steps=None, next_input=None, positions=None, seq_lens=None):
    """argmax of every row of bf16 logits [B, vocab] plus the decode bookkeeping, in place (see l3ci_greedy_step)."""
    assert logits.dim() == 2 and logits.stride(1) == 1
    ptr = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    with _on(logits):
        _check(load().l3ci_greedy_step(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0),
                                       ptr(out_tokens), out_tokens.stride(0) if out_tokens is not None else 0,
                                       out_tokens.shape[1] if out_tokens is not None and out_tokens.dim() == 2 else 1,
                                       ptr(steps), ptr(next_input), ptr(positions), ptr(seq_lens), _stream(logits)),
               "l3ci_greedy_step")


def top_p_step(logits, temperature: float, top_p: float, seed: int, out_tokens=None, steps=None, next_input=None,
               positions=None, seq_lens=None, nucleus_count=None, nucleus_mass=None):
    """One nucleus-sampling step over bf16 logits [B, vocab] plus the decode bookkeeping, in place (l3ci_top_p_step)."""
    assert logits.dim() == 2 and logits.stride(1) == 1
    ptr = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    with _on(logits):
        _check(load().l3ci_top_p_step(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0), temperature,
                                      top_p, seed, ptr(out_tokens), out_tokens.stride(0) if out_tokens is not None else 0,
                                      out_tokens.shape[1] if out_tokens is not None and out_tokens.dim() == 2 else 1,
                                      ptr(steps), ptr(next_input), ptr(positions), ptr(seq_lens), ptr(nucleus_count),
                                      ptr(nucleus_mass), _stream(logits)), "l3ci_top_p_step")


def rot_embed(x, freq):
    """`rot_embed(input, freq)` (custom_kernels/custom_kernels.cu:418-442): input [B,S,H,D] view, dense output."""
    import torch

    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.stride(3) == 1
    assert freq.dtype == torch.float32 and freq.is_contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    B, S, H, D = x.shape
    with _on(x):
        _check(load().l3ci_rot_embed(x.data_ptr(), freq.data_ptr(), out.data_ptr(), B, S, H, D, x.stride(0),
                                     x.stride(1), x.stride(2), _stream(x)), "l3ci_rot_embed")
    return out


def rot_embed_kv_cache(qkv, freq, cache_k, cache_v, start_pos: int, n_head: int, n_kv_head: int):
    """Fused form of model.py:100-108: returns rotated q [B,T,n_head,D], updates the caches in place."""
    import torch

    B, T, W = qkv.shape
    D = W // (n_head + 2 * n_kv_head)
    q_out = torch.empty((B, T, n_head, D), dtype=qkv.dtype, device=qkv.device)
    with _on(qkv):
        _check(load().l3ci_rot_embed_kv_cache(qkv.data_ptr(), freq.data_ptr(), q_out.data_ptr(), cache_k.data_ptr(),
                                              cache_v.data_ptr(), B, T, n_head, n_kv_head, D, qkv.stride(0),
                                              qkv.stride(1), cache_k.stride(0), cache_k.stride(1), start_pos,
                                              _stream(qkv)), "l3ci_rot_embed_kv_cache")
    return q_out


def rot_embed_kv_cache_at(qkv, freq_table, cache_k, cache_v, positions, n_head: int, n_kv_head: int):
    """Like `rot_embed_kv_cache`, with per-sequence positions (int32 [B] on the device) and the whole table."""
    import torch

    B, T, W = qkv.shape
    D = W // (n_head + 2 * n_kv_head)
    q_out = torch.empty((B, T, n_head, D), dtype=qkv.dtype, device=qkv.device)
    with _on(qkv):
        _check(load().l3ci_rot_embed_kv_cache_at(qkv.data_ptr(), freq_table.data_ptr(), freq_table.shape[0],
                                                 q_out.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                                                 positions.data_ptr(), B, T, n_head, n_kv_head, D, qkv.stride(0),
                                                 qkv.stride(1), cache_k.stride(0), cache_k.stride(1), cache_k.shape[1],
                                                 _stream(qkv)), "l3ci_rot_embed_kv_cache_at")
    return q_out


class DecodeScratch:
    """Zero-filled scratch of l3ci_flash_decode for one device; reusable across calls on one stream."""

    def __init__(self, B: int, Hq: int, Hkv: int, D: int, device):
        import torch

        with torch.cuda.device(device):
            self.bytes = int(load().l3ci_flash_decode_scratch_bytes(B, Hq, Hkv, D))
        if self.bytes == 0:
            raise L3ciError(ERR_INVALID, "l3ci_flash_decode_scratch_bytes", f"B={B} Hq={Hq} Hkv={Hkv} D={D}")
        self.buf = torch.zeros(self.bytes, dtype=torch.uint8, device=device)

    def poll(self) -> int:
        """Synchronises and returns the device-side status word (0 = fine)."""
        with _on(self.buf):
            return int(load().l3ci_flash_decode_poll(self.buf.data_ptr(), self.bytes, _stream(self.buf)))


def flash_decode_args(q, k, v, out=None, o_partial=None, lse=None, seq_lens=None, scratch: Optional[DecodeScratch] = None,
                      scale: float = 0.0, max_ctas: int = 0) -> FlashDecodeArgs:
    """Fills struct l3ci_flash_decode_args from [B,H,T,D]-shaped torch views (strides in elements)."""
    a = FlashDecodeArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.out = out.data_ptr() if out is not None else None
    a.o_partial = o_partial.data_ptr() if o_partial is not None else None
    a.lse = lse.data_ptr() if lse is not None else None
    a.seq_lens = seq_lens.data_ptr() if seq_lens is not None else None
    a.scratch = scratch.buf.data_ptr() if scratch is not None else None
    a.scratch_bytes = scratch.bytes if scratch is not None else 0
    a.B, a.Hq, a.Hkv, a.D, a.n_seq = q.shape[0], q.shape[1], k.shape[1], q.shape[3], k.shape[2]
    a.q_sb, a.q_sh = q.stride(0), q.stride(1)
    a.k_sb, a.k_sh, a.k_st = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_sh, a.v_st = v.stride(0), v.stride(1), v.stride(2)
    if out is not None:
        a.o_sb, a.o_sh = out.stride(0), out.stride(1)
    a.scale = scale
    a.max_ctas = max_ctas
    a.stream = _stream(q)
    return a


def flash_attention_decode(q, k, v, seq_lens=None, scratch: Optional[DecodeScratch] = None, scale: float = 0.0,
                           max_ctas: int = 0):
    """`flash_attention_decode(query, keys, values)` (custom_kernels/custom_kernels.cu:233-338).

    q [B,Hq,1,D], k/v [B,Hkv,S,D] (any strides with a contiguous last dimension); returns bf16 shaped and
    laid out like q.  `seq_lens` (int32 [B] on the device) is this library's addition for ragged batches.
    """
    import torch

    out = torch.empty_like(q)
    if scratch is None:
        scratch = DecodeScratch(q.shape[0], q.shape[1], k.shape[1], q.shape[3], q.device)
    a = flash_decode_args(q, k, v, out=out, seq_lens=seq_lens, scratch=scratch, scale=scale, max_ctas=max_ctas)
    with _on(q):
        _check(load().l3ci_flash_decode(C.byref(a)), "l3ci_flash_decode")
    return out


def flash_attention_decode_partial(q, k, v, seq_lens=None, scratch: Optional[DecodeScratch] = None,
                                   scale: float = 0.0, max_ctas: int = 0):
    """Attention over one KV shard as fp32 (o [B,Hq,D], lse [B,Hq]) for `lse_merge`."""
    import torch

    B, Hq, _, D = q.shape
    o = torch.empty((B, Hq, D), dtype=torch.float32, device=q.device)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    if scratch is None:
        scratch = DecodeScratch(B, Hq, k.shape[1], D, q.device)
    a = flash_decode_args(q, k, v, o_partial=o, lse=lse, seq_lens=seq_lens, scratch=scratch, scale=scale,
                          max_ctas=max_ctas)
    with _on(q):
        _check(load().l3ci_flash_decode(C.byref(a)), "l3ci_flash_decode")
    return o, lse


def prefill_attention(q, k, v, start_pos: int = 0, scale: float = 0.0, status=None, variant: int = 0):
    """Causal GQA attention of q [B,Hq,T,D] over k, v [B,Hkv,S,D]: query t sees keys j <= start_pos + t.  Returns a
    bf16 tensor laid out like q."""
    import torch

    B, Hq, T, D = q.shape
    out = torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device)
    a = PrefillArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.status = status.data_ptr() if status is not None else None
    a.B, a.Hq, a.Hkv, a.D, a.T, a.n_keys, a.start_pos = B, Hq, k.shape[1], D, T, k.shape[2], start_pos
    a.q_sb, a.q_sh, a.q_st = q.stride(0), q.stride(1), q.stride(2)
    a.k_sb, a.k_sh, a.k_st = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_sh, a.v_st = v.stride(0), v.stride(1), v.stride(2)
    a.o_sb, a.o_sh, a.o_st = out.stride(0), out.stride(1), out.stride(2)
    a.scale, a.variant, a.stream = scale, variant, _stream(q)
    with _on(q):
        _check(load().l3ci_prefill_attention(C.byref(a)), "l3ci_prefill_attention")
    return out


def lse_merge(o_parts, lse_parts):
    """Merges fp32 shard results o_parts [P,B,Hq,D], lse_parts [P,B,Hq] into bf16 [B,Hq,1,D]."""
    import torch

    P, B, Hq, D = o_parts.shape
    out = torch.empty((B, 1, Hq, D), dtype=torch.bfloat16, device=o_parts.device).transpose(1, 2)
    with _on(o_parts):
        _check(load().l3ci_lse_merge(o_parts.data_ptr(), lse_parts.data_ptr(), out.data_ptr(), P, B, Hq, D,
                                     out.stride(0), out.stride(1), _stream(o_parts)), "l3ci_lse_merge")
    return out


STATIC_SCRATCH_BYTES = 12 << 20  # L3CI_STATIC_SCRATCH_BYTES


def flash_attention_decode_static(q, k, v, seq_lens=None, scale: float = 0.0, max_ctas: int = 0):
    """`flash_attention_decode` for callers that cannot allocate device memory: the merge scratch is the
    library's built-in array (one per GPU, shared by every call on it; do not overlap calls).  The output
    tensor is still created here because this helper mirrors the reference call form; a caller that owns
    its output buffer fills `FlashDecodeArgs.out` itself and calls `l3ci_flash_decode_static` directly."""
    import torch

    out = torch.empty_like(q)
    a = flash_decode_args(q, k, v, out=out, seq_lens=seq_lens, scale=scale, max_ctas=max_ctas)
    with _on(q):
        _check(load().l3ci_flash_decode_static(C.byref(a)), "l3ci_flash_decode_static")
    return out


class device_wait_limit:
    """Context manager: device-side waits on other CTAs / GPUs of launches made inside give up after `ns`
    nanoseconds (l3ci_set_device_wait_limit_ns); the previous setting comes back on exit."""

    def __init__(self, ns: int):
        self.ns = ns

    def __enter__(self):
        self.prev = load().l3ci_set_device_wait_limit_ns(self.ns)
        return self

    def __exit__(self, *exc):
        load().l3ci_set_device_wait_limit_ns(self.prev)
        return False


class programmatic_launch:
    """Context manager: launches made inside use (True) or do not use (False) programmatic dependent launch
    (l3ci_set_programmatic_launch); the previous setting comes back on exit.  A CUDA graph keeps the kind of launch
    it was captured with."""

    def __init__(self, on: bool):
        self.on = bool(on)

    def __enter__(self):
        self.prev = load().l3ci_set_programmatic_launch(int(self.on))
        return self

    def __exit__(self, *exc):
        load().l3ci_set_programmatic_launch(self.prev)
        return False


def lse_exchange_merge(bufs, rank: int, ranks: int, epoch: int, out, B: int, Hq: int, D: int, status=None):
    """`l3ci_lse_exchange_merge` over a device int64 tensor of `ranks` buffer addresses; `out` is bf16 [B,Hq,1,D]
    (any strides over b and h), `status` an optional int32 device word."""
    with _on(out):
        _check(load().l3ci_lse_exchange_merge(bufs.data_ptr(), rank, ranks, epoch, out.data_ptr(), B, Hq, D,
                                              out.stride(0), out.stride(1),
                                              status.data_ptr() if status is not None else None, _stream(out)),
               "l3ci_lse_exchange_merge")
    return out


def flash_decode_exchange(q, k, v, bufs, rank: int, ranks: int, epoch: int = 0, out=None, seq_lens=None, status=None,
                          scale: float = 0.0, max_ctas: int = 0):
    """`l3ci_flash_decode_exchange`: attention of q over this rank's slice k, v of a sequence-sharded cache, merged
    with the other ranks' results in the same launch.  `bufs`: device int64 tensor of the ranks' exchange buffers."""
    import torch

    if out is None:
        out = torch.empty_like(q)
    a = flash_decode_args(q, k, v, out=out, seq_lens=seq_lens, scale=scale, max_ctas=max_ctas)
    with _on(q):
        _check(load().l3ci_flash_decode_exchange(C.byref(a), bufs.data_ptr(), rank, ranks, epoch,
                                                 status.data_ptr() if status is not None else None),
               "l3ci_flash_decode_exchange")
    return out
