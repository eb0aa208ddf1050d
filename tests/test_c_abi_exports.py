"""The C-ABI library loads without a GPU, exports every symbol the header declares, and rejects bad
arguments before touching CUDA.  CPU only (no compute calls)."""
import ctypes as C
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (REPO / "include" / "l3ci_b200.h").read_text()
    return sorted(set(re.findall(r"L3CI_API\s+[\w\s\*]+?\b(l3ci_\w+)\s*\(", text)))


def test_header_and_binding_agree(capi):
    assert _declared_symbols() == sorted(capi.EXPORTS)


def test_library_exports_every_declared_symbol(capi):
    lib = capi.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_status_strings(capi):
    lib = capi.load()
    assert re.fullmatch(r"\d+\.\d+\.\d+", lib.l3ci_version().decode())
    assert lib.l3ci_status_string(capi.OK) == b"ok"
    texts = {lib.l3ci_status_string(i) for i in range(7)}
    assert len(texts) == 7 and lib.l3ci_status_string(99) == b"unknown status"


def test_struct_layout_matches_header(capi):
    # 8 pointers + size_t, 5 int32 (+4 pad), 10 int64, float + int32, pointer
    assert C.sizeof(capi.FlashDecodeArgs) == 9 * 8 + 24 + 10 * 8 + 8 + 8
    assert capi.FlashDecodeArgs.q_sb.offset == 96 and capi.FlashDecodeArgs.stream.offset == 184


def test_argument_validation_happens_before_cuda(capi):
    lib = capi.load()
    fake = C.c_void_p(0x1000)  # never dereferenced: validation fails first
    assert lib.l3ci_rms_norm(fake, fake, fake, 4, 7, 7, 7, 1e-5, None) == capi.ERR_UNSUPPORTED
    assert b"multiple of 8" in lib.l3ci_last_error()
    assert lib.l3ci_rms_norm(None, fake, fake, 4, 8, 8, 8, 1e-5, None) == capi.ERR_INVALID
    assert lib.l3ci_rms_norm(C.c_void_p(0x1002), fake, fake, 4, 8, 8, 8, 1e-5, None) == capi.ERR_ALIGNMENT
    assert lib.l3ci_rms_norm(fake, fake, fake, 0, 8, 8, 8, 1e-5, None) == capi.OK  # nothing to do
    assert lib.l3ci_rot_embed(fake, fake, fake, 1, 1, 1, 63, 63, 63, 63, None) == capi.ERR_UNSUPPORTED
    assert lib.l3ci_rot_embed(fake, fake, fake, 0, 1, 1, 64, 64, 64, 64, None) == capi.OK
    assert lib.l3ci_rot_embed_kv_cache(fake, fake, fake, fake, fake, 1, 1, 4, 2, 64, 512, 512, 1024, 128, -1, None) == capi.ERR_INVALID
    assert lib.l3ci_lse_merge(fake, fake, fake, 0, 1, 1, 64, 64, 64, None) == capi.ERR_INVALID

    a = capi.FlashDecodeArgs()
    a.q = a.k = a.v = a.out = 0x1000
    a.B, a.Hq, a.Hkv, a.D, a.n_seq = 1, 32, 8, 96, 16
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_UNSUPPORTED
    assert b"Unsupported head size" in lib.l3ci_last_error()
    a.D, a.Hq, a.Hkv = 128, 34, 2
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_UNSUPPORTED  # ratio 17
    assert b"Unsupported QKV head ratio" in lib.l3ci_last_error()
    a.Hq, a.Hkv = 32, 5
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.ERR_INVALID
    a.Hkv, a.B = 8, 0
    assert lib.l3ci_flash_decode(C.byref(a)) == capi.OK  # empty batch
    assert lib.l3ci_flash_decode(None) == capi.ERR_INVALID
    assert lib.l3ci_flash_decode_scratch_bytes(1, 32, 5, 128) == 0
    # sizes the call would refuse: no kernel is chosen
    for bad in ((1, 32, 5, 128, 16, 0), (1, 32, 8, 96, 16, 0), (0, 32, 8, 128, 16, 0), (1, 32, 8, 128, 0, 1)):
        assert lib.l3ci_flash_decode_kernel_choice(*bad) == -1


def test_extension_module_mirrors_reference_binding(ext):
    import torch

    # the three names bound at custom_kernels/main.cpp:6-8, plus the additive ones
    for name in ("flash_attention_decode", "rms_norm", "rot_embed"):
        assert callable(getattr(ext, name))
    for name in ("rot_embed_kv_cache", "flash_attention_decode_partial", "lse_merge", "flash_decode_status"):
        assert callable(getattr(ext, name))
    assert ext.c_abi_version() == "0.2.0"
    x = torch.zeros(1, 2, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):  # no CPU fallback: CPU tensors are refused
        ext.rms_norm(x, torch.ones(8, dtype=torch.bfloat16), 1e-5)
    q = torch.zeros(1, 4, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ext.flash_attention_decode(q, q, q)
    with pytest.raises(RuntimeError):
        ext.rot_embed(torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16), torch.zeros(1, 64))


def test_device_wait_limit_setter_round_trips(capi):
    lib = capi.load()
    prev = lib.l3ci_set_device_wait_limit_ns(123)
    assert lib.l3ci_set_device_wait_limit_ns(prev) == 123
    assert lib.l3ci_set_device_wait_limit_ns(prev) == prev


def test_programmatic_launch_switch_round_trips(capi):
    lib = capi.load()
    prev = lib.l3ci_set_programmatic_launch(0)
    assert prev in (0, 1)
    assert lib.l3ci_set_programmatic_launch(1) == 0
    assert lib.l3ci_set_programmatic_launch(7) == 1       # any non-zero value means on
    assert lib.l3ci_set_programmatic_launch(prev) == 1
    with capi.programmatic_launch(False):
        assert lib.l3ci_set_programmatic_launch(0) == 0
    assert lib.l3ci_set_programmatic_launch(prev) == prev
