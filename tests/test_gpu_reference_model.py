"""The reference's own model code (model.py, unmodified) running on this build of `custom_kernels_extension`.

model.py imports the extension as `from custom_kernels import custom_kernels_extension` (model.py:23) and calls its
three functions from RMSNorm.forward (model.py:71) and CausalSelfAttention.forward (model.py:100-101, 118).  With
this package's directory on sys.path that import resolves to the sm_100a build, and nothing in model.py changes.
The file is taken from baseline/_ref/ (where `__graft_entry__.build()` puts it when the reference checkout is
present) or from the directory named by L3CI_REFERENCE_DIR; without it the tests are skipped.

Checked: `forward` with T > 1 and T == 1 and greedy `generate` of a small random-init LLaMA3 against the CPU
restatement of the same layers (oracle/decode_loop.py) on the same weights.
"""
import importlib.util
import os
import sys
import types
from pathlib import Path

import pytest
import torch

from conftest import REPO
from oracle.decode_loop import CpuDecoder

pytestmark = pytest.mark.gpu
REF_DIR = Path(os.environ.get("L3CI_REFERENCE_DIR", REPO / "baseline" / "_ref"))


def import_reference_model(pkg):
    """The reference's model.py as a module; `transformers` (imported at model.py:21 for the checkpoint loader only)
    is replaced by a stub while it loads."""
    if "l3ci_reference_model" in sys.modules:
        return sys.modules["l3ci_reference_model"]
    pkg.extension()   # puts the package directory on sys.path: `custom_kernels` resolves to this build
    saved = sys.modules.get("transformers")
    stub = types.ModuleType("transformers")
    stub.AutoModelForCausalLM = stub.AutoTokenizer = None
    sys.modules["transformers"] = stub
    try:
        spec = importlib.util.spec_from_file_location("l3ci_reference_model", REF_DIR / "model.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        if saved is not None:
            sys.modules["transformers"] = saved
        else:
            del sys.modules["transformers"]
    sys.modules["l3ci_reference_model"] = mod
    return mod


def build_reference_model(model_py, cfg_kwargs, weights, device):
    """LLaMA3(LlamaConfig(...)) constructed the way from_pretrained_llama3_hf does (model.py:282, 298-300: default
    dtype bf16, default device cuda), then loaded with `weights` (names of decode_loop.init_weights)."""
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            m = model_py.LLaMA3(model_py.LlamaConfig(**cfg_kwargs))
    finally:
        torch.set_default_dtype(old)
    sd = {"transformer.wte.weight": weights["wte"], "transformer.ln_f.weight": weights["ln_f"]}
    names = {"ln_1": "ln_1.weight", "attn": "attn.c_attn.weight", "proj": "attn.c_proj.weight", "ln_2": "ln_2.weight",
             "fc": "mlp.c_fc.weight", "fc2": "mlp.c_fc2.weight", "mlp_proj": "mlp.c_proj.weight"}
    for l in range(cfg_kwargs["n_layer"]):
        for ours, theirs in names.items():
            sd[f"transformer.h.{l}.{theirs}"] = weights[f"h{l}.{ours}"]
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not unexpected and all(k == "lm_head.weight" or "cache_" in k or k == "freqs_cis" for k in missing), (missing, unexpected)
    m.tokenizer = types.SimpleNamespace(pad_id=0, stop_tokens=[cfg_kwargs["vocab_size"] - 1])   # model.py:349, 361
    return m.eval()


@pytest.fixture(scope="module")
def setup(pkg, ext, device):
    if not (REF_DIR / "model.py").exists():
        pytest.skip(f"{REF_DIR / 'model.py'} is absent (the reference checkout was not there at build time)")
    model_py = import_reference_model(pkg)
    assert model_py.custom_kernels_extension is ext   # the reference's import found this build
    cfg_kwargs = dict(vocab_size=1000, n_layer=3, n_head=8, n_kv_head=2, n_embd=512, hidden_dim=1024, max_model_len=64,
                      max_gen_batch_size=4)
    # the reference hard-codes the rotary scaling factor 8 (model.py:29)
    cfg = pkg.decode_loop.DecoderConfig(vocab_size=1000, n_layer=3, n_head=8, n_kv_head=2, n_embd=512, hidden_dim=1024,
                                        rope_scale_factor=8.0)
    weights = pkg.decode_loop.init_weights(cfg, seed=5)
    return model_py, build_reference_model(model_py, cfg_kwargs, weights, device), cfg, weights


def test_forward_prefill_then_decode_step(setup, device):
    model_py, m, cfg, weights = setup
    B, P = 3, 20
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    cpu = CpuDecoder(cfg, weights, B, 64)
    with torch.inference_mode():
        logits, _ = m.forward(prompts.to(device), start_pos=0)                       # T > 1: model.py:114-116
        want = cpu.forward(prompts, 0, return_logits=True)
        assert logits.shape == (B, 1, cfg.vocab_size) and logits.dtype == torch.float32
        scale = want.abs().max().item()
        assert (logits[:, 0].cpu() - want).abs().max().item() < 0.05 * scale + 0.02
        nxt = want.argmax(-1, keepdim=True)
        logits, _ = m.forward(nxt.to(device), start_pos=P)                          # T == 1: the decode kernel
        want = cpu.forward(nxt, P, return_logits=True)
        assert (logits[:, 0].cpu() - want).abs().max().item() < 0.05 * scale + 0.02
    torch.cuda.synchronize()
    # the KV cache the reference's module wrote through rot_embed matches the restatement's
    ck = m.transformer.h[0].attn.cache_k[:B, :P + 1].float().cpu()
    assert (ck - cpu.cache_k[0][:B, :P + 1].float()).abs().max().item() < 0.1


def test_greedy_generate_tracks_the_cpu_loop(setup, device, ext):
    model_py, m, cfg, weights = setup
    B, P, G = 3, 20, 12
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(1, cfg.vocab_size - 1, (B, P), generator=g)
    out = m.generate(prompts.tolist(), G, temperature=0, ignore_eos=True)            # model.py:314-396
    torch.cuda.synchronize()
    assert ext.flash_decode_status(torch.zeros(1, device=device)) == 0
    toks = torch.tensor([o + [0] * (G - len(o)) for o in out])   # (cut after a stop token, if one was drawn)
    cpu = CpuDecoder(cfg, weights, B, 64)
    logits = cpu.forward(prompts, 0, return_logits=True)
    checked = 0
    for i in range(G):
        if any(len(o) <= i for o in out):
            break
        top2 = logits.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 0.05
        assert torch.equal(logits.argmax(-1)[clear], toks[clear, i])
        checked += int(clear.sum())
        if i + 1 < G:
            logits = cpu.forward(toks[:, i:i + 1], P + i, return_logits=True)
    assert checked >= B * G // 2
