"""The Hugging Face weight mapping (`decode_loop.weights_from_hf`, `config_from_hf`: the reference's
`adapt_llama_state_dict_keys_hf`, model.py:235-280) checked on the CPU: the CPU restatement of the decode loop on the
mapped weights against the Hugging Face implementation of the same architecture (rotate-half rotary embedding on
permuted weights there, adjacent pairs on un-permuted weights here)."""
import pytest
import torch

from oracle.decode_loop import CpuDecoder

transformers = pytest.importorskip("transformers")


@pytest.mark.parametrize("tie,factor", [(True, 32.0), (False, 8.0)])
def test_mapped_weights_give_the_hf_models_logits(pkg, tie, factor):
    cfg_hf = transformers.LlamaConfig(
        vocab_size=300, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0,
        rope_scaling={"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 8192},
        tie_word_embeddings=tie, attention_bias=False)
    torch.manual_seed(4)
    model = transformers.LlamaForCausalLM(cfg_hf).eval()
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() == 1:
                prm.add_(0.1 * torch.randn_like(prm))
            prm.copy_(prm.to(torch.bfloat16).float())
    cfg = pkg.decode_loop.config_from_hf(model.config)
    assert cfg.head_dim == 64 and cfg.rope_scale_factor == factor and cfg.rope_scaled
    weights = pkg.decode_loop.weights_from_hf(model.state_dict(), cfg)
    assert ("lm_head" in weights) == (not tie)
    B, T = 2, 12
    tokens = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=torch.Generator().manual_seed(1))
    cpu = CpuDecoder(cfg, weights, B, 32)
    ours = cpu.forward(tokens[:, :T], 0, return_logits=True)
    ours_next = cpu.forward(tokens[:, T:], T, return_logits=True)        # one decode step on the cache
    with torch.no_grad():
        ref = model(tokens).logits.float()
    # bf16 activations on our side, fp32 on the other: a few hundredths on logits of order one
    assert (ours - ref[:, T - 1]).abs().max().item() < 0.08
    assert (ours_next - ref[:, T]).abs().max().item() < 0.08
    # and the mapping matters: without the un-permutation the logits are far off
    broken = dict(weights)
    broken["h0.attn"] = torch.cat([model.state_dict()["model.layers.0.self_attn.q_proj.weight"].bfloat16(),
                                   weights["h0.attn"][cfg.n_head * cfg.head_dim:]], dim=0)
    off = CpuDecoder(cfg, broken, B, 32).forward(tokens[:, :T], 0, return_logits=True)
    assert (off - ref[:, T - 1]).abs().max().item() > 0.08
