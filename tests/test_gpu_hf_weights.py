"""Weights in the Hugging Face Llama layout through `weights_from_hf` / `config_from_hf` (the reference's
`adapt_llama_state_dict_keys_hf`, model.py:235-280): the decode loop on the extension kernels against the Hugging
Face implementation of the same architecture, an independent restatement of everything on the path (RMSNorm, rotary
embedding in its rotate-half form with the Llama-3 frequency scaling, GQA attention, the MLP).

No checkpoint is needed: the "checkpoint" is a small randomly initialised `LlamaForCausalLM`, evaluated in fp32 on
the CPU with its weights rounded to bf16."""
import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _hf_model(tie: bool, factor: float):
    cfg = transformers.LlamaConfig(
        vocab_size=1000, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
        num_key_value_heads=2, max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0,
        rope_scaling={"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 8192},
        tie_word_embeddings=tie, attention_bias=False)
    torch.manual_seed(11)
    model = transformers.LlamaForCausalLM(cfg).eval()
    with torch.no_grad():
        for prm in model.parameters():          # norm weights away from 1, everything representable in bf16
            if prm.dim() == 1:
                prm.add_(0.1 * torch.randn_like(prm))
            prm.copy_(prm.to(torch.bfloat16).float())
    return model


@pytest.mark.parametrize("tie,factor,prompt_len", [(True, 32.0, 9), (False, 8.0, 150)])
def test_decode_loop_on_hf_weights_tracks_the_hf_model(ext, pkg, device, tie, factor, prompt_len):
    model = _hf_model(tie, factor)
    cfg = pkg.decode_loop.config_from_hf(model.config)
    assert (cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd, cfg.hidden_dim) == (3, 8, 2, 512, 1024)
    assert cfg.rope_scaled and cfg.rope_scale_factor == factor and cfg.rope_theta == 500000.0
    weights = pkg.decode_loop.weights_from_hf(model.state_dict(), cfg)
    assert ("lm_head" in weights) == (not tie)
    B, G = 2, 10
    prompts = torch.randint(0, cfg.vocab_size, (B, prompt_len), generator=torch.Generator().manual_seed(2))
    dec = pkg.decode_loop.Llama3Decoder(ext, cfg, device, max_batch=B, max_len=prompt_len + G + 2, weights=weights)
    # logits of the prompt's last position: prefill (the tcgen05 kernel for the long prompt, mma.sync for the short)
    pos = torch.zeros(B, dtype=torch.int32, device=device)
    lens = torch.full((B,), prompt_len, dtype=torch.int32, device=device)
    ours = dec.forward(prompts.to(device), pos, lens).float().cpu()
    with torch.no_grad():
        ref = model(prompts).logits[:, -1].float()
    assert (ours - ref).abs().max().item() < 0.06, (ours - ref).abs().max().item()
    assert torch.equal(ours.argmax(-1), ref.argmax(-1)) or (ref.topk(2).values.diff().abs().min() < 0.05)
    # greedy generation (graph-replayed decode steps), the Hugging Face model teacher-forced with our tokens:
    # wherever its logits leave a clear winner, that is the token the loop chose
    toks = dec.generate(prompts.to(device), G, use_graph=True).cpu()
    torch.cuda.synchronize()
    seq = prompts.clone()
    checked = 0
    for i in range(G):
        with torch.no_grad():
            logits = model(seq).logits[:, -1].float()
        top2 = logits.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 0.05
        assert torch.equal(logits.argmax(-1)[clear], toks[clear, i]), i
        checked += int(clear.sum())
        seq = torch.cat([seq, toks[:, i:i + 1]], dim=1)
    assert checked >= B * G // 2
