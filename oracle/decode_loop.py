"""CPU restatement of the decode loop (test infrastructure): the same layer arithmetic as
llama3-custom-inference_b200/decode_loop.py, i.e. the reference's Block / CausalSelfAttention / MLP
(model.py:92-149, 203-232) with greedy decoding (model.py:370-371), built from the oracle's RMSNorm, RoPE and
attention and torch's CPU bf16 GEMMs.  Used to check the GPU loop on a small configuration and, on a bounded
sample, as the CPU baseline of the end-to-end benchmark."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .attention import sdpa_reference
from .rms_norm import rms_norm_reference
from .rope import freqs_cis_reference, rot_embed_reference


class CpuDecoder:
    def __init__(self, cfg, weights: dict, max_batch: int, max_len: int):
        self.cfg, self.w = cfg, weights
        D = cfg.n_embd // cfg.n_head
        self.cache_k = [torch.zeros(max_batch, max_len, cfg.n_kv_head, D, dtype=torch.bfloat16) for _ in range(cfg.n_layer)]
        self.cache_v = [torch.zeros(max_batch, max_len, cfg.n_kv_head, D, dtype=torch.bfloat16) for _ in range(cfg.n_layer)]
        self.freqs = freqs_cis_reference(D, max_len, cfg.rope_theta, getattr(cfg, "rope_scaled", True),
                                         scale_factor=cfg.rope_scale_factor,
                                         low_freq_factor=getattr(cfg, "rope_low_freq_factor", 1.0),
                                         high_freq_factor=getattr(cfg, "rope_high_freq_factor", 4.0),
                                         old_context_len=getattr(cfg, "rope_old_context_len", 8192))

    def forward(self, tokens: torch.Tensor, start_pos: int, return_logits: bool = False):
        cfg, w = self.cfg, self.w
        B, T = tokens.shape
        E, Hq, Hkv = cfg.n_embd, cfg.n_head, cfg.n_kv_head
        D = E // Hq
        x = F.embedding(tokens, w["wte"])
        freqs = self.freqs[start_pos:start_pos + T]
        for l in range(cfg.n_layer):
            p = f"h{l}."
            h = rms_norm_reference(x, w[p + "ln_1"], cfg.norm_eps)
            qkv = F.linear(h, w[p + "attn"])
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            q = rot_embed_reference(q.reshape(B, T, Hq, D), freqs)
            k = rot_embed_reference(k.reshape(B, T, Hkv, D), freqs)
            self.cache_k[l][:B, start_pos:start_pos + T] = k
            self.cache_v[l][:B, start_pos:start_pos + T] = v.reshape(B, T, Hkv, D)
            kk = self.cache_k[l][:B, :start_pos + T].transpose(1, 2)
            vv = self.cache_v[l][:B, :start_pos + T].transpose(1, 2)
            if T > 1:
                y = F.scaled_dot_product_attention(q.transpose(1, 2).float(), kk.float(), vv.float(), is_causal=True,
                                                   enable_gqa=True).to(torch.bfloat16)
            else:
                y = sdpa_reference(q.transpose(1, 2), kk, vv).to(torch.bfloat16)
            y = y.transpose(1, 2).reshape(B, T, E)
            x = x + F.linear(y, w[p + "proj"])
            h = rms_norm_reference(x, w[p + "ln_2"], cfg.norm_eps)
            x = x + F.linear(F.silu(F.linear(h, w[p + "fc2"])) * F.linear(h, w[p + "fc"]), w[p + "mlp_proj"])
        x = rms_norm_reference(x[:, -1:, :], w["ln_f"], cfg.norm_eps)
        logits = F.linear(x, w.get("lm_head", w["wte"])).float()[:, -1]
        return logits if return_logits else logits.argmax(dim=-1)
