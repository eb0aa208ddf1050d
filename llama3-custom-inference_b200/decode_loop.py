"""A Llama-3 decode loop around the extension kernels, for end-to-end tokens/s on random weights.

Host-side mirror of what the reference's model does around its three extension calls — `Block` /
`CausalSelfAttention` / `MLP` / `LLaMA3.forward` (model.py:92-149, 203-232) and the greedy branch of
`LLaMA3.generate` (model.py:363-381) — restricted to what the end-to-end benchmark needs: random-init
weights of the Llama-3.2-1B architecture (or any `DecoderConfig`), a batch of equal-length prompts, greedy or
top-p decoding with `ignore_eos`.  It is a harness, not a model library: no tokenizer; weights come from
`init_weights` (random) or from a Hugging Face Llama state dict through `weights_from_hf` / `config_from_hf`, which
restate the reference's key mapping and its un-permutation of the q and k projections (model.py:235-280).

What differs from the reference's loop, all on the caller's side of the kernels:
  * rotary embedding, the K/V cache write and the split of q|k|v are one call (`rot_embed_kv_cache` with
    per-sequence device positions) instead of two `rot_embed` calls and two cache copies (model.py:100-108);
  * decode attention reads the cache in place with device-side lengths (`seq_lens=`), so no tensor shape or
    host scalar changes from step to step;
  * which lets one decode step be captured in a CUDA graph and replayed: no per-step Python dispatch, no
    per-step mask construction (model.py:211) and no `all(eos_reached)` host sync (model.py:380).
  * the residual add runs inside the RMSNorm that follows it (`add_rms_norm`), `c_fc2` and `c_fc` are one GEMM
    over the stacked weight, and `silu(gate) * up` is one kernel (`silu_mul`) instead of two elementwise passes.
GEMMs and the embedding lookup are plain torch ops (cuBLAS); the token choice (greedy argmax, or nucleus sampling)
with its token bookkeeping is one kernel (`greedy_step` / `top_p_step`); prefill attention (torch SDPA in the reference, model.py:114-116) is `prefill_attention`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import rope_table

# Profiler range names of the reference's loop (model.py:99-109 "rot_embd" / "use_kv", :214-216 "layer", :364-366
# "forward"), kept so that a timeline of this loop reads like one of the reference's.  The fused RoPE + cache-write
# call carries both of the first two names.
_nvtx_push, _nvtx_pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop


@dataclass
class DecoderConfig:
    """Architecture numbers of model.py:153-165 (defaults: Llama-3.2-1B) plus the rotary scaling factor."""
    vocab_size: int = 128256
    n_layer: int = 16
    n_head: int = 32
    n_kv_head: int = 8
    n_embd: int = 2048
    hidden_dim: int = 8192
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scale_factor: float = 32.0      # (the reference's apply_scaling hard-codes 8, model.py:29; Llama-3.2 uses 32)
    rope_low_freq_factor: float = 1.0    # model.py:30-32
    rope_high_freq_factor: float = 4.0
    rope_old_context_len: int = 8192
    rope_scaled: bool = True

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head


class Llama3Decoder:
    """Random-init decoder-only transformer with a static KV cache on one GPU."""

    def __init__(self, ext, cfg: DecoderConfig, device, max_batch: int, max_len: int, seed: int = 42,
                 weights: Optional[dict] = None):
        self.ext, self.cfg, self.device = ext, cfg, torch.device(device)
        self.max_batch, self.max_len = max_batch, max_len
        E, F_, D = cfg.n_embd, cfg.hidden_dim, cfg.head_dim
        qkv_rows = (cfg.n_head + 2 * cfg.n_kv_head) * D
        if weights is None:
            weights = init_weights(cfg, seed)
        self.w = {k: v.to(self.device) for k, v in weights.items()}
        for l in range(cfg.n_layer):   # gate (c_fc2) and up (c_fc) projections as one [2F, E] GEMM operand
            self.w[f"h{l}.gate_up"] = torch.cat([self.w.pop(f"h{l}.fc2"), self.w.pop(f"h{l}.fc")], dim=0)
        bf16 = dict(dtype=torch.bfloat16, device=self.device)
        self.cache_k = [torch.zeros(max_batch, max_len, cfg.n_kv_head, D, **bf16) for _ in range(cfg.n_layer)]
        self.cache_v = [torch.zeros(max_batch, max_len, cfg.n_kv_head, D, **bf16) for _ in range(cfg.n_layer)]
        self.freqs = rope_table.precompute_freqs_cis(D, max_len, cfg.rope_theta, cfg.rope_scaled,
                                                     scale_factor=cfg.rope_scale_factor,
                                                     low_freq_factor=cfg.rope_low_freq_factor,
                                                     high_freq_factor=cfg.rope_high_freq_factor,
                                                     old_context_len=cfg.rope_old_context_len).to(self.device)
        assert self.w["h0.attn"].shape == (qkv_rows, E) and self.w["h0.gate_up"].shape == (2 * F_, E)
        self._graph = None
        self._kernel_for_batch = {}
        self.equal_lengths = True   # all sequences of a step have the same number of cached tokens (`generate`)

    def _decode_kernel(self, B: int) -> int:
        """`max_ctas` for the decode attention of a batch of B.  `generate` keeps all sequences at one length, which
        the library cannot see in device-side lengths: its own rule must assume a lopsided batch and keeps the
        persistent kernel for long caches.  With units known to be equal, the static deal is asked for (-1)
        wherever the library would take it for a batch of full-length caches."""
        if not self.equal_lengths:
            return 0
        if B in self._kernel_for_batch:
            return self._kernel_for_batch[B]
        cfg = self.cfg
        dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        choice = self.ext.flash_decode_kernel_choice(dev, B, cfg.n_head, cfg.n_kv_head, cfg.head_dim, self.max_len, False)
        self._kernel_for_batch[B] = -1 if choice > 0 else 0
        return self._kernel_for_batch[B]

    # ---- one forward pass over T new tokens per sequence ------------------------------------------------
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] int64; positions int32 [B] = tokens already cached per sequence; seq_lens int32 [B] =
        positions + T.  Returns the logits of the last position, bf16 [B, vocab]."""
        cfg, ext, w = self.cfg, self.ext, self.w
        B, T = tokens.shape
        E, D, Hq, Hkv = cfg.n_embd, cfg.head_dim, cfg.n_head, cfg.n_kv_head
        F_ = cfg.hidden_dim
        x = F.embedding(tokens, w["wte"])                                            # model.py:208
        h = ext.rms_norm(x, w["h0.ln_1"], cfg.norm_eps)                                # model.py:147, 71
        for l in range(cfg.n_layer):
            p = f"h{l}."
            _nvtx_push("layer")
            qkv = F.linear(h, w[p + "attn"])                                           # model.py:95
            _nvtx_push("rot_embd")
            _nvtx_push("use_kv")
            q = ext.rot_embed_kv_cache(qkv, self.freqs, self.cache_k[l], self.cache_v[l], 0, Hq, Hkv,
                                       positions=positions)                            # model.py:96-108
            _nvtx_pop()
            _nvtx_pop()
            if T > 1:
                # prefill: all sequences start at position 0 with T tokens (model.py:114-116)
                k = self.cache_k[l][:B, :T].transpose(1, 2)
                v = self.cache_v[l][:B, :T].transpose(1, 2)
                y = ext.prefill_attention(q.transpose(1, 2), k, v)                     # causal, GQA
            else:
                y = ext.flash_attention_decode(q.transpose(1, 2), self.cache_k[l][:B].transpose(1, 2),
                                               self.cache_v[l][:B].transpose(1, 2), seq_lens=seq_lens,
                                               max_ctas=self._decode_kernel(B))     # model.py:118
            y = y.transpose(1, 2).reshape(B, T, E)                                     # model.py:120
            x, h = ext.add_rms_norm(F.linear(y, w[p + "proj"]), x, w[p + "ln_2"], cfg.norm_eps)  # :121, 147-148
            gu = F.linear(h, w[p + "gate_up"])                                         # c_fc2 | c_fc, model.py:134
            m = F.linear(ext.silu_mul(gu[..., :F_], gu[..., F_:]), w[p + "mlp_proj"])
            nxt = w[f"h{l + 1}.ln_1"] if l + 1 < cfg.n_layer else w["ln_f"]
            x, h = ext.add_rms_norm(m, x, nxt, cfg.norm_eps)                           # model.py:148, next 147 / 217
            _nvtx_pop()
        # the reference widens the logits to fp32 first (model.py:226); the widening is monotonic, so the argmax
        # of the bf16 values is the same index
        # model.py:225; the head is tied to the embedding (model.py:189) unless the checkpoint brought its own
        return F.linear(h[:, -1, :], w.get("lm_head", w["wte"]))

    # ---- greedy generation --------------------------------------------------------------------------------
    @torch.inference_mode()
    def generate(self, prompts: torch.Tensor, max_gen_len: int, use_graph: bool = True, temperature: float = 0.0,
                 top_p: float = 0.9, seed: int = 0) -> torch.Tensor:
        """prompts int64 [B, P] (equal lengths, on the device).  Returns the generated tokens int64
        [B, max_gen_len].  With `use_graph` one decode step is captured in a CUDA graph and replayed.
        `temperature` 0 is greedy decoding (model.py:370-371); a positive temperature draws every token from the
        top-p nucleus of softmax(logits / temperature) (model.py:367-369), reproducibly for a given `seed`."""
        B, P = prompts.shape
        assert B <= self.max_batch and P + max_gen_len <= self.max_len
        dev = self.device
        out = torch.empty(B, max_gen_len, dtype=torch.int64, device=dev)
        positions = torch.zeros(B, dtype=torch.int32, device=dev)
        seq_lens = torch.full((B,), P, dtype=torch.int32, device=dev)
        steps = torch.zeros(B, dtype=torch.int64, device=dev)  # next free column of `out`, per sequence
        cur = torch.zeros(B, 1, dtype=torch.int64, device=dev)

        def pick(logits):
            # token choice, out[b, steps[b]] = token, cur[b] = token, steps / positions / seq_lens += 1: one kernel
            if temperature > 0:
                self.ext.top_p_step(logits, out, steps, cur.view(B), positions, seq_lens, temperature, top_p, seed)
            else:
                self.ext.greedy_step(logits, out, steps, cur.view(B), positions, seq_lens)  # model.py:370-381

        pick(self.forward(prompts, positions, seq_lens))                                # prefill; model.py:363-371
        # static state of the decode step: everything the step reads or writes lives in these tensors
        positions.fill_(P)
        seq_lens.fill_(P + 1)

        def step():
            _nvtx_push("forward")
            logits = self.forward(cur, positions, seq_lens)
            _nvtx_pop()
            pick(logits)

        n_steps = max_gen_len - 1
        if n_steps <= 0:
            return out
        if not use_graph:
            for _ in range(n_steps):
                step()
            return out
        # Capture needs every lazy allocation (decode workspace, cuBLAS handles) to have happened: run the step
        # once eagerly on a side stream, then capture the same step.
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
            n_steps -= 1
            graph = torch.cuda.CUDAGraph()
            if n_steps > 0:
                with torch.cuda.graph(graph, stream=side):
                    step()
                # the capture did not run the step: replay it for every remaining token
                for _ in range(n_steps):
                    graph.replay()
        torch.cuda.current_stream(dev).wait_stream(side)
        self._graph = graph
        return out


def config_from_hf(hf_config) -> DecoderConfig:
    """The architecture numbers `from_pretrained_llama3_hf` takes from a Hugging Face Llama config (model.py:290-296),
    plus the rotary parameters, which the reference hard-codes (model.py:29-32, 163) and the config carries."""
    rope = getattr(hf_config, "rope_parameters", None) or getattr(hf_config, "rope_scaling", None) or {}
    theta = rope.get("rope_theta", None) or getattr(hf_config, "rope_theta", None) or 500000.0
    scaled = rope.get("rope_type", rope.get("type", "default")) == "llama3"
    return DecoderConfig(vocab_size=hf_config.vocab_size, n_layer=hf_config.num_hidden_layers,
                         n_head=hf_config.num_attention_heads, n_kv_head=hf_config.num_key_value_heads,
                         n_embd=hf_config.hidden_size, hidden_dim=hf_config.intermediate_size,
                         norm_eps=hf_config.rms_norm_eps, rope_theta=float(theta), rope_scaled=scaled,
                         rope_scale_factor=float(rope.get("factor", 8.0)),
                         rope_low_freq_factor=float(rope.get("low_freq_factor", 1.0)),
                         rope_high_freq_factor=float(rope.get("high_freq_factor", 4.0)),
                         rope_old_context_len=int(rope.get("original_max_position_embeddings", 8192)))


def weights_from_hf(state_dict: dict, cfg: DecoderConfig) -> dict:
    """This loop's weights from a Hugging Face Llama state dict: the key mapping of `adapt_llama_state_dict_keys_hf`
    (model.py:235-280).  The q and k projections are un-permuted (model.py:244-245, 258-264): the Hugging Face
    conversion reorders each head's rows from the interleaved (even, odd) pair layout of the original weights to
    "first half, second half", and the rotary kernel here, like the reference's, rotates adjacent pairs."""
    D = cfg.head_dim

    def unpermute(w, n_heads):
        rows, cols = w.shape
        return w.view(n_heads, 2, rows // n_heads // 2, cols).transpose(1, 2).reshape(rows, cols)

    def get(name):
        return state_dict[name].detach().to(torch.bfloat16)

    w = {"wte": get("model.embed_tokens.weight"), "ln_f": get("model.norm.weight")}
    head = state_dict.get("lm_head.weight")
    if head is not None and head.data_ptr() != state_dict["model.embed_tokens.weight"].data_ptr():
        w["lm_head"] = head.detach().to(torch.bfloat16)   # an untied output projection (the 8B and 70B checkpoints)
    for l in range(cfg.n_layer):
        src, p = f"model.layers.{l}.", f"h{l}."
        q = unpermute(get(src + "self_attn.q_proj.weight"), cfg.n_head)
        k = unpermute(get(src + "self_attn.k_proj.weight"), cfg.n_kv_head)
        assert q.shape[0] == cfg.n_head * D and k.shape[0] == cfg.n_kv_head * D
        w[p + "attn"] = torch.cat([q, k, get(src + "self_attn.v_proj.weight")], dim=0)          # c_attn, model.py:255-266
        w[p + "proj"] = get(src + "self_attn.o_proj.weight")
        w[p + "ln_1"] = get(src + "input_layernorm.weight")
        w[p + "ln_2"] = get(src + "post_attention_layernorm.weight")
        w[p + "fc2"] = get(src + "mlp.gate_proj.weight")                                        # model.py:271
        w[p + "fc"] = get(src + "mlp.up_proj.weight")
        w[p + "mlp_proj"] = get(src + "mlp.down_proj.weight")
    return w


def init_weights(cfg: DecoderConfig, seed: int = 42) -> dict:
    """bf16 weights ~ N(0, 0.02) from a CPU generator, norm weights 1 (the benchmark's random-init model).
    Names follow the reference's module tree (model.py:83-84, 127-131, 140-143, 183-188)."""
    g = torch.Generator().manual_seed(seed)
    E, F_, D = cfg.n_embd, cfg.hidden_dim, cfg.head_dim

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=g) * 0.02).bfloat16()

    w = {"wte": mat(cfg.vocab_size, E), "ln_f": torch.ones(E, dtype=torch.bfloat16)}
    for l in range(cfg.n_layer):
        p = f"h{l}."
        w[p + "ln_1"] = torch.ones(E, dtype=torch.bfloat16)
        w[p + "attn"] = mat((cfg.n_head + 2 * cfg.n_kv_head) * D, E)
        w[p + "proj"] = mat(E, E)
        w[p + "ln_2"] = torch.ones(E, dtype=torch.bfloat16)
        w[p + "fc"] = mat(F_, E)
        w[p + "fc2"] = mat(F_, E)
        w[p + "mlp_proj"] = mat(E, F_)
    return w
