// Torch extension module `custom_kernels_extension`: the drop-in boundary.
//
// Exports the three functions the reference binds in custom_kernels/main.cpp:2-8
//   flash_attention_decode(query, keys, values) -> Tensor      (model.py:118, benchmark_kernel.py:25)
//   rms_norm(input, weight, eps) -> Tensor                     (model.py:71)
//   rot_embed(input, freq) -> Tensor                           (model.py:100-101)
// with the same positional signatures, return conventions (a freshly allocated tensor shaped
// like the input) and error type (RuntimeError through TORCH_CHECK), and adds keyword-only
// extras plus new functions; nothing here computes: every call validates its tensors, takes the
// device of the input and torch's current stream (the reference launches on the legacy default
// stream of whatever device is current, custom_kernels/custom_kernels.cu:274-275,386,439) and
// forwards raw pointers to the C ABI of include/l3ci_b200.h.
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <map>
#include <mutex>
#include <optional>
#include <tuple>
#include <utility>

#include "l3ci_b200.h"

namespace {

using torch::Tensor;

l3ci_stream_t current_stream() {
  return reinterpret_cast<l3ci_stream_t>(c10::cuda::getCurrentCUDAStream().stream());
}

void check_status(int status, const char* what) {
  TORCH_CHECK(status == L3CI_OK, what, ": ", l3ci_status_string(status), " (", l3ci_last_error(), ")");
}

void check_bf16_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bfloat16, got ", t.scalar_type());
}

// Scratch of the flash-decode kernel, one buffer per (device, stream), zero-filled when it is
// created and reused by later calls (the kernel leaves it ready).  The reference allocates its
// three scratch tensors on every call (custom_kernels/custom_kernels.cu:269-271).
struct Workspace {
  Tensor buf;
};
std::mutex g_ws_mutex;
std::map<std::pair<int, int64_t>, Workspace>& workspaces() {
  static auto* m = new std::map<std::pair<int, int64_t>, Workspace>();  // never destroyed: outlives CUDA teardown
  return *m;
}

Tensor& workspace_for(const Tensor& like, size_t bytes) {
  const auto stream = c10::cuda::getCurrentCUDAStream();
  const auto key = std::make_pair((int)like.get_device(), (int64_t)stream.id());
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  auto& all = workspaces();
  if (all.size() >= 16 && all.find(key) == all.end()) {
    // streams come and go (graph captures, side streams): the buffers of other streams are dropped rather than
    // kept for the life of the process; a stream that comes back gets a fresh zero-filled one
    for (auto it = all.begin(); it != all.end();) it = it->first.first == key.first ? all.erase(it) : std::next(it);
  }
  Workspace& ws = all[key];
  if (!ws.buf.defined() || (size_t)ws.buf.numel() < bytes) {
    ws.buf = torch::zeros({(int64_t)bytes}, torch::dtype(torch::kUInt8).device(like.device()));
  }
  return ws.buf;
}

struct DecodeShapes {
  int B, Hq, Hkv, D, n_seq;
};

DecodeShapes check_decode_inputs(const Tensor& q, const Tensor& k, const Tensor& v,
                                 const std::optional<Tensor>& seq_lens) {
  check_bf16_cuda(q, "query");
  check_bf16_cuda(k, "keys");
  check_bf16_cuda(v, "values");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "query, keys, values must be 4-D [B, H, T, D]");
  TORCH_CHECK(q.size(2) == 1, "flash_attention_decode takes one query token per sequence, got ", q.size(2));
  TORCH_CHECK(k.sizes() == v.sizes(), "keys and values must have the same shape");
  TORCH_CHECK(k.size(0) == q.size(0) && k.size(3) == q.size(3), "batch / head size of query and keys differ");
  TORCH_CHECK(k.get_device() == q.get_device() && v.get_device() == q.get_device(), "inputs on different devices");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1, "last dimension must be contiguous");
  if (seq_lens) {
    TORCH_CHECK(seq_lens->is_cuda() && seq_lens->scalar_type() == torch::kInt32 && seq_lens->dim() == 1 &&
                    seq_lens->size(0) == q.size(0) && seq_lens->is_contiguous(),
                "seq_lens must be a contiguous int32 CUDA tensor of shape [B]");
  }
  DecodeShapes s;
  s.B = (int)q.size(0);
  s.Hq = (int)q.size(1);
  s.Hkv = (int)k.size(1);
  s.n_seq = (int)k.size(2);
  s.D = (int)q.size(3);
  TORCH_CHECK(s.D == 64 || s.D == 128, "Unsupported head size for splitkv kernel: ", s.D);
  TORCH_CHECK(s.Hkv > 0 && s.Hq % s.Hkv == 0 && s.Hq / s.Hkv <= 16,
              "Unsupported QKV head ratio for splitkv kernel: ", s.Hq, "/", s.Hkv);
  return s;
}

void run_decode(const Tensor& q, const Tensor& k, const Tensor& v, const std::optional<Tensor>& seq_lens,
                Tensor* out, Tensor* o_partial, Tensor* lse, double scale, int64_t max_ctas,
                const DecodeShapes& s) {
  l3ci_flash_decode_args a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.out = out ? out->data_ptr() : nullptr;
  a.o_partial = o_partial ? o_partial->data_ptr<float>() : nullptr;
  a.lse = lse ? lse->data_ptr<float>() : nullptr;
  a.seq_lens = seq_lens ? seq_lens->data_ptr<int32_t>() : nullptr;
  a.B = s.B; a.Hq = s.Hq; a.Hkv = s.Hkv; a.D = s.D; a.n_seq = s.n_seq;
  a.q_sb = q.stride(0); a.q_sh = q.stride(1);
  a.k_sb = k.stride(0); a.k_sh = k.stride(1); a.k_st = k.stride(2);
  a.v_sb = v.stride(0); a.v_sh = v.stride(1); a.v_st = v.stride(2);
  if (out) { a.o_sb = out->stride(0); a.o_sh = out->stride(1); }
  a.scale = (float)scale;
  a.max_ctas = (int32_t)max_ctas;
  a.stream = current_stream();
  const size_t need = l3ci_flash_decode_scratch_bytes(s.B, s.Hq, s.Hkv, s.D);
  Tensor& ws = workspace_for(q, need);
  a.scratch = ws.data_ptr();
  a.scratch_bytes = (size_t)ws.numel();
  check_status(l3ci_flash_decode(&a), "flash_attention_decode");
}

// reference: custom_kernels/custom_kernels.cu:233-338
Tensor flash_attention_decode(Tensor query, Tensor keys, Tensor values, std::optional<Tensor> seq_lens,
                              std::optional<Tensor> out, double scale, int64_t max_ctas) {
  const DecodeShapes s = check_decode_inputs(query, keys, values, seq_lens);
  const c10::cuda::CUDAGuard guard(query.device());
  Tensor result = out ? *out : torch::empty_like(query);
  if (out) {
    check_bf16_cuda(result, "out");
    TORCH_CHECK(result.sizes() == query.sizes() && result.stride(3) == 1, "out must be shaped like query");
  }
  if (s.B == 0) return result;
  run_decode(query, keys, values, seq_lens, &result, nullptr, nullptr, scale, max_ctas, s);
  return result;
}

// Attention over a slice of the cached sequence, returned as fp32 (o, lse) for lse_merge.
// `out_o` / `out_lse` (contiguous fp32 [B,Hq,D] / [B,Hq]) let the caller choose where the result lands, e.g. in
// its slot of an exchange buffer that peers can address.
std::tuple<Tensor, Tensor> flash_attention_decode_partial(Tensor query, Tensor keys, Tensor values,
                                                          std::optional<Tensor> seq_lens, double scale,
                                                          int64_t max_ctas, std::optional<Tensor> out_o,
                                                          std::optional<Tensor> out_lse) {
  const DecodeShapes s = check_decode_inputs(query, keys, values, seq_lens);
  const c10::cuda::CUDAGuard guard(query.device());
  auto f32 = torch::dtype(torch::kFloat32).device(query.device());
  TORCH_CHECK(out_o.has_value() == out_lse.has_value(), "out_o and out_lse go together");
  if (out_o) {
    TORCH_CHECK(out_o->is_cuda() && out_o->scalar_type() == torch::kFloat32 && out_o->is_contiguous() &&
                    out_o->numel() == (int64_t)s.B * s.Hq * s.D && out_lse->is_cuda() &&
                    out_lse->scalar_type() == torch::kFloat32 && out_lse->is_contiguous() &&
                    out_lse->numel() == (int64_t)s.B * s.Hq && out_o->get_device() == query.get_device() &&
                    out_lse->get_device() == query.get_device(),
                "out_o / out_lse must be contiguous fp32 CUDA tensors of B*Hq*D / B*Hq elements");
  }
  Tensor o = out_o ? *out_o : torch::empty({s.B, s.Hq, s.D}, f32);
  Tensor lse = out_lse ? *out_lse : torch::empty({s.B, s.Hq}, f32);
  if (s.B == 0) return {o, lse};
  run_decode(query, keys, values, seq_lens, nullptr, &o, &lse, scale, max_ctas, s);
  return {o, lse};
}

// Causal attention for T > 1 new tokens (model.py:114-116 sends this case to torch's SDPA): query [B,Hq,T,D],
// keys / values [B,Hkv,S,D] (views of the cache are fine), query t sees keys j <= start_pos + t.  Returns a tensor
// laid out like `query`.
Tensor prefill_attention(Tensor query, Tensor keys, Tensor values, int64_t start_pos, double scale, int64_t variant) {
  check_bf16_cuda(query, "query");
  check_bf16_cuda(keys, "keys");
  check_bf16_cuda(values, "values");
  TORCH_CHECK(query.dim() == 4 && keys.dim() == 4 && values.dim() == 4, "query, keys, values must be 4-D");
  TORCH_CHECK(keys.sizes() == values.sizes() && keys.size(0) == query.size(0) && keys.size(3) == query.size(3),
              "shape mismatch between query, keys and values");
  TORCH_CHECK(query.stride(3) == 1 && keys.stride(3) == 1 && values.stride(3) == 1, "last axis must be contiguous");
  TORCH_CHECK(keys.get_device() == query.get_device() && values.get_device() == query.get_device(), "tensors on different devices");
  const int64_t B = query.size(0), Hq = query.size(1), T = query.size(2), D = query.size(3), Hkv = keys.size(1), S = keys.size(2);
  TORCH_CHECK(D == 64 || D == 128, "Unsupported head size for prefill_attention kernel: ", D);
  TORCH_CHECK(Hkv > 0 && Hq % Hkv == 0, "query heads must be a multiple of kv heads");
  TORCH_CHECK(start_pos >= 0 && start_pos + T <= S, "start_pos + T must not exceed the keys given");
  const c10::cuda::CUDAGuard guard(query.device());
  Tensor out = torch::empty_strided(query.sizes(), query.strides(), query.options());
  if (B == 0 || T == 0) return out;
  l3ci_prefill_args a{};
  a.q = query.data_ptr(); a.k = keys.data_ptr(); a.v = values.data_ptr(); a.out = out.data_ptr(); a.status = nullptr;
  a.B = (int32_t)B; a.Hq = (int32_t)Hq; a.Hkv = (int32_t)Hkv; a.D = (int32_t)D;
  a.T = (int32_t)T; a.n_keys = (int32_t)S; a.start_pos = (int32_t)start_pos;
  a.q_sb = query.stride(0); a.q_sh = query.stride(1); a.q_st = query.stride(2);
  a.k_sb = keys.stride(0); a.k_sh = keys.stride(1); a.k_st = keys.stride(2);
  a.v_sb = values.stride(0); a.v_sh = values.stride(1); a.v_st = values.stride(2);
  a.o_sb = out.stride(0); a.o_sh = out.stride(1); a.o_st = out.stride(2);
  a.scale = (float)scale;
  a.variant = (int32_t)variant;
  a.stream = current_stream();
  check_status(l3ci_prefill_attention(&a), "prefill_attention");
  return out;
}

// out[b, h, 0, :] = sum_p softmax_p(lse[p, b, h]) * o[p, b, h, :]
Tensor lse_merge(Tensor o_parts, Tensor lse_parts) {
  TORCH_CHECK(o_parts.is_cuda() && o_parts.scalar_type() == torch::kFloat32 && o_parts.dim() == 4 &&
                  o_parts.is_contiguous(),
              "o_parts must be a contiguous fp32 CUDA tensor [parts, B, Hq, D]");
  TORCH_CHECK(lse_parts.is_cuda() && lse_parts.scalar_type() == torch::kFloat32 && lse_parts.dim() == 3 &&
                  lse_parts.is_contiguous() && lse_parts.size(0) == o_parts.size(0) &&
                  lse_parts.size(1) == o_parts.size(1) && lse_parts.size(2) == o_parts.size(2),
              "lse_parts must be a contiguous fp32 CUDA tensor [parts, B, Hq]");
  const c10::cuda::CUDAGuard guard(o_parts.device());
  const int parts = (int)o_parts.size(0), B = (int)o_parts.size(1), Hq = (int)o_parts.size(2), D = (int)o_parts.size(3);
  // Same memory layout as the reference's result for a [B, 1, Hq, D].transpose(1, 2) query.
  Tensor out = torch::empty({B, 1, Hq, D}, torch::dtype(torch::kBFloat16).device(o_parts.device())).transpose(1, 2);
  check_status(l3ci_lse_merge(o_parts.data_ptr<float>(), lse_parts.data_ptr<float>(), out.data_ptr(), parts, B, Hq,
                              D, out.stride(0), out.stride(1), current_stream()),
               "lse_merge");
  return out;
}

// Exchange of shard results over peer memory fused with their merge (l3ci_lse_exchange_merge).  `bufs` is an
// int64 CUDA tensor [ranks] holding the base addresses of every rank's exchange buffer as this process sees
// them; this rank's own result must already be in its slot of parity epoch & 1.
Tensor lse_exchange_merge(Tensor bufs, int64_t rank, int64_t epoch, int64_t B, int64_t Hq, int64_t D,
                          std::optional<Tensor> status) {
  TORCH_CHECK(bufs.is_cuda() && bufs.scalar_type() == torch::kInt64 && bufs.dim() == 1 && bufs.is_contiguous(),
              "bufs must be a contiguous int64 CUDA tensor of buffer addresses");
  if (status)
    TORCH_CHECK(status->is_cuda() && status->scalar_type() == torch::kInt32 && status->numel() >= 1 &&
                    status->get_device() == bufs.get_device(),
                "status must be an int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(bufs.device());
  Tensor out = torch::empty({B, 1, Hq, D}, torch::dtype(torch::kBFloat16).device(bufs.device())).transpose(1, 2);
  check_status(l3ci_lse_exchange_merge(reinterpret_cast<void* const*>(bufs.data_ptr<int64_t>()), (int32_t)rank,
                                       (int32_t)bufs.size(0), (uint32_t)epoch, out.data_ptr(), (int32_t)B, (int32_t)Hq,
                                       (int32_t)D, out.stride(0), out.stride(1),
                                       status ? status->data_ptr<int32_t>() : nullptr, current_stream()),
               "lse_exchange_merge");
  return out;
}

// Decode attention over this rank's slice of a sequence-sharded cache, merged with the other ranks' results in the
// same launch (l3ci_flash_decode_exchange).  `bufs`: int64 CUDA tensor [ranks] of the ranks' exchange buffers as this
// process addresses them.  Returns false-y (None) when the sizes go to the kernel without a fused exchange, so that
// the caller can take the two-launch path.
std::optional<Tensor> flash_attention_decode_exchange(Tensor query, Tensor keys, Tensor values, Tensor bufs, int64_t rank,
                                                      int64_t epoch, std::optional<Tensor> seq_lens, std::optional<Tensor> out,
                                                      std::optional<Tensor> status, double scale, int64_t max_ctas) {
  const DecodeShapes s = check_decode_inputs(query, keys, values, seq_lens);
  TORCH_CHECK(bufs.is_cuda() && bufs.scalar_type() == torch::kInt64 && bufs.dim() == 1 && bufs.is_contiguous() &&
                  bufs.get_device() == query.get_device(),
              "bufs must be a contiguous int64 CUDA tensor of buffer addresses on the device of the inputs");
  if (status)
    TORCH_CHECK(status->is_cuda() && status->scalar_type() == torch::kInt32 && status->numel() >= 1 &&
                    status->get_device() == query.get_device(),
                "status must be an int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(query.device());
  Tensor result = out ? *out : torch::empty_like(query);
  if (out) {
    check_bf16_cuda(result, "out");
    TORCH_CHECK(result.sizes() == query.sizes() && result.stride(3) == 1, "out must be shaped like query");
  }
  if (s.B == 0) return result;
  l3ci_flash_decode_args a{};
  a.q = query.data_ptr(); a.k = keys.data_ptr(); a.v = values.data_ptr(); a.out = result.data_ptr();
  a.seq_lens = seq_lens ? seq_lens->data_ptr<int32_t>() : nullptr;
  a.B = s.B; a.Hq = s.Hq; a.Hkv = s.Hkv; a.D = s.D; a.n_seq = s.n_seq;
  a.q_sb = query.stride(0); a.q_sh = query.stride(1);
  a.k_sb = keys.stride(0); a.k_sh = keys.stride(1); a.k_st = keys.stride(2);
  a.v_sb = values.stride(0); a.v_sh = values.stride(1); a.v_st = values.stride(2);
  a.o_sb = result.stride(0); a.o_sh = result.stride(1);
  a.scale = (float)scale;
  a.max_ctas = (int32_t)max_ctas;
  a.stream = current_stream();
  const int st = l3ci_flash_decode_exchange(&a, reinterpret_cast<void* const*>(bufs.data_ptr<int64_t>()), (int32_t)rank,
                                            (int32_t)bufs.size(0), (uint32_t)epoch, status ? status->data_ptr<int32_t>() : nullptr);
  if (st == L3CI_ERR_UNSUPPORTED) return std::nullopt;
  check_status(st, "flash_attention_decode_exchange");
  return result;
}

// reference: custom_kernels/custom_kernels.cu:369-389
Tensor rms_norm(Tensor input, Tensor weight, double eps) {
  check_bf16_cuda(input, "input");
  check_bf16_cuda(weight, "weight");
  TORCH_CHECK(input.dim() >= 1 && weight.dim() == 1 && weight.size(0) == input.size(-1),
              "weight must have the size of the last input dimension");
  TORCH_CHECK(weight.get_device() == input.get_device(), "input and weight on different devices");
  const c10::cuda::CUDAGuard guard(input.device());
  const int64_t E = input.size(-1);
  Tensor x = input.is_contiguous() ? input : input.contiguous();
  Tensor w = weight.is_contiguous() ? weight : weight.contiguous();
  Tensor out = torch::empty_like(x);
  const int64_t rows = E ? x.numel() / E : 0;
  check_status(l3ci_rms_norm(x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, E, E, E, (float)eps, current_stream()),
               "rms_norm");
  return out;
}

// (x + residual) and its RMSNorm in one pass: returns (sum, normed).  model.py:147-148 as one kernel.
std::tuple<Tensor, Tensor> add_rms_norm(Tensor x, Tensor residual, Tensor weight, double eps) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(residual, "residual");
  check_bf16_cuda(weight, "weight");
  TORCH_CHECK(x.sizes() == residual.sizes() && weight.dim() == 1 && weight.size(0) == x.size(-1), "shape mismatch");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor xc = x.contiguous(), rc = residual.contiguous(), w = weight.contiguous();
  Tensor sum = torch::empty_like(xc), out = torch::empty_like(xc);
  const int64_t E = xc.size(-1);
  check_status(l3ci_add_rms_norm(xc.data_ptr(), rc.data_ptr(), w.data_ptr(), sum.data_ptr(), out.data_ptr(),
                                 E ? xc.numel() / E : 0, E, (float)eps, current_stream()),
               "add_rms_norm");
  return {sum, out};
}

// silu(gate) * up with the roundings of the two bf16 tensor ops it replaces (model.py:134).
Tensor silu_mul(Tensor gate, Tensor up) {
  check_bf16_cuda(gate, "gate");
  check_bf16_cuda(up, "up");
  TORCH_CHECK(gate.sizes() == up.sizes(), "gate and up must have the same shape");
  TORCH_CHECK(gate.dim() >= 1, "gate must have at least one dimension");
  const c10::cuda::CUDAGuard guard(gate.device());
  // rows of a [..., 2F] GEMM result split in halves stay in place: only the last axis must be contiguous
  const int64_t cols = gate.size(-1);
  auto rows2d = [&](const Tensor& t) {
    Tensor f = t.dim() == 2 ? t : t.reshape({-1, cols});  // a view whenever the leading axes collapse
    return f.stride(-1) == 1 ? f : f.contiguous();
  };
  Tensor g = rows2d(gate), u = rows2d(up);
  Tensor out = torch::empty(gate.sizes(), gate.options());
  check_status(l3ci_silu_mul(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.size(0), cols, g.stride(0), u.stride(0),
                             current_stream()),
               "silu_mul");
  return out;
}

// Greedy decode step in place: argmax of logits [B, vocab] (bf16) per row, token written to out_tokens[b, steps[b]]
// and next_input[b], steps / positions / seq_lens advanced by one.  model.py:370-381 as one kernel.
void greedy_step(Tensor logits, Tensor out_tokens, Tensor steps, Tensor next_input, Tensor positions, Tensor seq_lens) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [B, vocab] with a contiguous last axis");
  const int64_t B = logits.size(0);
  auto check = [&](const Tensor& t, at::ScalarType ty, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.device() == logits.device() && t.scalar_type() == ty, name, ": wrong device or dtype");
  };
  check(out_tokens, at::kLong, "out_tokens");
  check(steps, at::kLong, "steps");
  check(next_input, at::kLong, "next_input");
  check(positions, at::kInt, "positions");
  check(seq_lens, at::kInt, "seq_lens");
  TORCH_CHECK(out_tokens.dim() == 2 && out_tokens.size(0) == B && out_tokens.stride(1) == 1, "out_tokens must be [B, G]");
  TORCH_CHECK(steps.numel() == B && next_input.numel() == B && positions.numel() >= B && seq_lens.numel() >= B &&
                  steps.is_contiguous() && next_input.is_contiguous() && positions.is_contiguous() && seq_lens.is_contiguous(),
              "per-sequence state must be contiguous with one entry per row");
  const c10::cuda::CUDAGuard guard(logits.device());
  check_status(l3ci_greedy_step(logits.data_ptr(), B, logits.size(1), logits.stride(0), out_tokens.data_ptr<int64_t>(),
                                out_tokens.stride(0), out_tokens.size(1), steps.data_ptr<int64_t>(),
                                next_input.data_ptr<int64_t>(), positions.data_ptr<int32_t>(), seq_lens.data_ptr<int32_t>(),
                                current_stream()),
               "greedy_step");
}

// Nucleus sampling step in place (model.py:367-369 + sample_top_p, model.py:400-423, + the bookkeeping of
// model.py:373-381): one token per row of logits [B, vocab] (bf16) drawn from the top-p nucleus of
// softmax(logits / temperature); written like greedy_step writes its argmax.
void top_p_step(Tensor logits, Tensor out_tokens, Tensor steps, Tensor next_input, Tensor positions, Tensor seq_lens,
                double temperature, double top_p, int64_t seed) {
  check_bf16_cuda(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [B, vocab] with a contiguous last axis");
  TORCH_CHECK(temperature > 0 && top_p > 0, "temperature and top_p must be positive (temperature 0: greedy_step)");
  const int64_t B = logits.size(0);
  auto check = [&](const Tensor& t, at::ScalarType ty, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.device() == logits.device() && t.scalar_type() == ty, name, ": wrong device or dtype");
  };
  check(out_tokens, at::kLong, "out_tokens");
  check(steps, at::kLong, "steps");
  check(next_input, at::kLong, "next_input");
  check(positions, at::kInt, "positions");
  check(seq_lens, at::kInt, "seq_lens");
  TORCH_CHECK(out_tokens.dim() == 2 && out_tokens.size(0) == B && out_tokens.stride(1) == 1, "out_tokens must be [B, G]");
  TORCH_CHECK(steps.numel() == B && next_input.numel() == B && positions.numel() >= B && seq_lens.numel() >= B &&
                  steps.is_contiguous() && next_input.is_contiguous() && positions.is_contiguous() && seq_lens.is_contiguous(),
              "per-sequence state must be contiguous with one entry per row");
  const c10::cuda::CUDAGuard guard(logits.device());
  check_status(l3ci_top_p_step(logits.data_ptr(), B, logits.size(1), logits.stride(0), (float)temperature, (float)top_p,
                               (uint64_t)seed, out_tokens.data_ptr<int64_t>(), out_tokens.stride(0), out_tokens.size(1),
                               steps.data_ptr<int64_t>(), next_input.data_ptr<int64_t>(), positions.data_ptr<int32_t>(),
                               seq_lens.data_ptr<int32_t>(), nullptr, nullptr, current_stream()),
               "top_p_step");
}

// reference: custom_kernels/custom_kernels.cu:418-442
Tensor rot_embed(Tensor input, Tensor freq) {
  check_bf16_cuda(input, "input");
  TORCH_CHECK(input.dim() == 4, "input must be [B, S, H, D]");
  TORCH_CHECK(freq.is_cuda() && freq.scalar_type() == torch::kFloat32, "freq must be a float32 CUDA tensor");
  TORCH_CHECK(freq.get_device() == input.get_device(), "input and freq on different devices");
  TORCH_CHECK(freq.numel() >= input.size(1) * input.size(3), "freq must hold [S, D] values");
  TORCH_CHECK(input.stride(3) == 1, "last dimension must be contiguous");
  const c10::cuda::CUDAGuard guard(input.device());
  Tensor f = freq.is_contiguous() ? freq : freq.contiguous();
  Tensor out = torch::empty(input.sizes(), input.options());
  check_status(l3ci_rot_embed(input.data_ptr(), f.data_ptr<float>(), out.data_ptr(), input.size(0), input.size(1),
                              input.size(2), input.size(3), input.stride(0), input.stride(1), input.stride(2),
                              current_stream()),
               "rot_embed");
  return out;
}

// Rotary embedding of q and k plus the cache write of k and v in one pass (model.py:100-108).
// qkv: [B, T, (n_head + 2*n_kv_head) * D]; caches: [maxB, maxLen, n_kv_head, D].  Returns rotated
// q as [B, T, n_head, D]; cache_k / cache_v are updated in place at [:, start_pos : start_pos + T].
//
// With `positions` (int32 [B] on the device) every sequence has its own position: token t of sequence b
// is at positions[b] + t, `freq` is then the WHOLE table and `start_pos` is ignored.  Nothing on the host
// depends on the positions, so a decode step written this way can be captured in a CUDA graph.
Tensor rot_embed_kv_cache(Tensor qkv, Tensor freq, Tensor cache_k, Tensor cache_v, int64_t start_pos,
                          int64_t n_head, int64_t n_kv_head, std::optional<Tensor> positions) {
  check_bf16_cuda(qkv, "qkv");
  check_bf16_cuda(cache_k, "cache_k");
  check_bf16_cuda(cache_v, "cache_v");
  TORCH_CHECK(qkv.dim() == 3 && qkv.stride(2) == 1, "qkv must be [B, T, (n_head + 2*n_kv_head) * D] with a contiguous last dimension");
  TORCH_CHECK(n_head > 0 && n_kv_head > 0 && qkv.size(2) % (n_head + 2 * n_kv_head) == 0, "qkv width does not match the head counts");
  const int64_t B = qkv.size(0), T = qkv.size(1), D = qkv.size(2) / (n_head + 2 * n_kv_head);
  TORCH_CHECK(cache_k.dim() == 4 && cache_k.sizes() == cache_v.sizes() && cache_k.strides() == cache_v.strides(),
              "cache_k and cache_v must be [maxB, maxLen, n_kv_head, D] with equal layout");
  TORCH_CHECK(cache_k.size(2) == n_kv_head && cache_k.size(3) == D && cache_k.stride(3) == 1 && cache_k.stride(2) == D,
              "cache rows must be [n_kv_head, D] contiguous");
  TORCH_CHECK(B <= cache_k.size(0), "batch does not fit the cache");
  TORCH_CHECK(freq.is_cuda() && freq.scalar_type() == torch::kFloat32 && freq.numel() >= T * D, "freq must be float32 [T, D]");
  if (positions) {
    TORCH_CHECK(positions->is_cuda() && positions->scalar_type() == torch::kInt32 && positions->dim() == 1 &&
                    positions->size(0) == B && positions->is_contiguous() && positions->get_device() == qkv.get_device(),
                "positions must be a contiguous int32 CUDA tensor of shape [B]");
    TORCH_CHECK(freq.dim() == 2 && freq.size(1) == D, "with positions, freq must be the whole [rows, D] table");
  } else {
    TORCH_CHECK(start_pos >= 0 && start_pos + T <= cache_k.size(1), "step does not fit the cache");
  }
  TORCH_CHECK(cache_k.get_device() == qkv.get_device() && cache_v.get_device() == qkv.get_device() &&
                  freq.get_device() == qkv.get_device(),
              "tensors on different devices");
  const c10::cuda::CUDAGuard guard(qkv.device());
  Tensor f = freq.is_contiguous() ? freq : freq.contiguous();
  Tensor q_out = torch::empty({B, T, n_head, D}, qkv.options());
  if (positions) {
    check_status(l3ci_rot_embed_kv_cache_at(qkv.data_ptr(), f.data_ptr<float>(), f.size(0), q_out.data_ptr(),
                                            cache_k.data_ptr(), cache_v.data_ptr(), positions->data_ptr<int32_t>(), B, T,
                                            n_head, n_kv_head, D, qkv.stride(0), qkv.stride(1), cache_k.stride(0),
                                            cache_k.stride(1), cache_k.size(1), current_stream()),
                 "rot_embed_kv_cache");
    return q_out;
  }
  check_status(l3ci_rot_embed_kv_cache(qkv.data_ptr(), f.data_ptr<float>(), q_out.data_ptr(), cache_k.data_ptr(),
                                       cache_v.data_ptr(), B, T, n_head, n_kv_head, D, qkv.stride(0), qkv.stride(1),
                                       cache_k.stride(0), cache_k.stride(1), start_pos, current_stream()),
               "rot_embed_kv_cache");
  return q_out;
}

// Synchronises the current stream of `like`'s device and reports whether a device-side bounded
// wait ran out in an earlier flash_attention_decode call on it (0 = fine).
int64_t flash_decode_status(Tensor like) {
  TORCH_CHECK(like.is_cuda(), "pass any tensor on the device to query");
  const c10::cuda::CUDAGuard guard(like.device());
  const auto stream = c10::cuda::getCurrentCUDAStream();
  const auto key = std::make_pair((int)like.get_device(), (int64_t)stream.id());
  Tensor buf;
  {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = workspaces().find(key);
    if (it == workspaces().end() || !it->second.buf.defined()) return 0;
    buf = it->second.buf;
  }
  return l3ci_flash_decode_poll(buf.data_ptr(), (size_t)buf.numel(), current_stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("flash_attention_decode", torch::wrap_pybind_function(flash_attention_decode), "flash_attention_decode",
        py::arg("query"), py::arg("keys"), py::arg("values"), py::kw_only(), py::arg("seq_lens") = py::none(),
        py::arg("out") = py::none(), py::arg("scale") = 0.0, py::arg("max_ctas") = 0);
  m.def("rms_norm", torch::wrap_pybind_function(rms_norm), "rms_norm", py::arg("input"), py::arg("weight"),
        py::arg("eps"));
  m.def("add_rms_norm", torch::wrap_pybind_function(add_rms_norm), "add_rms_norm", py::arg("x"), py::arg("residual"),
        py::arg("weight"), py::arg("eps"));
  m.def("silu_mul", torch::wrap_pybind_function(silu_mul), "silu_mul", py::arg("gate"), py::arg("up"));
  m.def("greedy_step", torch::wrap_pybind_function(greedy_step), "greedy_step", py::arg("logits"), py::arg("out_tokens"),
        py::arg("steps"), py::arg("next_input"), py::arg("positions"), py::arg("seq_lens"));
  m.def("top_p_step", torch::wrap_pybind_function(top_p_step), "top_p_step", py::arg("logits"), py::arg("out_tokens"),
        py::arg("steps"), py::arg("next_input"), py::arg("positions"), py::arg("seq_lens"), py::arg("temperature"),
        py::arg("top_p"), py::arg("seed"));
  m.def("rot_embed", torch::wrap_pybind_function(rot_embed), "rot_embed", py::arg("input"), py::arg("freq"));
  m.def("rot_embed_kv_cache", torch::wrap_pybind_function(rot_embed_kv_cache), "rot_embed_kv_cache",
        py::arg("qkv"), py::arg("freq"), py::arg("cache_k"), py::arg("cache_v"), py::arg("start_pos"),
        py::arg("n_head"), py::arg("n_kv_head"), py::kw_only(), py::arg("positions") = py::none());
  m.def("flash_attention_decode_partial", torch::wrap_pybind_function(flash_attention_decode_partial),
        "flash_attention_decode_partial", py::arg("query"), py::arg("keys"), py::arg("values"), py::kw_only(),
        py::arg("seq_lens") = py::none(), py::arg("scale") = 0.0, py::arg("max_ctas") = 0,
        py::arg("out_o") = py::none(), py::arg("out_lse") = py::none());
  m.def("lse_exchange_merge", torch::wrap_pybind_function(lse_exchange_merge), "lse_exchange_merge", py::arg("bufs"),
        py::arg("rank"), py::arg("epoch"), py::arg("B"), py::arg("Hq"), py::arg("D"), py::kw_only(),
        py::arg("status") = py::none());
  // which decode kernel a call of these sizes takes on `device` (0 = persistent grid, else 16*C + W of the static deal)
  m.def("flash_decode_kernel_choice", [](int64_t device, int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t n_seq, bool ragged) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
    return (int64_t)l3ci_flash_decode_kernel_choice((int32_t)B, (int32_t)Hq, (int32_t)Hkv, (int32_t)D, (int32_t)n_seq,
                                                    ragged ? 1 : 0);
  }, py::arg("device"), py::arg("B"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"), py::arg("n_seq"), py::arg("ragged") = false);
  m.def("flash_attention_decode_exchange", torch::wrap_pybind_function(flash_attention_decode_exchange),
        "flash_attention_decode_exchange", py::arg("query"), py::arg("keys"), py::arg("values"), py::arg("bufs"),
        py::arg("rank"), py::arg("epoch") = 0, py::kw_only(), py::arg("seq_lens") = py::none(), py::arg("out") = py::none(),
        py::arg("status") = py::none(), py::arg("scale") = 0.0, py::arg("max_ctas") = 0);
  m.def("flash_decode_exchange_bytes", [](int64_t ranks, int64_t B, int64_t Hq, int64_t D) {
    return (int64_t)l3ci_flash_decode_exchange_bytes((int32_t)ranks, (int32_t)B, (int32_t)Hq, (int32_t)D);
  });
  m.def("lse_exchange_bytes", [](int64_t ranks, int64_t B, int64_t Hq, int64_t D) {
    return (int64_t)l3ci_lse_exchange_bytes((int32_t)ranks, (int32_t)B, (int32_t)Hq, (int32_t)D);
  });
  m.def("lse_merge", torch::wrap_pybind_function(lse_merge), "lse_merge", py::arg("o_parts"), py::arg("lse_parts"));
  m.def("prefill_attention", torch::wrap_pybind_function(prefill_attention), "prefill_attention", py::arg("query"),
        py::arg("keys"), py::arg("values"), py::kw_only(), py::arg("start_pos") = 0, py::arg("scale") = 0.0,
        py::arg("variant") = 0);
  m.def("flash_decode_status", torch::wrap_pybind_function(flash_decode_status), "flash_decode_status",
        py::arg("like"));
  m.def("c_abi_version", [] { return std::string(l3ci_version()); });
}
