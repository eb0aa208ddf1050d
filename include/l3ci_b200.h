/*
 * l3ci_b200.h — C ABI of the sm_100a decode kernels (libl3ci_b200.so).
 *
 * Plain pointers and sizes only: no torch types cross this boundary.  Every
 * pointer is a DEVICE pointer on the device that is current for the calling
 * thread unless the comment says "host".  All tensors are bf16 (2-byte,
 * round-to-nearest-even) unless stated; strides are in ELEMENTS, not bytes.
 * Every call is asynchronous on `stream` and returns an l3ci_status.
 *
 * Each entry point names the reference interface it replaces
 * (paths are relative to the reference project root).
 */
#ifndef L3CI_B200_H_
#define L3CI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define L3CI_API __attribute__((visibility("default")))
#else
#define L3CI_API
#endif

/* Same object as cudaStream_t / CUstream; 0 is the legacy default stream. */
typedef struct CUstream_st* l3ci_stream_t;

typedef enum l3ci_status {
  L3CI_OK = 0,
  L3CI_ERR_INVALID = 1,      /* null pointer, non-positive size, heads not divisible ...   */
  L3CI_ERR_UNSUPPORTED = 2,  /* head size not 64/128, or q/kv head ratio outside 1..16      */
  L3CI_ERR_ALIGNMENT = 3,    /* a row does not start on 16 bytes / stride not 8-element      */
  L3CI_ERR_SCRATCH = 4,      /* scratch buffer smaller than l3ci_flash_decode_scratch_bytes  */
  L3CI_ERR_CUDA = 5,         /* a CUDA runtime/driver call failed; see l3ci_last_error()     */
  L3CI_ERR_DEVICE_WAIT = 6   /* a bounded device-side wait ran out (read back by _poll)      */
} l3ci_status;

/* Static description of a status code. */
L3CI_API const char* l3ci_status_string(int status);
/* Thread-local detail text of the last failing call on this thread ("" if none). */
L3CI_API const char* l3ci_last_error(void);
/* Library version, "major.minor.patch". */
L3CI_API const char* l3ci_version(void);

/* Bound of the device-side waits on OTHER CTAs or OTHER GPUs (the arrival counters of l3ci_flash_decode's
 * persistent kernel, default 2 s; the peers' flags of l3ci_lse_exchange_merge, default 1 s), in nanoseconds,
 * for the launches made after this call by any thread of the process; 0 restores the defaults.  Returns the
 * previous setting.  A wait that runs out makes the kernel give up in order: it records
 * L3CI_ERR_DEVICE_WAIT (scratch header / status word), skips the rows it could not finish and returns,
 * so the context stays usable.  A host that watches for a lost peer sets a limit near its step time; the
 * tests use it to let a wait run out in milliseconds.  No counterpart in the reference (one GPU, no waits). */
L3CI_API uint64_t l3ci_set_device_wait_limit_ns(uint64_t ns);

/* Programmatic dependent launch, on (1, the default) or off (0), for the launches made after this call; returns the
 * previous setting.  When on, the streaming kernels of this library (decode attention's static-deal kernel where it
 * runs without clusters, RMSNorm,
 * SiLU*mul, the rotary kernels, the token-choice steps) are launched so that their grid may be set up on the SMs
 * while the previous kernel of the stream is still draining; each of them waits (griddepcontrol.wait) for that
 * kernel's completion and the visibility of its writes before its first global access, so results and stream order
 * are what they are without it: what overlaps is the launch itself and the start of the CTAs (about a microsecond
 * per launch between kernels of this library, e.g. RoPE + cache write -> attention in a decode step, also inside a
 * captured CUDA graph).  No counterpart in the reference (legacy-stream <<<>>> launches). */
L3CI_API int l3ci_set_programmatic_launch(int on);

/* ------------------------------------------------------------------------------------------
 * RMSNorm.   out[r, :] = bf16( (float(x[r, :]) * rsqrt(mean(x[r, :]^2) + eps)) * float(w) )
 * fp32 arithmetic, one rounding.  Replaces `rms_norm(input, weight, eps)` and
 * `custom_rms_norm_kernel` (custom_kernels/custom_kernels.cu:340-389, bound at
 * custom_kernels/main.cpp:7; caller model.py:70-72).  `rows` is B*S of the reference's
 * [B, S, E] input.  Rows must start on 16 bytes and `embed` be a multiple of 8.
 * ------------------------------------------------------------------------------------------ */
L3CI_API int l3ci_rms_norm(const void* x, const void* weight, void* out,
                           int64_t rows, int64_t embed,
                           int64_t x_row_stride, int64_t out_row_stride,
                           float eps, l3ci_stream_t stream);

/* Residual add fused into RMSNorm:  s = bf16(x + residual) (written to sum_out), out = rmsnorm(s) * w.
 * Does in one pass what Block.forward does with an elementwise add followed by ln_2 / the next block's
 * ln_1 (model.py:147-148).  All tensors dense [rows, embed]. */
L3CI_API int l3ci_add_rms_norm(const void* x, const void* residual, const void* weight,
                               void* sum_out, void* out, int64_t rows, int64_t embed, float eps,
                               l3ci_stream_t stream);

/* SwiGLU gate:  out = bf16( bf16(silu(gate)) * up ) over [rows, cols] (cols a multiple of 8), out dense,
 * gate and up with their own row strides in elements (so both may be halves of one [rows, 2*cols] GEMM
 * result).  The `F.silu(self.c_fc2(x)) * self.c_fc(x)` of MLP.forward (model.py:134) as one kernel. */
L3CI_API int l3ci_silu_mul(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                           int64_t gate_row_stride, int64_t up_row_stride, l3ci_stream_t stream);

/* Greedy decode step: for every row b of bf16 logits [rows, vocab] (row_stride elements apart),
 *   tok = argmax (ties: smallest index, as torch.argmax; NaN counts as the maximum);
 *   out_tokens[b * out_stride + steps[b]] = tok (if steps[b] < out_cols);  steps[b] += 1;
 *   next_input[b] = tok;  positions[b] += 1;  seq_lens[b] += 1.
 * Any of out_tokens / steps / next_input / positions / seq_lens may be null (without steps the token goes
 * to out_tokens[b * out_stride]).  One kernel for what the reference's greedy branch does with an argmax and
 * several elementwise launches per generated token (model.py:370-381). */
L3CI_API int l3ci_greedy_step(const void* logits, int64_t rows, int64_t vocab, int64_t row_stride,
                              int64_t* out_tokens, int64_t out_stride, int64_t out_cols, int64_t* steps,
                              int64_t* next_input, int32_t* positions, int32_t* seq_lens,
                              l3ci_stream_t stream);

/* Nucleus (top-p) sampling decode step: for every row b of bf16 logits [rows, vocab],
 *   probs = softmax(logits / temperature); nucleus = the entries whose PRECEDING probability mass, in descending
 *   order of probability (equal entries in index order), is <= top_p; tok = one draw from the nucleus with
 *   probabilities renormalised;
 * then the same bookkeeping as l3ci_greedy_step.  What `sample_top_p` does with a full-vocabulary sort, a
 * cumulative sum, a multinomial draw and a gather (model.py:367-369, 400-423), as one kernel without a sort.  The
 * draw of row b at step steps[b] (0 without steps) comes from a Philox4x32-10 stream keyed by `seed`: the same
 * (seed, row, step) gives the same token, different steps give independent draws, and nothing on the host changes
 * from step to step (the call can sit in a CUDA graph).  temperature and top_p must be positive (temperature 0 is
 * the greedy branch of the reference: l3ci_greedy_step).  Optional outputs for inspection: nucleus_count[b]
 * (entries kept) and nucleus_mass[b] (their probability mass before renormalisation).  Masses are summed in fp32:
 * an entry whose preceding mass is within ~1e-6 of top_p may fall on either side. */
L3CI_API int l3ci_top_p_step(const void* logits, int64_t rows, int64_t vocab, int64_t row_stride, float temperature,
                             float top_p, uint64_t seed, int64_t* out_tokens, int64_t out_stride, int64_t out_cols,
                             int64_t* steps, int64_t* next_input, int32_t* positions, int32_t* seq_lens,
                             int32_t* nucleus_count, float* nucleus_mass, l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Rotary embedding, interleaved-pair (Meta) convention:
 *   (x', y') = (x*c - y*s, x*s + y*c) for (x, y) = in[.., 2i], in[.., 2i+1] and
 *   (c, s) = freq[tok*D + 2i], freq[tok*D + 2i + 1]; fp32, products rounded separately,
 *   one rounding to bf16.
 * `x` is [B, S, H, D] with element strides (sb, ss, sh, 1); `freq` is fp32 [S, D];
 * `out` is dense [B, S, H, D].  Replaces `rot_embed(input, freq)` and
 * `custom_rot_embed_kernel` (custom_kernels/custom_kernels.cu:391-442, bound at
 * custom_kernels/main.cpp:8; callers model.py:100-101).
 * ------------------------------------------------------------------------------------------ */
L3CI_API int l3ci_rot_embed(const void* x, const float* freq, void* out,
                            int64_t B, int64_t S, int64_t H, int64_t D,
                            int64_t sb, int64_t ss, int64_t sh,
                            l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Rotary embedding fused with the KV-cache write: one pass over the fused projection output
 * qkv[B, T, (Hq + 2*Hkv) * D] (q heads, then k heads, then v heads along the last axis):
 *   q_out[b, t, h, :]                 = rope(q)       dense [B, T, Hq, D]
 *   cache_k[b, start_pos + t, h, :]   = rope(k)
 *   cache_v[b, start_pos + t, h, :]   = v
 * Replaces the two `rot_embed` calls plus the two cache copies of
 * CausalSelfAttention.forward (model.py:100-108).  `freq` is already sliced to the T
 * positions of this step, as model.py:209 does.  Caches are [maxB, maxLen, Hkv, D] with
 * element strides (cache_sb, cache_st, D, 1).
 * ------------------------------------------------------------------------------------------ */
L3CI_API int l3ci_rot_embed_kv_cache(const void* qkv, const float* freq, void* q_out,
                                     void* cache_k, void* cache_v,
                                     int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                                     int64_t qkv_sb, int64_t qkv_st,
                                     int64_t cache_sb, int64_t cache_st,
                                     int64_t start_pos, l3ci_stream_t stream);

/* The same pass with the position of every sequence read from device memory: token t of sequence b
 * sits at position positions[b] + t, takes row positions[b] + t of the WHOLE rotary table
 * `freq_table` (fp32 [freq_rows, D]) and is written to that row of the caches.  A position outside
 * the table or beyond cache_len is skipped.  This is the form a decode loop needs when it is captured
 * in a CUDA graph (no host-side start_pos) or when sequences of a batch are at different positions;
 * it extends model.py:100-108 / :209, which have one start_pos for the batch. */
L3CI_API int l3ci_rot_embed_kv_cache_at(const void* qkv, const float* freq_table, int64_t freq_rows,
                                        void* q_out, void* cache_k, void* cache_v,
                                        const int32_t* positions,
                                        int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                                        int64_t qkv_sb, int64_t qkv_st,
                                        int64_t cache_sb, int64_t cache_st, int64_t cache_len,
                                        l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Split-KV flash-decode attention for one query token per sequence over a GQA KV cache.
 * Replaces `flash_attention_decode(query, keys, values)` with its split-KV and combine
 * kernels (custom_kernels/custom_kernels.cu:13-177, 179-223, 233-338, bound at
 * custom_kernels/main.cpp:6; caller model.py:118, benchmark_kernel.py:25).
 * ------------------------------------------------------------------------------------------ */
typedef struct l3ci_flash_decode_args {
  const void* q;         /* [B, Hq, 1, D], element strides (q_sb, q_sh, -, 1)                  */
  const void* k;         /* [B, Hkv, n_seq, D], element strides (k_sb, k_sh, k_st, 1)          */
  const void* v;         /* [B, Hkv, n_seq, D], element strides (v_sb, v_sh, v_st, 1)          */
  void* out;             /* bf16 [B, Hq, 1, D], element strides (o_sb, o_sh, -, 1); may be NULL
                            when o_partial/lse are given                                       */
  float* o_partial;      /* optional fp32 [B, Hq, D] dense: softmax-normalised output of THIS
                            KV range, for a later l3ci_lse_merge across KV shards             */
  float* lse;            /* optional fp32 [B, Hq]: natural-log sum-exp of the scaled scores of
                            this KV range (-inf for an empty range); required with o_partial  */
  const int32_t* seq_lens; /* optional int32 [B]: valid tokens per sequence (clamped to
                            [0, n_seq]); NULL = every sequence has n_seq tokens               */
  void* scratch;         /* >= l3ci_flash_decode_scratch_bytes(...) bytes, 256-byte aligned,
                            zero-filled ONCE before its first use; the kernel leaves it ready
                            for the next call on the same stream, of any shape with
                            B * Hkv <= 65536 (beyond that: zero it again when the shape changes).
                            Two calls that overlap on the GPU must not share it                */
  size_t scratch_bytes;
  int32_t B, Hq, Hkv, D, n_seq;
  int64_t q_sb, q_sh;
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  int64_t o_sb, o_sh;
  float scale;           /* softmax scale; <= 0 selects 1/sqrt(D) (custom_kernels.cu:253)      */
  int32_t max_ctas;      /* 0 = library's choice between its two kernels: a persistent grid that  *
                          * fills the device and balances any mix of lengths, and one that deals  *
                          * units statically to warps, CTAs or clusters and merges in shared      *
                          * memory (Hq/Hkv <= 8; faster up to a few MB of cache per CTA).          *
                          * >0 = the persistent grid, capped at this size.  -1 = the static kernel *
                          * with its own split; -(16*C + W) = with C CTAs per unit (1, 2, 4, 8) and *
                          * W of a CTA's 8 warps per unit (1, 2, 4, 8; 8 if C > 1): tests, tuning.  */
  l3ci_stream_t stream;
} l3ci_flash_decode_args;

/* Bytes of scratch one call needs on the current device (depends on its SM count). */
L3CI_API size_t l3ci_flash_decode_scratch_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D);

/* Which kernel l3ci_flash_decode runs on the current device for a call of these sizes with max_ctas = 0
 * (ragged: seq_lens given): 0 = the persistent grid, else 16*C + W of the static deal (C CTAs per unit, W warps
 * per unit), the code that max_ctas = -(16*C + W) asks for.  -1 for sizes the call would refuse.  For logs and
 * benchmarks; the choice is a fit to measurements and may change between versions. */
L3CI_API int l3ci_flash_decode_kernel_choice(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t n_seq, int32_t ragged);

L3CI_API int l3ci_flash_decode(const l3ci_flash_decode_args* args);

/* ------------------------------------------------------------------------------------------
 * l3ci_flash_decode without any scratch from the caller.  (No counterpart in the reference, which
 * allocates three scratch tensors inside every call: custom_kernels/custom_kernels.cu:269-271.)
 *
 * Who needs it: a host that cannot create device memory at the moment it wants attention computed.
 * Typical cases are a serving process that handed the whole GPU to its own arena at start-up (the KV
 * cache is sized to fill the card, so a later cudaMalloc has nothing to take from and may not be
 * permitted by the embedding runtime at all), and code on a path where an allocation call would stall
 * or is forbidden by policy (a latency-critical decode loop that must not enter the driver's
 * allocator).  Such a caller still owns q, k, v and the output; only the merge scratch is missing.
 *
 * This entry point takes the same argument struct; its `scratch` and `scratch_bytes` fields are ignored.
 * The scratch is an L3CI_STATIC_SCRATCH_BYTES array that is part of the library's device code, so
 * every GPU on which the library is used carries it until the process ends.  The call makes no
 * cudaMalloc/cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *  - the shape must fit: l3ci_flash_decode_scratch_bytes(B, Hq, Hkv, D) <= L3CI_STATIC_SCRATCH_BYTES
 *    and B * Hkv <= 65536; otherwise L3CI_ERR_SCRATCH with a message that states both sizes
 *    (12 MiB covers head ratios up to 4 at head size 128, up to 9 at head size 64, on a 148-SM part);
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current); make that first call outside any stream capture;
 *  - all calls on a device share the one array and find in it what the previous call left: the entry
 *    point clears the part that has to start at zero itself (one small cudaMemsetAsync on `stream`),
 *    but two calls that overlap on the GPU (different streams, or different host threads without
 *    ordering) race on it.  Use one stream per device for this entry point, or l3ci_flash_decode with
 *    one scratch buffer per stream;
 *  - the device-side status word is not readable afterwards (l3ci_flash_decode_poll needs a caller
 *    buffer).
 * ------------------------------------------------------------------------------------------ */
#define L3CI_STATIC_SCRATCH_BYTES (12u << 20)
L3CI_API int l3ci_flash_decode_static(const l3ci_flash_decode_args* args);

/* Reads back (synchronising `stream`) the device-side status word kept in `scratch`:
 * L3CI_OK, or L3CI_ERR_DEVICE_WAIT if a bounded wait on a bulk copy ran out in an earlier
 * call.  Clears the word and the arrival counters so the scratch can be used again. */
L3CI_API int l3ci_flash_decode_poll(void* scratch, size_t scratch_bytes, l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Causal GQA attention for T > 1 new tokens per sequence (prefill / chunked prefill).
 *
 * The reference sends this case to PyTorch (model.py:114-116,
 * F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True) over cache rows [0, T)); this
 * entry point has no counterpart in its extension.  Query t of a sequence attends keys
 * j <= start_pos + t, j < n_keys (start_pos = 0, n_keys = T is the reference's call).
 * ------------------------------------------------------------------------------------------ */
typedef struct l3ci_prefill_args {
  const void* q;          /* bf16 [B, Hq, T, D] by strides (elements); last axis contiguous          */
  const void* k;          /* bf16 [B, Hkv, n_keys, D] by strides; rows 16-byte aligned               */
  const void* v;
  void* out;              /* bf16 [B, Hq, T, D] by strides                                            */
  int32_t* status;        /* optional device word that receives L3CI_ERR_DEVICE_WAIT if a bounded wait
                             on a bulk copy runs out; may be null                                      */
  int32_t B, Hq, Hkv, D;  /* D in {64, 128}; Hq a multiple of Hkv                                      */
  int32_t T, n_keys, start_pos;
  int64_t q_sb, q_sh, q_st, k_sb, k_sh, k_st, v_sb, v_sh, v_st, o_sb, o_sh, o_st;
  float scale;            /* <= 0: 1/sqrt(D)                                                           */
  int32_t variant;        /* 0: choose (tcgen05 kernel from 128 query rows on, where q and out rows are 16-byte
                             aligned); 1: the tcgen05 / tensor-memory kernel; 2: the mma.sync kernel   */
  l3ci_stream_t stream;
} l3ci_prefill_args;

L3CI_API int l3ci_prefill_attention(const l3ci_prefill_args* args);

/* ------------------------------------------------------------------------------------------
 * Log-sum-exp merge of `parts` partial results of the same queries over disjoint KV ranges
 * (the per-GPU results of a sequence-sharded cache):
 *   L = logsumexp_p lse[p, r];  out[r, :] = bf16( sum_p exp(lse[p, r] - L) * o[p, r, :] )
 * o is fp32 [parts, rows, D] dense, lse fp32 [parts, rows], rows = B*Hq; out is bf16 with
 * element strides (o_sb, o_sh) over (b, h).  Does for GPU shards what the reference's combine
 * kernel intends for its 64-token steps (custom_kernels/custom_kernels.cu:179-223).
 * ------------------------------------------------------------------------------------------ */
L3CI_API int l3ci_lse_merge(const float* o, const float* lse, void* out,
                            int32_t parts, int32_t B, int32_t Hq, int32_t D,
                            int64_t o_sb, int64_t o_sh, l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * The same merge with the exchange fused in: every rank pushes its shard result into its peers'
 * memory over NVLink and merges what the peers pushed to it, in ONE kernel, with no collective
 * library in between.  No counterpart in the reference (single GPU).
 *
 * Every rank owns a buffer of l3ci_lse_exchange_bytes(ranks, B, Hq, D) bytes, zero-filled once, that
 * all ranks of the box can address (CUDA IPC / torch symmetric memory); `bufs` is a DEVICE array of
 * `ranks` base pointers as seen from this process, bufs[rank] being the local one.  Layout (fp32):
 *   data    [2][ranks][B*Hq*D outputs, then B*Hq lse padded to a multiple of 4 floats]
 *   flags   [2][ranks][B*Hq] (uint32, after the data, padded to a multiple of 4 words)
 *   staging one more slot of the data layout
 *   control 4 words: call number, finished warps, 2 unused
 * A call with epoch e (1, 2, 3, ... the same on all ranks) uses parity e & 1.  Before the call the
 * rank's own shard result must be in ITS OWN slot [e & 1][rank] (l3ci_flash_decode with o_partial /
 * lse pointing there).  With epoch 0 the call number is kept on the device instead (control word 0
 * + 1, advanced by the kernel itself) and the rank's own result is expected in the staging slot, a
 * fixed address: such a call has no host-side state and can be captured in a CUDA graph; use one of
 * the two forms per buffer, not both.  The kernel waits at most one second for the peers' rows; if
 * that runs out it writes L3CI_ERR_DEVICE_WAIT to *status (optional device word) and leaves `out`
 * unwritten for those rows.  Every rank must call it, on its own GPU, once per epoch.
 * ------------------------------------------------------------------------------------------ */
L3CI_API size_t l3ci_lse_exchange_bytes(int32_t ranks, int32_t B, int32_t Hq, int32_t D);
L3CI_API int l3ci_lse_exchange_merge(void* const* bufs, int32_t rank, int32_t ranks, uint32_t epoch,
                                     void* out, int32_t B, int32_t Hq, int32_t D,
                                     int64_t o_sb, int64_t o_sh, int32_t* status,
                                     l3ci_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Decode attention over a sequence-sharded cache in ONE launch per GPU and step: l3ci_flash_decode on this GPU's
 * slice of the cached tokens, with the exchange of the per-GPU results and their log-sum-exp merge done in the
 * kernel's tail (every thread sends its finished output element to the peers as one 64-bit word {value, call
 * number} with a plain store over NVLink, polls its own buffer for the peers' words, merges).  No counterpart in
 * the reference (single GPU); does for GPU shards what its combine kernel intends for 64-token steps
 * (custom_kernels/custom_kernels.cu:179-223).
 *
 * `args` as for l3ci_flash_decode (k, v, n_seq, seq_lens describe THIS rank's slice; `out` receives the merged
 * attention on every rank; o_partial / lse must be null; scratch is not used).  `bufs` is a DEVICE array of
 * `ranks` (<= 8) base pointers, as seen from this process, of the ranks' exchange buffers of
 * l3ci_flash_decode_exchange_bytes(ranks, B, Hq, D) bytes each, zero-filled once, bufs[rank] the local one (CUDA IPC
 * / torch symmetric memory).  `epoch` numbers the calls (1, 2, 3, ... the same on all ranks); with 0 the number
 * is kept in the buffer and advanced by the kernel, so a step has no host state and can be captured in a CUDA
 * graph.  Every rank must make the call once per epoch.  The wait for the peers is bounded (1 s, see
 * l3ci_set_device_wait_limit_ns): when it runs out, *status (optional device word) becomes L3CI_ERR_DEVICE_WAIT and
 * the elements concerned stay unwritten.  Sizes that l3ci_flash_decode would hand to its persistent kernel
 * (Hq/Hkv > 8, very long or lopsided slices) return L3CI_ERR_UNSUPPORTED: use l3ci_flash_decode with o_partial /
 * lse followed by l3ci_lse_exchange_merge for those.
 * ------------------------------------------------------------------------------------------ */
L3CI_API size_t l3ci_flash_decode_exchange_bytes(int32_t ranks, int32_t B, int32_t Hq, int32_t D);
L3CI_API int l3ci_flash_decode_exchange(const l3ci_flash_decode_args* args, void* const* bufs, int32_t rank,
                                        int32_t ranks, uint32_t epoch, int32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* L3CI_B200_H_ */
