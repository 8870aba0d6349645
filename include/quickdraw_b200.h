/* quickdraw_b200 — C ABI of the sm_100a batch-one decode kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void*), launches asynchronously on that stream, allocates nothing, owns no device
 * memory and returns one of the QD_* codes below.  No C++ exception crosses this
 * boundary.  The functions mirror the host functions of the reference's kernel
 * backends; each declaration names the reference interface it replaces.
 *
 * Formats: bf16 activations; NVFP4 weights as uint8 codes [out, in/2] (low nibble =
 * even input), float8_e4m3fn block scales [out, in/group], fp32 global scale.
 */
#ifndef QUICKDRAW_B200_H
#define QUICKDRAW_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    QD_OK = 0,
    QD_ERR_ARG = 1,          /* contract violation detected before launch */
    QD_ERR_LAUNCH = 2,       /* the CUDA runtime refused the launch */
    QD_ERR_TIMEOUT = 3,      /* a bounded device-side wait ran out (status word) */
    QD_ERR_UNSUPPORTED = 4,  /* shape outside what the entry point covers */
    QD_ERR_TOO_LARGE = 5     /* the shape needs more than a fixed-capacity buffer holds */
};

int qd_version(void);
const char* qd_error_string(int code);

/* rms_norm(x, gamma, eps) — quickdraw/kernel/triton/norm.py:18-23, qwen.py:19-22.
 * x, out: [rows, width] bf16 (is_fp32 = 0) or fp32 (1); gamma fp32 [width]. */
int qd_rms_norm(const void* x, const float* gamma, void* out, int rows, int width, float eps,
                int is_fp32, void* stream);

/* The step's fused residual update — quickdraw/models/qwen.py:214-217.
 * normed = bf16(rms_norm(x + residual) * gamma), residual_out = bf16(x + residual);
 * residual may be NULL (zero); residual_out must not alias an input. */
int qd_add_rms_norm(const void* x, const void* residual, const float* gamma, void* normed,
                    void* residual_out, int width, float eps, void* stream);

/* nvfp4_gemv(x, proj, routing_weight=None) — quickdraw/kernel/cute/matvec.py:146-149,
 * quickdraw/kernel/triton/matvec.py:65-81, arithmetic qwen.py:36-54.
 * routing_weight: device fp32 scalar or NULL.  force_generic: 0 = the fastest kernel that
 * covers the shape (2048 / 4096 inputs, rows a multiple of 8, non-negative block scales: the
 * block-scaled FP4 tensor-core kernel, tcgen05 kind::mxf4nvf4, which reads codes and scales
 * straight from this layout and takes the activations as eight exact 2-bit digit planes;
 * else the streaming kernel), 2 = the streaming kernel (weights dequantised in registers,
 * mma.sync), 1 = the shape-generic kernel. */
int qd_nvfp4_gemv(const void* x, const void* codes, const void* scales, const float* global,
                  const float* routing_weight, void* y, int rows, int in_features,
                  int group_size, int force_generic, void* stream);

/* matmul(x, proj) for a chunk of tokens (prefill) — quickdraw/kernel/triton/matvec.py:118-163,
 * NVFP4 branch: y[t, n] = bf16( global * sum_k x[t, k] * bf16(e2m1[n, k] * e4m3 scale) ) on the
 * tensor cores (tcgen05, accumulator in tensor memory).  x bf16 [tokens, in_features]
 * contiguous, y bf16 [tokens, out_features]; in_features % 64 == 0, out_features % 8 == 0,
 * pointers 16-byte aligned.  status: device word, bit 0 is set if a bounded wait ran out. */
int qd_nvfp4_matmul(const void* x, const void* codes, const void* scales, const float* global, void* y,
                    int tokens, int out_features, int in_features, int group_size,
                    unsigned int* status, void* stream);

/* The same product for at most 32 token rows (the dense projections of a decode batch): every
 * weight tile is decoded once on the warp-level tensor-core instruction with the tokens as
 * columns; no 128-token tiles.  scratch: qd_nvfp4_matmul_rows_scratch_bytes(in_features) bytes,
 * 16-byte aligned, receives the token rows as f16; convert = 0 reuses what the previous call with
 * this scratch area converted (several projections of one input).  x_up (or NULL): the input rows
 * are bf16(bf16(silu(x)) * x_up), the SwiGLU of two projections (qwen.py:184, 191), formed on the
 * way in.  in_features % 512 == 0,
 * out_features % 16 == 0, else QD_ERR_UNSUPPORTED. */
long long qd_nvfp4_matmul_rows_scratch_bytes(int in_features);
int qd_nvfp4_matmul_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global, void* y,
                         int tokens, int out_features, int in_features, int group_size, void* scratch,
                         int convert, void* stream);
/* The same for up to three matrices that read the same input (q | k | v, qkv | z, gate | up) in one
 * launch; matrices past `count` are ignored (NULL). */
int qd_nvfp4_matmul_rows3(const void* x, const void* x_up, int tokens, int in_features, int group_size,
                          void* scratch, int convert, int count,
                          const void* codes0, const void* scales0, const float* global0, void* y0, int out0,
                          const void* codes1, const void* scales1, const float* global1, void* y1, int out1,
                          const void* codes2, const void* scales2, const float* global2, void* y2, int out2,
                          void* stream);

/* Activation quantiser of the FP4 x FP4 ("W4A4") product that quickdraw's todo.md:13 asks to
 * validate separately from the W4A16 path: x bf16 [tokens, in_features] -> E2M1 codes
 * [tokens, in_features / 2] (low nibble = even input), one E4M3 scale per sixteen inputs
 * [tokens, in_features / 16] and one fp32 scale for the chunk, i.e. the NVFP4Linear layout of
 * quickdraw/models/weights.py:29-47 for the activation operand.  global = amax / (6 * 448),
 * block scale = e4m3(block amax / (6 global)), code = e2m1(x / (scale * global)), all round to
 * nearest even.  amax_scratch: one device word.  in_features % 16 == 0, 16-byte aligned pointers. */
int qd_nvfp4_quantize_act(const void* x, int tokens, int in_features, void* codes, void* scales,
                          float* global, unsigned int* amax_scratch, void* stream);

/* matmul with both operands NVFP4 on the block-scaled tensor core (tcgen05.mma kind::mxf4nvf4,
 * one E4M3 scale per sixteen inputs of either operand read from tensor memory): y[t, n] =
 * bf16( x_global * w_global * sum_k xq[t, k] * wq[n, k] ), fp32 accumulation in tensor memory.
 * The prefill projection of quickdraw/kernel/triton/matvec.py:118-163 with the activations
 * quantised by qd_nvfp4_quantize_act.  in_features % 256 == 0, out_features % 128 == 0,
 * pointers 16-byte aligned.  wide_tiles: 1 = 256 weight rows per block and MMA (out_features
 * % 256 == 0), 0 = 128, -1 = the library chooses.  status: device word, bit 0 is set if a
 * bounded wait ran out. */
int qd_nvfp4_matmul_w4a4(const void* x_codes, const void* x_scales, const float* x_global,
                         const void* w_codes, const void* w_scales, const float* w_global, void* y,
                         int tokens, int out_features, int in_features, int wide_tiles,
                         unsigned int* status, void* stream);

/* grouped_matmul(x, bank, grouping, routing=None) for the routed experts of a chunk of tokens —
 * quickdraw/kernel/triton/moe.py:99-151.  Routes are the (token, slot) pairs of the chunk
 * sorted by expert (stable): order[r] = route index of sorted row r, rows [boundaries[e],
 * boundaries[e+1]) belong to expert e (int32, device).  by_token: the input row of sorted row r
 * is order[r] / topk (gate, up), else r (down).  scatter: the output row is order[r] (down),
 * else r.  routing (fp32 per route, or NULL) selects the routed double rounding
 * y = bf16(bf16(acc) * bf16(global * routing)).  max_rows_per_expert bounds the rows of any
 * one expert (routes is always a valid bound); nothing is synchronised with the host. */
int qd_nvfp4_grouped_matmul(const void* x, const void* codes, const void* scales, const float* global,
                            const int32_t* order, const int32_t* boundaries, const float* routing,
                            void* y, int routes, int experts, int topk, int out_features,
                            int in_features, int group_size, int by_token, int scatter,
                            int global_per_expert, int max_rows_per_expert, unsigned int* status,
                            void* stream);

/* The same product when an expert receives only a few rows (a short chunk, a decode batch):
 * every expert that got routes is read once, its NVFP4 rows decoded once per routes_per_pass
 * routes (8 or 32; 0 = the library's choice) and
 * multiplied on the warp-level tensor-core instruction (the grouped branch of
 * quickdraw/kernel/triton/moe.py:99-151 at small M).  Arguments as above; x_up (or NULL) as in
 * qd_nvfp4_matmul_rows.  scratch: qd_nvfp4_expert_rows_scratch_bytes(input rows, in_features) bytes,
 * 16-byte aligned, receives the input rows as f16 (input rows = routes / topk with by_token, else
 * routes); convert = 0 reuses what the previous call left there (the gate and up products of the
 * same tokens).  in_features
 * 512, 1024 or 2048, out_features a multiple of 16, else QD_ERR_UNSUPPORTED. */
long long qd_nvfp4_expert_rows_scratch_bytes(int rows, int in_features);
int qd_nvfp4_expert_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global,
                         const int32_t* order, const int32_t* boundaries, const float* routing, void* y,
                         int routes, int experts, int topk, int out_features, int in_features,
                         int group_size, int by_token, int scatter, int global_per_expert,
                         int routes_per_pass, void* scratch, int convert, void* stream);

/* Two banks of the same shape against the same routes in ONE launch: the gate and up products of the
 * routed experts (quickdraw/models/qwen.py:176-186).  y and y2 are what two calls of
 * qd_nvfp4_expert_rows with by_token = 1, no routing weights and results in sorted order give. */
int qd_nvfp4_expert_rows2(const void* x, const void* codes, const void* scales, const float* global, void* y,
                          const void* codes2, const void* scales2, const float* global2, void* y2,
                          const int32_t* order, const int32_t* boundaries,
                          int routes, int experts, int topk, int out_features, int in_features,
                          int group_size, int global_per_expert, int routes_per_pass, void* scratch, int convert,
                          void* stream);

/* The kernels of the chunk and batch entry points below wait, as their first instruction, for the
 * kernel before them in the stream and are launched as its programmatic dependents, so that their
 * launch overlaps its last blocks (512-token chunk: 32.2 -> 30.9 ms).  on = 0 launches them
 * ordinarily: measured faster while a step is captured into a CUDA graph.  Returns the old setting. */
int qd_set_chained_launches(int on);

/* ---- Sequence forms for a chunk of prompt tokens (the 2-D branches of
 * quickdraw/kernel/triton/{norm,delta,attention,moe}.py, qwen.py:66-241): the single-token
 * arithmetic row by row.  All activations bf16 [tokens, width] contiguous. */
int qd_seq_add_rms_norm(const void* x, const void* residual, const float* gamma, void* normed,
                        void* residual_out, int tokens, int width, float eps, void* stream);
/* y[t, n] = bf16(x[t] . w[n]) for a small bf16 matrix (router, shared gate, DeltaNet a / b). */
int qd_seq_bf16_matmul(const void* x, const void* w, void* y, int tokens, int rows, int width, void* stream);
/* Two such matrices of the same input in one launch (a and b; router and shared gate). */
int qd_seq_bf16_matmul2(const void* x, const void* w0, void* y0, int rows0, const void* w1, void* y1, int rows1,
                        int tokens, int width, void* stream);
/* short convolution walked along the chunk; conv_state ends with the last width - 1 inputs */
int qd_seq_gdn_conv(const void* mixed, const void* taps, void* conv_state, void* out, int tokens,
                    int channels, int width, void* stream);
/* delta-rule recurrence walked along the chunk; rec_state updated in place; a, b [tokens, value_heads] */
int qd_seq_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                          const void* dt_bias, float* rec_state, void* out, int tokens, int key_heads,
                          int value_heads, int key_dim, int value_dim, void* stream);
/* The same recurrence for a long run of tokens, 64 at a time on the tensor cores (closed form of
 * the delta rule within a chunk; the reference walks the run token by token,
 * quickdraw/kernel/triton/delta.py:57-81): tf32 operands, fp32 sums, about 1e-3 relative from
 * the token-by-token form.  key_dim 128, value_dim % 32 == 0, else QD_ERR_UNSUPPORTED.
 * scratch: qd_seq_gdn_chunk_scratch_bytes(tokens, value_heads) bytes, 16-byte aligned. */
long long qd_seq_gdn_chunk_scratch_bytes(int tokens, int value_heads);
int qd_seq_gdn_recurrence_chunked(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                  const void* dt_bias, float* rec_state, void* out, int tokens, int key_heads,
                                  int value_heads, int key_dim, int value_dim, void* scratch, void* stream);
/* q/k norm + RoPE + cache write for positions position0 .. position0 + tokens - 1, then causal
 * attention of every token over [0, its position], gated.  k_cache / v_cache: this layer's
 * [capacity, kv_heads, head_dim]; q_scratch bf16 [tokens, q_heads, head_dim]. */
int qd_seq_attention(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                     const void* k_norm, void* k_cache, void* v_cache, void* q_scratch, void* out,
                     int tokens, int position0, int capacity, int q_heads, int kv_heads, int head_dim,
                     int rotary_dim, float theta, float eps, void* stream);
int qd_seq_route_topk(const void* logits, int tokens, int experts, int topk, int32_t* ids, float* weights,
                      void* stream);
/* ---- Small-batch decode with per-sequence state: one token of each of `batch` independent
 * sequences per call.  The reference decodes one sequence (quickdraw/engine/engine.py:114-127);
 * these are its single-token operators (_conv_kernel / _delta_kernel of
 * quickdraw/kernel/triton/delta.py:37-121, _prepare / _attend of
 * quickdraw/kernel/triton/attention.py:10-100) with the sequence as one more grid dimension:
 * inputs and outputs hold one row set per sequence, the state of sequence b starts
 * `*_stride` elements after that of sequence b - 1.  The other operators of the step are the
 * chunk forms above (rows are independent there). */
int qd_batch_gdn_conv(const void* mixed, const void* taps, void* conv_state, long long state_stride,
                      void* out, int batch, int channels, int width, void* stream);
/* key_dim == 128 */
int qd_batch_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                            const void* dt_bias, float* rec_state, long long state_stride, void* out,
                            int batch, int key_heads, int value_heads, int key_dim, int value_dim,
                            void* stream);
/* positions: device int32 [batch], each < capacity; scratch: batch * qd_attn_scratch_floats()
 * floats; counters: batch * kv_heads zeroed uint32 (left zero). */
int qd_batch_attn_decode(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                         const void* k_norm, void* k_cache, void* v_cache, long long cache_stride,
                         void* out, float* scratch, unsigned int* counters, const int* positions,
                         int batch, int capacity, int q_heads, int kv_heads, int head_dim,
                         int rotary_dim, float theta, float eps, int splits, void* stream);

/* The same step as qd_batch_attn_decode in two launches: the chunk form's preparation (norm,
 * RoPE, cache rows written at every sequence's position; q_scratch bf16 [batch, q_heads,
 * head_dim]) and a kernel that gives every lane one cache position (32 row reads in flight per
 * warp, one warp reduction per head and 32 positions instead of one per position).  Same
 * arithmetic up to summation order.  head_dim a multiple of 32, rotary_dim a multiple of 64.
 * cache_stride 0: the rows are the tokens of one prompt chunk (ascending positions) sharing
 * one cache - the causal attention of the chunked prefill. */
int qd_batch_attention(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                       const void* k_norm, void* k_cache, void* v_cache, long long cache_stride,
                       void* q_scratch, void* out, float* scratch, unsigned int* counters,
                       const int* positions, int batch, int capacity, int q_heads, int kv_heads,
                       int head_dim, int rotary_dim, float theta, float eps, int splits, void* stream);

/* The stable order of the chunk's routes by expert (quickdraw/kernel/triton/moe.py:60-97, the
 * grouping the reference builds with a stable sort): ids int32 [routes], every id in
 * [0, experts); order int32 [routes] = route index of each sorted row, boundaries int32
 * [experts + 1] = first sorted row of each expert.  experts <= 1023. */
int qd_seq_group_routes(const int32_t* ids, int routes, int experts, int32_t* order, int32_t* boundaries,
                        void* stream);
/* contributions bf16 [tokens, topk, hidden] in route order, ids [tokens, topk], shared
 * [tokens, hidden], strength bf16 [tokens] */
int qd_seq_moe_combine(const void* contributions, const int32_t* ids, const void* shared,
                       const void* strength, void* out, int tokens, int hidden, int topk, void* stream);
/* qd_seq_moe_combine followed by qd_seq_add_rms_norm(x = its output, residual, gamma) in one launch;
 * hidden a multiple of 8, at most 4096, else QD_ERR_UNSUPPORTED. */
int qd_seq_moe_combine_norm(const void* contributions, const int32_t* ids, const void* shared, const void* strength,
                            const void* residual, const float* gamma, void* normed, void* residual_out,
                            int tokens, int hidden, int topk, float eps, void* stream);

/* expert_gemv(x, proj, ids, weights=None) — quickdraw/kernel/cute/matvec.py:152-154,
 * quickdraw/kernel/triton/matvec.py:84-99.  Bank [E, rows, in/2]; y [slots, rows];
 * x [in] or, with per_slot_input, [slots, in]; global fp32 scalar or [E]. */
int qd_nvfp4_expert_gemv(const void* x, const void* codes, const void* scales, const float* global,
                         const int32_t* ids, const float* routing, void* y, int rows,
                         int in_features, int group_size, int slots, int per_slot_input,
                         int global_per_expert, int force_generic, void* stream);

/* gate_up(x, gate, up, ids=None) — quickdraw/kernel/cute/matvec.py:157-159:
 * y = bf16(silu(bf16 gate.x)) * bf16(up.x); ids NULL for a plain projection pair. */
int qd_nvfp4_gate_up(const void* x, const void* gate_codes, const void* gate_scales,
                     const float* gate_global, const void* up_codes, const void* up_scales,
                     const float* up_global, const int32_t* ids, void* y, int rows,
                     int in_features, int group_size, int slots, int global_per_expert,
                     int force_generic, void* stream);

/* NVFP4Linear.dequantize without the bf16 cast — quickdraw/models/weights.py:21-26,46-55.
 * hardware_convert != 0 decodes the codes with the sm_100a e2m1x2 convert the streaming
 * kernels use, 0 with integer bit arithmetic. */
int qd_nvfp4_dequantize(const void* codes, const void* scales, float global, float* out,
                        long long rows, int in_features, int group_size, int hardware_convert,
                        void* stream);

/* F.linear on bf16 with a bf16 result (router, shared-expert gate, DeltaNet a/b, bf16 LM
 * head) — quickdraw/models/qwen.py:129-130,173,192. */
int qd_bf16_gemv(const void* x, const void* w, void* y, int rows, int width, void* stream);

/* fp8_gemv(x, proj) — quickdraw/kernel/triton/matvec.py:102-115, qwen.py:25-33. */
int qd_fp8_gemv(const void* x, const void* w, const float* w_scale, const float* in_scale, void* y,
                int rows, int width, int is_fp32, void* stream);
/* The same projection for a chunk of tokens or a decode batch (no counterpart in the reference, whose
 * prompt chunks go through fp8_gemv row by row): activations quantised once to E4M3 bytes
 * (q_scratch: tokens * in_features bytes, 16-byte aligned; convert = 0 reuses what the previous call
 * left there, for projections that share input and input scale), E4M3 x E4M3 products on
 * mma.sync.m16n8k32, fp32 sum, y = bf16((sum * in_scale) * w_scale).  in_features % 128 == 0,
 * out_features even, else QD_ERR_UNSUPPORTED. */
int qd_fp8_matmul(const void* x, const void* w, const float* w_scale, const float* in_scale, void* y,
                  int tokens, int out_features, int in_features, void* q_scratch, int convert, void* stream);

/* route(logits, topk) -> (int32 ids, fp32 weights) — quickdraw/kernel/cute/moe.py:87-98,
 * quickdraw/kernel/triton/moe.py:11-30, qwen.py:174-177.  experts <= 1024, topk <= 32. */
int qd_route_topk(const void* logits, int logits_fp32, int experts, int topk, int32_t* ids,
                  float* weights, void* stream);

/* _reduce — quickdraw/kernel/cute/moe.py:61-73, quickdraw/kernel/triton/moe.py:42-57:
 * out = bf16(sum over slots, ascending expert id) + bf16(shared * bf16(sigmoid(strength))). */
int qd_moe_combine(const void* contributions, const int32_t* ids, const void* shared,
                   const void* strength, void* out, int hidden, int topk, void* stream);

/* _silu_kernel — quickdraw/kernel/triton/moe.py:33-39. */
int qd_swiglu(const void* gate, const void* up, void* out, int n, void* stream);

/* ---- Gated-DeltaNet mixer core — quickdraw/kernel/triton/delta.py:37-121, qwen.py:134-164 */

/* _conv_kernel: depthwise causal conv of one token over [channels, width] taps; shifts the
 * [channels, width-1] history in place. */
int qd_gdn_conv(const void* mixed, const void* taps, void* conv_state, void* out, int channels,
                int width, void* stream);

/* _delta_kernel: l2norm(q,k), decay/beta gates, delta-rule update of the fp32 state
 * [value_heads, key_dim, value_dim] in place, out = bf16(S^T q).  key_dim <= 128. */
int qd_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                      const void* dt_bias, float* rec_state, void* out, int key_heads,
                      int value_heads, int key_dim, int value_dim, int pdl, void* stream);

/* _gate_kernel: per-head RMSNorm(o) * gamma * silu(z). */
int qd_gdn_gated_norm(const void* o, const void* z, const void* gamma, void* out, int heads,
                      int value_dim, float eps, void* stream);

/* ---- GQA decode attention — quickdraw/kernel/triton/attention.py:10-100, qwen.py:66-116.
 * _prepare and _attend in one launch: q/k RMSNorm (gamma = 1 + w), partial RoPE, cache write
 * at the position, split-context online softmax, sigmoid output gate.
 * qg [q_heads, 2*head_dim] (query | gate), k_new/v_new [kv_heads, head_dim], caches
 * [capacity, kv_heads, head_dim]; out [q_heads*head_dim].  position_dev (int32 device scalar)
 * overrides position_host when not NULL.  scratch: qd_attn_scratch_floats() floats;
 * counters: kv_heads zeroed uint32 (the kernel leaves them zero).  head_dim <= 256,
 * q_heads / kv_heads <= 8. */
int qd_attn_scratch_floats(int q_heads, int kv_heads, int head_dim, int splits);
int qd_attn_decode(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                   const void* k_norm, void* k_cache, void* v_cache, void* out, float* scratch,
                   unsigned int* counters, const int* position_dev, int position_host, int capacity,
                   int q_heads, int kv_heads, int head_dim, int rotary_dim, float theta, float eps,
                   int splits, int pdl, void* stream);

/* qd_attn_decode for callers that may not allocate device memory: plugins that run inside
 * another runtime's memory pool, code on a latency path that must not call the CUDA
 * allocator, or hosts that hand this library no workspace.  No counterpart in the
 * reference (its wrappers allocate their outputs and workspaces with torch).  Same
 * arguments and results as qd_attn_decode without the scratch and counter buffers: the
 * split-context partial sums live in a 1 MiB array built into the library, one per GPU that
 * loads it, held until the process exits.
 *  - Limit: qd_attn_scratch_floats(...) * 4 bytes must fit in 1 MiB minus 256 bytes
 *    (16 query / 2 KV heads of 256 with 32 splits need 516 KiB); otherwise QD_ERR_TOO_LARGE.
 *  - The first call on a device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - Every call uses the same array: two calls that overlap on the GPU (different streams,
 *    or graphs replayed concurrently) race on it.  Calls on one stream are safe.
 *  - Calls neither cudaMalloc/cudaFree nor any allocating routine. */
int qd_attn_decode_static(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                          const void* k_norm, void* k_cache, void* v_cache, void* out,
                          const int* position_dev, int position_host, int capacity, int q_heads,
                          int kv_heads, int head_dim, int rotary_dim, float theta, float eps,
                          int splits, void* stream);

/* ---- MoE tail — quickdraw/kernel/cute/moe.py:101-116 (expert_gemv(down, routed) +
 * shared down + _reduce in one launch).  hidden [topk+1, 512] (last row: shared expert).
 * Either `out` (combined bf16 [hidden_size]) or, for expert parallelism, `routed_out`
 * (fp32 partial sum over the experts in [expert_lo, expert_hi), bank pointers local to that
 * range) with `shared_out` (gated shared row); qd_moe_finish adds them after the all-reduce. */
int qd_moe_down_combine(const void* hidden, const int32_t* ids, const float* weights,
                        const void* down_codes, const void* down_scales, const float* down_global,
                        const void* shared_codes, const void* shared_scales, const float* shared_global,
                        const void* strength, void* out, float* routed_out, void* shared_out,
                        int hidden_size, int intermediate, int topk, int global_per_expert,
                        int expert_lo, int expert_hi, int pdl, void* stream);
int qd_moe_finish(const float* routed, const void* shared, void* out, int n, int pdl, void* stream);

/* ---- Whole decode step — quickdraw/models/qwen.py:196-241 behind Engine.decode_step
 * (quickdraw/engine/engine.py:114-127).  The caller owns every buffer; the model object is
 * a host-side table of pointers. */
typedef struct {
    const void* codes; const void* scales; const float* global;   /* NVFP4 projection */
} qd_fp4;

typedef struct {
    int is_attention;
    const float* gamma_in; const float* gamma_post;      /* fp32 [hidden]: 1 + layernorm weight */
    /* DeltaNet: qkv, z, out.  Attention: q(+gate), k, v, o. */
    qd_fp4 proj_a, proj_b, proj_c, proj_out;
    const void* in_proj_a; const void* in_proj_b;        /* bf16 [value_heads, hidden] */
    const void* conv1d; const void* a_log; const void* dt_bias; const void* head_norm;
    const void* q_norm; const void* k_norm;
    const void* router; const void* shared_expert_gate;  /* bf16 [experts, hidden], [1, hidden] */
    qd_fp4 experts_gate, experts_up, experts_down;       /* banks, local to [expert_lo, expert_hi) */
    qd_fp4 shared_gate, shared_up, shared_down;
    int experts_global_per_expert;
    int state_index;                                     /* index into rec/conv or kv arrays */
    /* Static FP8 mixers (FP8Linear, quickdraw/models/weights.py:58-74; fp8_gemv, qwen.py:25-33):
     * proj_a/b/c/out then hold E4M3 weights [out, in] in `codes`, NULL in `scales` and the fp32
     * weight scale in `global`; the projections that read the layer input share one activation
     * scale (merge_fp8_scales), the output projection has its own.  Persistent step only. */
    int mixers_fp8;
    const float* mixer_input_scale; const float* out_input_scale;
} qd_layer;

typedef struct {
    int hidden, layers, vocab;
    int q_heads, kv_heads, head_dim, rotary_dim;
    int key_heads, value_heads, key_dim, value_dim, conv_width;
    int experts, topk, intermediate;
    float eps, rope_theta;
    int expert_lo, expert_hi;                            /* owned expert range (expert parallel) */
    int vocab_lo, vocab_hi;                              /* owned LM-head rows; vocab_hi == 0: all of them */
    const void* embed;                                   /* bf16 [vocab, hidden] */
    const float* final_gamma;                            /* fp32 [hidden] */
    const void* lm_head;                                 /* bf16 rows [vocab_lo, vocab_hi) of [vocab, hidden] */
    /* The published checkpoint's LM head is NVFP4 (quickdraw/models/weights.py:164): when
     * lm_head_fp4.codes is set it replaces lm_head (same row range).  Persistent step only. */
    qd_fp4 lm_head_fp4;
} qd_model_config;

typedef struct {
    void* kv_k; void* kv_v;      /* bf16 [attention_layers, capacity, kv_heads, head_dim] */
    float* rec_state;            /* fp32 [linear_layers, value_heads, key_dim, value_dim] */
    void* conv_state;            /* bf16 [linear_layers, channels, conv_width - 1] */
    int capacity;
} qd_state;

typedef struct qd_model qd_model;

int qd_model_create(const qd_model_config* config, qd_model** out);
int qd_model_set_layer(qd_model* model, int index, const qd_layer* layer);
int qd_model_destroy(qd_model* model);
/* Bytes of zero-initialised device workspace one decode stream needs. */
long long qd_decode_workspace_bytes(const qd_model* model);

/* One token through every layer.  token: int64 device scalar; position: int32 device
 * scalar (preferred, graph-replayable) or host value.  Writes bf16 logits [vocab] and the
 * greedy next token (int64 device scalar, lowest index on ties).  flags: QD_FLAG_PDL makes
 * every launch a programmatic dependent of its predecessor, QD_FLAG_NO_LOGITS skips the LM
 * head (prompt tokens). */
enum { QD_FLAG_PDL = 1, QD_FLAG_NO_LOGITS = 2 };
int qd_decode_step(qd_model* model, const qd_state* state, const long long* token,
                   const int* position_dev, int position_host, void* workspace, void* logits_out,
                   long long* next_token, int flags, void* stream);
/* The same step as ONE cooperative launch: a persistent kernel, one block per SM, that walks
 * the phases of qwen.py:196-241 without any grid-wide barrier (blocks hand activations to each
 * other as tagged words in `workspace` and start a phase as soon as their own inputs exist)
 * and a weight ring that runs ahead across the phases.
 * The phase list ("program") holds device addresses of the model and of `workspace`, so it
 * is built once per (model, workspace) pair: qd_program_build fills a HOST buffer of
 * qd_program_bytes bytes, the caller copies it to the device and passes that copy here.
 * Needs a whole idle GPU (all blocks resident).  `trace` (optional, device) receives
 * [phase][16][blocks] nanosecond timestamps.
 *
 * Expert parallel (no counterpart in the reference, which is single-GPU): every rank runs
 * this launch on the same token with its own model slice (expert_lo/hi, vocab_lo/hi in the
 * config; banks and LM head local to the slice).  `exchange` names, per rank, the address in
 * THIS process of that rank's exchange area (qd_exchange_bytes bytes, zero-initialised before
 * the first step, peer-mapped, e.g. a symmetric-memory allocation).  A rank stores the routed
 * contributions of the experts it owns into every rank's area and reads all of them from its
 * own, so each rank adds the same eight bf16 rows in the same order as a single GPU would;
 * the ranks' best (logit, index) pairs meet the same way and every rank ends with the same
 * next token.  Logits: each rank writes rows [vocab_lo, vocab_hi) of `logits_out`.
 * exchange == NULL: single GPU.  Plain peer loads and stores only. */
typedef struct {
    int rank, world;                       /* world <= 8 */
    unsigned long long peer_base[8];
} qd_exchange;
long long qd_exchange_bytes(const qd_model* model);
long long qd_program_bytes(const qd_model* model);
int qd_program_build(const qd_model* model, void* workspace, void* host_out, long long bytes);
int qd_decode_step_persistent(const qd_model* model, const qd_state* state, const long long* token,
                              const int* position_dev, int position_host, void* workspace,
                              const void* program, const qd_exchange* exchange, void* logits_out,
                              long long* next_token, int flags, unsigned long long* trace, void* stream);
/* Bound of every device-side wait of the persistent kernel (default 200 000 us).  A wait that
 * runs out sets bit 0 of the status word (workspace + 256) and the kernel finishes the token
 * without waiting any further; the context stays usable. */
int qd_set_wait_limit_us(unsigned int microseconds);

/* Measurement helper: the streaming NVFP4 matvec over a bank of `matrices` equally shaped
 * [rows, in_features] matrices, one launch per matrix, so the working set can exceed L2. */
int qd_nvfp4_gemv_bank(const void* x, const void* codes, const void* scales, const float* global,
                       void* y, int rows, int in_features, int matrices, int pdl, void* stream);

#ifdef __cplusplus
}
#endif
#endif
