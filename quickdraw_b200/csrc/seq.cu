// Sequence forms of the per-token operators, for a chunk of prompt tokens (prefill).  The dense
// projections of a chunk run on the tensor cores (gemm.cu); everything here is the glue between
// them, with the arithmetic of the single-token kernels applied row by row (same rounding
// points): residual add + RMSNorm, small bf16 projections, the DeltaNet short convolution and
// recurrence walked along the chunk, attention preparation (q/k norm, RoPE, cache write) and
// causal attention over cache + chunk, routing and the MoE combine.
// Reference: the 2-D branches of quickdraw/kernel/triton/{delta,attention,moe,norm}.py and
// quickdraw/models/qwen.py:66-241.
#include "attn_mma.cuh"
#include "rowdot.cuh"

namespace {

using qd::AttnAcc;
using qd::attn_chunk;
using qd::kAttnQRow;
using qd::kAttnRow;
using qd::mma_bf16;

// ------------------------------------------------------------------ residual add + RMSNorm
__global__ void seq_add_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                                    const float* __restrict__ gamma, bf16* __restrict__ normed,
                                    bf16* __restrict__ residual_out, int width, float eps) {
    chain_enter();
    __shared__ float partial[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ld_bf16(x + base + i) + (residual ? ld_bf16(residual + base + i) : 0.f);
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += partial[w];
    const float inv = rsqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ld_bf16(x + base + i) + (residual ? ld_bf16(residual + base + i) : 0.f);
        normed[base + i] = __float2bfloat16_rn((v * inv) * gamma[i]);
        residual_out[base + i] = __float2bfloat16_rn(v);
    }
}

// The same with 16-byte accesses and the row kept in registers between the two passes (widths that
// are a multiple of 8, up to 4096; the sum of squares is taken in another order than above).
constexpr int kNormVecs = 2;            // 16-byte pieces per thread: 256 threads x 2 x 8 values
__global__ void __launch_bounds__(256)
seq_add_norm8_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual, const float* __restrict__ gamma,
                     bf16* __restrict__ normed, bf16* __restrict__ residual_out, int width, float eps) {
    chain_enter();
    __shared__ float partial[8];
    const size_t base = (size_t)blockIdx.x * width;
    const int tid = threadIdx.x, pieces = width / 8;
    float v[kNormVecs][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kNormVecs; ++k) {
        const int c = tid + k * 256;
        if (c >= pieces) break;
        const uint4 a = *reinterpret_cast<const uint4*>(x + base + 8 * c);
        uint4 r = make_uint4(0u, 0u, 0u, 0u);
        if (residual) r = *reinterpret_cast<const uint4*>(residual + base + 8 * c);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            v[k][2 * q] = __uint_as_float(aw[q] << 16) + __uint_as_float(rw[q] << 16);
            v[k][2 * q + 1] = __uint_as_float(aw[q] & 0xffff0000u) + __uint_as_float(rw[q] & 0xffff0000u);
            ss += v[k][2 * q] * v[k][2 * q] + v[k][2 * q + 1] * v[k][2 * q + 1];
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) partial[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += partial[w];
    const float inv = rsqrtf(total / (float)width + eps);
#pragma unroll
    for (int k = 0; k < kNormVecs; ++k) {
        const int c = tid + k * 256;
        if (c >= pieces) break;
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + 8 * c), g1 = *reinterpret_cast<const float4*>(gamma + 8 * c + 4);
        const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t n[4], o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            n[q] = qd::pack_bf16x2((v[k][2 * q] * inv) * gm[2 * q], (v[k][2 * q + 1] * inv) * gm[2 * q + 1]);
            o[q] = qd::pack_bf16x2(v[k][2 * q], v[k][2 * q + 1]);
        }
        *reinterpret_cast<uint4*>(normed + base + 8 * c) = make_uint4(n[0], n[1], n[2], n[3]);
        *reinterpret_cast<uint4*>(residual_out + base + 8 * c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// --------------------------------------------------- small bf16 projection of every token
// y[t, n] = bf16( sum_k x[t, k] w[n, k] ): one warp per (token, output row), 16-byte loads where
// the width allows them.
// A second matrix of the same input (w1, y1, rows1; or NULL) takes the blocks from first_block1 on.
__global__ void seq_bf16_matmul_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                                       int rows, int width, const bf16* __restrict__ w1, bf16* __restrict__ y1, int rows1,
                                       int first_block1) {
    chain_enter();
    const int lane = threadIdx.x & 31, t = blockIdx.y;
    int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w1 && (int)blockIdx.x >= first_block1) {
        n -= first_block1 * (blockDim.x >> 5);
        w = w1; y = y1; rows = rows1;
    }
    if (n >= rows) return;
    const bf16* row = w + (size_t)n * width;
    const bf16* xt = x + (size_t)t * width;
    float acc = 0.f;
    if ((width & 7) == 0) {
        for (int i = lane * 8; i < width; i += 256) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(row + i)), xv = __ldg(reinterpret_cast<const uint4*>(xt + i));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc += bf16_bits_to_float(ww[q] & 0xffffu) * bf16_bits_to_float(xx[q] & 0xffffu);
                acc += bf16_bits_to_float(ww[q] >> 16) * bf16_bits_to_float(xx[q] >> 16);
            }
        }
    } else {
        for (int i = lane; i < width; i += 32) acc += ld_bf16(row + i) * ld_bf16(xt + i);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)t * rows + n] = __float2bfloat16_rn(acc);
}

// The same for a tall matrix (the LM head over a batch of tokens) on the warp-level tensor-core
// instruction: the activations of up to 32 tokens sit in shared memory as bf16 (rows padded by
// 16 bytes against bank conflicts); a warp takes sixteen weight rows at a time and reads them
// once, straight from global memory into A fragments: lane (g, t) loads the 32 bytes of rows g
// and g + 8 at inputs 64 s + 16 t .. + 15 of step s (a quarter-warp reads two whole 128-byte
// lines), and the 16 inputs of token 8 nt + g at the same offsets are its B fragments, so every
// element of the 16 x 32 result is used.  fp32 accumulators, one bf16 rounding.
constexpr int kTallTokens = 32, kTallMaxWidth = 3072, kTallUnroll = 2, kTallWarps = 16;
__global__ void __launch_bounds__(kTallWarps * 32, 1)
seq_bf16_matmul_tall_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                            int tokens, int rows, int width, int groups_per_block, int input_parts) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char tall_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int t0 = blockIdx.y * kTallTokens, nt_rows = min(kTallTokens, tokens - t0);
    const int pieces = width / 8, x_row = 2 * width + 16;
    for (int i0 = tid; i0 < kTallTokens * pieces; i0 += kTallWarps * 32 * 8) {      // eight loads in flight per thread
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * kTallWarps * 32, row = i / pieces, col = i % pieces;
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (i < kTallTokens * pieces && row < nt_rows) v[u] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + row) * width) + col);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * kTallWarps * 32, row = i / pieces, col = i % pieces;
            if (i < kTallTokens * pieces) *reinterpret_cast<uint4*>(tall_smem + (size_t)row * x_row + col * 16) = v[u];
        }
    }
    __syncthreads();
    const unsigned char* xs = tall_smem + (size_t)g * x_row + t * 32;
    const int steps = width / 64;
    // sixteen weight rows (n0 ..) against the tile's tokens over steps [s_begin, s_end) of 64 inputs
    auto rows_times_tokens = [&](int n0, int s_begin, int s_end, float (&acc)[4][4]) {
        // rows past the matrix read its last row and store nothing
        const uint4* lo = reinterpret_cast<const uint4*>(w + (size_t)min(n0 + g, rows - 1) * width + t * 16);
        const uint4* hi = reinterpret_cast<const uint4*>(w + (size_t)min(n0 + g + 8, rows - 1) * width + t * 16);
        // two register buffers of kTallUnroll steps: the loads of one are in flight while the
        // other is multiplied (the warps of a block run in step, so nothing else would hide them)
        auto load = [&](uint4 (&a)[kTallUnroll][4], int s0) {
#pragma unroll
            for (int u = 0; u < kTallUnroll; ++u) {
                const int s = min(s0 + u, s_end - 1);
                a[u][0] = __ldg(lo + s * 8); a[u][1] = __ldg(lo + s * 8 + 1);
                a[u][2] = __ldg(hi + s * 8); a[u][3] = __ldg(hi + s * 8 + 1);
            }
        };
        auto multiply = [&](const uint4 (&a)[kTallUnroll][4], int s0) {
#pragma unroll
            for (int u = 0; u < kTallUnroll; ++u) {
                if (s0 + u >= s_end) break;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const unsigned char* src = xs + (size_t)nt * 8 * x_row + (s0 + u) * 128;
                    const uint4 b0 = lds128(src), b1 = lds128(src + 16);
                    mma_bf16(acc[nt], a[u][0].x, a[u][2].x, a[u][0].y, a[u][2].y, b0.x, b0.y);
                    mma_bf16(acc[nt], a[u][0].z, a[u][2].z, a[u][0].w, a[u][2].w, b0.z, b0.w);
                    mma_bf16(acc[nt], a[u][1].x, a[u][3].x, a[u][1].y, a[u][3].y, b1.x, b1.y);
                    mma_bf16(acc[nt], a[u][1].z, a[u][3].z, a[u][1].w, a[u][3].w, b1.z, b1.w);
                }
            }
        };
        uint4 even[kTallUnroll][4], odd[kTallUnroll][4];
        load(even, s_begin);
#pragma unroll 1
        for (int s0 = s_begin; s0 < s_end; s0 += 2 * kTallUnroll) {
            if (s0 + kTallUnroll < s_end) load(odd, s0 + kTallUnroll);
            multiply(even, s0);
            if (s0 + 2 * kTallUnroll < s_end) load(even, s0 + 2 * kTallUnroll);
            if (s0 + kTallUnroll < s_end) multiply(odd, s0 + kTallUnroll);
        }
    };
    // acc[nt][0..1] = row n0 + g, tokens 8 nt + 2 t and + 1; [2..3] = row n0 + g + 8
    auto store = [&](int n0, const float (&acc)[4][4]) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int token = 8 * nt + 2 * t + (c & 1), row = n0 + g + 8 * (c >> 1);
                if (token < nt_rows && row < rows) y[(size_t)(t0 + token) * rows + row] = __float2bfloat16_rn(acc[nt][c]);
            }
    };
    if (input_parts > 1) {
        // few rows (one pass per block): the warps beyond the row groups take parts of the inputs, the parts'
        // sums meet in shared memory behind the tokens and are added in order
        const int slot = warp % groups_per_block, part = warp / groups_per_block;
        const int n0 = (blockIdx.x * groups_per_block + slot) * 16;
        const bool active = n0 < rows && part < input_parts;
        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
        if (active) rows_times_tokens(n0, part * steps / input_parts, (part + 1) * steps / input_parts, acc);
        float4* meet = reinterpret_cast<float4*>(tall_smem + (size_t)kTallTokens * x_row);     // [part - 1][slot][nt][lane]
        if (active && part > 0) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
                meet[(((part - 1) * groups_per_block + slot) * 4 + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        }
        __syncthreads();
        if (active && part == 0) {
            for (int other = 1; other < input_parts; ++other)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const float4 v = meet[(((other - 1) * groups_per_block + slot) * 4 + nt) * 32 + lane];
                    acc[nt][0] += v.x; acc[nt][1] += v.y; acc[nt][2] += v.z; acc[nt][3] += v.w;
                }
            store(n0, acc);
        }
        return;
    }
    // many rows: only the first groups_per_block warps multiply (more blocks share the rows)
    for (int n0 = warp < groups_per_block ? (blockIdx.x * groups_per_block + warp) * 16 : rows; n0 < rows;
         n0 += gridDim.x * groups_per_block * 16) {
        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
        rows_times_tokens(n0, 0, steps, acc);
        store(n0, acc);
    }
}

// ------------------------------------------------------------- DeltaNet short convolution
// One thread per (token, channel): window = [history | new] ending at the token, tap products
// rounded to bf16, fp32 sum from the oldest tap on, SiLU, bf16.  A second kernel then leaves the
// last width - 1 inputs in the history (it runs after every read of the old history).
QD_DEVINL float conv_input(const bf16* __restrict__ mixed, const bf16* __restrict__ state, int index, int c,
                           int channels, int width) {
    return index < 0 ? ld_bf16(state + (size_t)c * (width - 1) + index + width - 1)
                     : ld_bf16(mixed + (size_t)index * channels + c);
}
__global__ void seq_conv_kernel(const bf16* __restrict__ mixed, const bf16* __restrict__ taps,
                                const bf16* __restrict__ state, bf16* __restrict__ out, int channels, int width) {
    chain_enter();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= channels) return;
    float acc = 0.f;
    for (int k = 0; k < width; ++k)
        acc += round_bf16(conv_input(mixed, state, t - (width - 1) + k, c, channels, width) * ld_bf16(taps + (size_t)c * width + k));
    out[(size_t)t * channels + c] = __float2bfloat16_rn(silu_precise(acc));
}
// The same arithmetic for width 4 with a thread per (pair of channels, run of sixteen tokens):
// the window slides through registers, so every input row is loaded once per run (4-byte loads,
// 128 bytes per warp) instead of once per tap.
constexpr int kConvRun = 16;
__global__ void __launch_bounds__(128)
seq_conv4_kernel(const bf16* __restrict__ mixed, const bf16* __restrict__ taps, const bf16* __restrict__ state,
                 bf16* __restrict__ out, int tokens, int channels) {
    chain_enter();
    const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x), t0 = blockIdx.y * kConvRun;
    if (c >= channels) return;
    const uint2 tp0 = *reinterpret_cast<const uint2*>(taps + (size_t)c * 4), tp1 = *reinterpret_cast<const uint2*>(taps + (size_t)c * 4 + 4);
    const float ta[4] = {bf16_bits_to_float(tp0.x & 0xffffu), bf16_bits_to_float(tp0.x >> 16),
                         bf16_bits_to_float(tp0.y & 0xffffu), bf16_bits_to_float(tp0.y >> 16)};
    const float tb[4] = {bf16_bits_to_float(tp1.x & 0xffffu), bf16_bits_to_float(tp1.x >> 16),
                         bf16_bits_to_float(tp1.y & 0xffffu), bf16_bits_to_float(tp1.y >> 16)};
    float wa[4], wb[4];                  // inputs t - 3 .. t of either channel
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int index = t0 - 3 + k;
        if (index < 0) {
            wa[k + 1] = ld_bf16(state + (size_t)c * 3 + index + 3);
            wb[k + 1] = ld_bf16(state + (size_t)(c + 1) * 3 + index + 3);
        } else {
            const uint32_t pair = *reinterpret_cast<const uint32_t*>(mixed + (size_t)index * channels + c);
            wa[k + 1] = bf16_bits_to_float(pair & 0xffffu); wb[k + 1] = bf16_bits_to_float(pair >> 16);
        }
    }
    const int count = min(kConvRun, tokens - t0);
    uint32_t fresh[kConvRun];
#pragma unroll
    for (int i = 0; i < kConvRun; ++i)
        fresh[i] = i < count ? __ldg(reinterpret_cast<const uint32_t*>(mixed + (size_t)(t0 + i) * channels + c)) : 0u;
#pragma unroll
    for (int i = 0; i < kConvRun; ++i) {
        if (i >= count) break;
        wa[0] = wa[1]; wa[1] = wa[2]; wa[2] = wa[3]; wa[3] = bf16_bits_to_float(fresh[i] & 0xffffu);
        wb[0] = wb[1]; wb[1] = wb[2]; wb[2] = wb[3]; wb[3] = bf16_bits_to_float(fresh[i] >> 16);
        float acc_a = 0.f, acc_b = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) { acc_a += round_bf16(wa[k] * ta[k]); acc_b += round_bf16(wb[k] * tb[k]); }
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(t0 + i) * channels + c) =
            __floats2bfloat162_rn(silu_precise(acc_a), silu_precise(acc_b));
    }
}
__global__ void seq_conv_state_kernel(const bf16* __restrict__ mixed, bf16* state, int tokens, int channels, int width) {
    chain_enter();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    bf16 keep[8];
    for (int j = 0; j < width - 1; ++j) {
        const int index = tokens - (width - 1) + j;
        keep[j] = index < 0 ? state[(size_t)c * (width - 1) + index + width - 1] : mixed[(size_t)index * channels + c];
    }
    for (int j = 0; j < width - 1; ++j) state[(size_t)c * (width - 1) + j] = keep[j];
}

// One decode step of `batch` independent sequences: thread = (sequence, channel), the
// single-token arithmetic on the sequence's own history (state_stride elements apart).
__global__ void batch_conv_kernel(const bf16* __restrict__ mixed, const bf16* __restrict__ taps, bf16* state,
                                  bf16* __restrict__ out, int channels, int width, long long state_stride) {
    chain_enter();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= channels) return;
    bf16* hist = state + (size_t)b * state_stride + (size_t)c * (width - 1);
    const float fresh = ld_bf16(mixed + (size_t)b * channels + c);
    float acc = 0.f;
    for (int k = 0; k < width - 1; ++k) acc += round_bf16(ld_bf16(hist + k) * ld_bf16(taps + (size_t)c * width + k));
    acc += round_bf16(fresh * ld_bf16(taps + (size_t)c * width + width - 1));
    for (int k = 0; k + 1 < width - 1; ++k) hist[k] = hist[k + 1];
    if (width > 1) hist[width - 2] = mixed[(size_t)b * channels + c];
    out[(size_t)b * channels + c] = __float2bfloat16_rn(silu_precise(acc));
}

// ------------------------------------------------- DeltaNet recurrence, key dimension 128
// Block = (value head, 32 value columns), four warps; a warp owns 8 columns, a lane one column
// and one quarter of the 128 keys: 32 state entries in registers for the whole chunk, the sums
// over keys finish with two shuffles, so the token loop has no block-wide barrier.  The inputs
// of 16 tokens at a time (normalised key and query in fp32, the gates, the value columns) are
// prepared in shared memory by the four warps, one batch ahead of the recurrence: the global
// loads of batch n + 1 are issued before batch n is walked and finished after it.
// Arithmetic per token as in the single-token kernel (quickdraw/kernel/triton/delta.py:41-78):
// S *= decay; pred = S^T k; S += k (x) beta (v - pred); out = S^T q.
constexpr int kRecBatch = 16;
#ifndef QD_REC_PARTS
#define QD_REC_PARTS 4
#endif
constexpr int kRecParts = QD_REC_PARTS;              // lanes that share a column (4 or 8), each with 128 / parts keys
                                                     // (8 was measured: twice the blocks, same time per chunk)
constexpr int kRecKeys = 128 / kRecParts;            // state entries per lane
constexpr int kRecPitch = kRecKeys + 4;              // floats per part in shared memory (+ 4: no bank conflicts)
constexpr int kRecCols = 4 * 32 / kRecParts;         // value columns per block (four warps)

struct RecPrefetch { uint2 k[kRecBatch / 4], q[kRecBatch / 4]; bf16 v[kRecBatch / 4], a[kRecBatch / 4], b[kRecBatch / 4]; };

__global__ void __launch_bounds__(128)
seq_recurrence128_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ b,
                         const bf16* __restrict__ a_log, const bf16* __restrict__ dt_bias, float* __restrict__ state,
                         bf16* __restrict__ out, int tokens, int hk, int hv, int dv, long long state_stride) {
    chain_enter();
    constexpr int dk = 128;
    // batched decode: grid z = sequence, one token each; rows and state move on by one sequence
    if (blockIdx.z) {
        const size_t z = blockIdx.z;
        qkv += z * (size_t)(2 * hk * dk + hv * dv);
        a += z * hv;
        b += z * hv;
        out += z * (size_t)hv * dv;
        state += z * state_stride;
    }
    __shared__ __align__(16) float skn[2][kRecBatch][kRecParts * kRecPitch];
    __shared__ __align__(16) float sqn[2][kRecBatch][kRecParts * kRecPitch];
    __shared__ float sv[2][kRecBatch][32];
    __shared__ float sgate[2][kRecBatch][2];
    const int head = blockIdx.x, c0 = blockIdx.y * kRecCols;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = lane & (kRecParts - 1), col = warp * (32 / kRecParts) + lane / kRecParts;
    const int key_head = head / (hv / hk);
    const bool col_ok = c0 + col < dv;
    const int channels = 2 * hk * dk + hv * dv;
    const float a_decay = ld_bf16(a_log + head), bias = ld_bf16(dt_bias + head);
    float* tile = state + (size_t)head * dk * dv + (size_t)quarter * kRecKeys * dv + c0 + col;
    float s[kRecKeys];
#pragma unroll
    for (int j = 0; j < kRecKeys; ++j) s[j] = col_ok ? tile[(size_t)j * dv] : 0.f;

    // warp w prepares tokens w, w + 4, w + 8, w + 12 of a batch; lane l holds keys 4l .. 4l + 3
    auto issue = [&](int batch, RecPrefetch& r) {
#pragma unroll
        for (int i = 0; i < kRecBatch / 4; ++i) {
            const int t = batch * kRecBatch + warp + 4 * i;
            if (t >= tokens) continue;
            const bf16* row = qkv + (size_t)t * channels;
            r.q[i] = __ldg(reinterpret_cast<const uint2*>(row + (size_t)key_head * dk + 4 * lane));
            r.k[i] = __ldg(reinterpret_cast<const uint2*>(row + (size_t)(hk + key_head) * dk + 4 * lane));
            r.v[i] = (lane < kRecCols && c0 + lane < dv) ? row[(size_t)2 * hk * dk + (size_t)head * dv + c0 + lane] : __float2bfloat16_rn(0.f);
            r.a[i] = a[(size_t)t * hv + head];
            r.b[i] = b[(size_t)t * hv + head];
        }
    };
    auto finish = [&](int batch, const RecPrefetch& r) {
        const int buf = batch & 1;
#pragma unroll
        for (int i = 0; i < kRecBatch / 4; ++i) {
            const int slot = warp + 4 * i;
            if (batch * kRecBatch + slot >= tokens) continue;
            const float q4[4] = {bf16_bits_to_float(r.q[i].x & 0xffffu), bf16_bits_to_float(r.q[i].x >> 16),
                                 bf16_bits_to_float(r.q[i].y & 0xffffu), bf16_bits_to_float(r.q[i].y >> 16)};
            const float k4[4] = {bf16_bits_to_float(r.k[i].x & 0xffffu), bf16_bits_to_float(r.k[i].x >> 16),
                                 bf16_bits_to_float(r.k[i].y & 0xffffu), bf16_bits_to_float(r.k[i].y >> 16)};
            float qq = 0.f, kk = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) { qq += q4[e] * q4[e]; kk += k4[e] * k4[e]; }
            const float qscale = rsqrtf(warp_sum(qq) + 1e-6f), kscale = rsqrtf(warp_sum(kk) + 1e-6f);
            const int at = ((4 * lane) / kRecKeys) * kRecPitch + (4 * lane) % kRecKeys;
            *reinterpret_cast<float4*>(&skn[buf][slot][at]) = make_float4(k4[0] * kscale, k4[1] * kscale, k4[2] * kscale, k4[3] * kscale);
            *reinterpret_cast<float4*>(&sqn[buf][slot][at]) =
                make_float4((q4[0] * qscale) / sqrtf((float)dk), (q4[1] * qscale) / sqrtf((float)dk),
                            (q4[2] * qscale) / sqrtf((float)dk), (q4[3] * qscale) / sqrtf((float)dk));
            sv[buf][slot][lane] = __bfloat162float(r.v[i]);
            if (lane == 0) {
                const float alpha = __bfloat162float(r.a[i]) + bias;
                sgate[buf][slot][0] = expf(-expf(a_decay) * softplus_precise(alpha));
                sgate[buf][slot][1] = sigmoid_precise(__bfloat162float(r.b[i]));
            }
        }
    };

    const int batches = (tokens + kRecBatch - 1) / kRecBatch;
    RecPrefetch pre;
    issue(0, pre);
    finish(0, pre);
    __syncthreads();
    for (int n = 0; n < batches; ++n) {
        const int buf = n & 1;
        if (n + 1 < batches) issue(n + 1, pre);
        const int count = min(kRecBatch, tokens - n * kRecBatch);
#pragma unroll 1
        for (int i = 0; i < count; ++i) {
            const float4* kp = reinterpret_cast<const float4*>(&skn[buf][i][quarter * kRecPitch]);
            const float4* qp = reinterpret_cast<const float4*>(&sqn[buf][i][quarter * kRecPitch]);
            const float decay = sgate[buf][i][0], beta = sgate[buf][i][1], v = sv[buf][i][col];
            float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
            for (int j = 0; j < kRecKeys / 4; ++j) {
                const float4 k4 = kp[j];
                s[4 * j] *= decay; s[4 * j + 1] *= decay; s[4 * j + 2] *= decay; s[4 * j + 3] *= decay;
                p0 += s[4 * j] * k4.x; p1 += s[4 * j + 1] * k4.y; p2 += s[4 * j + 2] * k4.z; p3 += s[4 * j + 3] * k4.w;
            }
            float pred = (p0 + p1) + (p2 + p3);
#pragma unroll
            for (int d = 1; d < kRecParts; d <<= 1) pred += __shfl_xor_sync(0xffffffffu, pred, d);
            const float corr = beta * (v - pred);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int j = 0; j < kRecKeys / 4; ++j) {
                const float4 k4 = kp[j], q4 = qp[j];
                s[4 * j] += k4.x * corr; s[4 * j + 1] += k4.y * corr; s[4 * j + 2] += k4.z * corr; s[4 * j + 3] += k4.w * corr;
                o0 += s[4 * j] * q4.x; o1 += s[4 * j + 1] * q4.y; o2 += s[4 * j + 2] * q4.z; o3 += s[4 * j + 3] * q4.w;
            }
            float o = (o0 + o1) + (o2 + o3);
#pragma unroll
            for (int d = 1; d < kRecParts; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
            if (quarter == 0 && col_ok)
                out[(size_t)(n * kRecBatch + i) * hv * dv + (size_t)head * dv + c0 + col] = __float2bfloat16_rn(o);
        }
        if (n + 1 < batches) finish(n + 1, pre);
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < kRecKeys; ++j)
        if (col_ok) tile[(size_t)j * dv] = s[j];
}

// ----------------------------------------------- DeltaNet recurrence, other key dimensions
// The single-token kernel (block = value head x 32 columns, 8 key groups x 32 columns, 16 state
// entries per thread) in a loop over the chunk; the state stays in registers in between.
__global__ void __launch_bounds__(256)
seq_recurrence_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ b,
                      const bf16* __restrict__ a_log, const bf16* __restrict__ dt_bias, float* __restrict__ state,
                      bf16* __restrict__ out, int tokens, int hk, int hv, int dk, int dv) {
    chain_enter();
    __shared__ float sq[128], sk[128];
    __shared__ float part[8][32];
    __shared__ float norms[2], gates[2];
    const int head = blockIdx.x, c0 = blockIdx.y * 32;
    const int tid = threadIdx.x, col = tid & 31, kg = tid >> 5;
    const int kpt = (dk + 7) / 8;
    const int key_head = head / (hv / hk);
    const bool col_ok = c0 + col < dv;
    const int channels = 2 * hk * dk + hv * dv;
    float* tile = state + (size_t)head * dk * dv + c0 + col;
    float s[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int key = kg * kpt + j;
        s[j] = (j < kpt && key < dk && col_ok) ? tile[(size_t)key * dv] : 0.f;
    }
    const float a_decay = ld_bf16(a_log + head), bias = ld_bf16(dt_bias + head);
    for (int t = 0; t < tokens; ++t) {
        const bf16* row = qkv + (size_t)t * channels;
        float qq = 0.f, kk = 0.f;
        for (int i = tid; i < dk; i += 256) {
            const float qv = ld_bf16(row + (size_t)key_head * dk + i), kv = ld_bf16(row + (size_t)hk * dk + (size_t)key_head * dk + i);
            sq[i] = qv; sk[i] = kv;
            qq += qv * qv; kk += kv * kv;
        }
        qq = warp_sum(qq); kk = warp_sum(kk);
        if (col == 0) { part[kg][0] = qq; part[kg][1] = kk; }
        __syncthreads();
        if (tid == 0) {
            float tq = 0.f, tk = 0.f;
            for (int w = 0; w < 8; ++w) { tq += part[w][0]; tk += part[w][1]; }
            norms[0] = rsqrtf(tq + 1e-6f);
            norms[1] = rsqrtf(tk + 1e-6f);
            const float alpha = ld_bf16(a + (size_t)t * hv + head) + bias;
            gates[0] = expf(-expf(a_decay) * softplus_precise(alpha));
            gates[1] = sigmoid_precise(ld_bf16(b + (size_t)t * hv + head));
        }
        __syncthreads();
        const float kscale = norms[1];
        const float decay = gates[0], beta = gates[1];
        const float v = col_ok ? ld_bf16(row + (size_t)2 * hk * dk + (size_t)head * dv + c0 + col) : 0.f;
        float pred = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int key = kg * kpt + j;
            if (j < kpt && key < dk) {
                s[j] *= decay;
                pred += s[j] * (sk[key] * kscale);
            }
        }
        part[kg][col] = pred;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += part[w][col];
        const float corr = beta * (v - total);
        __syncthreads();
        float o = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int key = kg * kpt + j;
            if (j < kpt && key < dk) {
                s[j] += (sk[key] * kscale) * corr;
                o += s[j] * ((sq[key] * norms[0]) / sqrtf((float)dk));
            }
        }
        part[kg][col] = o;
        __syncthreads();
        if (kg == 0 && col_ok) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) acc += part[w][col];
            out[(size_t)t * hv * dv + (size_t)head * dv + c0 + col] = __float2bfloat16_rn(acc);
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int key = kg * kpt + j;
        if (j < kpt && key < dk && col_ok) tile[(size_t)key * dv] = s[j];
    }
}

// --------------------------------------------------------------------- attention, step 1
// One warp per (token, head): RMSNorm with gamma = 1 + weight, partial RoPE at the token's
// position; query heads go to q_out (bf16), key heads and the values into the cache rows.
__global__ void seq_attn_prepare_kernel(const bf16* __restrict__ qg, const bf16* __restrict__ k_new,
                                        const bf16* __restrict__ v_new, const bf16* __restrict__ q_norm,
                                        const bf16* __restrict__ k_norm, bf16* __restrict__ k_cache,
                                        bf16* __restrict__ v_cache, bf16* __restrict__ q_out, int position0, int hq,
                                        int hk, int d, int rotary, float theta, float eps,
                                        const int* __restrict__ positions, long long cache_stride, int capacity) {
    chain_enter();
    const int t = blockIdx.y, head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= hq + hk) return;
    // a chunk of one sequence: consecutive positions of one cache; batched decode: row t is
    // sequence t at its own position in its own cache
    const int position = positions ? positions[t] : position0 + t;
    if (position < 0 || position >= capacity) return;      // a position outside the cache touches nothing
    if (positions) { k_cache += (size_t)t * cache_stride; v_cache += (size_t)t * cache_stride; }
    const bool is_q = head < hq;
    const bf16* src = is_q ? qg + ((size_t)t * hq + head) * 2 * d : k_new + ((size_t)t * hk + (head - hq)) * d;
    const bf16* gamma_w = is_q ? q_norm : k_norm;
    float v[8], g[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = j * 32 + lane;
        v[j] = i < d ? ld_bf16(src + i) : 0.f;
        g[j] = i < d ? ld_bf16(gamma_w + i) : 0.f;
        ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = round_bf16((v[j] * inv) * (1.0f + g[j]));
    const int hj = rotary / 64;          // registers per half of the rotary part (rotary / 2 a multiple of 32)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (j < hj) {
            const int f = j * 32 + lane;
            const float inv_freq = 1.0f / powf(theta, (float)(2 * f) / (float)rotary);
            const float angle = (float)position * inv_freq;
            const float c = round_bf16(cosf(angle)), sn = round_bf16(sinf(angle));
            const float lo = v[j], hi = v[j + hj];
            v[j] = round_bf16(lo * c + (-hi) * sn);
            v[j + hj] = round_bf16(hi * c + lo * sn);
        }
    }
    bf16* dst = is_q ? q_out + ((size_t)t * hq + head) * d : k_cache + ((size_t)position * hk + (head - hq)) * d;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = j * 32 + lane;
        if (i < d) dst[i] = __float2bfloat16_rn(v[j]);
    }
    if (!is_q) {
        const bf16* vs = v_new + ((size_t)t * hk + (head - hq)) * d;
        bf16* vd = v_cache + ((size_t)position * hk + (head - hq)) * d;
        for (int i = lane; i < d; i += 32) vd[i] = vs[i];
    }
}

// --------------------------------------------------------------------- attention, step 2
// Causal attention of every chunk token over the cache rows [0, position]: block = (token, KV
// head), warp = query head of the group; fp32 online softmax, lane = eight features; output
// bf16(attended) * bf16(sigmoid(gate)).
__global__ void __launch_bounds__(256)
seq_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ qg, const bf16* __restrict__ k_cache,
                const bf16* __restrict__ v_cache, bf16* __restrict__ out, int position0, int hq, int hk, int d) {
    chain_enter();
    const int t = blockIdx.y, kvh = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = hq / hk;
    if (warp >= G) return;
    const int head = kvh * G + warp;
    const int T = position0 + t + 1;
    const int f0 = lane * 8;
    const bool on = f0 < d;
    float qf[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) qf[j] = on ? ld_bf16(q + ((size_t)t * hq + head) * d + f0 + j) : 0.f;
    const float scale = rsqrtf((float)d);
    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < T; ++p) {
        float kf[8], vf[8];
        if (on) {
            const uint4 kr = *reinterpret_cast<const uint4*>(k_cache + ((size_t)p * hk + kvh) * d + f0);
            const uint4 vr = *reinterpret_cast<const uint4*>(v_cache + ((size_t)p * hk + kvh) * d + f0);
            const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kf[2 * j] = __uint_as_float(kw[j] << 16); kf[2 * j + 1] = __uint_as_float(kw[j] & 0xffff0000u);
                vf[2 * j] = __uint_as_float(vw[j] << 16); vf[2 * j + 1] = __uint_as_float(vw[j] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) { kf[j] = 0.f; vf[j] = 0.f; }
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += qf[j] * kf[j];
        const float sc = warp_sum(dot) * scale;
        const float nm = fmaxf(m, sc);
        const float fix = expf(m - nm), pr = expf(sc - nm);
        l = l * fix + pr;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = acc[j] * fix + pr * vf[j];
        m = nm;
    }
    if (on) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float attended = round_bf16(acc[j] / l);
            const float gate = round_bf16(sigmoid_precise(ld_bf16(qg + ((size_t)t * hq + head) * 2 * d + d + f0 + j)));
            out[((size_t)t * hq + head) * d + f0 + j] = __float2bfloat16_rn(attended * gate);
        }
    }
}

// ------------------------------------------------ batched decode attention, lane = position
// One decode step of `batch` sequences over their own caches (rows already prepared by the
// kernel above: q normalised and rotated in q, the new key/value rows in the caches).
// Block = (KV head, context split, sequence), 8 warps; a warp walks its share of the split in
// chunks of 32 positions:
//   scores   lane = one position: its key row against the G query heads (bf16 pairs from
//            shared memory, mixed-precision FMA), 32 independent row reads per warp in flight
//   softmax  per head over the chunk: one warp max and one warp sum per 32 positions
//   values   lane = eight features: the chunk's value rows (coalesced 512-byte rows) weighted
//            by the probabilities that went through shared memory
// then the warps, and across blocks the splits, are merged as in the single-sequence kernel
// (running maximum, sum and weighted values), output = bf16(attended) * bf16(sigmoid(gate)).
constexpr int kLaneAttnWarps = 8, kLaneAttnGroup = 8, kLaneAttnSplitMin = 256;

struct LaneAttnParams {
    const bf16* q;          // [batch, hq, d] prepared queries
    const bf16* qg;         // [batch, hq, 2 d] projection output (the gate is its second half)
    const bf16* k_cache; const bf16* v_cache; long long cache_stride;
    bf16* out;              // [batch, hq * d]
    float* partial;         // [batch, hk, splits, G, d + 2]
    unsigned int* counters; // [batch, hk], zero on entry and on exit
    const int* positions;
    int hq, hk, d, splits, capacity;
};

// The warps' running states (red: [warps][G][d + 2] = weighted values, maximum, sum) become the
// block's partial result; the last block of a (sequence, KV head) merges the splits, normalises
// and gates.  Every thread of the block calls it.
__device__ void lane_attn_finish(const LaneAttnParams& p, const float* __restrict__ red, size_t z, int kvh, int split,
                                 int active, int tid) {
    __shared__ int s_last;
    const int G = p.hq / p.hk, D = p.d, stride = D + 2;
    float* partial = p.partial + z * (size_t)p.hk * p.splits * G * stride;
    float* block_out = partial + (((size_t)kvh * p.splits + split) * G) * stride;
    for (int idx = tid; idx < G * D; idx += kLaneAttnWarps * 32) {
        const int h = idx / D, f = idx % D;
        float mm = -INFINITY;
        for (int w = 0; w < kLaneAttnWarps; ++w) mm = fmaxf(mm, red[((size_t)w * G + h) * stride + D]);
        float num = 0.f, den = 0.f;
        for (int w = 0; w < kLaneAttnWarps; ++w) {
            const float* src = red + ((size_t)w * G + h) * stride;
            const float wgt = src[D] == -INFINITY ? 0.f : expf(src[D] - mm);
            num += wgt * src[f];
            den += wgt * src[D + 1];
        }
        block_out[(size_t)h * stride + f] = num;
        if (f == 0) { block_out[(size_t)h * stride + D] = mm; block_out[(size_t)h * stride + D + 1] = den; }
    }
    __threadfence();
    __syncthreads();
    unsigned int* counter = p.counters + z * p.hk + kvh;
    if (tid == 0) s_last = atomicAdd(counter, 1u) == (unsigned int)p.splits - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- last block of this (sequence, KV head): merge the splits, normalise, gate
    for (int idx = tid; idx < G * D; idx += kLaneAttnWarps * 32) {
        const int h = idx / D, f = idx % D;
        float mm = -INFINITY;
        for (int s = 0; s < active; ++s) mm = fmaxf(mm, __ldcg(partial + (((size_t)kvh * p.splits + s) * G + h) * stride + D));
        float num = 0.f, den = 0.f;
        for (int s = 0; s < active; ++s) {
            const float* src = partial + (((size_t)kvh * p.splits + s) * G + h) * stride;
            const float sm_ = __ldcg(src + D);
            const float wgt = sm_ == -INFINITY ? 0.f : expf(sm_ - mm);
            num += wgt * __ldcg(src + f);
            den += wgt * __ldcg(src + D + 1);
        }
        const float attended = round_bf16(num / den);
        const int qh = kvh * G + h;
        const float gate = round_bf16(sigmoid_precise(ld_bf16(p.qg + (z * p.hq + qh) * 2 * (size_t)D + D + f)));
        p.out[(z * p.hq + qh) * (size_t)D + f] = __float2bfloat16_rn(attended * gate);
    }
    if (tid == 0) *counter = 0;
}

__global__ void __launch_bounds__(kLaneAttnWarps * 32)
batch_attn_lanes_kernel(const LaneAttnParams p) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char lane_attn_smem[];
    const int G = p.hq / p.hk, D = p.d, stride = D + 2;
    bf16* qs = reinterpret_cast<bf16*>(lane_attn_smem);                                  // [G][D]
    float* pbuf = reinterpret_cast<float*>(lane_attn_smem + (size_t)G * D * sizeof(bf16)); // [warps][32][8]
    float* red = pbuf + kLaneAttnWarps * 32 * kLaneAttnGroup;                            // [warps][G][D + 2]
    const int kvh = blockIdx.x, split = blockIdx.y;
    const size_t z = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = p.positions[z] + 1;
    if (T < 1 || T > p.capacity) return;      // a position outside the cache: the sequence's output is left alone
    int active = (T + kLaneAttnSplitMin - 1) / kLaneAttnSplitMin;
    if (active > p.splits) active = p.splits;
    const int per = ((T + active - 1) / active + 31) & ~31;
    const int t0 = split * per, t1 = min(T, t0 + per);
    const bool mine = split < active && t0 < t1;
    const bf16* kc = p.k_cache + z * p.cache_stride;
    const bf16* vc = p.v_cache + z * p.cache_stride;

    if (mine) {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + (z * p.hq + (size_t)kvh * G) * D);
        for (int i = tid; i < G * D / 8; i += kLaneAttnWarps * 32) reinterpret_cast<uint4*>(qs)[i] = __ldg(src + i);
    }
    __syncthreads();

    const int f0 = lane * 8;
    const bool lane_on = f0 < D;
    float m[kLaneAttnGroup], l[kLaneAttnGroup], acc[kLaneAttnGroup][8];
#pragma unroll
    for (int h = 0; h < kLaneAttnGroup; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;
    }
    const float scale = rsqrtf((float)D);
    float* mine_p = pbuf + warp * 32 * kLaneAttnGroup;
    if (mine) {
        for (int c = t0 + warp * 32; c < t1; c += kLaneAttnWarps * 32) {
            const int count = min(32, t1 - c);
            // ---- scores: this lane's position against every head
            const int tl = c + min(lane, count - 1);
            const bf16* krow = kc + ((size_t)tl * p.hk + kvh) * D;
            float score[kLaneAttnGroup];
#pragma unroll
            for (int h = 0; h < kLaneAttnGroup; ++h) score[h] = 0.f;
            for (int fb = 0; fb < D; fb += 32) {
                uint4 kk[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) kk[i] = __ldg(reinterpret_cast<const uint4*>(krow + fb) + i);
#pragma unroll
                for (int h = 0; h < kLaneAttnGroup; ++h) {
                    if (h < G) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint4 qq = *reinterpret_cast<const uint4*>(qs + h * D + fb + 8 * i);
                            score[h] = fma_bf16_lo(kk[i].x, qq.x, score[h]); score[h] = fma_bf16_hi(kk[i].x, qq.x, score[h]);
                            score[h] = fma_bf16_lo(kk[i].y, qq.y, score[h]); score[h] = fma_bf16_hi(kk[i].y, qq.y, score[h]);
                            score[h] = fma_bf16_lo(kk[i].z, qq.z, score[h]); score[h] = fma_bf16_hi(kk[i].z, qq.z, score[h]);
                            score[h] = fma_bf16_lo(kk[i].w, qq.w, score[h]); score[h] = fma_bf16_hi(kk[i].w, qq.w, score[h]);
                        }
                    }
                }
            }
            // ---- softmax over the chunk, per head
            float prob[kLaneAttnGroup];
#pragma unroll
            for (int h = 0; h < kLaneAttnGroup; ++h) {
                prob[h] = 0.f;
                if (h < G) {
                    const float sc = lane < count ? score[h] * scale : -INFINITY;
                    const float nm = fmaxf(m[h], warp_max(sc));
                    const float fix = expf(m[h] - nm);
                    prob[h] = lane < count ? expf(sc - nm) : 0.f;
                    l[h] = l[h] * fix + warp_sum(prob[h]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[h][j] *= fix;
                    m[h] = nm;
                }
            }
            __syncwarp();
            *reinterpret_cast<float4*>(mine_p + lane * kLaneAttnGroup) = make_float4(prob[0], prob[1], prob[2], prob[3]);
            *reinterpret_cast<float4*>(mine_p + lane * kLaneAttnGroup + 4) = make_float4(prob[4], prob[5], prob[6], prob[7]);
            __syncwarp();
            // ---- values: this lane's eight features of every position of the chunk
            if (lane_on) {
#pragma unroll 4
                for (int j = 0; j < count; ++j) {
                    const uint4 vr = __ldg(reinterpret_cast<const uint4*>(vc + ((size_t)(c + j) * p.hk + kvh) * D + f0));
                    const uint32_t vw[4] = {vr.x, vr.y, vr.z, vr.w};
                    float vf[8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) { vf[2 * q] = __uint_as_float(vw[q] << 16); vf[2 * q + 1] = __uint_as_float(vw[q] & 0xffff0000u); }
                    const float4 pa = *reinterpret_cast<const float4*>(mine_p + j * kLaneAttnGroup);
                    const float4 pb = *reinterpret_cast<const float4*>(mine_p + j * kLaneAttnGroup + 4);
                    const float pr[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                    for (int h = 0; h < kLaneAttnGroup; ++h) {
                        if (h < G) {
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[h][e] += pr[h] * vf[e];
                        }
                    }
                }
            }
        }
    }
    // ---- merge the warps of this block
#pragma unroll
    for (int h = 0; h < kLaneAttnGroup; ++h) {
        if (h < G) {
            float* dst = red + ((size_t)warp * G + h) * stride;
            if (lane_on) {
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[f0 + j] = acc[h][j];
            }
            if (lane == 0) { dst[D] = m[h]; dst[D + 1] = l[h]; }
        }
    }
    __syncthreads();
    lane_attn_finish(p, red, z, kvh, split, active, tid);
}

// ------------------------------------------------ batched decode attention on the tensor cores
// The same block layout (KV head, context split, sequence; 8 warps) for head dimension 256: a
// warp walks its share of the split sixteen positions at a time with the fragment arithmetic of
// attn_mma.cuh (scores S^T = K Q^T, running softmax, O^T += V^T P^T).  Every key and value
// element is needed by exactly one lane of the warp, so the rows go from the cache straight
// into the MMA fragments (no staging in shared memory): per chunk a lane loads 16 x 16 bytes of
// its two key rows, and, once the scores are out, 16 x 16 bytes of four value rows while the
// next chunk's keys are already on their way.  The lane-per-position kernel above spends its
// time in scalar FMAs (28 % of the HBM bandwidth at 32 sequences x 8192 positions).
struct AttnKeys { uint4 a[8], b[8]; };      // bytes 64 m + 16 t .. + 15 of key rows prow and 8 + prow

QD_DEVINL uint4 ld_stream16(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// rows past `last` (masked positions of the final chunk) read row `last`, which is initialised
QD_DEVINL void attn_load_keys(AttnKeys& k, const uint8_t* __restrict__ base, size_t row_bytes, int first, int last, int lane) {
    const int g = lane >> 2, t = lane & 3, prow = qd::attn_key_row(g);
    const uint8_t* r0 = base + (size_t)min(first + prow, last) * row_bytes + t * 16;
    const uint8_t* r1 = base + (size_t)min(first + 8 + prow, last) * row_bytes + t * 16;
#pragma unroll
    for (int m = 0; m < 8; ++m) { k.a[m] = ld_stream16(r0 + m * 64); k.b[m] = ld_stream16(r1 + m * 64); }
}

__global__ void __launch_bounds__(kLaneAttnWarps * 32, 1)
batch_attn_mma_kernel(const LaneAttnParams p) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char mma_attn_smem[];
    constexpr int D = 256;
    const int G = p.hq / p.hk, stride = D + 2;
    uint8_t* q_s = mma_attn_smem;                                                       // [8][kAttnQRow]
    float* red = reinterpret_cast<float*>(mma_attn_smem + 8 * kAttnQRow);               // [warps][G][D + 2]
    const int kvh = blockIdx.x, split = blockIdx.y;
    const size_t z = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int T = p.positions[z] + 1;
    if (T < 1 || T > p.capacity) return;      // a position outside the cache: the sequence's output is left alone
    int active = (T + kLaneAttnSplitMin - 1) / kLaneAttnSplitMin;
    if (active > p.splits) active = p.splits;
    const int per = ((T + active - 1) / active + 31) & ~31;
    const int t0 = split * per, t1 = min(T, t0 + per);
    const bool mine = split < active && t0 < t1;
    const size_t row_bytes = (size_t)p.hk * D * sizeof(bf16);
    const uint8_t* kc = reinterpret_cast<const uint8_t*>(p.k_cache + z * p.cache_stride + (size_t)kvh * D);
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(p.v_cache + z * p.cache_stride + (size_t)kvh * D);

    AttnAcc acc;
    acc.m = -INFINITY; acc.l = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc.out[i][0] = 0.f; acc.out[i][1] = 0.f; acc.out[i][2] = 0.f; acc.out[i][3] = 0.f; }
    if (mine) {
        AttnKeys keys;
        int c = t0 + warp * 16;
        if (c < t1) attn_load_keys(keys, kc, row_bytes, c, T - 1, lane);
        // query heads of this KV head (heads beyond the group: zeros)
        for (int i = tid; i < 8 * 32; i += kLaneAttnWarps * 32) {
            const int h = i >> 5, piece = i & 31;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (h < G) v = __ldg(reinterpret_cast<const uint4*>(p.q + (z * p.hq + (size_t)kvh * G + h) * D) + piece);
            reinterpret_cast<uint4*>(q_s + h * kAttnQRow)[piece] = v;
        }
        __syncthreads();
#pragma unroll 1
        for (; c < t1; c += kLaneAttnWarps * 16) {
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < 8; ++m)
                qd::attn_score_step(s0, s1, lds128(q_s + g * kAttnQRow + m * 64 + t * 16), keys.a[m], keys.b[m]);
            uint4 values[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint8_t* row = vc + (size_t)min(c + 4 * i + t, T - 1) * row_bytes + g * 64;
#pragma unroll
                for (int q = 0; q < 4; ++q) values[q][i] = ld_stream16(row + q * 16);
            }
            if (c + kLaneAttnWarps * 16 < t1) attn_load_keys(keys, kc, row_bytes, c + kLaneAttnWarps * 16, T - 1, lane);
            const qd::AttnProbs pr = qd::attn_softmax(acc, s0, s1, c, t1, lane);
#pragma unroll
            for (int q = 0; q < 4; ++q) qd::attn_value_step(acc, q, values[q][0], values[q][1], values[q][2], values[q][3], pr);
        }
    } else {
        __syncthreads();
    }
    // ---- the warp's state in the layout of the merge: lane (g, t) holds the statistics of head g
    // (the sum still spread over its four lanes) and out[i][c] = feature 32 g + 2 i + (c >> 1) of head 2 t + (c & 1)
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 1);
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 2);
    if (t == 0 && g < G) {
        float* dst = red + ((size_t)warp * G + g) * stride;
        dst[D] = acc.m; dst[D + 1] = acc.l;
    }
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int h = 2 * t + cc;
        if (h >= G) continue;
        float* dst = red + ((size_t)warp * G + h) * stride + 32 * g;
#pragma unroll
        for (int i = 0; i < 16; ++i) { dst[2 * i] = acc.out[i][cc]; dst[2 * i + 1] = acc.out[i][2 + cc]; }
    }
    __syncthreads();
    lane_attn_finish(p, red, z, kvh, split, active, tid);
}

// ------------------------------------------------ causal attention of a prompt chunk on the tensor cores
// The chunk's tokens sit at consecutive positions position0 .. position0 + tokens - 1 of ONE
// cache (rows already prepared by seq_attn_prepare_kernel).  Block = (sixteen consecutive tokens,
// KV head); a warp owns one token and its (up to eight) query heads of that KV head.  The block
// walks the cache in tiles of 64 positions: key and value rows of the tile are copied to shared
// memory once (cp.async, two tiles in flight) and read by all sixteen warps, which is what the
// lane-per-position kernel cannot do (there every token streams its whole history from L2).  A
// warp multiplies its heads with sixteen positions at a time on mma.sync (attn_mma.cuh: scores
// S^T = K Q^T, running softmax, O^T += V^T P^T with the probabilities as one bf16 piece) up to its
// own position; output = bf16(attended) * bf16(sigmoid(gate)) as in the decode kernels
// (quickdraw/kernel/triton/attention.py:53-100).  Head dimension 256, group of at most 8.
constexpr int kFlashTokens = 16, kFlashTile = 64, kFlashThreads = kFlashTokens * 32;
constexpr int kFlashTileBytes = 2 * kFlashTile * kAttnRow;      // key rows, then value rows
constexpr size_t kFlashSmem = (size_t)kFlashTokens * 8 * kAttnQRow + 2 * (size_t)kFlashTileBytes;

__global__ void __launch_bounds__(kFlashThreads, 1)
seq_flash_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ qg, const bf16* __restrict__ k_cache,
                           const bf16* __restrict__ v_cache, bf16* __restrict__ out, int tokens, int position0, int hq, int hk) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char flash_smem[];
    constexpr int D = 256;
    const int G = hq / hk, kvh = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int token0 = blockIdx.x * kFlashTokens, token = token0 + warp;
    const bool live = token < tokens;
    uint8_t* q_s = flash_smem + (size_t)warp * 8 * kAttnQRow;                      // this warp's query heads
    uint8_t* tiles = flash_smem + (size_t)kFlashTokens * 8 * kAttnQRow;
    // query heads of the warp's token (heads beyond the group, and a token beyond the chunk: zeros)
    for (int h = 0; h < 8; ++h) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (live && h < G) v = reinterpret_cast<const uint4*>(q + ((size_t)token * hq + kvh * G + h) * D)[lane];
        reinterpret_cast<uint4*>(q_s + h * kAttnQRow)[lane] = v;
    }
    // positions every token of the block may see: [0, last]; the warp's own limit is its position
    const int last = position0 + min(tokens, token0 + kFlashTokens) - 1;
    const int mine = live ? position0 + token + 1 : 0;                             // end of the warp's range
    const int ntiles = last / kFlashTile + 1;
    auto fetch = [&](int tile) {
        // 64 key rows and 64 value rows of 512 bytes: 32 sixteen-byte pieces per row, 4096 pieces in all
        uint8_t* dst = tiles + (size_t)(tile & 1) * kFlashTileBytes;
        const int first = tile * kFlashTile;
        for (int piece = tid; piece < 2 * kFlashTile * 32; piece += kFlashThreads) {
            const int row = piece >> 5, c = piece & 31, pos = first + (row & (kFlashTile - 1));
            const bf16* src = (row < kFlashTile ? k_cache : v_cache) + ((size_t)min(pos, last) * hk + kvh) * D;
            const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + (size_t)row * kAttnRow + c * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(reinterpret_cast<const uint8_t*>(src) + c * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    AttnAcc acc;
    acc.m = -INFINITY; acc.l = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc.out[i][0] = 0.f; acc.out[i][1] = 0.f; acc.out[i][2] = 0.f; acc.out[i][3] = 0.f; }
    fetch(0);
    for (int tile = 0; tile < ntiles; ++tile) {
        if (tile + 1 < ntiles) { fetch(tile + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                   // the tile (and, the first time, the queries) are in place
        const uint8_t* buf = tiles + (size_t)(tile & 1) * kFlashTileBytes;
        const int first = tile * kFlashTile;
#pragma unroll 1
        for (int c = 0; c < kFlashTile / 16; ++c) {
            const int start = first + 16 * c;
            if (start < mine)
                attn_chunk<false>(acc, q_s, buf + (size_t)(16 * c) * kAttnRow, buf + (size_t)(kFlashTile + 16 * c) * kAttnRow, start, mine, lane);
        }
        __syncthreads();                                   // everybody is done with this buffer before it is refilled
    }
    if (!live) return;
    // ---- normalise and gate: lane (g, t) holds out[i][c] = feature 32 g + 2 i + (c >> 1) of head 2 t + (c & 1)
    const int g = lane >> 2, t = lane & 3;
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 1);
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 2);
    const float l_even = __shfl_sync(0xffffffffu, acc.l, 8 * t), l_odd = __shfl_sync(0xffffffffu, acc.l, 8 * t + 4);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int h = 2 * t + cc;
        if (h >= G) continue;
        const int qh = kvh * G + h;
        const float den = cc ? l_odd : l_even;
        const bf16* gate_row = qg + ((size_t)token * hq + qh) * 2 * D + D;
        bf16* dst = out + ((size_t)token * hq + qh) * D;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int f = 32 * g + 2 * i;
            const float a0 = round_bf16(acc.out[i][cc] / den), a1 = round_bf16(acc.out[i][2 + cc] / den);
            const float g0 = round_bf16(sigmoid_precise(ld_bf16(gate_row + f))), g1 = round_bf16(sigmoid_precise(ld_bf16(gate_row + f + 1)));
            *reinterpret_cast<__nv_bfloat162*>(dst + f) = __floats2bfloat162_rn(a0 * g0, a1 * g1);
        }
    }
}

// ----------------------------------------------------------------------------- routing
__global__ void seq_route_kernel(const bf16* __restrict__ logits, int experts, int topk, int32_t* __restrict__ ids,
                                 float* __restrict__ weights) {
    chain_enter();
    const int t = blockIdx.x;
    qd::route_small(logits + (size_t)t * experts, experts, topk, ids + (size_t)t * topk, weights + (size_t)t * topk,
                    threadIdx.x);
}

// --------------------------------------------------------- routes of a chunk by expert
// The stable order of the chunk's (token, slot) routes by expert id, as the reference groups
// them (quickdraw/kernel/triton/moe.py:60-97): order[r] = route index of sorted row r,
// boundaries[e] = first sorted row of expert e.  One block; every warp owns a contiguous slice
// of the routes and a private row of per-expert counters in shared memory.  Pass 1 counts the
// slice (32 routes at a time: lanes with the same expert find one another with match_any, the
// lowest of them adds their number), a scan in (expert, warp) order turns the counters into
// first positions, pass 2 walks the slice again and places every route at its expert's
// running position plus its rank among the equal lanes below it.
__global__ void __launch_bounds__(1024)
seq_group_routes_kernel(const int32_t* __restrict__ ids, int routes, int experts, int32_t* __restrict__ order,
                        int32_t* __restrict__ boundaries) {
    chain_enter();
    extern __shared__ int32_t counters[];               // [warps][experts], then first[experts + 1]
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* first = counters + warps * experts;
    for (int i = threadIdx.x; i < warps * experts; i += blockDim.x) counters[i] = 0;
    __syncthreads();
    const int slice = ((routes + warps - 1) / warps + 31) & ~31;
    const int begin = min(routes, warp * slice), end = min(routes, begin + slice);
    int32_t* mine = counters + warp * experts;
    for (int r0 = begin; r0 < end; r0 += 32) {
        const int r = r0 + lane;
        const int e = r < end ? ids[r] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
    }
    __syncthreads();
    // totals per expert, their exclusive scan, then every warp's first position per expert
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int total = 0;
        for (int w = 0; w < warps; ++w) total += counters[w * experts + e];
        first[e + 1] = total;
    }
    if (threadIdx.x == 0) first[0] = 0;
    __syncthreads();
    if (warp == 0) {      // inclusive scan by one warp: a lane adds up its run of experts, the runs are scanned with shuffles
        const int run = (experts + 31) / 32, lo = min(experts, lane * run), hi = min(experts, lo + run);
        int sum = 0;
        for (int e = lo; e < hi; ++e) sum += first[e + 1];
        int inclusive = sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int below = __shfl_up_sync(0xffffffffu, inclusive, d);
            if (lane >= d) inclusive += below;
        }
        int running = inclusive - sum;
        for (int e = lo; e < hi; ++e) { running += first[e + 1]; first[e + 1] = running; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) boundaries[e] = first[e];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int at = first[e];
        for (int w = 0; w < warps; ++w) {
            const int n = counters[w * experts + e];
            counters[w * experts + e] = at;
            at += n;
        }
    }
    __syncthreads();
    for (int r0 = begin; r0 < end; r0 += 32) {
        const int r = r0 + lane;
        const int e = r < end ? ids[r] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        int at = 0;
        if (e >= 0) at = mine[e] + __popc(same & ((1u << lane) - 1u));
        __syncwarp();
        if (e >= 0 && lane == __ffs(same) - 1) mine[e] += __popc(same);
        __syncwarp();
        if (e >= 0) order[at] = r;
    }
}

// --------------------------------------------------------------------------- MoE combine
// out[t] = bf16( bf16(sum of the token's routed rows in ascending expert id) +
//                bf16(shared[t] * bf16(sigmoid(strength[t]))) )
__global__ void __launch_bounds__(256)
seq_combine_kernel(const bf16* __restrict__ contributions, const int32_t* __restrict__ ids,
                   const bf16* __restrict__ shared, const bf16* __restrict__ strength,
                   bf16* __restrict__ out, int hidden, int topk) {
    chain_enter();
    // block = one token; slot_of[n] = the slot with the n-th smallest expert id; a thread then
    // adds eight features of the token's rows in that order (16-byte loads)
    __shared__ int slot_of[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int32_t* my = ids + (size_t)t * topk;
    if (tid < topk) {
        const int e = my[tid];
        int rank = 0;
        for (int s = 0; s < topk; ++s) { const int o = my[s]; rank += (o < e) || (o == e && s < tid); }
        slot_of[rank] = tid;
    }
    __syncthreads();
    const bf16* rows = contributions + (size_t)t * topk * hidden;
    const float gate = round_bf16(sigmoid_precise(ld_bf16(strength + t)));
    if (hidden % 8 == 0 && !(((uintptr_t)contributions | (uintptr_t)shared | (uintptr_t)out) & 15u)) {
        for (int i = tid * 8; i < hidden; i += 256 * 8) {
            float routed[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
            for (int n = 0; n < topk; ++n) {
                const uint4 v = *reinterpret_cast<const uint4*>(rows + (size_t)slot_of[n] * hidden + i);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) { routed[2 * q] += bf16_bits_to_float(w[q] & 0xffffu); routed[2 * q + 1] += bf16_bits_to_float(w[q] >> 16); }
            }
            const uint4 sh = *reinterpret_cast<const uint4*>(shared + (size_t)t * hidden + i);
            const uint32_t sw[4] = {sh.x, sh.y, sh.z, sh.w};
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float lo = round_bf16(routed[2 * q]) + round_bf16(bf16_bits_to_float(sw[q] & 0xffffu) * gate);
                const float hi = round_bf16(routed[2 * q + 1]) + round_bf16(bf16_bits_to_float(sw[q] >> 16) * gate);
                o[q] = qd::pack_bf16x2(lo, hi);
            }
            *reinterpret_cast<uint4*>(out + (size_t)t * hidden + i) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    for (int i = tid; i < hidden; i += 256) {
        float routed = 0.f;
        for (int n = 0; n < topk; ++n) routed += ld_bf16(rows + (size_t)slot_of[n] * hidden + i);
        const float gated = round_bf16(ld_bf16(shared + (size_t)t * hidden + i) * gate);
        out[(size_t)t * hidden + i] = __float2bfloat16_rn(round_bf16(routed) + gated);
    }
}

// The combine above followed by the residual add + RMSNorm in front of the next layer (seq_add_norm8_kernel),
// a token per block: thread tid holds the same eight features (pieces tid and tid + 256) in both, so the
// layer output never goes to memory.  normed / residual_out as seq_add_norm8_kernel writes them for
// x = the combine's bf16 output.  hidden a multiple of 8, at most 4096.
__global__ void __launch_bounds__(256)
seq_combine_norm_kernel(const bf16* __restrict__ contributions, const int32_t* __restrict__ ids,
                        const bf16* __restrict__ shared, const bf16* __restrict__ strength,
                        const bf16* __restrict__ residual, const float* __restrict__ gamma,
                        bf16* __restrict__ normed, bf16* __restrict__ residual_out, int hidden, int topk, float eps) {
    chain_enter();
    __shared__ int slot_of[32];
    __shared__ float partial[8];
    const int t = blockIdx.x, tid = threadIdx.x, pieces = hidden / 8;
    const int32_t* my = ids + (size_t)t * topk;
    if (tid < topk) {
        const int e = my[tid];
        int rank = 0;
        for (int s = 0; s < topk; ++s) { const int o = my[s]; rank += (o < e) || (o == e && s < tid); }
        slot_of[rank] = tid;
    }
    __syncthreads();
    const bf16* rows = contributions + (size_t)t * topk * hidden;
    const float gate = round_bf16(sigmoid_precise(ld_bf16(strength + t)));
    const size_t base = (size_t)t * hidden;
    float v[kNormVecs][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kNormVecs; ++k) {
        const int c = tid + k * 256;
        if (c >= pieces) break;
        float routed[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int n = 0; n < topk; ++n) {
            const uint4 row = *reinterpret_cast<const uint4*>(rows + (size_t)slot_of[n] * hidden + 8 * c);
            const uint32_t w[4] = {row.x, row.y, row.z, row.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) { routed[2 * q] += bf16_bits_to_float(w[q] & 0xffffu); routed[2 * q + 1] += bf16_bits_to_float(w[q] >> 16); }
        }
        const uint4 sh = *reinterpret_cast<const uint4*>(shared + base + 8 * c);
        const uint4 r = *reinterpret_cast<const uint4*>(residual + base + 8 * c);
        const uint32_t sw[4] = {sh.x, sh.y, sh.z, sh.w}, rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            // the layer output as the combine rounds it, then the sum with the residual as the norm kernel forms it
            const float lo = round_bf16(round_bf16(routed[2 * q]) + round_bf16(bf16_bits_to_float(sw[q] & 0xffffu) * gate));
            const float hi = round_bf16(round_bf16(routed[2 * q + 1]) + round_bf16(bf16_bits_to_float(sw[q] >> 16) * gate));
            v[k][2 * q] = lo + __uint_as_float(rw[q] << 16);
            v[k][2 * q + 1] = hi + __uint_as_float(rw[q] & 0xffff0000u);
            ss += v[k][2 * q] * v[k][2 * q] + v[k][2 * q + 1] * v[k][2 * q + 1];
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) partial[tid >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += partial[w];
    const float inv = rsqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < kNormVecs; ++k) {
        const int c = tid + k * 256;
        if (c >= pieces) break;
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + 8 * c), g1 = *reinterpret_cast<const float4*>(gamma + 8 * c + 4);
        const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t n[4], o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            n[q] = qd::pack_bf16x2((v[k][2 * q] * inv) * gm[2 * q], (v[k][2 * q + 1] * inv) * gm[2 * q + 1]);
            o[q] = qd::pack_bf16x2(v[k][2 * q], v[k][2 * q + 1]);
        }
        *reinterpret_cast<uint4*>(normed + base + 8 * c) = make_uint4(n[0], n[1], n[2], n[3]);
        *reinterpret_cast<uint4*>(residual_out + base + 8 * c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace

extern "C" int qd_seq_add_rms_norm(const void* x, const void* residual, const float* gamma, void* normed,
                                   void* residual_out, int tokens, int width, float eps, void* stream) {
    QD_CHECK_ARG(x && gamma && normed && residual_out && tokens > 0 && width > 0);
    const uintptr_t align = (uintptr_t)x | (uintptr_t)residual | (uintptr_t)gamma | (uintptr_t)normed | (uintptr_t)residual_out;
    if (width % 8 == 0 && width <= 8 * 256 * kNormVecs && !(align & 15u))
        qd_launch(seq_add_norm8_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)residual, gamma,
                                                                       (bf16*)normed, (bf16*)residual_out, width, eps);
    else
        qd_launch(seq_add_norm_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)residual, gamma,
                                                                      (bf16*)normed, (bf16*)residual_out, width, eps);
    return qd_launch_status();
}

extern "C" int qd_seq_bf16_matmul(const void* x, const void* w, void* y, int tokens, int rows, int width, void* stream) {
    QD_CHECK_ARG(x && w && y && tokens > 0 && rows > 0 && width > 0);
    const uintptr_t align = (uintptr_t)x | (uintptr_t)w;
    if ((rows >= 4096 || tokens >= 64) && width % 64 == 0 && width <= kTallMaxWidth && !(align & 15u) && (tokens + 31) / 32 <= 65535) {
        // tall matrix or many tokens: every weight row is read once per tile of 32 tokens (tensor-core form)
        const size_t smem = (size_t)kTallTokens * (width * sizeof(bf16) + 16);
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
        static bool configured[64];
        if (!configured[dev]) {
            if (cudaFuncSetAttribute(seq_bf16_matmul_tall_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTallTokens * (kTallMaxWidth * 2 + 16)) != cudaSuccess)
                return QD_ERR_LAUNCH;
            configured[dev] = true;
        }
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        // sixteen row groups per block, fewer while the blocks do not fill the GPU; then the idle warps take
        // parts of the inputs (a power of two that divides the steps of 64 inputs), if the sums fit behind the tokens
        const int row_groups = (rows + 15) / 16, token_tiles = (tokens + 31) / 32;
        int per_block = kTallWarps;
        while (per_block > 1 && (long long)((row_groups + per_block - 1) / per_block) * token_tiles < sms &&
               (per_block > 2 || row_groups == 1)) per_block >>= 1;
        const int row_blocks = (row_groups + per_block - 1) / per_block;
        int parts = 1;
        if (row_blocks <= sms && per_block < kTallWarps) {
            parts = kTallWarps / per_block;
            while (parts > 1 && (width / 64) % parts != 0) parts >>= 1;
        }
        size_t launch_smem = smem;
        if (parts > 1) {
            launch_smem += (size_t)(parts - 1) * per_block * 4 * 32 * 16;
            if (launch_smem > (size_t)kTallTokens * (kTallMaxWidth * 2 + 16)) { parts = 1; launch_smem = smem; }
        }
        qd_launch(seq_bf16_matmul_tall_kernel, dim3(row_blocks < sms ? row_blocks : sms, token_tiles), dim3(kTallWarps * 32), launch_smem, (cudaStream_t)stream, true, 
            (const bf16*)x, (const bf16*)w, (bf16*)y, tokens, rows, width, per_block, parts);
        return qd_launch_status();
    }
    qd_launch(seq_bf16_matmul_kernel, dim3((rows + 7) / 8, tokens), dim3(256), 0, (cudaStream_t)stream, true,
              (const bf16*)x, (const bf16*)w, (bf16*)y, rows, width, (const bf16*)nullptr, (bf16*)nullptr, 0, 0);
    return qd_launch_status();
}

// Two small matrices of the same input in one launch (the a and b projections of a DeltaNet layer, the
// router and the shared-expert gate: quickdraw/models/qwen.py:120-131, 165-170); shapes that
// qd_seq_bf16_matmul gives to the tensor-core form go there one after the other.
extern "C" int qd_seq_bf16_matmul2(const void* x, const void* w0, void* y0, int rows0, const void* w1, void* y1, int rows1,
                                   int tokens, int width, void* stream) {
    QD_CHECK_ARG(x && w0 && y0 && w1 && y1 && tokens > 0 && rows0 > 0 && rows1 > 0 && width > 0);
    if (rows0 >= 4096 || rows1 >= 4096 || tokens >= 64 || tokens > 65535) {
        const int first = qd_seq_bf16_matmul(x, w0, y0, tokens, rows0, width, stream);
        return first != QD_OK ? first : qd_seq_bf16_matmul(x, w1, y1, tokens, rows1, width, stream);
    }
    const int blocks0 = (rows0 + 7) / 8, blocks1 = (rows1 + 7) / 8;
    qd_launch(seq_bf16_matmul_kernel, dim3(blocks0 + blocks1, tokens), dim3(256), 0, (cudaStream_t)stream, true,
              (const bf16*)x, (const bf16*)w0, (bf16*)y0, rows0, width, (const bf16*)w1, (bf16*)y1, rows1, blocks0);
    return qd_launch_status();
}

extern "C" int qd_seq_gdn_conv(const void* mixed, const void* taps, void* conv_state, void* out, int tokens,
                               int channels, int width, void* stream) {
    QD_CHECK_ARG(mixed && taps && out && tokens > 0 && channels > 0 && width >= 1 && width <= 8 && (width == 1 || conv_state));
    if (tokens > 65535) return QD_ERR_UNSUPPORTED;
    if (width == 4 && channels % 2 == 0 && tokens >= kConvRun && !(((uintptr_t)mixed | (uintptr_t)out) & 3u) && !((uintptr_t)taps & 7u))
        qd_launch(seq_conv4_kernel, dim3((channels / 2 + 127) / 128, (tokens + kConvRun - 1) / kConvRun), dim3(128), 0, (cudaStream_t)stream, true, 
            (const bf16*)mixed, (const bf16*)taps, (const bf16*)conv_state, (bf16*)out, tokens, channels);
    else
        qd_launch(seq_conv_kernel, dim3((channels + 127) / 128, tokens), dim3(128), 0, (cudaStream_t)stream, true, 
            (const bf16*)mixed, (const bf16*)taps, (const bf16*)conv_state, (bf16*)out, channels, width);
    if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    if (width > 1)
        qd_launch(seq_conv_state_kernel, dim3((channels + 127) / 128), dim3(128), 0, (cudaStream_t)stream, true, 
            (const bf16*)mixed, (bf16*)conv_state, tokens, channels, width);
    return qd_launch_status();
}

extern "C" int qd_seq_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                     const void* dt_bias, float* rec_state, void* out, int tokens, int key_heads,
                                     int value_heads, int key_dim, int value_dim, void* stream) {
    QD_CHECK_ARG(conv_qkv && a && b && a_log && dt_bias && rec_state && out && tokens > 0);
    QD_CHECK_ARG(key_heads > 0 && value_heads % key_heads == 0 && key_dim > 0 && value_dim > 0);
    if (key_dim > 128) return QD_ERR_UNSUPPORTED;
    if (key_dim == 128) {
        qd_launch(seq_recurrence128_kernel, dim3(value_heads, (value_dim + kRecCols - 1) / kRecCols), dim3(128), 0, (cudaStream_t)stream, true, 
            (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log, (const bf16*)dt_bias, rec_state,
            (bf16*)out, tokens, key_heads, value_heads, value_dim, 0);
        return qd_launch_status();
    }
    qd_launch(seq_recurrence_kernel, dim3(value_heads, (value_dim + 31) / 32), dim3(256), 0, (cudaStream_t)stream, true, 
        (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log, (const bf16*)dt_bias, rec_state,
        (bf16*)out, tokens, key_heads, value_heads, key_dim, value_dim);
    return qd_launch_status();
}

/* batched decode: one token of each of `batch` sequences */
extern "C" int qd_batch_gdn_conv(const void* mixed, const void* taps, void* conv_state, long long state_stride,
                                 void* out, int batch, int channels, int width, void* stream) {
    QD_CHECK_ARG(mixed && taps && out && batch > 0 && batch <= 65535 && channels > 0 && width >= 1 && width <= 8);
    QD_CHECK_ARG(width == 1 || (conv_state && (batch == 1 || state_stride >= (long long)channels * (width - 1))));
    qd_launch(batch_conv_kernel, dim3((channels + 127) / 128, batch), dim3(128), 0, (cudaStream_t)stream, true, 
        (const bf16*)mixed, (const bf16*)taps, (bf16*)conv_state, (bf16*)out, channels, width, state_stride);
    return qd_launch_status();
}

extern "C" int qd_batch_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                       const void* dt_bias, float* rec_state, long long state_stride, void* out,
                                       int batch, int key_heads, int value_heads, int key_dim, int value_dim,
                                       void* stream) {
    QD_CHECK_ARG(conv_qkv && a && b && a_log && dt_bias && rec_state && out && batch > 0 && batch <= 65535);
    QD_CHECK_ARG(key_heads > 0 && value_heads % key_heads == 0 && key_dim > 0 && value_dim > 0);
    QD_CHECK_ARG(batch == 1 || state_stride >= (long long)value_heads * key_dim * value_dim);
    if (key_dim != 128) return QD_ERR_UNSUPPORTED;
    qd_launch(seq_recurrence128_kernel, dim3(value_heads, (value_dim + kRecCols - 1) / kRecCols, batch), dim3(128), 0, (cudaStream_t)stream, true, 
        (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log, (const bf16*)dt_bias, rec_state,
        (bf16*)out, 1, key_heads, value_heads, value_dim, state_stride);
    return qd_launch_status();
}

extern "C" int qd_seq_attention(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                                const void* k_norm, void* k_cache, void* v_cache, void* q_scratch, void* out,
                                int tokens, int position0, int capacity, int q_heads, int kv_heads, int head_dim,
                                int rotary_dim, float theta, float eps, void* stream) {
    QD_CHECK_ARG(qg && k_new && v_new && q_norm && k_norm && k_cache && v_cache && q_scratch && out);
    QD_CHECK_ARG(tokens > 0 && position0 >= 0 && position0 + tokens <= capacity && kv_heads > 0 && q_heads % kv_heads == 0);
    if (head_dim > 256 || head_dim % 8 != 0 || q_heads / kv_heads > 8 || rotary_dim % 64 != 0 || rotary_dim > head_dim)
        return QD_ERR_UNSUPPORTED;
    const int heads = q_heads + kv_heads;
    qd_launch(seq_attn_prepare_kernel, dim3((heads + 7) / 8, tokens), dim3(256), 0, (cudaStream_t)stream, true, 
        (const bf16*)qg, (const bf16*)k_new, (const bf16*)v_new, (const bf16*)q_norm, (const bf16*)k_norm,
        (bf16*)k_cache, (bf16*)v_cache, (bf16*)q_scratch, position0, q_heads, kv_heads, head_dim, rotary_dim, theta, eps,
        nullptr, 0, capacity);
    if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    if (head_dim == 256 && tokens >= 2) {
        // the tensor-core kernel: every cache tile is shared by sixteen tokens
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
        static bool flash_configured[64];
        if (!flash_configured[dev]) {
            if (cudaFuncSetAttribute(seq_flash_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFlashSmem) != cudaSuccess)
                return QD_ERR_LAUNCH;
            flash_configured[dev] = true;
        }
        qd_launch(seq_flash_attention_kernel, dim3((tokens + kFlashTokens - 1) / kFlashTokens, kv_heads), dim3(kFlashThreads), kFlashSmem, (cudaStream_t)stream, true, (const bf16*)q_scratch, (const bf16*)qg, (const bf16*)k_cache,
                                                             (const bf16*)v_cache, (bf16*)out, tokens, position0, q_heads, kv_heads);
        return qd_launch_status();
    }
    qd_launch(seq_attn_kernel, dim3(kv_heads, tokens), dim3(256), 0, (cudaStream_t)stream, true, 
        (const bf16*)q_scratch, (const bf16*)qg, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, position0,
        q_heads, kv_heads, head_dim);
    return qd_launch_status();
}

/* batched decode attention: prepare (norm, RoPE, cache write at every sequence's position)
 * and the lane-per-position kernel */
extern "C" int qd_batch_attention(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                                  const void* k_norm, void* k_cache, void* v_cache, long long cache_stride,
                                  void* q_scratch, void* out, float* scratch, unsigned int* counters,
                                  const int* positions, int batch, int capacity, int q_heads, int kv_heads,
                                  int head_dim, int rotary_dim, float theta, float eps, int splits, void* stream) {
    QD_CHECK_ARG(qg && k_new && v_new && q_norm && k_norm && k_cache && v_cache && q_scratch && out && scratch && counters && positions);
    QD_CHECK_ARG(batch > 0 && batch <= 65535 && capacity > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && splits >= 1);
    // cache_stride 0: the rows are consecutive tokens of ONE sequence (a prompt chunk; positions
    // ascending), every row attends over the shared cache up to its own position
    QD_CHECK_ARG(batch == 1 || cache_stride == 0 || cache_stride >= (long long)capacity * kv_heads * head_dim);
    const int G = q_heads / kv_heads;
    if (head_dim > 256 || head_dim % 32 != 0 || G > kLaneAttnGroup || rotary_dim % 64 != 0 || rotary_dim > head_dim)
        return QD_ERR_UNSUPPORTED;
    const uintptr_t align = (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q_scratch;
    if ((align & 15u) || (cache_stride & 7)) return QD_ERR_UNSUPPORTED;
    const int heads = q_heads + kv_heads;
    qd_launch(seq_attn_prepare_kernel, dim3((heads + 7) / 8, batch), dim3(256), 0, (cudaStream_t)stream, true, 
        (const bf16*)qg, (const bf16*)k_new, (const bf16*)v_new, (const bf16*)q_norm, (const bf16*)k_norm,
        (bf16*)k_cache, (bf16*)v_cache, (bf16*)q_scratch, 0, q_heads, kv_heads, head_dim, rotary_dim, theta, eps,
        positions, cache_stride, capacity);
    if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    LaneAttnParams p;
    p.q = (const bf16*)q_scratch; p.qg = (const bf16*)qg; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
    p.cache_stride = cache_stride; p.out = (bf16*)out; p.partial = scratch; p.counters = counters; p.positions = positions;
    p.hq = q_heads; p.hk = kv_heads; p.d = head_dim; p.splits = splits; p.capacity = capacity;
    const size_t smem = (size_t)G * head_dim * sizeof(bf16) + sizeof(float) * (kLaneAttnWarps * 32 * kLaneAttnGroup +
                                                                                (size_t)kLaneAttnWarps * G * (head_dim + 2));
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(batch_attn_lanes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    if (smem > 100 * 1024) return QD_ERR_UNSUPPORTED;
    if (head_dim == 256) {          // tensor-core form
        const size_t mma_smem = 8 * kAttnQRow + sizeof(float) * (size_t)kLaneAttnWarps * G * (head_dim + 2);
        static bool mma_configured[64];
        if (!mma_configured[dev]) {
            if (cudaFuncSetAttribute(batch_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
                return QD_ERR_LAUNCH;
            mma_configured[dev] = true;
        }
        qd_launch(batch_attn_mma_kernel, dim3(kv_heads, splits, batch), dim3(kLaneAttnWarps * 32), mma_smem, (cudaStream_t)stream, true, p);
        return qd_launch_status();
    }
    qd_launch(batch_attn_lanes_kernel, dim3(kv_heads, splits, batch), dim3(kLaneAttnWarps * 32), smem, (cudaStream_t)stream, true, p);
    return qd_launch_status();
}

extern "C" int qd_seq_route_topk(const void* logits, int tokens, int experts, int topk, int32_t* ids, float* weights,
                                 void* stream) {
    QD_CHECK_ARG(logits && ids && weights && tokens > 0 && topk >= 1 && topk <= 32 && topk <= experts);
    if (experts > 256) return QD_ERR_UNSUPPORTED;
    qd_launch(seq_route_kernel, dim3(tokens), dim3(32), 0, (cudaStream_t)stream, true, (const bf16*)logits, experts, topk, ids, weights);
    return qd_launch_status();
}

extern "C" int qd_seq_group_routes(const int32_t* ids, int routes, int experts, int32_t* order, int32_t* boundaries,
                                   void* stream) {
    QD_CHECK_ARG(ids && order && boundaries && routes > 0 && experts > 0);
    if (experts > 1023) return QD_ERR_UNSUPPORTED;
    // as many warps as 40 KB of counters allow (32 at 256 experts, 8 at 1023)
    int warps = 32;
    while (warps > 1 && (size_t)warps * experts * 4 > 40960) warps >>= 1;
    const size_t smem = ((size_t)warps * experts + experts + 1) * sizeof(int32_t);
    qd_launch(seq_group_routes_kernel, dim3(1), dim3(warps * 32), smem, (cudaStream_t)stream, true, ids, routes, experts, order, boundaries);
    return qd_launch_status();
}

extern "C" int qd_seq_moe_combine(const void* contributions, const int32_t* ids, const void* shared,
                                  const void* strength, void* out, int tokens, int hidden, int topk, void* stream) {
    QD_CHECK_ARG(contributions && ids && shared && strength && out && tokens > 0 && hidden > 0 && topk > 0);
    if (topk > 32) return QD_ERR_UNSUPPORTED;
    qd_launch(seq_combine_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, true, 
        (const bf16*)contributions, ids, (const bf16*)shared, (const bf16*)strength, (bf16*)out, hidden, topk);
    return qd_launch_status();
}

// qd_seq_moe_combine followed by qd_seq_add_rms_norm(x = its output, residual, gamma) in one launch: the
// end of a layer and the norm in front of the next one (quickdraw/models/qwen.py:189-194, 203-207).
// hidden a multiple of 8, at most 4096, 16-byte aligned rows; QD_ERR_UNSUPPORTED otherwise.
extern "C" int qd_seq_moe_combine_norm(const void* contributions, const int32_t* ids, const void* shared, const void* strength,
                                       const void* residual, const float* gamma, void* normed, void* residual_out,
                                       int tokens, int hidden, int topk, float eps, void* stream) {
    QD_CHECK_ARG(contributions && ids && shared && strength && residual && gamma && normed && residual_out);
    QD_CHECK_ARG(tokens > 0 && hidden > 0 && topk > 0);
    if (topk > 32 || hidden % 8 != 0 || hidden > 8 * 256 * kNormVecs) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)contributions | (uintptr_t)shared | (uintptr_t)residual | (uintptr_t)gamma | (uintptr_t)normed | (uintptr_t)residual_out) & 15u)
        return QD_ERR_UNSUPPORTED;
    qd_launch(seq_combine_norm_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, true,
              (const bf16*)contributions, ids, (const bf16*)shared, (const bf16*)strength, (const bf16*)residual, gamma,
              (bf16*)normed, (bf16*)residual_out, hidden, topk, eps);
    return qd_launch_status();
}

