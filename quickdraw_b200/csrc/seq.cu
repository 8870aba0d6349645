// Sequence forms of the per-token operators, for a chunk of prompt tokens (prefill).  The dense
// projections of a chunk run on the tensor cores (gemm.cu); everything here is the glue between
// them, with the arithmetic of the single-token kernels applied row by row (same rounding
// points): residual add + RMSNorm, small bf16 projections, the DeltaNet short convolution and
// recurrence walked along the chunk, attention preparation (q/k norm, RoPE, cache write) and
// causal attention over cache + chunk, routing and the MoE combine.
// Reference: the 2-D branches of quickdraw/kernel/triton/{delta,attention,moe,norm}.py and
// quickdraw/models/qwen.py:66-241.
#include "rowdot.cuh"

namespace {

// ------------------------------------------------------------------ residual add + RMSNorm
__global__ void seq_add_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                                    const float* __restrict__ gamma, bf16* __restrict__ normed,
                                    bf16* __restrict__ residual_out, int width, float eps) {
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

// --------------------------------------------------- small bf16 projection of every token
// y[t, n] = bf16( sum_k x[t, k] w[n, k] ): one warp per (token, output row).
__global__ void seq_bf16_matmul_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                                       int rows, int width) {
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    if (n >= rows) return;
    const bf16* row = w + (size_t)n * width;
    const bf16* xt = x + (size_t)t * width;
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) acc += ld_bf16(row + i) * ld_bf16(xt + i);
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)t * rows + n] = __float2bfloat16_rn(acc);
}

// ------------------------------------------------------------- DeltaNet short convolution
// One thread per channel walks the chunk: window = [history | new], tap products rounded to
// bf16, fp32 sum, SiLU, bf16; the history ends up holding the last width - 1 inputs.
__global__ void seq_conv_kernel(const bf16* __restrict__ mixed, const bf16* __restrict__ taps, bf16* __restrict__ state,
                                bf16* __restrict__ out, int tokens, int channels, int width) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float hist[8], w[8];
    for (int t = 0; t < width - 1; ++t) hist[t] = ld_bf16(state + (size_t)c * (width - 1) + t);
    for (int t = 0; t < width; ++t) w[t] = ld_bf16(taps + (size_t)c * width + t);
    for (int t = 0; t < tokens; ++t) {
        const float fresh = ld_bf16(mixed + (size_t)t * channels + c);
        float acc = 0.f;
        for (int k = 0; k < width - 1; ++k) acc += round_bf16(hist[k] * w[k]);
        acc += round_bf16(fresh * w[width - 1]);
        for (int k = 0; k + 1 < width - 1; ++k) hist[k] = hist[k + 1];
        if (width > 1) hist[width - 2] = fresh;
        out[(size_t)t * channels + c] = __float2bfloat16_rn(silu_precise(acc));
    }
    for (int t = 0; t < width - 1; ++t) state[(size_t)c * (width - 1) + t] = __float2bfloat16_rn(hist[t]);
}

// ------------------------------------------------------------------- DeltaNet recurrence
// The single-token kernel (block = value head x 32 columns, 8 key groups x 32 columns, 16 state
// entries per thread) in a loop over the chunk; the state stays in registers in between.
__global__ void __launch_bounds__(256)
seq_recurrence_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ b,
                      const bf16* __restrict__ a_log, const bf16* __restrict__ dt_bias, float* __restrict__ state,
                      bf16* __restrict__ out, int tokens, int hk, int hv, int dk, int dv) {
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
                                        int hk, int d, int rotary, float theta, float eps) {
    const int t = blockIdx.y, head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= hq + hk) return;
    const int position = position0 + t;
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

// ----------------------------------------------------------------------------- routing
__global__ void seq_route_kernel(const bf16* __restrict__ logits, int experts, int topk, int32_t* __restrict__ ids,
                                 float* __restrict__ weights) {
    const int t = blockIdx.x;
    qd::route_small(logits + (size_t)t * experts, experts, topk, ids + (size_t)t * topk, weights + (size_t)t * topk,
                    threadIdx.x);
}

// --------------------------------------------------------------------------- MoE combine
// out[t] = bf16( bf16(sum of the token's routed rows in ascending expert id) +
//                bf16(shared[t] * bf16(sigmoid(strength[t]))) )
__global__ void seq_combine_kernel(const bf16* __restrict__ contributions, const int32_t* __restrict__ ids,
                                   const bf16* __restrict__ shared, const bf16* __restrict__ strength,
                                   bf16* __restrict__ out, int hidden, int topk) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= hidden) return;
    const int32_t* my = ids + (size_t)t * topk;
    const bf16* rows = contributions + (size_t)t * topk * hidden;
    float routed = 0.f;
    int last = -1;
    for (int n = 0; n < topk; ++n) {
        int pick = -1, pick_id = 0x7fffffff;
        for (int s = 0; s < topk; ++s) {
            const int e = my[s];
            if (e > last && e < pick_id) { pick = s; pick_id = e; }
        }
        if (pick < 0) break;
        last = pick_id;
        routed += ld_bf16(rows + (size_t)pick * hidden + i);
    }
    const float gate = round_bf16(sigmoid_precise(ld_bf16(strength + t)));
    const float gated = round_bf16(ld_bf16(shared + (size_t)t * hidden + i) * gate);
    out[(size_t)t * hidden + i] = __float2bfloat16_rn(round_bf16(routed) + gated);
}

}  // namespace

extern "C" int qd_seq_add_rms_norm(const void* x, const void* residual, const float* gamma, void* normed,
                                   void* residual_out, int tokens, int width, float eps, void* stream) {
    QD_CHECK_ARG(x && gamma && normed && residual_out && tokens > 0 && width > 0);
    seq_add_norm_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)residual, gamma,
                                                                  (bf16*)normed, (bf16*)residual_out, width, eps);
    return qd_launch_status();
}

extern "C" int qd_seq_bf16_matmul(const void* x, const void* w, void* y, int tokens, int rows, int width, void* stream) {
    QD_CHECK_ARG(x && w && y && tokens > 0 && rows > 0 && width > 0);
    seq_bf16_matmul_kernel<<<dim3((rows + 7) / 8, tokens), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, (const bf16*)w, (bf16*)y, rows, width);
    return qd_launch_status();
}

extern "C" int qd_seq_gdn_conv(const void* mixed, const void* taps, void* conv_state, void* out, int tokens,
                               int channels, int width, void* stream) {
    QD_CHECK_ARG(mixed && taps && out && tokens > 0 && channels > 0 && width >= 1 && width <= 8 && (width == 1 || conv_state));
    seq_conv_kernel<<<(channels + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        (const bf16*)mixed, (const bf16*)taps, (bf16*)conv_state, (bf16*)out, tokens, channels, width);
    return qd_launch_status();
}

extern "C" int qd_seq_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                     const void* dt_bias, float* rec_state, void* out, int tokens, int key_heads,
                                     int value_heads, int key_dim, int value_dim, void* stream) {
    QD_CHECK_ARG(conv_qkv && a && b && a_log && dt_bias && rec_state && out && tokens > 0);
    QD_CHECK_ARG(key_heads > 0 && value_heads % key_heads == 0 && key_dim > 0 && value_dim > 0);
    if (key_dim > 128) return QD_ERR_UNSUPPORTED;
    seq_recurrence_kernel<<<dim3(value_heads, (value_dim + 31) / 32), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log, (const bf16*)dt_bias, rec_state,
        (bf16*)out, tokens, key_heads, value_heads, key_dim, value_dim);
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
    seq_attn_prepare_kernel<<<dim3((heads + 7) / 8, tokens), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)qg, (const bf16*)k_new, (const bf16*)v_new, (const bf16*)q_norm, (const bf16*)k_norm,
        (bf16*)k_cache, (bf16*)v_cache, (bf16*)q_scratch, position0, q_heads, kv_heads, head_dim, rotary_dim, theta, eps);
    if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    seq_attn_kernel<<<dim3(kv_heads, tokens), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)q_scratch, (const bf16*)qg, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, position0,
        q_heads, kv_heads, head_dim);
    return qd_launch_status();
}

extern "C" int qd_seq_route_topk(const void* logits, int tokens, int experts, int topk, int32_t* ids, float* weights,
                                 void* stream) {
    QD_CHECK_ARG(logits && ids && weights && tokens > 0 && topk >= 1 && topk <= 32 && topk <= experts);
    if (experts > 256) return QD_ERR_UNSUPPORTED;
    seq_route_kernel<<<tokens, 32, 0, (cudaStream_t)stream>>>((const bf16*)logits, experts, topk, ids, weights);
    return qd_launch_status();
}

extern "C" int qd_seq_moe_combine(const void* contributions, const int32_t* ids, const void* shared,
                                  const void* strength, void* out, int tokens, int hidden, int topk, void* stream) {
    QD_CHECK_ARG(contributions && ids && shared && strength && out && tokens > 0 && hidden > 0 && topk > 0);
    seq_combine_kernel<<<dim3((hidden + 255) / 256, tokens), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)contributions, ids, (const bf16*)shared, (const bf16*)strength, (bf16*)out, hidden, topk);
    return qd_launch_status();
}
