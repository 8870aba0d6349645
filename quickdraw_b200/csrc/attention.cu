// Gated GQA decode attention over a contiguous bf16 KV cache, split along the context
// (reference: quickdraw/models/qwen.py:66-116, quickdraw/kernel/triton/attention.py:10-100).
//
// One kernel does the whole mixer core between the q/k/v projections and o_proj:
//   * per-head RMSNorm of q and k with gamma = 1 + weight, rounded to bf16;
//   * partial RoPE on the leading rotary_dim features (half-split pairing; cos/sin
//     rounded to bf16, rotation in fp32, result rounded to bf16);
//   * the new key/value row written into the cache at `position`;
//   * fp32 online softmax over [0, position], every KV head's rows read once for all
//     the query heads that share it; partial results of the context splits are merged
//     by the last block to finish;
//   * bf16(attended) * bf16(sigmoid(gate)).
// The position is a host integer or, for CUDA-graph replay, a device scalar.
#include "common.cuh"

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kAttnMaxGroup = 8;      // query heads per KV head
constexpr int kAttnMaxDim = 256;      // head_dim <= 256, multiple of 8
constexpr int kAttnSplitMin = 64;     // positions per split at least

struct AttnParams {
    const bf16* qg;        // [Hq, 2*D]  query | gate per head
    const bf16* k_new;     // [Hk, D] raw key projection
    const bf16* v_new;     // [Hk, D]
    const bf16* q_norm;    // [D]
    const bf16* k_norm;    // [D]
    bf16* k_cache;         // [capacity, Hk, D]
    bf16* v_cache;
    bf16* out;             // [Hq * D] gated attention output
    float* partial;        // [Hk, splits, G, D + 2] scratch
    unsigned int* counters;// [Hk], zero before the first launch; reset by the kernel
    const int* position_dev;
    unsigned int* status;  // optional status word (QD_STATUS_* bits)
    int position_host;
    int capacity;
    int hq, hk, d, rotary;
    float theta, eps;
    int splits;
    long long cache_stride;   // batched form only: elements between the caches of two sequences
};

// normalise + rotate one head held as D/32 (<= 8) strided features per lane: feature i = j*32 + lane.
QD_DEVINL void norm_rope_head(const bf16* __restrict__ src, const bf16* __restrict__ gamma_w, int d,
                              int rotary, float theta, float eps, int position, int lane,
                              float* __restrict__ dst_smem /* [d] */) {
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float v = ld_bf16(src + i); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32)
        dst_smem[i] = round_bf16((ld_bf16(src + i) * inv) * (1.0f + ld_bf16(gamma_w + i)));
    __syncwarp();
    const int half = rotary / 2;
    float rotated[kAttnMaxDim / 32];
    int n = 0;
    for (int i = lane; i < rotary; i += 32, ++n) {
        const int f = i % half;
        const float inv_freq = 1.0f / powf(theta, (float)(2 * f) / (float)rotary);
        const float angle = (float)position * inv_freq;
        const float c = round_bf16(cosf(angle)), s = round_bf16(sinf(angle));
        const float partner = i < half ? -dst_smem[i + half] : dst_smem[i - half];
        rotated[n] = round_bf16(dst_smem[i] * c + partner * s);
    }
    __syncwarp();
    n = 0;
    for (int i = lane; i < rotary; i += 32, ++n) dst_smem[i] = rotated[n];
    __syncwarp();
}

__global__ void __launch_bounds__(kAttnThreads)
attn_decode_kernel(const AttnParams p) {
    extern __shared__ float sm[];
    const int G = p.hq / p.hk, D = p.d;
    // batched form: grid z = sequence; every per-sequence array moves on by one sequence, the
    // position comes from the sequence's entry of the device array (z = 0: no offsets)
    const size_t z = blockIdx.z;
    const long long cache_offset = z ? (long long)z * p.cache_stride : 0;
    const bf16* const seq_qg = p.qg + z * (size_t)p.hq * 2 * D;
    const bf16* const seq_k_new = p.k_new + z * (size_t)p.hk * D;
    const bf16* const seq_v_new = p.v_new + z * (size_t)p.hk * D;
    bf16* const seq_k_cache = p.k_cache + cache_offset;
    bf16* const seq_v_cache = p.v_cache + cache_offset;
    bf16* const seq_out = p.out + z * (size_t)p.hq * D;
    float* const seq_partial = p.partial + z * (size_t)p.hk * p.splits * G * (D + 2);
    unsigned int* const seq_counters = p.counters + z * (size_t)p.hk;
    const int* const seq_position = p.position_dev ? p.position_dev + z : nullptr;
    float* q_s = sm;                              // [G][D] normalised, rotated, as fp32 of bf16
    float* k_s = q_s + G * D;                     // [D] new key
    float* red = k_s + D;                         // [warps][G][D + 2]
    __shared__ int s_last;
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    grid_launch_dependents();
    grid_dependency_wait();
    const int position = seq_position ? *seq_position : p.position_host;
    // A position outside the cache (possible only when it comes from the device scalar; host
    // values are checked before the launch) touches nothing: every block of the sequence
    // leaves, the output keeps its old contents and, where the caller gave one, the status
    // word says so.
    if (position < 0 || position >= p.capacity) {
        if (p.status && tid == 0) atomicOr(p.status, QD_STATUS_BAD_ARG);
        return;
    }
    const int T = position + 1;
    int active = (T + kAttnSplitMin - 1) / kAttnSplitMin;
    if (active > p.splits) active = p.splits;
    const int per = ((T + active - 1) / active + 7) & ~7;
    const int t0 = split * per;
    const int t1 = min(T, t0 + per);
    const bool mine = split < active && t0 < t1;

    if (mine) {
        for (int h = warp; h < G; h += kAttnWarps)
            norm_rope_head(seq_qg + (size_t)(kvh * G + h) * 2 * D, p.q_norm, D, p.rotary, p.theta, p.eps,
                           position, lane, q_s + h * D);
        const bool owns_new = position >= t0 && position < t1;
        if (owns_new && warp == kAttnWarps - 1) {
            norm_rope_head(seq_k_new + (size_t)kvh * D, p.k_norm, D, p.rotary, p.theta, p.eps, position, lane, k_s);
            bf16* krow = seq_k_cache + ((size_t)position * p.hk + kvh) * D;
            bf16* vrow = seq_v_cache + ((size_t)position * p.hk + kvh) * D;
            for (int i = lane; i < D; i += 32) {
                krow[i] = __float2bfloat16_rn(k_s[i]);
                vrow[i] = seq_v_new[(size_t)kvh * D + i];
            }
        }
    }
    __syncthreads();

    // per-warp online softmax over positions t0 + warp, t0 + warp + 8, ...
    // lane owns features [8*lane, 8*lane + 8) (D <= 256)
    const int f0 = lane * 8;
    const bool lane_on = f0 < D;
    float m[kAttnMaxGroup], l[kAttnMaxGroup], acc[kAttnMaxGroup][8];
#pragma unroll
    for (int h = 0; h < kAttnMaxGroup; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;
    }
    const float scale = rsqrtf((float)D);
    if (mine) {
        for (int t = t0 + warp; t < t1; t += kAttnWarps) {
            float kf[8], vf[8];
            if (lane_on) {
                if (t == position) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        kf[j] = k_s[f0 + j];
                        vf[j] = ld_bf16(seq_v_new + (size_t)kvh * D + f0 + j);
                    }
                } else {
                    const uint4 kr = *reinterpret_cast<const uint4*>(seq_k_cache + ((size_t)t * p.hk + kvh) * D + f0);
                    const uint4 vr = *reinterpret_cast<const uint4*>(seq_v_cache + ((size_t)t * p.hk + kvh) * D + f0);
                    const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        kf[2 * j] = __uint_as_float(kw[j] << 16); kf[2 * j + 1] = __uint_as_float(kw[j] & 0xffff0000u);
                        vf[2 * j] = __uint_as_float(vw[j] << 16); vf[2 * j + 1] = __uint_as_float(vw[j] & 0xffff0000u);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) { kf[j] = 0.f; vf[j] = 0.f; }
            }
#pragma unroll
            for (int h = 0; h < kAttnMaxGroup; ++h) {
                if (h < G) {
                    float dot = 0.f;
                    if (lane_on) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) dot += q_s[h * D + f0 + j] * kf[j];
                    }
                    const float sc = warp_sum(dot) * scale;
                    const float nm = fmaxf(m[h], sc);
                    const float fix = expf(m[h] - nm), pr = expf(sc - nm);
                    l[h] = l[h] * fix + pr;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[h][j] = acc[h][j] * fix + pr * vf[j];
                    m[h] = nm;
                }
            }
        }
    }
    // merge the warps of this block
    const int stride = D + 2;
#pragma unroll
    for (int h = 0; h < kAttnMaxGroup; ++h) {
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
    float* block_out = seq_partial + (((size_t)kvh * p.splits + split) * G) * stride;
    for (int idx = tid; idx < G * D; idx += kAttnThreads) {
        const int h = idx / D, f = idx % D;
        float mm = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, red[((size_t)w * G + h) * stride + D]);
        float num = 0.f, den = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) {
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
    if (tid == 0) {
        const unsigned int done = atomicAdd(seq_counters + kvh, 1u);
        s_last = done == (unsigned int)p.splits - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last block of this KV head: merge the splits, normalise, gate
    for (int idx = tid; idx < G * D; idx += kAttnThreads) {
        const int h = idx / D, f = idx % D;
        float mm = -INFINITY;
        for (int s = 0; s < active; ++s)
            mm = fmaxf(mm, __ldcg(seq_partial + (((size_t)kvh * p.splits + s) * G + h) * stride + D));
        float num = 0.f, den = 0.f;
        for (int s = 0; s < active; ++s) {
            const float* src = seq_partial + (((size_t)kvh * p.splits + s) * G + h) * stride;
            const float sm_ = __ldcg(src + D);
            const float wgt = sm_ == -INFINITY ? 0.f : expf(sm_ - mm);
            num += wgt * __ldcg(src + f);
            den += wgt * __ldcg(src + D + 1);
        }
        const float attended = round_bf16(num / den);
        const int qh = kvh * G + h;
        const float gate = round_bf16(sigmoid_precise(ld_bf16(seq_qg + (size_t)qh * 2 * D + D + f)));
        seq_out[(size_t)qh * D + f] = __float2bfloat16_rn(attended * gate);
    }
    if (tid == 0) seq_counters[kvh] = 0;
}

extern "C" int qd_attn_scratch_floats(int q_heads, int kv_heads, int head_dim, int splits) {
    return kv_heads * splits * (q_heads / kv_heads) * (head_dim + 2);
}

extern "C" int qd_attn_decode(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                              const void* k_norm, void* k_cache, void* v_cache, void* out, float* scratch,
                              unsigned int* counters, const int* position_dev, int position_host,
                              int capacity, int q_heads, int kv_heads, int head_dim, int rotary_dim,
                              float theta, float eps, int splits, int pdl, void* stream) {
    QD_CHECK_ARG(qg && k_new && v_new && q_norm && k_norm && k_cache && v_cache && out && scratch && counters);
    QD_CHECK_ARG(kv_heads > 0 && q_heads % kv_heads == 0 && splits >= 1 && capacity > 0);
    QD_CHECK_ARG(position_dev || (position_host >= 0 && position_host < capacity));
    QD_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0);
    const int G = q_heads / kv_heads;
    if (G > kAttnMaxGroup || head_dim > kAttnMaxDim || head_dim % 8 != 0) return QD_ERR_UNSUPPORTED;
    AttnParams p = {};
    p.qg = (const bf16*)qg; p.k_new = (const bf16*)k_new; p.v_new = (const bf16*)v_new;
    p.q_norm = (const bf16*)q_norm; p.k_norm = (const bf16*)k_norm;
    p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.out = (bf16*)out;
    p.partial = scratch; p.counters = counters; p.position_dev = position_dev; p.position_host = position_host;
    p.capacity = capacity; p.hq = q_heads; p.hk = kv_heads; p.d = head_dim; p.rotary = rotary_dim;
    p.theta = theta; p.eps = eps; p.splits = splits; p.cache_stride = 0;
    const size_t smem = sizeof(float) * ((size_t)G * head_dim + head_dim + (size_t)kAttnWarps * G * (head_dim + 2));
    if (smem > 100 * 1024) return QD_ERR_UNSUPPORTED;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    return qd_launch(attn_decode_kernel, dim3(kv_heads, splits), dim3(kAttnThreads), smem, (cudaStream_t)stream,
                     pdl != 0, p);
}

// ------------------------------------------------------------------------- batched form
// One decode step of `batch` independent sequences, each with its own cache and position
// (per-sequence state of small-batch decode): the single-sequence kernel with the sequence as
// grid z.  qg / k_new / v_new / out hold one row set per sequence, the caches of sequence b
// start cache_stride elements after those of sequence b - 1, positions is a device array,
// scratch holds batch * qd_attn_scratch_floats() floats, counters batch * kv_heads zeros.
extern "C" int qd_batch_attn_decode(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                                    const void* k_norm, void* k_cache, void* v_cache, long long cache_stride,
                                    void* out, float* scratch, unsigned int* counters, const int* positions,
                                    int batch, int capacity, int q_heads, int kv_heads, int head_dim,
                                    int rotary_dim, float theta, float eps, int splits, void* stream) {
    QD_CHECK_ARG(qg && k_new && v_new && q_norm && k_norm && k_cache && v_cache && out && scratch && counters && positions);
    QD_CHECK_ARG(batch > 0 && batch <= 65535 && kv_heads > 0 && q_heads % kv_heads == 0 && splits >= 1 && capacity > 0);
    QD_CHECK_ARG(cache_stride >= (long long)capacity * kv_heads * head_dim || batch == 1);
    QD_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0);
    const int G = q_heads / kv_heads;
    if (G > kAttnMaxGroup || head_dim > kAttnMaxDim || head_dim % 8 != 0) return QD_ERR_UNSUPPORTED;
    AttnParams p = {};
    p.qg = (const bf16*)qg; p.k_new = (const bf16*)k_new; p.v_new = (const bf16*)v_new;
    p.q_norm = (const bf16*)q_norm; p.k_norm = (const bf16*)k_norm;
    p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.out = (bf16*)out;
    p.partial = scratch; p.counters = counters; p.position_dev = positions; p.position_host = 0;
    p.capacity = capacity; p.hq = q_heads; p.hk = kv_heads; p.d = head_dim; p.rotary = rotary_dim;
    p.theta = theta; p.eps = eps; p.splits = splits; p.cache_stride = cache_stride;
    const size_t smem = sizeof(float) * ((size_t)G * head_dim + head_dim + (size_t)kAttnWarps * G * (head_dim + 2));
    if (smem > 100 * 1024) return QD_ERR_UNSUPPORTED;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    return qd_launch(attn_decode_kernel, dim3(kv_heads, splits, batch), dim3(kAttnThreads), smem, (cudaStream_t)stream,
                     false, p);
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for callers that cannot allocate device memory (see qd_attn_decode_static in the
// header).  One array per GPU that loads the library, held until the process exits: the
// split partials first, the per-KV-head completion counters in the last 256 bytes.
constexpr size_t kAttnStaticBytes = 1u << 20;
constexpr size_t kAttnStaticCounterBytes = 256;
static __device__ __align__(256) unsigned char qd_attn_static_scratch[kAttnStaticBytes];
static unsigned char* g_attn_static_ptr[64];     // device address of the array, per device ordinal

extern "C" int qd_attn_decode_static(const void* qg, const void* k_new, const void* v_new, const void* q_norm,
                                     const void* k_norm, void* k_cache, void* v_cache, void* out,
                                     const int* position_dev, int position_host, int capacity, int q_heads,
                                     int kv_heads, int head_dim, int rotary_dim, float theta, float eps,
                                     int splits, void* stream) {
    QD_CHECK_ARG(qg && k_new && v_new && q_norm && k_norm && k_cache && v_cache && out);
    QD_CHECK_ARG(kv_heads > 0 && q_heads % kv_heads == 0 && splits >= 1 && capacity > 0);
    QD_CHECK_ARG(position_dev || (position_host >= 0 && position_host < capacity));
    QD_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0);
    const int G = q_heads / kv_heads;
    if (G > kAttnMaxGroup || head_dim > kAttnMaxDim || head_dim % 8 != 0) return QD_ERR_UNSUPPORTED;
    const size_t need = sizeof(float) * (size_t)qd_attn_scratch_floats(q_heads, kv_heads, head_dim, splits);
    if (need > kAttnStaticBytes - kAttnStaticCounterBytes || (size_t)kv_heads * 4 > kAttnStaticCounterBytes)
        return QD_ERR_TOO_LARGE;      // the static array cannot hold this shape
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    if (!g_attn_static_ptr[dev]) {
        // The array's name is a host-side handle; the kernel needs its address on THIS device.
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, qd_attn_static_scratch) != cudaSuccess || !address) return QD_ERR_LAUNCH;
        g_attn_static_ptr[dev] = (unsigned char*)address;
    }
    unsigned char* base = g_attn_static_ptr[dev];
    unsigned int* counters = (unsigned int*)(base + kAttnStaticBytes - kAttnStaticCounterBytes);
    // The array keeps whatever the last call left; the counters must start at zero.
    if (cudaMemsetAsync(counters, 0, kAttnStaticCounterBytes, (cudaStream_t)stream) != cudaSuccess) return QD_ERR_LAUNCH;
    AttnParams p = {};
    p.qg = (const bf16*)qg; p.k_new = (const bf16*)k_new; p.v_new = (const bf16*)v_new;
    p.q_norm = (const bf16*)q_norm; p.k_norm = (const bf16*)k_norm;
    p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.out = (bf16*)out;
    p.partial = (float*)base; p.counters = counters; p.position_dev = position_dev; p.position_host = position_host;
    p.capacity = capacity; p.hq = q_heads; p.hk = kv_heads; p.d = head_dim; p.rotary = rotary_dim;
    p.theta = theta; p.eps = eps; p.splits = splits; p.cache_stride = 0;
    const size_t smem = sizeof(float) * ((size_t)G * head_dim + head_dim + (size_t)kAttnWarps * G * (head_dim + 2));
    if (smem > 100 * 1024) return QD_ERR_UNSUPPORTED;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    return qd_launch(attn_decode_kernel, dim3(kv_heads, splits), dim3(kAttnThreads), smem, (cudaStream_t)stream,
                     false, p);
}
