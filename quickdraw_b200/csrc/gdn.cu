// Gated-DeltaNet decode step: short convolution, gated delta-rule recurrence and the
// per-head gated RMSNorm (reference: quickdraw/models/qwen.py:119-165,
// quickdraw/kernel/triton/delta.py:37-91).
#include "common.cuh"

// ------------------------------------------------------------------ short convolution
// One thread per channel.  window = [history | new]; every tap product is rounded to
// bf16, the sum is fp32, SiLU, bf16; the history shifts left by one.
__global__ void gdn_conv_kernel(const bf16* __restrict__ mixed, const bf16* __restrict__ taps,
                                bf16* __restrict__ state, bf16* __restrict__ out, int channels, int width) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    bf16* hist = state + (size_t)c * (width - 1);
    const bf16* w = taps + (size_t)c * width;
    const float fresh = ld_bf16(mixed + c);
    float acc = 0.f;
    for (int t = 0; t < width - 1; ++t) {
        const float h = ld_bf16(hist + t);
        acc += round_bf16(h * ld_bf16(w + t));
        if (t > 0) hist[t - 1] = __float2bfloat16_rn(h);
    }
    acc += round_bf16(fresh * ld_bf16(w + width - 1));
    if (width > 1) hist[width - 2] = __float2bfloat16_rn(fresh);
    out[c] = __float2bfloat16_rn(silu_precise(acc));
}

extern "C" int qd_gdn_conv(const void* mixed, const void* taps, void* conv_state, void* out,
                           int channels, int width, void* stream) {
    QD_CHECK_ARG(mixed && taps && out && channels > 0 && width >= 1 && (width == 1 || conv_state));
    gdn_conv_kernel<<<(channels + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        (const bf16*)mixed, (const bf16*)taps, (bf16*)conv_state, (bf16*)out, channels, width);
    return qd_launch_status();
}

// ------------------------------------------------------------------------- recurrence
// Block = (value head, slice of 32 value columns); 8 key groups x 32 columns = 256 threads.
// Thread (kg, col) keeps KPT = ceil(Dk/8) state entries S[kg*KPT + j][col] in registers:
//   S *= decay;  pred = S^T k;  corr = beta (v - pred);  S += k corr^T;  o = S^T q.
// The state tile is fetched before the dependency wait: it was last written by the
// previous token's step, never by the kernel that precedes this one in the stream.
constexpr int kGdnKeyGroups = 8;
constexpr int kGdnCols = 32;
constexpr int kGdnMaxKpt = 16;

__global__ void __launch_bounds__(kGdnKeyGroups* kGdnCols)
gdn_recurrence_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ b,
                      const bf16* __restrict__ a_log, const bf16* __restrict__ dt_bias,
                      float* __restrict__ state, bf16* __restrict__ out, int hk, int hv, int dk, int dv) {
    __shared__ float sq[kGdnMaxKpt * kGdnKeyGroups], sk[kGdnMaxKpt * kGdnKeyGroups];
    __shared__ float part[kGdnKeyGroups][kGdnCols];
    __shared__ float norms[2], gates[2];
    const int head = blockIdx.x, c0 = blockIdx.y * kGdnCols;
    const int tid = threadIdx.x, col = tid & 31, kg = tid >> 5;
    const int kpt = (dk + kGdnKeyGroups - 1) / kGdnKeyGroups;
    const int key_head = head / (hv / hk);
    const bool col_ok = c0 + col < dv;
    float* tile = state + (size_t)head * dk * dv + c0 + col;

    float s[kGdnMaxKpt];
#pragma unroll
    for (int j = 0; j < kGdnMaxKpt; ++j) {
        const int key = kg * kpt + j;
        s[j] = (j < kpt && key < dk && col_ok) ? tile[(size_t)key * dv] : 0.f;
    }
    grid_launch_dependents();
    grid_dependency_wait();

    // q, k of the key head: l2-normalise (eps inside the root), q also scaled by Dk^-1/2
    const bf16* qh = qkv + (size_t)key_head * dk;
    const bf16* kh = qkv + (size_t)hk * dk + (size_t)key_head * dk;
    float qq = 0.f, kk = 0.f;
    for (int i = tid; i < dk; i += blockDim.x) {
        const float qv = ld_bf16(qh + i), kv = ld_bf16(kh + i);
        sq[i] = qv; sk[i] = kv;
        qq += qv * qv; kk += kv * kv;
    }
    qq = warp_sum(qq); kk = warp_sum(kk);
    if (col == 0) { part[kg][0] = qq; part[kg][1] = kk; }
    __syncthreads();
    if (tid == 0) {
        float tq = 0.f, tk = 0.f;
        for (int w = 0; w < kGdnKeyGroups; ++w) { tq += part[w][0]; tk += part[w][1]; }
        norms[0] = rsqrtf(tq + 1e-6f);
        norms[1] = rsqrtf(tk + 1e-6f);
        const float alpha = ld_bf16(a + head) + ld_bf16(dt_bias + head);
        gates[0] = expf(-expf(ld_bf16(a_log + head)) * softplus_precise(alpha));   // decay
        gates[1] = sigmoid_precise(ld_bf16(b + head));                              // beta
    }
    __syncthreads();
    const float kscale = norms[1];
    const float decay = gates[0], beta = gates[1];
    const float v = col_ok ? ld_bf16(qkv + (size_t)2 * hk * dk + (size_t)head * dv + c0 + col) : 0.f;

    float pred = 0.f;
#pragma unroll
    for (int j = 0; j < kGdnMaxKpt; ++j) {
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
    for (int w = 0; w < kGdnKeyGroups; ++w) total += part[w][col];
    const float corr = beta * (v - total);
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < kGdnMaxKpt; ++j) {
        const int key = kg * kpt + j;
        if (j < kpt && key < dk) {
            s[j] += (sk[key] * kscale) * corr;
            o += s[j] * ((sq[key] * norms[0]) / sqrtf((float)dk));
            if (col_ok) tile[(size_t)key * dv] = s[j];
        }
    }
    part[kg][col] = o;
    __syncthreads();
    if (kg == 0 && col_ok) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kGdnKeyGroups; ++w) acc += part[w][col];
        out[(size_t)head * dv + c0 + col] = __float2bfloat16_rn(acc);
    }
}

extern "C" int qd_gdn_recurrence(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                 const void* dt_bias, float* rec_state, void* out, int key_heads,
                                 int value_heads, int key_dim, int value_dim, int pdl, void* stream) {
    QD_CHECK_ARG(conv_qkv && a && b && a_log && dt_bias && rec_state && out);
    QD_CHECK_ARG(key_heads > 0 && value_heads % key_heads == 0 && key_dim > 0 && value_dim > 0);
    if (key_dim > kGdnMaxKpt * kGdnKeyGroups) return QD_ERR_UNSUPPORTED;
    dim3 grid(value_heads, (value_dim + kGdnCols - 1) / kGdnCols);
    return qd_launch(gdn_recurrence_kernel, grid, dim3(kGdnKeyGroups * kGdnCols), 0, (cudaStream_t)stream,
                     pdl != 0, (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log,
                     (const bf16*)dt_bias, rec_state, (bf16*)out, key_heads, value_heads, key_dim, value_dim);
}

// ------------------------------------------------------------------------- gated norm
// gated = bf16( rms_norm(o)[head] * gamma * silu(z) ), one warp per head.
__global__ void gdn_gated_norm_kernel(const bf16* __restrict__ o, const bf16* __restrict__ z,
                                      const bf16* __restrict__ gamma, bf16* __restrict__ out, int heads,
                                      int dv, float eps) {
    chain_enter();
    const int head = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (head >= heads) return;
    if (dv == 128 && !(((uintptr_t)o | (uintptr_t)z | (uintptr_t)gamma | (uintptr_t)out) & 7u)) {
        // four values per lane, 8-byte accesses
        const size_t at = (size_t)head * dv + 4 * lane;
        const uint2 ov = *reinterpret_cast<const uint2*>(o + at), zv = *reinterpret_cast<const uint2*>(z + at);
        const uint2 gv = *reinterpret_cast<const uint2*>(gamma + 4 * lane);
        const float v[4] = {bf16_bits_to_float(ov.x & 0xffffu), bf16_bits_to_float(ov.x >> 16), bf16_bits_to_float(ov.y & 0xffffu), bf16_bits_to_float(ov.y >> 16)};
        const float zz[4] = {bf16_bits_to_float(zv.x & 0xffffu), bf16_bits_to_float(zv.x >> 16), bf16_bits_to_float(zv.y & 0xffffu), bf16_bits_to_float(zv.y >> 16)};
        const float gg[4] = {bf16_bits_to_float(gv.x & 0xffffu), bf16_bits_to_float(gv.x >> 16), bf16_bits_to_float(gv.y & 0xffffu), bf16_bits_to_float(gv.y >> 16)};
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)dv + eps);
        float r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = ((v[i] * inv) * gg[i]) * silu_precise(zz[i]);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
        *reinterpret_cast<uint2*>(out + at) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) { const float v = ld_bf16(o + (size_t)head * dv + i); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const size_t idx = (size_t)head * dv + i;
        out[idx] = __float2bfloat16_rn(((ld_bf16(o + idx) * inv) * ld_bf16(gamma + i)) * silu_precise(ld_bf16(z + idx)));
    }
}

extern "C" int qd_gdn_gated_norm(const void* o, const void* z, const void* gamma, void* out, int heads,
                                 int value_dim, float eps, void* stream) {
    QD_CHECK_ARG(o && z && gamma && out && heads > 0 && value_dim > 0);
    qd_launch(gdn_gated_norm_kernel, dim3((heads + 3) / 4), dim3(128), 0, (cudaStream_t)stream, true, 
        (const bf16*)o, (const bf16*)z, (const bf16*)gamma, (bf16*)out, heads, value_dim, eps);
    return qd_launch_status();
}
