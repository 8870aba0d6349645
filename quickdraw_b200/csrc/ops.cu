// Shape-generic operators of the six-name kernel table: they accept every shape the
// reference accepts (row tails, group sizes down to 2, tiny heads) and define the
// arithmetic contract; the streaming kernels in stream.cu take over for the aligned
// shapes of the real model.
#include "stream.cuh"

// ------------------------------------------------------------------------- rms_norm
// reference: quickdraw/models/qwen.py:19-22, quickdraw/kernel/triton/norm.py:8-23
template <typename T>
__global__ void rms_norm_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                T* __restrict__ out, int width, float eps) {
    __shared__ float partial[32];
    const T* row = x + (size_t)blockIdx.x * width;
    T* dst = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = (float)row[i];
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += partial[w];
    const float inv = rsqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        dst[i] = (T)(((float)row[i] * inv) * gamma[i]);
}

extern "C" int qd_rms_norm(const void* x, const float* gamma, void* out, int rows, int width,
                           float eps, int is_fp32, void* stream) {
    QD_CHECK_ARG(x && gamma && out && rows >= 0 && width > 0);
    if (rows == 0) return QD_OK;
    const int threads = width >= 1024 ? 256 : 128;
    if (is_fp32)
        rms_norm_kernel<float><<<rows, threads, 0, (cudaStream_t)stream>>>(
            (const float*)x, gamma, (float*)out, width, eps);
    else
        rms_norm_kernel<bf16><<<rows, threads, 0, (cudaStream_t)stream>>>(
            (const bf16*)x, gamma, (bf16*)out, width, eps);
    return qd_launch_status();
}

// Fused residual update of the step (quickdraw/models/qwen.py:214-217): total = x + r in
// fp32, normed = bf16(rms_norm(total) * gamma), residual = bf16(total).
__global__ void add_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                                const float* __restrict__ gamma, bf16* __restrict__ normed,
                                bf16* __restrict__ residual_out, int width, float eps) {
    __shared__ float partial[32];
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ld_bf16(x + i) + (residual ? ld_bf16(residual + i) : 0.f);
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += partial[w];
    const float inv = rsqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = ld_bf16(x + i) + (residual ? ld_bf16(residual + i) : 0.f);
        normed[i] = __float2bfloat16_rn((v * inv) * gamma[i]);
        residual_out[i] = __float2bfloat16_rn(v);
    }
}

extern "C" int qd_add_rms_norm(const void* x, const void* residual, const float* gamma,
                               void* normed, void* residual_out, int width, float eps,
                               void* stream) {
    QD_CHECK_ARG(x && gamma && normed && residual_out && width > 0);
    QD_CHECK_ARG(residual_out != residual && residual_out != x);
    add_norm_kernel<<<1, 512, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, (const bf16*)residual, gamma, (bf16*)normed, (bf16*)residual_out, width, eps);
    return qd_launch_status();
}

// ------------------------------------------------------------------- NVFP4 matvec
// One warp per (row, slot).  reference arithmetic: quickdraw/models/qwen.py:36-54;
// bank / per-slot / routed / fused-up switches: quickdraw/kernel/cute/matvec.py:26-79.

QD_DEVINL float fp4_row_dot(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                            const bf16* __restrict__ x, int half_k, int group, int lane) {
    float acc = 0.f;
    for (int j = lane; j < half_k; j += 32) {
        const uint32_t byte = codes[j];
        const float s = e4m3_to_float(scales[(2 * j) / group]);
        const float even = e2m1_to_float(byte & 15u) * s;
        const float odd = e2m1_to_float(byte >> 4) * s;
        acc += even * ld_bf16(x + 2 * j) + odd * ld_bf16(x + 2 * j + 1);
    }
    return warp_sum(acc);
}

__global__ void nvfp4_generic_kernel(const Fp4Args a) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.y;
    if (warp >= a.rows) return;
    const int expert = a.ids ? a.ids[slot] : 0;
    const int half_k = a.in_features / 2;
    const int groups = a.in_features / a.group;
    const size_t row = (size_t)expert * a.rows + warp;
    const bf16* x = a.x + (a.per_slot_input ? (size_t)slot * a.in_features : 0);
    const float acc = fp4_row_dot(a.codes + row * half_k, a.scales + row * groups, x, half_k, a.group, lane);
    float g = a.global[a.global_per_expert ? expert : 0];
    float result;
    if (a.up_codes) {
        const float acc_up = fp4_row_dot(a.up_codes + row * half_k, a.up_scales + row * groups, x,
                                         half_k, a.group, lane);
        const float gate = round_bf16(acc * g);
        const float up = round_bf16(acc_up * a.up_global[a.global_per_expert ? expert : 0]);
        result = round_bf16(silu_precise(gate)) * up;
    } else if (a.routing) {
        g = round_bf16(g * a.routing[slot]);
        result = round_bf16(acc) * g;
    } else {
        result = acc * g;
    }
    if (lane == 0) a.y[(size_t)slot * a.rows + warp] = __float2bfloat16_rn(result);
}

int qd_stream_matvec_try(const Fp4Args& a, cudaStream_t stream);  // stream.cu; QD_ERR_UNSUPPORTED if not covered
int qd_umma_matvec_try(const Fp4Args& a, cudaStream_t stream);    // umma.cu; QD_ERR_UNSUPPORTED if not covered

static int nvfp4_dispatch(const Fp4Args& a, cudaStream_t stream, int force_generic) {
    QD_CHECK_ARG(a.x && a.codes && a.scales && a.global && a.y);
    QD_CHECK_ARG(a.rows >= 0 && a.in_features > 0 && a.group >= 2 && a.group % 2 == 0);
    QD_CHECK_ARG(a.in_features % a.group == 0 && a.slots >= 1);
    QD_CHECK_ARG(!(a.up_codes && a.routing));
    QD_CHECK_ARG(!a.up_codes || (a.up_scales && a.up_global));
    QD_CHECK_ARG(a.ids || (a.slots == 1 && !a.global_per_expert));
    if (a.rows == 0) return QD_OK;
    // 0: the fastest kernel that covers the shape (FP4 tensor core, then the streaming kernel);
    // 2: the streaming kernel (cross-check); any other value: the shape-generic kernel
    if (force_generic == 0) {
        const int rc = qd_umma_matvec_try(a, stream);
        if (rc != QD_ERR_UNSUPPORTED) return rc;
    }
    if (force_generic == 0 || force_generic == 2) {
        const int rc = qd_stream_matvec_try(a, stream);
        if (rc != QD_ERR_UNSUPPORTED) return rc;
    }
    const int warps_per_block = 8;
    dim3 grid((a.rows + warps_per_block - 1) / warps_per_block, a.slots);
    nvfp4_generic_kernel<<<grid, warps_per_block * 32, 0, stream>>>(a);
    return qd_launch_status();
}

extern "C" int qd_nvfp4_gemv(const void* x, const void* codes, const void* scales, const float* global,
                             const float* routing_weight, void* y, int rows, int in_features,
                             int group_size, int force_generic, void* stream) {
    Fp4Args a = {};
    a.x = (const bf16*)x; a.codes = (const uint8_t*)codes; a.scales = (const uint8_t*)scales;
    a.global = global; a.routing = routing_weight; a.y = (bf16*)y;
    a.rows = rows; a.in_features = in_features; a.group = group_size; a.slots = 1;
    return nvfp4_dispatch(a, (cudaStream_t)stream, force_generic);
}

extern "C" int qd_nvfp4_expert_gemv(const void* x, const void* codes, const void* scales,
                                    const float* global, const int32_t* ids, const float* routing,
                                    void* y, int rows, int in_features, int group_size, int slots,
                                    int per_slot_input, int global_per_expert, int force_generic,
                                    void* stream) {
    QD_CHECK_ARG(ids);
    Fp4Args a = {};
    a.x = (const bf16*)x; a.codes = (const uint8_t*)codes; a.scales = (const uint8_t*)scales;
    a.global = global; a.ids = ids; a.routing = routing; a.y = (bf16*)y;
    a.rows = rows; a.in_features = in_features; a.group = group_size; a.slots = slots;
    a.per_slot_input = per_slot_input; a.global_per_expert = global_per_expert;
    return nvfp4_dispatch(a, (cudaStream_t)stream, force_generic);
}

extern "C" int qd_nvfp4_gate_up(const void* x, const void* gate_codes, const void* gate_scales,
                                const float* gate_global, const void* up_codes, const void* up_scales,
                                const float* up_global, const int32_t* ids, void* y, int rows,
                                int in_features, int group_size, int slots, int global_per_expert,
                                int force_generic, void* stream) {
    QD_CHECK_ARG(up_codes);
    Fp4Args a = {};
    a.x = (const bf16*)x; a.codes = (const uint8_t*)gate_codes; a.scales = (const uint8_t*)gate_scales;
    a.global = gate_global; a.up_codes = (const uint8_t*)up_codes; a.up_scales = (const uint8_t*)up_scales;
    a.up_global = up_global; a.ids = ids; a.y = (bf16*)y;
    a.rows = rows; a.in_features = in_features; a.group = group_size; a.slots = slots;
    a.global_per_expert = global_per_expert;
    return nvfp4_dispatch(a, (cudaStream_t)stream, force_generic);
}

// Dequantise to fp32 (no bf16 cast): the bit-exactness probe for codes and block scales
// (quickdraw/models/weights.py:21-26,46-55).
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                     float global, float* __restrict__ out, size_t pairs, int in_features,
                                     int group, int fast) {
    const size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= pairs) return;
    const size_t row = j / (in_features / 2);
    const int col = (int)(j % (in_features / 2)) * 2;
    const float s = e4m3_to_float(scales[row * (in_features / group) + col / group]);
    const uint32_t byte = codes[j];
    float lo, hi;
    if (fast) {   // the hardware convert used by the streaming kernels
        const uint32_t h2 = e2m1x2_to_f16x2(byte);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        lo = f.x; hi = f.y;
    } else {
        lo = e2m1_to_float(byte & 15u); hi = e2m1_to_float(byte >> 4);
    }
    out[2 * j] = lo * s * global;
    out[2 * j + 1] = hi * s * global;
}

extern "C" int qd_nvfp4_dequantize(const void* codes, const void* scales, float global, float* out,
                                   long long rows, int in_features, int group_size, int hardware_convert,
                                   void* stream) {
    QD_CHECK_ARG(codes && scales && out && rows >= 0 && in_features > 0 && in_features % group_size == 0);
    const size_t pairs = (size_t)rows * (in_features / 2);
    if (pairs == 0) return QD_OK;
    nvfp4_dequant_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)codes, (const uint8_t*)scales, global, out, pairs, in_features, group_size,
        hardware_convert);
    return qd_launch_status();
}

// ------------------------------------------------------------------------ bf16 gemv
// y = bf16(W x) with fp32 accumulation; router, shared-expert gate, DeltaNet a/b and the
// bf16 LM head of the synthetic model (quickdraw/models/qwen.py:129-130,173,192).
__global__ void bf16_gemv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                 bf16* __restrict__ y, int rows, int width) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const bf16* row = w + (size_t)warp * width;
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) acc += ld_bf16(row + i) * ld_bf16(x + i);
    acc = warp_sum(acc);
    if (lane == 0) y[warp] = __float2bfloat16_rn(acc);
}

extern "C" int qd_bf16_gemv(const void* x, const void* w, void* y, int rows, int width, void* stream) {
    QD_CHECK_ARG(x && w && y && rows >= 0 && width > 0);
    if (rows == 0) return QD_OK;
    bf16_gemv_kernel<<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, (const bf16*)w, (bf16*)y, rows, width);
    return qd_launch_status();
}

// ------------------------------------------------------------------------- fp8 gemv
// Static-FP8 projection: q = e4m3(clamp(x / s_in, +-448)), y = sum (w * s_w) * (q * s_in)
// (quickdraw/models/qwen.py:25-33, quickdraw/kernel/triton/matvec.py:48-62).
template <typename T>
__global__ void fp8_gemv_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w,
                                const float* __restrict__ w_scale, const float* __restrict__ in_scale,
                                T* __restrict__ y, int rows, int width) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const float s_in = *in_scale, s_w = *w_scale;
    const uint8_t* row = w + (size_t)warp * width;
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) {
        const float scaled = fminf(fmaxf(__fdiv_rn((float)x[i], s_in), -448.f), 448.f);
        const uint8_t q = __nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3);
        acc += (e4m3_to_float(row[i]) * s_w) * (e4m3_to_float(q) * s_in);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[warp] = (T)acc;
}

extern "C" int qd_fp8_gemv(const void* x, const void* w, const float* w_scale, const float* in_scale,
                           void* y, int rows, int width, int is_fp32, void* stream) {
    QD_CHECK_ARG(x && w && w_scale && in_scale && y && rows >= 0 && width > 0);
    if (rows == 0) return QD_OK;
    if (is_fp32)
        fp8_gemv_kernel<float><<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
            (const float*)x, (const uint8_t*)w, w_scale, in_scale, (float*)y, rows, width);
    else
        fp8_gemv_kernel<bf16><<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
            (const bf16*)x, (const uint8_t*)w, w_scale, in_scale, (bf16*)y, rows, width);
    return qd_launch_status();
}

// --------------------------------------------------------------------------- routing
// fp32 softmax over E logits, top-k by repeated maximum with the lowest index winning
// ties, weights renormalised over the selection (quickdraw/models/qwen.py:174-177,
// quickdraw/kernel/triton/moe.py:11-30).  One warp; E <= 1024.
QD_DEVINL void route_warp(const bf16* __restrict__ logits_bf16, const float* __restrict__ logits_f32,
                          int experts, int topk, int32_t* ids, float* weights, int lane) {
    constexpr int PER = 32;
    float p[PER];
    float best = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        float v = -INFINITY;
        if (e < experts) v = logits_bf16 ? ld_bf16(logits_bf16 + e) : logits_f32[e];
        p[i] = v;
        best = fmaxf(best, v);
    }
    best = warp_max(best);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        p[i] = e < experts ? expf(p[i] - best) : -1.f;   // -1 marks "not a candidate"
        if (e < experts) sum += p[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < PER; ++i) if (p[i] >= 0.f) p[i] = p[i] / sum;
    float chosen_sum = 0.f;
    float my_weight = 0.f;   // lane s keeps the weight of selection s (topk <= 32)
    int my_id = 0;
    for (int s = 0; s < topk; ++s) {
        float v = -1.f; int idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (p[i] > v) { v = p[i]; idx = i * 32 + lane; }   // ascending index within the lane
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        chosen_sum += v;
        if (lane == (s & 31)) { my_weight = v; my_id = idx; }
        if ((idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PER; ++i) if (i == (idx >> 5)) p[i] = -1.f;
        }
    }
    if (lane < topk) { ids[lane] = my_id; weights[lane] = my_weight / chosen_sum; }
}

__global__ void route_kernel(const bf16* logits_bf16, const float* logits_f32, int experts, int topk,
                             int32_t* ids, float* weights) {
    route_warp(logits_bf16, logits_f32, experts, topk, ids, weights, threadIdx.x);
}

extern "C" int qd_route_topk(const void* logits, int logits_fp32, int experts, int topk, int32_t* ids,
                             float* weights, void* stream) {
    QD_CHECK_ARG(logits && ids && weights && experts >= 1 && experts <= 1024 && topk >= 1 &&
                 topk <= experts && topk <= 32);
    route_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
        logits_fp32 ? nullptr : (const bf16*)logits, logits_fp32 ? (const float*)logits : nullptr,
        experts, topk, ids, weights);
    return qd_launch_status();
}

// --------------------------------------------------------------------- MoE combine
// out = bf16(sum_slots contribution) + bf16(shared * bf16(sigmoid(strength logit)))
// (quickdraw/models/qwen.py:189-193, quickdraw/kernel/triton/moe.py:42-57).  The slots are
// summed in ascending expert id, the order of the reference loop.
__global__ void moe_combine_kernel(const bf16* __restrict__ contributions, const int32_t* __restrict__ ids,
                                   const bf16* __restrict__ shared, const bf16* __restrict__ strength,
                                   bf16* __restrict__ out, int hidden, int topk) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= hidden) return;
    float routed = 0.f;
    int last = -1;
    for (int n = 0; n < topk; ++n) {       // selection sort over at most 32 ids
        int pick = -1, pick_id = 0x7fffffff;
        for (int s = 0; s < topk; ++s) {
            const int e = ids ? ids[s] : s;
            if (e > last && e < pick_id) { pick = s; pick_id = e; }
        }
        if (pick < 0) break;
        last = pick_id;
        routed += ld_bf16(contributions + (size_t)pick * hidden + i);
    }
    const float gate = round_bf16(sigmoid_precise(ld_bf16(strength)));
    const float gated = round_bf16(ld_bf16(shared + i) * gate);
    out[i] = __float2bfloat16_rn(round_bf16(routed) + gated);
}

extern "C" int qd_moe_combine(const void* contributions, const int32_t* ids, const void* shared,
                              const void* strength, void* out, int hidden, int topk, void* stream) {
    QD_CHECK_ARG(contributions && shared && strength && out && hidden > 0 && topk >= 1 && topk <= 32);
    moe_combine_kernel<<<(hidden + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)contributions, ids, (const bf16*)shared, (const bf16*)strength, (bf16*)out, hidden, topk);
    return qd_launch_status();
}

// Elementwise helpers of the composed (non-fused) step.
__global__ void swiglu_kernel(const bf16* gate, const bf16* up, bf16* out, int n) {
    chain_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(round_bf16(silu_precise(ld_bf16(gate + i))) * ld_bf16(up + i));
}
// eight elements per thread (16-byte accesses)
__global__ void swiglu8_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out, int n8) {
    chain_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 g = gate[i], u = up[i];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float lo = round_bf16(silu_precise(__uint_as_float(gw[q] << 16))) * __uint_as_float(uw[q] << 16);
        const float hi = round_bf16(silu_precise(__uint_as_float(gw[q] & 0xffff0000u))) * __uint_as_float(uw[q] & 0xffff0000u);
        const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
        o[q] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}
extern "C" int qd_swiglu(const void* gate, const void* up, void* out, int n, void* stream) {
    QD_CHECK_ARG(gate && up && out && n >= 0);
    if (n == 0) return QD_OK;
    if (n % 8 == 0 && !(((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) & 15u))
        qd_launch(swiglu8_kernel, dim3((n / 8 + 255) / 256), dim3(256), 0, (cudaStream_t)stream, true, (const uint4*)gate, (const uint4*)up, (uint4*)out, n / 8);
    else
        qd_launch(swiglu_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)gate, (const bf16*)up, (bf16*)out, n);
    return qd_launch_status();
}

extern "C" int qd_version(void) { return 1; }

extern "C" const char* qd_error_string(int code) {
    switch (code) {
        case QD_OK: return "ok";
        case QD_ERR_ARG: return "invalid argument";
        case QD_ERR_LAUNCH: return "CUDA launch failed";
        case QD_ERR_TIMEOUT: return "bounded device wait ran out";
        case QD_ERR_UNSUPPORTED: return "shape not covered by this kernel";
        case QD_ERR_TOO_LARGE: return "shape exceeds the fixed capacity of a built-in buffer";
        default: return "unknown";
    }
}

// Kernels of the chunk and batch paths open with a wait for the kernel before them and are launched as
// its programmatic dependents, so that their launch overlaps its last blocks.  on = 0 launches them
// ordinarily (measured faster inside a captured graph, whose edges are cheaper than the overlap gains;
// the few-row products stay dependents of their conversion kernels either way).  Returns the old setting.
extern "C" int qd_set_chained_launches(int on) {
    int& current = qd_chain_switch();
    const int before = current;
    current = on != 0;
    return before;
}

