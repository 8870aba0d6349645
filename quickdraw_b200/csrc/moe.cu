// MoE tail of a decode step: the routed down projections, the shared expert's down
// projection and the combine, in one launch (reference: quickdraw/models/qwen.py:185-193,
// quickdraw/kernel/cute/moe.py:61-73,101-116).
//
// Every block owns a contiguous range of output rows and fetches, for those rows, the
// code and scale rows of all selected experts plus the shared expert with one batch of
// bulk copies.  Warp s works on slot s (one expert): its 512-wide hidden vector sits in
// registers, each half-warp takes alternate rows (a 512-input row is 16 lanes x 16 bytes).
// Rounding points: routed slot = bf16(bf16(acc) * bf16(global * routing weight)); slots are
// summed in fp32 in ascending expert id and rounded once; the shared row is
// bf16(acc * global), times bf16(sigmoid(gate logit)) rounded to bf16; final sum bf16.
#include "common.cuh"

namespace {

constexpr int kDownSlots = 9;        // top-8 + shared
constexpr int kDownMaxRows = 32;
constexpr int kDownWidth = 512;
constexpr int kDownRowBytes = kDownWidth / 2 + kDownWidth / 16;   // 288
constexpr int kDownThreads = (kDownSlots + 1) * 32;

struct DownParams {
    const bf16* hidden;                 // [topk + 1][512]; last row = shared expert
    const int32_t* ids; const float* weights;
    const uint8_t* dw; const uint8_t* ds; const float* dg; int g_per_expert;
    const uint8_t* sw; const uint8_t* ss; const float* sg;
    const bf16* strength;
    bf16* out;                          // combined output, or NULL in expert-parallel mode
    float* routed_out; bf16* shared_out;   // expert-parallel mode: partial sum + gated shared row
    int H, topk, expert_lo, expert_hi;
    unsigned int* status;
};

__global__ void __launch_bounds__(kDownThreads)
moe_down_kernel(const __grid_constant__ DownParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // per slot: codes [kDownMaxRows][256] then scales [kDownMaxRows][32]
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + kDownSlots * kDownMaxRows * kDownRowBytes);
    float* contrib = reinterpret_cast<float*>(bar + 1);        // [slots][kDownMaxRows]
    int* s_ids = reinterpret_cast<int*>(contrib + kDownSlots * kDownMaxRows);   // [16]
    float* s_w = reinterpret_cast<float*>(s_ids + 16);                          // [16]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = (int)((long long)p.H * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.H * (blockIdx.x + 1) / gridDim.x);
    const int n = r1 - r0;
    const int nslots = p.topk + 1;

    if (tid == 0) { mbar_init(bar, 1); mbar_fence_init(); }
    __syncthreads();
    grid_launch_dependents();
    grid_dependency_wait();
    if (tid < p.topk) { s_ids[tid] = p.ids[tid]; s_w[tid] = p.weights[tid]; }
    __syncthreads();

    if (warp == kDownSlots) {
        if (lane == 0 && n > 0) {
            uint32_t bytes = 0;
            for (int s = 0; s < nslots; ++s) {
                const bool shared = s == p.topk;
                const int e = shared ? 0 : s_ids[s];
                if (!shared && (e < p.expert_lo || e >= p.expert_hi)) continue;
                bytes += (uint32_t)n * kDownRowBytes;
            }
            mbar_expect_tx(bar, bytes);
            for (int s = 0; s < nslots; ++s) {
                const bool shared = s == p.topk;
                const int e = shared ? 0 : s_ids[s];
                if (!shared && (e < p.expert_lo || e >= p.expert_hi)) continue;
                const long long row = shared ? r0 : (long long)(e - p.expert_lo) * p.H + r0;
                const uint8_t* w = (shared ? p.sw : p.dw) + row * (kDownWidth / 2);
                const uint8_t* sc = (shared ? p.ss : p.ds) + row * (kDownWidth / 16);
                uint8_t* dst = smem + (size_t)s * kDownMaxRows * kDownRowBytes;
                bulk_load(dst, w, n * (kDownWidth / 2), bar);
                bulk_load(dst + kDownMaxRows * (kDownWidth / 2), sc, n * (kDownWidth / 16), bar);
            }
        }
    } else if (warp < nslots && n > 0) {
        const int s = warp;
        const bool shared = s == p.topk;
        const int e = shared ? 0 : s_ids[s];
        const bool owned = shared || (e >= p.expert_lo && e < p.expert_hi);
        const int hl = lane & 15, half = lane >> 4;
        // hidden slice of this lane: inputs [32 hl, 32 hl + 32) as packed f16, scaled to fit
        uint32_t xh[16];
        float amax = 0.f;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.hidden + (size_t)s * kDownWidth) + hl * 16;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            xh[j] = src[j];
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(xh[j] << 16)), fabsf(__uint_as_float(xh[j] & 0xffff0000u))));
        }
        amax = warp_max(amax);
        int ex = 0;
        if (amax > 0.f && amax < INFINITY) frexpf(amax, &ex);
        const int shift = ex > 15 ? ex - 15 : 0;
        const float down = ldexpf(1.f, -shift), mult = ldexpf(1.f, shift);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const __half2 h = __floats2half2_rn(__uint_as_float(xh[j] << 16) * down,
                                                __uint_as_float(xh[j] & 0xffff0000u) * down);
            xh[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        float scale;
        if (shared) scale = p.sg[0];
        else scale = round_bf16(p.dg[p.g_per_expert ? e - p.expert_lo : 0] * s_w[s]);
        const bool ok = !owned || mbar_wait(bar, 0, p.status);
        const uint8_t* base = smem + (size_t)s * kDownMaxRows * kDownRowBytes;
        // both half-warps run the same number of iterations (the shuffles below name all
        // 32 lanes); a half-warp past the last row recomputes it and does not store.
        for (int rr = 0; rr < n; rr += 2) {
            const bool live = rr + half < n;
            const int r = live ? rr + half : n - 1;
            float value = 0.f;
            if (owned && ok) {
                const uint4 w = lds128(base + r * (kDownWidth / 2) + hl * 16);
                const float2 sc = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(
                    base + kDownMaxRows * (kDownWidth / 2) + r * (kDownWidth / 16) + hl * 2));
                const uint32_t words[4] = {w.x, w.y, w.z, w.w};
                float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t h2[4];
                    e2m1x8_to_f16x2(words[q], h2);
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        g[(q >> 1) * 2] = fma_f16_lo(h2[b], xh[q * 4 + b], g[(q >> 1) * 2]);
                        g[(q >> 1) * 2 + 1] = fma_f16_hi(h2[b], xh[q * 4 + b], g[(q >> 1) * 2 + 1]);
                    }
                }
                float acc = fmaf(sc.x, g[0] + g[1], 0.f);
                acc = fmaf(sc.y, g[2] + g[3], acc);
                acc = group_sum<16>(acc) * mult;
                value = shared ? round_bf16(acc * scale) : round_bf16(round_bf16(acc) * scale);
            }
            if (hl == 0 && live) contrib[s * kDownMaxRows + r] = value;
        }
    }
    __syncthreads();
    // combine: one thread per row
    if (tid < n) {
        float routed = 0.f;
        int last = -1;
        for (int k = 0; k < p.topk; ++k) {       // ascending expert id
            int pick = -1, pick_id = 0x7fffffff;
            for (int s = 0; s < p.topk; ++s) {
                const int e = s_ids[s];
                if (e > last && e < pick_id) { pick = s; pick_id = e; }
            }
            if (pick < 0) break;
            last = pick_id;
            routed += contrib[pick * kDownMaxRows + tid];
        }
        const float gate = round_bf16(sigmoid_precise(ld_bf16(p.strength)));
        const float shared = round_bf16(contrib[p.topk * kDownMaxRows + tid] * gate);
        if (p.out) p.out[r0 + tid] = __float2bfloat16_rn(round_bf16(routed) + shared);
        if (p.routed_out) { p.routed_out[r0 + tid] = routed; p.shared_out[r0 + tid] = __float2bfloat16_rn(shared); }
    }
}

// Expert-parallel finish after the all-reduce of the routed partial sums:
// out = bf16(bf16(sum) + gated shared row).
__global__ void moe_finish_kernel(const float* __restrict__ routed, const bf16* __restrict__ shared,
                                  bf16* __restrict__ out, int n) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(round_bf16(routed[i]) + ld_bf16(shared + i));
}

}  // namespace

extern "C" int qd_moe_down_combine(const void* hidden, const int32_t* ids, const float* weights,
                                   const void* down_codes, const void* down_scales, const float* down_global,
                                   const void* shared_codes, const void* shared_scales,
                                   const float* shared_global, const void* strength, void* out,
                                   float* routed_out, void* shared_out, int hidden_size, int intermediate,
                                   int topk, int global_per_expert, int expert_lo, int expert_hi, int pdl,
                                   void* stream) {
    QD_CHECK_ARG(hidden && ids && weights && down_codes && down_scales && down_global && shared_codes &&
                 shared_scales && shared_global && strength);
    QD_CHECK_ARG((out != nullptr) != (routed_out != nullptr) && (!routed_out || shared_out));
    if (intermediate != kDownWidth || topk + 1 > kDownSlots || topk < 1) return QD_ERR_UNSUPPORTED;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = sms > 0 ? sms : 148;
    if ((hidden_size + grid - 1) / grid > kDownMaxRows) grid = (hidden_size + kDownMaxRows - 1) / kDownMaxRows;
    DownParams p;
    p.hidden = (const bf16*)hidden; p.ids = ids; p.weights = weights;
    p.dw = (const uint8_t*)down_codes; p.ds = (const uint8_t*)down_scales; p.dg = down_global;
    p.g_per_expert = global_per_expert;
    p.sw = (const uint8_t*)shared_codes; p.ss = (const uint8_t*)shared_scales; p.sg = shared_global;
    p.strength = (const bf16*)strength; p.out = (bf16*)out; p.routed_out = routed_out;
    p.shared_out = (bf16*)shared_out; p.H = hidden_size; p.topk = topk;
    p.expert_lo = expert_lo; p.expert_hi = expert_hi; p.status = nullptr;
    const size_t smem = (size_t)kDownSlots * kDownMaxRows * kDownRowBytes + 8 + kDownSlots * kDownMaxRows * 4 + 128;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[device]) {
        if (cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[device] = true;
    }
    return qd_launch(moe_down_kernel, dim3(grid), dim3(kDownThreads), smem, (cudaStream_t)stream, pdl != 0, p);
}

extern "C" int qd_moe_finish(const float* routed, const void* shared, void* out, int n, int pdl, void* stream) {
    QD_CHECK_ARG(routed && shared && out && n > 0);
    return qd_launch(moe_finish_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream, pdl != 0,
                     routed, (const bf16*)shared, (bf16*)out, n);
}
