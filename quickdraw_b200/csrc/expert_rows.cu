// Routed expert products when an expert gets only a few rows (a decode batch: one or two routes
// per expert; a short prompt chunk: a handful): every expert that received routes is read ONCE
// and multiplied with all of its rows.
//
// Same contract as qd_nvfp4_grouped_matmul (quickdraw/kernel/triton/moe.py:99-151: the (token,
// slot) routes of a chunk sorted by expert, rows [boundaries[e], boundaries[e + 1]) belong to
// expert e).  The tcgen05 grouped product expands an expert's weights to bf16 for a 128-token
// tile that holds a handful of rows; here the weights are decoded once per eight routes on the
// warp-level tensor-core instruction, with the routes as the columns of the B operand:
//   block = (expert, 64 to 256 weight rows: about 90 KB); its NVFP4 tile (codes and block scales, checkpoint
//   layout) is copied to shared memory with cp.async in two halves of the inputs, rows padded
//   against bank conflicts; two blocks share an SM, so one computes while the other loads;
//   the expert's input rows go to shared memory eight at a time as f16 (scaled down by a power
//   of two only if they would overflow);
//   a warp owns sixteen weight rows at a time (at 2048 inputs two warps share them, each with
//   one input quarter of either half): per 128 inputs a lane converts 32 codes of two rows (cvt.rn.f16x2.e2m1x2, exact f16 multiply with
//   the E4M3 scale) and feeds 8 MMAs (m16n8k16); fp32 accumulators, the two warps of a row
//   group meet in shared memory.
// Rounding as in the single-token kernels: fp32 sum, global scale last, one bf16 rounding;
// with routing weights the routed double rounding (quickdraw/models/qwen.py:44-53).
#include <algorithm>

#include "expert_rows.cuh"

namespace qd {
namespace {

constexpr int kRowsThreads = 256;
// Shape of a block per input width K and routes per pass (8 NT): PARTS warps share a group of
// sixteen rows (each takes a part of the inputs), the 8 / PARTS groups take ITERS turns:
// 16 * (8 / PARTS) * ITERS weight rows.  NT = 1 (a decode batch: one or two routes per expert):
// about 100 KB of shared memory, two blocks per SM.  NT = 4 (a short prompt chunk: some sixteen
// routes per expert, all multiplied with ONE decoding of the tile): the 32 input rows take up to
// 130 KB, one block per SM.
template <int K, int NT> struct RowsShape {
    static constexpr int kParts = K >= 2048 ? 2 : 1;
    static constexpr int kIters = (K <= 512 && NT == 1) ? 2 : 1;
    static constexpr int kGroups = 8 / kParts;
    static constexpr int kTile = 16 * kGroups * kIters;
    static constexpr int kBlocksPerSM = NT == 1 ? 2 : 1;
};

template <int K, int NT> constexpr size_t rows_smem_bytes() {
    return (size_t)RowsShape<K, NT>::kTile * (rows_code_row<K>() + rows_scale_row<K>()) + (size_t)8 * NT * rows_x_row<K>();
}

template <int K, int NT>
__global__ void __launch_bounds__(kRowsThreads, RowsShape<K, NT>::kBlocksPerSM) expert_rows_kernel(const RowsParams p) {
    extern __shared__ __align__(16) uint8_t rows_smem[];
    using Shape = RowsShape<K, NT>;
    constexpr int kParts = Shape::kParts, kIters = Shape::kIters, kGroups = Shape::kGroups, kRowsTile = Shape::kTile;
    constexpr int kTokens = 8 * NT;                         // routes per pass over the tile
    static_assert(kParts == 1 || kIters == 1, "one meeting buffer");
    const int e = blockIdx.y, r0 = blockIdx.x * kRowsTile;
    const int b0 = p.boundaries[e], b1 = p.boundaries[e + 1];
    if (b1 <= b0) return;
    constexpr int code_row = rows_code_row<K>(), scale_row = rows_scale_row<K>(), x_row = rows_x_row<K>();
    constexpr int kPieces = K / 8;                          // 16-byte pieces of a bf16 input row
    constexpr int kBatch = (kTokens * kPieces / kRowsThreads) < 16 ? (kTokens * kPieces / kRowsThreads) : 16;   // loads in flight per thread
    static_assert(kTokens * kPieces % (kBatch * kRowsThreads) == 0 && K % 512 == 0, "input width");
    const int R = p.out_features;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    uint8_t* w_codes = rows_smem;
    uint8_t* w_scales = w_codes + (size_t)kRowsTile * code_row;
    uint8_t* xt = w_scales + (size_t)kRowsTile * scale_row;                             // [8 NT][x_row] f16
    __shared__ float red[8];
    __shared__ int source[kTokens], route_of[kTokens];
    __shared__ float factor[kTokens];
    __shared__ float4 meet[NT][kGroups][32];
    // ---- the expert's weight tile, in two cp.async groups by half of the inputs (rows past the
    // matrix are not copied; the block scales travel with the first half)
    const int rows = min(kRowsTile, R - r0);
    const uint8_t* codes = p.codes + (long long)e * p.codes_stride + (long long)r0 * (K / 2);
    const uint8_t* scales = p.scales + (long long)e * p.scales_stride + (long long)r0 * (K / 16);
    for (int piece = tid; piece < rows * (K / 256); piece += kRowsThreads) {
        const int r = piece / (K / 256), c = piece % (K / 256);
        rows_cp16(w_scales + (size_t)r * scale_row + c * 16, scales + (size_t)r * (K / 16) + c * 16);
    }
    constexpr int half = K / 64;          // 16-byte pieces of a row's codes per half
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        for (int piece = tid; piece < rows * half; piece += kRowsThreads) {
            const int r = piece / half, c = h * half + piece % half;
            rows_cp16(w_codes + (size_t)r * code_row + c * 16, codes + (size_t)r * (K / 2) + c * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const float global = p.global[p.global_per_expert ? e : 0];
    const int group = warp % kGroups, part = warp / kGroups;   // sixteen rows; which part of either half of the inputs
#pragma unroll 1
    for (int first = b0; first < b1; first += kTokens) {
        const int n = min(kTokens, b1 - first), nts = (n + 7) >> 3;     // routes of this pass, groups of eight in use
        __syncthreads();                  // the pass before is done with xt, red, source and meet
        if (tid < kTokens) {              // where a route's input row lies, where its result goes, what multiplies it
            const int r = first + tid, route = tid < n ? p.order[r] : 0;
            source[tid] = tid < n ? (p.by_token ? route / p.topk : r) : -1;
            route_of[tid] = p.scatter ? route : r;
            factor[tid] = (p.routing && tid < n) ? round_bf16(global * p.routing[route]) : global;
        }
        __syncthreads();
        // ---- the input rows of this pass as f16 (up to kBatch 16-byte loads in flight per thread) and
        // their largest magnitude; `down`: power of two applied on the way
        auto stage = [&](float down) -> float {
            uint32_t biggest = 0u;
#pragma unroll 1
            for (int base = 0; base < nts * 8 * kPieces; base += kBatch * kRowsThreads) {
                uint4 v[kBatch];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const int idx = base + tid + i * kRowsThreads, j = idx / kPieces, c = idx % kPieces, row = source[j];
                    v[i] = row >= 0 ? reinterpret_cast<const uint4*>(p.x + (size_t)row * K)[c] : make_uint4(0u, 0u, 0u, 0u);
                }
                if (p.x_up) {             // the input is bf16(bf16(silu(x)) * x_up): SwiGLU of the gate / up rows on the way in
#pragma unroll
                    for (int i = 0; i < kBatch; ++i) {
                        const int idx = base + tid + i * kRowsThreads, j = idx / kPieces, c = idx % kPieces, row = source[j];
                        if (row < 0) continue;
                        const uint4 u = reinterpret_cast<const uint4*>(p.x_up + (size_t)row * K)[c];
                        const uint32_t gw[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, uw[4] = {u.x, u.y, u.z, u.w};
                        uint32_t o[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float lo = round_bf16(silu_precise(__uint_as_float(gw[q] << 16))) * __uint_as_float(uw[q] << 16);
                            const float hi = round_bf16(silu_precise(__uint_as_float(gw[q] & 0xffff0000u))) * __uint_as_float(uw[q] & 0xffff0000u);
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                            o[q] = *reinterpret_cast<const uint32_t*>(&pair);
                        }
                        v[i] = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const int idx = base + tid + i * kRowsThreads, j = idx / kPieces, c = idx % kPieces;
                    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        biggest = max(biggest, max(w[q] & 0x7fffu, (w[q] >> 16) & 0x7fffu));
                        o[q] = pack_f16x2(__uint_as_float(w[q] << 16) * down, __uint_as_float(w[q] & 0xffff0000u) * down);
                    }
                    *reinterpret_cast<uint4*>(xt + (size_t)j * x_row + x_piece(c) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
            return __uint_as_float(biggest << 16);
        };
        float top = warp_max(stage(1.f));
        if (lane == 0) red[warp] = top;
        __syncthreads();
        top = fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
        float up = 1.f;
        if (top >= 32768.f) {             // rare: the rows would leave f16; a power-of-two down-scale keeps them inside
            const int exponent = (int)((__float_as_uint(top) >> 23) & 0xffu) - 127;
            const int shift = exponent < 128 ? exponent - 14 : 0;
            up = __uint_as_float((uint32_t)(127 + shift) << 23);
            stage(__uint_as_float((uint32_t)(127 - shift) << 23));
            __syncthreads();
        }
        // ---- sixteen weight rows of this warp against the pass's routes, its part of either half
        constexpr int part_spans = K / 128 / (2 * kParts);
#pragma unroll 1
        for (int it = 0; it < kIters; ++it) {
            const int mine = (it * kGroups + group) * 16;
            const bool live = mine < rows;                 // a warp without rows computes on rows 0..15 and stores nothing
            const int slot0 = live ? mine : 0;
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = 0.f; acc[nt][1] = 0.f; acc[nt][2] = 0.f; acc[nt][3] = 0.f; }
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                if (first == b0 && it == 0) {              // block-uniform: this half of the tile has landed
                    if (h == 0) asm volatile("cp.async.wait_group 1;" ::: "memory");
                    else asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncthreads();
                }
#pragma unroll 2
                for (int s = 0; s < part_spans; ++s) {
                    const int span = (h * kParts + part) * part_spans + s;
                    const uint8_t* c0 = w_codes + (size_t)(slot0 + g) * code_row + span * 64 + t * 16;
                    const uint8_t* s0 = w_scales + (size_t)(slot0 + g) * scale_row + span * 8 + t * 2;
                    const uint4 w0 = lds128(c0), w1 = lds128(c0 + 8 * code_row);
                    const uint32_t p0 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0));
                    const uint32_t p1 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0 + 8 * scale_row));
                    const uint32_t sa0 = __byte_perm(p0, 0u, 0x1010), sb0 = __byte_perm(p0, 0u, 0x3232);
                    const uint32_t sa1 = __byte_perm(p1, 0u, 0x1010), sb1 = __byte_perm(p1, 0u, 0x3232);
                    const uint32_t ra[4] = {w0.x, w0.y, w0.z, w0.w}, rb[4] = {w1.x, w1.y, w1.z, w1.w};
                    // the lane's activations of this span: route 8 nt + g is its column of group nt
                    const uint8_t* xs0 = xt + (size_t)g * x_row;
                    const int piece0 = span * 16 + t * 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t h0[4], h1[4];
                        e2m1x8_to_f16x2(ra[j], h0);
                        e2m1x8_to_f16x2(rb[j], h1);
                        const uint32_t s_lo = j < 2 ? sa0 : sb0, s_hi = j < 2 ? sa1 : sb1;
#pragma unroll
                        for (int b = 0; b < 4; ++b) { h0[b] = hmul2(h0[b], s_lo); h1[b] = hmul2(h1[b], s_hi); }
                        const int at = x_piece(piece0 + j) * 16;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            if (NT == 1 || nt < nts) {
                                const uint4 u = lds128(xs0 + (size_t)nt * 8 * x_row + at);
                                mma_f16(acc[nt], h0[0], h1[0], h0[1], h1[1], u.x, u.y);
                                mma_f16(acc[nt], h0[2], h1[2], h0[3], h1[3], u.z, u.w);
                            }
                        }
                    }
                }
            }
            // ---- the warps of a row group meet; acc[nt][0..1] = row slot0 + g, routes 8 nt + 2 t and + 1; [2..3] = row + 8
            if (kParts == 2) {
                if (part == 1) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) meet[nt][group][lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
                }
                __syncthreads();
                if (part == 0) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const float4 other = meet[nt][group][lane];
                        acc[nt][0] += other.x; acc[nt][1] += other.y; acc[nt][2] += other.z; acc[nt][3] += other.w;
                    }
                }
            }
            if (part == 0 && live) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = 8 * nt + 2 * t + (c & 1), row = r0 + slot0 + g + 8 * (c >> 1);
                        if (j >= n || row >= R) continue;
                        const float sum = acc[nt][c] * up;
                        const float result = p.routing ? round_bf16(sum) * factor[j] : sum * factor[j];
                        p.y[(size_t)route_of[j] * R + row] = __float2bfloat16_rn(result);
                    }
            }
        }
    }
}

template <int K, int NT> int launch_rows(const RowsParams& p, cudaStream_t stream) {
    constexpr size_t smem = rows_smem_bytes<K, NT>();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(expert_rows_kernel<K, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    constexpr int tile = RowsShape<K, NT>::kTile;
    const dim3 grid((unsigned)((p.out_features + tile - 1) / tile), (unsigned)p.experts);
    expert_rows_kernel<K, NT><<<grid, kRowsThreads, smem, stream>>>(p);
    return qd_launch_status();
}
template <int K> int launch_rows_for(const RowsParams& p, bool many, cudaStream_t stream) {
    return many ? launch_rows<K, 4>(p, stream) : launch_rows<K, 1>(p, stream);
}

}  // namespace
}  // namespace qd

// The grouped product for few rows per expert (the contract of qd_nvfp4_grouped_matmul).  x_up (or NULL):
// the input rows are bf16(bf16(silu(x)) * x_up), the SwiGLU of the gate and up products
// (quickdraw/models/qwen.py:184, 191), computed while the rows are staged.
// in_features 512, 1024 or 2048, out_features a multiple of 16, group size 16, 16-byte aligned
// pointers; QD_ERR_UNSUPPORTED otherwise.  routes_per_pass: 8 or 32 routes multiplied per decoding of
// a weight tile, 0 = the library's choice (8).
extern "C" int qd_nvfp4_expert_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global,
                                    const int32_t* order, const int32_t* boundaries, const float* routing, void* y,
                                    int routes, int experts, int topk, int out_features, int in_features,
                                    int group_size, int by_token, int scatter, int global_per_expert,
                                    int routes_per_pass, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x && codes && scales && global && order && boundaries && y);
    QD_CHECK_ARG(routes > 0 && experts > 0 && experts <= 65535 && topk > 0 && out_features > 0 && in_features > 0);
    QD_CHECK_ARG(routes_per_pass == 0 || routes_per_pass == 8 || routes_per_pass == 32);
    if (group_size != 16 || out_features % 16 != 0) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)x_up | (uintptr_t)codes | (uintptr_t)scales) & 15u) return QD_ERR_UNSUPPORTED;
    RowsParams p = {};
    p.x = (const bf16*)x; p.x_up = (const bf16*)x_up; p.codes = (const uint8_t*)codes; p.scales = (const uint8_t*)scales; p.global = global;
    p.order = order; p.boundaries = boundaries; p.routing = routing; p.y = (bf16*)y;
    p.routes = routes; p.experts = experts; p.topk = topk; p.out_features = out_features;
    p.by_token = by_token; p.scatter = scatter; p.global_per_expert = global_per_expert;
    p.codes_stride = (long long)out_features * (in_features / 2);
    p.scales_stride = (long long)out_features * (in_features / 16);
    // Eight routes per pass unless the caller asks for 32: measured at 16 routes per expert (a 511-token
    // chunk) the two forms are within 10 % of each other (gate 105 against 118 us, down 101 against 98 us:
    // one decoding of the tile for all routes, but one block per SM and four times the MMAs per pass).
    const bool many = routes_per_pass == 32;
    switch (in_features) {
        case 512: return launch_rows_for<512>(p, many, (cudaStream_t)stream);
        case 1024: return launch_rows_for<1024>(p, many, (cudaStream_t)stream);
        case 2048: return launch_rows_for<2048>(p, many, (cudaStream_t)stream);
        default: return QD_ERR_UNSUPPORTED;
    }
}
