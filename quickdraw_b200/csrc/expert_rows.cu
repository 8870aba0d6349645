// Routed expert products when an expert gets only a few rows (a decode batch: one or two routes
// per expert; a short prompt chunk: a handful): every expert that received routes is read ONCE
// and multiplied with all of its rows.
//
// Same contract as qd_nvfp4_grouped_matmul (quickdraw/kernel/triton/moe.py:99-151: the (token,
// slot) routes of a chunk sorted by expert, rows [boundaries[e], boundaries[e + 1]) belong to
// expert e).  The tcgen05 grouped product expands an expert's weights to bf16 for a 128-token
// tile that holds a handful of rows; here the weights are decoded once per eight routes on the
// warp-level tensor-core instruction, with the routes as the columns of the B operand:
//   a first small kernel writes the input rows as f16 (a row scaled down by a power of two only if it
//   would leave f16; optionally the SwiGLU of two inputs) into a scratch area;
//   block = (expert, 64 to 256 weight rows: about 90 KB); its NVFP4 tile (codes and block scales, checkpoint
//   layout) is copied to shared memory with cp.async in two halves of the inputs, rows padded
//   against bank conflicts; two blocks share an SM, so one computes while the other loads;
//   the expert's input rows follow eight at a time through two buffers of half a row each (cp.async
//   from the scratch area: one half is multiplied while the next one, of this or of the next eight
//   routes, is on its way);
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
// about 110 KB of shared memory, two blocks per SM.  NT = 4 (a short prompt chunk: some sixteen
// routes per expert, all multiplied with ONE decoding of the tile): the two buffers of 32 half rows
// take up to 130 KB, one block per SM.
template <int K, int NT> struct RowsShape {
    static constexpr int kParts = K >= 2048 ? 2 : 1;
    static constexpr int kIters = (K <= 512 && NT == 1) ? 2 : 1;
    static constexpr int kGroups = 8 / kParts;
    static constexpr int kTile = 16 * kGroups * kIters;
    static constexpr int kBlocksPerSM = (NT == 1 || K <= 512) ? 2 : 1;
};

// The f16 input rows of a pass go through two buffers: a pass's rows in halves of the inputs (one half is
// multiplied while the next is copied), or whole when the row groups take turns (kIters = 2: every turn
// reads both halves).
template <int K, int NT> constexpr int rows_units_per_pass() { return RowsShape<K, NT>::kIters == 1 ? 2 : 1; }
template <int K, int NT> constexpr int rows_x_unit_row() { return 2 * K / rows_units_per_pass<K, NT>() + 16; }   // padded, bytes
template <int K, int NT> constexpr size_t rows_smem_bytes() {
    return (size_t)RowsShape<K, NT>::kTile * (rows_code_row<K>() + rows_scale_row<K>()) + (size_t)2 * 8 * NT * rows_x_unit_row<K, NT>();
}

template <int K, int NT>
__global__ void __launch_bounds__(kRowsThreads, RowsShape<K, NT>::kBlocksPerSM) expert_rows_kernel(const RowsParams p) {
    extern __shared__ __align__(16) uint8_t rows_smem[];
    using Shape = RowsShape<K, NT>;
    constexpr int kParts = Shape::kParts, kIters = Shape::kIters, kGroups = Shape::kGroups, kRowsTile = Shape::kTile;
    constexpr int kTokens = 8 * NT;                         // routes per pass over the tile
    constexpr int kUnits = rows_units_per_pass<K, NT>();    // copies of input rows per pass
    static_assert(kParts == 1 || kIters == 1, "one meeting buffer");
    // chain_enter() in two parts: the wait follows the fetch of the weight tile.  What is read before it
    // (the boundaries) was written before the conversion kernel let this one start; read past L1.
    grid_launch_dependents();
    const int e = blockIdx.y, r0 = blockIdx.x * kRowsTile;
    const int b0 = __ldcg(p.boundaries + e), b1 = __ldcg(p.boundaries + e + 1);
    if (b1 <= b0) return;
    constexpr int code_row = rows_code_row<K>(), scale_row = rows_scale_row<K>(), x_row = rows_x_unit_row<K, NT>();
    constexpr int kUnitPieces = K / 8 / kUnits;             // 16-byte pieces of an f16 input row per copy
    constexpr int kUnitBytes = kTokens * x_row;
    const int R = p.out_features;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    uint8_t* w_codes = rows_smem;
    uint8_t* w_scales = w_codes + (size_t)kRowsTile * code_row;
    uint8_t* xt = w_scales + (size_t)kRowsTile * scale_row;                             // [2][8 NT][x_row] f16
    __shared__ int route_of[kTokens];
    __shared__ float factor[kTokens], undo[kTokens];
    __shared__ float4 meet[NT][kGroups][32];
    const int units = ((b1 - b0 + kTokens - 1) / kTokens) * kUnits;
    // input rows of copy `unit` = (pass, part of the inputs) into buffer unit & 1
    auto issue_x = [&](int unit) {
        const int first = b0 + (unit / kUnits) * kTokens, n = min(kTokens, b1 - first), h = unit % kUnits;
        uint8_t* buffer = xt + (size_t)(unit & 1) * kUnitBytes;
        for (int idx = tid; idx < n * kUnitPieces; idx += kRowsThreads) {
            const int j = idx / kUnitPieces, c = idx % kUnitPieces;
            const int row = p.by_token ? p.order[first + j] / p.topk : first + j;
            rows_cp16(buffer + (size_t)j * x_row + x_piece(c) * 16, p.xf + ((size_t)row * K + (size_t)h * (K / kUnits)) * 2 + c * 16);
        }
    };
    // ---- three cp.async groups: the block scales and the first half of the codes, the first input rows,
    // the second half of the codes (rows past the matrix are not copied)
    const int rows = min(kRowsTile, R - r0);
    const bool second = blockIdx.z != 0;                    // the gate and up banks of the same routes share a launch
    const uint8_t* codes = (second ? p.codes2 : p.codes) + (long long)e * p.codes_stride + (long long)r0 * (K / 2);
    const uint8_t* scales = (second ? p.scales2 : p.scales) + (long long)e * p.scales_stride + (long long)r0 * (K / 16);
    bf16* y = second ? p.y2 : p.y;
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
        if (h == (p.dependent ? 1 : 0)) {
            // The weights do not depend on the kernel before this one (the writer of the f16 rows): as its
            // programmatic dependent the block fetches its whole tile while that kernel still runs and
            // waits for it here; in an ordinary launch the second half of the codes follows the rows.
            grid_dependency_wait();
            issue_x(0);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    }
    const float global = (second ? p.global2 : p.global)[p.global_per_expert ? e : 0];
    const int group = warp % kGroups, part = warp / kGroups;   // sixteen rows; which part of either half of the inputs
    int unit = 0;
#pragma unroll 1
    for (int first = b0; first < b1; first += kTokens) {
        const int n = min(kTokens, b1 - first), nts = (n + 7) >> 3;     // routes of this pass, groups of eight in use
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
                if (kUnits == 2 || (it == 0 && h == 0)) {  // block-uniform: the next copy of input rows is due
                    // this copy has landed (behind the first one the second half of the codes may be in flight) ...
                    if (unit == 0 && !p.dependent) asm volatile("cp.async.wait_group 1;" ::: "memory");
                    else asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncthreads();      // ... for everybody, and everybody is done with the copy before (and its pass)
                    if (unit % kUnits == 0 && tid < kTokens) {     // where a route's result goes, what multiplies it
                        const int r = first + tid, route = tid < n ? p.order[r] : 0;
                        route_of[tid] = p.scatter ? route : r;
                        factor[tid] = (p.routing && tid < n) ? round_bf16(global * p.routing[route]) : global;
                        undo[tid] = tid < n ? p.up[p.by_token ? route / p.topk : r] : 1.f;
                    }
                    if (unit + 1 < units) issue_x(unit + 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    if (kUnits == 1) __syncthreads();      // the epilogue of the first turn reads the route tables
                    ++unit;
                }
                if (kUnits == 1 && first == b0 && it == 0 && h == 1) {       // the second half of the codes (the next rows may be in flight)
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                    __syncthreads();
                }
                const uint8_t* xs0 = xt + (size_t)((unit - 1) & 1) * kUnitBytes + (size_t)g * x_row;
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
                    const int piece0 = (kUnits == 2 ? span - h * kParts * part_spans : span) * 16 + t * 4;
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
                        const float sum = acc[nt][c] * undo[j];
                        const float result = p.routing ? round_bf16(sum) * factor[j] : sum * factor[j];
                        y[(size_t)route_of[j] * R + row] = __float2bfloat16_rn(result);
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
    const dim3 grid((unsigned)((p.out_features + tile - 1) / tile), (unsigned)p.experts, p.codes2 ? 2u : 1u);
    // a programmatic dependent only behind its own conversion kernel (which holds it back until the routes are grouped)
    if (qd_launch(expert_rows_kernel<K, NT>, grid, dim3(kRowsThreads), smem, stream, p.dependent ? 2 : 0, p) != QD_OK) return QD_ERR_LAUNCH;
    return qd_launch_status();
}
template <int K> int launch_rows_for(const RowsParams& p, bool many, cudaStream_t stream) {
    return many ? launch_rows<K, 4>(p, stream) : launch_rows<K, 1>(p, stream);
}

}  // namespace
}  // namespace qd

// Bytes of the scratch area for the f16 copy of `rows` input rows and their scale factors.
extern "C" long long qd_nvfp4_expert_rows_scratch_bytes(int rows, int in_features) {
    return rows > 0 && in_features > 0 ? (long long)rows * in_features * 2 + (long long)rows * (long long)sizeof(float) : 0;
}

// The grouped product for few rows per expert (the contract of qd_nvfp4_grouped_matmul).  x_up (or NULL):
// the input rows are bf16(bf16(silu(x)) * x_up), the SwiGLU of the gate and up products
// (quickdraw/models/qwen.py:184, 191).  The input rows (routes / topk token rows with by_token, else one
// row per route) are first written as f16 into `scratch` (qd_nvfp4_expert_rows_scratch_bytes(rows,
// in_features) bytes, 16-byte aligned); convert = 0 reuses what the previous call with this scratch area
// wrote (the gate and up products of the same tokens).
// in_features 512, 1024 or 2048, out_features a multiple of 16, group size 16, 16-byte aligned
// pointers; QD_ERR_UNSUPPORTED otherwise.  routes_per_pass: 8 or 32 routes multiplied per decoding of
// a weight tile, 0 = the library's choice (8).
static int expert_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global, void* y,
                       const void* codes2, const void* scales2, const float* global2, void* y2,
                       const int32_t* order, const int32_t* boundaries, const float* routing,
                       int routes, int experts, int topk, int out_features, int in_features,
                       int group_size, int by_token, int scatter, int global_per_expert,
                       int routes_per_pass, void* scratch, int convert, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x && codes && scales && global && order && boundaries && y && scratch);
    QD_CHECK_ARG(!codes2 || (scales2 && global2 && y2));
    if (((uintptr_t)codes2 | (uintptr_t)scales2) & 15u) return QD_ERR_UNSUPPORTED;
    QD_CHECK_ARG(routes > 0 && experts > 0 && experts <= 65535 && topk > 0 && out_features > 0 && in_features > 0);
    QD_CHECK_ARG(routes_per_pass == 0 || routes_per_pass == 8 || routes_per_pass == 32);
    if (group_size != 16 || out_features % 16 != 0) return QD_ERR_UNSUPPORTED;
    if (in_features != 512 && in_features != 1024 && in_features != 2048) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)x_up | (uintptr_t)codes | (uintptr_t)scales | (uintptr_t)scratch) & 15u) return QD_ERR_UNSUPPORTED;
    const int in_rows = by_token ? routes / topk : routes;
    QD_CHECK_ARG(in_rows > 0);
    RowsParams p = {};
    p.xf = (const uint8_t*)scratch; p.up = reinterpret_cast<const float*>(p.xf + (size_t)in_rows * in_features * 2);
    p.codes = (const uint8_t*)codes; p.scales = (const uint8_t*)scales; p.global = global;
    p.codes2 = (const uint8_t*)codes2; p.scales2 = (const uint8_t*)scales2; p.global2 = global2; p.y2 = (bf16*)y2;
    p.order = order; p.boundaries = boundaries; p.routing = routing; p.y = (bf16*)y;
    p.routes = routes; p.experts = experts; p.topk = topk; p.out_features = out_features;
    p.by_token = by_token; p.scatter = scatter; p.global_per_expert = global_per_expert;
    p.codes_stride = (long long)out_features * (in_features / 2);
    p.scales_stride = (long long)out_features * (in_features / 16);
    p.dependent = convert != 0;
    if (convert) {
        const unsigned blocks = (unsigned)((in_rows + 7) / 8);
        uint8_t* xf = (uint8_t*)scratch;
        float* up = reinterpret_cast<float*>(xf + (size_t)in_rows * in_features * 2);
        if (in_features == 512) qd_launch(rows_to_f16_warp_kernel<512>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)x_up, in_rows, xf, up);
        else if (in_features == 1024) qd_launch(rows_to_f16_warp_kernel<1024>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)x_up, in_rows, xf, up);
        else qd_launch(rows_to_f16_warp_kernel<2048>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)x_up, in_rows, xf, up);
        if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    }
    // Eight routes per pass unless the caller asks for 32 (one decoding of the tile for up to 32 routes,
    // but one block per SM and four times the MMAs per pass).
    const bool many = routes_per_pass == 32;
    switch (in_features) {
        case 512: return launch_rows_for<512>(p, many, (cudaStream_t)stream);
        case 1024: return launch_rows_for<1024>(p, many, (cudaStream_t)stream);
        default: return launch_rows_for<2048>(p, many, (cudaStream_t)stream);
    }
}

// One bank (the contract described above; a second bank: qd_nvfp4_expert_rows2 below).
extern "C" int qd_nvfp4_expert_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global,
                                    const int32_t* order, const int32_t* boundaries, const float* routing, void* y,
                                    int routes, int experts, int topk, int out_features, int in_features,
                                    int group_size, int by_token, int scatter, int global_per_expert,
                                    int routes_per_pass, void* scratch, int convert, void* stream) {
    return expert_rows(x, x_up, codes, scales, global, y, nullptr, nullptr, nullptr, nullptr, order, boundaries, routing, routes, experts,
                       topk, out_features, in_features, group_size, by_token, scatter, global_per_expert, routes_per_pass, scratch,
                       convert, stream);
}

// Two banks of the same shape against the same routes in one launch (the gate and up products of the
// routed experts, quickdraw/models/qwen.py:176-186): y = bank(x), y2 = bank2(x), each as
// qd_nvfp4_expert_rows would give it with by_token = 1, no routing weights, results in sorted order.
extern "C" int qd_nvfp4_expert_rows2(const void* x, const void* codes, const void* scales, const float* global, void* y,
                                     const void* codes2, const void* scales2, const float* global2, void* y2,
                                     const int32_t* order, const int32_t* boundaries,
                                     int routes, int experts, int topk, int out_features, int in_features,
                                     int group_size, int global_per_expert, int routes_per_pass, void* scratch, int convert,
                                     void* stream) {
    QD_CHECK_ARG(codes2 && scales2 && global2 && y2);
    return expert_rows(x, nullptr, codes, scales, global, y, codes2, scales2, global2, y2, order, boundaries, nullptr, routes, experts,
                       topk, out_features, in_features, group_size, 1, 0, global_per_expert, routes_per_pass, scratch, convert, stream);
}
