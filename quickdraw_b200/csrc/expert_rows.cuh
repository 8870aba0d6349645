// Parameters and small helpers of the routed expert product for few routes per expert (expert_rows.cu).
#pragma once
#include "rowdot.cuh"
#include "rowmma.cuh"

namespace qd {

struct RowsParams {
    const bf16* x; const bf16* x_up; const uint8_t* codes; const uint8_t* scales; const float* global;
    const int32_t* order; const int32_t* boundaries; const float* routing; bf16* y;
    int routes, experts, topk, out_features, by_token, scatter, global_per_expert;
    long long codes_stride, scales_stride;
};

QD_DEVINL void rows_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// 16-byte piece c of an input row sits at piece c ^ (bit 3 of c << 1): the four pieces a
// quarter-warp reads at once (c = 4 t + q) then fall on different banks
QD_DEVINL int x_piece(int c) { return c ^ ((c >> 2) & 2); }

template <int K> constexpr int rows_code_row() { return K / 2 + 64; }      // padded row strides, bytes
template <int K> constexpr int rows_scale_row() { return K / 16 + 16; }
template <int K> constexpr int rows_x_row() { return 2 * K + 16; }

// bf16(bf16(silu(g)) * u) for eight values: the SwiGLU of gate and up rows on their way in
QD_DEVINL uint4 rows_swiglu8(const uint4& g, const uint4& u) {
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float lo = round_bf16(silu_precise(__uint_as_float(gw[q] << 16))) * __uint_as_float(uw[q] << 16);
        const float hi = round_bf16(silu_precise(__uint_as_float(gw[q] & 0xffff0000u))) * __uint_as_float(uw[q] & 0xffff0000u);
        const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
        o[q] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace qd
