// Parameters and small helpers of the products with few token rows: the routed expert product for few
// routes per expert (expert_rows.cu) and the dense projections of a decode batch (dense_rows.cu).
#pragma once
#include "rowdot.cuh"
#include "rowmma.cuh"

namespace qd {

struct RowsParams {
    const uint8_t* xf; const float* up; const uint8_t* codes; const uint8_t* scales; const float* global;
    const int32_t* order; const int32_t* boundaries; const float* routing; bf16* y;
    const uint8_t* codes2; const uint8_t* scales2; const float* global2; bf16* y2;    // a second bank of the same shape (blockIdx.z = 1)
    int routes, experts, topk, out_features, by_token, scatter, global_per_expert;
    int dependent;        // launched as the programmatic dependent of the kernel that writes xf and up
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


// Largest magnitude of eight bf16 values, as bf16 bits without the sign.
QD_DEVINL uint32_t rows_biggest8(const uint4& v, uint32_t biggest) {
    biggest = max(max(biggest, max(v.x & 0x7fffu, (v.x >> 16) & 0x7fffu)), max(v.y & 0x7fffu, (v.y >> 16) & 0x7fffu));
    return max(max(biggest, max(v.z & 0x7fffu, (v.z >> 16) & 0x7fffu)), max(v.w & 0x7fffu, (v.w >> 16) & 0x7fffu));
}
// The power-of-two shift that keeps a row with largest magnitude `top` inside f16 (0 for nearly every row).
QD_DEVINL int rows_shift(float top) {
    const int exponent = (int)((__float_as_uint(top) >> 23) & 0xffu) - 127;
    return (exponent > 14 && exponent < 128) ? exponent - 14 : 0;
}
QD_DEVINL uint4 rows_f16x8(const uint4& v, float down) {      // eight bf16 values times `down` as f16
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
        o[q] = pack_f16x2(__uint_as_float(w[q] << 16) * down, __uint_as_float(w[q] & 0xffff0000u) * down);
    return make_uint4(o[0], o[1], o[2], o[3]);
}

namespace {

// Token rows as f16, a block per row: xf [gridDim.x][K] (rows past `tokens` zero), up[t] = the power of
// two that undoes row t's down-scale.  x_up (or NULL): the rows are the SwiGLU of x (gate) and x_up.
__global__ void __launch_bounds__(256) rows_to_f16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ x_up, int tokens, int K,
                                                          uint8_t* __restrict__ xf, float* __restrict__ up) {
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    chain_enter();            // the product that reads these rows may start: it fetches weights until this kernel has finished
    uint4* out = reinterpret_cast<uint4*>(xf + (size_t)row * K * 2);
    if (row >= tokens) {
        for (int c = tid; c < K / 8; c += 256) out[c] = make_uint4(0u, 0u, 0u, 0u);
        if (tid == 0) up[row] = 1.f;
        return;
    }
    __shared__ float red[8];
    const uint4* in = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    const uint4* in_up = x_up ? reinterpret_cast<const uint4*>(x_up + (size_t)row * K) : nullptr;
    uint32_t biggest = 0u;
    for (int c = tid; c < K / 8; c += 256) biggest = rows_biggest8(in_up ? rows_swiglu8(in[c], in_up[c]) : in[c], biggest);
    float top = warp_max(__uint_as_float(biggest << 16));
    if (lane == 0) red[warp] = top;
    __syncthreads();
    top = fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
    const int shift = rows_shift(top);
    const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
    for (int c = tid; c < K / 8; c += 256) out[c] = rows_f16x8(in_up ? rows_swiglu8(in[c], in_up[c]) : in[c], down);
    if (tid == 0) up[row] = __uint_as_float((uint32_t)(127 + shift) << 23);
}

// The same for many rows, a warp per row, the row held in registers.
template <int K>
__global__ void __launch_bounds__(256) rows_to_f16_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ x_up, int rows,
                                                               uint8_t* __restrict__ xf, float* __restrict__ up) {
    constexpr int N = K / 256;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    // The routed product that follows reads the routes' boundaries before its own wait, so it may only be
    // scheduled once the kernels before this one have finished: wait first, then let it start (it fetches
    // its weight tile while this kernel runs).
    grid_dependency_wait();
    grid_launch_dependents();
    if (row >= rows) return;
    const uint4* in = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    uint4 v[N];
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = in[lane + 32 * i];
    if (x_up) {
        const uint4* in_up = reinterpret_cast<const uint4*>(x_up + (size_t)row * K);
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = rows_swiglu8(v[i], in_up[lane + 32 * i]);
    }
    uint32_t biggest = 0u;
#pragma unroll
    for (int i = 0; i < N; ++i) biggest = rows_biggest8(v[i], biggest);
    const int shift = rows_shift(warp_max(__uint_as_float(biggest << 16)));
    const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
    uint4* out = reinterpret_cast<uint4*>(xf + (size_t)row * K * 2);
#pragma unroll
    for (int i = 0; i < N; ++i) out[lane + 32 * i] = rows_f16x8(v[i], down);
    if (lane == 0) up[row] = __uint_as_float((uint32_t)(127 + shift) << 23);
}

}  // namespace
}  // namespace qd
