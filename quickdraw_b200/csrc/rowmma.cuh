// NVFP4 rows against one activation vector on the warp-level tensor-core instruction
// (mma.sync m16n8k16, f16 operands, fp32 accumulator).
//
// A tile of weight rows sits in shared memory in the checkpoint layout: codes
// [slots][K/2] bytes, then E4M3 block scales [slots][K/16] bytes.  The sixteen consumer
// warps of a block split the K inputs between them in spans of 128 inputs; a warp takes sixteen
// rows of its span at a time:
//   lane (g, t), g = lane / 4, t = lane % 4, loads sixteen code bytes (32 inputs) of row g
//   and of row g + 8, converts them with cvt.rn.f16x2.e2m1x2, multiplies each pair with the
//   block scale in f16 (exact: two significant bits times four) and feeds them to eight MMAs
//   as the A operand; the B operand is the lane's own 32 activations (f16 pairs, kept in
//   registers for the whole phase).
// Rows with odd g read the neighbouring span (span ^ 1), so that the eight rows of a
// quarter-warp do not collide on the shared-memory banks (row strides are multiples of 128
// bytes); because column n of B is supplied by the lanes of row n, only the diagonal of the
// 16 x 8 result is meaningful: D[g][g] and D[g + 8][g], held by lane (g, g / 2).
// The warps' partial sums meet in shared memory; one warp per tile (rotating) adds them in
// warp order and applies the row epilogue.  Global scale and bf16 rounding come last
// (quickdraw/models/qwen.py:36-54).
#pragma once
#include "stream.cuh"

namespace qd {

constexpr int kRowWarps = 16;               // consumer warps that share the K split
constexpr int kRowSlots = 32;               // partial sums per warp and tile (two groups of sixteen rows)
constexpr int kRowPartialFloats = kRowWarps * kRowSlots;

QD_DEVINL void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
QD_DEVINL uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// two E4M3 bytes -> f16x2 (low byte in the low half), exact
QD_DEVINL uint32_t e4m3x2_to_f16x2(uint16_t pair) {
    uint32_t d;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"(pair));
    return d;
}

// Span of 128 inputs that unit u of warp `warp` covers for the rows of lane group g.
template <int UNITS> QD_DEVINL int row_span(int warp, int u, int g) {
    return UNITS == 1 ? (warp ^ (g & 1)) : (UNITS * warp + (u ^ (g & 1)));
}

// The lane's activations for its spans: xf is the vector as f16 in natural order.
template <int UNITS>
QD_DEVINL void load_x_fragments(const uint8_t* __restrict__ xf, int warp, int lane, uint32_t (&xh)[UNITS][16]) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const uint8_t* src = xf + (row_span<UNITS>(warp, u, g) * 128 + t * 32) * 2;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = lds128(src + q * 16);
            xh[u][q * 4 + 0] = v.x; xh[u][q * 4 + 1] = v.y; xh[u][q * 4 + 2] = v.z; xh[u][q * 4 + 3] = v.w;
        }
    }
}

// Sixteen rows (slots slot0 + g and slot0 + g + 8) of one span: sixteen MMAs into acc.
// codes_row / scales_row: byte strides of a row.
QD_DEVINL void unit_mma(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, int codes_row,
                        int scales_row, int slot0, int span, int g, int t, const uint32_t (&xh)[16],
                        float (&acc_a)[4], float (&acc_b)[4]) {
    const uint8_t* c0 = codes + (slot0 + g) * codes_row + span * 64 + t * 16;
    const uint8_t* s0 = scales + (slot0 + g) * scales_row + span * 8 + t * 2;
    const uint4 w0 = lds128(c0), w1 = lds128(c0 + 8 * codes_row);
    const uint32_t p0 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0));
    const uint32_t p1 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0 + 8 * scales_row));
    const uint32_t sa0 = __byte_perm(p0, 0u, 0x1010), sb0 = __byte_perm(p0, 0u, 0x3232);   // first / second block of row g
    const uint32_t sa1 = __byte_perm(p1, 0u, 0x1010), sb1 = __byte_perm(p1, 0u, 0x3232);   // ... of row g + 8
    const uint32_t r0[4] = {w0.x, w0.y, w0.z, w0.w}, r1[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t h0[4], h1[4];
        e2m1x8_to_f16x2(r0[j], h0);
        e2m1x8_to_f16x2(r1[j], h1);
        const uint32_t s_lo = j < 2 ? sa0 : sb0, s_hi = j < 2 ? sa1 : sb1;
#pragma unroll
        for (int b = 0; b < 4; ++b) { h0[b] = hmul2(h0[b], s_lo); h1[b] = hmul2(h1[b], s_hi); }
        mma_f16(acc_a, h0[0], h1[0], h0[1], h1[1], xh[4 * j + 0], xh[4 * j + 1]);
        mma_f16(acc_b, h0[2], h1[2], h0[3], h1[3], xh[4 * j + 2], xh[4 * j + 3]);
    }
}

// The same for static-E4M3 rows (one byte per weight, no block scales: the matrix scale and the
// activation scale multiply the finished sum): lane (g, t) takes 32 weights of rows g and g + 8
// of its span, converts them to f16 (exact) and feeds the same sixteen MMAs.
QD_DEVINL void unit_mma_fp8(const uint8_t* __restrict__ rows, int row_bytes, int span, int g, int t,
                            const uint32_t (&xh)[16], float (&acc_a)[4], float (&acc_b)[4]) {
    const uint8_t* c0 = rows + g * row_bytes + span * 128 + t * 32;
    const uint4 a0 = lds128(c0), a1 = lds128(c0 + 16), b0 = lds128(c0 + 8 * row_bytes), b1 = lds128(c0 + 8 * row_bytes + 16);
    const uint32_t r0[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t r1[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {        // four weights of either row per word: one MMA
        const uint32_t h0 = e4m3x2_to_f16x2((uint16_t)(r0[j] & 0xffffu)), h1 = e4m3x2_to_f16x2((uint16_t)(r0[j] >> 16));
        const uint32_t k0 = e4m3x2_to_f16x2((uint16_t)(r1[j] & 0xffffu)), k1 = e4m3x2_to_f16x2((uint16_t)(r1[j] >> 16));
        if (j & 1) mma_f16(acc_b, h0, k0, h1, k1, xh[2 * j], xh[2 * j + 1]);
        else mma_f16(acc_a, h0, k0, h1, k1, xh[2 * j], xh[2 * j + 1]);
    }
}

// A warp's partial sums of a tile of up to sixteen FP8 rows ([rows][K] bytes).
template <int K>
QD_DEVINL void tile_partials_fp8(const uint8_t* __restrict__ base, const uint32_t (&xh)[K / 2048][16], int warp, int lane,
                                 float* __restrict__ partial) {
    constexpr int UNITS = K / 2048;
    const int g = lane >> 2, t = lane & 3;
    float aa[4] = {0.f, 0.f, 0.f, 0.f}, ab[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < UNITS; ++u) unit_mma_fp8(base, K, row_span<UNITS>(warp, u, g), g, t, xh[u], aa, ab);
    if (t == (g >> 1)) {
        partial[g] = (g & 1) ? aa[1] + ab[1] : aa[0] + ab[0];
        partial[g + 8] = (g & 1) ? aa[3] + ab[3] : aa[2] + ab[2];
    }
}

// A warp's partial sums of one tile: K = 2048 -> up to two groups of sixteen rows, one span
// each; K = 4096 -> one group, two spans.  partial: this warp's kRowSlots floats.
template <int K>
QD_DEVINL void tile_partials(const uint8_t* __restrict__ base, int slots_in_tile, int groups,
                             const uint32_t (&xh)[K / 2048][16], int warp, int lane, float* __restrict__ partial) {
    constexpr int UNITS = K / 2048;
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* scales = base + slots_in_tile * (K / 2);
#pragma unroll 1
    for (int grp = 0; grp < groups; ++grp) {
        float aa[4] = {0.f, 0.f, 0.f, 0.f}, ab[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < UNITS; ++u)
            unit_mma(base, scales, K / 2, K / 16, grp * 16, row_span<UNITS>(warp, u, g), g, t, xh[u], aa, ab);
        if (t == (g >> 1)) {
            const float lo = (g & 1) ? aa[1] + ab[1] : aa[0] + ab[0];
            const float hi = (g & 1) ? aa[3] + ab[3] : aa[2] + ab[2];
            partial[grp * 16 + g] = lo;
            partial[grp * 16 + g + 8] = hi;
        }
    }
}

// Sum over the warps' partials for slot `lane` (fixed order).
QD_DEVINL float tile_sum(const float* __restrict__ partials, int lane) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kRowWarps; ++w) s += partials[w * kRowSlots + lane];
    return s;
}

}  // namespace qd
