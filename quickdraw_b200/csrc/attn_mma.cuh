// Tensor-core (mma.sync m16n8k16, bf16) attention of up to eight query heads that share one KV
// head against sixteen cached positions at a time, with a running softmax in MMA fragment
// layout.  Shared by the attention phase of the persistent decode kernel (mega.cu) and the
// causal attention of the chunked prefill (seq.cu).
//
// Shared-memory layouts the chunk routine reads: query heads bf16 [8][kAttnQRow bytes] (heads
// beyond the group zeroed), key rows and value rows bf16 [positions][kAttnRow bytes]; both row
// strides are 512 bytes plus padding, so that the eight rows a quarter-warp touches fall into
// different banks.
#pragma once
#include "common.cuh"

namespace qd {

constexpr int kAttnRow = 528;                  // a 512-byte cache row of one KV head, padded against bank conflicts
constexpr int kAttnQRow = 576;                 // a query head in shared memory (bf16 [256], padded)

QD_DEVINL void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
QD_DEVINL uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

// Running state of one warp's share of the context, in MMA fragment layout.  Lane (g, t):
// softmax statistics of query head g; out[i][c]: feature 32 g + 2 i + (c >> 1) of head 2 t + (c & 1).
struct AttnAcc {
    float m, l;
    float out[16][4];
};

// Key row behind column g of a score tile (rows prow and 8 + prow of the chunk are lane (g, t)'s).
QD_DEVINL int attn_key_row(int g) { return (g & 1) ? 4 + (g >> 1) : (g >> 1); }

// Scores: 64 bytes of the query heads against the same bytes of the lane's two key rows.
QD_DEVINL void attn_score_step(float (&s0)[4], float (&s1)[4], const uint4& q4, const uint4& k0, const uint4& k1) {
    mma_bf16(s0, q4.x, 0u, q4.y, 0u, k0.x, k0.y);
    mma_bf16(s0, q4.z, 0u, q4.w, 0u, k0.z, k0.w);
    mma_bf16(s1, q4.x, 0u, q4.y, 0u, k1.x, k1.y);
    mma_bf16(s1, q4.z, 0u, q4.w, 0u, k1.z, k1.w);
}

// Probabilities of a chunk as the B operand of the value product, split into two bf16 pieces
// (sixteen bits of mantissa).
struct AttnProbs { uint32_t hi0, hi1, lo0, lo1; };

// Running softmax over the chunk's scores; rescales the accumulator.  first: context position of
// row 0 of the chunk; t1: end of the range (rows at or past it are masked).
QD_DEVINL AttnProbs attn_softmax(AttnAcc& acc, const float (&s0)[4], const float (&s1)[4], int first, int t1, int lane) {
    const int t = lane & 3;
    // the lane's four scores of head g: rows t, 4 + t, 8 + t, 12 + t of the chunk
    float sc[4] = {s0[0], s0[1], s1[0], s1[1]};
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sc[i] = (first + 4 * i + t < t1) ? sc[i] * 0.0625f : -INFINITY;      // 1 / sqrt(256)
        mx = fmaxf(mx, sc[i]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(acc.m, mx);
    const float alpha = acc.m == -INFINITY ? 0.f : expf(acc.m - m_new);
    float p[4], psum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { p[i] = sc[i] == -INFINITY ? 0.f : expf(sc[i] - m_new); psum += p[i]; }
    acc.l = acc.l * alpha + psum;
    acc.m = m_new;
    AttnProbs pr;
    pr.hi0 = pack_bf16x2(p[0], p[1]); pr.hi1 = pack_bf16x2(p[2], p[3]);
    pr.lo0 = pack_bf16x2(p[0] - __uint_as_float(pr.hi0 << 16), p[1] - __uint_as_float(pr.hi0 & 0xffff0000u));
    pr.lo1 = pack_bf16x2(p[2] - __uint_as_float(pr.hi1 << 16), p[3] - __uint_as_float(pr.hi1 & 0xffff0000u));
    const float a_even = __shfl_sync(0xffffffffu, alpha, 8 * t), a_odd = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc.out[i][0] *= a_even; acc.out[i][1] *= a_odd; acc.out[i][2] *= a_even; acc.out[i][3] *= a_odd;
    }
    return pr;
}

// Values: bytes 64 g + 16 q .. + 15 of the value rows t, 4 + t, 8 + t, 12 + t of the chunk.
// TWO_PIECES = false: the probabilities as one bf16 piece (eight bits of mantissa), half the MMAs: the
// form for long prompt chunks, where the value product is most of the arithmetic.
template <bool TWO_PIECES = true>
QD_DEVINL void attn_value_step(AttnAcc& acc, int q, const uint4& r0, const uint4& r1, const uint4& r2, const uint4& r3,
                               const AttnProbs& pr) {
    const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w}, w1[4] = {r1.x, r1.y, r1.z, r1.w};
    const uint32_t w2[4] = {r2.x, r2.y, r2.z, r2.w}, w3[4] = {r3.x, r3.y, r3.z, r3.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const uint32_t a0 = __byte_perm(w0[e], w1[e], 0x5410), a1 = __byte_perm(w0[e], w1[e], 0x7632);
        const uint32_t a2 = __byte_perm(w2[e], w3[e], 0x5410), a3 = __byte_perm(w2[e], w3[e], 0x7632);
        mma_bf16(acc.out[q * 4 + e], a0, a1, a2, a3, pr.hi0, pr.hi1);
        if (TWO_PIECES) mma_bf16(acc.out[q * 4 + e], a0, a1, a2, a3, pr.lo0, pr.lo1);
    }
}

// Sixteen positions of the context against the (up to) eight query heads of a KV head.
// krows / vrows: the chunk's key and value rows in shared memory (kAttnRow bytes apart);
// first: context position of row 0; t1: end of the block's split.
template <bool TWO_PIECES = true>
QD_DEVINL void attn_chunk(AttnAcc& acc, const uint8_t* __restrict__ q_s, const uint8_t* __restrict__ krows,
                          const uint8_t* __restrict__ vrows, int first, int t1, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int prow = attn_key_row(g);
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const uint4 q4 = lds128(q_s + g * kAttnQRow + m * 64 + t * 16);
        const uint4 k0 = lds128(krows + prow * kAttnRow + m * 64 + t * 16);
        const uint4 k1 = lds128(krows + (8 + prow) * kAttnRow + m * 64 + t * 16);
        attn_score_step(s0, s1, q4, k0, k1);
    }
    const AttnProbs pr = attn_softmax(acc, s0, s1, first, t1, lane);
    const uint8_t* vb = vrows + g * 64;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint4 r0 = lds128(vb + t * kAttnRow + q * 16);
        const uint4 r1 = lds128(vb + (4 + t) * kAttnRow + q * 16);
        const uint4 r2 = lds128(vb + (8 + t) * kAttnRow + q * 16);
        const uint4 r3 = lds128(vb + (12 + t) * kAttnRow + q * 16);
        attn_value_step<TWO_PIECES>(acc, q, r0, r1, r2, r3, pr);
    }
}

}  // namespace qd
