// Row-level device helpers shared by the streaming matvec kernel and the persistent decode
// kernel: the byte-cost partition of a segment list, the NVFP4 / bf16 row dot products with
// the activation slice in registers, and the top-k routing of one warp.
#pragma once
#include "stream.cuh"

namespace qd {

// Costs are counted in units of 16 bytes so that a whole launch fits 32-bit arithmetic.
template <int K> QD_DEVINL int seg_cost(int kind) {
    constexpr int fp4_row = (K / 2 + K / 16) / 16;
    return kind == SEG_BF16 ? 2 * K / 16 : kind == SEG_FP8 ? K / 16 : (kind == SEG_FP4_PAIR ? 2 * fp4_row : fp4_row);
}
// Rows of one ring stage; FP8 rows go sixteen (2048 inputs) or eight (4096) at a time: one group
// of the row engine.
template <int K> QD_DEVINL int seg_tile_rows(int kind) {
    return kind == SEG_FP8 ? (K == 2048 ? 16 : 8) : (kStreamStageBytes / 16) / seg_cost<K>(kind);
}
template <int K> QD_DEVINL unsigned ceil_div_cost(unsigned v, int kind) {   // constant divisors only
    constexpr unsigned fp4_row = (K / 2 + K / 16) / 16;
    return kind == SEG_BF16 ? (v + 2 * K / 16 - 1) / (2 * K / 16)
         : kind == SEG_FP8 ? (v + K / 16 - 1) / (K / 16)
         : kind == SEG_FP4_PAIR ? (v + 2 * fp4_row - 1) / (2 * fp4_row) : (v + fp4_row - 1) / fp4_row;
}
// Row range [ra, rb) of a segment that falls into the block's cost range [lo, hi).
template <int K> QD_DEVINL void seg_range(unsigned seg_start, int kind, int rows, unsigned lo, unsigned hi,
                                          int& ra, int& rb) {
    const unsigned fa = lo <= seg_start ? 0u : ceil_div_cost<K>(lo - seg_start, kind);
    const unsigned fb = hi <= seg_start ? 0u : ceil_div_cost<K>(hi - seg_start, kind);
    ra = (int)min(fa, (unsigned)rows);
    rb = (int)min(fb, (unsigned)rows);
}

QD_DEVINL uint32_t max_u16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
QD_DEVINL uint32_t pack_f16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

template <int KC>
QD_DEVINL float fp4_row_dot(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                            const uint32_t (&xh)[KC][16], int lane) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        const uint4 w = lds128(codes + (c * 32 + lane) * 16);
        const float2 s = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(scales + (c * 32 + lane) * 2));
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
        float g[4] = {0.f, 0.f, 0.f, 0.f};   // two chains per 16-input group
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t h2[4];
            e2m1x8_to_f16x2(words[q], h2);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t xv = xh[c][q * 4 + b];
                g[(q >> 1) * 2] = fma_f16_lo(h2[b], xv, g[(q >> 1) * 2]);
                g[(q >> 1) * 2 + 1] = fma_f16_hi(h2[b], xv, g[(q >> 1) * 2 + 1]);
            }
        }
        acc = fmaf(s.x, g[0] + g[1], acc);
        acc = fmaf(s.y, g[2] + g[3], acc);
    }
    return acc;
}

template <int NB>   // NB = K / 256 sixteen-byte chunks per lane
QD_DEVINL float bf16_row_dot(const uint8_t* __restrict__ row, const uint32_t (&xb)[NB * 4], int lane) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const uint4 w = lds128(row + (i * 32 + lane) * 16);
        a0 = fma_bf16_lo(w.x, xb[i * 4 + 0], a0); a1 = fma_bf16_hi(w.x, xb[i * 4 + 0], a1);
        a0 = fma_bf16_lo(w.y, xb[i * 4 + 1], a0); a1 = fma_bf16_hi(w.y, xb[i * 4 + 1], a1);
        a0 = fma_bf16_lo(w.z, xb[i * 4 + 2], a0); a1 = fma_bf16_hi(w.z, xb[i * 4 + 2], a1);
        a0 = fma_bf16_lo(w.w, xb[i * 4 + 3], a0); a1 = fma_bf16_hi(w.w, xb[i * 4 + 3], a1);
    }
    return a0 + a1;
}

// The same dot products with the activation slice fetched from shared memory as it is used
// (no register copy): for blocks that only see a few rows of a kind.  xf_t is the f16 vector
// in the transposed layout where the piece of (chunk c, quarter q, lane) sits at
// ((c * 4 + q) * 32 + lane) * 16 bytes; xs is the bf16 vector in natural order.
template <int KC>
QD_DEVINL float fp4_row_dot_smem(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                 const uint8_t* __restrict__ xf_t, int lane) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        const uint4 w = lds128(codes + (c * 32 + lane) * 16);
        const float2 s = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(scales + (c * 32 + lane) * 2));
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
        float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t h2[4];
            e2m1x8_to_f16x2(words[q], h2);
            const uint4 xq = lds128(xf_t + ((c * 4 + q) * 32 + lane) * 16);
            const uint32_t xv[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                g[(q >> 1) * 2] = fma_f16_lo(h2[b], xv[b], g[(q >> 1) * 2]);
                g[(q >> 1) * 2 + 1] = fma_f16_hi(h2[b], xv[b], g[(q >> 1) * 2 + 1]);
            }
        }
        acc = fmaf(s.x, g[0] + g[1], acc);
        acc = fmaf(s.y, g[2] + g[3], acc);
    }
    return acc;
}

template <int NB>
QD_DEVINL float bf16_row_dot_smem(const uint8_t* __restrict__ row, const uint8_t* __restrict__ xs, int lane) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const uint4 w = lds128(row + (i * 32 + lane) * 16);
        const uint4 x = lds128(xs + (i * 32 + lane) * 16);
        a0 = fma_bf16_lo(w.x, x.x, a0); a1 = fma_bf16_hi(w.x, x.x, a1);
        a0 = fma_bf16_lo(w.y, x.y, a0); a1 = fma_bf16_hi(w.y, x.y, a1);
        a0 = fma_bf16_lo(w.z, x.z, a0); a1 = fma_bf16_hi(w.z, x.z, a1);
        a0 = fma_bf16_lo(w.w, x.w, a0); a1 = fma_bf16_hi(w.w, x.w, a1);
    }
    return a0 + a1;
}

// top-k routing by one warp over at most 256 bf16 logits in global memory (written by other
// blocks of this launch, hence the cache-global loads): fp32 softmax, lowest index wins
// ties, weights renormalised (quickdraw/models/qwen.py:174-177).
QD_DEVINL void route_small(const bf16* logits, int experts, int topk, int32_t* ids, float* weights, int lane) {
    float p[8];
    float best = -INFINITY;
    const unsigned short* raw = reinterpret_cast<const unsigned short*>(logits);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = i * 32 + lane;
        p[i] = e < experts ? __uint_as_float((uint32_t)__ldcg(raw + e) << 16) : -INFINITY;
        best = fmaxf(best, p[i]);
    }
    best = warp_max(best);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = i * 32 + lane;
        p[i] = e < experts ? expf(p[i] - best) : -1.f;
        if (e < experts) sum += p[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < 8; ++i) if (p[i] >= 0.f) p[i] = p[i] / sum;
    float chosen = 0.f, mine = 0.f;
    int my_id = 0;
    for (int s = 0; s < topk; ++s) {
        float v = -1.f; int idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i) if (p[i] > v) { v = p[i]; idx = i * 32 + lane; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        chosen += v;
        if (lane == s) { mine = v; my_id = idx; }
        if ((idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (i == (idx >> 5)) p[i] = -1.f;
        }
    }
    if (lane < topk) { ids[lane] = my_id; weights[lane] = mine / chosen; }
}

}  // namespace qd
