// tcgen05 helpers for the block-scaled NVFP4 product (kind::mxf4nvf4): tensor memory,
// shared-memory matrix descriptors, the MMA itself, tiled TMA loads.
//
// How one activation vector meets the FP4 tensor core exactly: the MMA wants both operands as
// E2M1 with a UE4M3 scale per sixteen inputs.  The weights already are (codes and block
// scales straight from the checkpoint layout, no unpacking anywhere).  The activation vector x
// (bf16) is written as a 32-bit fixed-point number relative to its largest magnitude,
// |x| = t * 2^(E - 32) with |x| < 2^E (exact for every element within 2^-24 of the largest),
// and t is cut into sixteen 2-bit digits, most significant first; digit d with the sign of x is
// exactly the E2M1 code of +-d/2, so digit plane p becomes column p of the B operand, with the
// block scale 2^(8 - 2 (p mod 8)) for every block.  Columns 0..7 add up to the contribution of
// the upper sixteen bits, columns 8..15 to that of the lower sixteen times 2^16; together
// (c_hi + c_lo * 2^-16) * 2^(E - 9) = sum_k w_k s_k x_k with exact weights, exact activations
// and fp32 accumulation in tensor memory.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace qd {

QD_DEVINL void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
QD_DEVINL void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
QD_DEVINL void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
QD_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
QD_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
QD_DEVINL void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
QD_DEVINL void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
QD_DEVINL void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 128 rows x 16 columns x 64 inputs, both operands E2M1 from shared memory, one UE4M3 scale per
// sixteen inputs from tensor memory, fp32 accumulator in tensor memory.
QD_DEVINL void umma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                          uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate) : "memory");
}
// The same with the descriptors as halves: the upper 32 bits are the same for every tile of this
// layout (kDescHiSw128), the lower hold the start address, so a K step is an add of 2.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
QD_DEVINL uint32_t desc_lo_sw128(uint32_t addr) { return ((addr >> 4) & 0x3fffu) | (1u << 16); }
QD_DEVINL void umma_nvfp4_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa_tmem,
                             uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %7, 0;\n\t"
                 "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [%5], [%6], p;\n\t}"
                 ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem),
                   "r"(accumulate) : "memory");
}
// Instruction descriptor of that MMA: E2M1 A and B (format 1 at bits [7,10) and [10,13)), both
// K-major, N >> 3 at [17,23), UE4M3 scales (bit 23 = 0), M >> 4 at [24,29), scale-factor ids 0,
// K = 64.
constexpr uint32_t kUmmaNvfp4Desc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
constexpr int kPlanes = 16;                  // digit planes = columns of the B operand
constexpr int kPlaneChunkBytes = 2048;       // 16 plane rows x 128 bytes per 256 inputs

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes (256 FP4
// inputs), the 16-byte pieces of a row XOR-ed with the row index inside every 1024-byte group
// of 8 rows; the tile starts on a 1024-byte boundary.  Bits: [0,14) address >> 4, [16,30)
// leading byte offset >> 4 (unused here), [32,46) bytes between 8-row groups >> 4, [46,48)
// descriptor version 1, [61,64) layout type 2.  A K step of 64 inputs advances the start
// address by 32 bytes inside the row.
QD_DEVINL uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Tiled 2-D TMA load global -> shared; c0 = innermost coordinate (bytes here: the maps are over
// uint8, so c0 must be a multiple of 16), c1 = row.  Completion is counted in bytes on the mbarrier.
QD_DEVINL void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
QD_DEVINL void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// sixteen 32-bit columns of this warp's 32 lanes of tensor memory from registers
QD_DEVINL void tmem_store16(uint32_t addr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
QD_DEVINL void tmem_store1(uint32_t addr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(addr), "r"(v) : "memory");
}
// eight columns (fp32 bits) of this warp's 32 lanes
QD_DEVINL void tmem_load8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr) : "memory");
}

// sixteen columns (fp32 bits) of this warp's 32 lanes
QD_DEVINL void tmem_load16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(addr) : "memory");
}
// The sixteen result columns of a row -> the dot product before the vector's scale.
QD_DEVINL float plane_sum(const uint32_t (&v)[16]) {
    float hi = 0.f, lo = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) { hi += __uint_as_float(v[q]); lo += __uint_as_float(v[8 + q]); }
    return hi + lo * 1.52587890625e-05f;       // 2^-16
}

// ---- activation digit planes --------------------------------------------------------------
// Exponent E with |x| < 2^E for a vector whose largest magnitude is at most `top` (a float
// bound; zero and non-finite bounds give a harmless value).
QD_DEVINL int plane_exponent_of(float top) {
    const int e = (int)((__float_as_uint(top) >> 23) & 0xffu) - 127 + 1;
    return max(-90, min(e, 120));
}
// The factor that turns plane_sum into the dot product.
QD_DEVINL float plane_out_scale(int E) { return exp2f((float)(E - 9)); }
// UE4M3 block scale of plane p: 2^(8 - 2 (p mod 8)), four copies (one per block of sixteen
// inputs of a 64-input MMA step).
QD_DEVINL uint32_t plane_scale_word(int p) { return (uint32_t)((15 - 2 * (p & 7)) << 3) * 0x01010101u; }

// Four consecutive activations (floats holding bf16 values) -> eight 32-bit words: the low half
// of word p holds the E2M1 codes of digit plane 8 + p, the high half those of plane p (element j
// in nibble j).  Digit p of the upper and of the lower sixteen bits of t sit sixteen bits apart,
// so one shift and one mask move both.
QD_DEVINL void plane_pairs(const float (&x)[4], int E, uint32_t (&pairs)[8]) {
    const float up = exp2f((float)(32 - E));
    uint32_t t[4], sg = 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        t[j] = __float2uint_rz(fabsf(x[j]) * up);       // saturates; exact for bf16 inputs below 2^E
        sg |= (__float_as_uint(x[j]) >> 31) << (4 * j + 3);
    }
    sg |= sg << 16;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        uint32_t w = sg;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int shift = 14 - 2 * p - 4 * j;            // digit p of both halves to nibble j of both halves
            const uint32_t moved = shift >= 0 ? (t[j] >> shift) : (t[j] << -shift);
            w |= moved & (0x00030003u << (4 * j));
        }
        pairs[p] = w;
    }
}
// Byte offset of the 16-byte piece (plane row p, piece c of the 128-byte row) inside the
// 2048-byte block of one 256-input chunk of the B operand (two swizzled groups of 8 rows).
QD_DEVINL uint32_t plane_piece_offset(int p, int c) { return (uint32_t)(p * 128 + ((c ^ (p & 7)) << 4)); }
// The sixteen 16-bit plane words of four consecutive inputs starting at input `first` into the B operand.
QD_DEVINL void store_planes4(uint8_t* planes, int first, const float (&v)[4], int E) {
    uint32_t pw[8];
    plane_pairs(v, E, pw);
    uint8_t* dst = planes + (first >> 8) * kPlaneChunkBytes + ((first & 31) >> 1);
    const int piece = (first & 255) >> 5;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        *reinterpret_cast<unsigned short*>(dst + plane_piece_offset(q, piece)) = (unsigned short)(pw[q] >> 16);
        *reinterpret_cast<unsigned short*>(dst + plane_piece_offset(q + 8, piece)) = (unsigned short)pw[q];
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point table.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn umma_encode_fn();
// Map over a row-major uint8 matrix [rows][row_bytes] with a box of box_rows x box_bytes
// (box_bytes <= 128), 128-byte swizzle.  QD_* code.
int umma_make_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows);

}  // namespace qd
