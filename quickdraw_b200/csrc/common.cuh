// Shared device helpers for the sm_100a decode kernels.
//
// Number formats (reference: quickdraw/models/weights.py:14-26): an NVFP4 byte holds
// two E2M1 codes, low nibble = even input index; a block of 16 inputs shares one E4M3
// scale; one fp32 global scale multiplies the finished dot product.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quickdraw_b200.h"

typedef __nv_bfloat16 bf16;

#define QD_DEVINL __device__ __forceinline__

// Status word bits written by kernels (never trapped on; the host reads them).
#define QD_STATUS_WAIT_TIMEOUT 1u   // a bounded mbarrier/flag wait ran out
#define QD_STATUS_BAD_SHAPE 2u      // a kernel was asked for a shape it does not cover
#define QD_STATUS_BAD_ARG 4u        // a device-side argument (a position) was out of range; nothing was touched

// --------------------------------------------------------------------- conversions
QD_DEVINL float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
QD_DEVINL float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
QD_DEVINL float ld_bf16(const bf16* p) { return __bfloat162float(*p); }

// E2M1 code (4 bits) -> fp32, exact, sign bit kept for code 8 (-0).
QD_DEVINL float e2m1_to_float(uint32_t code) {
    const uint32_t m = code & 7u;
    const uint32_t mag = (m & 6u) ? ((((m >> 1) + 126u) << 23) | ((m & 1u) << 22))
                                  : ((m & 1u) ? 0x3F000000u : 0u);
    return __uint_as_float(mag | ((code & 8u) << 28));
}

// E4M3 (fn) byte -> fp32, exact (through the hardware fp8 -> f16 convert).
QD_DEVINL float e4m3_to_float(uint8_t code) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(code, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}

// two E4M3 bytes (low byte first) -> two fp32
QD_DEVINL float2 e4m3x2_to_float2(uint16_t pair) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// one NVFP4 byte -> f16x2 {low nibble, high nibble}; hardware convert on sm_100a.
QD_DEVINL uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t out;
    const uint16_t b = (uint16_t)byte;
    asm("{\n\t.reg .b8 lo, hi;\n\tmov.b16 {lo, hi}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, lo;\n\t}" : "=r"(out) : "h"(b));
    return out;
}
// four NVFP4 bytes (eight codes) of a 32-bit word -> four f16x2, byte 0 first.  The word is
// unpacked into its four bytes in ONE vector move (a two-level b32 -> b16 -> b8 unpack gave
// wrong bytes when inlined into a large kernel).
QD_DEVINL void e2m1x8_to_f16x2(uint32_t word, uint32_t (&out)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "r"(word));
}

// d = a(f16) * b(f16) + c(f32), one rounding, on the low / high halves of packed pairs.
QD_DEVINL float fma_f16_lo(uint32_t a2, uint32_t b2, float c) {
    float d;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %3;\n\t}" : "=f"(d) : "r"(a2), "r"(b2), "f"(c));
    return d;
}
QD_DEVINL float fma_f16_hi(uint32_t a2, uint32_t b2, float c) {
    float d;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.f16 %0, ah, bh, %3;\n\t}" : "=f"(d) : "r"(a2), "r"(b2), "f"(c));
    return d;
}
QD_DEVINL float fma_bf16_lo(uint32_t a2, uint32_t b2, float c) {
    float d;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %3;\n\t}" : "=f"(d) : "r"(a2), "r"(b2), "f"(c));
    return d;
}
QD_DEVINL float fma_bf16_hi(uint32_t a2, uint32_t b2, float c) {
    float d;
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, ah, bh, %3;\n\t}" : "=f"(d) : "r"(a2), "r"(b2), "f"(c));
    return d;
}

QD_DEVINL float sigmoidf_(float v) { return 1.0f / (1.0f + __expf(-v)); }
QD_DEVINL float sigmoid_precise(float v) { return 1.0f / (1.0f + expf(-v)); }
QD_DEVINL float silu_precise(float v) { return v / (1.0f + expf(-v)); }
// softplus with the identity above 20, as torch computes it.
QD_DEVINL float softplus_precise(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// -------------------------------------------------------------------- warp reduce
QD_DEVINL float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
QD_DEVINL float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int WIDTH>
QD_DEVINL float group_sum(float v) {   // butterfly over aligned groups of WIDTH lanes
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------ shared memory / mbarrier / TMA
QD_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

QD_DEVINL void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
QD_DEVINL void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
QD_DEVINL void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
QD_DEVINL void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
QD_DEVINL bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after QD_WAIT_LIMIT_NS of wall time, records the failure in
// *status and returns false so the caller can leave the kernel instead of spinning for ever.
// The polling loops stay rolled: unrolled, every poll would run through fresh code.
#define QD_WAIT_LIMIT_NS 200000000ull   /* 0.2 s of wall time */
QD_DEVINL unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, unsigned int* status) {
    const unsigned long long start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - start > QD_WAIT_LIMIT_NS) break;
    }
    if (status) atomicOr(status, QD_STATUS_WAIT_TIMEOUT);
    return false;
}
// The usual case (the barrier completes within a few polls) stays inline, so that no
// registers are saved around a call in the row loops.
QD_DEVINL bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, status);
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
QD_DEVINL void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
QD_DEVINL void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Programmatic dependent launch: a kernel may start before its predecessor in the
// stream has finished; everything that reads the predecessor's output, and every
// global write, comes after grid_dependency_wait().
QD_DEVINL void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
QD_DEVINL void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// First statement of a kernel that is launched as a programmatic dependent (qd_launch with pdl = true):
// the next kernel of the stream may be scheduled behind this one's blocks, then the kernel waits until
// the one before it has finished and its writes are visible.  Before this call a kernel must not touch
// anything another kernel of the stream writes; in an ordinary launch both instructions do nothing.
QD_DEVINL void chain_enter() { grid_launch_dependents(); grid_dependency_wait(); }

QD_DEVINL uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// ------------------------------------------------------------------------ host side
#define QD_CHECK_ARG(cond) do { if (!(cond)) return QD_ERR_ARG; } while (0)
static inline int qd_launch_status() { return cudaGetLastError() == cudaSuccess ? QD_OK : QD_ERR_LAUNCH; }

// Whether kernels that open with chain_enter() are launched as programmatic dependents (qd_set_chained_launches).
inline int& qd_chain_switch() { static int on = 1; return on; }

// Launch helper that optionally marks the kernel as a programmatic dependent of the previous one in
// the stream.  pdl: 0 = ordinary launch, 1 = dependent unless chained launches are switched off,
// 2 = always dependent (a kernel that fetches weights before its wait).
template <typename... KArgs, typename... Args>
static inline int qd_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, int pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (pdl == 2 || (pdl == 1 && qd_chain_switch())) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? QD_OK : QD_ERR_LAUNCH;
}
