// Static-FP8 projection of a chunk of tokens: y[t] = W q(x[t]) for an E4M3 matrix with scalar
// weight and activation scales (FP8Linear: quickdraw/models/weights.py:58-74; arithmetic of
// fp8_gemv, quickdraw/models/qwen.py:25-33: q(x) = e4m3(clamp(x / input_scale, +-448)), products
// exact, fp32 sum, both scales on the sum, one bf16 rounding).  The one-launch step takes such
// mixers token by token; this is the form for prompt chunks and decode batches.
//
//   quantiser   x bf16 [tokens, K] -> E4M3 bytes [tokens, K] (round to nearest even, saturating)
//   product     block = 128 tokens x 128 weight rows, eight warps of 64 x 32; both operands go
//               through a four-stage cp.async ring in chunks of 128 inputs (rows padded to 192
//               bytes: the 16-byte fragment loads of a quarter-warp fall on different banks) and
//               meet on mma.sync.m16n8k32 (e4m3 x e4m3, fp32 accumulators) with the tokens as
//               rows, so that a lane's two results are neighbouring outputs of one token.
#include "common.cuh"

namespace qd {
namespace {

constexpr int kF8Tile = 128, kF8Chunk = 128, kF8Row = kF8Chunk + 64, kF8Stages = 4, kF8Threads = 256;
constexpr int kF8StageBytes = 2 * kF8Tile * kF8Row;
constexpr size_t kF8Smem = (size_t)kF8Stages * kF8StageBytes;

__global__ void __launch_bounds__(256) fp8_quantize_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ in_scale,
                                                                uint2* __restrict__ q, long long n8) {
    chain_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float s = *in_scale;
    const uint4 v = x[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = __nv_cvt_float_to_fp8(__fdiv_rn(__uint_as_float(w[k] << 16), s), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float_to_fp8(__fdiv_rn(__uint_as_float(w[k] & 0xffff0000u), s), __NV_SATFINITE, __NV_E4M3);
        out[k >> 1] |= (lo | (hi << 8)) << (16 * (k & 1));
    }
    q[i] = make_uint2(out[0], out[1]);
}

QD_DEVINL void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
QD_DEVINL void f8_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kF8Threads, 1)
fp8_gemm_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ w, const float* __restrict__ w_scale,
                const float* __restrict__ in_scale, bf16* __restrict__ y, int tokens, int rows, int K) {
    chain_enter();
    extern __shared__ __align__(128) uint8_t f8_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int t0 = blockIdx.y * kF8Tile, r0 = blockIdx.x * kF8Tile;
    const int m0 = (warp & 1) * 64, n0 = (warp >> 1) * 32;          // the warp's 64 tokens x 32 rows of the tile
    const int chunks = K / kF8Chunk;
    // rows past the ends read the last valid row and are not stored
    auto issue = [&](int c) {
        uint8_t* st = f8_smem + (size_t)(c % kF8Stages) * kF8StageBytes;
#pragma unroll
        for (int i = 0; i < 2 * kF8Tile * 8 / kF8Threads; ++i) {
            const int piece = tid + i * kF8Threads, which = piece >> 10, row = (piece >> 3) & (kF8Tile - 1), col = piece & 7;
            const uint8_t* src = which ? w + (size_t)min(r0 + row, rows - 1) * K : q + (size_t)min(t0 + row, tokens - 1) * K;
            f8_cp16(st + (size_t)(which * kF8Tile + row) * kF8Row + col * 16, src + (size_t)c * kF8Chunk + col * 16);
        }
    };
#pragma unroll
    for (int c = 0; c < kF8Stages - 1; ++c) {
        if (c < chunks) issue(c);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[4][4][4];
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mi][ni][c] = 0.f;
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group 2;" ::: "memory");       // kF8Stages - 2 younger chunks may be in flight
        __syncthreads();                                           // chunk c is everybody's; chunk c - 1 is consumed
        if (c + kF8Stages - 1 < chunks) issue(c + kF8Stages - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const uint8_t* xa = f8_smem + (size_t)(c % kF8Stages) * kF8StageBytes;
        const uint8_t* wb = xa + (size_t)kF8Tile * kF8Row;
#pragma unroll
        for (int kk = 0; kk < kF8Chunk / 64; ++kk) {
            // lane (g, t) supplies bytes 16 t .. 16 t + 15 of every 64 on both sides: two MMAs per 16-byte load
            uint4 bw[4];
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) bw[ni] = lds128(wb + (size_t)(n0 + 8 * ni + g) * kF8Row + kk * 64 + t * 16);
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const uint4 lo = lds128(xa + (size_t)(m0 + 16 * mi + g) * kF8Row + kk * 64 + t * 16);
                const uint4 hi = lds128(xa + (size_t)(m0 + 16 * mi + g + 8) * kF8Row + kk * 64 + t * 16);
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    mma_e4m3(acc[mi][ni], lo.x, hi.x, lo.y, hi.y, bw[ni].x, bw[ni].y);
                    mma_e4m3(acc[mi][ni], lo.z, hi.z, lo.w, hi.w, bw[ni].z, bw[ni].w);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // acc[mi][ni][0..1] = token m0 + 16 mi + g, rows n0 + 8 ni + 2 t and + 1; [2..3] = token + 8
    const float s_in = *in_scale, s_w = *w_scale;
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int token = t0 + m0 + 16 * mi + g + 8 * half;
            if (token >= tokens) continue;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const int row = r0 + n0 + 8 * ni + 2 * t;
                if (row + 1 < rows)
                    *reinterpret_cast<__nv_bfloat162*>(y + (size_t)token * rows + row) =
                        __floats2bfloat162_rn((acc[mi][ni][2 * half] * s_in) * s_w, (acc[mi][ni][2 * half + 1] * s_in) * s_w);
                else if (row < rows)
                    y[(size_t)token * rows + row] = __float2bfloat16_rn((acc[mi][ni][2 * half] * s_in) * s_w);
            }
        }
}

}  // namespace
}  // namespace qd

// y [tokens, out_features] = q(x) W^T for a static-FP8 projection (see above).  q_scratch: tokens *
// in_features bytes, 16-byte aligned, receives the quantised rows; convert = 0 reuses what the
// previous call left there (projections that share input and input scale).  in_features a multiple
// of 128, out_features even; QD_ERR_UNSUPPORTED otherwise.
extern "C" int qd_fp8_matmul(const void* x, const void* w, const float* w_scale, const float* in_scale, void* y,
                             int tokens, int out_features, int in_features, void* q_scratch, int convert, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x && w && w_scale && in_scale && y && q_scratch && tokens > 0 && out_features > 0 && in_features > 0);
    if (in_features % kF8Chunk != 0 || out_features % 2 != 0 || (tokens + kF8Tile - 1) / kF8Tile > 65535) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)q_scratch) & 15u || ((uintptr_t)y & 3u)) return QD_ERR_UNSUPPORTED;
    if (convert) {
        const long long n8 = (long long)tokens * in_features / 8;
        qd_launch(fp8_quantize_rows_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, true, 
            (const uint4*)x, in_scale, (uint2*)q_scratch, n8);
        if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kF8Smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    const dim3 grid((unsigned)((out_features + kF8Tile - 1) / kF8Tile), (unsigned)((tokens + kF8Tile - 1) / kF8Tile));
    qd_launch(fp8_gemm_kernel, dim3(grid), dim3(kF8Threads), kF8Smem, (cudaStream_t)stream, true, 
        (const uint8_t*)q_scratch, (const uint8_t*)w, w_scale, in_scale, (bf16*)y, tokens, out_features, in_features);
    return qd_launch_status();
}
