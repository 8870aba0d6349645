// Block-scaled FP4 x FP4 product on the 5th generation tensor cores (tcgen05.mma
// kind::mxf4nvf4, scale_vec::4X): Y[T, N] = X[T, K] . W[N, K]^T with BOTH operands NVFP4, and
// the activation quantiser that produces X in that format.
//
// The reference multiplies bf16 activations with dequantised NVFP4 weights
// (quickdraw/kernel/triton/matvec.py:118-163); its notes (todo.md:13) name "W4A4 activation
// quantisation" as the step to validate separately from that W4A16 path.  This file is that
// step: qd_nvfp4_quantize_act writes the activations of a chunk of tokens as E2M1 codes, one
// E4M3 scale per sixteen inputs and one fp32 scale per tensor (the weight format of
// quickdraw/models/weights.py:29-47, so the same container describes both operands), and
// qd_nvfp4_matmul_w4a4 multiplies the two without expanding anything: codes travel HBM -> shared
// memory as tiled TMA loads in the layout the MMA reads, block scales travel the same way and
// are moved into tensor memory, the accumulator lives in tensor memory.  The result differs from
// the W4A16 product by the activation rounding only; the exact path stays qd_nvfp4_matmul.
//
// Tile: 128 tokens x 128 weight rows per block, K in stages of 256 inputs (a 128-byte row of
// codes, sixteen scales).  Two blocks share an SM (3 stages of 36 KB and 256 columns of tensor
// memory each), so one block's epilogue overlaps the other's K loop.
//   warp 0      TMA: per stage four boxes (codes and scales of both operands)
//   warp 1      allocates tensor memory, issues 4 MMAs of 128 x 128 x 64 per stage
//   warps 2..5  move the stage's block scales shared memory -> tensor memory (every warp fills
//               its own 32-lane quarter), then run the epilogue: one token per lane
// Every wait is bounded; a wait that runs out sets the status word and the block leaves.
#include <algorithm>

#include "umma.cuh"

namespace qd {
namespace {

constexpr int kTile = 128;                    // tokens per block (tensor-memory lanes)
// Weight rows per block = columns of one MMA: template parameter TN.  128: 3 stages of 36 KB and
// 256 tensor-memory columns, two blocks per SM.  256: 4 stages of 54 KB, all 512 columns, one block
// per SM; a block-scaled MMA takes the same 152 clocks for 256 columns as for 128.
constexpr int stages_of(int tn) { return tn == 128 ? 3 : 4; }
constexpr int kCodeBytes = kTile * 128;       // 128 rows x 256 inputs
constexpr int kScaleBytes = kTile * 16;       // 128 rows x 16 scales
constexpr int stage_bytes(int tn) { return (1 + tn / 128) * (kCodeBytes + kScaleBytes); }      // 36 / 54 KB
constexpr int kThreads4 = 6 * 32;
constexpr uint32_t tmem_cols(int tn) { return tn == 128 ? 256u : 512u; }
constexpr uint32_t kColAcc = 0;
// scale columns of a stage: 16 for the 128 tokens (four per 64-input step: rows l, l + 32, l + 64,
// l + 96 of lane l), then four per step and 128 weight rows
constexpr uint32_t sf_cols(int tn) { return 16u + 16u * (tn / 128); }
constexpr uint32_t desc_of(int tn) { return (1u << 7) | (1u << 10) | (((uint32_t)tn >> 3) << 17) | ((128u >> 4) << 24); }

struct Gemm4Params {
    const float* x_global; const float* w_global; bf16* y;
    int tokens, out_features, in_features;
    unsigned int* status;
};

struct Bars4 { uint64_t full[4], empty[4], sf_ready[4], done; };

template <int TN>
__global__ void __launch_bounds__(kThreads4, TN == 128 ? 2 : 1)
nvfp4_gemm_w4a4_kernel(const __grid_constant__ Gemm4Params p, const __grid_constant__ CUtensorMap x_codes,
                       const __grid_constant__ CUtensorMap x_scales, const __grid_constant__ CUtensorMap w_codes,
                       const __grid_constant__ CUtensorMap w_scales) {
    extern __shared__ __align__(1024) uint8_t gemm4_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm4_smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kStages4 = stages_of(TN), kStage4Bytes = stage_bytes(TN), kHalves = TN / 128;
    constexpr uint32_t kCols4 = tmem_cols(TN), kColSf = TN, kSfCols = sf_cols(TN);
    Bars4* bars = reinterpret_cast<Bars4*>(smem + kStages4 * kStage4Bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.y * kTile, n0 = blockIdx.x * TN;
    const int chunks = p.in_features / 256;

    if (tid == 0) {
        for (int s = 0; s < kStages4; ++s) { mbar_init(bars->full + s, 1); mbar_init(bars->empty + s, 1); mbar_init(bars->sf_ready + s, 4); }
        mbar_init(&bars->done, 1);
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, kCols4); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    auto stage = [&](int st) { return smem + (size_t)st * kStage4Bytes; };

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_map(&x_codes); tma_prefetch_map(&x_scales); tma_prefetch_map(&w_codes); tma_prefetch_map(&w_scales);
            for (int c = 0; c < chunks; ++c) {
                const int st = c % kStages4;
                if (!mbar_wait(bars->empty + st, ((c / kStages4) & 1) ^ 1, p.status)) break;
                // rows past the end of a matrix arrive as zeros; a box always counts in full
                mbar_expect_tx(bars->full + st, kStage4Bytes);
                uint8_t* base = stage(st);
                // codes: tokens, then the weight rows (128 at a time); scales in the same order
                uint8_t* sc = base + (1 + kHalves) * kCodeBytes;
                tma_load_2d(base, &x_codes, c * 128, t0, bars->full + st);
                tma_load_2d(sc, &x_scales, c * 16, t0, bars->full + st);
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    tma_load_2d(base + (1 + h) * kCodeBytes, &w_codes, c * 128, n0 + h * 128, bars->full + st);
                    tma_load_2d(sc + (1 + h) * kScaleBytes, &w_scales, c * 16, n0 + h * 128, bars->full + st);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int c = 0; c < chunks && ok; ++c) {
                const int st = c % kStages4;
                ok = mbar_wait(bars->full + st, (c / kStages4) & 1, p.status) &&
                     mbar_wait(bars->sf_ready + st, (c / kStages4) & 1, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = desc_lo_sw128(smem_u32(stage(st))), b_lo = desc_lo_sw128(smem_u32(stage(st) + kCodeBytes));
                const uint32_t sfa = tmem + kColSf + st * kSfCols, sfb = sfa + 16;
#pragma unroll
                for (int j = 0; j < 4; ++j)       // a 64-input step: 32 bytes further in both operands
                    umma_nvfp4_lo(tmem + kColAcc, a_lo + 2 * j, b_lo + 2 * j, desc_of(TN), sfa + j * 4, sfb + j * 4 * kHalves,
                                  (c | j) ? 1u : 0u);
                umma_commit(bars->empty + st);    // the stage (and its scale columns) is free once these MMAs are done
            }
            if (ok) umma_commit(&bars->done);
        }
    } else {
        // ---- block scales of every stage into tensor memory: lane l of a quarter holds, per
        //      64-input step, the scale words of rows l, l + 32, l + 64, l + 96 in four columns
        const uint32_t quarter = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        bool ok = true;
        for (int c = 0; c < chunks && ok; ++c) {
            const int st = c % kStages4;
            if (!mbar_wait(bars->full + st, (c / kStages4) & 1, p.status)) { ok = false; break; }
            const uint8_t* sc = stage(st) + (1 + kHalves) * kCodeBytes;
            {   // the tokens' scales: four columns per 64-input step
                uint32_t w[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint4 v = *reinterpret_cast<const uint4*>(sc + (lane + 32 * g) * 16);
                    w[0 + g] = v.x; w[4 + g] = v.y; w[8 + g] = v.z; w[12 + g] = v.w;
                }
                tmem_store16(quarter + kColSf + st * kSfCols, w);
            }
            // the weight rows' scales: 4 * kHalves columns per step (row l + 32 g of lane l in column g)
#pragma unroll
            for (int pair = 0; pair < kHalves; ++pair) {      // steps 2 pair, 2 pair + 1 (256 rows) or all four (128 rows)
                uint32_t w[16];
#pragma unroll
                for (int g = 0; g < 4 * kHalves; ++g) {
                    const uint4 v = *reinterpret_cast<const uint4*>(sc + kScaleBytes + (lane + 32 * g) * 16);
                    const uint32_t word[4] = {v.x, v.y, v.z, v.w};
                    if (kHalves == 1) { w[0 + g] = word[0]; w[4 + g] = word[1]; w[8 + g] = word[2]; w[12 + g] = word[3]; }
                    else { w[g] = word[2 * pair]; w[8 + g] = word[2 * pair + 1]; }
                }
                tmem_store16(quarter + kColSf + st * kSfCols + 16 + pair * 16, w);
            }
            tmem_store_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars->sf_ready + st);
        }
        // ---- epilogue: this lane's token, 128 outputs, both tensor scales after the sum
        if (ok && mbar_wait(&bars->done, 0, p.status)) {
            tc_fence_after();
            const float scale = p.x_global[0] * p.w_global[0];
            const int token = t0 + (warp & 3) * 32 + lane;
            bf16* out = p.y + (size_t)token * p.out_features + n0;
#pragma unroll 1
            for (int col = 0; col < TN; col += 16) {
                uint32_t v[16];
                tmem_load16(quarter + kColAcc + col, v);
                tmem_load_wait();
                if (token < p.tokens) {
                    uint32_t packed[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(v[2 * q]) * scale, __uint_as_float(v[2 * q + 1]) * scale);
                        packed[q] = *reinterpret_cast<const uint32_t*>(&two);
                    }
                    *reinterpret_cast<uint4*>(out + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(out + col + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kCols4);
}

// ---- activation quantiser --------------------------------------------------------------
// Largest magnitude of the chunk (bf16 magnitudes order like their bit patterns).
__global__ void act_amax_kernel(const uint4* __restrict__ x, long long n8, unsigned int* __restrict__ amax_bits) {
    uint32_t m = 0u;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = x[i];
        m = max(m, max(max(v.x & 0x7fffu, (v.x >> 16) & 0x7fffu), max(v.y & 0x7fffu, (v.y >> 16) & 0x7fffu)));
        m = max(m, max(max(v.z & 0x7fffu, (v.z >> 16) & 0x7fffu), max(v.w & 0x7fffu, (v.w >> 16) & 0x7fffu)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(amax_bits, m);
}

// Eight values -> eight E2M1 codes, round to nearest even, saturating; value 2i in the low
// nibble of byte i (the checkpoint's nibble order).
QD_DEVINL uint32_t e2m1x8(const float (&v)[16], int first) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(r)
        : "f"(v[first]), "f"(v[first + 1]), "f"(v[first + 2]), "f"(v[first + 3]), "f"(v[first + 4]), "f"(v[first + 5]),
          "f"(v[first + 6]), "f"(v[first + 7]));
    return r;
}
QD_DEVINL uint32_t e4m3_of(float v) {                 // round to nearest even, saturating
    unsigned short r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
    return (uint32_t)r & 0xffu;
}

// One thread per block of sixteen inputs: tensor scale g = amax / (6 * 448) (1 for a zero chunk),
// block scale s = e4m3(block amax / (6 g)), codes = e2m1(x / (s g)), everything round to
// nearest even; a block whose scale rounds to zero gets zero codes.
__global__ void act_quantize_kernel(const bf16* __restrict__ x, long long blocks, const unsigned int* __restrict__ amax_bits,
                                    uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, float* __restrict__ global) {
    const float amax = __uint_as_float(*amax_bits << 16);
    const float g = amax > 0.f ? amax / (6.f * 448.f) : 1.f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *global = g;
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const uint4 lo = reinterpret_cast<const uint4*>(x)[2 * b], hi = reinterpret_cast<const uint4*>(x)[2 * b + 1];
    const uint32_t raw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float v[16], top = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = __uint_as_float(raw[i] << 16);
        v[2 * i + 1] = __uint_as_float(raw[i] & 0xffff0000u);
        top = fmaxf(top, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    const uint32_t sbits = e4m3_of(top / (6.f * g));
    const float s = e4m3_to_float((uint8_t)sbits) * g;
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= inv;
    reinterpret_cast<uint2*>(codes)[b] = make_uint2(e2m1x8(v, 0), e2m1x8(v, 8));
    scales[b] = (uint8_t)sbits;
}

int scale_map_of(CUtensorMap* map, const void* base, long long rows, long long row_bytes) {
    EncodeTiledFn encode = umma_encode_fn();
    if (!encode) return QD_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {16, (cuuint32_t)kTile};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QD_OK : QD_ERR_LAUNCH;
}

}  // namespace
}  // namespace qd

extern "C" int qd_nvfp4_quantize_act(const void* x, int tokens, int in_features, void* codes, void* scales,
                                     float* global, unsigned int* amax_scratch, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x && codes && scales && global && amax_scratch && tokens > 0 && in_features > 0 && in_features % 16 == 0);
    QD_CHECK_ARG(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(codes)) & 15u) == 0);
    cudaStream_t s = (cudaStream_t)stream;
    const long long n = (long long)tokens * in_features;
    if (cudaMemsetAsync(amax_scratch, 0, 4, s) != cudaSuccess) return QD_ERR_LAUNCH;
    const int grid = (int)std::min<long long>((n / 8 + 255) / 256, 148 * 8);
    act_amax_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(x), n / 8, amax_scratch);
    const long long blocks = n / 16;
    act_quantize_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, s>>>(reinterpret_cast<const bf16*>(x), blocks, amax_scratch,
                                                                     reinterpret_cast<uint8_t*>(codes), reinterpret_cast<uint8_t*>(scales), global);
    return qd_launch_status();
}

extern "C" int qd_nvfp4_matmul_w4a4(const void* x_codes, const void* x_scales, const float* x_global, const void* w_codes,
                                    const void* w_scales, const float* w_global, void* y, int tokens, int out_features,
                                    int in_features, int wide_tiles, unsigned int* status, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x_codes && x_scales && x_global && w_codes && w_scales && w_global && y && tokens > 0);
    QD_CHECK_ARG(in_features > 0 && in_features % 256 == 0 && out_features > 0 && out_features % 128 == 0);
    QD_CHECK_ARG(((reinterpret_cast<uintptr_t>(x_codes) | reinterpret_cast<uintptr_t>(x_scales) | reinterpret_cast<uintptr_t>(w_codes) |
                   reinterpret_cast<uintptr_t>(w_scales) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0);
    alignas(64) CUtensorMap xc, xs, wc, ws;
    int rc = umma_make_map(&xc, x_codes, tokens, in_features / 2, 128, kTile);
    if (rc == QD_OK) rc = umma_make_map(&wc, w_codes, out_features, in_features / 2, 128, kTile);
    if (rc == QD_OK) rc = scale_map_of(&xs, x_scales, tokens, in_features / 16);
    if (rc == QD_OK) rc = scale_map_of(&ws, w_scales, out_features, in_features / 16);
    if (rc != QD_OK) return rc;
    Gemm4Params p = {};
    p.x_global = x_global; p.w_global = w_global; p.y = reinterpret_cast<bf16*>(y);
    p.tokens = tokens; p.out_features = out_features; p.in_features = in_features; p.status = status;
    // 256-row weight tiles where they still give every SM a tile or more; 128-row tiles otherwise
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long token_tiles = (tokens + kTile - 1) / kTile;
    const bool wide = wide_tiles >= 0 ? wide_tiles != 0 : (out_features % 256 == 0 && token_tiles * (out_features / 256) >= 2ll * sms);
    static bool configured[2][64];
    auto launch = [&](auto kernel, int tn) -> int {
        const size_t smem = (size_t)stages_of(tn) * stage_bytes(tn) + sizeof(Bars4) + 64 + 1024;
        if (!configured[tn == 256][dev]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return QD_ERR_LAUNCH;
            configured[tn == 256][dev] = true;
        }
        const dim3 grid((unsigned)(out_features / tn), (unsigned)token_tiles);
        kernel<<<grid, kThreads4, smem, (cudaStream_t)stream>>>(p, xc, xs, wc, ws);
        return qd_launch_status();
    };
    return wide ? launch(nvfp4_gemm_w4a4_kernel<256>, 256) : launch(nvfp4_gemm_w4a4_kernel<128>, 128);
}
