// NVFP4 matvec on the block-scaled FP4 tensor core (tcgen05.mma kind::mxf4nvf4).
//
// y = bf16((sum_k x_k * e2m1[n, k] * e4m3_scale[n, k / 16]) * global)  (reference:
// quickdraw/models/qwen.py:36-54, quickdraw/kernel/cute/matvec.py:26-72) with no unpacking
// instruction at all: the weight codes travel HBM -> shared memory as 2-D tiled TMA loads
// straight from the checkpoint layout (128-byte swizzle, the layout the MMA reads), the
// E4M3 block scales travel the same way and are moved into tensor memory by the four worker
// warps, and the activation vector enters as sixteen E2M1 digit planes (umma.cuh).  Per 128
// weight rows and 64 inputs one MMA of shape 128 x 16 x 64 does what 256 convert and 512
// multiply-add lane-operations did.
//
// Block = 4 worker warps (digit planes, scale factors into tensor memory, epilogue: one
// thread per weight row), one TMA warp, one MMA warp.  A block owns a contiguous range of
// rows (a multiple of the TMA box height) and walks it in tiles of up to 128 rows; the
// codes of a tile stream through a ring of 16 KB stages (128 rows x 256 inputs).
#include "umma.cuh"
#include "stream.cuh"

namespace qd {

EncodeTiledFn umma_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

int umma_make_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows) {
    EncodeTiledFn encode = umma_encode_fn();
    if (!encode) return QD_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_bytes & 15) || box_bytes > 128 || box_bytes % 16 || box_rows > 256)
        return QD_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QD_OK : QD_ERR_LAUNCH;
}

namespace {

constexpr int kWorkers = 128;                 // one per tensor-memory lane
constexpr int kThreads = kWorkers + 64;       // + TMA warp + MMA warp
constexpr int kStages = 8;                    // 128 rows x 128 bytes (256 inputs) each
constexpr int kStageBytes = 128 * 128;
constexpr int kMaxK = 4096;
constexpr int kTmemCols = 512;
constexpr int kColD = 0;                      // two accumulators of 16 columns
constexpr int kColSfb = 32;                   // two columns per 64-input step (the first one is read)
constexpr int kColSfa = 160;                  // K / 16 columns per buffer

struct UmmaParams {
    const bf16* x; const float* global; bf16* y;
    int rows, k, box_rows, rows_per_block;
    unsigned int* status;
};

struct Bars {
    uint64_t full[kStages], empty[kStages];
    uint64_t sc_full[2], sc_free[2], sfa_ready[2], d_full[2], d_free[2], b_ready;
};

__global__ void __launch_bounds__(kThreads, 1)
nvfp4_umma_matvec_kernel(const __grid_constant__ UmmaParams p, const __grid_constant__ CUtensorMap code_map,
                         const __grid_constant__ CUtensorMap scale_map) {
    extern __shared__ __align__(1024) uint8_t umma_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(umma_smem_raw) + 1023) & ~uintptr_t(1023));
    const int K = p.k, chunks = K / 256, halves = K / 2048;   // 256-input chunks; 128-byte groups of a scale row
    uint8_t* stages = smem;                                                   // [kStages][128 rows][128 B]
    uint8_t* planes = stages + kStages * kStageBytes;                         // [chunks][16 rows][128 B]
    uint8_t* scales = planes + (kMaxK / 256) * kPlaneChunkBytes;                          // [2][halves][128 rows][128 B]
    Bars* bars = reinterpret_cast<Bars*>(scales + 2 * 2 * 128 * 128);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
    float* red = reinterpret_cast<float*>(tmem_slot + 4);                     // [8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nbuf = K <= 2048 ? 2 : 1;                                       // scale-factor buffers in tensor memory
    const int r_begin = min(p.rows, (int)blockIdx.x * p.rows_per_block);
    const int r_end = min(p.rows, r_begin + p.rows_per_block);
    const int tiles = (r_end - r_begin + 127) / 128;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bars->full + s, 1); mbar_init(bars->empty + s, 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bars->sc_full + b, 1); mbar_init(bars->sc_free + b, 4);
            mbar_init(bars->sfa_ready + b, 4); mbar_init(bars->d_full + b, 1); mbar_init(bars->d_free + b, 4);
        }
        mbar_init(&bars->b_ready, 4);
        mbar_fence_init();
    }
    if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA warp
        if (lane == 0) {
            tma_prefetch_map(&code_map);
            tma_prefetch_map(&scale_map);
            int it = 0;
            bool ok = true;
            for (int ti = 0; ti < tiles && ok; ++ti) {
                const int r0 = r_begin + ti * 128, n = min(128, r_end - r0);
                const int sb = ti & 1;
                if (ti >= 2 && !mbar_wait(bars->sc_free + sb, ((ti >> 1) - 1) & 1, p.status)) break;
                // a box always delivers box_rows rows (rows past the end of the matrix arrive as zeros)
                const uint32_t boxed = (uint32_t)((n + p.box_rows - 1) / p.box_rows * p.box_rows);
                mbar_expect_tx(bars->sc_full + sb, boxed * (K / 16));
                for (int h = 0; h < halves; ++h)
                    for (int r = 0; r < n; r += p.box_rows)
                        tma_load_2d(scales + ((sb * 2 + h) * 128 + r) * 128, &scale_map, h * 128, r0 + r, bars->sc_full + sb);
                for (int c = 0; c < chunks; ++c, ++it) {
                    const int st = it % kStages;
                    if (!mbar_wait(bars->empty + st, ((it / kStages) & 1) ^ 1, p.status)) { ok = false; break; }
                    mbar_expect_tx(bars->full + st, boxed * 128);
                    for (int r = 0; r < n; r += p.box_rows)
                        tma_load_2d(stages + st * kStageBytes + r * 128, &code_map, c * 128, r0 + r, bars->full + st);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA warp
        if (lane == 0 && tiles > 0) {
            bool ok = mbar_wait(&bars->b_ready, 0, p.status);
            int it = 0;
            for (int ti = 0; ti < tiles && ok; ++ti) {
                const int fb = ti % nbuf, db = ti & 1;
                if (!mbar_wait(bars->sfa_ready + fb, (ti / nbuf) & 1, p.status)) break;
                if (ti >= 2 && !mbar_wait(bars->d_free + db, ((ti >> 1) - 1) & 1, p.status)) break;
                tc_fence_after();
                const uint32_t d_col = tmem + kColD + db * 16;
                for (int c = 0; c < chunks; ++c, ++it) {
                    const int st = it % kStages;
                    if (!mbar_wait(bars->full + st, (it / kStages) & 1, p.status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stages + st * kStageBytes), b_addr = smem_u32(planes + c * kPlaneChunkBytes);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int step = c * 4 + j;       // 64-input step of the row
                        umma_nvfp4(d_col, smem_desc_sw128(a_addr + j * 32), smem_desc_sw128(b_addr + j * 32), kUmmaNvfp4Desc,
                                   tmem + kColSfa + fb * (K / 16) + step * 4, tmem + kColSfb + step * 2, (c | j) ? 1u : 0u);
                    }
                    umma_commit(bars->empty + st);        // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(bars->d_full + db);
            }
        }
    } else {
        // ------------------------------------------------------------------ workers
        // 1. activation digit planes into the B operand, plane scales into tensor memory
        uint32_t m2 = 0u;
        for (int i = tid; i < K / 8; i += kWorkers) {
            const uint4 v = reinterpret_cast<const uint4*>(p.x)[i];
            m2 = max(m2, max(max(v.x & 0x7fffu, (v.x >> 16) & 0x7fffu), max(v.y & 0x7fffu, (v.y >> 16) & 0x7fffu)));
            m2 = max(m2, max(max(v.z & 0x7fffu, (v.z >> 16) & 0x7fffu), max(v.w & 0x7fffu, (v.w >> 16) & 0x7fffu)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m2 = max(m2, __shfl_xor_sync(0xffffffffu, m2, o));
        if (lane == 0) reinterpret_cast<uint32_t*>(red)[warp] = m2;
        named_barrier(1, kWorkers);
        m2 = max(max(reinterpret_cast<uint32_t*>(red)[0], reinterpret_cast<uint32_t*>(red)[1]),
                 max(reinterpret_cast<uint32_t*>(red)[2], reinterpret_cast<uint32_t*>(red)[3]));
        const int E = plane_exponent_of(__uint_as_float(m2 << 16));      // the largest |bf16| of the vector
        for (int i = tid; i < K / 4; i += kWorkers) {
            const uint2 v = reinterpret_cast<const uint2*>(p.x)[i];
            const float xv[4] = {__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                 __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u)};
            store_planes4(planes, 4 * i, xv, E);
        }
        // lanes 0..15 of every 32-lane quarter of tensor memory: plane p's scale, per 64-input step
        for (int step = 0; step < K / 64; ++step)
            tmem_store1(tmem + ((uint32_t)(warp * 32) << 16) + kColSfb + step * 2, plane_scale_word(lane & 15));
        tmem_store_wait();
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the plane bytes are read by the MMA (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->b_ready);
        const float out_scale = plane_out_scale(E) * p.global[0];

        // 2. per tile: block scales shared memory -> tensor memory, then (one tile behind) the epilogue
        auto epilogue = [&](int ti) {
            const int db = ti & 1;
            if (!mbar_wait(bars->d_full + db, (ti >> 1) & 1, p.status)) return;
            tc_fence_after();
            uint32_t v[16];
            tmem_load16(tmem + ((uint32_t)(warp * 32) << 16) + kColD + db * 16, v);
            tmem_load_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars->d_free + db);
            const float sum = plane_sum(v);
            const int row = r_begin + ti * 128 + tid;
            if (row < r_end) p.y[row] = __float2bfloat16_rn(sum * out_scale);
        };
        for (int ti = 0; ti < tiles; ++ti) {
            const int sb = ti & 1, fb = ti % nbuf;
            if (nbuf == 1 && ti >= 1) epilogue(ti - 1);       // one buffer: the MMAs of the tile before must be done
            if (!mbar_wait(bars->sc_full + sb, (ti >> 1) & 1, p.status)) break;
            // lane l of each quarter holds, for every 64-input step, the scale words of rows
            // l, l + 32, l + 64, l + 96 in four consecutive columns
            for (int c = 0; c < chunks; ++c) {
                uint32_t w[16];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int r = lane + 32 * g;
                    const uint8_t* row = scales + ((sb * 2 + (c >> 3)) * 128 + r) * 128;
                    const uint4 v = *reinterpret_cast<const uint4*>(row + (((c & 7) ^ (r & 7)) << 4));
                    w[0 + g] = v.x; w[4 + g] = v.y; w[8 + g] = v.z; w[12 + g] = v.w;
                }
                tmem_store16(tmem + ((uint32_t)(warp * 32) << 16) + kColSfa + fb * (K / 16) + c * 16, w);
            }
            tmem_store_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(bars->sfa_ready + fb); mbar_arrive(bars->sc_free + sb); }
            if (nbuf == 2 && ti >= 1) epilogue(ti - 1);
        }
        if (tiles > 0) epilogue(tiles - 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace qd

// NVFP4 matvec through the FP4 tensor core.  rows a multiple of 8, in_features 2048 or 4096,
// group size 16, non-negative block scales (they are read as unsigned E4M3), 16-byte aligned
// pointers.  QD_ERR_UNSUPPORTED otherwise.
int qd_umma_matvec_try(const Fp4Args& a, cudaStream_t stream) {
    using namespace qd;
    if (a.group != 16 || (a.in_features != 2048 && a.in_features != 4096) || a.rows % 8 != 0) return QD_ERR_UNSUPPORTED;
    if (a.routing || a.per_slot_input || a.slots != 1 || a.ids || a.up_codes) return QD_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.scales)) & 15u)
        return QD_ERR_UNSUPPORTED;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    UmmaParams p = {};
    p.x = a.x; p.global = a.global; p.y = a.y; p.rows = a.rows; p.k = a.in_features; p.status = nullptr;
    // rows per block: a multiple of the box height; big matrices take whole 128-row boxes
    int per = (a.rows + sms - 1) / sms;
    p.box_rows = per >= 128 ? 128 : 8;
    per = (per + p.box_rows - 1) / p.box_rows * p.box_rows;
    p.rows_per_block = per;
    const int grid = (a.rows + per - 1) / per;
    alignas(64) CUtensorMap code_map, scale_map;
    int rc = umma_make_map(&code_map, a.codes, a.rows, a.in_features / 2, 128, p.box_rows);
    if (rc != QD_OK) return rc;
    rc = umma_make_map(&scale_map, a.scales, a.rows, a.in_features / 16, 128, p.box_rows);
    if (rc != QD_OK) return rc;
    const size_t smem = (size_t)kStages * kStageBytes + (kMaxK / 256) * kPlaneChunkBytes + 2 * 2 * 128 * 128 + sizeof(Bars) + 64 + 1024;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(nvfp4_umma_matvec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    nvfp4_umma_matvec_kernel<<<grid, kThreads, smem, stream>>>(p, code_map, scale_map);
    return qd_launch_status();
}
