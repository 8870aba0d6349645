// y[t] = W x[t] for an NVFP4 matrix and up to 32 token rows (the dense projections of a decode
// batch: the 2-D NVFP4 branch of quickdraw/kernel/triton/matvec.py:118-163 at small M;
// arithmetic of quickdraw/models/qwen.py:36-54).
//
// The tcgen05 product expands a weight tile to bf16 for 128 tokens and walks the inputs in a
// serial chain of K steps: about 19 us for matrices that take 2 us to read.  Here every weight
// tile is decoded once on the warp-level tensor-core instruction with the tokens as the columns
// of the B operand, as in the routed form (expert_rows.cu):
//   a first small kernel writes the token rows as f16 (each row scaled down by a power of two
//   only if it would leave f16) into a scratch area that every block then reads from L2;
//   block = 64 (or 32) weight rows; the inputs go by in chunks of 512 through a three-stage
//   cp.async ring (weight codes, block scales and the f16 token rows of the chunk);
//   warp (group, part): sixteen rows, one part of the chunk's four spans of 128 inputs; a lane
//   converts 32 codes of two rows per span (cvt.rn.f16x2.e2m1x2, exact f16 multiply with the E4M3
//   scale) and feeds 8 MMAs (m16n8k16) per group of eight tokens; fp32 accumulators; the parts of
//   a row group meet in shared memory at the end.
// Rounding as everywhere: fp32 sum, global scale last, one bf16 rounding.
#include "expert_rows.cuh"

namespace qd {
namespace {

constexpr int kDenseTokens = 32, kDenseThreads = 256, kDenseChunk = 512, kDenseStages = 3;
constexpr int kDenseCodeRow = kDenseChunk / 2 + 64;       // padded row strides of a stage, bytes
constexpr int kDenseScaleRow = kDenseChunk / 16 + 16;
constexpr int kDenseXRow = kDenseChunk * 2 + 16;
template <int GROUPS> constexpr int dense_stage_bytes() {
    return 16 * GROUPS * (kDenseCodeRow + kDenseScaleRow) + kDenseTokens * kDenseXRow;
}

// Up to three matrices that read the same token rows share a launch (q | k | v, qkv | z, gate | up):
// the blocks are the tiles of the first matrix, then those of the second, ...
constexpr int kDenseMatrices = 3;
struct DenseMatrix {
    const uint8_t* codes; const uint8_t* scales; const float* global; bf16* y;
    int out_features, first_tile;     // first_tile: the block that holds rows 0 .. of this matrix (a huge value: unused)
};
struct DenseParams {
    const uint8_t* xf; const float* up;
    DenseMatrix m[kDenseMatrices];
    int tokens, in_features;
};

QD_DEVINL void dense_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// 16-byte piece c of a token row sits at piece c ^ (bit 3 of c << 1): the four pieces a
// quarter-warp reads at once (c = 4 t + j) then fall on different banks
QD_DEVINL int dense_piece(int c) { return c ^ ((c >> 2) & 2); }

template <int GROUPS>
__global__ void __launch_bounds__(kDenseThreads, 1) dense_rows_kernel(const DenseParams p) {
    constexpr int PARTS = 8 / GROUPS, TILE = 16 * GROUPS, SPANS = kDenseChunk / 128 / PARTS;
    constexpr int kStage = dense_stage_bytes<GROUPS>();
    static_assert(PARTS <= 4 && (PARTS - 1) * GROUPS * 4 * 32 * 16 <= kStage, "parts of a chunk; meeting area");
    extern __shared__ __align__(16) uint8_t dense_smem[];
    const int which = ((int)blockIdx.x >= p.m[1].first_tile) + ((int)blockIdx.x >= p.m[2].first_tile);
    const DenseMatrix& mx = p.m[which];
    const int K = p.in_features, R = mx.out_features, chunks = K / kDenseChunk;
    const int r0 = ((int)blockIdx.x - mx.first_tile) * TILE, rows = min(TILE, R - r0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int group = warp % GROUPS, part = warp / GROUPS;
    const bool live = group * 16 < rows;              // a warp without rows computes on rows 0..15 and stores nothing
    const int slot0 = live ? group * 16 : 0;
    const uint8_t* codes = mx.codes + (size_t)r0 * (K / 2);
    const uint8_t* scales = mx.scales + (size_t)r0 * (K / 16);

    auto issue_weights = [&](int c) {     // chunk c of the codes and block scales into its stage of the ring
        uint8_t* st = dense_smem + (size_t)(c % kDenseStages) * kStage;
        uint8_t* st_scales = st + TILE * kDenseCodeRow;
        for (int piece = tid; piece < rows * 16; piece += kDenseThreads) {
            const int r = piece >> 4, q = piece & 15;
            dense_cp16(st + r * kDenseCodeRow + q * 16, codes + (size_t)r * (K / 2) + c * (kDenseChunk / 2) + q * 16);
        }
        for (int piece = tid; piece < rows * 2; piece += kDenseThreads) {
            const int r = piece >> 1, q = piece & 1;
            dense_cp16(st_scales + r * kDenseScaleRow + q * 16, scales + (size_t)r * (K / 16) + c * (kDenseChunk / 16) + q * 16);
        }
    };
    auto issue_rows = [&](int c) {        // chunk c of the f16 token rows
        uint8_t* st_x = dense_smem + (size_t)(c % kDenseStages) * kStage + TILE * (kDenseCodeRow + kDenseScaleRow);
#pragma unroll
        for (int i = 0; i < kDenseTokens * 64 / kDenseThreads; ++i) {
            const int piece = tid + i * kDenseThreads, row = piece >> 6, q = piece & 63;
            dense_cp16(st_x + row * kDenseXRow + dense_piece(q) * 16, p.xf + ((size_t)row * K + (size_t)c * kDenseChunk) * 2 + q * 16);
        }
    };
    // The weights of the first chunks do not depend on the kernel before this one (the writer of the f16
    // token rows): as its programmatic dependent the block fetches them while that kernel still runs, and
    // only then waits for it (chain_enter() split around the fetch).
    grid_launch_dependents();
#pragma unroll
    for (int c = 0; c < kDenseStages; ++c)
        if (c < chunks) issue_weights(c);
    grid_dependency_wait();
#pragma unroll
    for (int c = 0; c < kDenseStages; ++c) {
        if (c < chunks) issue_rows(c);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group 2;" ::: "memory");       // kDenseStages - 1 younger groups may be in flight
        __syncthreads();
        const uint8_t* st = dense_smem + (size_t)(c % kDenseStages) * kStage;
        const uint8_t* st_scales = st + TILE * kDenseCodeRow;
        const uint8_t* st_x = st_scales + TILE * kDenseScaleRow + (size_t)g * kDenseXRow;
#pragma unroll
        for (int s = 0; s < SPANS; ++s) {
            const int span = part * SPANS + s;
            const uint8_t* c0 = st + (slot0 + g) * kDenseCodeRow + span * 64 + t * 16;
            const uint8_t* s0 = st_scales + (slot0 + g) * kDenseScaleRow + span * 8 + t * 2;
            const uint4 w0 = lds128(c0), w1 = lds128(c0 + 8 * kDenseCodeRow);
            const uint32_t p0 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0));
            const uint32_t p1 = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(s0 + 8 * kDenseScaleRow));
            const uint32_t sa0 = __byte_perm(p0, 0u, 0x1010), sb0 = __byte_perm(p0, 0u, 0x3232);
            const uint32_t sa1 = __byte_perm(p1, 0u, 0x1010), sb1 = __byte_perm(p1, 0u, 0x3232);
            const uint32_t ra[4] = {w0.x, w0.y, w0.z, w0.w}, rb[4] = {w1.x, w1.y, w1.z, w1.w};
            const int piece0 = span * 16 + t * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t h0[4], h1[4];
                e2m1x8_to_f16x2(ra[j], h0);
                e2m1x8_to_f16x2(rb[j], h1);
                const uint32_t s_lo = j < 2 ? sa0 : sb0, s_hi = j < 2 ? sa1 : sb1;
#pragma unroll
                for (int b = 0; b < 4; ++b) { h0[b] = hmul2(h0[b], s_lo); h1[b] = hmul2(h1[b], s_hi); }
                const int at = dense_piece(piece0 + j) * 16;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {        // token 8 nt + g is this lane's column
                    const uint4 u = lds128(st_x + (size_t)nt * 8 * kDenseXRow + at);
                    mma_f16(acc[nt], h0[0], h1[0], h0[1], h1[1], u.x, u.y);
                    mma_f16(acc[nt], h0[2], h1[2], h0[3], h1[3], u.z, u.w);
                }
            }
        }
        __syncthreads();                  // every warp is done with this stage
        if (c + kDenseStages < chunks) { issue_weights(c + kDenseStages); issue_rows(c + kDenseStages); }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ---- the parts of a row group meet (the ring is free: the loop ended with a barrier)
    float4* meet = reinterpret_cast<float4*>(dense_smem);
    if (PARTS > 1) {
        if (part > 0) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
                meet[(((part - 1) * GROUPS + group) * 4 + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        }
        __syncthreads();
    }
    if (part != 0 || !live) return;
#pragma unroll
    for (int other = 1; other < PARTS; ++other)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float4 v = meet[(((other - 1) * GROUPS + group) * 4 + nt) * 32 + lane];
            acc[nt][0] += v.x; acc[nt][1] += v.y; acc[nt][2] += v.z; acc[nt][3] += v.w;
        }
    // acc[nt][0..1] = row slot0 + g, tokens 8 nt + 2 t and + 1; [2..3] = row + 8
    const float global = *mx.global;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int token = 8 * nt + 2 * t + (c & 1), row = r0 + slot0 + g + 8 * (c >> 1);
            if (token >= p.tokens || row >= R) continue;
            mx.y[(size_t)token * R + row] = __float2bfloat16_rn(acc[nt][c] * p.up[token] * global);
        }
}

template <int GROUPS> int launch_dense(DenseParams p, int count, cudaStream_t stream) {
    constexpr int smem = kDenseStages * dense_stage_bytes<GROUPS>();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(dense_rows_kernel<GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    const int tile = 16 * GROUPS;
    int tiles = 0;
    for (int i = 0; i < kDenseMatrices; ++i) {
        p.m[i].first_tile = i < count ? tiles : 0x7fffffff;
        if (i < count) tiles += (p.m[i].out_features + tile - 1) / tile;
    }
    if (qd_launch(dense_rows_kernel<GROUPS>, dim3((unsigned)tiles), dim3(kDenseThreads), smem, stream, 2, p) != QD_OK) return QD_ERR_LAUNCH;
    return qd_launch_status();
}

}  // namespace
}  // namespace qd

// Bytes of the scratch area for the f16 token rows and their scale factors.
extern "C" long long qd_nvfp4_matmul_rows_scratch_bytes(int in_features) {
    return in_features > 0 ? (long long)qd::kDenseTokens * in_features * 2 + qd::kDenseTokens * (long long)sizeof(float) : 0;
}

// y_i [tokens, out_i] = x [tokens, in_features] W_i^T for tokens <= 32 and up to three matrices that
// read the same input (the contract of qd_nvfp4_matmul for each).  scratch:
// qd_nvfp4_matmul_rows_scratch_bytes(in_features) bytes, 16-byte aligned; convert = 0 reuses the token
// rows that the previous call with this scratch area converted.  x_up (or NULL): the input rows are
// bf16(bf16(silu(x)) * x_up), the SwiGLU of two projections.  Matrices past `count` are ignored (NULL).
// in_features a multiple of 512, out_features of 16, group size 16; QD_ERR_UNSUPPORTED otherwise.
extern "C" int qd_nvfp4_matmul_rows3(const void* x, const void* x_up, int tokens, int in_features, int group_size,
                                     void* scratch, int convert, int count,
                                     const void* codes0, const void* scales0, const float* global0, void* y0, int out0,
                                     const void* codes1, const void* scales1, const float* global1, void* y1, int out1,
                                     const void* codes2, const void* scales2, const float* global2, void* y2, int out2,
                                     void* stream) {
    using namespace qd;
    QD_CHECK_ARG(x && scratch && tokens > 0 && in_features > 0 && count >= 1 && count <= kDenseMatrices);
    if (tokens > kDenseTokens || group_size != 16 || in_features % kDenseChunk != 0) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)x_up | (uintptr_t)scratch) & 15u) return QD_ERR_UNSUPPORTED;
    const void* codes[3] = {codes0, codes1, codes2};
    const void* scales[3] = {scales0, scales1, scales2};
    const float* globals[3] = {global0, global1, global2};
    void* ys[3] = {y0, y1, y2};
    const int outs[3] = {out0, out1, out2};
    uint8_t* xf = (uint8_t*)scratch;
    float* up = reinterpret_cast<float*>(xf + (size_t)kDenseTokens * in_features * 2);
    DenseParams p = {};
    p.xf = xf; p.up = up; p.tokens = tokens; p.in_features = in_features;
    long long rows = 0;
    for (int i = 0; i < count; ++i) {
        QD_CHECK_ARG(codes[i] && scales[i] && globals[i] && ys[i] && outs[i] > 0);
        if (outs[i] % 16 != 0 || (((uintptr_t)codes[i] | (uintptr_t)scales[i]) & 15u)) return QD_ERR_UNSUPPORTED;
        p.m[i].codes = (const uint8_t*)codes[i]; p.m[i].scales = (const uint8_t*)scales[i]; p.m[i].global = globals[i];
        p.m[i].y = (bf16*)ys[i]; p.m[i].out_features = outs[i];
        rows += outs[i];
    }
    if (convert) {
        qd_launch(rows_to_f16_kernel, dim3(kDenseTokens), dim3(256), 0, (cudaStream_t)stream, true, (const bf16*)x, (const bf16*)x_up, tokens, in_features, xf, up);
        if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    }
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // 32-row tiles while they fit one wave of the GPU (twice the blocks, half the chain), else 64-row tiles
    return (rows + 31) / 32 > (sms > 0 ? sms : 148) ? launch_dense<4>(p, count, (cudaStream_t)stream)
                                                    : launch_dense<2>(p, count, (cudaStream_t)stream);
}

// One matrix: see qd_nvfp4_matmul_rows3.
extern "C" int qd_nvfp4_matmul_rows(const void* x, const void* x_up, const void* codes, const void* scales, const float* global, void* y,
                                    int tokens, int out_features, int in_features, int group_size, void* scratch,
                                    int convert, void* stream) {
    return qd_nvfp4_matmul_rows3(x, x_up, tokens, in_features, group_size, scratch, convert, 1, codes, scales, global, y, out_features,
                                 nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr, 0, stream);
}
