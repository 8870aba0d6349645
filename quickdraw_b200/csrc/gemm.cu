// Prefill / batched projection: Y[T, N] = X[T, K] . W[N, K]^T with NVFP4 weights on the 5th
// generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// Arithmetic (reference: quickdraw/kernel/triton/matvec.py:118-163, the prefill path of the
// projections): every weight is expanded to bf16(e2m1 * e4m3 block scale) - exact, the product
// has at most six significant bits - multiplied with the bf16 activations on the tensor cores
// with fp32 accumulation, the fp32 global scale multiplies the finished sum, one bf16 rounding.
//
// One block computes a 256-token x 256-row tile as two 128-token accumulators that share every
// expanded weight stage.  Roles:
//   warps 1..8  producers: 16-byte global loads of weight codes into registers (one K step
//               ahead), expansion to bf16, 16-byte stores into the shared-memory stage in the
//               tensor core's K-major core-matrix layout (8 rows x 16 bytes per core matrix, no
//               swizzle); warps 1..4 also run the epilogue
//   warp 9      plain product: one thread copies the 256 x 64 activation tile of every stage
//               with one tiled TMA load (cp.async.bulk.tensor, 128-byte swizzle; rows past the
//               end arrive as zeros) as soon as the stage is free
//               grouped product: idle - the rows of a tile are gathered through the route
//               order, so the producers copy them with 16-byte loads into the same layout
//   warp 0      allocates all 512 columns of tensor memory, issues 2 x 4 MMAs of 128x256x16 per
//               stage and commits them to the stage's "empty" barrier
// Stages: 3 x (32 KB activations + 32 KB weights) guarded by full / empty mbarriers.  Every wait
// is bounded; a wait that runs out sets the status word, the block frees its tensor memory and
// leaves.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int kTileM = 256;                 // tokens per tile: two halves of 128 (tensor memory lanes)
// weight rows per tile (tensor memory columns per accumulator): template parameter TN, 256 for
// large problems, 128 or 64 where 256 would leave most SMs without a tile
constexpr int kTileK = 64;                  // inputs per stage
// Tile heights: 256 tokens (two 128-token halves; the plain product and large grouped tiles) or
// 128 (grouped product with few rows per expert: 2 stages of 48 KB and 8 producer warps, so that
// two blocks share an SM and one block's prologue and epilogue overlap the other's K loop).
constexpr int stages_of(int tm) { return tm == 128 ? 2 : 3; }
constexpr int blocks_per_sm(int tm) { return tm == 128 ? 2 : 1; }
// Producer warps: 8 for the plain product (they only expand weights), 16 for the grouped product
// (they also gather the activation rows, and an expert's weights come from DRAM, not from L2:
// more warps keep more loads in flight; measured 171 -> 149 us on the gate bank of a
// 511-token chunk).  The block is warp 0 + producers + loader warp.
constexpr int producer_warps(bool dense, int tm) { return (dense || tm == 128) ? 8 : 16; }
constexpr int block_threads(bool dense, int tm) { return (2 + producer_warps(dense, tm)) * 32; }
// The producer warps work in kGroups groups on alternate K steps, so that two stages fill at
// the same time (measured: plain product 1 104 -> 1 138 TFLOP/s, grouped product unchanged).
#ifndef QD_GEMM_GROUPS
#define QD_GEMM_GROUPS 2
#endif
constexpr int groups_of(int tm) { return tm == 128 ? 1 : QD_GEMM_GROUPS; }
constexpr int group_threads(bool dense, int tm) { return producer_warps(dense, tm) * 32 / groups_of(tm); }
// Both operands of a stage use the 128-byte swizzled K-major layout: row r of the tile is 128
// bytes (64 inputs) at r * 128, its 16-byte piece c stored at piece c ^ (r & 7).  The TMA load
// writes it for the activations of the plain product; the producers write it themselves for
// the weights (and for the gathered activation rows of the grouped product).
constexpr int a_bytes(int tm) { return tm * kTileK * 2; }                  // 32 KB at 256 tokens
constexpr int kBBytesMax = 256 * kTileK * 2;                                // 32 KB at 256 rows
constexpr int stage_bytes(int tm) { return a_bytes(tm) + kBBytesMax; }

struct GemmParams {
    const bf16* x; const uint8_t* codes; const uint8_t* scales; const float* global; bf16* y;
    int tokens, out_features, in_features;
    unsigned int* status;
    // grouped form (routed experts of a chunk of tokens; order == NULL: plain matmul).  Routes =
    // (token, slot) pairs sorted by expert: order[r] = route index of sorted row r, rows
    // [boundaries[e], boundaries[e + 1]) belong to expert e.
    const int32_t* order; const int32_t* boundaries; const float* routing;
    int topk, experts, by_token, scatter, global_per_expert;
    long long codes_stride, scales_stride;       // bytes between experts of the bank
};

// ---- tcgen05 wrappers ------------------------------------------------------------------
QD_DEVINL void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
QD_DEVINL void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
QD_DEVINL void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
QD_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
QD_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
QD_DEVINL void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
QD_DEVINL void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
QD_DEVINL void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 columns of fp32: thread l of the warp gets lane (quadrant * 32 + l)
QD_DEVINL void tmem_load32(uint32_t addr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(addr) : "memory");
}
QD_DEVINL void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
QD_DEVINL void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle (rows of 128 bytes, 16-byte pieces
// XOR-ed with the row index inside every 1024-byte group of 8 rows; the tile starts on a
// 1024-byte boundary).  Bits: [0,14) address >> 4, [16,30) leading byte offset >> 4 (unused
// here), [32,46) bytes between 8-row groups >> 4 = 64, [46,48) descriptor version 1, [61,64)
// layout type 2.  A K step of 16 inputs advances the start address by 32 bytes inside the row.
QD_DEVINL uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Tiled 2-D TMA load global -> shared; c0 = innermost coordinate (elements; c0 * 2 bytes must be
// a multiple of 16), c1 = row.  Completion is counted in bytes on the mbarrier.
QD_DEVINL void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// (A and B must have the same format: a descriptor with bf16 activations and f16 weights, which
// would save the weights' f16 -> bf16 conversion, is rejected as an illegal instruction.)
// Instruction descriptor: fp32 accumulator (bits [4,6) = 1), bf16 A and B (bits [7,10) and
// [10,13) = 1), both K-major (bits 15, 16 = 0), N >> 3 at [17,23), M >> 4 at [24,29).
template <int TN>
constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// byte offset of the 16-byte piece (row, 8-input group kg) inside a swizzled stage tile
QD_DEVINL uint32_t piece_offset(int row, int kg) { return (uint32_t)(row * 128 + ((kg ^ (row & 7)) << 4)); }

// eight E2M1 codes (one 32-bit word, low nibble first) times an fp32 block scale -> eight bf16
// (hardware convert to f16 pairs; code * scale has at most six significant bits and stays inside
// the f16 range for every E4M3 scale, so the f16 product and the bf16 conversion are exact)
QD_DEVINL uint4 expand8(uint32_t word, float scale) {
    uint32_t h2[4], out[4];
    e2m1x8_to_f16x2(word, h2);
    const __half2 s2 = __float2half2_rn(scale);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const __half2 prod = __hmul2(*reinterpret_cast<const __half2*>(&h2[b]), s2);
        const float2 f = __half22float2(prod);
        const __nv_bfloat162 p = __floats2bfloat162_rn(f.x, f.y);
        out[b] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

template <bool DENSE, int TM>
struct StageRegs {
    static constexpr int kXPieces = TM * (kTileK / 8) / group_threads(DENSE, TM);   // 16-byte activation pieces per thread
    static constexpr int kWPieces = 256 * 2 / group_threads(DENSE, TM);             // 16-byte code pieces per thread
    uint4 wc[kWPieces];               // 16-byte pieces of codes (32 weights each)
    uint16_t ws[kWPieces];            // their two block scales each
};

// DENSE: plain product (activation tiles by TMA through `xmap`); otherwise the grouped product.
template <int TN, bool DENSE, int AHEAD, int TM>
__global__ void __launch_bounds__(block_threads(DENSE, TM), blocks_per_sm(TM))
nvfp4_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap xmap) {
    chain_enter();
    constexpr int kProducerWarps = producer_warps(DENSE, TM), kProducerThreads = group_threads(DENSE, TM);
    constexpr int kThreads = block_threads(DENSE, TM), kLoaderWarp = 1 + kProducerWarps;
    constexpr int kGroups = groups_of(TM), kStages = stages_of(TM), kTileM = TM;
    constexpr int kABytes = a_bytes(TM), kATmaBytes = kABytes, kStageBytes = stage_bytes(TM);
    constexpr int kXPieces = StageRegs<DENSE, TM>::kXPieces, kWPiecesPerThread = StageRegs<DENSE, TM>::kWPieces;
    constexpr int kTileN = TN;
    constexpr int kTmemCols = (TM / 128) * TN;   // one 128 x TN fp32 accumulator per token half
    constexpr uint32_t kInstrDesc = instr_desc<TN>();
    constexpr int kWPieces = TN * 2;             // 16-byte code pieces of a stage: (row, 32-input half)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the swizzled tiles need a 1024-byte boundary in the shared address space
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* done = empty + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * kTileN;
    const int K = p.in_features, nk = K / kTileK;
    // rows of this tile: [t0, t_end) of the activations, or of the sorted routes of one expert
    int t0 = blockIdx.x * kTileM, t_end = p.tokens, expert = 0;
    constexpr bool grouped = !DENSE;
    if (grouped) {
        // Block x is the x-th non-empty row tile in expert order (the grid holds an upper bound of
        // their number, not experts x tiles per expert): the boundaries go through shared memory
        // (the first stage is not in use yet), warp 0 sums the tiles of the experts until it
        // passes x.  Blocks past the last tile leave here, before any barrier object exists.
        __shared__ int found[2];
        int* bounds = reinterpret_cast<int*>(smem);
        for (int e = tid; e <= p.experts; e += kThreads) bounds[e] = p.boundaries[e];
        if (tid == 0) found[0] = -1;
        __syncthreads();
        if (warp == 0) {
            const int want = blockIdx.x;
            int total = 0;
            for (int e0 = 0; e0 < p.experts && total <= want; e0 += 32) {
                const int e = e0 + lane;
                const int tiles = e < p.experts ? (bounds[e + 1] - bounds[e] + kTileM - 1) / kTileM : 0;
                int incl = tiles;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += up;
                }
                const int before = total + incl - tiles;
                if (want >= before && want < before + tiles) { found[0] = e; found[1] = want - before; }
                total += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        expert = found[0];
        if (expert < 0) return;
        t0 = bounds[expert] + found[1] * kTileM;
        t_end = bounds[expert + 1];
    }
    const uint8_t* codes = p.codes + (long long)expert * p.codes_stride;
    const uint8_t* scales = p.scales + (long long)expert * p.scales_stride;
    const int halves = (t_end - t0 > 128) ? kTileM / 128 : 1;      // a half without rows is not multiplied

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full + s, kProducerWarps / kGroups + (DENSE ? 1 : 0)); mbar_init(empty + s, 1); }
        mbar_init(done, 1);
        mbar_fence_init();
        *failed = 0;
    }
    if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int s = 0; s < nk && ok; ++s) {
                const int st = s % kStages;
                ok = mbar_wait(full + st, (s / kStages) & 1, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a = smem_u32(smem + st * kStageBytes), b = a + kABytes;
#pragma unroll 1
                for (int h = 0; h < halves; ++h)
#pragma unroll
                    for (int j = 0; j < kTileK / 16; ++j) {
                        umma_bf16(tmem + h * kTileN, smem_desc_sw128(a + h * (kABytes / 2) + j * 32),
                                  smem_desc_sw128(b + j * 32), kInstrDesc, (s | j) ? 1u : 0u);
                    }
                umma_commit(empty + st);          // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(done);
            else *failed = 1;
        }
    } else if (warp == kLoaderWarp) {
        // ------------------------------------------------------- activation tiles by TMA
        if (DENSE && lane == 0) {
            for (int s = 0; s < nk; ++s) {
                const int st = s % kStages;
                if (s >= kStages && !mbar_wait(empty + st, ((s / kStages) - 1) & 1, p.status)) break;
                mbar_expect_tx(full + st, kATmaBytes);
                tma_load_2d(smem + st * kStageBytes, &xmap, s * kTileK, t0, full + st);
            }
        }
    } else {
        // ------------------------------------------------------------------- producers
        const int group = (tid - 32) / kProducerThreads;          // this warp's K steps: group, group + kGroups, ...
        const int pt = (tid - 32) % kProducerThreads;           // thread within the group
        StageRegs<DENSE, TM> cur, nxt, far;      // K steps s, s + 1 and (AHEAD == 2) s + 2
        // the eight activation rows this thread copies pieces of (piece = (row, 8-input group))
        const bf16* xrow[DENSE ? 1 : kXPieces];
        if (!DENSE) {
#pragma unroll
            for (int i = 0; i < (DENSE ? 1 : kXPieces); ++i) {
                const int t = t0 + ((pt + i * kProducerThreads) >> 3);
                xrow[i] = nullptr;
                if (t < t_end) {
                    const int src = p.by_token ? p.order[t] / p.topk : t;
                    xrow[i] = p.x + (size_t)src * K + (pt & 7) * 8;
                }
            }
        }
        if (!DENSE) {
            // an expert's weights are read once, from DRAM: ask for this thread's whole weight row
            // now, so that the K loop's loads (one step ahead) find it in L2
            const int n = n0 + pt;
            if (group == 0 && pt < kTileN && n < p.out_features) {   // (at least 256 threads per group)
                const uint8_t* row_codes = codes + (size_t)n * (K / 2);
                const uint8_t* row_scales = scales + (size_t)n * (K / 16);
                for (int off = 0; off < K / 2; off += 128) prefetch_l2(row_codes + off);
                for (int off = 0; off < K / 16; off += 128) prefetch_l2(row_scales + off);
            }
        }
        auto fetch = [&](int s, StageRegs<DENSE, TM>& r) {
            const int k0 = s * kTileK;
#pragma unroll
            for (int i = 0; i < kWPiecesPerThread; ++i) {   // weights: piece = (row, 32-input half of the stage)
                const int piece = pt + i * kProducerThreads, row = piece >> 1, half = piece & 1;
                const int n = n0 + row;
                if (piece < kWPieces && n < p.out_features) {
                    r.wc[i] = __ldg(reinterpret_cast<const uint4*>(codes + (size_t)n * (K / 2) + (k0 + half * 32) / 2));
                    r.ws[i] = __ldg(reinterpret_cast<const uint16_t*>(scales + (size_t)n * (K / 16) + (k0 + half * 32) / 16));
                } else {
                    r.wc[i] = make_uint4(0u, 0u, 0u, 0u);
                    r.ws[i] = 0;
                }
            }
        };
        auto store = [&](int st, int s, const StageRegs<DENSE, TM>& r) {
            uint8_t* a = smem + st * kStageBytes;
            uint8_t* b = a + kABytes;
            // rows without a token are not stored: an accumulator row depends on its own activation
            // row only, and rows past the end are never written out
            if (!DENSE) {
#pragma unroll
                for (int i = 0; i < (DENSE ? 1 : kXPieces); ++i) {
                    const int piece = pt + i * kProducerThreads;
                    // (the few rows an expert has come from L2 right here; holding them in registers
                    // a step ahead would cost the registers of a whole 256-row tile)
                    if (xrow[i])
                        *reinterpret_cast<uint4*>(a + piece_offset(piece >> 3, piece & 7)) =
                            __ldg(reinterpret_cast<const uint4*>(xrow[i] + s * kTileK));
                }
            }
#pragma unroll
            for (int i = 0; i < kWPiecesPerThread; ++i) {
                const int piece = pt + i * kProducerThreads, row = piece >> 1, half = piece & 1;
                if (piece >= kWPieces) continue;
                const float2 sc = e4m3x2_to_float2(r.ws[i]);
                const uint32_t words[4] = {r.wc[i].x, r.wc[i].y, r.wc[i].z, r.wc[i].w};
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4*>(b + piece_offset(row, half * 4 + q)) = expand8(words[q], q < 2 ? sc.x : sc.y);
            }
        };
        bool ok = true;
        if (group < nk) fetch(group, cur);
        if (AHEAD == 2 && group + kGroups < nk) fetch(group + kGroups, nxt);
        for (int s = group; s < nk && ok; s += kGroups) {
            if (AHEAD == 2) { if (s + 2 * kGroups < nk) fetch(s + 2 * kGroups, far); }
            else if (s + kGroups < nk) fetch(s + kGroups, nxt);
            const int st = s % kStages;
            if (s >= kStages) ok = mbar_wait(empty + st, ((s / kStages) - 1) & 1, p.status);
            if (!ok) break;
            store(st, s, cur);
            fence_async_proxy();          // the tensor core reads shared memory through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full + st);
            cur = nxt;
            if (AHEAD == 2) nxt = far;
        }
        // --------------------------------------------------------------------- epilogue
        if (warp <= 4) {
            ok = ok && mbar_wait(done, 0, p.status) && !*failed;
            tc_fence_after();
            if (ok) {
                const int quadrant = warp & 3;                 // the lanes this warp may read
                const float g = p.global[p.global_per_expert ? expert : 0];
#pragma unroll 1
                for (int h = 0; h < halves; ++h) {
                    const int t = t0 + h * 128 + quadrant * 32 + lane;
                    // where the row goes and, for the routed down projection, its routing weight:
                    // y = bf16( bf16(acc) * bf16(global * routing) )  (quickdraw/models/qwen.py:44-53)
                    int dst = t;
                    float row_scale = g;
                    bool routed = false;
                    if (grouped && t < t_end) {
                        const int route = p.order[t];
                        if (p.scatter) dst = route;
                        if (p.routing) { row_scale = round_bf16(g * p.routing[route]); routed = true; }
                    }
#pragma unroll 1
                    for (int c = 0; c < kTileN; c += 32) {
                        uint32_t v[32];
                        tmem_load32(tmem + ((uint32_t)(quadrant * 32) << 16) + h * kTileN + c, v);
                        tmem_load_wait();
                        if (t < t_end) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (n0 + c + j < p.out_features) {
                                    uint32_t o[4];
#pragma unroll
                                    for (int q = 0; q < 4; ++q) {
                                        float a0 = __uint_as_float(v[j + 2 * q]), a1 = __uint_as_float(v[j + 2 * q + 1]);
                                        if (routed) { a0 = round_bf16(a0); a1 = round_bf16(a1); }
                                        const __nv_bfloat162 hv = __floats2bfloat162_rn(a0 * row_scale, a1 * row_scale);
                                        o[q] = *reinterpret_cast<const uint32_t*>(&hv);
                                    }
                                    *reinterpret_cast<uint4*>(p.y + (size_t)dst * p.out_features + n0 + c + j) = make_uint4(o[0], o[1], o[2], o[3]);
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

// cuTensorMapEncodeTiled through the runtime's driver entry point table (the library does not
// link against the driver library).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// Tensor map of the activations X[tokens, in_features] (bf16, row-major) with a box of one
// stage tile: 64 inputs x 256 (or 128) tokens, 128-byte swizzle, zeros outside the tensor.
static int activation_map(const GemmParams& p, CUtensorMap* map, int tile_tokens) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return QD_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)p.in_features, (cuuint64_t)p.tokens};
    const cuuint64_t strides[1] = {(cuuint64_t)p.in_features * sizeof(bf16)};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)tile_tokens};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(p.x), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QD_OK : QD_ERR_LAUNCH;
}

template <int TN, bool DENSE, int AHEAD, int TM>
static int launch_variant(const GemmParams& p, int row_tiles, cudaStream_t stream) {
    // + 1024: the kernel moves its base up to a 1024-byte boundary
    const size_t smem = (size_t)stages_of(TM) * stage_bytes(TM) + (2 * stages_of(TM) + 1) * 8 + 16 + 1024;
    static bool configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(nvfp4_gemm_kernel<TN, DENSE, AHEAD, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    alignas(64) CUtensorMap map = {};
    if (DENSE) {
        const int rc = activation_map(p, &map, TM);
        if (rc != QD_OK) return rc;
    }
    dim3 grid(row_tiles, (p.out_features + TN - 1) / TN);
    return qd_launch(nvfp4_gemm_kernel<TN, DENSE, AHEAD, TM>, grid, dim3(block_threads(DENSE, TM)), smem, stream, true, p, map);
}

// The widest weight tile that still gives every SM a tile (narrower tiles expand fewer weights
// per block, so small problems finish sooner); `busy_row_tiles`: row tiles that will have rows.
template <bool DENSE, int TM>
static int launch_gemm(const GemmParams& p, int row_tiles, int busy_row_tiles, cudaStream_t stream) {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const long long wide = (long long)busy_row_tiles * ((p.out_features + 255) / 256);
    // weight codes are fetched two K steps ahead where the registers allow it (plain product)
    constexpr int kAhead = DENSE ? 2 : 1;
    // (narrower tiles to balance the last round of blocks do not pay: a 128-row block takes far
    // more than half the time of a 256-row block - gate bank of a 511-token chunk 143 -> 191 us)
    if (wide >= sms) return launch_variant<256, DENSE, kAhead, TM>(p, row_tiles, stream);
    if (4 * wide >= sms) return launch_variant<128, DENSE, kAhead, TM>(p, row_tiles, stream);
    return launch_variant<64, DENSE, kAhead, TM>(p, row_tiles, stream);
}

// matmul(x, proj) for a 2-D x — quickdraw/kernel/triton/matvec.py:153-163 (NVFP4 branch).
extern "C" int qd_nvfp4_matmul(const void* x, const void* codes, const void* scales, const float* global, void* y,
                               int tokens, int out_features, int in_features, int group_size,
                               unsigned int* status, void* stream) {
    QD_CHECK_ARG(x && codes && scales && global && y && tokens > 0 && out_features > 0 && in_features > 0);
    if (group_size != 16 || in_features % kTileK != 0 || out_features % 8 != 0) return QD_ERR_UNSUPPORTED;
    const uintptr_t align = (uintptr_t)x | (uintptr_t)codes | (uintptr_t)y;
    if (align & 15u) return QD_ERR_UNSUPPORTED;
    GemmParams p = {};
    p.x = (const bf16*)x; p.codes = (const uint8_t*)codes; p.scales = (const uint8_t*)scales; p.global = global;
    p.y = (bf16*)y; p.tokens = tokens; p.out_features = out_features; p.in_features = in_features; p.status = status;
    const int row_tiles = (tokens + kTileM - 1) / kTileM;
    // so few 256-token tiles that even 64-row weight tiles leave SMs idle: 128-token tiles, two
    // blocks per SM (measured on a 511-token chunk: better for the projections up to 4096 rows,
    // worse for 8192 rows, where 128-row weight tiles already fill the GPU)
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (4ll * row_tiles * ((out_features + 255) / 256) < (sms > 0 ? sms : 148)) {
        const int small_tiles = (tokens + 127) / 128;
        return launch_gemm<true, 128>(p, small_tiles, small_tiles, (cudaStream_t)stream);
    }
    return launch_gemm<true, 256>(p, row_tiles, row_tiles, (cudaStream_t)stream);
}

// grouped_matmul(x, bank, grouping, routing=None) — quickdraw/kernel/triton/moe.py:99-151: the
// routes (token, slot) of a chunk sorted by expert; every expert's rows go through that
// expert's matrix.  by_token: input row = order[r] / topk (gate, up), else the sorted row r
// (down).  scatter: output row = order[r] (down), else r.  routing (fp32 per route) selects the
// routed double rounding.  max_rows_per_expert bounds the rows any one expert can get (the
// number of routes is always a valid bound); no host synchronisation is needed.
extern "C" int qd_nvfp4_grouped_matmul(const void* x, const void* codes, const void* scales, const float* global,
                                       const int32_t* order, const int32_t* boundaries, const float* routing,
                                       void* y, int routes, int experts, int topk, int out_features,
                                       int in_features, int group_size, int by_token, int scatter,
                                       int global_per_expert, int max_rows_per_expert, unsigned int* status,
                                       void* stream) {
    QD_CHECK_ARG(x && codes && scales && global && order && boundaries && y);
    QD_CHECK_ARG(routes > 0 && experts > 0 && topk > 0 && out_features > 0 && in_features > 0 && max_rows_per_expert > 0);
    if (group_size != 16 || in_features % kTileK != 0 || out_features % 8 != 0) return QD_ERR_UNSUPPORTED;
    const uintptr_t align = (uintptr_t)x | (uintptr_t)codes | (uintptr_t)y;
    if (align & 15u) return QD_ERR_UNSUPPORTED;
    GemmParams p = {};
    p.x = (const bf16*)x; p.codes = (const uint8_t*)codes; p.scales = (const uint8_t*)scales; p.global = global;
    p.y = (bf16*)y; p.tokens = routes; p.out_features = out_features; p.in_features = in_features; p.status = status;
    p.order = order; p.boundaries = boundaries; p.routing = routing; p.topk = topk;
    p.experts = experts;
    p.by_token = by_token; p.scatter = scatter; p.global_per_expert = global_per_expert;
    p.codes_stride = (long long)out_features * (in_features / 2);
    p.scales_stride = (long long)out_features * (in_features / 16);
    // Few rows per expert (a chunk of some hundred tokens, a decode batch): 128-token tiles, two
    // blocks per SM.  Many rows: 256-token tiles, which expand an expert's weights once per 256.
    const bool small = (long long)routes <= 64ll * experts;
    const int tile = small ? 128 : 256;
    // non-empty row tiles: at most one partly filled tile per expert that received routes plus
    // the full ones, and never more than the caller's bound per expert allows
    const int busy = experts < routes ? experts : routes;
    const long long by_bound = (long long)experts * ((max_rows_per_expert + tile - 1) / tile);
    const long long by_count = (long long)busy + routes / tile;
    const int row_tiles = (int)(by_bound < by_count ? by_bound : by_count);
    return small ? launch_gemm<false, 128>(p, row_tiles, busy, (cudaStream_t)stream)
                 : launch_gemm<false, 256>(p, row_tiles, busy, (cudaStream_t)stream);
}
