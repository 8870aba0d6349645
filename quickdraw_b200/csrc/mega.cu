// Persistent decode kernel: one cooperative launch per token.
//
// The grid is one block per SM.  A block has sixteen consumer warps and one producer warp.
// The producer walks the program phase by phase and streams this block's share of every
// phase's weights into a ring of shared-memory stages (1-D bulk copies, full/empty
// mbarriers); it never waits for other blocks except where the weights to fetch depend on
// the routing, so at a grid barrier the ring already holds the start of the next phase.
// The consumers run the phases in order:
//     static prefetch (what no other block writes)  ->  grid barrier  ->  build the
//     activation vector  ->  rows of the ring  ->  arrive at the next barrier.
// Activations written by one block and read by another travel through L2: every such read
// is a cache-global load, every phase ends with a fence and a release on the barrier word.
//
// The arithmetic of every phase is that of the separate kernels (stream.cu, gdn.cu,
// moe.cu): same rounding points, same summation order; attention uses its own split of the
// context (reference: quickdraw/models/qwen.py:66-241).
//
// Every wait is bounded.  A wait that runs out sets the status word and an abort bit in
// the barrier word, which lets every other block fall through its barriers and leave.
#include "mega.cuh"
#include "rowdot.cuh"

namespace qd {
namespace {

constexpr int CW = kMegaConsumerWarps, CT = kMegaConsumers, NS = kMegaStages;
constexpr unsigned kAbortBit = 0x80000000u;
constexpr int kDownWidth = 512;
constexpr int kDownRowBytes = kDownWidth / 2 + kDownWidth / 16;   // 288
constexpr int kAttnStride = 256 + 2;
constexpr int kAttnScratchFloats = 8 * 4 * kAttnStride + 3 * 8 * kMegaAttnSplits + 64;   // attention merge buffers
constexpr int kDownSlots = 9;                                   // top-8 + shared
constexpr int kDownBufBytes = kDownSlots * kMegaDownRows * kDownRowBytes;   // down-projection rows of one layer
constexpr int kScratchFloats = kAttnScratchFloats > kDownBufBytes / 4 ? kAttnScratchFloats : kDownBufBytes / 4;

struct Smem {
    uint8_t* stages;
    bf16* xs;              // [4096] activation vector, bf16           (attention: q rows, fp32)
    uint32_t* xf;          // [2048] the same as f16 pairs             (attention: new key, trig table)
    float* scratch;        // attention merge / DeltaNet vectors / down contributions
    bf16* conv_taps; bf16* conv_state;
    MegaPhase* cph;        // [2] consumer copies of the current and the next phase
    MegaPhase* pph;        // producer copy
    uint64_t* full; uint64_t* empty;
    float* red;            // [96]: 0.. sums, 16.. amax, 32.. / 48.. argmax, 64.. / 80.. global scales of the segments
    int32_t* ids; float* weights;      // [8] routing of the current layer
    uint64_t* ids_bar;                 // completes once per layer, when the routing is in ids / weights
    uint64_t* down_bar;                // completes once per layer, when the down-projection rows have landed
    volatile int* abort;
    int* flag;
    float* rope;           // [2][128] bf16-rounded cos / sin of the step's position, per rotary frequency
};

extern __shared__ __align__(128) uint8_t mega_smem[];

QD_DEVINL Smem carve_smem(uint8_t* base) {
    Smem s;
    s.stages = base;                                  base += (size_t)NS * kStreamStageBytes;
    s.xs = reinterpret_cast<bf16*>(base);             base += 4096 * 2;
    s.xf = reinterpret_cast<uint32_t*>(base);         base += 2048 * 4;
    s.scratch = reinterpret_cast<float*>(base);       base += (size_t)kScratchFloats * 4;
    s.conv_taps = reinterpret_cast<bf16*>(base);      base += kMegaConvRows * kStreamConvWidth * 2;
    s.conv_state = reinterpret_cast<bf16*>(base);     base += kMegaConvRows * kStreamConvWidth * 2;
    s.cph = reinterpret_cast<MegaPhase*>(base);       base += 2 * sizeof(MegaPhase);
    s.pph = reinterpret_cast<MegaPhase*>(base);       base += sizeof(MegaPhase);
    s.full = reinterpret_cast<uint64_t*>(base);       base += NS * 8;
    s.empty = reinterpret_cast<uint64_t*>(base);      base += NS * 8;
    s.red = reinterpret_cast<float*>(base);           base += 96 * 4;
    s.ids = reinterpret_cast<int32_t*>(base);         base += 8 * 4;
    s.weights = reinterpret_cast<float*>(base);       base += 8 * 4;
    s.ids_bar = reinterpret_cast<uint64_t*>(base);    base += 8;
    s.down_bar = reinterpret_cast<uint64_t*>(base);   base += 8;
    s.abort = reinterpret_cast<volatile int*>(base);  base += 4;
    s.flag = reinterpret_cast<int*>(base);            base += 4;
    s.rope = reinterpret_cast<float*>(base);          base += 2 * 128 * 4;
    return s;
}
constexpr size_t kSmemBytes = (size_t)NS * kStreamStageBytes + 4096 * 2 + 2048 * 4 + (size_t)kScratchFloats * 4 +
                              2 * kMegaConvRows * kStreamConvWidth * 2 + 3 * sizeof(MegaPhase) + 2 * NS * 8 +
                              96 * 4 + 8 * 4 + 8 * 4 + 24 + 2 * 128 * 4;

QD_DEVINL float ldcg_bf16(const bf16* p) {
    return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
}
QD_DEVINL unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
QD_DEVINL void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
QD_DEVINL void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
QD_DEVINL void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Orders this thread's earlier shared-memory accesses before later bulk copies into the same bytes.
QD_DEVINL void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bounded wait until the barrier word reaches `target` (the abort bit makes it larger than
// any target).  On time-out: status bit, abort bit, false.
// Returns the word it saw (abort bit included); on time-out: status bit, abort bit.
__device__ __noinline__ unsigned grid_wait(unsigned* bar, unsigned target, unsigned* status) {
    unsigned v;
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
        if ((v = ld_acquire(bar)) >= target) return v;
    const unsigned long long start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if ((v = ld_acquire(bar)) >= target) return v;
        if (global_timer_ns() - start > QD_WAIT_LIMIT_NS) break;
    }
    atomicOr(status, QD_STATUS_WAIT_TIMEOUT);
    atomicOr(bar, kAbortBit);
    return kAbortBit;
}
// The consumers' side of the grid barrier in front of phase `pi`.
QD_DEVINL void phase_wait(const MegaParams& mp, const Smem& S, int pi, int tid) {
    // The acquire load orders thread 0's later reads after the other blocks' releases; the
    // block barrier hands that order on to the rest of the block.
    if (pi > 0 && tid == 0) {
        if (grid_wait(mp.bar, (unsigned)pi * gridDim.x, mp.status) & kAbortBit) *S.abort = 1;
    }
    named_barrier(1, CT);
}
// Profiling: sixteen nanosecond timestamps per phase and block.  Slots: 0 phase start (after
// the grid barrier), 1 phase end, 2 activation vector ready, 3 first tile landed, 4 / 5 first
// and last tile of the phase issued by the producer; 8.. are free for finer marks (QD_MARK,
// compiled in with -DQD_FINE_TRACE).
constexpr int kTraceSlots = 16;
QD_DEVINL void trace_mark(const MegaParams& mp, int pi, int slot) {
    if (mp.trace) mp.trace[((size_t)pi * kTraceSlots + slot) * gridDim.x + blockIdx.x] = global_timer_ns();
}
#ifdef QD_FINE_TRACE
#define QD_MARK(slot) do { if (tid == 0) trace_mark(mp, pi, slot); } while (0)
#else
#define QD_MARK(slot) do { } while (0)
#endif
QD_DEVINL void give_up(const MegaParams& mp, const Smem& S) {
    *S.abort = 1;
    atomicOr(mp.bar, kAbortBit);
}

// =========================================================================== producer
template <int K>
QD_DEVINL bool produce_stream(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int& it) {
    bool ids_ready = false;
    const unsigned lo = blockIdx.x * ph.quota + min(blockIdx.x, ph.remainder);
    const unsigned hi = (blockIdx.x + 1) * ph.quota + min(blockIdx.x + 1, ph.remainder);
    unsigned seg_start = 0;
#pragma unroll 1
    for (int i = 0; i < ph.nseg; ++i) {
        const MegaSeg& sg = ph.seg[i];
        int ra, rb;
        seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
        seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        if (ra >= rb) continue;
        int expert = 0;
        if (sg.slot >= 0) {
            // The routing of layer L completes phase L of the barrier; the producer is never
            // more than one layer away from it, so the parity names the phase.  Segments in
            // front of the first routed one have been issued by now.
            if (!ids_ready && !mbar_wait(S.ids_bar, ph.layer & 1, mp.status)) return false;
            ids_ready = true;
            expert = S.ids[sg.slot];
            if (expert < mp.expert_lo || expert >= mp.expert_hi) continue;
            expert -= mp.expert_lo;
        }
        const int tile_rows = seg_tile_rows<K>(sg.kind);
        const uint8_t* w = sg.w + (long long)expert * sg.w_stride;
        const uint8_t* s = sg.s ? sg.s + (long long)expert * sg.s_stride : nullptr;
        const uint8_t* w2 = sg.w2 ? sg.w2 + (long long)expert * sg.w_stride : nullptr;
        const uint8_t* s2 = sg.s2 ? sg.s2 + (long long)expert * sg.s_stride : nullptr;
#pragma unroll 1
        for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
            const int n = min(tile_rows, rb - r0);
            const int st = it % NS;
            if (*S.abort || !mbar_wait(S.empty + st, ((it / NS) & 1) ^ 1, mp.status)) return false;
            uint8_t* dst = S.stages + (size_t)st * kStreamStageBytes;
            uint64_t* full = S.full + st;
            if (sg.kind == SEG_BF16) {
                mbar_expect_tx(full, n * 2 * K);
                bulk_load(dst, w + (long long)r0 * 2 * K, n * 2 * K, full);
            } else if (sg.kind == SEG_FP4) {
                mbar_expect_tx(full, n * (K / 2 + K / 16));
                bulk_load(dst, w + (long long)r0 * (K / 2), n * (K / 2), full);
                bulk_load(dst + tile_rows * (K / 2), s + (long long)r0 * (K / 16), n * (K / 16), full);
            } else {
                mbar_expect_tx(full, 2 * n * (K / 2 + K / 16));
                uint8_t* sc = dst + 2 * tile_rows * (K / 2);
                bulk_load(dst, w + (long long)r0 * (K / 2), n * (K / 2), full);
                bulk_load(dst + tile_rows * (K / 2), w2 + (long long)r0 * (K / 2), n * (K / 2), full);
                bulk_load(sc, s + (long long)r0 * (K / 16), n * (K / 16), full);
                bulk_load(sc + tile_rows * (K / 16), s2 + (long long)r0 * (K / 16), n * (K / 16), full);
            }
        }
    }
    return true;
}

// Down projections: this block's output rows of every selected expert and of the shared
// expert, into their own buffer (the scratch area, idle between the mixer core and the MoE
// tail).  Issued as soon as the routing is known, so the rows land during the gate/up phase.
QD_DEVINL void produce_down(const MegaParams& mp, const MegaPhase& ph, const Smem& S) {
    const int H = mp.hidden;
    const int r0 = (int)((long long)H * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)H * (blockIdx.x + 1) / gridDim.x);
    const int n = r1 - r0, nslots = mp.topk + 1;
    uint8_t* dst = reinterpret_cast<uint8_t*>(S.scratch);
    uint32_t bytes = 0;
    for (int s = 0; s < nslots; ++s) {
        const bool shared = s == mp.topk;
        const int e = shared ? 0 : S.ids[s];
        if (shared || (e >= mp.expert_lo && e < mp.expert_hi)) bytes += (uint32_t)n * kDownRowBytes;
    }
    mbar_expect_tx(S.down_bar, bytes);
    if (n <= 0) return;
    for (int s = 0; s < nslots; ++s) {
        const bool shared = s == mp.topk;
        const int e = shared ? 0 : S.ids[s];
        if (!shared && (e < mp.expert_lo || e >= mp.expert_hi)) continue;
        const long long row = shared ? r0 : (long long)(e - mp.expert_lo) * H + r0;
        const uint8_t* w = (shared ? ph.sw : ph.dw) + row * (kDownWidth / 2);
        const uint8_t* sc = (shared ? ph.ss : ph.ds) + row * (kDownWidth / 16);
        uint8_t* d = dst + (size_t)s * kMegaDownRows * kDownRowBytes;
        bulk_load(d, w, n * (kDownWidth / 2), S.down_bar);
        bulk_load(d + kMegaDownRows * (kDownWidth / 2), sc, n * (kDownWidth / 16), S.down_bar);
    }
}

struct AttnSplit { int active, per; };
// How the context [0, T) is cut into splits of `per` positions, one block per (KV head, split).
QD_DEVINL AttnSplit attn_split(int T, int max_splits) {
    AttnSplit a;
    const int s = min(max_splits, T);
    a.per = (T + s - 1) / s;
    a.active = (T + a.per - 1) / a.per;
    return a;
}

constexpr int kAttnChunk = 16;                       // positions per pass = consumer warps
constexpr int kAttnRowBytes = 256 * 2;               // one cache row of a KV head (head_dim 256, bf16)

// Attention: the cache rows of this block's context split, sixteen positions per ring stage (K rows
// then V rows, one 512-byte bulk copy each).  The row of the step's own position is not in
// the cache yet; the consumers fill it in.  Rows of earlier positions were written by earlier
// steps, so these copies may run ahead of the grid barrier like any weight.
QD_DEVINL bool produce_attn(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int& it) {
    const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const int T = position + 1;
    const AttnSplit cut = attn_split(T, mp.attn_splits);
    const int kvh = blockIdx.x / cut.active, split = blockIdx.x % cut.active;
    if (kvh >= mp.hkv) return true;
    const int t0 = split * cut.per, t1 = min(T, t0 + cut.per);
    const size_t layer_elems = (size_t)mp.st.capacity * mp.hkv * 256;
    const uint8_t* k_cache = reinterpret_cast<const uint8_t*>(reinterpret_cast<const bf16*>(mp.st.kv_k) + (size_t)ph.state_index * layer_elems);
    const uint8_t* v_cache = reinterpret_cast<const uint8_t*>(reinterpret_cast<const bf16*>(mp.st.kv_v) + (size_t)ph.state_index * layer_elems);
#pragma unroll 1
    for (int c0 = t0; c0 < t1; c0 += kAttnChunk, ++it) {
        const int st = it % NS;
        if (*S.abort || !mbar_wait(S.empty + st, ((it / NS) & 1) ^ 1, mp.status)) return false;
        uint8_t* dst = S.stages + (size_t)st * kStreamStageBytes;
        int rows = 0;
        for (int tl = 0; tl < kAttnChunk; ++tl) rows += (c0 + tl < t1 && c0 + tl != position) ? 1 : 0;
        mbar_expect_tx(S.full + st, (uint32_t)rows * 2 * kAttnRowBytes);
        for (int tl = 0; tl < kAttnChunk; ++tl) {
            const int t = c0 + tl;
            if (t >= t1 || t == position) continue;
            const size_t off = ((size_t)t * mp.hkv + kvh) * kAttnRowBytes;
            bulk_load(dst + tl * kAttnRowBytes, k_cache + off, kAttnRowBytes, S.full + st);
            bulk_load(dst + (kAttnChunk + tl) * kAttnRowBytes, v_cache + off, kAttnRowBytes, S.full + st);
        }
    }
    return true;
}

QD_DEVINL void producer(const MegaParams& mp, const Smem& S, int lane) {
    int it = 0;
    bool ok = true;
#pragma unroll 1
    for (int pi = 0; pi < mp.nphases && ok; ++pi) {
        {
            const uint4* src = reinterpret_cast<const uint4*>(mp.program + pi);
            uint4* dst = reinterpret_cast<uint4*>(S.pph);
            for (int i = lane; i < (int)(sizeof(MegaPhase) / 16); i += 32) dst[i] = __ldg(src + i);
        }
        __syncwarp();
        const MegaPhase& ph = *S.pph;
        if (lane == 0 && ph.kind == MK_STREAM) {
            trace_mark(mp, pi, 4);
            if (ph.width == 2048) ok = produce_stream<2048>(mp, ph, S, it);
            else ok = produce_stream<4096>(mp, ph, S, it);
            // the routed gate/up phase also carries the down-projection pointers of its layer
            if (ok && ph.route) {
                ok = mbar_wait(S.ids_bar, ph.layer & 1, mp.status);
                if (ok) produce_down(mp, ph, S);
            }
            trace_mark(mp, pi, 5);
            if (!ok) give_up(mp, S);
        } else if (lane == 0 && ph.kind == MK_ATTN) {
            ok = produce_attn(mp, ph, S, it);
            if (!ok) give_up(mp, S);
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        __syncwarp();
    }
    // Never leave with copies in flight: the full barrier of a stage completes when its bytes
    // have landed, whether or not the consumers have used them (bounded).
    if (lane == 0) {
        for (int back = 1; back <= NS && back <= it; ++back) {
            const int j = it - back;
            mbar_wait(S.full + (j % NS), (j / NS) & 1, nullptr);
        }
    }
}

// Top-k routing by one warp over at most 256 bf16 logits written by other blocks: the same
// fp32 softmax, tie-break (lowest index) and renormalisation as route_small, with the
// eight selections done by integer warp reductions (probabilities are non-negative, so their
// bit patterns order like the values).
QD_DEVINL void route_fast(const bf16* logits, int experts, int topk, int32_t* ids, float* weights, int lane) {
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
#pragma unroll 1
    for (int s = 0; s < topk; ++s) {
        float v = -1.f; int slot = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) if (p[i] > v) { v = p[i]; slot = i; }
        const int top = __reduce_max_sync(0xffffffffu, __float_as_int(v));
        const int idx = __reduce_min_sync(0xffffffffu, __float_as_int(v) == top ? slot * 32 + lane : 0x7fffffff);
        const float value = __int_as_float(top);
        chosen += value;
        if (lane == s) { mine = value; my_id = idx; }
        if ((idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (i == (idx >> 5)) p[i] = -1.f;
        }
    }
    if (lane < topk) { ids[lane] = my_id; weights[lane] = mine / chosen; }
}

// ========================================================================== consumers
// One streaming phase: activation vector -> registers, then this block's rows of the ring.
template <int KC, bool WITH_BF16>
QD_DEVINL void stream_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int pi, int& it) {
    constexpr int K = KC * 1024;
    constexpr int EPC = K / CT;                 // elements a thread converts (4 or 8)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bf16* xs = S.xs;
    uint32_t* xf = S.xf;
    float* red = S.red;
    const unsigned lo = blockIdx.x * ph.quota + min(blockIdx.x, ph.remainder);
    const unsigned hi = (blockIdx.x + 1) * ph.quota + min(blockIdx.x + 1, ph.remainder);

    // ---- static prefetch: norm gamma, conv taps and history of this block's channels
    float gam[8];
    if constexpr (KC == 2) if (ph.prologue == PRO_ADD_NORM && tid < 256) {
        const float4 g0 = *reinterpret_cast<const float4*>(ph.gamma + tid * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(ph.gamma + tid * 8 + 4);
        gam[0] = g0.x; gam[1] = g0.y; gam[2] = g0.z; gam[3] = g0.w;
        gam[4] = g1.x; gam[5] = g1.y; gam[6] = g1.z; gam[7] = g1.w;
    }
    // global scales of the segments (one per projection; per-expert scales are read at the
    // segment, after the routing): in flight across the barrier like the other static inputs
    float seg_scale = 1.f;
    if (tid < 2 * kMegaMaxSeg) {
        const MegaSeg& sg = ph.seg[tid >> 1];
        const float* src = (tid & 1) ? sg.g2 : sg.g;
        if ((tid >> 1) < ph.nseg && src && !sg.g_per_expert) seg_scale = *src;
    }
    int conv_row0 = 0, conv_n = 0;
    bf16* conv_state = nullptr;
    unsigned short conv_tap_reg = 0, conv_state_reg = 0;     // one element of each per thread
    if constexpr (KC == 2) if (ph.conv_taps) {
        const int W = mp.conv_width;
        conv_state = reinterpret_cast<bf16*>(mp.st.conv_state) + (size_t)ph.state_index * mp.channels * (W - 1);
        unsigned seg_start = 0;
#pragma unroll 1
        for (int i = 0; i < ph.nseg; ++i) {
            const MegaSeg& sg = ph.seg[i];
            if (sg.epilogue == EP_CONV) {
                int ra, rb;
                seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
                conv_row0 = ra;
                conv_n = min(rb - ra, kMegaConvRows);
                // in flight across the grid barrier; stored to shared memory after it
                if (tid < conv_n * W)
                    conv_tap_reg = reinterpret_cast<const unsigned short*>(ph.conv_taps)[(size_t)ra * W + tid];
                if (tid < conv_n * (W - 1))
                    conv_state_reg = reinterpret_cast<const unsigned short*>(conv_state)[(size_t)ra * (W - 1) + tid];
            }
            seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        }
    }
    phase_wait(mp, S, pi, tid);
    if (tid == 0) trace_mark(mp, pi, 0);
    // (stored after the wait: thread 0 polls the barrier and must not sit on this load first)
    if (tid < 2 * kMegaMaxSeg) red[64 + (tid & 1) * 16 + (tid >> 1)] = seg_scale;
    if constexpr (KC == 2) if (ph.conv_taps) {
        if (tid < conv_n * mp.conv_width) reinterpret_cast<unsigned short*>(S.conv_taps)[tid] = conv_tap_reg;
        if (tid < conv_n * (mp.conv_width - 1)) reinterpret_cast<unsigned short*>(S.conv_state)[tid] = conv_state_reg;
    }

    // ---- routing for this layer (every block selects the same experts from the same logits)
    if constexpr (KC == 2) if (ph.route && warp == 0) {
        route_fast(ph.router_logits, mp.experts, mp.topk, S.ids, S.weights, lane);
        __syncwarp();
        if (blockIdx.x == 0 && lane < mp.topk) { ph.ids_out[lane] = S.ids[lane]; ph.weights_out[lane] = S.weights[lane]; }
        if (lane == 0) mbar_arrive(S.ids_bar);
    }

    if (KC == 4 || !ph.keep_x) {
        const bf16* xin = (KC == 2 && ph.from_token) ? mp.embed + (size_t)(*mp.token) * K : ph.x;
        uint32_t m2 = 0u;
        if (KC == 2 && ph.prologue == PRO_ADD_NORM) {
            // residual add + RMSNorm by the first 256 threads, eight elements each
            // (quickdraw/models/qwen.py:205-214)
            if (tid < 256) {
                float v[8];
                float ss = 0.f;
                const uint4 xa = __ldcg(reinterpret_cast<const uint4*>(xin + tid * 8));
                uint4 ra4 = make_uint4(0u, 0u, 0u, 0u);
                if (ph.residual) ra4 = __ldcg(reinterpret_cast<const uint4*>(ph.residual + tid * 8));
                const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w}, rw0[4] = {ra4.x, ra4.y, ra4.z, ra4.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    v[2 * q] = __uint_as_float(xw[q] << 16) + __uint_as_float(rw0[q] << 16);
                    v[2 * q + 1] = __uint_as_float(xw[q] & 0xffff0000u) + __uint_as_float(rw0[q] & 0xffff0000u);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
                ss = warp_sum(ss);
                QD_MARK(8);
                if (lane == 0) red[warp] = ss;
                named_barrier(2, 256);
                QD_MARK(9);
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) tot += red[w];
                const float inv = rsqrtf(tot / (float)K + mp.eps);
                uint32_t nw[4], rw[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const __nv_bfloat162 n2 = __floats2bfloat162_rn((v[2 * q] * inv) * gam[2 * q],
                                                                    (v[2 * q + 1] * inv) * gam[2 * q + 1]);
                    const __nv_bfloat162 r2 = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
                    nw[q] = *reinterpret_cast<const uint32_t*>(&n2);
                    rw[q] = *reinterpret_cast<const uint32_t*>(&r2);
                    m2 = max_u16x2(m2, nw[q] & 0x7fff7fffu);
                }
                const uint4 nv = make_uint4(nw[0], nw[1], nw[2], nw[3]);
                *reinterpret_cast<uint4*>(xs + tid * 8) = nv;
                if (blockIdx.x == 0) {
                    if (ph.x_out) *reinterpret_cast<uint4*>(ph.x_out + tid * 8) = nv;
                    *reinterpret_cast<uint4*>(ph.residual_out + tid * 8) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
                }
            }
        } else if (KC == 4 && ph.prologue == PRO_GATED_NORM) {
            // per-head RMSNorm of o, times gamma, times silu(z); one warp per 128-wide head
            // (quickdraw/models/qwen.py:161-164)
            constexpr int HPW = K / 128 / CW;          // heads per warp
            float o[HPW > 0 ? HPW : 1][4], zz[HPW > 0 ? HPW : 1][4], gm[4];
#pragma unroll
            for (int a = 0; a < HPW; ++a)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = (warp + a * CW) * 128 + j * 32 + lane;
                    o[a][j] = ldcg_bf16(xin + i);
                    zz[a][j] = ldcg_bf16(ph.z + i);
                }
#pragma unroll
            for (int j = 0; j < 4; ++j) gm[j] = ld_bf16(ph.head_gamma + j * 32 + lane);
            QD_MARK(8);
#pragma unroll
            for (int a = 0; a < HPW; ++a) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) ss += o[a][j] * o[a][j];
                ss = warp_sum(ss);
                const float inv = rsqrtf(ss / 128.f + mp.eps);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = (warp + a * CW) * 128 + j * 32 + lane;
                    const bf16 n = __float2bfloat16_rn(((o[a][j] * inv) * gm[j]) * silu_precise(zz[a][j]));
                    xs[i] = n;
                    m2 = max(m2, (uint32_t)(__bfloat16_as_ushort(n) & 0x7fffu));
                    if (blockIdx.x == 0 && ph.x_out) ph.x_out[i] = n;
                }
            }
        } else {
            for (int i = tid; i < K / 8; i += CT) {
                const uint4 v = __ldcg(reinterpret_cast<const uint4*>(xin) + i);
                reinterpret_cast<uint4*>(xs)[i] = v;
                m2 = max_u16x2(m2, v.x & 0x7fff7fffu); m2 = max_u16x2(m2, v.y & 0x7fff7fffu);
                m2 = max_u16x2(m2, v.z & 0x7fff7fffu); m2 = max_u16x2(m2, v.w & 0x7fff7fffu);
            }
        }
        QD_MARK(10);
        {
            uint32_t m = max(m2 & 0xffffu, m2 >> 16);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0) reinterpret_cast<uint32_t*>(red)[16 + warp] = m;
        }
    }
    named_barrier(1, CT);
    QD_MARK(11);
    // ---- the vector as f16 pairs, scaled down by a power of two only if it would overflow f16
    uint32_t xh[KC == 2 ? 2 : 1][16];      // 2048-wide phases keep the f16 slice in registers
    float out_mult;
    {
        uint32_t m = 0u;
#pragma unroll
        for (int w = 0; w < CW; ++w) m = max(m, reinterpret_cast<const uint32_t*>(red)[16 + w]);
        const int exponent = (int)(m >> 7) - 127;
        const int shift = exponent > 14 ? exponent - 14 : 0;
        const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
        out_mult = __uint_as_float((uint32_t)(127 + min(shift, 127)) << 23);
        if (KC == 4 || !ph.keep_x) {
            // f16 layout: the 16-byte piece a lane fetches as (chunk c, quarter q) sits at
            // ((c * 4 + q) * 32 + lane) * 16, so that a warp's fetch is one contiguous 512 bytes
            if (EPC == 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(xs + tid * 8);
                uint4 h;
                h.x = pack_f16x2(__uint_as_float(v.x << 16) * down, __uint_as_float(v.x & 0xffff0000u) * down);
                h.y = pack_f16x2(__uint_as_float(v.y << 16) * down, __uint_as_float(v.y & 0xffff0000u) * down);
                h.z = pack_f16x2(__uint_as_float(v.z << 16) * down, __uint_as_float(v.z & 0xffff0000u) * down);
                h.w = pack_f16x2(__uint_as_float(v.w << 16) * down, __uint_as_float(v.w & 0xffff0000u) * down);
                const int piece = tid;
                const int pos = ((piece >> 7) * 4 + (piece & 3)) * 32 + ((piece >> 2) & 31);
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(xf) + pos * 16) = h;
            } else {
                const uint2 v = *reinterpret_cast<const uint2*>(xs + tid * 4);
                uint2 h;
                h.x = pack_f16x2(__uint_as_float(v.x << 16) * down, __uint_as_float(v.x & 0xffff0000u) * down);
                h.y = pack_f16x2(__uint_as_float(v.y << 16) * down, __uint_as_float(v.y & 0xffff0000u) * down);
                const int piece = tid >> 1;
                const int pos = ((piece >> 7) * 4 + (piece & 3)) * 32 + ((piece >> 2) & 31);
                *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(xf) + pos * 16 + (tid & 1) * 8) = h;
            }
            named_barrier(1, CT);
            QD_MARK(12);
        }
    }
    bool have_xh = false;
    constexpr int NB = K / 256;
    if (tid == 0) trace_mark(mp, pi, 2);
    // ---- rows
    float best_val = -INFINITY;
    bool first_tile = true;
    int best_idx = 0x7fffffff;
    unsigned seg_start = 0;
    int turn = 0;                      // rows handed out so far: rotates the row -> warp map
    bool ok = !*S.abort;
#pragma unroll 1
    for (int i = 0; i < ph.nseg && ok; ++i) {
        const MegaSeg& sg = ph.seg[i];
        int ra, rb;
        seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
        seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        if (ra >= rb) continue;
        int expert = 0;
        if (KC == 2 && sg.slot >= 0) {
            expert = S.ids[sg.slot];
            if (expert < mp.expert_lo || expert >= mp.expert_hi) continue;
            expert -= mp.expert_lo;
        }
        // 2048-wide NVFP4 rows: the lane's f16 slice goes to registers when the first such
        // segment shows up; bf16 rows and 4096-wide rows (a block sees few of them) read the
        // vector from shared memory as they go
        if (KC == 2 && sg.kind != SEG_BF16 && !have_xh) {
#pragma unroll
            for (int c = 0; c < (KC == 2 ? 2 : 1); ++c)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 v = lds128(reinterpret_cast<const uint8_t*>(xf) + ((c * 4 + q) * 32 + lane) * 16);
                    xh[c][q * 4 + 0] = v.x; xh[c][q * 4 + 1] = v.y; xh[c][q * 4 + 2] = v.z; xh[c][q * 4 + 3] = v.w;
                }
            have_xh = true;
        }
        const int tile_rows = seg_tile_rows<K>(sg.kind);
        const float g1 = (sg.g && sg.g_per_expert) ? sg.g[expert] : red[64 + i];
        const float g2 = (sg.g2 && sg.g_per_expert) ? sg.g2[expert] : red[80 + i];
        bf16* y = (KC == 2 && sg.epilogue == EP_ARGMAX) ? mp.logits : sg.y;
#pragma unroll 1
        for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
            const int n = min(tile_rows, rb - r0);
            const int st = it % NS;
            if (!mbar_wait(S.full + st, (it / NS) & 1, mp.status)) { ok = false; break; }
            if (first_tile && tid == 0) trace_mark(mp, pi, 3);
            first_tile = false;
            const uint8_t* base = S.stages + (size_t)st * kStreamStageBytes;
#pragma unroll 1
            for (int r = (warp - turn) & (CW - 1); r < n; r += CW) {
                const int row = r0 + r;
                float result;
                if (WITH_BF16 && sg.kind == SEG_BF16) {
                    result = warp_sum(bf16_row_dot_smem<NB>(base + (size_t)r * 2 * K, reinterpret_cast<const uint8_t*>(xs), lane));
                } else {
                    const int halves = (KC == 2 && sg.kind == SEG_FP4_PAIR) ? 2 : 1;
                    const uint8_t* sc = base + halves * tile_rows * (K / 2);
                    float acc[2] = {0.f, 0.f};
#pragma unroll 1
                    for (int h = 0; h < halves; ++h) {
                        if constexpr (KC == 2)
                            acc[h] = warp_sum(fp4_row_dot<2>(base + (h * tile_rows + r) * (K / 2),
                                                             sc + (h * tile_rows + r) * (K / 16), xh, lane));
                        else
                            acc[h] = warp_sum(fp4_row_dot_smem<KC>(base + (h * tile_rows + r) * (K / 2),
                                                                   sc + (h * tile_rows + r) * (K / 16),
                                                                   reinterpret_cast<const uint8_t*>(xf), lane));
                    }
                    result = (acc[0] * out_mult) * g1;
                    if (halves == 2) {
                        const float up = round_bf16((acc[1] * out_mult) * g2);
                        result = round_bf16(silu_precise(round_bf16(result))) * up;
                    }
                }
                const bf16 rounded = __float2bfloat16_rn(result);
                if (KC == 2 && sg.epilogue == EP_CONV) {
                    // depthwise causal conv of this channel (quickdraw/models/qwen.py:134-136)
                    const int W = mp.conv_width, local = row - conv_row0;
                    float val = 0.f, tap = 0.f;
                    if (lane < W) {
                        tap = __bfloat162float(S.conv_taps[local * W + lane]);
                        val = lane < W - 1 ? __bfloat162float(S.conv_state[local * (W - 1) + lane]) : __bfloat162float(rounded);
                    }
                    // W <= 4 and lanes >= W hold zero: the last two butterfly steps are the whole sum
                    float conv = lane < W ? round_bf16(val * tap) : 0.f;
                    conv += __shfl_xor_sync(0xffffffffu, conv, 2);
                    conv += __shfl_xor_sync(0xffffffffu, conv, 1);
                    if (lane >= 1 && lane < W) conv_state[(size_t)row * (W - 1) + lane - 1] = __float2bfloat16_rn(val);
                    if (lane == 0) y[row] = __float2bfloat16_rn(silu_precise(conv));
                } else {
                    if (lane == 0) y[row] = rounded;
                    if (KC == 2 && sg.epilogue == EP_ARGMAX) {
                        const float v = __bfloat162float(rounded);
                        if (v > best_val || (v == best_val && row < best_idx)) { best_val = v; best_idx = row; }
                    }
                }
            }
            turn = (turn + n) & (CW - 1);
            __syncwarp();
            if (lane == 0) mbar_arrive(S.empty + st);
        }
    }
    if (!ok && lane == 0) give_up(mp, S);
    // ---- greedy argmax over the logits (ties: lowest index)
    if (KC == 2 && ph.argmax) {
        if (lane == 0) { red[32 + warp] = best_val; reinterpret_cast<int*>(red)[48 + warp] = best_idx; }
        named_barrier(1, CT);
        if (tid == 0) {
            float bv = red[32]; int bi = reinterpret_cast<int*>(red)[48];
            for (int w = 1; w < CW; ++w) {
                const float v = red[32 + w]; const int ix = reinterpret_cast<int*>(red)[48 + w];
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            mp.best_val[blockIdx.x] = bv;
            mp.best_idx[blockIdx.x] = bi;
            __threadfence();
            const unsigned int done = atomicAdd(mp.argmax_counter, 1u);
            if (done == gridDim.x - 1) {
                __threadfence();
                float fv = -INFINITY; int fi = 0x7fffffff;
                for (int b = 0; b < (int)gridDim.x; ++b) {
                    const float v = __ldcg(mp.best_val + b);
                    const int ix = __ldcg(mp.best_idx + b);
                    if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
                }
                *mp.next_token = fi == 0x7fffffff ? 0 : fi;
                *mp.argmax_counter = 0;
            }
        }
    }
}

// Gated delta-rule recurrence (quickdraw/models/qwen.py:139-160) for 128-wide key heads:
// block = (value head, 32 value columns), 256 threads = 8 key groups x 32 columns, 16 state
// entries per thread, fetched before the grid barrier (only this block ever touches them).
QD_DEVINL void gdn_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int pi) {
    constexpr int DK = 128, KPT = 16;
    const int tid = threadIdx.x, col = tid & 31, kg = tid >> 5;
    const int dv = mp.dv, hk = mp.hk, hv = mp.hv;
    const int slices = dv / 32;
    const int unit = blockIdx.x;
    const bool active = unit < hv * slices && tid < 256;
    const int head = active ? unit / slices : 0, c0 = active ? (unit % slices) * 32 : 0;
    float* qs = S.scratch;            // [128] q, normalised and scaled
    float* ks = qs + DK;              // [128] k, normalised
    float* part = ks + DK;            // [8][32]
    float* gates = part + 256;        // decay, beta
    float* tile = mp.st.rec_state + (size_t)ph.state_index * hv * DK * dv + (size_t)head * DK * dv + c0 + col;
    float s[KPT];
    if (active) {
#pragma unroll
        for (int j = 0; j < KPT; ++j) s[j] = tile[(size_t)(kg * KPT + j) * dv];
    }
    phase_wait(mp, S, pi, tid);
    if (tid == 0) trace_mark(mp, pi, 0);
    if (!active) return;
    const int key_head = head / (hv / hk);
    // everything this thread needs from the projections, in flight together
    const float v = ldcg_bf16(ph.qkv + (size_t)2 * hk * DK + (size_t)head * dv + c0 + col);
    float qv = 0.f, kv = 0.f, av = 0.f, bv = 0.f;
    if (tid < DK) {
        qv = ldcg_bf16(ph.qkv + (size_t)key_head * DK + tid);
        kv = ldcg_bf16(ph.qkv + (size_t)hk * DK + (size_t)key_head * DK + tid);
    }
    if (tid == DK) { av = ldcg_bf16(ph.a + head); bv = ldcg_bf16(ph.b + head); }
    const float qq = warp_sum(qv * qv), kk = warp_sum(kv * kv);
    if (col == 0) { part[kg * 32] = qq; part[kg * 32 + 1] = kk; }
    named_barrier(2, 256);
    if (tid < DK) {
        float tq = 0.f, tk = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { tq += part[w * 32]; tk += part[w * 32 + 1]; }
        qs[tid] = (qv * rsqrtf(tq + 1e-6f)) / sqrtf((float)DK);
        ks[tid] = kv * rsqrtf(tk + 1e-6f);
    } else if (tid == DK) {
        const float alpha = av + ld_bf16(ph.dt_bias + head);
        gates[0] = expf(-expf(ld_bf16(ph.a_log + head)) * softplus_precise(alpha));
        gates[1] = sigmoid_precise(bv);
    }
    named_barrier(2, 256);
    const float decay = gates[0], beta = gates[1];
    float pred = 0.f;
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        s[j] *= decay;
        pred += s[j] * ks[kg * KPT + j];
    }
    part[kg * 32 + col] = pred;
    named_barrier(2, 256);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += part[w * 32 + col];
    const float corr = beta * (v - total);
    named_barrier(2, 256);
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
        s[j] += ks[kg * KPT + j] * corr;
        o += s[j] * qs[kg * KPT + j];
        tile[(size_t)(kg * KPT + j) * dv] = s[j];
    }
    part[kg * 32 + col] = o;
    named_barrier(2, 256);
    if (kg == 0) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) acc += part[w * 32 + col];
        ph.mix_out[(size_t)head * dv + c0 + col] = __float2bfloat16_rn(acc);
    }
}

// RMSNorm with gamma = 1 + weight and partial RoPE of one head by one warp
// (quickdraw/models/qwen.py:76-92).  Feature i = j * 32 + lane, so with rotary / 2 a multiple
// of 32 the two features of a rotation pair sit in the same lane and nothing is exchanged.
// cos_t / sin_t: bf16-rounded table over the rotary / 2 frequencies.
QD_DEVINL void norm_rope_row(const bf16* __restrict__ src, const bf16* __restrict__ gamma_w, int d, int rotary,
                             float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int lane,
                             float* __restrict__ dst) {
    float v[8], g[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = j * 32 + lane;
        v[j] = i < d ? ldcg_bf16(src + i) : 0.f;
        g[j] = i < d ? ld_bf16(gamma_w + i) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = round_bf16((v[j] * inv) * (1.0f + g[j]));
    const int hj = rotary / 64;                 // registers per half of the rotary part
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (j < hj) {
            const float c = cos_t[j * 32 + lane], sn = sin_t[j * 32 + lane];
            const float lo = v[j], hi = v[j + hj];
            v[j] = round_bf16(lo * c + (-hi) * sn);
            v[j + hj] = round_bf16(hi * c + lo * sn);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = j * 32 + lane;
        if (i < d) dst[i] = v[j];
    }
}

// Gated GQA decode attention, first half (quickdraw/models/qwen.py:66-116): block = (KV head,
// context split).  The split is walked in chunks of sixteen positions staged in shared memory:
// scores (one warp per position, all query heads of the KV head), softmax update (one warp per
// head), weighted value sum (one thread per head and four features).  Writes the block's
// partials: unnormalised sum, running max and denominator per head.
QD_DEVINL void attn_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int pi, int& it) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = mp.hq / mp.hkv;
    constexpr int D = 256;
    const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const int T = position + 1;
    const AttnSplit cut = attn_split(T, mp.attn_splits);
    const int unit = blockIdx.x;
    const int kvh = unit / cut.active, split = unit % cut.active;
    const int t0 = split * cut.per, t1 = min(T, t0 + cut.per);
    const bool mine = kvh < mp.hkv;
    float* q_s = reinterpret_cast<float*>(S.xs);            // [G][D]
    float* k_s = reinterpret_cast<float*>(S.xf);            // [D] the new key
    const float* cos_t = S.rope;                            // [rotary / 2], filled at kernel start
    const float* sin_t = S.rope + 128;
    float* sc = k_s + 256;                                  // [8][16] scores of the chunk
    float* pr = sc + 8 * kAttnChunk;                        // [8][16] softmax numerators
    float* fix = pr + 8 * kAttnChunk;                       // [8] rescale of the running sums
    const size_t layer_elems = (size_t)mp.st.capacity * mp.hkv * D;
    bf16* k_cache = reinterpret_cast<bf16*>(mp.st.kv_k) + (size_t)ph.state_index * layer_elems;
    bf16* v_cache = reinterpret_cast<bf16*>(mp.st.kv_v) + (size_t)ph.state_index * layer_elems;

    phase_wait(mp, S, pi, tid);
    if (tid == 0) trace_mark(mp, pi, 0);
    if (!mine) return;
    const bool owns_new = position >= t0 && position < t1;
    if (warp < G)
        norm_rope_row(ph.qg + (size_t)(kvh * G + warp) * 2 * D, ph.q_norm, D, mp.rotary, mp.eps, cos_t, sin_t, lane,
                      q_s + warp * D);
    if (owns_new && warp == CW - 1) {
        norm_rope_row(ph.k_new + (size_t)kvh * D, ph.k_norm, D, mp.rotary, mp.eps, cos_t, sin_t, lane, k_s);
        __syncwarp();
        bf16* krow = k_cache + ((size_t)position * mp.hkv + kvh) * D;
        bf16* vrow = v_cache + ((size_t)position * mp.hkv + kvh) * D;
        for (int i = lane; i < D; i += 32) {
            krow[i] = __float2bfloat16_rn(k_s[i]);
            vrow[i] = __float2bfloat16_rn(ldcg_bf16(ph.v_new + (size_t)kvh * D + i));
        }
    }
    QD_MARK(9);
    const float scale = rsqrtf((float)D);
    float m_run = -INFINITY, l_run = 0.f;            // warp h < G: running max / denominator of head h
    float acc[4] = {0.f, 0.f, 0.f, 0.f};             // thread (head tid / 64, features 4 (tid % 64) ..)
    const int ph_head = tid >> 6, pf = (tid & 63) * 4;
    bool ok = !*S.abort;
    named_barrier(1, CT);                  // q_s (and k_s) are complete
    uint32_t qp[4][4];                     // features 8 lane .. 8 lane + 7 of this warp's four heads, packed bf16
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const int head = min((warp & 1) * 4 + h, G - 1);
        const float4 qa = *reinterpret_cast<const float4*>(q_s + head * D + lane * 8);
        const float4 qb = *reinterpret_cast<const float4*>(q_s + head * D + lane * 8 + 4);
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(qa.x, qa.y), p1 = __floats2bfloat162_rn(qa.z, qa.w);
        const __nv_bfloat162 p2 = __floats2bfloat162_rn(qb.x, qb.y), p3 = __floats2bfloat162_rn(qb.z, qb.w);
        qp[h][0] = *reinterpret_cast<const uint32_t*>(&p0); qp[h][1] = *reinterpret_cast<const uint32_t*>(&p1);
        qp[h][2] = *reinterpret_cast<const uint32_t*>(&p2); qp[h][3] = *reinterpret_cast<const uint32_t*>(&p3);
    }
#pragma unroll 1
    for (int c0 = t0; c0 < t1 && ok; c0 += kAttnChunk, ++it) {
        // the producer streams the chunks of the split through the ring, ahead of this loop
        const int st = it % NS;
        if (!mbar_wait(S.full + st, (it / NS) & 1, mp.status)) { ok = false; break; }
        QD_MARK(12);
        uint8_t* buf = S.stages + (size_t)st * kStreamStageBytes;
        if (owns_new && position >= c0 && position < c0 + kAttnChunk && warp == CW - 1) {
            // the step's own row: key from the normalised vector, value from the projection
            const int tl = position - c0;
            bf16* kd = reinterpret_cast<bf16*>(buf + tl * kAttnRowBytes);
            bf16* vd = reinterpret_cast<bf16*>(buf + (kAttnChunk + tl) * kAttnRowBytes);
            for (int i = lane; i < D; i += 32) {
                kd[i] = __float2bfloat16_rn(k_s[i]);
                vd[i] = __float2bfloat16_rn(ldcg_bf16(ph.v_new + (size_t)kvh * D + i));
            }
        }
        named_barrier(1, CT);
        // scores: warp = (two positions of the chunk, one half of the heads); its query features
        // stay in registers for the whole split
        {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int tl = (warp >> 1) + half * 8;
                const int t = c0 + tl;
                const uint4 kr = lds128(buf + tl * kAttnRowBytes + lane * 16);
                const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w};
                // bf16 x bf16 products are exact in the mixed-precision fma: no unpacking
                float dots[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    float dot = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        dot = fma_bf16_lo(qp[h][j], kw[j], dot);
                        dot = fma_bf16_hi(qp[h][j], kw[j], dot);
                    }
                    dots[h] = dot;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int h = 0; h < 4; ++h) dots[h] += __shfl_xor_sync(0xffffffffu, dots[h], o);
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const int head = (warp & 1) * 4 + h;
                    if (head < G && lane == h) sc[head * kAttnChunk + tl] = t < t1 ? dots[h] * scale : -INFINITY;
                }
            }
        }
        QD_MARK(13);
        named_barrier(1, CT);
        // softmax update: warp = head
        if (warp < G) {
            const float s_t = lane < kAttnChunk ? sc[warp * kAttnChunk + lane] : -INFINITY;
            const float nm = fmaxf(m_run, warp_max(s_t));
            const float p = s_t == -INFINITY ? 0.f : expf(s_t - nm);
            const float fx = m_run == -INFINITY ? 0.f : expf(m_run - nm);
            l_run = l_run * fx + warp_sum(p);
            m_run = nm;
            if (lane < kAttnChunk) pr[warp * kAttnChunk + lane] = p;
            if (lane == 0) fix[warp] = fx;
        }
        QD_MARK(14);
        named_barrier(1, CT);
        // weighted values: thread = (head, four features)
        if (ph_head < G) {
            const float fx = fix[ph_head];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] *= fx;
            const uint8_t* vb = buf + kAttnChunk * kAttnRowBytes + pf * 2;
            const int valid = min(kAttnChunk, t1 - c0);      // rows past the split hold stale bytes
#pragma unroll
            for (int t = 0; t < kAttnChunk; ++t) {
                if (t >= valid) break;
                const float p = pr[ph_head * kAttnChunk + t];
                const uint2 vv = *reinterpret_cast<const uint2*>(vb + t * kAttnRowBytes);
                acc[0] += p * __uint_as_float(vv.x << 16);
                acc[1] += p * __uint_as_float(vv.x & 0xffff0000u);
                acc[2] += p * __uint_as_float(vv.y << 16);
                acc[3] += p * __uint_as_float(vv.y & 0xffff0000u);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.empty + st);
    }
    if (!ok && lane == 0) give_up(mp, S);
    QD_MARK(10);
    float* block_out = mp.attn_partial + (((size_t)kvh * mp.attn_splits + split) * G) * kAttnStride;
    if (ph_head < G) {
        float* dst = block_out + (size_t)ph_head * kAttnStride + pf;
        *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(dst + 2) = make_float2(acc[2], acc[3]);
    }
    if (warp < G && lane == 0) {
        block_out[(size_t)warp * kAttnStride + 256] = m_run;
        block_out[(size_t)warp * kAttnStride + 257] = l_run;
    }
    QD_MARK(11);
}

// Second half: block = (query head, 32 output features); warp w merges the splits w, w + 16, ...
// (all its loads in flight at once), warp 0 merges the sixteen results, normalises and applies
// the sigmoid gate.
QD_DEVINL void attn_merge_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int pi) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = mp.hq / mp.hkv;
    constexpr int D = 256;
    const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const AttnSplit cut = attn_split(position + 1, mp.attn_splits);
    float* part = S.scratch;                  // [16 warps][34]: 32 sums, max, denominator
    phase_wait(mp, S, pi, tid);
    if (tid == 0) trace_mark(mp, pi, 0);
    const int units = mp.hq * (D / 32);
#pragma unroll 1
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int qh = unit / (D / 32), f = (unit % (D / 32)) * 32 + lane;
        const int kvh = qh / G, h = qh % G;
        const float* base = mp.attn_partial + ((size_t)kvh * mp.attn_splits * G + h) * kAttnStride;
        const float gate_raw = warp == 0 ? ldcg_bf16(ph.qg + (size_t)qh * 2 * D + D + f) : 0.f;
        constexpr int PER = (kMegaAttnSplits + CW - 1) / CW;      // splits per warp at most
        float ms[PER], ls[PER], as[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int sp = warp + CW * k;
            const float* src = base + (size_t)sp * G * kAttnStride;
            const bool on = sp < cut.active;
            ms[k] = on ? __ldcg(src + 256) : -INFINITY;
            ls[k] = on ? __ldcg(src + 257) : 0.f;
            as[k] = on ? __ldcg(src + f) : 0.f;
        }
        float mm = ms[0];
#pragma unroll
        for (int k = 1; k < PER; ++k) mm = fmaxf(mm, ms[k]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const float w = ms[k] == -INFINITY ? 0.f : expf(ms[k] - mm);
            num += w * as[k];
            den += w * ls[k];
        }
        part[warp * 34 + lane] = num;
        if (lane == 0) { part[warp * 34 + 32] = mm; part[warp * 34 + 33] = den; }
        named_barrier(1, CT);
        if (warp == 0) {
            float top = -INFINITY;
#pragma unroll
            for (int w = 0; w < CW; ++w) top = fmaxf(top, part[w * 34 + 32]);
            float n2 = 0.f, d2 = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) {
                const float mw = part[w * 34 + 32];
                const float wv = mw == -INFINITY ? 0.f : expf(mw - top);
                n2 += wv * part[w * 34 + lane];
                d2 += wv * part[w * 34 + 33];
            }
            const float attended = round_bf16(n2 / d2);
            const float gate = round_bf16(sigmoid_precise(gate_raw));
            ph.mix_out[(size_t)qh * D + f] = __float2bfloat16_rn(attended * gate);
        }
        named_barrier(1, CT);
    }
}

// One down-projection row (512 inputs) by a half-warp: lane hl holds inputs [32 hl, 32 hl + 32).
QD_DEVINL float down_row(const uint8_t* base, int r, int hl, const uint32_t (&xh)[16]) {
    const uint4 w = lds128(base + r * (kDownWidth / 2) + hl * 16);
    const float2 sc = e4m3x2_to_float2(*reinterpret_cast<const uint16_t*>(
        base + kMegaDownRows * (kDownWidth / 2) + r * (kDownWidth / 16) + hl * 2));
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t h2[4];
        e2m1x8_to_f16x2(words[q], h2);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            g[(q >> 1) * 2] = fma_f16_lo(h2[b], xh[q * 4 + b], g[(q >> 1) * 2]);
            g[(q >> 1) * 2 + 1] = fma_f16_hi(h2[b], xh[q * 4 + b], g[(q >> 1) * 2 + 1]);
        }
    }
    float acc = fmaf(sc.x, g[0] + g[1], 0.f);
    acc = fmaf(sc.y, g[2] + g[3], acc);
    return group_sum<16>(acc);
}

// Routed and shared down projections with the combine (quickdraw/models/qwen.py:185-193):
// warp s works on slot s, each half-warp on alternate rows, two rows in flight; rounding
// points as in moe.cu.  The rows were fetched into the scratch area during the gate/up phase.
QD_DEVINL void down_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int pi) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = mp.hidden;
    const int r0 = (int)((long long)H * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)H * (blockIdx.x + 1) / gridDim.x);
    const int n = r1 - r0, nslots = mp.topk + 1;
    float* contrib = reinterpret_cast<float*>(S.xs);                         // [slots][kMegaDownRows]
    int* order = reinterpret_cast<int*>(contrib + kDownSlots * kMegaDownRows);   // [topk]
    // the routing of this layer has been in shared memory since the gate/up phase: the global
    // scale of this warp's expert is a static input, fetched before the barrier
    const int s = warp;
    const bool worker = s < nslots;
    const bool shared = s == mp.topk;
    const int e = (worker && !shared) ? S.ids[s] : 0;
    const bool owned = worker && (shared || (e >= mp.expert_lo && e < mp.expert_hi));
    const int hl = lane & 15, half = lane >> 4;
    float global_scale = 0.f;
    if (worker) global_scale = shared ? ph.sg[0] : ph.dg[ph.g_per_expert ? e - mp.expert_lo : 0];
    phase_wait(mp, S, pi, tid);
    if (tid == 0) trace_mark(mp, pi, 0);
    const float strength = tid < kMegaDownRows ? ldcg_bf16(ph.strength) : 0.f;    // in flight during the rows
    bool ok = !*S.abort;
    if (worker && ok) {
        uint32_t xh[16];
        uint32_t m2 = 0u;          // largest |bf16| bit pattern, per 16-bit half
        const uint32_t* src = reinterpret_cast<const uint32_t*>(ph.hidden + (size_t)s * kDownWidth) + hl * 16;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + j));
            xh[j] = v.x; xh[j + 1] = v.y; xh[j + 2] = v.z; xh[j + 3] = v.w;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) m2 = max_u16x2(m2, xh[j] & 0x7fff7fffu);
        uint32_t m = max(m2 & 0xffffu, m2 >> 16);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        // |x| < 2^(exponent + 1); scale down by a power of two only if f16 would overflow
        // (non-finite inputs are left alone)
        const int exponent = (int)(m >> 7) - 127;
        const int shift = (exponent > 14 && exponent < 128) ? exponent - 14 : 0;
        const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
        const float mult = __uint_as_float((uint32_t)(127 + shift) << 23);
#pragma unroll
        for (int j = 0; j < 16; ++j) xh[j] = pack_f16x2(__uint_as_float(xh[j] << 16) * down,
                                                       __uint_as_float(xh[j] & 0xffff0000u) * down);
        const float scale = shared ? global_scale : round_bf16(global_scale * S.weights[s]);
        QD_MARK(8);
        ok = mbar_wait(S.down_bar, ph.layer & 1, mp.status);
        QD_MARK(9);
        const uint8_t* base = reinterpret_cast<const uint8_t*>(S.scratch) + (size_t)s * kMegaDownRows * kDownRowBytes;
        if (ok) {
#pragma unroll 1
            for (int rr = 0; rr < n; rr += 4) {
                // both half-warps run the same iterations (the shuffles name all 32 lanes); a
                // half-warp past the last row recomputes it and does not store
                const int ra = min(rr + half, n - 1), rb = min(rr + 2 + half, n - 1);
                float va = 0.f, vb = 0.f;
                if (owned) {
                    const float acc_a = down_row(base, ra, hl, xh) * mult;
                    const float acc_b = down_row(base, rb, hl, xh) * mult;
                    va = shared ? round_bf16(acc_a * scale) : round_bf16(round_bf16(acc_a) * scale);
                    vb = shared ? round_bf16(acc_b * scale) : round_bf16(round_bf16(acc_b) * scale);
                }
                if (hl == 0 && rr + half < n) contrib[s * kMegaDownRows + ra] = va;
                if (hl == 0 && rr + 2 + half < n) contrib[s * kMegaDownRows + rb] = vb;
            }
        }
    } else if (warp == CW - 1 && lane < mp.topk) {
        // slots in ascending expert id: the order the routed rows are summed in
        const int id = S.ids[lane];
        int rank = 0;
        for (int q = 0; q < mp.topk; ++q) rank += S.ids[q] < id;
        order[rank] = lane;
    }
    QD_MARK(10);
    if (!ok && lane == 0) give_up(mp, S);
    named_barrier(1, CT);
    QD_MARK(11);
    if (tid < n && ok) {
        float routed = 0.f;
        for (int k = 0; k < mp.topk; ++k) routed += contrib[order[k] * kMegaDownRows + tid];
        const float gate = round_bf16(sigmoid_precise(strength));
        const float shared_row = round_bf16(contrib[mp.topk * kMegaDownRows + tid] * gate);
        ph.out[r0 + tid] = __float2bfloat16_rn(round_bf16(routed) + shared_row);
    }
    // the scratch area goes back to the mixer core of the next layer and, after that, to the
    // next bulk copies: order this thread's reads and writes of it before those
    fence_proxy_async();
}

__global__ void __launch_bounds__(kMegaThreads, 1)
mega_kernel(const __grid_constant__ MegaParams mp) {
    const Smem S = carve_smem(mega_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((int)gridDim.x != mp.grid) {            // the program was laid out for another grid
        if (tid == 0) atomicOr(mp.status, QD_STATUS_BAD_SHAPE);
        return;
    }
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(S.full + s, 1); mbar_init(S.empty + s, CW); }
        mbar_init(S.ids_bar, 1);
        mbar_init(S.down_bar, 1);
        mbar_fence_init();
        *S.abort = 0;
        *S.flag = 0;
    }
    __syncthreads();
    if (warp == CW) {
        producer(mp, S, lane);
        return;
    }
    // rotation table of this step's position, once for all attention layers
    // (quickdraw/models/qwen.py:84-88: fp32 angle, cos / sin rounded to bf16)
    if (mp.rotary > 0) {
        const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
        for (int f = tid; f < mp.rotary / 2; f += CT) {
            const float inv_freq = 1.0f / powf(mp.theta, (float)(2 * f) / (float)mp.rotary);
            const float angle = (float)position * inv_freq;
            S.rope[f] = round_bf16(cosf(angle));
            S.rope[128 + f] = round_bf16(sinf(angle));
        }
    }
    // first phase parameters
    {
        const uint4* src = reinterpret_cast<const uint4*>(mp.program);
        uint4* dst = reinterpret_cast<uint4*>(S.cph);
        for (int i = tid; i < (int)(sizeof(MegaPhase) / 16); i += CT) dst[i] = __ldg(src + i);
    }
    named_barrier(1, CT);
    int it = 0;
#pragma unroll 1
    for (int pi = 0; pi < mp.nphases; ++pi) {
        const MegaPhase& ph = S.cph[pi & 1];
        if (pi + 1 < mp.nphases) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(mp.program + pi + 1);
            uint8_t* dst = reinterpret_cast<uint8_t*>(S.cph + ((pi + 1) & 1));
            for (int i = tid; i < (int)(sizeof(MegaPhase) / 16); i += CT) cp_async16(dst + i * 16, src + i * 16);
        }
        if (ph.kind == MK_STREAM) {
            if (ph.width == 2048) stream_phase<2, true>(mp, ph, S, pi, it);
            else stream_phase<4, false>(mp, ph, S, pi, it);
        } else if (ph.kind == MK_GDN) {
            gdn_phase(mp, ph, S, pi);
        } else if (ph.kind == MK_ATTN) {
            attn_phase(mp, ph, S, pi, it);
        } else if (ph.kind == MK_ATTN_MERGE) {
            attn_merge_phase(mp, ph, S, pi);
        } else {
            down_phase(mp, ph, S, pi);
        }
        cp_async_wait_all();
        fence_proxy_async();      // scratch and ring bytes this thread touched may be bulk-copy targets next
        if (tid == 0) trace_mark(mp, pi, 1);
        named_barrier(1, CT);
        // release: this block's writes (ordered before it by the block barrier) are visible to
        // whoever acquires the new count
        if (tid == 0 && pi + 1 < mp.nphases) red_release_add(mp.bar, 1u);
    }
    // the last block to leave resets the barrier words for the next launch
    if (tid == 0) {
        __threadfence();
        const unsigned int gone = atomicAdd(mp.exit_count, 1u);
        if (gone == gridDim.x - 1) {
            *mp.bar = 0u;
            *mp.exit_count = 0u;
            __threadfence();
        }
    }
}

}  // namespace

size_t mega_smem_bytes() { return kSmemBytes; }

int mega_launch(const MegaParams& p, cudaStream_t stream) {
    static bool configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    if (!configured[dev]) {
        int limit = 0;
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if ((size_t)limit < kSmemBytes) return QD_ERR_UNSUPPORTED;
        if (cudaFuncSetAttribute(mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid); cfg.blockDim = dim3(kMegaThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all blocks resident at once: they wait for each other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, mega_kernel, p) == cudaSuccess ? QD_OK : QD_ERR_LAUNCH;
}

}  // namespace qd
