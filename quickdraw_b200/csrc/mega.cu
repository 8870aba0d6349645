// Persistent decode kernel: one cooperative launch per token, no grid-wide barrier.
//
// The grid is one block per SM.  A block has sixteen consumer warps and one producer warp.
// The producer walks the program phase by phase and streams this block's share of every
// phase's weights (and, for attention, its slice of the KV cache) into a ring of
// shared-memory stages (bulk copies, full/empty mbarriers); it never waits for other blocks
// except where the weights to fetch depend on the routing, so when the consumers reach a
// phase the ring already holds its first tiles.
//
// Blocks hand activations to each other through L2 as tagged words (mega.cuh): a consumer
// re-reads the words it needs until they carry the tag of this launch and layer, so a phase
// starts in a block as soon as ITS inputs exist.  The residual stream never leaves the
// block: every block adds and normalises the whole hidden vector itself (it needs the whole
// vector for its rows anyway) and keeps the bf16 residual in registers.
//
// NVFP4 rows run on the warp-level tensor-core instruction with the inputs split over the
// sixteen warps (rowmma.cuh); attention is a split-context flash decode on the same
// instruction (all query heads of a KV head share each key/value tile).
//
// Arithmetic follows the separate kernels (stream.cu, gdn.cu, moe.cu, attention.cu): same
// rounding points (reference: quickdraw/models/qwen.py:66-241), fp32 sums in a different order.
//
// Every wait is bounded.  A wait that runs out sets the status word and the block's abort
// flag; the block then stops waiting, finishes the token with whatever it has (its outputs
// still carry their tags, so no other block waits for it) and leaves.
#include "mega.cuh"
#include "rowdot.cuh"
#include "attn_mma.cuh"
#include "rowmma.cuh"

namespace qd {
namespace {

constexpr int CW = kMegaConsumerWarps, CT = kMegaConsumers, NS = kMegaStages;
constexpr int kDownWidth = 512;
constexpr int kDownRowBytes = kDownWidth / 2 + kDownWidth / 16;   // 288
constexpr int kDownSlots = 9;                                     // top-8 + shared
constexpr int kDownSlotBytes = kMegaDownRows * kDownRowBytes;     // codes [16][256] then scales [16][32]
constexpr int kDownBufBytes = kDownSlots * kDownSlotBytes;        // down-projection rows of one layer
constexpr int kAttnStagePos = 32;              // positions per ring stage: K rows, then V rows
constexpr int kAttnWarps = 8;                  // warps that walk the context (a chunk of sixteen positions each)
constexpr int kAttnStride = 258;               // partial of one head: 256 sums, running max, denominator
constexpr int kAttnMergeFloats = 8 * 256 + 16; // one warp's partial in shared memory during the block merge
constexpr int kScratchBytes = kDownBufBytes > 4 * kAttnMergeFloats * 4 ? kDownBufBytes : 4 * kAttnMergeFloats * 4;

struct Smem {
    uint8_t* stages;
    bf16* xs;              // [4096] activation vector, bf16   (attention: query heads, new key; down: hidden vectors)
    uint8_t* xf;           // [4096] the same as f16, natural order
    uint8_t* scratch;      // down-projection rows / DeltaNet vectors / attention merge
    float* partials;       // [NS][16 warps][32] partial row sums of the tile in each stage
    bf16* conv_taps; bf16* conv_state;
    MegaPhase* cph;        // [2] consumer copies of the current and the next phase
    MegaPhase* pph;        // producer copy
    uint64_t* full; uint64_t* empty; uint64_t* ready;
    float* red;            // [160]: reductions, per-segment global scales, the f16 scale of the kept vector
    int32_t* ids; float* weights;      // [8] routing of the current layer
    uint64_t* ids_bar;                 // completes once per layer, when the routing is in ids / weights
    uint64_t* down_bar;                // completes once per layer, when the down-projection rows have landed
    volatile int* abort;
    float* rope;           // [2][128] bf16-rounded cos / sin of the step's position, per rotary frequency
};

extern __shared__ __align__(128) uint8_t mega_smem[];

constexpr size_t kSmemBytes = (size_t)NS * kStreamStageBytes + 4096 * 2 + 4096 * 2 + (size_t)kScratchBytes +
                              (size_t)NS * kRowPartialFloats * 4 + 2 * kMegaConvRows * kStreamConvWidth * 2 +
                              3 * sizeof(MegaPhase) + 3 * NS * 8 + 160 * 4 + 8 * 4 + 8 * 4 + 16 + 16 + 2 * 128 * 4;

QD_DEVINL Smem carve_smem(uint8_t* base) {
    Smem s;
    s.stages = base;                                  base += (size_t)NS * kStreamStageBytes;
    s.xs = reinterpret_cast<bf16*>(base);             base += 4096 * 2;
    s.xf = base;                                      base += 4096 * 2;
    s.scratch = base;                                 base += (size_t)kScratchBytes;
    s.partials = reinterpret_cast<float*>(base);      base += (size_t)NS * kRowPartialFloats * 4;
    s.conv_taps = reinterpret_cast<bf16*>(base);      base += kMegaConvRows * kStreamConvWidth * 2;
    s.conv_state = reinterpret_cast<bf16*>(base);     base += kMegaConvRows * kStreamConvWidth * 2;
    s.cph = reinterpret_cast<MegaPhase*>(base);       base += 2 * sizeof(MegaPhase);
    s.pph = reinterpret_cast<MegaPhase*>(base);       base += sizeof(MegaPhase);
    s.full = reinterpret_cast<uint64_t*>(base);       base += NS * 8;
    s.empty = reinterpret_cast<uint64_t*>(base);      base += NS * 8;
    s.ready = reinterpret_cast<uint64_t*>(base);      base += NS * 8;
    s.red = reinterpret_cast<float*>(base);           base += 160 * 4;
    s.ids = reinterpret_cast<int32_t*>(base);         base += 8 * 4;
    s.weights = reinterpret_cast<float*>(base);       base += 8 * 4;
    s.ids_bar = reinterpret_cast<uint64_t*>(base);    base += 8;
    s.down_bar = reinterpret_cast<uint64_t*>(base);   base += 8;
    s.abort = reinterpret_cast<volatile int*>(base);  base += 16;
    s.rope = reinterpret_cast<float*>(base);          base += 2 * 128 * 4;
    return s;
}

// ------------------------------------------------------------------ tagged words
// Loads and stores of the words blocks exchange: relaxed, GPU scope (system scope for the words
// other GPUs write or read), straight to and from L2.
QD_DEVINL uint4 ld_words4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
QD_DEVINL uint32_t ld_word(const void* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
QD_DEVINL uint32_t ld_word_sys(const void* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
QD_DEVINL uint2 ld_pair(const void* p) {       // one 64-bit {value, tag} word
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return make_uint2((uint32_t)v, (uint32_t)(v >> 32));
}
QD_DEVINL uint2 ld_pair_sys(const void* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return make_uint2((uint32_t)v, (uint32_t)(v >> 32));
}
QD_DEVINL void st_word(void* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
QD_DEVINL void st_word_sys(void* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
QD_DEVINL void st_pair_sys(void* p, uint32_t value, uint32_t tag) {
    const unsigned long long v = (unsigned long long)value | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// two {value, tag} words in one 16-byte store; each 64-bit half validates itself on the reader's side
QD_DEVINL void st_pairs2(void* p, uint32_t v0, uint32_t v1, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v0), "r"(tag), "r"(v1), "r"(tag) : "memory");
}
QD_DEVINL uint32_t make_word(bf16 v, uint32_t tag) { return (uint32_t)__bfloat16_as_ushort(v) | (tag << 16); }
QD_DEVINL float word_value(uint32_t w) { return __uint_as_float(w << 16); }
QD_DEVINL bool tags4(const uint4& v, uint32_t tag) {
    return ((v.x >> 16) == tag) & ((v.y >> 16) == tag) & ((v.z >> 16) == tag) & ((v.w >> 16) == tag);
}

struct Wait {                 // what a bounded wait needs, and the launch number for 32-bit tags
    unsigned int* status; volatile int* abort; unsigned long long limit_ns;
    unsigned int launch;
};
QD_DEVINL bool wait_expired(const Wait& w, unsigned long long start) {
    if (*w.abort) return true;
    if (global_timer_ns() - start <= w.limit_ns) return false;
    atomicOr(w.status, QD_STATUS_WAIT_TIMEOUT);
    *w.abort = 1;
    return true;
}
static __device__ __noinline__ uint4 wait_words4_slow(const tagged* p, uint32_t tag, Wait w) {
    const unsigned long long start = global_timer_ns();
    uint4 v;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) { v = ld_words4(p); if (tags4(v, tag)) return v; }
        if (wait_expired(w, start)) return v;
    }
}
// Four consecutive tagged words (16-byte aligned), re-read until all carry `tag`.
QD_DEVINL uint4 wait_words4(const tagged* p, uint32_t tag, const Wait& w) {
    const uint4 v = ld_words4(p);
    if (tags4(v, tag)) return v;
    return wait_words4_slow(p, tag, w);
}
static __device__ __noinline__ uint32_t wait_word_slow(const tagged* p, uint32_t tag, Wait w, bool sys) {
    const unsigned long long start = global_timer_ns();
    uint32_t v;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) { v = sys ? ld_word_sys(p) : ld_word(p); if ((v >> 16) == tag) return v; }
        if (wait_expired(w, start)) return v;
    }
}
QD_DEVINL uint32_t wait_word(const tagged* p, uint32_t tag, const Wait& w, bool sys = false) {
    const uint32_t v = sys ? ld_word_sys(p) : ld_word(p);
    if ((v >> 16) == tag) return v;
    return wait_word_slow(p, tag, w, sys);
}
static __device__ __noinline__ uint32_t wait_pair_slow(const uint2* p, uint32_t tag, Wait w, bool sys) {
    const unsigned long long start = global_timer_ns();
    uint2 v;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) { v = sys ? ld_pair_sys(p) : ld_pair(p); if (v.y == tag) return v.x; }
        if (wait_expired(w, start)) return v.x;
    }
}
// One {fp32 bits, 32-bit tag} word; returns the value bits.
QD_DEVINL uint32_t wait_pair(const uint2* p, uint32_t tag, const Wait& w, bool sys = false) {
    const uint2 v = sys ? ld_pair_sys(p) : ld_pair(p);
    if (v.y == tag) return v.x;
    return wait_pair_slow(p, tag, w, sys);
}

// Several items at once: all loads are in flight together (one trip to L2 when the data is
// there), then only the missing ones are read again.  on[i] = false leaves item i alone.
template <int N>
QD_DEVINL void wait_words_n(const tagged* const (&p)[N], const bool (&on)[N], uint32_t tag, uint32_t (&v)[N], const Wait& w,
                            bool sys = false) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = on[i] ? (sys ? ld_word_sys(p[i]) : ld_word(p[i])) : (tag << 16);
    bool all = true;
#pragma unroll
    for (int i = 0; i < N; ++i) all &= (v[i] >> 16) == tag;
    if (all) return;
    const unsigned long long start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int rep = 0; rep < 8; ++rep) {
            all = true;
#pragma unroll
            for (int i = 0; i < N; ++i)
                if ((v[i] >> 16) != tag) { v[i] = sys ? ld_word_sys(p[i]) : ld_word(p[i]); all &= (v[i] >> 16) == tag; }
            if (all) return;
        }
        if (wait_expired(w, start)) return;
    }
}
// PRELOADED: v already holds a first read of every item (issued earlier, so that its trip to L2
// overlapped other work).
template <int N, bool PRELOADED = false>
QD_DEVINL void wait_words4_n(const tagged* const (&p)[N], const bool (&on)[N], uint32_t tag, uint4 (&v)[N], const Wait& w) {
    const uint32_t filled = tag << 16;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        if (!on[i]) v[i] = make_uint4(filled, filled, filled, filled);
        else if (!PRELOADED) v[i] = ld_words4(p[i]);
    }
    bool all = true;
#pragma unroll
    for (int i = 0; i < N; ++i) all &= tags4(v[i], tag);
    if (all) return;
    const unsigned long long start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int rep = 0; rep < 8; ++rep) {
            all = true;
#pragma unroll
            for (int i = 0; i < N; ++i)
                if (!tags4(v[i], tag)) { v[i] = ld_words4(p[i]); all &= tags4(v[i], tag); }
            if (all) return;
        }
        if (wait_expired(w, start)) return;
    }
}
template <int N>
QD_DEVINL void wait_pairs_n(const uint2* const (&p)[N], const bool (&on)[N], uint32_t tag, uint32_t (&v)[N], const Wait& w) {
    uint2 t[N];
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = on[i] ? ld_pair(p[i]) : make_uint2(0u, tag);
    bool all = true;
#pragma unroll
    for (int i = 0; i < N; ++i) all &= t[i].y == tag;
    if (!all) {
        const unsigned long long start = global_timer_ns();
        for (;;) {
#pragma unroll 1
            for (int rep = 0; rep < 8 && !all; ++rep) {
                all = true;
#pragma unroll
                for (int i = 0; i < N; ++i)
                    if (t[i].y != tag) { t[i] = ld_pair(p[i]); all &= t[i].y == tag; }
            }
            if (all || wait_expired(w, start)) break;
        }
    }
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = t[i].x;
}

QD_DEVINL void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
QD_DEVINL void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Orders this thread's earlier shared-memory accesses before later bulk copies into the same bytes.
QD_DEVINL void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Profiling: sixteen nanosecond timestamps per phase and block.  Slots: 0 phase entered,
// 1 phase left, 2 activation vector ready, 3 first tile landed, 4 / 5 first and last tile of
// the phase issued by the producer.
constexpr int kTraceSlots = 16;
QD_DEVINL void trace_mark(const MegaParams& mp, int pi, int slot) {
    if (mp.trace) mp.trace[((size_t)pi * kTraceSlots + slot) * gridDim.x + blockIdx.x] = global_timer_ns();
}

// This block's share [lo, hi) of a streaming phase, in cost units over the concatenated segments.
QD_DEVINL void block_cost_range(const MegaPhase& ph, unsigned& lo, unsigned& hi) {
    if (ph.seg_blocks) {
        const unsigned s = blockIdx.x / ph.seg_blocks, j = blockIdx.x % ph.seg_blocks;
        const unsigned end = (min(s, (unsigned)ph.nseg - 1u) + 1u) * ph.seg_cost;
        lo = s < (unsigned)ph.nseg ? min(s * ph.seg_cost + j * ph.block_cost, end) : end;
        hi = min(lo + ph.block_cost, end);
    } else {
        lo = blockIdx.x * ph.quota + min(blockIdx.x, ph.remainder);
        hi = (blockIdx.x + 1) * ph.quota + min(blockIdx.x + 1, ph.remainder);
    }
}

// =========================================================================== producer
template <int K>
QD_DEVINL bool produce_stream(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int& it) {
    bool ids_ready = false;
    unsigned lo, hi;
    block_cost_range(ph, lo, hi);
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
            } else if (sg.kind == SEG_FP8) {
                mbar_expect_tx(full, n * K);
                bulk_load(dst, w + (long long)r0 * K, n * K, full);
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

// Down projections: this block's output rows of every selected expert this rank owns and of
// the shared expert, into their own buffer (the scratch area, idle between the mixer core and
// the MoE tail).  Issued as soon as the routing is known, so the rows land during the gate/up phase.
QD_DEVINL void produce_down(const MegaParams& mp, const MegaPhase& ph, const Smem& S) {
    const int H = mp.hidden;
    const int r0 = (int)((long long)H * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)H * (blockIdx.x + 1) / gridDim.x);
    const int n = r1 - r0, nslots = mp.topk + 1;
    uint8_t* dst = S.scratch;
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
        uint8_t* d = dst + (size_t)s * kDownSlotBytes;
        bulk_load(d, w, n * (kDownWidth / 2), S.down_bar);
        bulk_load(d + kMegaDownRows * (kDownWidth / 2), sc, n * (kDownWidth / 16), S.down_bar);
    }
}

struct AttnSplit { int active, per; };
// How the context [0, T) is cut into splits of `per` positions (a multiple of the stage), one
// block per (KV head, split).
QD_DEVINL AttnSplit attn_split(int T, int max_splits) {
    AttnSplit a;
    const int per = (T + max_splits - 1) / max_splits;
    a.per = max(kAttnStagePos, (per + kAttnStagePos - 1) / kAttnStagePos * kAttnStagePos);
    a.active = (T + a.per - 1) / a.per;
    return a;
}

// Attention: the cache rows of this block's context split, thirty-two positions per ring stage
// (K rows then V rows, one 512-byte bulk copy each, issued by the whole warp).  The row of the
// step's own position is not in the cache yet; the consumers fill it in.  Rows of earlier
// positions were written by earlier steps, so these copies may run ahead like any weight.
QD_DEVINL bool produce_attn(const MegaParams& mp, const MegaPhase& ph, const Smem& S, int& it, int lane) {
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
    for (int c0 = t0; c0 < t1; c0 += kAttnStagePos, ++it) {
        const int st = it % NS;
        int ok = 1;
        if (lane == 0) ok = (!*S.abort && mbar_wait(S.empty + st, ((it / NS) & 1) ^ 1, mp.status)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        uint8_t* dst = S.stages + (size_t)st * kStreamStageBytes;
        const int t = c0 + lane;
        const bool copy = t < t1 && t != position;
        const int rows = __popc(__ballot_sync(0xffffffffu, copy));
        if (lane == 0) mbar_expect_tx(S.full + st, (uint32_t)rows * 2 * 512);
        __syncwarp();
        if (copy) {
            const size_t off = ((size_t)t * mp.hkv + kvh) * 512;
            bulk_load(dst + lane * kAttnRow, k_cache + off, 512, S.full + st);
            bulk_load(dst + (kAttnStagePos + lane) * kAttnRow, v_cache + off, 512, S.full + st);
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
        if (ph.kind == MK_STREAM) {
            if (lane == 0) {
                trace_mark(mp, pi, 4);
                if (ph.width == 2048) ok = produce_stream<2048>(mp, ph, S, it);
                else ok = produce_stream<4096>(mp, ph, S, it);
                // the routed gate/up phase also carries the down-projection pointers of its layer
                if (ok && ph.route) {
                    ok = mbar_wait(S.ids_bar, ph.layer & 1, mp.status);
                    if (ok) produce_down(mp, ph, S);
                }
                trace_mark(mp, pi, 5);
                if (!ok) *S.abort = 1;
            }
            it = __shfl_sync(0xffffffffu, it, 0);
        } else if (ph.kind == MK_ATTN) {
            ok = produce_attn(mp, ph, S, it, lane);
            if (!ok && lane == 0) *S.abort = 1;
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

// Top-k routing by one warp; the lane holds the logits of experts 8 lane .. 8 lane + 7: fp32
// softmax, lowest index wins ties, weights renormalised (quickdraw/models/qwen.py:174-177).
// The eight selections are integer warp reductions (probabilities are non-negative, so their
// bit patterns order like the values).
QD_DEVINL void route_regs(float (&p)[8], int experts, int topk, int32_t* ids, float* weights, int lane) {
    float best = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (lane * 8 + i >= experts) p[i] = -INFINITY;
        best = fmaxf(best, p[i]);
    }
    best = warp_max(best);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const bool on = lane * 8 + i < experts;
        p[i] = on ? expf(p[i] - best) : -1.f;
        if (on) sum += p[i];
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
        const int idx = __reduce_min_sync(0xffffffffu, __float_as_int(v) == top ? lane * 8 + slot : 0x7fffffff);
        const float value = __int_as_float(top);
        chosen += value;
        if (lane == s) { mine = value; my_id = idx; }
        if ((idx >> 3) == lane) {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (i == (idx & 7)) p[i] = -1.f;
        }
    }
    if (lane < topk) { ids[lane] = my_id; weights[lane] = mine / chosen; }
}

// Power-of-two down-scale that keeps a vector whose largest magnitude is `top` inside f16.
QD_DEVINL void f16_scale(float top, float& down, float& up) {
    const int exponent = (int)((__float_as_uint(top) >> 23) & 0xffu) - 127;     // |x| < 2^(exponent + 1)
    const int shift = (exponent > 14 && exponent < 128) ? exponent - 14 : 0;
    down = __uint_as_float((uint32_t)(127 - shift) << 23);
    up = __uint_as_float((uint32_t)(127 + shift) << 23);
}

// Greedy choice at the end of the LM head: this block's best (value, index) over its warps, the
// last block to arrive reduces over the blocks and, expert parallel, over the ranks (ties: lowest
// index).  Out of line: it runs once per token, the streaming phase once per phase.
static __device__ __noinline__ void head_argmax(const MegaParams& mp, const Smem& S, const Wait& wt, uint32_t tag_base,
                                                float best_val, int best_idx) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* red = S.red;

    // over the lanes first (NVFP4 head rows end in different lanes; bf16 rows leave every lane equal)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_val, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (ov > best_val || (ov == best_val && oi < best_idx)) { best_val = ov; best_idx = oi; }
    }
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
            if (mp.world > 1) {
                // every rank tells every rank its best (value, index); two sets alternate
                // from launch to launch
                const uint32_t launch = tag_base >> 6;
                const uint32_t tag32 = (launch << 8) | 0xA5u;
                const long long slot = mp.argmax_offset + (long long)((launch & 1u) * mp.world) * 16;
                for (int r = 0; r < mp.world; ++r) {
                    uint8_t* dst = reinterpret_cast<uint8_t*>(mp.peer_base[r]) + slot + (long long)mp.rank * 16;
                    st_pair_sys(dst, __float_as_uint(fv), tag32);
                    st_pair_sys(dst + 8, (uint32_t)fi, tag32);
                }
                const uint8_t* own = reinterpret_cast<const uint8_t*>(mp.peer_base[mp.rank]) + slot;
                for (int r = 0; r < mp.world; ++r) {
                    const float v = __uint_as_float(wait_pair(reinterpret_cast<const uint2*>(own + r * 16), tag32, wt, true));
                    const int ix = (int)wait_pair(reinterpret_cast<const uint2*>(own + r * 16 + 8), tag32, wt, true);
                    if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
                }
            }
            *mp.next_token = fi == 0x7fffffff ? 0 : fi;
            *mp.argmax_counter = 0;
        }
    }
}

// Static FP8 activation (quickdraw/models/qwen.py:25-26): x / scale, clamped to the E4M3 range,
// rounded to nearest even; returned as the f16 that holds the E4M3 value exactly.
QD_DEVINL float fp8_quantised(float v, float in_scale) {
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(__fdiv_rn(v, in_scale), __NV_SATFINITE, __NV_E4M3);
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3)));
}

// ========================================================================== consumers
// One streaming phase: activation vector -> shared memory and registers, then this block's
// rows of the ring.  res: this thread's four elements of the bf16 residual stream.
template <int KC>
QD_DEVINL void stream_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, const Wait& wt, int pi, int& it,
                            float (&res)[4], uint32_t tag_base) {
    constexpr int K = KC * 1024;
    constexpr int UNITS = K / 2048;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bf16* xs = S.xs;
    uint8_t* xf = S.xf;
    float* red = S.red;
    const uint32_t tag = tag_base | (uint32_t)(ph.layer + 1);
    const uint32_t tag_x = ph.x_prev_layer ? tag - 1u : tag;
    unsigned lo, hi;
    block_cost_range(ph, lo, hi);

    // ---- first read of the activation words this thread needs: their trip to L2 overlaps the
    //      static loads below; they are checked, and read again if they have not arrived, later
    uint4 xin[4];
    const int mode = KC == 2 ? ((ph.keep_x || ph.from_token) ? 0 : 1) : (ph.prologue == PRO_GATED_NORM ? 2 : 3);
    const tagged* xsrc[4] = {ph.x, ph.x, ph.x, ph.x};
    bool xon[4] = {false, false, false, false};
    if (mode == 1) { xsrc[0] = ph.x + tid * 4; xon[0] = true; }
    if (mode == 2) {
        const int base0 = warp * 128 + lane * 4, base1 = (warp + CW) * 128 + lane * 4;
        xsrc[0] = ph.x + base0; xsrc[1] = ph.z + base0; xsrc[2] = ph.x + base1; xsrc[3] = ph.z + base1;
        xon[0] = xon[1] = xon[2] = xon[3] = true;
    }
    if (mode == 3) { xsrc[0] = ph.x + tid * 8; xsrc[1] = ph.x + tid * 8 + 4; xon[0] = xon[1] = true; }
#pragma unroll
    for (int i = 0; i < 4; ++i) if (xon[i]) xin[i] = ld_words4(xsrc[i]);

    // ---- static inputs (nothing another block writes): norm gamma, global scales of the
    //      segments, conv taps and history of this block's channels
    const bool q8 = ph.in_scale != nullptr;          // static FP8 projections: the vector is quantised first
    const float in_scale = q8 ? *ph.in_scale : 1.f;
    float4 gam = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (KC == 2) if (ph.prologue == PRO_ADD_NORM) gam = *reinterpret_cast<const float4*>(ph.gamma + tid * 4);
    if (tid < 2 * kMegaMaxSeg) {
        const MegaSeg& sg = ph.seg[tid >> 1];
        const float* src = (tid & 1) ? sg.g2 : sg.g;
        float v = 1.f;
        if ((tid >> 1) < ph.nseg && src && !sg.g_per_expert) v = *src;
        red[64 + (tid & 1) * 16 + (tid >> 1)] = v;
    }
    int conv_row0 = 0;
    bf16* conv_state = nullptr;
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
                const int conv_n = min(rb - ra, kMegaConvRows);
                if (tid < conv_n * W)
                    reinterpret_cast<unsigned short*>(S.conv_taps)[tid] =
                        reinterpret_cast<const unsigned short*>(ph.conv_taps)[(size_t)ra * W + tid];
                if (tid < conv_n * (W - 1))
                    reinterpret_cast<unsigned short*>(S.conv_state)[tid] =
                        reinterpret_cast<const unsigned short*>(conv_state)[(size_t)ra * (W - 1) + tid];
            }
            seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        }
    }

    wait_words4_n<4, true>(xsrc, xon, mode == 1 ? tag_x : tag, xin, wt);
    if (tid == 0) trace_mark(mp, pi, 6);

    // ---- the activation vector: bf16 (for bf16 rows) and f16 (for the tensor-core rows), the
    //      f16 copy scaled down by a power of two only if it would overflow
    float out_mult;
    if (KC == 4 || !ph.keep_x) {
        if (KC == 2) {
            // residual add + RMSNorm, four elements per thread (quickdraw/models/qwen.py:205-217)
            float v[4];
            if (ph.from_token) {
                const uint2 raw = *reinterpret_cast<const uint2*>(mp.embed + (size_t)(*mp.token) * K + tid * 4);
                v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
                v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
            } else {
                const uint4 w4 = xin[0];
                v[0] = word_value(w4.x) + res[0]; v[1] = word_value(w4.y) + res[1];
                v[2] = word_value(w4.z) + res[2]; v[3] = word_value(w4.w) + res[3];
            }
            const float g4[4] = {gam.x, gam.y, gam.z, gam.w};
            float ss = 0.f, top = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { ss += v[j] * v[j]; top = fmaxf(top, fabsf(v[j] * g4[j])); }
            ss = warp_sum(ss);
            top = warp_max(top);
            if (lane == 0) { red[warp] = ss; red[16 + warp] = top; }
            named_barrier(1, CT);
            float tot = 0.f, tmax = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) { tot += red[w]; tmax = fmaxf(tmax, red[16 + w]); }
            const float inv = rsqrtf(tot / (float)K + mp.eps);
            float down;
            f16_scale(tmax * inv * 1.01f, down, out_mult);
            float nrm[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                nrm[j] = round_bf16((v[j] * inv) * g4[j]);
                res[j] = round_bf16(v[j]);
            }
            const __nv_bfloat162 n01 = __floats2bfloat162_rn(nrm[0], nrm[1]), n23 = __floats2bfloat162_rn(nrm[2], nrm[3]);
            *reinterpret_cast<uint2*>(xs + tid * 4) = make_uint2(*reinterpret_cast<const uint32_t*>(&n01),
                                                                 *reinterpret_cast<const uint32_t*>(&n23));
            float f[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = q8 ? fp8_quantised(nrm[j], in_scale) : nrm[j] * down;
            if (q8) out_mult = in_scale;
            *reinterpret_cast<uint2*>(xf + tid * 8) = make_uint2(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]));
            if (tid == 0) red[96] = out_mult;
        } else if (KC == 4 && ph.prologue == PRO_GATED_NORM) {
            // per-head RMSNorm of o, times gamma, times silu(z); a warp per 128-wide head, four
            // consecutive features per lane (quickdraw/models/qwen.py:161-164)
            constexpr int HPW = K / 128 / CW;
            float nv[HPW][4];
            const uint2 graw = *reinterpret_cast<const uint2*>(ph.head_gamma + lane * 4);
            const float gm[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xffff0000u),
                                 __uint_as_float(graw.y << 16), __uint_as_float(graw.y & 0xffff0000u)};
            float top = 0.f;
#pragma unroll
            for (int a = 0; a < HPW; ++a) {
                const uint4 ow = xin[2 * a], zw = xin[2 * a + 1];
                const float o[4] = {word_value(ow.x), word_value(ow.y), word_value(ow.z), word_value(ow.w)};
                const float zz[4] = {word_value(zw.x), word_value(zw.y), word_value(zw.z), word_value(zw.w)};
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) ss += o[j] * o[j];
                ss = warp_sum(ss);
                const float inv = rsqrtf(ss / 128.f + mp.eps);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    nv[a][j] = round_bf16(((o[j] * inv) * gm[j]) * silu_precise(zz[j]));
                    top = fmaxf(top, fabsf(nv[a][j]));
                }
            }
            top = warp_max(top);
            if (lane == 0) red[16 + warp] = top;
            named_barrier(1, CT);
            float tmax = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) tmax = fmaxf(tmax, red[16 + w]);
            float down;
            f16_scale(tmax, down, out_mult);
#pragma unroll
            if (q8) out_mult = in_scale;
#pragma unroll
            for (int a = 0; a < HPW; ++a) {
                const int base = (warp + a * CW) * 128 + lane * 4;
                float f[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) f[j] = q8 ? fp8_quantised(nv[a][j], in_scale) : nv[a][j] * down;
                *reinterpret_cast<uint2*>(xf + base * 2) = make_uint2(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]));
            }
        } else {
            // the vector as it is (attention output): eight elements per thread
            const uint4 w0 = xin[0], w1 = xin[1];
            const float v[8] = {word_value(w0.x), word_value(w0.y), word_value(w0.z), word_value(w0.w),
                                word_value(w1.x), word_value(w1.y), word_value(w1.z), word_value(w1.w)};
            float top = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) top = fmaxf(top, fabsf(v[j]));
            top = warp_max(top);
            if (lane == 0) red[16 + warp] = top;
            named_barrier(1, CT);
            float tmax = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) tmax = fmaxf(tmax, red[16 + w]);
            float down;
            f16_scale(tmax, down, out_mult);
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = q8 ? fp8_quantised(v[j], in_scale) : v[j] * down;
            if (q8) out_mult = in_scale;
            *reinterpret_cast<uint4*>(xf + tid * 16) = make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]),
                                                                  pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
        }
        named_barrier(1, CT);
    } else {
        named_barrier(1, CT);    // the segment scales above are in shared memory
        out_mult = red[96];      // the vector (and its scale) the phase before left in shared memory
    }
    // ---- routing for this layer (every block selects the same experts from the same logits);
    //      the other warps go on with the shared expert's rows meanwhile
    if constexpr (KC == 2) if (ph.route && warp == 0) {
        float p[8];
        uint4 ab[2];
        {
            const bool have = lane * 8 < mp.experts;          // the expert count is a multiple of eight
            const tagged* const src[2] = {ph.router_logits + (have ? lane * 8 : 0), ph.router_logits + (have ? lane * 8 + 4 : 0)};
            const bool on[2] = {have, have};
            wait_words4_n<2>(src, on, tag, ab, wt);
        }
        const uint4 a = ab[0], b = ab[1];
        p[0] = word_value(a.x); p[1] = word_value(a.y); p[2] = word_value(a.z); p[3] = word_value(a.w);
        p[4] = word_value(b.x); p[5] = word_value(b.y); p[6] = word_value(b.z); p[7] = word_value(b.w);
        route_regs(p, mp.experts, mp.topk, S.ids, S.weights, lane);
        __syncwarp();
        if (blockIdx.x == 0 && lane < mp.topk) { ph.ids_out[lane] = S.ids[lane]; ph.weights_out[lane] = S.weights[lane]; }
        if (lane == 0) { mbar_arrive(S.ids_bar); trace_mark(mp, pi, 7); }
    }

    if (tid == 0) trace_mark(mp, pi, 2);
    uint32_t xh[UNITS][16];
    load_x_fragments<UNITS>(xf, warp, lane, xh);

    // ---- rows
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;
    bool first_tile = true, ids_ready = false;
    unsigned seg_start = 0;
    int turn = 0;                      // bf16 rows handed out so far: rotates the row -> warp map
    bool ok = true;
#pragma unroll 1
    for (int i = 0; i < ph.nseg && ok; ++i) {
        const MegaSeg& sg = ph.seg[i];
        int ra, rb;
        seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
        seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        if (ra >= rb) continue;
        int expert = 0;
        if (KC == 2 && sg.slot >= 0) {
            if (!ids_ready && !mbar_wait(S.ids_bar, ph.layer & 1, mp.status)) { ok = false; break; }
            ids_ready = true;
            expert = S.ids[sg.slot];
            if (expert < mp.expert_lo || expert >= mp.expert_hi) continue;
            expert -= mp.expert_lo;
        }
        const int tile_rows = seg_tile_rows<K>(sg.kind);
        const float g1 = (sg.g && sg.g_per_expert) ? sg.g[expert] : red[64 + i];
        const float g2 = (sg.g2 && sg.g_per_expert) ? sg.g2[expert] : red[80 + i];
#pragma unroll 1
        for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
            const int n = min(tile_rows, rb - r0);
            const int st = it % NS;
            if (!mbar_wait(S.full + st, (it / NS) & 1, mp.status)) { ok = false; break; }
            if (first_tile && tid == 0) trace_mark(mp, pi, 3);
            first_tile = false;
            const uint8_t* base = S.stages + (size_t)st * kStreamStageBytes;
            if (sg.kind == SEG_BF16) {
                if (lane == 0) mbar_arrive(S.ready + st);      // keeps the phase of `ready` in step with the ring
                if constexpr (KC == 2) {
#pragma unroll 1
                    for (int r = (warp - turn) & (CW - 1); r < n; r += CW) {
                        const int row = r0 + r;
                        const float result = warp_sum(bf16_row_dot_smem<K / 256>(base + (size_t)r * 2 * K,
                                                                                 reinterpret_cast<const uint8_t*>(xs), lane));
                        const bf16 rounded = __float2bfloat16_rn(result);
                        if (sg.epilogue == EP_ARGMAX) {
                            const int index = ph.row_lo + row;      // vocabulary index (the segment is this rank's shard)
                            if (lane == 0) mp.logits[index] = rounded;
                            const float v = __bfloat162float(rounded);
                            if (v > best_val || (v == best_val && index < best_idx)) { best_val = v; best_idx = index; }
                        } else if (lane == 0) {
                            st_word(sg.y + row, make_word(rounded, tag));
                        }
                    }
                    turn = (turn + n) & (CW - 1);
                }
            } else {
                const bool pair = KC == 2 && sg.kind == SEG_FP4_PAIR;
                const int groups = UNITS == 2 ? 1 : ((pair || n > 16) ? 2 : 1);
                float* mine = S.partials + st * kRowPartialFloats;
                if (sg.kind == SEG_FP8) tile_partials_fp8<K>(base, xh, warp, lane, mine + warp * kRowSlots);
                else tile_partials<K>(base, UNITS == 2 ? 16 : 32, groups, xh, warp, lane, mine + warp * kRowSlots);
                __syncwarp();
                if (lane == 0) mbar_arrive(S.ready + st);
                if (warp == (it & (CW - 1))) {
                    // this tile's finishing warp: lane = slot of the tile
                    if (!mbar_wait(S.ready + st, (it / NS) & 1, mp.status)) { ok = false; break; }
                    const float total = tile_sum(mine, lane);
                    float result = (total * out_mult) * g1;
                    if (pair) {
                        const float up_raw = __shfl_down_sync(0xffffffffu, total, 16);
                        const float up = round_bf16((up_raw * out_mult) * g2);
                        result = round_bf16(silu_precise(round_bf16(result))) * up;
                    }
                    const bf16 rounded = __float2bfloat16_rn(result);
                    const bool valid = lane < n && (!pair || lane < 16);
                    const int row = r0 + lane;
                    if (valid) {
                        if (KC == 2 && sg.epilogue == EP_CONV) {
                            // depthwise causal conv of this channel (quickdraw/models/qwen.py:134-136):
                            // history taps then the new value; products rounded to bf16, fp32 sum as
                            // (0 + 2) + (1 + 3)
                            const int W = mp.conv_width, local = row - conv_row0;
                            float prod[kStreamConvWidth];
#pragma unroll
                            for (int k = 0; k < kStreamConvWidth; ++k) {
                                float val = 0.f, tap = 0.f;
                                if (k < W) {
                                    tap = __bfloat162float(S.conv_taps[local * W + k]);
                                    val = k < W - 1 ? __bfloat162float(S.conv_state[local * (W - 1) + k]) : __bfloat162float(rounded);
                                    if (k >= 1) conv_state[(size_t)row * (W - 1) + k - 1] = __float2bfloat16_rn(val);
                                }
                                prod[k] = k < W ? round_bf16(val * tap) : 0.f;
                            }
                            const float conv = (prod[0] + prod[2]) + (prod[1] + prod[3]);
                            st_word(sg.y + row, make_word(__float2bfloat16_rn(silu_precise(conv)), tag));
                        } else if (KC == 2 && sg.epilogue == EP_ARGMAX) {
                            // an NVFP4 LM head: this lane's row is a vocabulary entry
                            const int index = ph.row_lo + row;
                            mp.logits[index] = rounded;
                            const float v = __bfloat162float(rounded);
                            if (v > best_val || (v == best_val && index < best_idx)) { best_val = v; best_idx = index; }
                        } else {
                            st_word(sg.y + row, make_word(rounded, tag));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(S.empty + st);
        }
    }
    if (tid == 0) trace_mark(mp, pi, 8);
    if (!ok && lane == 0) *S.abort = 1;
    if (KC == 2 && ph.argmax) head_argmax(mp, S, wt, tag_base, best_val, best_idx);
}

// Gated delta-rule recurrence (quickdraw/models/qwen.py:139-160) for 128-wide key heads:
// block = (value head, 32 value columns), 256 threads = 8 key groups x 32 columns, 16 state
// entries per thread, fetched before the inputs are waited for (only this block ever touches them).
QD_DEVINL void gdn_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, const Wait& wt, uint32_t tag_base) {
    constexpr int DK = 128, KPT = 16;
    const int tid = threadIdx.x, col = tid & 31, kg = tid >> 5;
    const int dv = mp.dv, hk = mp.hk, hv = mp.hv;
    const int slices = dv / 32;
    const int unit = blockIdx.x;
    if (unit >= hv * slices || tid >= 256) return;
    const uint32_t tag = tag_base | (uint32_t)(ph.layer + 1);
    const int head = unit / slices, c0 = (unit % slices) * 32;
    float* qs = reinterpret_cast<float*>(S.scratch);   // [128] q, normalised and scaled
    float* ks = qs + DK;              // [128] k, normalised
    float* part = ks + DK;            // [8][32]
    float* gates = part + 256;        // decay, beta
    float* tile = mp.st.rec_state + (size_t)ph.state_index * hv * DK * dv + (size_t)head * DK * dv + c0 + col;
    float s[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j) s[j] = tile[(size_t)(kg * KPT + j) * dv];
    const int key_head = head / (hv / hk);
    // everything this thread needs from the projections
    float v, qv = 0.f, kv = 0.f, av = 0.f, bv = 0.f;
    {
        const int kt = tid < DK ? tid : 0;
        const tagged* const src[5] = {ph.qkv + (size_t)2 * hk * DK + (size_t)head * dv + c0 + col,
                                      ph.qkv + (size_t)key_head * DK + kt,
                                      ph.qkv + (size_t)hk * DK + (size_t)key_head * DK + kt,
                                      ph.ab + head, ph.ab + hv + head};
        const bool on[5] = {true, tid < DK, tid < DK, tid == DK, tid == DK};
        uint32_t got[5];
        wait_words_n<5>(src, on, tag, got, wt);
        v = word_value(got[0]);
        if (tid < DK) { qv = word_value(got[1]); kv = word_value(got[2]); }
        if (tid == DK) { av = word_value(got[3]); bv = word_value(got[4]); }
    }
    const float qq = warp_sum(qv * qv), kk = warp_sum(kv * kv);
    if (col == 0) { part[kg * 32] = qq; part[kg * 32 + 1] = kk; }
    named_barrier(2, 256);
    if (tid < DK) {
        float tq = 0.f, tk = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) { tq += part[w * 32]; tk += part[w * 32 + 1]; }
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
        st_word(ph.mix_out + (size_t)head * dv + c0 + col, make_word(__float2bfloat16_rn(acc), tag));
    }
}

// RMSNorm with gamma = 1 + weight and partial RoPE of one head by one warp
// (quickdraw/models/qwen.py:76-92).  Feature i = j * 32 + lane, so with rotary / 2 a multiple
// of 32 the two features of a rotation pair sit in the same lane and nothing is exchanged.
// cos_t / sin_t: bf16-rounded table over the rotary / 2 frequencies.  dst: bf16 [d].
QD_DEVINL void norm_rope_row(const tagged* __restrict__ src, uint32_t tag, const Wait& wt, const bf16* __restrict__ gamma_w,
                             int d, int rotary, float eps, const float* __restrict__ cos_t,
                             const float* __restrict__ sin_t, int lane, bf16* __restrict__ dst) {
    float v[8], g[8];
    float ss = 0.f;
    {
        const tagged* p[8];
        bool on[8];
        uint32_t got[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { on[j] = j * 32 + lane < d; p[j] = src + (on[j] ? j * 32 + lane : 0); }
        wait_words_n<8>(p, on, tag, got, wt);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = on[j] ? word_value(got[j]) : 0.f;
            g[j] = on[j] ? ld_bf16(gamma_w + j * 32 + lane) : 0.f;
        }
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
        if (i < d) dst[i] = __float2bfloat16_rn(v[j]);
    }
}

// Gated GQA decode attention, first half (quickdraw/models/qwen.py:66-116): block = (KV head,
// context split).  The split arrives through the ring thirty-two positions at a time; warp
// w < 8 takes every eighth chunk of sixteen positions, the warps' results merge in shared
// memory, warp 0 writes the block's partial (unnormalised sums, running max, denominator).
QD_DEVINL void attn_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, const Wait& wt, int& it, uint32_t tag_base) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = mp.hq / mp.hkv;
    constexpr int D = 256;
    const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const int T = position + 1;
    const AttnSplit cut = attn_split(T, mp.attn_splits);
    const int unit = blockIdx.x;
    const int kvh = unit / cut.active, split = unit % cut.active;
    if (kvh >= mp.hkv) return;
    const uint32_t tag = tag_base | (uint32_t)(ph.layer + 1);
    const int t0 = split * cut.per, t1 = min(T, t0 + cut.per);
    uint8_t* q_s = reinterpret_cast<uint8_t*>(S.xs);                       // [8][kAttnQRow] bf16 query heads
    bf16* k_s = reinterpret_cast<bf16*>(q_s + 8 * kAttnQRow);              // [256] the new key
    bf16* v_s = k_s + D;                                                    // [256] the new value
    const float* cos_t = S.rope;
    const float* sin_t = S.rope + 128;
    const size_t layer_elems = (size_t)mp.st.capacity * mp.hkv * D;
    bf16* k_cache = reinterpret_cast<bf16*>(mp.st.kv_k) + (size_t)ph.state_index * layer_elems;
    bf16* v_cache = reinterpret_cast<bf16*>(mp.st.kv_v) + (size_t)ph.state_index * layer_elems;
    const bool owns_new = position >= t0 && position < t1;
    if (warp < 8) {
        if (warp < G) {
            norm_rope_row(ph.qg + (size_t)(kvh * G + warp) * 2 * D, tag, wt, ph.q_norm, D, mp.rotary, mp.eps, cos_t, sin_t,
                          lane, reinterpret_cast<bf16*>(q_s + warp * kAttnQRow));
        } else {
            for (int i = lane; i < D; i += 32) reinterpret_cast<bf16*>(q_s + warp * kAttnQRow)[i] = __float2bfloat16_rn(0.f);
        }
    } else if (owns_new && warp == CW - 1) {
        norm_rope_row(ph.kv_new + (size_t)kvh * D, tag, wt, ph.k_norm, D, mp.rotary, mp.eps, cos_t, sin_t, lane, k_s);
        bf16* krow = k_cache + ((size_t)position * mp.hkv + kvh) * D;
        bf16* vrow = v_cache + ((size_t)position * mp.hkv + kvh) * D;
        __syncwarp();
        {
            const tagged* p[8];
            bool on[8];
            uint32_t got[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { on[j] = true; p[j] = ph.kv_new + (size_t)(mp.hkv + kvh) * D + j * 32 + lane; }
            wait_words_n<8>(p, on, tag, got, wt);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = j * 32 + lane;
                const bf16 vv = __ushort_as_bfloat16((unsigned short)(got[j] & 0xffffu));
                v_s[i] = vv;
                vrow[i] = vv;
                krow[i] = k_s[i];
            }
        }
    }
    named_barrier(1, CT);                  // q_s (and the new row) are complete
    AttnAcc acc;
    acc.m = -INFINITY; acc.l = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc.out[i][0] = 0.f; acc.out[i][1] = 0.f; acc.out[i][2] = 0.f; acc.out[i][3] = 0.f; }
    bool ok = true;
    int chunk = 0;
#pragma unroll 1
    for (int c0 = t0; c0 < t1 && ok; c0 += kAttnStagePos, ++it) {
        const int st = it % NS;
        if (!mbar_wait(S.full + st, (it / NS) & 1, mp.status)) { ok = false; break; }
        uint8_t* buf = S.stages + (size_t)st * kStreamStageBytes;
        const bool has_new = owns_new && position >= c0 && position < c0 + kAttnStagePos;
        const bool ragged = c0 + kAttnStagePos > t1;
        if (has_new || ragged) {
            // the step's own row from the projections; value rows past the split hold stale bytes:
            // clear them (their probability is zero, but zero times a stale NaN is not)
            const int valid = min(kAttnStagePos, t1 - c0);
            for (int e = tid; e < (kAttnStagePos - valid) * (D / 8); e += CT) {
                const int r = valid + e / (D / 8), c = e % (D / 8);
                *reinterpret_cast<uint4*>(buf + (kAttnStagePos + r) * kAttnRow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            if (has_new && warp == CW - 1) {
                const int r = position - c0;
                for (int i = lane; i < D; i += 32) {
                    reinterpret_cast<bf16*>(buf + r * kAttnRow)[i] = k_s[i];
                    reinterpret_cast<bf16*>(buf + (kAttnStagePos + r) * kAttnRow)[i] = v_s[i];
                }
            }
            named_barrier(1, CT);
        }
        if (lane == 0) mbar_arrive(S.ready + st);      // keeps the phase of `ready` in step with the ring
#pragma unroll 1
        for (int h = 0; h < 2; ++h, ++chunk) {
            if (c0 + 16 * h >= t1) continue;
            if (warp == (chunk & (kAttnWarps - 1)))
                attn_chunk(acc, q_s, buf + (16 * h) * kAttnRow, buf + (kAttnStagePos + 16 * h) * kAttnRow, c0 + 16 * h, t1, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.empty + st);
    }
    if (!ok && lane == 0) *S.abort = 1;
    const int nchunks = (t1 - t0 + 15) / 16;
    const int active = min(kAttnWarps, nchunks);
    const int g = lane >> 2, t = lane & 3;
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 1);
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 2);
    // ---- merge of the warps: warps [s, 2 s) hand their state to warps [0, s)
    float* mbuf = reinterpret_cast<float*>(S.scratch);
#pragma unroll 1
    for (int s = kAttnWarps / 2; s >= 1; s >>= 1) {
        if (active <= s) continue;
        if (warp >= s && warp < 2 * s) {
            float* dst = mbuf + (size_t)(warp - s) * kAttnMergeFloats;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                *reinterpret_cast<float2*>(dst + (2 * t) * D + 32 * g + 2 * i) = make_float2(acc.out[i][0], acc.out[i][2]);
                *reinterpret_cast<float2*>(dst + (2 * t + 1) * D + 32 * g + 2 * i) = make_float2(acc.out[i][1], acc.out[i][3]);
            }
            if (t == 0) { dst[8 * D + g] = acc.m; dst[8 * D + 8 + g] = acc.l; }
        }
        named_barrier(1, CT);
        if (warp < s) {
            const float* src = mbuf + (size_t)warp * kAttnMergeFloats;
            const float m2 = src[8 * D + g], l2 = src[8 * D + 8 + g];
            const float m_new = fmaxf(acc.m, m2);
            const float f1 = acc.m == -INFINITY ? 0.f : expf(acc.m - m_new);
            const float f2 = m2 == -INFINITY ? 0.f : expf(m2 - m_new);
            acc.l = acc.l * f1 + l2 * f2;
            acc.m = m_new;
            const float f1e = __shfl_sync(0xffffffffu, f1, 8 * t), f1o = __shfl_sync(0xffffffffu, f1, 8 * t + 4);
            const float f2e = __shfl_sync(0xffffffffu, f2, 8 * t), f2o = __shfl_sync(0xffffffffu, f2, 8 * t + 4);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float2 e = *reinterpret_cast<const float2*>(src + (2 * t) * D + 32 * g + 2 * i);
                const float2 o = *reinterpret_cast<const float2*>(src + (2 * t + 1) * D + 32 * g + 2 * i);
                acc.out[i][0] = acc.out[i][0] * f1e + e.x * f2e;
                acc.out[i][2] = acc.out[i][2] * f1e + e.y * f2e;
                acc.out[i][1] = acc.out[i][1] * f1o + o.x * f2o;
                acc.out[i][3] = acc.out[i][3] * f1o + o.y * f2o;
            }
        }
        named_barrier(1, CT);
    }
    // ---- the block's partial: 64-bit {value, tag} words
    if (warp == 0) {
        const uint32_t tag32 = (wt.launch << 8) | (uint32_t)(ph.layer + 1);      // 24 bits of launch number: a split that is
        // not written for many launches (shorter contexts in between) must not be mistaken for a fresh one
        uint2* block_out = mp.attn_partial + (((size_t)kvh * mp.attn_splits + split) * 8) * kAttnStride;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            st_pairs2(block_out + (size_t)(2 * t) * kAttnStride + 32 * g + 2 * i, __float_as_uint(acc.out[i][0]),
                      __float_as_uint(acc.out[i][2]), tag32);
            st_pairs2(block_out + (size_t)(2 * t + 1) * kAttnStride + 32 * g + 2 * i, __float_as_uint(acc.out[i][1]),
                      __float_as_uint(acc.out[i][3]), tag32);
        }
        if (t == 0) st_pairs2(block_out + (size_t)g * kAttnStride + 256, __float_as_uint(acc.m), __float_as_uint(acc.l), tag32);
    }
}

// Second half: block = (query head, 32 output features); warp w merges the splits w, w + 16, ...
// (all its loads in flight at once), warp 0 merges the sixteen results, normalises and applies
// the sigmoid gate.
QD_DEVINL void attn_merge_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, const Wait& wt, uint32_t tag_base) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = mp.hq / mp.hkv;
    constexpr int D = 256;
    const int position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const AttnSplit cut = attn_split(position + 1, mp.attn_splits);
    const uint32_t tag = tag_base | (uint32_t)(ph.layer + 1);
    const uint32_t tag32 = (wt.launch << 8) | (uint32_t)(ph.layer + 1);      // 24 bits of launch number: a split that is
        // not written for many launches (shorter contexts in between) must not be mistaken for a fresh one
    float* part = reinterpret_cast<float*>(S.scratch);     // [16 warps][34]: 32 sums, max, denominator
    const int units = mp.hq * (D / 32);
#pragma unroll 1
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int qh = unit / (D / 32), f = (unit % (D / 32)) * 32 + lane;
        const int kvh = qh / G, h = qh % G;
        const uint2* base = mp.attn_partial + ((size_t)kvh * mp.attn_splits * 8 + h) * kAttnStride;
        constexpr int PER = (kMegaAttnSplits + CW - 1) / CW;      // splits per warp at most
        float ms[PER], ls[PER], as[PER];
        {
            const uint2* p[3 * PER];
            bool on[3 * PER];
            uint32_t got[3 * PER];
#pragma unroll
            for (int k = 0; k < PER; ++k) {
                const int sp = warp + CW * k;
                const bool have = sp < cut.active;
                const uint2* src = base + (size_t)(have ? sp : 0) * 8 * kAttnStride;
                p[3 * k] = src + 256; p[3 * k + 1] = src + 257; p[3 * k + 2] = src + f;
                on[3 * k] = on[3 * k + 1] = on[3 * k + 2] = have;
            }
            wait_pairs_n<3 * PER>(p, on, tag32, got, wt);
#pragma unroll
            for (int k = 0; k < PER; ++k) {
                const bool have = warp + CW * k < cut.active;
                ms[k] = have ? __uint_as_float(got[3 * k]) : -INFINITY;
                ls[k] = have ? __uint_as_float(got[3 * k + 1]) : 0.f;
                as[k] = have ? __uint_as_float(got[3 * k + 2]) : 0.f;
            }
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
            const float gate_raw = word_value(wait_word(ph.qg + (size_t)qh * 2 * D + D + f, tag, wt));
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
            st_word(ph.mix_out + (size_t)qh * D + f, make_word(__float2bfloat16_rn(attended * gate), tag));
        }
        named_barrier(1, CT);
    }
}

// Routed and shared down projections with the combine (quickdraw/models/qwen.py:185-193).
// The block owns up to sixteen output rows; their weight rows of every selected expert and of
// the shared expert were fetched into the scratch area during the gate/up phase.  A unit of
// work is (slot, span of 128 inputs): sixteen rows on the tensor cores, the units spread over
// the warps; then one thread per (slot, row) applies the scales and rounding points of moe.cu,
// and one thread per row adds the routed rows in ascending expert id and the gated shared row.
// Expert parallel: a rank multiplies the slots it owns and stores those contributions into
// every rank's copy of the layer's contribution table; the combine reads all eight slots
// from the local copy, so every rank forms the same sum in the same order as a single GPU.
QD_DEVINL void down_phase(const MegaParams& mp, const MegaPhase& ph, const Smem& S, const Wait& wt, uint32_t tag_base) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = mp.hidden;
    const int r0 = (int)((long long)H * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)H * (blockIdx.x + 1) / gridDim.x);
    const int n = r1 - r0, nslots = mp.topk + 1;
    const uint32_t tag = tag_base | (uint32_t)(ph.layer + 1);
    uint8_t* hx = reinterpret_cast<uint8_t*>(S.xs);                        // [slots][512] f16 (xs and xf are adjacent)
    float* dpart = S.partials;                                             // [36 units][16 rows]
    float* contrib = S.partials + 36 * 16;                                 // [slots][16]
    int* order = reinterpret_cast<int*>(contrib + kDownSlots * 16);        // [topk]
    float* smult = reinterpret_cast<float*>(order + 8);                    // [slots] f16 scale of each hidden vector
    float* red = S.red;
    // ---- the hidden vectors of the owned slots, 16 bytes (four words) per load: load k of
    //      thread tid covers words 4 (tid + 512 k) ..; slot = (tid >> 7) + 4 k
    float hv[3][4];
    float top[3] = {0.f, 0.f, 0.f};
    bool have[3];
    {
        const tagged* p[3];
        uint4 got[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const int idx = tid + CT * k, s = idx >> 7;
            have[k] = false;
            if (s < nslots) {
                const bool shared = s == mp.topk;
                const int e = shared ? 0 : S.ids[s];
                have[k] = shared || (e >= mp.expert_lo && e < mp.expert_hi);
            }
            p[k] = ph.hidden + (size_t)(have[k] ? idx : 0) * 4;
        }
        wait_words4_n<3>(p, have, tag, got, wt);
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            hv[k][0] = hv[k][1] = hv[k][2] = hv[k][3] = 0.f;
            if (have[k]) {
                hv[k][0] = word_value(got[k].x); hv[k][1] = word_value(got[k].y);
                hv[k][2] = word_value(got[k].z); hv[k][3] = word_value(got[k].w);
                top[k] = fmaxf(fmaxf(fabsf(hv[k][0]), fabsf(hv[k][1])), fmaxf(fabsf(hv[k][2]), fabsf(hv[k][3])));
            }
            top[k] = warp_max(top[k]);
            if (lane == 0) red[k * 16 + warp] = top[k];
        }
    }
    if (warp == CW - 1 && lane < mp.topk) {
        // slots in ascending expert id: the order the routed rows are summed in
        const int id = S.ids[lane];
        int rank = 0;
        for (int q = 0; q < mp.topk; ++q) rank += S.ids[q] < id;
        order[rank] = lane;
    }
    named_barrier(1, CT);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int idx = tid + CT * k, s = idx >> 7;
        if (s >= nslots) continue;
        const int w0 = (s & 3) * 4;
        const float tmax = fmaxf(fmaxf(red[k * 16 + w0], red[k * 16 + w0 + 1]), fmaxf(red[k * 16 + w0 + 2], red[k * 16 + w0 + 3]));
        float down, up;
        f16_scale(tmax, down, up);
        *reinterpret_cast<uint2*>(hx + (size_t)idx * 8) = make_uint2(pack_f16x2(hv[k][0] * down, hv[k][1] * down),
                                                                     pack_f16x2(hv[k][2] * down, hv[k][3] * down));
        if ((idx & 127) == 0) smult[s] = up;
    }
    bool ok = mbar_wait(S.down_bar, ph.layer & 1, mp.status);
    named_barrier(1, CT);
    // ---- units: (slot, span)
    {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll 1
        for (int u = warp; u < nslots * 4; u += CW) {
            const int s = u >> 2, span = (u & 3) ^ (g & 1);
            const bool shared = s == mp.topk;
            const int e = shared ? 0 : S.ids[s];
            if (!shared && (e < mp.expert_lo || e >= mp.expert_hi)) continue;
            uint32_t xh[16];
            const uint8_t* src = hx + ((size_t)s * kDownWidth + span * 128 + t * 32) * 2;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = lds128(src + q * 16);
                xh[q * 4 + 0] = v.x; xh[q * 4 + 1] = v.y; xh[q * 4 + 2] = v.z; xh[q * 4 + 3] = v.w;
            }
            const uint8_t* slot_base = S.scratch + (size_t)s * kDownSlotBytes;
            float aa[4] = {0.f, 0.f, 0.f, 0.f}, ab[4] = {0.f, 0.f, 0.f, 0.f};
            unit_mma(slot_base, slot_base + kMegaDownRows * (kDownWidth / 2), kDownWidth / 2, kDownWidth / 16, 0, span, g, t,
                     xh, aa, ab);
            if (t == (g >> 1)) {
                // the partial of span (u & 3) ^ (g & 1) of rows g and g + 8
                dpart[(s * 4 + span) * 16 + g] = (g & 1) ? aa[1] + ab[1] : aa[0] + ab[0];
                dpart[(s * 4 + span) * 16 + g + 8] = (g & 1) ? aa[3] + ab[3] : aa[2] + ab[2];
            }
        }
    }
    named_barrier(1, CT);
    // ---- one thread per (slot, row): scales and rounding
    if (tid < nslots * 16) {
        const int s = tid >> 4, r = tid & 15;
        const bool shared = s == mp.topk;
        const int e = shared ? 0 : S.ids[s];
        const bool owned = shared || (e >= mp.expert_lo && e < mp.expert_hi);
        if (owned && r < n) {
            const float acc = (((dpart[(s * 4 + 0) * 16 + r] + dpart[(s * 4 + 1) * 16 + r]) + dpart[(s * 4 + 2) * 16 + r]) +
                               dpart[(s * 4 + 3) * 16 + r]) * smult[s];
            float value;
            if (shared) {
                value = round_bf16(acc * ph.sg[0]);
            } else {
                const float global_scale = ph.dg[ph.g_per_expert ? e - mp.expert_lo : 0];
                value = round_bf16(round_bf16(acc) * round_bf16(global_scale * S.weights[s]));
            }
            contrib[s * 16 + r] = value;
            if (!shared && mp.world > 1) {
                const uint32_t word = make_word(__float2bfloat16_rn(value), tag);
                const long long off = mp.contrib_offset + ((long long)ph.layer * mp.topk * H + (long long)s * H + r0 + r) * 4;
                for (int rk = 0; rk < mp.world; ++rk)
                    st_word_sys(reinterpret_cast<uint8_t*>(mp.peer_base[rk]) + off, word);
            }
        }
    }
    named_barrier(1, CT);
    if (tid < n) {
        float routed = 0.f;
        if (mp.world > 1) {
            const tagged* mine = reinterpret_cast<const tagged*>(reinterpret_cast<const uint8_t*>(mp.peer_base[mp.rank]) +
                                                                  mp.contrib_offset) + (size_t)ph.layer * mp.topk * H;
            float c[8];
            {
                const tagged* p[8];
                bool on[8];
                uint32_t got[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) { on[k] = k < mp.topk; p[k] = mine + (size_t)order[on[k] ? k : 0] * H + r0 + tid; }
                wait_words_n<8>(p, on, tag, got, wt, true);
#pragma unroll
                for (int k = 0; k < 8; ++k) c[k] = on[k] ? word_value(got[k]) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) routed += c[k];
        } else {
            for (int k = 0; k < mp.topk; ++k) routed += contrib[order[k] * 16 + tid];
        }
        const float strength = word_value(wait_word(ph.strength, tag, wt));
        const float gate = round_bf16(sigmoid_precise(strength));
        const float shared_row = round_bf16(contrib[mp.topk * 16 + tid] * gate);
        st_word(ph.out + r0 + tid, make_word(__float2bfloat16_rn(round_bf16(routed) + shared_row), tag));
    }
    if (!ok && lane == 0) *S.abort = 1;
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
        for (int s = 0; s < NS; ++s) { mbar_init(S.full + s, 1); mbar_init(S.empty + s, CW); mbar_init(S.ready + s, CW); }
        mbar_init(S.ids_bar, 1);
        mbar_init(S.down_bar, 1);
        mbar_fence_init();
        *S.abort = 0;
    }
    // The launch number: part of every tag.  Read by every thread before any block can leave
    // (the last block to leave advances it).
    const uint32_t launch = *reinterpret_cast<volatile unsigned int*>(mp.epoch) + 1u;
    const uint32_t tag_base = (launch & 0x3ffu) << 6;
    __syncthreads();
    // A position outside the cache (it may come from a device scalar) touches nothing: every
    // block skips the token and the status word says so.
    const int step_position = mp.pos_dev ? *mp.pos_dev : mp.pos_host;
    const bool bad_position = step_position < 0 || step_position >= mp.st.capacity;
    if (bad_position) {
        if (tid == 0 && blockIdx.x == 0) atomicOr(mp.status, QD_STATUS_BAD_ARG);
    } else if (warp == CW) {
        producer(mp, S, lane);
    } else {
        Wait wt;
        wt.status = mp.status; wt.abort = S.abort; wt.limit_ns = (unsigned long long)mp.wait_limit_us * 1000ull; wt.launch = launch;
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
        float res[4] = {0.f, 0.f, 0.f, 0.f};
        int it = 0;
#pragma unroll 1
        for (int pi = 0; pi < mp.nphases; ++pi) {
            const MegaPhase& ph = S.cph[pi & 1];
            if (pi + 1 < mp.nphases) {
                const uint8_t* src = reinterpret_cast<const uint8_t*>(mp.program + pi + 1);
                uint8_t* dst = reinterpret_cast<uint8_t*>(S.cph + ((pi + 1) & 1));
                for (int i = tid; i < (int)(sizeof(MegaPhase) / 16); i += CT) cp_async16(dst + i * 16, src + i * 16);
            }
            if (tid == 0) trace_mark(mp, pi, 0);
            if (ph.kind == MK_STREAM) {
                if (ph.width == 2048) stream_phase<2>(mp, ph, S, wt, pi, it, res, tag_base);
                else stream_phase<4>(mp, ph, S, wt, pi, it, res, tag_base);
            } else if (ph.kind == MK_GDN) {
                gdn_phase(mp, ph, S, wt, tag_base);
            } else if (ph.kind == MK_ATTN) {
                attn_phase(mp, ph, S, wt, it, tag_base);
            } else if (ph.kind == MK_ATTN_MERGE) {
                attn_merge_phase(mp, ph, S, wt, tag_base);
            } else {
                down_phase(mp, ph, S, wt, tag_base);
            }
            cp_async_wait_all();
            fence_proxy_async();      // scratch and ring bytes this thread touched may be bulk-copy targets next
            if (tid == 0) trace_mark(mp, pi, 1);
            named_barrier(1, CT);
        }
    }
    // the last block to leave advances the launch number for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int gone = atomicAdd(mp.exit_count, 1u);
        if (gone == gridDim.x - 1) {
            *mp.epoch = launch;
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
