// Streaming matvec: one activation vector against a list of weight segments.
//
// Work split: the byte cost of all segments is cut into gridDim.x equal ranges; a block
// walks its range in tiles of whole rows.  A producer warp issues the bulk copies of a
// tile (codes and block scales are contiguous row blocks in the reference layout, so no
// repacking is needed) into a ring of shared-memory stages guarded by full/empty
// mbarriers; eight consumer warps take rows of the tile round-robin.  Each lane owns a
// fixed set of input positions, so its slice of the activation vector stays in
// registers for the whole kernel as packed f16 (scaled by a power of two when it would
// overflow f16; products of an E2M1 weight and a bf16 activation are exact in the
// mixed-precision fma, sums are fp32).
//
// Arithmetic contract (reference: quickdraw/models/qwen.py:36-54 and the rounding points
// of quickdraw/kernel/cute/matvec.py:62-77): fp32 accumulation, global scale applied to
// the finished sum, one bf16 rounding; SwiGLU rounds gate, up, silu(gate) and the product.
#include "stream.cuh"

namespace qd {

namespace {

struct TileCursor {      // identical walk for the producer and the consumers
    int seg, row, rows_here;
};

QD_DEVINL int seg_cost(const StreamSeg& s, int K) {
    const int fp4_row = K / 2 + K / 16;
    return s.kind == SEG_BF16 ? 2 * K : (s.kind == SEG_FP4_PAIR ? 2 * fp4_row : fp4_row);
}
QD_DEVINL int seg_tile_rows(const StreamSeg& s, int K) {
    return kStreamStageBytes / seg_cost(s, K);
}

// Row range [ra, rb) of segment `i` that falls into the block's byte range [lo, hi).
QD_DEVINL void seg_range(long long seg_start, int cost, int rows, long long lo, long long hi,
                         int& ra, int& rb) {
    const long long a = lo - seg_start, b = hi - seg_start;
    long long fa = a <= 0 ? 0 : (a + cost - 1) / cost;
    long long fb = b <= 0 ? 0 : (b + cost - 1) / cost;
    ra = (int)(fa > rows ? rows : fa);
    rb = (int)(fb > rows ? rows : fb);
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

// top-k routing by one warp, at most 256 experts (8 per lane); same rule as route_warp
// in ops.cu: fp32 softmax, lowest index wins ties, weights renormalised.
QD_DEVINL void route_small(const bf16* __restrict__ logits, int experts, int topk, int32_t* ids,
                           float* weights, int lane) {
    float p[8];
    float best = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = i * 32 + lane;
        p[i] = e < experts ? ld_bf16(logits + e) : -INFINITY;
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

template <int KC, bool WITH_BF16>
__global__ void __launch_bounds__(kStreamThreads, KC == 2 ? 2 : 1)
stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int K = KC * 1024;
    constexpr int CW = kStreamConsumerWarps;
    constexpr int NS = kStreamStages;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;
    bf16* xs = reinterpret_cast<bf16*>(smem + NS * kStreamStageBytes);           // [K]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + NS * kStreamStageBytes + K * 2);
    uint64_t* empty = full + NS;
    float* red = reinterpret_cast<float*>(empty + NS);      // [32] reduction scratch
    int32_t* s_ids = reinterpret_cast<int32_t*>(red + 32);  // [32]
    float* s_wts = reinterpret_cast<float*>(s_ids + 32);    // [32]
    int* s_abort = reinterpret_cast<int*>(s_wts + 32);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool routed = p.router_logits != nullptr || p.ids_in != nullptr;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, CW); }
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    grid_launch_dependents();

    // byte range of this block
    long long total = 0;
    for (int i = 0; i < p.nseg; ++i) total += (long long)p.seg[i].rows * seg_cost(p.seg[i], K);
    const long long lo = total * blockIdx.x / gridDim.x;
    const long long hi = total * (blockIdx.x + 1) / gridDim.x;

    if (warp == CW) {
        // ------------------------------------------------------------------ producer
        if (routed) {
            grid_dependency_wait();
            named_barrier(2, kStreamThreads);    // ids are in shared memory
        }
        if (lane == 0) {
            int it = 0;
            long long seg_start = 0;
            bool ok = true;
            for (int i = 0; i < p.nseg && ok; ++i) {
                const StreamSeg& sg = p.seg[i];
                const int cost = seg_cost(sg, K);
                int ra, rb;
                seg_range(seg_start, cost, sg.rows, lo, hi, ra, rb);
                seg_start += (long long)sg.rows * cost;
                int expert = 0;
                if (sg.slot >= 0) {
                    expert = s_ids[sg.slot];
                    if (expert < p.expert_lo || expert >= p.expert_hi) continue;
                    expert -= p.expert_lo;
                }
                const int tile_rows = seg_tile_rows(sg, K);
                const uint8_t* w = sg.w + (long long)expert * sg.w_stride;
                const uint8_t* s = sg.s ? sg.s + (long long)expert * sg.s_stride : nullptr;
                const uint8_t* w2 = sg.w2 ? sg.w2 + (long long)expert * sg.w_stride : nullptr;
                const uint8_t* s2 = sg.s2 ? sg.s2 + (long long)expert * sg.s_stride : nullptr;
                for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
                    const int n = min(tile_rows, rb - r0);
                    const int st = it % NS;
                    if (!mbar_wait(empty + st, ((it / NS) & 1) ^ 1, p.status)) { ok = false; break; }
                    uint8_t* dst = stages + st * kStreamStageBytes;
                    if (sg.kind == SEG_BF16) {
                        mbar_expect_tx(full + st, n * 2 * K);
                        bulk_load(dst, w + (long long)r0 * 2 * K, n * 2 * K, full + st);
                    } else if (sg.kind == SEG_FP4) {
                        mbar_expect_tx(full + st, n * (K / 2 + K / 16));
                        bulk_load(dst, w + (long long)r0 * (K / 2), n * (K / 2), full + st);
                        bulk_load(dst + tile_rows * (K / 2), s + (long long)r0 * (K / 16), n * (K / 16), full + st);
                    } else {
                        mbar_expect_tx(full + st, 2 * n * (K / 2 + K / 16));
                        uint8_t* sc = dst + 2 * tile_rows * (K / 2);
                        bulk_load(dst, w + (long long)r0 * (K / 2), n * (K / 2), full + st);
                        bulk_load(dst + tile_rows * (K / 2), w2 + (long long)r0 * (K / 2), n * (K / 2), full + st);
                        bulk_load(sc, s + (long long)r0 * (K / 16), n * (K / 16), full + st);
                        bulk_load(sc + tile_rows * (K / 16), s2 + (long long)r0 * (K / 16), n * (K / 16), full + st);
                    }
                }
            }
            if (!ok) *s_abort = 1;
            // Do not leave while copies are in flight: wait for the consumers to drain the ring
            // (bounded); every stage is empty again once its last tile has been released.
            for (int back = 1; back <= NS && back <= it; ++back) {
                const int j = it - back;
                mbar_wait(empty + (j % NS), (j / NS) & 1, ok ? p.status : nullptr);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    grid_dependency_wait();
    const int ctid = tid;                      // 0 .. CW*32-1
    constexpr int CT = CW * 32;
    const bf16* xin = p.token ? p.embed + (size_t)(*p.token) * K : p.x;
    // 1. activation vector into shared memory (bf16)
    if (p.prologue == PRO_ADD_NORM) {
        float v[K / CT];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < K / CT; ++j) {
            const int i = j * CT + ctid;
            v[j] = ld_bf16(xin + i) + (p.residual ? ld_bf16(p.residual + i) : 0.f);
            ss += v[j] * v[j];
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        named_barrier(1, CT);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) tot += red[w];
        const float inv = rsqrtf(tot / (float)K + p.eps);
#pragma unroll
        for (int j = 0; j < K / CT; ++j) {
            const int i = j * CT + ctid;
            const bf16 n = __float2bfloat16_rn((v[j] * inv) * p.gamma[i]);
            xs[i] = n;
            if (blockIdx.x == 0) {
                if (p.x_out) p.x_out[i] = n;
                p.residual_out[i] = __float2bfloat16_rn(v[j]);
            }
        }
    } else if (p.prologue == PRO_GATED_NORM) {
        // per-head RMSNorm of o, times gamma, times silu(z); one warp per head, 128 wide
        // (reference: quickdraw/models/qwen.py:161-164)
        for (int h = warp; h < K / 128; h += CW) {
            float o[4], ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { o[j] = ld_bf16(xin + h * 128 + j * 32 + lane); ss += o[j] * o[j]; }
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / 128.f + p.eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = h * 128 + j * 32 + lane;
                const float zz = ld_bf16(p.z + i);
                const bf16 n = __float2bfloat16_rn(((o[j] * inv) * ld_bf16(p.head_gamma + j * 32 + lane)) * silu_precise(zz));
                xs[i] = n;
                if (blockIdx.x == 0 && p.x_out) p.x_out[i] = n;
            }
        }
    } else {
        for (int i = ctid; i < K / 8; i += CT)
            reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(xin)[i];
    }
    // 2. routing (warp 0), published to the producer
    if (routed) {
        if (warp == 0) {
            if (p.ids_in) {
                if (lane < p.topk) s_ids[lane] = p.ids_in[lane];
            } else {
                route_small(p.router_logits, p.experts, p.topk, s_ids, s_wts, lane);
                __syncwarp();
                if (blockIdx.x == 0 && lane < p.topk) {
                    if (p.ids_out) p.ids_out[lane] = s_ids[lane];
                    if (p.weights_out) p.weights_out[lane] = s_wts[lane];
                }
            }
        }
        named_barrier(2, kStreamThreads);
    } else {
        named_barrier(1, CT);
    }
    // 3. this lane's activation slices into registers
    uint32_t xh[KC][16];
    float out_mult = 1.f;
    {
        float amax = 0.f;
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
#pragma unroll
        for (int c = 0; c < KC; ++c)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t pr = xw[(c * 32 + lane) * 16 + j];
                xh[c][j] = pr;
                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(pr << 16)), fabsf(__uint_as_float(pr & 0xffff0000u))));
            }
        amax = warp_max(amax);
        int e = 0;
        if (amax > 0.f && amax < INFINITY) frexpf(amax, &e);
        const int shift = e > 15 ? e - 15 : 0;
        const float down = ldexpf(1.f, -shift);
        out_mult = ldexpf(1.f, shift);
#pragma unroll
        for (int c = 0; c < KC; ++c)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t pr = xh[c][j];
                const __half2 h = __floats2half2_rn(__uint_as_float(pr << 16) * down,
                                                    __uint_as_float(pr & 0xffff0000u) * down);
                xh[c][j] = *reinterpret_cast<const uint32_t*>(&h);
            }
    }
    constexpr int NB = WITH_BF16 ? K / 256 : 1;
    uint32_t xb[NB * 4];
    if (WITH_BF16) {
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
#pragma unroll
        for (int i = 0; i < NB; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) xb[i * 4 + j] = xw[(i * 32 + lane) * 4 + j];
    }

    // 4. tiles
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;
    int it = 0;
    long long seg_start = 0;
    bool ok = true;
    for (int i = 0; i < p.nseg && ok; ++i) {
        const StreamSeg& sg = p.seg[i];
        const int cost = seg_cost(sg, K);
        int ra, rb;
        seg_range(seg_start, cost, sg.rows, lo, hi, ra, rb);
        seg_start += (long long)sg.rows * cost;
        int expert = 0;
        if (sg.slot >= 0) {
            expert = s_ids[sg.slot];
            if (expert < p.expert_lo || expert >= p.expert_hi) continue;
            expert -= p.expert_lo;
        }
        const int tile_rows = seg_tile_rows(sg, K);
        const float g1 = sg.g ? sg.g[sg.g_per_expert ? expert : 0] : 1.f;
        const float g2 = sg.g2 ? sg.g2[sg.g_per_expert ? expert : 0] : 1.f;
        for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
            const int n = min(tile_rows, rb - r0);
            const int st = it % NS;
            if (!mbar_wait(full + st, (it / NS) & 1, p.status)) { ok = false; break; }
            const uint8_t* base = stages + st * kStreamStageBytes;
            for (int r = warp; r < n; r += CW) {
                const int row = r0 + r;
                float result;
                if (sg.kind == SEG_BF16) {
                    if (WITH_BF16) result = warp_sum(bf16_row_dot<NB>(base + (size_t)r * 2 * K, xb, lane));
                    else result = 0.f;
                } else if (sg.kind == SEG_FP4) {
                    const float acc = warp_sum(fp4_row_dot<KC>(base + r * (K / 2),
                                                               base + tile_rows * (K / 2) + r * (K / 16), xh, lane));
                    result = (acc * out_mult) * g1;
                } else {
                    const uint8_t* sc = base + 2 * tile_rows * (K / 2);
                    const float ag = warp_sum(fp4_row_dot<KC>(base + r * (K / 2), sc + r * (K / 16), xh, lane));
                    const float au = warp_sum(fp4_row_dot<KC>(base + (tile_rows + r) * (K / 2),
                                                              sc + (tile_rows + r) * (K / 16), xh, lane));
                    const float gate = round_bf16((ag * out_mult) * g1);
                    const float up = round_bf16((au * out_mult) * g2);
                    result = round_bf16(silu_precise(gate)) * up;
                }
                const bf16 rounded = __float2bfloat16_rn(result);
                if (sg.epilogue == EP_CONV) {
                    // depthwise causal conv for this channel (quickdraw/models/qwen.py:134-136):
                    // lane t < W-1 holds history tap t, lane W-1 the new value.
                    const int W = p.conv_width;
                    bf16* hist = p.conv_state + (size_t)row * (W - 1);
                    float val = 0.f, tap = 0.f;
                    if (lane < W) {
                        tap = ld_bf16(p.conv_taps + (size_t)row * W + lane);
                        val = lane < W - 1 ? ld_bf16(hist + lane) : __bfloat162float(rounded);
                    }
                    const float conv = warp_sum(lane < W ? round_bf16(val * tap) : 0.f);
                    __syncwarp();
                    if (lane >= 1 && lane < W) hist[lane - 1] = __float2bfloat16_rn(val);
                    if (lane == 0) sg.y[row] = __float2bfloat16_rn(silu_precise(conv));
                } else {
                    if (lane == 0) sg.y[row] = rounded;
                    if (sg.epilogue == EP_ARGMAX) {
                        const float v = __bfloat162float(rounded);
                        if (v > best_val || (v == best_val && row < best_idx)) { best_val = v; best_idx = row; }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);
        }
    }
    // 5. greedy argmax over the EP_ARGMAX segment (ties: lowest index)
    if (p.best_val != nullptr) {
        if (lane == 0) { red[warp] = best_val; s_ids[warp + 16] = best_idx; }   // s_ids[16..] unused by routing
        named_barrier(1, CT);
        if (ctid == 0) {
            float bv = red[0]; int bi = s_ids[16];
            for (int w = 1; w < CW; ++w) {
                const float v = red[w]; const int ix = s_ids[16 + w];
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            p.best_val[blockIdx.x] = bv;
            p.best_idx[blockIdx.x] = bi;
            __threadfence();
            const unsigned int done = atomicAdd(p.counter, 1u);
            if (done == gridDim.x - 1) {
                __threadfence();
                float fv = -INFINITY; int fi = 0x7fffffff;
                for (int b = 0; b < (int)gridDim.x; ++b) {
                    const float v = reinterpret_cast<volatile float*>(p.best_val)[b];
                    const int ix = reinterpret_cast<volatile int*>(p.best_idx)[b];
                    if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
                }
                *p.token_out = fi == 0x7fffffff ? 0 : fi;
                *p.counter = 0;      // ready for the next launch / graph replay
            }
        }
    }
}

int g_sm_count = 0;

}  // namespace

int stream_sm_count() {
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

template <int KC, bool WITH_BF16>
static int launch_variant(const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
    constexpr int K = KC * 1024;
    const size_t smem = kStreamStages * kStreamStageBytes + K * 2 + 2 * kStreamStages * 8 + 32 * 4 * 3 + 16;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(stream_kernel<KC, WITH_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return QD_ERR_LAUNCH;
        configured = true;
    }
    return qd_launch(stream_kernel<KC, WITH_BF16>, dim3(grid), dim3(kStreamThreads), smem, stream, pdl, p);
}

int stream_launch(const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
    if (grid <= 0) grid = stream_sm_count();
    bool has_bf16 = false;
    for (int i = 0; i < p.nseg; ++i) has_bf16 |= p.seg[i].kind == SEG_BF16;
    if (p.width == 2048) return has_bf16 ? launch_variant<2, true>(p, grid, stream, pdl)
                                         : launch_variant<2, false>(p, grid, stream, pdl);
    if (p.width == 4096 && !has_bf16) return launch_variant<4, false>(p, grid, stream, pdl);
    return QD_ERR_UNSUPPORTED;
}

}  // namespace qd

// ------------------------------------------------------------ op-table entry (ops.cu)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int qd_stream_matvec_try(const Fp4Args& a, cudaStream_t stream) {
    using namespace qd;
    if (a.group != 16 || (a.in_features != 2048 && a.in_features != 4096)) return QD_ERR_UNSUPPORTED;
    if (a.routing || a.per_slot_input || a.slots > kStreamMaxSeg) return QD_ERR_UNSUPPORTED;
    if (!aligned16(a.x) || !aligned16(a.codes) || !aligned16(a.scales)) return QD_ERR_UNSUPPORTED;
    if (a.up_codes && (!aligned16(a.up_codes) || !aligned16(a.up_scales))) return QD_ERR_UNSUPPORTED;
    if (a.ids && (a.rows % 1) != 0) return QD_ERR_UNSUPPORTED;
    StreamParams p = {};
    p.width = a.in_features;
    p.prologue = PRO_NONE;
    p.x = a.x;
    p.nseg = a.slots;
    p.expert_lo = 0; p.expert_hi = 0x7fffffff;
    if (a.ids) { p.ids_in = a.ids; p.topk = a.slots; }
    for (int s = 0; s < a.slots; ++s) {
        StreamSeg& sg = p.seg[s];
        sg.w = a.codes; sg.s = a.scales; sg.g = a.global;
        sg.w2 = a.up_codes; sg.s2 = a.up_scales; sg.g2 = a.up_global;
        sg.y = a.y + (size_t)s * a.rows;
        sg.rows = a.rows;
        sg.kind = a.up_codes ? SEG_FP4_PAIR : SEG_FP4;
        sg.epilogue = EP_PLAIN;
        sg.slot = a.ids ? s : -1;
        sg.g_per_expert = a.global_per_expert;
        sg.w_stride = (long long)a.rows * (a.in_features / 2);
        sg.s_stride = (long long)a.rows * (a.in_features / 16);
    }
    return stream_launch(p, 0, stream, false);
}
