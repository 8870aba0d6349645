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
// Everything that does not depend on the previous launch (weights, norm gamma, conv taps
// and history) is fetched before the programmatic dependency wait; the code that runs once
// per block is kept short, because a block's first pass over cold code dominates the
// latency of a launch that only has a few tiles of work.
//
// Arithmetic contract (reference: quickdraw/models/qwen.py:36-54 and the rounding points
// of quickdraw/kernel/cute/matvec.py:62-77): fp32 accumulation, global scale applied to
// the finished sum, one bf16 rounding; SwiGLU rounds gate, up, silu(gate) and the product.
#include "stream.cuh"
#include "rowdot.cuh"

namespace qd {

int g_blocks_per_sm = 2;
unsigned long long* g_trace = nullptr;   // profiling: timestamps of every launch
int g_trace_launches = 0, g_trace_next = 0;
constexpr int kTraceStride = 1024 * 16;

namespace {


template <int KC, bool WITH_BF16>
__global__ void __launch_bounds__(kStreamThreads, KC == 2 ? 2 : 1)
stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int K = KC * 1024;
    constexpr int CW = kStreamConsumerWarps, CT = CW * 32, NS = kStreamStages;
    constexpr int EPT = K / CT;                       // prologue elements per thread (8 or 16)
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;
    bf16* xs = reinterpret_cast<bf16*>(smem + NS * kStreamStageBytes);                // [K]
    bf16* conv_taps_s = xs + K;                                                          // [rows][W]
    bf16* conv_state_s = conv_taps_s + kStreamConvRows * kStreamConvWidth;               // [rows][W-1]
    uint32_t* xf = reinterpret_cast<uint32_t*>(conv_state_s + kStreamConvRows * kStreamConvWidth);   // [K/2] f16 pairs
    uint64_t* full = reinterpret_cast<uint64_t*>(xf + K / 2);
    uint64_t* empty = full + NS;
    float* red = reinterpret_cast<float*>(empty + NS);      // [32]
    int32_t* s_ids = reinterpret_cast<int32_t*>(red + 32);  // [32]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, CW); }
        mbar_fence_init();
    }
    __syncthreads();
    grid_launch_dependents();
#define QD_TRACE(slot) do { if (p.trace && (tid == 0 || tid == CT)) p.trace[blockIdx.x * 16 + (tid ? 8 : 0) + (slot)] = global_timer_ns(); } while (0)
    QD_TRACE(0);

    // byte range of this block
    // total cost = quota * gridDim.x + remainder, split on the host
    const unsigned lo = blockIdx.x * p.quota + min(blockIdx.x, p.remainder);
    const unsigned hi = (blockIdx.x + 1) * p.quota + min(blockIdx.x + 1, p.remainder);

    if (warp == CW) {
        // ------------------------------------------------------------------ producer
        if (p.ids_in) grid_dependency_wait();      // bank entries depend on the routing
        if (lane == 0) {
            int it = 0;
            unsigned seg_start = 0;
            bool ok = true;
#pragma unroll 1
            for (int i = 0; i < p.nseg && ok; ++i) {
                const StreamSeg& sg = p.seg[i];
                int ra, rb;
                seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
                seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
                if (ra >= rb) continue;
                int expert = 0;
                if (sg.slot >= 0) {
                    expert = __ldcg(p.ids_in + sg.slot);
                    if (expert < p.expert_lo || expert >= p.expert_hi) continue;
                    expert -= p.expert_lo;
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
                    if (!mbar_wait(empty + st, ((it / NS) & 1) ^ 1, p.status)) { ok = false; break; }
                    uint8_t* dst = stages + st * kStreamStageBytes;
                    if (it == 0) QD_TRACE(1);
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
            QD_TRACE(2);
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
    // 0. before the dependency wait: norm gamma into registers, conv taps and history of this
    //    block's channels into shared memory (weights, and state the previous launch never writes)
    float gam[EPT];
    if (p.prologue == PRO_ADD_NORM) {
#pragma unroll
        for (int j = 0; j < EPT; j += 4) {
            const float4 gv = *reinterpret_cast<const float4*>(p.gamma + tid * EPT + j);
            gam[j] = gv.x; gam[j + 1] = gv.y; gam[j + 2] = gv.z; gam[j + 3] = gv.w;
        }
    }
    int conv_row0 = 0;
    {
        unsigned seg_start = 0;
#pragma unroll 1
        for (int i = 0; i < p.nseg; ++i) {
            const StreamSeg& sg = p.seg[i];
            if (sg.epilogue == EP_CONV) {
                int ra, rb;
                seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
                conv_row0 = ra;
                const int W = p.conv_width, n = min(rb - ra, kStreamConvRows);
                for (int e = tid; e < n * W; e += CT) conv_taps_s[e] = p.conv_taps[(size_t)ra * W + e];
                for (int e = tid; e < n * (W - 1); e += CT) conv_state_s[e] = p.conv_state[(size_t)ra * (W - 1) + e];
            }
            seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        }
    }
    grid_dependency_wait();
    QD_TRACE(5);
    const bf16* xin = p.token ? p.embed + (size_t)(*p.token) * K : p.x;
    uint32_t m2 = 0u;      // largest |bf16| bit pattern this thread produced, per 16-bit half
    // 1. activation vector into shared memory (bf16); thread i owns elements [EPT*i, EPT*i + EPT)
    if (p.prologue == PRO_ADD_NORM) {
        float v[EPT];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPT; j += 8) {
            const uint4 xa = *reinterpret_cast<const uint4*>(xin + tid * EPT + j);
            uint4 ra4 = make_uint4(0u, 0u, 0u, 0u);
            if (p.residual) ra4 = *reinterpret_cast<const uint4*>(p.residual + tid * EPT + j);
            const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w}, rw[4] = {ra4.x, ra4.y, ra4.z, ra4.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[j + 2 * q] = __uint_as_float(xw[q] << 16) + __uint_as_float(rw[q] << 16);
                v[j + 2 * q + 1] = __uint_as_float(xw[q] & 0xffff0000u) + __uint_as_float(rw[q] & 0xffff0000u);
            }
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) ss += v[j] * v[j];
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        named_barrier(1, CT);
        QD_TRACE(6);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) tot += red[w];
        const float inv = rsqrtf(tot / (float)K + p.eps);
#pragma unroll
        for (int j = 0; j < EPT; j += 8) {
            uint32_t nw[4], rw[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 n2 = __floats2bfloat162_rn((v[j + 2 * q] * inv) * gam[j + 2 * q],
                                                                (v[j + 2 * q + 1] * inv) * gam[j + 2 * q + 1]);
                const __nv_bfloat162 r2 = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                nw[q] = *reinterpret_cast<const uint32_t*>(&n2);
                rw[q] = *reinterpret_cast<const uint32_t*>(&r2);
                m2 = max_u16x2(m2, nw[q] & 0x7fff7fffu);
            }
            const uint4 nv = make_uint4(nw[0], nw[1], nw[2], nw[3]);
            *reinterpret_cast<uint4*>(xs + tid * EPT + j) = nv;
            if (blockIdx.x == 0) {
                if (p.x_out) *reinterpret_cast<uint4*>(p.x_out + tid * EPT + j) = nv;
                *reinterpret_cast<uint4*>(p.residual_out + tid * EPT + j) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
            }
        }
    } else if (p.prologue == PRO_GATED_NORM) {
        // per-head RMSNorm of o, times gamma, times silu(z); one warp per 128-wide head
        // (quickdraw/models/qwen.py:161-164)
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
                m2 = max(m2, (uint32_t)(__bfloat16_as_ushort(n) & 0x7fffu));
                if (blockIdx.x == 0 && p.x_out) p.x_out[i] = n;
            }
        }
    } else {
        for (int i = tid; i < K / 8; i += CT) {
            const uint4 v = reinterpret_cast<const uint4*>(xin)[i];
            reinterpret_cast<uint4*>(xs)[i] = v;
            m2 = max_u16x2(m2, v.x & 0x7fff7fffu); m2 = max_u16x2(m2, v.y & 0x7fff7fffu);
            m2 = max_u16x2(m2, v.z & 0x7fff7fffu); m2 = max_u16x2(m2, v.w & 0x7fff7fffu);
        }
    }
    {
        uint32_t m = max(m2 & 0xffffu, m2 >> 16);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) reinterpret_cast<uint32_t*>(red)[8 + warp] = m;
    }
    if (p.ids_in && warp == 0 && lane < p.topk) s_ids[lane] = __ldcg(p.ids_in + lane);
    QD_TRACE(7);
    named_barrier(1, CT);
    QD_TRACE(1);
    // 2. the vector as f16 pairs.  The largest bf16 magnitude (compared as a bit pattern)
    //    decides a common power-of-two down-scale so that nothing overflows f16 (one in the
    //    usual range); every thread converts its own slice into shared memory once, then each
    //    lane fetches the slices of its input positions.
    uint32_t xh[KC][16];
    float out_mult;
    {
        uint32_t m = 0u;
#pragma unroll
        for (int w = 0; w < CW; ++w) m = max(m, reinterpret_cast<const uint32_t*>(red)[8 + w]);
        const int exponent = (int)(m >> 7) - 127;            // |x| < 2^(exponent + 1)
        const int shift = exponent > 14 ? exponent - 14 : 0;
        const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
        out_mult = __uint_as_float((uint32_t)(127 + min(shift, 127)) << 23);
#pragma unroll
        for (int j = 0; j < EPT; j += 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xs + tid * EPT + j);
            uint4 h;
            h.x = pack_f16x2(__uint_as_float(v.x << 16) * down, __uint_as_float(v.x & 0xffff0000u) * down);
            h.y = pack_f16x2(__uint_as_float(v.y << 16) * down, __uint_as_float(v.y & 0xffff0000u) * down);
            h.z = pack_f16x2(__uint_as_float(v.z << 16) * down, __uint_as_float(v.z & 0xffff0000u) * down);
            h.w = pack_f16x2(__uint_as_float(v.w << 16) * down, __uint_as_float(v.w & 0xffff0000u) * down);
            *reinterpret_cast<uint4*>(xf + (tid * EPT + j) / 2) = h;
        }
        named_barrier(1, CT);
#pragma unroll
        for (int c = 0; c < KC; ++c)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = lds128(reinterpret_cast<const uint8_t*>(xf) + (c * 32 + lane) * 64 + q * 16);
                xh[c][q * 4 + 0] = v.x; xh[c][q * 4 + 1] = v.y; xh[c][q * 4 + 2] = v.z; xh[c][q * 4 + 3] = v.w;
            }
    }
    constexpr int NB = WITH_BF16 ? K / 256 : 1;
    uint32_t xb[NB * 4];
    if (WITH_BF16) {
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const uint4 v = lds128(reinterpret_cast<const uint8_t*>(xs) + (i * 32 + lane) * 16);
            xb[i * 4 + 0] = v.x; xb[i * 4 + 1] = v.y; xb[i * 4 + 2] = v.z; xb[i * 4 + 3] = v.w;
        }
    }
    QD_TRACE(2);

    // 3. tiles
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;
    int it = 0;
    unsigned seg_start = 0;
    bool ok = true;
#pragma unroll 1
    for (int i = 0; i < p.nseg && ok; ++i) {
        const StreamSeg& sg = p.seg[i];
        int ra, rb;
        seg_range<K>(seg_start, sg.kind, sg.rows, lo, hi, ra, rb);
        seg_start += (unsigned)sg.rows * seg_cost<K>(sg.kind);
        if (ra >= rb) continue;
        int expert = 0;
        if (sg.slot >= 0) {
            expert = s_ids[sg.slot];
            if (expert < p.expert_lo || expert >= p.expert_hi) continue;
            expert -= p.expert_lo;
        }
        const int tile_rows = seg_tile_rows<K>(sg.kind);
        const float g1 = sg.g ? sg.g[sg.g_per_expert ? expert : 0] : 1.f;
        const float g2 = sg.g2 ? sg.g2[sg.g_per_expert ? expert : 0] : 1.f;
#pragma unroll 1
        for (int r0 = ra; r0 < rb; r0 += tile_rows, ++it) {
            const int n = min(tile_rows, rb - r0);
            const int st = it % NS;
            if (!mbar_wait(full + st, (it / NS) & 1, p.status)) { ok = false; break; }
            if (it == 0) QD_TRACE(3);
            const uint8_t* base = stages + st * kStreamStageBytes;
#pragma unroll 1
            for (int r = warp; r < n; r += CW) {
                const int row = r0 + r;
                float result;
                if (sg.kind == SEG_BF16) {
                    if (WITH_BF16) result = warp_sum(bf16_row_dot<NB>(base + (size_t)r * 2 * K, xb, lane));
                    else result = 0.f;
                } else {
                    // one code path for plain rows and gate/up pairs: the pair's second half
                    // sits tile_rows rows further in both the code and the scale block
                    const int halves = sg.kind == SEG_FP4_PAIR ? 2 : 1;
                    const uint8_t* sc = base + halves * tile_rows * (K / 2);
                    float acc[2] = {0.f, 0.f};
#pragma unroll 1
                    for (int h = 0; h < halves; ++h)
                        acc[h] = warp_sum(fp4_row_dot<KC>(base + (h * tile_rows + r) * (K / 2),
                                                          sc + (h * tile_rows + r) * (K / 16), xh, lane));
                    result = (acc[0] * out_mult) * g1;
                    if (halves == 2) {
                        const float up = round_bf16((acc[1] * out_mult) * g2);
                        result = round_bf16(silu_precise(round_bf16(result))) * up;
                    }
                }
                const bf16 rounded = __float2bfloat16_rn(result);
                if (sg.epilogue == EP_CONV) {
                    // depthwise causal conv for this channel (quickdraw/models/qwen.py:134-136):
                    // lane t < W-1 holds history tap t, lane W-1 the new value.
                    const int W = p.conv_width, local = row - conv_row0;
                    float val = 0.f, tap = 0.f;
                    if (lane < W) {
                        tap = __bfloat162float(conv_taps_s[local * W + lane]);
                        val = lane < W - 1 ? __bfloat162float(conv_state_s[local * (W - 1) + lane]) : __bfloat162float(rounded);
                    }
                    const float conv = warp_sum(lane < W ? round_bf16(val * tap) : 0.f);
                    if (lane >= 1 && lane < W) p.conv_state[(size_t)row * (W - 1) + lane - 1] = __float2bfloat16_rn(val);
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
        if (sg.epilogue == EP_ROUTE) {
            // The block that completes the router rows selects the experts for the next launch.
            named_barrier(1, CT);
            if (warp == 0) {
                int last = 0;
                if (lane == 0) {
                    __threadfence();
                    const unsigned int before = atomicAdd(p.route_counter, (unsigned int)(rb - ra));
                    last = before + (unsigned int)(rb - ra) == (unsigned int)sg.rows;
                    if (last) __threadfence();
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    route_small(sg.y, sg.rows, p.route_topk, p.ids_out, p.weights_out, lane);
                    if (lane == 0) *p.route_counter = 0u;      // ready for the next launch / graph replay
                }
            }
        }
    }
    QD_TRACE(4);
    // 4. greedy argmax over the EP_ARGMAX segment (ties: lowest index)
    if (p.best_val != nullptr) {
        if (lane == 0) { red[warp] = best_val; s_ids[warp + 16] = best_idx; }   // s_ids[16..] is free
        named_barrier(1, CT);
        if (tid == 0) {
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
                    const float v = __ldcg(p.best_val + b);
                    const int ix = __ldcg(p.best_idx + b);
                    if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
                }
                *p.token_out = fi == 0x7fffffff ? 0 : fi;
                *p.counter = 0;      // ready for the next launch / graph replay
            }
        }
    }
}

int g_sm_count = 0;

template <int KC, bool WITH_BF16>
int launch_variant(const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
    constexpr int K = KC * 1024;
    const size_t smem = kStreamStages * kStreamStageBytes + K * 4 + 2 * kStreamConvRows * kStreamConvWidth * 2 +
                        2 * kStreamStages * 8 + 32 * 4 * 2 + 64;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(stream_kernel<KC, WITH_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return QD_ERR_LAUNCH;
        configured = true;
    }
    return qd_launch(stream_kernel<KC, WITH_BF16>, dim3(grid), dim3(kStreamThreads), smem, stream, pdl, p);
}

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

int stream_launch(const StreamParams& p_in, int grid, cudaStream_t stream, bool pdl) {
    StreamParams p = p_in;
    if (g_trace && g_trace_next < g_trace_launches) p.trace = g_trace + (size_t)(g_trace_next++) * kTraceStride;
    if (grid <= 0) grid = stream_sm_count() * (p.width == 2048 ? g_blocks_per_sm : 1);
    if (grid > 1024) grid = 1024;
    {
        unsigned long long total = 0;
        for (int i = 0; i < p.nseg; ++i) {
            const unsigned fp4_row = (p.width / 2 + p.width / 16) / 16;
            const unsigned cost = p.seg[i].kind == SEG_BF16 ? 2u * p.width / 16 : p.seg[i].kind == SEG_FP4_PAIR ? 2 * fp4_row : fp4_row;
            total += (unsigned long long)p.seg[i].rows * cost;
        }
        if (total + 1024 >= 0xffffffffull) return QD_ERR_UNSUPPORTED;
        p.quota = (unsigned)(total / grid);
        p.remainder = (unsigned)(total % grid);
    }
    bool has_bf16 = false;
    for (int i = 0; i < p.nseg; ++i) {
        has_bf16 |= p.seg[i].kind == SEG_BF16;
        if (p.seg[i].epilogue == EP_CONV) {
            // a block stages the taps and history of its conv rows in shared memory
            const long long rows_per_block = p.seg[i].rows / grid + 2;
            if (p.conv_width > kStreamConvWidth || p.conv_width < 1 || rows_per_block > kStreamConvRows)
                return QD_ERR_UNSUPPORTED;
        }
    }
    if (p.width == 2048) return has_bf16 ? launch_variant<2, true>(p, grid, stream, pdl)
                                         : launch_variant<2, false>(p, grid, stream, pdl);
    if (p.width == 4096 && !has_bf16 && p.prologue != PRO_ADD_NORM) return launch_variant<4, false>(p, grid, stream, pdl);
    return QD_ERR_UNSUPPORTED;
}

}  // namespace qd

// Profiling aid: after this call every streaming launch writes per-block timestamps (ns) into
// buffer + launch_index * 16384 (16 per block: 8 consumer slots, 8 producer slots), for the
// next `launches` launches.  buffer NULL switches it off.
extern "C" int qd_stream_trace(unsigned long long* buffer, int launches) {
    qd::g_trace = buffer; qd::g_trace_launches = launches; qd::g_trace_next = 0;
    return QD_OK;
}

// Tuning knob: blocks per SM the streaming kernel is launched with when the caller gives no
// grid (2048-wide inputs; 1 or 2).
extern "C" int qd_stream_blocks_per_sm(int n) {
    if (n < 1 || n > 2) return QD_ERR_ARG;
    qd::g_blocks_per_sm = n;
    return QD_OK;
}

// ------------------------------------------------------------ op-table entry (ops.cu)
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int qd_stream_matvec_try(const Fp4Args& a, cudaStream_t stream) {
    using namespace qd;
    if (a.group != 16 || (a.in_features != 2048 && a.in_features != 4096)) return QD_ERR_UNSUPPORTED;
    if (a.routing || a.per_slot_input || a.slots > kStreamMaxSeg) return QD_ERR_UNSUPPORTED;
    if (!aligned16(a.x) || !aligned16(a.codes) || !aligned16(a.scales)) return QD_ERR_UNSUPPORTED;
    if (a.up_codes && (!aligned16(a.up_codes) || !aligned16(a.up_scales))) return QD_ERR_UNSUPPORTED;
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
