// Streaming matvec: one activation vector against a list of weight segments.
//
// Work split: the byte cost of all segments is cut into gridDim.x equal ranges; a block
// walks its range in tiles of whole rows.  A producer warp issues the bulk copies of a
// tile (codes and block scales are contiguous row blocks in the reference layout, so no
// repacking is needed) into a ring of shared-memory stages guarded by full/empty
// mbarriers.  The sixteen consumer warps share every NVFP4 tile: each warp multiplies its
// slice of the inputs of all rows of the tile on the tensor cores (rowmma.cuh), the partial
// sums meet in shared memory and one warp per tile (rotating) finishes the rows.  bf16 rows
// (router, LM head, small projections) go row by row, a warp each.
//
// Everything that does not depend on the previous launch (weights, norm gamma, conv taps
// and history) is fetched before the programmatic dependency wait.
//
// Arithmetic contract (reference: quickdraw/models/qwen.py:36-54 and the rounding points
// of quickdraw/kernel/cute/matvec.py:62-77): weights dequantised exactly (code x block
// scale in f16), fp32 accumulation, global scale applied to the finished sum, one bf16
// rounding; SwiGLU rounds gate, up, silu(gate) and the product.
#include "stream.cuh"
#include "rowdot.cuh"
#include "rowmma.cuh"

namespace qd {

namespace {

template <int KC, bool WITH_BF16>
__global__ void __launch_bounds__(kStreamThreads, 1)
stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int K = KC * 1024;
    constexpr int CW = kStreamConsumerWarps, CT = CW * 32, NS = kStreamStages;
    constexpr int EPT = K / CT;                       // prologue elements per thread (4 or 8)
    constexpr int UNITS = K / 2048;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;
    bf16* xs = reinterpret_cast<bf16*>(smem + NS * kStreamStageBytes);                // [K] bf16
    uint8_t* xf = reinterpret_cast<uint8_t*>(xs + K);                                   // [K] f16
    float* partials = reinterpret_cast<float*>(xf + K * 2);                              // [NS][16 warps][32]
    bf16* conv_taps_s = reinterpret_cast<bf16*>(partials + NS * kRowPartialFloats);      // [rows][W]
    bf16* conv_state_s = conv_taps_s + kStreamConvRows * kStreamConvWidth;               // [rows][W-1]
    uint64_t* full = reinterpret_cast<uint64_t*>(conv_state_s + kStreamConvRows * kStreamConvWidth);
    uint64_t* empty = full + NS;
    uint64_t* ready = empty + NS;                             // partial sums of a tile are complete
    float* red = reinterpret_cast<float*>(ready + NS);       // [64]
    int32_t* s_ids = reinterpret_cast<int32_t*>(red + 64);   // [64]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, CW); mbar_init(ready + s, CW); }
        mbar_fence_init();
    }
    __syncthreads();
    grid_launch_dependents();

    // byte range of this block: total cost = quota * gridDim.x + remainder, split on the host
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
    const bf16* xin = p.token ? p.embed + (size_t)(*p.token) * K : p.x;
    uint32_t m2 = 0u;      // largest |bf16| bit pattern this thread produced, per 16-bit half
    // 1. activation vector into shared memory (bf16); thread i owns elements [EPT*i, EPT*i + EPT)
    if (p.prologue == PRO_ADD_NORM) {
        float v[EPT];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPT; j += 4) {
            const uint2 xa = *reinterpret_cast<const uint2*>(xin + tid * EPT + j);
            uint2 ra2 = make_uint2(0u, 0u);
            if (p.residual) ra2 = *reinterpret_cast<const uint2*>(p.residual + tid * EPT + j);
            const uint32_t xw[2] = {xa.x, xa.y}, rw[2] = {ra2.x, ra2.y};
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                v[j + 2 * q] = __uint_as_float(xw[q] << 16) + __uint_as_float(rw[q] << 16);
                v[j + 2 * q + 1] = __uint_as_float(xw[q] & 0xffff0000u) + __uint_as_float(rw[q] & 0xffff0000u);
            }
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) ss += v[j] * v[j];
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        named_barrier(1, CT);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) tot += red[w];
        const float inv = rsqrtf(tot / (float)K + p.eps);
#pragma unroll
        for (int j = 0; j < EPT; j += 4) {
            uint32_t nw[2], rw[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const __nv_bfloat162 n2 = __floats2bfloat162_rn((v[j + 2 * q] * inv) * gam[j + 2 * q],
                                                                (v[j + 2 * q + 1] * inv) * gam[j + 2 * q + 1]);
                const __nv_bfloat162 r2 = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                nw[q] = *reinterpret_cast<const uint32_t*>(&n2);
                rw[q] = *reinterpret_cast<const uint32_t*>(&r2);
                m2 = max_u16x2(m2, nw[q] & 0x7fff7fffu);
            }
            const uint2 nv = make_uint2(nw[0], nw[1]);
            *reinterpret_cast<uint2*>(xs + tid * EPT + j) = nv;
            if (blockIdx.x == 0) {
                if (p.x_out) *reinterpret_cast<uint2*>(p.x_out + tid * EPT + j) = nv;
                *reinterpret_cast<uint2*>(p.residual_out + tid * EPT + j) = make_uint2(rw[0], rw[1]);
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
        if (lane == 0) reinterpret_cast<uint32_t*>(red)[32 + warp] = m;
    }
    if (p.ids_in && warp == 0 && lane < p.topk) s_ids[lane] = __ldcg(p.ids_in + lane);
    named_barrier(1, CT);
    // 2. the vector as f16 in natural order.  The largest bf16 magnitude (compared as a bit
    //    pattern) decides a common power-of-two down-scale so that nothing overflows f16 (one in
    //    the usual range); every thread converts its own slice, then each lane fetches the
    //    slices of its spans.
    uint32_t xh[UNITS][16];
    float out_mult;
    {
        uint32_t m = 0u;
#pragma unroll
        for (int w = 0; w < CW; ++w) m = max(m, reinterpret_cast<const uint32_t*>(red)[32 + w]);
        const int exponent = (int)(m >> 7) - 127;            // |x| < 2^(exponent + 1)
        const int shift = (exponent > 14 && exponent < 128) ? exponent - 14 : 0;
        const float down = __uint_as_float((uint32_t)(127 - shift) << 23);
        out_mult = __uint_as_float((uint32_t)(127 + shift) << 23);
#pragma unroll
        for (int j = 0; j < EPT; j += 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(xs + tid * EPT + j);
            uint2 h;
            h.x = pack_f16x2(__uint_as_float(v.x << 16) * down, __uint_as_float(v.x & 0xffff0000u) * down);
            h.y = pack_f16x2(__uint_as_float(v.y << 16) * down, __uint_as_float(v.y & 0xffff0000u) * down);
            *reinterpret_cast<uint2*>(xf + (tid * EPT + j) * 2) = h;
        }
        named_barrier(1, CT);
        load_x_fragments<UNITS>(xf, warp, lane, xh);
    }

    // 3. tiles
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;
    int it = 0, turn = 0;
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
            const uint8_t* base = stages + st * kStreamStageBytes;
            if (sg.kind == SEG_BF16) {
                if (lane == 0) mbar_arrive(ready + st);      // keeps the phase of `ready` in step with the ring
                if (WITH_BF16) {
                    // rows rotate over the warps from tile to tile, so that consecutive tiles overlap
#pragma unroll 1
                    for (int r = (warp - turn) & (CW - 1); r < n; r += CW) {
                        const int row = r0 + r;
                        const float result = warp_sum(bf16_row_dot_smem<K / 256>(base + (size_t)r * 2 * K,
                                                                                 reinterpret_cast<const uint8_t*>(xs), lane));
                        const bf16 rounded = __float2bfloat16_rn(result);
                        if (lane == 0) sg.y[row] = rounded;
                        if (sg.epilogue == EP_ARGMAX) {
                            const float v = __bfloat162float(rounded);
                            if (v > best_val || (v == best_val && row < best_idx)) { best_val = v; best_idx = row; }
                        }
                    }
                    turn = (turn + n) & (CW - 1);
                }
            } else {
                const bool pair = sg.kind == SEG_FP4_PAIR;
                const int groups = UNITS == 2 ? 1 : ((pair || n > 16) ? 2 : 1);
                float* mine = partials + st * kRowPartialFloats;
                tile_partials<K>(base, UNITS == 2 ? 16 : 32, groups, xh, warp, lane, mine + warp * kRowSlots);
                __syncwarp();
                if (lane == 0) mbar_arrive(ready + st);
                if (warp == (it & (CW - 1))) {
                    // this tile's finishing warp: lane = slot of the tile
                    if (!mbar_wait(ready + st, (it / NS) & 1, p.status)) { ok = false; break; }
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
                        if (sg.epilogue == EP_CONV) {
                            // depthwise causal conv for this channel (quickdraw/models/qwen.py:134-136):
                            // history taps then the new value; products rounded to bf16, fp32 sum in the
                            // order of a two-step butterfly ((0 + 2) + (1 + 3) for four taps)
                            const int W = p.conv_width, local = row - conv_row0;
                            float prod[kStreamConvWidth];
#pragma unroll
                            for (int k = 0; k < kStreamConvWidth; ++k) {
                                float val = 0.f, tap = 0.f;
                                if (k < W) {
                                    tap = __bfloat162float(conv_taps_s[local * W + k]);
                                    val = k < W - 1 ? __bfloat162float(conv_state_s[local * (W - 1) + k]) : __bfloat162float(rounded);
                                    if (k >= 1) p.conv_state[(size_t)row * (W - 1) + k - 1] = __float2bfloat16_rn(val);
                                }
                                prod[k] = k < W ? round_bf16(val * tap) : 0.f;
                            }
                            const float conv = (prod[0] + prod[2]) + (prod[1] + prod[3]);
                            sg.y[row] = __float2bfloat16_rn(silu_precise(conv));
                        } else {
                            sg.y[row] = rounded;
                        }
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
    // 4. greedy argmax over the EP_ARGMAX segment (ties: lowest index)
    if (p.best_val != nullptr) {
        if (lane == 0) { red[warp] = best_val; s_ids[warp + 32] = best_idx; }
        named_barrier(1, CT);
        if (tid == 0) {
            float bv = red[0]; int bi = s_ids[32];
            for (int w = 1; w < CW; ++w) {
                const float v = red[w]; const int ix = s_ids[32 + w];
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

template <int KC, bool WITH_BF16>
int launch_variant(const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
    constexpr int K = KC * 1024;
    const size_t smem = (size_t)kStreamStages * kStreamStageBytes + K * 4 + (size_t)kStreamStages * kRowPartialFloats * 4 +
                        2 * kStreamConvRows * kStreamConvWidth * 2 + 3 * kStreamStages * 8 + 64 * 4 * 2 + 64;
    static bool configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(stream_kernel<KC, WITH_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    return qd_launch(stream_kernel<KC, WITH_BF16>, dim3(grid), dim3(kStreamThreads), smem, stream, pdl, p);
}

}  // namespace

int stream_sm_count() {
    static int counts[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (counts[dev] == 0) {
        cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev);
        if (counts[dev] <= 0) counts[dev] = 148;
    }
    return counts[dev];
}

int stream_launch(const StreamParams& p_in, int grid, cudaStream_t stream, bool pdl) {
    StreamParams p = p_in;
    if (grid <= 0) grid = stream_sm_count();
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
