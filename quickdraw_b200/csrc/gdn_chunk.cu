// Gated delta rule over a long run of tokens, 64 tokens at a time on the tensor cores.
//
// The reference walks a prompt token by token (quickdraw/kernel/triton/delta.py:57-81: per
// token S *= decay; pred = S^T k; S += k (x) beta (v - pred); out = S^T q), and so does the
// sequence kernel of seq.cu: about 750 clocks per token whatever the width, because every token
// waits for the one before.  Within a chunk of C = 64 tokens the same recurrence has a closed
// form.  With g_t the product of the decays of tokens 0..t of the chunk, u_t = beta_t (v_t - pred_t)
// and S_0 the state at the start of the chunk:
//   (I + L) U = B (V - G K S_0),   L[t][i] = beta_t (g_t / g_i) (k_t . k_i)  for i < t
//   O = G Q S_0 + A U,              A[t][i] = (g_t / g_i) (q_t . k_i)         for i <= t
//   S_C = g_C S_0 + (K scaled by g_C / g_t)^T U
// (B = diag(beta), G = diag(g)).  Two kernels:
//   prepare     block = (chunk, value head), all chunks in parallel: normalised keys and queries,
//               K K^T and Q K^T on mma.sync (tf32), L and A, T = (I + L)^-1 by forward substitution
//               in fp32 (a column per four lanes), T B and A written to a scratch area;
//   recurrence  block = (value head, 32 value columns), chunks in order: R = V - (G K) S_0,
//               U = (T B) R, O = (G Q) S_0 + A U, S = g_C S + K^T (U scaled by g_C / g_t), all on
//               mma.sync (tf32 operands, fp32 accumulation; row scalings applied to the sums,
//               not to the operands); the state stays in accumulator registers, its tf32 copy in
//               shared memory (transposed, like R and U: every operand fragment is one 16-byte
//               load) is the B operand; the next chunk's rows are loaded into registers and its
//               T B / A tiles by cp.async while this chunk is multiplied.
// Operands are rounded to tf32 (10 bits of mantissa), sums are fp32: the result differs from the
// token-by-token kernel by about 1e-3 relative, inside the tolerance the sequence forms are
// tested with.
#include "common.cuh"

namespace qd {
namespace {

constexpr int kC = 64;             // tokens per chunk
constexpr int kDK = 128;           // key dimension
constexpr int kCols = 32;          // value columns per recurrence block
// Row strides in shared memory: 16 floats of padding, so that the 16-byte fragment loads of a
// quarter-warp (rows g, g + 1; floats 4 t .. 4 t + 3) fall on different banks.
constexpr int kKP = kDK + 16;      // floats per row of a [*][128] tile
constexpr int kTP = kC + 16;       // ... of a [*][64] tile
constexpr int kTileFloats = kC * kTP;

QD_DEVINL float tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
QD_DEVINL void mma_tf32(float (&d)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
                   "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
QD_DEVINL void chunk_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// log of the decay of one token (<= 0)
QD_DEVINL float log_decay(float a, float a_log, float bias) { return -expf(a_log) * softplus_precise(a + bias); }

// Rows of eight tokens of a chunk (warp w: tokens 8 w .. 8 w + 7; lane l: keys 4 l .. 4 l + 3).
struct ChunkRows { uint2 k[8], q[8]; };
QD_DEVINL void load_rows(ChunkRows& r, const bf16* __restrict__ qkv, int t_base, int tokens, int channels, int hk, int key_head,
                         int warp, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = t_base + 8 * warp + i;
        r.k[i] = make_uint2(0u, 0u); r.q[i] = make_uint2(0u, 0u);
        if (t < tokens) {
            const bf16* row = qkv + (size_t)t * channels;
            r.q[i] = __ldg(reinterpret_cast<const uint2*>(row + (size_t)key_head * kDK + 4 * lane));
            r.k[i] = __ldg(reinterpret_cast<const uint2*>(row + (size_t)(hk + key_head) * kDK + 4 * lane));
        }
    }
}
// L2-normalised keys and queries (queries also scaled by 1 / sqrt(128)) as tf32 values.
QD_DEVINL void store_rows(const ChunkRows& r, float* __restrict__ Kn, float* __restrict__ Qn, int warp, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float q4[4] = {bf16_bits_to_float(r.q[i].x & 0xffffu), bf16_bits_to_float(r.q[i].x >> 16),
                             bf16_bits_to_float(r.q[i].y & 0xffffu), bf16_bits_to_float(r.q[i].y >> 16)};
        const float k4[4] = {bf16_bits_to_float(r.k[i].x & 0xffffu), bf16_bits_to_float(r.k[i].x >> 16),
                             bf16_bits_to_float(r.k[i].y & 0xffffu), bf16_bits_to_float(r.k[i].y >> 16)};
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) { qq += q4[e] * q4[e]; kk += k4[e] * k4[e]; }
        const float qscale = rsqrtf(warp_sum(qq) + 1e-6f) * 0.08838834764831845f, kscale = rsqrtf(warp_sum(kk) + 1e-6f);
        const int at = (8 * warp + i) * kKP + 4 * lane;
        *reinterpret_cast<float4*>(Kn + at) = make_float4(tf32(k4[0] * kscale), tf32(k4[1] * kscale), tf32(k4[2] * kscale), tf32(k4[3] * kscale));
        *reinterpret_cast<float4*>(Qn + at) = make_float4(tf32(q4[0] * qscale), tf32(q4[1] * qscale), tf32(q4[2] * qscale), tf32(q4[3] * qscale));
    }
}
QD_DEVINL float4 lds4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// Two k-steps of an MMA tile from 16-byte fragments.  The contraction index is permuted the same
// way on both sides: lane (g, t) supplies elements 4 t, 4 t + 1 (first step) and 4 t + 2, 4 t + 3
// (second step) of every 16, so one 16-byte load per row (A: rows g and g + 8; B: column g)
// feeds two MMAs.
QD_DEVINL void mma_pair(float (&d)[4], const float4& a_lo, const float4& a_hi, const float4& b) {
    mma_tf32(d, a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
    mma_tf32(d, a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
}

// ------------------------------------------------------------------------------- prepare
__global__ void __launch_bounds__(256, 2)
gdn_chunk_prepare_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ b,
                         const bf16* __restrict__ a_log, const bf16* __restrict__ dt_bias, float* __restrict__ scratch,
                         int tokens, int hk, int hv, int dv) {
    chain_enter();
    extern __shared__ __align__(16) float prep_smem[];
    float* Kn = prep_smem;                     // [64][kKP]
    float* Qn = Kn + kC * kKP;
    float* Lm = Qn + kC * kKP;                 // [64][kTP]: L, later T B
    float* Am = Lm + kTileFloats;              // [64][kTP]: A
    __shared__ float cum[kC], beta[kC];
    const int chunk = blockIdx.x, head = blockIdx.y, chunks = gridDim.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int key_head = head / (hv / hk), channels = 2 * hk * kDK + hv * dv, t_base = chunk * kC;
    if (tid < kC) {
        const int tok = t_base + tid;
        float lg = 0.f, bt = 0.f;
        if (tok < tokens) {
            lg = log_decay(ld_bf16(a + (size_t)tok * hv + head), ld_bf16(a_log + head), ld_bf16(dt_bias + head));
            bt = sigmoid_precise(ld_bf16(b + (size_t)tok * hv + head));
        }
        cum[tid] = lg; beta[tid] = bt;
    }
    ChunkRows rows;
    load_rows(rows, qkv, t_base, tokens, channels, hk, key_head, warp, lane);
    store_rows(rows, Kn, Qn, warp, lane);
    __syncthreads();
    if (tid == 0) {                            // inclusive sums of the log decays
        float s = 0.f;
        for (int i = 0; i < kC; ++i) { s += cum[i]; cum[i] = s; }
    }
    // ---- K K^T and Q K^T: warp = (16 rows, 32 columns)
    const int mt = warp & 3, nq = warp >> 2;
    float g1[4][4], g2[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) { g1[j][c] = 0.f; g2[j][c] = 0.f; }
#pragma unroll 2
    for (int kk = 0; kk < kDK / 16; ++kk) {
        const int at = (16 * mt + g) * kKP + 16 * kk + 4 * t;
        const float4 k_lo = lds4(Kn + at), k_hi = lds4(Kn + at + 8 * kKP), q_lo = lds4(Qn + at), q_hi = lds4(Qn + at + 8 * kKP);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 bk = lds4(Kn + ((nq * 4 + j) * 8 + g) * kKP + 16 * kk + 4 * t);
            mma_pair(g1[j], k_lo, k_hi, bk);
            mma_pair(g2[j], q_lo, q_hi, bk);
        }
    }
    __syncthreads();                           // cum is complete
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int row = 16 * mt + g + 8 * (c >> 1), col = (nq * 4 + j) * 8 + 2 * t + (c & 1);
            const float ratio = col <= row ? expf(cum[row] - cum[col]) : 0.f;
            Lm[row * kTP + col] = col < row ? beta[row] * ratio * g1[j][c] : 0.f;
            Am[row * kTP + col] = col <= row ? tf32(ratio * g2[j][c]) : 0.f;
        }
    __syncthreads();
    // ---- T = (I + L)^-1, row by row: four lanes share a column (lane part p holds rows 4 i + p)
    const int col = 8 * warp + g, p = t;
    float tc[kC / 4];
#pragma unroll
    for (int i = 0; i < kC / 4; ++i) tc[i] = 0.f;
#pragma unroll
    for (int row = 0; row < kC; ++row) {
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < kC / 4; ++i)
            if (4 * i < row) {                 // rows below `row` only (static bound; the last group is partial)
                const int r = 4 * i + p;
                if (r < row) part += Lm[row * kTP + r] * tc[i];
            }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        const float value = (row == col ? 1.f : 0.f) - part;
        if (p == (row & 3)) tc[row >> 2] = value;
    }
    __syncthreads();                           // every column is done with L
#pragma unroll
    for (int i = 0; i < kC / 4; ++i) Lm[(4 * i + p) * kTP + col] = tf32(tc[i] * beta[col]);
    __syncthreads();
    float4* dst = reinterpret_cast<float4*>(scratch + ((size_t)head * chunks + chunk) * 2 * kTileFloats);
    const float4* src = reinterpret_cast<const float4*>(Lm);      // T B, then A: contiguous
    for (int i = tid; i < 2 * kTileFloats / 4; i += 256) dst[i] = src[i];
}

// ---------------------------------------------------------------------------- recurrence
constexpr int kVP = kCols + 8;     // floats per row of the [64][32] value tile
__global__ void __launch_bounds__(256, 1)
gdn_chunk_recurrence_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ a, const bf16* __restrict__ a_log,
                            const bf16* __restrict__ dt_bias, float* __restrict__ state, bf16* __restrict__ out,
                            const float* __restrict__ scratch, int tokens, int hk, int hv, int dv) {
    chain_enter();
    extern __shared__ __align__(16) float rec_smem[];
    float* Kn = rec_smem;                      // [64 tokens][kKP]
    float* Qn = Kn + kC * kKP;
    float* TA = Qn + kC * kKP;                 // [2][T B | A][64][kTP]
    float* St = TA + 4 * kTileFloats;          // [32 columns][kKP]: the state at the start of the chunk, transposed, tf32
    float* Rt = St + kCols * kKP;              // [32 columns][kTP]: R transposed
    float* Ut = Rt + kCols * kTP;              // ... U
    float* Wt = Ut + kCols * kTP;              // ... U with row t scaled by g_C / g_t
    float* Vs = Wt + kCols * kTP;              // [64 tokens][kVP]: the value columns
    __shared__ float gam[kC], gend[kC], lg_s[kC];
    __shared__ float g_end;
    const int head = blockIdx.x, c0 = blockIdx.y * kCols;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int key_head = head / (hv / hk), channels = 2 * hk * kDK + hv * dv;
    const int chunks = (tokens + kC - 1) / kC;
    const float a_decay = ld_bf16(a_log + head), bias = ld_bf16(dt_bias + head);
    float* tile = state + (size_t)head * kDK * dv + c0;

    // the state: warp w owns keys 16 w .. 16 w + 15; acc[nt][c]: key 16 w + g + 8 (c >> 1), column 8 nt + 2 t + (c & 1)
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = tile[(size_t)(16 * warp + g + 8 * (c >> 1)) * dv + 8 * nt + 2 * t + (c & 1)];

    ChunkRows rows;
    bf16 vals[8];
    bf16 gate_raw = __float2bfloat16_rn(0.f);
    bool gate_on = false;
    auto issue = [&](int chunk) {              // the chunk's rows into registers, its T B / A tiles by cp.async
        const int t_base = chunk * kC;
        load_rows(rows, qkv, t_base, tokens, channels, hk, key_head, warp, lane);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int tok = t_base + 8 * warp + i;
            vals[i] = tok < tokens ? qkv[(size_t)tok * channels + (size_t)2 * hk * kDK + (size_t)head * dv + c0 + lane]
                                   : __float2bfloat16_rn(0.f);
        }
        gate_on = tid < kC && t_base + tid < tokens;             // the value is used in finish(): nothing waits for it here
        if (gate_on) gate_raw = a[(size_t)(t_base + tid) * hv + head];
        const float* src = scratch + ((size_t)head * chunks + chunk) * 2 * kTileFloats;
        float* dst = TA + (size_t)(chunk & 1) * 2 * kTileFloats;
        for (int i = tid; i < 2 * kTileFloats / 4; i += 256) chunk_cp16(dst + 4 * i, src + 4 * i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto finish = [&]() {                      // registers -> shared memory: rows, values, decays; the state's tf32 copy
        store_rows(rows, Kn, Qn, warp, lane);
#pragma unroll
        for (int i = 0; i < 8; ++i) Vs[(8 * warp + i) * kVP + lane] = __bfloat162float(vals[i]);
        if (tid < kC) lg_s[tid] = gate_on ? log_decay(__bfloat162float(gate_raw), a_decay, bias) : 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) St[(8 * nt + 2 * t + (c & 1)) * kKP + 16 * warp + g + 8 * (c >> 1)] = tf32(acc[nt][c]);
    };
    issue(0);
    finish();
    __syncthreads();
#pragma unroll 1
    for (int chunk = 0; chunk < chunks; ++chunk) {
        // ---- decays of the chunk: g_t (rows of K S and Q S), g_C / g_t (rows of U for the state), g_C
        if (warp == 0) {
            float v0 = lg_s[2 * lane], v1 = lg_s[2 * lane + 1] + v0, run = v1;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const float up = __shfl_up_sync(0xffffffffu, run, d); if (lane >= d) run += up; }
            const float before = run - v1, total = __shfl_sync(0xffffffffu, run, 31);
            gam[2 * lane] = expf(before + v0); gam[2 * lane + 1] = expf(before + v1);
            gend[2 * lane] = expf(total - before - v0); gend[2 * lane + 1] = expf(total - before - v1);
            if (lane == 0) g_end = expf(total);
        }
        __syncthreads();
        if (chunk + 1 < chunks) issue(chunk + 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const float* Tb = TA + (size_t)(chunk & 1) * 2 * kTileFloats;
        const float* Am = Tb + kTileFloats;
        const int mt = warp & 3, n0 = (warp >> 2) * 16;          // stages on [64][32]: 16 rows x 16 columns per warp
        const int row0 = 16 * mt + g;
        const float row_g[2] = {gam[row0], gam[row0 + 8]}, row_e[2] = {gend[row0], gend[row0 + 8]};
        const int frag = 4 * t;                                  // the lane's four elements of every sixteen
        // ---- R = V - G (K S_0)
        {
            float r[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < kDK / 16; ++kk) {
                const float4 a_lo = lds4(Kn + row0 * kKP + 16 * kk + frag), a_hi = lds4(Kn + (row0 + 8) * kKP + 16 * kk + frag);
                mma_pair(r[0], a_lo, a_hi, lds4(St + (n0 + g) * kKP + 16 * kk + frag));
                mma_pair(r[1], a_lo, a_hi, lds4(St + (n0 + 8 + g) * kKP + 16 * kk + frag));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int row = row0 + 8 * (c >> 1), col = n0 + 8 * j + 2 * t + (c & 1);
                    Rt[col * kTP + row] = tf32(Vs[row * kVP + col] - row_g[c >> 1] * r[j][c]);
                }
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // this chunk's T B and A (the next chunk's may be in flight)
        __syncthreads();
        // ---- U = (T B) R: T is lower triangular, so only the tokens up to the warp's rows count
        {
            float u[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            for (int kk = 0; kk <= mt; ++kk) {
                const float4 a_lo = lds4(Tb + row0 * kTP + 16 * kk + frag), a_hi = lds4(Tb + (row0 + 8) * kTP + 16 * kk + frag);
                mma_pair(u[0], a_lo, a_hi, lds4(Rt + (n0 + g) * kTP + 16 * kk + frag));
                mma_pair(u[1], a_lo, a_hi, lds4(Rt + (n0 + 8 + g) * kTP + 16 * kk + frag));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int row = row0 + 8 * (c >> 1), col = n0 + 8 * j + 2 * t + (c & 1);
                    Ut[col * kTP + row] = tf32(u[j][c]);
                    Wt[col * kTP + row] = tf32(u[j][c] * row_e[c >> 1]);
                }
        }
        __syncthreads();
        // ---- O = G (Q S_0) + A U
        {
            float o[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < kDK / 16; ++kk) {
                const float4 a_lo = lds4(Qn + row0 * kKP + 16 * kk + frag), a_hi = lds4(Qn + (row0 + 8) * kKP + 16 * kk + frag);
                mma_pair(o[0], a_lo, a_hi, lds4(St + (n0 + g) * kKP + 16 * kk + frag));
                mma_pair(o[1], a_lo, a_hi, lds4(St + (n0 + 8 + g) * kKP + 16 * kk + frag));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[j][c] *= row_g[c >> 1];
            for (int kk = 0; kk <= mt; ++kk) {
                const float4 a_lo = lds4(Am + row0 * kTP + 16 * kk + frag), a_hi = lds4(Am + (row0 + 8) * kTP + 16 * kk + frag);
                mma_pair(o[0], a_lo, a_hi, lds4(Ut + (n0 + g) * kTP + 16 * kk + frag));
                mma_pair(o[1], a_lo, a_hi, lds4(Ut + (n0 + 8 + g) * kTP + 16 * kk + frag));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int tok = chunk * kC + row0 + 8 * half;
                    if (tok < tokens)
                        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)tok * hv * dv + (size_t)head * dv + c0 + n0 + 8 * j + 2 * t) =
                            __floats2bfloat162_rn(o[j][2 * half], o[j][2 * half + 1]);
                }
        }
        // ---- S = g_C S + K^T W: warp w = keys 16 w .. 16 w + 15, all 32 columns; contraction over the tokens
        {
            const float scale = g_end;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[nt][c] *= scale;
#pragma unroll
            for (int kk = 0; kk < kC / 16; ++kk) {
                const float* ka = Kn + (16 * kk + frag) * kKP + 16 * warp + g;     // tokens 16 kk + 4 t .. + 3, keys g and g + 8
                const float4 a_lo = make_float4(ka[0], ka[kKP], ka[2 * kKP], ka[3 * kKP]);
                const float4 a_hi = make_float4(ka[8], ka[kKP + 8], ka[2 * kKP + 8], ka[3 * kKP + 8]);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) mma_pair(acc[nt], a_lo, a_hi, lds4(Wt + (8 * nt + g) * kTP + 16 * kk + frag));
            }
        }
        __syncthreads();                       // every warp is done with this chunk's tiles
        if (chunk + 1 < chunks) finish();
        __syncthreads();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) tile[(size_t)(16 * warp + g + 8 * (c >> 1)) * dv + 8 * nt + 2 * t + (c & 1)] = acc[nt][c];
}

constexpr size_t kPrepSmem = sizeof(float) * (2 * kC * kKP + 2 * kTileFloats);
constexpr size_t kRecSmem = sizeof(float) * (2 * kC * kKP + 4 * kTileFloats + kCols * kKP + 3 * kCols * kTP + kC * kVP);

}  // namespace
}  // namespace qd

// Bytes of the scratch area of qd_seq_gdn_recurrence_chunked for a run of `tokens` tokens.
extern "C" long long qd_seq_gdn_chunk_scratch_bytes(int tokens, int value_heads) {
    if (tokens <= 0 || value_heads <= 0) return 0;
    return (long long)((tokens + qd::kC - 1) / qd::kC) * value_heads * 2 * qd::kTileFloats * (long long)sizeof(float);
}

// The contract of qd_seq_gdn_recurrence (conv_qkv [tokens, 2 key_heads 128 + value_heads value_dim]
// after the short convolution, a / b [tokens, value_heads], rec_state fp32 updated in place, out
// bf16 [tokens, value_heads value_dim]) in the chunked form.  key_dim 128, value_dim a multiple of
// 32; QD_ERR_UNSUPPORTED otherwise.  scratch: qd_seq_gdn_chunk_scratch_bytes bytes, 16-byte aligned.
extern "C" int qd_seq_gdn_recurrence_chunked(const void* conv_qkv, const void* a, const void* b, const void* a_log,
                                             const void* dt_bias, float* rec_state, void* out, int tokens, int key_heads,
                                             int value_heads, int key_dim, int value_dim, void* scratch, void* stream) {
    using namespace qd;
    QD_CHECK_ARG(conv_qkv && a && b && a_log && dt_bias && rec_state && out && scratch && tokens > 0);
    QD_CHECK_ARG(key_heads > 0 && value_heads % key_heads == 0 && value_dim > 0);
    if (key_dim != kDK || value_dim % kCols != 0 || value_heads > 65535) return QD_ERR_UNSUPPORTED;
    if (((uintptr_t)conv_qkv & 7u) || ((uintptr_t)scratch & 15u) || ((2 * key_heads * kDK + value_heads * value_dim) % 4)) return QD_ERR_UNSUPPORTED;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return QD_ERR_LAUNCH;
    static bool configured[64];
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrepSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRecSmem) != cudaSuccess)
            return QD_ERR_LAUNCH;
        configured[dev] = true;
    }
    const int chunks = (tokens + kC - 1) / kC;
    qd_launch(gdn_chunk_prepare_kernel, dim3(chunks, value_heads), dim3(256), kPrepSmem, (cudaStream_t)stream, true, 
        (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)b, (const bf16*)a_log, (const bf16*)dt_bias, (float*)scratch,
        tokens, key_heads, value_heads, value_dim);
    if (qd_launch_status() != QD_OK) return QD_ERR_LAUNCH;
    qd_launch(gdn_chunk_recurrence_kernel, dim3(value_heads, value_dim / kCols), dim3(256), kRecSmem, (cudaStream_t)stream, true, 
        (const bf16*)conv_qkv, (const bf16*)a, (const bf16*)a_log, (const bf16*)dt_bias, rec_state, (bf16*)out,
        (const float*)scratch, tokens, key_heads, value_heads, value_dim);
    return qd_launch_status();
}
