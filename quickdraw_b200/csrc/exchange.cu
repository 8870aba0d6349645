// Sum of one small fp32 vector over the GPUs of a node, through peer memory (NVLink): the
// exchange of the expert-parallel decode step (one per layer: the [hidden] partial sums of the
// ranks' experts).  The reference is a single-GPU library and has no counterpart.
//
// Every rank owns a buffer that all ranks can address (symmetric allocation, peer pointers
// exchanged by the host): slots [2][world][n] floats and flags [2][world] words.  One block
// per rank and exchange:
//   1. stores its vector into slot [parity][rank] of every rank's buffer (plain stores over
//      NVLink), fences at system scope,
//   2. release-stores the exchange number into flag [parity][rank] of every rank,
//   3. waits until the flags of all ranks in its own buffer show this exchange number (the
//      wait is bounded by wall time: on time-out the status word gets a bit and the block goes
//      on with whatever it has),
//   4. sums the slots in rank order (the same order on every rank, so all ranks hold the same
//      bits) into its vector.
// Two slot sets alternate with the parity of the exchange number: a rank can run at most one
// exchange ahead of the slowest rank, because it needs that rank's flag to finish its own.
// The exchange number lives in device memory and is advanced by the kernel, so the launch can
// be replayed from a CUDA graph.  Nothing here uses multicast or TMA.
#include "common.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr unsigned long long kExchangeWaitNs = 2000000000ull;   // 2 s: ranks may start a step apart

struct ExchangeParams {
    unsigned long long peers[kMaxRanks];   // every rank's buffer as seen from this GPU
    float* vector;                         // in: this rank's partial, out: the sum
    unsigned int* epoch;                   // exchange number, local
    unsigned int* status;
    int rank, world, n;
};

QD_DEVINL size_t flags_offset(int world, int n) { return (((size_t)2 * world * n * sizeof(float)) + 127) & ~(size_t)127; }

QD_DEVINL void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
QD_DEVINL unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(512)
peer_all_reduce_kernel(const ExchangeParams p) {
    const int tid = threadIdx.x, W = p.world, n = p.n;
    const unsigned int e = *p.epoch + 1;
    const int parity = (int)(e & 1u);
    // 1. my vector into my slot of every rank's buffer
    for (int r = 0; r < W; ++r) {
        float4* dst = reinterpret_cast<float4*>(p.peers[r]) + ((size_t)(parity * W + p.rank) * n) / 4;
        for (int i = tid; i < n / 4; i += blockDim.x) dst[i] = reinterpret_cast<const float4*>(p.vector)[i];
    }
    __threadfence_system();
    __syncthreads();
    // 2. tell every rank, 3. wait for every rank
    if (tid < W) {
        unsigned int* theirs = reinterpret_cast<unsigned int*>(p.peers[tid] + flags_offset(W, n)) + parity * W + p.rank;
        st_release_sys(theirs, e);
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.peers[p.rank] + flags_offset(W, n)) + parity * W + tid;
        const unsigned long long start = global_timer_ns();
        bool seen = false;
        for (;;) {
#pragma unroll 1
            for (int i = 0; i < 32 && !seen; ++i) seen = ld_acquire_sys(mine) == e;
            if (seen || global_timer_ns() - start > kExchangeWaitNs) break;
        }
        if (!seen) atomicOr(p.status, QD_STATUS_WAIT_TIMEOUT);
    }
    __syncthreads();
    // 4. the sum in rank order, read past the L1 (the slots were written by other GPUs)
    const float4* slots = reinterpret_cast<const float4*>(p.peers[p.rank]) + ((size_t)parity * W * n) / 4;
    for (int i = tid; i < n / 4; i += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < W; ++r) {
            const float4 v = __ldcv(slots + (size_t)r * (n / 4) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(p.vector)[i] = acc;
    }
    if (tid == 0) *p.epoch = e;
}

}  // namespace

// bytes of the symmetric buffer every rank must provide (zero-filled before the first exchange)
extern "C" long long qd_peer_all_reduce_bytes(int world, int n) {
    if (world < 1 || world > kMaxRanks || n <= 0 || n % 4 != 0) return -1;
    return (long long)((((size_t)2 * world * n * sizeof(float)) + 127) & ~(size_t)127) + 2 * world * (long long)sizeof(unsigned int);
}

extern "C" int qd_peer_all_reduce(float* vector, const unsigned long long* peer_buffers, int rank, int world, int n,
                                  unsigned int* epoch, unsigned int* status, void* stream) {
    QD_CHECK_ARG(vector && peer_buffers && epoch && status && world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world);
    QD_CHECK_ARG(n > 0 && n % 4 == 0 && !((uintptr_t)vector & 15u));
    ExchangeParams p = {};
    for (int r = 0; r < world; ++r) {
        QD_CHECK_ARG(peer_buffers[r] && !(peer_buffers[r] & 127u));
        p.peers[r] = peer_buffers[r];
    }
    p.vector = vector; p.epoch = epoch; p.status = status; p.rank = rank; p.world = world; p.n = n;
    peer_all_reduce_kernel<<<1, 512, 0, (cudaStream_t)stream>>>(p);
    return qd_launch_status();
}
