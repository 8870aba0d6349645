// Program and parameter blocks of the persistent decode kernel (mega.cu).
//
// One cooperative launch runs a whole token: the host lays the token step out as a list of
// phases (the "program", built once per model and workspace); every phase is a piece of work
// spread over all blocks, and a grid-wide barrier separates a phase from the one that reads
// its results.  Weights reach shared memory through one ring of bulk copies per block whose
// producer warp runs ahead of the consumers across phase boundaries, so the weights of the
// next phases are already on chip while the blocks wait for each other.
#pragma once
#include "stream.cuh"

namespace qd {

constexpr int kMegaConsumerWarps = 16;
constexpr int kMegaConsumers = kMegaConsumerWarps * 32;
constexpr int kMegaThreads = kMegaConsumers + 32;     // + one producer warp
constexpr int kMegaStages = 6;                        // ring stages of kStreamStageBytes
constexpr int kMegaMaxSeg = 10;
constexpr int kMegaConvRows = 128;                    // conv channels one block can own
constexpr int kMegaAttnSplits = 64;                   // context splits per KV head at most
constexpr int kMegaDownRows = 16;                     // down-projection output rows per block at most

enum MegaKind { MK_STREAM = 0, MK_GDN = 1, MK_ATTN = 2, MK_DOWN = 3, MK_ATTN_MERGE = 4 };

struct alignas(8) MegaSeg {
    const uint8_t* w;  const uint8_t* s;  const float* g;      // codes / bf16 rows, scales, global
    const uint8_t* w2; const uint8_t* s2; const float* g2;     // "up" half of a pair
    bf16* y;                                                    // one bf16 per row (NULL: the logits)
    long long w_stride, s_stride;                               // bytes between experts of a bank
    int rows;
    short kind, epilogue;                                       // SegKind, SegEpilogue
    short slot, g_per_expert;                                   // slot >= 0: bank entry = ids[slot]
};

struct alignas(16) MegaPhase {
    MegaSeg seg[kMegaMaxSeg];
    int kind;                 // MegaKind
    int nseg, width, prologue;
    int uses_ids;             // segments are bank entries chosen by this layer's routing
    int route;                // the consumers select the experts before the phase
    int layer, state_index;
    int from_token;           // x = embedding row of the step's token
    int keep_x;               // x is the vector the previous streaming phase built
    unsigned quota, remainder;   // total cost = quota * grid + remainder
    int g_per_expert, argmax;
    // streaming phases
    const bf16* x; const bf16* residual; const float* gamma; bf16* residual_out; bf16* x_out;
    const bf16* z; const bf16* head_gamma; const bf16* conv_taps;
    const bf16* router_logits; int32_t* ids_out; float* weights_out;
    // DeltaNet recurrence
    const bf16* qkv; const bf16* a; const bf16* b; const bf16* a_log; const bf16* dt_bias; bf16* mix_out;
    // attention
    const bf16* qg; const bf16* k_new; const bf16* v_new; const bf16* q_norm; const bf16* k_norm;
    // MoE down projections and combine
    const bf16* hidden; const uint8_t* dw; const uint8_t* ds; const float* dg;
    const uint8_t* sw; const uint8_t* ss; const float* sg; const bf16* strength; bf16* out;
};
static_assert(sizeof(MegaPhase) % 16 == 0, "phases are copied in 16-byte pieces");

struct MegaParams {
    const MegaPhase* program; int nphases; int grid;
    qd_state st;
    const long long* token; const int* pos_dev; int pos_host;
    const bf16* embed; bf16* logits; long long* next_token;
    float* best_val; int* best_idx; unsigned int* argmax_counter;
    unsigned int* bar; unsigned int* exit_count; unsigned int* status;
    float* attn_partial; unsigned int* attn_counters; int attn_splits;
    int hk, hv, dk, dv;            // DeltaNet heads
    int hq, hkv, d, rotary;        // attention heads
    float theta, eps;
    int conv_width, topk, experts, hidden, channels;
    int expert_lo, expert_hi;
    unsigned long long* trace;     // optional: [phase][16][grid] timestamps (ns)
};

int mega_launch(const MegaParams& p, cudaStream_t stream);
size_t mega_smem_bytes();

}  // namespace qd
