// Program and parameter blocks of the persistent decode kernel (mega.cu).
//
// One cooperative launch runs a whole token: the host lays the token step out as a list of
// phases (the "program", built once per model and workspace); every phase is a piece of work
// spread over all blocks.  There is no grid-wide barrier: every activation that one block
// writes and another reads is a 32-bit word {bf16 value, 16-bit tag}, the tag naming the
// launch and the layer that produced it, and a reader simply re-reads its words until all of
// them carry the tag it expects (fp32 partial sums of the attention splits travel as 64-bit
// {value, tag} words).  A block therefore starts a phase as soon as the words it needs
// have arrived, and the wait costs one trip to L2 instead of a fence, an atomic and a poll.
// Weights reach shared memory through one ring of bulk copies per block whose producer warp
// runs ahead of the consumers across phase boundaries.
#pragma once
#include "stream.cuh"

namespace qd {

constexpr int kMegaConsumerWarps = 16;
constexpr int kMegaConsumers = kMegaConsumerWarps * 32;
constexpr int kMegaThreads = kMegaConsumers + 32;     // + one producer warp
constexpr int kMegaStages = 4;                        // ring stages of kStreamStageBytes
constexpr int kMegaMaxSeg = 10;
constexpr int kMegaConvRows = 128;                    // conv channels one block can own
constexpr int kMegaAttnSplits = 80;                   // context splits per KV head at most
constexpr int kMegaDownRows = 16;                     // down-projection output rows per block at most
constexpr int kMegaMaxLayers = 62;                    // the layer number is six bits of the tag
constexpr int kMegaMaxRanks = 8;                      // expert-parallel group size at most

enum MegaKind { MK_STREAM = 0, MK_GDN = 1, MK_ATTN = 2, MK_DOWN = 3, MK_ATTN_MERGE = 4 };

typedef uint32_t tagged;      // {bf16 bits, 16-bit tag}

struct alignas(8) MegaSeg {
    const uint8_t* w;  const uint8_t* s;  const float* g;      // codes / bf16 rows, scales, global
    const uint8_t* w2; const uint8_t* s2; const float* g2;     // "up" half of a pair
    tagged* y;                                                  // one word per row (NULL: the logits, plain bf16)
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
    int route;                // the consumers select the experts at the start of the phase
    int layer, state_index;
    int from_token;           // x = embedding row of the step's token
    int keep_x;               // x is the vector the previous streaming phase built
    int x_prev_layer;         // x carries the tag of the layer before (the MoE output)
    unsigned quota, remainder;   // total cost = quota * grid + remainder
    // equal segments (the routed gate/up phase): segment s belongs to blocks [s * seg_blocks,
    // (s + 1) * seg_blocks), block_cost of its seg_cost each, so that no block straddles two
    // experts and every block's share is whole tiles; seg_blocks == 0: the cost partition above
    unsigned seg_blocks, seg_cost, block_cost, pad1;
    int g_per_expert, argmax;
    int row_lo, pad0;         // LM head: vocabulary index of the segment's first row (this rank's shard)
    // streaming phases
    const float* in_scale;    // static FP8 projections of this phase: the activation scale (NULL: none)
    const tagged* x; const float* gamma;
    const tagged* z; const bf16* head_gamma; const bf16* conv_taps;
    const tagged* router_logits; int32_t* ids_out; float* weights_out;
    // DeltaNet recurrence
    const tagged* qkv; const tagged* ab; const bf16* a_log; const bf16* dt_bias; tagged* mix_out;
    // attention
    const tagged* qg; const tagged* kv_new; const bf16* q_norm; const bf16* k_norm;
    // MoE down projections and combine
    const tagged* hidden; const uint8_t* dw; const uint8_t* ds; const float* dg;
    const uint8_t* sw; const uint8_t* ss; const float* sg; const tagged* strength; tagged* out;
};
static_assert(sizeof(MegaPhase) % 16 == 0, "phases are copied in 16-byte pieces");

struct MegaParams {
    const MegaPhase* program; int nphases; int grid;
    qd_state st;
    const long long* token; const int* pos_dev; int pos_host;
    const bf16* embed; bf16* logits; long long* next_token;
    float* best_val; int* best_idx; unsigned int* argmax_counter;
    unsigned int* epoch; unsigned int* exit_count; unsigned int* status;
    uint2* attn_partial; int attn_splits;
    int hk, hv, dk, dv;            // DeltaNet heads
    int hq, hkv, d, rotary;        // attention heads
    float theta, eps;
    int conv_width, topk, experts, hidden, channels;
    int expert_lo, expert_hi;
    // expert parallel (world > 1): this rank's index and, per rank, the address of that rank's
    // exchange area in this process (peer memory); offsets inside the area are the same on
    // every rank
    int rank, world;
    unsigned long long peer_base[kMegaMaxRanks];
    long long contrib_offset;      // tagged [topk][hidden] per rank: routed contributions of the layer
    long long argmax_offset;       // uint2 [2][world] per rank: {value bits, index} and tag of the rank's best logit
    unsigned int wait_limit_us;    // bound of every wait, microseconds
    unsigned long long* trace;     // optional: [phase][16][grid] timestamps (ns)
};

int mega_launch(const MegaParams& p, cudaStream_t stream);
size_t mega_smem_bytes();

}  // namespace qd
