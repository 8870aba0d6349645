// Parameter block of the streaming matvec kernel (stream.cu).
//
// One launch multiplies ONE activation vector with a list of weight segments that share
// its width: NVFP4 row blocks, NVFP4 gate/up pairs (SwiGLU fused) and bf16 row blocks, all
// in the reference's checkpoint layout.  Weights travel global -> shared memory as 1-D
// bulk copies (TMA) through a ring of stages; every consumer warp keeps its slice of the
// activation vector in registers.
// A prologue can build the vector (residual add + RMSNorm, or the DeltaNet per-head gated
// norm), an epilogue can post-process each output row (short convolution, greedy argmax),
// and the block that completes the router rows can do the top-k routing for the next launch.
#pragma once
#include "common.cuh"

// Arguments of the op-table NVFP4 matvec family (ops.cu), shared with the streaming path.
struct Fp4Args {
    const bf16* x;
    const uint8_t* codes;  const uint8_t* scales;  const float* global;
    const uint8_t* up_codes; const uint8_t* up_scales; const float* up_global;
    const int32_t* ids; const float* routing;
    bf16* y;
    int rows, in_features, group, slots, per_slot_input, global_per_expert;
};

namespace qd {

constexpr int kStreamMaxSeg = 10;
constexpr int kStreamConsumerWarps = 16;   // they split the inputs of every NVFP4 row between them (rowmma.cuh)
constexpr int kStreamThreads = (kStreamConsumerWarps + 1) * 32;   // + one producer warp
constexpr int kStreamStages = 5;
constexpr int kStreamStageBytes = 36864;   // 32 NVFP4 rows of 2048 inputs, or 16 of 4096 (codes + scales)
constexpr int kStreamConvRows = 256;       // conv rows one block can stage
constexpr int kStreamConvWidth = 4;        // widest short convolution the fused epilogue takes

// SEG_FP8: static E4M3 rows [out][K] bytes with one fp32 scale per matrix (persistent kernel only)
enum SegKind { SEG_FP4 = 0, SEG_FP4_PAIR = 1, SEG_BF16 = 2, SEG_FP8 = 3 };
enum SegEpilogue { EP_PLAIN = 0, EP_CONV = 1, EP_ARGMAX = 2, EP_ROUTE = 3 };
enum Prologue { PRO_NONE = 0, PRO_ADD_NORM = 1, PRO_GATED_NORM = 2 };

struct StreamSeg {
    const uint8_t* w;  const uint8_t* s;  const float* g;     // codes / bf16 rows, scales, global
    const uint8_t* w2; const uint8_t* s2; const float* g2;    // "up" half of a pair
    bf16* y;                  // one bf16 per row
    long long w_stride, s_stride;   // bytes between experts of a bank
    int rows;
    int kind;                 // SegKind
    int epilogue;             // SegEpilogue
    int slot;                 // >= 0: expert id = ids[slot] selects the bank entry; -1: none
    int g_per_expert;         // global scale indexed by expert id
};

struct StreamParams {
    StreamSeg seg[kStreamMaxSeg];
    int nseg;
    int width;                // K: 2048 or 4096
    int prologue;
    // activation source
    const bf16* x;            // [K]
    const long long* token;   // when set, x = embed + (*token) * K (embedding row)
    const bf16* embed;
    const bf16* residual;     // PRO_ADD_NORM: may be null (first layer)
    const float* gamma;       // PRO_ADD_NORM: fp32 [K]
    float eps;
    bf16* residual_out;       // PRO_ADD_NORM: written by block 0
    bf16* x_out;              // prologue result, written by block 0 (may be null)
    const bf16* z;            // PRO_GATED_NORM: gate input [K]
    const bf16* head_gamma;   // PRO_GATED_NORM: bf16 [128]
    // expert ids of segments with slot >= 0 (device, written by an earlier launch or the caller)
    const int32_t* ids_in; int topk;
    int expert_lo, expert_hi; // owned expert range; routed segments outside it are skipped
    // EP_ROUTE: the segment's rows are router logits; the block that completes them selects
    // the top-k experts (quickdraw/models/qwen.py:174-177)
    int32_t* ids_out; float* weights_out; unsigned int* route_counter; int route_topk;
    // EP_CONV
    bf16* conv_state; const bf16* conv_taps; int conv_width;
    // EP_ARGMAX
    float* best_val; int* best_idx; unsigned int* counter; long long* token_out;
    unsigned int* status;
    unsigned int quota, remainder;   // filled by stream_launch: total cost = quota * grid + remainder
};

// grid <= 0 picks the default number of blocks per SM.  Returns a QD_* code.
int stream_launch(const StreamParams& p, int grid, cudaStream_t stream, bool pdl);
int stream_sm_count();

}  // namespace qd
