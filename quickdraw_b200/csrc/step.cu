// One decode step of the hybrid MoE model as a fixed sequence of fused launches, and the
// phase list of the same step for the persistent kernel
// (reference: quickdraw/models/qwen.py:196-241).  Per layer:
//   A  residual add + RMSNorm  ->  mixer input projections (+ short conv for DeltaNet)
//   M  DeltaNet recurrence, or split-context GQA attention
//   B  (DeltaNet: gated per-head norm ->) output projection
//   C  residual add + RMSNorm  ->  router logits, shared-expert gate logit, shared gate/up
//   D  top-k routing            ->  routed gate/up with SwiGLU
//   E  routed + shared down projections and the combine
// then   residual add + final RMSNorm -> bf16 LM head with greedy argmax.
// Every launch can be a programmatic dependent of the one before it, so its weight
// fetches overlap the predecessor's tail.  The model object is a host-side pointer table.
#include <new>
#include <vector>

#include "mega.cuh"

using namespace qd;

struct qd_model {
    qd_model_config cfg;
    std::vector<qd_layer> layers;
    std::vector<char> layer_set;
};

namespace {

struct Workspace {
    bf16 *resid[2], *xnorm, *big, *mid, *ab, *o, *mixed, *router_logits, *strength, *hidden, *moe_out, *shared_row;
    int32_t* ids; float* weights; float* routed_partial; float* attn_scratch;
    unsigned int* attn_counters; float* best_val; int* best_idx; unsigned int* argmax_counter;
    unsigned int* status; int* cursor; unsigned int* route_counter;
    // persistent kernel: the launch counter, the exit counter and the tagged activation words
    unsigned int* epoch; unsigned int* grid_exit;
    tagged *t_moe_out, *t_big, *t_mid, *t_ab, *t_o, *t_mixed, *t_router, *t_hidden;
    uint2* t_attn;
    size_t bytes;
};

constexpr int kAttnSplits = 32;
constexpr int kMaxGrid = 1024;

size_t align_up(size_t v) { return (v + 255) & ~size_t(255); }

Workspace carve(const qd_model_config& c, uint8_t* base) {
    Workspace w;
    size_t off = 0;
    auto take = [&](size_t bytes) { uint8_t* p = base ? base + off : nullptr; off += align_up(bytes); return p; };
    const int channels = 2 * c.key_heads * c.key_dim + c.value_heads * c.value_dim;
    const int q_width = c.q_heads * c.head_dim, kv_width = c.kv_heads * c.head_dim;
    const int value_width = c.value_heads * c.value_dim;
    const int big = channels > 2 * q_width ? channels : 2 * q_width;
    const int mid = value_width > 2 * kv_width ? value_width : 2 * kv_width;
    const int owide = value_width > q_width ? value_width : q_width;
    w.cursor = (int*)take(4);                       // which residual buffer is current
    w.status = (unsigned int*)take(4);
    w.argmax_counter = (unsigned int*)take(4);
    w.route_counter = (unsigned int*)take(4);
    w.attn_counters = (unsigned int*)take(4 * c.kv_heads);
    w.resid[0] = (bf16*)take(2 * c.hidden); w.resid[1] = (bf16*)take(2 * c.hidden);
    w.xnorm = (bf16*)take(2 * c.hidden);
    w.big = (bf16*)take(2 * big);
    w.mid = (bf16*)take(2 * mid);
    w.ab = (bf16*)take(2 * 2 * c.value_heads);
    w.o = (bf16*)take(2 * owide);
    w.mixed = (bf16*)take(2 * c.hidden);
    w.router_logits = (bf16*)take(2 * c.experts);
    w.strength = (bf16*)take(2);
    w.hidden = (bf16*)take(2 * (size_t)(c.topk + 1) * c.intermediate);
    w.ids = (int32_t*)take(4 * c.topk);
    w.weights = (float*)take(4 * c.topk);
    w.moe_out = (bf16*)take(2 * c.hidden);
    w.shared_row = (bf16*)take(2 * c.hidden);
    w.routed_partial = (float*)take(4 * c.hidden);
    w.attn_scratch = (float*)take(4 * (size_t)qd_attn_scratch_floats(c.q_heads, c.kv_heads, c.head_dim, kAttnSplits));
    w.best_val = (float*)take(4 * kMaxGrid);
    w.best_idx = (int*)take(4 * kMaxGrid);
    w.epoch = (unsigned int*)take(4);
    w.grid_exit = (unsigned int*)take(4);
    w.t_moe_out = (tagged*)take(4 * (size_t)c.hidden);
    w.t_big = (tagged*)take(4 * (size_t)big);
    w.t_mid = (tagged*)take(4 * (size_t)mid);
    w.t_ab = (tagged*)take(4 * 2 * (size_t)c.value_heads);
    w.t_o = (tagged*)take(4 * (size_t)owide);
    w.t_mixed = (tagged*)take(4 * (size_t)c.hidden);
    w.t_router = (tagged*)take(4 * ((size_t)c.experts + 4));          // logits, then the shared-expert gate logit
    w.t_hidden = (tagged*)take(4 * (size_t)(c.topk + 1) * c.intermediate);
    w.t_attn = (uint2*)take(8 * (size_t)c.kv_heads * kMegaAttnSplits * 8 * 258);
    w.bytes = off;
    return w;
}

bool fused_shape_ok(const qd_model_config& c) {
    return c.hidden == 2048 && c.value_heads * c.value_dim == 4096 && c.q_heads * c.head_dim == 4096 &&
           c.intermediate == 512 && c.key_dim <= 128 && c.value_dim == 128 && c.topk >= 1 && c.topk <= 8 &&
           c.experts <= 256 && c.head_dim <= 256 && c.q_heads / c.kv_heads <= 8 && c.conv_width >= 1 &&
           c.conv_width <= 32;
}

StreamSeg fp4_seg(const qd_fp4& w, int rows, bf16* y, int epilogue = EP_PLAIN) {
    StreamSeg s = {};
    s.w = (const uint8_t*)w.codes; s.s = (const uint8_t*)w.scales; s.g = w.global;
    s.y = y; s.rows = rows; s.kind = SEG_FP4; s.epilogue = epilogue; s.slot = -1;
    return s;
}
// a mixer projection: NVFP4, or static FP8 when the layer says so
StreamSeg mixer_seg(const qd_layer& ly, const qd_fp4& w, int rows, int epilogue = EP_PLAIN) {
    StreamSeg s = fp4_seg(w, rows, nullptr, epilogue);
    if (ly.mixers_fp8) { s.kind = SEG_FP8; s.s = nullptr; }
    return s;
}
StreamSeg bf16_seg(const void* w, int rows, bf16* y, int epilogue = EP_PLAIN) {
    StreamSeg s = {};
    s.w = (const uint8_t*)w; s.y = y; s.rows = rows; s.kind = SEG_BF16; s.epilogue = epilogue; s.slot = -1;
    return s;
}
StreamSeg pair_seg(const qd_fp4& gate, const qd_fp4& up, int rows, bf16* y) {
    StreamSeg s = fp4_seg(gate, rows, y);
    s.kind = SEG_FP4_PAIR;
    s.w2 = (const uint8_t*)up.codes; s.s2 = (const uint8_t*)up.scales; s.g2 = up.global;
    return s;
}

#define QD_TRY(expr) do { const int rc_ = (expr); if (rc_ != QD_OK) return rc_; } while (0)

int run_layers(qd_model* m, const qd_state* st, const long long* token, const int* pos_dev, int pos_host,
               void* workspace, int begin, int end, bool head, void* logits,
               long long* next_token, int flags, cudaStream_t stream) {
    const qd_model_config& c = m->cfg;
    if (!fused_shape_ok(c)) return QD_ERR_UNSUPPORTED;
    for (int L = begin; L < end; ++L)
        if (m->layers[L].mixers_fp8) return QD_ERR_UNSUPPORTED;      // static FP8 mixers: persistent step only
    if (head && c.lm_head_fp4.codes) return QD_ERR_UNSUPPORTED;      // NVFP4 LM head: persistent step only
    const bool pdl = flags & QD_FLAG_PDL;
    Workspace w = carve(c, (uint8_t*)workspace);
    const int H = c.hidden;
    const int channels = 2 * c.key_heads * c.key_dim + c.value_heads * c.value_dim;
    const int value_width = c.value_heads * c.value_dim;
    const int q_width = c.q_heads * c.head_dim, kv_width = c.kv_heads * c.head_dim;
    // Residual ping-pong: every add+norm flips it; two flips per layer, so the buffer index at
    // the start of layer L is always 0.
    for (int L = begin; L < end; ++L) {
        const qd_layer& ly = m->layers[L];
        if (!m->layer_set[L]) return QD_ERR_ARG;
        // ---- A
        StreamParams a = {};
        a.width = H; a.prologue = PRO_ADD_NORM; a.gamma = ly.gamma_in; a.eps = c.eps;
        a.residual_out = w.resid[1]; a.status = w.status; a.expert_hi = 0x7fffffff;
        if (L == 0) { a.token = token; a.embed = (const bf16*)c.embed; a.residual = nullptr; }
        else { a.x = w.moe_out; a.residual = w.resid[0]; }
        if (ly.is_attention) {
            a.nseg = 3;
            a.seg[0] = fp4_seg(ly.proj_a, 2 * q_width, w.big);
            a.seg[1] = fp4_seg(ly.proj_b, kv_width, w.mid);
            a.seg[2] = fp4_seg(ly.proj_c, kv_width, w.mid + kv_width);
        } else {
            a.nseg = 4;
            a.seg[0] = fp4_seg(ly.proj_a, channels, w.big, EP_CONV);
            a.seg[1] = fp4_seg(ly.proj_b, value_width, w.mid);
            a.seg[2] = bf16_seg(ly.in_proj_a, c.value_heads, w.ab);
            a.seg[3] = bf16_seg(ly.in_proj_b, c.value_heads, w.ab + c.value_heads);
            a.conv_state = (bf16*)st->conv_state + (size_t)ly.state_index * channels * (c.conv_width - 1);
            a.conv_taps = (const bf16*)ly.conv1d; a.conv_width = c.conv_width;
        }
        QD_TRY(stream_launch(a, 0, stream, pdl));
        // ---- M and B
        StreamParams b = {};
        b.width = 4096; b.status = w.status; b.expert_hi = 0x7fffffff; b.eps = c.eps;
        b.x = w.o; b.nseg = 1; b.seg[0] = fp4_seg(ly.proj_out, H, w.mixed);
        if (ly.is_attention) {
            const size_t layer_elems = (size_t)st->capacity * kv_width;
            QD_TRY(qd_attn_decode(w.big, w.mid, w.mid + kv_width, ly.q_norm, ly.k_norm,
                                  (bf16*)st->kv_k + ly.state_index * layer_elems,
                                  (bf16*)st->kv_v + ly.state_index * layer_elems, w.o, w.attn_scratch,
                                  w.attn_counters, pos_dev, pos_host, st->capacity, c.q_heads, c.kv_heads,
                                  c.head_dim, c.rotary_dim, c.rope_theta, c.eps, kAttnSplits, pdl, stream));
            b.prologue = PRO_NONE;
        } else {
            QD_TRY(qd_gdn_recurrence(w.big, w.ab, w.ab + c.value_heads, ly.a_log, ly.dt_bias,
                                     st->rec_state + (size_t)ly.state_index * c.value_heads * c.key_dim * c.value_dim,
                                     w.o, c.key_heads, c.value_heads, c.key_dim, c.value_dim, pdl, stream));
            b.prologue = PRO_GATED_NORM; b.z = w.mid; b.head_gamma = (const bf16*)ly.head_norm;
        }
        QD_TRY(stream_launch(b, 0, stream, pdl));
        // ---- C
        StreamParams cc = {};
        cc.width = H; cc.prologue = PRO_ADD_NORM; cc.gamma = ly.gamma_post; cc.eps = c.eps;
        cc.x = w.mixed; cc.residual = w.resid[1]; cc.residual_out = w.resid[0]; cc.x_out = w.xnorm;
        cc.status = w.status; cc.expert_hi = 0x7fffffff;
        cc.nseg = 3;
        cc.seg[0] = bf16_seg(ly.router, c.experts, w.router_logits, EP_ROUTE);
        cc.ids_out = w.ids; cc.weights_out = w.weights; cc.route_counter = w.route_counter; cc.route_topk = c.topk;
        cc.seg[1] = bf16_seg(ly.shared_expert_gate, 1, w.strength);
        cc.seg[2] = pair_seg(ly.shared_gate, ly.shared_up, c.intermediate, w.hidden + (size_t)c.topk * c.intermediate);
        QD_TRY(stream_launch(cc, 0, stream, pdl));
        // ---- D
        StreamParams d = {};
        d.width = H; d.prologue = PRO_NONE; d.x = w.xnorm; d.status = w.status;
        d.ids_in = w.ids; d.topk = c.topk;
        d.expert_lo = c.expert_lo; d.expert_hi = c.expert_hi;
        d.nseg = c.topk;
        for (int s = 0; s < c.topk; ++s) {
            StreamSeg sg = pair_seg(ly.experts_gate, ly.experts_up, c.intermediate, w.hidden + (size_t)s * c.intermediate);
            sg.slot = s; sg.g_per_expert = ly.experts_global_per_expert;
            sg.w_stride = (long long)c.intermediate * (H / 2);
            sg.s_stride = (long long)c.intermediate * (H / 16);
            d.seg[s] = sg;
        }
        QD_TRY(stream_launch(d, 0, stream, pdl));
        // ---- E
        QD_TRY(qd_moe_down_combine(w.hidden, w.ids, w.weights, ly.experts_down.codes, ly.experts_down.scales,
                                   ly.experts_down.global, ly.shared_down.codes, ly.shared_down.scales,
                                   ly.shared_down.global, w.strength, w.moe_out, nullptr, nullptr, H, c.intermediate,
                                   c.topk, ly.experts_global_per_expert, c.expert_lo, c.expert_hi, pdl, stream));
    }
    if (head) {
        StreamParams h = {};
        h.width = H; h.prologue = PRO_ADD_NORM; h.gamma = c.final_gamma; h.eps = c.eps;
        h.x = w.moe_out; h.residual = w.resid[0]; h.residual_out = w.resid[1];
        h.status = w.status; h.expert_hi = 0x7fffffff;
        h.nseg = 1;
        h.seg[0] = bf16_seg(c.lm_head, c.vocab, (bf16*)logits, EP_ARGMAX);
        h.best_val = w.best_val; h.best_idx = w.best_idx; h.counter = w.argmax_counter; h.token_out = next_token;
        int grid = stream_sm_count() * 2;
        if (grid > kMaxGrid) grid = kMaxGrid;
        QD_TRY(stream_launch(h, grid, stream, pdl));
    }
    return QD_OK;
}

}  // namespace

extern "C" int qd_model_create(const qd_model_config* config, qd_model** out) {
    QD_CHECK_ARG(config && out && config->layers > 0 && config->hidden > 0);
    qd_model* m = new (std::nothrow) qd_model();
    if (!m) return QD_ERR_ARG;
    m->cfg = *config;
    m->layers.resize(config->layers);
    m->layer_set.assign(config->layers, 0);
    *out = m;
    return QD_OK;
}

extern "C" int qd_model_set_layer(qd_model* model, int index, const qd_layer* layer) {
    QD_CHECK_ARG(model && layer && index >= 0 && index < model->cfg.layers);
    model->layers[index] = *layer;
    model->layer_set[index] = 1;
    return QD_OK;
}

extern "C" int qd_model_destroy(qd_model* model) {
    delete model;
    return QD_OK;
}

extern "C" long long qd_decode_workspace_bytes(const qd_model* model) {
    if (!model) return -1;
    return (long long)carve(model->cfg, nullptr).bytes;
}

extern "C" int qd_decode_step(qd_model* model, const qd_state* state, const long long* token,
                              const int* position_dev, int position_host, void* workspace, void* logits_out,
                              long long* next_token, int flags, void* stream) {
    QD_CHECK_ARG(model && state && token && workspace && logits_out && next_token);
    if (model->cfg.expert_lo != 0 || model->cfg.expert_hi < model->cfg.experts || model->cfg.vocab_hi != 0)
        return QD_ERR_UNSUPPORTED;      // model slices run through the persistent kernel only
    return run_layers(model, state, token, position_dev, position_host, workspace, 0, model->cfg.layers,
                      !(flags & QD_FLAG_NO_LOGITS), logits_out, next_token, flags, (cudaStream_t)stream);
}

extern "C" int qd_nvfp4_gemv_bank(const void* x, const void* codes, const void* scales, const float* global,
                                  void* y, int rows, int in_features, int matrices, int pdl, void* stream) {
    QD_CHECK_ARG(x && codes && scales && global && y && rows > 0 && matrices > 0);
    if (in_features != 2048 && in_features != 4096) return QD_ERR_UNSUPPORTED;
    for (int i = 0; i < matrices; ++i) {
        StreamParams p = {};
        p.width = in_features; p.prologue = PRO_NONE; p.x = (const bf16*)x; p.expert_hi = 0x7fffffff;
        p.nseg = 1;
        qd_fp4 w = {(const uint8_t*)codes + (size_t)i * rows * (in_features / 2),
                    (const uint8_t*)scales + (size_t)i * rows * (in_features / 16), global};
        p.seg[0] = fp4_seg(w, rows, (bf16*)y + (size_t)i * rows);
        QD_TRY(stream_launch(p, 0, (cudaStream_t)stream, pdl != 0));
    }
    return QD_OK;
}

// ------------------------------------------------------------- persistent kernel program
namespace {

unsigned int g_wait_limit_us = 200000;      // bound of every device-side wait of the persistent kernel

MegaSeg mega_seg(const StreamSeg& s, tagged* y) {
    MegaSeg m = {};
    m.w = s.w; m.s = s.s; m.g = s.g; m.w2 = s.w2; m.s2 = s.s2; m.g2 = s.g2; m.y = y;
    m.w_stride = s.w_stride; m.s_stride = s.s_stride; m.rows = s.rows;
    m.kind = (short)s.kind; m.epilogue = (short)s.epilogue; m.slot = (short)s.slot; m.g_per_expert = (short)s.g_per_expert;
    return m;
}

// Cost partition of a streaming phase over `grid` blocks; false if it does not fit.
bool mega_finish_stream(MegaPhase& ph, int grid) {
    unsigned long long total = 0;
    const unsigned fp4_row = (ph.width / 2 + ph.width / 16) / 16;
    for (int i = 0; i < ph.nseg; ++i) {
        const unsigned cost = ph.seg[i].kind == SEG_BF16 ? 2u * ph.width / 16 : ph.seg[i].kind == SEG_FP8 ? (unsigned)ph.width / 16
                              : ph.seg[i].kind == SEG_FP4_PAIR ? 2 * fp4_row : fp4_row;
        total += (unsigned long long)ph.seg[i].rows * cost;
        if (ph.seg[i].epilogue == EP_CONV && ph.seg[i].rows / grid + 2 > kMegaConvRows) return false;
    }
    if (total + 1024 >= 0xffffffffull) return false;
    ph.quota = (unsigned)(total / grid);
    ph.remainder = (unsigned)(total % grid);
    // Equal NVFP4 pair segments (shared expert + routed slots): a group of blocks per segment,
    // whole 16-pair tiles per block.  A block that straddles two experts would run a partial tile
    // of each, one tile more than its neighbours, and the phase ends with its slowest block.
    ph.seg_blocks = ph.seg_cost = ph.block_cost = 0;
    bool equal = ph.nseg > 1 && ph.nseg <= grid;
    for (int i = 0; i < ph.nseg && equal; ++i)
        equal = ph.seg[i].kind == SEG_FP4_PAIR && ph.seg[i].rows == ph.seg[0].rows;
    if (equal) {
        const unsigned blocks = (unsigned)(grid / ph.nseg), rows = (unsigned)ph.seg[0].rows;
        unsigned per = (rows + blocks - 1) / blocks;
        per = (per + 15) / 16 * 16;                      // pairs per block: whole tiles
        ph.seg_blocks = blocks;
        ph.seg_cost = rows * 2 * fp4_row;
        ph.block_cost = per * 2 * fp4_row;
    }
    return true;
}

// six phases per layer, one more (the split merge) per attention layer, and the LM head
int mega_phase_count(const qd_model* m) {
    int n = 6 * m->cfg.layers + 1;
    for (int L = 0; L < m->cfg.layers; ++L) n += m->layers[L].is_attention ? 1 : 0;
    return n;
}

bool mega_shape_ok(const qd_model_config& c, int grid) {
    return fused_shape_ok(c) && c.expert_lo >= 0 && c.expert_hi > c.expert_lo && c.conv_width <= kStreamConvWidth &&
           c.key_dim == 128 && c.value_dim % 32 == 0 && c.value_heads * (c.value_dim / 32) <= grid &&
           c.head_dim == 256 && c.rotary_dim <= 256 && c.rotary_dim % 64 == 0 && c.kv_heads >= 1 && c.kv_heads <= grid &&
           c.q_heads / c.kv_heads <= 8 && (c.hidden + grid - 1) / grid <= kMegaDownRows &&
           c.topk + 1 <= 9 && c.topk + 1 <= kMegaMaxSeg && c.conv_width <= 4 && grid <= kMaxGrid &&
           c.experts % 8 == 0 && c.layers <= kMegaMaxLayers && c.vocab_lo >= 0 &&
           (c.vocab_hi == 0 || (c.vocab_hi > c.vocab_lo && c.vocab_hi <= c.vocab));
}

int mega_attn_splits(const qd_model_config& c, int grid) {
    int s = grid / c.kv_heads;
    return s > kMegaAttnSplits ? kMegaAttnSplits : s;
}

// Exchange area of one rank (expert parallel): the routed contributions of every layer, then
// two sets of per-rank (best logit, index) pairs.
long long exchange_contrib_bytes(const qd_model_config& c) {
    return (long long)align_up((size_t)c.layers * c.topk * c.hidden * 4);
}

}  // namespace

extern "C" long long qd_exchange_bytes(const qd_model* model) {
    if (!model) return -1;
    return exchange_contrib_bytes(model->cfg) + 2 * kMegaMaxRanks * 16;
}

extern "C" int qd_set_wait_limit_us(unsigned int microseconds) {
    if (microseconds == 0) return QD_ERR_ARG;
    g_wait_limit_us = microseconds;
    return QD_OK;
}

extern "C" long long qd_program_bytes(const qd_model* model) {
    if (!model) return -1;
    return (long long)mega_phase_count(model) * (long long)sizeof(MegaPhase);
}

extern "C" int qd_program_build(const qd_model* model, void* workspace, void* host_out, long long bytes) {
    QD_CHECK_ARG(model && workspace && host_out);
    const qd_model_config& c = model->cfg;
    const int grid = stream_sm_count();
    if (!mega_shape_ok(c, grid)) return QD_ERR_UNSUPPORTED;
    if (bytes < qd_program_bytes(model)) return QD_ERR_ARG;
    Workspace w = carve(c, (uint8_t*)workspace);
    MegaPhase* out = (MegaPhase*)host_out;
    const int H = c.hidden;
    const int channels = 2 * c.key_heads * c.key_dim + c.value_heads * c.value_dim;
    const int value_width = c.value_heads * c.value_dim;
    const int q_width = c.q_heads * c.head_dim, kv_width = c.kv_heads * c.head_dim;
    int n = 0;
    for (int L = 0; L < c.layers; ++L) {
        if (!model->layer_set[L]) return QD_ERR_ARG;
        const qd_layer& ly = model->layers[L];
        // ---- A: residual add + norm -> mixer input projections
        MegaPhase a = {};
        a.kind = MK_STREAM; a.width = H; a.prologue = PRO_ADD_NORM; a.layer = L; a.state_index = ly.state_index;
        a.gamma = ly.gamma_in;
        if (L == 0) a.from_token = 1;
        else { a.x = w.t_moe_out; a.x_prev_layer = 1; }
        if (ly.is_attention) {
            a.nseg = 3;
            a.seg[0] = mega_seg(mixer_seg(ly, ly.proj_a, 2 * q_width), w.t_big);
            a.seg[1] = mega_seg(mixer_seg(ly, ly.proj_b, kv_width), w.t_mid);
            a.seg[2] = mega_seg(mixer_seg(ly, ly.proj_c, kv_width), w.t_mid + kv_width);
        } else {
            a.nseg = 4;
            a.seg[0] = mega_seg(mixer_seg(ly, ly.proj_a, channels, EP_CONV), w.t_big);
            a.seg[1] = mega_seg(mixer_seg(ly, ly.proj_b, value_width), w.t_mid);
            a.seg[2] = mega_seg(bf16_seg(ly.in_proj_a, c.value_heads, nullptr), w.t_ab);
            a.seg[3] = mega_seg(bf16_seg(ly.in_proj_b, c.value_heads, nullptr), w.t_ab + c.value_heads);
            a.conv_taps = (const bf16*)ly.conv1d;
        }
        if (ly.mixers_fp8) {
            if (!ly.mixer_input_scale || !ly.out_input_scale) return QD_ERR_ARG;
            a.in_scale = ly.mixer_input_scale;
        }
        if (!mega_finish_stream(a, grid)) return QD_ERR_UNSUPPORTED;
        out[n++] = a;
        // ---- M: mixer core
        MegaPhase m = {};
        m.layer = L; m.state_index = ly.state_index; m.mix_out = w.t_o;
        if (ly.is_attention) {
            m.kind = MK_ATTN;
            m.qg = w.t_big; m.kv_new = w.t_mid;
            m.q_norm = (const bf16*)ly.q_norm; m.k_norm = (const bf16*)ly.k_norm;
            out[n++] = m;
            m.kind = MK_ATTN_MERGE;       // second half: merge of the context splits, gate
        } else {
            m.kind = MK_GDN;
            m.qkv = w.t_big; m.ab = w.t_ab;
            m.a_log = (const bf16*)ly.a_log; m.dt_bias = (const bf16*)ly.dt_bias;
        }
        out[n++] = m;
        // ---- B: output projection
        MegaPhase b = {};
        b.kind = MK_STREAM; b.width = 4096; b.layer = L; b.x = w.t_o;
        b.nseg = 1; b.seg[0] = mega_seg(mixer_seg(ly, ly.proj_out, H), w.t_mixed);
        if (ly.mixers_fp8) b.in_scale = ly.out_input_scale;
        if (ly.is_attention) b.prologue = PRO_NONE;
        else { b.prologue = PRO_GATED_NORM; b.z = w.t_mid; b.head_gamma = (const bf16*)ly.head_norm; }
        if (!mega_finish_stream(b, grid)) return QD_ERR_UNSUPPORTED;
        out[n++] = b;
        // ---- C: residual add + norm -> router logits, shared gate logit
        MegaPhase cc = {};
        cc.kind = MK_STREAM; cc.width = H; cc.prologue = PRO_ADD_NORM; cc.layer = L;
        cc.gamma = ly.gamma_post; cc.x = w.t_mixed;
        cc.nseg = 2;
        cc.seg[0] = mega_seg(bf16_seg(ly.router, c.experts, nullptr), w.t_router);
        cc.seg[1] = mega_seg(bf16_seg(ly.shared_expert_gate, 1, nullptr), w.t_router + c.experts);
        if (!mega_finish_stream(cc, grid)) return QD_ERR_UNSUPPORTED;
        out[n++] = cc;
        // ---- D: routing; the shared expert's gate/up (its weights do not wait for the routing),
        //         then the routed gate/up pairs, all on the vector phase C built
        MegaPhase d = {};
        d.kind = MK_STREAM; d.width = H; d.prologue = PRO_NONE; d.layer = L; d.keep_x = 1; d.route = 1; d.uses_ids = 1;
        d.router_logits = w.t_router; d.ids_out = w.ids; d.weights_out = w.weights;
        d.nseg = c.topk + 1;
        d.seg[0] = mega_seg(pair_seg(ly.shared_gate, ly.shared_up, c.intermediate, nullptr),
                            w.t_hidden + (size_t)c.topk * c.intermediate);
        for (int s = 0; s < c.topk; ++s) {
            StreamSeg sg = pair_seg(ly.experts_gate, ly.experts_up, c.intermediate, nullptr);
            sg.slot = s; sg.g_per_expert = ly.experts_global_per_expert;
            sg.w_stride = (long long)c.intermediate * (H / 2);
            sg.s_stride = (long long)c.intermediate * (H / 16);
            d.seg[s + 1] = mega_seg(sg, w.t_hidden + (size_t)s * c.intermediate);
        }
        if (!mega_finish_stream(d, grid)) return QD_ERR_UNSUPPORTED;
        // ---- E: down projections and combine.  Phase D carries the same weight pointers: its
        //         producer fetches the down-projection rows as soon as the routing is known.
        MegaPhase e = {};
        e.kind = MK_DOWN; e.layer = L; e.uses_ids = 1;
        e.hidden = w.t_hidden; e.dw = (const uint8_t*)ly.experts_down.codes; e.ds = (const uint8_t*)ly.experts_down.scales;
        e.dg = ly.experts_down.global; e.g_per_expert = ly.experts_global_per_expert;
        e.sw = (const uint8_t*)ly.shared_down.codes; e.ss = (const uint8_t*)ly.shared_down.scales; e.sg = ly.shared_down.global;
        e.strength = w.t_router + c.experts; e.out = w.t_moe_out;
        d.dw = e.dw; d.ds = e.ds; d.sw = e.sw; d.ss = e.ss;
        out[n++] = d;
        out[n++] = e;
    }
    // ---- head: residual add + final norm -> this rank's LM head rows with greedy argmax
    MegaPhase h = {};
    h.kind = MK_STREAM; h.width = H; h.prologue = PRO_ADD_NORM; h.layer = c.layers; h.argmax = 1;
    h.gamma = c.final_gamma; h.x = w.t_moe_out; h.x_prev_layer = 1;
    h.nseg = 1;
    const int vocab_lo = c.vocab_hi ? c.vocab_lo : 0, vocab_hi = c.vocab_hi ? c.vocab_hi : c.vocab;
    h.seg[0] = c.lm_head_fp4.codes ? mega_seg(fp4_seg(c.lm_head_fp4, vocab_hi - vocab_lo, nullptr, EP_ARGMAX), nullptr)
                                   : mega_seg(bf16_seg(c.lm_head, vocab_hi - vocab_lo, nullptr, EP_ARGMAX), nullptr);
    h.row_lo = vocab_lo;
    if (!mega_finish_stream(h, grid)) return QD_ERR_UNSUPPORTED;
    out[n++] = h;
    return n == mega_phase_count(model) ? QD_OK : QD_ERR_ARG;
}

extern "C" int qd_decode_step_persistent(const qd_model* model, const qd_state* state, const long long* token,
                                         const int* position_dev, int position_host, void* workspace,
                                         const void* program, const qd_exchange* exchange, void* logits_out,
                                         long long* next_token, int flags, unsigned long long* trace, void* stream) {
    QD_CHECK_ARG(model && state && token && workspace && program && next_token);
    QD_CHECK_ARG((flags & QD_FLAG_NO_LOGITS) || logits_out);
    QD_CHECK_ARG(position_dev || (position_host >= 0 && position_host < state->capacity));
    const qd_model_config& c = model->cfg;
    const int grid = stream_sm_count();
    if (!mega_shape_ok(c, grid)) return QD_ERR_UNSUPPORTED;
    const bool sharded = c.expert_lo != 0 || c.expert_hi < c.experts || c.vocab_hi != 0;
    QD_CHECK_ARG(!sharded || (exchange && exchange->world > 1));
    Workspace w = carve(c, (uint8_t*)workspace);
    MegaParams p = {};
    p.program = (const MegaPhase*)program;
    // Under expert parallelism the LM head always runs: its exchange of the ranks' best logits is
    // also what keeps a rank from starting the next token while another still reads this one's
    // contributions.
    const bool skip_head = (flags & QD_FLAG_NO_LOGITS) && !(exchange && exchange->world > 1);
    QD_CHECK_ARG(skip_head || logits_out);
    p.nphases = mega_phase_count(model) - (skip_head ? 1 : 0);
    p.grid = grid;
    p.st = *state;
    p.token = token; p.pos_dev = position_dev; p.pos_host = position_host;
    p.embed = (const bf16*)c.embed; p.logits = (bf16*)logits_out; p.next_token = next_token;
    p.best_val = w.best_val; p.best_idx = w.best_idx; p.argmax_counter = w.argmax_counter;
    p.epoch = w.epoch; p.exit_count = w.grid_exit; p.status = w.status;
    p.attn_partial = w.t_attn; p.attn_splits = mega_attn_splits(c, grid);
    p.hk = c.key_heads; p.hv = c.value_heads; p.dk = c.key_dim; p.dv = c.value_dim;
    p.hq = c.q_heads; p.hkv = c.kv_heads; p.d = c.head_dim; p.rotary = c.rotary_dim;
    p.theta = c.rope_theta; p.eps = c.eps;
    p.conv_width = c.conv_width; p.topk = c.topk; p.experts = c.experts; p.hidden = c.hidden;
    p.channels = 2 * c.key_heads * c.key_dim + c.value_heads * c.value_dim;
    p.expert_lo = c.expert_lo; p.expert_hi = c.expert_hi;
    p.rank = 0; p.world = 1;
    if (exchange && exchange->world > 1) {
        QD_CHECK_ARG(exchange->world <= kMegaMaxRanks && exchange->rank >= 0 && exchange->rank < exchange->world);
        p.rank = exchange->rank; p.world = exchange->world;
        for (int r = 0; r < p.world; ++r) {
            QD_CHECK_ARG(exchange->peer_base[r] != 0 && (exchange->peer_base[r] & 15ull) == 0);
            p.peer_base[r] = exchange->peer_base[r];
        }
        p.contrib_offset = 0;
        p.argmax_offset = exchange_contrib_bytes(c);
    }
    p.wait_limit_us = g_wait_limit_us;
    p.trace = trace;
    return mega_launch(p, (cudaStream_t)stream);
}
