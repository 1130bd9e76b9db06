// gpt2_forward: the driver the reference's kernels plug into.  The reference ships only the
// kernels (README.md:19 names llm.c's train_gpt2_fp32.cu as the program they were dropped into);
// the operator order is the one drawn in images/gpt2/gpt2_flow.png and listed in README.md:9-15,
// with every layernorm except the first fused with the residual add before it
// (README.md:255-256).  Forward only, so one set of per-layer activations is reused by all
// layers; parameters keep the flat fp32 layout documented in include/b200gpt2.h.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <new>
#include <utility>
#include <vector>
#include "../api/ctx.h"
#include "../kernels/kernels.h"

struct b200_gpt2 {
    b200_ctx* ctx = nullptr;
    b200_gpt2_config cfg{};
    int max_B = 0, max_T = 0;
    size_t n_params = 0;
    size_t off[17] = {};
    float* params = nullptr;
    float* params_r = nullptr;     // TF32-rounded copy of the five weight matrices (same offsets; round_operands)
    float* qkv_small = nullptr;    // scratch of the 3xTF32 attention (allocated by set_options)
    bool weights_rounded = false;
    uint16_t* params_h = nullptr;  // bf16 copy of the weight matrices (same offsets) for the bf16 modes
    uint16_t* params_l = nullptr;  // what that rounding dropped, again as bf16 (B200_BF16X3)
    bool params_h_ready = false, params_l_ready = false;
    // activations, sized for max_B * max_T rows
    float *residual = nullptr, *ln_out = nullptr, *qkv = nullptr, *atty = nullptr,
          *branch = nullptr, *fch = nullptr, *logits = nullptr;
    int* tokens = nullptr;
    int* argmax = nullptr;
    unsigned long long* argmax_keys = nullptr;  // per row: best (value, column) of the lm-head's fused arg-max; zero between forwards
    float* last_logits = nullptr;               // logits of the last position of every sequence, gathered for the host [max rows/64][Vp]
    float *kcache = nullptr, *vcache = nullptr;  // [L][max_B][max_T][C] each (b200_gpt2_enable_kv_cache)
    bool keep_kv = false;                        // the forward being enqueued also fills the cache
    int* pos_dev = nullptr;                      // position of the decode step being run
    float* resid2 = nullptr;                     // second residual buffer of the decode step [16][C]
    float* att_partial = nullptr;                // decode attention: softmax states of the position splits
    unsigned int* att_counters = nullptr;        // ... and their arrival counters (zero between launches)
    int* gen_tokens = nullptr;                   // greedy generation: prompt and continuation [max_B][max_T]
    cudaEvent_t host_done[2] = {nullptr, nullptr};  // forward_host_enqueue / _wait: results of a slot are on the host
    int* h_slot_status = nullptr;                // pinned: the device status word as seen behind each slot's work
    int* d_slot_status = nullptr;                // the same two words as the device addresses them
    // Host-buffer forward without copies: device views of the caller's pinned buffers, written by
    // the kernel behind the lm-head (null: the model's own buffers).  Set around one enqueue_forward.
    struct HostDst { int* ids = nullptr; float* last = nullptr; int* status = nullptr; } host_dst;
    // b200_gpt2_forward_sample: what the lm-head's epilogue computes besides (or instead of) the arg-max;
    // set around one enqueue_forward
    const b200::GemmRowStats* row_stats = nullptr;
    float2* lse_part = nullptr;                  // log-sum-exp partials [max rows][2 * ceil(Vp / 256)]
    std::map<int, cudaGraphExec_t> decode_graphs;  // by B (the position is read from pos_dev)
    int round_operands = 1, gemm_mode = B200_BF16X3, lmhead_mode = B200_BF16X3, use_graph = 0;
    int att_mode = -1;  // -1: split-operand attention exactly when gemm_mode is B200_TF32X3
    // tensor parallelism (Megatron style): this rank's share of the attention heads, of the MLP
    // width and of the vocabulary; with tp_size == 1 these are the full dimensions
    int tp_size = 1, tp_rank = 0;
    int attn_c = 0;    // channels of the local heads (nh_local * 64)
    int nh_local = 0;
    int mlp_c = 0;     // local width of the MLP hidden layer (4C / tp_size)
    int vp_local = 0;  // local width of the logits
    int vp_row0 = 0;   // first row of wte used by the local lm-head
    b200_allreduce_fn allreduce = nullptr;
    void* allreduce_user = nullptr;
    // the all-reduces of a projection run on a stream of their own, chunk by chunk under the GEMM
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t tp_ev[9] = {};  // [0..7] chunk computed, [8] all chunks reduced
    // Row chunks of a projection (1: one GEMM, then one all-reduce on the compute stream) and the SMs
    // the later chunks' GEMMs leave to the communication kernels running beside them.  Measured on
    // two B200s (GPT-2 XL, 8192 rows): 40.7 ms per step unchunked, 44.0 with 2 chunks, 48.5 with 4
    // (42.9 / 47.7 with 16 SMs set aside) - the shorter GEMMs and smaller messages cost more than
    // the overlap hides - so chunking is off unless asked for.
    int tp_chunks = 1;
    int tp_reserve_sms = 0;
    // Two-way tensor parallelism without an all-reduce (b200_gpt2_tp_peer_*): the projection GEMM
    // stores every tile of its partial sum a second time, into the peer GPU's memory, while it
    // computes; a word written after the GEMM tells the peer that the sum is complete, and the fused
    // residual + layernorm adds the two partial sums itself.  Two receive buffers, used in turn:
    // the peer's GEMM number e + 2 - the next writer of the buffer my layernorm number e reads -
    // is behind its layernorm e + 1, which waited for my GEMM e + 1, which follows my layernorm e.
    float* peer_in[2] = {nullptr, nullptr};   // local: receives the peer's partial sums
    unsigned int* peer_word = nullptr;         // local: [0] the peer's epoch of completed GEMMs
    float* peer_out[2] = {nullptr, nullptr};  // the peer's peer_in, mapped into this process
    unsigned int* peer_word_remote = nullptr;  // the peer's peer_word, mapped
    CUtensorMap* peer_maps = nullptr;          // device copies of the tensor maps over peer_out[0..1], per projection width
    int peer_maps_rows = 0;
    unsigned int peer_epoch = 0;
    bool peer_on = false;
    // Sequence-parallel hand-over for any group size (b200_gpt2_tp_sp_*): rank r owns rows [r, r+1) * M / n of
    // the residual stream.  A projection GEMM stores every tile of its partial sum only to the owner of the
    // tile's rows (into the slot of the source rank; TMA stores over NVLink under the GEMM), the owner's
    // layernorm adds the n partial sums for its rows and writes the normalised rows into every rank's
    // layernorm output, and two epoch words per peer order it all: per projection each rank sends
    // (n-1)/n of the activation twice, like an all-reduce, the first half hidden under the GEMM.
    bool sp_on = false;
    float* sp_recv = nullptr;                 // local [2 (epoch parity)][max_B * max_T * C]: [source rank][own rows][C]
    unsigned int* sp_words = nullptr;         // local: [s] projections completed by rank s, [16 + s] layernorms completed by rank s
    float* sp_recv_peer[8] = {};              // the peers' sp_recv / layernorm output / words, mapped (own entries unused)
    float* sp_ln_peer[8] = {};
    unsigned int* sp_words_peer[8] = {};
    CUtensorMap* sp_maps = nullptr;           // device [2][8]: by parity and owner, over the owner's slot for this rank
    int sp_maps_rows = 0;
    unsigned int sp_epoch = 0;
    std::map<std::pair<std::pair<int, int>, int>, cudaGraphExec_t> graphs;  // by (B, T, results)
    // per-operator timing (b200_gpt2_set_profile): one event pair per kernel launch
    bool profile = false;
    std::vector<cudaEvent_t> ev_pool;
    std::vector<int> ev_cat;     // category of each recorded pair
    size_t ev_used = 0;          // events handed out since the last read-out
    double prof_ms[B200_PROF_NUM] = {};
    long prof_launches[B200_PROF_NUM] = {};
};

namespace {

int tp_heads(int NH, int n, int r) { return NH / n + (r < NH % n ? 1 : 0); }
int tp_head0(int NH, int n, int r) { return r * (NH / n) + (r < NH % n ? r : NH % n); }

// offsets of the 16 parameter tensors in the (rank-local) flat layout
size_t local_param_offsets(const b200_gpt2_config* cfg, int attn_c, int mlp_c, size_t* offsets) {
    const size_t C = cfg->channels, L = cfg->num_layers, Vp = cfg->padded_vocab_size, mT = cfg->max_seq_len;
    const size_t A = attn_c, F = mlp_c;
    const size_t sizes[16] = {Vp * C, mT * C, L * C, L * C, L * 3 * A * C, L * 3 * A, L * C * A, L * C,
                              L * C, L * C, L * F * C, L * F, L * C * F, L * C, C, C};
    size_t o = 0;
    for (int i = 0; i < 16; ++i) { if (offsets) offsets[i] = o; o += sizes[i]; }
    if (offsets) offsets[16] = o;
    return o;
}

// fills the rank-local dimensions; returns false if the model cannot be split this way
bool set_tp_dims(b200_gpt2* m, int tp_size, int tp_rank) {
    const b200_gpt2_config& c = m->cfg;
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size || tp_size > c.num_heads) return false;
    if ((4 * c.channels) % tp_size || ((4 * c.channels) / tp_size) % 4) return false;
    m->tp_size = tp_size;
    m->tp_rank = tp_rank;
    m->nh_local = tp_heads(c.num_heads, tp_size, tp_rank);
    m->attn_c = m->nh_local * 64;
    m->mlp_c = 4 * c.channels / tp_size;
    // the lm-head is split over the vocabulary when it divides evenly (logits stay sharded),
    // otherwise every rank computes all of it
    if (c.padded_vocab_size % tp_size == 0 && (c.padded_vocab_size / tp_size) % 4 == 0) {
        m->vp_local = c.padded_vocab_size / tp_size;
        m->vp_row0 = tp_rank * m->vp_local;
    } else {
        m->vp_local = c.padded_vocab_size;
        m->vp_row0 = 0;
    }
    m->n_params = local_param_offsets(&m->cfg, m->attn_c, m->mlp_c, m->off);
    return true;
}

}  // namespace

namespace {

// hands out a start/stop event pair for category `cat` and records the start
int prof_begin(b200_gpt2* m, int cat) {
    if (m->ev_used + 2 > m->ev_pool.size()) {
        for (int i = 0; i < 256; ++i) {
            cudaEvent_t e;
            B200_CUDA(m->ctx, cudaEventCreate(&e));
            m->ev_pool.push_back(e);
        }
    }
    m->ev_cat.push_back(cat);
    B200_CUDA(m->ctx, cudaEventRecord(m->ev_pool[m->ev_used], m->ctx->stream));
    m->ev_used += 2;
    return B200_OK;
}
int prof_end(b200_gpt2* m) {
    B200_CUDA(m->ctx, cudaEventRecord(m->ev_pool[m->ev_used - 1], m->ctx->stream));
    return B200_OK;
}

int tp_allreduce(b200_gpt2* m, float* buf, size_t count) {
    if (!m->allreduce) return B200_ERR_STATE;
    return m->allreduce(m->allreduce_user, buf, count, m->ctx->stream) == 0 ? B200_OK : B200_ERR_CUDA;
}

// Tensor parallel: out[M,N] = inp[M,K] . w^T + bias as a partial sum, then summed over the ranks.
// The rows are cut into chunks; each chunk's all-reduce is issued on the communication stream as
// soon as its GEMM has been queued, so the transfer of chunk c runs under the GEMM of chunk c+1 and
// only the last chunk's all-reduce is exposed.  The compute stream continues once every chunk is
// reduced.  (Row chunks do not change any element's arithmetic: a GEMM row depends on its own
// input row only.)
int tp_projection_overlapped(b200_gpt2* m, float* out, const float* inp, const float* w, const float* bias, int M, int K, int N, int chunks) {
    using namespace b200;
    b200_ctx* ctx = m->ctx;
    const int Mc = M / chunks;
    const int all_sms = ctx->num_sms;
    for (int c = 0; c < chunks; ++c) {
        float* o = out + (size_t)c * Mc * N;
        // The GEMMs are persistent, one CTA per SM: with every SM taken, the communication kernel of
        // the previous chunk could only start as CTAs of this GEMM retire, and the GEMM's last CTAs
        // would queue behind it.  From the second chunk on the grid leaves a few SMs free instead.
        if (c > 0 && m->tp_reserve_sms > 0 && all_sms - m->tp_reserve_sms >= 32) ctx->num_sms = (all_sms - m->tp_reserve_sms) & ~1;
        int st = launch_gemm_tf32(ctx, o, inp + (size_t)c * Mc * K, w, bias, nullptr, Mc, K, N, 0, m->gemm_mode);
        ctx->num_sms = all_sms;
        if (st != B200_OK) return st;
        B200_CUDA(ctx, cudaEventRecord(m->tp_ev[c], ctx->stream));
        B200_CUDA(ctx, cudaStreamWaitEvent(m->comm_stream, m->tp_ev[c], 0));
        if (m->allreduce(m->allreduce_user, o, (size_t)Mc * N, m->comm_stream) != 0) return B200_ERR_CUDA;
    }
    B200_CUDA(ctx, cudaEventRecord(m->tp_ev[8], m->comm_stream));
    B200_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, m->tp_ev[8], 0));
    return B200_OK;
}

// how many row chunks a tensor-parallel projection is cut into (1: GEMM, then one all-reduce on the compute stream)
int tp_chunks(const b200_gpt2* m, int M, bool prof) {
    int n = m->tp_chunks;
    if (prof || !m->comm_stream) return 1;  // per-launch timing wants the all-reduce on the timed stream
    while (n > 1 && (M % (n * 256) || M / n < 1024)) --n;
    return n;
}

// results, what is prepared for the host behind the lm-head:
//   RES_ARGMAX  the lm-head GEMM also leaves, per position, the arg-max over the real vocabulary
//               in m->argmax (found in its epilogue while the logits are on their way out: no
//               second pass over the 1.6 GB of logits)
//   RES_LAST    the logits of the last position of every sequence, contiguous in m->last_logits
//   RES_STATUS  the status word, written to the pinned word the host will look at
//   RES_NO_LOGITS  (with RES_ARGMAX) nobody reads the full logits: the lm-head writes only the
//               32-row blocks that hold a sequence's last position - the arg-max is taken from
//               the accumulators, so 1.6 GB of stores per step fall away
enum : int { RES_ARGMAX = 1, RES_LAST = 2, RES_STATUS = 4, RES_NO_LOGITS = 8 };
int enqueue_forward(b200_gpt2* m, const int* tokens, int B, int T, int results) {
    const bool with_argmax = (results & RES_ARGMAX) != 0;
    using namespace b200;
    b200_ctx* ctx = m->ctx;
    const b200_gpt2_config& c = m->cfg;
    const int C = c.channels, L = c.num_layers, Vp = c.padded_vocab_size;
    const int A = m->attn_c, NH = m->nh_local, F = m->mlp_c;  // rank-local widths
    const int M = B * T;
    const float* P = m->params;
    const size_t* off = m->off;
    // GEMM modes.  bf16 modes: the operands of the GEMMs are bf16 (B200_BF16) or pairs of bf16 planes
    // (B200_BF16X3: value = hi + lo); the weights come from the bf16 copies of the parameters, and
    // layernorm, attention and the GELU GEMM write their outputs in that form into the same
    // activation buffers (two bf16 planes take exactly the room of the fp32 tensor).  Everything
    // between the GEMMs stays fp32.
    const bool hb = m->gemm_mode == B200_BF16, hx = m->gemm_mode == B200_BF16X3;
    const bool hl = m->lmhead_mode == B200_BF16, hlx = m->lmhead_mode == B200_BF16X3;
    const bool g_tf32 = !hb && !hx;
    const int rnd = (m->round_operands && m->gemm_mode == B200_TF32) ? ROUND_OUT_TF32 : 0;
    const int grnd = rnd ? GEMM_ROUND_OUT_TF32 : 0;
    // single-pass TF32 GEMMs read the rounded-to-nearest copy of the weights
    const float* W = (m->round_operands && m->params_r && m->gemm_mode == B200_TF32) ? m->params_r : P;
    const float* W_head = (m->round_operands && m->params_r && m->lmhead_mode == B200_TF32) ? m->params_r : P;
    const uint16_t* PH = m->params_h;
    const uint16_t* PL = m->params_l;
    uint16_t* ln_h = reinterpret_cast<uint16_t*>(m->ln_out);
    uint16_t* atty_h = reinterpret_cast<uint16_t*>(m->atty);
    uint16_t* fch_h = reinterpret_cast<uint16_t*>(m->fch);
    const int ln_flags = hx ? OUT_BF16X2 : (hb ? OUT_BF16 : rnd);
    // the tensor-parallel all-reduce needs the branch as a buffer of its own
    const int accum = (m->tp_size == 1) ? GEMM_ACCUM_OUT : 0;
    int st;
    const bool prof = m->profile;
    const int tpc = (m->tp_size > 1 && g_tf32 && m->gemm_mode == B200_TF32) ? tp_chunks(m, M, prof) : 1;
    // two-way tensor parallelism over peer memory instead of all-reduces (see the model's peer_* fields)
    const bool peer = m->peer_on && m->tp_size == 2 && ((g_tf32 && m->gemm_mode == B200_TF32) || hx) && tpc == 1;
    if (peer) {
        // (a tensor-parallel forward is never replayed from a graph, so the epochs below are live values)
        if (m->peer_maps_rows != M) {
            CUtensorMap host_maps[2];
            for (int i = 0; i < 2; ++i) {
                st = b200_get_tensor_map(ctx, &host_maps[i], m->peer_out[i], (uint64_t)M, (uint64_t)C, (uint64_t)C, 32, 32);
                if (st != B200_OK) return st;
            }
            B200_CUDA(ctx, cudaMemcpyAsync(m->peer_maps, host_maps, sizeof(host_maps), cudaMemcpyHostToDevice, ctx->stream));
            m->peer_maps_rows = M;
        }
    }
    unsigned int peer_e = 0;
    // the sequence-parallel hand-over (see the model's sp_* fields): rows in whole 256-row tiles per rank
    const int spn = m->tp_size;
    const bool sp = m->sp_on && spn > 1 && !peer && ((g_tf32 && m->gemm_mode == B200_TF32) || hx) && tpc == 1 && M % (spn * 256) == 0;
    if (m->sp_on && spn > 1 && !sp && !m->allreduce) { ctx->last_error = "the hand-over needs B*T to be a multiple of 256 * tp_size (or an all-reduce to fall back on)"; return B200_ERR_SHAPE; }
    const int sp_rows = sp ? M / spn : 0;
    const size_t sp_par_stride = (size_t)m->max_B * m->max_T * C;  // floats between the two parity halves of a receive buffer
    unsigned int* sp_sig1[8] = {};
    unsigned int* sp_sig2[8] = {};
    float* sp_dst[8] = {};
    if (sp) {
        for (int p = 0; p < spn; ++p) {
            sp_dst[p] = p == m->tp_rank ? m->ln_out : m->sp_ln_peer[p];
            if (p == m->tp_rank) continue;
            sp_sig1[p] = m->sp_words_peer[p] + m->tp_rank;
            sp_sig2[p] = m->sp_words_peer[p] + 16 + m->tp_rank;
        }
        if (m->sp_maps_rows != M) {
            CUtensorMap host_maps[16];
            for (int par = 0; par < 2; ++par)
                for (int o = 0; o < 8; ++o) {
                    const int oo = o < spn ? o : 0;
                    float* base = (oo == m->tp_rank ? m->sp_recv : m->sp_recv_peer[oo]) + par * sp_par_stride + (size_t)m->tp_rank * sp_rows * C;
                    st = b200_get_tensor_map(ctx, &host_maps[par * 8 + o], base, (uint64_t)sp_rows, (uint64_t)C, (uint64_t)C, 32, 32);
                    if (st != B200_OK) return st;
                }
            B200_CUDA(ctx, cudaMemcpyAsync(m->sp_maps, host_maps, sizeof(host_maps), cudaMemcpyHostToDevice, ctx->stream));
            m->sp_maps_rows = M;
        }
    }
    unsigned int sp_e = 0;
    // what follows a projection in this mode: tell the peers, wait for theirs, normalise the own rows into
    // every rank's layernorm output, tell the peers, wait for theirs
#define SP_AFTER_PROJECTION(lnw, lnb, lnflags)                                                                                          \
    do {                                                                                                                                \
        STEP(B200_PROF_ALLREDUCE, launch_peer_signal_many(ctx, sp_sig1, spn, sp_e));                                                    \
        STEP(B200_PROF_ALLREDUCE, launch_peer_wait_many(ctx, m->sp_words, spn, m->tp_rank, sp_e));                                      \
        STEP(B200_PROF_FUSED_RES_LN, launch_layernorm_sp(ctx, m->residual, m->sp_recv + (sp_e & 1) * sp_par_stride, sp_dst, spn, sp_rows, \
                                                         m->tp_rank * sp_rows, (lnw), (lnb), M, C, (lnflags)));                         \
        STEP(B200_PROF_ALLREDUCE, launch_peer_signal_many(ctx, sp_sig2, spn, sp_e));                                                    \
        STEP(B200_PROF_ALLREDUCE, launch_peer_wait_many(ctx, m->sp_words + 16, spn, m->tp_rank, sp_e));                                 \
    } while (0)
#define SP_BEFORE_PROJECTION()                                                                                  \
    do {                                                                                                        \
        if (sp) { sp_e = ++m->sp_epoch; ctx->next_gemm_out2 = m->sp_maps + (sp_e & 1) * 8; ctx->next_gemm_out2_rows = sp_rows; } \
    } while (0)
#define STEP(cat, call)                                             \
    do {                                                            \
        if (prof) { st = prof_begin(m, (cat)); if (st != B200_OK) return st; } \
        st = (call);                                                \
        if (st != B200_OK) return st;                               \
        if (prof) { st = prof_end(m); if (st != B200_OK) return st; } \
    } while (0)
    STEP(B200_PROF_ENCODER, launch_encoder(ctx, m->residual, tokens, P + off[0], P + off[1], B, T, C, Vp));
    STEP(B200_PROF_LAYERNORM, launch_layernorm(ctx, m->ln_out, nullptr, nullptr, m->residual, P + off[2], P + off[3], M, C, ln_flags));
    for (int l = 0; l < L; ++l) {
        const size_t o_qkvw = off[4] + (size_t)l * 3 * A * C, o_apw = off[6] + (size_t)l * C * A;
        const size_t o_fcw = off[10] + (size_t)l * F * C, o_fpw = off[12] + (size_t)l * C * F;
        const float* qkvb = P + off[5] + (size_t)l * 3 * A;
        const float* apb = P + off[7] + (size_t)l * C;
        const float* ln2w = P + off[8] + (size_t)l * C;
        const float* ln2b = P + off[9] + (size_t)l * C;
        const float* fcb = P + off[11] + (size_t)l * F;
        const float* fpb = P + off[13] + (size_t)l * C;
        // The single-pass attention kernel multiplies q, k and v on the TF32 pipe as they are.
        // Storing them rounded-to-nearest makes them exact TF32 values, so the tensor core's
        // truncation no longer shrinks every product (a systematic bias); what is left is
        // unbiased rounding noise that the softmax-weighted sums average down.  The 3xTF32
        // attention needs the unrounded values.
        const bool att_x3 = (g_tf32 || hx) && (m->att_mode < 0 ? m->gemm_mode == B200_TF32X3 : m->att_mode == B200_TF32X3) && m->qkv_small;
        // fp16 attention: the QKV GEMM writes q, k, v as two fp16 planes into the same buffer
        // (not while the forward also fills the fp32 key/value cache)
        const bool att_split = hx && !m->keep_kv && (m->att_mode < 0 || m->att_mode == B200_BF16X3);
        const int qkv_flags = (!att_x3 && (m->round_operands || m->gemm_mode != B200_TF32)) ? GEMM_ROUND_OUT_TF32 : 0;
        uint16_t* qkv_h = reinterpret_cast<uint16_t*>(m->qkv);
#ifdef B200_QKV_FULL_LO
        const int qkv_lo_col0 = 0;
#else
        const int qkv_lo_col0 = (2 * A) % 64 == 0 ? 2 * A : 0;  // the attention reads only v's second plane
#endif
        if (att_split) STEP(B200_PROF_GEMM_QKV, launch_gemm_bf16x3(ctx, nullptr, qkv_h, ln_h, PH + o_qkvw, PL + o_qkvw, qkvb, M, C, 3 * A, GEMM_PLANES_FP16,
                                                                    nullptr, 0, 0, nullptr, qkv_lo_col0));
        else if (hx) STEP(B200_PROF_GEMM_QKV, launch_gemm_bf16x3(ctx, m->qkv, nullptr, ln_h, PH + o_qkvw, PL + o_qkvw, qkvb, M, C, 3 * A, qkv_flags));
        else if (hb) STEP(B200_PROF_GEMM_QKV, launch_gemm_bf16(ctx, m->qkv, nullptr, ln_h, PH + o_qkvw, qkvb, M, C, 3 * A, qkv_flags));
        else STEP(B200_PROF_GEMM_QKV, launch_gemm_tf32(ctx, m->qkv, m->ln_out, W + o_qkvw, qkvb, nullptr, M, C, 3 * A, qkv_flags, m->gemm_mode));
        if (m->keep_kv) {
            const size_t per_layer = (size_t)m->max_B * m->max_T * C;
            st = launch_kv_append(ctx, m->kcache + l * per_layer, m->vcache + l * per_layer, m->qkv, B, T, C, 0, m->max_T);
            if (st != B200_OK) return st;
        }
        if (att_split) {
            STEP(B200_PROF_ATTENTION, launch_attention_split(ctx, m->atty, nullptr, qkv_h, B, T, A, NH, OUT_BF16X2));
        } else if (att_x3 && hx) {
            // the split-operand attention writes fp32: through the (free) branch buffer, then split
            STEP(B200_PROF_ATTENTION, launch_attention_x3(ctx, m->branch, m->qkv_small, nullptr, m->qkv, B, T, A, NH));
            STEP(B200_PROF_ATTENTION, launch_convert_bf16(ctx, atty_h, m->branch, (size_t)M * A, atty_h + (size_t)M * A));
        } else if (att_x3) STEP(B200_PROF_ATTENTION, launch_attention_x3(ctx, m->atty, m->qkv_small, nullptr, m->qkv, B, T, A, NH));
        else STEP(B200_PROF_ATTENTION, launch_attention(ctx, m->atty, nullptr, m->qkv, B, T, A, NH, hx ? OUT_BF16X2 : (hb ? OUT_BF16 : rnd)));
        // Without tensor parallelism the projection adds its result straight onto the residual
        // stream (its tiles leave as TMA reductions: the same single fp32 add per element that the
        // fused residual + layernorm kernel would do), and a plain layernorm follows: 50 MB less
        // traffic per block than writing the branch and reading it back.
        float* proj_out = accum ? m->residual : m->branch;
        if (hx) {
            if (peer) { peer_e = ++m->peer_epoch; ctx->next_gemm_out2 = m->peer_maps + (peer_e & 1); }
            SP_BEFORE_PROJECTION();
            STEP(B200_PROF_GEMM_ATTPROJ, launch_gemm_bf16x3(ctx, proj_out, nullptr, atty_h, PH + o_apw, PL + o_apw, apb, M, A, C, accum));
        }
        else if (hb) STEP(B200_PROF_GEMM_ATTPROJ, launch_gemm_bf16(ctx, proj_out, nullptr, atty_h, PH + o_apw, apb, M, A, C, accum));
        else if (tpc > 1) STEP(B200_PROF_GEMM_ATTPROJ, tp_projection_overlapped(m, proj_out, m->atty, W + o_apw, apb, M, A, C, tpc));
        else {
            if (peer) { peer_e = ++m->peer_epoch; ctx->next_gemm_out2 = m->peer_maps + (peer_e & 1); }
            SP_BEFORE_PROJECTION();
            STEP(B200_PROF_GEMM_ATTPROJ, launch_gemm_tf32(ctx, proj_out, m->atty, W + o_apw, apb, nullptr, M, A, C, accum, m->gemm_mode));
        }
        if (accum) {
            STEP(B200_PROF_LAYERNORM, launch_layernorm(ctx, m->ln_out, nullptr, nullptr, m->residual, ln2w, ln2b, M, C, ln_flags));
        } else {
            // tensor parallel: every rank holds a partial sum over its heads; one all-reduce per block
            // (already issued, chunk by chunk, when the projection ran overlapped)
            if (sp) {
                SP_AFTER_PROJECTION(ln2w, ln2b, ln_flags);
            } else {
                if (peer) {
                    STEP(B200_PROF_ALLREDUCE, launch_peer_signal(ctx, m->peer_word_remote, peer_e));
                    STEP(B200_PROF_ALLREDUCE, launch_peer_wait(ctx, m->peer_word, peer_e));
                } else if (m->tp_size > 1 && tpc == 1) STEP(B200_PROF_ALLREDUCE, tp_allreduce(m, m->branch, (size_t)M * C));
                STEP(B200_PROF_FUSED_RES_LN, launch_fused_residual_layernorm(ctx, m->residual, m->ln_out, nullptr, nullptr, m->residual,
                                                     m->branch, ln2w, ln2b, M, C, ln_flags, peer ? m->peer_in[peer_e & 1] : nullptr));
            }
        }
        if (hx) {
            STEP(B200_PROF_GEMM_FC, launch_gemm_bf16x3(ctx, nullptr, fch_h, ln_h, PH + o_fcw, PL + o_fcw, fcb, M, C, F, GEMM_GELU));
            if (peer) { peer_e = ++m->peer_epoch; ctx->next_gemm_out2 = m->peer_maps + (peer_e & 1); }
            SP_BEFORE_PROJECTION();
            STEP(B200_PROF_GEMM_FCPROJ, launch_gemm_bf16x3(ctx, proj_out, nullptr, fch_h, PH + o_fpw, PL + o_fpw, fpb, M, F, C, accum));
        } else if (hb) {
            STEP(B200_PROF_GEMM_FC, launch_gemm_bf16(ctx, nullptr, fch_h, ln_h, PH + o_fcw, fcb, M, C, F, GEMM_GELU));
            STEP(B200_PROF_GEMM_FCPROJ, launch_gemm_bf16(ctx, proj_out, nullptr, fch_h, PH + o_fpw, fpb, M, F, C, accum));
        } else {
            STEP(B200_PROF_GEMM_FC, launch_gemm_tf32(ctx, m->fch, m->ln_out, W + o_fcw, fcb, nullptr, M, C, F, GEMM_GELU | grnd, m->gemm_mode));
            if (tpc > 1) STEP(B200_PROF_GEMM_FCPROJ, tp_projection_overlapped(m, proj_out, m->fch, W + o_fpw, fpb, M, F, C, tpc));
            else {
                if (peer) { peer_e = ++m->peer_epoch; ctx->next_gemm_out2 = m->peer_maps + (peer_e & 1); }
                SP_BEFORE_PROJECTION();
                STEP(B200_PROF_GEMM_FCPROJ, launch_gemm_tf32(ctx, proj_out, m->fch, W + o_fpw, fpb, nullptr, M, F, C, accum, m->gemm_mode));
            }
        }
        const float* nw = (l + 1 < L) ? P + off[2] + (size_t)(l + 1) * C : P + off[14];
        const float* nb = (l + 1 < L) ? P + off[3] + (size_t)(l + 1) * C : P + off[15];
        const int head_flags = hlx ? OUT_BF16X2 : (hl ? OUT_BF16 : ((m->round_operands && m->lmhead_mode == B200_TF32) ? ROUND_OUT_TF32 : 0));
        const int next_flags = (l + 1 < L) ? ln_flags : head_flags;
        if (accum) {
            STEP(B200_PROF_LAYERNORM, launch_layernorm(ctx, m->ln_out, nullptr, nullptr, m->residual, nw, nb, M, C, next_flags));
        } else {
            if (sp) {
                SP_AFTER_PROJECTION(nw, nb, next_flags);
            } else {
                if (peer) {
                    STEP(B200_PROF_ALLREDUCE, launch_peer_signal(ctx, m->peer_word_remote, peer_e));
                    STEP(B200_PROF_ALLREDUCE, launch_peer_wait(ctx, m->peer_word, peer_e));
                } else if (m->tp_size > 1 && tpc == 1) STEP(B200_PROF_ALLREDUCE, tp_allreduce(m, m->branch, (size_t)M * C));
                STEP(B200_PROF_FUSED_RES_LN, launch_fused_residual_layernorm(ctx, m->residual, m->ln_out, nullptr, nullptr, m->residual,
                                                     m->branch, nw, nb, M, C, next_flags, peer ? m->peer_in[peer_e & 1] : nullptr));
            }
        }
    }
    const size_t o_head = off[0] + (size_t)m->vp_row0 * C;
    const int store_period = (with_argmax && (results & RES_NO_LOGITS)) ? T : 0;
    unsigned long long* keys = with_argmax ? m->argmax_keys : nullptr;
    if (m->row_stats && !hlx && m->lmhead_mode != B200_TF32) { ctx->last_error = "sampling in the lm-head: lmhead_mode B200_BF16X3 or B200_TF32"; return B200_ERR_STATE; }
    if (hlx) STEP(B200_PROF_GEMM_LMHEAD, launch_gemm_bf16x3(ctx, m->logits, nullptr, ln_h, PH + o_head, PL + o_head, nullptr, M, C, m->vp_local, 0,
                                                          keys, c.vocab_size, store_period, m->row_stats));
    else if (hl) STEP(B200_PROF_GEMM_LMHEAD, launch_gemm_bf16(ctx, m->logits, nullptr, ln_h, PH + o_head, nullptr, M, C, m->vp_local, 0,
                                                              keys, c.vocab_size, store_period));
    else STEP(B200_PROF_GEMM_LMHEAD, launch_gemm_tf32(ctx, m->logits, m->ln_out, W_head + o_head, nullptr, nullptr, M, C,
                                                      m->vp_local, 0, m->lmhead_mode, keys, c.vocab_size, store_period, m->row_stats));
    if (results) {
        st = launch_host_results(ctx, m->host_dst.ids ? m->host_dst.ids : m->argmax, with_argmax ? m->argmax_keys : nullptr, M,
                                 (results & RES_LAST) ? (m->host_dst.last ? m->host_dst.last : m->last_logits) : nullptr,
                                 m->logits, B, T, m->vp_local, (results & RES_STATUS) ? m->host_dst.status : nullptr);
        if (st != B200_OK) return st;
    }
#undef STEP
#undef SP_AFTER_PROJECTION
#undef SP_BEFORE_PROJECTION
    return B200_OK;
}

// bf16 copies of the weight matrices (and of wte for the lm-head), made from the parameters as
// they are at the first forward of a bf16 mode; with_lo: also the plane of what the rounding dropped
int bf16_weights_once(b200_gpt2* m, bool with_lo) {
    using namespace b200;
    if (m->params_h_ready && (!with_lo || m->params_l_ready)) return B200_OK;
    b200_ctx* ctx = m->ctx;
    if (!m->params_h) B200_CUDA(ctx, cudaMalloc(&m->params_h, m->n_params * sizeof(uint16_t)));
    if (with_lo && !m->params_l) B200_CUDA(ctx, cudaMalloc(&m->params_l, m->n_params * sizeof(uint16_t)));
    const int idx[5] = {0, 4, 6, 10, 12};  // wte, qkvw, attprojw, fcw, fcprojw
    for (int i = 0; i < 5; ++i) {
        int st = launch_convert_bf16(ctx, m->params_h + m->off[idx[i]], m->params + m->off[idx[i]], m->off[idx[i] + 1] - m->off[idx[i]],
                                     with_lo ? m->params_l + m->off[idx[i]] : nullptr);
        if (st != B200_OK) return st;
    }
    m->params_h_ready = true;
    if (with_lo) m->params_l_ready = true;
    return B200_OK;
}

// TF32-rounded (to nearest) copy of the weight matrices for the single-pass TF32 GEMMs; the
// parameters themselves are never modified (the encoder, the decode step and the other modes
// read them as loaded)
int round_weights_once(b200_gpt2* m) {
    using namespace b200;
    if (m->weights_rounded) return B200_OK;
    b200_ctx* ctx = m->ctx;
    const size_t* off = m->off;
    if (!m->params_r) B200_CUDA(ctx, cudaMalloc(&m->params_r, m->n_params * sizeof(float)));
    const int idx[5] = {0, 4, 6, 10, 12};  // wte (lm-head), qkvw, attprojw, fcw, fcprojw
    for (int i = 0; i < 5; ++i) {
        const size_t n = off[idx[i] + 1] - off[idx[i]];
        B200_CUDA(ctx, cudaMemcpyAsync(m->params_r + off[idx[i]], m->params + off[idx[i]], n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        int st = launch_round_tf32_inplace(ctx, m->params_r + off[idx[i]], n);
        if (st != B200_OK) return st;
    }
    m->weights_rounded = true;
    return B200_OK;
}

// what a forward needs done to the weights for the current modes
int prepare_weights(b200_gpt2* m) {
    const bool x3 = m->gemm_mode == B200_BF16X3 || m->lmhead_mode == B200_BF16X3;
    if (x3 || m->gemm_mode == B200_BF16 || m->lmhead_mode == B200_BF16) {
        int st = bf16_weights_once(m, x3);
        if (st != B200_OK) return st;
    }
    if (m->round_operands && (m->gemm_mode == B200_TF32 || m->lmhead_mode == B200_TF32)) return round_weights_once(m);
    return B200_OK;
}

}  // namespace

extern "C" {

size_t b200_gpt2_param_offsets(const b200_gpt2_config* cfg, size_t* offsets) {
    const size_t C = cfg->channels, L = cfg->num_layers, Vp = cfg->padded_vocab_size, mT = cfg->max_seq_len;
    const size_t sizes[16] = {Vp * C, mT * C, L * C, L * C, L * 3 * C * C, L * 3 * C, L * C * C, L * C,
                              L * C, L * C, L * 4 * C * C, L * 4 * C, L * C * 4 * C, L * C, C, C};
    size_t o = 0;
    for (int i = 0; i < 16; ++i) { if (offsets) offsets[i] = o; o += sizes[i]; }
    if (offsets) offsets[16] = o;
    return o;
}

size_t b200_gpt2_param_offsets_tp(const b200_gpt2_config* cfg, int tp_size, int tp_rank, size_t* offsets) {
    if (!cfg || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size || tp_size > cfg->num_heads || (4 * cfg->channels) % tp_size)
        return 0;
    return local_param_offsets(cfg, tp_heads(cfg->num_heads, tp_size, tp_rank) * 64, 4 * cfg->channels / tp_size, offsets);
}

int b200_gpt2_shard_params_host(const b200_gpt2_config* cfg, int tp_size, int tp_rank, const float* full, float* local) {
    if (!cfg || !full || !local) return B200_ERR_NULL;
    size_t fo[17], lo[17];
    b200_gpt2_param_offsets(cfg, fo);
    if (b200_gpt2_param_offsets_tp(cfg, tp_size, tp_rank, lo) == 0) return B200_ERR_SHAPE;
    const size_t C = cfg->channels, L = cfg->num_layers;
    const size_t A = (size_t)tp_heads(cfg->num_heads, tp_size, tp_rank) * 64, a0 = (size_t)tp_head0(cfg->num_heads, tp_size, tp_rank) * 64;
    const size_t F = 4 * C / tp_size, f0 = (size_t)tp_rank * F;
    const int same[] = {0, 1, 2, 3, 8, 9, 14, 15};  // wte, wpe and the layernorm tensors are replicated
    for (int t : same) memcpy(local + lo[t], full + fo[t], (fo[t + 1] - fo[t]) * sizeof(float));
    for (size_t l = 0; l < L; ++l) {
        for (size_t part = 0; part < 3; ++part) {  // q, k, v rows of the local heads
            memcpy(local + lo[4] + (l * 3 * A + part * A) * C, full + fo[4] + (l * 3 * C + part * C + a0) * C, A * C * sizeof(float));
            memcpy(local + lo[5] + l * 3 * A + part * A, full + fo[5] + l * 3 * C + part * C + a0, A * sizeof(float));
        }
        for (size_t o = 0; o < C; ++o) {  // input columns of the two projections
            memcpy(local + lo[6] + (l * C + o) * A, full + fo[6] + (l * C + o) * C + a0, A * sizeof(float));
            memcpy(local + lo[12] + (l * C + o) * F, full + fo[12] + (l * C + o) * 4 * C + f0, F * sizeof(float));
        }
        memcpy(local + lo[10] + l * F * C, full + fo[10] + (l * 4 * C + f0) * C, F * C * sizeof(float));
        memcpy(local + lo[11] + l * F, full + fo[11] + l * 4 * C + f0, F * sizeof(float));
        // the projection biases are added once: by rank 0
        for (int t : {7, 13}) {
            if (tp_rank == 0) memcpy(local + lo[t] + l * C, full + fo[t] + l * C, C * sizeof(float));
            else memset(local + lo[t] + l * C, 0, C * sizeof(float));
        }
    }
    return B200_OK;
}

int b200_gpt2_create(b200_gpt2** out, b200_ctx* ctx, const b200_gpt2_config* cfg, int max_B, int max_T) {
    return b200_gpt2_create_tp(out, ctx, cfg, max_B, max_T, 1, 0);
}

int b200_gpt2_set_tp_overlap(b200_gpt2* m, int chunks, int reserve_sms) {
    if (!m) return B200_ERR_NULL;
    if (chunks < 1 || chunks > 8 || reserve_sms < 0 || reserve_sms > 64) return B200_ERR_SHAPE;
    m->tp_chunks = chunks;
    m->tp_reserve_sms = reserve_sms;
    return B200_OK;
}

// ---- two-way tensor parallelism over peer memory -------------------------------------------------
int b200_gpt2_tp_peer_export(b200_gpt2* m, unsigned char* handles) {
    if (!m || !handles) return B200_ERR_NULL;
    if (m->tp_size != 2) { m->ctx->last_error = "peer hand-over is for a tensor-parallel group of two"; return B200_ERR_STATE; }
    b200_ctx* ctx = m->ctx;
    b200_device_guard guard(ctx);
    const size_t bytes = (size_t)m->max_B * m->max_T * m->cfg.channels * sizeof(float);
    for (int i = 0; i < 2; ++i)
        if (!m->peer_in[i]) B200_CUDA(ctx, cudaMalloc(&m->peer_in[i], bytes));
    if (!m->peer_word) {
        B200_CUDA(ctx, cudaMalloc(&m->peer_word, 256));
        B200_CUDA(ctx, cudaMemset(m->peer_word, 0, 256));
    }
    if (!m->peer_maps) B200_CUDA(ctx, cudaMalloc(&m->peer_maps, 2 * sizeof(CUtensorMap)));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->peer_in[0])); memcpy(handles, &h, 64);
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->peer_in[1])); memcpy(handles + 64, &h, 64);
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->peer_word)); memcpy(handles + 128, &h, 64);
    return B200_OK;
}

int b200_gpt2_tp_peer_connect(b200_gpt2* m, const unsigned char* peer_handles) {
    if (!m || !peer_handles) return B200_ERR_NULL;
    if (m->tp_size != 2 || !m->peer_word) { m->ctx->last_error = "b200_gpt2_tp_peer_export comes first"; return B200_ERR_STATE; }
    if (m->peer_word_remote) { m->ctx->last_error = "the model is connected to its peer already"; return B200_ERR_STATE; }
    b200_ctx* ctx = m->ctx;
    b200_device_guard guard(ctx);
    cudaIpcMemHandle_t h;
    void* q = nullptr;
    for (int i = 0; i < 2; ++i) {
        memcpy(&h, peer_handles + 64 * i, 64);
        B200_CUDA(ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
        m->peer_out[i] = static_cast<float*>(q);
    }
    memcpy(&h, peer_handles + 128, 64);
    B200_CUDA(ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
    m->peer_word_remote = static_cast<unsigned int*>(q);
    m->peer_maps_rows = 0;
    m->peer_epoch = 0;
    m->peer_on = true;
    return B200_OK;
}

int b200_gpt2_tp_peer_enable(b200_gpt2* m, int on) {
    if (!m) return B200_ERR_NULL;
    if (on && !m->peer_word_remote) { m->ctx->last_error = "not connected to a peer"; return B200_ERR_STATE; }
    m->peer_on = on != 0;
    return B200_OK;
}

// ---- sequence-parallel hand-over for a tensor-parallel group of 2..8 ranks ---------------------------
int b200_gpt2_tp_sp_export(b200_gpt2* m, unsigned char* handles) {
    if (!m || !handles) return B200_ERR_NULL;
    if (m->tp_size < 2 || m->tp_size > 8) { m->ctx->last_error = "the hand-over is for tensor-parallel groups of 2 to 8"; return B200_ERR_STATE; }
    b200_ctx* ctx = m->ctx;
    b200_device_guard guard(ctx);
    const size_t bytes = (size_t)2 * m->max_B * m->max_T * m->cfg.channels * sizeof(float);
    if (!m->sp_recv) B200_CUDA(ctx, cudaMalloc(&m->sp_recv, bytes));
    if (!m->sp_words) {
        B200_CUDA(ctx, cudaMalloc(&m->sp_words, 256));
        B200_CUDA(ctx, cudaMemset(m->sp_words, 0, 256));
    }
    if (!m->sp_maps) B200_CUDA(ctx, cudaMalloc(&m->sp_maps, 16 * sizeof(CUtensorMap)));
    cudaIpcMemHandle_t h;
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->sp_recv)); memcpy(handles, &h, 64);
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->ln_out)); memcpy(handles + 64, &h, 64);
    B200_CUDA(ctx, cudaIpcGetMemHandle(&h, m->sp_words)); memcpy(handles + 128, &h, 64);
    return B200_OK;
}

int b200_gpt2_tp_sp_connect(b200_gpt2* m, const unsigned char* all_handles) {
    if (!m || !all_handles) return B200_ERR_NULL;
    if (m->tp_size < 2 || m->tp_size > 8 || !m->sp_words) { m->ctx->last_error = "b200_gpt2_tp_sp_export comes first"; return B200_ERR_STATE; }
    for (int p = 0; p < 8; ++p)
        if (m->sp_words_peer[p]) { m->ctx->last_error = "the model is connected to its peers already"; return B200_ERR_STATE; }
    b200_ctx* ctx = m->ctx;
    b200_device_guard guard(ctx);
    for (int p = 0; p < m->tp_size; ++p) {
        if (p == m->tp_rank) continue;
        cudaIpcMemHandle_t h;
        void* q = nullptr;
        memcpy(&h, all_handles + 192 * p, 64);
        B200_CUDA(ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
        m->sp_recv_peer[p] = static_cast<float*>(q);
        memcpy(&h, all_handles + 192 * p + 64, 64);
        B200_CUDA(ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
        m->sp_ln_peer[p] = static_cast<float*>(q);
        memcpy(&h, all_handles + 192 * p + 128, 64);
        B200_CUDA(ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
        m->sp_words_peer[p] = static_cast<unsigned int*>(q);
    }
    m->sp_maps_rows = 0;
    m->sp_epoch = 0;
    m->sp_on = true;
    m->peer_on = false;
    return B200_OK;
}

int b200_gpt2_tp_sp_enable(b200_gpt2* m, int on) {
    if (!m) return B200_ERR_NULL;
    bool connected = false;
    for (int p = 0; p < 8; ++p) connected = connected || m->sp_words_peer[p] != nullptr;
    if (on && !connected) { m->ctx->last_error = "not connected to the peers"; return B200_ERR_STATE; }
    m->sp_on = on != 0;
    return B200_OK;
}

int b200_gpt2_set_allreduce(b200_gpt2* m, b200_allreduce_fn fn, void* user) {
    if (!m) return B200_ERR_NULL;
    m->allreduce = fn;
    m->allreduce_user = user;
    return B200_OK;
}

int b200_gpt2_create_tp(b200_gpt2** out, b200_ctx* ctx, const b200_gpt2_config* cfg, int max_B, int max_T,
                        int tp_size, int tp_rank) {
    if (!out || !ctx || !cfg) return B200_ERR_NULL;
    *out = nullptr;
    if (cfg->channels <= 0 || cfg->num_heads <= 0 || cfg->channels % cfg->num_heads ||
        cfg->channels / cfg->num_heads != 64 || cfg->channels % 4 || cfg->channels > 4096 ||
        cfg->num_layers <= 0 || cfg->padded_vocab_size % 4 || cfg->vocab_size > cfg->padded_vocab_size ||
        cfg->vocab_size <= 0 || max_B <= 0 || max_T <= 0 || max_T > cfg->max_seq_len || max_T % 64)
        return B200_ERR_SHAPE;
    b200_gpt2* m = new (std::nothrow) b200_gpt2();
    if (!m) return B200_ERR_CUDA;
    m->ctx = ctx; m->cfg = *cfg; m->max_B = max_B; m->max_T = max_T;
    if (!set_tp_dims(m, tp_size, tp_rank)) { delete m; return B200_ERR_SHAPE; }
    const size_t M = (size_t)max_B * max_T, C = cfg->channels, Vp = m->vp_local;
    const size_t A = m->attn_c, F = m->mlp_c;
    cudaError_t e = cudaSetDevice(ctx->device);
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes); };
    alloc((void**)&m->params, m->n_params * 4);
    alloc((void**)&m->residual, M * C * 4);
    alloc((void**)&m->ln_out, M * C * 4);
    alloc((void**)&m->qkv, M * 3 * A * 4);
    alloc((void**)&m->atty, M * A * 4);
    alloc((void**)&m->branch, M * C * 4);
    alloc((void**)&m->fch, M * F * 4);
    alloc((void**)&m->logits, M * Vp * 4);
    alloc((void**)&m->tokens, M * 4);
    alloc((void**)&m->argmax, M * 4);
    alloc((void**)&m->argmax_keys, M * 8);
    alloc((void**)&m->last_logits, (M / 64 + 1) * Vp * 4);
    if (e == cudaSuccess) e = cudaMemset(m->argmax_keys, 0, M * 8);
    if (tp_size > 1) {
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking);
        for (int i = 0; i < 9 && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&m->tp_ev[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        b200_fail_cuda(ctx, e, "cudaMalloc (b200_gpt2_create)");
        b200_gpt2_destroy(m);
        return B200_ERR_CUDA;
    }
    *out = m;
    return B200_OK;
}

int b200_gpt2_destroy(b200_gpt2* m) {
    if (!m) return B200_ERR_NULL;
    cudaSetDevice(m->ctx->device);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    for (auto& g : m->decode_graphs) cudaGraphExecDestroy(g.second);
    if (m->pos_dev) cudaFree(m->pos_dev);
    if (m->resid2) cudaFree(m->resid2);
    if (m->att_partial) cudaFree(m->att_partial);
    if (m->att_counters) cudaFree(m->att_counters);
    if (m->gen_tokens) cudaFree(m->gen_tokens);
    for (cudaEvent_t e : m->host_done) if (e) cudaEventDestroy(e);
    if (m->h_slot_status) cudaFreeHost(m->h_slot_status);
    for (cudaEvent_t e : m->ev_pool) cudaEventDestroy(e);
    for (cudaEvent_t e : m->tp_ev) if (e) cudaEventDestroy(e);
    if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
    for (float* q : m->peer_out) if (q) cudaIpcCloseMemHandle(q);
    for (int i = 0; i < 8; ++i) {
        if (m->sp_recv_peer[i]) cudaIpcCloseMemHandle(m->sp_recv_peer[i]);
        if (m->sp_ln_peer[i]) cudaIpcCloseMemHandle(m->sp_ln_peer[i]);
        if (m->sp_words_peer[i]) cudaIpcCloseMemHandle(m->sp_words_peer[i]);
    }
    if (m->sp_recv) cudaFree(m->sp_recv);
    if (m->sp_words) cudaFree(m->sp_words);
    if (m->sp_maps) cudaFree(m->sp_maps);
    if (m->peer_word_remote) cudaIpcCloseMemHandle(m->peer_word_remote);
    for (float* q : m->peer_in) if (q) cudaFree(q);
    if (m->peer_word) cudaFree(m->peer_word);
    if (m->peer_maps) cudaFree(m->peer_maps);
    void* ptrs[] = {m->params, m->params_h, m->params_l, m->params_r, m->qkv_small, m->residual, m->ln_out, m->qkv, m->atty, m->branch,
                    m->fch, m->logits, m->tokens, m->argmax, m->argmax_keys, m->last_logits, m->kcache, m->vcache, m->lse_part};
    for (void* p : ptrs) if (p) cudaFree(p);
    delete m;
    return B200_OK;
}

float* b200_gpt2_params(b200_gpt2* m) { return m ? m->params : nullptr; }
float* b200_gpt2_logits(b200_gpt2* m) { return m ? m->logits : nullptr; }

int b200_gpt2_load_params_host(b200_gpt2* m, const float* host_params, size_t count) {
    if (!m || !host_params) return B200_ERR_NULL;
    if (count != m->n_params) return B200_ERR_SHAPE;
    B200_CUDA(m->ctx, cudaMemcpyAsync(m->params, host_params, count * 4, cudaMemcpyHostToDevice, m->ctx->stream));
    B200_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
    m->weights_rounded = false;
    m->params_h_ready = m->params_l_ready = false;
    return B200_OK;
}

int b200_gpt2_load_params_file(b200_gpt2* m, const char* path, size_t header_bytes) {
    if (!m || !path) return B200_ERR_NULL;
    if (m->tp_size > 1) return B200_ERR_STATE;
    b200_ctx* ctx = m->ctx;
    FILE* f = fopen(path, "rb");
    if (!f) { ctx->last_error = std::string("cannot open ") + path; return B200_ERR_STATE; }
    int st = B200_OK;
    const unsigned long long want = (unsigned long long)header_bytes + (unsigned long long)m->n_params * 4ull;
    if (fseek(f, 0, SEEK_END) != 0 || (unsigned long long)ftell(f) != want) {
        ctx->last_error = std::string(path) + ": size is not header_bytes + 4 * parameter count";
        st = B200_ERR_SHAPE;
    } else if (fseek(f, (long)header_bytes, SEEK_SET) != 0) {
        ctx->last_error = std::string("cannot seek in ") + path;
        st = B200_ERR_STATE;
    }
    // two pinned staging buffers: the disk read of one piece overlaps the copy of the previous one
    constexpr size_t kPiece = (size_t)32 << 20;
    void* stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaSetDevice(ctx->device);
    for (int i = 0; i < 2 && st == B200_OK; ++i) {
        cudaError_t e = cudaMallocHost(&stage[i], kPiece);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming);
        if (e != cudaSuccess) st = b200_fail_cuda(ctx, e, "pinned staging buffers");
    }
    const size_t total = m->n_params * sizeof(float);
    size_t off_bytes = 0;
    for (int i = 0; st == B200_OK && off_bytes < total; i ^= 1) {
        const size_t n = total - off_bytes < kPiece ? total - off_bytes : kPiece;
        cudaError_t e = cudaEventSynchronize(done[i]);  // the copy that last used this buffer is done
        if (e != cudaSuccess) { st = b200_fail_cuda(ctx, e, "cudaEventSynchronize"); break; }
        if (fread(stage[i], 1, n, f) != n) { ctx->last_error = std::string("short read from ") + path; st = B200_ERR_STATE; break; }
        e = cudaMemcpyAsync(reinterpret_cast<char*>(m->params) + off_bytes, stage[i], n, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaEventRecord(done[i], ctx->stream);
        if (e != cudaSuccess) { st = b200_fail_cuda(ctx, e, "cudaMemcpyAsync (parameters)"); break; }
        off_bytes += n;
    }
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 2; ++i) {
        if (done[i]) cudaEventDestroy(done[i]);
        if (stage[i]) cudaFreeHost(stage[i]);
    }
    fclose(f);
    m->weights_rounded = false;
    m->params_h_ready = m->params_l_ready = false;
    return st;
}

int b200_gpt2_set_options(b200_gpt2* m, int round_operands, int gemm_mode, int lmhead_mode, int use_graph) {
    if (!m) return B200_ERR_NULL;
    if (gemm_mode < B200_TF32 || gemm_mode > B200_BF16X3 || lmhead_mode < B200_TF32 || lmhead_mode > B200_BF16X3) return B200_ERR_SHAPE;
    // tensor-parallel models: single-pass TF32 or the split-bf16 arithmetic (the plain bf16 mode is not wired for them)
    if ((gemm_mode == B200_BF16 || lmhead_mode == B200_BF16) && m->tp_size > 1) return B200_ERR_STATE;
    if (m->round_operands != round_operands || m->gemm_mode != gemm_mode || m->lmhead_mode != lmhead_mode) {
        for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
        m->graphs.clear();
    }
    if ((m->att_mode < 0 ? gemm_mode == B200_TF32X3 : m->att_mode == B200_TF32X3) && !m->qkv_small) {
        cudaSetDevice(m->ctx->device);
        B200_CUDA(m->ctx, cudaMalloc(&m->qkv_small, (size_t)m->max_B * m->max_T * 3 * m->attn_c * sizeof(float)));
    }
    m->round_operands = round_operands;
    m->gemm_mode = gemm_mode;
    m->lmhead_mode = lmhead_mode;
    m->use_graph = use_graph;
    return B200_OK;
}

int b200_gpt2_set_attention_mode(b200_gpt2* m, int mode) {
    if (!m) return B200_ERR_NULL;
    if (mode != -1 && mode != B200_TF32 && mode != B200_TF32X3 && mode != B200_BF16X3) return B200_ERR_SHAPE;
    if (mode != m->att_mode) {
        for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
        m->graphs.clear();
    }
    m->att_mode = mode;
    if ((mode < 0 ? m->gemm_mode == B200_TF32X3 : mode == B200_TF32X3) && !m->qkv_small) {
        cudaSetDevice(m->ctx->device);
        B200_CUDA(m->ctx, cudaMalloc(&m->qkv_small, (size_t)m->max_B * m->max_T * 3 * m->attn_c * sizeof(float)));
    }
    return B200_OK;
}

static int forward_impl(b200_gpt2* m, const int* tokens, int B, int T, int results) {
    if (!m || !tokens) return B200_ERR_NULL;
    if (B <= 0 || T <= 0 || T % 64 || T > m->max_T) return B200_ERR_SHAPE;
    if ((size_t)B * T > (size_t)m->max_B * m->max_T) return B200_ERR_LIMIT;
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    {
        int st = prepare_weights(m);
        if (st != B200_OK) return st;
    }
    if (m->tp_size > 1 && !m->allreduce && !m->peer_on && !m->sp_on) return B200_ERR_STATE;  // some way to sum over the group
    if (!m->use_graph || ctx->stream == nullptr || m->profile || m->tp_size > 1) return enqueue_forward(m, tokens, B, T, results);

    // CUDA-graph replay: the graph reads token ids from the model's own token buffer
    if (tokens != m->tokens)
        B200_CUDA(ctx, cudaMemcpyAsync(m->tokens, tokens, (size_t)B * T * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    auto key = std::make_pair(std::make_pair(B, T), results);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        // warm the tensor-map cache and function attributes outside of capture
        int st = enqueue_forward(m, m->tokens, B, T, results);
        if (st != B200_OK) return st;
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaGraph_t graph = nullptr;
        const uint64_t launches_before = ctx->launches;
        B200_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        st = enqueue_forward(m, m->tokens, B, T, results);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        ctx->launches = launches_before;
        if (st != B200_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (e != cudaSuccess) return b200_fail_cuda(ctx, e, "cudaStreamEndCapture");
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return b200_fail_cuda(ctx, e, "cudaGraphInstantiate");
        it = m->graphs.emplace(key, exec).first;
    }
    B200_CUDA(ctx, cudaGraphLaunch(it->second, ctx->stream));
    // kernels inside the replayed graph: encoder, first layernorm, 7 per layer (8 with the
    // 3xTF32 attention's split pass), lm-head
    ctx->launches += 2 + (m->gemm_mode == B200_TF32X3 ? 8ull : 7ull) * m->cfg.num_layers + 1 + (results ? 1 : 0);
    return B200_OK;
}

int b200_gpt2_forward(b200_gpt2* m, const int* tokens, int B, int T) { return forward_impl(m, tokens, B, T, 0); }

int b200_gpt2_forward_sample(b200_gpt2* m, const int* tokens, int B, int T, float temperature, unsigned int seed,
                             int* ids_out, float* lse_out, int store_logits) {
    if (!m || !tokens || !ids_out) return B200_ERR_NULL;
    if (B <= 0 || T <= 0 || T % 64 || T > m->max_T) return B200_ERR_SHAPE;
    if ((size_t)B * T > (size_t)m->max_B * m->max_T) return B200_ERR_LIMIT;
    if (m->tp_size > 1) return B200_ERR_STATE;  // a rank sees only its slice of the vocabulary
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    const int slots = 2 * ((m->cfg.padded_vocab_size + 255) / 256);
    if (lse_out && !m->lse_part)
        B200_CUDA(ctx, cudaMalloc(&m->lse_part, (size_t)m->max_B * m->max_T * slots * sizeof(float2)));
    int st = prepare_weights(m);
    if (st != B200_OK) return st;
    b200::GemmRowStats rs;
    rs.inv_temp = temperature > 0.f ? 1.0f / temperature : 0.f;  // <= 0: greedy
    rs.seed = seed;
    rs.stream0 = 0u;
    rs.lse_part = lse_out ? m->lse_part : nullptr;
    rs.lse_slots = slots;
    m->row_stats = &rs;
    m->host_dst.ids = ids_out;
    st = enqueue_forward(m, tokens, B, T, RES_ARGMAX | (store_logits ? 0 : RES_NO_LOGITS));
    m->row_stats = nullptr;
    m->host_dst = {};
    if (st != B200_OK) return st;
    if (lse_out) return b200::launch_lse_reduce(ctx, lse_out, m->lse_part, B * T, slots);
    return B200_OK;
}

// Device address of a pinned (page-locked, mapped) host buffer, or null for any other memory.
static void* device_view(const void* p) {
    if (!p) return nullptr;
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return (a.type == cudaMemoryTypeHost) ? a.devicePointer : nullptr;
}

int b200_gpt2_forward_host_enqueue(b200_gpt2* m, const int* tokens_host, int B, int T, float* logits_host,
                                   float* last_logits_host, int* argmax_host, int slot) {
    if (!m || !tokens_host) return B200_ERR_NULL;
    if (slot < 0 || slot > 1) return B200_ERR_SHAPE;
    if (B <= 0 || T <= 0 || T % 64 || T > m->max_T) return B200_ERR_SHAPE;
    if ((size_t)B * T > (size_t)m->max_B * m->max_T) return B200_ERR_LIMIT;
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    const size_t M = (size_t)B * T, Vp = m->vp_local;  // a tensor-parallel rank returns its slice of the vocabulary
    if (argmax_host && m->vp_local != m->cfg.padded_vocab_size) return B200_ERR_STATE;  // needs all logits
    if (!m->h_slot_status) {
        B200_CUDA(ctx, cudaSetDevice(ctx->device));
        B200_CUDA(ctx, cudaHostAlloc(&m->h_slot_status, 2 * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
        m->h_slot_status[0] = m->h_slot_status[1] = 0;
        B200_CUDA(ctx, cudaHostGetDevicePointer(&m->d_slot_status, m->h_slot_status, 0));
        for (int i = 0; i < 2; ++i) B200_CUDA(ctx, cudaEventCreateWithFlags(&m->host_done[i], cudaEventDisableTiming));
    }
    // Buffers in pinned host memory are read and written by kernels (one in front of the encoder
    // fetches the token ids, the one behind the lm-head writes ids, last-position logits and the
    // status word): no copy is queued in front of or behind the forward, each of which would
    // cost a drained GPU and tens of microseconds.  Pageable buffers, and everything when the
    // forward is replayed as a graph (whose kernel arguments are fixed), go through copies.
    const bool replay = m->use_graph && ctx->stream != nullptr && !m->profile && m->tp_size == 1;
    const int* tok_view = (replay || !b200_aligned16(tokens_host)) ? nullptr : static_cast<const int*>(device_view(tokens_host));
    int* ids_view = replay ? nullptr : static_cast<int*>(device_view(argmax_host));
    float* last_view = (replay || !b200_aligned16(last_logits_host)) ? nullptr : static_cast<float*>(device_view(last_logits_host));
    int* status_view = replay ? nullptr : m->d_slot_status + slot;
    if (tok_view) {
        const int fs = b200::launch_fetch_ints(ctx, m->tokens, tok_view, (int)M);
        if (fs != B200_OK) return fs;
    } else {
        B200_CUDA(ctx, cudaMemcpyAsync(m->tokens, tokens_host, M * 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    m->host_dst.ids = ids_view;
    m->host_dst.last = last_view;
    m->host_dst.status = status_view;
    int st = forward_impl(m, m->tokens, B, T,
                          (argmax_host ? RES_ARGMAX : 0) | (last_logits_host ? RES_LAST : 0) | (status_view ? RES_STATUS : 0) |
                              ((argmax_host && !logits_host) ? RES_NO_LOGITS : 0));
    m->host_dst = {};
    if (st != B200_OK) return st;
    if (argmax_host && !ids_view) B200_CUDA(ctx, cudaMemcpyAsync(argmax_host, m->argmax, M * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (last_logits_host && !last_view)  // gathered behind the lm-head: one plain copy
        B200_CUDA(ctx, cudaMemcpyAsync(last_logits_host, m->last_logits, (size_t)B * Vp * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (logits_host)
        B200_CUDA(ctx, cudaMemcpyAsync(logits_host, m->logits, M * Vp * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (!status_view)
        B200_CUDA(ctx, cudaMemcpyAsync(m->h_slot_status + slot, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA(ctx, cudaEventRecord(m->host_done[slot], ctx->stream));
    return B200_OK;
}

int b200_gpt2_forward_host_wait(b200_gpt2* m, int slot);

int b200_gpt2_forward_host(b200_gpt2* m, const int* tokens_host, int B, int T, float* logits_host,
                           float* last_logits_host, int* argmax_host) {
    const int st = b200_gpt2_forward_host_enqueue(m, tokens_host, B, T, logits_host, last_logits_host, argmax_host, 0);
    return st != B200_OK ? st : b200_gpt2_forward_host_wait(m, 0);
}

int b200_gpt2_forward_host_wait(b200_gpt2* m, int slot) {
    if (!m) return B200_ERR_NULL;
    if (slot < 0 || slot > 1) return B200_ERR_SHAPE;
    if (!m->h_slot_status) return B200_ERR_STATE;  // nothing was enqueued
    b200_ctx* ctx = m->ctx;
    B200_CUDA(ctx, cudaEventSynchronize(m->host_done[slot]));
    const int word = m->h_slot_status[slot];
    if (word != 0) {
        m->h_slot_status[slot] = 0;
        // cleared behind whatever is already queued; a step enqueued meanwhile reports the word too
        B200_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, 256, ctx->stream));
        B200_CUDA(ctx, cudaMemsetAsync(ctx->d_split_flags, 0, ctx->split_flag_words * sizeof(unsigned int), ctx->stream));
        // a forward that gave up may have left arg-max keys behind; the next one starts from zero again
        B200_CUDA(ctx, cudaMemsetAsync(m->argmax_keys, 0, (size_t)m->max_B * m->max_T * 8, ctx->stream));
        ctx->last_error = "device status word = " + std::to_string(word);
        return word == 201 ? B200_ERR_SHAPE : B200_ERR_TIMEOUT;
    }
    return B200_OK;
}

int b200_gpt2_enable_kv_cache(b200_gpt2* m) {
    if (!m) return B200_ERR_NULL;
    if (m->tp_size > 1) return B200_ERR_STATE;
    if (m->kcache) return B200_OK;
    b200_ctx* ctx = m->ctx;
    const size_t n = (size_t)m->cfg.num_layers * m->max_B * m->max_T * m->cfg.channels;
    B200_CUDA(ctx, cudaSetDevice(ctx->device));
    B200_CUDA(ctx, cudaMalloc(&m->kcache, n * sizeof(float)));
    cudaError_t e = cudaMalloc(&m->vcache, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&m->pos_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&m->resid2, (size_t)16 * m->cfg.channels * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&m->att_partial, (size_t)16 * m->cfg.num_heads * 8 * 66 * sizeof(float));  // up to 8 position splits
    if (e == cudaSuccess) e = cudaMalloc(&m->att_counters, (size_t)16 * m->cfg.num_heads * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(m->att_counters, 0, (size_t)16 * m->cfg.num_heads * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&m->gen_tokens, (size_t)m->max_B * m->max_T * sizeof(int));
    if (e != cudaSuccess) {
        cudaFree(m->kcache);
        if (m->vcache) cudaFree(m->vcache);
        m->kcache = m->vcache = nullptr;
        return b200_fail_cuda(ctx, e, "cudaMalloc (kv cache)");
    }
    return B200_OK;
}

int b200_gpt2_prefill(b200_gpt2* m, const int* tokens, int B, int T) {
    if (!m || !tokens) return B200_ERR_NULL;
    if (!m->kcache) return B200_ERR_STATE;
    if (B <= 0 || B > m->max_B || T <= 0 || T % 64 || T > m->max_T) return B200_ERR_SHAPE;
    b200_device_guard on_device(m->ctx);
    {
        int st = prepare_weights(m);
        if (st != B200_OK) return st;
    }
    m->keep_kv = true;  // eager (the replayed graphs are those of the plain forward)
    const int st = enqueue_forward(m, tokens, B, T, false);
    m->keep_kv = false;
    return st;
}

// One token per sequence: the forward's operator sequence on B rows, with the attention reading
// keys and values of positions 0..pos out of the cache.  The position comes from m->pos_dev.
static int enqueue_decode(b200_gpt2* m, const int* tokens, int B) {
    using namespace b200;
    b200_ctx* ctx = m->ctx;
    const b200_gpt2_config& c = m->cfg;
    const int C = c.channels, L = c.num_layers, Vp = c.padded_vocab_size, NH = c.num_heads;
    const float* P = m->params;
    const size_t* off = m->off;
    const size_t per_layer = (size_t)m->max_B * m->max_T * C;
    int st;
#define DSTEP(call) do { st = (call); if (st != B200_OK) return st; } while (0)
    // The residual stream alternates between two buffers: every GEMM that follows a layernorm
    // forms "residual + branch" and its layernorm itself (all of its CTAs, each for itself) and
    // one of them stores the new residual - into the other buffer, because the old one is still
    // being read.  C above the prologue's limit: the separate kernels, as in the full forward.
    float* ra = m->residual;
    float* rb = m->resid2;
    const bool fuse_ln = C <= 1664;
    // narrow projections are computed in K slices by more CTAs; the prologue that consumes them adds the slices up
    const int ks_att = fuse_ln ? skinny_gemm_k_splits(ctx, C, C) : 1;
    const int ks_fc = fuse_ln ? skinny_gemm_k_splits(ctx, 4 * C, C) : 1;
    DSTEP(launch_decode_encoder(ctx, ra, tokens, P + off[0], P + off[1], m->pos_dev, B, C, Vp));
    const float* branch = nullptr;  // what the next layernorm adds to the residual first
    for (int l = 0; l < L; ++l) {
        const float* qkvw = P + off[4] + (size_t)l * 3 * C * C;
        const float* qkvb = P + off[5] + (size_t)l * 3 * C;
        const float *ln1w = P + off[2] + (size_t)l * C, *ln1b = P + off[3] + (size_t)l * C;
        const float *ln2w = P + off[8] + (size_t)l * C, *ln2b = P + off[9] + (size_t)l * C;
        if (fuse_ln) {
            DSTEP(launch_skinny_gemm(ctx, m->qkv, ra, qkvw, qkvb, B, C, 3 * C, 0, branch, ln1w, ln1b, rb, 1, ks_fc));
            std::swap(ra, rb);
        } else {
            if (branch) {
                DSTEP(launch_fused_residual_layernorm(ctx, rb, m->ln_out, nullptr, nullptr, ra, branch, ln1w, ln1b, B, C, 0));
                std::swap(ra, rb);
            } else {
                DSTEP(launch_layernorm(ctx, m->ln_out, nullptr, nullptr, ra, ln1w, ln1b, B, C, 0));
            }
            DSTEP(launch_skinny_gemm(ctx, m->qkv, m->ln_out, qkvw, qkvb, B, C, 3 * C, 0));
        }
        DSTEP(launch_decode_attention(ctx, m->atty, m->qkv, m->kcache + l * per_layer, m->vcache + l * per_layer, B, C, NH, m->pos_dev, m->max_T, m->att_partial, m->att_counters));
        DSTEP(launch_skinny_gemm(ctx, m->branch, m->atty, P + off[6] + (size_t)l * C * C, P + off[7] + (size_t)l * C, B, C, C, 0,
                                 nullptr, nullptr, nullptr, nullptr, ks_att));
        const float* fcw = P + off[10] + (size_t)l * 4 * C * C;
        const float* fcb = P + off[11] + (size_t)l * 4 * C;
        if (fuse_ln) {
            DSTEP(launch_skinny_gemm(ctx, m->fch, ra, fcw, fcb, B, C, 4 * C, 1, m->branch, ln2w, ln2b, rb, 1, ks_att));
        } else {
            DSTEP(launch_fused_residual_layernorm(ctx, rb, m->ln_out, nullptr, nullptr, ra, m->branch, ln2w, ln2b, B, C, 0));
            DSTEP(launch_skinny_gemm(ctx, m->fch, m->ln_out, fcw, fcb, B, C, 4 * C, 1));
        }
        std::swap(ra, rb);
        DSTEP(launch_skinny_gemm(ctx, m->branch, m->fch, P + off[12] + (size_t)l * C * 4 * C, P + off[13] + (size_t)l * C, B, 4 * C, C, 0,
                                 nullptr, nullptr, nullptr, nullptr, ks_fc));
        branch = m->branch;
    }
    // final layernorm and lm-head
    if (fuse_ln) {
        DSTEP(launch_skinny_gemm(ctx, m->logits, ra, P + off[0], nullptr, B, C, Vp, 0, branch, P + off[14], P + off[15], rb, 1, ks_fc));
    } else {
        DSTEP(launch_fused_residual_layernorm(ctx, rb, m->ln_out, nullptr, nullptr, ra, branch, P + off[14], P + off[15], B, C, 0));
        DSTEP(launch_skinny_gemm(ctx, m->logits, m->ln_out, P + off[0], nullptr, B, C, Vp, 0));
    }
#undef DSTEP
    return B200_OK;
}

int b200_gpt2_decode_step(b200_gpt2* m, const int* tokens, int B, int pos) {
    if (!m || !tokens) return B200_ERR_NULL;
    if (!m->kcache) return B200_ERR_STATE;
    if (B <= 0 || B > 16 || B > m->max_B || pos < 0 || pos >= m->max_T) return B200_ERR_SHAPE;
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    int st = b200::launch_set_int(ctx, m->pos_dev, pos);
    if (st != B200_OK) return st;
    if (!m->use_graph || ctx->stream == nullptr) return enqueue_decode(m, tokens, B);

    // CUDA-graph replay (one graph per B; the position is data): the graph reads the token ids
    // from the model's own token buffer
    if (tokens != m->tokens)
        B200_CUDA(ctx, cudaMemcpyAsync(m->tokens, tokens, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    auto it = m->decode_graphs.find(B);
    if (it == m->decode_graphs.end()) {
        st = enqueue_decode(m, m->tokens, B);  // function attributes are set outside of capture; the step is idempotent
        if (st != B200_OK) return st;
        B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaGraph_t graph = nullptr;
        const uint64_t launches_before = ctx->launches;
        B200_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        st = enqueue_decode(m, m->tokens, B);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        ctx->launches = launches_before;
        if (st != B200_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (e != cudaSuccess) return b200_fail_cuda(ctx, e, "cudaStreamEndCapture");
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return b200_fail_cuda(ctx, e, "cudaGraphInstantiate");
        it = m->decode_graphs.emplace(B, exec).first;
    }
    B200_CUDA(ctx, cudaGraphLaunch(it->second, ctx->stream));
    ctx->launches += (m->cfg.channels <= 1664 ? 2 + 5ull * m->cfg.num_layers : 3 + 7ull * m->cfg.num_layers);  // set_int is counted by its launcher
    return B200_OK;
}

int b200_gpt2_decode_step_host(b200_gpt2* m, const int* tokens_host, int B, int pos, float* logits_host,
                               int* argmax_host) {
    if (!m || !tokens_host) return B200_ERR_NULL;
    if (B <= 0 || B > 16 || B > m->max_B) return B200_ERR_SHAPE;
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    const size_t Vp = m->cfg.padded_vocab_size;
    B200_CUDA(ctx, cudaMemcpyAsync(m->tokens, tokens_host, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
    int st = b200_gpt2_decode_step(m, m->tokens, B, pos);
    if (st != B200_OK) return st;
    if (argmax_host) {
        st = b200::launch_argmax_rows(ctx, m->argmax, m->logits, B, m->cfg.vocab_size, (int)Vp);
        if (st != B200_OK) return st;
        B200_CUDA(ctx, cudaMemcpyAsync(argmax_host, m->argmax, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    if (logits_host)
        B200_CUDA(ctx, cudaMemcpyAsync(logits_host, m->logits, (size_t)B * Vp * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return b200_ctx_sync_check(ctx);
}

int b200_gpt2_generate(b200_gpt2* m, const int* prompt_host, int B, int T0, int n_new, float temperature,
                       int top_k, float top_p, unsigned int seed, int* out_host) {
    if (!m || !prompt_host || !out_host) return B200_ERR_NULL;
    if (!m->kcache) return B200_ERR_STATE;
    if (B <= 0 || B > 16 || B > m->max_B || T0 < 1 || n_new < 1 || T0 + n_new > m->max_T || top_k < 0) return B200_ERR_SHAPE;
    b200_ctx* ctx = m->ctx;
    b200_device_guard on_device(ctx);
    const int V = m->cfg.vocab_size, Vp = m->cfg.padded_vocab_size;
    // gen holds the prompt [B,T0] and, behind it, the continuation [B,n_new]; m->argmax doubles as
    // the current column of token ids [B] (m->tokens belongs to the decode step's graph replay)
    int* gen = m->gen_tokens;
    int* rec = gen + (size_t)B * T0;
    B200_CUDA(ctx, cudaMemcpyAsync(gen, prompt_host, (size_t)B * T0 * 4, cudaMemcpyHostToDevice, ctx->stream));
    int st;
    if (T0 % 64 == 0) {
        st = b200_gpt2_prefill(m, gen, B, T0);
        if (st != B200_OK) return st;
        // arg-max of the last prompt position of every sequence: rows T0-1, 2*T0-1, ... of the logits
        for (int b = 0; b < B; ++b) {
            st = b200::launch_sample_rows(ctx, m->argmax + b, m->logits + ((size_t)b * T0 + T0 - 1) * Vp, 1, V, Vp,
                                          temperature, seed, (unsigned)T0 * 16u + b, top_k, top_p);
            if (st != B200_OK) return st;
        }
    } else {
        for (int t = 0; t < T0; ++t) {
            // column t of the prompt, gathered into a contiguous [B] (the decode step reads B ids in a row)
            B200_CUDA(ctx, cudaMemcpy2DAsync(m->argmax, 4, gen + t, (size_t)T0 * 4, 4, B, cudaMemcpyDeviceToDevice, ctx->stream));
            st = b200_gpt2_decode_step(m, m->argmax, B, t);
            if (st != B200_OK) return st;
        }
        st = b200::launch_sample_rows(ctx, m->argmax, m->logits, B, V, Vp, temperature, seed, (unsigned)T0 * 16u, top_k, top_p);
        if (st != B200_OK) return st;
    }
    for (int i = 0; i < n_new; ++i) {
        // m->argmax holds generated token i of every sequence: record it, then feed it at position T0 + i
        B200_CUDA(ctx, cudaMemcpy2DAsync(rec + i, (size_t)n_new * 4, m->argmax, 4, 4, B, cudaMemcpyDeviceToDevice, ctx->stream));
        if (i + 1 == n_new) break;
        st = b200_gpt2_decode_step(m, m->argmax, B, T0 + i);
        if (st != B200_OK) return st;
        // the token that will stand at position T0 + i + 1 of sequence b uses noise stream 16 * position + b
        st = b200::launch_sample_rows(ctx, m->argmax, m->logits, B, V, Vp, temperature, seed, (unsigned)(T0 + i + 1) * 16u, top_k, top_p);
        if (st != B200_OK) return st;
    }
    B200_CUDA(ctx, cudaMemcpyAsync(out_host, rec, (size_t)B * n_new * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return b200_ctx_sync_check(ctx);
}

int b200_gpt2_generate_greedy(b200_gpt2* m, const int* prompt_host, int B, int T0, int n_new, int* out_host) {
    return b200_gpt2_generate(m, prompt_host, B, T0, n_new, 0.f, 0, 0.f, 0u, out_host);
}

int b200_gpt2_set_profile(b200_gpt2* m, int enabled) {
    if (!m) return B200_ERR_NULL;
    m->profile = enabled != 0;
    return B200_OK;
}

int b200_gpt2_read_profile(b200_gpt2* m, double* ms, long* launches) {
    if (!m) return B200_ERR_NULL;
    b200_ctx* ctx = m->ctx;
    B200_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (size_t i = 0; i < m->ev_cat.size(); ++i) {
        float t = 0.f;
        B200_CUDA(ctx, cudaEventElapsedTime(&t, m->ev_pool[2 * i], m->ev_pool[2 * i + 1]));
        m->prof_ms[m->ev_cat[i]] += t;
        m->prof_launches[m->ev_cat[i]]++;
    }
    m->ev_cat.clear();
    m->ev_used = 0;
    for (int c = 0; c < B200_PROF_NUM; ++c) {
        if (ms) ms[c] = m->prof_ms[c];
        if (launches) launches[c] = m->prof_launches[c];
        m->prof_ms[c] = 0.0;
        m->prof_launches[c] = 0;
    }
    return B200_OK;
}

void* b200_gpt2_activation(b200_gpt2* m, const char* name) {
    if (!m || !name) return nullptr;
    if (!strcmp(name, "residual") || !strcmp(name, "encoded")) return m->residual;
    if (!strcmp(name, "ln_out")) return m->ln_out;
    if (!strcmp(name, "qkv")) return m->qkv;
    if (!strcmp(name, "atty")) return m->atty;
    if (!strcmp(name, "branch")) return m->branch;
    if (!strcmp(name, "fch")) return m->fch;
    if (!strcmp(name, "argmax")) return m->argmax;
    return nullptr;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Forward pass without any device allocation.
//
// Some callers must not allocate device memory: code that runs after an application has handed
// every byte of the GPU to its own pool, plugin hosts that forbid driver allocations once
// initialisation is over, and latency-critical serving loops that cannot afford the implicit
// device-wide synchronisation of cudaMalloc / cudaFree.  For them the per-layer activations of
// the forward (the scratch memory that b200_gpt2_create normally allocates) live in the
// file-scope array below, which every GPU that loads this library holds until the process exits.
constexpr size_t kStaticScratchRowElems = (size_t)B200_STATIC_MAX_TOKEN_CHANNELS;  // max B*T*C
// residual, ln_out, atty, branch: 1 each; qkv: 3; fch: 4  (units of B*T*C floats)
constexpr size_t kStaticScratchFloats = 11 * kStaticScratchRowElems;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

namespace {
// In host code the name g_static_scratch is only a stand-in; the device address has to be asked
// for, once per device, with that device current.  Looking it up loads this file's module, and
// the first launch of each kernel loads that kernel's code - both may allocate device memory - so
// the set-up also loads every kernel the static forward can launch.
std::mutex g_static_mu;
float* g_static_addr[64] = {};

int static_prepare(b200_ctx* ctx, float** scratch) {
    if (ctx->device < 0 || ctx->device >= 64) { ctx->last_error = "b200_gpt2_forward_static: device index beyond 63"; return B200_ERR_LIMIT; }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_addr[ctx->device]) {
        int cur = -1;
        B200_CUDA(ctx, cudaGetDevice(&cur));
        if (cur != ctx->device) B200_CUDA(ctx, cudaSetDevice(ctx->device));
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        int st = (e != cudaSuccess || !p) ? b200_fail_cuda(ctx, e, "cudaGetSymbolAddress(g_static_scratch)") : B200_OK;
        if (st == B200_OK) st = b200::preload_rowwise_kernels(ctx);
        if (st == B200_OK) st = b200::preload_gemm_kernels(ctx);
        if (st == B200_OK) st = b200::preload_attention_kernel(ctx);
        if (cur != ctx->device) cudaSetDevice(cur);  // leave the caller's current device as it was
        if (st != B200_OK) return st;
        g_static_addr[ctx->device] = static_cast<float*>(p);
    }
    if (scratch) *scratch = g_static_addr[ctx->device];
    return B200_OK;
}
}  // namespace

extern "C" int b200_gpt2_static_prepare(b200_ctx* ctx) {
    if (!ctx) return B200_ERR_NULL;
    return static_prepare(ctx, nullptr);
}

extern "C" int b200_gpt2_forward_static(b200_ctx* ctx, const b200_gpt2_config* cfg, const float* params,
                                        const int* tokens, int B, int T, float* logits) {
    if (!ctx || !cfg || !params || !tokens || !logits) return B200_ERR_NULL;
    if (!b200_aligned16(params) || !b200_aligned16(logits)) return B200_ERR_ALIGN;
    if (cfg->channels <= 0 || cfg->num_heads <= 0 || cfg->channels % cfg->num_heads ||
        cfg->channels / cfg->num_heads != 64 || cfg->channels > 4096 || cfg->num_layers <= 0 ||
        cfg->padded_vocab_size % 4 || cfg->vocab_size <= 0 || cfg->vocab_size > cfg->padded_vocab_size ||
        B <= 0 || T <= 0 || T % 64 || T > cfg->max_seq_len)
        return B200_ERR_SHAPE;
    const size_t MC = (size_t)B * T * cfg->channels;
    if (MC > kStaticScratchRowElems) {
        ctx->last_error = "b200_gpt2_forward_static: B*T*C = " + std::to_string(MC) + " exceeds the built-in scratch of " +
                          std::to_string(kStaticScratchRowElems) + " (B200_STATIC_MAX_TOKEN_CHANNELS); use b200_gpt2_create / b200_gpt2_forward";
        return B200_ERR_LIMIT;
    }
    float* scratch = nullptr;
    int st = static_prepare(ctx, &scratch);  // a no-op after b200_gpt2_static_prepare or an earlier call on this device
    if (st != B200_OK) return st;
    b200_device_guard on_device(ctx);  // launches go to ctx->stream, which belongs to ctx->device
    // a view of the caller's parameters and logits plus the built-in scratch; nothing is owned
    b200_gpt2 view;
    view.ctx = ctx;
    view.cfg = *cfg;
    view.max_B = B;
    view.max_T = T;
    if (!set_tp_dims(&view, 1, 0)) return B200_ERR_SHAPE;
    view.params = const_cast<float*>(params);  // read only: weights are not rounded on this path
    view.round_operands = 0;                   // the arithmetic of b200_gpt2_forward with round_operands = 0
    view.gemm_mode = view.lmhead_mode = B200_TF32;  // ... and single-pass TF32 GEMMs: no copies of the weights
    view.residual = scratch;
    view.ln_out = scratch + MC;
    view.atty = scratch + 2 * MC;
    view.branch = scratch + 3 * MC;
    view.qkv = scratch + 4 * MC;
    view.fch = scratch + 7 * MC;
    view.logits = logits;
    // every region is written in full before it is read, so nothing has to be cleared between calls
    return enqueue_forward(&view, tokens, B, T, false);
}
