// The Qwen3 forward pass behind el::Backend::eval of the reference (src/model.h:42-51): weight table, KV cache,
// the layer loop (CpuModel::forward order, src/model.cpp:157-234), prompt chunking and the captured decode step.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "split.cuh"
#include "decode.cuh"

namespace elb {

namespace {

struct HostTensor {
    int type = -1;
    int64_t rows = 0, n = 0;
    const uint8_t* bytes = nullptr;
    size_t nbytes = 0;
};

struct Seg {
    Weight* w = nullptr;
    int64_t col = 0;  // first output column of this segment
};

struct Layer {
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    std::vector<Seg> qkv;  // neighbours of equal type are one matrix (upload_lin of the reference, :1509-1528)
    Weight *wo = nullptr, *gu = nullptr, *down = nullptr;
};

bool env_on(const char* name) {
    const char* v = std::getenv(name);
    return v && v[0] == '1';
}

}  // namespace

struct Model {
    elb_config cfg{};
    int n_ctx = 0, device = 0, max_batch = 512, n_seq = 1;
    bool finalized = false;
    std::vector<HostTensor> pending;  // [3 + n_layer * 11], valid until finalize
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    Weight *embd = nullptr, *head = nullptr;  // head == embd when tied
    float* output_norm = nullptr;
    std::vector<Layer> layers;
    float* rope = nullptr;
    float *kcache = nullptr, *vcache = nullptr;
    float *x = nullptr, *qkv = nullptr, *att = nullptr, *act = nullptr, *logits = nullptr;
    int8_t* limbs = nullptr;
    float *inv_scale = nullptr, *xsum = nullptr;
    void* kv16 = nullptr;             // keys and values of one layer as fp16 pairs (tensor-core prompt attention)
    float* tc_part = nullptr;         // partial tiles and arrival counters of the fp16 tensor-core GEMM's k splits
    unsigned* tc_counters = nullptr;
    int32_t* tokens_dev = nullptr;
    int* pos_dev = nullptr;
    int32_t* tokens_host = nullptr;  // pinned
    int* pos_host = nullptr;         // pinned
    int8_t* dlimbs[4] = {nullptr, nullptr, nullptr, nullptr};  // single-token limb buffers (see body_decode)
    float* dinv = nullptr;   // [4] their 2^-k
    unsigned* done = nullptr;  // [4] post-op arrival counters
    float* attn_part = nullptr;
    unsigned* attn_counters = nullptr;
    int attn_split = 1;
    cudaGraphExec_t graph = nullptr;
    bool use_graph = true, use_pdl = true;
    int nl_qkv = 4, nl_wo = 3, nl_gu = 3, nl_down = 4;  // limbs per linear (reference defaults, :1871-1877)
    float last_ms = 0.f;
    int64_t last_launches = 0, launches = 0, graph_launches_ = 0;
    int last_rows = 1, decode_calls = 0;
    size_t weight_bytes = 0;
    // persistent decode kernel (quantized models whose step fits in shared memory)
    bool use_mega = false;
    DkParams dk{};
    float* norm_arena = nullptr;  // the norm vectors of all layers, layer after layer: attn_norm [E], ffn_norm [E], q_norm, k_norm [head_dim]
    int dk_slot = 0, dk_grid = 0;  // dk_slot: bytes of one warp's ring of weight units
    float* xbuf = nullptr;  // persistent kernel: residual stream [2][E]
    TpPeerBuf xarea;        // persistent kernel: flags, partial sums and logits, visible to all tensor-parallel ranks
    unsigned* xctl = nullptr;
    int8_t* gact = nullptr;  // persistent kernel: limbs of the FFN activation when they do not fit in shared memory
    float* logits_step = nullptr;  // where a single-token step leaves its logits (m->logits unless the persistent kernel runs)
    unsigned* sync_words = nullptr;  // barrier counter, step index, advance flag, launch count, then 2 x [n_layer][2] amax slots
    int* pos_steps = nullptr;        // positions of a batch of single-token steps (persistent kernel)
    int* err_host = nullptr;         // pinned, mapped: raised by the kernel when a barrier wait runs out
    // tensor parallelism (tp.size == 1: none). H, HKV, F are this rank's share of heads and of the FFN dimension.
    TpDims tp{};
    TpComm* comm = nullptr;
    TpReduce* tpr = nullptr;  // single-token all-reduce through peer memory (null: NCCL)
    TpRows* tprows = nullptr; // all-reduce of a small batch of rows through peer memory (null: NCCL)
    int H = 0, HKV = 0;
    int64_t F = 0;
    // several sequences (n_seq > 1): rows of a batch carry their own sequence and position
    int *seq_dev = nullptr, *posv_dev = nullptr;   // [max_batch]
    float* logits_rows = nullptr;                  // [n_seq][n_vocab] logits of the wanted rows of a batch
    float* rows_part = nullptr;                    // attention partial results of a batch
    unsigned* rows_counters = nullptr;
    int rows_split = 1;
    uint8_t* top_dev = nullptr;      // device-side logits post-processing: lse, ids, logits
    uint8_t* top_host = nullptr;     // pinned
    uint8_t *top_rows_dev = nullptr, *top_rows_host = nullptr;  // the same for every wanted row of a batch: [n_seq][TOP_BYTES]
    uint32_t* mask_dev = nullptr;    // allowed-token bits of a constrained pick
    float* ap_part = nullptr;        // partial results of the chunked prompt attention
    unsigned* ap_counters = nullptr;
    float* xr = nullptr;            // [max_batch][E] this rank's partial sums before the all-reduce
    float* logits_local = nullptr;  // [vchunk] this rank's rows of the head
    std::vector<std::vector<uint8_t>> shard_store;  // column cuts of wo / down, valid until finalize
};

namespace {

int64_t slot_of(const Model* m, int role, int layer) { return role <= ELB_OUTPUT_NORM ? role : 3 + int64_t(layer) * 11 + (role - 3); }

// dst: device memory for the vector (null: *out is allocated)
int upload_f32(const HostTensor& t, float** out, float* dst = nullptr) {
    if (!t.bytes) return fail(ELB_ERR_STATE, "model: a norm tensor is missing");
    if (t.type != ELB_F32 && t.type != ELB_F16) return fail(ELB_ERR_UNSUPPORTED, "model: norm weights must be F32 or F16");
    if (t.rows <= 0 || t.n <= 0 || t.nbytes != size_t(t.rows) * size_t(t.n) * (t.type == ELB_F32 ? 4 : 2))
        return fail(ELB_ERR_INVALID, "model: a norm tensor's byte count does not match its shape");
    std::vector<float> v(size_t(t.rows * t.n));
    if (t.type == ELB_F32) {
        std::memcpy(v.data(), t.bytes, v.size() * 4);
    } else if (t.type == ELB_F16) {
        const uint16_t* h = reinterpret_cast<const uint16_t*>(t.bytes);
        for (size_t i = 0; i < v.size(); ++i) v[i] = __half2float(__ushort_as_half(h[i]));
    } else {
        return fail(ELB_ERR_UNSUPPORTED, "model: norm weights must be F32 or F16");
    }
    if (dst) *out = dst;
    else ELB_CUDA(cudaMalloc(out, v.size() * 4));
    ELB_CUDA(cudaMemcpy(*out, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    return ELB_OK;
}

// consecutive tensors of one type and row length -> one weight; returns segments with their output columns
int upload_linear(Model* m, std::initializer_list<const HostTensor*> parts, int flags, std::vector<Seg>* out) {
    std::vector<const HostTensor*> group;
    int64_t col = 0;
    auto flush = [&]() -> int {
        if (group.empty()) return ELB_OK;
        int64_t rows = 0;
        size_t bytes = 0;
        for (auto* t : group) { rows += t->rows; bytes += t->nbytes; }
        Seg s;
        s.col = col;
        if (group.size() == 1) {
            ELB_TRY(weight_create(m->device, group[0]->type, rows, group[0]->n, group[0]->bytes, bytes, flags, &s.w));
        } else {
            std::vector<uint8_t> cat(bytes);
            size_t off = 0;
            for (auto* t : group) { std::memcpy(cat.data() + off, t->bytes, t->nbytes); off += t->nbytes; }
            ELB_TRY(weight_create(m->device, group[0]->type, rows, group[0]->n, cat.data(), bytes, flags, &s.w));
        }
        ELB_TRY(gemv_prepare(s.w));
        m->weight_bytes += s.w->tiled_bytes;
        out->push_back(s);
        col += rows;
        group.clear();
        return ELB_OK;
    };
    for (auto* t : parts) {
        if (!t->bytes) return fail(ELB_ERR_STATE, "model: a weight tensor is missing");
        if (!group.empty() && (group[0]->type != t->type || group[0]->n != t->n)) ELB_TRY(flush());
        group.push_back(t);
    }
    return flush();
}

int upload_pair(Model* m, const HostTensor& gate, const HostTensor& up, Weight** out) {
    if (!gate.bytes || !up.bytes) return fail(ELB_ERR_STATE, "model: ffn_gate / ffn_up missing");
    if (gate.type != up.type || gate.n != up.n || gate.rows != up.rows)
        return fail(ELB_ERR_UNSUPPORTED, "model: ffn_gate and ffn_up must have the same type and shape");
    std::vector<uint8_t> cat(gate.nbytes + up.nbytes);
    std::memcpy(cat.data(), gate.bytes, gate.nbytes);
    std::memcpy(cat.data() + gate.nbytes, up.bytes, up.nbytes);
    ELB_TRY(weight_create(m->device, gate.type, gate.rows, gate.n, cat.data(), cat.size(), ELB_W_PLANES | ELB_W_PAIR, out));
    ELB_TRY(gemv_prepare(*out));
    m->weight_bytes += (*out)->tiled_bytes;
    return ELB_OK;
}

int check_shape(const HostTensor& t, int64_t rows, int64_t n, const char* what) {
    if (t.bytes && (t.rows != rows || t.n != n)) return fail(ELB_ERR_UNSUPPORTED, std::string("model: unexpected shape of ") + what);
    return ELB_OK;
}

// ---- one linear layer over B tokens (linear() of the reference, :1706-1780), limbs already split when quantized
int linear_tokens(Model* m, const Weight* w, const float* xin, int64_t ldx, const float* norm_w, int B, float* y,
                  int64_t ldy, const float* resid, int epi, int nl) {
    ++m->launches;
    if (gemm_f16_tc_usable(w, B)) {  // F16, and Q8_0 held as fp16 pairs
        ++m->launches;  // the hi / lo split of the rows
        return gemm_f16_tc_launch(w, xin, ldx, norm_w, m->cfg.eps, B, m->limbs, m->inv_scale, y, ldy, resid, epi, m->stream, m->use_pdl,
                                  m->tc_part, m->tc_counters);
    }
    if (w->type == ELB_F16) return gemm_f16_launch(w, xin, ldx, norm_w, m->cfg.eps, B, y, ldy, resid, epi, m->stream);
    if (gemm_tc_usable(w, B)) return gemm_tc_launch(w, m->limbs, m->inv_scale, m->xsum, B, nl, y, ldy, resid, epi, m->stream, m->use_pdl);
    return gemm_planes_launch(w, m->limbs, m->inv_scale, m->xsum, B, y, ldy, resid, epi, m->stream);
}

int split_tokens(Model* m, const float* xin, int64_t ldx, int n, int nl, const float* norm_w, int B, bool any_quant) {
    if (!any_quant) return ELB_OK;
    ++m->launches;
    return split_launch(xin, ldx, B, n, nl, norm_w, m->cfg.eps, m->limbs, m->inv_scale, m->xsum, m->stream, m->use_pdl);
}

// xr (every rank's partial sums of B rows) -> x on every rank: through peer memory for a small batch, NCCL otherwise
int rows_all_reduce(Model* m, int B) {
    const size_t n = size_t(B) * m->cfg.n_embd;
    if (m->tprows && n <= m->tprows->n_max) return tp_rows_all_reduce(m->tprows, m->xr, m->x, n, m->stream);
    return tp_all_reduce(m->comm, m->xr, m->x, n, m->stream);
}

// Rows of one sequence at consecutive positions (seq0, pos0 + b), or (mixed) row b at posv_dev[b] of sequence seq_dev[b].
int body_prefill(Model* m, int B, int pos0, int seq0 = 0, bool mixed = false) {
    const elb_config& c = m->cfg;
    const int E = c.n_embd, F = int(m->F), H = m->H, HKV = m->HKV, QD = H * 128, KD = HKV * 128, QKV = QD + 2 * KD;
    const float scale = 1.0f / std::sqrt(float(c.head_dim));
    // row-parallel linears (wo, down): every rank writes its partial sums to xr (rank 0 adds the residual), the
    // all-reduce leaves the new residual stream in x on every rank
    const bool tp = m->tp.size > 1;
    float* yo = tp ? m->xr : m->x;
    const float* res = !tp || m->tp.rank == 0 ? m->x : nullptr;
    const int epi_o = res ? EPI_ADD : EPI_STORE;
    for (int l = 0; l < c.n_layer; ++l) {
        Layer& L = m->layers[size_t(l)];
        const size_t seq_stride = size_t(m->n_ctx) * KD;
        float* kc = m->kcache + (size_t(l) * m->n_seq + (mixed ? 0 : seq0)) * seq_stride;
        float* vc = m->vcache + (size_t(l) * m->n_seq + (mixed ? 0 : seq0)) * seq_stride;
        bool q = false;
        for (auto& s : L.qkv) q |= !gemm_f16_tc_usable(s.w, B) && s.w->type != ELB_F16;
        ELB_TRY(split_tokens(m, m->x, E, E, m->nl_qkv, L.attn_norm, B, q));
        for (auto& s : L.qkv) ELB_TRY(linear_tokens(m, s.w, m->x, E, L.attn_norm, B, m->qkv + s.col, QKV, nullptr, EPI_STORE, m->nl_qkv));
        if (mixed) {
            ELB_TRY(qkv_post_launch(m->qkv, QKV, L.q_norm, L.k_norm, m->rope, 0, B, kc, vc, H, HKV, c.rope_dim, c.eps, m->stream,
                                    m->posv_dev, m->seq_dev, seq_stride));
            ELB_TRY(attn_rows_launch(m->qkv, QKV, kc, vc, seq_stride, m->posv_dev, m->seq_dev, m->att, QD, m->rows_part,
                                     m->rows_counters, B, H, HKV, m->rows_split, scale, m->stream));
        } else {
            ELB_TRY(qkv_post_launch(m->qkv, QKV, L.q_norm, L.k_norm, m->rope, pos0, B, kc, vc, H, HKV, c.rope_dim, c.eps, m->stream));
            if (m->kv16 && attn_prefill_tc_usable(H, HKV, QKV, QD)) {
                ELB_TRY(attn_prefill_tc_launch(m->qkv, QKV, kc, vc, m->att, QD, pos0, B, H, HKV, scale, m->stream, m->ap_part, m->ap_counters, m->kv16));
                ++m->launches;  // the fp16 split of the layer's keys and values
            } else {
                ELB_TRY(attn_prefill_launch(m->qkv, QKV, kc, vc, m->att, QD, pos0, B, H, HKV, scale, m->stream, m->ap_part, m->ap_counters));
            }
        }
        m->launches += 2;
        ELB_TRY(split_tokens(m, m->att, QD, QD, m->nl_wo, nullptr, B, L.wo->type != ELB_F16 && !gemm_f16_tc_usable(L.wo, B)));
        ELB_TRY(linear_tokens(m, L.wo, m->att, QD, nullptr, B, yo, E, res, epi_o, m->nl_wo));
        if (tp) ELB_TRY(rows_all_reduce(m, B));
        ELB_TRY(split_tokens(m, m->x, E, E, m->nl_gu, L.ffn_norm, B, L.gu->type != ELB_F16 && !gemm_f16_tc_usable(L.gu, B)));
        ELB_TRY(linear_tokens(m, L.gu, m->x, E, L.ffn_norm, B, m->act, F, nullptr, EPI_SILU, m->nl_gu));
        ELB_TRY(split_tokens(m, m->act, F, F, m->nl_down, nullptr, B, L.down->type != ELB_F16 && !gemm_f16_tc_usable(L.down, B)));
        ELB_TRY(linear_tokens(m, L.down, m->act, F, nullptr, B, yo, E, res, epi_o, m->nl_down));
        if (tp) ELB_TRY(rows_all_reduce(m, B));
    }
    return ELB_OK;
}

// Where the activation of a single-token matvec comes from: limbs left in `lim` by the producer's post-op (quantized
// weights), or the fp32 vector itself, normalised inside the kernel (F16 weights).
struct ActIn {
    const int8_t* lim;
    const float* inv_scale;
    const float* x;
    const float* norm_w;
};

int gemv(Model* m, const Weight* w, const ActIn& in, float* y, const float* resid, int epi, const PostOp& post) {
    GemvArgs a;
    a.limbs = in.lim; a.inv_scale = in.inv_scale;
    a.x = in.x; a.norm_w = in.norm_w; a.eps = m->cfg.eps;
    a.prologue = in.norm_w ? PRO_RMSNORM : PRO_PLAIN;
    a.y = y; a.resid = resid; a.epilogue = epi; a.pdl = m->use_pdl; a.post = post;
    ++m->launches;
    return gemv_launch(w, a, m->stream);
}

// post-op that leaves the limbs of `src` (optionally RMSNorm'ed) in slot `slot` of the model's limb buffers; none when
// the consumer does not read limbs
PostOp make_post(Model* m, bool wanted, const float* src, int n, const float* norm_w, int nl, int slot) {
    PostOp po;
    if (!wanted) return po;
    po.kind = 1; po.src = src; po.n = n; po.nl = nl; po.norm_w = norm_w; po.eps = m->cfg.eps;
    po.limbs = m->dlimbs[slot]; po.inv_scale = m->dinv + slot; po.done = m->done + slot;
    return po;
}

// the head on limbs already in slot 0 (or on xrow for F16 weights); under tensor parallelism every rank computes its
// vocabulary rows and the all-gather assembles the logits on all of them
int head_gemv(Model* m, const float* xrow) {
    if (m->tp.size == 1)
        return gemv(m, m->head, ActIn{m->dlimbs[0], m->dinv, xrow, m->output_norm}, m->logits, nullptr, EPI_STORE, PostOp{});
    ELB_TRY(gemv(m, m->head, ActIn{m->dlimbs[0], m->dinv, xrow, m->output_norm}, m->logits_local, nullptr, EPI_STORE, PostOp{}));
    return tp_all_gather(m->comm, m->logits_local, m->logits, size_t(m->tp.vchunk), m->stream);
}

// final norm + head on one row of x (the reference runs the head as a B=1 matvec too, :1833-1837); stand-alone split
int head_logits(Model* m, const float* xrow) {
    const int E = m->cfg.n_embd;
    if (m->head->type != ELB_F16) {
        ELB_TRY(prep_limbs_launch(xrow, E, m->output_norm, m->cfg.eps, 4, m->dlimbs[0], m->dinv, false, m->stream));
        ++m->launches;
    }
    return head_gemv(m, xrow);
}

// one token: everything through the matvec kernels; position and token id are read from device memory so that the
// step can be captured once and replayed. Limb buffers: 0 = input of qkv / head, 1 = input of wo, 2 = input of gate|up,
// 3 = input of down; each is filled by the post-op of the kernel that produces the vector.
int body_decode(Model* m) {
    const elb_config& c = m->cfg;
    const int E = c.n_embd, F = int(m->F), H = m->H, HKV = m->HKV, QD = H * 128, KD = HKV * 128;
    const float scale = 1.0f / std::sqrt(float(c.head_dim));
    const bool tp = m->tp.size > 1;
    float* yo = tp ? m->xr : m->x;
    const float* res = !tp || m->tp.rank == 0 ? m->x : nullptr;
    const int epi_o = res ? EPI_ADD : EPI_STORE;
    // after a row-parallel matvec: all-reduce the partial sums into x, then split x for the next matvec (single GPU:
    // that split is the matvec's own post-op)
    auto reduce_then_split = [&](bool wanted, const float* norm_w, int nl, int slot) -> int {
        if (m->tpr) {  // one kernel: exchange through peer memory, sum, (norm +) split
            ++m->launches;
            return tp_reduce_split_launch(m->tpr, m->xr, m->x, E, norm_w, c.eps, nl, wanted ? m->dlimbs[slot] : nullptr,
                                          m->dinv + slot, m->stream);
        }
        ELB_TRY(tp_all_reduce(m->comm, m->xr, m->x, size_t(E), m->stream));
        if (!wanted) return ELB_OK;
        ++m->launches;
        return prep_limbs_launch(m->x, E, norm_w, c.eps, nl, m->dlimbs[slot], m->dinv + slot, false, m->stream);
    };
    if (m->use_mega) {
        ++m->launches;
        return decode_step_launch(m->dk, m->dk_slot, m->dk_grid, m->stream);
    }
    auto quant = [](const Weight* w) { return w->type != ELB_F16; };
    auto qkv_quant = [&](const Layer& L) { bool q = false; for (auto& s : L.qkv) q |= quant(s.w); return q; };
    ELB_TRY(launch_gather_rows(m->embd, m->tokens_dev, 1, m->x, m->stream));
    ++m->launches;
    if (qkv_quant(m->layers[0])) {
        ELB_TRY(prep_limbs_launch(m->x, E, m->layers[0].attn_norm, c.eps, m->nl_qkv, m->dlimbs[0], m->dinv, m->use_pdl, m->stream));
        ++m->launches;
    }
    for (int l = 0; l < c.n_layer; ++l) {
        Layer& L = m->layers[size_t(l)];
        const bool last = l + 1 == c.n_layer;
        for (auto& s : L.qkv)
            ELB_TRY(gemv(m, s.w, ActIn{m->dlimbs[0], m->dinv, m->x, L.attn_norm}, m->qkv + s.col, nullptr, EPI_STORE, PostOp{}));
        AttnDecodeArgs a{m->qkv, L.q_norm, L.k_norm, m->rope, m->pos_dev,
                         m->kcache + size_t(l) * m->n_seq * m->n_ctx * KD, m->vcache + size_t(l) * m->n_seq * m->n_ctx * KD, m->att, m->attn_part,
                         m->attn_counters, H, HKV, c.rope_dim, m->attn_split, c.eps, scale, m->use_pdl,
                         make_post(m, quant(L.wo), m->att, QD, nullptr, m->nl_wo, 1)};
        ELB_TRY(attn_decode_launch(a, m->stream));
        ++m->launches;
        ELB_TRY(gemv(m, L.wo, ActIn{m->dlimbs[1], m->dinv + 1, m->att, nullptr}, yo, res, epi_o,
                     make_post(m, !tp && quant(L.gu), m->x, E, L.ffn_norm, m->nl_gu, 2)));
        if (tp) ELB_TRY(reduce_then_split(quant(L.gu), L.ffn_norm, m->nl_gu, 2));
        ELB_TRY(gemv(m, L.gu, ActIn{m->dlimbs[2], m->dinv + 2, m->x, L.ffn_norm}, m->act, nullptr, EPI_SILU,
                     make_post(m, quant(L.down), m->act, F, nullptr, m->nl_down, 3)));
        const bool next_quant = last ? quant(m->head) : qkv_quant(m->layers[size_t(l) + 1]);
        const float* next_norm = last ? m->output_norm : m->layers[size_t(l) + 1].attn_norm;
        ELB_TRY(gemv(m, L.down, ActIn{m->dlimbs[3], m->dinv + 3, m->act, nullptr}, yo, res, epi_o,
                     make_post(m, !tp && next_quant, m->x, E, next_norm, last ? 4 : m->nl_qkv, 0)));
        if (tp) ELB_TRY(reduce_then_split(next_quant, next_norm, last ? 4 : m->nl_qkv, 0));
    }
    return head_gemv(m, m->x);
}

// Enqueue one single-token step on the model's stream (token id and position already on the device). The first
// step runs eagerly (it also sets the kernels' launch attributes), the second is captured, later ones replay the graph.
int enqueue_decode_step(Model* m) {
    if (!m->use_graph || m->decode_calls++ == 0) return body_decode(m);
    if (!m->graph) {
        cudaGraph_t g = nullptr;
        ELB_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const int64_t before = m->launches;
        const int rc = body_decode(m);
        m->graph_launches_ = m->launches - before;
        m->launches = before;
        const cudaError_t e = cudaStreamEndCapture(m->stream, &g);
        if (rc != ELB_OK) { if (g) cudaGraphDestroy(g); return rc; }
        ELB_CUDA(e);
        const cudaError_t ei = cudaGraphInstantiate(&m->graph, g, 0);
        cudaGraphDestroy(g);
        ELB_CUDA(ei);
    }
    ELB_CUDA(cudaGraphLaunch(m->graph, m->stream));
    m->launches += m->graph_launches_;
    return ELB_OK;
}

// `top`: instead of copying the logits out, reduce them on the device to the k best tokens and the log-sum-exp
struct TopOut { int k; int32_t* ids; float* vals; double* lse; const uint32_t* allowed; };

int chunk(Model* m, const int32_t* tokens, int B, int pos0, float* logits, const TopOut* top = nullptr) {
    std::memcpy(m->tokens_host, tokens, size_t(B) * sizeof(int32_t));
    *m->pos_host = pos0;
    ELB_CUDA(cudaMemcpyAsync(m->tokens_dev, m->tokens_host, size_t(B) * sizeof(int32_t), cudaMemcpyHostToDevice, m->stream));
    ELB_CUDA(cudaMemcpyAsync(m->use_mega && B == 1 ? m->pos_steps : m->pos_dev, m->pos_host, sizeof(int), cudaMemcpyHostToDevice, m->stream));
    ELB_CUDA(cudaEventRecord(m->ev0, m->stream));
    m->last_rows = B;
    if (B == 1) {
        ELB_TRY(enqueue_decode_step(m));
    } else {
        ELB_TRY(launch_gather_rows(m->embd, m->tokens_dev, B, m->x, m->stream));
        ++m->launches;
        ELB_TRY(body_prefill(m, B, pos0));
        if (logits || top) ELB_TRY(head_logits(m, m->x + size_t(B - 1) * m->cfg.n_embd));
    }
    const float* dev_logits = B == 1 && m->use_mega ? m->logits_step : m->logits;
    if (top) {
        if (top->allowed)  // (pageable source: staged by the runtime before the call returns)
            ELB_CUDA(cudaMemcpyAsync(m->mask_dev, top->allowed, size_t((m->cfg.n_vocab + 31) / 32) * 4, cudaMemcpyHostToDevice, m->stream));
        ELB_TRY(logits_top_launch(dev_logits, m->cfg.n_vocab, top->k, m->top_dev, m->stream, top->allowed ? m->mask_dev : nullptr));
        ++m->launches;
    }
    ELB_CUDA(cudaEventRecord(m->ev1, m->stream));
    if (logits)
        ELB_CUDA(cudaMemcpyAsync(logits, dev_logits, size_t(m->cfg.n_vocab) * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
    if (top) ELB_CUDA(cudaMemcpyAsync(m->top_host, m->top_dev, TOP_BYTES, cudaMemcpyDeviceToHost, m->stream));
    ELB_CUDA(cudaStreamSynchronize(m->stream));
    if (top) {  // layout of the result: lse (double), then k ids, then k logits
        const uint8_t* r = m->top_host;
        std::memcpy(top->lse, r, sizeof(double));
        std::memcpy(top->ids, r + 8, size_t(top->k) * sizeof(int32_t));
        std::memcpy(top->vals, r + 8 + 4 * TOP_MAXK, size_t(top->k) * sizeof(float));
    }
    if (m->err_host && *m->err_host) return fail(ELB_ERR_CUDA, "decode kernel: a grid barrier wait ran out");
    if ((m->tpr && *m->tpr->err_host) || (m->tprows && *m->tprows->err_host))
        return fail(ELB_ERR_CUDA, "tensor parallel: a peer did not arrive at an all-reduce in time");
    ELB_TRY(gemm_tc_check());
    ELB_TRY(gemm_f16_tc_check());
    float ms = 0.f;
    ELB_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    m->last_ms += ms;
    return ELB_OK;
}

}  // namespace

// Fill the parameters of the persistent decode kernel; it is used when every weight is quantized and the step's
// shared memory (rings + the longest activation's limbs) fits on one SM. ELB_NO_MEGA=1 keeps the kernel-per-op path.
// local_ok: false when this rank already failed earlier in its set-up. Under tensor parallelism it still walks through
// the collectives of this function (the other ranks are on their way into them) with "failed" as its answer.
int setup_decode_kernel(Model* m, bool local_ok = true) {
    const elb_config& c = m->cfg;
    if (env_on("ELB_NO_MEGA") || (m->tp.size > 1 && env_on("ELB_TP_NO_MEGA"))) return ELB_OK;
    DeviceInfo di;
    ELB_TRY(device_info(m->device, &di));
    auto kind_of = [](const Weight* w) {  // alone in its phase, whole tiles per CTA
        return DkKind{int(w->tiles), int(w->units_per_tile), int(w->rows), int(w->n), int(w->tiles), 0, 0, 0};
    };
    // row-parallel matrices (few row tiles, long rows): equal unit ranges, when every CTA's range is at least one tile
    // long, so that no tile has more than two contributors
    auto kind_balanced = [&](const Weight* w) {
        DkKind d = kind_of(w);
        d.balanced = w->tiles * w->units_per_tile / di.sm_count >= w->units_per_tile ? 1 : 0;
        return d;
    };
    auto same_shape = [](const Weight* a, const Weight* b) {
        return a->tiles == b->tiles && a->units_per_tile == b->units_per_tile && a->rows == b->rows && a->n == b->n;
    };
    bool quant = m->head->type != ELB_F16 && m->embd->type != ELB_F32;
    const size_t nq = m->layers[0].qkv.size();
    for (const Layer& L : m->layers) {
        quant = quant && L.qkv.size() == nq && L.wo->type != ELB_F16 && L.gu->type != ELB_F16 && L.down->type != ELB_F16;
        for (auto& s : L.qkv) quant = quant && s.w->type != ELB_F16;
    }
    // this rank's dimensions; the longest FFN cut of any rank sizes the shared memory, so that all ranks decide alike
    int Fmax = int(m->F);
    for (int r = 0; r < m->tp.size; ++r) {
        TpDims d;
        ELB_TRY(tp_dims(c, r, m->tp.size, &d));
        Fmax = std::max(Fmax, int(d.f1 - d.f0));
    }
    const int E = c.n_embd, F = int(m->F), QD = m->H * 128, KD = m->HKV * 128;
    // (the residual stream is split two blocks per warp and pass, other activations three: longer ones go to global memory)
    if (!quant || nq > 3 || E % 256 || F % 256 || QD % 256 || E > 2 * 256 * decode_warps() || QD > 3 * 256 * decode_warps() ||
        c.n_layer > DK_MAX_LAYERS)
        return ELB_OK;
    // the kernel takes the shape of each kind of matrix from layer 0: every layer must repeat it (block formats may differ)
    for (const Layer& L : m->layers) {
        const Layer& L0 = m->layers[0];
        bool same = same_shape(L.wo, L0.wo) && same_shape(L.gu, L0.gu) && same_shape(L.down, L0.down);
        for (size_t i = 0; i < nq; ++i) same = same && same_shape(L.qkv[i].w, L0.qkv[i].w) && L.qkv[i].col == L0.qkv[i].col;
        if (!same) return ELB_OK;
    }
    DkParams& p = m->dk;
    p = DkParams{};
    p.kind[6] = kind_of(m->head);
    p.W[c.n_layer][0] = m->head->tiled;
    p.wtype[c.n_layer][0] = uint8_t(m->head->type);
    int unit_max = m->head->unit_bytes, unit_min = m->head->unit_bytes;  // largest and smallest unit of the step
    int slots = 0, cta_tiles = 0;
    auto account = [&](const Weight* w) {
        unit_max = std::max(unit_max, w->unit_bytes);
        unit_min = std::min(unit_min, w->unit_bytes);
        const int64_t per_cta = (w->tiles + di.sm_count - 1) / di.sm_count * w->units_per_tile;
        const int64_t per_warp = (per_cta + decode_warps() - 1) / decode_warps();
        slots = std::max(slots, int((per_warp + w->units_per_tile - 1) / w->units_per_tile + 2));
        cta_tiles = std::max(cta_tiles, int((w->tiles + di.sm_count - 1) / di.sm_count + 2));
    };
    account(m->head);
    for (int l = 0; l < c.n_layer; ++l) {
        const Layer& L = m->layers[size_t(l)];
        int group = 0;
        for (size_t i = 0; i < nq; ++i) group += int(L.qkv[i].w->tiles);
        for (size_t i = 0, off = 0; i < nq; ++i) {  // q, k, v share one phase: the CTAs cut the tiles of all three together
            if (l == 0) {
                p.kind[i] = kind_of(L.qkv[i].w);
                p.kind[i].group_tiles = group;
                p.kind[i].group_off = int(off);
                p.qkv_col[i] = int(L.qkv[i].col);
            }
            off += size_t(L.qkv[i].w->tiles);
            p.W[l][i] = L.qkv[i].w->tiled;
            p.wtype[l][i] = uint8_t(L.qkv[i].w->type);
            account(L.qkv[i].w);
        }
        if (l == 0) { p.kind[3] = kind_balanced(L.wo); p.kind[4] = kind_of(L.gu); p.kind[5] = kind_balanced(L.down); }
        const Weight* rest[3] = {L.wo, L.gu, L.down};
        for (int i = 0; i < 3; ++i) {
            p.W[l][nq + i] = rest[i]->tiled;
            p.wtype[l][nq + i] = uint8_t(rest[i]->type);
            account(rest[i]);
        }
    }
    if (nq > 1 && !env_on("ELB_DK_EVEN_TILES")) {  // q|k|v cut by cost: a tile's units times the time a unit of its format takes
        auto unit_cost = [](int type) { return type == ELB_Q6_K ? 1455 : type == ELB_Q8_0 ? 481 : 875; };  // SM clocks, measured
        long long off = 0;
        for (size_t i = 0; i < nq; ++i) {
            long long sum = 0;
            for (int l = 0; l < c.n_layer; ++l) sum += unit_cost(p.wtype[l][i]);
            p.kind[i].cost = int(sum / c.n_layer) * p.kind[i].upt;
            p.kind[i].group_cost_off = int(off);
            off += (long long)p.kind[i].cost * p.kind[i].tiles;
        }
        if (off < (1ll << 30))
            for (size_t i = 0; i < nq; ++i) p.kind[i].group_cost = int(off);
    }
    p.norms = m->norm_arena;
    p.norm_stride = int(2 * E + 2 * c.head_dim);
    p.kc = m->kcache;  // sequence 0
    p.vc = m->vcache;
    p.kv_stride = size_t(m->n_seq) * m->n_ctx * KD;
    if (local_ok && cudaMalloc(&m->xbuf, size_t(2) * E * sizeof(float)) != cudaSuccess) {  // residual stream [2][E]
        cudaGetLastError();
        local_ok = false;
        fail(ELB_ERR_MEMORY, "decode kernel set-up: out of device memory");
    }
    // exchange area: flags, partial sums [2 sets][ranks][2][E], logits; mapped into every rank under tensor parallelism
    const int N = m->tp.size;
    const int pv = 2;  // (one vector per rank with whole tiles measured slower at two ranks: 6.74 against 6.57 ms on the 32B shape)
    // (under tensor parallelism every partial sum travels with a sequence number in the same 8-byte word)
    const size_t part_floats = size_t(2) * N * pv * E * (N > 1 ? 2 : 1), logit_floats = size_t(std::max<int64_t>(c.n_vocab, m->tp.vchunk * N));
    const size_t xbytes = 256 + (part_floats + logit_floats) * sizeof(float);
    if (N > 1) {
        bool mapped = false;
        ELB_TRY(tp_peer_alloc(m->comm, m->device, xbytes, m->stream, &m->xarea, &mapped, local_ok));
        if (!local_ok) return ELB_ERR_MEMORY;  // (every rank has seen it: none of them maps, none waits for this one)
        if (!mapped) return ELB_OK;  // no peer mapping: the kernel-per-op path with NCCL stays
    } else {
        if (!local_ok) return ELB_ERR_MEMORY;
        ELB_CUDA(cudaMalloc(&m->xarea.local, xbytes));
        ELB_CUDA(cudaMemset(m->xarea.local, 0, xbytes));
        m->xarea.peer[0] = m->xarea.local;
        m->xarea.size = 1;
    }
    int* err_dev = nullptr;
    auto local_words = [&]() -> int {
        ELB_CUDA(cudaMalloc(&m->xctl, 2 * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(m->xctl, 0, 2 * sizeof(unsigned)));
        ELB_CUDA(cudaMalloc(&m->sync_words, size_t(4 + 4 * c.n_layer) * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(m->sync_words, 0, size_t(4 + 4 * c.n_layer) * sizeof(unsigned)));
        ELB_CUDA(cudaMalloc(&m->pos_steps, size_t(m->max_batch) * sizeof(int)));
        ELB_CUDA(cudaHostAlloc(&m->err_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
        *m->err_host = 0;
        ELB_CUDA(cudaHostGetDevicePointer(&err_dev, m->err_host, 0));
        return ELB_OK;
    };
    int rc_local = local_words();  // a failure is carried to the agreement below, not returned before it
    p.n_layer = c.n_layer; p.n_qkv = int(nq);
    p.output_norm = m->output_norm;
    p.embd = m->embd->tiled; p.embd_type = m->embd->type;
    p.E = E; p.F = F; p.H = m->H; p.HKV = m->HKV; p.rope_dim = c.rope_dim; p.n_ctx = m->n_ctx;
    p.nsplit = std::max(1, std::min({decode_max_split(), m->attn_split, di.sm_count / m->HKV}));
    p.tp_rank = m->tp.rank; p.tp_size = N; p.pv = pv; p.v0 = int(m->tp.v0); p.xctl = m->xctl;
    for (int q = 0; q < N; ++q) {
        uint8_t* base = static_cast<uint8_t*>(m->xarea.peer[q]);
        p.flag_peer[q] = reinterpret_cast<unsigned*>(base);
        p.part_peer[q] = reinterpret_cast<float*>(base + 256);
        p.logits_peer[q] = p.part_peer[q] + part_floats;
    }
    p.eps = c.eps; p.scale = 1.0f / std::sqrt(float(c.head_dim));
    p.nl_qkv = m->nl_qkv; p.nl_wo = m->nl_wo; p.nl_gu = m->nl_gu; p.nl_down = m->nl_down;
    p.token = m->tokens_dev; p.pos = m->pos_steps; p.rope = m->rope;
    p.x = m->x; p.qkv = m->qkv; p.att = m->att; p.act = m->act; p.logits = m->logits;
    p.xbuf = m->xbuf; p.bar = m->sync_words; p.ctl = m->sync_words + 1; p.amax = m->sync_words + 4;
    p.attn_part = m->attn_part; p.attn_counters = m->attn_counters;
    p.err = err_dev; p.slots = slots; p.cta_tiles = cta_tiles; p.n_max = std::max({E, Fmax, QD});
    m->dk_grid = di.sm_count;
    // 32-bit unit arithmetic in the kernel
    bool small = true;
    for (int l = 0; l < c.n_layer; ++l)
        for (const Weight* w : {m->layers[size_t(l)].wo, m->layers[size_t(l)].gu, m->layers[size_t(l)].down, m->head})
            if (w->tiles * w->units_per_tile * int64_t(di.sm_count) >= (int64_t(1) << 31) || w->max_grid < di.sm_count) small = false;
    // The rings of the warps take whatever shared memory the activation limbs and the reduction buffers leave; a ring
    // shorter than ELB_DK_MIN_RING bytes (default: 8 KB, three to four units) would leave the weight stream too little
    // run-ahead, and the long FFN activation then goes to global memory instead.
    bool fits = false;
    int min_ring = std::max(8192, 2 * unit_max);
    if (const char* v = std::getenv("ELB_DK_MIN_RING")) min_ring = std::max(2 * unit_max, std::atoi(v));
    auto try_fit = [&]() -> int {
        m->dk_slot = decode_ring_bytes(p, unit_max, unit_min, m->device);
        if (const char* v = std::getenv("ELB_DK_RING")) m->dk_slot = std::min(m->dk_slot, std::max(2 * unit_max, std::atoi(v) / 128 * 128));  // (experiments)
        fits = false;
        if (m->dk_slot >= min_ring) ELB_TRY(decode_step_fits(p, m->dk_slot, m->device, &fits));
        return ELB_OK;
    };
    auto local_fit = [&]() -> int {
        ELB_TRY(try_fit());
        if ((!fits || env_on("ELB_DK_GACT")) && Fmax > std::max(E, QD)) {  // (the variable forces the mode, for tests)
            // the limbs of the FFN activation do not fit next to the rings: keep them in global memory (one more grid
            // barrier per layer, ffn_down reads them through L2); every rank decides from the longest FFN cut, so all
            // decide alike
            p.act_global = 1;
            p.n_max = std::max(E, QD);
            ELB_TRY(try_fit());
            if (fits) {
                ELB_CUDA(cudaMalloc(&m->gact, decode_act_bytes(Fmax)));
                p.gact = m->gact;
            }
        }
        return ELB_OK;
    };
    if (rc_local == ELB_OK) rc_local = local_fit();
    fits = fits && small && rc_local == ELB_OK;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->device) != cudaSuccess) { cudaGetLastError(); coop = 0; }
    bool all = false;  // under tensor parallelism every rank must take the same path: its kernels wait for the peers'
    ELB_TRY(tp_agree(m->comm, fits && coop, m->stream, &all));
    if (rc_local != ELB_OK) return rc_local;  // (after the agreement: the other ranks fell back to the kernel-per-op path together)
    m->use_mega = all;
    if (m->use_mega) m->logits_step = p.logits_peer[m->tp.rank];  // the kernel leaves the logits in the exchange area
    if (m->use_mega && env_on("ELB_DK_PROF")) {
        ELB_CUDA(cudaMalloc(&p.prof, size_t(c.n_layer) * 32 * sizeof(unsigned long long)));
        ELB_CUDA(cudaMemset(p.prof, 0, size_t(c.n_layer) * 32 * sizeof(unsigned long long)));
        ELB_CUDA(cudaMalloc(&p.prof_cta, size_t(di.sm_count) * 16 * sizeof(unsigned long long)));
        ELB_CUDA(cudaMemset(p.prof_cta, 0, size_t(di.sm_count) * 16 * sizeof(unsigned long long)));
        p.prof_layer = c.n_layer / 2;
    }
    return ELB_OK;
}

int model_create(const elb_config* cfg, int n_ctx, int device, Model** out) {
    return model_create_tp(cfg, n_ctx, device, 0, 1, nullptr, out);
}

int model_create_tp(const elb_config* cfg, int n_ctx, int device, int rank, int size, const void* id128, Model** out) {
    if (!cfg || !out) return fail(ELB_ERR_INVALID, "model_create: null argument");
    if (size > 1 && !id128) return fail(ELB_ERR_INVALID, "model_create: tensor parallelism needs the communicator id");
    if (n_ctx <= 0) return fail(ELB_ERR_INVALID, "model_create: context length must be positive");
    if (cfg->n_layer <= 0 || cfg->n_layer > 512 || cfg->n_embd <= 0 || cfg->n_head <= 0 || cfg->n_head_kv <= 0 ||
        cfg->n_head % cfg->n_head_kv != 0 || cfg->n_ff <= 0 || cfg->n_vocab <= 0 || cfg->rope_dim <= 0 ||
        cfg->rope_dim % 2 != 0 || cfg->rope_dim > cfg->head_dim)
        return fail(ELB_ERR_INVALID, "model_create: invalid configuration");
    if (cfg->head_dim != 128) return fail(ELB_ERR_UNSUPPORTED, "model_create: only head_dim = 128 is supported");
    if (cfg->n_head / cfg->n_head_kv > 8) return fail(ELB_ERR_UNSUPPORTED, "model_create: at most 8 query heads per KV head");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) {
        cudaGetLastError();
        return fail(ELB_ERR_CUDA, "model_create: no such CUDA device");
    }
    TpDims tp;
    ELB_TRY(tp_dims(*cfg, rank, size, &tp));
    auto* m = new Model;
    m->cfg = *cfg;
    m->tp = tp;
    m->H = tp.H; m->HKV = tp.HKV; m->F = tp.f1 - tp.f0;
    m->n_ctx = n_ctx;
    m->device = device;
    if (size > 1) {
        const int rc = tp_comm_create(device, rank, size, id128, &m->comm);
        if (rc != ELB_OK) { delete m; return rc; }
    }
    m->max_batch = cfg->max_batch > 0 ? cfg->max_batch : 512;
    m->n_seq = cfg->n_seq > 0 ? cfg->n_seq : 1;
    m->pending.resize(size_t(3 + cfg->n_layer * 11));
    m->layers.resize(size_t(cfg->n_layer));
    m->use_graph = !env_on("ELB_NO_GRAPH");
    m->use_pdl = !env_on("ELB_NO_PDL");
    if (const char* v = std::getenv("ELB_NL3")) {  // bit mask like the reference's EL_NL3: 1 qkv, 2 wo, 4 gate/up, 8 down
        const int mask = std::atoi(v);
        m->nl_qkv = mask & 1 ? 3 : 4; m->nl_wo = mask & 2 ? 3 : 4; m->nl_gu = mask & 4 ? 3 : 4; m->nl_down = mask & 8 ? 3 : 4;
    }
    *out = m;
    return ELB_OK;
}

int model_set_tensor(Model* m, int role, int layer, int type, int64_t rows, int64_t n, const void* bytes, size_t nbytes) {
    if (!m || !bytes) return fail(ELB_ERR_INVALID, "set_tensor: null argument");
    if (m->finalized) return fail(ELB_ERR_STATE, "set_tensor: model already finalized");
    if (role < 0 || role > ELB_DOWN) return fail(ELB_ERR_INVALID, "set_tensor: unknown role");
    if (role > ELB_OUTPUT_NORM && (layer < 0 || layer >= m->cfg.n_layer)) return fail(ELB_ERR_RANGE, "set_tensor: layer out of range");
    m->pending[size_t(slot_of(m, role, layer))] = HostTensor{type, rows, n, static_cast<const uint8_t*>(bytes), nbytes};
    return ELB_OK;
}

void model_destroy(Model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    if (m->graph) cudaGraphExecDestroy(m->graph);
    if (m->head && m->head != m->embd) weight_destroy(m->head);  // also a row view of embd (tied head under TP)
    weight_destroy(m->embd);
    for (Layer& L : m->layers) {
        for (auto& s : L.qkv) weight_destroy(s.w);
        weight_destroy(L.wo); weight_destroy(L.gu); weight_destroy(L.down);
    }
    cudaFree(m->norm_arena);
    for (void* p : {(void*)m->output_norm, (void*)m->rope, (void*)m->kcache, (void*)m->vcache, (void*)m->x, (void*)m->qkv,
                    (void*)m->att, (void*)m->act, (void*)m->logits, (void*)m->limbs, (void*)m->inv_scale, (void*)m->xsum,
                    (void*)m->tokens_dev, (void*)m->pos_dev, (void*)m->attn_part, (void*)m->attn_counters, (void*)m->dlimbs[0],
                    (void*)m->dlimbs[1], (void*)m->dlimbs[2], (void*)m->dlimbs[3], (void*)m->dinv, (void*)m->done})
        cudaFree(p);
    cudaFree(m->xbuf); cudaFree(m->xctl); cudaFree(m->gact); cudaFree(m->tc_part); cudaFree(m->tc_counters); cudaFree(m->kv16);
    if (m->xarea.local) tp_peer_free(&m->xarea, m->tp.rank); cudaFree(m->sync_words); cudaFree(m->pos_steps);
    cudaFree(m->xr); cudaFree(m->logits_local);
    cudaFree(m->ap_part); cudaFree(m->ap_counters); cudaFree(m->top_dev); cudaFree(m->mask_dev);
    if (m->top_host) cudaFreeHost(m->top_host);
    cudaFree(m->top_rows_dev);
    if (m->top_rows_host) cudaFreeHost(m->top_rows_host);
    cudaFree(m->seq_dev); cudaFree(m->posv_dev); cudaFree(m->logits_rows); cudaFree(m->rows_part); cudaFree(m->rows_counters);
    tp_reduce_destroy(m->tpr);
    tp_rows_destroy(m->tprows);
    tp_comm_destroy(m->comm);
    if (m->err_host) cudaFreeHost(m->err_host);
    if (m->tokens_host) cudaFreeHost(m->tokens_host);
    if (m->pos_host) cudaFreeHost(m->pos_host);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

// everything of finalize that concerns this rank alone: uploads, re-layout, allocations; no collective in here
static int finalize_local(Model* m) {
    ELB_CUDA(cudaSetDevice(m->device));
    const elb_config& c = m->cfg;
    const int64_t E = c.n_embd, V = c.n_vocab, B = m->max_batch;
    auto P = [&](int role, int layer) -> const HostTensor& { return m->pending[size_t(slot_of(m, role, layer))]; };
    {   // global shapes, then (tensor parallel) every tensor is replaced by this rank's cut of it
        const int64_t F = c.n_ff, QD = int64_t(c.n_head) * 128, KD = int64_t(c.n_head_kv) * 128;

    // shapes (read_tensors of the reference, src/model.cpp:66-103)
    ELB_TRY(check_shape(P(ELB_TOK_EMBD, 0), V, E, "token_embd"));
    ELB_TRY(check_shape(P(ELB_OUTPUT, 0), V, E, "output"));
    for (int l = 0; l < c.n_layer; ++l) {
        ELB_TRY(check_shape(P(ELB_WQ, l), QD, E, "attn_q"));
        ELB_TRY(check_shape(P(ELB_WK, l), KD, E, "attn_k"));
        ELB_TRY(check_shape(P(ELB_WV, l), KD, E, "attn_v"));
        ELB_TRY(check_shape(P(ELB_WO, l), E, QD, "attn_output"));
        ELB_TRY(check_shape(P(ELB_GATE, l), F, E, "ffn_gate"));
        ELB_TRY(check_shape(P(ELB_UP, l), F, E, "ffn_up"));
        ELB_TRY(check_shape(P(ELB_DOWN, l), E, F, "ffn_down"));
    }
    // norm vectors (expect_shape {E} / {head_dim} of the reference, src/model.cpp:76,92-95): the kernels read E or
    // head_dim floats from them whatever the caller said their length was
    auto check_vec = [&](const HostTensor& t, int64_t len, const char* what) -> int {
        if (t.bytes && t.rows * t.n != len) return fail(ELB_ERR_UNSUPPORTED, std::string("model: unexpected shape of ") + what);
        return ELB_OK;
    };
    ELB_TRY(check_vec(P(ELB_OUTPUT_NORM, 0), E, "output_norm"));
    for (int l = 0; l < c.n_layer; ++l) {
        ELB_TRY(check_vec(P(ELB_ATTN_NORM, l), E, "attn_norm"));
        ELB_TRY(check_vec(P(ELB_FFN_NORM, l), E, "ffn_norm"));
        ELB_TRY(check_vec(P(ELB_Q_NORM, l), c.head_dim, "attn_q_norm"));
        ELB_TRY(check_vec(P(ELB_K_NORM, l), c.head_dim, "attn_k_norm"));
    }
    }
    if (m->tp.size > 1) {
        for (int role = ELB_OUTPUT; role <= ELB_DOWN; ++role) {
            if (role != ELB_OUTPUT && role < ELB_WQ) continue;
            for (int l = 0; l < (role == ELB_OUTPUT ? 1 : c.n_layer); ++l) {
                HostTensor& t = m->pending[size_t(slot_of(m, role, l))];
                if (!t.bytes) continue;
                TpShard sh;
                ELB_TRY(tp_shard_shape(c, m->tp, role, t.type, t.rows, t.n, &sh));
                if (sh.contiguous) {
                    t.bytes += size_t(sh.row0) * size_t(sh.src_row_bytes);
                } else {
                    m->shard_store.emplace_back(sh.nbytes);
                    ELB_TRY(tp_shard_copy(sh, t.bytes, t.nbytes, m->shard_store.back().data()));
                    t.bytes = m->shard_store.back().data();
                }
                t.rows = sh.rows; t.n = sh.n; t.nbytes = sh.nbytes;
            }
        }
    }
    const int64_t F = m->F, QD = int64_t(m->H) * 128, KD = int64_t(m->HKV) * 128, QKV = QD + 2 * KD;

    // device memory budget before anything is allocated (pre-flight check of the reference, :1578-1591)
    const size_t kv_bytes = size_t(c.n_layer) * size_t(m->n_seq) * size_t(m->n_ctx) * size_t(KD) * sizeof(float);
    const int64_t maxn = std::max({E, QD, F});
    size_t need = 2 * kv_bytes + size_t(B) * size_t(E + QKV + QD + F) * 4 + size_t(V) * 4 + size_t(4) * B * maxn + size_t(B) * (maxn / 32 + 1) * 4;
    for (const HostTensor& t : m->pending)
        if (t.bytes && t.rows > 1) need += t.nbytes + (t.type != ELB_F16 && &t != &P(ELB_TOK_EMBD, 0) && &t != &P(ELB_OUTPUT, 0) ? size_t(t.rows) * t.n * 2 + size_t(t.rows) * (t.n / 32) * 4 : 0);
    size_t free_b = 0, total_b = 0;
    ELB_CUDA(cudaMemGetInfo(&free_b, &total_b));
    if (need + (256ull << 20) > free_b) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "not enough device memory: %.0f MB needed, %.0f MB free (lower n_ctx)", need / 1048576.0, free_b / 1048576.0);
        return fail(ELB_ERR_MEMORY, msg);
    }

    ELB_CUDA(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    ELB_CUDA(cudaEventCreate(&m->ev0));
    ELB_CUDA(cudaEventCreate(&m->ev1));

    const HostTensor& emb = P(ELB_TOK_EMBD, 0);
    if (!emb.bytes) return fail(ELB_ERR_STATE, "model: token_embd missing");
    // with several sequences the head runs as a matrix product over the rows of a batch: digit planes for it too
    const int head_flags = m->n_seq > 1 && m->tp.size == 1 ? ELB_W_PLANES : 0;
    const bool tied = !P(ELB_OUTPUT, 0).bytes;
    ELB_TRY(weight_create(m->device, emb.type, emb.rows, emb.n, emb.bytes, emb.nbytes, tied ? head_flags : 0, &m->embd));
    ELB_TRY(gemv_prepare(m->embd));
    const HostTensor& outw = P(ELB_OUTPUT, 0);
    if (outw.bytes) {
        ELB_TRY(weight_create(m->device, outw.type, outw.rows, outw.n, outw.bytes, outw.nbytes, head_flags, &m->head));
        ELB_TRY(gemv_prepare(m->head));
    } else if (m->tp.size > 1) {
        ELB_TRY(weight_view_rows(m->embd, m->tp.v0, m->tp.v1 - m->tp.v0, &m->head));  // this rank's rows of the tied table
        ELB_TRY(gemv_prepare(m->head));
    } else {
        m->head = m->embd;  // tied embeddings (src/model.cpp:73-74 of the reference)
    }
    m->weight_bytes += m->head->tiled_bytes;
    ELB_TRY(upload_f32(P(ELB_OUTPUT_NORM, 0), &m->output_norm));
    // the norm vectors of all layers in one piece of memory at a fixed stride: kernels address layer l by arithmetic
    const size_t norm_stride = size_t(2) * E + 2 * size_t(c.head_dim);
    ELB_CUDA(cudaMalloc(&m->norm_arena, size_t(c.n_layer) * norm_stride * sizeof(float)));
    for (int l = 0; l < c.n_layer; ++l) {
        Layer& L = m->layers[size_t(l)];
        float* base = m->norm_arena + size_t(l) * norm_stride;
        ELB_TRY(upload_f32(P(ELB_ATTN_NORM, l), &L.attn_norm, base));
        ELB_TRY(upload_f32(P(ELB_FFN_NORM, l), &L.ffn_norm, base + E));
        ELB_TRY(upload_f32(P(ELB_Q_NORM, l), &L.q_norm, base + 2 * E));
        ELB_TRY(upload_f32(P(ELB_K_NORM, l), &L.k_norm, base + 2 * E + c.head_dim));
        ELB_TRY(upload_linear(m, {&P(ELB_WQ, l), &P(ELB_WK, l), &P(ELB_WV, l)}, ELB_W_PLANES, &L.qkv));
        std::vector<Seg> one;
        ELB_TRY(upload_linear(m, {&P(ELB_WO, l)}, ELB_W_PLANES, &one));
        L.wo = one[0].w;
        ELB_TRY(upload_pair(m, P(ELB_GATE, l), P(ELB_UP, l), &L.gu));
        one.clear();
        ELB_TRY(upload_linear(m, {&P(ELB_DOWN, l)}, ELB_W_PLANES, &one));
        L.down = one[0].w;
    }

    // RoPE table: angle in double, rounded to float (src/model.cpp:105-109, 23-32; src/cuda/model_cuda.cu:1610-1619)
    {
        const int half = c.rope_dim / 2;
        std::vector<float> cs(size_t(m->n_ctx) * half * 2);
        std::vector<double> inv(static_cast<size_t>(half));
        for (int i = 0; i < half; ++i) inv[size_t(i)] = std::pow(c.rope_base, -2.0 * i / c.rope_dim);
        for (int p = 0; p < m->n_ctx; ++p)
            for (int i = 0; i < half; ++i) {
                const double th = p * inv[size_t(i)];
                cs[(size_t(p) * half + i) * 2] = float(std::cos(th));
                cs[(size_t(p) * half + i) * 2 + 1] = float(std::sin(th));
            }
        ELB_CUDA(cudaMalloc(&m->rope, cs.size() * 4));
        ELB_CUDA(cudaMemcpy(m->rope, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    }
    ELB_CUDA(cudaMalloc(&m->kcache, kv_bytes));
    ELB_CUDA(cudaMalloc(&m->vcache, kv_bytes));
    ELB_CUDA(cudaMemset(m->kcache, 0, kv_bytes));
    ELB_CUDA(cudaMemset(m->vcache, 0, kv_bytes));
    ELB_CUDA(cudaMalloc(&m->x, size_t(B) * E * 4));
    ELB_CUDA(cudaMalloc(&m->qkv, size_t(B) * QKV * 4));
    ELB_CUDA(cudaMalloc(&m->att, size_t(B) * QD * 4));
    ELB_CUDA(cudaMalloc(&m->act, size_t(B) * F * 4));
    ELB_CUDA(cudaMalloc(&m->logits, size_t(std::max<int64_t>(V, m->tp.vchunk * m->tp.size)) * 4));
    if (m->tp.size > 1) {
        ELB_CUDA(cudaMalloc(&m->xr, size_t(B) * E * 4));
        ELB_CUDA(cudaMalloc(&m->logits_local, size_t(m->tp.vchunk) * 4));
    }
    ELB_CUDA(cudaMalloc(&m->limbs, size_t(4) * B * maxn));
    ELB_CUDA(cudaMalloc(&m->inv_scale, size_t(B) * 4));
    ELB_CUDA(cudaMalloc(&m->tc_part, gemm_f16_tc_part_bytes()));
    ELB_CUDA(cudaMalloc(&m->tc_counters, size_t(gemm_f16_tc_counters()) * sizeof(unsigned)));
    ELB_CUDA(cudaMemset(m->tc_counters, 0, size_t(gemm_f16_tc_counters()) * sizeof(unsigned)));
    ELB_CUDA(cudaMalloc(&m->xsum, size_t(B) * (maxn / 32 + 1) * 4));
    ELB_CUDA(cudaMalloc(&m->tokens_dev, size_t(B) * sizeof(int32_t)));
    ELB_CUDA(cudaMalloc(&m->pos_dev, sizeof(int)));
    if (m->n_seq > 1) {
        DeviceInfo dinfo;
        ELB_TRY(device_info(m->device, &dinfo));
        ELB_CUDA(cudaMalloc(&m->seq_dev, size_t(B) * sizeof(int)));
        ELB_CUDA(cudaMalloc(&m->posv_dev, size_t(B) * sizeof(int)));
        ELB_CUDA(cudaMalloc(&m->logits_rows, size_t(m->n_seq) * V * sizeof(float)));
        // key splits of the batched attention: enough CTAs for two per SM when one row per sequence is in the batch
        m->rows_split = int(std::max<int64_t>(1, std::min<int64_t>(8, (2 * dinfo.sm_count + int64_t(m->n_seq) * m->HKV - 1) / (int64_t(m->n_seq) * m->HKV))));
        const int group = c.n_head / c.n_head_kv;
        ELB_CUDA(cudaMalloc(&m->rows_part, size_t(B) * m->HKV * m->rows_split * group * (128 + 2) * sizeof(float)));
        ELB_CUDA(cudaMalloc(&m->rows_counters, size_t(B) * m->HKV * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(m->rows_counters, 0, size_t(B) * m->HKV * sizeof(unsigned)));
    }
    ELB_CUDA(cudaMallocHost(&m->tokens_host, size_t(B) * sizeof(int32_t)));
    ELB_CUDA(cudaMallocHost(&m->pos_host, sizeof(int)));
    {
        const int64_t ns[4] = {E, QD, E, F};
        for (int i = 0; i < 4; ++i) ELB_CUDA(cudaMalloc(&m->dlimbs[i], act_bytes(int(ns[i]))));
        ELB_CUDA(cudaMalloc(&m->dinv, 4 * sizeof(float)));
        ELB_CUDA(cudaMalloc(&m->done, 4 * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(m->done, 0, 4 * sizeof(unsigned)));
    }
    // decode attention: a fixed number of key splits so that the launch shape does not depend on the position
    DeviceInfo di;
    ELB_TRY(device_info(m->device, &di));
    m->attn_split = std::max(1, std::min(32, (di.sm_count + m->HKV - 1) / m->HKV));
    if (const char* v = std::getenv("ELB_ATTN_SPLIT")) m->attn_split = std::max(1, std::min(32, std::atoi(v)));
    const int group = c.n_head / c.n_head_kv;
    ELB_CUDA(cudaMalloc(&m->attn_part, size_t(m->HKV) * m->attn_split * group * std::max(128 + 2, decode_part_stride()) * 4));
    ELB_CUDA(cudaMalloc(&m->attn_counters, size_t(m->HKV) * sizeof(unsigned)));
    ELB_CUDA(cudaMemset(m->attn_counters, 0, size_t(m->HKV) * sizeof(unsigned)));
    ELB_CUDA(cudaMalloc(&m->top_dev, TOP_BYTES));
    ELB_CUDA(cudaMallocHost(&m->top_host, TOP_BYTES));
    ELB_CUDA(cudaMalloc(&m->top_rows_dev, size_t(m->n_seq) * TOP_BYTES));
    ELB_CUDA(cudaMallocHost(&m->top_rows_host, size_t(m->n_seq) * TOP_BYTES));
    ELB_CUDA(cudaMalloc(&m->mask_dev, size_t((V + 31) / 32) * 4));
    ELB_CUDA(cudaMalloc(&m->ap_part, attn_prefill_scratch_floats(m->max_batch, m->H, m->HKV) * sizeof(float)));
    ELB_CUDA(cudaMalloc(&m->ap_counters, attn_prefill_counters(m->max_batch, m->H, m->HKV) * sizeof(unsigned)));
    ELB_CUDA(cudaMemset(m->ap_counters, 0, attn_prefill_counters(m->max_batch, m->H, m->HKV) * sizeof(unsigned)));
    ELB_CUDA(cudaMalloc(&m->kv16, attn_prefill_tc_scratch_halves(m->n_ctx, m->HKV * 128) * 2));
    // test hook: a rank that fails on its own once everything local is in place (as it would running out of memory)
    if (const char* v = std::getenv("ELB_TEST_FAIL_FINALIZE_RANK"))
        if (m->tp.size > 1 && std::atoi(v) == m->tp.rank) return fail(ELB_ERR_MEMORY, "finalize: injected failure of this rank (test)");
    return ELB_OK;
}

// Under tensor parallelism the ranks set up peer memory with collectives. A rank that fails on its own (out of memory
// while uploading, say) must not leave the others waiting in one: the ranks first agree that the local part worked
// everywhere, every rank then passes through the same collectives whatever happens to it locally, and a last agreement
// makes the outcome the same on all of them - all finalized, or an error on every rank.
int model_finalize(Model* m) {
    if (!m) return fail(ELB_ERR_INVALID, "finalize: null model");
    if (m->finalized) return fail(ELB_ERR_STATE, "finalize: called twice");
    int rc = finalize_local(m);
    const bool tp = m->tp.size > 1 && m->comm;
    const char* other = "finalize: another rank of the tensor-parallel group failed to set up its model";
    if (tp) {
        bool all = false;
        const int rc_a = tp_agree(m->comm, rc == ELB_OK, m->stream, &all);
        if (rc != ELB_OK) return rc;
        if (rc_a != ELB_OK) return rc_a;
        if (!all) return fail(ELB_ERR_STATE, other);
        if (!env_on("ELB_TP_NCCL")) {
            rc = tp_reduce_create(m->comm, m->device, m->tp.rank, m->tp.size, m->cfg.n_embd, m->stream, &m->tpr);
            // (a rank that failed above still walks through this one's collectives, with "failed" as its answer)
            const int rc2 = tp_rows_create(m->comm, m->device, m->tp.rank, m->tp.size, size_t(16) * m->cfg.n_embd, m->stream, &m->tprows,
                                           rc == ELB_OK);
            if (rc == ELB_OK) rc = rc2;
        }
    } else if (rc != ELB_OK) {
        return rc;
    }
    const int rc_k = setup_decode_kernel(m, rc == ELB_OK);
    if (rc == ELB_OK) rc = rc_k;
    if (tp) {
        bool all = false;
        const int rc_a = tp_agree(m->comm, rc == ELB_OK, m->stream, &all);
        if (rc != ELB_OK) return rc;
        if (rc_a != ELB_OK) return rc_a;
        if (!all) return fail(ELB_ERR_STATE, other);
    } else if (rc != ELB_OK) {
        return rc;
    }
    m->pending.clear();
    m->pending.shrink_to_fit();
    m->shard_store.clear();
    m->shard_store.shrink_to_fit();
    m->finalized = true;
    return ELB_OK;
}

namespace { struct TopOut; }
int model_eval_impl(Model* m, const int32_t* tokens, int n, int pos0, float* logits, const TopOut* top);

int model_eval_top(Model* m, const int32_t* tokens, int n, int pos0, int k, int32_t* ids, float* vals, double* lse,
                   const uint32_t* allowed) {
    if (!ids || !vals || !lse) return fail(ELB_ERR_INVALID, "eval_top: null argument");
    if (k < 1 || k > TOP_MAXK || (m && k > m->cfg.n_vocab)) return fail(ELB_ERR_INVALID, "eval_top: k must be between 1 and 64 (and at most n_vocab)");
    const TopOut top{k, ids, vals, lse, allowed};
    return model_eval_impl(m, tokens, n, pos0, nullptr, &top);
}

int model_eval(Model* m, const int32_t* tokens, int n, int pos0, float* logits) { return model_eval_impl(m, tokens, n, pos0, logits, nullptr); }

int model_eval_impl(Model* m, const int32_t* tokens, int n, int pos0, float* logits, const TopOut* top) {
    if (!m || !tokens) return fail(ELB_ERR_INVALID, "eval: null argument");
    if (!m->finalized) return fail(ELB_ERR_STATE, "eval: model not finalized");
    if (n <= 0) return fail(ELB_ERR_INVALID, "eval: empty token sequence");
    if (pos0 < 0 || int64_t(pos0) + n > m->n_ctx) return fail(ELB_ERR_RANGE, "eval: context window full");
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= m->cfg.n_vocab) return fail(ELB_ERR_RANGE, "eval: token id out of range");
    ELB_CUDA(cudaSetDevice(m->device));
    m->last_ms = 0.f;
    const int64_t before = m->launches;
    for (int done = 0; done < n;) {
        const int b = std::min(m->max_batch, n - done);
        const bool last = done + b == n;
        ELB_TRY(chunk(m, tokens + done, b, pos0 + done, last ? logits : nullptr, last ? top : nullptr));
        done += b;
    }
    m->last_launches = m->launches - before;
    return ELB_OK;
}

// Rows of several sequences in one pass: the prompt-chunk path with per-row sequence and position (body_prefill, mixed)
// or, when all rows belong to one sequence at consecutive positions, exactly the prompt-chunk path on that sequence's
// cache. The head runs over the wanted rows only.
namespace { struct TopRows { int k; int32_t* ids; float* vals; double* lse; }; }
static int eval_batch_impl(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want,
                           float* logits, const TopRows* top);

int model_eval_batch(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want,
                     float* logits) {
    return eval_batch_impl(m, n, tokens, seq, pos, want, logits, nullptr);
}

// the wanted rows' logits reduced on the device: ids[r][k], vals[r][k], lse[r] for wanted row r (in row order)
int model_eval_batch_top(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want, int k,
                         int32_t* ids, float* vals, double* lse) {
    if (!ids || !vals || !lse) return fail(ELB_ERR_INVALID, "eval_batch_top: null argument");
    if (k < 1 || k > TOP_MAXK || (m && k > m->cfg.n_vocab)) return fail(ELB_ERR_INVALID, "eval_batch_top: k must be between 1 and 64 (and at most n_vocab)");
    const TopRows top{k, ids, vals, lse};
    return eval_batch_impl(m, n, tokens, seq, pos, want, nullptr, &top);
}

static int eval_batch_impl(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want,
                           float* logits, const TopRows* top) {
    if (!m || !tokens || !seq || !pos) return fail(ELB_ERR_INVALID, "eval_batch: null argument");
    if (!m->finalized) return fail(ELB_ERR_STATE, "eval_batch: model not finalized");
    if (n <= 0) return fail(ELB_ERR_INVALID, "eval_batch: empty batch");
    if (n > m->max_batch) return fail(ELB_ERR_RANGE, "eval_batch: more rows than max_batch");
    bool uniform = true;
    std::vector<int> rows;  // wanted rows
    for (int i = 0; i < n; ++i) {
        if (tokens[i] < 0 || tokens[i] >= m->cfg.n_vocab) return fail(ELB_ERR_RANGE, "eval_batch: token id out of range");
        if (seq[i] < 0 || seq[i] >= m->n_seq) return fail(ELB_ERR_RANGE, "eval_batch: sequence index out of range");
        if (pos[i] < 0 || pos[i] >= m->n_ctx) return fail(ELB_ERR_RANGE, "eval_batch: context window full");
        uniform = uniform && seq[i] == seq[0] && pos[i] == pos[0] + i;
        if ((logits || top) && (!want || want[i])) rows.push_back(i);
    }
    for (int i = 0; i < n; ++i)  // rows of one sequence: increasing, consecutive positions
        for (int j = i + 1; j < n; ++j)
            if (seq[j] == seq[i]) {
                if (pos[j] != pos[i] + 1) return fail(ELB_ERR_INVALID, "eval_batch: rows of a sequence must be at consecutive positions");
                break;
            }
    if (!uniform && m->n_seq == 1) return fail(ELB_ERR_INVALID, "eval_batch: one sequence needs consecutive positions");
    if (int(rows.size()) > m->n_seq) return fail(ELB_ERR_UNSUPPORTED, "eval_batch: more wanted rows than sequences");
    if (m->tp.size > 1 && rows.size() > 1) return fail(ELB_ERR_UNSUPPORTED, "eval_batch: one wanted row under tensor parallelism");
    ELB_CUDA(cudaSetDevice(m->device));
    const int E = m->cfg.n_embd;
    const int64_t V = m->cfg.n_vocab, before = m->launches;
    std::memcpy(m->tokens_host, tokens, size_t(n) * sizeof(int32_t));
    ELB_CUDA(cudaMemcpyAsync(m->tokens_dev, m->tokens_host, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice, m->stream));
    if (!uniform) {
        // (pageable source: the copies are staged by the runtime before the call returns)
        ELB_CUDA(cudaMemcpyAsync(m->seq_dev, seq, size_t(n) * sizeof(int), cudaMemcpyHostToDevice, m->stream));
        ELB_CUDA(cudaMemcpyAsync(m->posv_dev, pos, size_t(n) * sizeof(int), cudaMemcpyHostToDevice, m->stream));
    }
    ELB_CUDA(cudaEventRecord(m->ev0, m->stream));
    ELB_TRY(launch_gather_rows(m->embd, m->tokens_dev, n, m->x, m->stream));
    ++m->launches;
    ELB_TRY(body_prefill(m, n, pos[0], seq[0], !uniform));
    m->last_rows = n;
    float* out_dev = nullptr;
    if (rows.size() == 1) {
        ELB_TRY(head_logits(m, m->x + size_t(rows[0]) * E));
        out_dev = m->logits;
    } else if (rows.size() > 1) {
        float* xh = m->x;
        if (int(rows.size()) != n) {  // compact the wanted rows (act is free after the last layer)
            xh = m->act;
            for (size_t r = 0; r < rows.size(); ++r)
                ELB_CUDA(cudaMemcpyAsync(xh + r * E, m->x + size_t(rows[r]) * E, size_t(E) * sizeof(float), cudaMemcpyDeviceToDevice, m->stream));
        }
        const int R = int(rows.size());
        if (m->head->type != ELB_F16 && !m->head->planes && !gemm_f16_tc_usable(m->head, R)) {  // no digit planes: row by row
            for (int r = 0; r < R; ++r) {
                ELB_TRY(prep_limbs_launch(xh + size_t(r) * E, E, m->output_norm, m->cfg.eps, 4, m->dlimbs[0], m->dinv, false, m->stream));
                ++m->launches;
                ELB_TRY(gemv(m, m->head, ActIn{m->dlimbs[0], m->dinv, xh + size_t(r) * E, m->output_norm}, m->logits_rows + size_t(r) * V,
                             nullptr, EPI_STORE, PostOp{}));
            }
        } else {
            ELB_TRY(split_tokens(m, xh, E, E, 4, m->output_norm, R, m->head->type != ELB_F16 && !gemm_f16_tc_usable(m->head, R)));
            ELB_TRY(linear_tokens(m, m->head, xh, E, m->output_norm, R, m->logits_rows, V, nullptr, EPI_STORE, 4));
        }
        out_dev = m->logits_rows;
    }
    if (out_dev && top) {  // k best tokens and the log-sum-exp of every wanted row, on the device
        ELB_TRY(logits_top_rows_launch(out_dev, int(V), V, int(rows.size()), top->k, m->top_rows_dev, m->stream));
        ++m->launches;
    }
    ELB_CUDA(cudaEventRecord(m->ev1, m->stream));
    if (out_dev && top) ELB_CUDA(cudaMemcpyAsync(m->top_rows_host, m->top_rows_dev, rows.size() * TOP_BYTES, cudaMemcpyDeviceToHost, m->stream));
    else if (out_dev) ELB_CUDA(cudaMemcpyAsync(logits, out_dev, rows.size() * size_t(V) * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
    ELB_CUDA(cudaStreamSynchronize(m->stream));
    ELB_TRY(gemm_tc_check());
    ELB_TRY(gemm_f16_tc_check());
    if (out_dev && top)
        for (size_t r = 0; r < rows.size(); ++r) {  // layout per row: lse (double), then k ids, then k logits
            const uint8_t* src = m->top_rows_host + r * TOP_BYTES;
            std::memcpy(top->lse + r, src, sizeof(double));
            std::memcpy(top->ids + r * top->k, src + 8, size_t(top->k) * sizeof(int32_t));
            std::memcpy(top->vals + r * top->k, src + 8 + 4 * TOP_MAXK, size_t(top->k) * sizeof(float));
        }
    ELB_CUDA(cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    m->last_launches = m->launches - before;
    return ELB_OK;
}

// n single-token steps at positions pos0.. enqueued back to back without reading logits back (the tg loop of the
// reference's bench command, src/main.cpp:639, minus its per-token host round trip); device time of the whole run.
int model_eval_steps(Model* m, const int32_t* tokens, int n, int pos0, float* device_ms) {
    if (!m || !tokens || !device_ms) return fail(ELB_ERR_INVALID, "eval_steps: null argument");
    if (!m->finalized) return fail(ELB_ERR_STATE, "eval_steps: model not finalized");
    if (n <= 0) return fail(ELB_ERR_INVALID, "eval_steps: empty token sequence");
    if (pos0 < 0 || int64_t(pos0) + n > m->n_ctx) return fail(ELB_ERR_RANGE, "eval_steps: context window full");
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= m->cfg.n_vocab) return fail(ELB_ERR_RANGE, "eval_steps: token id out of range");
    ELB_CUDA(cudaSetDevice(m->device));
    int32_t* pin = nullptr;  // [n] tokens, [n] positions, then the control words; pinned so that the copies stay asynchronous
    ELB_CUDA(cudaMallocHost(&pin, (size_t(2) * n + 4) * sizeof(int32_t)));
    for (int i = 0; i < n; ++i) { pin[i] = tokens[i]; pin[n + i] = pos0 + i; }
    int32_t* ctl = pin + 2 * n;
    ctl[0] = 0; ctl[1] = 1; ctl[2] = 0; ctl[3] = 0;  // {index 0, advance} to start a batch, {index 0, stay} to end it
    const int64_t before = m->launches;
    int rc = ELB_OK;
    cudaEventRecord(m->ev0, m->stream);
    if (m->use_mega) {
        // the persistent kernel walks the token / position arrays by itself: one upload per batch of steps
        for (int done = 0; done < n && rc == ELB_OK; done += m->max_batch) {
            const int b = std::min(m->max_batch, n - done);
            cudaMemcpyAsync(m->tokens_dev, pin + done, size_t(b) * sizeof(int32_t), cudaMemcpyHostToDevice, m->stream);
            cudaMemcpyAsync(m->pos_steps, pin + n + done, size_t(b) * sizeof(int), cudaMemcpyHostToDevice, m->stream);
            cudaMemcpyAsync(m->dk.ctl, ctl, 2 * sizeof(unsigned), cudaMemcpyHostToDevice, m->stream);
            for (int i = 0; i < b && rc == ELB_OK; ++i) rc = enqueue_decode_step(m);
        }
        cudaMemcpyAsync(m->dk.ctl, ctl + 2, 2 * sizeof(unsigned), cudaMemcpyHostToDevice, m->stream);
    } else {
        for (int i = 0; i < n && rc == ELB_OK; ++i) {
            cudaMemcpyAsync(m->tokens_dev, pin + i, sizeof(int32_t), cudaMemcpyHostToDevice, m->stream);
            cudaMemcpyAsync(m->pos_dev, pin + n + i, sizeof(int), cudaMemcpyHostToDevice, m->stream);
            rc = enqueue_decode_step(m);
        }
    }
    cudaEventRecord(m->ev1, m->stream);
    const cudaError_t e = cudaStreamSynchronize(m->stream);
    cudaFreeHost(pin);
    if (rc != ELB_OK) return rc;
    ELB_CUDA(e);
    if (m->err_host && *m->err_host) return fail(ELB_ERR_CUDA, "decode kernel: a grid barrier wait ran out");
    if ((m->tpr && *m->tpr->err_host) || (m->tprows && *m->tprows->err_host))
        return fail(ELB_ERR_CUDA, "tensor parallel: a peer did not arrive at an all-reduce in time");
    ELB_CUDA(cudaEventElapsedTime(device_ms, m->ev0, m->ev1));
    m->last_ms = *device_ms;
    m->last_launches = m->launches - before;
    if (m->use_mega && m->dk.prof) {  // diagnostics: phase times of the last step, CTA 0, averaged over the layers
        std::vector<unsigned long long> t(size_t(m->cfg.n_layer) * 32);
        cudaMemcpy(t.data(), m->dk.prof, t.size() * 8, cudaMemcpyDeviceToHost);
        static const char* names[15] = {"", "convert qkv", "matvec qkv", "barrier", "attention", "barrier", "convert wo", "matvec wo", "barrier", "convert gu", "matvec gu", "barrier", "convert down", "matvec down", "barrier"};
        double layer_total = 0;
        for (int ev = 1; ev < 15; ++ev) {
            double sum = 0;
            for (int l = 0; l < m->cfg.n_layer; ++l) sum += double(t[size_t(l) * 32 + ev] - t[size_t(l) * 32 + ev - 1]);
            std::fprintf(stderr, "[dk prof] %-13s %7.2f us\n", names[ev], sum / m->cfg.n_layer / 1000.0);
            layer_total += sum / m->cfg.n_layer / 1000.0;
        }
        std::fprintf(stderr, "[dk prof] layer total   %7.2f us\n", layer_total);
        if (m->dk.prof_cta) {  // every CTA's arrival at and release from the five barriers of one layer
            std::vector<unsigned long long> a(size_t(m->dk_grid) * 16);
            cudaMemcpy(a.data(), m->dk.prof_cta, a.size() * 8, cudaMemcpyDeviceToHost);
            static const char* bn[5] = {"after q|k|v", "after attention", "after attn_output", "after gate|up", "after ffn_down"};
            for (int b = 0; b < 5; ++b) {
                unsigned long long first = ~0ull, last = 0, rel_first = ~0ull, rel_last = 0;
                int who = 0;
                for (int cta = 0; cta < m->dk_grid; ++cta) {
                    const unsigned long long arr = a[size_t(cta) * 16 + 2 * b], rel = a[size_t(cta) * 16 + 2 * b + 1];
                    if (arr < first) first = arr;
                    if (arr > last) { last = arr; who = cta; }
                    if (rel < rel_first) rel_first = rel;
                    if (rel > rel_last) rel_last = rel;
                }
                std::fprintf(stderr, "[dk prof] barrier %-18s arrivals spread over %6.2f us (last: CTA %d), first release %5.2f us and last release %5.2f us after the last arrival\n",
                             bn[b], (last - first) / 1000.0, who, (double(rel_first) - double(last)) / 1000.0, (double(rel_last) - double(last)) / 1000.0);
            }
        }
    }
    m->last_rows = 1;
    return ELB_OK;
}

int model_stats(const Model* m, float* ms, int64_t* launches) {
    if (!m) return fail(ELB_ERR_INVALID, "stats: null model");
    if (ms) *ms = m->last_ms;
    if (launches) *launches = m->last_launches;
    return ELB_OK;
}

int model_hidden(Model* m, float* out) {
    if (!m || !out || !m->finalized) return fail(ELB_ERR_STATE, "hidden: model not ready");
    ELB_CUDA(cudaMemcpy(out, m->x + size_t(m->last_rows - 1) * m->cfg.n_embd, size_t(m->cfg.n_embd) * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

int model_config(const Model* m, elb_config* out) {
    if (!m || !out) return fail(ELB_ERR_INVALID, "config: null argument");
    *out = m->cfg;
    return ELB_OK;
}
size_t model_weight_bytes(const Model* m) { return m->weight_bytes; }
size_t model_kv_bytes_per_token(const Model* m) { return size_t(2) * m->cfg.n_layer * m->HKV * 128 * sizeof(float); }
int model_device(const Model* m) { return m->device; }

}  // namespace elb
