// Tensor parallelism over the GPUs of one box: how each tensor of the model is cut for rank r of N (host code, no
// device needed), and the NCCL communicator the forward pass calls for its two all-reduces per layer.
// The reference runs on one GPU; the cut is the usual column/row split of its layer (CpuModel::forward,
// src/model.cpp:157-234), which keeps every head and every SwiGLU element on one rank:
//   attn_q/k/v   rows of whole heads      H/N query heads, HKV/N key-value heads per rank
//   attn_output  columns of those heads   partial sums -> all-reduce
//   ffn_gate/up  rows [f0, f1)            f0, f1 multiples of 256 (uneven when F/256 is not a multiple of N)
//   ffn_down     columns [f0, f1)         partial sums -> all-reduce
//   output head  rows [v0, v1)            whole 16-row tiles; logits are all-gathered
//   norms, token embedding               replicated
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace elb {

int tp_dims(const elb_config& c, int rank, int size, TpDims* d) {
    if (size < 1 || rank < 0 || rank >= size) return fail(ELB_ERR_INVALID, "tensor parallel: rank outside [0, size)");
    if (c.n_head_kv % size || c.n_head % size)
        return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: the number of ranks must divide the KV and query head counts");
    d->rank = rank; d->size = size;
    d->H = c.n_head / size;
    d->HKV = c.n_head_kv / size;
    if (size > 1 && (int64_t(d->H) * c.head_dim) % 256)
        return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: query heads per rank x head_dim must be a multiple of 256");
    if (size > 1 && c.n_ff % 256) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: n_ff must be a multiple of 256");
    if (size == 1) {
        d->f0 = 0; d->f1 = c.n_ff;
    } else {
        const int64_t nb = c.n_ff / 256;
        if (nb < size) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: fewer 256-blocks in n_ff than ranks");
        d->f0 = nb * rank / size * 256;
        d->f1 = nb * (rank + 1) / size * 256;
    }
    const int64_t tiles = (int64_t(c.n_vocab) + 15) / 16;
    if (tiles < size) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: vocabulary smaller than 16 rows per rank");
    d->vchunk = (tiles + size - 1) / size * 16;
    d->v0 = std::min<int64_t>(d->vchunk * rank, c.n_vocab);
    d->v1 = std::min<int64_t>(d->vchunk * (rank + 1), c.n_vocab);
    if (d->v1 <= d->v0) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: a rank would own no vocabulary rows");
    return ELB_OK;
}

namespace {

// bytes of `cols` consecutive values of a row, starting at a multiple of the type's block; -1 when not block aligned
int64_t col_bytes(int type, int64_t cols) {
    switch (type) {
        case ELB_F32: return cols * 4;
        case ELB_F16: return cols * 2;
        case ELB_Q8_0: return cols % QK8_0 ? -1 : cols / QK8_0 * Q8_0_BYTES;
        case ELB_Q4_K: return cols % QK_K ? -1 : cols / QK_K * Q4_K_BYTES;
        case ELB_Q6_K: return cols % QK_K ? -1 : cols / QK_K * Q6_K_BYTES;
        default: return -1;
    }
}

}  // namespace

int tp_shard_shape(const elb_config& c, const TpDims& d, int role, int type, int64_t rows, int64_t n, TpShard* s) {
    s->row0 = 0; s->rows = rows; s->col0 = 0; s->n = n;
    const int64_t hd = c.head_dim;
    switch (role) {
        case ELB_WQ: s->row0 = int64_t(d.rank) * d.H * hd; s->rows = int64_t(d.H) * hd; break;
        case ELB_WK:
        case ELB_WV: s->row0 = int64_t(d.rank) * d.HKV * hd; s->rows = int64_t(d.HKV) * hd; break;
        case ELB_WO: s->col0 = int64_t(d.rank) * d.H * hd; s->n = int64_t(d.H) * hd; break;
        case ELB_GATE:
        case ELB_UP: s->row0 = d.f0; s->rows = d.f1 - d.f0; break;
        case ELB_DOWN: s->col0 = d.f0; s->n = d.f1 - d.f0; break;
        case ELB_OUTPUT: s->row0 = d.v0; s->rows = d.v1 - d.v0; break;
        default: break;  // norms and the token embedding are replicated
    }
    if (s->row0 + s->rows > rows || s->col0 + s->n > n) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: tensor smaller than its shard");
    const int64_t rb = col_bytes(type, s->n), full = col_bytes(type, n), off = col_bytes(type, s->col0);
    if (rb < 0 || full < 0 || off < 0) return fail(ELB_ERR_UNSUPPORTED, "tensor parallel: column cut not on a block boundary of this type");
    s->row_bytes = rb; s->src_row_bytes = full; s->src_col_off = off;
    s->nbytes = size_t(rb) * size_t(s->rows);
    s->contiguous = s->n == n;
    return ELB_OK;
}

int tp_shard_copy(const TpShard& s, const uint8_t* src, size_t src_bytes, uint8_t* dst) {
    if (!src || !dst) return fail(ELB_ERR_INVALID, "tensor parallel: null buffer");
    if (size_t(s.src_row_bytes) * size_t(s.row0 + s.rows) > src_bytes) return fail(ELB_ERR_INVALID, "tensor parallel: source tensor too short");
    for (int64_t r = 0; r < s.rows; ++r)
        std::memcpy(dst + size_t(r) * s.row_bytes, src + size_t(s.row0 + r) * s.src_row_bytes + s.src_col_off, size_t(s.row_bytes));
    return ELB_OK;
}

// ---------------------------------------------------------------- NCCL, resolved at run time
// The library is found with dlopen so that single-GPU users need no NCCL: a process that already loaded one (PyTorch
// brings its own) gets that copy, others the system's.
namespace {

struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string why;
};

Nccl* nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            n.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (n.handle) break;
        }
        if (!n.handle) { n.why = "NCCL not found (libnccl.so.2)"; return; }
        auto sym = [&](const char* s) { void* p = dlsym(n.handle, s); if (!p) n.why = std::string("NCCL lacks ") + s; return p; };
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
        n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(sym("ncclAllReduce"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
    });
    return &n;
}

int nccl_fail(Nccl* n, ncclResult_t r, const char* what) {
    return fail(ELB_ERR_CUDA, std::string(what) + ": " + (n->GetErrorString ? n->GetErrorString(r) : "NCCL error"));
}

}  // namespace

struct TpComm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1;
    // staging for the small set-up collectives (IPC handles, agreement flags), allocated with the communicator so that
    // a rank whose later allocations fail can still take part in them: [68 send][68 * 8 receive][16 flag]
    uint8_t* d_small = nullptr;
};
constexpr size_t TP_SMALL_RECV = 128, TP_SMALL_FLAG = 128 + 68 * 8 + 32, TP_SMALL_BYTES = TP_SMALL_FLAG + 16;

int tp_unique_id(void* id128) {
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
    if (!id128) return fail(ELB_ERR_INVALID, "tp_unique_id: null buffer");
    Nccl* n = nccl();
    if (!n->why.empty()) return fail(ELB_ERR_UNSUPPORTED, n->why);
    ncclUniqueId id;
    const ncclResult_t r = n->GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(n, r, "ncclGetUniqueId");
    std::memcpy(id128, &id, 128);
    return ELB_OK;
}

int tp_comm_create(int device, int rank, int size, const void* id128, TpComm** out) {
    if (!id128 || !out) return fail(ELB_ERR_INVALID, "tp_comm_create: null argument");
    Nccl* n = nccl();
    if (!n->why.empty()) return fail(ELB_ERR_UNSUPPORTED, n->why);
    ELB_CUDA(cudaSetDevice(device));
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    auto* c = new TpComm;
    c->rank = rank; c->size = size;
    const ncclResult_t r = n->CommInitRank(&c->comm, size, id, rank);
    if (r != ncclSuccess) { delete c; return nccl_fail(n, r, "ncclCommInitRank"); }
    if (cudaMalloc(&c->d_small, TP_SMALL_BYTES) != cudaSuccess) {
        cudaGetLastError();
        tp_comm_destroy(c);
        return fail(ELB_ERR_MEMORY, "tp_comm_create: out of device memory");
    }
    *out = c;
    return ELB_OK;
}

void tp_comm_destroy(TpComm* c) {
    if (!c) return;
    if (c->comm) nccl()->CommDestroy(c->comm);
    cudaFree(c->d_small);
    delete c;
}

int tp_all_reduce(TpComm* c, const float* in, float* out, size_t count, cudaStream_t s) {
    const ncclResult_t r = nccl()->AllReduce(in, out, count, ncclFloat, ncclSum, c->comm, s);
    return r == ncclSuccess ? ELB_OK : nccl_fail(nccl(), r, "ncclAllReduce");
}

int tp_all_gather(TpComm* c, const float* in, float* out, size_t count_per_rank, cudaStream_t s) {
    const ncclResult_t r = nccl()->AllGather(in, out, count_per_rank, ncclFloat, c->comm, s);
    return r == ncclSuccess ? ELB_OK : nccl_fail(nccl(), r, "ncclAllGather");
}


// ---------------------------------------------------------------- peer-visible buffers (one process per GPU)
// Every rank allocates `bytes` of device memory, zeroes it, and the ranks exchange CUDA IPC handles through the
// communicator; peer[r] is rank r's buffer as mapped into this process (peer[rank] = the local one). `ok` comes back
// false on every rank when any rank could not map a peer (the caller then keeps to NCCL).
int tp_peer_alloc(TpComm* c, int device, size_t bytes, cudaStream_t s, TpPeerBuf* out, bool* ok, bool local_ok) {
    *ok = false;
    *out = TpPeerBuf{};
    if (!c || c->size < 2 || c->size > 8) return ELB_OK;
    // A rank whose own part fails (out of memory, no IPC handle) does NOT return before the two collectives below: the
    // other ranks are on their way into them. It takes part with "failed" as its answer, and every rank sees it.
    int good = local_ok ? 1 : 0;
    if (cudaSetDevice(device) != cudaSuccess) good = 0;
    out->size = c->size;
    if (good && (cudaMalloc(&out->local, bytes) != cudaSuccess || cudaMemset(out->local, 0, bytes) != cudaSuccess)) good = 0;
    cudaIpcMemHandle_t mine{};
    if (good && cudaIpcGetMemHandle(&mine, out->local) != cudaSuccess) good = 0;
    if (!good) cudaGetLastError();
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle is 64 bytes");
    uint8_t *d_send = c->d_small, *d_recv = c->d_small + TP_SMALL_RECV;
    float* d_flag = reinterpret_cast<float*>(c->d_small + TP_SMALL_FLAG);
    uint8_t pack[68];
    std::memcpy(pack, &mine, 64);
    std::memcpy(pack + 64, &good, 4);
    std::vector<uint8_t> all(size_t(68) * c->size);
    int rc = ELB_OK;
    auto cleanup = [&](int code) { tp_peer_free(out, c->rank); return code; };
    // (a failing copy or collective here is a broken stream or communicator: nothing the other ranks could be told through)
    if (cudaMemcpyAsync(d_send, pack, 68, cudaMemcpyHostToDevice, s) != cudaSuccess) return cleanup(fail(ELB_ERR_CUDA, "tp_peer_alloc: staging copy failed"));
    ncclResult_t r = nccl()->AllGather(d_send, d_recv, 68, ncclInt8, c->comm, s);
    if (r != ncclSuccess) return cleanup(nccl_fail(nccl(), r, "ncclAllGather (peer handles)"));
    if (cudaMemcpyAsync(all.data(), d_recv, all.size(), cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return cleanup(fail(ELB_ERR_CUDA, "tp_peer_alloc: reading the handles failed"));
    for (int p = 0; p < c->size; ++p) {
        int g = 0;
        std::memcpy(&g, all.data() + size_t(p) * 68 + 64, 4);
        good &= g;
    }
    for (int p = 0; p < c->size && good; ++p) {
        if (p == c->rank) { out->peer[p] = out->local; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, all.data() + size_t(p) * 68, 64);
        if (cudaIpcOpenMemHandle(&out->peer[p], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            out->peer[p] = nullptr;
            good = 0;
        }
    }
    // every rank must take the same path: agree on the outcome
    float flag = good ? 0.f : 1.f;
    if (cudaMemcpyAsync(d_flag, &flag, 4, cudaMemcpyHostToDevice, s) != cudaSuccess) return cleanup(fail(ELB_ERR_CUDA, "tp_peer_alloc: staging copy failed"));
    r = nccl()->AllReduce(d_flag, d_flag, 1, ncclFloat, ncclSum, c->comm, s);
    if (r != ncclSuccess) return cleanup(nccl_fail(nccl(), r, "ncclAllReduce (peer mapping outcome)"));
    if (cudaMemcpyAsync(&flag, d_flag, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return cleanup(fail(ELB_ERR_CUDA, "tp_peer_alloc: reading the outcome failed"));
    *ok = flag == 0.f;
    if (!*ok) tp_peer_free(out, c->rank);
    return rc;
}

// true on every rank only when `mine` is true on every rank (collective; one rank: its own answer)
int tp_agree(TpComm* c, bool mine, cudaStream_t s, bool* all) {
    *all = mine;
    if (!c || c->size < 2) return ELB_OK;
    float flag = mine ? 0.f : 1.f, *d_flag = reinterpret_cast<float*>(c->d_small + TP_SMALL_FLAG);
    if (cudaMemcpyAsync(d_flag, &flag, sizeof(float), cudaMemcpyHostToDevice, s) != cudaSuccess) return fail(ELB_ERR_CUDA, "tp_agree: staging copy failed");
    const ncclResult_t r = nccl()->AllReduce(d_flag, d_flag, 1, ncclFloat, ncclSum, c->comm, s);
    if (r != ncclSuccess) return nccl_fail(nccl(), r, "ncclAllReduce (agreement)");
    if (cudaMemcpyAsync(&flag, d_flag, sizeof(float), cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return fail(ELB_ERR_CUDA, "tp_agree: reading the outcome failed");
    *all = flag == 0.f;
    return ELB_OK;
}

void tp_peer_free(TpPeerBuf* b, int rank) {
    if (!b) return;
    for (int p = 0; p < b->size; ++p)
        if (p != rank && b->peer[p]) cudaIpcCloseMemHandle(b->peer[p]);
    cudaFree(b->local);
    *b = TpPeerBuf{};
}

}  // namespace elb
