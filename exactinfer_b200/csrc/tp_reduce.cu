// All-reduce of one activation vector across the tensor-parallel ranks through peer memory, fused with what follows it
// in the decode chain: the new residual stream and its (RMSNorm +) limb split for the next matvec.
//
// A single-token all-reduce moves 10-20 KB: its cost is latency, not bandwidth. One kernel (one CTA) per rank:
//   1. push: the rank's partial sums are stored into slot [parity][rank] of EVERY rank's buffer (plain peer stores
//      over NVLink), then a system-scope release store raises flag [parity][rank] on every rank to the sequence number;
//   2. wait (bounded) until all `size` local flags carry the sequence number;
//   3. sum the slots in rank order - the same order and the same values on every rank, so all ranks hold bit-identical
//      results - write x, and run the limb split on the values still in registers.
// Two parities: a rank can be at most one reduction ahead of a peer (it needs the peer's flag of reduction s to
// finish s), so slot [s & 1] is never overwritten while a peer still reads reduction s - 2... s.
// The waits are bounded: a rank that never arrives raises the error word; the kernel still returns.
#include <algorithm>

#include "common.cuh"
#include "split.cuh"

namespace elb {

namespace {

constexpr unsigned TPR_SPIN_LIMIT = 1u << 24;  // x ~100 ns: about two seconds
constexpr size_t TPR_FLAG_BYTES = 256;  // flag words [2 parities][8 ranks], padded

struct TprParams {
    float* slots[8];      // rank p's slot area as mapped here
    unsigned* flags[8];   // rank p's flag words as mapped here
    int rank, size, n_max, n;
    const float* part;
    float* x;
    const float* norm_w;
    float eps;
    int nl;
    int8_t* limbs;
    float* inv_scale;
    unsigned* seq;
    int* err;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(SPLIT_THREADS) k_tp_reduce_split(const TprParams p) {
    __shared__ double red8[SPLIT_WARPS];
    __shared__ int s_dead;
    const int tid = threadIdx.x;
    const unsigned s = *p.seq, epoch = s + 1;
    const int par = int(s & 1u);
    if (tid == 0) s_dead = 0;
    // 1. push this rank's partial sums to every other rank (its own stay in registers)
    float4 mine[SPLIT_V4];
#pragma unroll
    for (int j = 0; j < SPLIT_V4; ++j) {
        const int idx = (j * SPLIT_THREADS + tid) * 4;
        mine[j] = idx < p.n ? __ldcg(reinterpret_cast<const float4*>(p.part + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const size_t my_slot = (size_t(par) * p.size + p.rank) * p.n_max;
    for (int q = 0; q < p.size; ++q) {
        const int peer = (p.rank + 1 + q) % p.size;  // spread the first stores over the links
        if (peer == p.rank) continue;
#pragma unroll
        for (int j = 0; j < SPLIT_V4; ++j) {
            const int idx = (j * SPLIT_THREADS + tid) * 4;
            if (idx < p.n) *reinterpret_cast<float4*>(p.slots[peer] + my_slot + idx) = mine[j];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.size && tid != p.rank) st_release_sys(p.flags[tid] + par * 8 + p.rank, epoch);
    // 2. wait for every peer's flag on this rank
    if (tid < p.size && tid != p.rank) {
        const unsigned* f = p.flags[p.rank] + par * 8 + tid;
        unsigned it = 0;
        while (ld_acquire_sys(f) != epoch) {
            if (++it > TPR_SPIN_LIMIT) {
                s_dead = 1;
                atomicExch(p.err, 1);
                break;
            }
            if (it > 64) __nanosleep(100);
        }
    }
    __syncthreads();
    // 3. sum in rank order, write x, split
    float4 v[SPLIT_V4];
#pragma unroll
    for (int j = 0; j < SPLIT_V4; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!s_dead) {
        for (int r = 0; r < p.size; ++r) {
            const float* src = p.slots[p.rank] + (size_t(par) * p.size + r) * p.n_max;
#pragma unroll
            for (int j = 0; j < SPLIT_V4; ++j) {
                const int idx = (j * SPLIT_THREADS + tid) * 4;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < p.n) a = r == p.rank ? mine[j] : __ldcg(reinterpret_cast<const float4*>(src + idx));
                if (r == 0) v[j] = a;
                else { v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w; }
            }
        }
#pragma unroll
        for (int j = 0; j < SPLIT_V4; ++j) {
            const int idx = (j * SPLIT_THREADS + tid) * 4;
            if (idx < p.n) *reinterpret_cast<float4*>(p.x + idx) = v[j];
        }
    }
    if (p.limbs) {
        const int k = block_split_values(v, p.n, p.norm_w, p.eps, p.nl, p.limbs, red8);
        if (tid == 0) *p.inv_scale = k <= 126 ? __int_as_float((127 - k) << 23) : ldexpf(1.0f, -k);
    }
    if (tid == 0) *p.seq = epoch;
}

// ---------------------------------------------------------------- a few rows at once (batched steps, short prompt chunks)

// All-reduce of up to n_max floats (a batch of 2..16 activation rows: 20-330 KB) without flags, fences or barriers: every
// value travels to the other ranks as one 8-byte word {value, tag}, tag = number of this reduction (never zero, never
// repeated), and an 8-byte store is delivered whole, so a reader that sees the tag has the value. Every thread owns a
// few pairs of values: it stores them into this rank's slot on every peer, then reads the same positions of every
// rank's slot on its own GPU (polling, bounded, until the tag is there) and adds them in rank order - the same sums in
// the same order on all ranks. Two sets of slots in turn: a rank finishes reduction k only with every peer's data of
// k, so by the time a peer's stores of k + 2 arrive it is done reading k.
constexpr unsigned TPR_ROWS_SPIN = 1u << 22;

struct TprRowsParams {
    uint2* slots[8];  // rank q's slots as mapped here: [2 sets][size][n_max]
    int rank, size, set;
    size_t n_max, n;  // n even
    const float* in;
    float* out;
    unsigned tag;
    int* err;
};

__global__ void __launch_bounds__(256) k_tp_rows_allreduce(const TprRowsParams p) {
    const size_t pairs = p.n / 2, stride = size_t(gridDim.x) * blockDim.x, first = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t mine = (size_t(p.set) * p.size + p.rank) * p.n_max;
    for (size_t i = first; i < pairs; i += stride) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(p.in) + i);
        const uint2 w0 = make_uint2(__float_as_uint(v.x), p.tag), w1 = make_uint2(__float_as_uint(v.y), p.tag);
        for (int q = 1; q < p.size; ++q) {
            uint2* dst = p.slots[(p.rank + q) % p.size] + mine + 2 * i;
            dst[0] = w0;
            dst[1] = w1;
        }
    }
    bool dead = false;
    for (size_t i = first; i < pairs; i += stride) {
        float2 acc = make_float2(0.f, 0.f);
        for (int r = 0; r < p.size; ++r) {
            float2 a;
            if (r == p.rank) {
                a = __ldcg(reinterpret_cast<const float2*>(p.in) + i);
            } else {
                const uint2* src = p.slots[p.rank] + (size_t(p.set) * p.size + r) * p.n_max + 2 * i;
                uint4 w;
                unsigned it = 0;
                while (true) {
                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
                    if ((w.y == p.tag && w.w == p.tag) || dead) break;
                    if (++it > TPR_ROWS_SPIN) {  // a peer never sent: report, and stop waiting for anything else
                        dead = true;
                        atomicExch(p.err, 1);
                        break;
                    }
                    if (it > 64) __nanosleep(100);
                }
                a = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
            }
            if (r == 0) acc = a;
            else { acc.x = __fadd_rn(acc.x, a.x); acc.y = __fadd_rn(acc.y, a.y); }
        }
        reinterpret_cast<float2*>(p.out)[i] = acc;
    }
}

}  // namespace

int tp_rows_create(TpComm* c, int device, int rank, int size, size_t n_max, cudaStream_t s, TpRows** out, bool caller_ok) {
    *out = nullptr;
    if (size < 2 || size > 8 || n_max == 0) return ELB_OK;
    auto* r = new TpRows;
    r->rank = rank; r->size = size; r->n_max = (n_max + 1) / 2 * 2;
    bool ok = false;
    bool local_ok = caller_ok && cudaSetDevice(device) == cudaSuccess &&
                    cudaHostAlloc(&r->err_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess;
    if (local_ok) {
        *r->err_host = 0;
        local_ok = cudaHostGetDevicePointer(&r->err_dev, r->err_host, 0) == cudaSuccess;
    }
    if (!local_ok) cudaGetLastError();
    const int rc = tp_peer_alloc(c, device, size_t(2) * size * r->n_max * sizeof(uint2), s, &r->buf, &ok, local_ok);
    if (rc != ELB_OK || !ok) {  // every rank gets here together: all keep to NCCL
        tp_rows_destroy(r);
        if (rc != ELB_OK) return rc;
        return local_ok || !caller_ok ? ELB_OK : fail(ELB_ERR_MEMORY, "tp_rows: out of memory");
    }
    *out = r;
    return ELB_OK;
}

void tp_rows_destroy(TpRows* r) {
    if (!r) return;
    tp_peer_free(&r->buf, r->rank);
    if (r->err_host) cudaFreeHost(r->err_host);
    delete r;
}

int tp_rows_all_reduce(TpRows* r, const float* in, float* out, size_t n, cudaStream_t s) {
    if (!r || !in || !out || n == 0 || n > r->n_max || n % 2 || in == out) return fail(ELB_ERR_INVALID, "tp_rows: bad argument");
    TprRowsParams p{};
    for (int q = 0; q < r->size; ++q) p.slots[q] = static_cast<uint2*>(r->buf.peer[q]);
    p.rank = r->rank; p.size = r->size; p.n_max = r->n_max; p.n = n; p.in = in; p.out = out; p.err = r->err_dev;
    p.tag = ++r->count;
    if (p.tag == 0) p.tag = ++r->count;  // (after 2^32 reductions: zero is what an unwritten slot holds)
    p.set = int(r->count & 1u);
    const size_t pairs = n / 2;
    const int grid = int(std::min<size_t>((pairs + 255) / 256, 148));
    k_tp_rows_allreduce<<<grid, 256, 0, s>>>(p);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

namespace {

}  // namespace

int tp_reduce_create(TpComm* c, int device, int rank, int size, int n_max, cudaStream_t s, TpReduce** out) {
    *out = nullptr;
    if (size < 2 || size > 8 || n_max > SPLIT_V4 * 4 * SPLIT_THREADS || n_max % 4) return ELB_OK;
    auto* r = new TpReduce;
    r->rank = rank; r->size = size; r->n_max = n_max;
    bool ok = false;
    const size_t bytes = TPR_FLAG_BYTES + size_t(2) * size * n_max * sizeof(float);
    // the local pieces first, so that a rank that cannot have them says so IN the collectives of tp_peer_alloc
    // instead of leaving before them
    bool local_ok = cudaSetDevice(device) == cudaSuccess && cudaMalloc(&r->seq, sizeof(unsigned)) == cudaSuccess &&
                    cudaMemset(r->seq, 0, sizeof(unsigned)) == cudaSuccess &&
                    cudaHostAlloc(&r->err_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess;
    if (local_ok) {
        *r->err_host = 0;
        local_ok = cudaHostGetDevicePointer(&r->err_dev, r->err_host, 0) == cudaSuccess;
    }
    if (!local_ok) cudaGetLastError();
    const int rc = tp_peer_alloc(c, device, bytes, s, &r->buf, &ok, local_ok);
    if (rc != ELB_OK || !ok) {  // every rank gets here together: all keep to NCCL, the rank that failed reports why
        tp_reduce_destroy(r);
        if (rc != ELB_OK) return rc;
        return local_ok ? ELB_OK : fail(ELB_ERR_MEMORY, "tp_reduce: out of memory");
    }
    *out = r;
    return ELB_OK;
}

void tp_reduce_destroy(TpReduce* r) {
    if (!r) return;
    tp_peer_free(&r->buf, r->rank);
    cudaFree(r->seq);
    if (r->err_host) cudaFreeHost(r->err_host);
    delete r;
}

int tp_reduce_split_launch(TpReduce* r, const float* part, float* x, int n, const float* norm_w, float eps, int nl,
                           int8_t* limbs, float* inv_scale, cudaStream_t s) {
    if (!r || !part || !x || n <= 0 || n > r->n_max || n % 4) return fail(ELB_ERR_INVALID, "tp_reduce: bad argument");
    if (limbs && (n % 256 || !inv_scale)) return fail(ELB_ERR_INVALID, "tp_reduce: the split needs a multiple of 256 values");
    TprParams p{};
    for (int q = 0; q < r->size; ++q) {
        p.flags[q] = reinterpret_cast<unsigned*>(r->buf.peer[q]);
        p.slots[q] = reinterpret_cast<float*>(static_cast<uint8_t*>(r->buf.peer[q]) + TPR_FLAG_BYTES);
    }
    p.rank = r->rank; p.size = r->size; p.n_max = r->n_max; p.n = n;
    p.part = part; p.x = x; p.norm_w = norm_w; p.eps = eps; p.nl = nl; p.limbs = limbs; p.inv_scale = inv_scale;
    p.seq = r->seq; p.err = r->err_dev;
    k_tp_reduce_split<<<1, SPLIT_THREADS, 0, s>>>(p);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
