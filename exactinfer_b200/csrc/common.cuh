// Shared declarations of libelb: error handling, device helpers, and the tiled weight layouts.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/elb.h"

namespace elb {

// ---------------------------------------------------------------- errors (no exceptions cross the C ABI)
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define ELB_CUDA(expr)                                                                                         \
    do {                                                                                                       \
        cudaError_t e_ = (expr);                                                                               \
        if (e_ != cudaSuccess)                                                                                 \
            return ::elb::fail(ELB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));              \
    } while (0)

#define ELB_TRY(expr)                \
    do {                             \
        int rc_ = (expr);            \
        if (rc_ != ELB_OK) return rc_; \
    } while (0)

// ---------------------------------------------------------------- block formats (src/quant.h:20-41 of the reference)
constexpr int QK8_0 = 32, QK_K = 256;
constexpr int Q8_0_BYTES = 34, Q4_K_BYTES = 144, Q6_K_BYTES = 210;
constexpr int TILE_ROWS = 16;  // rows of one weight tile = M of mma.m16n8k*

// Tiled device layouts. A weight is cut into tiles of 16 consecutive rows; within a tile, "lane" means the
// lane of the warp that consumes it, lane = 4*g + t, which owns rows g and g+8 of the tile (the A-fragment rows
// of mma.m16n8k32/k16) and 8 (Q4_K, Q8_0) or 4 (Q6_K) consecutive k positions of each sub-block. The bytes of a
// tile are exactly the bytes of its 16 rows in the file, only permuted — nothing is widened or rounded.
//
// Q4_K, per (tile, 256-block): 2304 B = 16 * 144
//     [  0, 256)  headers: for g in 0..7: 16 B of row g (fp16 d, fp16 dmin, 12 packed scale bytes), 16 B of row g+8
//     [256,2304)  qs: for pair j in 0..3 (sub-blocks 2j low nibbles, 2j+1 high nibbles): lane * 16 B =
//                 row g bytes [32j+8t, +8) then row g+8 bytes [32j+8t, +8)
constexpr int Q4K_UNIT = 16 * Q4_K_BYTES;
// Q6_K, per (tile, 256-block): 3360 B = 16 * 210
//     [   0,  32)  fp16 d of rows g=0..7 interleaved as (row g, row g+8)
//     [  32, 288)  int8 scales: for g: 16 B of row g, 16 B of row g+8
//     [ 288,2336)  low nibbles: for quad c in 0..3 (sub-blocks 4c..4c+3): lane * 16 B = words i=0..3 (sub-block
//                  4c+i): byte j = value k=16(4c+i)+4t+j of row g in the low nibble, of row g+8 in the high nibble
//     [2336,3360)  high 2 bits: for quad c: lane * 8 B = word for row g, word for row g+8; in each word byte j
//                  holds, at bits 2i..2i+1, the top two bits of value k=16(4c+i)+4t+j
constexpr int Q6K_UNIT = 16 * Q6_K_BYTES;
// Q8_0, per (tile, group of 4 32-blocks): 2176 B = 16 * 4 * 34
//     [  0, 128)  fp16 d: for g: (row g blocks 0..3), (row g+8 blocks 0..3)  -> 16 B per g
//     [128,2176)  qs: for block i in 0..3: lane * 16 B = row g bytes [8t, +8) then row g+8 bytes [8t, +8)
constexpr int Q8_UNIT = 16 * 4 * Q8_0_BYTES;
constexpr int Q8_GROUP = 4;  // 32-blocks per unit (row length must be a multiple of 128)

struct Weight {
    int device = 0;
    int type = 0;          // ggml type id
    int64_t rows = 0;      // logical rows (2x the per-matrix rows for a gate|up pair)
    int64_t n = 0;         // row length
    int64_t tiles = 0;     // ceil(rows / 16)
    int64_t units_per_tile = 0;
    int unit_bytes = 0;
    bool pair = false;     // gate|up interleaved in 8-row groups
    bool view = false;     // rows of another weight: tiled memory is borrowed, not owned
    uint8_t* tiled = nullptr;  // tiled layout (quantized types) or plain row-major fp16 (F16)
    size_t tiled_bytes = 0;
    // digit planes for the tensor-core path: plane p holds digit p of the integer weight, row-major [rows16][n]
    int n_planes = 0;
    int8_t* planes = nullptr;  // [n_planes][tiles*16][n]
    __half* pl_d = nullptr;    // [tiles*16][n/blk] block scale d (blk = 256, Q8_0: 32)
    float* pl_dm = nullptr;    // Q4_K: [tiles*16][n/32] fl(dmin * m)
    // Q8_0 on the fp16 tensor-core path: the weight d * q (18 significant bits) as an exact sum of two fp16 values,
    // [2][tiles*16][n] (hi, then lo); present instead of the digit plane unless some d * q leaves the fp16 range
    __half* f16pair = nullptr;
    // scratch of the split-K matvec (per weight so that matvecs of different weights may overlap)
    float* part = nullptr;     // [grid][2][16]
    unsigned* counters = nullptr;  // [tiles]
    int max_grid = 0;
    // activation limbs for the operator-level entry points (the model keeps its own): [4][n] int8, then 2^-k
    int8_t* xlimbs = nullptr;
    float* xinv = nullptr;
};

// ---------------------------------------------------------------- device helpers
__device__ __forceinline__ float h2f_bits(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 6-bit scale / min of sub-block j from the 12 packed bytes (q4k_scale_min, src/quant.h:44-52 of the reference)
__host__ __device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, int& sc, int& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// exact int -> float for |v| <= 2^22 (adds 1.5*2^23 in the integer domain, subtracts it as a float)
__device__ __forceinline__ float i2f_small(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// mma.sync m16n8k32 / m16n8k16, A unsigned or signed 8-bit, B signed 8-bit, int32 accumulate (exact)
// Integer tensor-core products of one warp, C = A * B with a zero accumulator (the callers scale every product before
// they add it up, so there is nothing to accumulate into; passing the zeros as inputs spares four moves per MMA).
#define ELB_MMA_K32(NAME, TA)                                                                                          \
    __device__ __forceinline__ void NAME(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, \
                                         uint32_t b1) {                                                               \
        asm("mma.sync.aligned.m16n8k32.row.col.s32." TA ".s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};" \
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])                                                          \
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));                                           \
    }
#define ELB_MMA_K16(NAME, TA)                                                                                \
    __device__ __forceinline__ void NAME(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {              \
        asm("mma.sync.aligned.m16n8k16.row.col.s32." TA ".s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};" \
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])                                                \
            : "r"(a0), "r"(a1), "r"(b0), "r"(0));                                                            \
    }
ELB_MMA_K32(mma_u8s8_k32, "u8")
ELB_MMA_K32(mma_s8s8_k32, "s8")
ELB_MMA_K16(mma_u8s8_k16, "u8")
ELB_MMA_K16(mma_s8s8_k16, "s8")
#undef ELB_MMA_K32
#undef ELB_MMA_K16
// accumulating form: c += A * B
__device__ __forceinline__ void mma_s8s8_k32_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x * 2^k as two exact multiplications by powers of two (|k| can exceed the exponent range of one float);
// bit-identical to ldexpf(x, k) wherever the result is a normal float or zero, which covers every value that
// survives the rounding to an integer
struct Pow2 { float s1, s2; };
__device__ __forceinline__ Pow2 make_pow2(int k) {
    const int k1 = k >> 1, k2 = k - k1;
    return Pow2{__int_as_float((k1 + 127) << 23), __int_as_float((k2 + 127) << 23)};
}

// programmatic dependent launch: let the next kernel of the stream start its prologue / wait for the previous one
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------- host-side declarations shared between files
struct DeviceInfo {
    int sm_count = 0;
    size_t smem_optin = 0;
};
int device_info(int device, DeviceInfo* out);
// Raise a kernel's dynamic shared memory limit to at least `smem` bytes on the CURRENT device. The attribute is kept per
// device by the runtime, so what has been set is remembered per (kernel, device): any thread, any device, any order.
int ensure_dyn_smem(const void* kernel, size_t smem);

// weights.cu
int weight_create(int device, int type, int64_t rows_one, int64_t n, const void* bytes, size_t nbytes, int flags,
                  Weight** out);
void weight_destroy(Weight* w);
// rows [row0, row0 + rows) of `base` as a weight of its own (row0 a multiple of 16; not for gate|up pairs); the tiled
// memory stays owned by `base`, which must outlive the view. No digit planes.
int weight_view_rows(const Weight* base, int64_t row0, int64_t rows, Weight** out);
int get_rows_dev(const Weight* w, int64_t row0, int64_t count, float* d_out, cudaStream_t s);
int launch_gather_rows(const Weight* w, const int32_t* d_tokens, int count, float* d_out, cudaStream_t s);

// gemv.cu — decode matvec. Prologue: what the kernel does to x before the limb split; epilogue: what it does
// with the row sums.
enum { PRO_PLAIN = 0, PRO_RMSNORM = 1 };
enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SILU = 2 };
// What a producer kernel leaves for the next matvec once its whole output is written (run by its last CTA).
struct PostOp {
    int kind = 0;                   // 0: nothing; 1: limbs of src (of RMSNorm(src) * norm_w when norm_w is set)
    const float* src = nullptr;     // the producer's fp32 output vector
    int n = 0, nl = 4;
    const float* norm_w = nullptr;
    float eps = 0.f;
    int8_t* limbs = nullptr;        // [4][n]
    float* inv_scale = nullptr;     // [1]
    unsigned* done = nullptr;       // arrival counter of the producer's CTAs (zero between launches)
};
struct GemvArgs {
    const int8_t* limbs = nullptr;     // quantized weights: pre-split activation [4][n] and its 2^-k (device)
    const float* inv_scale = nullptr;
    const float* x = nullptr;          // F16 weights: fp32 activation [n], optionally RMSNorm'ed in the kernel
    const float* norm_w = nullptr;
    float eps = 0.f;
    int prologue = PRO_PLAIN;
    float* y = nullptr;                // [rows] (EPI_SILU: [rows/2])
    const float* resid = nullptr;      // EPI_ADD: y = resid + W x (may alias y)
    int epilogue = EPI_STORE;
    bool pdl = false;                  // launch with programmatic stream serialization
    PostOp post;
    int32_t *dbgP = nullptr, *dbgI = nullptr, *dbgJ = nullptr;  // parity dumps
};
int gemv_prepare(Weight* w);  // allocates the split-K scratch (once per weight)
int prep_limbs_launch(const float* x, int n, const float* norm_w, float eps, int nl, int8_t* limbs, float* inv_scale,
                      bool pdl, cudaStream_t s);
int gemv_launch(const Weight* w, const GemvArgs& a, cudaStream_t s);
int matvec_static(const Weight* w, const float* d_x, float* d_y, int nl, cudaStream_t s);

// linear.cu — several tokens at once
// pdl: launch with programmatic stream serialization (the kernel sets itself up while its predecessor still runs and
// waits for it before it touches global memory)
int split_launch(const float* d_x, int64_t ldx, int64_t b, int n, int nl, const float* d_norm_w, float eps,
                 int8_t* d_limbs, float* d_inv_scale, float* d_xsum, cudaStream_t s, bool pdl = false);
int gemm_planes_launch(const Weight* w, const int8_t* d_limbs, const float* d_inv_scale, const float* d_xsum, int B,
                       float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s);
// gemm_tc.cu — tcgen05 path for the two-plane weights (Q4_K, Q6_K)
bool gemm_tc_usable(const Weight* w, int B);
int gemm_tc_launch(const Weight* w, const int8_t* d_limbs, const float* d_inv_scale, const float* d_xsum, int B, int nl,
                   float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s, bool pdl = false,
                   int32_t* d_dbg_acc = nullptr);  // d_dbg_acc: [B][n/256][nl + 1][rows16] accumulator columns (parity checks)
int gemm_tc_check();
int gemm_f16_launch(const Weight* w, const float* d_x, int64_t ldx, const float* d_norm_w, float eps, int B, float* d_y,
                    int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s);
// gemm_f16_tc.cu - tcgen05 path for F16 weights and for Q8_0 weights held as fp16 pairs: the token rows are split into
// fp16 hi / lo halves (d_scratch: 4 * B * n bytes) with 2^-k per row in d_inv_scale, then one tensor-core GEMM with fp32
// accumulators in tensor memory. d_part (gemm_f16_tc_part_bytes() bytes) and d_counters (gemm_f16_tc_counters() zeroed
// words) let a matrix of few tiles be cut along k over more CTAs; null: no cut.
bool gemm_f16_tc_usable(const Weight* w, int B);
size_t gemm_f16_tc_part_bytes();
int gemm_f16_tc_counters();
int gemm_f16_tc_launch(const Weight* w, const float* d_x, int64_t ldx, const float* d_norm_w, float eps, int B, void* d_scratch,
                       float* d_inv_scale, float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s, bool pdl,
                       float* d_part = nullptr, unsigned* d_counters = nullptr);
int gemm_f16_tc_check();
int gemm_f16_tc_wait_expiry(cudaStream_t s);  // test hook: a bounded wait that must run out

// attn.cu
struct AttnDecodeArgs {
    const float* qkv; const float *q_norm, *k_norm; const float* rope; const int* pos;
    float *kc, *vc, *att, *part; unsigned* counters;
    int H, HKV, rope_dim, nsplit; float eps, scale; bool pdl;
    PostOp post;
};
int attn_decode_launch(const AttnDecodeArgs& a, cudaStream_t s);
int qkv_post_launch(float* qkv, int64_t ld, const float* q_norm, const float* k_norm, const float* rope, int pos0, int B,
                    float* kc, float* vc, int H, int HKV, int rope_dim, float eps, cudaStream_t s,
                    const int* posv = nullptr, const int* seqv = nullptr, size_t seq_stride = 0);
// rows of several sequences (row b: position posv[b] of sequence seqv[b]); part [B][HKV][nsplit][group][130], counters [B][HKV]
int attn_rows_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, size_t seq_stride, const int* posv,
                     const int* seqv, float* att, int64_t ld_att, float* part, unsigned* counters, int B, int H, int HKV,
                     int nsplit, float scale, cudaStream_t s);
int attn_prefill_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, float* att, int64_t ld_att,
                        int pos0, int B, int H, int HKV, float scale, cudaStream_t s, float* part = nullptr,
                        unsigned* counters = nullptr);
// attn_tc.cu - the same on the tensor cores (fp16 pairs); kv16: attn_prefill_tc_scratch_halves(n_ctx, HKV * 128) halves
bool attn_prefill_tc_usable(int H, int HKV, int64_t ld, int64_t ld_att);
size_t attn_prefill_tc_scratch_halves(int n_ctx, int KD);
int attn_prefill_tc_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, float* att, int64_t ld_att, int pos0,
                           int B, int H, int HKV, float scale, cudaStream_t s, float* part, unsigned* counters, void* kv16);
size_t attn_prefill_scratch_floats(int max_batch, int H, int HKV);  // `part` of attn_prefill_launch
size_t attn_prefill_counters(int max_batch, int H, int HKV);        // `counters` (zero before the first launch)
int rmsnorm_launch(float* out, const float* x, const float* w, int n, float eps, int rows, cudaStream_t s);
// log-sum-exp (double) and the k best entries by (value descending, index ascending) of logits[n]; out: double lse, then
// TOP_MAXK int32 ids, then TOP_MAXK floats
constexpr int TOP_MAXK = 64;
constexpr size_t TOP_BYTES = 8 + size_t(TOP_MAXK) * 8;
int logits_top_launch(const float* logits, int n, int k, uint8_t* out, cudaStream_t s, const uint32_t* d_allowed = nullptr);
int logits_top_rows_launch(const float* logits, int n, int64_t ld, int rows, int k, uint8_t* out, cudaStream_t s);


}  // namespace elb

// tp.cu: tensor-parallel cut of the model's tensors (host arithmetic) and the NCCL communicator
namespace elb {
struct TpDims {
    int rank = 0, size = 1;
    int H = 0, HKV = 0;                  // heads of this rank
    int64_t f0 = 0, f1 = 0;              // this rank's slice of the FFN dimension
    int64_t v0 = 0, v1 = 0, vchunk = 0;  // this rank's vocabulary rows; vchunk = rows per rank in the gathered logits
};
struct TpShard {
    int64_t row0 = 0, rows = 0, col0 = 0, n = 0;
    int64_t row_bytes = 0, src_row_bytes = 0, src_col_off = 0;
    size_t nbytes = 0;
    bool contiguous = true;  // a row slice: the shard is one byte range of the source
};
int tp_dims(const elb_config& c, int rank, int size, TpDims* d);
int tp_shard_shape(const elb_config& c, const TpDims& d, int role, int type, int64_t rows, int64_t n, TpShard* s);
int tp_shard_copy(const TpShard& s, const uint8_t* src, size_t src_bytes, uint8_t* dst);
struct TpComm;
int tp_unique_id(void* id128);
int tp_comm_create(int device, int rank, int size, const void* id128, TpComm** out);
void tp_comm_destroy(TpComm* c);
int tp_all_reduce(TpComm* c, const float* in, float* out, size_t count, cudaStream_t s);
int tp_all_gather(TpComm* c, const float* in, float* out, size_t count_per_rank, cudaStream_t s);
struct TpPeerBuf {
    void* local = nullptr;
    void* peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int size = 0;
};
int tp_peer_alloc(TpComm* c, int device, size_t bytes, cudaStream_t s, TpPeerBuf* out, bool* ok, bool local_ok = true);
void tp_peer_free(TpPeerBuf* b, int rank);
int tp_agree(TpComm* c, bool mine, cudaStream_t s, bool* all);

// tp_reduce.cu: all-reduce of one activation vector through peer memory, fused with the limb split that follows it
struct TpReduce {
    TpPeerBuf buf;       // per rank: flags [2][8] words, then slots [2][size][n_max] floats
    int rank = 0, size = 1, n_max = 0;
    unsigned* seq = nullptr;  // device counter of reductions done
    int* err_host = nullptr;  // pinned, mapped: raised when a peer did not arrive in time
    int* err_dev = nullptr;
};
int tp_reduce_create(TpComm* c, int device, int rank, int size, int n_max, cudaStream_t s, TpReduce** out);  // *out null: unavailable
void tp_reduce_destroy(TpReduce* r);
// x[n] = sum over ranks (rank order) of their `part`; then, when limbs != null, the split of x (RMSNorm first when
// norm_w != null) as prep_limbs_launch leaves it. Collective: every rank launches it with the same n.
int tp_reduce_split_launch(TpReduce* r, const float* part, float* x, int n, const float* norm_w, float eps, int nl,
                           int8_t* limbs, float* inv_scale, cudaStream_t s);
// the same for a small batch of rows (up to n_max floats), without the split: every value crosses NVLink with its tag in
// one 8-byte word, no flags, no fences (k_tp_rows_allreduce)
struct TpRows {
    TpPeerBuf buf;       // per rank: slots [2 sets][size][n_max] of {value, tag}
    int rank = 0, size = 1;
    size_t n_max = 0;
    unsigned count = 0;  // reductions so far (the next one's tag); all ranks call in step
    int* err_host = nullptr;  // pinned, mapped: raised when a peer's data did not arrive in time
    int* err_dev = nullptr;
};
// collective; *out null: unavailable. caller_ok false: this rank has already failed and only walks through the collectives
int tp_rows_create(TpComm* c, int device, int rank, int size, size_t n_max, cudaStream_t s, TpRows** out, bool caller_ok = true);
void tp_rows_destroy(TpRows* r);
int tp_rows_all_reduce(TpRows* r, const float* in, float* out, size_t n, cudaStream_t s);  // out != in, n even, n <= n_max
}  // namespace elb

// model.cu
namespace elb {
struct Model;
int model_create(const elb_config* cfg, int n_ctx, int device, Model** out);
int model_create_tp(const elb_config* cfg, int n_ctx, int device, int rank, int size, const void* id128, Model** out);
int model_set_tensor(Model* m, int role, int layer, int type, int64_t rows, int64_t n, const void* bytes, size_t nbytes);
int model_finalize(Model* m);
int model_load_gguf(const char* path, int n_ctx, int device, int max_batch, int n_seq, int tp_rank, int tp_size,
                    const void* id128, Model** out);  // gguf_load.cu
int model_config(const Model* m, elb_config* out);
void model_destroy(Model* m);
int model_eval(Model* m, const int32_t* tokens, int n, int pos0, float* logits);
int model_eval_steps(Model* m, const int32_t* tokens, int n, int pos0, float* device_ms);
int model_eval_top(Model* m, const int32_t* tokens, int n, int pos0, int k, int32_t* ids, float* vals, double* lse,
                   const uint32_t* allowed = nullptr);
int model_eval_batch(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want,
                     float* logits);
int model_eval_batch_top(Model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos, const uint8_t* want, int k,
                         int32_t* ids, float* vals, double* lse);
int model_stats(const Model* m, float* ms, int64_t* launches);
int model_hidden(Model* m, float* out);
size_t model_weight_bytes(const Model* m);
size_t model_kv_bytes_per_token(const Model* m);
}  // namespace elb
