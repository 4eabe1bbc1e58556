// Prompt-chunk linear layer with F16 weights on the 5th-generation tensor cores:
// Y[token][row] = sum_k W[row][k] * x[token][k], W in fp16 as it lies in the file, x = 2^-k (hi + lo) with hi and lo in
// fp16 (the row is scaled so that its largest magnitude lands in [2^14, 2^15), hi = fp16(x 2^k), lo = fp16(x 2^k - hi):
// 22 significant bits; k_split of the reference, src/cuda/model_cuda.cu:371-395). Every product W * hi and W * lo is exact
// in fp32; both are accumulated in one fp32 accumulator in tensor memory (tcgen05.mma kind::f16), which takes the place
// of the reference's 64-wide tensor-core slices summed in registers (k_gemm_tc, src/cuda/model_cuda.cu:402-492).
//
// Warp roles (192 threads): warps 0-3 epilogue (warp w drains TMEM lanes 32w.. = weight rows), warp 4 TMA producer,
// warp 5 MMA issuer and TMEM owner. Operands arrive by TMA (no multicast) into a ring of 128-byte-swizzled K-major
// tiles (64 k per stage); two accumulators, so that the drain of one tile overlaps the MMAs of the next. A persistent
// grid walks the output tiles. Every mbarrier wait is bounded: on timeout the kernel raises an error word and winds down.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace elb {

namespace {

constexpr int FT_ROWS = 128, FT_K = 64, FT_THREADS = 192;
constexpr unsigned FT_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t f_smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void f_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(f_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void f_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(f_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void f_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(f_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool f_mbar_wait(uint64_t* bar, uint32_t parity) {  // bounded; false when it ran out
    const uint32_t a = f_smem_u32(bar);
    for (unsigned it = 0; it < FT_SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void f_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(f_smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(f_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void f_tma_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(f_smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(f_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void f_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void f_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, fp16 x fp16 -> fp32, issued by one thread
__device__ __forceinline__ void f_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void f_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(f_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void f_tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle; 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t f_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3FFFF) >> 4);
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulator, fp16 A and B, both K-major, M x N
__host__ __device__ constexpr uint32_t f_idesc(int M, int N) {
    return (1u << 4) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

struct FtParams {
    const float* inv_scale;  // [B] 2^-k of each token row
    float* Y;
    const float* resid;
    int64_t rows16, rows, ldy;
    int B, n, epilogue;
    int row_tiles, tok_tiles;
    int* err;
};

template <int T> struct FtShape {
    static constexpr int STAGES = T >= 128 ? 4 : 6;
    static constexpr int A_BYTES = FT_ROWS * 128;  // 128 rows x 64 halves
    static constexpr int B_BYTES = T * 128;        // T tokens x 64 halves, once for hi and once for lo
    static constexpr int STAGE = A_BYTES + 2 * B_BYTES;
    static constexpr int SMEM = STAGES * STAGE + 256 + 1024;
    static constexpr int TMEM_COLS = 2 * T < 32 ? 32 : 2 * T;  // two accumulators (a power of two >= 32)
};

template <int T>
__global__ void __launch_bounds__(FT_THREADS, 1) k_gemm_f16_tc(const __grid_constant__ CUtensorMap mapW,
                                                               const __grid_constant__ CUtensorMap mapX, const FtParams p) {
    using S = FtShape<T>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE);
    uint64_t* full = bars;                     // [STAGES] TMA -> MMA
    uint64_t* empty = bars + S::STAGES;        // [STAGES] MMA -> TMA
    uint64_t* tfull = bars + 2 * S::STAGES;    // [2] MMA -> epilogue
    uint64_t* tempty = tfull + 2;              // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = p.n / FT_K, n_tiles = p.row_tiles * p.tok_tiles;
    if (tid == 0) {
        for (int s = 0; s < S::STAGES; ++s) { f_mbar_init(full + s, 1); f_mbar_init(empty + s, 1); }
        for (int a = 0; a < 2; ++a) { f_mbar_init(tfull + a, 1); f_mbar_init(tempty + a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(f_smem_u32(tmem_slot)), "n"(S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();  // everything above touched shared memory only; from here on the kernel reads what earlier kernels wrote
    f_fence_before();
    __syncthreads();
    f_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 4) {
        if (lane == 0) {  // ---- TMA producer
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int row0 = tile / p.tok_tiles * FT_ROWS, tok0 = tile % p.tok_tiles * T;
                for (int kt = 0; kt < nk && ok; ++kt, ++it) {
                    const int s = it % S::STAGES;
                    ok = f_mbar_wait(empty + s, ((it / S::STAGES) & 1) ^ 1);
                    if (!ok) break;
                    f_mbar_expect_tx(full + s, S::STAGE);
                    uint8_t* st = smem + s * S::STAGE;
                    f_tma_2d(st, &mapW, kt * FT_K, row0, full + s);
                    f_tma_3d(st + S::A_BYTES, &mapX, kt * FT_K, tok0, 0, full + s);
                    f_tma_3d(st + S::A_BYTES + S::B_BYTES, &mapX, kt * FT_K, tok0, 1, full + s);
                }
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {  // ---- MMA issuer
            constexpr uint32_t idesc = f_idesc(FT_ROWS, T);
            int it = 0, nt = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++nt) {
                const int acc = nt & 1;
                ok = f_mbar_wait(tempty + acc, ((nt >> 1) & 1) ^ 1);  // the accumulator has been drained
                if (!ok) break;
                f_fence_after();
                const uint32_t d = tmem_base + acc * T;
                for (int kt = 0; kt < nk && ok; ++kt, ++it) {
                    const int s = it % S::STAGES;
                    ok = f_mbar_wait(full + s, (it / S::STAGES) & 1);
                    if (!ok) break;
                    f_fence_after();
                    const uint32_t a0 = f_smem_u32(smem + s * S::STAGE), bh = a0 + S::A_BYTES, bl = bh + S::B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < FT_K / 16; ++ks) {  // 16 halves = 32 bytes per MMA
                        f_mma(d, f_desc(a0 + ks * 32), f_desc(bh + ks * 32), idesc, (kt | ks) != 0);
                        f_mma(d, f_desc(a0 + ks * 32), f_desc(bl + ks * 32), idesc, 1);
                    }
                    f_commit(empty + s);  // the stage is free once these MMAs have read it
                }
                if (ok) f_commit(tfull + acc);  // the tile is complete
            }
        }
    } else {  // ---- epilogue: warp w drains TMEM lanes 32w.. (weight rows), all T tokens
        int nt = 0;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++nt) {
            const int acc = nt & 1;
            const int row0 = tile / p.tok_tiles * FT_ROWS, tok0 = tile % p.tok_tiles * T;
            const int64_t R = row0 + warp * 32 + lane;
            ok = f_mbar_wait(tfull + acc, (nt >> 1) & 1);
            if (!ok) break;
            f_fence_after();
            const uint32_t tbase = tmem_base + acc * T + (uint32_t(warp * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < T; c += 16) {
                float v[16];
                f_tmem_ld16(tbase + c, v);
                if (c + 16 >= T) {  // accumulator in registers: the issuer may overwrite it
                    f_fence_before();
                    __syncwarp();
                    if (lane == 0) f_mbar_arrive(tempty + acc);
                }
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    const int tok = tok0 + c + t;
                    const bool tok_ok = tok < p.B;
                    const float y = v[t] * (tok_ok ? __ldcg(p.inv_scale + tok) : 0.f);
                    if (p.epilogue == EPI_SILU) {  // tile rows 0..7 gate, 8..15 up (16-row groups): partner is 8 lanes up
                        const float up = __shfl_down_sync(0xffffffffu, y, 8);
                        const int64_t o = R / 16 * 8 + (R & 7);
                        if (tok_ok && (lane & 8) == 0 && o < p.rows / 2)
                            p.Y[int64_t(tok) * p.ldy + o] = __fmul_rn(__fdiv_rn(y, 1.0f + expf(-y)), up);
                    } else if (tok_ok && R < p.rows) {
                        const int64_t o = int64_t(tok) * p.ldy + R;
                        p.Y[o] = p.epilogue == EPI_ADD ? p.resid[o] + y : y;
                    }
                }
            }
        }
    }
    if (!ok) atomicExch(p.err, 3);
    pdl_launch_dependents();
    f_fence_before();
    __syncthreads();
    if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(S::TMEM_COLS) : "memory");
}

// ---------------------------------------------------------------- hi / lo split of the token rows

// One block per token row: optional RMSNorm (src/ops.cpp:155-160, sum of squares in double), scale 2^k that brings the
// row's largest magnitude into [2^14, 2^15), hi = fp16(x 2^k), lo = fp16(x 2^k - hi); inv_scale = 2^-k.
__global__ void __launch_bounds__(256) k_split_f16(const float* __restrict__ X, int64_t ldx, int n, const float* __restrict__ norm_w,
                                                   float eps, __half* __restrict__ hi, __half* __restrict__ lo,
                                                   float* __restrict__ inv_scale) {
    __shared__ double red8[8];
    __shared__ float redf[8];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int64_t b = blockIdx.x;
    const float* x = X + b * ldx;
    float inv = 1.0f;
    if (norm_w) {
        double ss = 0.0;
        for (int i = tid; i < n; i += 256) { const double v = __ldcg(x + i); ss += v * v; }
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red8[tid >> 5] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < 8; ++i) ss += red8[i];
        inv = float(1.0 / sqrt(ss / n + double(eps)));
    }
    auto val = [&](int i) { return norm_w ? __fmul_rn(__fmul_rn(__ldcg(x + i), inv), norm_w[i]) : __ldcg(x + i); };
    float m = 0.f;
    for (int i = tid; i < n; i += 256) m = fmaxf(m, fabsf(val(i)));
    m = warp_max(m);
    if ((tid & 31) == 0) redf[tid >> 5] = m;
    __syncthreads();
    m = redf[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, redf[i]);
    int e = 0;
    if (m > 0.f) frexpf(m, &e);
    const int k = m > 0.f ? 15 - e : 0;
    const Pow2 sc = make_pow2(k);
    for (int i = tid; i < n; i += 256) {
        const float v = val(i) * sc.s1 * sc.s2;
        const __half h = __float2half_rn(v);
        hi[b * n + i] = h;
        lo[b * n + i] = __float2half_rn(v - __half2float(h));
    }
    if (tid == 0) inv_scale[b] = ldexpf(1.0f, -k);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn f_encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}
// fp16 tensor [d2][d1][k] (k contiguous), box [1][box1][64], 128-byte swizzle, zero fill outside
int f_make_map(CUtensorMap* map, const void* base, uint64_t k, uint64_t d1, uint64_t d2, uint32_t box1) {
    EncodeFn fn = f_encode_fn();
    if (!fn) return fail(ELB_ERR_CUDA, "matmul: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[3] = {k, d1, d2};
    const cuuint64_t strides[2] = {k * 2, k * d1 * 2};
    const cuuint32_t box[3] = {FT_K, box1, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, d2 > 1 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ELB_ERR_CUDA, "matmul: tensor map encoding failed (F16)");
    return ELB_OK;
}

int* f_error_word() {  // pinned, mapped: raised by a kernel whose bounded wait ran out
    static int* host = [] {
        int* p = nullptr;
        if (cudaHostAlloc(&p, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return static_cast<int*>(nullptr);
        *p = 0;
        return p;
    }();
    return host;
}

}  // namespace

bool gemm_f16_tc_usable(const Weight* w, int B) {
    static const bool off = [] { const char* v = std::getenv("ELB_NO_TC"); return v && v[0] == '1'; }();
    return !off && w->type == ELB_F16 && w->n % FT_K == 0 && B >= 16 && f_encode_fn() != nullptr;
}

int gemm_f16_tc_check() {  // after a synchronize: did the kernel give up on a wait?
    int* e = f_error_word();
    if (e && *e) {
        *e = 0;
        return fail(ELB_ERR_CUDA, "matmul: a bounded wait in the F16 tensor-core kernel ran out");
    }
    return ELB_OK;
}

// scratch: room for hi and lo, 2 * B * n halves (the model's limb buffer has exactly that size)
int gemm_f16_tc_launch(const Weight* w, const float* d_x, int64_t ldx, const float* d_norm_w, float eps, int B, void* d_scratch,
                       float* d_inv_scale, float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s, bool pdl) {
    if (!gemm_f16_tc_usable(w, B)) return fail(ELB_ERR_STATE, "matmul: F16 tensor-core path not usable for this weight");
    if (epilogue == EPI_SILU && !w->pair) return fail(ELB_ERR_INVALID, "matmul: SwiGLU epilogue needs a paired weight");
    int* err_host = f_error_word();
    int* err_dev = nullptr;
    if (!err_host || cudaHostGetDevicePointer(&err_dev, err_host, 0) != cudaSuccess) return fail(ELB_ERR_CUDA, "matmul: no error word");
    const int n = int(w->n);
    __half* hi = static_cast<__half*>(d_scratch);
    __half* lo = hi + size_t(B) * n;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(unsigned(B));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        ELB_CUDA(cudaLaunchKernelEx(&cfg, k_split_f16, d_x, ldx, n, d_norm_w, eps, hi, lo, d_inv_scale));
    }
    const int64_t rows16 = w->tiles * 16;
    const int T = B > 64 ? 128 : B > 32 ? 64 : 32;
    CUtensorMap mapW, mapX;
    ELB_TRY(f_make_map(&mapW, w->tiled, uint64_t(n), uint64_t(rows16), 1, FT_ROWS));
    ELB_TRY(f_make_map(&mapX, hi, uint64_t(n), uint64_t(B), 2, uint32_t(T)));
    const int row_tiles = int((rows16 + FT_ROWS - 1) / FT_ROWS), tok_tiles = (B + T - 1) / T;
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    FtParams p{d_inv_scale, d_y, d_resid, rows16, w->rows, ldy, B, n, epilogue, row_tiles, tok_tiles, err_dev};
    const int grid = int(std::min<int64_t>(int64_t(row_tiles) * tok_tiles, di.sm_count));
    auto launch = [&](auto kernel, int smem) -> int {
        ELB_TRY(ensure_dyn_smem(reinterpret_cast<const void*>(kernel), size_t(smem)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(unsigned(grid));
        cfg.blockDim = dim3(FT_THREADS);
        cfg.dynamicSmemBytes = size_t(smem);
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        ELB_CUDA(cudaLaunchKernelEx(&cfg, kernel, mapW, mapX, p));
        return ELB_OK;
    };
    if (T == 128) ELB_TRY(launch(k_gemm_f16_tc<128>, FtShape<128>::SMEM));
    else if (T == 64) ELB_TRY(launch(k_gemm_f16_tc<64>, FtShape<64>::SMEM));
    else ELB_TRY(launch(k_gemm_f16_tc<32>, FtShape<32>::SMEM));
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
