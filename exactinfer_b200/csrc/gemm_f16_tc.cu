// Linear layer over a batch of token rows with F16 or Q8_0 weights on the 5th-generation tensor cores:
// Y[token][row] = sum_k W[row][k] * x[token][k], W in fp16 as it lies in the file, x = 2^-k (hi + lo) with hi and lo in
// fp16 (the row is scaled so that its largest magnitude lands in [2^14, 2^15), hi = fp16(x 2^k), lo = fp16(x 2^k - hi):
// 22 significant bits; k_split of the reference, src/cuda/model_cuda.cu:371-395). Every product W * hi and W * lo is exact
// in fp32; both are accumulated in one fp32 accumulator in tensor memory (tcgen05.mma kind::f16), which takes the place
// of the reference's 64-wide tensor-core slices summed in registers (k_gemm_tc, src/cuda/model_cuda.cu:402-492).
// A Q8_0 weight d * q has 18 significant bits: it is held as the exact sum Whi + Wlo of two fp16 values (weights.cu) and
// contributes Whi * hi + Whi * lo + Wlo * hi (Wlo * lo is 2^-22 of the product and left out), so that the block scale
// travels inside the operand and a row's 32-value blocks accumulate in one pass.
//
// Few output tiles (a 64-row batch against a 2048-row matrix is 16 tiles for 148 SMs): the k range of a tile is cut
// into splits that different CTAs accumulate; each leaves its fp32 partial tile in scratch memory and the CTA that
// arrives last adds the partial tiles in split order, so the result does not depend on which CTA that was.
//
// Warp roles (192 threads): warps 0-3 epilogue (warp w drains TMEM lanes 32w.. = weight rows), warp 4 TMA producer,
// warp 5 MMA issuer and TMEM owner. Operands arrive by TMA into a ring of 128-byte-swizzled K-major
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
constexpr int FT_SEG = 2;  // k tiles (of 64) accumulated in tensor memory before the sum moves to registers
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
__device__ __forceinline__ bool f_mbar_wait(uint64_t* bar, uint32_t parity, unsigned limit = FT_SPIN_LIMIT) {  // bounded; false when it ran out
    const uint32_t a = f_smem_u32(bar);
    for (unsigned it = 0; it < limit; ++it) {
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
__device__ __forceinline__ void f_tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
          "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
          "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void f_tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
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
    int splits;          // k splits per output tile
    float* part;         // [tile][split][128 rows][T] partial tiles (splits > 1)
    unsigned* counters;  // [tile] arrivals; the last arrival reduces and zeroes its counter
    int* err;
};

template <int T, bool WLO> struct FtShape {
    static constexpr int A_BYTES = FT_ROWS * 128;  // 128 rows x 64 halves (once more for the lo half of a Q8_0 weight)
    static constexpr int B_BYTES = T * 128;        // T tokens x 64 halves, once for hi and once for lo
    static constexpr int STAGE = (WLO ? 2 : 1) * A_BYTES + 2 * B_BYTES;
    static constexpr int STAGES = (200 * 1024) / STAGE > 6 ? 6 : (200 * 1024) / STAGE;
    static constexpr int SMEM = STAGES * STAGE + 256 + 1024;
    static constexpr int TMEM_COLS = 4 * T;  // two accumulators and the finished tile (3 T columns; a power of two)
};

// k tiles [k0, k1) of split s of a tile
__device__ __forceinline__ void ft_k_range(int nk, int splits, int s, int& k0, int& k1) {
    k0 = int(int64_t(nk) * s / splits);
    k1 = int(int64_t(nk) * (s + 1) / splits);
}

template <int T, bool WLO>
__global__ void __launch_bounds__(FT_THREADS, 1) k_gemm_f16_tc(const __grid_constant__ CUtensorMap mapW,
                                                               const __grid_constant__ CUtensorMap mapX, const FtParams p) {
    using S = FtShape<T, WLO>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE);
    uint64_t* full = bars;                     // [STAGES] TMA -> MMA
    uint64_t* empty = bars + S::STAGES;        // [STAGES] MMA -> TMA
    uint64_t* tfull = bars + 2 * S::STAGES;    // [2] MMA -> epilogue
    uint64_t* tempty = tfull + 2;              // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    unsigned* last_slot = tmem_slot + 1;  // split mode: non-zero when this CTA is the tile's last arrival
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = p.n / FT_K, n_items = p.row_tiles * p.tok_tiles * p.splits;  // item = tile * splits + split
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
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int tile = item / p.splits;
                const int row0 = tile / p.tok_tiles * FT_ROWS, tok0 = tile % p.tok_tiles * T;
                int k0, k1;
                ft_k_range(nk, p.splits, item % p.splits, k0, k1);
                for (int kt = k0; kt < k1 && ok; ++kt, ++it) {
                    const int s = it % S::STAGES;
                    ok = f_mbar_wait(empty + s, ((it / S::STAGES) & 1) ^ 1);
                    if (!ok) break;
                    f_mbar_expect_tx(full + s, S::STAGE);
                    uint8_t* st = smem + s * S::STAGE;
                    if (WLO) {
                        f_tma_3d(st, &mapW, kt * FT_K, row0, 0, full + s);
                        f_tma_3d(st + S::A_BYTES, &mapW, kt * FT_K, row0, 1, full + s);
                        st += S::A_BYTES;
                    } else {
                        f_tma_2d(st, &mapW, kt * FT_K, row0, full + s);
                    }
                    f_tma_3d(st + S::A_BYTES, &mapX, kt * FT_K, tok0, 0, full + s);
                    f_tma_3d(st + S::A_BYTES + S::B_BYTES, &mapX, kt * FT_K, tok0, 1, full + s);
                }
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {  // ---- MMA issuer
            constexpr uint32_t idesc = f_idesc(FT_ROWS, T);
            int it = 0, ns = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int k0, k1;
                ft_k_range(nk, p.splits, item % p.splits, k0, k1);
                for (int ks0 = k0; ks0 < k1 && ok; ks0 += FT_SEG, ++ns) {  // one segment into one accumulator
                    const int acc = ns & 1, ks1 = min(ks0 + FT_SEG, k1);
                    ok = f_mbar_wait(tempty + acc, ((ns >> 1) & 1) ^ 1);  // the accumulator has been drained
                    if (!ok) break;
                    f_fence_after();
                    const uint32_t d = tmem_base + acc * T;
                    for (int kt = ks0; kt < ks1 && ok; ++kt, ++it) {
                        const int s = it % S::STAGES;
                        ok = f_mbar_wait(full + s, (it / S::STAGES) & 1);
                        if (!ok) break;
                        f_fence_after();
                        const uint32_t a0 = f_smem_u32(smem + s * S::STAGE), bh = a0 + (WLO ? 2 : 1) * S::A_BYTES, bl = bh + S::B_BYTES;
#pragma unroll
                        for (int ks = 0; ks < FT_K / 16; ++ks) {  // 16 halves = 32 bytes per MMA
                            f_mma(d, f_desc(a0 + ks * 32), f_desc(bh + ks * 32), idesc, (kt != ks0) | (ks != 0));
                            f_mma(d, f_desc(a0 + ks * 32), f_desc(bl + ks * 32), idesc, 1);
                            if (WLO) f_mma(d, f_desc(a0 + S::A_BYTES + ks * 32), f_desc(bh + ks * 32), idesc, 1);
                        }
                        f_commit(empty + s);  // the stage is free once these MMAs have read it
                    }
                    if (ok) f_commit(tfull + acc);  // the segment is complete
                }
            }
        }
    } else {  // ---- epilogue: warp w drains TMEM lanes 32w.. (weight rows), all T tokens
        int ns = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int tile = item / p.splits;
            const int row0 = tile / p.tok_tiles * FT_ROWS, tok0 = tile % p.tok_tiles * T;
            const int64_t R = row0 + warp * 32 + lane;
            int k0, k1;
            ft_k_range(nk, p.splits, item % p.splits, k0, k1);
            // The tensor core adds into its fp32 accumulator with truncation, a bias that grows with the length of the
            // chain: a segment of FT_SEG k tiles is accumulated there, the segments are added here with rounding.
            float accf[T];
#pragma unroll
            for (int i = 0; i < T; ++i) accf[i] = 0.f;
            for (int ks0 = k0; ks0 < k1 && ok; ks0 += FT_SEG, ++ns) {
                const int acc = ns & 1;
                ok = f_mbar_wait(tfull + acc, (ns >> 1) & 1);
                if (!ok) break;
                f_fence_after();
                const uint32_t tbase = tmem_base + acc * T + (uint32_t(warp * 32) << 16);
#pragma unroll
                for (int c = 0; c < T; c += 32) {
                    float v[32];
                    f_tmem_ld32(tbase + c, v);
#pragma unroll
                    for (int t = 0; t < 32; ++t) accf[c + t] += v[t];
                }
                f_fence_before();  // accumulator in registers: the issuer may overwrite it
                __syncwarp();
                if (lane == 0) f_mbar_arrive(tempty + acc);
            }
            if (!ok) break;
            if (p.splits > 1) {
                float* dst = p.part + (size_t(item) * FT_ROWS + warp * 32 + lane) * T;
#pragma unroll
                for (int t = 0; t < T; t += 4) __stcg(reinterpret_cast<float4*>(dst + t), make_float4(accf[t], accf[t + 1], accf[t + 2], accf[t + 3]));
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
                if (tid == 0) {
                    const unsigned seen = atomicAdd(p.counters + tile, 1u);
                    *last_slot = seen == unsigned(p.splits - 1);
                    if (seen == unsigned(p.splits - 1)) p.counters[tile] = 0;  // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = *last_slot != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");  // everyone has read the slot before the next item writes it
                if (!last) continue;
                __threadfence();
                // the partial tiles in split order, whichever CTA came last (its own included, read back like the others)
                const float* mine = p.part + (size_t(tile) * p.splits * FT_ROWS + warp * 32 + lane) * T;
#pragma unroll
                for (int t = 0; t < T; t += 4) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(mine + t));
                    accf[t] = a.x; accf[t + 1] = a.y; accf[t + 2] = a.z; accf[t + 3] = a.w;
                }
                // (32 tokens of two partial tiles are requested before the first of them is added: the loop is a chain
                // of round trips to L2 otherwise; the order of the additions stays split 1, 2, 3, ...)
                for (int s2 = 1; s2 < p.splits; s2 += 2) {
                    const float* q0 = mine + size_t(s2) * FT_ROWS * T;
                    const bool two = s2 + 1 < p.splits;
                    const float* q1 = two ? q0 + size_t(FT_ROWS) * T : q0;
#pragma unroll
                    for (int c = 0; c < T; c += 32) {
                        float4 a[8], b[8];
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            a[t] = __ldcg(reinterpret_cast<const float4*>(q0 + c) + t);
                            b[t] = __ldcg(reinterpret_cast<const float4*>(q1 + c) + t);
                        }
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            accf[c + 4 * t] += a[t].x; accf[c + 4 * t + 1] += a[t].y; accf[c + 4 * t + 2] += a[t].z; accf[c + 4 * t + 3] += a[t].w;
                        }
                        if (two) {
#pragma unroll
                            for (int t = 0; t < 8; ++t) {
                                accf[c + 4 * t] += b[t].x; accf[c + 4 * t + 1] += b[t].y; accf[c + 4 * t + 2] += b[t].z; accf[c + 4 * t + 3] += b[t].w;
                            }
                        }
                    }
                }
            }
            // The finished tile goes back to tensor memory, from where a compact loop writes it out 32 tokens at a
            // time (a loop over the register array would have to be unrolled: code that runs once per tile, straight
            // from instruction memory).
            const uint32_t tdone = tmem_base + 2 * T + (uint32_t(warp * 32) << 16);
#pragma unroll
            for (int c = 0; c < T; c += 32) f_tmem_st32(tdone + c, *reinterpret_cast<const float(*)[32]>(&accf[c]));
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < T; c += 32) {
                float v[32];
                f_tmem_ld32(tdone + c, v);
                // every load of the 32 tokens before the first store: Y may be the residual stream itself, and a load
                // that has to wait for the store before it turns the chunk into a chain of memory round trips
                float sc[32], r[32];
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    const int tok = tok0 + c + t;
                    sc[t] = tok < p.B ? __ldcg(p.inv_scale + tok) : 0.f;
                    r[t] = p.epilogue == EPI_ADD && tok < p.B && R < p.rows ? __ldcg(p.resid + int64_t(tok) * p.ldy + R) : 0.f;
                }
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    const int tok = tok0 + c + t;
                    const bool tok_ok = tok < p.B;
                    const float y = v[t] * sc[t];
                    if (p.epilogue == EPI_SILU) {  // tile rows 0..7 gate, 8..15 up (16-row groups): partner is 8 lanes up
                        const float up = __shfl_down_sync(0xffffffffu, y, 8);
                        const int64_t o = R / 16 * 8 + (R & 7);
                        if (tok_ok && (lane & 8) == 0 && o < p.rows / 2)
                            p.Y[int64_t(tok) * p.ldy + o] = __fmul_rn(__fdiv_rn(y, 1.0f + expf(-y)), up);
                    } else if (tok_ok && R < p.rows) {
                        p.Y[int64_t(tok) * p.ldy + R] = p.epilogue == EPI_ADD ? r[t] + y : y;
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

// The kernel's bounded wait on a barrier that nobody arrives at (a short limit): it must give up, raise the error word
// and return, leaving the context usable. Host-made failure for the tests; nothing faults.
__global__ void k_wait_expiry(int* err) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        f_mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!f_mbar_wait(&bar, 0, 1u << 12)) atomicExch(err, 3);
    }
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
    // the row is read once and kept in registers (rows of up to 256 * SF_MAX values; longer rows read it three times)
    constexpr int SF_MAX = 24;
    const bool in_regs = n <= 256 * SF_MAX;
    float v[SF_MAX];
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < SF_MAX; ++j) v[j] = tid + 256 * j < n ? __ldcg(x + tid + 256 * j) : 0.f;
    }
    float inv = 1.0f;
    if (norm_w) {
        double ss = 0.0;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < SF_MAX; ++j) ss += double(v[j]) * double(v[j]);
        } else {
            for (int i = tid; i < n; i += 256) { const double t = __ldcg(x + i); ss += t * t; }
        }
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red8[tid >> 5] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < 8; ++i) ss += red8[i];
        inv = float(1.0 / sqrt(ss / n + double(eps)));
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < SF_MAX; ++j)
                if (tid + 256 * j < n) v[j] = __fmul_rn(__fmul_rn(v[j], inv), norm_w[tid + 256 * j]);
        }
    }
    auto val = [&](int i) { return norm_w ? __fmul_rn(__fmul_rn(__ldcg(x + i), inv), norm_w[i]) : __ldcg(x + i); };
    float m = 0.f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < SF_MAX; ++j) m = fmaxf(m, fabsf(v[j]));
    } else {
        for (int i = tid; i < n; i += 256) m = fmaxf(m, fabsf(val(i)));
    }
    m = warp_max(m);
    if ((tid & 31) == 0) redf[tid >> 5] = m;
    __syncthreads();
    m = redf[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, redf[i]);
    int e = 0;
    if (m > 0.f) frexpf(m, &e);
    const int k = m > 0.f ? 15 - e : 0;
    const Pow2 sc = make_pow2(k);
    auto put = [&](int i, float xv) {
        const float s = xv * sc.s1 * sc.s2;
        const __half h = __float2half_rn(s);
        hi[b * n + i] = h;
        lo[b * n + i] = __float2half_rn(s - __half2float(h));
    };
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < SF_MAX; ++j)
            if (tid + 256 * j < n) put(tid + 256 * j, v[j]);
    } else {
        for (int i = tid; i < n; i += 256) put(i, val(i));
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
        if (cudaHostAlloc(&p, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return static_cast<int*>(nullptr);
        *p = 0;
        return p;
    }();
    return host;
}

}  // namespace

bool gemm_f16_tc_usable(const Weight* w, int B) {
    static const bool off = [] { const char* v = std::getenv("ELB_NO_TC"); return v && v[0] == '1'; }();
    static const int min_b = [] { const char* v = std::getenv("ELB_TC_MIN_ROWS"); return v ? std::max(1, atoi(v)) : 2; }();
    const bool fp16 = w->type == ELB_F16 || (w->type == ELB_Q8_0 && w->f16pair);
    return !off && fp16 && w->n % FT_K == 0 && B >= min_b && f_encode_fn() != nullptr;
}

int gemm_f16_tc_wait_expiry(cudaStream_t s) {  // launches the probe; gemm_f16_tc_check() after a synchronize reports it
    int* err_host = f_error_word();
    int* err_dev = nullptr;
    if (!err_host || cudaHostGetDevicePointer(&err_dev, err_host, 0) != cudaSuccess) return fail(ELB_ERR_CUDA, "selftest: no error word");
    k_wait_expiry<<<1, 32, 0, s>>>(err_dev);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

int gemm_f16_tc_check() {  // after a synchronize: did the kernel give up on a wait?
    int* e = f_error_word();
    if (e && *e) {
        *e = 0;
        return fail(ELB_ERR_CUDA, "matmul: a bounded wait in the F16 tensor-core kernel ran out");
    }
    return ELB_OK;
}

size_t gemm_f16_tc_part_bytes() { return size_t(2) * 148 * FT_ROWS * 128 * sizeof(float); }  // two items per SM at T = 128
int gemm_f16_tc_counters() { return 4096; }

// scratch: room for hi and lo, 2 * B * n halves (the model's limb buffer has exactly that size). d_part / d_counters:
// gemm_f16_tc_part_bytes() bytes and gemm_f16_tc_counters() zeroed words for the k splits, or null (no splits).
int gemm_f16_tc_launch(const Weight* w, const float* d_x, int64_t ldx, const float* d_norm_w, float eps, int B, void* d_scratch,
                       float* d_inv_scale, float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s, bool pdl,
                       float* d_part, unsigned* d_counters) {
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
    const bool wlo = w->type == ELB_Q8_0;
    CUtensorMap mapW, mapX;
    if (wlo) ELB_TRY(f_make_map(&mapW, w->f16pair, uint64_t(n), uint64_t(rows16), 2, FT_ROWS));
    else ELB_TRY(f_make_map(&mapW, w->tiled, uint64_t(n), uint64_t(rows16), 1, FT_ROWS));
    ELB_TRY(f_make_map(&mapX, hi, uint64_t(n), uint64_t(B), 2, uint32_t(T)));
    const int row_tiles = int((rows16 + FT_ROWS - 1) / FT_ROWS), tok_tiles = (B + T - 1) / T;
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    const int64_t tiles = int64_t(row_tiles) * tok_tiles;
    int splits = 1;
    static const int max_splits = [] { const char* v = std::getenv("ELB_TC_SPLITS"); return v ? std::max(1, atoi(v)) : 16; }();
    if (d_part && d_counters && tiles < di.sm_count && tiles <= gemm_f16_tc_counters()) {
        splits = int(std::min<int64_t>({int64_t(di.sm_count) / tiles, int64_t(n / FT_K / 4), int64_t(max_splits)}));
        splits = std::max(splits, 1);
        while (splits > 1 && size_t(tiles) * splits * FT_ROWS * T * sizeof(float) > gemm_f16_tc_part_bytes()) --splits;
    }
    FtParams p{d_inv_scale, d_y, d_resid, rows16, w->rows, ldy, B, n, epilogue, row_tiles, tok_tiles, splits, d_part, d_counters, err_dev};
    const int grid = int(std::min<int64_t>(tiles * splits, di.sm_count));
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
    if (wlo) {
        if (T == 128) ELB_TRY(launch(k_gemm_f16_tc<128, true>, FtShape<128, true>::SMEM));
        else if (T == 64) ELB_TRY(launch(k_gemm_f16_tc<64, true>, FtShape<64, true>::SMEM));
        else ELB_TRY(launch(k_gemm_f16_tc<32, true>, FtShape<32, true>::SMEM));
    } else {
        if (T == 128) ELB_TRY(launch(k_gemm_f16_tc<128, false>, FtShape<128, false>::SMEM));
        else if (T == 64) ELB_TRY(launch(k_gemm_f16_tc<64, false>, FtShape<64, false>::SMEM));
        else ELB_TRY(launch(k_gemm_f16_tc<32, false>, FtShape<32, false>::SMEM));
    }
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
