// Prompt-chunk linear layer on the 5th-generation tensor cores: Y[token][row] = sum_k W[row][k] * x[token][k] with
// W = W0 + 256 W1 (int8 digit planes of the integer weight sc*q, built at upload) and x = 2^-k * sum_l a_l 256^l
// (int8 limbs), every product exact in int32.
//
// One tcgen05 accumulator holds all digit products of equal weight 256^j: column (j, token) accumulates
// W0 . a_j + W1 . a_(j-1), j = 0..NL. Both MMAs of a k-step read the limb tile from the same shared-memory buffer:
// its rows are ordered (limb, token) with a block of T zero rows in front and behind, and the operand of the W1
// product is simply the same buffer addressed T rows earlier. So a 128-row x T-token tile costs 2 MMAs of
// M=128, N=(NL+1)T, K=32 per 32 k, one accumulator of (NL+1)T TMEM columns (two, for double buffering), and the limb
// combination sum_j 256^j R_j is one Horner chain per (row, token) per 256-block in the epilogue, where the fp16
// block scale d (and Q4_K's dmin*m term) is applied in fp32.
//
// Warp roles (576 threads): warps 0-15 epilogue (warp w drains TMEM lanes 32(w%4).. = weight rows, for quarter w/4 of
// the tile's tokens), warp 16 TMA producer, warp 17 MMA issuer and TMEM owner. Operands arrive by TMA into a 3-stage ring of
// 128-byte-swizzled K-major tiles; TMEM accumulators are double buffered so that the drain of one 256-block overlaps
// the MMAs of the next. Every mbarrier wait is bounded: on timeout the kernel raises an error word and winds down.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace elb {

constexpr int TC_ROWS = 128, TC_KSTAGE = 128, TC_STAGES = 3, TC_EPI_WARPS = 16, TC_THREADS = (TC_EPI_WARPS + 2) * 32;
constexpr int TC_TOK_PARTS = TC_EPI_WARPS / 4;  // epilogue warps per TMEM lane quarter: each takes a share of the tile's tokens
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;

// ---------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait; false when it ran out (the error word is raised by the caller)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    for (unsigned it = 0; it < TC_SPIN_LIMIT; ++it) {
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

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, int8 x int8 -> int32, issued by one thread
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive columns of this warp's 32 TMEM lanes -> 16 registers per thread (thread = lane = weight row)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, int (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle; 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3FFFF) >> 4);  // start address, 16-byte units
    d |= uint64_t(1024 >> 4) << 32;         // stride between 8-row groups
    d |= uint64_t(1) << 46;                 // descriptor version of this architecture
    d |= uint64_t(2) << 61;                 // 128-byte swizzle
    return d;
}
// Instruction descriptor for kind::i8: int32 accumulator, signed 8-bit A and B, both K-major, M x N
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// ---------------------------------------------------------------- the kernel

// diagnostics (ELB_TC_PROF=1): clock cycles the MMA issuer of CTA 0 spent waiting for a drained accumulator, waiting for
// operands, and in total, summed over launches
__device__ unsigned long long g_tc_prof[12];


struct TcParams {
    const __half* pl_d;      // [rows16][n/256] block scale
    const float* pl_dm;      // Q4_K: [rows16][n/32] fl(dmin*m); else null
    const float* xsum;       // [B][n/32] sum of the fixed-point activation over each 32-slice
    const float* inv_scale;  // [B] 2^-k
    float* Y;
    const float* resid;
    int64_t rows16, rows, ldy;
    int B, n, epilogue;
    int row_tiles, tok_tiles;  // row_tiles * tok_tiles output tiles, token tiles of one row tile adjacent
    int waves;                 // whole tiles per CTA: CTA c computes tiles c, c + grid, ... (waves of them)
    int per;                   // the tiles behind the whole waves are cut in (tile, 256-block) units, `per` per CTA:
                               // CTA c owns units [c * per, (c + 1) * per) of them
    float* scratch;            // [grid][T][TC_ROWS] partial sums of a tile piece that does not hold the tile's first block
    unsigned* flags;           // [grid] launch number once the CTA's scratch is written
    unsigned* ctl;             // {launches completed, CTAs of this launch that are done}: kept by the kernel itself, so a
                               // launch replayed from a graph numbers itself like any other
    int* err;
    int prof;
    int32_t* dbgA;             // parity checks: the int32 accumulator columns as they leave tensor memory,
                               // [B][n/256][NL + 1][rows16]; null in normal use
};

// A grid of one CTA per SM walks the output tiles in whole waves; the tiles that do not fill a wave would leave most
// SMs idle for a whole tile's time, so they are cut by (tile, 256-block) units instead: every CTA gets the same number
// of consecutive units, a tile is shared by the CTA that holds its first blocks and one or more CTAs after it. Those
// leave their partial sums (fp32, after the block scales) in `scratch` and the CTA with the first blocks adds them in
// CTA order and writes the tile. The shared tiles come first: a CTA's share of them is at most two pieces, the piece
// without a tile's first blocks first, so nobody waits long, and the whole tiles after them keep neighbouring CTAs on
// neighbouring tiles (the weight tile of a row is fetched from HBM once for all its token tiles).
struct Piece { int tile, kb0, kb1; };
// Piece i of this CTA: 0 and 1 are its share of the shared tiles (a share is no longer than a tile, so it touches at
// most two), 2 + w is its tile of whole wave w. False when the CTA has no such piece. Everything is recomputed from
// the launch parameters, so that the walk costs the three roles one register.
__device__ __forceinline__ bool piece_at(const int i, const int per, const int waves, const int n_tiles, const int nkb, Piece& pc) {
    const int tile0 = waves * int(gridDim.x);  // the shared tiles follow the whole waves
    if (i >= 2) {
        pc.tile = int(blockIdx.x) + (i - 2) * int(gridDim.x);
        pc.kb0 = 0;
        pc.kb1 = nkb;
        return pc.tile < n_tiles;  // (the last wave may be a partial one when nothing is shared: ELB_TC_NO_SPLIT)
    }
    const int units = max(n_tiles - tile0, 0) * nkb;
    const int u0 = min(int(blockIdx.x) * per, units), u1 = min(u0 + per, units);
    const int tl = u0 / nkb, k0 = u0 - tl * nkb, k1 = min(nkb, k0 + (u1 - u0));
    if (i == 0) {
        pc.tile = tile0 + tl;
        pc.kb0 = k0;
        pc.kb1 = k1;
        return u0 < u1;
    }
    pc.tile = tile0 + tl + 1;
    pc.kb0 = 0;
    pc.kb1 = u1 - (tl + 1) * nkb;
    return pc.kb1 > 0;
}

// Tokens per tile. The accumulator has (NL + 1) * T columns, twice (double buffering) in the 512 TMEM columns: at most 64
// tokens for three limbs, 48 for four. Small batches (decode steps of several sequences) take narrower tiles, so that
// the tensor core and the epilogue do not work on columns that hold no token.
constexpr int tc_wide(int nl) { return nl == 4 ? 48 : 64; }

template <int NL, int TT> struct TcShape {
    static constexpr int T = TT;                      // tokens per tile
    static constexpr int N = (NL + 1) * T;            // accumulator columns: (digit weight j, token)
    static constexpr int ZB = T * 128;                // one block of zero rows
    static constexpr int LB = NL * T * 128;           // limb rows of one stage
    static constexpr int A_BYTES = TC_ROWS * 128;     // one plane tile of one stage
    static constexpr int LIMB_AREA = ZB + TC_STAGES * (LB + ZB);
    static constexpr int XS_BYTES = 2 * T * 8 * 4;    // sum(X) of the tile's tokens over the 8 sub-blocks of a block, x2
    static constexpr int SC_BYTES = 2 * TC_ROWS * 9 * 4;  // fl(dmin*m) [8] and d of the tile's rows for one block, x2
    static constexpr int SMEM = LIMB_AREA + TC_STAGES * 2 * A_BYTES + 256 + XS_BYTES + SC_BYTES + 1024;  // + barriers + slack
};

// DBG: also writes the int32 accumulator columns to p.dbgA (parity checks; its own instantiation, because the extra
// addressing does not fit into the 96 registers of the production kernel without spills)
template <int NL, int TT, bool DBG = false>
__global__ void __launch_bounds__(TC_THREADS, 1) k_gemm_tc(const __grid_constant__ CUtensorMap mapW,
                                                          const __grid_constant__ CUtensorMap mapX, const TcParams p) {
    using S = TcShape<NL, TT>;
    constexpr int T = S::T, N = S::N;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* limb_area = smem;
    uint8_t* a_area = smem + S::LIMB_AREA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(a_area + TC_STAGES * 2 * S::A_BYTES);
    uint64_t* full = bars;                   // [TC_STAGES] TMA -> MMA
    uint64_t* empty = bars + TC_STAGES;      // [TC_STAGES] MMA -> TMA
    uint64_t* tfull = bars + 2 * TC_STAGES;  // [2] MMA -> epilogue
    uint64_t* tempty = tfull + 2;            // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    float* xs_s = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [2][T][8]
    float* dm_s = xs_s + 2 * T * 8;            // [2][TC_ROWS][8]
    float* d_s = dm_s + 2 * TC_ROWS * 8;       // [2][TC_ROWS]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = p.n / 256, n_tiles = p.row_tiles * p.tok_tiles;
    int* s_fail = reinterpret_cast<int*>(tmem_slot + 1);
    unsigned* s_seq = reinterpret_cast<unsigned*>(tmem_slot + 2);

    // zero blocks in front of, between and behind the limb stages
    for (int z = 0; z <= TC_STAGES; ++z) {
        uint4* zp = reinterpret_cast<uint4*>(limb_area + z * (S::LB + S::ZB));
        for (int i = tid; i < S::ZB / 16; i += TC_THREADS) zp[i] = make_uint4(0, 0, 0, 0);
    }
    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull + a, 1); mbar_init(tempty + a, TC_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zero rows are read by the tensor core
    if (warp == TC_EPI_WARPS + 1) tmem_alloc(tmem_slot, 512);
    // Launched with programmatic stream serialization this kernel starts while its predecessor still runs: everything
    // above touched shared memory only. From here on it reads what earlier kernels wrote (limbs, sums, the residual, the
    // launch counter) and writes what they may still read.
    pdl_wait();
    if (tid == 0) {
        *s_fail = 0;
        // the count moves only when every CTA of a launch is done, hence after every CTA of it has read it
        *s_seq = *reinterpret_cast<volatile unsigned*>(p.ctl) + 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == TC_EPI_WARPS) {
        if (lane == 0) {  // ---- TMA producer
            int it = 0;  // stages filled so far, over all pieces of this CTA
            Piece pc;
            for (int pi = 0; pi < 2 + p.waves && ok; ++pi) {
            if (!piece_at(pi, p.per, p.waves, n_tiles, nkb, pc)) continue;
            const int row0 = pc.tile / p.tok_tiles * TC_ROWS, tok0 = pc.tile % p.tok_tiles * T;
            for (int kt = 2 * pc.kb0; kt < 2 * pc.kb1 && ok; ++kt, ++it) {
                const int s = it % TC_STAGES;
                ok = mbar_wait(empty + s, ((it / TC_STAGES) & 1) ^ 1);
                if (!ok) break;
                mbar_expect_tx(full + s, 2 * S::A_BYTES + S::LB);
                const int k0 = kt * TC_KSTAGE;
                tma_load_3d(a_area + (s * 2 + 0) * S::A_BYTES, &mapW, k0, row0, 0, full + s);
                tma_load_3d(a_area + (s * 2 + 1) * S::A_BYTES, &mapW, k0, row0, 1, full + s);
                uint8_t* lb = limb_area + S::ZB + s * (S::LB + S::ZB);
                for (int l = 0; l < NL; ++l) tma_load_3d(lb + l * S::ZB, &mapX, k0, tok0, l, full + s);
            }
            }
        }
    } else if (warp == TC_EPI_WARPS + 1) {
        if (lane == 0) {  // ---- MMA issuer
            constexpr uint32_t idesc = idesc_i8(TC_ROWS, N);
            int it = 0;
            long long w_acc = 0, w_ops = 0;
            const long long t_start = clock64();
            Piece pc;
            for (int pi = 0; pi < 2 + p.waves && ok; ++pi)
            for (int kt = piece_at(pi, p.per, p.waves, n_tiles, nkb, pc) ? 2 * pc.kb0 : 2 * pc.kb1; kt < 2 * pc.kb1 && ok; ++kt, ++it) {
                const int s = it % TC_STAGES, kb = it >> 1, acc = kb & 1;  // kb: 256-blocks issued so far (nk is even)
                long long t0 = clock64();
                if ((kt & 1) == 0) {  // first half of a 256-block: its accumulator must have been drained
                    ok = mbar_wait(tempty + acc, ((kb >> 1) & 1) ^ 1);
                    if (!ok) break;
                }
                long long t1 = clock64();
                ok = mbar_wait(full + s, (it / TC_STAGES) & 1);
                if (!ok) break;
                w_acc += t1 - t0;
                w_ops += clock64() - t1;
                tc_fence_after();
                const uint32_t a0 = smem_u32(a_area + (s * 2 + 0) * S::A_BYTES), a1 = a0 + S::A_BYTES;
                const uint32_t b0 = smem_u32(limb_area + S::ZB + s * (S::LB + S::ZB)), b1 = b0 - S::ZB;
                const uint32_t d = tmem_base + acc * 256;
#pragma unroll
                for (int ks = 0; ks < TC_KSTAGE / 32; ++ks) {
                    mma_i8(d, smem_desc(a0 + ks * 32), smem_desc(b0 + ks * 32), idesc, ((kt & 1) | ks) != 0);
                    mma_i8(d, smem_desc(a1 + ks * 32), smem_desc(b1 + ks * 32), idesc, 1);
                }
                mma_commit(empty + s);                    // the stage is free once these MMAs have read it
                if (kt & 1) mma_commit(tfull + acc);      // the 256-block is complete
            }
            if (p.prof && blockIdx.x == 0) {
                atomicAdd(&g_tc_prof[0], (unsigned long long)w_acc);
                atomicAdd(&g_tc_prof[1], (unsigned long long)w_ops);
                atomicAdd(&g_tc_prof[2], (unsigned long long)(clock64() - t_start));
                atomicAdd(&g_tc_prof[3], 1ull);
            }
        }
    } else {  // ---- epilogue: warp w drains TMEM lanes 32(w%4).. (weight rows) for tokens [th*TH, (th+1)*TH), th = w/4
        constexpr int TH = T / TC_TOK_PARTS;  // tokens per epilogue warp
        static_assert(TH % 4 == 0, "token share of an epilogue warp is loaded four columns at a time");
        constexpr int XPT = (T * 8 + TC_EPI_WARPS * 32 - 1) / (TC_EPI_WARPS * 32);  // sum(X) values staged per thread
        static_assert(TC_EPI_WARPS * 32 >= 3 * TC_ROWS, "one scale value per staging thread");
        const int etid = warp * 32 + lane;
        const int q4 = warp & 3, th = warp >> 2, my_row = q4 * 32 + lane;
        const int nblk = p.n / 256, nsub = p.n / 32;
        int kbt = 0;  // 256-blocks drained so far, over all tiles of this CTA
        Piece pc;
        for (int pi = 0; pi < 2 + p.waves && ok; ++pi) {
        if (!piece_at(pi, p.per, p.waves, n_tiles, nkb, pc)) continue;
        const int row0 = pc.tile / p.tok_tiles * TC_ROWS, tok0 = pc.tile % p.tok_tiles * T;
        const int64_t R = row0 + my_row;
        float accf[TH];
#pragma unroll
        for (int t = 0; t < TH; ++t) accf[t] = 0.f;
        // Per 256-block the epilogue needs the block scale d and (Q4_K) the eight fl(dmin*m) of every row of the tile and
        // sum(X) over the eight 32-slices of every token of the tile. Thread = weight row would make those loads one
        // cache line per lane; instead all epilogue threads fetch them together (two threads per row for dmin*m, one
        // per row for d, the rest sum(X)), one block ahead, and pass them on through shared memory.
        float xreg[XPT];
        float4 screg = make_float4(0.f, 0.f, 0.f, 0.f);
        auto fetch = [&](int kb) {
#pragma unroll
            for (int q = 0; q < XPT; ++q) {
                const int i = etid + q * TC_EPI_WARPS * 32;
                const int tok = min(tok0 + (i >> 3), p.B - 1);
                xreg[q] = p.pl_dm && i < T * 8 ? __ldcg(p.xsum + int64_t(tok) * nsub + kb * 8 + (i & 7)) : 0.f;
            }
            if (etid < 2 * TC_ROWS) {
                const int64_t r = row0 + (etid >> 1);
                screg = p.pl_dm && r < p.rows16 ? __ldg(reinterpret_cast<const float4*>(p.pl_dm + r * nsub + kb * 8 + 4 * (etid & 1)))
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
            } else if (etid < 3 * TC_ROWS) {
                const int64_t r = row0 + etid - 2 * TC_ROWS;
                screg.x = r < p.rows16 ? __half2float(p.pl_d[r * nblk + kb]) : 0.f;
            }
        };
        const bool is_tail = pc.kb0 > 0, is_open = pc.kb0 == 0 && pc.kb1 < nkb;
        const int kb_end = pc.kb1;
        fetch(pc.kb0);
        for (int kb = pc.kb0; kb < kb_end && ok; ++kb, ++kbt) {
            const int acc = kbt & 1;
            float* xb = xs_s + acc * (T * 8);
            float* dmb = dm_s + acc * (TC_ROWS * 8);
            float* db = d_s + acc * TC_ROWS;
#pragma unroll
            for (int q = 0; q < XPT; ++q) {
                const int i = etid + q * TC_EPI_WARPS * 32;
                if (i < T * 8) xb[i] = xreg[q];
            }
            if (etid < 2 * TC_ROWS) *reinterpret_cast<float4*>(dmb + etid * 4) = screg;
            else if (etid < 3 * TC_ROWS) db[etid - 2 * TC_ROWS] = screg.x;
            if (kb + 1 < kb_end) fetch(kb + 1);
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");  // epilogue warps only
            // Q4_K: minus sum over the 8 sub-blocks of fl(dmin*m) * sum(X). It does not need the accumulator: it runs
            // while the tensor core is still working on this block.
            if (p.pl_dm) {
                const float4 dm0 = *reinterpret_cast<const float4*>(dmb + my_row * 8), dm1 = *reinterpret_cast<const float4*>(dmb + my_row * 8 + 4);
                const float* xt = xb + th * TH * 8;
#pragma unroll
                for (int t = 0; t < TH; t += 2) {
                    const float4 xa0 = *reinterpret_cast<const float4*>(xt + t * 8), xa1 = *reinterpret_cast<const float4*>(xt + t * 8 + 4);
                    const float4 xc0 = *reinterpret_cast<const float4*>(xt + t * 8 + 8), xc1 = *reinterpret_cast<const float4*>(xt + t * 8 + 12);
                    float sa = dm0.x * xa0.x, sc = dm0.x * xc0.x;
                    sa = fmaf(dm0.y, xa0.y, sa); sc = fmaf(dm0.y, xc0.y, sc);
                    sa = fmaf(dm0.z, xa0.z, sa); sc = fmaf(dm0.z, xc0.z, sc);
                    sa = fmaf(dm0.w, xa0.w, sa); sc = fmaf(dm0.w, xc0.w, sc);
                    sa = fmaf(dm1.x, xa1.x, sa); sc = fmaf(dm1.x, xc1.x, sc);
                    sa = fmaf(dm1.y, xa1.y, sa); sc = fmaf(dm1.y, xc1.y, sc);
                    sa = fmaf(dm1.z, xa1.z, sa); sc = fmaf(dm1.z, xc1.z, sc);
                    sa = fmaf(dm1.w, xa1.w, sa); sc = fmaf(dm1.w, xc1.w, sc);
                    accf[t] -= sa;
                    accf[t + 1] -= sc;
                }
            }
            const float d = db[my_row];
            ok = mbar_wait(tfull + acc, (kbt >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tbase = tmem_base + acc * 256 + (uint32_t(q4 * 32) << 16) + th * TH;
            // sum_j 256^j v_j with few int->float conversions: neighbouring columns are joined in int32 first
            // (|v_j| < 2^23, so v_j + 256 v_{j+1} fits), as the reference joins its limb pairs (I0 = P0 + 256 P1,
            // src/cuda/model_cuda.cu:962-994); the top column of four limbs is small enough for the exact
            // add-a-constant conversion
            auto join = [&](const int(&w)[NL + 1][4], const int t0) {
                if constexpr (DBG) {
#pragma unroll
                    for (int j = 0; j <= NL; ++j)
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const int tok = tok0 + th * TH + t0 + t;
                            if (tok < p.B && R < p.rows16) p.dbgA[((int64_t(tok) * nblk + kb) * (NL + 1) + j) * p.rows16 + R] = w[j][t];
                        }
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int i01 = w[0][t] + (w[1][t] << 8), i23 = w[2][t] + (w[3][t] << 8);
                    float f = NL == 4 ? fmaf(i2f_small(w[NL][t]), 65536.0f, float(i23)) : float(i23);
                    f = fmaf(f, 65536.0f, float(i01));
                    accf[t0 + t] = fmaf(d, f, accf[t0 + t]);
                }
            };
            auto release = [&]() {  // accumulator in registers: the issuer may overwrite it
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty + acc);
            };
            if constexpr (TH <= 12) {  // every load of the drain is issued before the one wait, eight columns at a time
                int v[NL + 1][TH];
#pragma unroll
                for (int j = 0; j <= NL; ++j) {
                    if constexpr (TH >= 8) {
                        tmem_ld8(tbase + j * T, *reinterpret_cast<int(*)[8]>(&v[j][0]));
                        if constexpr (TH == 12) tmem_ld4(tbase + j * T + 8, *reinterpret_cast<int(*)[4]>(&v[j][8]));
                    } else {
                        tmem_ld4(tbase + j * T, *reinterpret_cast<int(*)[4]>(&v[j][0]));
                    }
                }
                tmem_ld_wait();
                release();
                if constexpr (DBG) {
#pragma unroll
                    for (int j = 0; j <= NL; ++j)
#pragma unroll
                        for (int t = 0; t < TH; ++t) {
                            const int tok = tok0 + th * TH + t;
                            if (tok < p.B && R < p.rows16) p.dbgA[((int64_t(tok) * nblk + kb) * (NL + 1) + j) * p.rows16 + R] = v[j][t];
                        }
                }
#pragma unroll
                for (int t = 0; t < TH; ++t) {
                    const int i01 = v[0][t] + (v[1][t] << 8), i23 = v[2][t] + (v[3][t] << 8);
                    float f = NL == 4 ? fmaf(i2f_small(v[NL][t]), 65536.0f, float(i23)) : float(i23);
                    f = fmaf(f, 65536.0f, float(i01));
                    accf[t] = fmaf(d, f, accf[t]);
                }
            } else {
                // Sixteen tokens of four columns would not leave room in the 96 registers a thread of this kernel can
                // have: the drain goes four tokens at a time, two such chunks in flight (the loads of chunk c + 1 are
                // issued before chunk c is worked on, so their latency is covered).
                int v[2][NL + 1][4];
#pragma unroll
                for (int j = 0; j <= NL; ++j) tmem_ld4(tbase + j * T, v[0][j]);
#pragma unroll
                for (int c = 0; c < TH / 4; ++c) {
                    tmem_ld_wait();
                    if (c + 1 < TH / 4) {
#pragma unroll
                        for (int j = 0; j <= NL; ++j) tmem_ld4(tbase + j * T + (c + 1) * 4, v[(c + 1) & 1][j]);
                    } else {
                        release();
                    }
                    join(v[c & 1], c * 4);
                }
            }
        }
        if (ok && is_tail) {  // not the tile's first blocks: leave the partial sums to the CTA that holds them
            float* sl = p.scratch + (size_t(blockIdx.x) * T + th * TH) * TC_ROWS + my_row;  // a warp stores 32 neighbours
#pragma unroll
            for (int t = 0; t < TH; ++t) sl[t * TC_ROWS] = accf[t];
            // (no fence per thread: the barrier orders the stores before thread 0, whose release store publishes them)
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
            if (etid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + blockIdx.x), "r"(*s_seq) : "memory");
            continue;
        }
        if (ok && is_open) {  // the tile's first blocks but not its last: add the pieces of the CTAs after this one
            const int c_last = ((pc.tile - p.waves * int(gridDim.x) + 1) * nkb - 1) / p.per;
            // the pieces finish at about the same time: the lanes of one warp wait for one flag each, then everybody
            // fetches the pieces, a few of them in flight at once, and adds them in CTA order
            if (warp == 0) {
                const unsigned seq = *s_seq;
                for (int c2 = int(blockIdx.x) + 1 + lane; c2 <= c_last; c2 += 32) {
                    unsigned seen = 0, it2 = 0;
                    do {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.flags + c2) : "memory");
                    } while (seen != seq && ++it2 < TC_SPIN_LIMIT);
                    if (seen != seq) *s_fail = 1;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
            if (*s_fail) ok = false;
            constexpr int G = TH >= 16 ? 1 : 16 / TH;  // pieces fetched together
            for (int c2 = int(blockIdx.x) + 1; c2 <= c_last && ok; c2 += G) {
                float part[G][TH >= 16 ? 4 : TH];
#pragma unroll
                for (int t0 = 0; t0 < TH; t0 += 4 * (TH >= 16 ? 1 : TH / 4)) {
                    constexpr int W = TH >= 16 ? 4 : TH;
#pragma unroll
                    for (int q = 0; q < G; ++q) {
                        const int cq = min(c2 + q, c_last);  // (a piece past the last one is read again and not added)
                        const float* sl = p.scratch + (size_t(cq) * T + th * TH + t0) * TC_ROWS + my_row;
#pragma unroll
                        for (int j = 0; j < W; ++j) part[q][j] = __ldcg(sl + j * TC_ROWS);
                    }
#pragma unroll
                    for (int q = 0; q < G; ++q)
                        if (c2 + q <= c_last) {
#pragma unroll
                            for (int j = 0; j < W; ++j) accf[t0 + j] += part[q][j];
                        }
                }
            }
        }
        if (ok) {
            // every load before the first store: Y may be the residual stream itself, and a load that has to wait for
            // the store before it turns the tile's output into a chain of memory round trips
            float sc[TH], res[TH];
#pragma unroll
            for (int t = 0; t < TH; ++t) {
                const int tok = tok0 + th * TH + t;
                sc[t] = tok < p.B ? __ldcg(p.inv_scale + tok) : 0.f;
                res[t] = p.epilogue == EPI_ADD && tok < p.B && R < p.rows ? __ldcg(p.resid + int64_t(tok) * p.ldy + R) : 0.f;
            }
#pragma unroll
            for (int t = 0; t < TH; ++t) {
                const int tok = tok0 + th * TH + t;
                const bool tok_ok = tok < p.B;
                const float y = accf[t] * sc[t];
                if (p.epilogue == EPI_SILU) {  // tile rows 0..7 gate, 8..15 up (16-row groups): partner is 8 lanes up
                    const float up = __shfl_down_sync(0xffffffffu, y, 8);
                    const int64_t o = R / 16 * 8 + (R & 7);
                    if (tok_ok && (lane & 8) == 0 && o < p.rows / 2)
                        p.Y[int64_t(tok) * p.ldy + o] = __fmul_rn(__fdiv_rn(y, 1.0f + expf(-y)), up);
                } else if (tok_ok && R < p.rows) {
                    const int64_t o = int64_t(tok) * p.ldy + R;
                    p.Y[o] = p.epilogue == EPI_ADD ? res[t] + y : y;
                }
            }
        }
        }
    }
    if (!ok) atomicExch(p.err, 2);
    // The next kernel of the stream may be launched now and set itself up while this CTA winds down (it still waits for
    // the whole grid before it reads anything). Not earlier: blocks that sit next to a working CTA for the length of a
    // large GEMM cost it issue slots (measured on the 32B shape: +3.7 % prompt time).
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == TC_EPI_WARPS + 1) tmem_dealloc(tmem_base, 512);
    if (tid == 0) {  // the last CTA to finish closes the launch (both words are read by the next launch only)
        if (atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1) {
            p.ctl[1] = 0;
            atomicAdd(p.ctl, 1u);
        }
    }
}

// ---------------------------------------------------------------- host side

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// int8 tensor [d2][d1][k] (k contiguous), box [1][box1][128], 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* map, const void* base, uint64_t k, uint64_t d1, uint64_t d2, uint32_t box1) {
    EncodeFn fn = encode_fn();
    if (!fn) return fail(ELB_ERR_CUDA, "matmul: cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[3] = {k, d1, d2};
    const cuuint64_t strides[2] = {k, k * d1};
    const cuuint32_t box[3] = {128, box1, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ELB_ERR_CUDA, "matmul: tensor map encoding failed");
    return ELB_OK;
}

int* error_word() {  // pinned, mapped: raised by a kernel whose bounded wait ran out
    static int* host = [] {
        int* p = nullptr;
        if (cudaHostAlloc(&p, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return static_cast<int*>(nullptr);
        *p = 0;
        return p;
    }();
    return host;
}

}  // namespace

static bool tc_prof_on() {
    static const bool on = [] { const char* v = std::getenv("ELB_TC_PROF"); return v && v[0] == '1'; }();
    return on;
}

bool gemm_tc_usable(const Weight* w, int B) {
    static const bool off = [] { const char* v = std::getenv("ELB_NO_TC"); return v && v[0] == '1'; }();
    // (batches below 16 rows run on the 16-token tile: the rows that are not there come in as zeros and are not stored)
    static const int min_b = [] { const char* v = std::getenv("ELB_TC_MIN_ROWS"); return v ? std::max(1, atoi(v)) : 2; }();
    return !off && w->planes && w->n_planes == 2 && w->n % 256 == 0 && w->n % 16 == 0 && B >= min_b && encode_fn() != nullptr;
}

int gemm_tc_check() {  // after a synchronize: did a tensor-core GEMM give up on a wait?
    if (tc_prof_on()) {
        unsigned long long h[12] = {};
        if (cudaMemcpyFromSymbol(h, g_tc_prof, sizeof h) == cudaSuccess && h[3])
            std::fprintf(stderr, "[tc prof] launches %llu: MMA issuer of CTA 0 waited %.1f%% for accumulators, %.1f%% for operands\n", h[3],
                         100.0 * double(h[0]) / double(h[2]), 100.0 * double(h[1]) / double(h[2]));
    }
    int* e = error_word();
    if (e && *e) {
        *e = 0;
        return fail(ELB_ERR_CUDA, "matmul: a bounded wait in the tensor-core kernel ran out");
    }
    return ELB_OK;
}

int gemm_tc_launch(const Weight* w, const int8_t* d_limbs, const float* d_inv_scale, const float* d_xsum, int B, int nl,
                   float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s, bool pdl, int32_t* d_dbg_acc) {
    if (!gemm_tc_usable(w, B)) return fail(ELB_ERR_STATE, "matmul: tensor-core path not usable for this weight");
    if (epilogue == EPI_SILU && !w->pair) return fail(ELB_ERR_INVALID, "matmul: SwiGLU epilogue needs a paired weight");
    int* err_host = error_word();
    int* err_dev = nullptr;
    if (!err_host || cudaHostGetDevicePointer(&err_dev, err_host, 0) != cudaSuccess) return fail(ELB_ERR_CUDA, "matmul: no error word");
    const int64_t rows16 = w->tiles * 16;
    CUtensorMap mapW, mapX;
    const bool four = nl >= 4;
    // tokens per tile: the widest tile for prompt chunks; 16 or 32 when that covers the batch (or wastes less of it)
    const int wide = tc_wide(four ? 4 : 3);
    const int T = B <= 16 ? 16 : B <= 32 ? 32 : B <= 64 && (B + 31) / 32 * 32 < (B + wide - 1) / wide * wide ? 32 : wide;
    ELB_TRY(make_map(&mapW, w->planes, uint64_t(w->n), uint64_t(rows16), 2, TC_ROWS));
    ELB_TRY(make_map(&mapX, d_limbs, uint64_t(w->n), uint64_t(B), 4, uint32_t(T)));
    const int row_tiles = int((rows16 + TC_ROWS - 1) / TC_ROWS), tok_tiles = (B + T - 1) / T;
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    const int64_t n_tiles = int64_t(row_tiles) * tok_tiles, nkb = w->n / 256;
    if (n_tiles * nkb >= (int64_t(1) << 31)) return fail(ELB_ERR_UNSUPPORTED, "matmul: too many tiles for 32-bit arithmetic");
    // persistent, one CTA per SM: whole waves of tiles, then the rest in equal shares of (tile, 256-block) units
    static const bool no_split = [] { const char* v = std::getenv("ELB_TC_NO_SPLIT"); return v && v[0] == '1'; }();
    const int waves = int(no_split ? (n_tiles + di.sm_count - 1) / di.sm_count : n_tiles / di.sm_count);
    const int64_t units = std::max<int64_t>(n_tiles - int64_t(waves) * di.sm_count, 0) * nkb;
    const int grid_n = waves > 0 ? int(std::min<int64_t>(n_tiles, di.sm_count)) : int(std::min<int64_t>(units, di.sm_count));
    const int per = int((units + grid_n - 1) / grid_n);
    // scratch of the shared tiles and the launch counter, once per device
    static thread_local float* scratch[64] = {};
    static thread_local unsigned* flags[64] = {};
    static thread_local unsigned* ctl[64] = {};
    if (!scratch[w->device]) {
        ELB_CUDA(cudaMalloc(&scratch[w->device], size_t(di.sm_count) * TC_ROWS * 64 * sizeof(float)));
        ELB_CUDA(cudaMalloc(&flags[w->device], size_t(di.sm_count) * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(flags[w->device], 0, size_t(di.sm_count) * sizeof(unsigned)));
        ELB_CUDA(cudaMalloc(&ctl[w->device], 2 * sizeof(unsigned)));
        ELB_CUDA(cudaMemset(ctl[w->device], 0, 2 * sizeof(unsigned)));
    }
    TcParams p{w->pl_d, w->pl_dm, d_xsum, d_inv_scale, d_y, d_resid, rows16, w->rows, ldy, B, int(w->n), epilogue,
               row_tiles, tok_tiles, waves, per, scratch[w->device], flags[w->device], ctl[w->device], err_dev, tc_prof_on() ? 1 : 0, d_dbg_acc};
    const dim3 grid{unsigned(grid_n)};
    auto launch = [&](auto kernel, int smem) -> int {
        ELB_TRY(ensure_dyn_smem(reinterpret_cast<const void*>(kernel), size_t(smem)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = size_t(smem);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        ELB_CUDA(cudaLaunchKernelEx(&cfg, kernel, mapW, mapX, p));
        return ELB_OK;
    };
#define ELB_TC_CASE(NL_, T_)                                                                            \
    if ((four ? 4 : 3) == NL_ && T == T_) {                                                             \
        if (d_dbg_acc) ELB_TRY(launch(k_gemm_tc<NL_, T_, true>, TcShape<NL_, T_>::SMEM));               \
        else ELB_TRY(launch(k_gemm_tc<NL_, T_, false>, TcShape<NL_, T_>::SMEM));                        \
    }
    ELB_TC_CASE(3, 16) ELB_TC_CASE(3, 32) ELB_TC_CASE(3, 64) ELB_TC_CASE(4, 16) ELB_TC_CASE(4, 32) ELB_TC_CASE(4, 48)
#undef ELB_TC_CASE
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
