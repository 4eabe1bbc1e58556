// One decode step (one token, batch 1) as ONE persistent cooperative kernel.
//
// At batch 1 every layer is a chain of five dependent steps (qkv matvec, attention, output projection, gate|up, down),
// each a few microseconds of HBM traffic on this GPU: launched as separate kernels they are bound by launch and
// dependency latency, not by bandwidth. Here one CTA per SM stays resident for the whole step and walks the chain with
// grid-wide barriers between the steps:
//   * every working warp owns a fixed, contiguous share of the (row tile, k block) units of every weight matrix of the
//     step, in execution order — one long "unit stream" — and one more warp, which does nothing else, keeps every
//     working warp's ring in shared memory as full as it gets (a byte ring: units of different block formats lie back
//     to back; every unit is one bulk copy that reports to an mbarrier), no matter which phase the CTA is in: HBM
//     keeps streaming through barriers, attention and activation conversion, and the working warps spend no
//     instruction on requesting data;
//   * the activation of a matvec is converted to int8 limbs redundantly by every CTA (shared memory), from the fp32
//     vector and a global maximum (atomicMax, order independent) or the sums that the producing phase left: no serial
//     single-CTA section;
//   * no phase ends with an exchange between CTAs: q, k, v and gate|up are cut in whole row tiles; attn_output and
//     ffn_down, which have few row tiles and long rows, are cut in equal unit ranges instead, a row tile then has at most
//     two contributing CTAs: the one with the tile's first blocks adds the residual stream to its partial sums, the other
//     leaves its partial sums in a second buffer, and the next conversion adds the two on every CTA: deterministic;
//   * everything a phase needs to find its data (matrix shapes, base pointers, block formats) lies in the kernel's
//     parameter block, and the code is kept small (loops are rolled, the phases are functions): a kernel of this length
//     runs every piece of its code once per layer, so it is bound by instruction fetch as soon as it outgrows the
//     instruction cache.
// Barrier waits are bounded: on timeout the kernel raises an error word, drains its copies and leaves.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "split.cuh"
#include "gemv_core.cuh"
#include "layout.cuh"
#include "decode.cuh"

namespace elb {

constexpr int DK_THREADS = 512, DK_WARPS = DK_THREADS / 32;  // the working warps
// The CTA is launched with one more warpgroup (four warps, the unit in which registers can be handed over): its first
// warp is the producer, the other three leave at once. Registers per thread: the compiler sizes the kernel for
// 65536 / 640 = 96; the extra warpgroup then shrinks to DK_REGS_PRODUCER and the working warps grow to DK_REGS_WORKER.
// The working warps can only take what the extra warpgroup has given back (registers the CTA never held are not in
// its pool, and a warp asking for more than the pool holds waits for ever): 4 * 32 * (96 - 32) = 8192 registers released,
// 16 * 32 * (112 - 96) = 8192 taken.
constexpr int DK_CTA_THREADS = DK_THREADS + 128;
constexpr int DK_REGS_LAUNCH = 96, DK_REGS_WORKER = 112, DK_REGS_PRODUCER = 32;
static_assert(4 * 32 * (DK_REGS_LAUNCH - DK_REGS_PRODUCER) >= DK_THREADS * (DK_REGS_WORKER - DK_REGS_LAUNCH),
              "the working warps would wait for registers that nobody releases");
constexpr int DK_NBAR = 8;  // mbarriers per warp = most units a warp can have requested and not yet consumed
// How long the producer warp sleeps when no ring has room (ns). It shares a scheduler with four working warps:
// 500-1000 ns measured 0.6 % faster per step than 40 ns, 2000 ns 2 % slower (the rings run dry).
#ifndef DK_PRODUCER_NAP
#define DK_PRODUCER_NAP 500
#endif
constexpr int DK_HD = 128, DK_KT = 40, DK_KS = DK_HD + 4, DK_MAXG = 8;  // DK_KS: row stride of the K tile (float4 reads without bank conflicts)
constexpr int DK_MAXSPLIT = 18;         // key splits of one KV head (their partial results are staged in the K/V tile area)
constexpr int DK_PS = DK_HD + 4;        // floats per (split, head) of the attention's partial results: 128 outputs, m, l, padding
constexpr unsigned DK_SPIN_LIMIT = 1u << 22;
constexpr unsigned DK_XSPIN_LIMIT = 1u << 24;  // waits on another GPU (x ~100 ns: about two seconds)
constexpr unsigned DK_MBAR_LIMIT = 1u << 17;   // tries of one wait for a weight unit (each try blocks for a while in hardware)

// CTA barrier of the working warps (the producer warp runs on its own): a named barrier over DK_THREADS threads
__device__ __forceinline__ void dk_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DK_THREADS) : "memory"); }

// ---------------------------------------------------------------- grid barrier (bounded)

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// All CTAs arrive, then leave together. `target` is the arrival count that completes this CTA's next barrier (the
// counter is never reset: a launch starts from launches * barriers per launch * CTAs). Returns false when the wait ran
// out (or an earlier one did): the caller stops working, every later barrier returns at once.
// peers: the barrier covers the CTAs of ALL tensor-parallel ranks: exchange number x (counted from the first launch,
// the same on every rank) is complete when every rank's CTAs have arrived. Every CTA waits for the local arrivals; CTA 0
// then raises this rank's flag of set x & 1 on every peer (system-scope release); every CTA waits for the peers' flags
// in its own rank's flag words. What a CTA stored to its peers before the barrier is fenced once, by its arriving thread.
__device__ __noinline__ bool grid_barrier(const DkParams& p, unsigned& target, int* s_dead, bool peers = false, unsigned x = 0, int ev = -1) {
    dk_sync();
    if (ev >= 0 && threadIdx.x == 0) {  // diagnostics: when this CTA arrived
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.prof_cta[blockIdx.x * 16 + 2 * ev] = t;
    }
    if (threadIdx.x == 0 && !*s_dead) {
        if (peers) __threadfence_system();  // the CTA's peer stores (ordered before this thread by the CTA barrier)
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar) : "memory");  // orders the CTA's writes before it
        target += gridDim.x;
        unsigned it = 0;
        bool dead = false;
        while (!dead && int(ld_acquire(p.bar) - target) < 0)
            if (++it > DK_SPIN_LIMIT) dead = true; else if (it > 2048) __nanosleep(64);
        // (no fence here: the acquire load that saw the last arrival synchronises with every CTA's release, and the
        // CTA barrier below carries that to the other threads)
        if (peers) {
            const int set = int(x & 1u);
            unsigned* mine = p.flag_peer[p.tp_rank];
            if (blockIdx.x == 0 && !dead)
                for (int q = 0; q < p.tp_size; ++q)
                    if (q != p.tp_rank) st_release_sys(p.flag_peer[q] + set * 8 + p.tp_rank, x + 1);
            for (int q = 0; q < p.tp_size && !dead; ++q) {  // every CTA watches the peers' flags itself: no second hop
                if (q == p.tp_rank) continue;
                it = 0;
                while (!dead && ld_acquire_sys(mine + set * 8 + q) != x + 1)
                    if (++it > DK_XSPIN_LIMIT) dead = true; else if (it > 256) __nanosleep(100);
            }
        }
        if (dead) {
            *s_dead = 1;
            atomicExch(p.err, 1);
        }
    }
    if (ev >= 0 && threadIdx.x == 0) {  // ... and when it saw the barrier complete
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.prof_cta[blockIdx.x * 16 + 2 * ev + 1] = t;
    }
    dk_sync();
    return !*s_dead;
}

// ---------------------------------------------------------------- activation -> limbs in shared memory

// The split activation of a matvec: int8 limbs [4][n_pad], the sums of each limb over the 32-wide (Q4_K's min term) and
// 16-wide (Q6_K's offset) sub-blocks as two balanced base-256 digits each, in the layout the matvec's extra MMA reads
// (split.cuh), and one power-of-two scale per 256-block: here every 256-block is split on its own, with the shift
// k = 8 nl - 2 - e of its own largest magnitude (k_split8 of the reference, src/cuda/model_cuda.cu:701-729, applied per
// block; the matvec multiplies each block's exact integer sums by 2^-k of that block). A block is then converted
// without knowing anything about the rest of the vector: no maximum over the whole vector has to be agreed on.
struct ActSmem {
    int8_t* lim;    // [4][n_pad]
    int8_t* sd32;   // [n/256][8][8]
    int8_t* sd16;   // [n/256][8][16]
    float* bscale;  // [n/256] 2^-k of each block
    int n_pad;
};
__host__ __device__ inline size_t dk_act_bytes(int n) {  // limbs, sums, scales (a multiple of 16)
    return (size_t(4) * (n + 32) + size_t(n / 256) * 192 + size_t(n / 256) * 4 + 15) / 16 * 16;
}
__device__ __forceinline__ ActSmem act_at(int8_t* base, int n) {
    ActSmem a;
    a.lim = base;
    a.n_pad = n + 32;
    a.sd32 = a.lim + 4 * a.n_pad;
    a.sd16 = a.sd32 + (n / 256) * 64;
    a.bscale = reinterpret_cast<float*>(a.sd16 + (n / 256) * 128);
    return a;
}
__device__ __forceinline__ int sd_need(int type) { return type == ELB_Q4_K ? 1 : type == ELB_Q6_K ? 2 : 0; }
__device__ __forceinline__ int unit_bytes_of(int type) { return type == ELB_Q4_K ? Q4K_UNIT : type == ELB_Q6_K ? Q6K_UNIT : Q8_UNIT; }
// 1 / sqrt(x) in double from the single-precision estimate and two Newton steps (relative error ~1e-27 of the exact
// value before the last rounding): what the reference's 1.0 / sqrt(x) in double gives, after rounding to float,
// without the division and square root routines
__device__ __forceinline__ double rsqrt_d(double x) {
    double y = double(rsqrtf(float(x)));
    y = y * fma(-0.5 * x, y * y, 1.5);
    y = y * fma(-0.5 * x, y * y, 1.5);
    return y;
}
__device__ __forceinline__ float pow2_neg(int k) { return k <= 126 ? __int_as_float((127 - k) << 23) : ldexpf(1.0f, -k); }

// Four consecutive fixed-point values -> one packed word of each of the 4 limbs (balanced base-256 digits: adding 128 at
// every byte position turns them into the ordinary digits of v + 0x80808080; a 4x4 byte transpose groups them by limb).
__device__ __forceinline__ void limb_words(const float4& f, const Pow2 sc, uint32_t (&w)[4]) {
    const uint32_t a = (uint32_t(__float2int_rn(f.x * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t b = (uint32_t(__float2int_rn(f.y * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t c = (uint32_t(__float2int_rn(f.z * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t d = (uint32_t(__float2int_rn(f.w * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t ab01 = __byte_perm(a, b, 0x5140), ab23 = __byte_perm(a, b, 0x7362);  // a0 b0 a1 b1 | a2 b2 a3 b3
    const uint32_t cd01 = __byte_perm(c, d, 0x5140), cd23 = __byte_perm(c, d, 0x7362);
    w[0] = __byte_perm(ab01, cd01, 0x5410);
    w[1] = __byte_perm(ab01, cd01, 0x7632);
    w[2] = __byte_perm(ab23, cd23, 0x5410);
    w[3] = __byte_perm(ab23, cd23, 0x7632);
}

// One warp splits 256-block b of a vector: lane holds its values 8*lane .. 8*lane+7 in v0, v1. Writes limbs, sub-block
// sums (shuffles over the 2 / 4 neighbouring lanes that hold the rest of a sub-block; the sums of two limbs travel in
// the halves of one word: |sum of 32 int8| < 2^12) and the block's scale. Every lane of the warp must call this together.
__device__ __forceinline__ void split_block(const float4& v0, const float4& v1, const int b, const int nl, const ActSmem& a,
                                            const int sd_mask, const int lane) {
    float m = fmaxf(absmax4(v0), absmax4(v1));
    m = warp_max(m);
    const int k = split_shift(m, nl);
    const Pow2 sc = make_pow2(k);
    uint32_t w0[4], w1[4];
    limb_words(v0, sc, w0);
    limb_words(v1, sc, w1);
    const int idx = b * 256 + lane * 8;
#pragma unroll
    for (int l = 0; l < 4; ++l) *reinterpret_cast<uint2*>(a.lim + l * a.n_pad + idx) = make_uint2(w0[l], w1[l]);
    if (sd_mask) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // limbs 2h and 2h+1 together
            const int sa = __dp4a(int(w1[2 * h]), 0x01010101, __dp4a(int(w0[2 * h]), 0x01010101, 0));
            const int sb = __dp4a(int(w1[2 * h + 1]), 0x01010101, __dp4a(int(w0[2 * h + 1]), 0x01010101, 0));
            int pk = sa + (sb << 16);  // (the low half may borrow from the high one: undone when they are taken apart)
            const int p16 = pk + __shfl_xor_sync(0xffffffffu, pk, 1);
            const int p32 = p16 + __shfl_xor_sync(0xffffffffu, p16, 2);
#pragma unroll
            for (int wd = 0; wd < 2; ++wd) {
                if (!(sd_mask & (wd ? 1 : 2))) continue;
                const int pw = wd ? p32 : p16, per = wd ? 8 : 16, si = wd ? lane >> 2 : lane >> 1;
                if ((lane & (wd ? 3 : 1)) != 0) continue;
                int8_t* sd = wd ? a.sd32 : a.sd16;
                const int s_lo = int(short(pw & 0xFFFF)), s_hi = (pw - s_lo) >> 16;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int sum = e ? s_hi : s_lo, l = 2 * h + e;
                    const int lo = ((sum + 128) & 255) - 128;
                    sd[(b * 8 + l) * per + si] = int8_t(lo);
                    sd[(b * 8 + 4 + l) * per + si] = int8_t((sum - lo) >> 8);
                }
            }
        }
    }
    if (lane == 0) a.bscale[b] = pow2_neg(k);
}

// Activation of the next matvec -> split blocks [b0, b1) of the vector A (+ B when B is not null: the two buffers of
// partial sums a row-parallel matvec left, the first of which already holds the residual stream), read through L2
// (written by other CTAs before the last barrier); warp w takes blocks b0 + w, b0 + w + 16, ...
//  * NORM (the residual stream in front of attn_norm / ffn_norm / output_norm): the blocks of (A + B) * norm_w are
//    split and the factor 1 / sqrt(mean(x^2) + eps) of the RMSNorm (src/ops.cpp:155-160 of the reference, sum of squares
//    in double) is returned for the matvec to apply to its row sums: no block has to wait for the sum over the vector.
//    CTA c also stores its slice of A + B to `out` (when not null), the residual stream the next row-parallel matvec
//    adds to.
//  * otherwise the blocks of A are split as they are; returns 1.
// Ends with a CTA barrier: the limbs are visible to every warp.
template <bool NORM>
__device__ __noinline__ float convert_act(const float* A, const float* B, float* out, const int n, const int b0, const int b1,
                                          const float* norm_w, const float eps, const int nl, const ActSmem a, double* red,
                                          const int sd_mask) {
    constexpr int NB = NORM ? 2 : 3;  // blocks of a warp in flight together: every load of a pass is issued before the first use
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q4 = n / 4, lo = out ? range_lo(q4, gridDim.x, blockIdx.x) : 0, hi = out ? range_lo(q4, gridDim.x, blockIdx.x + 1) : 0;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    double ss = 0.0;
#pragma unroll 1
    for (int bb = b0 + warp; bb < b1; bb += NB * DK_WARPS) {
        float4 v[NB][2], w[NB][2];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int b = bb + j * DK_WARPS;
            const bool on = b < b1;
            const float4* pa = reinterpret_cast<const float4*>(A + size_t(b) * 256) + lane * 2;
            v[j][0] = on ? __ldcg(pa) : z;
            v[j][1] = on ? __ldcg(pa + 1) : z;
            if (NORM) {
                const float4* pb = reinterpret_cast<const float4*>(B + size_t(b) * 256) + lane * 2;
                w[j][0] = on && B ? __ldcg(pb) : z;
                w[j][1] = on && B ? __ldcg(pb + 1) : z;
            }
        }
        if (NORM) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = bb + j * DK_WARPS;
                const bool on = b < b1;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float4& x = v[j][h];
                    x.x = __fadd_rn(x.x, w[j][h].x); x.y = __fadd_rn(x.y, w[j][h].y);
                    x.z = __fadd_rn(x.z, w[j][h].z); x.w = __fadd_rn(x.w, w[j][h].w);
                    w[j][h] = on ? __ldg(reinterpret_cast<const float4*>(norm_w + size_t(b) * 256) + lane * 2 + h) : z;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int b = bb + j * DK_WARPS;
            if (b >= b1) continue;  // (warp-uniform)
            if (NORM) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float4& x = v[j][h];
                    const int i4 = b * 64 + lane * 2 + h;
                    if (i4 >= lo && i4 < hi) *reinterpret_cast<float4*>(out + size_t(i4) * 4) = x;
                    ss += double(x.x) * x.x + double(x.y) * x.y + double(x.z) * x.z + double(x.w) * x.w;
                    x.x = __fmul_rn(x.x, w[j][h].x); x.y = __fmul_rn(x.y, w[j][h].y);
                    x.z = __fmul_rn(x.z, w[j][h].z); x.w = __fmul_rn(x.w, w[j][h].w);
                }
            }
            split_block(v[j][0], v[j][1], b, nl, a, sd_mask, lane);
        }
    }
    if (NORM) {
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
    }
    dk_sync();
    float inv = 1.0f;
    if (NORM) {
        double S = 0.0;
#pragma unroll
        for (int i = 0; i < DK_WARPS; ++i) S += red[i];  // fixed order
        inv = float(rsqrt_d(S / n + double(eps)));
    }
    return inv;
}

// Tensor parallelism: a row-parallel matvec stores every partial sum, on every rank, as an 8-byte word {value, number of
// the exchange + 1}: data and "it has arrived" travel in one store, so there is neither a fence behind the peer stores nor
// a barrier in front of the reduction. CTA c waits (bounded) for its slice of the two vectors of every rank in its own
// rank's copy of the set, adds them in rank order — the same order on every rank, so the residual stream stays
// bit-identical everywhere (rank 0's first vector carries the old stream) — and stores the slice to `out`; the CTAs then
// meet at the grid barrier of this GPU and the conversion reads `out` alone. A set is written again two exchanges
// later, when every rank has passed the barrier behind this reduction.
__device__ __noinline__ void reduce_ranks(const DkParams& p, const uint2* set, float* out, const unsigned tag, int* s_dead) {
    const int q4 = p.E / 4, lo = range_lo(q4, gridDim.x, blockIdx.x), hi = range_lo(q4, gridDim.x, blockIdx.x + 1);
    const int nv = p.tp_size * p.pv;
#pragma unroll 1
    for (int i4 = lo + int(threadIdx.x); i4 < hi; i4 += DK_THREADS) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int q = 0; q < nv; ++q) {
            const uint4* src = reinterpret_cast<const uint4*>(set + size_t(q) * p.E + size_t(i4) * 4);
            uint4 a, b;
            unsigned it = 0;
            while (true) {
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 1) : "memory");
                if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) break;
                if (++it > DK_XSPIN_LIMIT || *reinterpret_cast<volatile int*>(s_dead)) {
                    if (!*reinterpret_cast<volatile int*>(s_dead)) { *s_dead = 1; atomicExch(p.err, 1); }
                    break;
                }
                if (it > 64) __nanosleep(100);
            }
            if (q == 0) {
                v = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
            } else {
                v.x = __fadd_rn(v.x, __uint_as_float(a.x)); v.y = __fadd_rn(v.y, __uint_as_float(a.z));
                v.z = __fadd_rn(v.z, __uint_as_float(b.x)); v.w = __fadd_rn(v.w, __uint_as_float(b.z));
            }
        }
        reinterpret_cast<float4*>(out)[i4] = v;
    }
}

__device__ __forceinline__ void dk_stamp(const DkParams& p, int l, int ev) {
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.prof[l * 32 + ev] = t;
    }
}

// ---------------------------------------------------------------- the unit stream of one warp

// Matrices of the step in execution order: per layer qkv segments, wo, gate|up, down; then the head. Matrix `i` of
// layer `l` (l == n_layer, i == 0: the head). Every layer has the same shapes, so the way a matrix is shared between
// CTAs and warps depends only on its kind.
__device__ __forceinline__ int kind_li(const DkParams& p, int l, int i) { return l >= p.n_layer ? 6 : i < p.n_qkv ? i : 3 + i - p.n_qkv; }

// The CTA's share of a matrix as a range of units [cA, cB), cut into equal ranges for its warps [wA, wB).
// Whole tiles of the matrix's group by default (no tile is shared between CTAs: the phase ends without any exchange;
// a group with fewer tiles than CTAs occupies the first CTAs only); equal unit ranges for a balanced matrix.
struct WarpRange { int cA, cB, wA, wB; };
__device__ __noinline__ WarpRange warp_range(const DkKind& m, int warp) {
    const int c = blockIdx.x;
    WarpRange r;
    if (m.balanced) {
        const int U = m.tiles * m.upt;
        r.cA = range_lo(U, gridDim.x, c);
        r.cB = range_lo(U, gridDim.x, c + 1);
    } else {
        const int G = min(int(gridDim.x), m.group_tiles);
        if (m.group_cost > 0) {  // CTA c takes the tiles whose cost position lies in [C c / G, C (c + 1) / G)
            auto bound = [&](int cc) {  // first tile of this matrix at or behind the cost position of boundary cc
                const long long rel = (long long)m.group_cost * cc / G - m.group_cost_off;
                return rel <= 0 ? 0 : int(min((rel + m.cost - 1) / m.cost, (long long)m.tiles));
            };
            r.cA = (c < G ? bound(c) : m.tiles) * m.upt;
            r.cB = (c < G ? bound(c + 1) : m.tiles) * m.upt;
        } else {
            const int gA = c < G ? range_lo(m.group_tiles, G, c) : 0, gB = c < G ? range_lo(m.group_tiles, G, c + 1) : 0;
            r.cA = min(max(gA - m.group_off, 0), m.tiles) * m.upt;
            r.cB = min(max(gB - m.group_off, 0), m.tiles) * m.upt;
        }
    }
    r.wA = r.cA + range_lo(r.cB - r.cA, DK_WARPS, warp);
    r.wB = r.cA + range_lo(r.cB - r.cA, DK_WARPS, warp + 1);
    return r;
}

// The shares of a warp (and of its CTA) in the matrices of every kind are computed once, when the kernel starts, and
// kept in shared memory: warp[kind] = {wA, wB} and tiles[kind] = {first row tile, last row tile} of this warp's share,
// cta[kind] = {cA, cB}.
struct Sched {
    const int2* warp;   // this warp's [DK_KINDS]
    const int2* tiles;  // all warps' [DK_WARPS][DK_KINDS]
    const int2* cta;    // [DK_KINDS]
};

// Prefetch cursor: the next unit of a warp's stream that has not been requested yet.
struct Cursor {
    int l, i, u, end, unit_bytes;  // matrix i of layer l (l > n_layer: the stream has ended)
    const uint8_t* W;
};
__device__ __forceinline__ bool cursor_live(const DkParams& p, const Cursor& c) { return c.l <= p.n_layer; }
__device__ __forceinline__ void cursor_next_matrix(const DkParams& p, Cursor& c) {
    if (c.l >= p.n_layer || ++c.i == p.n_qkv + 3) { c.i = 0; ++c.l; }
}
__device__ __forceinline__ void cursor_seek(const DkParams& p, Cursor& c, const int2* sched_warp) {  // first non-empty range from (l, i) on
    while (cursor_live(p, c)) {
        const int2 r = sched_warp[kind_li(p, c.l, c.i)];
        if (r.x < r.y) {
            c.u = r.x; c.end = r.y; c.W = p.W[c.l][c.i]; c.unit_bytes = unit_bytes_of(p.wtype[c.l][c.i]);
            return;
        }
        cursor_next_matrix(p, c);
    }
}

// The ring of one working warp: `bytes` bytes of shared memory that the units of the warp's stream pass through in
// order. A unit is requested with one bulk copy (global -> shared, completion counted in bytes on an mbarrier) by the
// producer warp (its lane w serves working warp w) and consumed by the working warp; its place is given up when the
// arithmetic on it is done. Units are placed back to back; one that would cross the end of the ring starts at offset 0
// instead and the bytes left over count as used until the consumer has passed them too (consumer and producer walk the
// same sequence of unit sizes, so both take the same decisions). Unit number q of the warp (counted from the start of
// the kernel) reports to mbarrier q % DK_NBAR, whose phase for it has parity (q / DK_NBAR) & 1; the ring is at most
// DK_NBAR of the smallest units long, so no more than DK_NBAR units are ever on request. The consumer tells the producer
// how far it has come through one word of shared memory: the number of bytes it has given up since the kernel started.
struct RingShared {       // in shared memory, one set for the CTA
    unsigned freed[DK_WARPS];    // bytes given up by working warp w so far (gaps included)
    unsigned issued[DK_WARPS];   // units requested for warp w in all, written when the producer ends
    int producer_done;
};
struct Ring {             // consumer side, in registers of the working warp
    uint32_t base;        // shared-memory addresses (32 bit) of the ring's first byte and of its first mbarrier
    uint32_t bars;
    int bytes;
    int c_off;            // offset of the next unit to consume (before the wrap rule is applied)
    unsigned c_seq;       // units given up so far
    unsigned freed;       // bytes given up so far
    uint32_t freed_out;   // where the producer reads it (shared-memory address)
};

__device__ __forceinline__ uint32_t dk_smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ const uint8_t* dk_smem_ptr(uint32_t a) { return static_cast<const uint8_t*>(__cvta_shared_to_generic(size_t(a))); }

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// The producer warp: lane w < DK_WARPS walks the stream of working warp w and requests its units as room appears in that
// warp's ring. All lanes run in step, so the bookkeeping is paid once for the sixteen rings. Ends when every stream
// has been requested to its end, when the step is given up (dead flag), or when nothing has moved for too long.
__device__ __noinline__ void producer_warp(const DkParams& p, const uint32_t ring0, const int ring_bytes, const uint32_t bars0,
                                           const int2* sched_all, RingShared* rs, const int* s_dead, const int lane) {
    const bool mine = lane < DK_WARPS;
    const int2* sched_warp = sched_all + (mine ? lane : 0) * DK_KINDS;
    Cursor c;
    c.l = 0;
    c.i = 0;
    c.u = c.end = c.unit_bytes = 0;
    c.W = nullptr;
    if (mine) cursor_seek(p, c, sched_warp);
    else c.l = p.n_layer + 1;
    const uint32_t base = ring0 + uint32_t(lane * ring_bytes), bars = bars0 + uint32_t(lane * DK_NBAR) * 8u;
    unsigned issued = 0, seq = 0, idle = 0;
    int off = 0;
    const volatile unsigned* freed = rs->freed + (mine ? lane : 0);
    while (true) {
        const bool live = cursor_live(p, c);
        if (!__any_sync(0xffffffffu, live)) break;
        bool did = false;
        if (live) {
            const int ub = c.unit_bytes;
            const bool wrap = off + ub > ring_bytes;
            const int need = wrap ? ring_bytes - off + ub : ub;
            if (int(issued - *freed) + need <= ring_bytes) {
                if (wrap) off = 0;
                const uint32_t bar = bars + (seq % DK_NBAR) * 8u;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(ub) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(base + uint32_t(off)), "l"(c.W + size_t(c.u) * ub), "r"(ub), "r"(bar)
                             : "memory");
                issued += unsigned(need);
                off += ub;
                ++seq;
                did = true;
                if (++c.u == c.end) {
                    cursor_next_matrix(p, c);
                    cursor_seek(p, c, sched_warp);
                }
            }
        }
        if (__any_sync(0xffffffffu, did)) {
            idle = 0;
        } else {
            if (*reinterpret_cast<const volatile int*>(s_dead) || ++idle > DK_SPIN_LIMIT) break;
            __nanosleep(DK_PRODUCER_NAP);
        }
    }
    if (mine) rs->issued[lane] = seq;
    __syncwarp();
    if (lane == 0) {
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&rs->producer_done) = 1;
    }
}

// Wait (bounded) until the oldest requested unit, of `ub` bytes, has arrived; returns where it lies. On timeout the
// dead flag and the error word are raised and the caller goes on with whatever the ring holds: the next grid barrier
// ends the step.
__device__ __forceinline__ uint32_t ring_front(const DkParams& p, Ring& r, int ub, int* s_dead) {
    if (r.c_off + ub > r.bytes) {  // the producer skipped the end of the ring for this unit
        r.freed += unsigned(r.bytes - r.c_off);
        r.c_off = 0;
    }
    const uint32_t bar = r.bars + (r.c_seq % DK_NBAR) * 8u, parity = (r.c_seq / DK_NBAR) & 1u;
    bool done = false;
#pragma unroll 1
    for (unsigned it = 0; it < DK_MBAR_LIMIT && !done; ++it) done = mbar_try(bar, parity);
    if (!done && !*s_dead) {
        *s_dead = 1;
        atomicExch(p.err, 1);
    }
    return r.base + uint32_t(r.c_off);
}
// The unit at the front has been used up by every lane (the caller has synchronised the warp): its bytes are free again.
__device__ __forceinline__ void ring_pop(Ring& r, int ub, int lane) {
    r.c_off += ub;
    r.freed += unsigned(ub);
    ++r.c_seq;
    if (lane == 0) asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(r.freed_out), "r"(r.freed) : "memory");
}
// Before the kernel ends: the producer must have stopped and every copy it requested must have landed (bounded waits).
__device__ __noinline__ void ring_drain(Ring& r, const RingShared* rs, int warp) {
    unsigned it = 0;
    while (!*reinterpret_cast<const volatile int*>(&rs->producer_done) && ++it < DK_SPIN_LIMIT) __nanosleep(100);
    const unsigned end = *reinterpret_cast<const volatile unsigned*>(&rs->issued[warp]);
    for (; r.c_seq != end; ++r.c_seq) {
        const uint32_t bar = r.bars + (r.c_seq % DK_NBAR) * 8u, parity = (r.c_seq / DK_NBAR) & 1u;
        bool done = false;
        for (unsigned j = 0; j < DK_MBAR_LIMIT && !done; ++j) done = mbar_try(bar, parity);
    }
}

// ---------------------------------------------------------------- one matvec phase

enum { DK_EPI_STORE = 0, DK_EPI_PART = 1, DK_EPI_SILU = 2, DK_EPI_LOGITS = 3 };

struct PhaseSmem {
    Sched sched;
    ActSmem act;
    float* red;      // [DK_WARPS][slots][16] row sums of each warp's share, per row tile it touches
    float* outs;     // [cta_tiles][16] row sums of the CTA's share
    double* red8;    // [DK_WARPS]
    int* flags;      // [4]: attention: last-arriver flag (0); dead (2)
};

template <int TYPE, bool CG>
__device__ void run_units(const DkParams& p, const int upt, const int wA, const int wB, Ring& rg, const PhaseSmem& s, int warp,
                          int lane) {
    const int g = lane >> 2, t = lane & 3;
    constexpr int UB = TYPE == ELB_Q4_K ? Q4K_UNIT : TYPE == ELB_Q6_K ? Q6K_UNIT : Q8_UNIT;
    const int8_t* sd = TYPE == ELB_Q6_K ? s.act.sd16 : s.act.sd32;
    Acc a{{0.f, 0.f}, {0.f, 0.f}};
    int slot = 0;
    int b = wA % upt;
    const float wt = t < 2 ? (t & 1 ? 65536.0f : 1.0f) : 0.0f;
    const float wtm = (t & 1 ? 65536.0f : 1.0f) * (t & 2 ? 256.0f : 1.0f);
    DbgOut dbg{nullptr, nullptr, nullptr, 0, 0, 0, 0};
#pragma unroll 1
    for (int u = wA; u < wB; ++u) {
        Unit<TYPE> cur;
        load_unit(cur, dk_smem_ptr(ring_front(p, rg, UB, &s.flags[2])), lane);
        compute_unit<false, CG>(cur, b, s.act.lim, s.act.n_pad, sd, lane, a, dbg, s.act.bscale);
        __syncwarp();  // every lane has its fragments of the unit in registers and has used them
        ring_pop(rg, UB, lane);
        if (++b == upt || u + 1 == wB) {
            float v0 = a.acc[0] * wt - a.accm[0] * wtm, v1 = a.acc[1] * wt - a.accm[1] * wtm;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (t == 0) {
                s.red[(warp * p.slots + slot) * 16 + g] = v0;
                s.red[(warp * p.slots + slot) * 16 + g + 8] = v1;
            }
            ++slot;
            a = Acc{{0.f, 0.f}, {0.f, 0.f}};
            b = 0;
        }
    }
}

// What the epilogue of a matvec needs besides its sums
struct EpiArgs {
    int epi;
    float* y;               // STORE / SILU: output vector
    float inv;              // factor of the row sums: 1 / rms of the RMSNorm in front of the matvec, or 1
    int xset;               // PART: set of partial-sum buffers
    unsigned tag;           // PART under tensor parallelism: number of the exchange + 1, stored with every partial sum
    const float* x_old;     // PART: the residual stream the first contributor of a tile adds (null: nothing is added)
};

// y = W * act for one matrix; the activation limbs are already in shared memory (GACT: in global memory, written by other
// CTAs before the last barrier, read through L2). Ends with this CTA's share written:
//   DK_EPI_STORE      y[row] = sum                       (whole tiles)
//   DK_EPI_SILU       y[o] = silu(gate) * up              (whole tiles of a gate|up pair)
//   DK_EPI_PART       partial sums of a balanced matrix: the CTA that holds a tile's first unit writes x_old + sum to
//                     vector 0, the one that holds its last unit (when it is another CTA) its sum to vector 1 of this
//                     rank's pair in set `xset`; a CTA that holds the whole tile writes zeros to vector 1. Stored on every
//                     tensor-parallel rank; the consumer adds the vectors.
//   DK_EPI_LOGITS     y[v0 + row] = sum on every tensor-parallel rank (this rank's vocabulary rows of the head)
template <bool GACT>
__device__ __forceinline__ void matvec_phase(const DkParams& p, const int type, const int kind, const EpiArgs& ea, Ring& rg,
                                          const PhaseSmem& s, bool after_matrix, bool gact) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, upt = p.kind[kind].upt, rows = p.kind[kind].rows;
    const int2 rc = s.sched.cta[kind], rw = s.sched.warp[kind];
    // the residual stream the first contributor of a row tile adds: asked for now, used after the units
    float xo = 0.f;
    if (ea.x_old && rc.x < rc.y) {
        const int Xf0 = rc.x / upt;
        const int64_t r = 16 * int64_t(Xf0) + tid;
        if (tid < ((rc.y - 1) / upt - Xf0 + 1) * 16 && r < rows && rc.x <= (Xf0 + (tid >> 4)) * upt) xo = __ldcg(ea.x_old + r);
    }
    // the reduction buffers may still be read by the previous matrix of the same phase (q, k, v); the first matrix
    // comes straight from the conversion, which ends with a CTA barrier
    if (after_matrix) dk_sync();
    if (GACT && gact) {  // (only the kernel for models with a long FFN activation carries this code)
        switch (type) {
            case ELB_Q4_K: run_units<ELB_Q4_K, GACT>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
            case ELB_Q6_K: run_units<ELB_Q6_K, GACT>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
            default: run_units<ELB_Q8_0, GACT>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
        }
    } else {
        switch (type) {
            case ELB_Q4_K: run_units<ELB_Q4_K, false>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
            case ELB_Q6_K: run_units<ELB_Q6_K, false>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
            default: run_units<ELB_Q8_0, false>(p, upt, rw.x, rw.y, rg, s, warp, lane); break;
        }
    }
    dk_sync();
    if (rc.x >= rc.y) return;  // (the whole CTA: it has no share of this matrix)
    const int Xf = rc.x / upt, ntl = (rc.y - 1) / upt - Xf + 1;
    // Row sums of the CTA's tiles: (row tile, row pair g / g+8) by (warp, half warp), the sixteen lanes of a half add the
    // contributions of the sixteen working warps in a fixed tree.
    {
        const int w = lane & 15, half = lane >> 4;
        const int2 tl = s.sched.tiles[w * DK_KINDS + kind];  // first and last row tile of warp w's share
#pragma unroll 1
        for (int pr = warp; pr < ntl * 8; pr += DK_WARPS) {
            const int Xt = Xf + (pr >> 3), row = (pr & 7) + 8 * half;
            float v = Xt >= tl.x && Xt <= tl.y ? s.red[(w * p.slots + (Xt - tl.x)) * 16 + row] : 0.f;
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            if (w == 0) s.outs[(pr >> 3) * 16 + row] = v * ea.inv;
        }
    }
    dk_sync();
    if (ea.epi == DK_EPI_SILU) {  // rows g = gate, g+8 = up of output row 8X+g (SwiGLU, src/model.cpp:222-225 of the reference)
#pragma unroll 1
        for (int e = tid; e < ntl * 8; e += DK_THREADS) {
            const int64_t o = 8 * int64_t(Xf) + e;
            if (o < rows / 2) {
                const float v0 = s.outs[(e >> 3) * 16 + (e & 7)], v1 = s.outs[(e >> 3) * 16 + (e & 7) + 8];
                ea.y[o] = __fmul_rn(__fdiv_rn(v0, 1.0f + expf(-v0)), v1);
            }
        }
        return;
    }
#pragma unroll 1
    for (int e = tid; e < ntl * 16; e += DK_THREADS) {
        const int Xt = Xf + (e >> 4);
        const int64_t r = 16 * int64_t(Xf) + e;
        if (r >= rows) continue;
        float v = s.outs[e];
        if (ea.epi == DK_EPI_PART) {
            const bool first = rc.x <= Xt * upt, last = rc.y >= (Xt + 1) * upt;
            if (first && ea.x_old) v = __fadd_rn(e == tid ? xo : __ldcg(ea.x_old + r), v);  // (a CTA has few row tiles: e == tid)
            const size_t pair = (size_t(ea.xset) * p.tp_size + p.tp_rank) * p.pv * p.E;  // this rank's vectors of the set
            if (p.tp_size == 1) {
                float* base = p.part_peer[0] + pair;
                base[(first ? 0 : p.E) + r] = v;
                if (first && last && p.pv == 2) base[p.E + r] = 0.f;
            } else {  // every rank receives {value, tag} in one 8-byte store
#pragma unroll 1
                for (int q = 0; q < p.tp_size; ++q) {
                    uint2* base = reinterpret_cast<uint2*>(p.part_peer[q]) + pair;
                    base[(first ? 0 : p.E) + r] = make_uint2(__float_as_uint(v), ea.tag);
                    if (first && last && p.pv == 2) base[p.E + r] = make_uint2(0u, ea.tag);
                }
            }
        } else if (ea.epi == DK_EPI_LOGITS) {
#pragma unroll 1
            for (int q = 0; q < p.tp_size; ++q) p.logits_peer[q][p.v0 + r] = v;
        } else {
            ea.y[r] = v;
        }
    }
}

// ---------------------------------------------------------------- attention phase (one token)

// RMSNorm over one 128-wide head followed by NEOX RoPE (src/ops.cpp:155-160, src/model.cpp:23-32 of the reference);
// one warp per head, lane owns elements lane, lane+32, lane+64, lane+96.
__device__ __forceinline__ void dk_head_norm_rope(const float* src, const float* w, const float2* cs, int rope_dim, float eps,
                                                  float* dst, int lane) {
    float v[4], wn[4];
    float2 c[2];  // cos / sin of this lane's rotation pairs: asked for together with the head, used last
    const int half = rope_dim / 2;
#pragma unroll
    for (int j = 0; j < 2; ++j) c[j] = lane + 32 * j < half ? __ldg(cs + lane + 32 * j) : make_float2(1.f, 0.f);
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = __ldcg(src + lane + 32 * j);
        wn[j] = __ldg(w + lane + 32 * j);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += double(v[j]) * v[j];
    ss = warp_sum(ss);
    const float inv = float(rsqrt_d(ss / DK_HD + double(eps)));
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __fmul_rn(__fmul_rn(v[j], inv), wn[j]);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = lane + 32 * j;
        if (i < half) {
            const float a = dst[i], b = dst[i + half];
            dst[i] = __fsub_rn(__fmul_rn(a, c[j].x), __fmul_rn(b, c[j].y));
            dst[i + half] = __fadd_rn(__fmul_rn(a, c[j].y), __fmul_rn(b, c[j].x));
        }
    }
    __syncwarp();
}

struct AttnSmem {
    float* qs;    // [DK_MAXG][128]
    float* knew;  // [128]
    float* vnew;  // [128]
    float* Ks;    // [DK_KT][DK_KS]; Ks and Vs together also stage the partial results the last split combines
    float* Vs;    // [DK_KT][128]
    float* Ps;    // [DK_MAXG][DK_KT]
    float* corr;  // [DK_MAXG], then m [DK_MAXG], l [DK_MAXG]
    int* flags;
};
constexpr int DK_ATTN_FLOATS = DK_MAXG * DK_HD + 2 * DK_HD + DK_KT * DK_KS + DK_KT * DK_HD + DK_MAXG * DK_KT + 3 * DK_MAXG;
static_assert(DK_MAXSPLIT * 4 * DK_PS <= DK_KT * DK_KS + DK_KT * DK_HD, "the staged partial results of four heads must fit in the K/V tile area");

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}

// Key splits of one KV head at T keys: a split should have a tile's worth of keys (fewer, longer splits keep the
// combination short at small contexts), and there are at most p.nsplit of them.
__device__ __forceinline__ int attn_splits(const DkParams& p, int T) { return max(1, min(p.nsplit, (T + DK_KT - 1) / DK_KT)); }

// K and V rows t0 .. t0+nk-1 of one KV head -> shared memory with cp.async (row `pos`, which this step appends, is
// filled in from shared memory by the caller). One commit group.
__device__ __forceinline__ void attn_fetch_kv(const float* kc, const float* vc, const AttnSmem& s, int KD, int kvh, int t0, int nk, int pos) {
    const uint32_t ks = dk_smem_u32(s.Ks), vs = dk_smem_u32(s.Vs);
    for (int idx = threadIdx.x; idx < nk * (DK_HD / 4); idx += DK_THREADS) {
        const int j = idx / (DK_HD / 4), cc = (idx % (DK_HD / 4)) * 4, t = t0 + j;
        if (t == pos) continue;
        const size_t off = size_t(t) * KD + kvh * DK_HD + cc;
        cp_async16(ks + uint32_t(j * DK_KS + cc) * 4u, kc + off);
        cp_async16(vs + uint32_t(j * DK_HD + cc) * 4u, vc + off);
    }
    ring_commit();
}

// The first key / value tile of this CTA's attention part does not depend on the token in flight (its own row comes
// from shared memory): it is requested as soon as the q|k|v matvec has released the scratch area, so that it travels
// while the CTAs meet at the barrier in front of the attention.
__device__ __forceinline__ void attn_prefetch(const DkParams& p, const int l, const AttnSmem& s) {
    const int c = blockIdx.x, pos = p.pos[p.ctl[0]], T = pos + 1, ns = attn_splits(p, T);
    if (c >= p.HKV * ns) return;
    const int kvh = c / ns, split = c - kvh * ns;
    const int t_begin = range_lo(T, ns, split), t_end = range_lo(T, ns, split + 1);
    attn_fetch_kv(p.kc + size_t(l) * p.kv_stride, p.vc + size_t(l) * p.kv_stride, s, p.HKV * DK_HD, kvh, t_begin, min(DK_KT, t_end - t_begin), pos);
}

// CTA c < HKV * splits works on KV head c / splits, key split c % splits: q/k norm + RoPE, KV append, flash decode
// over its keys (DK_KT at a time, fetched while the heads are normalised), partial results to the scratch buffer; the
// last split of a KV head to arrive combines them in split order and writes att (and max|att|).
// Semantics: src/model.cpp:176-214 of the reference.
__device__ __forceinline__ void attn_phase(const DkParams& p, const int l, const AttnSmem& s) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, c = blockIdx.x;
    const int pos = p.pos[p.ctl[0]], T = pos + 1, ns = attn_splits(p, T);
    if (c >= p.HKV * ns) return;
    const int kvh = c / ns, split = c - kvh * ns, group = p.H / p.HKV, QD = p.H * DK_HD, KD = p.HKV * DK_HD;
    float* const kc = p.kc + size_t(l) * p.kv_stride;
    float* const vc = p.vc + size_t(l) * p.kv_stride;
    const float* const q_norm = p.norms + size_t(l) * p.norm_stride + 2 * p.E;
    const float* const k_norm = q_norm + DK_HD;
    const int t_begin = range_lo(T, ns, split), t_end = range_lo(T, ns, split + 1);  // equal key ranges
    // (the first tile was requested by attn_prefetch before the barrier)
    const float2* cs = reinterpret_cast<const float2*>(p.rope) + size_t(pos) * (p.rope_dim / 2);
    float* m_s = s.corr + DK_MAXG;
    float* l_s = s.corr + 2 * DK_MAXG;
    for (int h = warp; h < group + 1; h += DK_WARPS) {
        if (h < group) dk_head_norm_rope(p.qkv + (kvh * group + h) * DK_HD, q_norm, cs, p.rope_dim, p.eps, s.qs + h * DK_HD, lane);
        else dk_head_norm_rope(p.qkv + QD + kvh * DK_HD, k_norm, cs, p.rope_dim, p.eps, s.knew, lane);
    }
    if (tid >= DK_THREADS - DK_HD) s.vnew[tid - (DK_THREADS - DK_HD)] = __ldcg(p.qkv + QD + KD + kvh * DK_HD + tid - (DK_THREADS - DK_HD));
    if (tid < DK_MAXG) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    dk_sync();
    if (split == 0 && tid < DK_HD) {  // KV append (src/model.cpp:186-189): only row `pos` is written
        kc[size_t(pos) * KD + kvh * DK_HD + tid] = s.knew[tid];
        vc[size_t(pos) * KD + kvh * DK_HD + tid] = s.vnew[tid];
    }
    float acc[2] = {0.f, 0.f};  // outputs (head tid/128 + 4i, dim tid%128)
    const int od = tid & (DK_HD - 1), oh = tid >> 7;
#pragma unroll 1
    for (int t0 = t_begin; t0 < t_end; t0 += DK_KT) {
        const int nk = min(DK_KT, t_end - t0);
        if (t0 != t_begin) {
            dk_sync();  // the previous tile has been consumed
            attn_fetch_kv(kc, vc, s, KD, kvh, t0, nk, pos);
        }
        if (pos >= t0 && pos < t0 + nk && tid < DK_HD) {  // the row this step appends: from shared memory, not from the cache
            s.Ks[(pos - t0) * DK_KS + tid] = s.knew[tid];
            s.Vs[(pos - t0) * DK_HD + tid] = s.vnew[tid];
        }
        ring_wait<0>();
        dk_sync();
        // scores and softmax bookkeeping of head `warp` over the tile: lane = key (a tile has up to two keys per lane);
        // the 128 products of a score are added in four interleaved partial sums
        if (warp < group) {
            constexpr int NP = (DK_KT + 31) / 32;
            float sc[NP], mx = -INFINITY;
            const float4* q = reinterpret_cast<const float4*>(s.qs + warp * DK_HD);
#pragma unroll
            for (int pass = 0; pass < NP; ++pass) {
                const int j = pass * 32 + lane;
                sc[pass] = -INFINITY;
                if (pass * 32 < nk) {  // (warp-uniform)
                    const float4* kr = reinterpret_cast<const float4*>(s.Ks + min(j, nk - 1) * DK_KS);
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
                    for (int i = 0; i < DK_HD / 4; ++i) {
                        const float4 qv = q[i], kv = kr[i];
                        a0 = fmaf(qv.x, kv.x, a0);
                        a1 = fmaf(qv.y, kv.y, a1);
                        a2 = fmaf(qv.z, kv.z, a2);
                        a3 = fmaf(qv.w, kv.w, a3);
                    }
                    if (j < nk) sc[pass] = __fmul_rn((a0 + a1) + (a2 + a3), p.scale);
                }
                mx = fmaxf(mx, sc[pass]);
            }
            const float m_old = m_s[warp], m_new = fmaxf(m_old, warp_max(mx));
            float sum = 0.f;
#pragma unroll
            for (int pass = 0; pass < NP; ++pass) {
                const int j = pass * 32 + lane;
                const float pj = j < nk ? expf(sc[pass] - m_new) : 0.f;
                if (j < nk) s.Ps[warp * DK_KT + j] = pj;
                sum += pj;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float cr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                s.corr[warp] = cr;
                l_s[warp] = l_s[warp] * cr + sum;
                m_s[warp] = m_new;
            }
        }
        dk_sync();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int h = oh + 4 * i;
            if (h >= group) continue;
            float a = acc[i] * s.corr[h];
#pragma unroll 8
            for (int j = 0; j < nk; ++j) a = fmaf(s.Ps[h * DK_KT + j], s.Vs[j * DK_HD + od], a);
            acc[i] = a;
        }
    }
    dk_sync();
    float* mine = p.attn_part + (size_t(kvh) * p.nsplit + split) * group * DK_PS;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int h = oh + 4 * i;
        if (h < group) mine[h * DK_PS + od] = acc[i];
    }
    if (tid < group) {
        mine[tid * DK_PS + DK_HD] = m_s[tid];
        mine[tid * DK_PS + DK_HD + 1] = l_s[tid];
    }
    dk_sync();
    if (tid == 0) {
        // release: the CTA's partial results (ordered before this thread by the barrier) are visible to whoever reads
        // the count; acquire: the last arriver sees everybody else's
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.attn_counters + kvh) : "memory");
        s.flags[0] = old == unsigned(ns - 1);
        if (s.flags[0]) p.attn_counters[kvh] = 0;
    }
    dk_sync();
    if (!s.flags[0]) return;
    // (thread 0's acquire and the barrier above order the other parts' results before the copies below)
    // The last split combines: the partial results of four heads at a time are staged in the K/V tile area (asynchronous
    // copies in a rolled loop: one round trip for all of them), then thread (head, dimension) walks the splits in order.
    const float* base = p.attn_part + size_t(kvh) * p.nsplit * group * DK_PS;
    float* stage = s.Ks;  // [ns][4][DK_PS]
#pragma unroll 1
    for (int hq = 0; hq < group; hq += 4) {
        const int nh = min(4, group - hq), chunks = nh * (DK_PS / 4);  // 16-byte pieces per split
        if (hq) dk_sync();  // the previous four heads have been read
#pragma unroll 1
        for (int idx = tid; idx < ns * chunks; idx += DK_THREADS) {
            const int q = idx / chunks, o = (idx - q * chunks) * 4;
            cp_async16(dk_smem_u32(stage + q * 4 * DK_PS + o), base + (size_t(q) * group + hq) * DK_PS + o);
        }
        ring_commit();
        ring_wait<0>();
        dk_sync();
        if (oh < nh) {
            const float* ps = stage + oh * DK_PS;
            float M = -INFINITY;
#pragma unroll 1
            for (int q = 0; q < ns; ++q) M = fmaxf(M, ps[q * 4 * DK_PS + DK_HD]);
            float Lsum = 0.f, o = 0.f;
#pragma unroll 1
            for (int q = 0; q < ns; ++q) {  // fixed split order
                const float mq = ps[q * 4 * DK_PS + DK_HD];
                if (mq == -INFINITY) continue;
                const float w = expf(mq - M);
                Lsum = fmaf(ps[q * 4 * DK_PS + DK_HD + 1], w, Lsum);
                o = fmaf(ps[q * 4 * DK_PS + od], w, o);
            }
            p.att[(kvh * group + hq + oh) * DK_HD + od] = o / Lsum;
        }
    }
}

// ---------------------------------------------------------------- the step

__host__ __device__ inline size_t dk_scratch_bytes(int n_max) {
    const size_t act = dk_act_bytes(n_max), attn = size_t(DK_ATTN_FLOATS) * 4;
    return ((act > attn ? act : attn) + 15) / 16 * 16;
}
// grid barriers of one launch (the arrival counter runs on from launch to launch)
__host__ __device__ inline unsigned dk_barriers_per_launch(const DkParams& p) {
    // Per layer: behind q|k|v, attention, attn_output, gate|up, ffn_down. Tensor parallel: the barriers behind the two
    // row-parallel matvecs move behind the reductions of their partial sums (the first conversion of a launch has nothing
    // to reduce, the head's has), and the logits meet at one more.
    const unsigned per_layer = 5u + (p.act_global ? 1u : 0u);
    return 1u + per_layer * unsigned(p.n_layer) + (p.tp_size > 1 ? 1u : 0u);
}

// token embedding (get_row, src/ops.cpp:76-82 of the reference): the CTAs decode slices of the row into the residual buffer
__device__ __noinline__ void embed_token(const DkParams& p, float* x, unsigned step) {
    const int64_t R = p.token[step];
    const int lo = range_lo(p.E, gridDim.x, blockIdx.x), hi = range_lo(p.E, gridDim.x, blockIdx.x + 1);
#pragma unroll 1
    for (int k = lo + int(threadIdx.x); k < hi; k += DK_THREADS)
        x[k] = p.embd_type == ELB_F16 ? __half2float(reinterpret_cast<const __half*>(p.embd)[R * p.E + k])
                                      : elem_value(p.embd_type, tiled_elem(p.embd_type, p.embd, p.E, R, k));
}

template <bool GACT>
__global__ void __launch_bounds__(DK_CTA_THREADS, 1) k_decode_step(const __grid_constant__ DkParams p, const int ring_bytes) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // shared memory: rings | scratch (limbs of the running matvec, or the attention tiles) | reduction buffers | mbarriers | tables
    uint8_t* scratch = smem + size_t(DK_WARPS) * ring_bytes;
    uint8_t* tail = scratch + dk_scratch_bytes(p.n_max);
    PhaseSmem s;
    s.red = reinterpret_cast<float*>(tail);
    s.outs = s.red + DK_WARPS * p.slots * 16;
    s.red8 = reinterpret_cast<double*>(s.outs + p.cta_tiles * 16);
    s.flags = reinterpret_cast<int*>(s.red8 + DK_WARPS);
    uint64_t* bars0 = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(s.flags + 4) + 7) & ~uintptr_t(7));
    int2* sched_w = reinterpret_cast<int2*>(bars0 + DK_WARPS * DK_NBAR);  // [DK_WARPS][DK_KINDS] unit ranges
    int2* sched_t = sched_w + DK_WARPS * DK_KINDS;                         // [DK_WARPS][DK_KINDS] row tile ranges
    int2* sched_c = sched_t + DK_WARPS * DK_KINDS;                         // [DK_KINDS]
    RingShared* rshared = reinterpret_cast<RingShared*>(sched_c + DK_KINDS);
    const int wk = warp < DK_WARPS ? warp : 0;
    s.sched.warp = sched_w + wk * DK_KINDS;
    s.sched.tiles = sched_t;
    s.sched.cta = sched_c;
    Ring rg;
    rg.base = dk_smem_u32(smem) + uint32_t(wk * ring_bytes);
    rg.bars = dk_smem_u32(bars0 + wk * DK_NBAR);
    rg.bytes = ring_bytes;
    rg.c_off = 0;
    rg.c_seq = rg.freed = 0u;
    rg.freed_out = dk_smem_u32(rshared->freed + wk);
    AttnSmem as;
    as.qs = reinterpret_cast<float*>(scratch);
    as.knew = as.qs + DK_MAXG * DK_HD;
    as.vnew = as.knew + DK_HD;
    as.Ks = as.vnew + DK_HD;
    as.Vs = as.Ks + DK_KT * DK_KS;
    as.Ps = as.Vs + DK_KT * DK_HD;
    as.corr = as.Ps + DK_MAXG * DK_KT;
    as.flags = s.flags;
    if (tid == 0) { s.flags[2] = 0; rshared->producer_done = 0; }
    if (tid < DK_WARPS) { rshared->freed[tid] = 0u; rshared->issued[tid] = 0u; }
    if (warp < DK_WARPS && lane < DK_KINDS) {  // this warp's share of every kind of matrix (kinds the model does not have: empty)
        const int kind = lane;
        WarpRange r{0, 0, 0, 0};
        if (kind >= 3 || kind < p.n_qkv) r = warp_range(p.kind[kind], warp);
        const int upt = max(p.kind[kind].upt, 1);
        sched_w[warp * DK_KINDS + kind] = make_int2(r.wA, r.wB);
        sched_t[warp * DK_KINDS + kind] = r.wA < r.wB ? make_int2(r.wA / upt, (r.wB - 1) / upt) : make_int2(0, -1);
        if (warp == 0) sched_c[kind] = make_int2(r.cA, r.cB);
    }
    if (warp < DK_WARPS && lane == 0) {
#pragma unroll 1
        for (int i = 0; i < DK_NBAR; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rg.bars + i * 8u), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();  // the only barrier of all twenty warps

    // the weight stream starts here: from now to the end of the step the producer warp keeps every ring as full as it gets
    if (warp >= DK_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(DK_REGS_PRODUCER));
        if (warp == DK_WARPS) producer_warp(p, dk_smem_u32(smem), ring_bytes, dk_smem_u32(bars0), sched_w, rshared, &s.flags[2], lane);
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DK_REGS_WORKER));
    int* dead = &s.flags[2];
    const unsigned step = p.ctl[0], epoch = p.ctl[2];
    unsigned nb = epoch * dk_barriers_per_launch(p) * gridDim.x;  // arrivals before this launch

    embed_token(p, p.xbuf, step);
    bool ok = grid_barrier(p, nb, dead);
    int cur = 0;  // which half of xbuf holds the residual stream (without the pending partial sums)
    // exchanges (row-parallel matvec -> all ranks) are numbered from the first launch; number x uses set x & 1
    unsigned xn = epoch * unsigned(2 * p.n_layer + 1);
    const bool tp = p.tp_size > 1;
    float* const my_part = p.part_peer[p.tp_rank];  // this rank's copy of the partial-sum sets
    int pending = -1;  // set whose partial sums the next residual conversion adds (-1: none yet in this launch)
    unsigned pending_tag = 0;  // tensor parallel: the tag those partial sums carry
    int8_t* const lim_smem = reinterpret_cast<int8_t*>(scratch);

    // The step as ONE loop over its matvec stages - per layer q|k|v (0), attn_output (1), gate|up (2), ffn_down (3),
    // then the head (4) - so that the conversion, the matvec and the attention code exist once in the kernel.
    const int n_stages = 4 * p.n_layer + 1;
#pragma unroll 1
    for (int stage = 0; stage < n_stages && ok; ++stage) {
        const bool head = stage + 1 == n_stages;
        const int l = head ? p.n_layer : stage >> 2, k = head ? 4 : stage & 3;
        const float* const layer_norms = p.norms + size_t(l) * p.norm_stride;  // (not read for the head)
        if (k == 0) dk_stamp(p, l, 0);
        const bool pc = p.prof_cta && l == p.prof_layer;  // diagnostics: every CTA stamps this layer's barriers
        if (k == 1) {  // attention sits between q|k|v and attn_output
            attn_phase(p, l, as);
            dk_stamp(p, l, 4);
            if (!(ok = grid_barrier(p, nb, dead, false, 0, pc ? 1 : -1))) break;
            dk_stamp(p, l, 5);
        }
        // the stage's activation: where it comes from, how it is normalised, which matrices consume it
        const float *src = nullptr, *norm_w = nullptr;
        EpiArgs ea{DK_EPI_PART, nullptr, 1.0f, int(xn & 1u), xn + 1u, nullptr};
        int n = p.E, nl = 4, nm = 1;
        int i0 = p.n_qkv, kind0 = 3;  // the stage's first matrix: index within the layer, kind
        bool resid = true;
        switch (k) {
            case 0: norm_w = layer_norms; nl = p.nl_qkv; i0 = 0; kind0 = 0; nm = p.n_qkv; ea.epi = DK_EPI_STORE; ea.y = p.qkv; break;
            case 1: resid = false; src = p.att; n = p.H * DK_HD; nl = p.nl_wo; break;
            case 2: norm_w = layer_norms + p.E; nl = p.nl_gu; i0 = p.n_qkv + 1; kind0 = 4; ea.epi = DK_EPI_SILU; ea.y = p.act; break;
            case 3: resid = false; src = p.act; n = p.F; nl = p.nl_down; i0 = p.n_qkv + 2; kind0 = 5; break;
            default: norm_w = p.output_norm; ea.epi = DK_EPI_LOGITS; i0 = 0; kind0 = 6; break;
        }
        int need = 0;
        for (int i = 0; i < nm; ++i) need |= sd_need(p.wtype[l][i0 + i]);
        const bool gact = GACT && k == 3;
        const int nblk = n / 256;
        if (gact) {  // the CTAs split equal ranges of blocks into global memory and meet; ffn_down reads them through L2
            s.act = act_at(p.gact, n);
            convert_act<false>(src, nullptr, nullptr, n, range_lo(nblk, gridDim.x, blockIdx.x), range_lo(nblk, gridDim.x, blockIdx.x + 1),
                               nullptr, p.eps, nl, s.act, s.red8, need);
            if (!(ok = grid_barrier(p, nb, dead))) break;
        } else {
            s.act = act_at(lim_smem, n);
            if (!resid) {
                convert_act<false>(src, nullptr, nullptr, n, 0, nblk, nullptr, p.eps, nl, s.act, s.red8, need);
            } else if (pending < 0) {  // the embedding: nothing to add, the residual stream is where it is
                ea.inv = convert_act<true>(p.xbuf + cur * p.E, nullptr, nullptr, n, 0, nblk, norm_w, p.eps, nl, s.act, s.red8, need);
            } else {
                // the new residual stream: the partial sums of the last row-parallel matvec (its first buffer carries the
                // old stream); it goes to the other half of xbuf, after the last layer to p.x
                float* const xnew = head ? p.x : p.xbuf + (cur ^ 1) * p.E;
                const float* const set = my_part + size_t(pending) * p.tp_size * p.pv * p.E;
                if (tp) {
                    reduce_ranks(p, reinterpret_cast<const uint2*>(my_part) + size_t(pending) * p.tp_size * p.pv * p.E, xnew, pending_tag, dead);
                    if (!(ok = grid_barrier(p, nb, dead))) break;
                    ea.inv = convert_act<true>(xnew, nullptr, nullptr, n, 0, nblk, norm_w, p.eps, nl, s.act, s.red8, need);
                } else {
                    ea.inv = convert_act<true>(set, set + p.E, xnew, n, 0, nblk, norm_w, p.eps, nl, s.act, s.red8, need);
                }
                cur ^= 1;
            }
        }
        // the residual stream a row-parallel matvec adds to its partial sums (under tensor parallelism: rank 0 alone)
        ea.x_old = ea.epi == DK_EPI_PART && p.tp_rank == 0 ? p.xbuf + cur * p.E : nullptr;
        const int sb = k == 0 ? 0 : 3 * k + 2;  // profile stamps of the stage: conversion, matvec, barrier
        if (!head) dk_stamp(p, l, sb + 1);
        for (int i = 0; i < nm; ++i) {
            EpiArgs e2 = ea;
            if (k == 0) e2.y = ea.y + p.qkv_col[i];
            matvec_phase<GACT>(p, p.wtype[l][i0 + i], kind0 + i, e2, rg, s, i > 0, gact);
        }
        if (!head) dk_stamp(p, l, sb + 2);
        if (k == 0) attn_prefetch(p, l, as);
        if (k == 1 || k == 3) {
            // a row-parallel matvec: on one GPU its partial sums meet at the grid barrier; under tensor parallelism they
            // carry their own arrival tag and the reduction waits for them, no barrier here
            if (!tp) ok = grid_barrier(p, nb, dead, false, 0, pc ? (k == 1 ? 2 : 4) : -1);
            pending = int(xn & 1u);
            pending_tag = xn + 1u;
            ++xn;
        } else if (head && tp) {  // the logits rows of all ranks: fenced peer stores and flags
            ok = grid_barrier(p, nb, dead, true, xn);
            ++xn;
        } else if (!head) {
            ok = grid_barrier(p, nb, dead, false, 0, pc ? (k == 0 ? 0 : 3) : -1);
        }
        if (!head) dk_stamp(p, l, sb + 3);
    }
    ring_drain(rg, rshared, warp);  // (nothing is left in flight after a whole step; after a timeout the copies still land here)
    if (blockIdx.x == 0 && tid == 0) {  // every CTA read ctl before its first barrier: safe to move on
        p.ctl[2] = epoch + 1;
        if (p.ctl[1]) p.ctl[0] = step + 1;
    }
}

// everything but the rings
static size_t decode_fixed_smem(const DkParams& p) {
    return dk_scratch_bytes(p.n_max) + size_t(DK_WARPS) * p.slots * 16 * 4 + size_t(p.cta_tiles) * 16 * 4 + DK_WARPS * 8 + 4 * 4 + 16 +
           size_t(DK_WARPS) * DK_NBAR * 8 + size_t(2 * DK_WARPS + 1) * DK_KINDS * 8 + sizeof(RingShared);
}
size_t decode_smem_bytes(const DkParams& p, int ring_bytes) { return size_t(DK_WARPS) * ring_bytes + decode_fixed_smem(p); }

// Bytes per warp ring when the kernel takes all the shared memory a CTA can have (a multiple of 128), capped so that a
// warp cannot have more than DK_NBAR of the smallest units on request; 0 when not even two of the largest units fit.
int decode_ring_bytes(const DkParams& p, int max_unit, int min_unit, int device) {
    DeviceInfo di;
    if (device_info(device, &di) != ELB_OK) return 0;
    const size_t fixed = decode_fixed_smem(p);
    if (di.smem_optin < fixed + size_t(DK_WARPS) * 2 * max_unit) return 0;
    size_t per = (di.smem_optin - fixed) / DK_WARPS / 128 * 128;
    per = std::min(per, size_t(DK_NBAR) * min_unit / 128 * 128);
    return per >= size_t(2) * max_unit ? int(per) : 0;
}

static const void* decode_kernel(const DkParams& p) {
    return p.act_global ? reinterpret_cast<const void*>(k_decode_step<true>) : reinterpret_cast<const void*>(k_decode_step<false>);
}

int decode_step_launch(const DkParams& p, int ring_bytes, int grid, cudaStream_t s) {
    const size_t smem = decode_smem_bytes(p, ring_bytes);
    ELB_TRY(ensure_dyn_smem(decode_kernel(p), smem));
    void* args[] = {const_cast<DkParams*>(&p), const_cast<int*>(&ring_bytes)};
    ELB_CUDA(cudaLaunchCooperativeKernel(decode_kernel(p), dim3(grid), dim3(DK_CTA_THREADS), args, smem, s));
    return ELB_OK;
}

// can one CTA per SM of the step kernel be resident with this much shared memory?
int decode_step_fits(const DkParams& p, int ring_bytes, int device, bool* fits) {
    DeviceInfo di;
    ELB_TRY(device_info(device, &di));
    const size_t smem = decode_smem_bytes(p, ring_bytes);
    *fits = false;
    if (smem > di.smem_optin) return ELB_OK;
    ELB_TRY(ensure_dyn_smem(decode_kernel(p), smem));
    int per_sm = 0;
    if (p.act_global) ELB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_step<true>, DK_CTA_THREADS, smem));
    else ELB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_decode_step<false>, DK_CTA_THREADS, smem));
    *fits = per_sm >= 1;
    return ELB_OK;
}

int decode_threads() { return DK_THREADS; }
int decode_warps() { return DK_WARPS; }
int decode_max_split() { return DK_MAXSPLIT; }
int decode_part_stride() { return DK_PS; }
size_t decode_act_bytes(int n) { return dk_act_bytes(n); }


}  // namespace elb
