// Decode matvec y = W x for one token: a bandwidth kernel.
//
// The activation is split once per CTA into exact int8 limbs (k_split8 semantics of the reference,
// src/cuda/model_cuda.cu:701-729) held in shared memory. Weights stream from HBM in their file encoding, one
// 128-bit load per lane per 1 KB micro-tile, straight into mma.sync A-fragments (16 weight rows x 32 k); the limbs
// are the B-fragments (columns = limbs), so one integer MMA forms the four limb dot products of 16 rows over one
// sub-block exactly in int32. Integer sub-block scales are applied in int32; one conversion to fp32 per 256-block.
//
// Work split: the (row tile, k block) units of the matrix are cut into equal contiguous ranges, one per CTA and
// within a CTA one per warp, whatever the matrix shape. Partial row sums meet in shared memory (fixed warp order) and,
// where a row tile is shared by several CTAs, in a scratch buffer summed by the last CTA to arrive (fixed CTA order):
// results are deterministic and need no floating-point atomics.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "split.cuh"

namespace elb {

constexpr int GEMV_THREADS = 256, GEMV_WARPS = GEMV_THREADS / 32;
constexpr int LIMB_PAD = 32;  // limb row stride n + 32 bytes: the four limb rows fall in different bank groups

struct GemvParams {
    const uint8_t* W;
    int64_t tiles, upt, rows;
    int n;
    const int8_t* limbs;     // [4][n] pre-split activation (global)
    const float* inv_scale;  // [1]
    float* y;
    const float* resid;
    float* part;
    unsigned* counters;
    int epilogue, slots;
    int32_t *dbgP, *dbgI, *dbgJ;
    PostOp post;
};

// ---------------------------------------------------------------- units: registers of one lane

template <int TYPE> struct Unit;
template <> struct Unit<ELB_Q4_K> { uint4 h0, h1, q[4]; };
template <> struct Unit<ELB_Q6_K> { uint32_t dd; uint4 s0, s1, ql[4]; uint2 qh[4]; };
template <> struct Unit<ELB_Q8_0> { uint2 d0, d1; uint4 q[4]; };

// A unit travels HBM -> shared memory with cp.async (a per-warp ring, so that several units per warp are in flight
// without holding registers), then shared memory -> registers right before it is used. The image in shared memory
// is byte for byte the unit in the tiled layout.
__device__ __forceinline__ void issue_unit(uint8_t* slot, const uint8_t* src, int unit_bytes, int lane) {
    const unsigned dst = unsigned(__cvta_generic_to_shared(slot));
    for (int o = lane * 16; o < unit_bytes; o += 512)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + o), "l"(src + o));
}
__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ring_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint4 lds4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint2 lds2(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }

__device__ __forceinline__ void load_unit(Unit<ELB_Q4_K>& u, const uint8_t* base, int lane) {
    const int g = lane >> 2;
    u.h0 = lds4(base + g * 32);
    u.h1 = lds4(base + g * 32 + 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) u.q[j] = lds4(base + 256 + j * 512 + lane * 16);
}
__device__ __forceinline__ void load_unit(Unit<ELB_Q6_K>& u, const uint8_t* base, int lane) {
    const int g = lane >> 2;
    u.dd = *reinterpret_cast<const uint32_t*>(base + g * 4);
    u.s0 = lds4(base + 32 + g * 32);
    u.s1 = lds4(base + 32 + g * 32 + 16);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        u.ql[c] = lds4(base + 288 + c * 512 + lane * 16);
        u.qh[c] = lds2(base + 2336 + c * 256 + lane * 8);
    }
}
__device__ __forceinline__ void load_unit(Unit<ELB_Q8_0>& u, const uint8_t* base, int lane) {
    const int g = lane >> 2;
    u.d0 = lds2(base + g * 16);
    u.d1 = lds2(base + g * 16 + 8);
#pragma unroll
    for (int i = 0; i < 4; ++i) u.q[i] = lds4(base + 128 + i * 512 + lane * 16);
}

__device__ __forceinline__ uint32_t sel4(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Accumulators of one lane for the tile in progress: rows g (index 0) and g+8 (index 1).
//   acc  : sum over blocks of d * (I[2t'] + 256 I[2t'+1]),  t' = t & 1 — the limb pair this lane's C columns hold
//   accm : the correction term with its own fp scale (Q4_K: dmin * sum m*S; Q6_K: 32 d * sum sc*S), digit pair of lane t
struct Acc { float acc[2], accm[2]; };

struct DbgOut {
    int32_t *P, *I, *J;
    int64_t row_g;  // global row of this lane's row g (row g+8 = +8), rows beyond the matrix are not written
    int64_t rows;
    int nsub, nblk;
};

// ---- Q4_K: one 256-block of 16 rows
template <bool DBG>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q4_K>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t* sd, int lane, Acc& a, const DbgOut& dbg) {
    const int g = lane >> 2, t = lane & 3;
    const int8_t* lcol = lim + (g & 3) * n_pad + b * QK_K + 8 * t;
    // 6-bit scales and mins of rows g and g+8 as packed bytes (q4k_scale_min of the reference, src/quant.h:44-52)
    const uint32_t sg[2] = {u.h0.y & 0x3F3F3F3Fu, (u.h0.w & 0x0F0F0F0Fu) | ((u.h0.y >> 2) & 0x30303030u)};
    const uint32_t sh[2] = {u.h1.y & 0x3F3F3F3Fu, (u.h1.w & 0x0F0F0F0Fu) | ((u.h1.y >> 2) & 0x30303030u)};
    const uint32_t mg[2] = {u.h0.z & 0x3F3F3F3Fu, ((u.h0.w >> 4) & 0x0F0F0F0Fu) | ((u.h0.z >> 2) & 0x30303030u)};
    const uint32_t mh[2] = {u.h1.z & 0x3F3F3F3Fu, ((u.h1.w >> 4) & 0x0F0F0F0Fu) | ((u.h1.z >> 2) & 0x30303030u)};
    int I[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 q = u.q[j];
#pragma unroll
        for (int odd = 0; odd < 2; ++odd) {
            const int sub = 2 * j + odd;
            const uint2 bf = __ldg(reinterpret_cast<const uint2*>(lcol + sub * 32));
            int C[4] = {0, 0, 0, 0};
            if (odd == 0)
                mma_u8s8_k32(C, q.x & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, bf.x, bf.y);
            else
                mma_u8s8_k32(C, (q.x >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu,
                             (q.w >> 4) & 0x0F0F0F0Fu, bf.x, bf.y);
            const int s0 = (sg[sub >> 2] >> (8 * (sub & 3))) & 0xFF, s1 = (sh[sub >> 2] >> (8 * (sub & 3))) & 0xFF;
            I[0] += s0 * C[0];
            I[1] += s0 * C[1];
            I[2] += s1 * C[2];
            I[3] += s1 * C[3];
            if (DBG && dbg.P && t < 2) {
                const int64_t s = int64_t(b) * 8 + sub;
                if (dbg.row_g < dbg.rows) {
                    dbg.P[(dbg.row_g * dbg.nsub + s) * 4 + 2 * t] = C[0];
                    dbg.P[(dbg.row_g * dbg.nsub + s) * 4 + 2 * t + 1] = C[1];
                }
                if (dbg.row_g + 8 < dbg.rows) {
                    dbg.P[((dbg.row_g + 8) * dbg.nsub + s) * 4 + 2 * t] = C[2];
                    dbg.P[((dbg.row_g + 8) * dbg.nsub + s) * 4 + 2 * t + 1] = C[3];
                }
            }
        }
    }
    const float dg = h2f_bits(u.h0.x & 0xFFFFu), dh = h2f_bits(u.h1.x & 0xFFFFu);
    a.acc[0] += dg * fmaf(float(I[1]), 256.0f, float(I[0]));
    a.acc[1] += dh * fmaf(float(I[3]), 256.0f, float(I[2]));
    // min term: J[col] = sum over the 8 sub-blocks of m * (digit `col>>2` of the limb sum S of limb `col&3`)
    const uint32_t a0 = t == 0 ? mg[0] : t == 1 ? mg[1] : 0u, a1 = t == 0 ? mh[0] : t == 1 ? mh[1] : 0u;
    const uint32_t b0 = __ldg(reinterpret_cast<const uint32_t*>(sd + (b * 8 + g) * 8 + 4 * (t & 1)));
    int J[4] = {0, 0, 0, 0};
    mma_u8s8_k16(J, a0, a1, b0);
    const float ng = h2f_bits(u.h0.x >> 16), nh = h2f_bits(u.h1.x >> 16);
    a.accm[0] += ng * fmaf(float(J[1]), 256.0f, float(J[0]));
    a.accm[1] += nh * fmaf(float(J[3]), 256.0f, float(J[2]));
    if (DBG) {
        // digits of J sit in lanes t (low) and t+2 (high): bring them together
        int Jh[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) Jh[i] = __shfl_down_sync(0xffffffffu, J[i], 2);
        if (t < 2) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int64_t row = dbg.row_g + 8 * r;
                if (row >= dbg.rows) continue;
                const int64_t o = (row * dbg.nblk + b) * 4 + 2 * t;
                if (dbg.I) { dbg.I[o] = I[2 * r]; dbg.I[o + 1] = I[2 * r + 1]; }
                if (dbg.J) { dbg.J[o] = J[2 * r] + 256 * Jh[2 * r]; dbg.J[o + 1] = J[2 * r + 1] + 256 * Jh[2 * r + 1]; }
            }
        }
    }
}

// ---- Q6_K: one 256-block of 16 rows; sub-blocks of 16 with int8 scales; q6 is fed unsigned (0..63) and the
// offset -32 * sum sc*S comes from one extra MMA over the limb sums S of the 16-wide sub-blocks.
template <bool DBG>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q6_K>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t* sd, int lane, Acc& a, const DbgOut& dbg) {
    const int g = lane >> 2, t = lane & 3;
    const int8_t* lcol = lim + (g & 3) * n_pad + b * QK_K + 4 * t;
    int I[4] = {0, 0, 0, 0};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 ql = u.ql[c];
        const uint2 qh = u.qh[c];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = 4 * c + i;
            const uint32_t w = sel4(ql, i);
            const uint32_t a0 = (w & 0x0F0F0F0Fu) | (((qh.x >> (2 * i)) & 0x03030303u) << 4);
            const uint32_t a1 = ((w >> 4) & 0x0F0F0F0Fu) | (((qh.y >> (2 * i)) & 0x03030303u) << 4);
            const uint32_t bf = __ldg(reinterpret_cast<const uint32_t*>(lcol + s * 16));
            int C[4] = {0, 0, 0, 0};
            mma_u8s8_k16(C, a0, a1, bf);
            const int s0 = int(int8_t(sel4(u.s0, s >> 2) >> (8 * (s & 3)))), s1 = int(int8_t(sel4(u.s1, s >> 2) >> (8 * (s & 3))));
            I[0] += s0 * C[0];
            I[1] += s0 * C[1];
            I[2] += s1 * C[2];
            I[3] += s1 * C[3];
            if (DBG && dbg.P && t < 2) {
                // the parity dump wants sum (q6-32)*a: subtract 32 * S, S recomputed from the limbs
                const int64_t sidx = int64_t(b) * 16 + s;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int l = 2 * t + e;
                    int S = 0;
                    for (int k = 0; k < 16; ++k) S += lim[l * n_pad + b * QK_K + s * 16 + k];
                    if (dbg.row_g < dbg.rows) dbg.P[(dbg.row_g * dbg.nsub + sidx) * 4 + l] = C[e] - 32 * S;
                    if (dbg.row_g + 8 < dbg.rows) dbg.P[((dbg.row_g + 8) * dbg.nsub + sidx) * 4 + l] = C[2 + e] - 32 * S;
                }
            }
        }
    }
    const float dg = h2f_bits(u.dd & 0xFFFFu), dh = h2f_bits(u.dd >> 16);
    a.acc[0] += dg * fmaf(float(I[1]), 256.0f, float(I[0]));
    a.acc[1] += dh * fmaf(float(I[3]), 256.0f, float(I[2]));
    const uint32_t b0 = __ldg(reinterpret_cast<const uint32_t*>(sd + (b * 8 + g) * 16 + 4 * t));
    int J[4] = {0, 0, 0, 0};
    mma_s8s8_k16(J, sel4(u.s0, t), sel4(u.s1, t), b0);
    a.accm[0] += (32.0f * dg) * fmaf(float(J[1]), 256.0f, float(J[0]));
    a.accm[1] += (32.0f * dh) * fmaf(float(J[3]), 256.0f, float(J[2]));
    if (DBG) {
        int Jh[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) Jh[i] = __shfl_down_sync(0xffffffffu, J[i], 2);
        if (t < 2 && dbg.I) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int64_t row = dbg.row_g + 8 * r;
                if (row >= dbg.rows) continue;
                const int64_t o = (row * dbg.nblk + b) * 4 + 2 * t;
                dbg.I[o] = I[2 * r] - 32 * (J[2 * r] + 256 * Jh[2 * r]);
                dbg.I[o + 1] = I[2 * r + 1] - 32 * (J[2 * r + 1] + 256 * Jh[2 * r + 1]);
                if (dbg.J) { dbg.J[o] = 0; dbg.J[o + 1] = 0; }
            }
        }
    }
}

// ---- Q8_0: four 32-blocks of 16 rows; fp16 scale per block, so fp32 after every MMA
template <bool DBG>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q8_0>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t*, int lane, Acc& a, const DbgOut& dbg) {
    const int g = lane >> 2, t = lane & 3;
    const int8_t* lcol = lim + (g & 3) * n_pad + b * (QK8_0 * Q8_GROUP) + 8 * t;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 q = u.q[i];
        const uint2 bf = __ldg(reinterpret_cast<const uint2*>(lcol + i * 32));
        int C[4] = {0, 0, 0, 0};
        mma_s8s8_k32(C, q.x, q.z, q.y, q.w, bf.x, bf.y);
        const uint32_t d0w = i < 2 ? u.d0.x : u.d0.y, d1w = i < 2 ? u.d1.x : u.d1.y;
        const float dg = h2f_bits((d0w >> (16 * (i & 1))) & 0xFFFFu), dh = h2f_bits((d1w >> (16 * (i & 1))) & 0xFFFFu);
        a.acc[0] += dg * fmaf(i2f_small(C[1]), 256.0f, i2f_small(C[0]));
        a.acc[1] += dh * fmaf(i2f_small(C[3]), 256.0f, i2f_small(C[2]));
        if (DBG && t < 2) {
            const int64_t s = int64_t(b) * 4 + i;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int64_t row = dbg.row_g + 8 * r;
                if (row >= dbg.rows) continue;
                const int64_t o = (row * dbg.nsub + s) * 4 + 2 * t;
                if (dbg.P) { dbg.P[o] = C[2 * r]; dbg.P[o + 1] = C[2 * r + 1]; }
                if (dbg.I) { dbg.I[o] = C[2 * r]; dbg.I[o + 1] = C[2 * r + 1]; }
                if (dbg.J) { dbg.J[o] = 0; dbg.J[o + 1] = 0; }
            }
        }
    }
}

// ---------------------------------------------------------------- prologue: x -> limbs (+ limb sums) in shared memory

// The split activation (limbs and their sub-block sums, layout in split.cuh) is read straight from global memory
// through L1: every SM touches the same few tens of KB, so after a first sweep the B-fragments are L1 hits and no
// shared memory, copy phase or block barrier stands between a warp and its first MMA. This warms L1 up.
__device__ __forceinline__ void prefetch_act(const int8_t* act, int n) {
    const int lines = int((act_bytes(n) + 127) / 128);
    for (int i = threadIdx.x; i < lines; i += GEMV_THREADS) asm volatile("prefetch.global.L1 [%0];" ::"l"(act + size_t(i) * 128));
}

// ---------------------------------------------------------------- epilogue for rows g / g+8 of tile X

__device__ __forceinline__ void epilogue(const GemvParams& p, int64_t X, int g, float v0, float v1) {
    const int64_t r0 = 16 * X + g, r1 = r0 + 8;
    if (p.epilogue == EPI_SILU) {  // rows g = gate, g+8 = up of output row 8X+g (SwiGLU, src/model.cpp:222-225)
        const int64_t o = 8 * X + g;
        if (o < p.rows / 2) p.y[o] = __fmul_rn(__fdiv_rn(v0, 1.0f + expf(-v0)), v1);
        return;
    }
    if (p.epilogue == EPI_ADD) {
        if (r0 < p.rows) p.y[r0] = p.resid[r0] + v0;
        if (r1 < p.rows) p.y[r1] = p.resid[r1] + v1;
        return;
    }
    if (r0 < p.rows) p.y[r0] = v0;
    if (r1 < p.rows) p.y[r1] = v1;
}

// ---------------------------------------------------------------- the kernel

// start of part i when `total` items are cut into `parts` contiguous ranges (total * parts < 2^31, checked on the host)
__host__ __device__ __forceinline__ int range_lo(int total, int parts, int i) { return int(unsigned(total) * unsigned(i) / unsigned(parts)); }

template <int TYPE, bool DBG, int DEPTH>
__global__ void __launch_bounds__(GEMV_THREADS, 2) k_gemv(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n_pad = p.n, upt = int(p.upt);
    constexpr int UNIT_BYTES = TYPE == ELB_Q4_K ? Q4K_UNIT : TYPE == ELB_Q6_K ? Q6K_UNIT : Q8_UNIT;
    const int8_t* lim = p.limbs;
    const int8_t* sd = p.limbs + (TYPE == ELB_Q6_K ? act_sd16_off(p.n) : act_sd32_off(p.n));
    float* red = reinterpret_cast<float*>(smem);  // [warps][slots][16]
    uint8_t* ring = reinterpret_cast<uint8_t*>(red + GEMV_WARPS * p.slots * 16) + size_t(warp) * DEPTH * UNIT_BYTES;
    __shared__ double red8[GEMV_WARPS];
    __shared__ int s_last[2], s_wfirst[GEMV_WARPS], s_wlast[GEMV_WARPS];  // tiles touched by each warp

    const int U = int(p.tiles) * upt, G = gridDim.x, c = blockIdx.x;
    const int cA = range_lo(U, G, c), cB = range_lo(U, G, c + 1);
    const int wA = cA + range_lo(cB - cA, GEMV_WARPS, warp), wB = cA + range_lo(cB - cA, GEMV_WARPS, warp + 1);

    // weights do not depend on the previous kernel: fill the ring before waiting for it. One commit group per unit,
    // empty groups included, so that "all but the newest DEPTH-1 groups" always means "the unit about to be used".
    const uint8_t* src = p.W + size_t(wA) * UNIT_BYTES;
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) {
        if (wA + d < wB) issue_unit(ring + d * UNIT_BYTES, src + size_t(d) * UNIT_BYTES, UNIT_BYTES, lane);
        ring_commit();
    }
    pdl_launch_dependents();
    pdl_wait();
    prefetch_act(p.limbs, p.n);
    const float inv_scale = __ldcg(p.inv_scale);

    Acc a{{0.f, 0.f}, {0.f, 0.f}};
    int slot = 0, rs = 0;           // rs: ring slot of the unit in hand
    int X = wA / upt, b = wA - X * upt;  // tile and block of the unit in hand
    if (lane == 0) { s_wfirst[warp] = X; s_wlast[warp] = wB > wA ? (wB - 1) / upt : X - 1; }
    const float wt = t < 2 ? (t & 1 ? 65536.0f : 1.0f) : 0.0f;
    const float wtm = (t & 1 ? 65536.0f : 1.0f) * (t & 2 ? 256.0f : 1.0f);
    for (int u = wA; u < wB; ++u) {
        {   // refill the slot that the previous iteration finished reading
            const int fs = rs == 0 ? DEPTH - 1 : rs - 1;
            if (u + DEPTH - 1 < wB) issue_unit(ring + fs * UNIT_BYTES, src + size_t(u - wA + DEPTH - 1) * UNIT_BYTES, UNIT_BYTES, lane);
            ring_commit();
        }
        ring_wait<DEPTH - 1>();
        __syncwarp();
        Unit<TYPE> cur;
        load_unit(cur, ring + rs * UNIT_BYTES, lane);
        rs = rs + 1 == DEPTH ? 0 : rs + 1;
        DbgOut dbg{p.dbgP, p.dbgI, p.dbgJ, int64_t(16) * X + g, p.rows, p.n / (TYPE == ELB_Q6_K ? 16 : 32), p.n / (TYPE == ELB_Q8_0 ? 32 : QK_K)};
        compute_unit<DBG>(cur, b, lim, n_pad, sd, lane, a, dbg);
        __syncwarp();  // every lane has its registers before the slot is refilled
        if (++b == upt || u + 1 == wB) {  // tile finished for this warp: row sums over the 4 lanes of a row
            float v0 = a.acc[0] * wt - a.accm[0] * wtm, v1 = a.acc[1] * wt - a.accm[1] * wtm;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (t == 0) {
                red[(warp * p.slots + slot) * 16 + g] = v0;
                red[(warp * p.slots + slot) * 16 + g + 8] = v1;
            }
            ++slot;
            a = Acc{{0.f, 0.f}, {0.f, 0.f}};
            if (b == upt) { b = 0; ++X; }
        }
    }
    ring_wait<0>();
    __syncthreads();

    // CTA-level sums in warp order; complete tiles go out, shared tiles go to the scratch buffer
    const int Xf = cA / upt, Xl = (cB - 1) / upt, ntl = Xl - Xf + 1;
    const bool part_first = Xf * upt < cA || (Xf + 1) * upt > cB;
    const bool part_last = Xl != Xf && (Xl + 1) * upt > cB;
    for (int e = tid; e < ntl * 8; e += GEMV_THREADS) {
        const int Xt = Xf + (e >> 3), gg = e & 7;
        float v0 = 0.f, v1 = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_WARPS; ++w) {
            const int f = s_wfirst[w];
            if (Xt < f || Xt > s_wlast[w]) continue;
            v0 += red[(w * p.slots + (Xt - f)) * 16 + gg];
            v1 += red[(w * p.slots + (Xt - f)) * 16 + gg + 8];
        }
        const bool partial = (Xt == Xf && part_first) || (Xt == Xl && part_last);
        if (!partial) {
            epilogue(p, Xt, gg, v0 * inv_scale, v1 * inv_scale);
        } else {
            float* dst = p.part + (c * 2 + (Xt == Xf ? 0 : 1)) * 16;
            dst[gg] = v0;
            dst[gg + 8] = v1;
        }
    }
    if (part_first || part_last) {  // uniform over the CTA
    __threadfence();
    __syncthreads();
    if (tid < 2) {
        s_last[tid] = 0;
        if (tid == 0 ? part_first : part_last) {
            const int Xt = tid == 0 ? Xf : Xl;
            const int c_lo = ((Xt * upt + 1) * G - 1) / U, c_hi = ((Xt + 1) * upt * G - 1) / U;
            const unsigned old = atomicAdd(&p.counters[Xt], 1u);
            if (old == unsigned(c_hi - c_lo)) {
                s_last[tid] = 1;
                p.counters[Xt] = 0;  // ready for the next launch; every other CTA has already arrived
            }
        }
    }
    __syncthreads();
    if (s_last[0] || s_last[1]) __threadfence();
    if (tid < 16 && s_last[tid >> 3]) {
        const int i = tid >> 3, gg = tid & 7, Xt = i == 0 ? Xf : Xl;
        const int c_lo = ((Xt * upt + 1) * G - 1) / U, c_hi = ((Xt + 1) * upt * G - 1) / U;
        float v0 = 0.f, v1 = 0.f;
        for (int cc = c_lo; cc <= c_hi; ++cc) {  // fixed CTA order
            const int first_tile = range_lo(U, G, cc) / upt;
            const float* srcp = p.part + (cc * 2 + (Xt == first_tile ? 0 : 1)) * 16;
            v0 += __ldcg(srcp + gg);
            v1 += __ldcg(srcp + gg + 8);
        }
        epilogue(p, Xt, gg, v0 * inv_scale, v1 * inv_scale);
    }
    }
    post_op(p.post, G, &s_last[0], red8);
}

// ---------------------------------------------------------------- F16 weights: fp32 FMA, two rows (g, g+8) per warp

struct GemvF16Params {
    const __half* W;
    int64_t tiles, rows;
    int n;
    const float* x;
    const float* norm_w;
    float eps;
    float* y;
    const float* resid;
    int prologue, epilogue;
    PostOp post;
};

__global__ void __launch_bounds__(GEMV_THREADS, 2) k_gemv_f16(const GemvF16Params p) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* xs = reinterpret_cast<float*>(smem);
    __shared__ double red8[GEMV_WARPS];
    __shared__ int s_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, n = p.n;
    pdl_launch_dependents();
    pdl_wait();
    float inv = 1.0f;
    if (p.prologue == PRO_RMSNORM) {
        double ss = 0.0;
        for (int i = tid; i < n; i += GEMV_THREADS) { const double v = p.x[i]; ss += v * v; }
        ss = block_sum(ss, red8, tid);
        inv = float(1.0 / sqrt(ss / n + double(p.eps)));
    }
    for (int i = tid; i < n; i += GEMV_THREADS) {
        const float v = p.x[i];
        xs[i] = p.prologue == PRO_RMSNORM ? __fmul_rn(__fmul_rn(v, inv), p.norm_w[i]) : v;
    }
    __syncthreads();
    const int pairs = int(p.tiles) * 8, GW = gridDim.x * GEMV_WARPS, wg = blockIdx.x * GEMV_WARPS + warp;
    for (int pr = range_lo(pairs, GW, wg); pr < range_lo(pairs, GW, wg + 1); ++pr) {
        const int64_t X = pr >> 3;
        const int g = pr & 7;
        const __half* w0 = p.W + (16 * X + g) * n;
        const __half* w1 = w0 + 8 * int64_t(n);
        float s0 = 0.f, s1 = 0.f;
        for (int k = lane * 8; k < n; k += 256) {
            const uint4 a = ldg_stream(w0 + k), b = ldg_stream(w1 + k);
            const float4 x0 = *reinterpret_cast<const float4*>(xs + k), x1 = *reinterpret_cast<const float4*>(xs + k + 4);
            const __half2* ah = reinterpret_cast<const __half2*>(&a);
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 fa = __half22float2(ah[q]), fb = __half22float2(bh[q]);
                s0 = fmaf(fa.x, xv[2 * q], s0);
                s0 = fmaf(fa.y, xv[2 * q + 1], s0);
                s1 = fmaf(fb.x, xv[2 * q], s1);
                s1 = fmaf(fb.y, xv[2 * q + 1], s1);
            }
        }
        s0 = warp_sum(s0);
        s1 = warp_sum(s1);
        if (lane == 0) {
            GemvParams q{};
            q.rows = p.rows; q.y = p.y; q.resid = p.resid; q.epilogue = p.epilogue;
            epilogue(q, X, g, s0, s1);
        }
    }
    post_op(p.post, gridDim.x, &s_flag, red8);
}

// Stand-alone limb split of one vector (one block): the first matvec of a chain, and the operator-level entry points.
__global__ void __launch_bounds__(SPLIT_THREADS) k_prep_limbs(const float* x, int n, const float* norm_w, float eps, int nl,
                                                             int8_t* limbs, float* inv_scale) {
    __shared__ double red8[SPLIT_WARPS];
    pdl_launch_dependents();
    pdl_wait();
    block_split(x, n, norm_w, eps, nl, limbs, inv_scale, red8);
}

// ---------------------------------------------------------------- host side

int gemv_prepare(Weight* w) {
    if (w->type == ELB_F16 || w->part) return ELB_OK;
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    w->max_grid = di.sm_count * 2;
    ELB_CUDA(cudaMalloc(&w->part, size_t(w->max_grid) * 2 * 16 * sizeof(float)));
    ELB_CUDA(cudaMalloc(&w->counters, size_t(w->tiles) * sizeof(unsigned)));
    ELB_CUDA(cudaMemset(w->counters, 0, size_t(w->tiles) * sizeof(unsigned)));
    ELB_CUDA(cudaMalloc(&w->xlimbs, act_bytes(int(w->n))));
    ELB_CUDA(cudaMalloc(&w->xinv, sizeof(float)));
    return ELB_OK;
}

template <typename K, typename P>
static int launch(K kernel, int grid, size_t smem, bool pdl, cudaStream_t s, const P& params) {
    static thread_local const void* configured[16] = {};
    static thread_local size_t configured_smem[16] = {};
    // raise the dynamic shared memory limit once per kernel (and again if a larger row length shows up)
    int slot = -1;
    for (int i = 0; i < 16; ++i)
        if (configured[i] == (const void*)kernel || !configured[i]) { slot = i; break; }
    if (slot >= 0 && (configured[slot] != (const void*)kernel || configured_smem[slot] < smem)) {
        ELB_CUDA(cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        configured[slot] = (const void*)kernel;
        configured_smem[slot] = smem;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    ELB_CUDA(cudaLaunchKernelEx(&cfg, kernel, params));
    return ELB_OK;
}

int prep_limbs_launch(const float* x, int n, const float* norm_w, float eps, int nl, int8_t* limbs, float* inv_scale,
                      bool pdl, cudaStream_t s) {
    if (nl < 2 || nl > 4) return fail(ELB_ERR_INVALID, "split: limb count must be 2, 3 or 4");
    if (n % 256) return fail(ELB_ERR_UNSUPPORTED, "split: vector length must be a multiple of 256");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(SPLIT_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    ELB_CUDA(cudaLaunchKernelEx(&cfg, k_prep_limbs, x, n, norm_w, eps, nl, limbs, inv_scale));
    return ELB_OK;
}

int gemv_launch(const Weight* w, const GemvArgs& a, cudaStream_t s) {
    if (!w || !a.y) return fail(ELB_ERR_INVALID, "matvec: null argument");
    if (a.epilogue == EPI_ADD && !a.resid) return fail(ELB_ERR_INVALID, "matvec: residual epilogue without residual");
    if (a.epilogue == EPI_SILU && !w->pair) return fail(ELB_ERR_INVALID, "matvec: SwiGLU epilogue needs a paired weight");
    if (a.post.kind && (!a.post.src || !a.post.limbs || !a.post.inv_scale || !a.post.done || a.post.n % 256))
        return fail(ELB_ERR_INVALID, "matvec: incomplete post-op");
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    if (w->type == ELB_F16) {
        if (!a.x) return fail(ELB_ERR_INVALID, "matvec: F16 weights take the fp32 activation");
        if (a.prologue == PRO_RMSNORM && !a.norm_w) return fail(ELB_ERR_INVALID, "matvec: RMSNorm prologue without weight");
        GemvF16Params p{reinterpret_cast<const __half*>(w->tiled), w->tiles, w->rows, int(w->n), a.x, a.norm_w, a.eps, a.y,
                        a.resid, a.prologue, a.epilogue, a.post};
        const size_t smem = size_t(w->n) * sizeof(float);
        if (smem > di.smem_optin) return fail(ELB_ERR_UNSUPPORTED, "matvec: row too long for shared memory");
        const int grid = int(std::min<int64_t>((w->tiles * 8 + GEMV_WARPS - 1) / GEMV_WARPS, int64_t(di.sm_count) * 2));
        return launch(k_gemv_f16, grid, smem, a.pdl, s, p);
    }
    if (!a.limbs || !a.inv_scale) return fail(ELB_ERR_INVALID, "matvec: quantized weights take the pre-split activation");
    if (!w->part) return fail(ELB_ERR_STATE, "matvec: weight scratch not prepared");
    if (w->tiles * w->units_per_tile * int64_t(w->max_grid) >= (int64_t(1) << 31) || w->tiles * 8 * int64_t(w->max_grid) * GEMV_WARPS >= (int64_t(1) << 31))
        return fail(ELB_ERR_UNSUPPORTED, "matvec: matrix too large for 32-bit unit indexing");
    const int64_t U = w->tiles * w->units_per_tile;
    // Grid: equal contiguous unit ranges, one CTA per SM (tiles on CTA borders are finished through the scratch buffer).
    static const int grid_override = [] { const char* v = std::getenv("ELB_GEMV_GRID"); return v ? std::atoi(v) : 0; }();
    int64_t grid64 = std::min<int64_t>(U, di.sm_count);  // one CTA per SM: the next kernel's CTAs fit beside them
    if (grid_override > 0) grid64 = std::min<int64_t>({U, int64_t(grid_override), int64_t(w->max_grid)});
    const int grid = int(grid64);
    const int64_t per_cta = (U + grid - 1) / grid, per_warp = (per_cta + GEMV_WARPS - 1) / GEMV_WARPS;
    const int slots = int((per_warp + w->units_per_tile - 1) / w->units_per_tile + 2);
    const size_t fixed = size_t(GEMV_WARPS) * slots * 16 * sizeof(float);
    // ring depth: as deep as two resident CTAs per SM allow (at most 4 units per warp), else one CTA per SM
    const size_t per_depth = size_t(GEMV_WARPS) * w->unit_bytes, two_cta_budget = (di.smem_optin + 1024) / 2 - 1024;
    static const int depth_override = [] { const char* v = std::getenv("ELB_GEMV_DEPTH"); return v ? std::atoi(v) : 0; }();
    int depth = fixed < two_cta_budget ? int((two_cta_budget - fixed) / per_depth) : 0;
    if (depth < 2) depth = fixed < di.smem_optin ? int((di.smem_optin - fixed) / per_depth) : 0;
    if (depth < 2) return fail(ELB_ERR_UNSUPPORTED, "matvec: row too long for shared memory");
    depth = std::min(depth, 6);
    if (depth_override >= 2 && depth_override <= 6 && fixed + depth_override * per_depth <= di.smem_optin) depth = depth_override;
    const bool dbg = a.dbgP || a.dbgI || a.dbgJ;
    if (dbg) depth = 2;
    if (depth == 5) depth = 4;
    const size_t smem = fixed + depth * per_depth;
    GemvParams p{w->tiled, w->tiles, w->units_per_tile, w->rows, int(w->n), a.limbs, a.inv_scale, a.y, a.resid,
                 w->part, w->counters, a.epilogue, slots, a.dbgP, a.dbgI, a.dbgJ, a.post};
#define ELB_GEMV_CASE(T)                                                                        \
    case T:                                                                                     \
        if (dbg) return launch(k_gemv<T, true, 2>, grid, smem, a.pdl, s, p);                     \
        if (depth == 2) return launch(k_gemv<T, false, 2>, grid, smem, a.pdl, s, p);             \
        if (depth == 3) return launch(k_gemv<T, false, 3>, grid, smem, a.pdl, s, p);             \
        if (depth <= 5) return launch(k_gemv<T, false, 4>, grid, smem, a.pdl, s, p);             \
        return launch(k_gemv<T, false, 6>, grid, smem, a.pdl, s, p);
    switch (w->type) {
        ELB_GEMV_CASE(ELB_Q4_K)
        ELB_GEMV_CASE(ELB_Q6_K)
        ELB_GEMV_CASE(ELB_Q8_0)
        default: return fail(ELB_ERR_UNSUPPORTED, "matvec: unsupported weight type");
    }
#undef ELB_GEMV_CASE
}

}  // namespace elb
