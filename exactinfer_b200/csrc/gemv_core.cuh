// Core of the limb-exact matvec, shared by the stand-alone kernel (gemv.cu) and the persistent decode kernel
// (decode.cu): one "unit" = the 16-row x 256-k (Q4_K, Q6_K) or 16-row x 128-k (Q8_0) piece of a tiled weight, how it
// travels HBM -> shared memory ring -> registers, and the integer MMA arithmetic on it.
//
// compute_unit: weights are the A-fragments of mma.sync.m16n8k32 / m16n8k16 (16 weight rows), the activation limbs the
// B-fragments (column = limb), so one MMA forms the four limb dot products of 16 rows over one sub-block exactly in
// int32. Integer sub-block scales are applied in int32; one conversion to fp32 per super-block. `lim` points at
// limbs [4][n_pad] and `sd` at the limb sub-block sums (layout in split.cuh), in shared or global memory.
#pragma once

#include "common.cuh"

namespace elb {

// start of part i when `total` items are cut into `parts` contiguous ranges (total * parts < 2^31, checked on the host)
__host__ __device__ __forceinline__ int range_lo(int total, int parts, int i) { return int(unsigned(total) * unsigned(i) / unsigned(parts)); }

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

// activation fragments: plain loads (the compiler picks LDS or LDG from the pointer; global ones hit L1)
// CG: through L2 only, for limbs in global memory that other CTAs of the SAME kernel wrote (L1 is not coherent)
template <bool CG, class T> __device__ __forceinline__ T ld_act(const T* p) {
    if constexpr (CG) return __ldcg(p);
    else return *p;
}

// prmt.b32 in its default mode: selector nibble k < 8 copies byte k of {a, b}; 8 + k fills the byte with byte k's sign
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
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
// bscale (optional): the activation was split block by block, 256-block b with its own power-of-two scale bscale[b];
// the block's sums are multiplied by it before they join the row sums (null: one scale for the whole vector, applied
// by the caller at the end).
template <bool DBG, bool CG = false>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q4_K>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t* sd, int lane, Acc& a, const DbgOut& dbg, const float* bscale = nullptr) {
    const int g = lane >> 2, t = lane & 3;
    const int8_t* lcol = lim + (g & 3) * n_pad + b * QK_K + 8 * t;
    // 6-bit scales and mins of rows g and g+8 as packed bytes (q4k_scale_min of the reference, src/quant.h:44-52)
    const uint32_t sg[2] = {u.h0.y & 0x3F3F3F3Fu, (u.h0.w & 0x0F0F0F0Fu) | ((u.h0.y >> 2) & 0x30303030u)};
    const uint32_t sh[2] = {u.h1.y & 0x3F3F3F3Fu, (u.h1.w & 0x0F0F0F0Fu) | ((u.h1.y >> 2) & 0x30303030u)};
    const uint32_t mg[2] = {u.h0.z & 0x3F3F3F3Fu, ((u.h0.w >> 4) & 0x0F0F0F0Fu) | ((u.h0.z >> 2) & 0x30303030u)};
    const uint32_t mh[2] = {u.h1.z & 0x3F3F3F3Fu, ((u.h1.w >> 4) & 0x0F0F0F0Fu) | ((u.h1.z >> 2) & 0x30303030u)};
    // even sub-blocks: low nibbles; odd sub-blocks: the high nibbles stay where they are (16 q, still a u8), their
    // products are accumulated apart and divided by 16 once per block (exact: every term is a multiple of 16)
    int I[4] = {0, 0, 0, 0}, I16[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 q = u.q[j];
#pragma unroll
        for (int odd = 0; odd < 2; ++odd) {
            const int sub = 2 * j + odd;
            const uint2 bf = ld_act<CG>(reinterpret_cast<const uint2*>(lcol + sub * 32));
            const uint32_t mask = odd ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
            int C[4];
            mma_u8s8_k32(C, q.x & mask, q.z & mask, q.y & mask, q.w & mask, bf.x, bf.y);
            const int s0 = int(__byte_perm(sg[sub >> 2], 0u, 0x4440 + (sub & 3))), s1 = int(__byte_perm(sh[sub >> 2], 0u, 0x4440 + (sub & 3)));
            if (odd) {
                I16[0] += s0 * C[0]; I16[1] += s0 * C[1]; I16[2] += s1 * C[2]; I16[3] += s1 * C[3];
            } else {
                I[0] += s0 * C[0]; I[1] += s0 * C[1]; I[2] += s1 * C[2]; I[3] += s1 * C[3];
            }
            if (DBG && dbg.P && t < 2) {
                const int sh4 = odd ? 4 : 0;
                const int64_t s = int64_t(b) * 8 + sub;
                if (dbg.row_g < dbg.rows) {
                    dbg.P[(dbg.row_g * dbg.nsub + s) * 4 + 2 * t] = C[0] >> sh4;
                    dbg.P[(dbg.row_g * dbg.nsub + s) * 4 + 2 * t + 1] = C[1] >> sh4;
                }
                if (dbg.row_g + 8 < dbg.rows) {
                    dbg.P[((dbg.row_g + 8) * dbg.nsub + s) * 4 + 2 * t] = C[2] >> sh4;
                    dbg.P[((dbg.row_g + 8) * dbg.nsub + s) * 4 + 2 * t + 1] = C[3] >> sh4;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) I[i] += I16[i] >> 4;
    const float xs = bscale ? ld_act<CG>(bscale + b) : 1.0f;
    const float dg = h2f_bits(u.h0.x & 0xFFFFu) * xs, dh = h2f_bits(u.h1.x & 0xFFFFu) * xs;
    a.acc[0] += dg * fmaf(float(I[1]), 256.0f, float(I[0]));
    a.acc[1] += dh * fmaf(float(I[3]), 256.0f, float(I[2]));
    // min term: J[col] = sum over the 8 sub-blocks of m * (digit `col>>2` of the limb sum S of limb `col&3`)
    const uint32_t a0 = t == 0 ? mg[0] : t == 1 ? mg[1] : 0u, a1 = t == 0 ? mh[0] : t == 1 ? mh[1] : 0u;
    const uint32_t b0 = ld_act<CG>(reinterpret_cast<const uint32_t*>(sd + (b * 8 + g) * 8 + 4 * (t & 1)));
    int J[4];
    mma_u8s8_k16(J, a0, a1, b0);
    const float ng = h2f_bits(u.h0.x >> 16) * xs, nh = h2f_bits(u.h1.x >> 16) * xs;
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
template <bool DBG, bool CG = false>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q6_K>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t* sd, int lane, Acc& a, const DbgOut& dbg, const float* bscale = nullptr) {
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
            // the two high bits of each q6 moved to bits 4-5 of its byte with one shift and one mask
            const uint32_t hx = (i < 2 ? qh.x << (4 - 2 * i) : qh.x >> (2 * i - 4)) & 0x30303030u;
            const uint32_t hy = (i < 2 ? qh.y << (4 - 2 * i) : qh.y >> (2 * i - 4)) & 0x30303030u;
            const uint32_t a0 = (w & 0x0F0F0F0Fu) | hx;
            const uint32_t a1 = ((w >> 4) & 0x0F0F0F0Fu) | hy;
            const uint32_t bf = ld_act<CG>(reinterpret_cast<const uint32_t*>(lcol + s * 16));
            int C[4];
            mma_u8s8_k16(C, a0, a1, bf);
            // int8 scale of sub-block s, sign-extended by the byte permute (selector 8+k replicates byte k's sign)
            const uint32_t sel = 0x8880u + 0x1111u * (s & 3);
            const int s0 = int(prmt(sel4(u.s0, s >> 2), 0u, sel)), s1 = int(prmt(sel4(u.s1, s >> 2), 0u, sel));
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
    const float xs = bscale ? ld_act<CG>(bscale + b) : 1.0f;
    const float dg = h2f_bits(u.dd & 0xFFFFu) * xs, dh = h2f_bits(u.dd >> 16) * xs;
    a.acc[0] += dg * fmaf(float(I[1]), 256.0f, float(I[0]));
    a.acc[1] += dh * fmaf(float(I[3]), 256.0f, float(I[2]));
    const uint32_t b0 = ld_act<CG>(reinterpret_cast<const uint32_t*>(sd + (b * 8 + g) * 16 + 4 * t));
    int J[4];
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
template <bool DBG, bool CG = false>
__device__ __forceinline__ void compute_unit(const Unit<ELB_Q8_0>& u, int b, const int8_t* lim, int n_pad,
                                             const int8_t*, int lane, Acc& a, const DbgOut& dbg, const float* bscale = nullptr) {
    const int g = lane >> 2, t = lane & 3;
    const float xs = bscale ? ld_act<CG>(bscale + (b >> 1)) : 1.0f;  // a unit is half a 256-block
    const int8_t* lcol = lim + (g & 3) * n_pad + b * (QK8_0 * Q8_GROUP) + 8 * t;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 q = u.q[i];
        const uint2 bf = ld_act<CG>(reinterpret_cast<const uint2*>(lcol + i * 32));
        int C[4];
        mma_s8s8_k32(C, q.x, q.z, q.y, q.w, bf.x, bf.y);
        const uint32_t d0w = i < 2 ? u.d0.x : u.d0.y, d1w = i < 2 ? u.d1.x : u.d1.y;
        const float dg = h2f_bits((d0w >> (16 * (i & 1))) & 0xFFFFu) * xs, dh = h2f_bits((d1w >> (16 * (i & 1))) & 0xFFFFu) * xs;
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


}  // namespace elb
