// Limb split of one activation vector by one thread block (k_split8 of the reference, src/cuda/model_cuda.cu:701-729,
// optionally with RMSNorm in front, src/ops.cpp:155-160): used as a stand-alone kernel and as the "post-op" that the
// last CTA of a producing kernel runs, so that the consuming matvec finds its limbs ready in global memory.
#pragma once

#include "common.cuh"

namespace elb {

constexpr int SPLIT_THREADS = 256, SPLIT_WARPS = SPLIT_THREADS / 32;
constexpr int SPLIT_V4 = 10;  // float4 per thread kept in registers: vectors of up to 10240 values need one pass

__device__ __forceinline__ float block_max(float v, float* red, int tid) {
    v = warp_max(v);
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float m = red[0];
#pragma unroll
    for (int i = 1; i < SPLIT_WARPS; ++i) m = fmaxf(m, red[i]);
    __syncthreads();
    return m;
}
__device__ __forceinline__ double block_sum(double v, double* red, int tid) {
    v = warp_sum(v);
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    double s = red[0];
#pragma unroll
    for (int i = 1; i < SPLIT_WARPS; ++i) s += red[i];
    __syncthreads();
    return s;
}

// Layout of one split activation vector in global memory (all int8): limbs [4][n], then the sums of each limb over
// the 32-wide sub-blocks and over the 16-wide sub-blocks as two balanced base-256 digits each, in the order the
// matvec's extra MMA reads them: sd32[n/256][col = limb + 4*digit][8 sub-blocks], sd16[n/256][col][16 sub-blocks].
__host__ __device__ __forceinline__ size_t act_bytes(int n) { return size_t(4) * n + size_t(n / 256) * (64 + 128); }
__host__ __device__ __forceinline__ size_t act_sd32_off(int n) { return size_t(4) * n; }
__host__ __device__ __forceinline__ size_t act_sd16_off(int n) { return size_t(4) * n + size_t(n / 256) * 64; }

// Four consecutive fixed-point values (index idx, a multiple of 4) -> one packed word of each of the 4 limbs (rows of
// `stride` bytes at lim), plus the
// limb sums of the enclosing 16- and 32-wide sub-blocks (shuffles over the 4 / 8 neighbouring lanes, which hold the rest
// of the sub-block: every lane of the warp must call this together). Balanced base-256 digits: adding 128 at every
// byte position turns them into the ordinary base-256 digits of v + 0x80808080, so the four limbs of one value are the
// bytes of (v + 0x80808080) ^ 0x80808080; a 4x4 byte transpose then groups them by limb.
__device__ __forceinline__ void split4(const float4& f, const Pow2 sc, int8_t* lim, int stride, int8_t* sd32, int8_t* sd16,
                                       int idx, bool valid) {
    const uint32_t a = (uint32_t(__float2int_rn(f.x * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t b = (uint32_t(__float2int_rn(f.y * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t c = (uint32_t(__float2int_rn(f.z * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t d = (uint32_t(__float2int_rn(f.w * sc.s1 * sc.s2)) + 0x80808080u) ^ 0x80808080u;
    const uint32_t ab01 = __byte_perm(a, b, 0x5140), ab23 = __byte_perm(a, b, 0x7362);  // a0 b0 a1 b1 | a2 b2 a3 b3
    const uint32_t cd01 = __byte_perm(c, d, 0x5140), cd23 = __byte_perm(c, d, 0x7362);
    const uint32_t w[4] = {__byte_perm(ab01, cd01, 0x5410), __byte_perm(ab01, cd01, 0x7632),   // limb 0, limb 1
                           __byte_perm(ab23, cd23, 0x5410), __byte_perm(ab23, cd23, 0x7632)};  // limb 2, limb 3
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
        if (valid) *reinterpret_cast<uint32_t*>(lim + size_t(l) * stride + idx) = w[l];
        int s = __dp4a(int(w[l]), 0x01010101, 0);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);  // sum over 16 values (lanes 4j..4j+3)
        const int s32 = s + __shfl_xor_sync(0xffffffffu, s, 4);
        if (valid && (lane & 3) == 0) {
            const int sub = idx >> 4, blk = sub >> 4, si = sub & 15;
            const int lo = ((s + 128) & 255) - 128;
            sd16[(blk * 8 + l) * 16 + si] = int8_t(lo);
            sd16[(blk * 8 + 4 + l) * 16 + si] = int8_t((s - lo) >> 8);
        }
        if (valid && (lane & 7) == 0) {
            const int sub = idx >> 5, blk = sub >> 3, si = sub & 7;
            const int lo = ((s32 + 128) & 255) - 128;
            sd32[(blk * 8 + l) * 8 + si] = int8_t(lo);
            sd32[(blk * 8 + 4 + l) * 8 + si] = int8_t((s32 - lo) >> 8);
        }
    }
}

__device__ __forceinline__ float4 norm4(const float4& v, float inv, const float4& w) {
    return make_float4(__fmul_rn(__fmul_rn(v.x, inv), w.x), __fmul_rn(__fmul_rn(v.y, inv), w.y),
                       __fmul_rn(__fmul_rn(v.z, inv), w.z), __fmul_rn(__fmul_rn(v.w, inv), w.w));
}
__device__ __forceinline__ float absmax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}
__device__ __forceinline__ int split_shift(float m, int nl) {  // k = 8 nl - 2 - e with m = f * 2^e, f in [0.5, 1)
    int e = 0;
    if (m > 0.f) frexpf(m, &e);
    return m > 0.f ? 8 * nl - 2 - e : 0;
}

// One block of SPLIT_THREADS threads: the split vector `out` (layout above; limbs beyond nl come out zero because
// |X| < 2^(8 nl - 2); n must be a multiple of 256) and *inv_scale = 2^-k. src is read through L2 (it may have been written by other CTAs of
// the running kernel). red: 8 doubles of shared memory.
// The split of a vector that the block already holds in registers: thread tid owns float4 number j * SPLIT_THREADS + tid
// in v[j] (zero beyond n). Returns k.
__device__ __forceinline__ int block_split_values(float4 (&v)[SPLIT_V4], int n, const float* norm_w, float eps, int nl,
                                                  int8_t* out, double* red) {
    const int tid = threadIdx.x;
    if (norm_w) {
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < SPLIT_V4; ++j)
            ss += double(v[j].x) * v[j].x + double(v[j].y) * v[j].y + double(v[j].z) * v[j].z + double(v[j].w) * v[j].w;
        ss = block_sum(ss, red, tid);
        const float inv = float(1.0 / sqrt(ss / n + double(eps)));
#pragma unroll
        for (int j = 0; j < SPLIT_V4; ++j) {
            const int idx = (j * SPLIT_THREADS + tid) * 4;
            if (idx < n) v[j] = norm4(v[j], inv, __ldg(reinterpret_cast<const float4*>(norm_w + idx)));
        }
    }
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < SPLIT_V4; ++j) m = fmaxf(m, absmax4(v[j]));
    const int k = split_shift(block_max(m, reinterpret_cast<float*>(red), tid), nl);
    const Pow2 sc = make_pow2(k);
#pragma unroll
    for (int j = 0; j < SPLIT_V4; ++j) {
        const int idx = (j * SPLIT_THREADS + tid) * 4;
        if (j * SPLIT_THREADS * 4 < n) split4(v[j], sc, out, n, out + act_sd32_off(n), out + act_sd16_off(n), idx, idx < n);  // warp-uniform guard: n % 128 == 0
    }
    return k;
}

__device__ __forceinline__ void block_split(const float* src, int n, const float* norm_w, float eps, int nl, int8_t* out,
                                            float* inv_scale, double* red) {
    const int tid = threadIdx.x;
    int k = 0;
    if (n <= SPLIT_V4 * 4 * SPLIT_THREADS) {  // all loads of the pass are in flight before the first use
        float4 v[SPLIT_V4];
#pragma unroll
        for (int j = 0; j < SPLIT_V4; ++j) {
            const int idx = (j * SPLIT_THREADS + tid) * 4;
            v[j] = idx < n ? __ldcg(reinterpret_cast<const float4*>(src + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        k = block_split_values(v, n, norm_w, eps, nl, out, red);
    } else {  // long vectors: passes over src, the later ones served by cache
        float inv = 1.0f;
        if (norm_w) {
            double ss = 0.0;
            for (int i = tid * 4; i < n; i += SPLIT_THREADS * 4) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(src + i));
                ss += double(f.x) * f.x + double(f.y) * f.y + double(f.z) * f.z + double(f.w) * f.w;
            }
            inv = float(1.0 / sqrt(block_sum(ss, red, tid) / n + double(eps)));
        }
        float m = 0.f;
        for (int i = tid * 4; i < n; i += SPLIT_THREADS * 4) {
            float4 f = __ldcg(reinterpret_cast<const float4*>(src + i));
            if (norm_w) f = norm4(f, inv, __ldg(reinterpret_cast<const float4*>(norm_w + i)));
            m = fmaxf(m, absmax4(f));
        }
        k = split_shift(block_max(m, reinterpret_cast<float*>(red), tid), nl);
        const Pow2 sc = make_pow2(k);
        for (int i = tid * 4; i < n; i += SPLIT_THREADS * 4) {
            float4 f = __ldcg(reinterpret_cast<const float4*>(src + i));
            if (norm_w) f = norm4(f, inv, __ldg(reinterpret_cast<const float4*>(norm_w + i)));
            split4(f, sc, out, n, out + act_sd32_off(n), out + act_sd16_off(n), i, true);
        }
    }
    if (tid == 0) *inv_scale = k <= 126 ? __int_as_float((127 - k) << 23) : ldexpf(1.0f, -k);  // 2^-k
}

// Called by every thread of every CTA of a producer kernel once the CTA's share of the output is written.
// The CTA that arrives last (of `n_ctas`) runs the split; returns after it is done. s_flag: one int of shared memory.
__device__ __forceinline__ void post_op(const PostOp& po, int n_ctas, int* s_flag, double* red) {
    if (po.kind == 0) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned old = atomicAdd(po.done, 1u);
        *s_flag = old == unsigned(n_ctas - 1);
        if (*s_flag) *po.done = 0;  // every CTA has arrived: ready for the next launch
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    block_split(po.src, po.n, po.norm_w, po.eps, po.nl, po.limbs, po.inv_scale, red);
}

}  // namespace elb
