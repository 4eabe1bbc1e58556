// Attention and the small per-head kernels around it, fp32 throughout (the KV cache stays fp32, as in the reference).
//
//   k_attn_decode   one token: per-head q/k RMSNorm + RoPE + KV store fused in front of a split-K flash decode; all
//                   q heads of a KV group share one pass over K/V; splits meet in a scratch buffer summed by the
//                   last CTA to arrive, in split order (deterministic).
//   k_qkv_post      prompt chunk: per-head q/k RMSNorm + RoPE in place, K/V rows stored to the cache.
//   k_attn_prefill  prompt chunk: causal tiled attention, 32 queries of one head per CTA, online softmax.
// Semantics follow CpuModel::forward of the reference (src/model.cpp:176-214): scale = 1/sqrt(float(D)), scores
// accumulated in dimension order without FMA contraction, max-subtracted softmax.
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "split.cuh"

namespace elb {

constexpr int D = 128;  // head_dim (checked at model creation)

// RMSNorm over one 128-wide head followed by NEOX RoPE (rmsnorm + rope, src/ops.cpp:155-160, src/model.cpp:23-32).
// One warp per head; lane owns elements lane, lane+32, lane+64, lane+96. Result goes to dst (shared or global).
__device__ __forceinline__ void head_norm_rope(const float* src, const float* w, const float2* cs, int rope_dim,
                                               float eps, float* dst, int lane) {
    float v[4];
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = src[lane + 32 * j];
        ss += double(v[j]) * v[j];
    }
    ss = warp_sum(ss);
    const float inv = float(1.0 / sqrt(ss / D + double(eps)));
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], inv), w[lane + 32 * j]);
    if (rope_dim == D) {  // pairs (i, i+64): both halves of a pair live in this lane
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 c = cs[lane + 32 * j];
            const float a = v[j], b = v[j + 2];
            v[j] = __fsub_rn(__fmul_rn(a, c.x), __fmul_rn(b, c.y));
            v[j + 2] = __fadd_rn(__fmul_rn(a, c.y), __fmul_rn(b, c.x));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = v[j];
    } else {  // partial rotary: pairs (i, i + rope_dim/2), the rest passes through
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = v[j];
        __syncwarp();
        const int half = rope_dim / 2;
        for (int i = lane; i < half; i += 32) {
            const float2 c = cs[i];
            const float a = dst[i], b = dst[i + half];
            dst[i] = __fsub_rn(__fmul_rn(a, c.x), __fmul_rn(b, c.y));
            dst[i + half] = __fadd_rn(__fmul_rn(a, c.y), __fmul_rn(b, c.x));
        }
    }
    __syncwarp();
}

// ---------------------------------------------------------------- decode

constexpr int AD_THREADS = 256, AD_KT = 32, AD_MAXG = 8, AD_LDK = D + 1, AD_MAXSPLIT = 32;

struct AttnDecodeParams {
    const float* qkv;  // [QD + 2 KD] of this token, q and k not yet normalised
    const float *q_norm, *k_norm;
    const float2* rope;  // [n_ctx][rope_dim/2] (cos, sin)
    const int* pos;      // device scalar
    float *kc, *vc;      // this layer's cache [n_ctx][KD]
    float* att;          // [QD]
    float* part;         // [HKV][nsplit][group][D + 2]
    unsigned* counters;  // [HKV]
    int H, HKV, rope_dim, nsplit;
    float eps, scale;
    PostOp post;
};

__global__ void __launch_bounds__(AD_THREADS) k_attn_decode(const AttnDecodeParams p) {
    __shared__ float qs[AD_MAXG][D];
    __shared__ float knew[D], vnew[D];
    __shared__ float Ks[AD_KT][AD_LDK];
    __shared__ float Vs[AD_KT][D];
    __shared__ float Ps[AD_MAXG][AD_KT];
    __shared__ float corr_s[AD_MAXG], m_s[AD_MAXG], l_s[AD_MAXG];
    __shared__ int s_last;
    __shared__ double red8[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, split = blockIdx.y, group = p.H / p.HKV, QD = p.H * D, KD = p.HKV * D;
    pdl_launch_dependents();
    pdl_wait();
    const int pos = *p.pos, T = pos + 1;
    const float2* cs = p.rope + size_t(pos) * (p.rope_dim / 2);

    for (int h = warp; h < group + 1; h += AD_THREADS / 32) {
        if (h < group) head_norm_rope(p.qkv + (kvh * group + h) * D, p.q_norm, cs, p.rope_dim, p.eps, qs[h], lane);
        else head_norm_rope(p.qkv + QD + kvh * D, p.k_norm, cs, p.rope_dim, p.eps, knew, lane);
    }
    if (tid < D) vnew[tid] = p.qkv[QD + KD + kvh * D + tid];
    __syncthreads();
    if (split == 0 && tid < D) {  // KV append (src/model.cpp:186-189): only row `pos` is written
        p.kc[size_t(pos) * KD + kvh * D + tid] = knew[tid];
        p.vc[size_t(pos) * KD + kvh * D + tid] = vnew[tid];
    }
    if (tid < AD_MAXG) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }

    // this split's key range, in whole tiles
    const int tiles = (T + AD_KT - 1) / AD_KT, per = (tiles + p.nsplit - 1) / p.nsplit;
    const int t_begin = min(T, split * per * AD_KT), t_end = min(T, (split + 1) * per * AD_KT);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // outputs (head tid/128 + 2i, dim tid%128)
    const int od = tid & (D - 1), oh = tid >> 7;

    for (int t0 = t_begin; t0 < t_end; t0 += AD_KT) {
        const int nk = min(AD_KT, t_end - t0);
        __syncthreads();
        for (int idx = tid; idx < AD_KT * (D / 4); idx += AD_THREADS) {
            const int j = idx / (D / 4), c = (idx % (D / 4)) * 4;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (j < nk) {
                const int t = t0 + j;
                if (t == pos) {  // the row this kernel appends: take it from shared memory, not from the cache
                    kv = *reinterpret_cast<const float4*>(&knew[c]);
                    vv = *reinterpret_cast<const float4*>(&vnew[c]);
                } else {
                    kv = *reinterpret_cast<const float4*>(p.kc + size_t(t) * KD + kvh * D + c);
                    vv = *reinterpret_cast<const float4*>(p.vc + size_t(t) * KD + kvh * D + c);
                }
            }
            Ks[j][c] = kv.x; Ks[j][c + 1] = kv.y; Ks[j][c + 2] = kv.z; Ks[j][c + 3] = kv.w;
            *reinterpret_cast<float4*>(&Vs[j][c]) = vv;
        }
        __syncthreads();
        // scores: warp = head, lane = key; dimension order, multiply then add (no contraction), as the CPU path does
        if (warp < group) {
            float s = -INFINITY;
            if (lane < nk) {
                float a = 0.f;
#pragma unroll 8
                for (int i = 0; i < D; ++i) a = __fadd_rn(a, __fmul_rn(qs[warp][i], Ks[lane][i]));
                s = __fmul_rn(a, p.scale);
            }
            const float m_old = m_s[warp], m_new = fmaxf(m_old, warp_max(s));
            const float pj = lane < nk ? expf(s - m_new) : 0.f;
            const float sum = warp_sum(pj);
            Ps[warp][lane] = pj;
            if (lane == 0) {
                const float c = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                corr_s[warp] = c;
                l_s[warp] = l_s[warp] * c + sum;
                m_s[warp] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = oh + 2 * i;
            if (h >= group) continue;
            float a = acc[i] * corr_s[h];
            for (int j = 0; j < nk; ++j) a = fmaf(Ps[h][j], Vs[j][od], a);
            acc[i] = a;
        }
    }
    __syncthreads();

    if (p.nsplit == 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = oh + 2 * i;
            if (h < group) p.att[(kvh * group + h) * D + od] = acc[i] / l_s[h];
        }
    } else {
        // partial result of this split: [group][D] accumulators, then m and l per head
        float* mine = p.part + (size_t(kvh) * p.nsplit + split) * group * (D + 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = oh + 2 * i;
            if (h < group) mine[h * (D + 2) + od] = acc[i];
        }
        if (tid < group) {
            mine[tid * (D + 2) + D] = m_s[tid];
            mine[tid * (D + 2) + D + 1] = l_s[tid];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned old = atomicAdd(&p.counters[kvh], 1u);
            s_last = old == unsigned(p.nsplit - 1);
            if (s_last) p.counters[kvh] = 0;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            const float* base = p.part + size_t(kvh) * p.nsplit * group * (D + 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int h = oh + 2 * i;
                if (h >= group) continue;
                // all loads of a pass are issued before the first use (the split count is at most AD_MAXSPLIT)
                float ms[AD_MAXSPLIT], ls[AD_MAXSPLIT], as[AD_MAXSPLIT];
#pragma unroll
                for (int s = 0; s < AD_MAXSPLIT; ++s) {
                    const float* ps = base + (size_t(s < p.nsplit ? s : 0) * group + h) * (D + 2);
                    ms[s] = s < p.nsplit ? __ldcg(ps + D) : -INFINITY;
                    ls[s] = __ldcg(ps + D + 1);
                    as[s] = __ldcg(ps + od);
                }
                float M = -INFINITY;
#pragma unroll
                for (int s = 0; s < AD_MAXSPLIT; ++s) M = fmaxf(M, ms[s]);
                float L = 0.f, o = 0.f;
#pragma unroll
                for (int s = 0; s < AD_MAXSPLIT; ++s) {  // fixed split order
                    if (ms[s] == -INFINITY) continue;
                    const float w = expf(ms[s] - M);
                    L = fmaf(ls[s], w, L);
                    o = fmaf(as[s], w, o);
                }
                p.att[(kvh * group + h) * D + od] = o / L;
            }
        }
    }
    post_op(p.post, gridDim.x * gridDim.y, &s_last, red8);
}

// ---------------------------------------------------------------- prompt chunk

// grid (B, ceil((H + 2 HKV) / 8)), blocks of 8 warps, one warp per (token, head). q heads: norm + rope in place. k heads: norm + rope in place and
// store to the cache row pos0 + b. v heads: store.
// posv / seqv (both or neither): row b sits at position posv[b] of sequence seqv[b], whose cache starts seq_stride
// floats after kc / vc; without them row b sits at position pos0 + b of the cache at kc / vc.
__global__ void __launch_bounds__(256) k_qkv_post(float* qkv, int64_t ld, const float* q_norm, const float* k_norm,
                                                 const float2* rope, int pos0, float* kc, float* vc, int H, int HKV,
                                                 int rope_dim, float eps, const int* posv, const int* seqv,
                                                 size_t seq_stride) {
    const int b = blockIdx.x, hd = blockIdx.y * 8 + threadIdx.y, lane = threadIdx.x, QD = H * D, KD = HKV * D;
    if (hd >= H + 2 * HKV) return;  // (warps only: nothing below synchronises the block)
    const int pos = posv ? posv[b] : pos0 + b;
    if (seqv) { kc += size_t(seqv[b]) * seq_stride; vc += size_t(seqv[b]) * seq_stride; }
    float* row = qkv + int64_t(b) * ld;
    const float2* cs = rope + size_t(pos) * (rope_dim / 2);
    if (hd < H) {
        head_norm_rope(row + hd * D, q_norm, cs, rope_dim, eps, row + hd * D, lane);
    } else if (hd < H + HKV) {
        float* k = row + QD + (hd - H) * D;
        head_norm_rope(k, k_norm, cs, rope_dim, eps, k, lane);
        for (int i = lane; i < D; i += 32) kc[size_t(pos) * KD + (hd - H) * D + i] = k[i];
    } else {
        const float* v = row + QD + KD + (hd - H - HKV) * D;
        for (int i = lane; i < D; i += 32) vc[size_t(pos) * KD + (hd - H - HKV) * D + i] = v[i];
    }
}

constexpr int AP_Q = 32, AP_K = 32, AP_THREADS = 256, AP_LD = D + 1;
constexpr size_t AP_SMEM = size_t(AP_Q * AP_LD + AP_K * AP_LD + AP_K * D + AP_Q * (AP_K + 1)) * sizeof(float);

// grid (H, ceil(B/32)). Query b of the chunk sits at position pos0 + b and sees keys 0..pos0+b (causal).
__global__ void __launch_bounds__(AP_THREADS) k_attn_prefill(const float* __restrict__ qkv, int64_t ld,
                                                             const float* __restrict__ kc, const float* __restrict__ vc,
                                                             float* __restrict__ att, int64_t ld_att, int pos0, int B, int H,
                                                             int HKV, float scale) {
    extern __shared__ __align__(16) float sm[];
    float (*Qs)[AP_LD] = reinterpret_cast<float (*)[AP_LD]>(sm);
    float (*Ks)[AP_LD] = reinterpret_cast<float (*)[AP_LD]>(sm + AP_Q * AP_LD);
    float (*Vs)[D] = reinterpret_cast<float (*)[D]>(sm + AP_Q * AP_LD + AP_K * AP_LD);
    float (*Ps)[AP_K + 1] = reinterpret_cast<float (*)[AP_K + 1]>(sm + AP_Q * AP_LD + AP_K * AP_LD + AP_K * D);
    const int tid = threadIdx.x, hd = blockIdx.x, q0 = blockIdx.y * AP_Q, KD = HKV * D, kvh = hd / (H / HKV);
    const int qi = tid >> 3, sub = tid & 7;  // 8 threads per query row
    const int nq = min(AP_Q, B - q0);
    for (int idx = tid; idx < AP_Q * D; idx += AP_THREADS) {
        const int r = idx / D, c = idx % D;
        Qs[r][c] = r < nq ? qkv[int64_t(q0 + r) * ld + hd * D + c] : 0.f;
    }
    float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    const int my_last = pos0 + q0 + qi;            // last key this query may see
    const int T = pos0 + q0 + nq;                  // keys needed by the tile
    for (int t0 = 0; t0 < T; t0 += AP_K) {
        __syncthreads();
        for (int idx = tid; idx < AP_K * (D / 4); idx += AP_THREADS) {
            const int j = idx / (D / 4), c = (idx % (D / 4)) * 4;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (t0 + j < T) {
                kv = *reinterpret_cast<const float4*>(kc + size_t(t0 + j) * KD + kvh * D + c);
                vv = *reinterpret_cast<const float4*>(vc + size_t(t0 + j) * KD + kvh * D + c);
            }
            Ks[j][c] = kv.x; Ks[j][c + 1] = kv.y; Ks[j][c + 2] = kv.z; Ks[j][c + 3] = kv.w;
            *reinterpret_cast<float4*>(&Vs[j][c]) = vv;
        }
        __syncthreads();
        float s[4] = {0.f, 0.f, 0.f, 0.f};  // keys sub + 8i
#pragma unroll 4
        for (int d = 0; d < D; ++d) {
            const float q = Qs[qi][d];
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] = __fadd_rn(s[i], __fmul_rn(q, Ks[sub + 8 * i][d]));
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s[i] = t0 + sub + 8 * i <= my_last ? __fmul_rn(s[i], scale) : -INFINITY;
            mx = fmaxf(mx, s[i]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m, mx);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float pj = s[i] == -INFINITY ? 0.f : expf(s[i] - m_new);
            Ps[qi][sub + 8 * i] = pj;
            sum += pj;
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * corr + sum;
        m = m_new;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= corr;
        const int nk = min(AP_K, T - t0);
        for (int j = 0; j < nk; ++j) {
            const float pj = Ps[qi][j];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = fmaf(pj, Vs[j][sub + 8 * i], acc[i]);
        }
    }
    if (qi < nq) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < 16; ++i) att[int64_t(q0 + qi) * ld_att + hd * D + sub + 8 * i] = acc[i] * inv;
    }
}

// Prompt chunk, all query heads of one KV head together: a CTA holds 64 query rows (group heads x 64/group tokens), so
// every K/V tile is loaded once for the whole group, and each thread keeps a 4-row x 2-key block of scores and a
// 4-row x 8-dim block of outputs in registers. Same arithmetic as k_attn_prefill: scores in dimension order, multiply
// then add, online softmax over 32-key tiles, causal.
// The keys of a query tile are cut into chunks of `kchunk` key tiles, one CTA per (query tile, chunk): late query tiles
// see many more keys than early ones, and without the cut the longest tile alone sets the kernel's duration. A query
// tile with one chunk writes its output directly; otherwise every chunk leaves (acc, m, l) in `part` and the last
// chunk to arrive adds them in chunk order (deterministic). grid (HKV, number of (query tile, chunk) items).
constexpr int AG_ROWS = 64, AG_K = 32, AG_LD = D + 4, AG_THREADS = 256, AG_LDP = AG_K + 1, AG_MAXCHUNK = 8;
constexpr size_t AG_SMEM = size_t(AG_ROWS * AG_LD + AG_K * AG_LD + AG_K * D + AG_ROWS * AG_LDP) * sizeof(float);
constexpr int AG_PART = AG_ROWS * (D + 2);  // floats per partial result

__host__ __device__ __forceinline__ int ag_chunks(int pos0, int B, int TQ, int i, int kchunk) {  // chunks of query tile i
    const int T = pos0 + min(B, (i + 1) * TQ);
    return ((T + AG_K - 1) / AG_K + kchunk - 1) / kchunk;
}

__global__ void __launch_bounds__(AG_THREADS) k_attn_prefill_gqa(const float* __restrict__ qkv, int64_t ld,
                                                                 const float* __restrict__ kc, const float* __restrict__ vc,
                                                                 float* __restrict__ att, int64_t ld_att, int pos0, int B,
                                                                 int H, int HKV, float scale, int kchunk, float* part,
                                                                 unsigned* counters) {
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;                        // [64][AG_LD]
    float* Ks = Qs + AG_ROWS * AG_LD;      // [32][AG_LD]
    float* Vs = Ks + AG_K * AG_LD;         // [32][D]
    float* Ps = Vs + AG_K * D;             // [64][33]
    __shared__ int s_last;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int kvh = blockIdx.x, group = H / HKV, TQ = AG_ROWS / group, KD = HKV * D, n_qt = (B + TQ - 1) / TQ;
    int qt = 0, chunk = int(blockIdx.y), n_chunks = ag_chunks(pos0, B, TQ, 0, kchunk);  // item -> (query tile, chunk)
    while (chunk >= n_chunks && qt + 1 < n_qt) {
        chunk -= n_chunks;
        ++qt;
        n_chunks = ag_chunks(pos0, B, TQ, qt, kchunk);
    }
    const int q0 = qt * TQ;
    const int nq = min(TQ, B - q0);
    for (int idx = tid; idx < AG_ROWS * (D / 4); idx += AG_THREADS) {  // row r = head * TQ + token
        const int r = idx / (D / 4), c = (idx % (D / 4)) * 4, h = r / TQ, t = r - h * TQ;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nq) v = *reinterpret_cast<const float4*>(qkv + int64_t(q0 + t) * ld + (kvh * group + h) * D + c);
        *reinterpret_cast<float4*>(Qs + r * AG_LD + c) = v;
    }
    int last[4];  // last key each of this thread's rows may see
    float m[4], l[4], acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i, t = r % TQ;
        last[i] = t < nq ? pos0 + q0 + t : -1;
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
    }
    const int T = min(pos0 + q0 + nq, (chunk + 1) * kchunk * AG_K);  // keys of this chunk: [chunk * kchunk * 32, T)
    for (int t0 = chunk * kchunk * AG_K; t0 < T; t0 += AG_K) {
        __syncthreads();
        for (int idx = tid; idx < AG_K * (D / 4); idx += AG_THREADS) {
            const int j = idx / (D / 4), c = (idx % (D / 4)) * 4;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (t0 + j < T) {
                kv = *reinterpret_cast<const float4*>(kc + size_t(t0 + j) * KD + kvh * D + c);
                vv = *reinterpret_cast<const float4*>(vc + size_t(t0 + j) * KD + kvh * D + c);
            }
            *reinterpret_cast<float4*>(Ks + j * AG_LD + c) = kv;
            *reinterpret_cast<float4*>(Vs + j * D + c) = vv;
        }
        __syncthreads();
        float sc[4][2];  // rows ty*4+i, keys tx and tx+16
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = 0.f;
#pragma unroll 4
        for (int d4 = 0; d4 < D / 4; ++d4) {
            float4 q[4], k[2];
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = *reinterpret_cast<const float4*>(Qs + (ty * 4 + i) * AG_LD + d4 * 4);
#pragma unroll
            for (int j = 0; j < 2; ++j) k[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * AG_LD + d4 * 4);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float a = sc[i][j];
                    a = __fadd_rn(a, __fmul_rn(q[i].x, k[j].x));
                    a = __fadd_rn(a, __fmul_rn(q[i].y, k[j].y));
                    a = __fadd_rn(a, __fmul_rn(q[i].z, k[j].z));
                    a = __fadd_rn(a, __fmul_rn(q[i].w, k[j].w));
                    sc[i][j] = a;
                }
        }
        float corr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                sc[i][j] = t0 + tx + 16 * j <= last[i] ? __fmul_rn(sc[i][j], scale) : -INFINITY;
                mx = fmaxf(mx, sc[i][j]);
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_new = fmaxf(m[i], mx);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float pj = sc[i][j] == -INFINITY ? 0.f : expf(sc[i][j] - m_new);
                Ps[(ty * 4 + i) * AG_LDP + tx + 16 * j] = pj;
                sum += pj;
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            corr[i] = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
            l[i] = l[i] * corr[i] + sum;
            m[i] = m_new;
        }
        __syncwarp();  // a row's 16 threads are half a warp
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[i][c] *= corr[i];
        const int nk = min(AG_K, T - t0);
        for (int j = 0; j < nk; ++j) {  // outputs: dims tx*4..+3 and 64+tx*4..+3
            const float4 v0 = *reinterpret_cast<const float4*>(Vs + j * D + tx * 4);
            const float4 v1 = *reinterpret_cast<const float4*>(Vs + j * D + 64 + tx * 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float pj = Ps[(ty * 4 + i) * AG_LDP + j];
                acc[i][0] = fmaf(pj, v0.x, acc[i][0]); acc[i][1] = fmaf(pj, v0.y, acc[i][1]);
                acc[i][2] = fmaf(pj, v0.z, acc[i][2]); acc[i][3] = fmaf(pj, v0.w, acc[i][3]);
                acc[i][4] = fmaf(pj, v1.x, acc[i][4]); acc[i][5] = fmaf(pj, v1.y, acc[i][5]);
                acc[i][6] = fmaf(pj, v1.z, acc[i][6]); acc[i][7] = fmaf(pj, v1.w, acc[i][7]);
            }
        }
        __syncwarp();
    }
    if (n_chunks > 1) {  // leave this chunk's result; the last chunk of the query tile to arrive adds them all
        float* base = part + (size_t(kvh) * n_qt + qt) * AG_MAXCHUNK * AG_PART;
        float* mine = base + size_t(chunk) * AG_PART;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float* o = mine + (ty * 4 + i) * (D + 2);
            *reinterpret_cast<float2*>(o + tx * 4) = make_float2(acc[i][0], acc[i][1]);  // rows of D + 2 floats: 8-byte aligned
            *reinterpret_cast<float2*>(o + tx * 4 + 2) = make_float2(acc[i][2], acc[i][3]);
            *reinterpret_cast<float2*>(o + 64 + tx * 4) = make_float2(acc[i][4], acc[i][5]);
            *reinterpret_cast<float2*>(o + 64 + tx * 4 + 2) = make_float2(acc[i][6], acc[i][7]);
            if (tx == 0) { o[D] = m[i]; o[D + 1] = l[i]; }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            unsigned* cnt = counters + size_t(kvh) * n_qt + qt;
            const unsigned old = atomicAdd(cnt, 1u);
            s_last = old == unsigned(n_chunks - 1);
            if (s_last) *cnt = 0;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = ty * 4 + i;
            float M = -INFINITY;
            for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, __ldcg(base + size_t(c) * AG_PART + r * (D + 2) + D));
            float L = 0.f;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) acc[i][c8] = 0.f;
            for (int c = 0; c < n_chunks; ++c) {  // fixed chunk order
                const float* ps = base + size_t(c) * AG_PART + r * (D + 2);
                const float mc = __ldcg(ps + D);
                if (mc == -INFINITY) continue;
                const float w = expf(mc - M);
                L = fmaf(__ldcg(ps + D + 1), w, L);
                const float2 a0 = __ldcg(reinterpret_cast<const float2*>(ps + tx * 4)), a1 = __ldcg(reinterpret_cast<const float2*>(ps + tx * 4 + 2));
                const float2 b0 = __ldcg(reinterpret_cast<const float2*>(ps + 64 + tx * 4)), b1 = __ldcg(reinterpret_cast<const float2*>(ps + 64 + tx * 4 + 2));
                acc[i][0] = fmaf(a0.x, w, acc[i][0]); acc[i][1] = fmaf(a0.y, w, acc[i][1]);
                acc[i][2] = fmaf(a1.x, w, acc[i][2]); acc[i][3] = fmaf(a1.y, w, acc[i][3]);
                acc[i][4] = fmaf(b0.x, w, acc[i][4]); acc[i][5] = fmaf(b0.y, w, acc[i][5]);
                acc[i][6] = fmaf(b1.x, w, acc[i][6]); acc[i][7] = fmaf(b1.y, w, acc[i][7]);
            }
            l[i] = L;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i, h = r / TQ, t = r - h * TQ;
        if (t >= nq) continue;
        const float inv = 1.0f / l[i];
        float* o = att + int64_t(q0 + t) * ld_att + (kvh * group + h) * D;
        *reinterpret_cast<float4*>(o + tx * 4) = make_float4(acc[i][0] * inv, acc[i][1] * inv, acc[i][2] * inv, acc[i][3] * inv);
        *reinterpret_cast<float4*>(o + 64 + tx * 4) = make_float4(acc[i][4] * inv, acc[i][5] * inv, acc[i][6] * inv, acc[i][7] * inv);
    }
}

// ---------------------------------------------------------------- rows of several sequences

// Row b of the batch is one token of sequence seqv[b] at position posv[b]; its q heads are normalised and rotated and
// its K/V row is in the cache already (k_qkv_post). Grid (B, HKV, nsplit): all q heads of a KV group share one pass
// over keys 0..posv[b] of that sequence; key splits meet in `part` and the last split to arrive adds them in split order.
// The same arithmetic as k_attn_decode (src/model.cpp:191-214 of the reference).
struct AttnRowsParams {
    const float* qkv;
    int64_t ld;
    const float *kc, *vc;  // this layer's cache of sequence 0; sequence s starts seq_stride floats later
    size_t seq_stride;
    const int *posv, *seqv;
    float* att;
    int64_t ld_att;
    float* part;         // [B][HKV][nsplit][group][D + 2]
    unsigned* counters;  // [B][HKV]
    int H, HKV, nsplit;
    float scale;
};

// Key / value tiles arrive by cp.async, the next tile while the current one is worked on: a CTA streams its whole key
// range (a sequence's context when there are enough rows to fill the GPU without a key split), so the bytes in flight
// per SM, not the arithmetic, set the pace.
constexpr int AR_LDK = D + 4;  // key row stride: 16-byte aligned rows, conflict-free 128-bit reads (lane = key)
constexpr int AR_KT = 24;       // keys per tile: two tiles of K and V are 50 KB, four CTAs per SM
constexpr size_t AR_SMEM = size_t(2) * AR_KT * (AR_LDK + D) * sizeof(float);

__global__ void __launch_bounds__(AD_THREADS) k_attn_rows(const AttnRowsParams p) {
    extern __shared__ __align__(16) float ar_tiles[];
    float* Ks = ar_tiles;                    // [2][AR_KT][AR_LDK]
    float* Vs = Ks + 2 * AR_KT * AR_LDK;     // [2][AR_KT][D]
    __shared__ __align__(16) float qs[AD_MAXG][D];
    __shared__ float Ps[AD_MAXG][32];  // (a warp writes all 32 lanes)
    __shared__ float corr_s[AD_MAXG], m_s[AD_MAXG], l_s[AD_MAXG];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, group = p.H / p.HKV, KD = p.HKV * D;
    const int T = p.posv[b] + 1;
    const float* kc = p.kc + size_t(p.seqv[b]) * p.seq_stride;
    const float* vc = p.vc + size_t(p.seqv[b]) * p.seq_stride;
    for (int idx = tid; idx < group * D; idx += AD_THREADS) qs[idx / D][idx % D] = p.qkv[int64_t(b) * p.ld + (kvh * group) * D + idx];
    if (tid < AD_MAXG) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    const int tiles = (T + AR_KT - 1) / AR_KT, per = (tiles + p.nsplit - 1) / p.nsplit;
    const int t_begin = min(T, split * per * AR_KT), t_end = min(T, (split + 1) * per * AR_KT);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // outputs (head tid/128 + 2i, dim tid%128)
    const int od = tid & (D - 1), oh = tid >> 7;
    auto fetch = [&](int buf, int t0, int nk) {
        const unsigned ks = unsigned(__cvta_generic_to_shared(Ks + buf * AR_KT * AR_LDK));
        const unsigned vs = unsigned(__cvta_generic_to_shared(Vs + buf * AR_KT * D));
        for (int idx = tid; idx < nk * (D / 4); idx += AD_THREADS) {
            const int j = idx / (D / 4), c = (idx % (D / 4)) * 4;
            const size_t off = size_t(t0 + j) * KD + kvh * D + c;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ks + unsigned(j * AR_LDK + c) * 4u), "l"(kc + off));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vs + unsigned(j * D + c) * 4u), "l"(vc + off));
        }
        asm volatile("cp.async.commit_group;");
    };
    if (t_begin < t_end) fetch(0, t_begin, min(AR_KT, t_end - t_begin));
    int buf = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += AR_KT, buf ^= 1) {
        const int nk = min(AR_KT, t_end - t0);
        if (t0 + AR_KT < t_end) {  // the other buffer was released by the barrier that ended the previous tile
            fetch(buf ^ 1, t0 + AR_KT, min(AR_KT, t_end - t0 - AR_KT));
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
        const float* Kb = Ks + buf * AR_KT * AR_LDK;
        const float* Vb = Vs + buf * AR_KT * D;
        if (warp < group) {  // scores: warp = head, lane = key; dimension order, multiply then add, as the CPU path does
            float sc = -INFINITY;
            if (lane < nk) {
                float a = 0.f;
                const float4* q = reinterpret_cast<const float4*>(qs[warp]);
                const float4* kr = reinterpret_cast<const float4*>(Kb + lane * AR_LDK);
#pragma unroll 8
                for (int i = 0; i < D / 4; ++i) {
                    const float4 qv = q[i], kv = kr[i];
                    a = __fadd_rn(a, __fmul_rn(qv.x, kv.x));
                    a = __fadd_rn(a, __fmul_rn(qv.y, kv.y));
                    a = __fadd_rn(a, __fmul_rn(qv.z, kv.z));
                    a = __fadd_rn(a, __fmul_rn(qv.w, kv.w));
                }
                sc = __fmul_rn(a, p.scale);
            }
            const float m_old = m_s[warp], m_new = fmaxf(m_old, warp_max(sc));
            const float pj = lane < nk ? expf(sc - m_new) : 0.f;
            const float sum = warp_sum(pj);
            Ps[warp][lane] = pj;
            if (lane == 0) {
                const float c = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                corr_s[warp] = c;
                l_s[warp] = l_s[warp] * c + sum;
                m_s[warp] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = oh + 2 * i;
            if (h >= group) continue;
            float a = acc[i] * corr_s[h];
            if (nk == AR_KT) {  // a whole tile: fixed trip count, the loads run ahead of the additions
#pragma unroll
                for (int j = 0; j < AR_KT; ++j) a = fmaf(Ps[h][j], Vb[j * D + od], a);
            } else {
                for (int j = 0; j < nk; ++j) a = fmaf(Ps[h][j], Vb[j * D + od], a);
            }
            acc[i] = a;
        }
        __syncthreads();  // the tile and Ps are free again
    }
    __syncthreads();
    float* out = p.att + int64_t(b) * p.ld_att;
    if (p.nsplit == 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int h = oh + 2 * i;
            if (h < group) out[(kvh * group + h) * D + od] = acc[i] / l_s[h];
        }
        return;
    }
    float* base = p.part + (size_t(b) * p.HKV + kvh) * p.nsplit * group * (D + 2);
    float* mine = base + size_t(split) * group * (D + 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int h = oh + 2 * i;
        if (h < group) mine[h * (D + 2) + od] = acc[i];
    }
    if (tid < group) {
        mine[tid * (D + 2) + D] = m_s[tid];
        mine[tid * (D + 2) + D + 1] = l_s[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned* cnt = p.counters + size_t(b) * p.HKV + kvh;
        const unsigned old = atomicAdd(cnt, 1u);
        s_last = old == unsigned(p.nsplit - 1);
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int h = oh + 2 * i;
        if (h >= group) continue;
        float M = -INFINITY;
        for (int q = 0; q < p.nsplit; ++q) M = fmaxf(M, __ldcg(base + (size_t(q) * group + h) * (D + 2) + D));
        float L = 0.f, o = 0.f;
        for (int q = 0; q < p.nsplit; ++q) {  // fixed split order
            const float* ps = base + (size_t(q) * group + h) * (D + 2);
            const float mq = __ldcg(ps + D);
            if (mq == -INFINITY) continue;
            const float w = expf(mq - M);
            L = fmaf(__ldcg(ps + D + 1), w, L);
            o = fmaf(__ldcg(ps + od), w, o);
        }
        out[(kvh * group + h) * D + od] = o / L;
    }
}

int attn_rows_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, size_t seq_stride, const int* posv,
                     const int* seqv, float* att, int64_t ld_att, float* part, unsigned* counters, int B, int H, int HKV,
                     int nsplit, float scale, cudaStream_t s) {
    if (H % HKV || H / HKV > AD_MAXG) return fail(ELB_ERR_UNSUPPORTED, "attention: at most 8 query heads per KV head");
    if (nsplit < 1 || nsplit > AD_MAXSPLIT) return fail(ELB_ERR_INVALID, "attention: split count out of range");
    AttnRowsParams p{qkv, ld, kc, vc, seq_stride, posv, seqv, att, ld_att, part, counters, H, HKV, nsplit, scale};
    ELB_TRY(ensure_dyn_smem((const void*)k_attn_rows, AR_SMEM));
    k_attn_rows<<<dim3(B, HKV, nsplit), AD_THREADS, AR_SMEM, s>>>(p);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

// ---------------------------------------------------------------- RMSNorm over rows (el::rmsnorm, src/ops.cpp:155-160)
__global__ void __launch_bounds__(256) k_rmsnorm_rows(float* out, const float* x, const float* w, int n, float eps) {
    __shared__ double red8[8];
    const int tid = threadIdx.x;
    const float* xr = x + int64_t(blockIdx.x) * n;
    float* o = out + int64_t(blockIdx.x) * n;
    double ss = 0.0;
    for (int i = tid; i < n; i += 256) { const double v = xr[i]; ss += v * v; }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red8[tid >> 5] = ss;
    __syncthreads();
    ss = 0.0;
    for (int i = 0; i < 8; ++i) ss += red8[i];
    const float inv = float(1.0 / sqrt(ss / n + double(eps)));
    for (int i = tid; i < n; i += 256) o[i] = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
}

// ---------------------------------------------------------------- logits post-processing
// What the reference's generate loop does on the host with the n_vocab logits of every token (src/main.cpp:309-320):
// log-sum-exp in double precision and the k best tokens ordered by (logit descending, id ascending). One block.
// allowed != nullptr: bit i of the array says whether token i may be picked (the log-sum-exp still covers all tokens).
// Block b reduces row b: logits + b * ld -> out + b * TOP_BYTES (one row: one block).
__global__ void __launch_bounds__(1024) k_logits_top(const float* __restrict__ logits, int n, int k, uint8_t* __restrict__ out,
                                                     const uint32_t* __restrict__ allowed, int64_t ld) {
    logits += int64_t(blockIdx.x) * ld;
    out += size_t(blockIdx.x) * TOP_BYTES;
    __shared__ double red_d[32];
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    __shared__ float s_val;
    __shared__ int s_idx;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -INFINITY;
    for (int i = tid; i < n; i += 1024) mx = fmaxf(mx, logits[i]);
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
    for (int w = 1; w < 32; ++w) mx = fmaxf(mx, red_f[w]);
    double sum = 0.0;
    for (int i = tid; i < n; i += 1024) sum += exp(double(logits[i]) - double(mx));
    sum = warp_sum(sum);
    if (lane == 0) red_d[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < 32; ++w) t += red_d[w];  // fixed order
        *reinterpret_cast<double*>(out) = double(mx) + log(t);
    }
    int32_t* ids = reinterpret_cast<int32_t*>(out + 8);
    float* vals = reinterpret_cast<float*>(out + 8 + 4 * TOP_MAXK);
    float pv = INFINITY;  // the previous pick: candidates come strictly after it in the order
    int pi = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < n; i += 1024) {
            const float v = logits[i];
            const bool after = (v < pv || (v == pv && i > pi)) && (!allowed || ((allowed[i >> 5] >> (i & 31)) & 1u));
            if (after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        __syncthreads();  // red_f / red_i free
        if (lane == 0) { red_f[warp] = bv; red_i[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 0; w < 32; ++w)
                if (red_f[w] > bv || (red_f[w] == bv && red_i[w] < bi)) { bv = red_f[w]; bi = red_i[w]; }
            s_val = bv; s_idx = bi;
            ids[r] = bi == 0x7fffffff ? -1 : bi;  // fewer than k tokens allowed: -1 from here on
            vals[r] = bv;
        }
        __syncthreads();
        pv = s_val; pi = s_idx;
    }
}

int logits_top_launch(const float* logits, int n, int k, uint8_t* out, cudaStream_t s, const uint32_t* d_allowed) {
    if (!logits || !out || n < 1 || k < 1 || k > TOP_MAXK || k > n) return fail(ELB_ERR_INVALID, "logits_top: bad argument");
    k_logits_top<<<1, 1024, 0, s>>>(logits, n, k, out, d_allowed, 0);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

// rows of logits [rows][ld] -> out [rows][TOP_BYTES], one block per row
int logits_top_rows_launch(const float* logits, int n, int64_t ld, int rows, int k, uint8_t* out, cudaStream_t s) {
    if (!logits || !out || n < 1 || rows < 1 || k < 1 || k > TOP_MAXK || k > n) return fail(ELB_ERR_INVALID, "logits_top: bad argument");
    k_logits_top<<<rows, 1024, 0, s>>>(logits, n, k, out, nullptr, ld);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

// ---------------------------------------------------------------- host side

int attn_decode_launch(const AttnDecodeArgs& a, cudaStream_t s) {
    if (a.H % a.HKV || a.H / a.HKV > AD_MAXG) return fail(ELB_ERR_UNSUPPORTED, "attention: at most 8 query heads per KV head");
    if (a.nsplit < 1 || a.nsplit > AD_MAXSPLIT) return fail(ELB_ERR_INVALID, "attention: split count out of range");
    AttnDecodeParams p{a.qkv, a.q_norm, a.k_norm, reinterpret_cast<const float2*>(a.rope), a.pos, a.kc, a.vc, a.att, a.part,
                       a.counters, a.H, a.HKV, a.rope_dim, a.nsplit, a.eps, a.scale, a.post};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.HKV, a.nsplit);
    cfg.blockDim = dim3(AD_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    ELB_CUDA(cudaLaunchKernelEx(&cfg, k_attn_decode, p));
    return ELB_OK;
}

int qkv_post_launch(float* qkv, int64_t ld, const float* q_norm, const float* k_norm, const float* rope, int pos0, int B,
                    float* kc, float* vc, int H, int HKV, int rope_dim, float eps, cudaStream_t s, const int* posv,
                    const int* seqv, size_t seq_stride) {
    k_qkv_post<<<dim3(B, (H + 2 * HKV + 7) / 8), dim3(32, 8), 0, s>>>(qkv, ld, q_norm, k_norm, reinterpret_cast<const float2*>(rope), pos0, kc,
                                                   vc, H, HKV, rope_dim, eps, posv, seqv, seq_stride);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

size_t attn_prefill_scratch_floats(int max_batch, int H, int HKV) {  // partial results of the chunked prompt attention
    const int group = std::max(1, H / HKV), TQ = AG_ROWS % group == 0 ? AG_ROWS / group : AG_ROWS;
    return size_t(HKV) * size_t((max_batch + TQ - 1) / TQ) * AG_MAXCHUNK * AG_PART;
}
size_t attn_prefill_counters(int max_batch, int H, int HKV) {
    const int group = std::max(1, H / HKV), TQ = AG_ROWS % group == 0 ? AG_ROWS / group : AG_ROWS;
    return size_t(HKV) * size_t((max_batch + TQ - 1) / TQ);
}

int attn_prefill_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, float* att, int64_t ld_att,
                        int pos0, int B, int H, int HKV, float scale, cudaStream_t s, float* part, unsigned* counters) {
    ELB_TRY(ensure_dyn_smem((const void*)k_attn_prefill, AP_SMEM));
    ELB_TRY(ensure_dyn_smem((const void*)k_attn_prefill_gqa, AG_SMEM));
    const int group = H / HKV;
    static const bool old_kernel = [] { const char* v = std::getenv("ELB_ATTN_SIMPLE"); return v && v[0] == '1'; }();
    if (!old_kernel && H % HKV == 0 && AG_ROWS % group == 0 && ld % 4 == 0 && ld_att % 4 == 0) {
        const int TQ = AG_ROWS / group, n_qt = (B + TQ - 1) / TQ;
        // chunks of 4 key tiles (128 keys), longer when the context is long enough to need more than AG_MAXCHUNK of them;
        // without scratch memory one chunk per query tile
        const int tiles_max = (pos0 + B + AG_K - 1) / AG_K;
        const int kchunk = part && counters ? std::max(4, (tiles_max + AG_MAXCHUNK - 1) / AG_MAXCHUNK) : tiles_max;
        int items = 0;
        for (int i = 0; i < n_qt; ++i) items += ag_chunks(pos0, B, TQ, i, kchunk);
        k_attn_prefill_gqa<<<dim3(HKV, items), AG_THREADS, AG_SMEM, s>>>(qkv, ld, kc, vc, att, ld_att, pos0, B, H, HKV, scale,
                                                                         kchunk, part, counters);
        ELB_CUDA(cudaGetLastError());
        return ELB_OK;
    }
    k_attn_prefill<<<dim3(H, (B + AP_Q - 1) / AP_Q), AP_THREADS, AP_SMEM, s>>>(qkv, ld, kc, vc, att, ld_att, pos0, B, H, HKV,
                                                                             scale);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

int rmsnorm_launch(float* out, const float* x, const float* w, int n, float eps, int rows, cudaStream_t s) {
    k_rmsnorm_rows<<<rows, 256, 0, s>>>(out, x, w, n, eps);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
