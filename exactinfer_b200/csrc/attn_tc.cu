// Prompt-chunk attention on the tensor cores (mma.sync.m16n8k16, fp16 operands, fp32 accumulators).
//
// The reference computes prompt attention in fp32 (scores in dimension order, online softmax, src/model.cpp:191-214 and
// k_attn_prefill of src/cuda/model_cuda.cu). fp16 alone would lose 13 bits of every operand, so every operand goes in as
// an exact pair x = hi + lo of fp16 values (22 significant bits) and a product a*b is formed as a_hi*b_hi + a_hi*b_lo +
// a_lo*b_hi (each exact in fp32; the fourth term is 2^-22 of the product and left out): Q K^T and P V both cost three
// MMAs per step instead of one, and stay within the rounding of the fp32 path (parity tests hold the same bars).
//
// k_kv_split16 writes the layer's keys as K_hi, K_lo [keys][KD] and its values transposed as V^T_hi, V^T_lo [KD][keys]
// (what the B operand of P V wants: two neighbouring keys of one dimension in one 32-bit word), zero-padded to a multiple
// of 64 keys, once per prompt chunk and layer - every query tile would otherwise convert the same keys again.
// k_attn_prefill_tc: a CTA of four warps holds 64 query rows (all q heads of a KV head x 64/group tokens, as
// k_attn_prefill_gqa), a warp 16 of them; Q as fp16 pairs in registers, 64-key tiles of K and V^T in shared memory
// (padded rows, conflict-free fragment loads), scores and outputs in MMA accumulator fragments, online softmax on the
// fragments. The three products of every step are a chain of their own, started from zero, and join the running score or
// output in fp32 registers with rounding (the tensor core's own accumulation truncates toward zero). Keys are cut into chunks per query tile with
// the same partial-result layout and last-arrival combination as k_attn_prefill_gqa (deterministic chunk order).
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace elb {

namespace {

constexpr int D = 128;
constexpr int AT_ROWS = 64, AT_K = 64, AT_THREADS = 128, AT_MAXCHUNK = 8;
constexpr int AT_LDK = D + 8;      // halves per key row in shared memory: 272 bytes, fragment loads hit 32 banks
constexpr int AT_LDV = AT_K + 8;   // halves per dimension row of V^T: 144 bytes
constexpr int AT_PART = AT_ROWS * (D + 2);  // floats per partial result (layout of k_attn_prefill_gqa)
constexpr size_t AT_SMEM = size_t(2) * (AT_K * AT_LDK + D * AT_LDV + AT_ROWS * AT_LDK) * sizeof(__half);
constexpr float AT_PSCALE = 16384.0f;  // probabilities (<= 1) are split as p * 2^14: small ones keep their bits in fp16

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// d = a * b (the accumulator input is zero): the start of a short chain
__device__ __forceinline__ void mma_f16_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
// (x, y) -> fp16 pair hi (packed) and the packed remainder lo = (x - hi.x, y - hi.y), exact in fp32
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 f = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - f.x, y - f.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(dst))), "l"(src));
}

__host__ __device__ __forceinline__ int at_chunks(int pos0, int B, int TQ, int i, int kchunk) {  // chunks of query tile i
    const int T = pos0 + min(B, (i + 1) * TQ);
    return ((T + AT_K - 1) / AT_K + kchunk - 1) / kchunk;
}

// keys [0, T) of one layer and sequence -> fp16 pairs; grid (Tp / 32, KD / 64), 256 threads
__global__ void __launch_bounds__(256) k_kv_split16(const float* __restrict__ kc, const float* __restrict__ vc, int T, int Tp, int KD,
                                                    __half* __restrict__ kh, __half* __restrict__ kl, __half* __restrict__ vth,
                                                    __half* __restrict__ vtl) {
    __shared__ float vs[32][65];
    const int t0 = blockIdx.x * 32, d0 = blockIdx.y * 64, tid = threadIdx.x;
    for (int i = tid; i < 32 * 32; i += 256) {  // keys: 32 x 32 pairs of dimensions
        const int j = i >> 5, c = (i & 31) * 2;
        float2 k = make_float2(0.f, 0.f);
        if (t0 + j < T) k = *reinterpret_cast<const float2*>(kc + size_t(t0 + j) * KD + d0 + c);
        uint32_t hi, lo;
        split2(k.x, k.y, hi, lo);
        *reinterpret_cast<uint32_t*>(kh + size_t(t0 + j) * KD + d0 + c) = hi;
        *reinterpret_cast<uint32_t*>(kl + size_t(t0 + j) * KD + d0 + c) = lo;
    }
    for (int i = tid; i < 32 * 64; i += 256) {
        const int j = i >> 6, c = i & 63;
        vs[j][c] = t0 + j < T ? vc[size_t(t0 + j) * KD + d0 + c] : 0.f;
    }
    __syncthreads();
    for (int i = tid; i < 64 * 16; i += 256) {  // values transposed: 64 dimensions x 16 pairs of keys
        const int c = i >> 4, j = (i & 15) * 2;
        uint32_t hi, lo;
        split2(vs[j][c], vs[j + 1][c], hi, lo);
        *reinterpret_cast<uint32_t*>(vth + size_t(d0 + c) * Tp + t0 + j) = hi;
        *reinterpret_cast<uint32_t*>(vtl + size_t(d0 + c) * Tp + t0 + j) = lo;
    }
}

struct AtParams {
    const float* qkv;
    int64_t ld;
    const __half *kh, *kl, *vth, *vtl;  // [Tp][KD], [Tp][KD], [KD][Tp], [KD][Tp]
    int Tp, KD;
    float* att;
    int64_t ld_att;
    int pos0, B, H, HKV, kchunk;  // kchunk: 64-key tiles per chunk
    float scale;
    float* part;
    unsigned* counters;
};

__global__ void __launch_bounds__(AT_THREADS, 2) k_attn_prefill_tc(const AtParams p) {
    extern __shared__ __align__(16) uint8_t at_smem[];
    __half* Kh = reinterpret_cast<__half*>(at_smem);  // [64][AT_LDK]
    __half* Kl = Kh + AT_K * AT_LDK;
    __half* Vh = Kl + AT_K * AT_LDK;                  // [128][AT_LDV]  (V^T: row = dimension)
    __half* Vl = Vh + D * AT_LDV;
    __half* Qh = Vl + D * AT_LDV;                     // [64 rows][AT_LDK]
    __half* Ql = Qh + AT_ROWS * AT_LDK;
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x, group = p.H / p.HKV, TQ = AT_ROWS / group, n_qt = (p.B + TQ - 1) / TQ;
    int qt = 0, chunk = int(blockIdx.y), n_chunks = at_chunks(p.pos0, p.B, TQ, 0, p.kchunk);  // item -> (query tile, chunk)
    while (chunk >= n_chunks && qt + 1 < n_qt) {
        chunk -= n_chunks;
        ++qt;
        n_chunks = at_chunks(p.pos0, p.B, TQ, qt, p.kchunk);
    }
    const int q0 = qt * TQ, nq = min(TQ, p.B - q0);
    // this lane's two rows (row r = head * TQ + token): r0 = 16 warp + g, r1 = r0 + 8
    int last[2], head[2], tokq[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + 8 * i;
        head[i] = r / TQ;
        tokq[i] = r - head[i] * TQ;
        last[i] = tokq[i] < nq ? p.pos0 + q0 + tokq[i] : -1;
    }
    const __half* qh_row = Qh + (warp * 16 + g) * AT_LDK + 2 * t;  // (row g, dims 2t..), +8 rows, +8 dims
    const __half* ql_row = Ql + (warp * 16 + g) * AT_LDK + 2 * t;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const int T = min(p.pos0 + q0 + nq, (chunk + 1) * p.kchunk * AT_K);  // keys of this chunk: [chunk * kchunk * 64, T)
    // The K buffer is free once every warp has its scores, the V buffer once every warp has its outputs: the next
    // tile's keys travel during P V and its values during Q K^T. One commit group per request, in the order
    // K0, V0, K1, V1, ... (empty groups past the last tile), so "all but the newest group" is always the one needed next.
    auto load_k = [&](int t0) {
        if (t0 < T)
            for (int i = tid; i < AT_K * 16; i += AT_THREADS) {  // 64 keys x 16 pieces of 16 bytes, hi and lo
                const int j = i >> 4, c = (i & 15) * 8;
                cp16(Kh + j * AT_LDK + c, p.kh + size_t(t0 + j) * p.KD + kvh * D + c);
                cp16(Kl + j * AT_LDK + c, p.kl + size_t(t0 + j) * p.KD + kvh * D + c);
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto load_v = [&](int t0) {
        if (t0 < T)
            for (int i = tid; i < D * 8; i += AT_THREADS) {  // V^T: 128 dimensions x 8 pieces of 16 bytes
                const int d = i >> 3, c = (i & 7) * 8;
                cp16(Vh + d * AT_LDV + c, p.vth + size_t(kvh * D + d) * p.Tp + t0 + c);
                cp16(Vl + d * AT_LDV + c, p.vtl + size_t(kvh * D + d) * p.Tp + t0 + c);
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int t_first = chunk * p.kchunk * AT_K;
    load_k(t_first);
    load_v(t_first);
    // Q as fp16 pairs in shared memory (row r = head * TQ + token), read as A fragments per 16-dimension step
    for (int i = tid; i < AT_ROWS * 64; i += AT_THREADS) {
        const int r = i >> 6, c = (i & 63) * 2, h = r / TQ, tk = r - h * TQ;
        float2 q = make_float2(0.f, 0.f);
        if (tk < nq) q = *reinterpret_cast<const float2*>(p.qkv + int64_t(q0 + tk) * p.ld + (kvh * group + h) * D + c);
        uint32_t hi, lo;
        split2(q.x, q.y, hi, lo);
        *reinterpret_cast<uint32_t*>(Qh + r * AT_LDK + c) = hi;
        *reinterpret_cast<uint32_t*>(Ql + r * AT_LDK + c) = lo;
    }
    for (int t0 = t_first; t0 < T; t0 += AT_K) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile's keys (its values may still travel)
        __syncthreads();
        // ---- scores S[16 rows][64 keys] = Q K^T
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        // The tensor core adds into its accumulator with truncation (measured: 2^24 + 3.5 -> 2^24 + 2), a bias that grows
        // with the chain. The three products of one 16-dimension step form a chain of their own, started from zero, and
        // join the score in fp32 registers with rounding. Four key tiles' operands at a time, product by product, so that
        // MMAs which follow one another are independent.
#pragma unroll 2
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t qh[4], ql[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int off = ks * 16 + 8 * (i & 1) * AT_LDK + 8 * (i >> 1);
                qh[i] = *reinterpret_cast<const uint32_t*>(qh_row + off);
                ql[i] = *reinterpret_cast<const uint32_t*>(ql_row + off);
            }
#pragma unroll
            for (int n4 = 0; n4 < 8; n4 += 4) {
                uint32_t bh[4][2], bl[4][2];
                float tmp[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half* kh_row = Kh + ((n4 + j) * 8 + g) * AT_LDK + 2 * t + ks * 16;
                    const __half* kl_row = Kl + ((n4 + j) * 8 + g) * AT_LDK + 2 * t + ks * 16;
                    bh[j][0] = *reinterpret_cast<const uint32_t*>(kh_row); bh[j][1] = *reinterpret_cast<const uint32_t*>(kh_row + 8);
                    bl[j][0] = *reinterpret_cast<const uint32_t*>(kl_row); bl[j][1] = *reinterpret_cast<const uint32_t*>(kl_row + 8);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16_z(tmp[j], ql, bh[j][0], bh[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16(tmp[j], qh, bl[j][0], bl[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16(tmp[j], qh, bh[j][0], bh[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[n4 + j][0] += tmp[j][0]; s[n4 + j][1] += tmp[j][1]; s[n4 + j][2] += tmp[j][2]; s[n4 + j][3] += tmp[j][3];
                }
            }
        }
        __syncthreads();  // every warp has its scores: the key buffer is free
        load_k(t0 + AT_K);
        // ---- online softmax on the fragments: lane holds rows g (c0, c1) and g+8 (c2, c3), keys nt*8 + 2t, +1
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = t0 + nt * 8 + 2 * t + e;
                    float& v = s[nt][2 * i + e];
                    v = key <= last[i] ? __fmul_rn(v, p.scale) : -INFINITY;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[i], mx);
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float& v = s[nt][2 * i + e];
                    v = v == -INFINITY ? 0.f : expf(v - m_new);
                    sum += v;
                }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            corr[i] = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
            l[i] = l[i] * corr[i] + sum;
            m[i] = m_new;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile's values (the next keys may still travel)
        __syncthreads();
        // ---- outputs: O = O * corr + P V, every 16-key step a chain of three MMAs from zero that joins O with rounding
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            o[nt][0] *= corr[0]; o[nt][1] *= corr[0]; o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step: score tiles 2kk and 2kk+1 are the A fragment
            uint32_t ph[4], pl[4];
            split2(s[2 * kk][0] * AT_PSCALE, s[2 * kk][1] * AT_PSCALE, ph[0], pl[0]);
            split2(s[2 * kk][2] * AT_PSCALE, s[2 * kk][3] * AT_PSCALE, ph[1], pl[1]);
            split2(s[2 * kk + 1][0] * AT_PSCALE, s[2 * kk + 1][1] * AT_PSCALE, ph[2], pl[2]);
            split2(s[2 * kk + 1][2] * AT_PSCALE, s[2 * kk + 1][3] * AT_PSCALE, ph[3], pl[3]);
#pragma unroll
            for (int n4 = 0; n4 < 16; n4 += 4) {
                uint32_t bh[4][2], bl[4][2];
                float tmp[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int d = (n4 + j) * 8 + g;
                    const __half* vh_row = Vh + d * AT_LDV + kk * 16 + 2 * t;
                    const __half* vl_row = Vl + d * AT_LDV + kk * 16 + 2 * t;
                    bh[j][0] = *reinterpret_cast<const uint32_t*>(vh_row); bh[j][1] = *reinterpret_cast<const uint32_t*>(vh_row + 8);
                    bl[j][0] = *reinterpret_cast<const uint32_t*>(vl_row); bl[j][1] = *reinterpret_cast<const uint32_t*>(vl_row + 8);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16_z(tmp[j], pl, bh[j][0], bh[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16(tmp[j], ph, bl[j][0], bl[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_f16(tmp[j], ph, bh[j][0], bh[j][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    o[n4 + j][0] += tmp[j][0]; o[n4 + j][1] += tmp[j][1]; o[n4 + j][2] += tmp[j][2]; o[n4 + j][3] += tmp[j][3];
                }
            }
        }
        __syncthreads();  // every warp has its outputs: the value buffer is free
        load_v(t0 + AT_K);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // lane's outputs: row g (+8 i): dimensions nt*8 + 2t, +1 of o[nt][2i], o[nt][2i+1]; the 2^14 of the split goes out (exact)
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        o[nt][0] *= 1.0f / AT_PSCALE; o[nt][1] *= 1.0f / AT_PSCALE; o[nt][2] *= 1.0f / AT_PSCALE; o[nt][3] *= 1.0f / AT_PSCALE;
    }
    if (n_chunks > 1) {  // leave this chunk's result; the last chunk of the query tile to arrive adds them all
        float* base = p.part + (size_t(kvh) * n_qt + qt) * AT_MAXCHUNK * AT_PART;
        float* mine = base + size_t(chunk) * AT_PART;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float* dst = mine + (warp * 16 + g + 8 * i) * (D + 2);
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(dst + nt * 8 + 2 * t) = make_float2(o[nt][2 * i], o[nt][2 * i + 1]);
            if (t == 0) { dst[D] = m[i]; dst[D + 1] = l[i]; }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            unsigned* cnt = p.counters + size_t(kvh) * n_qt + qt;
            const unsigned old = atomicAdd(cnt, 1u);
            s_last = old == unsigned(n_chunks - 1);
            if (s_last) *cnt = 0;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = warp * 16 + g + 8 * i;
            float M = -INFINITY;
            for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, __ldcg(base + size_t(c) * AT_PART + r * (D + 2) + D));
            float L = 0.f;
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) o[nt][2 * i] = o[nt][2 * i + 1] = 0.f;
            for (int c = 0; c < n_chunks; ++c) {  // fixed chunk order
                const float* ps = base + size_t(c) * AT_PART + r * (D + 2);
                const float mc = __ldcg(ps + D);
                if (mc == -INFINITY) continue;
                const float w = expf(mc - M);
                L = fmaf(__ldcg(ps + D + 1), w, L);
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) {
                    const float2 a = __ldcg(reinterpret_cast<const float2*>(ps + nt * 8 + 2 * t));
                    o[nt][2 * i] = fmaf(a.x, w, o[nt][2 * i]);
                    o[nt][2 * i + 1] = fmaf(a.y, w, o[nt][2 * i + 1]);
                }
            }
            l[i] = L;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (last[i] < 0) continue;
        const float inv = 1.0f / l[i];
        float* dst = p.att + int64_t(q0 + tokq[i]) * p.ld_att + (kvh * group + head[i]) * D;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2*>(dst + nt * 8 + 2 * t) = make_float2(o[nt][2 * i] * inv, o[nt][2 * i + 1] * inv);
    }
}

}  // namespace

// halves of scratch for a context of n_ctx keys and KD = HKV * 128 cached values per key
size_t attn_prefill_tc_scratch_halves(int n_ctx, int KD) { return size_t(4) * size_t((n_ctx + AT_K - 1) / AT_K * AT_K) * KD; }

// ELB_ATTN_TC=0 selects the fp32 kernel of attn.cu instead.
bool attn_prefill_tc_usable(int H, int HKV, int64_t ld, int64_t ld_att) {
    static const bool on = [] { const char* v = std::getenv("ELB_ATTN_TC"); return !(v && v[0] == '0'); }();
    return on && HKV > 0 && H % HKV == 0 && AT_ROWS % (H / HKV) == 0 && ld % 2 == 0 && ld_att % 2 == 0;
}

// part / counters: the scratch of attn_prefill_launch (same sizes); kv16: attn_prefill_tc_scratch_halves(n_ctx, HKV * 128) halves
int attn_prefill_tc_launch(const float* qkv, int64_t ld, const float* kc, const float* vc, float* att, int64_t ld_att, int pos0,
                           int B, int H, int HKV, float scale, cudaStream_t s, float* part, unsigned* counters, void* kv16) {
    if (!attn_prefill_tc_usable(H, HKV, ld, ld_att) || !kv16 || !part || !counters)
        return fail(ELB_ERR_STATE, "attention: tensor-core prompt attention not usable here");
    const int T = pos0 + B, Tp = (T + AT_K - 1) / AT_K * AT_K, KD = HKV * D, group = H / HKV, TQ = AT_ROWS / group;
    __half* kh = static_cast<__half*>(kv16);
    __half* kl = kh + size_t(Tp) * KD;
    __half* vth = kl + size_t(Tp) * KD;
    __half* vtl = vth + size_t(Tp) * KD;
    k_kv_split16<<<dim3(Tp / 32, KD / 64), 256, 0, s>>>(kc, vc, T, Tp, KD, kh, kl, vth, vtl);
    ELB_CUDA(cudaGetLastError());
    ELB_TRY(ensure_dyn_smem(reinterpret_cast<const void*>(k_attn_prefill_tc), AT_SMEM));
    const int n_qt = (B + TQ - 1) / TQ, tiles_max = Tp / AT_K;
    // chunks of >= 256 keys (a CTA's fixed costs - Q, first tile, partial result - are worth several tiles), at most 8 per query tile
    static const int min_chunk = [] { const char* v = std::getenv("ELB_ATTN_TC_CHUNK"); return v ? std::max(1, atoi(v)) : 4; }();
    const int kchunk = std::max(min_chunk, (tiles_max + AT_MAXCHUNK - 1) / AT_MAXCHUNK);
    int items = 0;
    for (int i = 0; i < n_qt; ++i) items += at_chunks(pos0, B, TQ, i, kchunk);
    AtParams p{qkv, ld, kh, kl, vth, vtl, Tp, KD, att, ld_att, pos0, B, H, HKV, kchunk, scale, part, counters};
    k_attn_prefill_tc<<<dim3(HKV, items), AT_THREADS, AT_SMEM, s>>>(p);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
