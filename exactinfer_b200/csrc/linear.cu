// Multi-token linear layers: limb split of the activations and the integer GEMM over the int8 digit planes.
//
// k_split_rows   X[b][n] (optionally RMSNorm'ed on the fly) -> limbs[4][b][n] int8, inv_scale[b], xsum[b][n/32]
// k_gemm_planes  mma.sync.m16n8k32 int8 GEMM, C[row][token,limb] exact in int32, scales per 256-block (per 32 for
//                Q8_0) — the portable tensor-core path (and the cross-check for the tcgen05 kernel).
#include <algorithm>

#include "common.cuh"

namespace elb {

// ---------------------------------------------------------------- limb split (k_split8 of the reference)

// One block per row. The row stays in registers (float4 j * 256 + tid of the row, up to SR_V4 * 1024 values); longer
// rows take the general kernel below.
constexpr int SR_V4 = 10;

__global__ void __launch_bounds__(256) k_split_rows(const float* __restrict__ X, int64_t ldx, int n, int nl,
                                                    const float* __restrict__ norm_w, float eps, int8_t* __restrict__ limbs,
                                                    int64_t limb_stride, float* __restrict__ inv_scale,
                                                    float* __restrict__ xsum) {
    __shared__ double red8[8];
    __shared__ float redf[8];
    const int tid = threadIdx.x, lane = tid & 31;
    const int64_t b = blockIdx.x;
    const float* x = X + b * ldx;
    pdl_launch_dependents();
    pdl_wait();  // the rows come from the kernel before this one
    float4 v[SR_V4];
#pragma unroll
    for (int j = 0; j < SR_V4; ++j) {
        const int idx = (j * 256 + tid) * 4;
        v[j] = idx < n ? __ldcg(reinterpret_cast<const float4*>(x + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (norm_w) {
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < SR_V4; ++j)
            ss += double(v[j].x) * v[j].x + double(v[j].y) * v[j].y + double(v[j].z) * v[j].z + double(v[j].w) * v[j].w;
        ss = warp_sum(ss);
        if (lane == 0) red8[tid >> 5] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < 8; ++i) ss += red8[i];
        const float inv = float(1.0 / sqrt(ss / n + double(eps)));
#pragma unroll
        for (int j = 0; j < SR_V4; ++j) {
            const int idx = (j * 256 + tid) * 4;
            if (idx < n) {
                const float4 w = __ldg(reinterpret_cast<const float4*>(norm_w + idx));
                v[j] = make_float4(__fmul_rn(__fmul_rn(v[j].x, inv), w.x), __fmul_rn(__fmul_rn(v[j].y, inv), w.y),
                                   __fmul_rn(__fmul_rn(v[j].z, inv), w.z), __fmul_rn(__fmul_rn(v[j].w, inv), w.w));
            }
        }
    }
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < SR_V4; ++j) m = fmaxf(m, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
    m = warp_max(m);
    if (lane == 0) redf[tid >> 5] = m;
    __syncthreads();
    m = redf[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, redf[i]);
    int e = 0;
    if (m > 0.f) frexpf(m, &e);
    const int k = m > 0.f ? 8 * nl - 2 - e : 0;
    int8_t* out = limbs + b * n;
    const Pow2 sc = make_pow2(k);
#pragma unroll
    for (int j = 0; j < SR_V4; ++j) {
        if (j * 1024 >= n) break;  // warp-uniform: n is a multiple of 32, so a warp's 128 values are all inside or all outside
        const int idx = (j * 256 + tid) * 4;
        const bool valid = idx < n;
        const int i0 = __float2int_rn(v[j].x * sc.s1 * sc.s2), i1 = __float2int_rn(v[j].y * sc.s1 * sc.s2);
        const int i2 = __float2int_rn(v[j].z * sc.s1 * sc.s2), i3 = __float2int_rn(v[j].w * sc.s1 * sc.s2);
        // balanced digits of one value = bytes of (v + 0x80808080) ^ 0x80808080; a 4x4 byte transpose groups them by limb
        const uint32_t a = (uint32_t(i0) + 0x80808080u) ^ 0x80808080u, bb = (uint32_t(i1) + 0x80808080u) ^ 0x80808080u;
        const uint32_t c = (uint32_t(i2) + 0x80808080u) ^ 0x80808080u, d = (uint32_t(i3) + 0x80808080u) ^ 0x80808080u;
        const uint32_t ab01 = __byte_perm(a, bb, 0x5140), ab23 = __byte_perm(a, bb, 0x7362);
        const uint32_t cd01 = __byte_perm(c, d, 0x5140), cd23 = __byte_perm(c, d, 0x7362);
        if (valid) {
            *reinterpret_cast<uint32_t*>(out + idx) = __byte_perm(ab01, cd01, 0x5410);
            *reinterpret_cast<uint32_t*>(out + limb_stride + idx) = __byte_perm(ab01, cd01, 0x7632);
            *reinterpret_cast<uint32_t*>(out + 2 * limb_stride + idx) = __byte_perm(ab23, cd23, 0x5410);
            *reinterpret_cast<uint32_t*>(out + 3 * limb_stride + idx) = __byte_perm(ab23, cd23, 0x7632);
        }
        if (xsum) {  // sum of the fixed-point values over each 32-slice (8 lanes), exact in 64 bits, rounded once
            long long sum = (long long)i0 + i1 + i2 + i3;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if (valid && (lane & 7) == 0) xsum[b * (n / 32) + (idx >> 5)] = float(sum);
        }
    }
    if (tid == 0) inv_scale[b] = ldexpf(1.0f, -k);
}

// rows longer than SR_V4 * 1024 values: passes over global memory
__global__ void __launch_bounds__(256) k_split_rows_long(const float* __restrict__ X, int64_t ldx, int n, int nl,
                                                         const float* __restrict__ norm_w, float eps, int8_t* __restrict__ limbs,
                                                         int64_t limb_stride, float* __restrict__ inv_scale,
                                                         float* __restrict__ xsum) {
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
    const int k = m > 0.f ? 8 * nl - 2 - e : 0;
    int8_t* out = limbs + b * n;
    const Pow2 sc = make_pow2(k);
    for (int i = tid; i < n; i += 256) {
        int v = __float2int_rn(val(i) * sc.s1 * sc.s2);
#pragma unroll
        for (int l = 0; l < 3; ++l) {
            const int a = ((v + 128) & 255) - 128;
            out[l * limb_stride + i] = int8_t(a);
            v = (v - a) >> 8;
        }
        out[3 * limb_stride + i] = int8_t(v);
    }
    if (tid == 0) inv_scale[b] = ldexpf(1.0f, -k);
    if (xsum) {  // sum of the fixed-point values over each 32-slice, exact in int64, rounded once
        for (int c = tid; c < n / 32; c += 256) {
            long long s = 0;
            for (int i = 0; i < 32; ++i) s += __float2int_rn(val(32 * c + i) * sc.s1 * sc.s2);
            xsum[b * (n / 32) + c] = float(s);
        }
    }
}

int split_launch(const float* d_x, int64_t ldx, int64_t b, int n, int nl, const float* d_norm_w, float eps,
                 int8_t* d_limbs, float* d_inv_scale, float* d_xsum, cudaStream_t s, bool pdl) {
    if (nl < 2 || nl > 4) return fail(ELB_ERR_INVALID, "split: limb count must be 2, 3 or 4");
    const bool fast = n <= SR_V4 * 1024 && n % 32 == 0 && ldx % 4 == 0 && (b * int64_t(n)) % 4 == 0 &&
                      reinterpret_cast<uintptr_t>(d_x) % 16 == 0 && (!d_norm_w || reinterpret_cast<uintptr_t>(d_norm_w) % 16 == 0);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(b));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // (rows too long for registers take several passes over global memory: launched early, that kernel ran slower -
    // 4.6 % of the 32B prompt time - so only the one-pass kernel is)
    cfg.numAttrs = pdl && fast ? 1 : 0;
    const int64_t limb_stride = b * int64_t(n);
    if (fast) ELB_CUDA(cudaLaunchKernelEx(&cfg, k_split_rows, d_x, ldx, n, nl, d_norm_w, eps, d_limbs, limb_stride, d_inv_scale, d_xsum));
    else ELB_CUDA(cudaLaunchKernelEx(&cfg, k_split_rows_long, d_x, ldx, n, nl, d_norm_w, eps, d_limbs, limb_stride, d_inv_scale, d_xsum));
    return ELB_OK;
}

// ---------------------------------------------------------------- plane GEMM with mma.sync

constexpr int GM_ROWS = 64, GM_TOK = 32, GM_K = 128, GM_PAD = 16, GM_LD = GM_K + GM_PAD, GM_THREADS = 128;

struct GemmParams {
    const int8_t* planes;  // [npl][rows16][n]
    const __half* pl_d;
    const float* pl_dm;
    const int8_t* limbs;   // [4][B][n]
    const float* inv_scale;
    const float* xsum;
    float* Y;
    const float* resid;
    int64_t rows16, rows, ldy;
    int B, n, npl, blk, epilogue;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned sa = unsigned(__cvta_generic_to_shared(smem));
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

template <int NPL>
__global__ void __launch_bounds__(GM_THREADS) k_gemm_planes(const GemmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int W_STAGE = NPL * GM_ROWS * GM_LD, A_STAGE = 4 * GM_TOK * GM_LD, STAGE = W_STAGE + A_STAGE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int64_t row0 = int64_t(blockIdx.x) * GM_ROWS;
    const int tok0 = blockIdx.y * GM_TOK;
    const int nk = p.n / GM_K;

    auto load_stage = [&](int st, int kt) {
        int8_t* ws = reinterpret_cast<int8_t*>(smem) + st * STAGE;
        int8_t* as = ws + W_STAGE;
        const int k0 = kt * GM_K;
        for (int idx = tid; idx < NPL * GM_ROWS * (GM_K / 16); idx += GM_THREADS) {
            const int pl = idx / (GM_ROWS * (GM_K / 16)), r = (idx / (GM_K / 16)) % GM_ROWS, c = idx % (GM_K / 16);
            const bool ok = row0 + r < p.rows16;
            cp_async16(ws + (pl * GM_ROWS + r) * GM_LD + c * 16,
                       p.planes + (int64_t(pl) * p.rows16 + (ok ? row0 + r : 0)) * p.n + k0 + c * 16, ok);
        }
        for (int idx = tid; idx < 4 * GM_TOK * (GM_K / 16); idx += GM_THREADS) {
            const int l = idx / (GM_TOK * (GM_K / 16)), r = (idx / (GM_K / 16)) % GM_TOK, c = idx % (GM_K / 16);
            const bool ok = tok0 + r < p.B;
            cp_async16(as + (l * GM_TOK + r) * GM_LD + c * 16,
                       p.limbs + (int64_t(l) * p.B + (ok ? tok0 + r : 0)) * p.n + k0 + c * 16, ok);
        }
        cp_async_commit();
    };

    int acc[NPL][4][4][4];  // [plane][token frag][limb][C reg]
    float yacc[4][4];       // [token frag][C reg]
#pragma unroll
    for (int a = 0; a < NPL; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int d = 0; d < 4; ++d) acc[a][b][c][d] = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int d = 0; d < 4; ++d) yacc[b][d] = 0.f;

    const int64_t rg = row0 + warp * 16 + g;  // this lane's rows: rg and rg + 8
    // drain: integer sums -> fp32 with the block scale; `kb` = index of the scale block just finished
    auto drain = [&](int kb) {
        const int nblk = p.n / p.blk;
        const float d0 = rg < p.rows16 ? __half2float(p.pl_d[rg * nblk + kb]) : 0.f;
        const float d1 = rg + 8 < p.rows16 ? __half2float(p.pl_d[(rg + 8) * nblk + kb]) : 0.f;
#pragma unroll
        for (int nf = 0; nf < 4; ++nf)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float f = 0.f;
#pragma unroll
                for (int l = 3; l >= 0; --l) {
                    int v = acc[0][nf][l][e];
                    if (NPL == 2) v += 256 * acc[NPL - 1][nf][l][e];
                    f = fmaf(f, 256.0f, float(v));
#pragma unroll
                    for (int a = 0; a < NPL; ++a) acc[a][nf][l][e] = 0;
                }
                yacc[nf][e] = fmaf(e < 2 ? d0 : d1, f, yacc[nf][e]);
            }
        if (p.pl_dm) {  // Q4_K min term of this 256-block: sum over its 8 sub-blocks of fl(dmin*m) * sum(X)
            const int nsub = p.n / 32;
#pragma unroll
            for (int nf = 0; nf < 4; ++nf)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t r = rg + (e < 2 ? 0 : 8);
                    const int tok = tok0 + nf * 8 + 2 * t + (e & 1);
                    if (r >= p.rows16 || tok >= p.B) continue;
                    const float* dm = p.pl_dm + r * nsub + kb * 8;
                    const float* xs = p.xsum + int64_t(tok) * nsub + kb * 8;
                    float s = 0.f;
#pragma unroll
                    for (int q = 0; q < 8; ++q) s = fmaf(__ldg(dm + q), __ldg(xs + q), s);
                    yacc[nf][e] -= s;
                }
        }
    };

    load_stage(0, 0);
    for (int kt = 0; kt < nk; ++kt) {
        if (kt + 1 < nk) {
            load_stage((kt + 1) & 1, kt + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int8_t* ws = reinterpret_cast<const int8_t*>(smem) + (kt & 1) * STAGE;
        const int8_t* as = ws + W_STAGE;
#pragma unroll
        for (int ks = 0; ks < GM_K / 32; ++ks) {
            uint32_t af[NPL][4];
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
                const int8_t* base = ws + (pl * GM_ROWS + warp * 16 + g) * GM_LD + ks * 32 + 4 * t;
                af[pl][0] = *reinterpret_cast<const uint32_t*>(base);
                af[pl][1] = *reinterpret_cast<const uint32_t*>(base + 8 * GM_LD);
                af[pl][2] = *reinterpret_cast<const uint32_t*>(base + 16);
                af[pl][3] = *reinterpret_cast<const uint32_t*>(base + 8 * GM_LD + 16);
            }
#pragma unroll
            for (int nf = 0; nf < 4; ++nf)
#pragma unroll
                for (int l = 0; l < 4; ++l) {
                    const int8_t* bb = as + (l * GM_TOK + nf * 8 + g) * GM_LD + ks * 32 + 4 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bb), b1 = *reinterpret_cast<const uint32_t*>(bb + 16);
#pragma unroll
                    for (int pl = 0; pl < NPL; ++pl)
                        mma_s8s8_k32_acc(acc[pl][nf][l], af[pl][0], af[pl][1], af[pl][2], af[pl][3], b0, b1);
                }
            const int kdone = kt * GM_K + (ks + 1) * 32;
            if (kdone % p.blk == 0) drain(kdone / p.blk - 1);
        }
        __syncthreads();
    }

#pragma unroll
    for (int nf = 0; nf < 4; ++nf)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = tok0 + nf * 8 + 2 * t + e;
            if (tok >= p.B) continue;
            const float is = p.inv_scale[tok];
            const float v0 = yacc[nf][e] * is, v1 = yacc[nf][2 + e] * is;  // rows rg, rg+8
            if (p.epilogue == EPI_SILU) {
                const int64_t o = rg / 16 * 8 + rg % 16;  // rg % 16 = g < 8: gate row; rg+8: the matching up row
                if (o < p.rows / 2) p.Y[int64_t(tok) * p.ldy + o] = __fmul_rn(__fdiv_rn(v0, 1.0f + expf(-v0)), v1);
            } else {
                float* y = p.Y + int64_t(tok) * p.ldy;
                const float* r = p.epilogue == EPI_ADD ? p.resid + int64_t(tok) * p.ldy : nullptr;
                if (rg < p.rows) y[rg] = r ? r[rg] + v0 : v0;
                if (rg + 8 < p.rows) y[rg + 8] = r ? r[rg + 8] + v1 : v1;
            }
        }
}

// Q8_0: one digit plane and a scale per 32 values, so every MMA (K = 32) is complete by itself: its four int32 results
// per limb are joined (limb pairs in int32, |P_l| < 2^19) and go straight into the fp32 sums with the block scale,
// acc += d * Horner_256(P_l) per 32 values as the reference does (src/cuda/model_cuda.cu:968-973). A warp owns RF
// fragments of 16 rows, so every limb fragment fetched from shared memory feeds RF MMAs.
template <int RF>
__global__ void __launch_bounds__(GM_THREADS) k_gemm_q8(const GemmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int ROWS = GM_ROWS * RF, W_STAGE = ROWS * GM_LD, A_STAGE = 4 * GM_TOK * GM_LD, STAGE = W_STAGE + A_STAGE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int64_t row0 = int64_t(blockIdx.x) * ROWS;
    const int tok0 = blockIdx.y * GM_TOK;
    const int nk = p.n / GM_K, nblk = p.n / 32;

    auto load_stage = [&](int st, int kt) {
        int8_t* ws = reinterpret_cast<int8_t*>(smem) + st * STAGE;
        int8_t* as = ws + W_STAGE;
        const int k0 = kt * GM_K;
        for (int idx = tid; idx < ROWS * (GM_K / 16); idx += GM_THREADS) {
            const int r = idx / (GM_K / 16), c = idx % (GM_K / 16);
            const bool ok = row0 + r < p.rows16;
            cp_async16(ws + r * GM_LD + c * 16, p.planes + (ok ? row0 + r : 0) * p.n + k0 + c * 16, ok);
        }
        for (int idx = tid; idx < 4 * GM_TOK * (GM_K / 16); idx += GM_THREADS) {
            const int l = idx / (GM_TOK * (GM_K / 16)), r = (idx / (GM_K / 16)) % GM_TOK, c = idx % (GM_K / 16);
            const bool ok = tok0 + r < p.B;
            cp_async16(as + (l * GM_TOK + r) * GM_LD + c * 16,
                       p.limbs + (int64_t(l) * p.B + (ok ? tok0 + r : 0)) * p.n + k0 + c * 16, ok);
        }
        cp_async_commit();
    };

    float yacc[RF][4][4];  // [row fragment][token fragment][C reg]
#pragma unroll
    for (int a = 0; a < RF; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int d = 0; d < 4; ++d) yacc[a][b][d] = 0.f;
    const int64_t rg0 = row0 + warp * 16 * RF + g;  // this lane's rows: rg0 + 16 rf and 8 more

    load_stage(0, 0);
    for (int kt = 0; kt < nk; ++kt) {
        if (kt + 1 < nk) {
            load_stage((kt + 1) & 1, kt + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        // the four block scales of this stage for the lane's rows: one 8-byte load per row
        float ds[RF][2][4];
#pragma unroll
        for (int rf = 0; rf < RF; ++rf)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t r = rg0 + 16 * rf + 8 * h;
                uint2 raw = make_uint2(0u, 0u);
                if (r < p.rows16) raw = __ldg(reinterpret_cast<const uint2*>(p.pl_d + r * nblk + kt * (GM_K / 32)));
                const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x), hi = *reinterpret_cast<const __half2*>(&raw.y);
                ds[rf][h][0] = __low2float(lo); ds[rf][h][1] = __high2float(lo);
                ds[rf][h][2] = __low2float(hi); ds[rf][h][3] = __high2float(hi);
            }
        __syncthreads();
        const int8_t* ws = reinterpret_cast<const int8_t*>(smem) + (kt & 1) * STAGE;
        const int8_t* as = ws + W_STAGE;
#pragma unroll
        for (int ks = 0; ks < GM_K / 32; ++ks) {
            uint32_t af[RF][4];
#pragma unroll
            for (int rf = 0; rf < RF; ++rf) {
                const int8_t* base = ws + (warp * 16 * RF + rf * 16 + g) * GM_LD + ks * 32 + 4 * t;
                af[rf][0] = *reinterpret_cast<const uint32_t*>(base);
                af[rf][1] = *reinterpret_cast<const uint32_t*>(base + 8 * GM_LD);
                af[rf][2] = *reinterpret_cast<const uint32_t*>(base + 16);
                af[rf][3] = *reinterpret_cast<const uint32_t*>(base + 8 * GM_LD + 16);
            }
#pragma unroll
            for (int nf = 0; nf < 4; ++nf) {
                int c[RF][4][4];
#pragma unroll
                for (int l = 0; l < 4; ++l) {
                    const int8_t* bb = as + (l * GM_TOK + nf * 8 + g) * GM_LD + ks * 32 + 4 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bb), b1 = *reinterpret_cast<const uint32_t*>(bb + 16);
#pragma unroll
                    for (int rf = 0; rf < RF; ++rf) mma_s8s8_k32(c[rf][l], af[rf][0], af[rf][1], af[rf][2], af[rf][3], b0, b1);
                }
#pragma unroll
                for (int rf = 0; rf < RF; ++rf)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i01 = c[rf][0][e] + (c[rf][1][e] << 8), i23 = c[rf][2][e] + (c[rf][3][e] << 8);
                        const float f = fmaf(float(i23), 65536.0f, float(i01));
                        yacc[rf][nf][e] = fmaf(ds[rf][e >> 1][ks], f, yacc[rf][nf][e]);
                    }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int rf = 0; rf < RF; ++rf)
#pragma unroll
        for (int nf = 0; nf < 4; ++nf)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tok0 + nf * 8 + 2 * t + e;
                if (tok >= p.B) continue;
                const int64_t rg = rg0 + 16 * rf;
                const float is = p.inv_scale[tok];
                const float v0 = yacc[rf][nf][e] * is, v1 = yacc[rf][nf][2 + e] * is;  // rows rg, rg+8
                if (p.epilogue == EPI_SILU) {
                    const int64_t o = rg / 16 * 8 + rg % 16;  // rg % 16 = g < 8: gate row; rg+8: the matching up row
                    if (o < p.rows / 2) p.Y[int64_t(tok) * p.ldy + o] = __fmul_rn(__fdiv_rn(v0, 1.0f + expf(-v0)), v1);
                } else {
                    float* y = p.Y + int64_t(tok) * p.ldy;
                    const float* r = p.epilogue == EPI_ADD ? p.resid + int64_t(tok) * p.ldy : nullptr;
                    if (rg < p.rows) y[rg] = r ? r[rg] + v0 : v0;
                    if (rg + 8 < p.rows) y[rg + 8] = r ? r[rg + 8] + v1 : v1;
                }
            }
}

int gemm_planes_launch(const Weight* w, const int8_t* d_limbs, const float* d_inv_scale, const float* d_xsum, int B,
                       float* d_y, int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s) {
    if (!w->planes) return fail(ELB_ERR_STATE, "matmul: weight was created without ELB_W_PLANES");
    if (w->n % GM_K) return fail(ELB_ERR_UNSUPPORTED, "matmul: row length must be a multiple of 128");
    if (epilogue == EPI_SILU && !w->pair) return fail(ELB_ERR_INVALID, "matmul: SwiGLU epilogue needs a paired weight");
    GemmParams p{w->planes, w->pl_d, w->pl_dm, d_limbs, d_inv_scale, d_xsum, d_y, d_resid, w->tiles * 16, w->rows, ldy,
                 B, int(w->n), w->n_planes, w->type == ELB_Q8_0 ? 32 : 256, epilogue};
    const int64_t rows16 = w->tiles * 16;
    const unsigned tok_tiles = unsigned((B + GM_TOK - 1) / GM_TOK);
    ELB_TRY(ensure_dyn_smem((const void*)k_gemm_q8<1>, size_t(2 * (1 * GM_ROWS + 4 * GM_TOK) * GM_LD)));
    ELB_TRY(ensure_dyn_smem((const void*)k_gemm_q8<2>, size_t(2 * (2 * GM_ROWS + 4 * GM_TOK) * GM_LD)));
    ELB_TRY(ensure_dyn_smem((const void*)k_gemm_planes<2>, size_t(2 * (2 * GM_ROWS + 4 * GM_TOK) * GM_LD)));
    if (w->n_planes == 1) {  // Q8_0: 128-row tiles when that still leaves a few CTAs for every SM
        DeviceInfo di;
        ELB_TRY(device_info(w->device, &di));
        const int64_t tiles128 = (rows16 + 2 * GM_ROWS - 1) / (2 * GM_ROWS);
        if (tiles128 * tok_tiles >= 3 * int64_t(di.sm_count)) {
            k_gemm_q8<2><<<dim3(unsigned(tiles128), tok_tiles), GM_THREADS, 2 * size_t(2 * GM_ROWS + 4 * GM_TOK) * GM_LD, s>>>(p);
        } else {
            k_gemm_q8<1><<<dim3(unsigned((rows16 + GM_ROWS - 1) / GM_ROWS), tok_tiles), GM_THREADS,
                           2 * size_t(GM_ROWS + 4 * GM_TOK) * GM_LD, s>>>(p);
        }
    } else {
        k_gemm_planes<2><<<dim3(unsigned((rows16 + GM_ROWS - 1) / GM_ROWS), tok_tiles), GM_THREADS,
                             2 * size_t(2 * GM_ROWS + 4 * GM_TOK) * GM_LD, s>>>(p);
    }
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

// ---------------------------------------------------------------- F16 weights, several tokens: fp32 FMA tiles
// (the F16 tensor-core path is separate; this keeps the model path complete and exact to fp32 rounding)
__global__ void __launch_bounds__(256) k_gemm_f16(const __half* __restrict__ W, const float* __restrict__ X, int64_t ldx,
                                                  const float* __restrict__ norm_w, float eps, float* __restrict__ Y,
                                                  int64_t ldy, const float* __restrict__ resid, int64_t rows16,
                                                  int64_t rows, int B, int n, int epilogue) {
    // tile: 32 tokens x 32 weight rows, K step 32; thread (ty, tx) owns tokens ty*2.. and rows tx*... 2x2
    __shared__ float Xs[32][33];
    __shared__ float Ws[32][33];
    __shared__ float inv_s[32];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int tok0 = blockIdx.y * 32;
    const int64_t row0 = int64_t(blockIdx.x) * 32;
    if (norm_w) {  // per-token RMSNorm scale, sum of squares in double
        const int warp = tid >> 5, lane = tid & 31;
        for (int r = warp; r < 32; r += 8) {
            double ss = 0.0;
            if (tok0 + r < B)
                for (int i = lane; i < n; i += 32) { const double v = X[int64_t(tok0 + r) * ldx + i]; ss += v * v; }
            ss = warp_sum(ss);
            if (lane == 0) inv_s[r] = float(1.0 / sqrt(ss / n + double(eps)));
        }
        __syncthreads();
    }
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < n; k0 += 32) {
        for (int idx = tid; idx < 32 * 32; idx += 256) {
            const int r = idx / 32, c = idx % 32;
            float xv = 0.f;
            if (tok0 + r < B) {
                xv = X[int64_t(tok0 + r) * ldx + k0 + c];
                if (norm_w) xv = __fmul_rn(__fmul_rn(xv, inv_s[r]), norm_w[k0 + c]);
            }
            Xs[r][c] = xv;
            Ws[r][c] = row0 + r < rows16 ? __half2float(W[(row0 + r) * n + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            const float x0 = Xs[ty * 2][c], x1 = Xs[ty * 2 + 1][c], w0 = Ws[tx][c], w1 = Ws[tx + 16][c];
            acc[0][0] = fmaf(x0, w0, acc[0][0]);
            acc[0][1] = fmaf(x0, w1, acc[0][1]);
            acc[1][0] = fmaf(x1, w0, acc[1][0]);
            acc[1][1] = fmaf(x1, w1, acc[1][1]);
        }
        __syncthreads();
    }
    // rows: row0 + tx and row0 + tx + 16. For SwiGLU pairs the 16-row tiles hold gate in rows 0..7 and up in 8..15:
    // tx and tx+16 are in different tiles, so pair gate/up through shared memory.
    if (epilogue == EPI_SILU) {
        for (int i = 0; i < 2; ++i) {
            Ws[ty * 2 + i][tx] = acc[i][0];
            Ws[ty * 2 + i][tx + 16] = acc[i][1];
        }
        __syncthreads();
        for (int idx = tid; idx < 32 * 16; idx += 256) {
            const int r = idx / 16, q = idx % 16, tile = q / 8, gg = q % 8;
            const int tok = tok0 + r;
            const int64_t o = (row0 / 16 + tile) * 8 + gg;
            if (tok < B && o < rows / 2) {
                const float gt = Ws[r][tile * 16 + gg], up = Ws[r][tile * 16 + gg + 8];
                Y[int64_t(tok) * ldy + o] = __fmul_rn(__fdiv_rn(gt, 1.0f + expf(-gt)), up);
            }
        }
        return;
    }
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 2; ++j) {
            const int tok = tok0 + ty * 2 + i;
            const int64_t r = row0 + tx + 16 * j;
            if (tok < B && r < rows) {
                const int64_t o = int64_t(tok) * ldy + r;
                Y[o] = epilogue == EPI_ADD ? resid[o] + acc[i][j] : acc[i][j];
            }
        }
}

int gemm_f16_launch(const Weight* w, const float* d_x, int64_t ldx, const float* d_norm_w, float eps, int B, float* d_y,
                    int64_t ldy, const float* d_resid, int epilogue, cudaStream_t s) {
    if (w->n % 32) return fail(ELB_ERR_UNSUPPORTED, "matmul: F16 row length must be a multiple of 32");
    const dim3 grid(unsigned((w->tiles * 16 + 31) / 32), unsigned((B + 31) / 32));
    k_gemm_f16<<<grid, 256, 0, s>>>(reinterpret_cast<const __half*>(w->tiled), d_x, ldx, d_norm_w, eps, d_y, ldy, d_resid,
                                    w->tiles * 16, w->rows, B, int(w->n), epilogue);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
