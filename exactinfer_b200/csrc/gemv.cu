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
#include <string>

#include <mutex>

#include "common.cuh"
#include "split.cuh"
#include "gemv_core.cuh"

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
    // raise the dynamic shared memory limit once per kernel and device (and again if a larger row length shows up)
    ELB_TRY(ensure_dyn_smem((const void*)kernel, smem));
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

// ---------------------------------------------------------------- matvec without any allocation
//
// Some hosts cannot call cudaMalloc where they need a matvec: a real-time or serving thread that must not take the
// driver's allocation lock, code that runs after the process has handed all of its device memory to a pool it does not
// control, or a caller that is inside a region where allocation is forbidden by its own rules. For them the working
// memory of the matvec (the limb-split activation, the split-K partial sums and their arrival counters) lives in one
// statically sized array in device memory instead of buffers allocated per weight.
//
// The array is part of the library image on every GPU that loads it (NOALLOC_BYTES, about 208 KB, until the process
// exits). Every call uses the same array and leaves its contents behind: two calls that overlap on the GPU (different
// streams, different threads) corrupt each other — issue them one after the other.
constexpr int NOALLOC_MAX_N = 16384;        // longest activation vector
constexpr int NOALLOC_MAX_TILES = 16384;    // row tiles of 16 rows: up to 262144 rows
constexpr int NOALLOC_MAX_GRID = 512;       // CTAs whose partial sums fit
constexpr size_t NOALLOC_ACT_OFF = 0;
constexpr size_t NOALLOC_INV_OFF = (size_t(4) * NOALLOC_MAX_N + size_t(NOALLOC_MAX_N / 256) * 192 + 255) / 256 * 256;
constexpr size_t NOALLOC_PART_OFF = NOALLOC_INV_OFF + 256;
constexpr size_t NOALLOC_CNT_OFF = NOALLOC_PART_OFF + size_t(NOALLOC_MAX_GRID) * 2 * 16 * sizeof(float);
constexpr size_t NOALLOC_BYTES = NOALLOC_CNT_OFF + size_t(NOALLOC_MAX_TILES) * sizeof(unsigned);

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

// Device address of the array on `device` (which must be current). In host code the array's name is only a handle for
// the runtime, not an address a kernel could use, so the address is asked for once per device and remembered.
static int noalloc_scratch(int device, unsigned char** out) {
    static unsigned char* cache[64] = {};
    static std::mutex mu;  // serving threads may make their first calls at the same time
    if (device < 0 || device >= 64) return fail(ELB_ERR_INVALID, "matvec_static: device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(ELB_ERR_CUDA, std::string("matvec_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        cache[device] = static_cast<unsigned char*>(p);
    }
    *out = cache[device];
    return ELB_OK;
}

int matvec_static(const Weight* w, const float* d_x, float* d_y, int nl, cudaStream_t s) {
    if (!w || !d_x || !d_y) return fail(ELB_ERR_INVALID, "matvec_static: null argument");
    if (nl == 0) nl = 4;
    ELB_CUDA(cudaSetDevice(w->device));
    GemvArgs a;
    a.x = d_x;
    a.y = d_y;
    if (w->type == ELB_F16) return gemv_launch(w, a, s);  // fp32 path: no working memory at all
    if (w->n > NOALLOC_MAX_N)
        return fail(ELB_ERR_UNSUPPORTED, "matvec_static: row length " + std::to_string(w->n) + " exceeds the static limit of " + std::to_string(NOALLOC_MAX_N));
    if (w->tiles > NOALLOC_MAX_TILES)
        return fail(ELB_ERR_UNSUPPORTED, "matvec_static: " + std::to_string(w->rows) + " rows exceed the static limit of " + std::to_string(NOALLOC_MAX_TILES * 16));
    DeviceInfo di;
    ELB_TRY(device_info(w->device, &di));
    if (di.sm_count > NOALLOC_MAX_GRID) return fail(ELB_ERR_UNSUPPORTED, "matvec_static: more SMs than the static partial-sum area covers");
    unsigned char* base = nullptr;
    ELB_TRY(noalloc_scratch(w->device, &base));
    int8_t* act = reinterpret_cast<int8_t*>(base + NOALLOC_ACT_OFF);
    float* inv = reinterpret_cast<float*>(base + NOALLOC_INV_OFF);
    // the arrival counters must start at zero whatever an earlier (possibly failed) call left behind
    ELB_CUDA(cudaMemsetAsync(base + NOALLOC_CNT_OFF, 0, size_t(w->tiles) * sizeof(unsigned), s));
    ELB_TRY(prep_limbs_launch(d_x, int(w->n), nullptr, 0.f, nl, act, inv, false, s));
    Weight view = *w;  // same weight, working memory redirected to the static array (nothing is allocated or freed)
    view.part = reinterpret_cast<float*>(base + NOALLOC_PART_OFF);
    view.counters = reinterpret_cast<unsigned*>(base + NOALLOC_CNT_OFF);
    view.max_grid = std::min(w->max_grid > 0 ? w->max_grid : NOALLOC_MAX_GRID, NOALLOC_MAX_GRID);
    a.limbs = act;
    a.inv_scale = inv;
    return gemv_launch(&view, a, s);
}

}  // namespace elb

// C entry point of the allocation-free matvec (declared in include/elb.h). It lives in this file because the static
// array does: its device address is looked up here (cudaGetSymbolAddress, on the first call per device).
extern "C" int elb_matvec_static(const elb_weight* w, const float* d_x, float* d_y, int nl) {
    const elb::Weight* ww = reinterpret_cast<const elb::Weight*>(w);
    const int rc = elb::matvec_static(ww, d_x, d_y, nl, nullptr);
    if (rc != ELB_OK) return rc;
    if (cudaStreamSynchronize(nullptr) != cudaSuccess) return elb::fail(ELB_ERR_CUDA, "matvec_static: kernel failed");
    return ELB_OK;
}

