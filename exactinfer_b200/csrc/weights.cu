// Weight upload: file bytes -> tiled device layout (a pure permutation), optional int8 digit planes for the
// tensor-core path, and the row decoders (embedding gather / parity checks) that read the tiled layout back.
#include <vector>
#include <cstdlib>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "layout.cuh"

namespace elb {

// ---------------------------------------------------------------- permutation: file layout -> tiled layout

#define ELB_GRID_STRIDE(o, total) \
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < (total); o += (int64_t)gridDim.x * blockDim.x)

__global__ void k_tile_q4k(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t nb,
                           int64_t total, bool pair) {
    ELB_GRID_STRIDE(o, total) dst[o] = tile_byte_q4k(src, o, rows, nb, pair);
}
__global__ void k_tile_q8(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t nb32,
                          int64_t total, bool pair) {
    ELB_GRID_STRIDE(o, total) dst[o] = tile_byte_q8(src, o, rows, nb32, pair);
}
__global__ void k_tile_q6k(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t nb,
                           int64_t total, bool pair) {
    ELB_GRID_STRIDE(o, total) dst[o] = tile_byte_q6k(src, o, rows, nb, pair);
}
// F16: plain row-major copy with the pair interleave / zero padding applied
__global__ void k_tile_f16(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int64_t rows, int64_t n,
                           int64_t total, bool pair) {
    ELB_GRID_STRIDE(o, total) {
        const int64_t r = src_row(o / n, rows, pair);
        dst[o] = r < 0 ? uint16_t(0) : src[r * n + o % n];
    }
}

// out[count][n] = rows [row0, row0+count) decoded; row indices are tiled rows (= logical rows unless paired)
__global__ void k_get_rows(int type, const uint8_t* __restrict__ tiled, int64_t n, int64_t row0, int64_t count,
                           float* __restrict__ out) {
    const int64_t total = count * n;
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = row0 + o / n, k = o % n;
        if (type == ELB_F16) out[o] = __half2float(reinterpret_cast<const __half*>(tiled)[R * n + k]);
        else out[o] = elem_value(type, tiled_elem(type, tiled, n, R, k));
    }
}

// Embedding gather for a chunk of tokens: out[b][n] = row tokens[b] (get_row, src/ops.cpp:76-82 of the reference)
__global__ void k_gather_rows(int type, const uint8_t* __restrict__ tiled, int64_t n, const int32_t* __restrict__ tokens,
                              float* __restrict__ out) {
    const int64_t R = tokens[blockIdx.x];
    float* o = out + (int64_t)blockIdx.x * n;
    for (int64_t k = threadIdx.x; k < n; k += blockDim.x) {
        if (type == ELB_F16) o[k] = __half2float(reinterpret_cast<const __half*>(tiled)[R * n + k]);
        else o[k] = elem_value(type, tiled_elem(type, tiled, n, R, k));
    }
}

// ---------------------------------------------------------------- int8 digit planes for the tensor-core path
// Integer weight w = sc*q (Q4_K: 0..945, Q6_K: -4064..4096, Q8_0: q). Balanced base-256 digits w = w0 + 256*w1 with
// w0 in [-128,127]; Q8_0 needs one plane. Exact: the planes hold the same integers as the file.
__global__ void k_planes(int type, const uint8_t* __restrict__ tiled, int64_t rows16, int64_t n, int8_t* __restrict__ p0,
                         int8_t* __restrict__ p1, __half* __restrict__ pl_d, float* __restrict__ pl_dm) {
    const int64_t total = rows16 * n;
    const int blk = type == ELB_Q8_0 ? QK8_0 : QK_K;
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = o / n, k = o % n;
        const QElem e = tiled_elem(type, tiled, n, R, k);
        const int w = e.sc * e.q;
        const int w0 = ((w + 128) & 255) - 128;
        p0[o] = int8_t(w0);
        if (p1) p1[o] = int8_t((w - w0) >> 8);
        if (k % blk == 0) pl_d[R * (n / blk) + k / blk] = __float2half_rn(e.d);  // exact: d came from fp16
        if (pl_dm && k % 32 == 0) pl_dm[R * (n / 32) + k / 32] = __fmul_rn(e.dmin, float(e.mn));
    }
}

// Q8_0 for the fp16 tensor cores: v = d * q is exact in fp32 (11 x 7 significant bits) and a multiple of 2^-24, hi =
// fp16(v), lo = v - hi has at most 8 significant bits and is again a multiple of 2^-24: hi + lo = v exactly. *bad is
// raised when that fails (hi overflows: |d * q| > 65504).
__global__ void k_q8_pair(const uint8_t* __restrict__ tiled, int64_t rows16, int64_t n, __half* __restrict__ hi,
                          __half* __restrict__ lo, int* __restrict__ bad) {
    const int64_t total = rows16 * n;
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
        const QElem e = tiled_elem(ELB_Q8_0, tiled, n, o / n, o % n);
        const float v = __fmul_rn(e.d, float(e.sc * e.q));
        const __half h = __float2half_rn(v);
        const float r = v - __half2float(h);
        const __half l = __float2half_rn(r);
        if (isinf(__half2float(h)) || __half2float(l) != r) *bad = 1;
        hi[o] = h;
        lo[o] = l;
    }
}

int launch_gather_rows(const Weight* w, const int32_t* d_tokens, int count, float* d_out, cudaStream_t s) {
    k_gather_rows<<<count, 256, 0, s>>>(w->type, w->tiled, w->n, d_tokens, d_out);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

int device_info(int device, DeviceInfo* out) {
    static DeviceInfo cache[64];
    if (device < 0 || device >= 64) return fail(ELB_ERR_INVALID, "device index out of range");
    if (cache[device].sm_count == 0) {
        int sms = 0, smem = 0;
        ELB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        ELB_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        cache[device].smem_optin = size_t(smem);
        cache[device].sm_count = sms;
    }
    *out = cache[device];
    return ELB_OK;
}

int ensure_dyn_smem(const void* kernel, size_t smem) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> done;
    int device = 0;
    ELB_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = done[{kernel, device}];
    if (have >= smem && have > 0) return ELB_OK;
    ELB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
    return ELB_OK;
}

static int row_bytes_of(int type, int64_t n, int64_t* out) {
    switch (type) {
        case ELB_F16: *out = n * 2; return n % 8 == 0 ? ELB_OK : fail(ELB_ERR_UNSUPPORTED, "F16 row length must be a multiple of 8");
        case ELB_Q8_0:
            *out = n / QK8_0 * Q8_0_BYTES;
            return n % (QK8_0 * Q8_GROUP) == 0 ? ELB_OK : fail(ELB_ERR_UNSUPPORTED, "Q8_0 row length must be a multiple of 128");
        case ELB_Q4_K: *out = n / QK_K * Q4_K_BYTES; return n % QK_K == 0 ? ELB_OK : fail(ELB_ERR_UNSUPPORTED, "Q4_K row length must be a multiple of 256");
        case ELB_Q6_K: *out = n / QK_K * Q6_K_BYTES; return n % QK_K == 0 ? ELB_OK : fail(ELB_ERR_UNSUPPORTED, "Q6_K row length must be a multiple of 256");
        default: return fail(ELB_ERR_UNSUPPORTED, "weight type not supported on this path (F16, Q8_0, Q4_K, Q6_K only)");
    }
}

int weight_create(int device, int type, int64_t rows_one, int64_t n, const void* bytes, size_t nbytes, int flags,
                  Weight** out) {
    if (!out || !bytes || rows_one <= 0 || n <= 0) return fail(ELB_ERR_INVALID, "weight_create: bad argument");
    const bool pair = flags & ELB_W_PAIR;
    if (pair && rows_one % 8) return fail(ELB_ERR_UNSUPPORTED, "paired weights need a row count that is a multiple of 8");
    int64_t rb = 0;
    ELB_TRY(row_bytes_of(type, n, &rb));
    const int64_t rows = pair ? 2 * rows_one : rows_one;
    if (size_t(rb * rows) != nbytes) return fail(ELB_ERR_INVALID, "weight_create: byte count does not match rows x row bytes");
    ELB_CUDA(cudaSetDevice(device));

    auto* w = new Weight;
    w->device = device; w->type = type; w->rows = rows; w->n = n; w->pair = pair;
    w->tiles = (rows + 15) / 16;
    switch (type) {
        case ELB_Q4_K: w->units_per_tile = n / QK_K; w->unit_bytes = Q4K_UNIT; break;
        case ELB_Q6_K: w->units_per_tile = n / QK_K; w->unit_bytes = Q6K_UNIT; break;
        case ELB_Q8_0: w->units_per_tile = n / (QK8_0 * Q8_GROUP); w->unit_bytes = Q8_UNIT; break;
        default: w->units_per_tile = 0; w->unit_bytes = 0; break;
    }
    w->tiled_bytes = type == ELB_F16 ? size_t(w->tiles) * 16 * n * 2 : size_t(w->tiles) * w->units_per_tile * w->unit_bytes;

    uint8_t* raw = nullptr;
    auto cleanup = [&](int rc) { if (raw) cudaFree(raw); weight_destroy(w); return rc; };
    if (cudaMalloc(&raw, nbytes) != cudaSuccess || cudaMalloc(&w->tiled, w->tiled_bytes) != cudaSuccess) {
        cudaGetLastError();
        return cleanup(fail(ELB_ERR_MEMORY, "weight_create: out of device memory"));
    }
    if (cudaMemcpy(raw, bytes, nbytes, cudaMemcpyHostToDevice) != cudaSuccess)
        return cleanup(fail(ELB_ERR_CUDA, "weight_create: upload failed"));
    const int64_t total = int64_t(w->tiled_bytes);
    const int grid = int(std::min<int64_t>((total + 255) / 256, 148 * 32));
    switch (type) {
        case ELB_Q4_K: k_tile_q4k<<<grid, 256>>>(raw, w->tiled, rows, n / QK_K, total, pair); break;
        case ELB_Q6_K: k_tile_q6k<<<grid, 256>>>(raw, w->tiled, rows, n / QK_K, total, pair); break;
        case ELB_Q8_0: k_tile_q8<<<grid, 256>>>(raw, w->tiled, rows, n / QK8_0, total, pair); break;
        default:
            k_tile_f16<<<grid, 256>>>(reinterpret_cast<const uint16_t*>(raw), reinterpret_cast<uint16_t*>(w->tiled), rows,
                                      n, total / 2, pair);
    }
    if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)
        return cleanup(fail(ELB_ERR_CUDA, "weight_create: re-layout kernel failed"));
    cudaFree(raw);
    raw = nullptr;

    if ((flags & ELB_W_PLANES) && type == ELB_Q8_0 && n % 64 == 0) {
        static const bool off = [] { const char* v = std::getenv("ELB_Q8_PLANES"); return v && v[0] == '1'; }();
        const int64_t rows16 = w->tiles * 16;
        int* bad = nullptr;
        if (!off && cudaMalloc(&bad, sizeof(int)) == cudaSuccess && cudaMemset(bad, 0, sizeof(int)) == cudaSuccess &&
            cudaMalloc(&w->f16pair, size_t(2) * rows16 * n * sizeof(__half)) == cudaSuccess) {
            const int64_t tot = rows16 * n;
            k_q8_pair<<<int(std::min<int64_t>((tot + 255) / 256, 148 * 32)), 256>>>(w->tiled, rows16, n, w->f16pair,
                                                                                   w->f16pair + rows16 * n, bad);
            int h_bad = 1;
            if (cudaGetLastError() != cudaSuccess || cudaMemcpy(&h_bad, bad, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
                cudaFree(bad);
                return cleanup(fail(ELB_ERR_CUDA, "weight_create: fp16 pair kernel failed"));
            }
            if (h_bad) {  // out of the fp16 range: this weight stays on the digit plane
                cudaFree(w->f16pair);
                w->f16pair = nullptr;
            }
        }
        cudaGetLastError();
        cudaFree(bad);
    }
    if ((flags & ELB_W_PLANES) && type != ELB_F16 && !w->f16pair) {
        const int64_t rows16 = w->tiles * 16;
        w->n_planes = type == ELB_Q8_0 ? 1 : 2;
        const int blk = type == ELB_Q8_0 ? QK8_0 : QK_K;
        bool ok = cudaMalloc(&w->planes, size_t(w->n_planes) * rows16 * n) == cudaSuccess &&
                  cudaMalloc(&w->pl_d, size_t(rows16) * (n / blk) * sizeof(__half)) == cudaSuccess;
        if (ok && type == ELB_Q4_K) ok = cudaMalloc(&w->pl_dm, size_t(rows16) * (n / 32) * sizeof(float)) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            return cleanup(fail(ELB_ERR_MEMORY, "weight_create: out of device memory for the digit planes"));
        }
        const int64_t tot = rows16 * n;
        k_planes<<<int(std::min<int64_t>((tot + 255) / 256, 148 * 32)), 256>>>(
            type, w->tiled, rows16, n, w->planes, w->n_planes == 2 ? w->planes + rows16 * n : nullptr, w->pl_d, w->pl_dm);
        if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)
            return cleanup(fail(ELB_ERR_CUDA, "weight_create: plane decode kernel failed"));
    }
    *out = w;
    return ELB_OK;
}

int weight_view_rows(const Weight* base, int64_t row0, int64_t rows, Weight** out) {
    if (!base || !out || rows <= 0 || row0 < 0 || row0 + rows > base->rows) return fail(ELB_ERR_INVALID, "weight_view_rows: bad range");
    if (row0 % 16 || base->pair) return fail(ELB_ERR_UNSUPPORTED, "weight_view_rows: the first row must be a multiple of 16 of an unpaired weight");
    auto* w = new Weight;
    w->device = base->device; w->type = base->type; w->rows = rows; w->n = base->n; w->view = true;
    w->tiles = (rows + 15) / 16;
    w->units_per_tile = base->units_per_tile; w->unit_bytes = base->unit_bytes;
    const size_t tile_bytes = base->type == ELB_F16 ? size_t(16) * base->n * 2 : size_t(base->units_per_tile) * base->unit_bytes;
    w->tiled = base->tiled + size_t(row0 / 16) * tile_bytes;
    w->tiled_bytes = size_t(w->tiles) * tile_bytes;
    *out = w;
    return ELB_OK;
}

void weight_destroy(Weight* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    if (w->view) w->tiled = nullptr;
    cudaFree(w->tiled); cudaFree(w->planes); cudaFree(w->f16pair); cudaFree(w->pl_d); cudaFree(w->pl_dm); cudaFree(w->part); cudaFree(w->counters); cudaFree(w->xlimbs); cudaFree(w->xinv);
    delete w;
}

int get_rows_dev(const Weight* w, int64_t row0, int64_t count, float* d_out, cudaStream_t s) {
    if (!w || !d_out || count <= 0) return fail(ELB_ERR_INVALID, "get_rows: bad argument");
    if (row0 < 0 || row0 + count > w->rows) return fail(ELB_ERR_RANGE, "get_rows: row out of range");
    const int64_t total = count * w->n;
    k_get_rows<<<int(std::min<int64_t>((total + 255) / 256, 148 * 16)), 256, 0, s>>>(w->type, w->tiled, w->n, row0, count, d_out);
    ELB_CUDA(cudaGetLastError());
    return ELB_OK;
}

}  // namespace elb
