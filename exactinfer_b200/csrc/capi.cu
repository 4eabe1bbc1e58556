// extern "C" surface of libelb.so (declared in include/elb.h): status codes in, no exceptions out.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace elb {
static thread_local std::string g_error;
void set_error(const std::string& msg) { g_error = msg; }
int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

namespace {
// RAII device scratch for the host-pointer convenience entry points
struct Dev {
    void* p = nullptr;
    ~Dev() { if (p) cudaFree(p); }
    int alloc(size_t n) {
        if (cudaMalloc(&p, std::max<size_t>(n, 16)) != cudaSuccess) {
            cudaGetLastError();
            return fail(ELB_ERR_MEMORY, "out of device memory");
        }
        return ELB_OK;
    }
    template <class T> T* as() const { return static_cast<T*>(p); }
};
}  // namespace
}  // namespace elb

using namespace elb;

// the opaque handles of the header are the internal structs

static Weight* W(elb_weight* w) { return reinterpret_cast<Weight*>(w); }
static const Weight* W(const elb_weight* w) { return reinterpret_cast<const Weight*>(w); }
static Model* M(elb_model* m) { return reinterpret_cast<Model*>(m); }
static const Model* M(const elb_model* m) { return reinterpret_cast<const Model*>(m); }

extern "C" {

const char* elb_last_error(void) { return g_error.c_str(); }

int elb_device_count(void) {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error(e != cudaSuccess ? cudaGetErrorString(e) : "no CUDA device");
        return 0;
    }
    int ok = 0;
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10) ++ok;
    }
    if (!ok) set_error("no device of compute capability 10.x (the kernels are built for sm_100a only)");
    return ok;
}

int elb_malloc(int device, size_t bytes, void** out) {
    if (!out) return fail(ELB_ERR_INVALID, "elb_malloc: null out");
    ELB_CUDA(cudaSetDevice(device));
    if (cudaMalloc(out, std::max<size_t>(bytes, 16)) != cudaSuccess) {
        cudaGetLastError();
        return fail(ELB_ERR_MEMORY, "elb_malloc: out of device memory");
    }
    return ELB_OK;
}
int elb_free(void* p) { ELB_CUDA(cudaFree(p)); return ELB_OK; }
int elb_host_alloc(size_t bytes, void** out) { ELB_CUDA(cudaMallocHost(out, std::max<size_t>(bytes, 16))); return ELB_OK; }
int elb_host_free(void* p) { ELB_CUDA(cudaFreeHost(p)); return ELB_OK; }
int elb_memcpy_h2d(void* dst, const void* src, size_t bytes) { ELB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); return ELB_OK; }
int elb_memcpy_d2h(void* dst, const void* src, size_t bytes) { ELB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost)); return ELB_OK; }
int elb_device_mem_info(int device, size_t* free_bytes, size_t* total_bytes) {
    if (!free_bytes || !total_bytes) return fail(ELB_ERR_INVALID, "elb_device_mem_info: null argument");
    ELB_CUDA(cudaSetDevice(device));
    ELB_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
    return ELB_OK;
}
int elb_selftest_wait_expiry(int device) {
    ELB_CUDA(cudaSetDevice(device));
    ELB_TRY(gemm_f16_tc_wait_expiry(nullptr));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    return gemm_f16_tc_check();  // ELB_ERR_CUDA when the wait ran out and was reported, as it must
}
int elb_device_sync(int device) {
    ELB_CUDA(cudaSetDevice(device));
    ELB_CUDA(cudaDeviceSynchronize());
    return ELB_OK;
}

// ---------------------------------------------------------------- weights

int elb_weight_create(int device, int ggml_type, int64_t rows, int64_t n, const void* bytes, size_t nbytes, int flags,
                      elb_weight** out) {
    if (elb_device_count() == 0) return fail(ELB_ERR_CUDA, std::string("no usable CUDA device: ") + g_error);
    Weight* w = nullptr;
    ELB_TRY(weight_create(device, ggml_type, rows, n, bytes, nbytes, flags, &w));
    const int rc = gemv_prepare(w);
    if (rc != ELB_OK) { weight_destroy(w); return rc; }
    *out = reinterpret_cast<elb_weight*>(w);
    return ELB_OK;
}
void elb_weight_destroy(elb_weight* w) { weight_destroy(W(w)); }
int64_t elb_weight_rows(const elb_weight* w) { return W(w)->rows; }
int64_t elb_weight_cols(const elb_weight* w) { return W(w)->n; }
size_t elb_weight_device_bytes(const elb_weight* w) { return W(w)->tiled_bytes; }

int elb_get_rows_dev(const elb_weight* w, int64_t row0, int64_t count, float* d_out) {
    if (!w) return fail(ELB_ERR_INVALID, "get_rows: null weight");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    ELB_TRY(get_rows_dev(W(w), row0, count, d_out, nullptr));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    return ELB_OK;
}
int elb_get_rows(const elb_weight* w, int64_t row0, int64_t count, float* out) {
    if (!w || !out) return fail(ELB_ERR_INVALID, "get_rows: null argument");
    if (count <= 0) return fail(ELB_ERR_INVALID, "get_rows: count must be positive");
    if (row0 < 0 || row0 + count > W(w)->rows) return fail(ELB_ERR_RANGE, "get_rows: row out of range");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    Dev d;
    ELB_TRY(d.alloc(size_t(count) * W(w)->n * 4));
    ELB_TRY(elb_get_rows_dev(w, row0, count, d.as<float>()));
    ELB_CUDA(cudaMemcpy(out, d.p, size_t(count) * W(w)->n * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

// split (quantized weights) + matvec on stream s; dbg may carry the parity dump pointers
static int matvec_on(const Weight* w, const float* d_x, float* d_y, int nl, cudaStream_t s, const GemvArgs* dbg) {
    GemvArgs a;
    if (dbg) a = *dbg;
    a.x = d_x; a.y = d_y;
    if (w->type != ELB_F16) {
        ELB_TRY(prep_limbs_launch(d_x, int(w->n), nullptr, 0.f, nl == 0 ? 4 : nl, w->xlimbs, w->xinv, false, s));
        a.limbs = w->xlimbs; a.inv_scale = w->xinv;
    }
    return gemv_launch(w, a, s);
}

int elb_matvec_dev(const elb_weight* w, const float* d_x, float* d_y, int nl) {
    if (!w) return fail(ELB_ERR_INVALID, "matvec: null weight");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    ELB_TRY(matvec_on(W(w), d_x, d_y, nl, nullptr, nullptr));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    return ELB_OK;
}
int elb_matvec(const elb_weight* w, const float* x, float* y, int nl) {
    if (!w || !x || !y) return fail(ELB_ERR_INVALID, "matvec: null argument");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    Dev dx, dy;
    ELB_TRY(dx.alloc(size_t(W(w)->n) * 4));
    ELB_TRY(dy.alloc(size_t(W(w)->rows) * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(W(w)->n) * 4, cudaMemcpyHostToDevice));
    ELB_TRY(elb_matvec_dev(w, dx.as<float>(), dy.as<float>(), nl));
    ELB_CUDA(cudaMemcpy(y, dy.p, size_t(W(w)->rows) * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

static int matmul_dev_on(const Weight* w, const float* d_x, int64_t b, float* d_y, int nl, cudaStream_t s, Dev* scratch) {
    if (b <= 0) return fail(ELB_ERR_INVALID, "matmul: token count must be positive");
    if (w->pair) return fail(ELB_ERR_UNSUPPORTED, "matmul: paired weights are only used inside the model");
    const size_t limb_bytes = size_t(4) * b * w->n, inv_off = (limb_bytes + 255) / 256 * 256;
    if (w->type == ELB_F16 || gemm_f16_tc_usable(w, int(b))) {
        if (!gemm_f16_tc_usable(w, int(b))) return gemm_f16_launch(w, d_x, w->n, nullptr, 0.f, int(b), d_y, w->rows, nullptr, EPI_STORE, s);
        // hi and lo halves, 2^-k per row, then the partial tiles and arrival counters of the k splits
        const size_t part_off = (inv_off + size_t(b) * 4 + 255) / 256 * 256, cnt_off = part_off + gemm_f16_tc_part_bytes();
        if (!scratch->p) {
            ELB_TRY(scratch->alloc(cnt_off + size_t(gemm_f16_tc_counters()) * 4));
            ELB_CUDA(cudaMemsetAsync(scratch->as<int8_t>() + cnt_off, 0, size_t(gemm_f16_tc_counters()) * 4, s));
        }
        int8_t* base = scratch->as<int8_t>();
        return gemm_f16_tc_launch(w, d_x, w->n, nullptr, 0.f, int(b), base, reinterpret_cast<float*>(base + inv_off), d_y, w->rows,
                                  nullptr, EPI_STORE, s, false, reinterpret_cast<float*>(base + part_off),
                                  reinterpret_cast<unsigned*>(base + cnt_off));
    }
    const size_t xs_off = inv_off + (size_t(b) * 4 + 255) / 256 * 256, total = xs_off + size_t(b) * (w->n / 32) * 4;
    if (!scratch->p) ELB_TRY(scratch->alloc(total));
    int8_t* limbs = scratch->as<int8_t>();
    float* inv = reinterpret_cast<float*>(limbs + inv_off);
    float* xs = reinterpret_cast<float*>(limbs + xs_off);
    ELB_TRY(split_launch(d_x, w->n, b, int(w->n), nl == 0 ? 4 : nl, nullptr, 0.f, limbs, inv, xs, s));
    if (gemm_tc_usable(w, int(b))) return gemm_tc_launch(w, limbs, inv, xs, int(b), nl == 0 ? 4 : nl, d_y, w->rows, nullptr, EPI_STORE, s);
    return gemm_planes_launch(w, limbs, inv, xs, int(b), d_y, w->rows, nullptr, EPI_STORE, s);
}

int elb_matmul_acc(const elb_weight* w, const float* x, int64_t b, int nl, int32_t* A) {
    if (!w || !x || !A) return fail(ELB_ERR_INVALID, "matmul_acc: null argument");
    const Weight* ww = W(w);
    if (b <= 0 || b > 4096) return fail(ELB_ERR_INVALID, "matmul_acc: token count out of range");
    if (nl == 0) nl = 4;
    if (nl != 3 && nl != 4) return fail(ELB_ERR_INVALID, "matmul_acc: 3 or 4 limbs");
    ELB_CUDA(cudaSetDevice(ww->device));
    if (!gemm_tc_usable(ww, int(b))) return fail(ELB_ERR_UNSUPPORTED, "matmul_acc: the weight does not run on the int8 tensor-core kernel");
    const int64_t rows16 = ww->tiles * 16, nblk = ww->n / 256;
    const size_t limb_bytes = size_t(4) * b * ww->n, inv_off = (limb_bytes + 255) / 256 * 256;
    const size_t xs_off = inv_off + (size_t(b) * 4 + 255) / 256 * 256, total = xs_off + size_t(b) * (ww->n / 32) * 4;
    const size_t nA = size_t(b) * nblk * (nl + 1) * rows16;
    Dev dx, dy, scratch, dA;
    ELB_TRY(dx.alloc(size_t(b) * ww->n * 4));
    ELB_TRY(dy.alloc(size_t(b) * ww->rows * 4));
    ELB_TRY(scratch.alloc(total));
    ELB_TRY(dA.alloc(nA * 4));
    ELB_CUDA(cudaMemset(dA.p, 0, nA * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(b) * ww->n * 4, cudaMemcpyHostToDevice));
    int8_t* limbs = scratch.as<int8_t>();
    float* inv = reinterpret_cast<float*>(limbs + inv_off);
    float* xs = reinterpret_cast<float*>(limbs + xs_off);
    ELB_TRY(split_launch(dx.as<float>(), ww->n, b, int(ww->n), nl, nullptr, 0.f, limbs, inv, xs, nullptr));
    ELB_TRY(gemm_tc_launch(ww, limbs, inv, xs, int(b), nl, dy.as<float>(), ww->rows, nullptr, EPI_STORE, nullptr, false, dA.as<int32_t>()));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    ELB_TRY(gemm_tc_check());
    std::vector<int32_t> tmp(nA);
    ELB_CUDA(cudaMemcpy(tmp.data(), dA.p, nA * 4, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < size_t(b) * nblk * (nl + 1); ++i)  // rows16 -> rows
        std::memcpy(A + i * ww->rows, tmp.data() + i * rows16, size_t(ww->rows) * 4);
    return ELB_OK;
}

int elb_matmul_dev(const elb_weight* w, const float* d_x, int64_t b, float* d_y, int nl) {
    if (!w) return fail(ELB_ERR_INVALID, "matmul: null weight");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    Dev scratch;
    ELB_TRY(matmul_dev_on(W(w), d_x, b, d_y, nl, nullptr, &scratch));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    ELB_TRY(gemm_f16_tc_check());
    return gemm_tc_check();
}
int elb_matmul(const elb_weight* w, const float* x, int64_t b, float* y, int nl) {
    if (!w || !x || !y) return fail(ELB_ERR_INVALID, "matmul: null argument");
    if (b <= 0) return fail(ELB_ERR_INVALID, "matmul: token count must be positive");
    ELB_CUDA(cudaSetDevice(W(w)->device));
    Dev dx, dy;
    ELB_TRY(dx.alloc(size_t(b) * W(w)->n * 4));
    ELB_TRY(dy.alloc(size_t(b) * W(w)->rows * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(b) * W(w)->n * 4, cudaMemcpyHostToDevice));
    ELB_TRY(elb_matmul_dev(w, dx.as<float>(), b, dy.as<float>(), nl));
    ELB_CUDA(cudaMemcpy(y, dy.p, size_t(b) * W(w)->rows * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

int elb_rmsnorm(float* out, const float* x, const float* w, int n, float eps, int rows) {
    if (!out || !x || !w || n <= 0 || rows <= 0) return fail(ELB_ERR_INVALID, "rmsnorm: bad argument");
    if (elb_device_count() == 0) return fail(ELB_ERR_CUDA, std::string("no usable CUDA device: ") + g_error);
    Dev dx, dw, dy;
    ELB_TRY(dx.alloc(size_t(rows) * n * 4));
    ELB_TRY(dw.alloc(size_t(n) * 4));
    ELB_TRY(dy.alloc(size_t(rows) * n * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(rows) * n * 4, cudaMemcpyHostToDevice));
    ELB_CUDA(cudaMemcpy(dw.p, w, size_t(n) * 4, cudaMemcpyHostToDevice));
    ELB_TRY(rmsnorm_launch(dy.as<float>(), dx.as<float>(), dw.as<float>(), n, eps, rows, nullptr));
    ELB_CUDA(cudaMemcpy(out, dy.p, size_t(rows) * n * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

int elb_split_limbs(int device, const float* x, int64_t b, int64_t n, int nl, int8_t* limbs, float* inv_scale) {
    if (!x || !limbs || !inv_scale || b <= 0 || n <= 0 || n % 32) return fail(ELB_ERR_INVALID, "split_limbs: bad argument");
    if (elb_device_count() == 0) return fail(ELB_ERR_CUDA, std::string("no usable CUDA device: ") + g_error);
    ELB_CUDA(cudaSetDevice(device));
    Dev dx, dl, di;
    ELB_TRY(dx.alloc(size_t(b) * n * 4));
    ELB_TRY(dl.alloc(size_t(4) * b * n));
    ELB_TRY(di.alloc(size_t(b) * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(b) * n * 4, cudaMemcpyHostToDevice));
    ELB_TRY(split_launch(dx.as<float>(), n, b, int(n), nl, nullptr, 0.f, dl.as<int8_t>(), di.as<float>(), nullptr, nullptr));
    ELB_CUDA(cudaMemcpy(limbs, dl.p, size_t(nl) * b * n, cudaMemcpyDeviceToHost));
    ELB_CUDA(cudaMemcpy(inv_scale, di.p, size_t(b) * 4, cudaMemcpyDeviceToHost));
    return ELB_OK;
}

int elb_limb_sums(const elb_weight* w, const float* x, int nl, int32_t* P, int32_t* I, int32_t* J) {
    if (!w || !x) return fail(ELB_ERR_INVALID, "limb_sums: null argument");
    const Weight* ww = W(w);
    if (ww->type == ELB_F16) return fail(ELB_ERR_UNSUPPORTED, "limb_sums: F16 weights are not multiplied through limbs");
    if (nl == 0) nl = 4;
    ELB_CUDA(cudaSetDevice(ww->device));
    const int sub = ww->type == ELB_Q6_K ? 16 : 32, blk = ww->type == ELB_Q8_0 ? 32 : 256;
    const size_t nP = size_t(ww->rows) * (ww->n / sub) * 4, nI = size_t(ww->rows) * (ww->n / blk) * 4;
    Dev dx, dy, dP, dI, dJ;
    ELB_TRY(dx.alloc(size_t(ww->n) * 4));
    ELB_TRY(dy.alloc(size_t(ww->rows) * 4));
    ELB_TRY(dP.alloc(nP * 4));
    ELB_TRY(dI.alloc(nI * 4));
    ELB_TRY(dJ.alloc(nI * 4));
    ELB_CUDA(cudaMemset(dJ.p, 0, nI * 4));
    ELB_CUDA(cudaMemcpy(dx.p, x, size_t(ww->n) * 4, cudaMemcpyHostToDevice));
    GemvArgs a;
    a.dbgP = dP.as<int32_t>(); a.dbgI = dI.as<int32_t>(); a.dbgJ = dJ.as<int32_t>();
    ELB_TRY(matvec_on(ww, dx.as<float>(), dy.as<float>(), nl, nullptr, &a));
    ELB_CUDA(cudaStreamSynchronize(nullptr));
    // device arrays carry 4 limb slots; compact to nl
    auto fetch = [&](int32_t* dst, const Dev& src, size_t n4) -> int {
        if (!dst) return ELB_OK;
        std::vector<int32_t> tmp(n4);
        ELB_CUDA(cudaMemcpy(tmp.data(), src.p, n4 * 4, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n4 / 4; ++i)
            for (int l = 0; l < nl; ++l) dst[i * nl + l] = tmp[i * 4 + l];
        return ELB_OK;
    };
    ELB_TRY(fetch(P, dP, nP));
    ELB_TRY(fetch(I, dI, nI));
    ELB_TRY(fetch(J, dJ, nI));
    return ELB_OK;
}

// ---------------------------------------------------------------- model

int elb_model_create(const elb_config* cfg, int n_ctx, int device, elb_model** out) {
    if (elb_device_count() == 0) return fail(ELB_ERR_CUDA, std::string("no usable CUDA device: ") + g_error);
    Model* m = nullptr;
    ELB_TRY(model_create(cfg, n_ctx, device, &m));
    *out = reinterpret_cast<elb_model*>(m);
    return ELB_OK;
}
int elb_model_create_tp(const elb_config* cfg, int n_ctx, int device, int tp_rank, int tp_size, const void* id128,
                        elb_model** out) {
    if (elb_device_count() == 0) return fail(ELB_ERR_CUDA, std::string("no usable CUDA device: ") + g_error);
    Model* m = nullptr;
    ELB_TRY(model_create_tp(cfg, n_ctx, device, tp_rank, tp_size, id128, &m));
    *out = reinterpret_cast<elb_model*>(m);
    return ELB_OK;
}
int elb_tp_unique_id(void* id128) { return tp_unique_id(id128); }
int elb_tp_dims(const elb_config* cfg, int tp_rank, int tp_size, int* n_head, int* n_head_kv, int64_t* f0, int64_t* f1,
                int64_t* v0, int64_t* v1) {
    if (!cfg) return fail(ELB_ERR_INVALID, "tp_dims: null configuration");
    TpDims d;
    ELB_TRY(tp_dims(*cfg, tp_rank, tp_size, &d));
    if (n_head) *n_head = d.H;
    if (n_head_kv) *n_head_kv = d.HKV;
    if (f0) *f0 = d.f0;
    if (f1) *f1 = d.f1;
    if (v0) *v0 = d.v0;
    if (v1) *v1 = d.v1;
    return ELB_OK;
}
int elb_tp_shard_shape(const elb_config* cfg, int tp_rank, int tp_size, int role, int ggml_type, int64_t rows, int64_t n,
                       int64_t* out_rows, int64_t* out_n, size_t* out_nbytes) {
    if (!cfg) return fail(ELB_ERR_INVALID, "tp_shard_shape: null configuration");
    TpDims d;
    TpShard s;
    ELB_TRY(tp_dims(*cfg, tp_rank, tp_size, &d));
    ELB_TRY(tp_shard_shape(*cfg, d, role, ggml_type, rows, n, &s));
    if (out_rows) *out_rows = s.rows;
    if (out_n) *out_n = s.n;
    if (out_nbytes) *out_nbytes = s.nbytes;
    return ELB_OK;
}
int elb_tp_shard_copy(const elb_config* cfg, int tp_rank, int tp_size, int role, int ggml_type, int64_t rows, int64_t n,
                      const void* bytes, size_t nbytes, void* out, size_t out_nbytes) {
    if (!cfg) return fail(ELB_ERR_INVALID, "tp_shard_copy: null configuration");
    TpDims d;
    TpShard s;
    ELB_TRY(tp_dims(*cfg, tp_rank, tp_size, &d));
    ELB_TRY(tp_shard_shape(*cfg, d, role, ggml_type, rows, n, &s));
    if (out_nbytes < s.nbytes) return fail(ELB_ERR_INVALID, "tp_shard_copy: output buffer too small");
    return tp_shard_copy(s, static_cast<const uint8_t*>(bytes), nbytes, static_cast<uint8_t*>(out));
}
int elb_model_set_tensor(elb_model* m, int role, int layer, int ggml_type, int64_t rows, int64_t n, const void* bytes,
                         size_t nbytes) {
    return model_set_tensor(M(m), role, layer, ggml_type, rows, n, bytes, nbytes);
}
int elb_model_finalize(elb_model* m) { return model_finalize(M(m)); }
int elb_model_load_gguf(const char* path, int n_ctx, int device, int max_batch, int n_seq, elb_model** out) {
    if (!out) return fail(ELB_ERR_INVALID, "load_gguf: null argument");
    Model* m = nullptr;
    ELB_TRY(model_load_gguf(path, n_ctx, device, max_batch, n_seq, 0, 1, nullptr, &m));  // the file is checked before any device is touched
    *out = reinterpret_cast<elb_model*>(m);
    return ELB_OK;
}
int elb_model_load_gguf_tp(const char* path, int n_ctx, int device, int max_batch, int n_seq, int tp_rank, int tp_size,
                           const void* id128, elb_model** out) {
    if (!out) return fail(ELB_ERR_INVALID, "load_gguf: null argument");
    Model* m = nullptr;
    ELB_TRY(model_load_gguf(path, n_ctx, device, max_batch, n_seq, tp_rank, tp_size, id128, &m));
    *out = reinterpret_cast<elb_model*>(m);
    return ELB_OK;
}
int elb_model_config(const elb_model* m, elb_config* out) { return model_config(M(m), out); }
void elb_model_destroy(elb_model* m) { model_destroy(M(m)); }
int elb_model_eval(elb_model* m, const int32_t* tokens, int n, int pos0, float* logits) {
    return model_eval(M(m), tokens, n, pos0, logits);
}
int elb_model_eval_top(elb_model* m, const int32_t* tokens, int n, int pos0, int k, int32_t* ids, float* top_logits,
                       double* lse) {
    return model_eval_top(M(m), tokens, n, pos0, k, ids, top_logits, lse);
}
int elb_model_eval_top_masked(elb_model* m, const int32_t* tokens, int n, int pos0, int k, const uint32_t* allowed,
                              int32_t* ids, float* top_logits, double* lse) {
    if (!allowed) return fail(ELB_ERR_INVALID, "eval_top_masked: null mask");
    return model_eval_top(M(m), tokens, n, pos0, k, ids, top_logits, lse, allowed);
}
int elb_model_eval_batch(elb_model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos,
                         const uint8_t* want, float* logits) {
    return model_eval_batch(M(m), n, tokens, seq, pos, want, logits);
}
int elb_model_eval_batch_top(elb_model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos,
                             const uint8_t* want, int k, int32_t* ids, float* top_logits, double* lse) {
    return model_eval_batch_top(M(m), n, tokens, seq, pos, want, k, ids, top_logits, lse);
}
int elb_model_eval_steps(elb_model* m, const int32_t* tokens, int n, int pos0, float* device_ms) {
    return model_eval_steps(M(m), tokens, n, pos0, device_ms);
}
int elb_model_last_eval_stats(const elb_model* m, float* device_ms, int64_t* kernel_launches) {
    return model_stats(M(m), device_ms, kernel_launches);
}
int elb_model_hidden(elb_model* m, float* out) { return model_hidden(M(m), out); }
size_t elb_model_weight_bytes(const elb_model* m) { return model_weight_bytes(M(m)); }
size_t elb_model_kv_bytes_per_token(const elb_model* m) { return model_kv_bytes_per_token(M(m)); }

// ---------------------------------------------------------------- microbenchmarks

int elb_bench_matvec(elb_weight* const* ws, int n_w, const float* d_x, float* d_y, int nl, int iters, float* avg_ms) {
    if (!ws || n_w <= 0 || iters <= 0 || !avg_ms) return fail(ELB_ERR_INVALID, "bench_matvec: bad argument");
    ELB_CUDA(cudaSetDevice(W(ws[0])->device));
    cudaStream_t s;
    ELB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaEvent_t e0, e1;
    ELB_CUDA(cudaEventCreate(&e0));
    ELB_CUDA(cudaEventCreate(&e1));
    // warm-up: split + matvec once per weight (sets the launch attributes and leaves each weight's limbs in place);
    // the timed region is a captured chain of `iters` matvec launches over the weights in rotation, launched
    // back to back the way the decode step launches them (programmatic dependent launch).
    int rc = ELB_OK;
    for (int i = 0; i < n_w && rc == ELB_OK; ++i) rc = matvec_on(W(ws[i]), d_x, d_y, nl, s, nullptr);
    cudaStreamSynchronize(s);
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    const bool pdl = !(std::getenv("ELB_NO_PDL") && std::getenv("ELB_NO_PDL")[0] == '1');
    if (rc == ELB_OK && cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) rc = fail(ELB_ERR_CUDA, "bench_matvec: capture failed");
    if (rc == ELB_OK) {
        for (int i = 0; i < iters && rc == ELB_OK; ++i) {
            const Weight* w = W(ws[i % n_w]);
            GemvArgs a;
            a.x = d_x; a.y = d_y; a.limbs = w->xlimbs; a.inv_scale = w->xinv; a.pdl = pdl && i > 0;
            rc = gemv_launch(w, a, s);
        }
        const cudaError_t ec = cudaStreamEndCapture(s, &g);
        if (rc == ELB_OK && (ec != cudaSuccess || cudaGraphInstantiate(&ge, g, 0) != cudaSuccess)) rc = fail(ELB_ERR_CUDA, "bench_matvec: graph build failed");
    }
    float ms = 0.f;
    cudaError_t e = cudaSuccess;
    if (rc == ELB_OK) {
        cudaGraphLaunch(ge, s);  // one untimed replay
        cudaStreamSynchronize(s);
        cudaEventRecord(e0, s);
        cudaGraphLaunch(ge, s);
        cudaEventRecord(e1, s);
        e = cudaStreamSynchronize(s);
        cudaEventElapsedTime(&ms, e0, e1);
    }
    if (ge) cudaGraphExecDestroy(ge);
    if (g) cudaGraphDestroy(g);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(s);
    if (rc != ELB_OK) return rc;
    ELB_CUDA(e);
    *avg_ms = ms / iters;
    return ELB_OK;
}

int elb_bench_matmul(elb_weight* const* ws, int n_w, const float* d_x, int64_t b, float* d_y, int nl, int iters,
                     float* avg_ms) {
    if (!ws || n_w <= 0 || iters <= 0 || !avg_ms) return fail(ELB_ERR_INVALID, "bench_matmul: bad argument");
    ELB_CUDA(cudaSetDevice(W(ws[0])->device));
    cudaStream_t s;
    ELB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaEvent_t e0, e1;
    ELB_CUDA(cudaEventCreate(&e0));
    ELB_CUDA(cudaEventCreate(&e1));
    Dev scratch;
    int rc = ELB_OK;
    for (int i = 0; i < n_w && rc == ELB_OK; ++i) rc = matmul_dev_on(W(ws[i]), d_x, b, d_y, nl, s, &scratch);
    cudaStreamSynchronize(s);
    cudaEventRecord(e0, s);
    for (int i = 0; i < iters && rc == ELB_OK; ++i) rc = matmul_dev_on(W(ws[i % n_w]), d_x, b, d_y, nl, s, &scratch);
    cudaEventRecord(e1, s);
    const cudaError_t e = cudaStreamSynchronize(s);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(s);
    if (rc != ELB_OK) return rc;
    ELB_CUDA(e);
    *avg_ms = ms / iters;
    return ELB_OK;
}

}  // extern "C"
