// TEST INFRASTRUCTURE — not part of the product.
//
// A plain-C surface over the reference's own CPU path, compiled together with the reference's UNMODIFIED
// sources (src/quant.cpp, src/ops.cpp, src/model.cpp, src/gguf.cpp) where they lie; see the Makefile in this
// directory. The result, oracle/_ref/libelref.so, is used (a) to pin oracle.c's restatement, (b) to generate
// the golden fixtures under tests/golden, and (c) as the timed CPU baseline. Nothing in the product links it.
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "gguf.h"
#include "model.h"
#include "ops.h"
#include "quant.h"

namespace {
thread_local std::string g_err;

el::Tensor make_tensor(int ggml_type, int64_t rows, int64_t n, const void* bytes, uint64_t nbytes) {
    el::Tensor t;
    t.name = "oracle";
    t.type = el::GgmlType(uint32_t(ggml_type));
    t.ne = {uint64_t(n), uint64_t(rows)};
    t.numel = uint64_t(rows) * uint64_t(n);
    t.nbytes = nbytes;
    t.data = static_cast<const uint8_t*>(bytes);
    return t;
}

struct RefModel {
    std::unique_ptr<el::Gguf> gguf;
    std::unique_ptr<el::Backend> be;
};
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

void ref_set_threads(int n) { el::set_threads(n); }
int ref_threads() { return el::threads(); }

// el::get_row / convert_row (src/ops.cpp:43-82) on `rows` consecutive rows starting at row0.
int ref_dequant_rows(int ggml_type, int64_t rows_total, int64_t n, const void* bytes, uint64_t nbytes, int64_t row0,
                     int64_t rows, float* out) {
    try {
        const el::Tensor t = make_tensor(ggml_type, rows_total, n, bytes, nbytes);
        for (int64_t r = 0; r < rows; ++r) el::get_row(t, uint64_t(row0 + r), out + r * n);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

// el::matvec (src/ops.cpp:126-153)
int ref_matvec(int ggml_type, int64_t rows, int64_t n, const void* bytes, uint64_t nbytes, const float* x, float* y) {
    try {
        const el::Tensor t = make_tensor(ggml_type, rows, n, bytes, nbytes);
        el::matvec(t, x, y);
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

// el::rmsnorm (src/ops.cpp:155-160)
void ref_rmsnorm(float* out, const float* x, const float* w, int n, float eps) { el::rmsnorm(out, x, w, n, eps); }

// el::q4k_scale_min (src/quant.h:44-52)
void ref_q4k_scale_min(int j, const uint8_t* q, int* sc, int* m) { el::q4k_scale_min(j, q, *sc, *m); }

// make_cpu_backend over a GGUF file (src/model.cpp:236-238)
void* ref_model_open(const char* path, int n_ctx) {
    try {
        auto m = std::make_unique<RefModel>();
        m->gguf = std::make_unique<el::Gguf>(path);
        m->be = el::make_cpu_backend(*m->gguf, n_ctx);
        return m.release();
    } catch (const std::exception& e) {
        g_err = e.what();
        return nullptr;
    }
}

int ref_model_config(void* h, int* out10) {
    const el::Config& c = static_cast<RefModel*>(h)->be->cfg();
    const int v[10] = {c.n_layer, c.n_embd, c.n_ff, c.n_head, c.n_head_kv, c.head_dim, c.n_vocab, c.rope_dim,
                       c.n_ctx_train, static_cast<RefModel*>(h)->be->n_ctx()};
    std::memcpy(out10, v, sizeof v);
    return 0;
}

// Backend::eval (src/model.h:48-50). Returns 0 ok, 2 invalid_argument, 3 out_of_range, 1 other.
int ref_model_eval(void* h, const int32_t* tokens, int n, int pos0, float* logits) {
    try {
        static_cast<RefModel*>(h)->be->eval(tokens, n, pos0, logits);
        return 0;
    } catch (const std::invalid_argument& e) {
        g_err = e.what();
        return 2;
    } catch (const std::out_of_range& e) {
        g_err = e.what();
        return 3;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

void ref_model_close(void* h) { delete static_cast<RefModel*>(h); }

}  // extern "C"
