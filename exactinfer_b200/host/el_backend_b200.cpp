// Drop-in replacement for the reference's CUDA translation unit (src/cuda/model_cuda.cu) and its stub
// (src/cuda_stub.cpp): it defines exactly the two symbols those define — el::cuda_available and el::make_cuda_backend
// (src/model.h:56-57) — and an el::Backend (src/model.h:42-51) whose eval() runs on libelb.so through the C ABI of
// include/elb.h. It is compiled against the reference's own headers (model.h, ops.h, gguf.h); nothing else of the
// reference changes: main.cpp's make_backend (src/main.cpp:125-132) picks it up as "--backend cuda".
//
//   g++ -std=c++20 -I<reference>/src -I<this repo>/include -c el_backend_b200.cpp
//   link with the reference's objects (without cuda_stub / model_cuda) and -lelb
#include <stdexcept>
#include <string>

#include "elb.h"
#include "model.h"
#include "ops.h"

namespace el {

namespace {

// status code -> the exception type the reference's CUDA backend throws for the same condition
// (src/cuda/model_cuda.cu:40-44, 1649-1652)
[[noreturn]] void raise(int rc) {
    const std::string msg = elb_last_error();
    switch (rc) {
        case ELB_ERR_INVALID: throw std::invalid_argument(msg);
        case ELB_ERR_RANGE: throw std::out_of_range(msg);
        default: throw std::runtime_error(msg);
    }
}
void check(int rc) {
    if (rc != ELB_OK) raise(rc);
}

class B200Model final : public Backend {
public:
    B200Model(const Gguf& g, int n_ctx) : c_(read_config(g)), n_ctx_(n_ctx) {
        if (n_ctx_ <= 0) throw std::runtime_error("baglam uzunlugu pozitif olmali");
        const ModelTensors t = read_tensors(g, c_);  // fills c_.n_vocab, validates shapes and types
        elb_config cfg{};
        cfg.n_layer = c_.n_layer; cfg.n_embd = c_.n_embd; cfg.n_ff = c_.n_ff; cfg.n_head = c_.n_head;
        cfg.n_head_kv = c_.n_head_kv; cfg.head_dim = c_.head_dim; cfg.n_vocab = c_.n_vocab; cfg.rope_dim = c_.rope_dim;
        cfg.rope_base = c_.rope_base; cfg.eps = c_.eps; cfg.max_batch = 512;
        check(elb_model_create(&cfg, n_ctx_, 0, &m_));
        try {
            set(ELB_TOK_EMBD, 0, *t.tok_embd);
            if (t.output != t.tok_embd) set(ELB_OUTPUT, 0, *t.output);  // tied head otherwise (src/model.cpp:73-74)
            set(ELB_OUTPUT_NORM, 0, *t.output_norm);
            for (int l = 0; l < c_.n_layer; ++l) {
                const LayerTensors& L = t.layers[size_t(l)];
                set(ELB_ATTN_NORM, l, *L.attn_norm); set(ELB_FFN_NORM, l, *L.ffn_norm);
                set(ELB_Q_NORM, l, *L.q_norm); set(ELB_K_NORM, l, *L.k_norm);
                set(ELB_WQ, l, *L.wq); set(ELB_WK, l, *L.wk); set(ELB_WV, l, *L.wv); set(ELB_WO, l, *L.wo);
                set(ELB_GATE, l, *L.gate); set(ELB_UP, l, *L.up); set(ELB_DOWN, l, *L.down);
            }
            check(elb_model_finalize(m_));  // uploads; the mapped file is not needed by the backend afterwards
        } catch (...) {
            elb_model_destroy(m_);
            throw;
        }
    }
    ~B200Model() override { elb_model_destroy(m_); }

    const Config& cfg() const override { return c_; }
    int n_ctx() const override { return n_ctx_; }
    const char* name() const override { return "cuda"; }
    void eval(const int32_t* tokens, int n, int pos0, float* logits) override {
        check(elb_model_eval(m_, tokens, n, pos0, logits));
    }

private:
    void set(int role, int layer, const Tensor& t) {
        const int64_t n = int64_t(t.ne[0]), rows = int64_t(t.rows());
        check(elb_model_set_tensor(m_, role, layer, int(uint32_t(t.type)), rows, n, t.data, size_t(t.nbytes)));
    }
    Config c_;
    int n_ctx_;
    elb_model* m_ = nullptr;
};

}  // namespace

bool cuda_available(std::string* why) {
    if (elb_device_count() > 0) return true;
    if (why) *why = elb_last_error();
    return false;
}

std::unique_ptr<Backend> make_cuda_backend(const Gguf& g, int n_ctx) {
    std::string why;
    if (!cuda_available(&why)) throw std::runtime_error("CUDA kullanilamiyor: " + why);
    return std::make_unique<B200Model>(g, n_ctx);
}

}  // namespace el
