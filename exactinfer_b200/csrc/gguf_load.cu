// A model straight from a GGUF file: the file is mapped, its metadata gives the configuration (the keys read_config of
// the reference reads, src/model.cpp:38-64), its tensor directory gives every tensor of el::ModelTensors by name
// (read_tensors, src/model.cpp:66-103), and the tensors go from the mapping to elb_model_set_tensor without a copy.
// Host code only; GGUF versions 2 and 3, little endian. Rejects what the reference rejects: other architectures,
// RoPE scaling, bias tensors, key_length != value_length.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace elb {

namespace {

struct Cursor8 {  // bounds-checked reader over the mapping
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (size_t(end - p) < sizeof(T)) { ok = false; p = end; return v; }
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > uint64_t(end - p)) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char*>(p), size_t(n));
        p += n;
        return s;
    }
    void skip(uint64_t n) {
        if (n > uint64_t(end - p)) { ok = false; p = end; } else p += n;
    }
};

enum { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };

size_t scalar_size(uint32_t t) {
    switch (t) {
        case T_U8: case T_I8: case T_BOOL: return 1;
        case T_U16: case T_I16: return 2;
        case T_U32: case T_I32: case T_F32: return 4;
        case T_U64: case T_I64: case T_F64: return 8;
        default: return 0;
    }
}

struct Meta {  // the scalar and string values of the metadata (arrays are skipped: the forward pass needs none)
    std::map<std::string, double> num;
    std::map<std::string, std::string> str;
};

struct TensorInfo {
    std::vector<uint64_t> ne;
    uint32_t type = 0;
    uint64_t offset = 0;
};

bool read_value(Cursor8& c, uint32_t type, const std::string& key, Meta* m) {
    switch (type) {
        case T_U8: m->num[key] = c.get<uint8_t>(); break;
        case T_I8: m->num[key] = c.get<int8_t>(); break;
        case T_U16: m->num[key] = c.get<uint16_t>(); break;
        case T_I16: m->num[key] = c.get<int16_t>(); break;
        case T_U32: m->num[key] = c.get<uint32_t>(); break;
        case T_I32: m->num[key] = c.get<int32_t>(); break;
        case T_F32: m->num[key] = c.get<float>(); break;
        case T_BOOL: m->num[key] = c.get<uint8_t>(); break;
        case T_U64: m->num[key] = double(c.get<uint64_t>()); break;
        case T_I64: m->num[key] = double(c.get<int64_t>()); break;
        case T_F64: m->num[key] = c.get<double>(); break;
        case T_STR: m->str[key] = c.str(); break;
        case T_ARR: {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = c.get<uint64_t>();
            if (et == T_STR) {
                for (uint64_t i = 0; i < n && c.ok; ++i) c.skip(c.get<uint64_t>());
            } else if (scalar_size(et)) {
                if (n > (uint64_t(1) << 40)) return false;
                c.skip(n * scalar_size(et));
            } else {
                return false;  // nested arrays: not produced by any writer of these models
            }
            break;
        }
        default: return false;
    }
    return c.ok;
}

int64_t tensor_bytes(uint32_t type, uint64_t n, uint64_t rows) {
    if (n > (uint64_t(1) << 31) || rows > (uint64_t(1) << 31)) return -1;  // n * rows * 4 stays far below 2^63
    switch (type) {
        case ELB_F32: return int64_t(n * rows * 4);
        case ELB_F16: return int64_t(n * rows * 2);
        case ELB_Q8_0: return n % QK8_0 ? -1 : int64_t(n / QK8_0 * Q8_0_BYTES * rows);
        case ELB_Q4_K: return n % QK_K ? -1 : int64_t(n / QK_K * Q4_K_BYTES * rows);
        case ELB_Q6_K: return n % QK_K ? -1 : int64_t(n / QK_K * Q6_K_BYTES * rows);
        default: return -1;
    }
}

struct Mapping {
    int fd = -1;
    void* base = MAP_FAILED;
    size_t size = 0;
    ~Mapping() {
        if (base != MAP_FAILED) munmap(base, size);
        if (fd >= 0) close(fd);
    }
};

}  // namespace

int model_load_gguf(const char* path, int n_ctx, int device, int max_batch, int n_seq, int tp_rank, int tp_size,
                    const void* id128, Model** out) {
    if (!path || !out) return fail(ELB_ERR_INVALID, "load_gguf: null argument");
    Mapping map;
    map.fd = open(path, O_RDONLY);
    if (map.fd < 0) return fail(ELB_ERR_INVALID, std::string("load_gguf: cannot open ") + path);
    struct stat st;
    if (fstat(map.fd, &st) != 0 || st.st_size < 24) return fail(ELB_ERR_INVALID, "load_gguf: file too short");
    map.size = size_t(st.st_size);
    map.base = mmap(nullptr, map.size, PROT_READ, MAP_PRIVATE, map.fd, 0);
    if (map.base == MAP_FAILED) return fail(ELB_ERR_MEMORY, "load_gguf: cannot map the file");
    const uint8_t* base = static_cast<const uint8_t*>(map.base);
    Cursor8 c{base, base + map.size};
    if (c.get<uint32_t>() != 0x46554747u) return fail(ELB_ERR_INVALID, "load_gguf: not a GGUF file");
    const uint32_t version = c.get<uint32_t>();
    if (version != 2 && version != 3) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: GGUF version 2 or 3 expected");
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (n_tensors > (1u << 20) || n_kv > (1u << 20)) return fail(ELB_ERR_INVALID, "load_gguf: implausible header");
    Meta meta;
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        if (!c.ok || !read_value(c, type, key, &meta)) return fail(ELB_ERR_INVALID, "load_gguf: damaged metadata at key " + key);
    }
    std::map<std::string, TensorInfo> dir;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        const std::string name = c.str();
        TensorInfo t;
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd > 4) return fail(ELB_ERR_INVALID, "load_gguf: damaged tensor directory");
        for (uint32_t d = 0; d < nd; ++d) t.ne.push_back(c.get<uint64_t>());
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail(ELB_ERR_INVALID, "load_gguf: damaged tensor directory");
        dir[name] = t;
    }
    const uint64_t align = meta.num.count("general.alignment") ? uint64_t(meta.num["general.alignment"]) : 32;
    if (align == 0 || (align & (align - 1))) return fail(ELB_ERR_INVALID, "load_gguf: alignment is not a power of two");
    const uint64_t data0 = (uint64_t(c.p - base) + align - 1) / align * align;

    // configuration (defaults as the reference's)
    const std::string arch = meta.str.count("general.architecture") ? meta.str["general.architecture"] : "";
    if (arch != "qwen3") return fail(ELB_ERR_UNSUPPORTED, "load_gguf: unsupported architecture '" + arch + "' (qwen3 only)");
    auto num = [&](const char* k, double dflt, bool required, bool* missing) {
        const std::string key = arch + "." + k;
        if (meta.num.count(key)) return meta.num[key];
        if (required) *missing = true;
        return dflt;
    };
    bool missing = false;
    elb_config cfg{};
    cfg.n_layer = int(num("block_count", 0, true, &missing));
    cfg.n_embd = int(num("embedding_length", 0, true, &missing));
    cfg.n_ff = int(num("feed_forward_length", 0, true, &missing));
    cfg.n_head = int(num("attention.head_count", 0, true, &missing));
    if (missing) return fail(ELB_ERR_INVALID, "load_gguf: a required qwen3.* key is missing");
    cfg.n_head_kv = int(num("attention.head_count_kv", cfg.n_head, false, &missing));
    cfg.head_dim = int(num("attention.key_length", cfg.n_head ? cfg.n_embd / cfg.n_head : 0, false, &missing));
    if (int(num("attention.value_length", cfg.head_dim, false, &missing)) != cfg.head_dim)
        return fail(ELB_ERR_UNSUPPORTED, "load_gguf: key_length != value_length");
    cfg.rope_dim = int(num("rope.dimension_count", cfg.head_dim, false, &missing));
    cfg.rope_base = num("rope.freq_base", 10000.0, false, &missing);
    cfg.eps = float(num("attention.layer_norm_rms_epsilon", 1e-6, false, &missing));
    cfg.max_batch = max_batch;
    cfg.n_seq = n_seq;
    const std::string scaling = arch + ".rope.scaling.type";
    if (meta.str.count(scaling) && meta.str[scaling] != "none") return fail(ELB_ERR_UNSUPPORTED, "load_gguf: RoPE scaling is not supported");

    auto find = [&](const std::string& name) -> const TensorInfo* {
        auto it = dir.find(name);
        return it == dir.end() ? nullptr : &it->second;
    };
    const TensorInfo* emb = find("token_embd.weight");
    if (!emb || emb->ne.size() != 2 || emb->ne[0] != uint64_t(cfg.n_embd)) return fail(ELB_ERR_INVALID, "load_gguf: token_embd.weight missing or of the wrong shape");
    cfg.n_vocab = int(emb->ne[1]);

    // Every tensor of the model is looked up, sized and bounds-checked before a device or a communicator is touched
    // (expect_shape of the reference, src/model.cpp:76,92-95: the norm vectors have E, the head norms head_dim values).
    if (cfg.n_layer <= 0 || cfg.n_layer > 512 || cfg.n_embd <= 0 || cfg.n_ff <= 0 || cfg.n_head <= 0 || cfg.n_head_kv <= 0 || cfg.head_dim <= 0)
        return fail(ELB_ERR_INVALID, "load_gguf: implausible model dimensions");
    auto vet = [&](const std::string& name, bool required, uint64_t want_n, uint64_t want_rows) -> int {
        const TensorInfo* t = find(name);
        if (!t) return required ? fail(ELB_ERR_INVALID, "load_gguf: tensor " + name + " is missing") : ELB_OK;
        const uint64_t n = t->ne.empty() ? 0 : t->ne[0], rows = t->ne.size() > 1 ? t->ne[1] : 1;
        if (t->ne.size() > 2 || n == 0) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: unexpected rank of " + name);
        if (n != want_n || rows != want_rows) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: unexpected shape of " + name);
        const int64_t bytes = tensor_bytes(t->type, n, rows);
        if (bytes < 0) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: tensor type of " + name + " is not supported (F32, F16, Q8_0, Q4_K, Q6_K)");
        if (data0 > map.size || t->offset > map.size - data0 || uint64_t(bytes) > map.size - data0 - t->offset)
            return fail(ELB_ERR_INVALID, "load_gguf: tensor " + name + " runs past the end of the file");
        return ELB_OK;
    };
    {
        const uint64_t E = uint64_t(cfg.n_embd), V = uint64_t(cfg.n_vocab), F = uint64_t(cfg.n_ff), D = uint64_t(cfg.head_dim);
        const uint64_t QD = uint64_t(cfg.n_head) * D, KD = uint64_t(cfg.n_head_kv) * D;
        ELB_TRY(vet("token_embd.weight", true, E, V));
        ELB_TRY(vet("output.weight", false, E, V));
        ELB_TRY(vet("output_norm.weight", true, E, 1));
        for (int l = 0; l < cfg.n_layer; ++l) {
            const std::string b = "blk." + std::to_string(l) + ".";
            ELB_TRY(vet(b + "attn_norm.weight", true, E, 1));
            ELB_TRY(vet(b + "ffn_norm.weight", true, E, 1));
            ELB_TRY(vet(b + "attn_q_norm.weight", true, D, 1));
            ELB_TRY(vet(b + "attn_k_norm.weight", true, D, 1));
            ELB_TRY(vet(b + "attn_q.weight", true, E, QD));
            ELB_TRY(vet(b + "attn_k.weight", true, E, KD));
            ELB_TRY(vet(b + "attn_v.weight", true, E, KD));
            ELB_TRY(vet(b + "attn_output.weight", true, QD, E));
            ELB_TRY(vet(b + "ffn_gate.weight", true, E, F));
            ELB_TRY(vet(b + "ffn_up.weight", true, E, F));
            ELB_TRY(vet(b + "ffn_down.weight", true, F, E));
        }
    }

    Model* m = nullptr;
    // under tensor parallelism every rank maps the whole file; model_set_tensor keeps this rank's cut of each tensor,
    // so only those pages of the mapping are read for the column-parallel matrices
    ELB_TRY(model_create_tp(&cfg, n_ctx, device, tp_rank, tp_size, id128, &m));
    auto give = [&](const std::string& name, int role, int layer, bool required) -> int {
        const TensorInfo* t = find(name);
        if (!t) return required ? fail(ELB_ERR_INVALID, "load_gguf: tensor " + name + " is missing") : ELB_OK;
        const uint64_t n = t->ne.empty() ? 0 : t->ne[0], rows = t->ne.size() > 1 ? t->ne[1] : 1;
        if (t->ne.size() > 2 || n == 0) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: unexpected rank of " + name);
        const int64_t bytes = tensor_bytes(t->type, n, rows);
        if (bytes < 0) return fail(ELB_ERR_UNSUPPORTED, "load_gguf: tensor type of " + name + " is not supported (F32, F16, Q8_0, Q4_K, Q6_K)");
        // (compared without forming data0 + offset + bytes: the offset comes from the file and may be close to 2^64)
        if (data0 > map.size || t->offset > map.size - data0 || uint64_t(bytes) > map.size - data0 - t->offset)
            return fail(ELB_ERR_INVALID, "load_gguf: tensor " + name + " runs past the end of the file");
        return model_set_tensor(m, role, layer, int(t->type), int64_t(rows), int64_t(n), base + data0 + t->offset, size_t(bytes));
    };
    int rc = give("token_embd.weight", ELB_TOK_EMBD, 0, true);
    if (rc == ELB_OK) rc = give("output.weight", ELB_OUTPUT, 0, false);  // absent: tied head
    if (rc == ELB_OK) rc = give("output_norm.weight", ELB_OUTPUT_NORM, 0, true);
    static const struct { const char* name; int role; } per_layer[] = {
        {"attn_norm.weight", ELB_ATTN_NORM}, {"ffn_norm.weight", ELB_FFN_NORM}, {"attn_q_norm.weight", ELB_Q_NORM},
        {"attn_k_norm.weight", ELB_K_NORM}, {"attn_q.weight", ELB_WQ}, {"attn_k.weight", ELB_WK}, {"attn_v.weight", ELB_WV},
        {"attn_output.weight", ELB_WO}, {"ffn_gate.weight", ELB_GATE}, {"ffn_up.weight", ELB_UP}, {"ffn_down.weight", ELB_DOWN}};
    for (int l = 0; l < cfg.n_layer && rc == ELB_OK; ++l) {
        const std::string b = "blk." + std::to_string(l) + ".";
        for (const char* bias : {"attn_q.bias", "attn_k.bias", "attn_v.bias", "attn_output.bias"})
            if (find(b + bias)) rc = fail(ELB_ERR_UNSUPPORTED, "load_gguf: bias tensor " + b + bias + " is not expected");
        for (const auto& t : per_layer)
            if (rc == ELB_OK) rc = give(b + t.name, t.role, l, true);
    }
    if (rc == ELB_OK) rc = model_finalize(m);  // uploads from the mapping; nothing of it is needed afterwards
    if (rc != ELB_OK) {
        model_destroy(m);
        return rc;
    }
    *out = m;
    return ELB_OK;
}

}  // namespace elb
