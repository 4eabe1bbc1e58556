/* exactinfer forward pass for NVIDIA B200 (sm_100a) — C ABI of libelb.so.
 *
 * Plain pointers and sizes only. Every function returns an elb_status (0 = ok) unless noted; after a failure
 * elb_last_error() describes it (thread-local string). Nothing here throws, allocates with a foreign allocator
 * or falls back to the CPU: without a CUDA device every compute entry point fails with ELB_ERR_CUDA.
 *
 * Each entry point cites the interface of the reference project (burakcelik1061-star/exactinfer) that it stands
 * in for, as path:line inside that project.
 */
#ifndef ELB_H
#define ELB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ELB_OK = 0,
    ELB_ERR_CUDA = 1,         /* a CUDA call failed, or no usable device (std::runtime_error in the reference) */
    ELB_ERR_INVALID = 2,      /* bad argument, e.g. n <= 0 (std::invalid_argument, src/cuda/model_cuda.cu:1649) */
    ELB_ERR_RANGE = 3,        /* context full or token id out of range (std::out_of_range, :1650-1652) */
    ELB_ERR_UNSUPPORTED = 4,  /* tensor type / shape the path does not cover (std::runtime_error, :1428,1542) */
    ELB_ERR_MEMORY = 5,       /* not enough device memory (std::runtime_error, :1586-1590) */
    ELB_ERR_STATE = 6         /* call order, e.g. eval before finalize */
} elb_status;

/* ggml tensor type ids, as stored in GGUF (src/gguf.h:22-25) */
enum { ELB_F32 = 0, ELB_F16 = 1, ELB_Q8_0 = 8, ELB_Q4_K = 12, ELB_Q6_K = 14 };

const char* elb_last_error(void);

/* ---- device -------------------------------------------------------------------------------------------------
 * el::cuda_available (src/model.h:56, src/cuda/model_cuda.cu:1894-1907): number of devices with compute
 * capability 10.x; 0 with the reason in elb_last_error() when there is none. */
int elb_device_count(void);
/* Raw device / pinned-host buffers for callers that keep activations on the GPU (tests, microbenchmarks). */
int elb_malloc(int device, size_t bytes, void** out);
int elb_free(void* dptr);
int elb_host_alloc(size_t bytes, void** out); /* pinned */
int elb_host_free(void* hptr);
int elb_memcpy_h2d(void* dst, const void* src, size_t bytes);
int elb_memcpy_d2h(void* dst, const void* src, size_t bytes);
int elb_device_sync(int device);
/* Free and total device memory in bytes (cudaMemGetInfo; the reference's pre-flight check reads the same figures,
 * src/cuda/model_cuda.cu:1578-1591). */
int elb_device_mem_info(int device, size_t* free_bytes, size_t* total_bytes);
/* Self-test of the failure path (no counterpart in the reference, whose kernels have no device-side waits): runs the
 * tensor-core kernels' bounded barrier wait on a barrier that nobody arrives at, with a short limit. The wait must give
 * up and report: the call returns ELB_ERR_CUDA (elb_last_error names the wait) and the device stays usable; ELB_OK
 * would mean the expiry went unnoticed. Nothing faults or hangs. */
int elb_selftest_wait_expiry(int device);

/* ---- weights ------------------------------------------------------------------------------------------------
 * One weight matrix W[rows][n] in a ggml block format, uploaded and re-laid out for the GPU kernels
 * (upload_group, src/cuda/model_cuda.cu:1450-1506). `bytes` is the tensor exactly as it lies in the GGUF file
 * (el::Tensor::data, src/gguf.h:27-36). Supported: F16, Q8_0, Q4_K, Q6_K (wtype_of, :1421-1431).
 *
 * flags: ELB_W_PLANES also builds the int8 digit planes the tensor-core (prefill) path reads;
 *        ELB_W_PAIR interleaves two equally shaped matrices given back to back in `bytes` (gate then up) in
 *        8-row groups, so that the SwiGLU epilogue finds gate[r] and up[r] in one thread (`rows` = rows of ONE
 *        of them; the weight then has 2*rows rows). */
typedef struct elb_weight elb_weight;
enum { ELB_W_PLANES = 1, ELB_W_PAIR = 2 };
int elb_weight_create(int device, int ggml_type, int64_t rows, int64_t n, const void* bytes, size_t nbytes, int flags,
                      elb_weight** out);
void elb_weight_destroy(elb_weight* w);
int64_t elb_weight_rows(const elb_weight* w);
int64_t elb_weight_cols(const elb_weight* w);
size_t elb_weight_device_bytes(const elb_weight* w); /* bytes the decode path streams per matvec */

/* ---- operators (src/ops.h:11-29). Pointers named d_* are device pointers, the others host pointers. ---------- */

/* el::get_row (src/ops.h:20, src/ops.cpp:76-82) for `count` consecutive rows from row0, decoded on the device
 * with the reference's fp32 operation order (src/quant.cpp:7-60): out[count][n], bit-exact. */
int elb_get_rows(const elb_weight* w, int64_t row0, int64_t count, float* out);
int elb_get_rows_dev(const elb_weight* w, int64_t row0, int64_t count, float* d_out);

/* el::matvec (src/ops.h:23, src/ops.cpp:126-153): y[r] = sum_j W[r][j] * x[j]. Quantized types split x into
 * `nl` (3 or 4) exact int8 limbs (k_split8, src/cuda/model_cuda.cu:701-729) and accumulate quant x limb products
 * in int32; F16 weights use fp32 FMA. nl = 0 picks 4. */
int elb_matvec(const elb_weight* w, const float* x, float* y, int nl);
int elb_matvec_dev(const elb_weight* w, const float* d_x, float* d_y, int nl);

/* The same matvec for callers that must not allocate: a serving or real-time thread that cannot take the driver's
 * allocation lock, a host that has already given all device memory to a pool it does not control, or any code inside
 * a section where allocation is ruled out. No counterpart in the reference project (its backend allocates freely).
 * Pointers are device pointers. The call allocates and frees nothing (no cudaMalloc / cudaFree, no library
 * allocator): its working memory — the limb-split activation, split-K partial sums, arrival counters — is one static
 * array of about 208 KB that every GPU loading this library carries until the process exits.
 * Limits: row length n <= 16384, at most 262144 rows; larger weights are refused with ELB_ERR_UNSUPPORTED and a
 * message that names the limit. The first call on a device looks up the array's device address; make that first call
 * outside any stream capture. All calls share the array and leave their data in it: calls that overlap on the GPU
 * (several streams or threads) race — issue them one after another. Result: identical to elb_matvec_dev. */
int elb_matvec_static(const elb_weight* w, const float* d_x, float* d_y, int nl);

/* Y[b][rows] = X[b][n] * W^T for b tokens (linear() with B > 1, src/cuda/model_cuda.cu:1706-1780): limb split once,
 * then the int8 tensor-core GEMM over the digit planes (needs ELB_W_PLANES). */
int elb_matmul(const elb_weight* w, const float* x, int64_t b, float* y, int nl);
int elb_matmul_dev(const elb_weight* w, const float* d_x, int64_t b, float* d_y, int nl);

/* el::rmsnorm (src/ops.h:26, src/ops.cpp:155-160) over `rows` rows of length n (sum of squares in double). */
int elb_rmsnorm(float* out, const float* x, const float* w, int n, float eps, int rows);

/* k_split8 (src/cuda/model_cuda.cu:701-729): limbs[nl][b][n] int8, inv_scale[b] = 2^-k. */
int elb_split_limbs(int device, const float* x, int64_t b, int64_t n, int nl, int8_t* limbs, float* inv_scale);

/* Exact int32 sums the matvec forms, for parity checks (src/cuda/model_cuda.cu:943-1012):
 *   P[rows][n/sub][nl]  = sum over one sub-block (32 values; 16 for Q6_K) of limb * quant   (sub-block partials)
 *   I[rows][n/blk][nl]  = sum over the sub-blocks of a super-block of scale * P             (blk 256; 32 for Q8_0)
 *   J[rows][n/blk][nl]  = Q4_K only: sum of min * (sum of the limb over the sub-block); zero otherwise
 * Any of P, I, J may be NULL. Computed by the same device code path as elb_matvec. */
int elb_limb_sums(const elb_weight* w, const float* x, int nl, int32_t* P, int32_t* I, int32_t* J);
/* The same check for the multi-token kernel (k_gemm_tc of the reference forms these sums in mma.sync fragments,
 * src/cuda/model_cuda.cu:402-492; here they are tcgen05 accumulators in tensor memory): the int32 accumulator columns
 * of every (token, 256-block) as they leave tensor memory, A[b][n/256][nl + 1][rows]. With the weight w = sc * q written
 * as balanced digits w = w0 + 256 w1, column c holds sum(w0 * limb_c + w1 * limb_(c-1)), so that
 * sum over c of 256^c A[..][c][row] = sum over l of 256^l I[row][block][l] of elb_limb_sums, exactly.
 * Q4_K and Q6_K weights created with ELB_W_PLANES, b >= 2, nl = 3 or 4 (0 = 4); ELB_ERR_UNSUPPORTED otherwise. */
int elb_matmul_acc(const elb_weight* w, const float* x, int64_t b, int nl, int32_t* A);

/* ---- model (el::Backend, src/model.h:42-57) -------------------------------------------------------------------*/
typedef struct {
    int32_t n_layer, n_embd, n_ff, n_head, n_head_kv, head_dim, n_vocab, rope_dim; /* el::Config, src/model.h:17-23 */
    double rope_base;
    float eps;
    int32_t max_batch; /* prompt chunk length; 0 = 512 (make_cuda_backend, src/cuda/model_cuda.cu:1912) */
    int32_t n_seq;     /* sequences that share the model, each with its own n_ctx rows of KV cache; 0 = 1 (the reference
                          keeps one sequence per process) */
} elb_config;

/* tensor roles, in the order of el::ModelTensors / el::LayerTensors (src/model.h:25-36) */
enum {
    ELB_TOK_EMBD = 0, ELB_OUTPUT = 1, ELB_OUTPUT_NORM = 2, ELB_ATTN_NORM = 3, ELB_FFN_NORM = 4, ELB_Q_NORM = 5,
    ELB_K_NORM = 6, ELB_WQ = 7, ELB_WK = 8, ELB_WV = 9, ELB_WO = 10, ELB_GATE = 11, ELB_UP = 12, ELB_DOWN = 13
};

typedef struct elb_model elb_model;

/* CudaModel constructor (src/cuda/model_cuda.cu:1539-1635), split so that the caller streams tensors in:
 * create -> set_tensor for every tensor of el::ModelTensors (ELB_OUTPUT may be omitted: tied head,
 * src/model.cpp:73-74) -> finalize (allocates the fp32 KV cache for n_ctx positions and the scratch buffers,
 * builds the RoPE table from double-precision angles, checks device memory). head_dim must be 128. */
int elb_model_create(const elb_config* cfg, int n_ctx, int device, elb_model** out);
/* The library keeps `bytes` by reference until elb_model_finalize returns (the reference's loader hands out pointers
 * into its file mapping the same way, src/gguf.cpp): the caller must keep them valid until then, and may free them after. */
int elb_model_set_tensor(elb_model* m, int role, int layer, int ggml_type, int64_t rows, int64_t n, const void* bytes,
                         size_t nbytes);
int elb_model_finalize(elb_model* m);
void elb_model_destroy(elb_model* m);
/* The same constructor straight from a GGUF file (versions 2 and 3): what Gguf::open + read_config + read_tensors +
 * make_cuda_backend do together in the reference (src/gguf.cpp:204-258, src/model.cpp:38-103,
 * src/cuda/model_cuda.cu:1900-1913). The file is mapped, its metadata gives the configuration (same keys and
 * defaults), every tensor is handed over from the mapping and the model is finalized; the mapping is released before
 * the call returns. Rejected as in the reference: architectures other than qwen3, RoPE scaling, bias tensors,
 * key_length != value_length, tensor types other than F32 / F16 / Q8_0 / Q4_K / Q6_K. max_batch and n_seq as in
 * elb_config (0 = defaults). */
int elb_model_load_gguf(const char* path, int n_ctx, int device, int max_batch, int n_seq, elb_model** out);
/* The configuration a model was created with (n_vocab and the rest, e.g. after elb_model_load_gguf). */
int elb_model_config(const elb_model* m, elb_config* out);

/* Backend::eval (src/model.h:48-50; CudaModel::eval, src/cuda/model_cuda.cu:1648-1658): tokens[0..n) are processed
 * at positions pos0..pos0+n-1 and written to the KV cache (only rows [pos0, pos0+n) are touched); when logits is
 * not NULL the LAST token's n_vocab fp32 logits are written to that host buffer. Synchronous.
 * n <= 0 -> ELB_ERR_INVALID; pos0 < 0, pos0+n > n_ctx or a token outside [0, n_vocab) -> ELB_ERR_RANGE. */
int elb_model_eval(elb_model* m, const int32_t* tokens, int n, int pos0, float* logits);

/* elb_model_eval with the logits reduced on the device to what a sampler of the reference's kind needs
 * (src/main.cpp:309-320 computes this on the host from all n_vocab floats of every token): the log-sum-exp of the last
 * token's logits in double precision, and the k best tokens ordered by (logit descending, id ascending) with their
 * logits, so that logprob = top_logits[i] - *lse. 1 <= k <= 64. Only 8 + 8k bytes cross to the host. No counterpart in
 * the reference's backend interface. */
int elb_model_eval_top(elb_model* m, const int32_t* tokens, int n, int pos0, int k, int32_t* ids, float* top_logits,
                       double* lse);
/* The same with a token mask, for constrained decoding (the reference's matcher walks the host copy of the logits in rank
 * order until it finds an allowed token, src/main.cpp:232-246, src/constrain.h:51-56): bit i of allowed[(n_vocab+31)/32]
 * says whether token i may be picked; the k best ALLOWED tokens come back (ids -1 when fewer are allowed), the
 * log-sum-exp still covers the whole vocabulary, so top_logits[i] - *lse is the token's true log-probability. */
int elb_model_eval_top_masked(elb_model* m, const int32_t* tokens, int n, int pos0, int k, const uint32_t* allowed,
                              int32_t* ids, float* top_logits, double* lse);

/* Rows of several sequences in one pass (no counterpart in the reference, which serves one sequence at a time:
 * src/main.cpp:499-505 keeps a single `cached` prefix). Row i is token tokens[i] at position pos[i] of sequence seq[i]
 * (0 <= seq[i] < n_seq); the rows of one sequence must come in increasing, consecutive positions, continuing what that
 * sequence has cached, exactly as elb_model_eval requires of its tokens. Each row attends to positions 0..pos[i] of its
 * own sequence; only the KV rows (seq[i], pos[i]) are written. n <= max_batch. When logits is not NULL it receives one
 * row of n_vocab floats for every row i with want[i] != 0, in row order (want == NULL: every row); at most n_seq rows
 * may be wanted. A prompt goes in as rows of one sequence (want only the last), a batched decode step as one row per
 * sequence. elb_model_eval(tokens, n, pos0) is the same as rows (seq 0, pos0 + i) with only the last row wanted. */
int elb_model_eval_batch(elb_model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos,
                         const uint8_t* want, float* logits);
/* elb_model_eval_batch with every wanted row's logits reduced on the device as elb_model_eval_top reduces one row's
 * (the sampler of src/main.cpp:309-320 once per sequence): for wanted row r, in row order, ids[r * k .. r * k + k) and
 * top_logits[...] hold its k best tokens by (logit descending, id ascending) and lse[r] its log-sum-exp over the whole
 * vocabulary in double precision. A batched decode step of 64 sequences then returns 64 * (8 + 8 k) bytes to the host
 * instead of 64 * n_vocab floats (39 MB). 1 <= k <= 64. */
int elb_model_eval_batch_top(elb_model* m, int n, const int32_t* tokens, const int32_t* seq, const int32_t* pos,
                             const uint8_t* want, int k, int32_t* ids, float* top_logits, double* lse);

/* n single-token steps at positions pos0.., enqueued back to back without reading logits back (the tg loop of the
 * reference's bench command, src/main.cpp:639, without its per-token host round trip). device_ms receives the device
 * time of the whole run (CUDA events on the model's stream). Same argument checks as elb_model_eval. */
int elb_model_eval_steps(elb_model* m, const int32_t* tokens, int n, int pos0, float* device_ms);

/* Same step, measured: device time in milliseconds of the last elb_model_eval (CUDA events on the model's own
 * stream, host<->device copies excluded), and the number of this library's kernels that call launched. */
int elb_model_last_eval_stats(const elb_model* m, float* device_ms, int64_t* kernel_launches);
/* Residual stream of the last evaluated token, E floats (for layer-level parity checks). */
int elb_model_hidden(elb_model* m, float* out);
size_t elb_model_weight_bytes(const elb_model* m); /* bytes one decode step streams from the weight tensors */
size_t elb_model_kv_bytes_per_token(const elb_model* m);

/* ---- tensor parallelism over the GPUs of one box (one process per GPU). The reference is single-GPU; these calls have
 * no counterpart there. The cut keeps whole heads and whole SwiGLU elements on a rank: attn_q/k/v and ffn_gate/up by
 * rows, attn_output and ffn_down by columns (their partial sums are all-reduced over NCCL, one all-reduce per
 * attention block and one per MLP block), the head by rows (logits are all-gathered); norms and the token embedding
 * are replicated. tp_size must divide n_head and n_head_kv; n_ff is cut in multiples of 256, unevenly if need be.
 *
 * elb_tp_dims / elb_tp_shard_shape / elb_tp_shard_copy are host arithmetic and need no GPU: the share of rank
 * tp_rank in the heads, the FFN range [f0, f1), the vocabulary rows [v0, v1), and the cut of one tensor (role as in
 * elb_model_set_tensor) as shape, byte size and bytes. */
int elb_tp_dims(const elb_config* cfg, int tp_rank, int tp_size, int* n_head, int* n_head_kv, int64_t* f0, int64_t* f1,
                int64_t* v0, int64_t* v1);
int elb_tp_shard_shape(const elb_config* cfg, int tp_rank, int tp_size, int role, int ggml_type, int64_t rows, int64_t n,
                       int64_t* out_rows, int64_t* out_n, size_t* out_nbytes);
int elb_tp_shard_copy(const elb_config* cfg, int tp_rank, int tp_size, int role, int ggml_type, int64_t rows, int64_t n,
                      const void* bytes, size_t nbytes, void* out, size_t out_nbytes);
/* 128-byte NCCL id: rank 0 makes one and hands it to the other ranks by any means it has (a file, a socket,
 * torch.distributed); every rank passes it to elb_model_create_tp, which joins the communicator (collective call). */
int elb_tp_unique_id(void* id128);
/* Like elb_model_create for rank tp_rank of tp_size; cfg is the WHOLE model's configuration and elb_model_set_tensor
 * still receives the whole tensors: elb_model_finalize uploads only this rank's cut. elb_model_eval must then be
 * called by all ranks with the same arguments; every rank receives the full logits. */
int elb_model_create_tp(const elb_config* cfg, int n_ctx, int device, int tp_rank, int tp_size, const void* id128,
                        elb_model** out);
/* elb_model_load_gguf for one rank of a tensor-parallel group: every rank maps the same file and uploads its own cut
 * of each tensor (the per-rank slicing that upload_group / upload_lin, src/cuda/model_cuda.cu:1450-1528, would need for
 * a sharded model; the reference has no such path). Collective like elb_model_create_tp. */
int elb_model_load_gguf_tp(const char* path, int n_ctx, int device, int max_batch, int n_seq, int tp_rank, int tp_size,
                           const void* id128, elb_model** out);

/* ---- timing helpers for microbenchmarks: run the device-pointer matvec `iters` times over `n_w` weights in
 * rotation (so that the working set exceeds L2) and return the average device time per call in ms. */
int elb_bench_matvec(elb_weight* const* ws, int n_w, const float* d_x, float* d_y, int nl, int iters, float* avg_ms);
int elb_bench_matmul(elb_weight* const* ws, int n_w, const float* d_x, int64_t b, float* d_y, int nl, int iters,
                     float* avg_ms);

#ifdef __cplusplus
}
#endif
#endif /* ELB_H */
