// Parameters of the persistent decode kernel (decode.cu), filled by the model (model.cu).
#pragma once

#include "common.cuh"

namespace elb {

// Everything the kernel needs to know about the step's matrices travels in its parameter block (constant memory, no
// pointer chasing through global memory on the way to a weight): the shape of each KIND of matrix, which is the same in
// every layer, and per layer only the base pointer and block format of each of its matrices.
constexpr int DK_MAX_LAYERS = 96;  // layers a model may have to run on this kernel
constexpr int DK_KINDS = 7;        // 0..2 qkv segment, 3 attn_output, 4 gate|up, 5 ffn_down, 6 head
constexpr int DK_LAYER_MATS = 6;   // matrices of a layer in execution order: n_qkv segments, attn_output, gate|up, ffn_down

struct DkKind {  // one kind of weight matrix, in tiled layout
    int tiles, upt, rows, n;
    // How the CTAs share the matrix. group_tiles / group_off: the matrix is tiles [group_off, group_off + tiles) of a
    // group of matrices that run in one phase (q, k, v) and the CTAs cut the group's tiles, whole tiles each.
    // balanced: the CTAs cut the (tile, k block) units into equal ranges instead; a tile then has up to two
    // contributors, which leave their partial sums in two buffers for the consumer to add (wo, down).
    int group_tiles, group_off, balanced, pad;
    // The matrices of a group may differ in block format and so in the time a tile takes (a Q6_K unit costs 1.66 Q4_K
    // units): the CTAs cut the group by cost, not by tile count. cost: of one tile of this matrix; group_cost_off: cost
    // of the group's matrices before this one; group_cost: of the whole group (0: cut by tiles).
    int cost, group_cost_off, group_cost, pad2;
};

struct DkParams {
    DkKind kind[DK_KINDS];
    const uint8_t* W[DK_MAX_LAYERS + 1][DK_LAYER_MATS];  // [layer][matrix in execution order]; [n_layer][0] is the head
    uint8_t wtype[DK_MAX_LAYERS + 1][8];                 // their block formats (ggml type ids)
    int n_layer, n_qkv;     // every layer has the same number of qkv segments
    int qkv_col[3];         // first output column of each qkv segment
    const float* norms;     // per layer norm_stride floats: attn_norm [E], ffn_norm [E], q_norm [128], k_norm [128]
    int norm_stride;
    float *kc, *vc;         // KV cache of layer 0 (sequence 0) [n_ctx][KD]; layer l lies l * kv_stride floats further
    size_t kv_stride;
    const float* output_norm;
    const uint8_t* embd;    // token embedding table, tiled layout
    int embd_type;
    int E, F, H, HKV, rope_dim, n_ctx, nsplit;
    float eps, scale;
    int nl_qkv, nl_wo, nl_gu, nl_down;
    const int32_t* token;   // device arrays: token id and position of step i of the running batch of steps
    const int* pos;
    unsigned* ctl;          // [0] index of the step to run, [1] non-zero: the kernel moves the index on when it ends,
                            // [2] launches so far (barrier targets and the parity of the amax slots derive from it)
    const float* rope;      // [n_ctx][rope_dim/2][2]
    float *x, *qkv, *att, *act, *logits;
    int8_t* gact;           // limbs + sub-block sums of the FFN activation in global memory, used when they do not fit in
    int act_global;         // shared memory next to the rings (long n_ff): then set, and ffn_down reads them through L2
    float* xbuf;            // [2][E] residual stream, alternating: a conversion reads one and writes the other
    // Partial sums of the row-parallel matvecs (attn_output, ffn_down), added by the next conversion. Two sets, used in
    // turn by successive exchanges; a set holds, for every tensor-parallel rank, two vectors of E floats (the two
    // contributors a row tile can have on that rank). part_peer[q] is rank q's copy as mapped into this process (peer
    // memory; part_peer[tp_rank] is the local one): every rank stores its partial sums into its slot on ALL ranks, and
    // after the exchange barrier every rank adds the same 2 * tp_size vectors in the same order.
    int tp_rank, tp_size;   // 1 rank: a single GPU, the exchange barrier is the grid barrier
    int pv;                 // vectors per rank in a set: 2 (a row tile can have two contributing CTAs) or 1 (whole tiles per CTA)
    float* part_peer[8];    // [2 sets][tp_size][pv][E]
    unsigned* flag_peer[8]; // rank q's arrival flags [2 sets][8 ranks]
    float* logits_peer[8];  // rank q's logits [n_vocab padded]: every rank stores its vocabulary rows on all ranks
    int v0;                 // first vocabulary row of this rank
    unsigned* xctl;         // local words: [0] exchanges so far, [1] release word of the exchange barrier
    unsigned* amax;         // [2][n_layer][2] bit patterns of max|att|, max|act| of each layer; launch e uses half e & 1
                            // (zero when it starts) and zeroes the other half for launch e + 1
    float* attn_part;       // [HKV][nsplit][group][130]
    unsigned* attn_counters;  // [HKV]
    unsigned* bar;          // grid barrier counter: counts arrivals for ever (compared modulo 2^32)
    int* err;               // raised when a barrier wait ran out
    int slots;              // row-tile slots per warp in the reduction buffer
    int cta_tiles;          // most row tiles a CTA's share of a matrix can touch
    int n_max;              // longest activation vector
    unsigned long long* prof;  // diagnostics (ELB_DK_PROF=1): [n_layer][32] nanosecond stamps of CTA 0, else null
    unsigned long long* prof_cta;  // diagnostics: [CTAs][16] stamps of every CTA at the barriers of layer prof_layer (arrival, release)
    int prof_layer;
};

// one token at the position / token id stored on the device (step ctl[0] of the arrays); nothing to reset between launches.
// ring_bytes: size of one warp's ring of weight units in shared memory (decode_ring_bytes); grid: one CTA per SM.
int decode_step_launch(const DkParams& p, int ring_bytes, int grid, cudaStream_t s);
int decode_step_fits(const DkParams& p, int ring_bytes, int device, bool* fits);
size_t decode_smem_bytes(const DkParams& p, int ring_bytes);
int decode_ring_bytes(const DkParams& p, int max_unit, int min_unit, int device);
int decode_threads();
int decode_warps();
int decode_max_split();    // most key splits of one KV head
int decode_part_stride();  // floats per (key split, head) of attn_part
size_t decode_act_bytes(int n);  // bytes of a split activation of n values (limbs, sub-block sums, block scales)

}  // namespace elb
