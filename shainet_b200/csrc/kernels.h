// Internal launch interfaces of libshainet_attn's kernels (host side).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "common.cuh"

namespace shainet {

// One sequence's device KV cache, [num_kv_heads, capacity, head_dim] per tensor, and
// the number of positions held BEFORE the rows of this call.  Elements are fp32, or
// bfloat16 for a cache created in that format: the launch arguments then say so
// (kv_elem_bytes = 2) and the kernels reinterpret these pointers.
struct SeqDesc {
    float* k;
    float* v;
    int start;
    int capacity;
};

// A launch covers `batch` sequences of `T` new tokens each (rows = batch*T).
// batch == 1 passes its descriptor by value in `one`; batched decode passes a
// device array in `many` (T == 1).
struct SeqRef {
    SeqDesc one;
    const SeqDesc* many;
};

struct HeadShape {
    int num_heads;
    int num_kv_heads;
    int head_dim;
};

struct PrepArgs {
    const float* q;        // [rows, num_heads*head_dim]
    const float* k_new;    // [rows, num_kv_heads*head_dim]
    const float* v_new;
    const float* b_q;      // nullable biases (Qwen2)
    const float* b_k;
    const float* b_v;
    const float* q_norm;   // nullable per-head RMSNorm weights (Qwen3), [head_dim]
    const float* k_norm;
    const float* inv_freq; // [head_dim/2]
    double eps;
    float* q_rot;          // [rows, num_heads*head_dim]
    SeqRef seqs;
    int batch, T;
    HeadShape hs;
    int round_q_tf32;      // round the rotated q to nearest TF32 (it feeds the tensor-core prefill kernel)
    int kv_elem_bytes;     // 4: fp32 cache rows; 2: rows rounded to bfloat16 (nearest even) as they are appended
    AttnStatus* status;    // nullable: receives a bounded wait's failure
};

struct AttnArgs {
    const float* q_rot;    // rotated queries [rows, num_heads*head_dim]
    float* out;            // [rows, num_heads*head_dim]
    SeqRef seqs;
    int batch, T;
    HeadShape hs;
    float scale;
    // split-K only
    float* part_o;         // [rows, num_heads, max_splits, head_dim]
    float* part_ml;        // [rows, num_heads, max_splits, 2]
    int chunk_rows;        // cache rows per split (multiple of the warp tile)
    int max_splits;        // grid.x
    int prefill_one_cta;   // tensor-core prefill: never pair CTAs
    AttnStatus* status;
};

// Where the fused decode kernel also delivers its result when kv-head groups
// are spread over GPUs: every rank's exchange buffer (plain peer stores over
// NVLink, no multicast), at this rank's slot.
constexpr int MAX_PEERS = 16;
// Delivery of the merged head rows into every rank's exchange buffer.  Each float
// travels as one 8-byte word {value, epoch}: an aligned 8-byte store is indivisible,
// so the receiver needs no fence and no separate flag; it polls the words
// themselves and unpacks them.
struct GatherTarget {
    unsigned long long* peer_words[MAX_PEERS];  // word area of every rank's exchange buffer (this rank's own included)
    int world;
    long long out_offset;     // in floats (= words): this rank's block of head rows
    long long lse_offset;     // this rank's block of log-sum-exp values, or -1
    unsigned epoch;           // never 0
};

// One decode token per sequence, everything in one launch (T == 1).
struct FusedArgs {
    const float* q;        // [batch, num_heads*head_dim] raw projections
    const float* k_new;    // [batch, num_kv_heads*head_dim]
    const float* v_new;
    const float* b_q;
    const float* b_k;
    const float* b_v;
    const float* q_norm;
    const float* k_norm;
    const float* inv_freq;
    double eps;
    float* out;            // [batch, num_heads*head_dim]
    SeqRef seqs;
    int batch;
    HeadShape hs;
    float scale;
    float* part_o;         // [batch, num_heads, max_splits, head_dim]
    float* part_ml;        // [batch, num_heads, max_splits, 2]
    float* part2_o;        // [batch, num_heads, max_groups, head_dim]: merged groups of splits
    float* part2_ml;       // [batch, num_heads, max_groups, 2]
    unsigned* tickets;     // [batch*num_kv_heads] group-level + [batch*num_kv_heads*max_groups] split-level, zero between launches
    int chunk_rows;
    int max_splits;
    int max_groups;
    unsigned epoch;        // this launch's tag in the {value, epoch} partial words: never 0, never reused while old words exist
    int stream_merge;      // partials travel as {value, epoch} words and are folded by CTAs that poll them (single
                           // sequence, grid fully resident); part_o / part_ml then point at 8-byte words, not floats
    int unsafe_tail;       // newest cache rows a still-running previous grid may be writing
    int inputs_ready;      // caller vouches that q/k_new/v_new do not come from the previous grid
    int pos_delta;         // RoPE position of the new token minus the rows already cached (0 unless the sequence is split over ranks)
    int no_append;         // attend over the cached rows only: k_new/v_new are not used, nothing is appended
    int kv_elem_bytes;     // 4: fp32 cache; 2: bfloat16 cache (the new row is rounded before it is stored and attended to)
    GatherTarget gather;   // peer delivery of the merged result (world == 0: none)
    float* lse_out;        // nullable [batch, num_heads]: max + ln(sum) of every row's softmax, for merging partial results
    AttnStatus* status;
};

// Fused (bias +) per-head RMSNorm + RoPE for q and k, and the append of the
// rotated k rows and raw v rows into the cache.
cudaError_t launch_prep_append(const PrepArgs& a, cudaStream_t s);

// Any head_dim <= 256 (even), any group size, any T: one CTA per (head, row).
cudaError_t launch_attn_generic(const AttnArgs& a, cudaStream_t s);

// Split-K flash-decode for head_dim in {64,128} and group size in {1,2,4,8,16}.
bool splitk_supported(const HeadShape& hs);
int splitk_tile_rows(const HeadShape& hs, int kv_elem_bytes, bool batched);   // rows per warp tile: fp32 (4) or bfloat16 (2) caches, one sequence or a batch
int splitk_ctas_per_sm(const HeadShape& hs);
size_t splitk_scratch_floats(const HeadShape& hs, int rows, int max_splits);
int fused_merge_groups(int max_splits);
cudaError_t launch_attn_splitk(const AttnArgs& a, cudaStream_t s);
// Fused norm/RoPE/append + split-K decode + split merge, launched with
// programmatic stream serialization.
cudaError_t launch_decode_fused(const FusedArgs& a, cudaStream_t s);

// Causal prefill on the tcgen05 tensor cores (TF32): head_dim 64 or 128, one
// sequence, q already rotated, cache already appended.  Rows of the cache
// beyond the appended length must hold finite values (the caches are zeroed
// when allocated).
bool prefill_tc_supported(const HeadShape& hs);
cudaError_t launch_attn_prefill_tc(const AttnArgs& a, cudaStream_t s);

// Merge of attention results computed over disjoint parts of one sequence by
// different ranks: `gathered` holds, per rank, [heads_per_rank*head_dim] outputs
// followed by [heads_per_rank] log-sum-exp values; consecutive `seq_parts` ranks
// form one head group.  out_full is [groups*heads_per_rank*head_dim].
cudaError_t launch_merge_parts(const float* gathered, int world, int seq_parts, int heads_per_rank, int head_dim,
                               float* out_full, cudaStream_t s);

// Bounded wait for the words of all ranks' (row, log-sum-exp) pairs of one exchange slot, merged per head group.
cudaError_t launch_gather_merge(const unsigned long long* words, int world, int seq_parts, int heads_per_rank, int head_dim,
                                unsigned epoch, unsigned long long limit_ns, float* out_full, AttnStatus* status,
                                cudaStream_t s);
// Bounded wait until `count` exchange words carry `epoch`; unpacks them into `data`.
cudaError_t launch_gather_wait(const unsigned long long* words, float* data, long long count, unsigned epoch,
                               unsigned long long limit_ns, AttnStatus* status, cudaStream_t s);

// Standard-normal fill of `len` positions per kv head (benchmark caches); elem_bytes 2 stores
// the same values rounded to bfloat16.
cudaError_t launch_fill_normal(float* base, int num_kv_heads, int capacity, int head_dim, int len,
                               unsigned long long seed, int elem_bytes, cudaStream_t s);

// Rows [row0, row0 + rows) of every kv head copied between two caches of possibly different
// element sizes (4 = fp32, 2 = bfloat16; fp32 -> bfloat16 rounds to nearest even) and capacities.
cudaError_t launch_kv_convert(const void* src, int src_elem_bytes, int src_capacity, void* dst, int dst_elem_bytes,
                              int dst_capacity, int num_kv_heads, int head_dim, int row0, int rows, cudaStream_t s);

// y[M, N] = x[M, K] . dequant(q[N, K], scales[N, ceil(K/32)]) with optional fused pieces:
// gamma != null: x is RMS-normalised first (f64 sum and scaling, weight gamma[K], eps);
// q2 != null: SwiGLU, y[M, N] = silu(x . W) * (x . W2) with silu in f64 (q2/scales2 shaped like q/scales);
// bias != null: + bias[N]; residual != null: residual[M, N] + result; argmax != null: every
// row's word receives max over its finite outputs of (order-preserving key << 32 | ~index)
// by atomicMax (the words must be zero before the launch).
struct Q8GemvArgs {
    const float* x;
    const signed char* q;
    const float* scales;
    const signed char* q2;
    const float* scales2;
    float* y;
    const float* residual;
    const float* bias;
    const float* gamma;
    double eps;
    unsigned long long* argmax;
    int M, N, K;
};
bool q8_fast_path(int K);
cudaError_t launch_q8_gemv(const Q8GemvArgs& a, int sm_count, cudaStream_t s);
// x[t] = table[ids[t]] for `rows` tokens; also zeroes n_words arg-max words.
cudaError_t launch_embed_rows(const int* ids_dev, const float* table, float* x, int rows, int d_model, int vocab,
                              unsigned long long* argmax_words, int n_words, cudaStream_t s);
// tokens[m] = index held by arg-max word m; the last one also goes to *next_id and history[history_pos] when given.
cudaError_t launch_argmax_decode(const unsigned long long* words, int* tokens, int n, int* next_id, int* history,
                                 int history_pos, cudaStream_t s);

// Sets the calling thread's message for shainet_attn_last_error().
void set_last_error_message(const char* msg);

// Drop-in bodies for the reference's two exported kernels.
cudaError_t launch_ref_append(const float* staging, float* kc, float* vc, int new_tokens, int start_pos,
                              int num_kv_heads, int head_dim, int capacity, cudaStream_t s);

}  // namespace shainet
