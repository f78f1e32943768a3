/* libshainet_attn — C ABI of the B200 (sm_100a) attention path for SHAInet's
 * LLaMA/Qwen decoder block: (bias +) per-head RMSNorm + RoPE + KV-cache append +
 * grouped-query causal attention over the cache, for prefill and decode.
 *
 * Plain C, plain pointers and sizes.  Every function returns an int status
 * (0 = ok, negative = error, see SHAINET_ATTN_E_*) and never prints or aborts;
 * shainet_attn_last_error() gives the message of the calling thread's last
 * failure.  File:line citations name the reference code each entry replaces
 * (paths inside the SHAInet project).
 *
 * Threading: a context and the caches created from it are used by one host
 * thread at a time (the contract of the reference's mutex-serialised Network).
 * Streams: the *_dev entries enqueue on the stream they are given and return at
 * once.  Calls that read or replace what those kernels use - kv_export, kv_import,
 * kv_set_rope*, kv_set_qk_norm, kv_set_bias, kv_fill_normal, ctx_sync - synchronise
 * only the context's own stream: a caller that launched on a stream of its own
 * synchronises that stream first (ctx_sync also reports a kernel-side wait failure
 * only once the stream that ran the kernel has been synchronised).
 * There is no CPU fallback: without a CUDA device every call fails.
 */
#ifndef SHAINET_ATTN_H
#define SHAINET_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SHAINET_ATTN_VERSION 101

#define SHAINET_ATTN_OK 0
#define SHAINET_ATTN_E_INVALID (-1)      /* bad argument / shape / null pointer / misaligned pointer */
#define SHAINET_ATTN_E_CUDA (-2)         /* a CUDA runtime call failed */
#define SHAINET_ATTN_E_NOMEM (-3)        /* device or pinned allocation failed */
#define SHAINET_ATTN_E_UNSUPPORTED (-4)  /* shape outside what the kernels cover */
#define SHAINET_ATTN_E_DEVICE_WAIT (-5)  /* a kernel gave up on a bounded wait */
#define SHAINET_ATTN_E_STATE (-6)        /* call sequence error (e.g. import past capacity) */

/* forward flags */
#define SHAINET_ATTN_F_GENERIC 1u  /* force the shape-agnostic kernel */
#define SHAINET_ATTN_F_SPLITK 2u   /* force the split-K decode kernel (error if unsupported) */
#define SHAINET_ATTN_F_TENSOR 4u   /* force the tcgen05 prefill kernel (error if unsupported) */
#define SHAINET_ATTN_F_UNFUSED 8u  /* decode as three launches (RoPE/append, split-K, merge) instead of one */
/* The caller vouches that q/k_new/v_new (device-pointer entries only) were
 * complete before the kernel launched immediately before this call on the same
 * stream began, i.e. they are not that kernel's output.  The fused decode
 * kernel then starts its RoPE/norm prologue and its streaming while that
 * kernel is still draining, and only waits for it before touching the scratch
 * the two share.  Without the flag nothing is assumed. */
#define SHAINET_ATTN_F_INPUTS_READY 16u   /* ignored for the first launch after kv_truncate / kv_reset: the rows it
                                             rewrites may still be read by the launch ahead of it */
/* Merge the split partials of the fused decode kernel with "last finisher"
 * tickets even where the flag-polling merge would be chosen (testing). */
#define SHAINET_ATTN_F_TICKET_MERGE 32u
/* Tensor-core prefill with one CTA per two query tiles even where a pair of CTAs (cluster of two, cta_group::2)
 * would be chosen, i.e. at head_dim 128 with an even group size (measurement and testing; the pair is the faster one). */
#define SHAINET_ATTN_F_TENSOR_1CTA 64u

typedef struct shainet_attn_ctx shainet_attn_ctx;
typedef struct shainet_attn_kv shainet_attn_kv;

/* ---- probing: replaces CUDA.fully_available? in LlamaBlock#gpu_attention?
 * (src/shainet/transformer/llama_block.cr:484-492, src/shainet/cuda.cr:778-780). */
int shainet_attn_version(void);
int shainet_attn_device_count(void);
const char* shainet_attn_last_error(void);

/* ---- context: owns the stream used by the host-pointer entry, the rotated-q
 * buffer, the split-K partials, pinned staging and the device status word.
 * Replaces the class-level @@gpu_staging/@@gpu_attn_out/@@gpu_attn_ws/
 * @@staging_host scratch (src/shainet/transformer/llama_block.cr:57-68, 421-429). */
int shainet_attn_ctx_create(shainet_attn_ctx** out, int device);
int shainet_attn_ctx_destroy(shainet_attn_ctx* ctx);
/* Waits for the context's stream and reports a kernel-side bounded-wait failure. */
int shainet_attn_ctx_sync(shainet_attn_ctx* ctx);
/* Bytes of device memory the context's scratch currently holds. */
size_t shainet_attn_ctx_scratch_bytes(shainet_attn_ctx* ctx);
/* Kernel timing for roofline reports: while enabled, every forward call
 * brackets its attention kernel(s) (not the RoPE/append kernel) with CUDA
 * events on the launching stream.  _read waits for them, returns the summed
 * device time and the number of bracketed launches since _enable(1), and
 * clears the record.  The reference only has wall-clock prints
 * (examples/prof.cr:19-37). */
int shainet_attn_ctx_timing_enable(shainet_attn_ctx* ctx, int enable);
int shainet_attn_ctx_timing_read(shainet_attn_ctx* ctx, double* total_ms, int* launches);

/* ---- KV cache of one block: two device buffers [num_kv_heads, capacity,
 * head_dim] fp32 (the layout of src/shainet/native/cuda_kernels.cu:689-694),
 * grown x2 (min 256) device-to-device.  Replaces @k_cache/@v_cache/@cache_len,
 * the device mirror and ensure_gpu_cache! (llama_block.cr:45-56, 497-520),
 * clear_cache! (:116-122) and finalize (:124-130).  num_heads/num_kv_heads are
 * the heads THIS cache serves (a rank's slice when kv-head groups are sharded).
 * RoPE defaults to theta = 10000 as LlamaBlock.new does (:74). */
int shainet_attn_kv_create(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                           int head_dim, int initial_capacity);
/* Element format of the cache rows.  The reference keeps fp32 rows only
 * (Array(Array(Float32)), llama_block.cr:45-48; float buffers, :50-56), so F32 is what
 * shainet_attn_kv_create makes and what every parity statement about the reference
 * refers to.  BF16 has no counterpart in the reference: it is an opt-in that halves the
 * bytes a decode step streams.  With it the rotated k row and the v row of every new
 * token are rounded to bfloat16 (round to nearest, ties to even) as they are appended,
 * and attention - still fp32 arithmetic, fp32 q, fp32 output - runs over the rounded
 * rows, the new token's own row included.  The result is therefore what the F32 path
 * gives on a cache whose rows were rounded that way, not what the reference gives on
 * unrounded rows.  Every entry that takes a cache accepts either format (single-token
 * decode and batched decode read bfloat16 directly; the other kernels read an fp32 image
 * of the rows that the context keeps as scratch) except shainet_attn_kv_device_ptrs
 * and batched decode with a kernel-forcing flag, which answer
 * SHAINET_ATTN_E_UNSUPPORTED.  kv_export widens exactly; kv_import and kv_fill_normal round. */
#define SHAINET_ATTN_KV_F32 0
#define SHAINET_ATTN_KV_BF16 1
int shainet_attn_kv_create_fmt(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                               int head_dim, int initial_capacity, int format);
int shainet_attn_kv_format(const shainet_attn_kv* kv);       /* SHAINET_ATTN_KV_*, or negative status */
/* A cache that grows without moving (no counterpart in the reference, whose ensure_gpu_cache!, llama_block.cr:497-520,
 * allocates max(256, need, 2 x old) rows and uploads the whole cache again).  Device ADDRESSES for max_capacity rows
 * per kv head (rounded up so that a kv head's range is a whole number of pages) are reserved at creation; physical
 * memory is mapped behind them, page by page (the driver's granularity, 2 MB), as rows are appended, reserved or
 * imported.  Growth therefore copies nothing and invalidates nothing: kv_device_ptrs stay valid for the cache's life,
 * kv_capacity is the reserved row count from the start, and memory in use follows the length, not a doubling policy.
 * Every entry accepts such a cache (to the kernels it is an ordinary cache of that capacity); appending past
 * max_capacity answers SHAINET_ATTN_E_INVALID, a driver without virtual memory management SHAINET_ATTN_E_UNSUPPORTED. */
int shainet_attn_kv_create_reserved(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                                    int head_dim, int max_capacity, int format);
int shainet_attn_kv_destroy(shainet_attn_kv* kv);
int shainet_attn_kv_reset(shainet_attn_kv* kv);              /* clear_cache!: length 0, buffers kept */
int shainet_attn_kv_len(const shainet_attn_kv* kv);          /* @cache_len, or negative status */
int shainet_attn_kv_capacity(const shainet_attn_kv* kv);     /* @gpu_cache_cap */
int shainet_attn_kv_reserve(shainet_attn_kv* kv, int total_len);
/* Drops the newest positions: the length becomes len (<= current length).
 * clear_cache! (llama_block.cr:116-122) is the len = 0 case; a partial
 * roll-back lets a caller replay or discard speculative rows. */
int shainet_attn_kv_truncate(shainet_attn_kv* kv, int len);

/* inv_freq(i) = f32(1 / theta^(2i/head_dim)) computed in double on the host
 * exactly as llama_block.cr:669-675 does. */
int shainet_attn_kv_set_rope_theta(shainet_attn_kv* kv, double theta);
/* Explicit table of head_dim/2 inverse frequencies (LlamaBlock#rope_freqs,
 * llama_block.cr:25-28; LLaMA-3 scaling from hf_loader.cr:235-265). */
int shainet_attn_kv_set_rope(shainet_attn_kv* kv, const float* inv_freq_host, int half);
/* Qwen3 per-head RMSNorm weights (head_dim floats each, either may be NULL)
 * and its epsilon (LlamaBlock#q_norm/#k_norm, llama_block.cr:19-23, 615-641). */
int shainet_attn_kv_set_qk_norm(shainet_attn_kv* kv, const float* q_weight_host, const float* k_weight_host,
                                double eps);
/* Qwen2 projection biases, sizes num_heads*head_dim, num_kv_heads*head_dim x2;
 * any may be NULL (LlamaBlock#b_q/#b_k/#b_v, llama_block.cr:35-43, 585-601). */
int shainet_attn_kv_set_bias(shainet_attn_kv* kv, const float* b_q_host, const float* b_k_host,
                             const float* b_v_host);

/* Cache contents to/from host arrays laid out [num_kv_heads, len, head_dim]
 * (K rows are stored rotated, as the reference stores them).  Import sets the
 * length to len. */
int shainet_attn_kv_export(shainet_attn_kv* kv, float* k_host, float* v_host, int len);
int shainet_attn_kv_import(shainet_attn_kv* kv, const float* k_host, const float* v_host, int len);
/* Fills len positions of K and V with N(0,1) values generated on the device
 * from seed and sets the length (synthetic long contexts for benchmarks). */
int shainet_attn_kv_fill_normal(shainet_attn_kv* kv, int len, uint64_t seed);
/* Raw device pointers of the current buffers (invalidated by growth); F32 caches only. */
int shainet_attn_kv_device_ptrs(shainet_attn_kv* kv, float** k_dev, float** v_dev);

/* ---- the drop-in for attention_heads_gpu (llama_block.cr:407-479) and the
 * host K-RoPE/append loop before it (:266-286): q [new_tokens, num_heads*head_dim],
 * k_new/v_new [new_tokens, num_kv_heads*head_dim] are the projection outputs on
 * the host, NOT yet biased, normalised or rotated; out [new_tokens,
 * num_heads*head_dim] receives the attention output (input of o_proj).
 * Positions start at the cache's current length, which grows by new_tokens.
 * scale is LlamaBlock's f32(1/sqrt(head_dim)) (:249).  Blocking. */
int shainet_attn_forward_host(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                              const float* v_new, float* out, int new_tokens, float scale, unsigned flags);

/* Same with device pointers (16-byte aligned) on a caller stream (a
 * cudaStream_t passed as void*; NULL = the context's own stream, so the legacy
 * default stream has to be named as cudaStreamLegacy).  Asynchronous. */
int shainet_attn_forward_dev(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q_dev, const float* k_new_dev,
                             const float* v_new_dev, float* out_dev, int new_tokens, float scale, unsigned flags,
                             void* stream);

/* ---- one sequence split over several GPUs.  The reference is single-device
 * (no cudaSetDevice, no collective anywhere in src/); these three entries serve
 * the partition "kv-head groups over ranks, and positions round-robin over the
 * ranks of a group when there are more ranks than kv heads".
 *
 * forward_dev_at: one decode token whose RoPE position is `position` (>= the
 * rows this rank's cache holds).  append != 0: this rank stores the token's k/v
 * row and attends over its rows including it; append == 0: it only attends over
 * the rows it already holds (k_new/v_new may be NULL).  Fused decode kernel only.
 * set_lse_out: while non-NULL, every fused decode call also writes max + ln(sum)
 * of each (sequence, head) softmax to lse_dev[batch*num_heads].
 * merge_parts: gathered_dev holds, per rank, heads_per_rank*head_dim outputs then
 * heads_per_rank log-sum-exp values; every `seq_parts` consecutive ranks form a
 * head group whose results are merged into out_full_dev
 * [world/seq_parts * heads_per_rank * head_dim]. */
int shainet_attn_forward_dev_at(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q_dev, const float* k_new_dev,
                                const float* v_new_dev, float* out_dev, int position, int append, float scale,
                                unsigned flags, void* stream);
int shainet_attn_ctx_set_lse_out(shainet_attn_ctx* ctx, float* lse_dev);
int shainet_attn_merge_parts(shainet_attn_ctx* ctx, const float* gathered_dev, int world, int seq_parts,
                             int heads_per_rank, int head_dim, float* out_full_dev, void* stream);

/* ---- exchange of head outputs between the GPUs of one box, fused into the
 * decode kernel (no counterpart in the reference, which is single-device).
 * Every rank owns one exchange buffer of data_floats floats (the same number on
 * every rank) followed by as many 8-byte {value, epoch} words.  comm_create
 * allocates it and returns an inter-process handle (SHAINET_ATTN_COMM_HANDLE_BYTES
 * bytes) that the host code passes around by whatever means it has; comm_open
 * maps the other ranks' buffers (handles: world consecutive handles in rank
 * order).  comm_set_target arms the NEXT fused decode call: the CTAs that merge
 * its split partials store every head row (and, if lse_offset_floats >= 0,
 * every head's log-sum-exp) into the word areas of ALL ranks at the given
 * offsets, each float as one indivisible 8-byte store {value, epoch} over NVLink
 * (no multicast, no copy engine, no fence, no flag).  comm_wait enqueues a kernel
 * that polls the words [offset, offset + count) of this rank's buffer until each
 * carries `epoch` (bounded, ~1 s, then SHAINET_ATTN_E_DEVICE_WAIT at the next
 * sync) and writes the values to the float area, where comm_data_ptr / comm_read
 * and merge_parts find them.  Epochs are non-zero and differ between successive
 * uses of a word; a word may be rewritten once its owner's stream has passed the
 * wait that unpacked it. */
#define SHAINET_ATTN_COMM_HANDLE_BYTES 64
int shainet_attn_comm_create(shainet_attn_ctx* ctx, size_t data_floats, void* handle_out);
int shainet_attn_comm_open(shainet_attn_ctx* ctx, const void* handles, int world, int rank);
int shainet_attn_comm_set_target(shainet_attn_ctx* ctx, long long out_offset_floats, long long lse_offset_floats, unsigned epoch);
int shainet_attn_comm_wait(shainet_attn_ctx* ctx, long long offset_floats, long long count_floats, unsigned epoch, void* stream);
/* comm_set_target + forward_dev_at + comm_wait in one call (one decode token of one
 * layer on a rank of a sharded model): the host cost of a layer is one foreign call. */
int shainet_attn_forward_dev_exchange(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                                      const float* v_new, float* out, int position, int append, float scale, unsigned flags,
                                      long long out_offset_floats, long long lse_offset_floats, long long wait_offset_floats,
                                      long long wait_count_floats, unsigned epoch, void* stream);
/* The same for a sequence that is split over the ranks of a head group (more ranks than
 * kv heads): every rank delivers its head rows and log-sum-exp values into the slot
 * [slot_offset, slot_offset + world * heads * (head_dim + 1)) of every rank, laid out
 * [rank][heads * head_dim rows | heads log-sum-exp]; one kernel then waits for the words
 * of all ranks and merges the seq_parts ranks of each head group straight into
 * out_full_dev [world / seq_parts * heads * head_dim] (what merge_parts would produce). */
int shainet_attn_forward_dev_exchange_merge(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                                            const float* v_new, float* out, int position, int append, float scale,
                                            unsigned flags, long long slot_offset_floats, int seq_parts, unsigned epoch,
                                            float* out_full_dev, void* stream);
/* How long comm_wait and forward_dev_exchange[_merge] let their kernel poll for the
 * other ranks' words before giving up (default 1000 ms).  The poll starts when the
 * waiting kernel starts, so the limit has to cover how late the slowest rank's host
 * thread may be with the matching call (a first-call set-up, paging, a garbage
 * collection pause in the host language) plus its kernel's run time.  A rank that is
 * later than this makes every other rank's next sync return
 * SHAINET_ATTN_E_DEVICE_WAIT; their contexts stay usable, but the token's exchanged
 * rows are incomplete and the step has to be redone (roll the caches back with
 * kv_truncate and call again with a fresh epoch).  Waits between the CTAs of one
 * kernel on one GPU are not affected (fixed, ~1 s). */
int shainet_attn_comm_set_wait_limit_ms(shainet_attn_ctx* ctx, int milliseconds);
/* Asynchronous copy of a range of this rank's float area to host memory. */
int shainet_attn_comm_read(shainet_attn_ctx* ctx, long long offset_floats, float* host_dst, size_t floats, void* stream);
int shainet_attn_comm_data_ptr(shainet_attn_ctx* ctx, float** data_dev);

/* One decode token for each of `batch` sequences in lock step, one launch:
 * q [batch, q_dim], k_new/v_new [batch, kv_dim], out [batch, q_dim] on the
 * device.  All caches share one head shape, RoPE table and norm weights (those
 * of kvs[0]).  The reference has no batched entry (Network#run is batch 1,
 * src/shainet/basic/network_run.cr:294-315); this serves ragged batched decode. */
int shainet_attn_forward_batched_dev(shainet_attn_ctx* ctx, shainet_attn_kv* const* kvs, int batch,
                                     const float* q_dev, const float* k_new_dev, const float* v_new_dev,
                                     float* out_dev, float scale, unsigned flags, void* stream);

/* ---- symbol-compatible replacements for the two kernels the reference loads
 * with dlsym from libshainet_cuda_kernels.so (src/shainet/cuda.cr:838-891;
 * definitions src/shainet/native/cuda_kernels.cu:713-726 and :808-825).  Same
 * names, argument order and meaning: device pointers, legacy default stream,
 * q already rotated, ws a scratch of num_heads*new_tokens*(start_pos+new_tokens)
 * floats.  Errors are printed like the reference does. */
void kv_cache_append_f32(const float* staging, float* kc, float* vc, int new_tokens, int start_pos,
                         int num_kv_heads, int head_dim, int capacity);
void attention_kv_f32(const float* q, const float* kc, const float* vc, float* out, float* ws, int new_tokens,
                      int start_pos, int num_heads, int heads_per_kv, int head_dim, int capacity, float scale);

/* ---- Q8_0 weights and the decode step around attention, resident on the device.
 *
 * A Q8_0 weight is the reference's QuantizedCudaMatrix
 * (src/shainet/math/quantized_cuda_matrix.cr:8-153): int8 values q[N][K] (output-major)
 * and one fp32 scale per 32 consecutive K of an output, scales[N][ceil(K/32)], for a
 * weight that maps K inputs to N outputs.  q8_create quantises a host fp32 matrix
 * [K, N] (input-major, the layout the reference's loader produces) exactly as
 * from_simple does (:74-115); q8_create_raw uploads already quantised host arrays;
 * q8_wrap adopts device arrays the caller owns (the q_ptr / scale_ptr of an existing
 * QuantizedCudaMatrix) without copying.  q8_gemv_dev is gemv_into (:143-153):
 * y[M, N] = x[M, K] . dequant(W) on device pointers.  gemm_q8_f32 is the
 * symbol-compatible replacement for the kernel wrapper the reference loads with dlsym
 * (src/shainet/native/cuda_kernels.cu:616-629; src/shainet/cuda.cr gemm_q8_f32):
 * device pointers, legacy default stream, errors printed. */
typedef struct shainet_attn_q8 shainet_attn_q8;
int shainet_attn_q8_create(shainet_attn_ctx* ctx, shainet_attn_q8** out, const float* w_host, int K, int N);
int shainet_attn_q8_create_raw(shainet_attn_ctx* ctx, shainet_attn_q8** out, const signed char* q_host,
                               const float* scales_host, int K, int N);
int shainet_attn_q8_wrap(shainet_attn_ctx* ctx, shainet_attn_q8** out, const signed char* q_dev, const float* scales_dev,
                         int K, int N);
int shainet_attn_q8_destroy(shainet_attn_q8* w);
int shainet_attn_q8_export(const shainet_attn_q8* w, signed char* q_host, float* scales_host);
int shainet_attn_q8_gemv_dev(shainet_attn_ctx* ctx, const shainet_attn_q8* w, const float* x_dev, float* y_dev, int M,
                             void* stream);
void gemm_q8_f32(const float* x, const signed char* q, const float* scales, float* y, int M, int N, int K);

/* One decoder block with every step on the device: LlamaBlock#forward_cached
 * (src/shainet/transformer/llama_block.cr:189-196) = norm1 (RMSNorm,
 * src/shainet/transformer/rms_norm.cr:18-37) -> q/k/v projections (:253-255, 726-768)
 * -> the attention of this library on `kv` -> o_proj (:298) -> residual -> norm2 ->
 * SwiGLU FFN (src/shainet/transformer/swiglu_ff.cr:76-91) -> residual.  x and out are
 * [new_tokens, d_model].  The block borrows kv and the weights (they must outlive it)
 * and keeps its own stacked copy of the q/k/v weights so that one launch serves all
 * three.  norm2/gate/up/down may all be NULL: the block then ends after the first
 * residual (models whose FFN stays with the caller, e.g. mixture-of-experts layers).
 * eps is the RMSNorm epsilon (LlamaBlock.new's eps, :76).  forward_host makes one
 * host-to-device copy (x) and one device-to-host copy (the block output) per call
 * where the reference makes sixteen; forward_dev makes none. */
typedef struct shainet_attn_block shainet_attn_block;
int shainet_attn_block_create(shainet_attn_ctx* ctx, shainet_attn_block** out, shainet_attn_kv* kv, int d_model,
                              const float* norm1_host, const shainet_attn_q8* wq, const shainet_attn_q8* wk,
                              const shainet_attn_q8* wv, const shainet_attn_q8* wo, const float* norm2_host,
                              const shainet_attn_q8* gate, const shainet_attn_q8* up, const shainet_attn_q8* down,
                              double eps);
int shainet_attn_block_destroy(shainet_attn_block* block);
int shainet_attn_block_forward_dev(shainet_attn_ctx* ctx, shainet_attn_block* block, const float* x_dev, float* out_dev,
                                   int new_tokens, void* stream);
int shainet_attn_block_forward_host(shainet_attn_ctx* ctx, shainet_attn_block* block, const float* x, float* out,
                                    int new_tokens);

/* The token loop: Network#run(Array(Int32)) with use_kv_cache
 * (src/shainet/basic/network_run.cr:185-264, 294-315) = embedding gather
 * (src/shainet/text/embedding_layer.cr:129-156) -> blocks -> final RMSNorm (:210-212)
 * -> Q8_0 lm_head on the last row (:1465-1487) -> bias (:222-226), and
 * Sampler.greedy (src/shainet/text/sampler.cr:38-53: first index of the largest finite
 * logit, 0 if none).  embedding_host is [vocab, d_model] fp32; final_norm_host and
 * lm_bias_host may be NULL.  decoder_run takes n_tokens ids (a prompt, or one token),
 * appends them to every block's cache and returns the last row's logits [vocab]
 * and/or its greedy token (either pointer may be NULL); it is blocking.
 * decoder_generate runs the prompt and then steps - 1 further tokens, each step
 * embedding the previous step's arg-max straight from device memory, and returns
 * the `steps` greedy tokens with one copy at the end: no token, logit or activation
 * visits the host in between. */
typedef struct shainet_attn_decoder shainet_attn_decoder;
int shainet_attn_decoder_create(shainet_attn_ctx* ctx, shainet_attn_decoder** out, shainet_attn_block* const* blocks,
                                int n_layers, const float* embedding_host, int vocab, const float* final_norm_host,
                                const shainet_attn_q8* lm_head, const float* lm_bias_host, double eps);
int shainet_attn_decoder_destroy(shainet_attn_decoder* dec);
int shainet_attn_decoder_run(shainet_attn_ctx* ctx, shainet_attn_decoder* dec, const int32_t* token_ids, int n_tokens,
                             float* logits_host, int32_t* next_token_host);
int shainet_attn_decoder_generate(shainet_attn_ctx* ctx, shainet_attn_decoder* dec, const int32_t* prompt_ids, int n_prompt,
                                  int steps, int32_t* tokens_host);

/* ---- decode without allocating.  This entry has no counterpart in the
 * reference.  It is for hosts that cannot let a library allocate device memory:
 * a server that gave the GPU's whole memory budget to its own pool at start-up
 * (a cudaMalloc made later from inside a library may fail or upset that plan),
 * or a latency-critical token loop where cudaMalloc/cudaFree are unwelcome
 * because they synchronise the whole device.  It computes what
 * attention_kv_f32 computes for new_tokens == 1 - q [num_heads*head_dim] already
 * rotated, the new K/V row already appended at start_pos, visible rows
 * 0..start_pos - on the caller's stream, and returns a status code.  Its split
 * partials live in a fixed 4 MiB array inside the library image (held by every GPU that loads the library, until exit)
 * instead of a buffer grown on demand; it calls no cudaMalloc, cudaFree or
 * allocating library routine.  Limits: head_dim 64 or 128; 1/2/4/8/16 query
 * heads per kv head; num_heads * splits * (head_dim + 2) <= 1,048,576 floats
 * (splits is the planner's count, at most two CTAs per SM spread over the kv
 * heads) - anything larger is refused with SHAINET_ATTN_E_UNSUPPORTED.  All calls
 * share the array: calls that overlap on the GPU race and must be ordered by
 * the caller.  The first call made with a given device current looks up the
 * array's device address (thread-safe); make that call before any stream
 * capture starts.  The returned status covers argument checks, the set-up and
 * the launch.  Without a context there is no device status word, so a
 * kernel-side bounded wait that runs out (SHAINET_ATTN_E_DEVICE_WAIT elsewhere)
 * is NOT reported by this entry; the same holds for attention_kv_f32 above. */
int shainet_attn_decode_noalloc(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                float* out_dev, int start_pos, int num_heads, int heads_per_kv, int head_dim,
                                int capacity, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SHAINET_ATTN_H */
