// Device-resident decode step around the attention path: Q8_0 weights, the whole
// LlamaBlock#forward_cached and the Network#run token loop behind the C ABI of
// include/shainet_attn.h.
//
// The reference keeps activations on the host and crosses to the device and back for
// every projection: per decoded token and layer four blocking copies around the q/k/v/o
// GEMVs (src/shainet/transformer/llama_block.cr:726-768), two around attention
// (:469-477) and six around the FFN (src/shainet/transformer/swiglu_ff.cr:115-127), with
// RMSNorm, residuals, SiLU, the embedding gather, the final norm, the lm_head bias and
// the arg-max on the host (src/shainet/basic/network_run.cr:185-264).  Here one token is
// a chain of kernels on one stream with nothing on the host in between:
//
//   embedding row -> per layer [ RMSNorm + q|k|v GEMV -> fused norm/RoPE/append/attention
//   -> o_proj GEMV + residual -> RMSNorm + gate|up GEMV + SwiGLU -> down GEMV + residual ]
//   -> final RMSNorm + lm_head GEMV + bias + arg-max -> token id
//
// Every kernel of the chain is launched with programmatic stream serialization and
// requests its weights before it waits for its predecessor; it releases its own dependents
// only after that wait, so no kernel overlaps anything older than its direct predecessor.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "host_state.h"

using namespace shainet;

struct shainet_attn_q8 {
    shainet_attn_ctx* ctx = nullptr;
    signed char* q = nullptr;   // [N, K]
    float* scales = nullptr;    // [N, ceil(K/32)]
    int K = 0, N = 0;
    bool owns = false;
};

struct shainet_attn_block {
    shainet_attn_ctx* ctx = nullptr;
    shainet_attn_kv* kv = nullptr;
    int d_model = 0, q_dim = 0, kv_dim = 0, ffn = 0;
    float* norm1 = nullptr;     // device, [d_model]
    float* norm2 = nullptr;
    signed char* qkv_q = nullptr;   // the three projections stacked: [q_dim + 2 kv_dim, d_model]
    float* qkv_s = nullptr;
    const shainet_attn_q8* wo = nullptr;
    const shainet_attn_q8* gate = nullptr;
    const shainet_attn_q8* up = nullptr;
    const shainet_attn_q8* down = nullptr;
    double eps = 1e-6;
    float scale = 0.0f;
};

struct shainet_attn_decoder {
    shainet_attn_ctx* ctx = nullptr;
    std::vector<shainet_attn_block*> blocks;
    float* embedding = nullptr;   // device, [vocab, d_model] fp32 (the reference gathers rows on the host from fp32)
    float* final_norm = nullptr;  // device, nullable
    float* lm_bias = nullptr;     // device, nullable
    const shainet_attn_q8* lm_head = nullptr;
    int vocab = 0, d_model = 0;
    double eps = 1e-6;
    int* ids_dev = nullptr;       // [ids_cap] token ids of the current call
    int ids_cap = 0;
    int* ids_pin = nullptr;       // pinned staging of the same size
    int* history_dev = nullptr;   // [history_cap] tokens produced by generate
    int history_cap = 0;
    int* next_id = nullptr;       // device: the token the next step embeds
    int* token_dev = nullptr;     // device: arg-max of the last call
    unsigned long long* argmax_word = nullptr;
    float* logits = nullptr;      // device, [vocab]
};

namespace {

// Q8_0 of a host fp32 weight [K, N] (input-major, the layout of SimpleMatrix after the
// loader's transpose), as QuantizedCudaMatrix.from_simple does it
// (src/shainet/math/quantized_cuda_matrix.cr:74-115): per output column and block of 32
// consecutive K, scale = max|w| / 127 (1 for an all-zero block), q = round(w * (1/scale))
// clamped to +-127; q stored output-major [N, K], scales [N, blocks].
void quantize_q8_0(const float* w, int K, int N, signed char* q, float* scales) {
    const int blocks = (K + 31) / 32;
    for (int col = 0; col < N; ++col) {
        for (int b = 0; b < blocks; ++b) {
            const int base = b * 32, lim = std::min(base + 32, K);
            float max_abs = 0.0f;
            for (int k = base; k < lim; ++k) max_abs = std::max(max_abs, fabsf(w[(size_t)k * N + col]));
            const float scale = max_abs > 0.0f ? max_abs / 127.0f : 1.0f;
            const float inv = 1.0f / scale;
            scales[(size_t)col * blocks + b] = scale;
            for (int k = base; k < lim; ++k) {
                float qv = nearbyintf(w[(size_t)k * N + col] * inv);   // Float32#round: ties to even
                qv = qv > 127.0f ? 127.0f : (qv < -127.0f ? -127.0f : qv);
                q[(size_t)col * K + k] = (signed char)qv;
            }
        }
    }
}

int q8_new(shainet_attn_ctx* ctx, shainet_attn_q8** out, int K, int N) {
    if (!ctx || !out) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (K <= 0 || N <= 0) return fail(SHAINET_ATTN_E_INVALID, "weight shape %d x %d", K, N);
    shainet_attn_q8* w = new (std::nothrow) shainet_attn_q8();
    if (!w) return fail(SHAINET_ATTN_E_NOMEM, "out of host memory");
    w->ctx = ctx;
    w->K = K;
    w->N = N;
    *out = w;
    return SHAINET_ATTN_OK;
}

int gemv(shainet_attn_ctx* ctx, const float* x, const signed char* q, const float* scales, const signed char* q2,
         const float* scales2, float* y, int M, int N, int K, const float* gamma, double eps, const float* residual,
         const float* bias, unsigned long long* argmax, cudaStream_t s) {
    Q8GemvArgs a{};
    a.x = x;
    a.q = q;
    a.scales = scales;
    a.q2 = q2;
    a.scales2 = scales2;
    a.y = y;
    a.residual = residual;
    a.bias = bias;
    a.gamma = gamma;
    a.eps = eps;
    a.argmax = argmax;
    a.M = M;
    a.N = N;
    a.K = K;
    if ((size_t)K * sizeof(float) > 200 * 1024) return fail(SHAINET_ATTN_E_UNSUPPORTED, "input width %d exceeds what one CTA stages in shared memory", K);
    CU(launch_q8_gemv(a, ctx->sm_count, s));
    ctx->last_fused = false;
    ctx->after_chain_kernel = true;
    return SHAINET_ATTN_OK;
}

enum { ACT_QKV = 0, ACT_ATTN = 1, ACT_H = 2, ACT_HIDDEN = 3, ACT_A = 4, ACT_B = 5 };

// LlamaBlock#forward_cached (llama_block.cr:189-196) on device pointers.
int block_forward(shainet_attn_block* b, const float* x, float* out, int T, cudaStream_t s) {
    shainet_attn_ctx* ctx = b->ctx;
    const int d = b->d_model, qd = b->q_dim, kd = b->kv_dim;
    int rc = grow(ctx->act[ACT_QKV], (size_t)T * (qd + 2 * kd), s);
    if (!rc) rc = grow(ctx->act[ACT_ATTN], (size_t)T * qd, s);
    if (!rc && b->gate) rc = grow(ctx->act[ACT_H], (size_t)T * d, s);
    if (!rc && b->gate) rc = grow(ctx->act[ACT_HIDDEN], (size_t)T * b->ffn, s);
    if (rc) return rc;
    float* qbuf = ctx->act[ACT_QKV].p;
    float* kbuf = qbuf + (size_t)T * qd;
    float* vbuf = kbuf + (size_t)T * kd;
    const int kb = (d + 31) / 32;
    if (T == 1) {
        // one launch for q|k|v: the stacked weight's rows are the three projections' columns
        rc = gemv(ctx, x, b->qkv_q, b->qkv_s, nullptr, nullptr, qbuf, 1, qd + 2 * kd, d, b->norm1, b->eps, nullptr, nullptr, nullptr, s);
        if (rc) return rc;
    } else {
        const int n0[3] = {0, qd, qd + kd}, nn[3] = {qd, kd, kd};
        float* dst[3] = {qbuf, kbuf, vbuf};
        for (int i = 0; i < 3; ++i) {
            rc = gemv(ctx, x, b->qkv_q + (size_t)n0[i] * d, b->qkv_s + (size_t)n0[i] * kb, nullptr, nullptr, dst[i], T, nn[i], d,
                      b->norm1, b->eps, nullptr, nullptr, nullptr, s);
            if (rc) return rc;
        }
    }
    float* attn = ctx->act[ACT_ATTN].p;
    rc = forward_device(ctx, b->kv, qbuf, kbuf, vbuf, attn, T, b->scale, 0, s);
    if (rc) return rc;
    float* h = b->gate ? ctx->act[ACT_H].p : out;
    rc = gemv(ctx, attn, b->wo->q, b->wo->scales, nullptr, nullptr, h, T, d, qd, nullptr, 0.0, x, nullptr, nullptr, s);
    if (rc || !b->gate) return rc;
    float* hidden = ctx->act[ACT_HIDDEN].p;
    rc = gemv(ctx, h, b->gate->q, b->gate->scales, b->up->q, b->up->scales, hidden, T, b->ffn, d, b->norm2, b->eps, nullptr, nullptr,
              nullptr, s);
    if (rc) return rc;
    return gemv(ctx, hidden, b->down->q, b->down->scales, nullptr, nullptr, out, T, d, b->ffn, nullptr, 0.0, h, nullptr, nullptr, s);
}

int decoder_reserve_ids(shainet_attn_decoder* dec, int n) {
    if (dec->ids_cap >= n) return SHAINET_ATTN_OK;
    CU(cudaStreamSynchronize(dec->ctx->stream));
    if (dec->ids_dev) CU(cudaFree(dec->ids_dev));
    if (dec->ids_pin) CU(cudaFreeHost(dec->ids_pin));
    dec->ids_dev = nullptr;
    dec->ids_pin = nullptr;
    dec->ids_cap = 0;
    const int cap = std::max(n, 64);
    CU(cudaMalloc(&dec->ids_dev, sizeof(int) * cap));
    CU(cudaMallocHost(&dec->ids_pin, sizeof(int) * cap));
    dec->ids_cap = cap;
    return SHAINET_ATTN_OK;
}

// One Network#run call on the device: T token ids at ids_dev -> logits of the last row and
// its greedy token (token_dev, next_id, optionally history[history_pos]).
int decoder_step(shainet_attn_decoder* dec, const int* ids_dev, int T, int history_pos, cudaStream_t s) {
    shainet_attn_ctx* ctx = dec->ctx;
    const int d = dec->d_model;
    int rc = grow(ctx->act[ACT_A], (size_t)T * d, s);
    if (!rc) rc = grow(ctx->act[ACT_B], (size_t)T * d, s);
    if (rc) return rc;
    float* cur = ctx->act[ACT_A].p;
    float* nxt = ctx->act[ACT_B].p;
    CU(launch_embed_rows(ids_dev, dec->embedding, cur, T, d, dec->vocab, dec->argmax_word, 1, s));
    for (shainet_attn_block* b : dec->blocks) {
        rc = block_forward(b, cur, nxt, T, s);
        if (rc) return rc;
        std::swap(cur, nxt);
    }
    // final norm and lm_head see the last row only (network_run.cr:1471-1477), bias added after (:222-226)
    const float* last = cur + (size_t)(T - 1) * d;
    rc = gemv(ctx, last, dec->lm_head->q, dec->lm_head->scales, nullptr, nullptr, dec->logits, 1, dec->vocab, d, dec->final_norm, dec->eps,
              nullptr, dec->lm_bias, dec->argmax_word, s);
    if (rc) return rc;
    CU(launch_argmax_decode(dec->argmax_word, dec->token_dev, 1, dec->next_id, history_pos >= 0 ? dec->history_dev : nullptr,
                            history_pos >= 0 ? history_pos : 0, s));
    return SHAINET_ATTN_OK;
}

}  // namespace

extern "C" {

int shainet_attn_q8_create(shainet_attn_ctx* ctx, shainet_attn_q8** out, const float* w_host, int K, int N) {
    if (!ctx || !out || !w_host) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (K <= 0 || N <= 0) return fail(SHAINET_ATTN_E_INVALID, "weight shape %d x %d", K, N);
    std::vector<signed char> q((size_t)N * K);
    std::vector<float> sc((size_t)N * ((K + 31) / 32));
    quantize_q8_0(w_host, K, N, q.data(), sc.data());
    return shainet_attn_q8_create_raw(ctx, out, q.data(), sc.data(), K, N);
}

int shainet_attn_q8_create_raw(shainet_attn_ctx* ctx, shainet_attn_q8** out, const signed char* q_host, const float* scales_host,
                               int K, int N) {
    if (!q_host || !scales_host) return fail(SHAINET_ATTN_E_INVALID, "null weight pointer");
    int rc = q8_new(ctx, out, K, N);
    if (rc) return rc;
    shainet_attn_q8* w = *out;
    DeviceGuard g(ctx->device);
    const size_t qb = (size_t)N * K, sb = (size_t)N * ((K + 31) / 32) * sizeof(float);
    cudaError_t e = cudaMalloc(&w->q, qb);
    if (e == cudaSuccess) e = cudaMalloc(&w->scales, sb);
    if (e == cudaSuccess) e = cudaMemcpy(w->q, q_host, qb, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->scales, scales_host, sb, cudaMemcpyHostToDevice);
    w->owns = true;
    if (e != cudaSuccess) {
        shainet_attn_q8_destroy(w);
        *out = nullptr;
        return fail_cuda(e, "upload of a Q8_0 weight");
    }
    return SHAINET_ATTN_OK;
}

int shainet_attn_q8_wrap(shainet_attn_ctx* ctx, shainet_attn_q8** out, const signed char* q_dev, const float* scales_dev, int K,
                         int N) {
    if (!q_dev || !scales_dev) return fail(SHAINET_ATTN_E_INVALID, "null weight pointer");
    int rc = q8_new(ctx, out, K, N);
    if (rc) return rc;
    (*out)->q = const_cast<signed char*>(q_dev);
    (*out)->scales = const_cast<float*>(scales_dev);
    (*out)->owns = false;
    return SHAINET_ATTN_OK;
}

int shainet_attn_q8_destroy(shainet_attn_q8* w) {
    if (!w) return SHAINET_ATTN_OK;
    if (w->owns) {
        DeviceGuard g(w->ctx->device);
        cudaStreamSynchronize(w->ctx->stream);
        if (w->q) cudaFree(w->q);
        if (w->scales) cudaFree(w->scales);
        cudaGetLastError();
    }
    delete w;
    return SHAINET_ATTN_OK;
}

int shainet_attn_q8_export(const shainet_attn_q8* w, signed char* q_host, float* scales_host) {
    if (!w || !q_host || !scales_host) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    DeviceGuard g(w->ctx->device);
    CU(cudaMemcpy(q_host, w->q, (size_t)w->N * w->K, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(scales_host, w->scales, (size_t)w->N * ((w->K + 31) / 32) * sizeof(float), cudaMemcpyDeviceToHost));
    return SHAINET_ATTN_OK;
}

int shainet_attn_q8_gemv_dev(shainet_attn_ctx* ctx, const shainet_attn_q8* w, const float* x_dev, float* y_dev, int M, void* stream) {
    if (!ctx || !w || !x_dev || !y_dev) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (w->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "weight belongs to another context");
    if (M < 0) return fail(SHAINET_ATTN_E_INVALID, "negative row count");
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    return gemv(ctx, x_dev, w->q, w->scales, nullptr, nullptr, y_dev, M, w->N, w->K, nullptr, 0.0, nullptr, nullptr, nullptr, s);
}

// Same name, arguments and meaning as the reference's exported wrapper
// (src/shainet/native/cuda_kernels.cu:616-629): device pointers, legacy default stream.
void gemm_q8_f32(const float* x, const signed char* q, const float* scales, float* y, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return;
    Q8GemvArgs a{};
    a.x = x;
    a.q = q;
    a.scales = scales;
    a.y = y;
    a.M = M;
    a.N = N;
    a.K = K;
    int sm = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = (size_t)K * sizeof(float) > 200 * 1024 ? cudaErrorInvalidValue : launch_q8_gemv(a, sm, cudaStreamLegacy);
    if (e != cudaSuccess) printf("CUDA Error in gemm_q8_f32: %s\n", cudaGetErrorString(e));
}

int shainet_attn_block_create(shainet_attn_ctx* ctx, shainet_attn_block** out, shainet_attn_kv* kv, int d_model,
                              const float* norm1_host, const shainet_attn_q8* wq, const shainet_attn_q8* wk,
                              const shainet_attn_q8* wv, const shainet_attn_q8* wo, const float* norm2_host,
                              const shainet_attn_q8* gate, const shainet_attn_q8* up, const shainet_attn_q8* down, double eps) {
    if (!ctx || !out || !kv || !norm1_host || !wq || !wk || !wv || !wo) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (kv->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "cache belongs to another context");
    const int qd = kv->hs.num_heads * kv->hs.head_dim, kd = kv->hs.num_kv_heads * kv->hs.head_dim;
    if (d_model <= 0 || d_model % 4 != 0) return fail(SHAINET_ATTN_E_INVALID, "d_model %d must be a positive multiple of 4", d_model);
    if (wq->K != d_model || wq->N != qd || wk->K != d_model || wk->N != kd || wv->K != d_model || wv->N != kd || wo->K != qd ||
        wo->N != d_model)
        return fail(SHAINET_ATTN_E_INVALID, "projection shapes do not match d_model %d, q_dim %d, kv_dim %d", d_model, qd, kd);
    const bool has_ffn = gate || up || down || norm2_host;
    if (has_ffn) {
        if (!gate || !up || !down || !norm2_host) return fail(SHAINET_ATTN_E_INVALID, "the FFN needs norm2, gate, up and down together");
        if (gate->K != d_model || up->K != d_model || gate->N != up->N || down->K != gate->N || down->N != d_model)
            return fail(SHAINET_ATTN_E_INVALID, "FFN weight shapes do not match d_model %d", d_model);
    }
    DeviceGuard g(ctx->device);
    shainet_attn_block* b = new (std::nothrow) shainet_attn_block();
    if (!b) return fail(SHAINET_ATTN_E_NOMEM, "out of host memory");
    b->ctx = ctx;
    b->kv = kv;
    b->d_model = d_model;
    b->q_dim = qd;
    b->kv_dim = kd;
    b->ffn = has_ffn ? gate->N : 0;
    b->wo = wo;
    b->gate = gate;
    b->up = up;
    b->down = down;
    b->eps = eps;
    b->scale = (float)(1.0 / sqrt((double)kv->hs.head_dim));   // llama_block.cr:249
    const int kb = (d_model + 31) / 32;
    const size_t n_all = (size_t)qd + 2 * kd;
    cudaError_t e = cudaMalloc(&b->qkv_q, n_all * d_model);
    if (e == cudaSuccess) e = cudaMalloc(&b->qkv_s, n_all * kb * sizeof(float));
    const shainet_attn_q8* parts[3] = {wq, wk, wv};
    size_t row = 0;
    for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
        e = cudaMemcpy(b->qkv_q + row * d_model, parts[i]->q, (size_t)parts[i]->N * d_model, cudaMemcpyDeviceToDevice);
        if (e == cudaSuccess)
            e = cudaMemcpy(b->qkv_s + row * kb, parts[i]->scales, (size_t)parts[i]->N * kb * sizeof(float), cudaMemcpyDeviceToDevice);
        row += parts[i]->N;
    }
    if (e != cudaSuccess) {
        shainet_attn_block_destroy(b);
        return fail_cuda(e, "stacking the q/k/v projections");
    }
    int rc = upload_vec(b->norm1, norm1_host, (size_t)d_model);
    if (!rc && has_ffn) rc = upload_vec(b->norm2, norm2_host, (size_t)d_model);
    if (rc) {
        shainet_attn_block_destroy(b);
        return rc;
    }
    *out = b;
    return SHAINET_ATTN_OK;
}

int shainet_attn_block_destroy(shainet_attn_block* b) {
    if (!b) return SHAINET_ATTN_OK;
    DeviceGuard g(b->ctx->device);
    cudaStreamSynchronize(b->ctx->stream);
    for (void* p : {(void*)b->qkv_q, (void*)b->qkv_s, (void*)b->norm1, (void*)b->norm2})
        if (p) cudaFree(p);
    cudaGetLastError();
    delete b;
    return SHAINET_ATTN_OK;
}

int shainet_attn_block_forward_dev(shainet_attn_ctx* ctx, shainet_attn_block* b, const float* x_dev, float* out_dev, int new_tokens,
                                   void* stream) {
    if (!ctx || !b || b->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "null or foreign block");
    if (new_tokens < 0) return fail(SHAINET_ATTN_E_INVALID, "new_tokens %d < 0", new_tokens);
    if (new_tokens == 0) return SHAINET_ATTN_OK;
    if (!x_dev || !out_dev || !aligned16(x_dev) || !aligned16(out_dev)) return fail(SHAINET_ATTN_E_INVALID, "null or misaligned tensor pointer");
    DeviceGuard g(ctx->device);
    return block_forward(b, x_dev, out_dev, new_tokens, stream ? (cudaStream_t)stream : ctx->stream);
}

int shainet_attn_block_forward_host(shainet_attn_ctx* ctx, shainet_attn_block* b, const float* x, float* out, int new_tokens) {
    if (!ctx || !b || b->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "null or foreign block");
    if (new_tokens < 0) return fail(SHAINET_ATTN_E_INVALID, "new_tokens %d < 0", new_tokens);
    if (new_tokens == 0) return SHAINET_ATTN_OK;
    if (!x || !out) return fail(SHAINET_ATTN_E_INVALID, "null tensor pointer");
    DeviceGuard g(ctx->device);
    cudaStream_t s = ctx->stream;
    const size_t n = (size_t)new_tokens * b->d_model;
    int rc = grow(ctx->dev_in, n, s);
    if (!rc) rc = grow(ctx->dev_out, n, s);
    if (rc) return rc;
    CU(cudaMemcpyAsync(ctx->dev_in.p, x, n * sizeof(float), cudaMemcpyHostToDevice, s));
    rc = block_forward(b, ctx->dev_in.p, ctx->dev_out.p, new_tokens, s);
    if (rc) return rc;
    CU(cudaMemcpyAsync(out, ctx->dev_out.p, n * sizeof(float), cudaMemcpyDeviceToHost, s));
    return shainet_attn_ctx_sync(ctx);
}

int shainet_attn_decoder_create(shainet_attn_ctx* ctx, shainet_attn_decoder** out, shainet_attn_block* const* blocks, int n_layers,
                                const float* embedding_host, int vocab, const float* final_norm_host,
                                const shainet_attn_q8* lm_head, const float* lm_bias_host, double eps) {
    if (!ctx || !out || !blocks || !embedding_host || !lm_head) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (n_layers <= 0 || vocab <= 0) return fail(SHAINET_ATTN_E_INVALID, "bad layer count or vocabulary size");
    const int d = blocks[0] ? blocks[0]->d_model : 0;
    for (int l = 0; l < n_layers; ++l)
        if (!blocks[l] || blocks[l]->ctx != ctx || blocks[l]->d_model != d) return fail(SHAINET_ATTN_E_INVALID, "block %d is null, foreign or of another width", l);
    if (lm_head->K != d || lm_head->N != vocab) return fail(SHAINET_ATTN_E_INVALID, "lm_head is %d x %d, expected %d x %d", lm_head->K, lm_head->N, d, vocab);
    DeviceGuard g(ctx->device);
    shainet_attn_decoder* dec = new (std::nothrow) shainet_attn_decoder();
    if (!dec) return fail(SHAINET_ATTN_E_NOMEM, "out of host memory");
    dec->ctx = ctx;
    dec->blocks.assign(blocks, blocks + n_layers);
    dec->vocab = vocab;
    dec->d_model = d;
    dec->lm_head = lm_head;
    dec->eps = eps;
    cudaError_t e = cudaMalloc(&dec->embedding, (size_t)vocab * d * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(dec->embedding, embedding_host, (size_t)vocab * d * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&dec->logits, (size_t)vocab * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&dec->next_id, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&dec->token_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&dec->argmax_word, sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(dec->argmax_word, 0, sizeof(unsigned long long));
    int rc = e == cudaSuccess ? SHAINET_ATTN_OK : fail_cuda(e, "decoder buffers");
    if (!rc && final_norm_host) rc = upload_vec(dec->final_norm, final_norm_host, (size_t)d);
    if (!rc && lm_bias_host) rc = upload_vec(dec->lm_bias, lm_bias_host, (size_t)vocab);
    if (rc) {
        shainet_attn_decoder_destroy(dec);
        return rc;
    }
    *out = dec;
    return SHAINET_ATTN_OK;
}

int shainet_attn_decoder_destroy(shainet_attn_decoder* dec) {
    if (!dec) return SHAINET_ATTN_OK;
    DeviceGuard g(dec->ctx->device);
    cudaStreamSynchronize(dec->ctx->stream);
    for (void* p : {(void*)dec->embedding, (void*)dec->final_norm, (void*)dec->lm_bias, (void*)dec->ids_dev, (void*)dec->history_dev,
                    (void*)dec->next_id, (void*)dec->token_dev, (void*)dec->argmax_word, (void*)dec->logits})
        if (p) cudaFree(p);
    if (dec->ids_pin) cudaFreeHost(dec->ids_pin);
    cudaGetLastError();
    delete dec;
    return SHAINET_ATTN_OK;
}

int shainet_attn_decoder_run(shainet_attn_ctx* ctx, shainet_attn_decoder* dec, const int32_t* token_ids, int n_tokens,
                             float* logits_host, int32_t* next_token_host) {
    if (!ctx || !dec || dec->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "null or foreign decoder");
    if (n_tokens <= 0 || !token_ids) return fail(SHAINET_ATTN_E_INVALID, "no token ids");
    DeviceGuard g(ctx->device);
    cudaStream_t s = ctx->stream;
    int rc = decoder_reserve_ids(dec, n_tokens);
    if (rc) return rc;
    memcpy(dec->ids_pin, token_ids, sizeof(int) * (size_t)n_tokens);
    CU(cudaMemcpyAsync(dec->ids_dev, dec->ids_pin, sizeof(int) * (size_t)n_tokens, cudaMemcpyHostToDevice, s));
    rc = decoder_step(dec, dec->ids_dev, n_tokens, -1, s);
    if (rc) return rc;
    if (logits_host) CU(cudaMemcpyAsync(logits_host, dec->logits, sizeof(float) * (size_t)dec->vocab, cudaMemcpyDeviceToHost, s));
    if (next_token_host) CU(cudaMemcpyAsync(next_token_host, dec->token_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
    return shainet_attn_ctx_sync(ctx);
}

int shainet_attn_decoder_generate(shainet_attn_ctx* ctx, shainet_attn_decoder* dec, const int32_t* prompt_ids, int n_prompt,
                                  int steps, int32_t* tokens_host) {
    if (!ctx || !dec || dec->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "null or foreign decoder");
    if (n_prompt <= 0 || !prompt_ids || steps <= 0 || !tokens_host) return fail(SHAINET_ATTN_E_INVALID, "no prompt, no steps or no output array");
    DeviceGuard g(ctx->device);
    cudaStream_t s = ctx->stream;
    int rc = decoder_reserve_ids(dec, n_prompt);
    if (rc) return rc;
    if (dec->history_cap < steps) {
        CU(cudaStreamSynchronize(s));
        if (dec->history_dev) CU(cudaFree(dec->history_dev));
        dec->history_dev = nullptr;
        dec->history_cap = 0;
        CU(cudaMalloc(&dec->history_dev, sizeof(int) * (size_t)std::max(steps, 256)));
        dec->history_cap = std::max(steps, 256);
    }
    // grow every cache once, up front: growth synchronises the stream
    for (shainet_attn_block* b : dec->blocks) {
        rc = shainet_attn_kv_reserve(b->kv, b->kv->len + n_prompt + steps);
        if (rc) return rc;
    }
    memcpy(dec->ids_pin, prompt_ids, sizeof(int) * (size_t)n_prompt);
    CU(cudaMemcpyAsync(dec->ids_dev, dec->ids_pin, sizeof(int) * (size_t)n_prompt, cudaMemcpyHostToDevice, s));
    rc = decoder_step(dec, dec->ids_dev, n_prompt, 0, s);
    for (int i = 1; i < steps && !rc; ++i) rc = decoder_step(dec, dec->next_id, 1, i, s);   // the token never visits the host
    if (rc) return rc;
    CU(cudaMemcpyAsync(tokens_host, dec->history_dev, sizeof(int) * (size_t)steps, cudaMemcpyDeviceToHost, s));
    return shainet_attn_ctx_sync(ctx);
}

}  // extern "C"
