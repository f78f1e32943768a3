// Host side of libshainet_attn: contexts, KV caches, kernel selection and the
// C ABI declared in include/shainet_attn.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <string>
#include <utility>
#include <vector>

#include "host_state.h"

using namespace shainet;

namespace {

thread_local std::string g_last_error;

constexpr size_t SMALL_COPY = 1 << 20;  // host entry: stage through pinned memory below this
constexpr int SPLITK_MAX_T = 16;      // rows per call the decode kernel takes before the generic one
constexpr int TENSOR_MIN_T = 64;      // rows per call from which the tensor-core prefill kernel takes over

}  // namespace

namespace shainet {

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int fail_cuda(cudaError_t e, const char* what) {
    const int code = (e == cudaErrorMemoryAllocation) ? SHAINET_ATTN_E_NOMEM : SHAINET_ATTN_E_CUDA;
    cudaGetLastError();  // clear the sticky-free error state
    return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace shainet

namespace {

int grow_pinned(float*& p, size_t& cap, size_t floats) {
    if (cap >= floats && p) return SHAINET_ATTN_OK;
    if (p) CU(cudaFreeHost(p));
    p = nullptr;
    cap = 0;
    size_t want = std::max(floats, (size_t)4096);
    CU(cudaMallocHost(&p, want * sizeof(float)));
    cap = want;
    return SHAINET_ATTN_OK;
}

// ---- virtual-memory management (driver API, looked up once) for caches that grow without moving ----
struct VmmApi {
    CUresult (*address_reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    bool ok = false;
};

const VmmApi& vmm_api() {
    static VmmApi api = [] {
        VmmApi a;
        auto get = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn;
        };
        a.ok = get("cuMemAddressReserve", (void**)&a.address_reserve) && get("cuMemAddressFree", (void**)&a.address_free) &&
               get("cuMemCreate", (void**)&a.create) && get("cuMemRelease", (void**)&a.release) && get("cuMemMap", (void**)&a.map) &&
               get("cuMemUnmap", (void**)&a.unmap) && get("cuMemSetAccess", (void**)&a.set_access) &&
               get("cuMemGetAllocationGranularity", (void**)&a.granularity);
        cudaGetLastError();
        return a;
    }();
    return api;
}

CUmemAllocationProp vmm_prop(int device) {
    CUmemAllocationProp p{};
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = device;
    return p;
}

// Maps (and zeroes) pages behind every kv head of both tensors until `rows` rows of each are backed.
int kv_map_rows(shainet_attn_kv* kv, int rows, cudaStream_t s) {
    const VmmApi& api = vmm_api();
    const size_t row_bytes = (size_t)kv->hs.head_dim * kv->es;
    const size_t head_stride = (size_t)kv->cap * row_bytes;
    const size_t need = ((size_t)rows * row_bytes + kv->page_bytes - 1) / kv->page_bytes;
    if (need <= kv->pages_per_head) return SHAINET_ATTN_OK;
    const CUmemAllocationProp prop = vmm_prop(kv->ctx->device);
    CUmemAccessDesc acc{};
    acc.location = prop.location;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    const size_t first = kv->pages_per_head * kv->page_bytes, bytes = (need - kv->pages_per_head) * kv->page_bytes;
    for (float* base : {kv->k, kv->v}) {
        for (int h = 0; h < kv->hs.num_kv_heads; ++h) {
            const CUdeviceptr at = (CUdeviceptr)base + (size_t)h * head_stride + first;
            CUmemGenericAllocationHandle hd;
            CUresult r = api.create(&hd, bytes, &prop, 0);
            if (r != CUDA_SUCCESS)
                return fail(r == CUDA_ERROR_OUT_OF_MEMORY ? SHAINET_ATTN_E_NOMEM : SHAINET_ATTN_E_CUDA, "cuMemCreate of %zu bytes failed (%d)", bytes, (int)r);
            r = api.map(at, bytes, 0, hd, 0);
            if (r == CUDA_SUCCESS) r = api.set_access(at, bytes, &acc, 1);
            if (r != CUDA_SUCCESS) {
                api.release(hd);
                return fail(SHAINET_ATTN_E_CUDA, "mapping %zu bytes of cache failed (%d)", bytes, (int)r);
            }
            kv->mappings.push_back({(unsigned long long)at, (unsigned long long)bytes, (unsigned long long)hd});
            // rows past the appended length are read (and masked) by the tensor-core prefill kernel: they start at zero
            CU(cudaMemsetAsync((void*)at, 0, bytes, s));
        }
    }
    CU(cudaStreamSynchronize(s));
    kv->pages_per_head = need;
    return SHAINET_ATTN_OK;
}

// Capacity policy of ensure_gpu_cache! (llama_block.cr:500): max(256, need, 2*old),
// but the live rows move device-to-device instead of being re-uploaded.
int kv_ensure(shainet_attn_kv* kv, int total_len, cudaStream_t s) {
    if (kv->reserved) {
        if (total_len > kv->cap)
            return fail(SHAINET_ATTN_E_INVALID, "%d rows exceed the %d this cache reserved addresses for", total_len, kv->cap);
        // whole 128-row tiles of the prefill kernel are always backed
        return kv_map_rows(kv, std::min(kv->cap, (total_len + 127) / 128 * 128), s);
    }
    if (kv->cap >= total_len && kv->k) return SHAINET_ATTN_OK;
    const long long want = std::max<long long>(256, std::max<long long>(total_len, 2ll * kv->cap));
    if (want > 0x7fffffffll) return fail(SHAINET_ATTN_E_INVALID, "cache capacity overflow");
    const int new_cap = (int)want;
    const size_t es = (size_t)kv->es;
    const size_t bytes = (size_t)kv->hs.num_kv_heads * new_cap * kv->hs.head_dim * es;
    float *nk = nullptr, *nv = nullptr;
    cudaError_t e = cudaMalloc(&nk, bytes);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc(k cache)");
    e = cudaMalloc(&nv, bytes);
    if (e != cudaSuccess) {
        cudaFree(nk);
        return fail_cuda(e, "cudaMalloc(v cache)");
    }
    // Rows past the appended length are read (and masked) by the tensor-core
    // prefill kernel; they must be finite, so fresh buffers start at zero.
    e = cudaMemsetAsync(nk, 0, bytes, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(nv, 0, bytes, s);
    if (e == cudaSuccess && kv->k && kv->len > 0) {
        const size_t row_bytes = (size_t)kv->len * kv->hs.head_dim * es;
        const size_t src_pitch = (size_t)kv->cap * kv->hs.head_dim * es;
        const size_t dst_pitch = (size_t)new_cap * kv->hs.head_dim * es;
        e = cudaMemcpy2DAsync(nk, dst_pitch, kv->k, src_pitch, row_bytes, kv->hs.num_kv_heads, cudaMemcpyDeviceToDevice, s);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(nv, dst_pitch, kv->v, src_pitch, row_bytes, kv->hs.num_kv_heads, cudaMemcpyDeviceToDevice, s);
    }
    // The old buffers are freed below, and a first allocation may be followed by work on
    // another stream (a cache created on the context's stream, then used on the caller's):
    // either way the zero fill and the move have to be complete when this returns.
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        cudaFree(nk);
        cudaFree(nv);
        return fail_cuda(e, "cache growth (zero fill / move of the live rows)");
    }
    if (kv->k) {
        CU(cudaFree(kv->k));
        CU(cudaFree(kv->v));
    }
    kv->k = nk;
    kv->v = nv;
    kv->cap = new_cap;
    return SHAINET_ATTN_OK;
}

int check_status(shainet_attn_ctx* ctx) {
    if (ctx->status_host && ctx->status_host->code != DEV_OK) {
        const int where = ctx->status_host->where;
        ctx->status_host->code = DEV_OK;
        ctx->status_host->where = 0;
        if (ctx->tickets) cudaMemset(ctx->tickets, 0, ctx->tickets_cap * sizeof(unsigned));  // an unwound kernel may leave counts
        return fail(SHAINET_ATTN_E_DEVICE_WAIT, "a kernel gave up on a bounded wait (site %d)", where);
    }
    return SHAINET_ATTN_OK;
}

enum class Kernel { Generic, SplitK, Tensor };

int ensure_tickets(shainet_attn_ctx* ctx, size_t n, cudaStream_t s) {
    if (ctx->tickets_cap >= n && ctx->tickets) return SHAINET_ATTN_OK;
    if (ctx->tickets) {
        CU(cudaStreamSynchronize(s));
        CU(cudaFree(ctx->tickets));
        ctx->tickets = nullptr;
        ctx->tickets_cap = 0;
    }
    const size_t want = std::max<size_t>(n, 256);
    CU(cudaMalloc(&ctx->tickets, want * sizeof(unsigned)));
    CU(cudaMemset(ctx->tickets, 0, want * sizeof(unsigned)));
    ctx->tickets_cap = want;
    return SHAINET_ATTN_OK;
}

int pick_kernel(const HeadShape& hs, int batch, int T, unsigned flags, Kernel* out) {
    const bool sk_ok = splitk_supported(hs);
    const bool tc_ok = prefill_tc_supported(hs) && batch == 1;
    if (flags & SHAINET_ATTN_F_TENSOR) {
        if (!tc_ok) return fail(SHAINET_ATTN_E_UNSUPPORTED, "tensor-core prefill needs head_dim 64 or 128 and a single sequence");
        *out = Kernel::Tensor;
        return SHAINET_ATTN_OK;
    }
    if (flags & SHAINET_ATTN_F_SPLITK) {
        if (!sk_ok) return fail(SHAINET_ATTN_E_UNSUPPORTED, "split-K decode needs head_dim 64/128 and group size 1/2/4/8/16");
        *out = Kernel::SplitK;
        return SHAINET_ATTN_OK;
    }
    if (flags & SHAINET_ATTN_F_GENERIC) {
        *out = Kernel::Generic;
        return SHAINET_ATTN_OK;
    }
    *out = (sk_ok && T <= SPLITK_MAX_T) ? Kernel::SplitK : (tc_ok && T >= TENSOR_MIN_T) ? Kernel::Tensor : Kernel::Generic;
    return SHAINET_ATTN_OK;
}

// Rows of cache per split so that about one CTA lands on every SM.
void plan_splits(int sm_count, const HeadShape& hs, int rows, long long total_visible, int max_visible,
                 int waves, int* chunk_rows, int* max_splits, int kv_elem_bytes = 4, bool batched = false) {
    const int tw = splitk_tile_rows(hs, kv_elem_bytes, batched);
    const long long ctas = std::max<long long>(1, (long long)sm_count * splitk_ctas_per_sm(hs) * waves);
    long long chunk = (total_visible * hs.num_kv_heads + ctas - 1) / ctas;
    const long long min_chunk = 4ll * tw;  // one tile per consumer warp
    chunk = std::max(chunk, min_chunk);
    chunk = (chunk + tw - 1) / tw * tw;
    if (chunk > 0x3fffffff) chunk = 0x3fffffff / tw * tw;
    *chunk_rows = (int)chunk;
    *max_splits = (int)((max_visible + chunk - 1) / chunk);
    (void)rows;
}

int run_attention_untimed(shainet_attn_ctx* ctx, const HeadShape& hs, SeqRef seqs, int batch, int T,
                          long long total_visible, int max_visible, const float* q_rot, float* out, float scale,
                          unsigned flags, cudaStream_t s);

int run_attention(shainet_attn_ctx* ctx, const HeadShape& hs, SeqRef seqs, int batch, int T, long long total_visible,
                  int max_visible, const float* q_rot, float* out, float scale, unsigned flags, cudaStream_t s) {
    if (!ctx->timing)
        return run_attention_untimed(ctx, hs, seqs, batch, T, total_visible, max_visible, q_rot, out, scale, flags, s);
    std::pair<cudaEvent_t, cudaEvent_t> ev;
    if (!ctx->ev_pool.empty()) {
        ev = ctx->ev_pool.back();
        ctx->ev_pool.pop_back();
    } else {
        CU(cudaEventCreate(&ev.first));
        CU(cudaEventCreate(&ev.second));
    }
    CU(cudaEventRecord(ev.first, s));
    int rc = run_attention_untimed(ctx, hs, seqs, batch, T, total_visible, max_visible, q_rot, out, scale, flags, s);
    CU(cudaEventRecord(ev.second, s));
    ctx->timed.push_back(ev);
    return rc;
}

int run_attention_untimed(shainet_attn_ctx* ctx, const HeadShape& hs, SeqRef seqs, int batch, int T,
                          long long total_visible, int max_visible, const float* q_rot, float* out, float scale,
                          unsigned flags, cudaStream_t s) {
    Kernel kern;
    int rc = pick_kernel(hs, batch, T, flags, &kern);
    if (rc) return rc;
    AttnArgs a{};
    a.q_rot = q_rot;
    a.out = out;
    a.seqs = seqs;
    a.batch = batch;
    a.T = T;
    a.hs = hs;
    a.scale = scale;
    a.status = ctx->status_dev;
    a.prefill_one_cta = (flags & SHAINET_ATTN_F_TENSOR_1CTA) ? 1 : 0;
    if (kern == Kernel::Generic) {
        if (hs.head_dim > 256) return fail(SHAINET_ATTN_E_UNSUPPORTED, "head_dim %d > 256", hs.head_dim);
        CU(launch_attn_generic(a, s));
        return SHAINET_ATTN_OK;
    }
    if (kern == Kernel::Tensor) {
        CU(launch_attn_prefill_tc(a, s));
        return SHAINET_ATTN_OK;
    }
    const int rows = batch * T;
    plan_splits(ctx->sm_count, hs, rows, total_visible, max_visible, batch > 1 ? 8 : 1, &a.chunk_rows, &a.max_splits);
    if (a.max_splits > 1) {
        const size_t need = splitk_scratch_floats(hs, rows, a.max_splits);
        rc = grow(ctx->part, need, s);
        if (rc) return rc;
        a.part_o = ctx->part.p;
        a.part_ml = ctx->part.p + (size_t)rows * hs.num_heads * a.max_splits * hs.head_dim;
    }
    CU(launch_attn_splitk(a, s));
    return SHAINET_ATTN_OK;
}

int validate_forward(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const void* q, const void* k, const void* v,
                     const void* out, int new_tokens) {
    if (!ctx || !kv) return fail(SHAINET_ATTN_E_INVALID, "null context or cache");
    if (kv->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "cache belongs to another context");
    if (new_tokens < 0) return fail(SHAINET_ATTN_E_INVALID, "new_tokens %d < 0", new_tokens);
    if (new_tokens > 0 && (!q || !k || !v || !out)) return fail(SHAINET_ATTN_E_INVALID, "null tensor pointer");
    if ((long long)kv->len + new_tokens > 0x7fffffffll) return fail(SHAINET_ATTN_E_INVALID, "cache length overflow");
    return SHAINET_ATTN_OK;
}

// One call = `batch` sequences x T new tokens: norm/RoPE/append + attention.
// `par` supplies the shared head shape, RoPE table, norm weights and biases.
int run_step(shainet_attn_ctx* ctx, const shainet_attn_kv* par, SeqRef seqs, int batch, int T, long long total_visible,
             int max_visible, const float* q, const float* k_new, const float* v_new, float* out, float scale,
             unsigned flags, cudaStream_t s, int pos_delta = 0, int no_append = 0) {
    const HeadShape hs = par->hs;
    const bool fused = T == 1 && splitk_supported(hs) &&
                       !(flags & (SHAINET_ATTN_F_GENERIC | SHAINET_ATTN_F_UNFUSED | SHAINET_ATTN_F_TENSOR));
    int rc;
    if (!fused && (pos_delta != 0 || no_append))
        return fail(SHAINET_ATTN_E_UNSUPPORTED, "a split sequence is served by the fused decode kernel only (head_dim 64/128, group size 1/2/4/8/16)");
    if (!fused && ctx->gather_armed) {
        ctx->gather_armed = false;
        return fail(SHAINET_ATTN_E_UNSUPPORTED, "peer delivery is done by the fused decode kernel only (one new token, head_dim 64/128)");
    }
    if (!fused && par->es != 4 && seqs.many != nullptr)
        return fail(SHAINET_ATTN_E_UNSUPPORTED, "batched decode over bfloat16 caches is served by the fused decode kernel only");
    if (!fused) {
        ctx->last_fused = false;
        rc = grow(ctx->q_rot, (size_t)batch * T * hs.num_heads * hs.head_dim, s);
        if (rc) return rc;
        PrepArgs p{};
        p.q = q;
        p.k_new = k_new;
        p.v_new = v_new;
        p.b_q = par->b_q;
        p.b_k = par->b_k;
        p.b_v = par->b_v;
        p.q_norm = par->q_norm;
        p.k_norm = par->k_norm;
        p.inv_freq = par->inv_freq;
        p.eps = par->eps;
        p.q_rot = ctx->q_rot.p;
        p.seqs = seqs;
        p.batch = batch;
        p.T = T;
        p.hs = hs;
        Kernel kern;
        rc = pick_kernel(hs, batch, T, flags, &kern);
        if (rc) return rc;
        p.round_q_tf32 = kern == Kernel::Tensor ? 1 : 0;
        p.kv_elem_bytes = par->es;
        p.status = ctx->status_dev;
        CU(launch_prep_append(p, s));
        if (par->es != 4) {
            // These attention kernels read fp32 rows.  A bfloat16 cache is widened (exactly) into
            // a scratch image first; the capacity of the image is a whole number of the
            // tensor-core kernel's 128-row tiles, and it never holds anything but finite values.
            const int cap_s = (max_visible + 127) / 128 * 128;
            const size_t per = (size_t)hs.num_kv_heads * cap_s * hs.head_dim;
            float* before = ctx->kv_f32.p;
            rc = grow(ctx->kv_f32, 2 * per, s);
            if (rc) return rc;
            if (ctx->kv_f32.p != before) CU(cudaMemsetAsync(ctx->kv_f32.p, 0, ctx->kv_f32.cap * sizeof(float), s));
            float* wk = ctx->kv_f32.p;
            float* wv = wk + per;
            CU(launch_kv_convert(seqs.one.k, par->es, seqs.one.capacity, wk, 4, cap_s, hs.num_kv_heads, hs.head_dim, 0, max_visible, s));
            CU(launch_kv_convert(seqs.one.v, par->es, seqs.one.capacity, wv, 4, cap_s, hs.num_kv_heads, hs.head_dim, 0, max_visible, s));
            seqs.one = SeqDesc{wk, wv, seqs.one.start, cap_s};
        }
        return run_attention(ctx, hs, seqs, batch, T, total_visible, max_visible, ctx->q_rot.p, out, scale, flags, s);
    }
    FusedArgs f{};
    f.q = q;
    f.k_new = k_new;
    f.v_new = v_new;
    f.b_q = par->b_q;
    f.b_k = par->b_k;
    f.b_v = par->b_v;
    f.q_norm = par->q_norm;
    f.k_norm = par->k_norm;
    f.inv_freq = par->inv_freq;
    f.eps = par->eps;
    f.out = out;
    f.seqs = seqs;
    f.batch = batch;
    f.hs = hs;
    f.scale = scale;
    f.status = ctx->status_dev;
    plan_splits(ctx->sm_count, hs, batch, total_visible, max_visible, batch > 1 ? 4 : 1, &f.chunk_rows, &f.max_splits, par->es,
                seqs.many != nullptr);
    f.max_groups = fused_merge_groups(f.max_splits);
    // A single sequence whose grid is fully resident merges through {value, epoch} words
    // (8 bytes per partial float) polled by the merging CTAs; batched decode keeps float
    // partials and the two-level tickets.
    f.stream_merge = batch == 1 && f.max_splits > 1 && !(flags & SHAINET_ATTN_F_TICKET_MERGE) &&
                     (long long)f.max_splits * hs.num_kv_heads <= (long long)ctx->sm_count * splitk_ctas_per_sm(hs);
    if (f.max_splits > 1 && f.stream_merge) {
        // a buffer of its own, written by nothing but this merge: a stale word can then
        // only carry an older epoch
        const size_t nw = 2 * splitk_scratch_floats(hs, batch, f.max_splits);
        float* before = ctx->part_words.p;
        rc = grow(ctx->part_words, nw, s);
        if (rc) return rc;
        if (ctx->part_words.p != before) CU(cudaMemsetAsync(ctx->part_words.p, 0, ctx->part_words.cap * sizeof(float), s));
        f.part_o = ctx->part_words.p;
        f.part_ml = f.part_o + 2 * (size_t)batch * hs.num_heads * f.max_splits * hs.head_dim;
    } else if (f.max_splits > 1) {
        const size_t n1 = (splitk_scratch_floats(hs, batch, f.max_splits) + 3) & ~(size_t)3;  // keeps the second table 16-byte aligned
        const size_t n2 = splitk_scratch_floats(hs, batch, f.max_groups);
        rc = grow(ctx->part, n1 + n2, s);
        if (rc) return rc;
        f.part_o = ctx->part.p;
        f.part_ml = f.part_o + (size_t)batch * hs.num_heads * f.max_splits * hs.head_dim;
        f.part2_o = ctx->part.p + n1;
        f.part2_ml = f.part2_o + (size_t)batch * hs.num_heads * f.max_groups * hs.head_dim;
    }
    // tickets (two levels) for the batched merge
    const size_t n_tickets = (size_t)batch * hs.num_kv_heads * (1 + f.max_groups);
    rc = ensure_tickets(ctx, n_tickets, s);
    if (rc) return rc;
    f.tickets = ctx->tickets;
    if (f.stream_merge) {
        // a fresh epoch per launch; at the wrap of the counter every old word is wiped
        if (ctx->epoch == 0xffffffffu) {
            CU(cudaMemsetAsync(ctx->part_words.p, 0, ctx->part_words.cap * sizeof(float), s));
            ctx->epoch = 0;
        }
        f.epoch = ++ctx->epoch;
    }
    // A fused kernel may start while the previous fused kernel still runs; that
    // one can be appending the newest row of this very cache.
    f.unsafe_tail = (ctx->last_fused || ctx->after_chain_kernel) ? 1 : 0;
    ctx->after_chain_kernel = false;
    f.inputs_ready = ((flags & SHAINET_ATTN_F_INPUTS_READY) && !ctx->rows_rewound) ? 1 : 0;
    ctx->rows_rewound = false;
    f.pos_delta = pos_delta;
    f.no_append = no_append;
    f.kv_elem_bytes = par->es;
    f.lse_out = ctx->lse_out;
    f.gather.world = 0;
    if (ctx->gather_armed) {
        ctx->gather_armed = false;
        if (!f.stream_merge)
            return fail(SHAINET_ATTN_E_UNSUPPORTED, "peer delivery needs the flag-merged single-sequence decode kernel (context too short, batched, or tickets forced)");
        const size_t need = (size_t)ctx->gather_out_off + (size_t)hs.num_heads * hs.head_dim;
        if (need > ctx->comm_data_floats || (ctx->gather_lse_off >= 0 && (size_t)ctx->gather_lse_off + hs.num_heads > ctx->comm_data_floats))
            return fail(SHAINET_ATTN_E_INVALID, "peer delivery target outside the exchange buffer");
        GatherTarget& gt = f.gather;
        gt.world = ctx->comm_world;
        for (int p = 0; p < ctx->comm_world; ++p)
            gt.peer_words[p] = reinterpret_cast<unsigned long long*>(ctx->comm_peer[p] + ctx->comm_data_floats * sizeof(float));
        gt.out_offset = ctx->gather_out_off;
        gt.lse_offset = ctx->gather_lse_off;
        gt.epoch = ctx->gather_epoch;
    }
    std::pair<cudaEvent_t, cudaEvent_t> ev{};
    if (ctx->timing) {
        if (!ctx->ev_pool.empty()) {
            ev = ctx->ev_pool.back();
            ctx->ev_pool.pop_back();
        } else {
            CU(cudaEventCreate(&ev.first));
            CU(cudaEventCreate(&ev.second));
        }
        CU(cudaEventRecord(ev.first, s));
    }
    CU(launch_decode_fused(f, s));
    if (ctx->timing) {
        CU(cudaEventRecord(ev.second, s));
        ctx->timed.push_back(ev);
    }
    ctx->last_fused = true;
    return SHAINET_ATTN_OK;
}

}  // namespace

namespace shainet {

int grow(DevBuf& b, size_t floats, cudaStream_t s) {
    if (b.cap >= floats && b.p) return SHAINET_ATTN_OK;
    const size_t old_cap = b.cap;
    if (b.p) {
        CU(cudaStreamSynchronize(s));
        CU(cudaFree(b.p));
        b.p = nullptr;
        b.cap = 0;
    }
    size_t want = std::max(floats, old_cap * 2);
    want = (want + 63) & ~(size_t)63;
    CU(cudaMalloc(&b.p, want * sizeof(float)));
    b.cap = want;
    return SHAINET_ATTN_OK;
}

int upload_vec(float*& dst, const float* host, size_t n) {
    if (!host) {
        if (dst) CU(cudaFree(dst));
        dst = nullptr;
        return SHAINET_ATTN_OK;
    }
    if (!dst) CU(cudaMalloc(&dst, n * sizeof(float)));
    CU(cudaMemcpy(dst, host, n * sizeof(float), cudaMemcpyHostToDevice));
    return SHAINET_ATTN_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int forward_device(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new, const float* v_new,
                   float* out, int T, float scale, unsigned flags, cudaStream_t s) {
    const int cap_before = kv->cap;
    int rc = kv_ensure(kv, kv->len + T, s);
    if (rc) return rc;
    if (kv->cap != cap_before) ctx->last_fused = false;  // growth synchronised the stream
    SeqRef seqs{};
    seqs.one = SeqDesc{kv->k, kv->v, kv->len, kv->cap};
    seqs.many = nullptr;
    const long long total_visible = (long long)T * kv->len + (long long)T * (T + 1) / 2;
    rc = run_step(ctx, kv, seqs, 1, T, total_visible, kv->len + T, q, k_new, v_new, out, scale, flags, s);
    if (rc) return rc;
    kv->len += T;
    return SHAINET_ATTN_OK;
}

void set_last_error_message(const char* msg) { g_last_error = msg ? msg : ""; }
}  // namespace shainet

extern "C" {

int shainet_attn_version(void) { return SHAINET_ATTN_VERSION; }

int shainet_attn_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

const char* shainet_attn_last_error(void) { return g_last_error.c_str(); }

int shainet_attn_ctx_create(shainet_attn_ctx** out, int device) {
    if (!out) return fail(SHAINET_ATTN_E_INVALID, "null out pointer");
    *out = nullptr;
    int n = shainet_attn_device_count();
    if (n <= 0) return fail(SHAINET_ATTN_E_CUDA, "no CUDA device (this library has no CPU path)");
    if (device < 0 || device >= n) return fail(SHAINET_ATTN_E_INVALID, "device %d out of range [0,%d)", device, n);
    DeviceGuard g(device);
    if (!g.ok) return fail(SHAINET_ATTN_E_CUDA, "cudaSetDevice(%d) failed", device);
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(SHAINET_ATTN_E_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    shainet_attn_ctx* c = new (std::nothrow) shainet_attn_ctx();
    if (!c) return fail(SHAINET_ATTN_E_NOMEM, "out of host memory");
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaHostAlloc(&c->status_host, sizeof(AttnStatus), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        c->status_host->code = DEV_OK;
        c->status_host->where = 0;
        e = cudaHostGetDevicePointer(&c->status_dev, c->status_host, 0);
    }
    for (int i = 0; i < SEQ_RING && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&c->seq_ev[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
        shainet_attn_ctx_destroy(c);
        return fail_cuda(e, "context setup");
    }
    *out = c;
    return SHAINET_ATTN_OK;
}

int shainet_attn_ctx_destroy(shainet_attn_ctx* c) {
    if (!c) return SHAINET_ATTN_OK;
    if (c->live_caches != 0) return fail(SHAINET_ATTN_E_STATE, "%d caches still alive", c->live_caches);
    DeviceGuard g(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (DevBuf* b : {&c->q_rot, &c->part, &c->part_words, &c->dev_in, &c->dev_out, &c->kv_f32})
        if (b->p) cudaFree(b->p);
    if (c->pin_in) cudaFreeHost(c->pin_in);
    if (c->pin_out) cudaFreeHost(c->pin_out);
    if (c->status_host) cudaFreeHost(c->status_host);
    if (c->seq_host) cudaFreeHost(c->seq_host);
    if (c->seq_dev) cudaFree(c->seq_dev);
    if (c->tickets) cudaFree(c->tickets);
    for (int p = 0; p < c->comm_world; ++p)
        if (p != c->comm_rank && c->comm_peer[p]) cudaIpcCloseMemHandle(c->comm_peer[p]);
    if (c->comm_base) cudaFree(c->comm_base);
    for (int i = 0; i < SEQ_RING; ++i)
        if (c->seq_ev[i]) cudaEventDestroy(c->seq_ev[i]);
    for (auto* v : {&c->timed, &c->ev_pool})
        for (auto& ev : *v) {
            cudaEventDestroy(ev.first);
            cudaEventDestroy(ev.second);
        }
    if (c->stream) cudaStreamDestroy(c->stream);
    cudaGetLastError();
    delete c;
    return SHAINET_ATTN_OK;
}

int shainet_attn_ctx_sync(shainet_attn_ctx* c) {
    if (!c) return fail(SHAINET_ATTN_E_INVALID, "null context");
    DeviceGuard g(c->device);
    CU(cudaStreamSynchronize(c->stream));
    return check_status(c);
}

int shainet_attn_ctx_timing_enable(shainet_attn_ctx* c, int enable) {
    if (!c) return fail(SHAINET_ATTN_E_INVALID, "null context");
    c->timing = enable != 0;
    return SHAINET_ATTN_OK;
}

int shainet_attn_ctx_timing_read(shainet_attn_ctx* c, double* total_ms, int* launches) {
    if (!c || !total_ms || !launches) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    DeviceGuard g(c->device);
    double sum = 0.0;
    for (auto& ev : c->timed) {
        CU(cudaEventSynchronize(ev.second));
        float ms = 0.0f;
        CU(cudaEventElapsedTime(&ms, ev.first, ev.second));
        sum += ms;
    }
    *total_ms = sum;
    *launches = (int)c->timed.size();
    c->ev_pool.insert(c->ev_pool.end(), c->timed.begin(), c->timed.end());
    c->timed.clear();
    return SHAINET_ATTN_OK;
}

size_t shainet_attn_ctx_scratch_bytes(shainet_attn_ctx* c) {
    if (!c) return 0;
    return (c->q_rot.cap + c->part.cap + c->part_words.cap + c->dev_in.cap + c->dev_out.cap + c->kv_f32.cap) * sizeof(float);
}

int shainet_attn_kv_create(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                           int head_dim, int initial_capacity) {
    return shainet_attn_kv_create_fmt(ctx, out, num_heads, num_kv_heads, head_dim, initial_capacity, SHAINET_ATTN_KV_F32);
}

int shainet_attn_kv_format(const shainet_attn_kv* kv) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    return kv->es == 2 ? SHAINET_ATTN_KV_BF16 : SHAINET_ATTN_KV_F32;
}

int shainet_attn_kv_create_fmt(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                               int head_dim, int initial_capacity, int format) {
    if (!ctx || !out) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (format != SHAINET_ATTN_KV_F32 && format != SHAINET_ATTN_KV_BF16)
        return fail(SHAINET_ATTN_E_INVALID, "unknown cache format %d", format);
    // LlamaBlock.new's checks (llama_block.cr:80-89)
    if (num_kv_heads <= 0 || num_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(SHAINET_ATTN_E_INVALID, "num_heads must be divisible by num_kv_heads");
    if (head_dim <= 0) return fail(SHAINET_ATTN_E_INVALID, "head_dim must be positive");
    if (head_dim % 2 != 0) return fail(SHAINET_ATTN_E_UNSUPPORTED, "odd head_dim %d", head_dim);
    if (head_dim > 256) return fail(SHAINET_ATTN_E_UNSUPPORTED, "head_dim %d > 256", head_dim);
    if (initial_capacity < 0) return fail(SHAINET_ATTN_E_INVALID, "negative capacity");
    DeviceGuard g(ctx->device);
    shainet_attn_kv* kv = new (std::nothrow) shainet_attn_kv();
    if (!kv) return fail(SHAINET_ATTN_E_NOMEM, "out of host memory");
    kv->ctx = ctx;
    kv->hs = HeadShape{num_heads, num_kv_heads, head_dim};
    kv->es = format == SHAINET_ATTN_KV_BF16 ? 2 : 4;
    ctx->live_caches++;
    int rc = shainet_attn_kv_set_rope_theta(kv, 10000.0);
    if (rc == SHAINET_ATTN_OK && initial_capacity > 0) rc = kv_ensure(kv, initial_capacity, ctx->stream);
    if (rc != SHAINET_ATTN_OK) {
        std::string keep = g_last_error;
        shainet_attn_kv_destroy(kv);
        g_last_error = keep;
        return rc;
    }
    *out = kv;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_create_reserved(shainet_attn_ctx* ctx, shainet_attn_kv** out, int num_heads, int num_kv_heads,
                                    int head_dim, int max_capacity, int format) {
    if (!out) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    *out = nullptr;
    if (max_capacity <= 0) return fail(SHAINET_ATTN_E_INVALID, "the reserved capacity must be positive");
    const VmmApi& api = vmm_api();
    if (!api.ok) return fail(SHAINET_ATTN_E_UNSUPPORTED, "the driver does not offer virtual memory management");
    shainet_attn_kv* kv = nullptr;
    int rc = shainet_attn_kv_create_fmt(ctx, &kv, num_heads, num_kv_heads, head_dim, 0, format);
    if (rc) return rc;
    DeviceGuard g(ctx->device);
    const CUmemAllocationProp prop = vmm_prop(ctx->device);
    size_t gran = 0;
    CUresult r = api.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
    if (r != CUDA_SUCCESS || gran == 0) {
        shainet_attn_kv_destroy(kv);
        return fail(SHAINET_ATTN_E_CUDA, "cuMemGetAllocationGranularity failed (%d)", (int)r);
    }
    // every kv head's range starts on a page: round the capacity up until its bytes are a whole number of pages
    const size_t row_bytes = (size_t)head_dim * kv->es;
    size_t a = gran, b = row_bytes;
    while (b) {
        const size_t t = a % b;
        a = b;
        b = t;
    }
    const size_t rows_unit = gran / a;   // smallest row count whose bytes are a multiple of the granularity
    const size_t cap = ((size_t)max_capacity + rows_unit - 1) / rows_unit * rows_unit;
    if (cap > 0x7fffffffull) {
        shainet_attn_kv_destroy(kv);
        return fail(SHAINET_ATTN_E_INVALID, "reserved capacity overflow");
    }
    const size_t total = cap * row_bytes * num_kv_heads;
    CUdeviceptr pk = 0, pv = 0;
    r = api.address_reserve(&pk, total, gran, 0, 0);
    if (r == CUDA_SUCCESS) r = api.address_reserve(&pv, total, gran, 0, 0);
    if (r != CUDA_SUCCESS) {
        if (pk) api.address_free(pk, total);
        shainet_attn_kv_destroy(kv);
        return fail(SHAINET_ATTN_E_NOMEM, "reserving %zu bytes of device addresses failed (%d)", total, (int)r);
    }
    kv->reserved = true;
    kv->page_bytes = gran;
    kv->cap = (int)cap;
    kv->k = reinterpret_cast<float*>(pk);
    kv->v = reinterpret_cast<float*>(pv);
    *out = kv;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_destroy(shainet_attn_kv* kv) {
    if (!kv) return SHAINET_ATTN_OK;
    DeviceGuard g(kv->ctx->device);
    cudaStreamSynchronize(kv->ctx->stream);
    if (kv->reserved) {
        const VmmApi& api = vmm_api();
        const size_t total = (size_t)kv->cap * kv->hs.head_dim * kv->es * kv->hs.num_kv_heads;
        for (const shainet_attn_kv::Mapping& m : kv->mappings) {
            api.unmap((CUdeviceptr)m.at, (size_t)m.bytes);
            api.release((CUmemGenericAllocationHandle)m.handle);
        }
        kv->mappings.clear();
        if (kv->k) api.address_free((CUdeviceptr)kv->k, total);
        if (kv->v) api.address_free((CUdeviceptr)kv->v, total);
        kv->k = kv->v = nullptr;
    }
    for (float* p : {kv->k, kv->v, kv->inv_freq, kv->q_norm, kv->k_norm, kv->b_q, kv->b_k, kv->b_v})
        if (p) cudaFree(p);
    cudaGetLastError();
    kv->ctx->live_caches--;
    delete kv;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_reset(shainet_attn_kv* kv) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    kv->len = 0;  // buffers stay; stale rows are rewritten before they become visible
    kv->ctx->rows_rewound = true;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_truncate(shainet_attn_kv* kv, int len) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    if (len < 0 || len > kv->len) return fail(SHAINET_ATTN_E_STATE, "truncate to %d of a cache of %d", len, kv->len);
    if (len < kv->len) kv->ctx->rows_rewound = true;
    kv->len = len;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_len(const shainet_attn_kv* kv) { return kv ? kv->len : fail(SHAINET_ATTN_E_INVALID, "null cache"); }

int shainet_attn_kv_capacity(const shainet_attn_kv* kv) {
    return kv ? kv->cap : fail(SHAINET_ATTN_E_INVALID, "null cache");
}

int shainet_attn_kv_reserve(shainet_attn_kv* kv, int total_len) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    if (total_len < 0) return fail(SHAINET_ATTN_E_INVALID, "negative length");
    DeviceGuard g(kv->ctx->device);
    return kv_ensure(kv, total_len, kv->ctx->stream);
}

int shainet_attn_kv_set_rope_theta(shainet_attn_kv* kv, double theta) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    if (!(theta > 0.0)) return fail(SHAINET_ATTN_E_INVALID, "rope theta must be positive");
    const int half = kv->hs.head_dim / 2;
    std::vector<float> f(half);
    for (int i = 0; i < half; ++i) f[i] = (float)(1.0 / pow(theta, 2.0 * (double)i / (double)kv->hs.head_dim));
    return shainet_attn_kv_set_rope(kv, f.data(), half);
}

int shainet_attn_kv_set_rope(shainet_attn_kv* kv, const float* inv_freq_host, int half) {
    if (!kv || !inv_freq_host) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (half != kv->hs.head_dim / 2) return fail(SHAINET_ATTN_E_INVALID, "rope table has %d entries, head_dim/2 is %d", half, kv->hs.head_dim / 2);
    DeviceGuard g(kv->ctx->device);
    CU(cudaStreamSynchronize(kv->ctx->stream));
    return upload_vec(kv->inv_freq, inv_freq_host, (size_t)half);
}

int shainet_attn_kv_set_qk_norm(shainet_attn_kv* kv, const float* qw, const float* kw, double eps) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    DeviceGuard g(kv->ctx->device);
    CU(cudaStreamSynchronize(kv->ctx->stream));
    int rc = upload_vec(kv->q_norm, qw, (size_t)kv->hs.head_dim);
    if (rc) return rc;
    rc = upload_vec(kv->k_norm, kw, (size_t)kv->hs.head_dim);
    if (rc) return rc;
    kv->eps = eps;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_set_bias(shainet_attn_kv* kv, const float* bq, const float* bk, const float* bv) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    DeviceGuard g(kv->ctx->device);
    CU(cudaStreamSynchronize(kv->ctx->stream));
    const size_t qd = (size_t)kv->hs.num_heads * kv->hs.head_dim, kd = (size_t)kv->hs.num_kv_heads * kv->hs.head_dim;
    int rc = upload_vec(kv->b_q, bq, qd);
    if (rc) return rc;
    rc = upload_vec(kv->b_k, bk, kd);
    if (rc) return rc;
    return upload_vec(kv->b_v, bv, kd);
}

int shainet_attn_kv_export(shainet_attn_kv* kv, float* k_host, float* v_host, int len) {
    if (!kv || !k_host || !v_host) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (len < 0 || len > kv->len) return fail(SHAINET_ATTN_E_STATE, "export of %d rows from a cache of %d", len, kv->len);
    if (len == 0) return SHAINET_ATTN_OK;
    DeviceGuard g(kv->ctx->device);
    cudaStream_t s = kv->ctx->stream;
    CU(cudaStreamSynchronize(s));
    const size_t row_bytes = (size_t)len * kv->hs.head_dim * sizeof(float);
    if (kv->es != 4) {
        // widened (exactly) on the device, one tensor at a time, through the context's fp32 image
        const size_t per = (size_t)kv->hs.num_kv_heads * len * kv->hs.head_dim;
        float* before = kv->ctx->kv_f32.p;
        int rc = grow(kv->ctx->kv_f32, per, s);
        if (rc) return rc;
        if (kv->ctx->kv_f32.p != before) CU(cudaMemsetAsync(kv->ctx->kv_f32.p, 0, kv->ctx->kv_f32.cap * sizeof(float), s));
        float* host[2] = {k_host, v_host};
        const float* dev[2] = {kv->k, kv->v};
        for (int t = 0; t < 2; ++t) {
            CU(launch_kv_convert(dev[t], kv->es, kv->cap, kv->ctx->kv_f32.p, 4, len, kv->hs.num_kv_heads, kv->hs.head_dim, 0, len, s));
            CU(cudaMemcpyAsync(host[t], kv->ctx->kv_f32.p, per * sizeof(float), cudaMemcpyDeviceToHost, s));
            CU(cudaStreamSynchronize(s));
        }
        return SHAINET_ATTN_OK;
    }
    const size_t pitch = (size_t)kv->cap * kv->hs.head_dim * sizeof(float);
    if (kv->reserved) {
        // a pitched copy would be checked over the unmapped addresses between the kv heads: one copy per head
        for (int h = 0; h < kv->hs.num_kv_heads; ++h) {
            CU(cudaMemcpy(reinterpret_cast<char*>(k_host) + h * row_bytes, reinterpret_cast<const char*>(kv->k) + h * pitch, row_bytes, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(reinterpret_cast<char*>(v_host) + h * row_bytes, reinterpret_cast<const char*>(kv->v) + h * pitch, row_bytes, cudaMemcpyDeviceToHost));
        }
        return SHAINET_ATTN_OK;
    }
    CU(cudaMemcpy2D(k_host, row_bytes, kv->k, pitch, row_bytes, kv->hs.num_kv_heads, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy2D(v_host, row_bytes, kv->v, pitch, row_bytes, kv->hs.num_kv_heads, cudaMemcpyDeviceToHost));
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_import(shainet_attn_kv* kv, const float* k_host, const float* v_host, int len) {
    if (!kv || (len > 0 && (!k_host || !v_host))) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (len < 0) return fail(SHAINET_ATTN_E_INVALID, "negative length");
    DeviceGuard g(kv->ctx->device);
    kv->len = 0;
    int rc = kv_ensure(kv, len, kv->ctx->stream);
    if (rc) return rc;
    if (len > 0 && kv->es != 4) {
        // uploaded as fp32, one tensor at a time, and rounded to bfloat16 (nearest even) on the device
        cudaStream_t s = kv->ctx->stream;
        const size_t per = (size_t)kv->hs.num_kv_heads * len * kv->hs.head_dim;
        float* before = kv->ctx->kv_f32.p;
        rc = grow(kv->ctx->kv_f32, per, s);
        if (rc) return rc;
        if (kv->ctx->kv_f32.p != before) CU(cudaMemsetAsync(kv->ctx->kv_f32.p, 0, kv->ctx->kv_f32.cap * sizeof(float), s));
        const float* host[2] = {k_host, v_host};
        float* dev[2] = {kv->k, kv->v};
        for (int t = 0; t < 2; ++t) {
            CU(cudaMemcpyAsync(kv->ctx->kv_f32.p, host[t], per * sizeof(float), cudaMemcpyHostToDevice, s));
            CU(launch_kv_convert(kv->ctx->kv_f32.p, 4, len, dev[t], kv->es, kv->cap, kv->hs.num_kv_heads, kv->hs.head_dim, 0, len, s));
            CU(cudaStreamSynchronize(s));
        }
    } else if (len > 0) {
        CU(cudaStreamSynchronize(kv->ctx->stream));
        const size_t row_bytes = (size_t)len * kv->hs.head_dim * sizeof(float);
        const size_t pitch = (size_t)kv->cap * kv->hs.head_dim * sizeof(float);
        if (kv->reserved) {
            for (int h = 0; h < kv->hs.num_kv_heads; ++h) {
                CU(cudaMemcpy(reinterpret_cast<char*>(kv->k) + h * pitch, reinterpret_cast<const char*>(k_host) + h * row_bytes, row_bytes, cudaMemcpyHostToDevice));
                CU(cudaMemcpy(reinterpret_cast<char*>(kv->v) + h * pitch, reinterpret_cast<const char*>(v_host) + h * row_bytes, row_bytes, cudaMemcpyHostToDevice));
            }
        } else {
            CU(cudaMemcpy2D(kv->k, pitch, k_host, row_bytes, row_bytes, kv->hs.num_kv_heads, cudaMemcpyHostToDevice));
            CU(cudaMemcpy2D(kv->v, pitch, v_host, row_bytes, row_bytes, kv->hs.num_kv_heads, cudaMemcpyHostToDevice));
        }
    }
    kv->len = len;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_fill_normal(shainet_attn_kv* kv, int len, uint64_t seed) {
    if (!kv) return fail(SHAINET_ATTN_E_INVALID, "null cache");
    if (len < 0) return fail(SHAINET_ATTN_E_INVALID, "negative length");
    DeviceGuard g(kv->ctx->device);
    kv->len = 0;
    int rc = kv_ensure(kv, len, kv->ctx->stream);
    if (rc) return rc;
    CU(launch_fill_normal(kv->k, kv->hs.num_kv_heads, kv->cap, kv->hs.head_dim, len, 2 * seed, kv->es, kv->ctx->stream));
    CU(launch_fill_normal(kv->v, kv->hs.num_kv_heads, kv->cap, kv->hs.head_dim, len, 2 * seed + 1, kv->es, kv->ctx->stream));
    CU(cudaStreamSynchronize(kv->ctx->stream));
    kv->len = len;
    return SHAINET_ATTN_OK;
}

int shainet_attn_kv_device_ptrs(shainet_attn_kv* kv, float** k_dev, float** v_dev) {
    if (!kv || !k_dev || !v_dev) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (kv->es != 4) return fail(SHAINET_ATTN_E_UNSUPPORTED, "the rows of a bfloat16 cache are not fp32: use shainet_attn_kv_export");
    *k_dev = kv->k;
    *v_dev = kv->v;
    return SHAINET_ATTN_OK;
}

int shainet_attn_forward_host(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                              const float* v_new, float* out, int T, float scale, unsigned flags) {
    int rc = validate_forward(ctx, kv, q, k_new, v_new, out, T);
    if (rc) return rc;
    if (T == 0) return SHAINET_ATTN_OK;
    DeviceGuard g(ctx->device);
    cudaStream_t s = ctx->stream;
    const size_t qn = (size_t)T * kv->hs.num_heads * kv->hs.head_dim;
    const size_t kn = (size_t)T * kv->hs.num_kv_heads * kv->hs.head_dim;
    const size_t in_n = qn + 2 * kn;
    rc = grow(ctx->dev_in, in_n, s);
    if (rc) return rc;
    rc = grow(ctx->dev_out, qn, s);
    if (rc) return rc;
    float* dq = ctx->dev_in.p;
    float* dk = dq + qn;
    float* dv = dk + kn;
    const bool small = in_n * sizeof(float) <= SMALL_COPY;
    if (small) {
        // One pinned blob, one H2D: q | k | v.
        rc = grow_pinned(ctx->pin_in, ctx->pin_in_cap, in_n);
        if (rc) return rc;
        rc = grow_pinned(ctx->pin_out, ctx->pin_out_cap, qn);
        if (rc) return rc;
        memcpy(ctx->pin_in, q, qn * sizeof(float));
        memcpy(ctx->pin_in + qn, k_new, kn * sizeof(float));
        memcpy(ctx->pin_in + qn + kn, v_new, kn * sizeof(float));
        CU(cudaMemcpyAsync(dq, ctx->pin_in, in_n * sizeof(float), cudaMemcpyHostToDevice, s));
    } else {
        CU(cudaMemcpyAsync(dq, q, qn * sizeof(float), cudaMemcpyHostToDevice, s));
        CU(cudaMemcpyAsync(dk, k_new, kn * sizeof(float), cudaMemcpyHostToDevice, s));
        CU(cudaMemcpyAsync(dv, v_new, kn * sizeof(float), cudaMemcpyHostToDevice, s));
    }
    // One decode token through the fused kernel: its merging CTAs store the few result
    // rows straight into the pinned (device-visible) host buffer, which saves the
    // device-to-host copy operation and its latency.
    const bool direct_out = small && T == 1 && splitk_supported(kv->hs) &&
                            !(flags & (SHAINET_ATTN_F_GENERIC | SHAINET_ATTN_F_UNFUSED | SHAINET_ATTN_F_TENSOR));
    rc = forward_device(ctx, kv, dq, dk, dv, direct_out ? ctx->pin_out : ctx->dev_out.p, T, scale, flags, s);
    if (rc) return rc;
    if (small) {
        if (!direct_out) CU(cudaMemcpyAsync(ctx->pin_out, ctx->dev_out.p, qn * sizeof(float), cudaMemcpyDeviceToHost, s));
        CU(cudaStreamSynchronize(s));
        memcpy(out, ctx->pin_out, qn * sizeof(float));
    } else {
        CU(cudaMemcpyAsync(out, ctx->dev_out.p, qn * sizeof(float), cudaMemcpyDeviceToHost, s));
        CU(cudaStreamSynchronize(s));
    }
    return check_status(ctx);
}

int shainet_attn_forward_dev(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                             const float* v_new, float* out, int T, float scale, unsigned flags, void* stream) {
    int rc = validate_forward(ctx, kv, q, k_new, v_new, out, T);
    if (rc) return rc;
    if (T == 0) return SHAINET_ATTN_OK;
    if (!aligned16(q) || !aligned16(k_new) || !aligned16(v_new) || !aligned16(out))
        return fail(SHAINET_ATTN_E_INVALID, "device pointers must be 16-byte aligned");
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    return forward_device(ctx, kv, q, k_new, v_new, out, T, scale, flags, s);
}

int shainet_attn_ctx_set_lse_out(shainet_attn_ctx* ctx, float* lse_dev) {
    if (!ctx) return fail(SHAINET_ATTN_E_INVALID, "null context");
    ctx->lse_out = lse_dev;
    return SHAINET_ATTN_OK;
}

int shainet_attn_forward_dev_at(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                                const float* v_new, float* out, int position, int append, float scale, unsigned flags,
                                void* stream) {
    int rc = validate_forward(ctx, kv, q, append ? k_new : q, append ? v_new : q, out, 1);
    if (rc) return rc;
    if (!aligned16(q) || !aligned16(out) || (append && (!aligned16(k_new) || !aligned16(v_new))))
        return fail(SHAINET_ATTN_E_INVALID, "device pointers must be 16-byte aligned");
    if (position < kv->len) return fail(SHAINET_ATTN_E_INVALID, "position %d is before the %d rows this cache already holds", position, kv->len);
    if (!append && kv->len == 0) return fail(SHAINET_ATTN_E_STATE, "nothing to attend to: the cache is empty and the token is not appended");
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    const int cap_before = kv->cap;
    rc = kv_ensure(kv, kv->len + (append ? 1 : 0), s);
    if (rc) return rc;
    if (kv->cap != cap_before) ctx->last_fused = false;
    SeqRef seqs{};
    seqs.one = SeqDesc{kv->k, kv->v, kv->len, kv->cap};
    seqs.many = nullptr;
    const int visible = kv->len + (append ? 1 : 0);
    rc = run_step(ctx, kv, seqs, 1, 1, visible, visible, q, k_new, v_new, out, scale, flags, s, position - kv->len, append ? 0 : 1);
    if (rc) return rc;
    if (append) kv->len += 1;
    return SHAINET_ATTN_OK;
}

int shainet_attn_merge_parts(shainet_attn_ctx* ctx, const float* gathered_dev, int world, int seq_parts, int heads_per_rank,
                             int head_dim, float* out_full_dev, void* stream) {
    if (!ctx || !gathered_dev || !out_full_dev) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (world <= 0 || seq_parts <= 0 || world % seq_parts != 0 || heads_per_rank <= 0 || head_dim <= 0)
        return fail(SHAINET_ATTN_E_INVALID, "bad partition: %d ranks in groups of %d", world, seq_parts);
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    ctx->last_fused = false;
    CU(launch_merge_parts(gathered_dev, world, seq_parts, heads_per_rank, head_dim, out_full_dev, s));
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_create(shainet_attn_ctx* ctx, size_t data_floats, void* handle_out) {
    if (!ctx || !handle_out) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (ctx->comm_base) return fail(SHAINET_ATTN_E_STATE, "exchange buffer already created");
    if (data_floats == 0 || data_floats % 4 != 0) return fail(SHAINET_ATTN_E_INVALID, "exchange buffer size must be a positive multiple of 4 floats");
    DeviceGuard g(ctx->device);
    const size_t bytes = data_floats * (sizeof(float) + sizeof(unsigned long long));
    CU(cudaMalloc(&ctx->comm_base, bytes));
    CU(cudaMemset(ctx->comm_base, 0, bytes));   // epoch 0 = nothing delivered
    ctx->comm_data_floats = data_floats;
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, ctx->comm_base));
    static_assert(sizeof(h) == SHAINET_ATTN_COMM_HANDLE_BYTES, "handle size");
    memcpy(handle_out, &h, sizeof h);
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_open(shainet_attn_ctx* ctx, const void* handles, int world, int rank) {
    if (!ctx || !handles) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (!ctx->comm_base) return fail(SHAINET_ATTN_E_STATE, "create the exchange buffer first");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) return fail(SHAINET_ATTN_E_INVALID, "bad world/rank %d/%d", world, rank);
    if (ctx->comm_world) return fail(SHAINET_ATTN_E_STATE, "exchange buffers already opened");
    DeviceGuard g(ctx->device);
    for (int p = 0; p < world; ++p) {
        if (p == rank) {
            ctx->comm_peer[p] = ctx->comm_base;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const unsigned char*>(handles) + (size_t)p * sizeof h, sizeof h);
        void* ptr = nullptr;
        CU(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        ctx->comm_peer[p] = static_cast<unsigned char*>(ptr);
    }
    ctx->comm_world = world;
    ctx->comm_rank = rank;
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_set_target(shainet_attn_ctx* ctx, long long out_offset_floats, long long lse_offset_floats, unsigned epoch) {
    if (!ctx) return fail(SHAINET_ATTN_E_INVALID, "null context");
    if (!ctx->comm_world) return fail(SHAINET_ATTN_E_STATE, "exchange buffers are not opened");
    if (out_offset_floats < 0 || out_offset_floats % 4 != 0) return fail(SHAINET_ATTN_E_INVALID, "output offset must be a non-negative multiple of 4 floats");
    if (epoch == 0) return fail(SHAINET_ATTN_E_INVALID, "epoch 0 is the empty state of the exchange buffer");
    ctx->gather_out_off = out_offset_floats;
    ctx->gather_lse_off = lse_offset_floats;
    ctx->gather_epoch = epoch;
    ctx->gather_armed = true;
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_wait(shainet_attn_ctx* ctx, long long offset_floats, long long count_floats, unsigned epoch, void* stream) {
    if (!ctx) return fail(SHAINET_ATTN_E_INVALID, "null context");
    if (!ctx->comm_world) return fail(SHAINET_ATTN_E_STATE, "exchange buffers are not opened");
    if (offset_floats < 0 || count_floats < 0 || (size_t)(offset_floats + count_floats) > ctx->comm_data_floats)
        return fail(SHAINET_ATTN_E_INVALID, "range outside the exchange buffer");
    if (epoch == 0) return fail(SHAINET_ATTN_E_INVALID, "epoch 0 is the empty state of the exchange buffer");
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    float* data = reinterpret_cast<float*>(ctx->comm_base);
    const unsigned long long* words = reinterpret_cast<const unsigned long long*>(ctx->comm_base + ctx->comm_data_floats * sizeof(float));
    CU(launch_gather_wait(words + offset_floats, data + offset_floats, count_floats, epoch, ctx->peer_wait_ns, ctx->status_dev, s));
    return SHAINET_ATTN_OK;
}

int shainet_attn_forward_dev_exchange(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                                      const float* v_new, float* out, int position, int append, float scale, unsigned flags,
                                      long long out_offset_floats, long long lse_offset_floats, long long wait_offset_floats,
                                      long long wait_count_floats, unsigned epoch, void* stream) {
    int rc = shainet_attn_comm_set_target(ctx, out_offset_floats, lse_offset_floats, epoch);
    if (rc) return rc;
    rc = shainet_attn_forward_dev_at(ctx, kv, q, k_new, v_new, out, position, append, scale, flags, stream);
    if (rc) {
        ctx->gather_armed = false;
        return rc;
    }
    return shainet_attn_comm_wait(ctx, wait_offset_floats, wait_count_floats, epoch, stream);
}

int shainet_attn_forward_dev_exchange_merge(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new,
                                            const float* v_new, float* out, int position, int append, float scale,
                                            unsigned flags, long long slot_offset_floats, int seq_parts, unsigned epoch,
                                            float* out_full_dev, void* stream) {
    if (!ctx || !kv || !out_full_dev) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (!ctx->comm_world) return fail(SHAINET_ATTN_E_STATE, "exchange buffers are not opened");
    if (seq_parts <= 0 || seq_parts > MAX_PEERS || ctx->comm_world % seq_parts != 0)
        return fail(SHAINET_ATTN_E_INVALID, "bad partition: %d ranks in groups of %d", ctx->comm_world, seq_parts);
    const long long heads = kv->hs.num_heads, hd = kv->hs.head_dim;
    const long long pay = heads * (hd + 1);            // a rank's block: head rows, then log-sum-exp values
    if (slot_offset_floats < 0 || (size_t)(slot_offset_floats + ctx->comm_world * pay) > ctx->comm_data_floats)
        return fail(SHAINET_ATTN_E_INVALID, "exchange slot outside the buffer");
    const long long mine = slot_offset_floats + ctx->comm_rank * pay;
    int rc = shainet_attn_comm_set_target(ctx, mine, mine + heads * hd, epoch);
    if (rc) return rc;
    rc = shainet_attn_forward_dev_at(ctx, kv, q, k_new, v_new, out, position, append, scale, flags, stream);
    if (rc) {
        ctx->gather_armed = false;
        return rc;
    }
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    const unsigned long long* words = reinterpret_cast<const unsigned long long*>(ctx->comm_base + ctx->comm_data_floats * sizeof(float));
    CU(launch_gather_merge(words + slot_offset_floats, ctx->comm_world, seq_parts, (int)heads, (int)hd, epoch,
                           ctx->peer_wait_ns, out_full_dev, ctx->status_dev, s));
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_set_wait_limit_ms(shainet_attn_ctx* ctx, int milliseconds) {
    if (!ctx) return fail(SHAINET_ATTN_E_INVALID, "null context");
    if (milliseconds < 1 || milliseconds > 600000) return fail(SHAINET_ATTN_E_INVALID, "wait limit %d ms outside [1, 600000]", milliseconds);
    ctx->peer_wait_ns = (unsigned long long)milliseconds * 1000000ull;
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_read(shainet_attn_ctx* ctx, long long offset_floats, float* host_dst, size_t floats, void* stream) {
    if (!ctx || !host_dst) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (!ctx->comm_base) return fail(SHAINET_ATTN_E_STATE, "no exchange buffer");
    if (offset_floats < 0 || (size_t)offset_floats + floats > ctx->comm_data_floats)
        return fail(SHAINET_ATTN_E_INVALID, "range outside the exchange buffer");
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    CU(cudaMemcpyAsync(host_dst, reinterpret_cast<const float*>(ctx->comm_base) + offset_floats, floats * sizeof(float),
                       cudaMemcpyDeviceToHost, s));
    return SHAINET_ATTN_OK;
}

int shainet_attn_comm_data_ptr(shainet_attn_ctx* ctx, float** data_dev) {
    if (!ctx || !data_dev) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (!ctx->comm_base) return fail(SHAINET_ATTN_E_STATE, "no exchange buffer");
    *data_dev = reinterpret_cast<float*>(ctx->comm_base);
    return SHAINET_ATTN_OK;
}

int shainet_attn_forward_batched_dev(shainet_attn_ctx* ctx, shainet_attn_kv* const* kvs, int batch, const float* q,
                                     const float* k_new, const float* v_new, float* out, float scale, unsigned flags,
                                     void* stream) {
    if (!ctx || !kvs) return fail(SHAINET_ATTN_E_INVALID, "null pointer");
    if (batch < 0) return fail(SHAINET_ATTN_E_INVALID, "negative batch");
    if (batch == 0) return SHAINET_ATTN_OK;
    if (!q || !k_new || !v_new || !out) return fail(SHAINET_ATTN_E_INVALID, "null tensor pointer");
    if (!aligned16(q) || !aligned16(k_new) || !aligned16(v_new) || !aligned16(out))
        return fail(SHAINET_ATTN_E_INVALID, "device pointers must be 16-byte aligned");
    if (batch > 65535) return fail(SHAINET_ATTN_E_UNSUPPORTED, "batch %d > 65535", batch);
    const shainet_attn_kv* first = kvs[0];
    if (!first) return fail(SHAINET_ATTN_E_INVALID, "null cache in batch");
    for (int b = 0; b < batch; ++b) {
        const shainet_attn_kv* kv = kvs[b];
        if (!kv || kv->ctx != ctx) return fail(SHAINET_ATTN_E_INVALID, "cache %d is null or of another context", b);
        if (kv->hs.num_heads != first->hs.num_heads || kv->hs.num_kv_heads != first->hs.num_kv_heads ||
            kv->hs.head_dim != first->hs.head_dim)
            return fail(SHAINET_ATTN_E_INVALID, "cache %d has a different head shape", b);
        if (kv->es != first->es) return fail(SHAINET_ATTN_E_INVALID, "cache %d has a different element format", b);
        for (int c = 0; c < b; ++c)
            if (kvs[c] == kv) return fail(SHAINET_ATTN_E_INVALID, "cache %d appears twice in the batch", b);
        if (kv->len == 0x7fffffff) return fail(SHAINET_ATTN_E_INVALID, "cache length overflow");
    }
    DeviceGuard g(ctx->device);
    cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
    int rc;
    for (int b = 0; b < batch; ++b) {
        rc = kv_ensure(kvs[b], kvs[b]->len + 1, s);
        if (rc) return rc;
    }
    if (ctx->seq_cap < batch) {
        CU(cudaStreamSynchronize(s));
        for (int i = 0; i < SEQ_RING; ++i) CU(cudaEventSynchronize(ctx->seq_ev[i]));
        if (ctx->seq_host) CU(cudaFreeHost(ctx->seq_host));
        if (ctx->seq_dev) CU(cudaFree(ctx->seq_dev));
        ctx->seq_host = nullptr;
        ctx->seq_dev = nullptr;
        ctx->seq_cap = 0;
        const int cap = std::max(batch, 64);
        CU(cudaMallocHost(&ctx->seq_host, sizeof(SeqDesc) * cap * SEQ_RING));
        CU(cudaMalloc(&ctx->seq_dev, sizeof(SeqDesc) * cap * SEQ_RING));
        ctx->seq_cap = cap;
    }
    const int slot = ctx->seq_slot;
    ctx->seq_slot = (slot + 1) % SEQ_RING;
    CU(cudaEventSynchronize(ctx->seq_ev[slot]));  // the upload that last used this slot has run
    SeqDesc* hd = ctx->seq_host + (size_t)slot * ctx->seq_cap;
    SeqDesc* dd = ctx->seq_dev + (size_t)slot * ctx->seq_cap;
    long long total_visible = 0;
    int max_visible = 0;
    for (int b = 0; b < batch; ++b) {
        hd[b] = SeqDesc{kvs[b]->k, kvs[b]->v, kvs[b]->len, kvs[b]->cap};
        total_visible += kvs[b]->len + 1;
        max_visible = std::max(max_visible, kvs[b]->len + 1);
    }
    CU(cudaMemcpyAsync(dd, hd, sizeof(SeqDesc) * batch, cudaMemcpyHostToDevice, s));
    CU(cudaEventRecord(ctx->seq_ev[slot], s));
    SeqRef seqs{};
    seqs.many = dd;
    rc = run_step(ctx, first, seqs, batch, 1, total_visible, max_visible, q, k_new, v_new, out, scale, flags, s);
    if (rc) return rc;
    for (int b = 0; b < batch; ++b) kvs[b]->len += 1;
    return SHAINET_ATTN_OK;
}

// ---- reference-signature entry points (legacy default stream) ----

void kv_cache_append_f32(const float* staging, float* kc, float* vc, int new_tokens, int start_pos,
                         int num_kv_heads, int head_dim, int capacity) {
    cudaError_t e = launch_ref_append(staging, kc, vc, new_tokens, start_pos, num_kv_heads, head_dim, capacity, 0);
    if (e != cudaSuccess) printf("CUDA Error in kv_cache_append_f32: %s\n", cudaGetErrorString(e));
}

void attention_kv_f32(const float* q, const float* kc, const float* vc, float* out, float* ws, int new_tokens,
                      int start_pos, int num_heads, int heads_per_kv, int head_dim, int capacity, float scale) {
    if (new_tokens <= 0 || num_heads <= 0 || heads_per_kv <= 0 || num_heads % heads_per_kv != 0) return;
    AttnArgs a{};
    a.q_rot = q;
    a.out = out;
    a.seqs.one = SeqDesc{const_cast<float*>(kc), const_cast<float*>(vc), start_pos, capacity};
    a.seqs.many = nullptr;
    a.batch = 1;
    a.T = new_tokens;
    a.hs = HeadShape{num_heads, num_heads / heads_per_kv, head_dim};
    a.scale = scale;
    a.status = nullptr;
    cudaError_t e = cudaSuccess;
    const int total_len = start_pos + new_tokens;
    bool done = false;
    if (splitk_supported(a.hs) && new_tokens <= SPLITK_MAX_T && aligned16(q) && aligned16(kc) && aligned16(vc) && aligned16(out)) {
        int sm = 148, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
        const long long tv = (long long)new_tokens * start_pos + (long long)new_tokens * (new_tokens + 1) / 2;
        plan_splits(sm, a.hs, new_tokens, tv, total_len, 1, &a.chunk_rows, &a.max_splits);
        // The caller's scratch holds num_heads*new_tokens*total_len floats; use it
        // for the split partials when they fit, otherwise take fewer splits.
        const long long ws_floats = (long long)num_heads * new_tokens * total_len;
        while (a.max_splits > 1 && (long long)splitk_scratch_floats(a.hs, new_tokens, a.max_splits) > ws_floats) {
            a.chunk_rows *= 2;
            a.max_splits = (total_len + a.chunk_rows - 1) / a.chunk_rows;
        }
        if (a.max_splits == 1 || (ws && aligned16(ws))) {
            a.part_o = ws;
            a.part_ml = ws + (size_t)new_tokens * num_heads * a.max_splits * head_dim;
            e = launch_attn_splitk(a, 0);
            done = true;
        }
    }
    if (!done) {
        if (head_dim > 256 || head_dim <= 0) {
            printf("CUDA Error in attention_kv_f32: head_dim %d not supported\n", head_dim);
            return;
        }
        e = launch_attn_generic(a, 0);
    }
    if (e != cudaSuccess) printf("CUDA Error in attention_kv_f32: %s\n", cudaGetErrorString(e));
}

}  // extern "C"
