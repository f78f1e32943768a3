// Fused (bias +) per-head RMSNorm + RoPE + KV-cache append.
//
// Replaces, in one launch, the host loops of the reference between the q/k/v
// projections and the attention kernel:
//   add_bias!            src/shainet/transformer/llama_block.cr:585-601
//   apply_head_rmsnorm!  src/shainet/transformer/llama_block.cr:615-641
//   K RoPE + append      src/shainet/transformer/llama_block.cr:266-286
//   Q RoPE               src/shainet/transformer/llama_block.cr:440-467
//   kv_cache_append_f32  src/shainet/native/cuda_kernels.cu:695-726
//
// Every arithmetic step uses the reference's order with explicitly rounded,
// unfused fp32 operations (the Crystal build does not contract a*b+c), so the
// cache contents differ from the host path only by the ulp-level difference
// between the device's and libm's cosf/sinf.
#include <cuda_bf16.h>

#include "kernels.h"

namespace shainet {

namespace {

constexpr int PREP_WARPS = 4;
constexpr int PREP_THREADS = PREP_WARPS * 32;

// One CTA per new token.  All of the token's q, k and v heads are staged in
// shared memory (rows padded by one float), so that
//   * cos/sin of the token's position are computed once and shared by every head,
//   * the per-head sum of squares keeps the host loop's strictly sequential
//     order, but 32 heads run their chains side by side (one per lane) instead
//     of one lane working while 31 wait.
__global__ void __launch_bounds__(PREP_THREADS) prep_append_kernel(PrepArgs a) {
    extern __shared__ __align__(16) float prep_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads, hd = a.hs.head_dim;
    const int per_row = H + 2 * KV;
    const int half = hd >> 1;
    // Rows arrive by bulk copies (TMA engine) when they are 16-byte multiples at 16-byte addresses: all of a
    // token's 24 KB are then in flight at once without holding registers.  Such rows are padded by four floats
    // (the copies need 16-byte destinations); otherwise by one (conflict-free column walks).
    const bool vec = (hd & 3) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(a.k_new) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.v_new) & 15u) == 0;
    const int stride = vec ? hd + 4 : hd + 1;
    uint64_t* bar = reinterpret_cast<uint64_t*>(prep_smem);   // 16 bytes reserved
    float* buf = prep_smem + 4;          // [per_row][stride], 16-byte aligned
    float* cs = buf + (size_t)per_row * stride;   // [half]
    float* sn = cs + half;               // [half]
    float* inv = sn + half;              // [H + KV]

    const int r = blockIdx.x;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int pos = sd.start + t;
    const float fpos = (float)pos;

    for (int i = threadIdx.x; i < half; i += PREP_THREADS) {
        const float angle = __fmul_rn(fpos, a.inv_freq[i]);
        float s_, c_;
        sincosf(angle, &s_, &c_);
        cs[i] = c_;
        sn[i] = s_;
    }
    // Stage the token's rows in shared memory.
    auto slot_src = [&](int slot, const float*& src, const float*& bias) {
        if (slot < H) {
            src = a.q + ((size_t)r * H + slot) * hd;
            bias = a.b_q ? a.b_q + (size_t)slot * hd : nullptr;
        } else if (slot < H + KV) {
            src = a.k_new + ((size_t)r * KV + (slot - H)) * hd;
            bias = a.b_k ? a.b_k + (size_t)(slot - H) * hd : nullptr;
        } else {
            src = a.v_new + ((size_t)r * KV + (slot - H - KV)) * hd;
            bias = a.b_v ? a.b_v + (size_t)(slot - H - KV) * hd : nullptr;
        }
    };
    if (vec) {
        if (threadIdx.x == 0) {
            mbar_init(bar, 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            mbar_arrive_expect_tx(bar, (uint32_t)per_row * hd * 4);
            for (int slot = 0; slot < per_row; ++slot) {
                const float* src;
                const float* bias;
                slot_src(slot, src, bias);
                bulk_g2s(buf + (size_t)slot * stride, src, (uint32_t)hd * 4, bar);
            }
        }
        if (!mbar_wait(bar, 0, a.status, 31)) return;   // bounded; the whole CTA sees the same outcome
        if (a.b_q != nullptr || a.b_k != nullptr || a.b_v != nullptr) {
            for (int slot = warp; slot < per_row; slot += PREP_WARPS) {
                const float* src;
                const float* bias;
                slot_src(slot, src, bias);
                if (bias == nullptr) continue;
                float* row = buf + (size_t)slot * stride;
                for (int d = lane; d < hd; d += 32) row[d] = __fadd_rn(row[d], bias[d]);
            }
        }
    } else {
        for (int slot = warp; slot < per_row; slot += PREP_WARPS) {
            const float* src;
            const float* bias;
            slot_src(slot, src, bias);
            float* row = buf + (size_t)slot * stride;
            for (int d = lane; d < hd; d += 32) {
                float x = src[d];
                if (bias) x = __fadd_rn(x, bias[d]);
                row[d] = x;
            }
        }
    }
    __syncthreads();
    const bool normed = a.q_norm != nullptr || a.k_norm != nullptr;
    if (normed) {
        for (int slot = threadIdx.x; slot < H + KV; slot += PREP_THREADS) {
            // Sequential fp32 sum in ascending d, as the host loop does.
            const float* row = buf + (size_t)slot * stride;
            float ss = 0.0f;
            for (int d = 0; d < hd; ++d) ss = __fadd_rn(ss, __fmul_rn(row[d], row[d]));
            const float mean = __fdiv_rn(ss, (float)hd);
            inv[slot] = (float)(1.0 / sqrt((double)mean + a.eps));
        }
        __syncthreads();
    }
    for (int slot = warp; slot < per_row; slot += PREP_WARPS) {
        const float* row = buf + (size_t)slot * stride;
        if (slot >= H + KV) {
            const size_t e0 = ((size_t)(slot - H - KV) * sd.capacity + pos) * hd;
            if (a.kv_elem_bytes == 2) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sd.v) + e0;
                for (int d = lane; d < hd; d += 32) dst[d] = __float2bfloat16_rn(row[d]);
            } else {
                float* dst = sd.v + e0;
                for (int d = lane; d < hd; d += 32) dst[d] = row[d];
            }
            continue;
        }
        const bool is_q = slot < H;
        const float* w = is_q ? a.q_norm : a.k_norm;
        const size_t k0 = is_q ? 0 : ((size_t)(slot - H) * sd.capacity + pos) * hd;
        const bool k16 = !is_q && a.kv_elem_bytes == 2;   // bfloat16 cache: rotated k rows are rounded to nearest even
        float* dst = is_q ? a.q_rot + ((size_t)r * H + slot) * hd : sd.k + k0;
        __nv_bfloat16* dst16 = reinterpret_cast<__nv_bfloat16*>(sd.k) + k0;
        const float iv = normed ? inv[slot] : 1.0f;
        for (int i = lane; i < half; i += 32) {
            float x0 = row[i], x1 = row[i + half];
            if (w) {
                x0 = __fmul_rn(__fmul_rn(x0, iv), w[i]);
                x1 = __fmul_rn(__fmul_rn(x1, iv), w[i + half]);
            }
            const float c = cs[i], s_ = sn[i];
            float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s_));
            float y1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s_));
            if (a.round_q_tf32 && is_q) {
                // q only: the cache keeps full fp32 rows
                unsigned u0, u1;
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u0) : "f"(y0));
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u1) : "f"(y1));
                y0 = __uint_as_float(u0);
                y1 = __uint_as_float(u1);
            }
            if (k16) {
                dst16[i] = __float2bfloat16_rn(y0);
                dst16[i + half] = __float2bfloat16_rn(y1);
            } else {
                dst[i] = y0;
                dst[i + half] = y1;
            }
        }
    }
}

// The same kernel for head_dim 64 and 128 with rows that arrive by bulk copies (16-byte aligned inputs): the loops are
// unrolled, a lane's cos/sin and norm weights stay in registers over all of the token's heads, and the sequential sums
// read four floats per load.  Arithmetic and its order are those of the kernel above; it only issues a third of the
// instructions (the general kernel is bound by its instruction count, not by memory).
template <int HD>
__global__ void __launch_bounds__(PREP_THREADS) prep_append_hd_kernel(PrepArgs a) {
    extern __shared__ __align__(16) float prep_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads;
    const int per_row = H + 2 * KV;
    constexpr int HALF = HD / 2, STRIDE = HD + 4, PL = HALF / 32;   // rotation pairs per lane
    uint64_t* bar = reinterpret_cast<uint64_t*>(prep_smem);   // 16 bytes reserved
    float* buf = prep_smem + 4;          // [per_row][STRIDE], 16-byte aligned
    float* inv = buf + (size_t)per_row * STRIDE;   // [H + KV]

    const int r = blockIdx.x;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int pos = sd.start + t;
    const float fpos = (float)pos;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(bar, (uint32_t)per_row * HD * 4);
        for (int slot = 0; slot < per_row; ++slot) {
            const float* src = slot < H ? a.q + ((size_t)r * H + slot) * HD
                             : slot < H + KV ? a.k_new + ((size_t)r * KV + (slot - H)) * HD
                                             : a.v_new + ((size_t)r * KV + (slot - H - KV)) * HD;
            bulk_g2s(buf + (size_t)slot * STRIDE, src, (uint32_t)HD * 4, bar);
        }
    }
    // this lane's rotation pairs (i, i + HALF), i = lane + 32 k: angle, norm weights
    float cs[PL], sn[PL], wq0[PL], wq1[PL], wk0[PL], wk1[PL];
#pragma unroll
    for (int k = 0; k < PL; ++k) {
        const int i = lane + 32 * k;
        sincosf(__fmul_rn(fpos, a.inv_freq[i]), &sn[k], &cs[k]);
        wq0[k] = a.q_norm ? a.q_norm[i] : 1.0f;
        wq1[k] = a.q_norm ? a.q_norm[i + HALF] : 1.0f;
        wk0[k] = a.k_norm ? a.k_norm[i] : 1.0f;
        wk1[k] = a.k_norm ? a.k_norm[i + HALF] : 1.0f;
    }
    if (!mbar_wait(bar, 0, a.status, 31)) return;   // bounded; the whole CTA sees the same outcome
    if (a.b_q != nullptr || a.b_k != nullptr || a.b_v != nullptr) {
        for (int slot = warp; slot < per_row; slot += PREP_WARPS) {
            const float* bias = slot < H ? (a.b_q ? a.b_q + (size_t)slot * HD : nullptr)
                              : slot < H + KV ? (a.b_k ? a.b_k + (size_t)(slot - H) * HD : nullptr)
                                              : (a.b_v ? a.b_v + (size_t)(slot - H - KV) * HD : nullptr);
            if (bias == nullptr) continue;
            float* row = buf + (size_t)slot * STRIDE;
#pragma unroll
            for (int d = lane; d < HD; d += 32) row[d] = __fadd_rn(row[d], bias[d]);
        }
        __syncthreads();
    }
    const bool normed = a.q_norm != nullptr || a.k_norm != nullptr;
    if (normed) {
        for (int slot = threadIdx.x; slot < H + KV; slot += PREP_THREADS) {
            // sequential fp32 sum in ascending d, as the host loop does; four floats per load
            const float4* row = reinterpret_cast<const float4*>(buf + (size_t)slot * STRIDE);
            float ss = 0.0f;
#pragma unroll
            for (int d4 = 0; d4 < HD / 4; ++d4) {
                const float4 v = row[d4];
                ss = __fadd_rn(ss, __fmul_rn(v.x, v.x));
                ss = __fadd_rn(ss, __fmul_rn(v.y, v.y));
                ss = __fadd_rn(ss, __fmul_rn(v.z, v.z));
                ss = __fadd_rn(ss, __fmul_rn(v.w, v.w));
            }
            const float mean = __fdiv_rn(ss, (float)HD);
            inv[slot] = (float)(1.0 / sqrt((double)mean + a.eps));
        }
        __syncthreads();
    }
    for (int slot = warp; slot < per_row; slot += PREP_WARPS) {
        const float* row = buf + (size_t)slot * STRIDE;
        if (slot >= H + KV) {
            const size_t e0 = ((size_t)(slot - H - KV) * sd.capacity + pos) * HD;
            if (a.kv_elem_bytes == 2) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sd.v) + e0;
#pragma unroll
                for (int d = lane; d < HD; d += 32) dst[d] = __float2bfloat16_rn(row[d]);
            } else {
                float* dst = sd.v + e0;
#pragma unroll
                for (int d = lane; d < HD; d += 32) dst[d] = row[d];
            }
            continue;
        }
        const bool is_q = slot < H;
        const bool has_w = (is_q ? a.q_norm : a.k_norm) != nullptr;
        const size_t k0 = is_q ? 0 : ((size_t)(slot - H) * sd.capacity + pos) * HD;
        const bool k16 = !is_q && a.kv_elem_bytes == 2;
        float* dst = is_q ? a.q_rot + ((size_t)r * H + slot) * HD : sd.k + k0;
        __nv_bfloat16* dst16 = reinterpret_cast<__nv_bfloat16*>(sd.k) + k0;
        const float iv = normed ? inv[slot] : 1.0f;
#pragma unroll
        for (int k = 0; k < PL; ++k) {
            const int i = lane + 32 * k;
            float x0 = row[i], x1 = row[i + HALF];
            if (has_w) {
                x0 = __fmul_rn(__fmul_rn(x0, iv), is_q ? wq0[k] : wk0[k]);
                x1 = __fmul_rn(__fmul_rn(x1, iv), is_q ? wq1[k] : wk1[k]);
            }
            float y0 = __fsub_rn(__fmul_rn(x0, cs[k]), __fmul_rn(x1, sn[k]));
            float y1 = __fadd_rn(__fmul_rn(x1, cs[k]), __fmul_rn(x0, sn[k]));
            if (a.round_q_tf32 && is_q) {
                unsigned u0, u1;
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u0) : "f"(y0));
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u1) : "f"(y1));
                y0 = __uint_as_float(u0);
                y1 = __uint_as_float(u1);
            }
            if (k16) {
                dst16[i] = __float2bfloat16_rn(y0);
                dst16[i + HALF] = __float2bfloat16_rn(y1);
            } else {
                dst[i] = y0;
                dst[i + HALF] = y1;
            }
        }
    }
}

// Scatter of already-rotated staging rows, the reference kernel's contract:
// staging = K chunks [kv_head][t][d] followed by V chunks in the same layout.
__global__ void ref_append_kernel(const float4* __restrict__ staging, float* __restrict__ kc, float* __restrict__ vc,
                                  int new_tokens, int start_pos, int num_kv_heads, int hd4, int capacity) {
    const long long chunk = (long long)new_tokens * hd4;
    const long long total = (long long)num_kv_heads * chunk;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < 2 * total;
         idx += (long long)gridDim.x * blockDim.x) {
        const bool is_v = idx >= total;
        const long long rr = is_v ? idx - total : idx;
        const long long kv_h = rr / chunk;
        const long long rem = rr - kv_h * chunk;
        float4* base = reinterpret_cast<float4*>(is_v ? vc : kc);
        base[(kv_h * capacity + start_pos) * hd4 + rem] = staging[idx];
    }
}

__global__ void ref_append_scalar_kernel(const float* __restrict__ staging, float* __restrict__ kc,
                                         float* __restrict__ vc, int new_tokens, int start_pos, int num_kv_heads,
                                         int hd, int capacity) {
    const long long chunk = (long long)new_tokens * hd;
    const long long total = (long long)num_kv_heads * chunk;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < 2 * total;
         idx += (long long)gridDim.x * blockDim.x) {
        const bool is_v = idx >= total;
        const long long rr = is_v ? idx - total : idx;
        const long long kv_h = rr / chunk;
        const long long rem = rr - kv_h * chunk;
        (is_v ? vc : kc)[(kv_h * capacity + start_pos) * hd + rem] = staging[idx];
    }
}

// Counter-based standard normal: SplitMix64 of (seed, index) -> Box-Muller.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void fill_normal_kernel(float* base, int num_kv_heads, int capacity, int hd, int len,
                                   unsigned long long seed, int elem_bytes) {
    const long long per_head = (long long)len * hd;
    const long long pairs = ((long long)num_kv_heads * per_head + 1) / 2;
    for (long long pidx = (long long)blockIdx.x * blockDim.x + threadIdx.x; pidx < pairs;
         pidx += (long long)gridDim.x * blockDim.x) {
        const unsigned long long bits = splitmix64(seed * 0xD1342543DE82EF95ull + (unsigned long long)pidx);
        const float u1 = ((float)(unsigned)(bits >> 40) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
        const float u2 = (float)(unsigned)((bits >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
        const float rad = sqrtf(-2.0f * logf(u1));
        float s, c;
        sincospif(2.0f * u2, &s, &c);
        const float z[2] = {rad * c, rad * s};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const long long e = 2 * pidx + k;
            if (e < (long long)num_kv_heads * per_head) {
                const long long h = e / per_head, rem = e - h * per_head;
                const long long at = h * (long long)capacity * hd + rem;
                if (elem_bytes == 2) reinterpret_cast<__nv_bfloat16*>(base)[at] = __float2bfloat16_rn(z[k]);
                else base[at] = z[k];
            }
        }
    }
}

// Rows [row0, row0 + rows) of every kv head, two elements per thread and step (head_dim is even).
__global__ void kv_convert_kernel(const void* src, int src_es, long long src_pitch, void* dst, int dst_es,
                                  long long dst_pitch, int num_kv_heads, long long row_elems0, long long elems) {
    const long long pairs_per_head = elems / 2;
    const long long total = pairs_per_head * num_kv_heads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long h = i / pairs_per_head, e = row_elems0 + 2 * (i - h * pairs_per_head);
        float2 v;
        if (src_es == 4) {
            v = *reinterpret_cast<const float2*>(static_cast<const float*>(src) + h * src_pitch + e);
        } else {
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(src) + h * src_pitch + e);
            v = __bfloat1622float2(b);
        }
        if (dst_es == 4) {
            *reinterpret_cast<float2*>(static_cast<float*>(dst) + h * dst_pitch + e) = v;
        } else {
            __nv_bfloat162 b;
            b.x = __float2bfloat16_rn(v.x);
            b.y = __float2bfloat16_rn(v.y);
            *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(dst) + h * dst_pitch + e) = b;
        }
    }
}

}  // namespace

cudaError_t launch_kv_convert(const void* src, int src_elem_bytes, int src_capacity, void* dst, int dst_elem_bytes,
                              int dst_capacity, int num_kv_heads, int head_dim, int row0, int rows, cudaStream_t s) {
    if (rows <= 0 || num_kv_heads <= 0) return cudaSuccess;
    if ((src_elem_bytes != 4 && src_elem_bytes != 2) || (dst_elem_bytes != 4 && dst_elem_bytes != 2) || (head_dim & 1))
        return cudaErrorInvalidValue;
    const long long elems = (long long)rows * head_dim;
    const long long total = elems / 2 * num_kv_heads;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    kv_convert_kernel<<<(unsigned)blocks, 256, 0, s>>>(src, src_elem_bytes, (long long)src_capacity * head_dim, dst,
                                                        dst_elem_bytes, (long long)dst_capacity * head_dim, num_kv_heads,
                                                        (long long)row0 * head_dim, elems);
    return cudaGetLastError();
}

cudaError_t launch_prep_append(const PrepArgs& a, cudaStream_t s) {
    const long long rows = (long long)a.batch * a.T;
    if (rows == 0) return cudaSuccess;
    const int per_row = a.hs.num_heads + 2 * a.hs.num_kv_heads;
    const size_t smem = (4 + (size_t)per_row * (a.hs.head_dim + 4) + a.hs.head_dim + a.hs.num_heads + a.hs.num_kv_heads) * sizeof(float);
    if (smem > 48 * 1024) {
        if (smem > 227 * 1024) return cudaErrorInvalidValue;
        cudaError_t e = cudaFuncSetAttribute(prep_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k_new) | reinterpret_cast<uintptr_t>(a.v_new)) & 15u) == 0;
    if (aligned && smem <= 48 * 1024 && a.hs.head_dim == 128) prep_append_hd_kernel<128><<<(unsigned)rows, PREP_THREADS, smem, s>>>(a);
    else if (aligned && smem <= 48 * 1024 && a.hs.head_dim == 64) prep_append_hd_kernel<64><<<(unsigned)rows, PREP_THREADS, smem, s>>>(a);
    else prep_append_kernel<<<(unsigned)rows, PREP_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_ref_append(const float* staging, float* kc, float* vc, int new_tokens, int start_pos,
                              int num_kv_heads, int head_dim, int capacity, cudaStream_t s) {
    const long long total = 2ll * num_kv_heads * new_tokens * head_dim;
    if (total == 0) return cudaSuccess;
    const bool vec = (head_dim % 4 == 0) && ((((uintptr_t)staging) | ((uintptr_t)kc) | ((uintptr_t)vc)) % 16 == 0);
    const long long work = vec ? total / 4 : total;
    long long blocks = (work + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (vec)
        ref_append_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(staging), kc, vc, new_tokens,
                                                          start_pos, num_kv_heads, head_dim / 4, capacity);
    else
        ref_append_scalar_kernel<<<(unsigned)blocks, 256, 0, s>>>(staging, kc, vc, new_tokens, start_pos, num_kv_heads,
                                                                 head_dim, capacity);
    return cudaGetLastError();
}

cudaError_t launch_fill_normal(float* base, int num_kv_heads, int capacity, int head_dim, int len,
                               unsigned long long seed, int elem_bytes, cudaStream_t s) {
    const long long pairs = ((long long)num_kv_heads * len * head_dim + 1) / 2;
    if (pairs == 0) return cudaSuccess;
    long long blocks = (pairs + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    fill_normal_kernel<<<(unsigned)blocks, 256, 0, s>>>(base, num_kv_heads, capacity, head_dim, len, seed, elem_bytes);
    return cudaGetLastError();
}

}  // namespace shainet
