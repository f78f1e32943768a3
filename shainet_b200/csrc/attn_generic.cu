// Shape-agnostic causal attention over the KV cache: any even head_dim <= 256,
// any query-heads-per-kv-head ratio, any number of new tokens.  One CTA per
// (query head, row); each warp streams a strided subset of the visible cache
// rows with a single-pass (online) softmax and the four warps are merged in
// shared memory, so no global scratch is needed.
//
// Same contract as the reference's attention_kv_kernel
// (src/shainet/native/cuda_kernels.cu:734-806): visible = start_pos + i + 1,
// query head h reads kv head h / heads_per_kv, out = softmax(scale * q.K^T) V.
// It serves the shapes the tuned kernels do not cover (the reference's spec
// shapes use head_dim 4 and 8).
#include <math.h>
#include "kernels.h"

namespace shainet {

namespace {

constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_C = 8;  // head_dim <= 256

__global__ void __launch_bounds__(GEN_WARPS * 32) attn_generic_kernel(AttnArgs a) {
    extern __shared__ float gen_smem[];  // [GEN_WARPS][hd + 2]
    const int h = blockIdx.x;
    const int r = blockIdx.y;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads, hd = a.hs.head_dim;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int visible = sd.start + t + 1;
    const int kv_h = h / (H / KV);
    const float* kh = sd.k + (size_t)kv_h * sd.capacity * hd;
    const float* vh = sd.v + (size_t)kv_h * sd.capacity * hd;
    const float* qv = a.q_rot + ((size_t)r * H + h) * hd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float q[GEN_MAX_C], o[GEN_MAX_C];
#pragma unroll
    for (int c = 0; c < GEN_MAX_C; ++c) {
        const int d = lane + 32 * c;
        q[c] = d < hd ? qv[d] : 0.0f;
        o[c] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int j = warp; j < visible; j += GEN_WARPS) {
        const float* kr = kh + (size_t)j * hd;
        const float* vr = vh + (size_t)j * hd;
        float dot = 0.0f;
        float vv[GEN_MAX_C];
#pragma unroll
        for (int c = 0; c < GEN_MAX_C; ++c) {
            const int d = lane + 32 * c;
            if (d < hd) {
                dot = fmaf(q[c], kr[d], dot);
                vv[c] = vr[d];
            } else {
                vv[c] = 0.0f;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float s = dot * a.scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);  // m = -inf on the first row gives 0
        const float p = expf(s - m_new);
        l = fmaf(l, alpha, p);
#pragma unroll
        for (int c = 0; c < GEN_MAX_C; ++c) o[c] = fmaf(o[c], alpha, p * vv[c]);
        m = m_new;
    }

    float* mine = gen_smem + warp * (hd + 2);
#pragma unroll
    for (int c = 0; c < GEN_MAX_C; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) mine[d] = o[c];
    }
    if (lane == 0) {
        mine[hd] = m;
        mine[hd + 1] = l;
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) M = fmaxf(M, gen_smem[w * (hd + 2) + hd]);
    float wgt[GEN_WARPS], L = 0.0f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) {
        const float mw = gen_smem[w * (hd + 2) + hd];
        wgt[w] = (mw == -INFINITY) ? 0.0f : expf(mw - M);
        L = fmaf(wgt[w], gen_smem[w * (hd + 2) + hd + 1], L);
    }
    const float invL = 1.0f / L;
    float* orow = a.out + ((size_t)r * H + h) * hd;
    for (int d = threadIdx.x; d < hd; d += GEN_WARPS * 32) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < GEN_WARPS; ++w) acc = fmaf(wgt[w], gen_smem[w * (hd + 2) + d], acc);
        orow[d] = acc * invL;
    }
}

}  // namespace

cudaError_t launch_attn_generic(const AttnArgs& a, cudaStream_t s) {
    const long long rows = (long long)a.batch * a.T;
    if (rows == 0) return cudaSuccess;
    if (rows > 65535) {
        // grid.y limit: issue in slabs of rows
        AttnArgs part = a;
        if (a.batch != 1) return cudaErrorInvalidValue;
        // Only a single sequence can have this many rows; walk T in slabs by
        // shifting the row origin through q/out pointers and `start`.
        const size_t stride = (size_t)a.hs.num_heads * a.hs.head_dim;
        for (long long r0 = 0; r0 < rows; r0 += 32768) {
            const int n = (int)((rows - r0) < 32768 ? (rows - r0) : 32768);
            part.q_rot = a.q_rot + r0 * stride;
            part.out = a.out + r0 * stride;
            part.T = n;
            part.seqs.one.start = a.seqs.one.start + (int)r0;
            cudaError_t e = launch_attn_generic(part, s);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    dim3 grid(a.hs.num_heads, (unsigned)rows);
    const size_t smem = (size_t)GEN_WARPS * (a.hs.head_dim + 2) * sizeof(float);
    attn_generic_kernel<<<grid, GEN_WARPS * 32, smem, s>>>(a);
    return cudaGetLastError();
}

}  // namespace shainet
