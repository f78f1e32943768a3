// Split-K flash-decode over the fp32 KV cache, CUDA cores, sm_100a.
//
// Replaces the reference's attention_kv_kernel
// (src/shainet/native/cuda_kernels.cu:734-806) for decode rows.  The reference
// launches one 128-thread CTA per (query head, token): 32 CTAs for a 32-head
// model, every query head of a group re-reading its kv head's K and V, scores
// round-tripping through a global scratch.  Here:
//
//  * the visible cache rows of one kv head are cut into `chunk_rows`-sized
//    splits; one CTA per (split, kv head, row) streams its slice ONCE for all
//    G = heads_per_kv query heads of the group;
//  * a producer warp moves K and V tiles global -> shared with 1-D bulk
//    asynchronous copies (the TMA engine; no tensor map, no multicast) through
//    a ring of mbarrier-guarded stages, so tens of KB per SM are in flight
//    without holding registers;
//  * each consumer warp owns whole tiles: q lives in registers (16 lanes per K
//    row, 128-bit shared loads), the 16 x G partial dot products of a batch of
//    rows are reduce-scattered across the half-warp so every lane ends with one
//    score, the softmax is the single-pass (online) form kept per warp, and
//    P.V runs with one lane per four output columns;
//  * per-split (max, sum, unnormalised output) go to a small scratch and a
//    second kernel merges the splits.
//
// All waits are bounded (see mbar_wait); a timed-out wait records a status
// word and the kernel unwinds.
#include <math.h>
#include "kernels.h"

namespace shainet {

namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int SK_MAX_STAGES = 32;

// Tile geometry.  R*G = 16 scores per half-warp per batch, so a batch is
// BR = 2*16/G rows; a warp tile is a whole number of batches.  The ring has a
// multiple of NW stages so that every stage is always consumed by the same
// warp: an mbarrier phase wait is only meaningful for a waiter that saw the
// previous phase, which a fixed stage->warp map guarantees.
template <int HD, int G>
struct SKDefault {
    static constexpr int BR = 2 * (16 / G);
    static constexpr int TW = BR > 8 ? BR : 8;                         // rows per warp tile
    static constexpr int NW = (2 * TW * HD * 4 > 16 * 1024) ? 4 : 8;   // consumer warps
    static constexpr int SMEM_KB = 200;                                // one CTA per SM
    static constexpr int CTAS_PER_SM = 1;
};

template <int HD, int G, int TW_ = SKDefault<HD, G>::TW, int NW_ = SKDefault<HD, G>::NW,
          int SMEM_KB_ = SKDefault<HD, G>::SMEM_KB, int CTAS_ = SKDefault<HD, G>::CTAS_PER_SM, bool MATH_ = true>
struct SK {
    static constexpr int NW = NW_;                     // consumer warps
    static constexpr int CPL = HD / 64;                // 16-byte chunks per lane per K row
    static constexpr int R = 16 / G;                   // rows per half-warp per batch
    static constexpr int BR = 2 * R;                   // rows per batch
    static constexpr int TW = TW_;                     // rows per warp tile
    static constexpr int NB = TW / BR;                 // batches per tile
    static constexpr int TILE_FLOATS = TW * HD;        // per tensor
    static constexpr int STAGE_FLOATS = 2 * TILE_FLOATS;
    static constexpr int RPI = 128 / HD;               // V rows covered by one warp-wide 128-bit load
    static constexpr int WARP_SCRATCH = 32 + 16;       // p[BR*G = 32] + alpha[G <= 16]
    static constexpr int THREADS = (NW + 1) * 32;
    static constexpr int CTAS_PER_SM = CTAS_;
    static constexpr bool MATH = MATH_;
    static constexpr int FIXED_BYTES = NW * WARP_SCRATCH * 4 + 2 * SK_MAX_STAGES * 8;
    static constexpr int NS_RAW = (SMEM_KB_ * 1024 - FIXED_BYTES) / (STAGE_FLOATS * 4);
    static constexpr int NS_CAP = NS_RAW > SK_MAX_STAGES ? SK_MAX_STAGES : NS_RAW;
    static constexpr int NS = NS_CAP / NW * NW;        // ring stages, a multiple of NW
    static constexpr int MERGE_FLOATS = NW * G * (HD + 2);
    static constexpr size_t SMEM_BYTES = (size_t)NS * STAGE_FLOATS * 4 + FIXED_BYTES;
    static_assert(HD == 64 || HD == 128, "head_dim");
    static_assert(G == 1 || G == 2 || G == 4 || G == 8 || G == 16, "group size");
    static_assert(TW % BR == 0, "a warp tile is a whole number of batches");
    static_assert(NS >= NW, "ring shorter than the number of consumer warps");
    static_assert(MERGE_FLOATS <= NS * STAGE_FLOATS, "merge area must fit in the ring");
};

// 16-lane reduce-scatter of 16 values: on return acc[0] of lane i (i = lane & 15)
// holds the sum over the half-warp of the callers' acc[i].
__device__ __forceinline__ void reduce_scatter16(float (&acc)[16], int lane) {
#pragma unroll
    for (int step = 0; step < 4; ++step) {
        const int off = 8 >> step;
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (k < off) {
                const float lo = acc[k], hi = acc[k + off];
                const float send = up ? lo : hi;
                const float keep = up ? hi : lo;
                acc[k] = keep + __shfl_xor_sync(FULL, send, off);
            }
        }
    }
}

template <int HD, int G, class C>
__global__ void __launch_bounds__(C::THREADS, C::CTAS_PER_SM) attn_splitk_kernel(AttnArgs a) {
    constexpr int NS = C::NS;
    extern __shared__ __align__(1024) unsigned char sk_smem_raw[];
    float* stages = reinterpret_cast<float*>(sk_smem_raw);
    float* warp_scratch = stages + (size_t)NS * C::STAGE_FLOATS;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(warp_scratch + C::NW * C::WARP_SCRATCH);
    uint64_t* empty_bar = full_bar + NS;

    const int split = blockIdx.x, kv_h = blockIdx.y, r = blockIdx.z;
    const int H = a.hs.num_heads;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int visible = sd.start + t + 1;
    const int row0 = split * a.chunk_rows;
    if (row0 >= visible) return;  // whole CTA: this sequence has fewer splits
    const int row1 = min(row0 + a.chunk_rows, visible);
    const int ntiles = (row1 - row0 + C::TW - 1) / C::TW;
    const float* kbase = sd.k + ((size_t)kv_h * sd.capacity + row0) * HD;
    const float* vbase = sd.v + ((size_t)kv_h * sd.capacity + row0) * HD;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();

    // Per-warp running state (consumers only; declared here so the merge below sees it).
    float o[G][4];
    float m_run = -INFINITY, l_run = 0.0f;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 4; ++k) o[g][k] = 0.0f;

    if (warp == C::NW) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int i = 0; i < ntiles; ++i) {
                const int s = i % NS;
                if (i >= NS && !mbar_wait(&empty_bar[s], ((i / NS) - 1) & 1, a.status, 1)) break;
                const int nrows = min(C::TW, (row1 - row0) - i * C::TW);
                const uint32_t bytes = (uint32_t)nrows * HD * 4;
                float* ks = stages + (size_t)s * C::STAGE_FLOATS;
                float* vs = ks + C::TILE_FLOATS;
                mbar_arrive_expect_tx(&full_bar[s], 2 * bytes);
                bulk_g2s(ks, kbase + (size_t)i * C::TILE_FLOATS, bytes, &full_bar[s]);
                bulk_g2s(vs, vbase + (size_t)i * C::TILE_FLOATS, bytes, &full_bar[s]);
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int i16 = lane & 15, hw = lane >> 4;
        const int my_r = hw * C::R + i16 / G;  // row in batch of this lane's score (its head is i16 % G)
        float* ps = warp_scratch + warp * C::WARP_SCRATCH;
        float* as = ps + 32;

        // q for the G heads of this kv head, this lane's 4*CPL columns of each.
        float4 q[G][C::CPL];
        {
            const float* qrow = a.q_rot + ((size_t)r * H + (size_t)kv_h * G) * HD;
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int c = 0; c < C::CPL; ++c)
                    q[g][c] = *reinterpret_cast<const float4*>(qrow + (size_t)g * HD + (c * 16 + i16) * 4);
        }

        for (int i = warp; i < ntiles; i += C::NW) {
            const int s = i % NS;
            if (!mbar_wait(&full_bar[s], (i / NS) & 1, a.status, 2)) break;
            const float* ks = stages + (size_t)s * C::STAGE_FLOATS;
            const float* vs = ks + C::TILE_FLOATS;
            const int nrows = min(C::TW, (row1 - row0) - i * C::TW);

#pragma unroll
            for (int bb = 0; bb < (C::MATH ? C::NB : 0); ++bb) {
                const int base = bb * C::BR;
                if (base >= nrows) break;  // warp-uniform
                // ---- scores: acc[rr*G + g] for the R rows of this half-warp ----
                float acc[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) acc[k] = 0.0f;
#pragma unroll
                for (int rr = 0; rr < C::R; ++rr) {
                    const float* krow = ks + (size_t)(base + hw * C::R + rr) * HD;
#pragma unroll
                    for (int c = 0; c < C::CPL; ++c) {
                        const float4 kk = lds128(krow + (c * 16 + i16) * 4);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            float v = acc[rr * G + g];
                            v = fmaf(q[g][c].x, kk.x, v);
                            v = fmaf(q[g][c].y, kk.y, v);
                            v = fmaf(q[g][c].z, kk.z, v);
                            v = fmaf(q[g][c].w, kk.w, v);
                            acc[rr * G + g] = v;
                        }
                    }
                }
                reduce_scatter16(acc, lane);
                float sc = acc[0] * a.scale;
                if (base + my_r >= nrows) sc = -INFINITY;  // rows past the end of the slice
                // ---- online softmax for head my_g ----
                float bmax = sc;
#pragma unroll
                for (int off = G; off < 32; off <<= 1) bmax = fmaxf(bmax, __shfl_xor_sync(FULL, bmax, off));
                const float m_new = fmaxf(m_run, bmax);
                const float alpha = exp2f((m_run - m_new) * LOG2E);  // 0 while m_run is -inf
                const float p = exp2f((sc - m_new) * LOG2E);
                l_run = fmaf(l_run, alpha, p);
                m_run = m_new;
                __syncwarp();  // previous batch's reads of ps/as are done
                ps[lane] = p;  // index = row_in_batch * G + head
                if (lane < G) as[lane] = alpha;
                const bool rescale = __any_sync(FULL, alpha != 1.0f);
                __syncwarp();
                if (rescale) {
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float al = as[g];
#pragma unroll
                        for (int k = 0; k < 4; ++k) o[g][k] *= al;
                    }
                }
                // ---- o += P.V ----
#pragma unroll
                for (int rr = 0; rr < C::BR; rr += C::RPI) {
                    const int row = base + rr + (C::RPI == 2 ? hw : 0);
                    if (base + rr >= nrows) break;  // warp-uniform
                    if (row < nrows) {
                        const int col = (C::RPI == 2 ? i16 : lane) * 4;
                        const float4 vv = lds128(vs + (size_t)row * HD + col);
                        const float* prow = ps + (row - base) * G;
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            const float pg = prow[g];
                            o[g][0] = fmaf(pg, vv.x, o[g][0]);
                            o[g][1] = fmaf(pg, vv.y, o[g][1]);
                            o[g][2] = fmaf(pg, vv.z, o[g][2]);
                            o[g][3] = fmaf(pg, vv.w, o[g][3]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }

        // Sum of p over the lanes that share a head.
#pragma unroll
        for (int off = G; off < 32; off <<= 1) l_run += __shfl_xor_sync(FULL, l_run, off);
        if (C::RPI == 2) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int k = 0; k < 4; ++k) o[g][k] += __shfl_xor_sync(FULL, o[g][k], 16);
        }
    }

    // All tiles are consumed (or abandoned after a timeout): every bulk copy
    // that was issued has landed, so the stage memory can be reused.
    __syncthreads();
    float* mo = stages;                               // [NW][G][HD]
    float* mm = mo + (size_t)C::NW * G * HD;          // [NW][G]
    float* ml = mm + C::NW * G;                       // [NW][G]
    if (warp < C::NW) {
        if (lane < G) {
            mm[warp * G + lane] = m_run;  // lane < G holds head `lane`
            ml[warp * G + lane] = l_run;
        }
        if (C::RPI == 1 || lane < 16) {
#pragma unroll
            for (int g = 0; g < G; ++g)
                *reinterpret_cast<float4*>(mo + ((size_t)warp * G + g) * HD + lane * 4) =
                    make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
        }
    }
    __syncthreads();
    const int nsplit_here = (visible + a.chunk_rows - 1) / a.chunk_rows;
    for (int e = threadIdx.x; e < G * HD; e += C::THREADS) {
        const int g = e / HD, d = e - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < C::NW; ++w) M = fmaxf(M, mm[w * G + g]);
        float L = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < C::NW; ++w) {
            const float mw = mm[w * G + g];
            const float wt = (mw == -INFINITY) ? 0.0f : exp2f((mw - M) * LOG2E);
            L = fmaf(wt, ml[w * G + g], L);
            acc = fmaf(wt, mo[((size_t)w * G + g) * HD + d], acc);
        }
        const int h = kv_h * G + g;
        if (nsplit_here == 1) {
            a.out[((size_t)r * H + h) * HD + d] = acc / L;
        } else {
            const size_t pidx = ((size_t)r * H + h) * a.max_splits + split;
            a.part_o[pidx * HD + d] = acc;
            if (d == 0) {
                a.part_ml[pidx * 2] = M;
                a.part_ml[pidx * 2 + 1] = L;
            }
        }
    }
}

// Merge of the per-split partials: out = sum_s w_s o_s / sum_s w_s l_s with
// w_s = exp(m_s - max m).  One CTA per (query head, row), one thread per column.
template <int HD>
__global__ void __launch_bounds__(HD) attn_combine_kernel(AttnArgs a) {
    const int h = blockIdx.x, r = blockIdx.y;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int visible = sd.start + t + 1;
    const int ns = (visible + a.chunk_rows - 1) / a.chunk_rows;
    if (ns <= 1) return;  // the split kernel already wrote the row
    const size_t p0 = ((size_t)r * a.hs.num_heads + h) * a.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, a.part_ml[(p0 + s) * 2]);
    float L = 0.0f, acc = 0.0f;
    const int d = threadIdx.x;
    for (int s = 0; s < ns; ++s) {
        const float w = exp2f((a.part_ml[(p0 + s) * 2] - M) * LOG2E);
        L = fmaf(w, a.part_ml[(p0 + s) * 2 + 1], L);
        acc = fmaf(w, a.part_o[(p0 + s) * HD + d], acc);
    }
    a.out[((size_t)r * a.hs.num_heads + h) * HD + d] = acc / L;
}

template <int HD, int G, class C = SK<HD, G>>
cudaError_t launch_sk(const AttnArgs& a, cudaStream_t s) {
    const size_t smem = C::SMEM_BYTES;
    static unsigned long long configured = 0;  // bit per device
    cudaError_t e;
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64 || !(configured >> dev & 1ull)) {
        e = cudaFuncSetAttribute(attn_splitk_kernel<HD, G, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev < 64) configured |= 1ull << dev;
    }
    const int rows = a.batch * a.T;
    dim3 grid(a.max_splits, a.hs.num_kv_heads, rows);
    attn_splitk_kernel<HD, G, C><<<grid, C::THREADS, smem, s>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (a.max_splits > 1) {
        dim3 cg(a.hs.num_heads, rows);
        attn_combine_kernel<HD><<<cg, HD, 0, s>>>(a);
        e = cudaGetLastError();
    }
    return e;
}

template <int HD>
cudaError_t dispatch_g(const AttnArgs& a, cudaStream_t s) {
    switch (a.hs.num_heads / a.hs.num_kv_heads) {
        case 1: return launch_sk<HD, 1>(a, s);
        case 2: return launch_sk<HD, 2>(a, s);
        case 4: return launch_sk<HD, 4>(a, s);
        case 8: return launch_sk<HD, 8>(a, s);
        case 16: return launch_sk<HD, 16>(a, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

bool splitk_supported(const HeadShape& hs) {
    const int g = hs.num_heads / hs.num_kv_heads;
    return (hs.head_dim == 64 || hs.head_dim == 128) && (g == 1 || g == 2 || g == 4 || g == 8 || g == 16);
}

int splitk_tile_rows(const HeadShape& hs) {
    const int g = hs.num_heads / hs.num_kv_heads;
    const int br = 2 * (16 / g);
    return br > 8 ? br : 8;
}

size_t splitk_scratch_floats(const HeadShape& hs, int rows, int max_splits) {
    return (size_t)rows * hs.num_heads * max_splits * (hs.head_dim + 2);
}

cudaError_t launch_attn_splitk(const AttnArgs& a, cudaStream_t s) {
    if (a.batch * a.T == 0) return cudaSuccess;
    if (a.hs.head_dim == 64) return dispatch_g<64>(a, s);
    if (a.hs.head_dim == 128) return dispatch_g<128>(a, s);
    return cudaErrorInvalidValue;
}

}  // namespace shainet
