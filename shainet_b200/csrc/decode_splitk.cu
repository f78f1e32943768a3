// Split-K flash-decode over the fp32 KV cache, CUDA cores, sm_100a.
//
// Replaces the reference's attention_kv_kernel
// (src/shainet/native/cuda_kernels.cu:734-806) for decode rows, and in its fused
// form also the host loops in front of it (bias, per-head RMSNorm, RoPE, cache
// append: src/shainet/transformer/llama_block.cr:257-286, 440-467, 585-641).
// The reference launches one 128-thread CTA per (query head, token): 32 CTAs
// for a 32-head model, every query head of a group re-reading its kv head's K
// and V, scores round-tripping through a global scratch.  Here:
//
//  * the visible cache rows of one kv head are cut into `chunk_rows`-sized
//    splits; one CTA per (split, kv head, row) streams its slice ONCE for all
//    G = heads_per_kv query heads of the group;
//  * a producer warp moves K and V tiles global -> shared with 1-D bulk
//    asynchronous copies (the TMA engine; no tensor map, no multicast) through
//    a ring of mbarrier-guarded stages, so ~100 KB per SM are in flight
//    without holding registers;
//  * each consumer warp owns whole tiles: q lives in registers (16 lanes per K
//    row, 128-bit shared loads), the 16 x G partial dot products of a batch of
//    rows are reduce-scattered across the half-warp so every lane ends with one
//    score, the softmax is the single-pass (online) form kept per warp, and
//    P.V runs with one lane per four output columns; multiply-adds are issued
//    as packed fp32 pairs (fma.rn.f32x2);
//  * per-split (max, sum, unnormalised output) go to a small scratch.  The
//    plain kernel leaves the merge to a second kernel; the fused kernel lets
//    the last CTA of each kv head (an atomic ticket, no waiting) do it.
//
// The fused kernel is launched with programmatic stream serialization: it
// prefetches cache tiles that no running kernel can still be writing, then
// waits for the previous grid, then lets the next grid start.  Consecutive
// layers therefore hand SMs over one CTA at a time instead of draining the GPU
// between launches.
//
// All waits are bounded (see mbar_wait); a timed-out wait records a status
// word and the kernel unwinds.
#include <cuda_bf16.h>
#include <math.h>
#include <stdio.h>
#include <atomic>
#include <mutex>
#include <type_traits>
#include "kernels.h"

namespace shainet {

namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int SK_MAX_STAGES = 32;
constexpr bool LAZY_RESCALE = false;

// Packed fp32 pairs: sm_100 executes fma.rn.f32x2 on a 64-bit register pair,
// two fused multiply-adds per issued instruction.
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ ulonglong2 lds128x2(const void* p) { return *reinterpret_cast<const ulonglong2*>(p); }

// Four consecutive cache elements of a shared-memory tile, `off` elements into the row that starts at
// element `row0`, as two packed fp32 pairs.  ES = 4: fp32 rows, one 16-byte load.  ES = 2: bfloat16 rows,
// one 8-byte load; a bfloat16 is the upper half of the fp32 of the same value, so each pair costs a shift
// and a mask.  The fp32 form keeps the row pointer as a pointer and the bfloat16 form sums the indices first:
// each is the grouping the compiler turns into the loop without spills for that element size (the other way
// round the group-size-8 fp32 instance spills 88 bytes per thread and a launch takes 1 us longer).
template <int ES>
struct KvRow {
    const float* row;   // ES = 4
    const float* tile;  // ES = 2
    size_t row0;
    __device__ __forceinline__ KvRow(const float* t, size_t r0) : row(t + r0), tile(t), row0(r0) {}
    __device__ __forceinline__ ulonglong2 at(int off) const {
        if constexpr (ES == 4) {
            return lds128x2(row + off);
        } else {
            const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(tile) + (row0 + off));
            ulonglong2 r;
            asm("mov.b64 %0, {%1, %2};" : "=l"(r.x) : "r"(w.x << 16), "r"(w.x & 0xffff0000u));
            asm("mov.b64 %0, {%1, %2};" : "=l"(r.y) : "r"(w.y << 16), "r"(w.y & 0xffff0000u));
            return r;
        }
    }
};

// The value a cache of element size ES keeps for x.
template <int ES>
__device__ __forceinline__ float kv_rounded(float x) {
    if constexpr (ES == 4) return x;
    else return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Tile geometry.  R*G = 16 scores per half-warp per batch, so a batch is
// BR = 2*16/G rows; a warp tile is a whole number of batches.  The ring has a
// multiple of NW stages so that every stage is always consumed by the same
// warp: an mbarrier phase wait is only meaningful for a waiter that saw the
// previous phase, which a fixed stage->warp map guarantees.
template <int HD, int G>
struct SKDefault {
    static constexpr int BR = 2 * (16 / G);
    static constexpr int TW = BR > 8 ? BR : 8;                         // rows per warp tile
    static constexpr int NW = 4;                                       // consumer warps (5, or 3 x 3 CTAs, measured slower)
    static constexpr bool BIG = 2 * TW * HD * 4 > 16 * 1024;           // ring + extras would not fit twice per SM
    static constexpr int SMEM_KB = BIG ? 216 : 110;                    // 2 x (110 + 1 KB reserved) fits 227 KB
    static constexpr int CTAS_PER_SM = BIG ? 1 : 2;
};

template <int HD, int G, int ES_ = 4, int TW_ = SKDefault<HD, G>::TW, int NW_ = SKDefault<HD, G>::NW,
          int SMEM_KB_ = SKDefault<HD, G>::SMEM_KB, int CTAS_ = SKDefault<HD, G>::CTAS_PER_SM>
struct SK {
    static constexpr int ES = ES_;                     // bytes per cache element: 4 (fp32) or 2 (bfloat16)
    static constexpr int NW = NW_;                     // consumer warps
    static constexpr int CPL = HD / 64;                // 16-byte chunks per lane per K row
    static constexpr int R = 16 / G;                   // rows per half-warp per batch
    static constexpr int BR = 2 * R;                   // rows per batch
    static constexpr int TW = TW_;                     // rows per warp tile
    static constexpr int NB = TW / BR;                 // batches per tile
    static constexpr int TILE_FLOATS = TW * HD * ES / 4;   // per tensor, in 4-byte units
    static constexpr int STAGE_FLOATS = 2 * TILE_FLOATS;
    static constexpr int RPI = 128 / HD;               // V rows covered by one warp-wide 128-bit load
    static constexpr int WARP_SCRATCH = 2 * 2 * (32 + 16); // two buffers of (p,p)[BR*G = 32] + (alpha,alpha)[G <= 16], as floats
    static constexpr int THREADS = (NW + 1) * 32;
    static constexpr int CTAS_PER_SM = CTAS_;
    // fused kernel extras: rotated q of the group (rows padded by 4 floats so that
    // lanes walking different rows hit different banks), a one-batch tile for the
    // new k row, the new v row, per-row inverse RMS values
    static constexpr int QS_STRIDE = HD + 4;
    static constexpr int QS_FLOATS = G * QS_STRIDE;
    static constexpr int XK_FLOATS = BR * HD;
    static constexpr int XV_FLOATS = HD;
    static constexpr int EXTRA_FLOATS = QS_FLOATS + XK_FLOATS + XV_FLOATS + 8 + 24;
    static constexpr int FIXED_BYTES = (NW * WARP_SCRATCH + EXTRA_FLOATS) * 4 + 2 * SK_MAX_STAGES * 8;
    static constexpr int NS_RAW = (SMEM_KB_ * 1024 - FIXED_BYTES) / (STAGE_FLOATS * 4);
    static constexpr int NS_CAP = NS_RAW > SK_MAX_STAGES ? SK_MAX_STAGES : NS_RAW;
    static constexpr int NS = NS_CAP / NW * NW;        // ring stages, a multiple of NW
    static constexpr int MERGE_FLOATS = NW * G * (HD + 2);
    static constexpr size_t SMEM_BYTES = (size_t)NS * STAGE_FLOATS * 4 + FIXED_BYTES;
    static_assert(HD == 64 || HD == 128, "head_dim");
    static_assert(ES == 4 || ES == 2, "cache element size");
    static_assert(G == 1 || G == 2 || G == 4 || G == 8 || G == 16, "group size");
    static_assert(TW % BR == 0, "a warp tile is a whole number of batches");
    static_assert(NS >= NW, "ring shorter than the number of consumer warps");
    static_assert(MERGE_FLOATS <= NS * STAGE_FLOATS, "merge area must fit in the ring");
};

// bfloat16 caches: a warp tile of twice the rows, so that a bulk copy moves as many bytes
// as with fp32 rows and twice the batches overlap inside a tile (batched decode on the
// Qwen3-8B shape: 0.49 ms per layer against 0.77 ms with the fp32 kernel's row count); three
// times the rows for batched decode at group sizes 4 and up (0.43 ms; a single sequence, whose
// CTAs have few tiles each, is slower with them: 29.6 against 27.0 us on the Qwen3-30B-A3B shape).
template <int HD, int G, int MUL>
using SKB = SK<HD, G, 2, MUL * SKDefault<HD, G>::TW>;
constexpr int skb_mul(int g, bool batched) { return batched && g >= 4 ? 3 : 2; }

// Carve-up of the dynamic shared memory, common to both kernels.
template <class C>
struct Smem {
    float* stages;
    float* warp_scratch;
    float* qs;   // [G][HD] rotated q (fused kernel)
    float* xk;   // [BR][HD], row 0 = the new rotated k row (fused kernel, last split)
    float* xv;   // [HD] the new v row
    int* flag;   // ticket broadcast
    float* inv;  // [G + 1] inverse RMS of the q rows and of the new k row
    uint64_t* full_bar;
    uint64_t* empty_bar;
    __device__ explicit Smem(unsigned char* raw) {
        stages = reinterpret_cast<float*>(raw);
        warp_scratch = stages + (size_t)C::NS * C::STAGE_FLOATS;
        qs = warp_scratch + C::NW * C::WARP_SCRATCH;
        xk = qs + C::QS_FLOATS;
        xv = xk + C::XK_FLOATS;
        flag = reinterpret_cast<int*>(xv + C::XV_FLOATS);
        inv = xv + C::XV_FLOATS + 8;
        full_bar = reinterpret_cast<uint64_t*>(xv + C::XV_FLOATS + 8 + 24);
        empty_bar = full_bar + SK_MAX_STAGES;
    }
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

// Running state of one consumer warp.
template <int G>
struct WarpState {
    f32x2 o[G][2];  // this lane's four output columns of every head, as two packed pairs
    float m, l;     // running max / partial sum for head (lane & 15) % G
    __device__ void init() {
#pragma unroll
        for (int g = 0; g < G; ++g) o[g][0] = o[g][1] = 0ull;
        m = -INFINITY;
        l = 0.0f;
    }
};

// q of the G heads, this lane's 4*CPL columns of each, as packed pairs
// (columns 0-1 and 2-3 of every 16-byte chunk).  qrow: [G][HD], global or shared.
template <int HD, int G, class C>
__device__ __forceinline__ void load_q(ulonglong2 (&q)[G][C::CPL], const float* qrow, int row_stride, int i16) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < C::CPL; ++c)
            q[g][c] = *reinterpret_cast<const ulonglong2*>(qrow + (size_t)g * row_stride + (c * 16 + i16) * 4);
}

// Scores of one batch: acc2[rr*G + g] for the R rows of this half-warp; even and
// odd columns accumulate in the two halves of a packed pair.
template <int HD, int G, class C>
__device__ __forceinline__ void score_batch(const float* ks, int base, int hw, int i16, const ulonglong2 (&q)[G][C::CPL],
                                            f32x2 (&acc2)[16]) {
#pragma unroll
    for (int k = 0; k < 16; ++k) acc2[k] = 0ull;
#pragma unroll
    for (int rr = 0; rr < C::R; ++rr) {
        const KvRow<C::ES> krow(ks, (size_t)(base + hw * C::R + rr) * HD);
#pragma unroll
        for (int c = 0; c < C::CPL; ++c) {
            const ulonglong2 kk = krow.at((c * 16 + i16) * 4);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                acc2[rr * G + g] = ffma2(q[g][c].x, kk.x, acc2[rr * G + g]);
                acc2[rr * G + g] = ffma2(q[g][c].y, kk.y, acc2[rr * G + g]);
            }
        }
    }
}

// A complete warp tile (all TW rows valid): no masks and no branches, so the
// whole tile is one basic block; the next batch's score FMAs are issued before
// the current batch's reduction and softmax, whose shuffle and exponent
// latencies they hide.  p and alpha alternate between two scratch buffers, one
// warp barrier per batch.
template <int HD, int G, class C>
__device__ __forceinline__ void consume_full_tile(const float* ks, const float* vs, const ulonglong2 (&q)[G][C::CPL],
                                                  WarpState<G>& st, f32x2* scratch, int lane, float scale) {
    const int i16 = lane & 15, hw = lane >> 4;
    f32x2 acc2[16];
    score_batch<HD, G, C>(ks, 0, hw, i16, q, acc2);
#pragma unroll
    for (int bb = 0; bb < C::NB; ++bb) {
        const int base = bb * C::BR;
        f32x2* ps = scratch + (bb & 1) * 48;
        f32x2* as = ps + 32;
        float acc[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float lo, hi;
            unpack2(acc2[k], lo, hi);
            acc[k] = lo + hi;
        }
        if (bb + 1 < C::NB) score_batch<HD, G, C>(ks, base + C::BR, hw, i16, q, acc2);
        reduce_scatter16(acc, lane);
        const float sc = acc[0] * scale;
        float bmax = sc;
#pragma unroll
        for (int off = G; off < 32; off <<= 1) bmax = fmaxf(bmax, __shfl_xor_sync(FULL, bmax, off));
        const float m_new = fmaxf(st.m, bmax);
        const float alpha = exp2f((st.m - m_new) * LOG2E);  // 0 while the running max is -inf
        const float p = exp2f((sc - m_new) * LOG2E);
        st.l = fmaf(st.l, alpha, p);
        st.m = m_new;
        ps[lane] = pack2(p, p);  // index = row_in_batch * G + head
        if (lane < G) as[lane] = pack2(alpha, alpha);
        const bool rescale = !LAZY_RESCALE || __any_sync(FULL, alpha != 1.0f);
        __syncwarp();
        if (rescale) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const f32x2 al = as[g];
                st.o[g][0] = fmul2(st.o[g][0], al);
                st.o[g][1] = fmul2(st.o[g][1], al);
            }
        }
#pragma unroll
        for (int rr = 0; rr < C::BR; rr += C::RPI) {
            const int rb = rr + (C::RPI == 2 ? hw : 0);
            const int col = (C::RPI == 2 ? i16 : lane) * 4;
            const ulonglong2 vv = KvRow<C::ES>(vs, (size_t)(base + rb) * HD).at(col);
            const f32x2* prow = ps + rb * G;
            if constexpr (G >= 2) {
#pragma unroll
                for (int g = 0; g < G; g += 2) {
                    const ulonglong2 pp = *reinterpret_cast<const ulonglong2*>(prow + g);
                    st.o[g][0] = ffma2(pp.x, vv.x, st.o[g][0]);
                    st.o[g][1] = ffma2(pp.x, vv.y, st.o[g][1]);
                    st.o[g + 1][0] = ffma2(pp.y, vv.x, st.o[g + 1][0]);
                    st.o[g + 1][1] = ffma2(pp.y, vv.y, st.o[g + 1][1]);
                }
            } else {
                const f32x2 pg = prow[0];
                st.o[0][0] = ffma2(pg, vv.x, st.o[0][0]);
                st.o[0][1] = ffma2(pg, vv.y, st.o[0][1]);
            }
        }
    }
}

// One warp tile: `nrows` valid rows of K (ks) and V (vs) in shared memory, elements of ES bytes.
template <int HD, int G, class C, int ES>
__device__ __forceinline__ void consume_tile(const float* ks, const float* vs, int nrows, const ulonglong2 (&q)[G][C::CPL],
                                             WarpState<G>& st, f32x2* ps, f32x2* as, int lane, float scale, int nbatches) {
    const int i16 = lane & 15, hw = lane >> 4;
    const int my_r = hw * C::R + i16 / G;  // row in batch of this lane's score (its head is i16 % G)
#pragma unroll
    for (int bb = 0; bb < C::NB; ++bb) {
        const int base = bb * C::BR;
        if (bb >= nbatches || base >= nrows) break;  // warp-uniform
        // ---- scores: acc[rr*G + g] for the R rows of this half-warp; even and odd
        // columns accumulate in the two halves of a packed pair ----
        f32x2 acc2[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) acc2[k] = 0ull;
#pragma unroll
        for (int rr = 0; rr < C::R; ++rr) {
            const KvRow<ES> krow(ks, (size_t)(base + hw * C::R + rr) * HD);
#pragma unroll
            for (int c = 0; c < C::CPL; ++c) {
                const ulonglong2 kk = krow.at((c * 16 + i16) * 4);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    acc2[rr * G + g] = ffma2(q[g][c].x, kk.x, acc2[rr * G + g]);
                    acc2[rr * G + g] = ffma2(q[g][c].y, kk.y, acc2[rr * G + g]);
                }
            }
        }
        float acc[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float lo, hi;
            unpack2(acc2[k], lo, hi);
            acc[k] = lo + hi;
        }
        reduce_scatter16(acc, lane);
        float sc = acc[0] * scale;
        if (base + my_r >= nrows) sc = -INFINITY;  // rows past the end of the slice
        // ---- online softmax for this lane's head ----
        float bmax = sc;
#pragma unroll
        for (int off = G; off < 32; off <<= 1) bmax = fmaxf(bmax, __shfl_xor_sync(FULL, bmax, off));
        const float m_new = fmaxf(st.m, bmax);
        const float alpha = exp2f((st.m - m_new) * LOG2E);  // 0 while the running max is -inf
        const float p = exp2f((sc - m_new) * LOG2E);
        st.l = fmaf(st.l, alpha, p);
        st.m = m_new;
        __syncwarp();  // previous batch's reads of ps/as are done
        ps[lane] = pack2(p, p);  // index = row_in_batch * G + head
        if (lane < G) as[lane] = pack2(alpha, alpha);
        const bool rescale = __any_sync(FULL, alpha != 1.0f);
        __syncwarp();
        if (rescale) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const f32x2 al = as[g];
                st.o[g][0] = fmul2(st.o[g][0], al);
                st.o[g][1] = fmul2(st.o[g][1], al);
            }
        }
        // ---- o += P.V ----
#pragma unroll
        for (int rr = 0; rr < C::BR; rr += C::RPI) {
            const int row = base + rr + (C::RPI == 2 ? hw : 0);
            if (base + rr >= nrows) break;  // warp-uniform
            if (row < nrows) {
                const int col = (C::RPI == 2 ? i16 : lane) * 4;
                const ulonglong2 vv = KvRow<ES>(vs, (size_t)row * HD).at(col);
                const f32x2* prow = ps + (row - base) * G;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const f32x2 pg = prow[g];
                    st.o[g][0] = ffma2(pg, vv.x, st.o[g][0]);
                    st.o[g][1] = ffma2(pg, vv.y, st.o[g][1]);
                }
            }
        }
    }
}

// After the last tile: fold the lanes that share a head (sum) and, for
// head_dim 64, the two half-warps that each took every other V row.
template <int HD, int G, class C>
__device__ __forceinline__ void finish_warp(WarpState<G>& st) {
#pragma unroll
    for (int off = G; off < 32; off <<= 1) st.l += __shfl_xor_sync(FULL, st.l, off);
    if (C::RPI == 2) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                float lo, hi;
                unpack2(st.o[g][k], lo, hi);
                lo += __shfl_xor_sync(FULL, lo, 16);
                hi += __shfl_xor_sync(FULL, hi, 16);
                st.o[g][k] = pack2(lo, hi);
            }
    }
}

// Consumer warps park their state in the (now idle) ring.
template <int HD, int G, class C>
__device__ __forceinline__ void park_state(const WarpState<G>& st, float* ring, int warp, int lane) {
    float* mo = ring;                              // [NW][G][HD]
    float* mm = mo + (size_t)C::NW * G * HD;       // [NW][G]
    float* ml = mm + C::NW * G;                    // [NW][G]
    if (lane < G) {  // lane < G holds head `lane`
        mm[warp * G + lane] = st.m;
        ml[warp * G + lane] = st.l;
    }
    if (C::RPI == 1 || lane < 16) {
#pragma unroll
        for (int g = 0; g < G; ++g)
            *reinterpret_cast<ulonglong2*>(mo + ((size_t)warp * G + g) * HD + lane * 4) = make_ulonglong2(st.o[g][0], st.o[g][1]);
    }
}

// Merge of the NW warps' states for element (g, d): unnormalised o, max and sum.
template <int HD, int G, class C>
__device__ __forceinline__ void merge_warps(const float* ring, int g, int d, float& acc, float& M, float& L) {
    const float* mo = ring;
    const float* mm = mo + (size_t)C::NW * G * HD;
    const float* ml = mm + C::NW * G;
    M = -INFINITY;
#pragma unroll
    for (int w = 0; w < C::NW; ++w) M = fmaxf(M, mm[w * G + g]);
    L = 0.0f;
    acc = 0.0f;
#pragma unroll
    for (int w = 0; w < C::NW; ++w) {
        const float mw = mm[w * G + g];
        const float wt = (mw == -INFINITY) ? 0.0f : exp2f((mw - M) * LOG2E);
        L = fmaf(wt, ml[w * G + g], L);
        acc = fmaf(wt, mo[((size_t)w * G + g) * HD + d], acc);
    }
}

template <class C>
__device__ __forceinline__ void init_barriers(Smem<C>& sm) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NS; ++s) {
            mbar_init(&sm.full_bar[s], 1);
            mbar_init(&sm.empty_bar[s], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
}

// Producer: tiles [first, last) of a slice starting at kbase/vbase with `rows` rows.
template <int HD, class C>
__device__ __forceinline__ bool produce_tiles(Smem<C>& sm, const float* kbase, const float* vbase, int rows, int first,
                                              int last, AttnStatus* status) {
    for (int i = first; i < last; ++i) {
        const int s = i % C::NS;
        if (i >= C::NS && !mbar_wait(&sm.empty_bar[s], ((i / C::NS) - 1) & 1, status, 1)) return false;
        const int nrows = min(C::TW, rows - i * C::TW);
        const uint32_t bytes = (uint32_t)nrows * HD * C::ES;
        float* ks = sm.stages + (size_t)s * C::STAGE_FLOATS;
        float* vs = ks + C::TILE_FLOATS;
        mbar_arrive_expect_tx(&sm.full_bar[s], 2 * bytes);
        bulk_g2s(ks, kbase + (size_t)i * C::TILE_FLOATS, bytes, &sm.full_bar[s]);
        bulk_g2s(vs, vbase + (size_t)i * C::TILE_FLOATS, bytes, &sm.full_bar[s]);
    }
    return true;
}

template <int HD, int G, class C>
__device__ __forceinline__ void consume_slice(Smem<C>& sm, int ntiles, int rows, const ulonglong2 (&q)[G][C::CPL],
                                              WarpState<G>& st, int warp, int lane, float scale, AttnStatus* status) {
    f32x2* ps = reinterpret_cast<f32x2*>(sm.warp_scratch + warp * C::WARP_SCRATCH);  // (p,p) per (row, head)
    f32x2* as = ps + 32;                                                             // (alpha,alpha) per head
    for (int i = warp; i < ntiles; i += C::NW) {
        const int s = i % C::NS;
        if (!mbar_wait(&sm.full_bar[s], (i / C::NS) & 1, status, 2)) break;
        const float* ks = sm.stages + (size_t)s * C::STAGE_FLOATS;
        const float* vs = ks + C::TILE_FLOATS;
        const int nrows = min(C::TW, rows - i * C::TW);
        if (nrows == C::TW) {
            consume_full_tile<HD, G, C>(ks, vs, q, st, ps, lane, scale);
        } else {
            __syncwarp();
            consume_tile<HD, G, C, C::ES>(ks, vs, nrows, q, st, ps, as, lane, scale, C::NB);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty_bar[s]);
    }
}

// ---------------------------------------------------------------------------
// Plain split-K kernel: q already rotated, cache already appended.
// ---------------------------------------------------------------------------
template <int HD, int G, class C>
__global__ void __launch_bounds__(C::THREADS, C::CTAS_PER_SM) attn_splitk_kernel(AttnArgs a) {
    extern __shared__ __align__(1024) unsigned char sk_smem_raw[];
    Smem<C> sm(sk_smem_raw);
    const int split = blockIdx.x, kv_h = blockIdx.y, r = blockIdx.z;
    const int H = a.hs.num_heads;
    const int b = r / a.T, t = r % a.T;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[b] : a.seqs.one;
    const int visible = sd.start + t + 1;
    const int row0 = split * a.chunk_rows;
    if (row0 >= visible) return;  // whole CTA: this sequence has fewer splits
    const int row1 = min(row0 + a.chunk_rows, visible);
    const int rows = row1 - row0;
    const int ntiles = (rows + C::TW - 1) / C::TW;
    static_assert(C::ES == 4, "the plain split-K kernel reads fp32 caches");
    const float* kbase = sd.k + ((size_t)kv_h * sd.capacity + row0) * HD;
    const float* vbase = sd.v + ((size_t)kv_h * sd.capacity + row0) * HD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    init_barriers(sm);

    WarpState<G> st;
    st.init();
    if (warp == C::NW) {
        if (lane == 0) produce_tiles<HD, C>(sm, kbase, vbase, rows, 0, ntiles, a.status);
    } else {
        ulonglong2 q[G][C::CPL];
        load_q<HD, G, C>(q, a.q_rot + ((size_t)r * H + (size_t)kv_h * G) * HD, HD, lane & 15);
        consume_slice<HD, G, C>(sm, ntiles, rows, q, st, warp, lane, a.scale, a.status);
        finish_warp<HD, G, C>(st);
    }
    // All tiles are consumed (or abandoned after a timeout): every bulk copy
    // that was issued has landed, so the ring can be reused.
    __syncthreads();
    if (warp < C::NW) park_state<HD, G, C>(st, sm.stages, warp, lane);
    __syncthreads();
    const int nsplit_here = (visible + a.chunk_rows - 1) / a.chunk_rows;
    for (int e = threadIdx.x; e < G * HD; e += C::THREADS) {
        const int g = e / HD, d = e - g * HD;
        float acc, M, L;
        merge_warps<HD, G, C>(sm.stages, g, d, acc, M, L);
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

// Merge of `count` partials (max, sum, unnormalised output) of the G heads of
// (row r, kv head kv_h), entries first..first+count-1 of a [row][head][stride]
// table, by the whole CTA.  `final` writes the normalised output row; otherwise
// the merged partial goes to entry dst_index of a second table.
constexpr int MERGE_GROUP = 8;  // splits merged by the last CTA of each group

template <int HD, int G, int THREADS>
__device__ void merge_partials(const float* po, const float* pml, size_t stride, int first, int count, int r, int kv_h,
                               int H, bool final, float* out, float* dst_o, float* dst_ml, size_t dst_stride,
                               int dst_index, float* lse_out) {
    // Every thread owns up to NT (head, four columns) tasks and walks the partials
    // in rounds of 8: the (max, sum) pairs and the output quads of a round are
    // all requested, for all of the thread's tasks, before any is used, so a
    // round costs one L2 latency.  Weights are recomputed per thread instead of
    // being staged through shared memory.
    constexpr int D4 = HD / 4;
    constexpr int NT = (G * D4 + THREADS - 1) / THREADS;
    const size_t head0 = (size_t)r * H + (size_t)kv_h * G;
    float M[NT], L[NT];
    float4 acc[NT];
    const float2* ml[NT];
    const float4* src[NT];
    bool on[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int task = threadIdx.x + t * THREADS;
        on[t] = task < G * D4;
        const int g = on[t] ? task / D4 : 0, d4 = on[t] ? task - g * D4 : 0;
        const size_t e0 = (head0 + g) * stride + first;
        ml[t] = reinterpret_cast<const float2*>(pml) + e0;
        src[t] = reinterpret_cast<const float4*>(po + e0 * HD) + d4;
        M[t] = -INFINITY;
        L[t] = 0.0f;
        acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s0 = 0; s0 < count; s0 += 8) {
        float2 mv[NT][8];
        float4 v[NT][8];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const bool in = on[t] && s0 + k < count;
                mv[t][k] = in ? __ldcg(ml[t] + s0 + k) : make_float2(-INFINITY, 0.f);
                v[t][k] = in ? __ldcg(src[t] + (size_t)(s0 + k) * D4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float Mc = M[t];
#pragma unroll
            for (int k = 0; k < 8; ++k) Mc = fmaxf(Mc, mv[t][k].x);
            const float resc = (M[t] == -INFINITY) ? 0.0f : exp2f((M[t] - Mc) * LOG2E);
            L[t] *= resc;
            acc[t].x *= resc; acc[t].y *= resc; acc[t].z *= resc; acc[t].w *= resc;
            M[t] = Mc;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float wt = (mv[t][k].x == -INFINITY) ? 0.0f : exp2f((mv[t][k].x - Mc) * LOG2E);
                L[t] = fmaf(wt, mv[t][k].y, L[t]);
                acc[t].x = fmaf(wt, v[t][k].x, acc[t].x);
                acc[t].y = fmaf(wt, v[t][k].y, acc[t].y);
                acc[t].z = fmaf(wt, v[t][k].z, acc[t].z);
                acc[t].w = fmaf(wt, v[t][k].w, acc[t].w);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (!on[t]) continue;
        const int task = threadIdx.x + t * THREADS;
        const int g = task / D4, d4 = task - g * D4;
        if (final) {
            const float inv = 1.0f / L[t];
            *(reinterpret_cast<float4*>(out + (head0 + g) * HD) + d4) =
                make_float4(acc[t].x * inv, acc[t].y * inv, acc[t].z * inv, acc[t].w * inv);
            if (lse_out && d4 == 0) lse_out[head0 + g] = M[t] + logf(L[t]);
        } else {
            const size_t e = (head0 + g) * dst_stride + dst_index;
            *(reinterpret_cast<float4*>(dst_o + e * HD) + d4) = acc[t];
            if (d4 == 0) *(reinterpret_cast<float2*>(dst_ml) + e) = make_float2(M[t], L[t]);
        }
    }
}

// Split partials that travel as {value, epoch} words: a CTA publishes its partial with
// plain 8-byte stores (each indivisible), and the merging CTA polls the words
// themselves, so the last partial costs one store and one load on the critical
// path instead of fence + flag + flag poll + load.  One call folds all `count`
// partials of 64 columns of one query head: 16 threads per partial, THREADS/16
// partials side by side, 8 partials requested per thread before the first is used.
template <int HD, int THREADS>
__device__ bool merge_head_words(const unsigned long long* po, const unsigned long long* pml, size_t e0, int count,
                                 unsigned epoch, float* smem, float* out_row, float* lse_out, const GatherTarget& gt,
                                 size_t head_index, int half, AttnStatus* status) {
    constexpr int D4 = 16;
    constexpr int NPG = THREADS / D4;
    constexpr int MAXB = 8;
    const int pg = threadIdx.x / D4, d4 = threadIdx.x - pg * D4;
    const int col = half * 64 + d4 * 4;
    const unsigned long long* src = po + e0 * HD + col;
    const unsigned long long* ml = pml + e0 * 2;
    float M = -INFINITY, L = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok = true;
    const unsigned long long t0 = globaltimer_ns();
    auto ld2 = [](const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
        asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    };
    if (pg < NPG) {
        for (int s0 = pg; s0 < count && ok; s0 += NPG * MAXB) {
            unsigned long long w[MAXB][6];
#pragma unroll
            for (int k = 0; k < MAXB; ++k) {
                const int sidx = s0 + k * NPG;
                if (sidx < count) {
                    ld2(src + (size_t)sidx * HD, w[k][0], w[k][1]);
                    ld2(src + (size_t)sidx * HD + 2, w[k][2], w[k][3]);
                    ld2(ml + (size_t)sidx * 2, w[k][4], w[k][5]);
                }
            }
            // words that do not carry this launch's epoch yet are requested again, all of
            // them in one round, until none is left (bounded)
            while (true) {
                bool all = true;
#pragma unroll
                for (int k = 0; k < MAXB; ++k) {
                    const int sidx = s0 + k * NPG;
                    if (sidx < count) {
                        bool good = true;
#pragma unroll
                        for (int j = 0; j < 6; ++j) good = good && (unsigned)(w[k][j] >> 32) == epoch;
                        if (!good) {
                            all = false;
                            ld2(src + (size_t)sidx * HD, w[k][0], w[k][1]);
                            ld2(src + (size_t)sidx * HD + 2, w[k][2], w[k][3]);
                            ld2(ml + (size_t)sidx * 2, w[k][4], w[k][5]);
                        }
                    }
                }
                if (all) break;
                if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                    if (status != nullptr && atomicCAS(&status->code, DEV_OK, DEV_WAIT_TIMEOUT) == DEV_OK) status->where = 3;
                    ok = false;
                    break;
                }
            }
            float2 mv[MAXB];
            float4 v[MAXB];
#pragma unroll
            for (int k = 0; k < MAXB; ++k) {
                const int sidx = s0 + k * NPG;
                if (sidx < count) {
                    v[k] = make_float4(__uint_as_float((unsigned)w[k][0]), __uint_as_float((unsigned)w[k][1]),
                                       __uint_as_float((unsigned)w[k][2]), __uint_as_float((unsigned)w[k][3]));
                    mv[k] = make_float2(__uint_as_float((unsigned)w[k][4]), __uint_as_float((unsigned)w[k][5]));
                } else {
                    v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                    mv[k] = make_float2(-INFINITY, 0.f);
                }
            }
            float Mc = M;
#pragma unroll
            for (int k = 0; k < MAXB; ++k) Mc = fmaxf(Mc, mv[k].x);
            const float resc = (M == -INFINITY) ? 0.0f : exp2f((M - Mc) * LOG2E);
            L *= resc;
            acc.x *= resc; acc.y *= resc; acc.z *= resc; acc.w *= resc;
            M = Mc;
#pragma unroll
            for (int k = 0; k < MAXB; ++k) {
                const float wt = (mv[k].x == -INFINITY) ? 0.0f : exp2f((mv[k].x - Mc) * LOG2E);
                L = fmaf(wt, mv[k].y, L);
                acc.x = fmaf(wt, v[k].x, acc.x);
                acc.y = fmaf(wt, v[k].y, acc.y);
                acc.z = fmaf(wt, v[k].z, acc.z);
                acc.w = fmaf(wt, v[k].w, acc.w);
            }
        }
        float4* sa = reinterpret_cast<float4*>(smem);                 // [NPG][D4]
        float2* sm2 = reinterpret_cast<float2*>(smem + NPG * D4 * 4);  // [NPG][D4]
        sa[pg * D4 + d4] = acc;
        sm2[pg * D4 + d4] = make_float2(M, L);
    }
    ok = __syncthreads_and(ok);
    if (ok && pg == 0) {
        const float4* sa = reinterpret_cast<const float4*>(smem);
        const float2* sm2 = reinterpret_cast<const float2*>(smem + NPG * D4 * 4);
        float Mt = -INFINITY;
#pragma unroll
        for (int g = 0; g < NPG; ++g) Mt = fmaxf(Mt, sm2[g * D4 + d4].x);
        float Lt = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int g = 0; g < NPG; ++g) {
            const float2 q = sm2[g * D4 + d4];
            const float wt = (q.x == -INFINITY) ? 0.0f : exp2f((q.x - Mt) * LOG2E);
            const float4 a4 = sa[g * D4 + d4];
            Lt = fmaf(wt, q.y, Lt);
            o.x = fmaf(wt, a4.x, o.x);
            o.y = fmaf(wt, a4.y, o.y);
            o.z = fmaf(wt, a4.z, o.z);
            o.w = fmaf(wt, a4.w, o.w);
        }
        const float inv = 1.0f / Lt;
        const float4 res = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
        *reinterpret_cast<float4*>(out_row + col) = res;
        const bool writes_lse = half == 0 && d4 == 0;
        if (lse_out && writes_lse) *lse_out = Mt + logf(Lt);
        // the same row into every rank's exchange buffer as {value, epoch} words:
        // plain 8-byte stores to peer memory, nothing to fence and nobody to wait for
        if (gt.world > 0) {
            const unsigned long long e = (unsigned long long)gt.epoch << 32;
            const unsigned long long w0 = e | __float_as_uint(res.x), w1 = e | __float_as_uint(res.y);
            const unsigned long long w2 = e | __float_as_uint(res.z), w3 = e | __float_as_uint(res.w);
            const unsigned long long wl = e | __float_as_uint(Mt + logf(Lt));
            for (int p = 0; p < gt.world; ++p) {
                unsigned long long* dst = gt.peer_words[p] + gt.out_offset + head_index * HD + col;
                asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(dst), "l"(w0), "l"(w1) : "memory");
                asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(w2), "l"(w3) : "memory");
                if (gt.lse_offset >= 0 && writes_lse)
                    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(gt.peer_words[p] + gt.lse_offset + head_index), "l"(wl) : "memory");
            }
        }
    }
    __syncthreads();
    return ok;
}

// The calling CTA has published something and takes a ticket; true for the
// CTA that took the last of `expected` tickets (it also resets the counter for
// the next launch).  Nobody waits for anybody.
__device__ __forceinline__ bool take_last_ticket(unsigned* ticket, int expected, int* flag) {
    // barrier, then one acquire-release atomic by thread 0: the CTA's stores are
    // released with it, the other CTAs' stores are acquired by the last taker
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(ticket) : "memory");
        const int last = t == (unsigned)(expected - 1);
        if (last) *ticket = 0u;
        *flag = last;
    }
    __syncthreads();
    return *flag != 0;
}

// ---------------------------------------------------------------------------
// Fused decode kernel: one new token per sequence.  Prologue = bias, per-head
// RMSNorm and RoPE of the group's q heads (every CTA) and of the new k row, and
// the append of k/v (the CTA whose slice ends at the new position); then the
// split-K stream; then the last CTA of each (row, kv head) merges the splits.
// ---------------------------------------------------------------------------

template <int HD, int G, class C>
__global__ void __launch_bounds__(C::THREADS, C::CTAS_PER_SM) attn_decode_fused_kernel(FusedArgs a) {
    extern __shared__ __align__(1024) unsigned char sk_smem_raw[];
    Smem<C> sm(sk_smem_raw);
    const int split = blockIdx.x, kv_h = blockIdx.y, r = blockIdx.z;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads;
    const SeqDesc sd = a.seqs.many ? a.seqs.many[r] : a.seqs.one;
    const int start = sd.start;     // rows already cached; the new token's row index if it is appended
    const int visible = start + (a.no_append ? 0 : 1);
    const int row0 = split * a.chunk_rows;
    if (row0 >= visible) return;    // whole CTA: this sequence has fewer splits (an exit counts as its trigger)
    const int row1 = min(row0 + a.chunk_rows, visible);
    const bool owns_new = !a.no_append && row1 == visible;   // this slice ends with the new token
    const int rows = (owns_new ? start : row1) - row0;  // rows that come from the cache
    const int ntiles = (rows + C::TW - 1) / C::TW;
    // Tiles that end at or below `safe_end` cannot be under construction by the
    // grid that may still be running; they are fetched before waiting for it.
    // When the caller vouches for the inputs (inputs_ready) the consumers do not
    // wait either, so every such tile may go out early, not just a ring's worth.
    const int safe_end = start - a.unsafe_tail;
    const int n_safe = min(ntiles, row0 + rows <= safe_end ? ntiles : max(0, (safe_end - row0) / C::TW));
    const int n_early = a.inputs_ready ? n_safe : min(n_safe, C::NS);
    // element size C::ES: a bfloat16 cache is addressed through the same (float-typed) pointers
    const size_t slice_off = ((size_t)kv_h * sd.capacity + row0) * HD * C::ES;
    const float* kbase = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(sd.k) + slice_off);
    const float* vbase = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(sd.v) + slice_off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    init_barriers(sm);

    WarpState<G> st;
    st.init();
    if (warp == C::NW) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const bool ok = produce_tiles<HD, C>(sm, kbase, vbase, rows, 0, n_early, a.status);
            grid_dependency_wait();
            grid_launch_dependents();
            if (ok) produce_tiles<HD, C>(sm, kbase, vbase, rows, n_early, ntiles, a.status);
        }
    } else {
        // ---------------- consumers ----------------
        // Everything that does not depend on this call's inputs happens before the
        // wait for the previous grid: norm weights, and the rotation of this
        // position (lane owns the pairs (i, i + HD/2), i = lane + 32k).
        constexpr int PL = HD / 64;                  // rotation pairs per lane
        constexpr int MAXIT = (G + 2 + C::NW - 1) / C::NW;
        const float fpos = (float)(start + a.pos_delta);   // RoPE position of the new token
        float rc[PL], rs[PL], wq0[PL], wq1[PL], wk0[PL], wk1[PL];
#pragma unroll
        for (int k = 0; k < PL; ++k) {
            const int i = lane + 32 * k;
            sincosf(__fmul_rn(fpos, a.inv_freq[i]), &rs[k], &rc[k]);
            wq0[k] = a.q_norm ? a.q_norm[i] : 1.0f;
            wq1[k] = a.q_norm ? a.q_norm[i + HD / 2] : 1.0f;
            wk0[k] = a.k_norm ? a.k_norm[i] : 1.0f;
            wk1[k] = a.k_norm ? a.k_norm[i + HD / 2] : 1.0f;
        }
        const int items = G + (owns_new ? 2 : 0);   // q rows of the group, then the new k row, then the new v row
        // Ask L2 for this warp's input rows now: whoever still writes them does so through
        // L2, so the loads after the wait see the final values and no longer go to DRAM.
#pragma unroll
        for (int n = 0; n < MAXIT; ++n) {
            const int it = warp + n * C::NW;
            if (it < items && lane < HD / 32) {
                const float* src = it < G ? a.q + ((size_t)r * H + kv_h * G + it) * HD
                                          : (it == G ? a.k_new : a.v_new) + ((size_t)r * KV + kv_h) * HD;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(src + lane * 32));
            }
        }
        if (!a.inputs_ready) grid_dependency_wait();   // q, k_new, v_new may come from the previous grid
        // (1) all of this warp's rows in one round of loads: x[n][c] = column lane + 32c
        float x[MAXIT][2 * PL];
#pragma unroll
        for (int n = 0; n < MAXIT; ++n) {
            const int it = warp + n * C::NW;
#pragma unroll
            for (int c = 0; c < 2 * PL; ++c) x[n][c] = 0.0f;
            if (it < items) {
                const float* src;
                const float* bias;
                if (it < G) {
                    const int h = kv_h * G + it;
                    src = a.q + ((size_t)r * H + h) * HD;
                    bias = a.b_q ? a.b_q + (size_t)h * HD : nullptr;
                } else if (it == G) {
                    src = a.k_new + ((size_t)r * KV + kv_h) * HD;
                    bias = a.b_k ? a.b_k + (size_t)kv_h * HD : nullptr;
                } else {
                    src = a.v_new + ((size_t)r * KV + kv_h) * HD;
                    bias = a.b_v ? a.b_v + (size_t)kv_h * HD : nullptr;
                }
#pragma unroll
                for (int c = 0; c < 2 * PL; ++c) {
                    x[n][c] = __ldcg(src + lane + 32 * c);   // written by the grid ahead while this one was resident: L2 only
                    if (bias) x[n][c] = __fadd_rn(x[n][c], bias[lane + 32 * c]);
                }
            }
        }
        // (2) norm (warp-tree sum of squares; the prefill kernel keeps the reference's
        // sequential order, the two differ by the rounding of the sum), rotation with
        // the reference's unfused arithmetic, then shared memory and, for k and v, the cache.
        // The rows of a warp go through each stage together (no per-row branches around
        // the shuffles), so their shuffle and double-precision latencies overlap.
        float inv[MAXIT];
#pragma unroll
        for (int n = 0; n < MAXIT; ++n) inv[n] = 1.0f;
        if (a.q_norm != nullptr || a.k_norm != nullptr) {   // models without per-head norms skip the sums and the f64 root
            float ss[MAXIT];
#pragma unroll
            for (int n = 0; n < MAXIT; ++n) {
                ss[n] = 0.0f;
#pragma unroll
                for (int c = 0; c < 2 * PL; ++c) ss[n] = fmaf(x[n][c], x[n][c], ss[n]);   // rows past `items` hold zeros
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                for (int n = 0; n < MAXIT; ++n) ss[n] += __shfl_xor_sync(FULL, ss[n], off);
#pragma unroll
            for (int n = 0; n < MAXIT; ++n) inv[n] = (float)(1.0 / sqrt((double)(ss[n] / (float)HD) + a.eps));
        }
#pragma unroll
        for (int n = 0; n < MAXIT; ++n) {
            const int it = warp + n * C::NW;
            if (it >= items) break;   // warp-uniform
            float* row = it < G ? sm.qs + it * C::QS_STRIDE : (it == G ? sm.xk : sm.xv);
            if (it <= G) {
                const bool normed = (it < G ? a.q_norm : a.k_norm) != nullptr;
#pragma unroll
                for (int k = 0; k < PL; ++k) {
                    float x0 = x[n][k], x1 = x[n][k + PL];
                    if (normed) {
                        x0 = __fmul_rn(__fmul_rn(x0, inv[n]), it < G ? wq0[k] : wk0[k]);
                        x1 = __fmul_rn(__fmul_rn(x1, inv[n]), it < G ? wq1[k] : wk1[k]);
                    }
                    x[n][k] = __fsub_rn(__fmul_rn(x0, rc[k]), __fmul_rn(x1, rs[k]));
                    x[n][k + PL] = __fadd_rn(__fmul_rn(x1, rc[k]), __fmul_rn(x0, rs[k]));
                }
            }
            if (it >= G) {  // the new row is attended to as the cache will hold it
#pragma unroll
                for (int c = 0; c < 2 * PL; ++c) x[n][c] = kv_rounded<C::ES>(x[n][c]);
            }
#pragma unroll
            for (int c = 0; c < 2 * PL; ++c) row[lane + 32 * c] = x[n][c];
            if (it >= G) {  // append to the cache
                const size_t e0 = ((size_t)kv_h * sd.capacity + start) * HD;
                if constexpr (C::ES == 4) {
                    float* dst = (it == G ? sd.k : sd.v) + e0;
#pragma unroll
                    for (int c = 0; c < 2 * PL; ++c) dst[lane + 32 * c] = x[n][c];
                } else {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(it == G ? sd.k : sd.v) + e0;
#pragma unroll
                    for (int c = 0; c < 2 * PL; ++c) dst[lane + 32 * c] = __float2bfloat16_rn(x[n][c]);
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(C::NW * 32) : "memory");  // consumers only: qs/xk/xv complete
        ulonglong2 q[G][C::CPL];
        load_q<HD, G, C>(q, sm.qs, C::QS_STRIDE, lane & 15);
        consume_slice<HD, G, C>(sm, ntiles, rows, q, st, warp, lane, a.scale, a.status);
        if (owns_new && warp == (ntiles % C::NW)) {
            // the new token's own row, from shared memory (one valid row)
            f32x2* ps = reinterpret_cast<f32x2*>(sm.warp_scratch + warp * C::WARP_SCRATCH);
            consume_tile<HD, G, C, 4>(sm.xk, sm.xv, 1, q, st, ps, ps + 32, lane, a.scale, 1);
        }
        finish_warp<HD, G, C>(st);
    }
    __syncthreads();  // every issued copy has landed; the ring is free
    if (a.inputs_ready) grid_dependency_wait();  // the shared scratch below may still be in use by the previous grid
    if (warp < C::NW) park_state<HD, G, C>(st, sm.stages, warp, lane);
    __syncthreads();
    const int nsplit_here = (visible + a.chunk_rows - 1) / a.chunk_rows;
    const bool words = a.stream_merge && nsplit_here > 1;   // partials as {value, epoch} words
    unsigned long long* pw = reinterpret_cast<unsigned long long*>(a.part_o);
    unsigned long long* pmlw = reinterpret_cast<unsigned long long*>(a.part_ml);
    const unsigned long long ew = (unsigned long long)a.epoch << 32;
    // Fold the NW warp states: the per-head weights once (G threads), then four
    // columns per thread and iteration.
    {
        const float* mo = sm.stages;                              // [NW][G][HD]
        const float* mm = mo + (size_t)C::NW * G * HD;            // [NW][G]
        const float* ml = mm + C::NW * G;                         // [NW][G]
        float* wts = sm.warp_scratch;                             // [NW][G] weights, then max[G], sum[G]
        if (threadIdx.x < G) {
            const int g = threadIdx.x;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < C::NW; ++w) M = fmaxf(M, mm[w * G + g]);
            float L = 0.0f;
#pragma unroll
            for (int w = 0; w < C::NW; ++w) {
                const float mw = mm[w * G + g];
                const float wt = (mw == -INFINITY) ? 0.0f : exp2f((mw - M) * LOG2E);
                wts[w * G + g] = wt;
                L = fmaf(wt, ml[w * G + g], L);
            }
            wts[C::NW * G + g] = M;
            wts[C::NW * G + G + g] = L;
        }
        __syncthreads();
        for (int e4 = threadIdx.x; e4 < G * HD / 4; e4 += C::THREADS) {
            const int g = e4 / (HD / 4), d = (e4 - g * (HD / 4)) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < C::NW; ++w) {
                const float wt = wts[w * G + g];
                const float4 o = *reinterpret_cast<const float4*>(mo + ((size_t)w * G + g) * HD + d);
                acc.x = fmaf(wt, o.x, acc.x);
                acc.y = fmaf(wt, o.y, acc.y);
                acc.z = fmaf(wt, o.z, acc.z);
                acc.w = fmaf(wt, o.w, acc.w);
            }
            const float M = wts[C::NW * G + g], L = wts[C::NW * G + G + g];
            const int h = kv_h * G + g;
            if (nsplit_here == 1) {
                *reinterpret_cast<float4*>(a.out + ((size_t)r * H + h) * HD + d) =
                    make_float4(acc.x / L, acc.y / L, acc.z / L, acc.w / L);
                if (a.lse_out && d == 0) a.lse_out[(size_t)r * H + h] = M + logf(L);
            } else {
                const size_t pidx = ((size_t)r * H + h) * a.max_splits + split;
                if (words) {
                    unsigned long long* dst = pw + pidx * HD + d;
                    asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(dst), "l"(ew | __float_as_uint(acc.x)),
                                 "l"(ew | __float_as_uint(acc.y))
                                 : "memory");
                    asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(ew | __float_as_uint(acc.z)),
                                 "l"(ew | __float_as_uint(acc.w))
                                 : "memory");
                    if (d == 0) {
                        asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(pmlw + pidx * 2), "l"(ew | __float_as_uint(M)),
                                     "l"(ew | __float_as_uint(L))
                                     : "memory");
                    }
                } else {
                    *reinterpret_cast<float4*>(a.part_o + pidx * HD + d) = acc;
                    if (d == 0) {
                        a.part_ml[pidx * 2] = M;
                        a.part_ml[pidx * 2 + 1] = L;
                    }
                }
            }
        }
    }
    if (nsplit_here == 1) return;
    if (a.stream_merge) {
        // The first CTAs of the kv head fold the partials, 64 columns of one query head at
        // a time; they poll the words themselves (bounded), nobody else waits for anything.
        constexpr int HALVES = HD / 64;
        const int nm = min(G * HALVES, nsplit_here);
        if (split >= nm) return;
        __syncthreads();   // the ring area is reused as merge scratch: every thread is done with merge_warps
        for (int m = split; m < G * HALVES; m += nm) {
            const int g = m / HALVES, half = m - g * HALVES;
            const size_t hrow = (size_t)r * H + (size_t)kv_h * G + g;
            if (!merge_head_words<HD, C::THREADS>(pw, pmlw, hrow * a.max_splits, nsplit_here, a.epoch, sm.stages,
                                                  a.out + hrow * HD, a.lse_out ? a.lse_out + hrow : nullptr, a.gather, hrow,
                                                  half, a.status))
                return;
        }
        return;
    }
    // ---- two-level merge by "last finisher" tickets: the last CTA of each group
    // of MERGE_GROUP splits folds the group, the last group folds the groups ----
    const int ngroups = (nsplit_here + MERGE_GROUP - 1) / MERGE_GROUP;
    const int grp = split / MERGE_GROUP;
    const int gsize = min(MERGE_GROUP, nsplit_here - grp * MERGE_GROUP);
    const size_t rk = (size_t)r * KV + kv_h;
    if (!take_last_ticket(a.tickets + a.batch * KV + rk * a.max_groups + grp, gsize, sm.flag)) return;
    if (ngroups == 1) {
        merge_partials<HD, G, C::THREADS>(a.part_o, a.part_ml, a.max_splits, 0, nsplit_here, r, kv_h, H, true, a.out, nullptr,
                                          nullptr, 0, 0, a.lse_out);
        return;
    }
    merge_partials<HD, G, C::THREADS>(a.part_o, a.part_ml, a.max_splits, grp * MERGE_GROUP, gsize, r, kv_h, H, false, nullptr,
                                      a.part2_o, a.part2_ml, a.max_groups, grp, nullptr);
    if (!take_last_ticket(a.tickets + rk, ngroups, sm.flag)) return;
    merge_partials<HD, G, C::THREADS>(a.part2_o, a.part2_ml, a.max_groups, 0, ngroups, r, kv_h, H, true, a.out, nullptr,
                                      nullptr, 0, 0, a.lse_out);
}

template <class K>
cudaError_t set_smem_once(K kernel, size_t smem, std::atomic<unsigned long long>& configured) {
    // one bit per device; two threads that race here both set the attribute, which is harmless
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64 || !(configured.load(std::memory_order_acquire) >> dev & 1ull)) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev < 64) configured.fetch_or(1ull << dev, std::memory_order_release);
    }
    return cudaSuccess;
}

template <int HD, int G, class C = SK<HD, G>>
cudaError_t launch_sk(const AttnArgs& a, cudaStream_t s) {
    static std::atomic<unsigned long long> configured{0};  // bit per device
    cudaError_t e = set_smem_once(attn_splitk_kernel<HD, G, C>, C::SMEM_BYTES, configured);
    if (e != cudaSuccess) return e;
    const int rows = a.batch * a.T;
    dim3 grid(a.max_splits, a.hs.num_kv_heads, rows);
    attn_splitk_kernel<HD, G, C><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (a.max_splits > 1) {
        dim3 cg(a.hs.num_heads, rows);
        attn_combine_kernel<HD><<<cg, HD, 0, s>>>(a);
        e = cudaGetLastError();
    }
    return e;
}

template <int HD, int G, class C = SK<HD, G>>
cudaError_t launch_fused(const FusedArgs& a, cudaStream_t s) {
    static std::atomic<unsigned long long> configured{0};
    cudaError_t e = set_smem_once(attn_decode_fused_kernel<HD, G, C>, C::SMEM_BYTES, configured);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.max_splits, a.hs.num_kv_heads, a.batch);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<HD, G, C>, a);
}

template <class A, class F>
cudaError_t dispatch_g(const A& a, F&& f) {
    switch (a.hs.num_heads / a.hs.num_kv_heads) {
        case 1: return f(std::integral_constant<int, 1>{});
        case 2: return f(std::integral_constant<int, 2>{});
        case 4: return f(std::integral_constant<int, 4>{});
        case 8: return f(std::integral_constant<int, 8>{});
        case 16: return f(std::integral_constant<int, 16>{});
        default: return cudaErrorInvalidValue;
    }
}

// Receiver side of the exchange: every thread polls its {value, epoch} words until
// they carry this epoch (bounded) and writes the values to the float area.
// Launched with programmatic stream serialization: it polls while the kernel ahead
// of it still runs, and the kernel behind it in the stream may become resident at
// once and prefetch what does not depend on this wait; that kernel's own
// grid-dependency wait then covers this kernel's completion.  The wait limit
// therefore has to cover the run time of the kernel ahead as well.
constexpr int GATHER_WAIT_THREADS = 256;
__global__ void __launch_bounds__(GATHER_WAIT_THREADS) gather_wait_kernel(const unsigned long long* words, float* data,
                                                                          long long count, unsigned epoch,
                                                                          unsigned long long limit_ns, AttnStatus* status) {
    grid_launch_dependents();
    const unsigned long long t0 = globaltimer_ns();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        while (true) {
            unsigned long long w;
            asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(words + i) : "memory");
            if ((unsigned)(w >> 32) == epoch) {
                data[i] = __uint_as_float((unsigned)w);
                break;
            }
            if (globaltimer_ns() - t0 > limit_ns) {
                if (status != nullptr && atomicCAS(&status->code, DEV_OK, DEV_WAIT_TIMEOUT) == DEV_OK) status->where = 21;
                return;
            }
        }
    }
    // The words may arrive while the kernel ahead in the stream (this rank's own
    // decode kernel) is still finishing; completing only after it keeps the
    // stream's order for whatever follows.
    grid_dependency_wait();
}

// out_full[(g*Hr + h)*hd + d] = sum_p w_p o_p / sum_p w_p with w_p = exp(lse_p - max lse)
__global__ void merge_parts_kernel(const float* __restrict__ gathered, int seq_parts, int heads_per_rank, int head_dim,
                                   float* __restrict__ out_full) {
    const int g = blockIdx.y, h = blockIdx.x;
    const size_t rank_stride = (size_t)heads_per_rank * (head_dim + 1);
    float mx = -INFINITY;
    for (int p = 0; p < seq_parts; ++p)
        mx = fmaxf(mx, gathered[(size_t)(g * seq_parts + p) * rank_stride + (size_t)heads_per_rank * head_dim + h]);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f, wsum = 0.0f;
        for (int p = 0; p < seq_parts; ++p) {
            const float* base = gathered + (size_t)(g * seq_parts + p) * rank_stride;
            const float lse = base[(size_t)heads_per_rank * head_dim + h];
            const float w = (lse == -INFINITY) ? 0.0f : expf(lse - mx);
            wsum += w;
            acc = fmaf(w, base[(size_t)h * head_dim + d], acc);
        }
        out_full[((size_t)g * heads_per_rank + h) * head_dim + d] = acc / wsum;
    }
}

// Wait and merge in one kernel, for a sequence that is split over the ranks of a head
// group: block (h, g) polls the {value, epoch} words of head h of the seq_parts ranks of
// group g (rows and log-sum-exp values, bounded) and writes the merged row; nothing is
// unpacked in between.  Launched like gather_wait_kernel.
__global__ void __launch_bounds__(128) gather_merge_kernel(const unsigned long long* words, int seq_parts,
                                                           int heads_per_rank, int head_dim, unsigned epoch,
                                                           unsigned long long limit_ns, float* __restrict__ out_full,
                                                           AttnStatus* status) {
    grid_launch_dependents();
    const int g = blockIdx.y, h = blockIdx.x;
    const size_t rank_stride = (size_t)heads_per_rank * (head_dim + 1);
    const unsigned long long t0 = globaltimer_ns();
    bool ok = true;
    auto take = [&](const unsigned long long* p) -> float {
        while (true) {
            unsigned long long w;
            asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
            if ((unsigned)(w >> 32) == epoch) return __uint_as_float((unsigned)w);
            if (globaltimer_ns() - t0 > limit_ns) {
                if (status != nullptr && atomicCAS(&status->code, DEV_OK, DEV_WAIT_TIMEOUT) == DEV_OK) status->where = 22;
                ok = false;
                return 0.0f;
            }
        }
    };
    constexpr int MAXP = 16;   // ranks per head group (MAX_PEERS)
    float lse[MAXP];
    float mx = -INFINITY;
    for (int p = 0; p < seq_parts && p < MAXP; ++p) {
        lse[p] = take(words + (size_t)(g * seq_parts + p) * rank_stride + (size_t)heads_per_rank * head_dim + h);
        mx = fmaxf(mx, lse[p]);
    }
    for (int d = threadIdx.x; d < head_dim && ok; d += blockDim.x) {
        float acc = 0.0f, wsum = 0.0f;
        for (int p = 0; p < seq_parts && p < MAXP; ++p) {
            const float o = take(words + (size_t)(g * seq_parts + p) * rank_stride + (size_t)h * head_dim + d);
            const float w = (lse[p] == -INFINITY) ? 0.0f : expf(lse[p] - mx);
            wsum += w;
            acc = fmaf(w, o, acc);
        }
        if (ok) out_full[((size_t)g * heads_per_rank + h) * head_dim + d] = acc / wsum;
    }
    grid_dependency_wait();
}

}  // namespace

cudaError_t launch_gather_wait(const unsigned long long* words, float* data, long long count, unsigned epoch,
                               unsigned long long limit_ns, AttnStatus* status, cudaStream_t s) {
    if (count <= 0) return cudaSuccess;
    cudaLaunchConfig_t cfg{};
    long long blocks = (count + 2 * GATHER_WAIT_THREADS - 1) / (2 * GATHER_WAIT_THREADS);   // two words per thread
    if (blocks > 64) blocks = 64;
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(GATHER_WAIT_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_wait_kernel, words, data, count, epoch, limit_ns, status);
}

cudaError_t launch_gather_merge(const unsigned long long* words, int world, int seq_parts, int heads_per_rank, int head_dim,
                                unsigned epoch, unsigned long long limit_ns, float* out_full, AttnStatus* status,
                                cudaStream_t s) {
    if (seq_parts <= 0 || seq_parts > MAX_PEERS || world % seq_parts != 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(heads_per_rank, world / seq_parts);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_merge_kernel, words, seq_parts, heads_per_rank, head_dim, epoch, limit_ns, out_full,
                              status);
}

cudaError_t launch_merge_parts(const float* gathered, int world, int seq_parts, int heads_per_rank, int head_dim,
                               float* out_full, cudaStream_t s) {
    if (seq_parts <= 0 || world % seq_parts != 0) return cudaErrorInvalidValue;
    dim3 grid(heads_per_rank, world / seq_parts);
    merge_parts_kernel<<<grid, 128, 0, s>>>(gathered, seq_parts, heads_per_rank, head_dim, out_full);
    return cudaGetLastError();
}

bool splitk_supported(const HeadShape& hs) {
    const int g = hs.num_heads / hs.num_kv_heads;
    return (hs.head_dim == 64 || hs.head_dim == 128) && (g == 1 || g == 2 || g == 4 || g == 8 || g == 16);
}

int splitk_tile_rows(const HeadShape& hs, int kv_elem_bytes, bool batched) {
    const int g = hs.num_heads / hs.num_kv_heads;
    const int br = 2 * (16 / g);
    const int tw = br > 8 ? br : 8;          // SKDefault::TW
    return kv_elem_bytes == 2 ? skb_mul(g, batched) * tw : tw;  // SKB
}

int splitk_ctas_per_sm(const HeadShape& hs) {
    return 2 * splitk_tile_rows(hs, 4, false) * hs.head_dim * 4 > 16 * 1024 ? 1 : 2;  // SKDefault::CTAS_PER_SM
}

size_t splitk_scratch_floats(const HeadShape& hs, int rows, int max_splits) {
    return (size_t)rows * hs.num_heads * max_splits * (hs.head_dim + 2);
}

int fused_merge_groups(int max_splits) { return (max_splits + MERGE_GROUP - 1) / MERGE_GROUP; }

cudaError_t launch_attn_splitk(const AttnArgs& a, cudaStream_t s) {
    if (a.batch * a.T == 0) return cudaSuccess;
    if (a.hs.head_dim == 64) return dispatch_g(a, [&](auto g) { return launch_sk<64, decltype(g)::value>(a, s); });
    if (a.hs.head_dim == 128) return dispatch_g(a, [&](auto g) { return launch_sk<128, decltype(g)::value>(a, s); });
    return cudaErrorInvalidValue;
}

cudaError_t launch_decode_fused(const FusedArgs& a, cudaStream_t s) {
    if (a.batch == 0) return cudaSuccess;
    if (a.kv_elem_bytes == 2) {
        const bool batched = a.seqs.many != nullptr;   // the planner made the slices for this tile size (splitk_tile_rows)
        auto go = [&](auto hd) {
            constexpr int HD = decltype(hd)::value;
            return dispatch_g(a, [&](auto g) {
                constexpr int G = decltype(g)::value;
                if (batched) return launch_fused<HD, G, SKB<HD, G, skb_mul(G, true)>>(a, s);
                return launch_fused<HD, G, SKB<HD, G, skb_mul(G, false)>>(a, s);
            });
        };
        if (a.hs.head_dim == 64) return go(std::integral_constant<int, 64>{});
        if (a.hs.head_dim == 128) return go(std::integral_constant<int, 128>{});
        return cudaErrorInvalidValue;
    }
    if (a.kv_elem_bytes != 4) return cudaErrorInvalidValue;
    if (a.hs.head_dim == 64) return dispatch_g(a, [&](auto g) { return launch_fused<64, decltype(g)::value>(a, s); });
    if (a.hs.head_dim == 128) return dispatch_g(a, [&](auto g) { return launch_fused<128, decltype(g)::value>(a, s); });
    return cudaErrorInvalidValue;
}

}  // namespace shainet

// ---------------------------------------------------------------------------
// Decode without any allocation.
//
// Some hosts cannot let a library allocate device memory on their behalf: an
// inference server that has handed the GPU's whole memory budget to its own
// pool at start-up (a later cudaMalloc from inside a library can fail, or
// fragment what the pool planned for), and a latency-critical token loop in
// which cudaMalloc/cudaFree are unwelcome because they synchronise the whole
// device and stall every stream.  For them this entry point runs the plain
// split-K decode kernel and its merge kernel with the per-split partials kept
// in a fixed array that is part of the library image instead of in a buffer the
// context grows on demand.  It calls no cudaMalloc, no cudaFree and no library
// routine that allocates.
//
// Limits and rules, all consequences of the array being one fixed global:
//  * it is NOALLOC_SCRATCH_FLOATS floats (4 MiB) and every GPU whose context
//    loads this library holds it until the process exits;
//  * a call needs num_heads * splits * (head_dim + 2) floats of it, where
//    splits is the planner's count (at most two CTAs per SM spread over the kv
//    heads); a shape that needs more is refused with SHAINET_ATTN_E_UNSUPPORTED;
//  * all calls share the array and it keeps whatever the last call left there.
//    Nothing in it has to start at zero: every entry the merge kernel reads was
//    written by the split kernel of the same call.  For the same reason two
//    calls that overlap on the GPU (different streams, no ordering between
//    them) race on it and give wrong results; order them;
//  * the address of the array is looked up once per device, by the first call
//    made with that device current (cudaGetSymbolAddress; the symbol's name is
//    only a host-side handle, never a device address).  Make that first call
//    before any stream capture begins.  The look-up is serialised by a mutex, so
//    threads may make their first calls concurrently;
//  * there is no context and therefore no device status word: should one of the
//    kernel's bounded waits on its shared-memory pipeline ever run out (~1 s;
//    only a programming error can cause it), the kernel leaves its loop and the
//    call has long returned 0.  A device-side wait failure is NOT reported by
//    this entry; callers that need the report use a context and forward_dev.
// ---------------------------------------------------------------------------
namespace shainet {
namespace {

constexpr size_t NOALLOC_SCRATCH_FLOATS = size_t(1) << 20;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

struct NoAllocDevice {
    float* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[64];
std::mutex g_noalloc_mutex;   // guards the one-time set-up per device

}  // namespace
}  // namespace shainet

extern "C" int shainet_attn_decode_noalloc(const float* q_dev, const float* k_cache_dev, const float* v_cache_dev,
                                            float* out_dev, int start_pos, int num_heads, int heads_per_kv, int head_dim,
                                            int capacity, float scale, void* stream) {
    using namespace shainet;
    char msg[256];
    if (!q_dev || !k_cache_dev || !v_cache_dev || !out_dev) {
        set_last_error_message("shainet_attn_decode_noalloc: null pointer");
        return -1;  // SHAINET_ATTN_E_INVALID
    }
    if (num_heads <= 0 || heads_per_kv <= 0 || num_heads % heads_per_kv != 0 || start_pos < 0 || capacity <= start_pos) {
        set_last_error_message("shainet_attn_decode_noalloc: bad head counts, or start_pos outside the cache capacity");
        return -1;
    }
    if (((reinterpret_cast<uintptr_t>(q_dev) | reinterpret_cast<uintptr_t>(k_cache_dev) | reinterpret_cast<uintptr_t>(v_cache_dev) |
          reinterpret_cast<uintptr_t>(out_dev)) & 15u) != 0) {
        set_last_error_message("shainet_attn_decode_noalloc: device pointers must be 16-byte aligned");
        return -1;
    }
    const HeadShape hs{num_heads, num_heads / heads_per_kv, head_dim};
    if (!splitk_supported(hs)) {
        set_last_error_message("shainet_attn_decode_noalloc: needs head_dim 64 or 128 and 1, 2, 4, 8 or 16 query heads per kv head");
        return -4;  // SHAINET_ATTN_E_UNSUPPORTED
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_last_error_message("shainet_attn_decode_noalloc: no usable current device");
        return -2;  // SHAINET_ATTN_E_CUDA
    }
    NoAllocDevice nd;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        NoAllocDevice& slot = g_noalloc_dev[dev];
        if (!slot.scratch) {
            // One-time set-up for this device: resolve the array's device address.
            float* ptr = nullptr;
            int sms = 0;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || !ptr) {
                cudaGetLastError();
                snprintf(msg, sizeof msg, "shainet_attn_decode_noalloc: set-up failed: %s", cudaGetErrorString(e));
                set_last_error_message(msg);
                return -2;
            }
            slot.sm_count = sms;
            slot.scratch = ptr;
        }
        nd = slot;
    }
    AttnArgs a{};
    a.q_rot = q_dev;
    a.out = out_dev;
    a.seqs.one = SeqDesc{const_cast<float*>(k_cache_dev), const_cast<float*>(v_cache_dev), start_pos, capacity};
    a.seqs.many = nullptr;
    a.batch = 1;
    a.T = 1;
    a.hs = hs;
    a.scale = scale;
    a.status = nullptr;
    const int visible = start_pos + 1;
    const int tw = splitk_tile_rows(hs, 4, false);
    const long long ctas = (long long)nd.sm_count * splitk_ctas_per_sm(hs);
    long long chunk = ((long long)visible * hs.num_kv_heads + ctas - 1) / ctas;
    if (chunk < 4ll * tw) chunk = 4ll * tw;
    chunk = (chunk + tw - 1) / tw * tw;
    a.chunk_rows = (int)chunk;
    a.max_splits = (int)((visible + chunk - 1) / chunk);
    const size_t need = splitk_scratch_floats(hs, 1, a.max_splits);
    if (need > NOALLOC_SCRATCH_FLOATS) {
        snprintf(msg, sizeof msg,
                 "shainet_attn_decode_noalloc: %d heads x %d splits x (head_dim + 2) = %zu floats exceeds the fixed scratch of %zu floats",
                 num_heads, a.max_splits, need, NOALLOC_SCRATCH_FLOATS);
        set_last_error_message(msg);
        return -4;
    }
    a.part_o = nd.scratch;
    a.part_ml = nd.scratch + (size_t)num_heads * a.max_splits * head_dim;
    e = launch_attn_splitk(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        cudaGetLastError();
        snprintf(msg, sizeof msg, "shainet_attn_decode_noalloc: launch failed: %s", cudaGetErrorString(e));
        set_last_error_message(msg);
        return -2;
    }
    return 0;
}
