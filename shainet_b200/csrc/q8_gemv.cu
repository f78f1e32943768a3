// Q8_0 weight-times-activation kernels for the decode step of SHAInet's LLaMA/Qwen
// block, sm_100a.
//
// Replaces the reference's gemm_q8_f32_kernel (src/shainet/native/cuda_kernels.cu:581-629:
// one 256-thread CTA per output element, every thread striding over K one int8 at a time)
// and, through the fused prologue and epilogues, the host loops around it:
//   * RMSNorm of the input row (src/shainet/transformer/rms_norm.cr:18-37: sum of squares and
//     the division in f64, fp32 store) as a prologue;
//   * residual add (SimpleMatrix#+, llama_block.cr:189-196) as an epilogue;
//   * SwiGLU, hidden = silu(gate) * up with silu in f64 (swiglu_ff.cr:76-91), as an epilogue
//     of a launch that walks the gate and the up weight side by side;
//   * lm_head bias add (basic/network_run.cr:222-226) and the greedy arg-max over the
//     logits (text/sampler.cr:38-53: first index of the largest finite value).
//
// Weight layout is the reference's (quantized_cuda_matrix.cr:74-115): int8 q[N][K]
// (output-major) and one fp32 scale per 32 consecutive K of an output, scales[N][K/32].
//
// The work is HBM-bound: 1 byte per weight plus 4 bytes per 32 weights, nothing else of
// size.  A warp owns a pair of output columns (for SwiGLU: gate column j and up column j)
// and walks K in segments of 2048: every lane loads 16 weights of a column with one
// 128-bit load, four such loads per column and segment, eight in flight per lane before
// the first is used, and the next segment's loads are issued before the current one is
// consumed.  int8 -> fp32 costs one byte-permute and half a packed add per weight: the
// byte is dropped into the mantissa of 2^23 (after flipping its sign bit) and 2^23 + 128
// is subtracted, which is exact.  The activation row sits in shared memory, permuted so
// that the 128-bit loads of a warp are conflict-free, and is shared by the two columns.
//
// Every kernel is launched with programmatic stream serialization: it requests its first
// weights BEFORE waiting for the previous kernel in the stream (weights never depend on
// it), waits, lets its own dependents start, and reads the activations.
#include <math.h>
#include <atomic>
#include "kernels.h"

namespace shainet {

bool q8_fast_path(int K);

namespace {

constexpr int Q8_THREADS = 256;
constexpr int Q8_WARPS = Q8_THREADS / 32;
constexpr int Q8_CHUNK = 512;    // K covered by one 128-bit load per lane
constexpr int Q8_SEG = 2048;     // K per unit of work: four chunks
constexpr unsigned FULL = 0xffffffffu;
constexpr int Q8_CTAS_PER_SM = 2;         // grid cap per SM (one per SM measured 15 % slower on the 16-layer decode chain)

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Four int8 of one 32-bit word (sign bits already flipped) -> four exact floats.
__device__ __forceinline__ void bytes_to_floats(unsigned u, float (&f)[4]) {
    constexpr float MAGIC = 8388736.0f;   // 2^23 + 128
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - MAGIC;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - MAGIC;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - MAGIC;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - MAGIC;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(FULL, v, off);
    return v;
}

// Order-preserving map of a float onto an unsigned (larger float -> larger key).
__device__ __forceinline__ unsigned float_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// The activations (x, the residual, token ids, arg-max words) are written by the kernel
// ahead in the stream while this kernel may already be resident, so they are read with
// L2-only loads (__ldcg) after the wait, never through the non-coherent path, which may
// keep a line from before the write.  Weights, scales, norm weights and biases are
// constants and do take that path.
//
// Activation rows into shared memory, optionally RMS-normalised, in the permuted order
// the main loop reads: element k of a row (chunk = k / 512, r = k % 512) goes to
// chunk*512 + ((r % 16) / 4)*128 + (r / 16)*4 + r % 4, so lane l's j-th float4 of a
// chunk is at chunk*512 + j*128 + l*4 and a warp's 128-bit loads touch 512 consecutive bytes.
// Each thread owns up to Q8_XREG float4 of a row (destination order); the norm weights for
// them are constants and are fetched before the wait for the previous kernel.
constexpr int Q8_XREG = 4;   // covers K <= 4096 from registers; wider rows re-read x from L2

template <int MB>
__device__ __forceinline__ void stage_rows(const Q8GemvArgs& a, int m0, int rows, float* xs, double* red,
                                           const float4 (&gam)[Q8_XREG]) {
    const int K = a.K;
    const int n4 = K >> 2;
    const bool in_regs = n4 <= Q8_XREG * Q8_THREADS;
    for (int m = 0; m < MB; ++m) {
        const bool live = m < rows;
        const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)(m0 + (live ? m : 0)) * K);
        float4* dst = reinterpret_cast<float4*>(xs + (size_t)m * K);
        // destination float4 d = chunk*128 + j*32 + l  <-  source float4 chunk*128 + l*4 + j
        auto source_of = [](int d) { return ((d >> 7) << 7) + ((d & 31) << 2) + ((d >> 5) & 3); };
        float4 xr[Q8_XREG];
        double sq = 0.0;
#pragma unroll
        for (int it = 0; it < Q8_XREG; ++it) {
            const int d = threadIdx.x + it * Q8_THREADS;
            xr[it] = (live && d < n4) ? __ldcg(src + source_of(d)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (a.gamma == nullptr) {
            if (in_regs) {
#pragma unroll
                for (int it = 0; it < Q8_XREG; ++it) {
                    const int d = threadIdx.x + it * Q8_THREADS;
                    if (d < n4) dst[d] = xr[it];
                }
            } else {
                for (int d = threadIdx.x; d < n4; d += Q8_THREADS)
                    dst[d] = live ? __ldcg(src + source_of(d)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            continue;
        }
        // rms_norm.cr:29-31: sq_sum over f64(x)^2, rms = sqrt(sq_sum / cols + eps)
        if (in_regs) {
#pragma unroll
            for (int it = 0; it < Q8_XREG; ++it) {
                const float4 v = xr[it];
                sq += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
            }
        } else {
            for (int d = threadIdx.x; d < n4; d += Q8_THREADS) {
                const float4 v = live ? __ldcg(src + d) : make_float4(0.f, 0.f, 0.f, 0.f);
                sq += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
            }
        }
        sq = warp_sum(sq);
        if (m > 0) __syncthreads();   // red[] of the previous row has been read
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
        __syncthreads();
        double tot = 0.0;
#pragma unroll
        for (int w = 0; w < Q8_WARPS; ++w) tot += red[w];
        // 1 / rms; rsqrt is within an ulp of the f64 quotient, far below the fp32 rounding that follows
        const double inv_rms = rsqrt(tot / (double)K + a.eps);
        // rms_norm.cr:32: f32((f64 x / rms) * f64 g), the division as a product with 1/rms
        auto normed = [&](float4 v, float4 g) {
            v.x = (float)(((double)v.x * inv_rms) * (double)g.x);
            v.y = (float)(((double)v.y * inv_rms) * (double)g.y);
            v.z = (float)(((double)v.z * inv_rms) * (double)g.z);
            v.w = (float)(((double)v.w * inv_rms) * (double)g.w);
            return v;
        };
        if (in_regs) {
#pragma unroll
            for (int it = 0; it < Q8_XREG; ++it) {
                const int d = threadIdx.x + it * Q8_THREADS;
                if (d < n4) dst[d] = normed(xr[it], gam[it]);
            }
        } else {
            for (int d = threadIdx.x; d < n4; d += Q8_THREADS) {
                const int s = source_of(d);
                const float4 v = live ? __ldcg(src + s) : make_float4(0.f, 0.f, 0.f, 0.f);
                dst[d] = normed(v, __ldg(reinterpret_cast<const float4*>(a.gamma) + s));
            }
        }
    }
    __syncthreads();
}

struct Unit {
    uint4 w[2][4];   // [column of the pair][chunk]: 16 weights each
    float s[2][4];   // their block scales
};

template <bool SWIGLU>
__device__ __forceinline__ void load_unit(const Q8GemvArgs& a, int pair, int seg, int lane, Unit& u) {
    const int kb = a.K >> 5;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int n = SWIGLU ? pair : 2 * pair + c;
        const bool valid = n < a.N;
        const signed char* qbase = (SWIGLU && c == 1) ? a.q2 : a.q;
        const float* sbase = (SWIGLU && c == 1) ? a.scales2 : a.scales;
        const signed char* qrow = qbase + (size_t)(valid ? n : 0) * a.K + (size_t)seg * Q8_SEG + lane * 16;
        const float* srow = sbase + (size_t)(valid ? n : 0) * kb + seg * (Q8_SEG / 32) + (lane >> 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            u.w[c][j] = valid ? ldg_stream_v4(qrow + j * Q8_CHUNK) : make_uint4(0u, 0u, 0u, 0u);
            u.s[c][j] = valid ? __ldg(srow + j * (Q8_CHUNK / 32)) : 0.0f;
        }
    }
}

template <int MB>
__device__ __forceinline__ void consume_unit(const Unit& u, const float* xs, int K, int seg, int lane, float (&acc)[MB][2]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float4 xv[MB][4];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
                xv[m][jj] = *reinterpret_cast<const float4*>(xs + (size_t)m * K + (seg * 4 + j) * Q8_CHUNK + jj * 128 + lane * 4);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const unsigned words[4] = {u.w[c][j].x ^ 0x80808080u, u.w[c][j].y ^ 0x80808080u, u.w[c][j].z ^ 0x80808080u,
                                       u.w[c][j].w ^ 0x80808080u};
            float part[MB];
#pragma unroll
            for (int m = 0; m < MB; ++m) part[m] = 0.0f;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float f[4];
                bytes_to_floats(words[jj], f);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    part[m] = fmaf(f[0], xv[m][jj].x, part[m]);
                    part[m] = fmaf(f[1], xv[m][jj].y, part[m]);
                    part[m] = fmaf(f[2], xv[m][jj].z, part[m]);
                    part[m] = fmaf(f[3], xv[m][jj].w, part[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[m][c] = fmaf(part[m], u.s[c][j], acc[m][c]);
        }
    }
}

// y[m0 .. m0+MB) x all N columns; gridDim.y walks the row tiles.
template <int MB, bool SWIGLU>
__global__ void __launch_bounds__(Q8_THREADS, MB == 1 ? 2 : 1) q8_gemv_kernel(Q8GemvArgs a) {
    extern __shared__ __align__(16) float q8_xs[];   // [MB][K] permuted activations
    __shared__ double red[Q8_WARPS];
    __shared__ unsigned long long best_sh[4];        // MB <= 4
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * MB;
    const int rows = min(MB, a.M - m0);
    const int nseg = a.K / Q8_SEG;
    const int pairs = SWIGLU ? a.N : (a.N + 1) / 2;
    const int gw = blockIdx.x * Q8_WARPS + warp, tw = gridDim.x * Q8_WARPS;

    // weights first: they do not depend on the kernel ahead in the stream
    Unit cur;
    if (gw < pairs) load_unit<SWIGLU>(a, gw, 0, lane, cur);
    float4 gam[Q8_XREG];   // norm weights of this thread's slots of a row: constants too
#pragma unroll
    for (int it = 0; it < Q8_XREG; ++it) {
        const int d = threadIdx.x + it * Q8_THREADS;
        gam[it] = (a.gamma != nullptr && d < (a.K >> 2) && (a.K >> 2) <= Q8_XREG * Q8_THREADS)
                      ? __ldg(reinterpret_cast<const float4*>(a.gamma) + ((d >> 7) << 7) + ((d & 31) << 2) + ((d >> 5) & 3))
                      : make_float4(1.f, 1.f, 1.f, 1.f);
    }
    // Dependents are released only after this kernel's own wait has returned: at most one
    // kernel then runs ahead of its predecessor, so a kernel's early phase can never overlap
    // anything older than the kernel directly ahead of it in the stream.
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x < 4) best_sh[threadIdx.x] = 0ull;
    stage_rows<MB>(a, m0, rows, q8_xs, red, gam);

    unsigned long long best[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) best[m] = 0ull;

    for (int pair = gw; pair < pairs; pair += tw) {
        float acc[MB][2];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m][0] = acc[m][1] = 0.0f;
        for (int seg = 0; seg < nseg; ++seg) {
            // request the next unit before using this one
            Unit nxt;
            const bool more_seg = seg + 1 < nseg;
            const int npair = more_seg ? pair : pair + tw;
            const bool have_next = npair < pairs;
            if (have_next) load_unit<SWIGLU>(a, npair, more_seg ? seg + 1 : 0, lane, nxt);
            consume_unit<MB>(cur, q8_xs, a.K, seg, lane, acc);
            if (have_next) cur = nxt;
        }
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc[m][c] += __shfl_xor_sync(FULL, acc[m][c], off);
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                if (m >= rows) break;
                const size_t row = (size_t)(m0 + m) * a.N;
                if (SWIGLU) {
                    // swiglu_ff.cr:83-88: the element access widens to f64, silu in f64, fp32 store
                    const double g = (double)acc[m][0], up = (double)acc[m][1];
                    a.y[row + pair] = (float)((g / (1.0 + exp(-g))) * up);
                } else {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int n = 2 * pair + c;
                        if (n >= a.N) break;
                        float v = acc[m][c];
                        if (a.bias != nullptr) v = __fadd_rn(v, a.bias[n]);
                        if (a.residual != nullptr) v = __fadd_rn(__ldcg(a.residual + row + n), v);
                        a.y[row + n] = v;
                        if (a.argmax != nullptr && isfinite(v)) {
                            const unsigned long long cand = ((unsigned long long)float_key(v) << 32) | (0xffffffffu - (unsigned)n);
                            best[m] = cand > best[m] ? cand : best[m];
                        }
                    }
                }
            }
        }
    }
    if (a.argmax != nullptr) {
        // one atomic per CTA and row: the largest key wins, among equal values the smallest index
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MB; ++m)
                if (best[m] != 0ull) atomicMax(&best_sh[m], best[m]);
        }
        __syncthreads();
        if (threadIdx.x < rows && best_sh[threadIdx.x] != 0ull) atomicMax(a.argmax + m0 + threadIdx.x, best_sh[threadIdx.x]);
    }
}

// ---------------------------------------------------------------------------
// Single-row GEMV with the weights streamed through shared memory by the TMA engine.
//
// A stage is four output columns x 2048 inputs: four 2 KB bulk copies of int8 weights and
// four 256-byte copies of their scales land on one mbarrier.  A producer thread keeps a ring
// of such stages full; each of eight consumer warps owns the stages whose slot number equals
// its index modulo eight (an mbarrier parity wait is only valid for a waiter that has seen
// the previous phase, which a fixed slot -> warp map guarantees).  The ring is filled before
// the wait for the previous kernel, so a kernel that becomes resident while its predecessor
// still runs already holds its first 72 KB of weights per SM when the activations arrive.
// A CTA owns a contiguous range of column quads; its warps leave one partial sum per
// (quad, 2048-input segment, column) in shared memory and the CTA folds the segments in
// order at the end, so results do not depend on timing.
// ---------------------------------------------------------------------------
constexpr int RG_NW = 8;
constexpr int RG_THREADS = (RG_NW + 1) * 32;
constexpr int RG_COLS = 4;
constexpr int RG_WBYTES = RG_COLS * Q8_SEG;              // 8192
constexpr int RG_SBYTES = RG_COLS * (Q8_SEG / 32) * 4;   // 1024
constexpr int RG_STAGE = RG_WBYTES + RG_SBYTES;          // 9216
constexpr int RG_CTAS_PER_SM = 2;   // sixteen consumer warps per SM; one CTA per SM measured 40 % slower on the decode chain

typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 fadd2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

template <int NS, bool SWIGLU>
__global__ void __launch_bounds__(RG_THREADS, 2) q8_gemv_ring_kernel(Q8GemvArgs a, int quads_per_cta) {
    extern __shared__ __align__(128) unsigned char rg_raw[];
    unsigned char* ring = rg_raw;                                             // [NS][RG_STAGE]
    float* xs = reinterpret_cast<float*>(rg_raw + (size_t)NS * RG_STAGE);     // [K] permuted activations
    const int nseg = a.K / Q8_SEG;
    const int vmul = SWIGLU ? 2 : 1;
    float* part = xs + a.K;                                                   // [local stages][RG_COLS]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(part + (size_t)quads_per_cta * vmul * nseg * RG_COLS);
    uint64_t* empty_bar = full_bar + NS;
    double* red = reinterpret_cast<double*>(empty_bar + NS);                  // [RG_NW]
    unsigned long long* best_sh = reinterpret_cast<unsigned long long*>(red + RG_NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quads = a.N / RG_COLS;
    const int q0 = blockIdx.x * quads_per_cta;
    const int q1 = min(quads, q0 + quads_per_cta);
    const int n_local = q1 > q0 ? (q1 - q0) * vmul * nseg : 0;   // stages of this CTA; stage i = ((quad - q0) * vmul + matrix) * nseg + seg
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        *best_sh = 0ull;
        fence_mbar_init();
    }
    __syncthreads();

    auto issue = [&](int i) {
        const int slot = i % NS;
        const int seg = i % nseg, v = i / nseg;
        const int quad = q0 + v / vmul;
        const bool second = SWIGLU && (v & 1);
        const signed char* qb = (second ? a.q2 : a.q) + (size_t)quad * RG_COLS * a.K + (size_t)seg * Q8_SEG;
        const float* sb = (second ? a.scales2 : a.scales) + (size_t)quad * RG_COLS * (a.K >> 5) + seg * (Q8_SEG / 32);
        unsigned char* st = ring + (size_t)slot * RG_STAGE;
        mbar_arrive_expect_tx(&full_bar[slot], RG_STAGE);
#pragma unroll
        for (int c = 0; c < RG_COLS; ++c) {
            bulk_g2s(st + c * Q8_SEG, qb + (size_t)c * a.K, Q8_SEG, &full_bar[slot]);
            bulk_g2s(st + RG_WBYTES + c * (Q8_SEG / 8), sb + (size_t)c * (a.K >> 5), Q8_SEG / 8, &full_bar[slot]);
        }
    };

    if (warp == RG_NW) {
        // ---------------- producer: weights are constants, nothing to wait for but free slots ----------------
        if (lane == 0) {
            for (int i = 0; i < n_local; ++i) {
                if (i >= NS && !mbar_wait(&empty_bar[i % NS], ((i / NS) - 1) & 1, nullptr, 0)) break;
                issue(i);
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int n4 = a.K >> 2;
        auto source_of = [](int d) { return ((d >> 7) << 7) + ((d & 31) << 2) + ((d >> 5) & 3); };
        float4 gam[Q8_XREG];
        const bool in_regs = n4 <= Q8_XREG * RG_NW * 32;
#pragma unroll
        for (int it = 0; it < Q8_XREG; ++it) {
            const int d = threadIdx.x + it * RG_NW * 32;
            gam[it] = (a.gamma != nullptr && in_regs && d < n4) ? __ldg(reinterpret_cast<const float4*>(a.gamma) + source_of(d))
                                                                : make_float4(1.f, 1.f, 1.f, 1.f);
        }
        pdl_wait();
        pdl_launch_dependents();
        // activations into shared memory (permuted), RMS-normalised if asked (rms_norm.cr:18-37)
        const float4* src = reinterpret_cast<const float4*>(a.x);
        float4* dst = reinterpret_cast<float4*>(xs);
        if (a.gamma == nullptr && !in_regs) {
            // a wide row without a norm (the FFN's down projection): eight loads in flight per thread
            for (int base = threadIdx.x; base < n4; base += 8 * RG_NW * 32) {
                float4 t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int d = base + u * RG_NW * 32;
                    t[u] = d < n4 ? __ldcg(src + source_of(d)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int d = base + u * RG_NW * 32;
                    if (d < n4) dst[d] = t[u];
                }
            }
        }
        float4 xr[Q8_XREG];
#pragma unroll
        for (int it = 0; it < Q8_XREG; ++it) {
            const int d = threadIdx.x + it * RG_NW * 32;
            xr[it] = (in_regs && d < n4) ? __ldcg(src + source_of(d)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        double inv_rms = 1.0;
        if (a.gamma != nullptr) {
            double sq = 0.0;
            if (in_regs) {
#pragma unroll
                for (int it = 0; it < Q8_XREG; ++it) {
                    const float4 v = xr[it];
                    sq += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
                }
            } else {
                for (int d = threadIdx.x; d < n4; d += RG_NW * 32) {
                    const float4 v = __ldcg(src + d);
                    sq += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
                }
            }
            sq = warp_sum(sq);
            if (lane == 0) red[warp] = sq;
            asm volatile("bar.sync 1, %0;" ::"n"(RG_NW * 32) : "memory");
            double tot = 0.0;
#pragma unroll
            for (int w = 0; w < RG_NW; ++w) tot += red[w];
            inv_rms = rsqrt(tot / (double)a.K + a.eps);
        }
        auto normed = [&](float4 v, float4 g) {
            v.x = (float)(((double)v.x * inv_rms) * (double)g.x);
            v.y = (float)(((double)v.y * inv_rms) * (double)g.y);
            v.z = (float)(((double)v.z * inv_rms) * (double)g.z);
            v.w = (float)(((double)v.w * inv_rms) * (double)g.w);
            return v;
        };
        if (in_regs) {
#pragma unroll
            for (int it = 0; it < Q8_XREG; ++it) {
                const int d = threadIdx.x + it * RG_NW * 32;
                if (d < n4) dst[d] = a.gamma != nullptr ? normed(xr[it], gam[it]) : xr[it];
            }
        } else if (a.gamma != nullptr) {
            for (int d = threadIdx.x; d < n4; d += RG_NW * 32) {
                const int sidx = source_of(d);
                dst[d] = normed(__ldcg(src + sidx), __ldg(reinterpret_cast<const float4*>(a.gamma) + sidx));
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(RG_NW * 32) : "memory");

        const f32x2 neg_magic = pk2(-8388736.0f, -8388736.0f);   // -(2^23 + 128)
        for (int i = warp; i < n_local; i += RG_NW) {
            const int slot = i % NS;
            if (!mbar_wait(&full_bar[slot], (i / NS) & 1, nullptr, 0)) break;
            const unsigned char* st = ring + (size_t)slot * RG_STAGE;
            const float* sc = reinterpret_cast<const float*>(st + RG_WBYTES);
            const int seg = i % nseg;
            float acc[RG_COLS];
#pragma unroll
            for (int c = 0; c < RG_COLS; ++c) acc[c] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                ulonglong2 xv[4];   // 16 activations of this lane as packed pairs
#pragma unroll
                for (int jj = 0; jj < 4; ++jj)
                    xv[jj] = *reinterpret_cast<const ulonglong2*>(xs + (seg * 4 + j) * Q8_CHUNK + jj * 128 + lane * 4);
#pragma unroll
                for (int c = 0; c < RG_COLS; ++c) {
                    const uint4 w = *reinterpret_cast<const uint4*>(st + c * Q8_SEG + j * Q8_CHUNK + lane * 16);
                    const float scale = sc[c * (Q8_SEG / 32) + j * (Q8_CHUNK / 32) + (lane >> 1)];
                    const unsigned words[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
                    f32x2 p2 = 0ull;
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const unsigned u = words[jj];
                        const f32x2 lo = fadd2(pk2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)),
                                                   __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651))), neg_magic);
                        const f32x2 hi = fadd2(pk2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)),
                                                   __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653))), neg_magic);
                        p2 = ffma2(lo, xv[jj].x, p2);
                        p2 = ffma2(hi, xv[jj].y, p2);
                    }
                    float plo, phi;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(plo), "=f"(phi) : "l"(p2));
                    acc[c] = fmaf(plo + phi, scale, acc[c]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot]);   // the stage's bytes are in registers / consumed
#pragma unroll
            for (int c = 0; c < RG_COLS; ++c)
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc[c] += __shfl_xor_sync(FULL, acc[c], off);
            if (lane == 0) *reinterpret_cast<float4*>(part + (size_t)i * RG_COLS) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
    }
    __syncthreads();
    // fold the segments of every column in order and finish the row
    const int cols_local = (q1 > q0 ? q1 - q0 : 0) * RG_COLS;
    unsigned long long best = 0ull;
    for (int e = threadIdx.x; e < cols_local; e += RG_THREADS) {
        const int ql = e / RG_COLS, c = e - ql * RG_COLS;
        const int n = (q0 + ql) * RG_COLS + c;
        float v0 = 0.0f, v1 = 0.0f;
        for (int sg = 0; sg < nseg; ++sg) {
            v0 += part[((size_t)(ql * vmul) * nseg + sg) * RG_COLS + c];
            if (SWIGLU) v1 += part[((size_t)(ql * vmul + 1) * nseg + sg) * RG_COLS + c];
        }
        if (SWIGLU) {
            const double g = (double)v0, up = (double)v1;
            a.y[n] = (float)((g / (1.0 + exp(-g))) * up);
        } else {
            float v = v0;
            if (a.bias != nullptr) v = __fadd_rn(v, a.bias[n]);
            if (a.residual != nullptr) v = __fadd_rn(__ldcg(a.residual + n), v);
            a.y[n] = v;
            if (a.argmax != nullptr && isfinite(v)) {
                const unsigned long long cand = ((unsigned long long)float_key(v) << 32) | (0xffffffffu - (unsigned)n);
                best = cand > best ? cand : best;
            }
        }
    }
    if (a.argmax != nullptr) {
        if (best != 0ull) atomicMax(best_sh, best);
        __syncthreads();
        if (threadIdx.x == 0 && *best_sh != 0ull) atomicMax(a.argmax, *best_sh);
    }
}

template <int NS, bool SWIGLU>
cudaError_t launch_ring(const Q8GemvArgs& a, int sm_count, cudaStream_t s) {
    const int quads = a.N / RG_COLS;
    int ctas = quads < sm_count * RG_CTAS_PER_SM ? quads : sm_count * RG_CTAS_PER_SM;
    const int qpc = (quads + ctas - 1) / ctas;
    ctas = (quads + qpc - 1) / qpc;
    const int nseg = a.K / Q8_SEG, vmul = SWIGLU ? 2 : 1;
    const size_t smem = (size_t)NS * RG_STAGE + (size_t)a.K * 4 + (size_t)qpc * vmul * nseg * RG_COLS * 4 + 2 * NS * 8 + RG_NW * 8 + 16;
    auto kern = q8_gemv_ring_kernel<NS, SWIGLU>;
    static std::atomic<unsigned long long> configured{0};   // bit per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64 || !(configured.load(std::memory_order_acquire) >> dev & 1ull)) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        if (dev < 64) configured.fetch_or(1ull << dev, std::memory_order_release);
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(RG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a, qpc);
}

constexpr int RG_NS = 8;   // ring stages (a multiple of the consumer warps): 72 KB

bool ring_ok(const Q8GemvArgs& a, int sm_count) {
    if (a.M != 1 || !q8_fast_path(a.K) || a.N % RG_COLS != 0) return false;
    // Long streams (the lm_head, 295 MB at a 128 K vocabulary) run faster through the register
    // kernel (4.6 against 3.8 TB/s measured); the ring pays off where a kernel is short and its
    // first 72 KB per CTA are already on chip when the activations arrive.
    if ((size_t)a.N * a.K * (a.q2 ? 2 : 1) > ((size_t)64 << 20)) return false;
    const int quads = a.N / RG_COLS;
    const int ctas = quads < sm_count * RG_CTAS_PER_SM ? quads : sm_count * RG_CTAS_PER_SM;
    const int qpc = (quads + ctas - 1) / ctas;
    const size_t smem = (size_t)RG_NS * RG_STAGE + (size_t)a.K * 4 + (size_t)qpc * (a.q2 ? 2 : 1) * (a.K / Q8_SEG) * RG_COLS * 4 + 512;
    return smem <= 200 * 1024;
}

// Any K (ragged last block included), any N: one warp per output element.  Small shapes
// of tests and models whose K is not a multiple of 2048; not a tuned path.
template <bool SWIGLU>
__global__ void __launch_bounds__(Q8_THREADS) q8_gemv_generic_kernel(Q8GemvArgs a) {
    extern __shared__ __align__(16) float q8_xs[];   // [K] activations of row blockIdx.y (normalised if asked)
    __shared__ double red[Q8_WARPS];
    __shared__ unsigned long long best_sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0) best_sh = 0ull;
    const float* xrow = a.x + (size_t)m * a.K;
    double inv_rms = 1.0;
    if (a.gamma != nullptr) {
        double sq = 0.0;
        for (int k = threadIdx.x; k < a.K; k += Q8_THREADS) {
            const double v = (double)__ldcg(xrow + k);
            sq += v * v;
        }
        sq = warp_sum(sq);
        if (lane == 0) red[warp] = sq;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < Q8_WARPS; ++w) tot += red[w];
        inv_rms = 1.0 / sqrt(tot / (double)a.K + a.eps);
    }
    for (int k = threadIdx.x; k < a.K; k += Q8_THREADS) {
        const float xv = __ldcg(xrow + k);
        q8_xs[k] = a.gamma != nullptr ? (float)(((double)xv * inv_rms) * (double)a.gamma[k]) : xv;
    }
    __syncthreads();
    const int kb = (a.K + 31) / 32;
    unsigned long long best = 0ull;
    for (int n = blockIdx.x * Q8_WARPS + warp; n < a.N; n += gridDim.x * Q8_WARPS) {
        float acc[2] = {0.0f, 0.0f};
        for (int c = 0; c < (SWIGLU ? 2 : 1); ++c) {
            const signed char* qrow = (c == 1 ? a.q2 : a.q) + (size_t)n * a.K;
            const float* srow = (c == 1 ? a.scales2 : a.scales) + (size_t)n * kb;
            float p = 0.0f;
            for (int k = lane; k < a.K; k += 32) p = fmaf((float)qrow[k] * q8_xs[k], srow[k >> 5], p);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) p += __shfl_xor_sync(FULL, p, off);
            acc[c] = p;
        }
        if (lane == 0) {
            const size_t row = (size_t)m * a.N;
            if (SWIGLU) {
                const double g = (double)acc[0], up = (double)acc[1];
                a.y[row + n] = (float)((g / (1.0 + exp(-g))) * up);
            } else {
                float v = acc[0];
                if (a.bias != nullptr) v = __fadd_rn(v, a.bias[n]);
                if (a.residual != nullptr) v = __fadd_rn(__ldcg(a.residual + row + n), v);
                a.y[row + n] = v;
                if (a.argmax != nullptr && isfinite(v)) {
                    const unsigned long long cand = ((unsigned long long)float_key(v) << 32) | (0xffffffffu - (unsigned)n);
                    best = cand > best ? cand : best;
                }
            }
        }
    }
    if (a.argmax != nullptr) {
        if (lane == 0 && best != 0ull) atomicMax(&best_sh, best);
        __syncthreads();
        if (threadIdx.x == 0 && best_sh != 0ull) atomicMax(a.argmax + m, best_sh);
    }
}

// x[t] = table[ids[t]] (EmbeddingLayer#embed_cpu, text/embedding_layer.cr:129-156) and the
// reset of the arg-max words the step's lm_head launch will fill.
__global__ void embed_rows_kernel(const int* ids, const float* __restrict__ table, float* x,
                                  int d_model, int vocab, unsigned long long* argmax_words, int n_words) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t == 0 && threadIdx.x < n_words) argmax_words[threadIdx.x] = 0ull;
    int id = __ldcg(ids + t);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const float4* src = reinterpret_cast<const float4*>(table + (size_t)id * d_model);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)t * d_model);
    for (int i = threadIdx.x; i < d_model / 4; i += blockDim.x) dst[i] = __ldg(src + i);
}

// token[m] = index packed in the arg-max word of row m (0 when no finite logit was seen,
// as Sampler.greedy returns); also stored where the next step's embedding reads its id.
__global__ void argmax_decode_kernel(const unsigned long long* words, int* tokens, int n, int* next_id, int* history,
                                     int history_pos) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= n) return;
    const unsigned long long w = __ldcg(words + m);
    const int tok = w == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(w & 0xffffffffull));
    tokens[m] = tok;
    if (m == n - 1) {
        if (next_id != nullptr) *next_id = tok;
        if (history != nullptr) history[history_pos] = tok;
    }
}

template <class Kern>
cudaError_t launch_pdl(Kern kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, const Q8GemvArgs& a) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <int MB, bool SWIGLU>
cudaError_t launch_fast(const Q8GemvArgs& a, int sm_count, cudaStream_t s) {
    const size_t smem = (size_t)MB * a.K * sizeof(float);
    auto kern = q8_gemv_kernel<MB, SWIGLU>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int pairs = SWIGLU ? a.N : (a.N + 1) / 2;
    const int row_tiles = (a.M + MB - 1) / MB;
    int gx = (pairs + Q8_WARPS - 1) / Q8_WARPS;
    const int cap = sm_count * Q8_CTAS_PER_SM;
    if (gx > cap) gx = cap;
    return launch_pdl(kern, dim3(gx, row_tiles), dim3(Q8_THREADS), smem, s, a);
}

}  // namespace

bool q8_fast_path(int K) { return K > 0 && K % Q8_SEG == 0 && (size_t)K * sizeof(float) <= 200 * 1024; }

cudaError_t launch_q8_gemv(const Q8GemvArgs& a, int sm_count, cudaStream_t s) {
    if (a.M <= 0 || a.N <= 0) return cudaSuccess;
    if (a.K <= 0) return cudaErrorInvalidValue;
    const bool swiglu = a.q2 != nullptr;
    if (q8_fast_path(a.K) && (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 && (!swiglu || (reinterpret_cast<uintptr_t>(a.q2) & 15u) == 0) &&
        (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && (a.gamma == nullptr || (reinterpret_cast<uintptr_t>(a.gamma) & 15u) == 0)) {
        if (ring_ok(a, sm_count)) return swiglu ? launch_ring<RG_NS, true>(a, sm_count, s) : launch_ring<RG_NS, false>(a, sm_count, s);
        // Rows are taken four at a time while that fits shared memory; a row tile re-reads the weights.
        const bool four = a.M >= 3 && (size_t)4 * a.K * sizeof(float) <= 160 * 1024;
        const bool two = !four && a.M >= 2 && (size_t)2 * a.K * sizeof(float) <= 160 * 1024;
        if (swiglu) {
            if (four) return launch_fast<4, true>(a, sm_count, s);
            if (two) return launch_fast<2, true>(a, sm_count, s);
            return launch_fast<1, true>(a, sm_count, s);
        }
        if (four) return launch_fast<4, false>(a, sm_count, s);
        if (two) return launch_fast<2, false>(a, sm_count, s);
        return launch_fast<1, false>(a, sm_count, s);
    }
    const size_t smem = (size_t)a.K * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    int gx = (a.N + Q8_WARPS - 1) / Q8_WARPS;
    if (gx > sm_count * 4) gx = sm_count * 4;
    if (swiglu) {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(q8_gemv_generic_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        return launch_pdl(q8_gemv_generic_kernel<true>, dim3(gx, a.M), dim3(Q8_THREADS), smem, s, a);
    }
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(q8_gemv_generic_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(q8_gemv_generic_kernel<false>, dim3(gx, a.M), dim3(Q8_THREADS), smem, s, a);
}

cudaError_t launch_embed_rows(const int* ids_dev, const float* table, float* x, int rows, int d_model, int vocab,
                              unsigned long long* argmax_words, int n_words, cudaStream_t s) {
    if (rows <= 0) return cudaSuccess;
    if (d_model % 4 != 0 || n_words > 128) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, embed_rows_kernel, ids_dev, table, x, d_model, vocab, argmax_words, n_words);
}

cudaError_t launch_argmax_decode(const unsigned long long* words, int* tokens, int n, int* next_id, int* history,
                                 int history_pos, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((n + 127) / 128);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, argmax_decode_kernel, words, tokens, n, next_id, history, history_pos);
}

}  // namespace shainet
