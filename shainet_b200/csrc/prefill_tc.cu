// Causal prefill attention over the KV cache on the 5th-generation tensor
// cores (tcgen05, TF32 inputs, fp32 accumulation in tensor memory), sm_100a.
//
// Replaces the reference's attention_kv_kernel
// (src/shainet/native/cuda_kernels.cu:734-806) when many new tokens arrive at
// once: that kernel runs one 128-thread CTA per (head, token), forms scores
// with scalar FMAs through a global scratch of heads x T x L floats (which
// overflows Int32 at 32 x 8192 x 8192, src/shainet/transformer/llama_block.cr:418)
// and never touches a tensor core.
//
// Two kernels.  With head_dim 128 and an even group size a cluster of two CTAs
// works as one tensor core (cta_group::2) on two query heads of one kv head:
// attn_prefill_pair_kernel, further down.  Otherwise (head_dim 64, or one query
// head per kv head) attn_prefill_tc2_kernel: one CTA owns two tiles of 128 query rows that
// see the same K/V tiles and walks the visible cache positions in tiles of 64:
//
//   S  = Q K^T      tcgen05.mma kind::tf32, A and B from shared memory (K-major),
//                   accumulator in tensor memory (two score buffers per query tile)
//   P  = exp2(S*c - max), written back over S in tensor memory
//   O += P V        tcgen05.mma with A from tensor memory, B = the V tile from
//                   shared memory (MN-major), accumulating in tensor memory
//
// Q, K and V tiles arrive by TMA (2-D tiled, 128-byte swizzle, no multicast)
// into mbarrier-guarded buffers.  Warp 0 is the TMA producer, warp 1 allocates
// tensor memory and issues the MMAs, warps 4-7 and 8-11 are the softmax
// warpgroups of the two query tiles: each thread owns one query row (= one TMEM
// lane), so row maxima and sums need no shuffles.  Every wait is bounded.
//
// The softmax is the same max-subtracted form as the reference's
// (llama_block.cr:346-373); TF32 rounds the inputs of both contractions to 10
// mantissa bits, which is the 2e-3 tolerance class of this path.
#include <cuda.h>
#include <math.h>
#include "kernels.h"

namespace shainet {

namespace {

constexpr float PF_LOG2E = 1.4426950408889634f;
// The tensor core drops the 13 low mantissa bits of an fp32 operand (truncation
// toward zero): every K and V element loses x * d with d in [0, 2^-10 / m) for a
// mantissa m in [1, 2), i.e. 2^-11 * ln 2 on average.  The cache stays fp32, so
// instead of rounding it the mean loss is put back as a constant factor on the
// scores (K) and on the output (V); what remains is zero-mean, like rounding to
// nearest.  q is rounded to nearest TF32 where it is written; P is handed over
// as fp32 bits and treated like V.
constexpr float PF_TRUNC_GAIN = 1.0f + 0.693147f / 2048.0f;

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// ---- a pair of CTAs (cluster of two) working as one tensor core: cta_group::2 ----
// The tile of the MMA is 256 rows, 128 per CTA; each CTA holds half of the B operand in its own
// shared memory and the hardware passes the halves across, so an SM reads half as many K/V bytes
// from shared memory per flop.  One thread of the even CTA issues for both.

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of the object at the same offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// TMA load into this CTA's shared memory that reports its bytes to a barrier of either CTA of the pair
// (`bar_cluster` is a shared::cluster address).  No multicast: every CTA fetches its own half.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}

// Arrival (once all MMAs issued so far by this thread have completed) on a barrier given by its
// shared::cluster address: the local one or the peer's copy.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// Bounded wait on a barrier of this CTA whose arrivals may come from the peer CTA.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, AttnStatus* status, int where) {
    const uint32_t addr = smem_u32(bar);
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            uint32_t ok;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                : "=r"(ok)
                : "r"(addr), "r"(parity)
                : "memory");
            if (ok) return true;
        }
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            if (status != nullptr && atomicCAS(&status->code, DEV_OK, DEV_WAIT_TIMEOUT) == DEV_OK) status->where = where;
            return false;
        }
    }
}

__device__ __forceinline__ void mma_ss_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_ts_tf32_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Shared-memory matrix descriptor (Blackwell version field set).
//  * K-major operand (Q, K): rows of 128 bytes swizzled in 16-byte chunks
//    (layout type 2 = SWIZZLE_128B), 8-row groups every 1024 bytes (SBO); the
//    leading offset is not used.
//  * MN-major 32-bit operand (V): the only layout the tensor core accepts is
//    the 128-byte span swizzled in 32-byte chunks (layout type 1 =
//    SWIZZLE_128B_BASE32B): rows (positions, the contraction index) of 128 bytes =
//    32 head-dim columns, 4-row groups every 512 bytes (SBO), further blocks of
//    32 columns every `lbo_bytes`.
constexpr uint32_t LAYOUT_SW128 = 2, LAYOUT_SW128_BASE32B = 1;

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version
    d |= (uint64_t)layout << 61;
    return d;
}

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return smem_desc(saddr, lbo_bytes, sbo_bytes, LAYOUT_SW128);
}

// Instruction descriptor: fp32 accumulate, TF32 A and B, dense.
__host__ __device__ constexpr uint32_t idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct PrefillArgs {
    float* out;    // [T, num_heads*head_dim]
    int T;         // new tokens (query rows)
    int start;     // cache positions before them
    int num_heads;
    int num_kv_heads;
    int capacity;
    float scale;
    AttnStatus* status;
};

// ---------------------------------------------------------------------------
// Two query tiles per CTA.  Both tiles walk the same K/V tiles (two query heads
// of one kv head over the same rows, or two consecutive row tiles of one head),
// so every K/V byte fetched from L2 feeds twice the tensor work.  The output
// accumulators stay in tensor memory: P.V accumulates straight into them, and a
// row is rescaled there only when its running maximum has grown by more than
// 2^8 since the scale in use was chosen (the probabilities then stay below 2^8,
// far inside fp32 range; the final division by the row sum, kept at the same
// scale, makes the result independent of the choice).  One warpgroup per tile
// does the softmax, one thread issues all MMAs, one thread all TMA loads.
// ---------------------------------------------------------------------------
template <int HD>
struct PF2 {
    static constexpr int BM = 128;              // query rows per tile, two tiles per CTA
    static constexpr int BN = 64;               // cache positions per K/V tile
    static constexpr int NBOX = HD / 32;        // 128-byte column blocks per row
    static constexpr int Q_BYTES = BM * HD * 4;   // one tile
    static constexpr int KV_BYTES = BN * HD * 4;  // one of K, V
    static constexpr int BAR_BYTES = 256;
    static constexpr size_t SMEM_BYTES = 1024 + 2 * Q_BYTES + 3 * KV_BYTES + BAR_BYTES;  // Q x2, K x2, V x1
    static constexpr int TMEM_S = 0;            // [tile][buffer] score/probability blocks of BN columns
    static constexpr int TMEM_O = 4 * BN;       // [tile] output accumulators of HD columns
    static constexpr int TMEM_COLS = 512;
    static constexpr int THREADS = 384;
    static constexpr float RESCALE_STEP = 8.0f; // log2 units
};

struct Prefill2Args {
    PrefillArgs p;
    int pair_heads;  // 1: tiles = heads 2y, 2y+1 over the same rows; 0: tiles = row tiles 2x, 2x+1 of head y
};

template <int HD>
__global__ void __launch_bounds__(PF2<HD>::THREADS, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, Prefill2Args pa) {
    using C = PF2<HD>;
    const PrefillArgs& a = pa.p;
    extern __shared__ unsigned char pf_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;                         // [2][Q_BYTES]
    unsigned char* k_s = base + 2 * C::Q_BYTES;        // [2][KV_BYTES]
    unsigned char* v_s = k_s + 2 * C::KV_BYTES;        // [KV_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + C::KV_BYTES);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* k_empty = k_full + 2;     // 2
    uint64_t* v_full = k_empty + 2;     // 1
    uint64_t* v_empty = v_full + 1;     // 1
    uint64_t* s_full = v_empty + 1;     // [tile][buffer] = 4
    uint64_t* p_full = s_full + 4;      // 4
    uint64_t* o_done = p_full + 4;      // [tile] = 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the two tiles of this CTA; heaviest (latest rows) first
    const int x = gridDim.x - 1 - blockIdx.x;
    int th[2], ti0[2], trows[2], tn[2];
    if (pa.pair_heads) {
        th[0] = 2 * blockIdx.y;
        th[1] = th[0] + 1;
        ti0[0] = ti0[1] = x * C::BM;
    } else {
        th[0] = th[1] = blockIdx.y;
        ti0[0] = 2 * x * C::BM;
        ti0[1] = ti0[0] + C::BM;
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        trows[t] = max(0, min(C::BM, a.T - ti0[t]));
        tn[t] = trows[t] > 0 ? (a.start + ti0[t] + trows[t] + C::BN - 1) / C::BN : 0;
    }
    const int n = max(tn[0], tn[1]);
    const int kv_h = th[0] / (a.num_heads / a.num_kv_heads);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&o_done[i], 1);
        }
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const int active = (tn[0] > 0) + (tn[1] > 0);
            mbar_arrive_expect_tx(q_full, active * C::Q_BYTES);
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (tn[t] > 0)
                    for (int c = 0; c < C::NBOX; ++c)
                        tma_load_2d(q_s + t * C::Q_BYTES + c * (C::BM * 128), &tm_q, th[t] * HD + 32 * c, ti0[t], q_full);
            const int y0 = kv_h * a.capacity;
            auto load_k = [&](int j) {
                const int st = j & 1;
                mbar_arrive_expect_tx(&k_full[st], C::KV_BYTES);
                for (int c = 0; c < C::NBOX; ++c)
                    tma_load_2d(k_s + st * C::KV_BYTES + c * (C::BN * 128), &tm_k, 32 * c, y0 + j * C::BN, &k_full[st]);
            };
            if (n > 0) load_k(0);
            for (int j = 0; j < n; ++j) {
                // K one tile ahead of V: the scores of tile j+1 are issued before P.V of tile j
                if (j + 1 < n) {
                    if (j + 1 >= 2 && !mbar_wait(&k_empty[(j + 1) & 1], (((j + 1) >> 1) - 1) & 1, a.status, 31)) break;
                    load_k(j + 1);
                }
                if (j >= 1 && !mbar_wait(v_empty, (j - 1) & 1, a.status, 32)) break;
                mbar_arrive_expect_tx(v_full, C::KV_BYTES);
                for (int c = 0; c < C::NBOX; ++c)
                    tma_load_2d(v_s + c * (C::BN * 128), &tm_v, 32 * c, y0 + j * C::BN, v_full);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_tf32(C::BM, C::BN, 0, 0);
            constexpr uint32_t idesc_pv = idesc_tf32(C::BM, HD, 0, 1);
            const uint32_t q_addr = smem_u32(q_s), k_addr0 = smem_u32(k_s), v_addr = smem_u32(v_s);
            auto scores = [&](int j) {   // S[t][j & 1] = Q_t K(j)^T for the tiles that still see tile j
                const uint32_t k_addr = k_addr0 + (j & 1) * C::KV_BYTES;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j >= tn[t]) continue;
                    const uint32_t d = tmem + C::TMEM_S + (t * 2 + (j & 1)) * C::BN;
#pragma unroll
                    for (int kk = 0; kk < HD / 8; ++kk) {
                        const uint64_t ad = smem_desc_sw128(q_addr + t * C::Q_BYTES + (kk >> 2) * (C::BM * 128) + (kk & 3) * 32, 16, 1024);
                        const uint64_t bd = smem_desc_sw128(k_addr + (kk >> 2) * (C::BN * 128) + (kk & 3) * 32, 16, 1024);
                        mma_ss_tf32(d, ad, bd, idesc_qk, kk > 0);
                    }
                    tc_commit(&s_full[t * 2 + (j & 1)]);
                }
                tc_commit(&k_empty[j & 1]);
            };
            bool ok = n > 0 && mbar_wait(q_full, 0, a.status, 33);
            if (ok && (ok = mbar_wait(&k_full[0], 0, a.status, 34))) {
                tc_fence_after();
                scores(0);
            }
            for (int j = 0; ok && j < n; ++j) {
                if (j + 1 < n) {
                    if (!(ok = mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, a.status, 35))) break;
                    tc_fence_after();
                    scores(j + 1);
                }
                if (!(ok = mbar_wait(v_full, j & 1, a.status, 36))) break;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j >= tn[t]) continue;
                    const int b = j & 1;
                    if (!(ok = mbar_wait(&p_full[t * 2 + b], (j >> 1) & 1, a.status, 37))) break;
                    tc_fence_after();
                    const uint32_t d = tmem + C::TMEM_O + t * HD;
                    const uint32_t p = tmem + C::TMEM_S + (t * 2 + b) * C::BN;
#pragma unroll
                    for (int kk = 0; kk < C::BN / 8; ++kk) {
                        const uint64_t bd = smem_desc(v_addr + kk * 1024, C::BN * 128, 512, LAYOUT_SW128_BASE32B);
                        mma_ts_tf32(d, p + kk * 8, bd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(&o_done[t]);
                }
                if (!ok) break;
                tc_commit(v_empty);
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax: one warpgroup per tile, one query row per thread ----------------
        const int t = (warp - 4) >> 2;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                 // row inside the tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int row_pos = a.start + ti0[t] + r;       // last visible cache position of this row
        const float sl2 = a.scale * PF_LOG2E * PF_TRUNC_GAIN;
        const uint32_t oa = tmem + lane_addr + C::TMEM_O + t * HD;
        const int nt = tn[t];
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < nt; ++j) {
            const int b = j & 1;
            if (!(ok = mbar_wait(&s_full[t * 2 + b], (j >> 1) & 1, a.status, 38))) break;
            tc_fence_after();
            uint32_t s0[32], s1[32];
            const uint32_t sa = tmem + lane_addr + C::TMEM_S + (t * 2 + b) * C::BN;
            tmem_ld32(sa, s0);
            tmem_ld32(sa + 32, s1);
            tmem_wait_ld();
            const int c0 = j * C::BN;
            if (c0 + C::BN - 1 > row_pos) {             // tile crosses this row's causal boundary
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if (c0 + c > row_pos) s0[c] = 0xff800000u;        // -inf
                    if (c0 + 32 + c > row_pos) s1[c] = 0xff800000u;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
            const float m_cand = fmaxf(m, mx * sl2);    // the positive factor commutes with max
            // P.V of tile j-1 is awaited once per tile, so this barrier never runs more
            // than one phase ahead of its waiters (a parity wait cannot tell two apart):
            // here if the accumulator must be rescaled, otherwise after the exponentials,
            // by which time it has long completed.
            bool o_seen = j == 0;
            if (__any_sync(0xffffffffu, m_cand - m > C::RESCALE_STEP)) {   // always on the first tile (m = -inf)
                const float alpha = ex2_approx(m - m_cand);
                m = m_cand;
                l *= alpha;
                if (j > 0) {
                    // O_t is stable once P.V of tile j-1 has completed, and P.V of tile j
                    // cannot start before this warpgroup hands over P
                    if (!(ok = mbar_wait(&o_done[t], (j - 1) & 1, a.status, 39))) break;
                    o_seen = true;
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < HD / 32; ++ch) {
                        uint32_t v[32];
                        tmem_ld32(oa + ch * 32, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                        tmem_st32(oa + ch * 32, v);
                    }
                }
            }
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(s0[c]), sl2, -m));
                const float p1 = ex2_approx(fmaf(__uint_as_float(s1[c]), sl2, -m));
                s0[c] = __float_as_uint(p0);
                s1[c] = __float_as_uint(p1);
                sum0 += p0;
                sum1 += p1;
            }
            l += sum0 + sum1;
            tmem_st32(sa, s0);
            tmem_st32(sa + 32, s1);
            tmem_wait_st();
            if (!o_seen && !(ok = mbar_wait(&o_done[t], (j - 1) & 1, a.status, 41))) break;
            tc_fence_before();
            mbar_arrive(&p_full[t * 2 + b]);
        }
        if (ok && nt > 0 && (ok = mbar_wait(&o_done[t], (nt - 1) & 1, a.status, 40))) {
            tc_fence_after();
            const float inv = PF_TRUNC_GAIN * PF_TRUNC_GAIN / l;   // V and P are both truncated by the tensor core
            float* dst = a.out + ((size_t)(ti0[t] + r) * a.num_heads + th[t]) * HD;
#pragma unroll
            for (int ch = 0; ch < HD / 32; ++ch) {
                uint32_t v[32];
                tmem_ld32(oa + ch * 32, v);
                tmem_wait_ld();
                if (r < trows[t]) {
#pragma unroll
                    for (int d = 0; d < 32; d += 4)
                        *reinterpret_cast<float4*>(dst + ch * 32 + d) =
                            make_float4(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv,
                                        __uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// One query tile per CTA, two CTAs per cluster working as one tensor core
// (cta_group::2): the pair's tiles are two query heads of one kv head over the
// same 128 rows, the MMA tile is 256 rows, and each CTA holds half of every K
// tile (64 of 128 positions) and half of every V tile (HD/2 of the columns).
// With one tile per CTA tensor memory has room for score blocks of 128
// positions (two buffers) beside the output accumulator, so the Q tile - the A
// operand, re-read from shared memory for every K tile - is read half as often
// per flop as with 64-position blocks, and the B operands are read half as
// often again because the pair shares them.  Eight softmax warps: the two warps
// of a tensor-memory lane quadrant take 64 columns each of their 32 rows and
// agree on the row maximum through shared memory.
// ---------------------------------------------------------------------------
template <int HD>
struct PFP {
    static constexpr int BM = 128;               // query rows per CTA
    static constexpr int BN = 128;               // cache positions per step
    static constexpr int NBOX = HD / 32;
    static constexpr int Q_BYTES = BM * HD * 4;
    static constexpr int K_ROWS = BN / 2;        // this CTA's positions of a K tile
    static constexpr int K_BYTES = K_ROWS * HD * 4;
    static constexpr int V_BOXES = NBOX / 2;     // this CTA's 32-column blocks of a V tile
    static constexpr int V_BYTES = BN * (HD / 2) * 4;
    // Three score buffers: the scores of step j+2 are issued before P.V of step j, so a step's softmax has the time of
    // three groups of MMAs (scores j+2, P.V j, scores j+3) before its probabilities are needed.  K therefore runs two
    // tiles ahead of V.
    static constexpr int SB = 3;
    static constexpr int KS = 3, VS = 2;
    static constexpr int XCHG_BYTES = 2 * 2 * BM * 4;   // [parity][half][row] row maxima; reused for the row sums
    static constexpr int BAR_BYTES = 256;
    static constexpr size_t SMEM_BYTES = Q_BYTES + KS * K_BYTES + VS * V_BYTES + XCHG_BYTES + BAR_BYTES;   // 1024-aligned base
    static constexpr int TMEM_S = 0;             // [buffer] score/probability blocks of BN columns
    static constexpr int TMEM_O = SB * BN;       // output accumulator, HD columns
    static constexpr int TMEM_COLS = 512;
    static constexpr int THREADS = 384;
    static constexpr float RESCALE_STEP = 8.0f;
};

template <int HD>
__global__ void __launch_bounds__(PFP<HD>::THREADS, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, PrefillArgs a) {
    using C = PFP<HD>;
    constexpr int KS = C::KS, VS = C::VS, SB = C::SB;
    extern __shared__ __align__(1024) unsigned char pfp_smem_raw[];
    unsigned char* q_s = pfp_smem_raw;
    unsigned char* k_s = q_s + C::Q_BYTES;           // [KS][K_BYTES]
    unsigned char* v_s = k_s + KS * C::K_BYTES;      // [VS][V_BYTES]
    float* xchg = reinterpret_cast<float*>(v_s + VS * C::V_BYTES);   // [2][2][BM]
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(xchg) + C::XCHG_BYTES);
    uint64_t* q_full = bars;             // 1
    uint64_t* k_full = bars + 1;         // KS
    uint64_t* k_empty = k_full + KS;     // KS
    uint64_t* v_full = k_empty + KS;     // VS
    uint64_t* v_empty = v_full + VS;     // VS
    uint64_t* s_full = v_empty + VS;     // SB
    uint64_t* p_full = s_full + SB;      // SB
    uint64_t* o_done = p_full + SB;      // 1
    uint64_t* x_bar = o_done + 1;        // 4: the two warps of a lane quadrant meet here
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(x_bar + 4);
    static_assert((1 + 2 * KS + 2 * VS + 2 * SB + 1 + 4) * 8 + 4 <= C::BAR_BYTES, "barrier area");
    static_assert(C::TMEM_O + HD <= C::TMEM_COLS, "tensor memory columns");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    // heaviest (latest rows) first
    const int x = (int)(gridDim.x >> 1) - 1 - (int)(blockIdx.x >> 1);
    const int head = 2 * (int)blockIdx.y + (int)rank;
    const int ti0 = x * C::BM;
    const int trows = max(0, min(C::BM, a.T - ti0));
    const int n = trows > 0 ? (a.start + ti0 + trows + C::BN - 1) / C::BN : 0;   // the same in both CTAs of the pair
    const int kv_h = head / (a.num_heads / a.num_kv_heads);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KS; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < VS; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < SB; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 16);    // the leader's counts the softmax warps of both CTAs
        }
        mbar_init(o_done, 1);
        for (int i = 0; i < 4; ++i) mbar_init(&x_bar[i], 64);
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer: this CTA's halves, reported to the leader's barriers ----------------
        if (lane == 0 && n > 0) {
            auto at_leader = [&](uint64_t* bar) { return map_to_cta(smem_u32(bar), 0u); };
            if (leader) mbar_arrive_expect_tx(q_full, 2 * C::Q_BYTES);
            for (int c = 0; c < C::NBOX; ++c)
                tma_load_2d_pair(q_s + c * (C::BM * 128), &tm_q, head * HD + 32 * c, ti0, at_leader(q_full));
            const int y0 = kv_h * a.capacity;
            int jk = 0;
            bool okp = true;
            for (int j = 0; okp && j < n; ++j) {
                while (jk < n && jk <= j + KS - 1) {
                    const int st = jk % KS;
                    if (jk >= KS && !mbar_wait(&k_empty[st], ((jk / KS) - 1) & 1, a.status, 51)) {
                        okp = false;
                        break;
                    }
                    if (leader) mbar_arrive_expect_tx(&k_full[st], 2 * C::K_BYTES);
                    for (int c = 0; c < C::NBOX; ++c)
                        tma_load_2d_pair(k_s + st * C::K_BYTES + c * (C::K_ROWS * 128), &tm_k, 32 * c,
                                         y0 + jk * C::BN + (int)rank * C::K_ROWS, at_leader(&k_full[st]));
                    ++jk;
                }
                if (!okp) break;
                const int sv = j % VS;
                if (j >= VS && !mbar_wait(&v_empty[sv], ((j / VS) - 1) & 1, a.status, 52)) break;
                if (leader) mbar_arrive_expect_tx(&v_full[sv], 2 * C::V_BYTES);
                for (int c = 0; c < C::V_BOXES; ++c)
                    tma_load_2d_pair(v_s + sv * C::V_BYTES + c * (C::BN * 128), &tm_v, 32 * ((int)rank * C::V_BOXES + c),
                                     y0 + j * C::BN, at_leader(&v_full[sv]));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread of the leader, for both CTAs ----------------
        if (lane == 0 && leader && n > 0) {
            constexpr uint32_t idesc_qk = idesc_tf32(2 * C::BM, C::BN, 0, 0);
            constexpr uint32_t idesc_pv = idesc_tf32(2 * C::BM, HD, 0, 1);
            const uint32_t q_addr = smem_u32(q_s), k_addr0 = smem_u32(k_s), v_addr0 = smem_u32(v_s);
            auto commit = [&](uint64_t* bar) {   // this CTA's barrier and the peer's copy of it
                tc_commit_pair(smem_u32(bar));
                tc_commit_pair(map_to_cta(smem_u32(bar), 1u));
            };
            // A descriptor differs from the one of the tile's first bytes only in its address field (bits 0-13, in
            // units of 16 bytes; every address here is below 256 KB): built once, then one 64-bit add per MMA by this
            // single issuing thread.
            const uint64_t q_desc0 = smem_desc_sw128(q_addr, 16, 1024);
            auto scores = [&](int j) {
                const uint64_t k_desc0 = smem_desc_sw128(k_addr0 + (j % KS) * C::K_BYTES, 16, 1024);
                const uint32_t d = tmem + C::TMEM_S + (j % SB) * C::BN;
#pragma unroll
                for (int kk = 0; kk < HD / 8; ++kk) {
                    const uint64_t ad = q_desc0 + (uint64_t)(((kk >> 2) * (C::BM * 128) + (kk & 3) * 32) >> 4);
                    const uint64_t bd = k_desc0 + (uint64_t)(((kk >> 2) * (C::K_ROWS * 128) + (kk & 3) * 32) >> 4);
                    mma_ss_tf32_pair(d, ad, bd, idesc_qk, kk > 0);
                }
                commit(&s_full[j % SB]);
                commit(&k_empty[j % KS]);
            };
            // scores run SB - 1 steps ahead of P.V
            bool ok = mbar_wait(q_full, 0, a.status, 53);
            for (int j = 0; ok && j < SB - 1 && j < n; ++j) {
                if (!(ok = mbar_wait(&k_full[j % KS], 0, a.status, 54))) break;
                tc_fence_after();
                scores(j);
            }
            for (int j = 0; ok && j < n; ++j) {
                const int ja = j + SB - 1;
                if (ja < n) {
                    if (!(ok = mbar_wait(&k_full[ja % KS], (ja / KS) & 1, a.status, 55))) break;
                    tc_fence_after();
                    scores(ja);
                }
                const int sv = j % VS;
                if (!(ok = mbar_wait(&v_full[sv], (j / VS) & 1, a.status, 56))) break;
                if (!(ok = mbar_wait_cluster(&p_full[j % SB], (j / SB) & 1, a.status, 57))) break;
                tc_fence_after();
                const uint32_t d = tmem + C::TMEM_O;
                const uint32_t p = tmem + C::TMEM_S + (j % SB) * C::BN;
                const uint64_t v_desc0 = smem_desc(v_addr0 + sv * C::V_BYTES, C::BN * 128, 512, LAYOUT_SW128_BASE32B);
#pragma unroll
                for (int kk = 0; kk < C::BN / 8; ++kk)
                    mma_ts_tf32_pair(d, p + kk * 8, v_desc0 + (uint64_t)(kk * 1024 >> 4), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                commit(o_done);
                commit(&v_empty[sv]);
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax: thread = (query row, half of the block's columns) ----------------
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const int r = quad * 32 + lane;                 // row inside the tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int row_pos = a.start + ti0 + r;          // last visible cache position of this row
        const float sl2 = a.scale * PF_LOG2E * PF_TRUNC_GAIN;
        const uint32_t oa = tmem + lane_addr + C::TMEM_O + half * (HD / 2);   // this thread's half of the output columns
        const uint32_t p_leader = map_to_cta(smem_u32(&p_full[0]), 0u);   // the leader's p_full[0]; the others follow at 8 bytes
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n; ++j) {
            const int b = j % SB;
            if (!(ok = mbar_wait(&s_full[b], (j / SB) & 1, a.status, 58))) break;
            tc_fence_after();
            uint32_t s0[32], s1[32];
            const uint32_t sa = tmem + lane_addr + C::TMEM_S + b * C::BN + half * 64;
            tmem_ld32(sa, s0);
            tmem_ld32(sa + 32, s1);
            tmem_wait_ld();
            const int c0 = j * C::BN + half * 64;
            if (c0 + 63 > row_pos) {                    // these columns cross this row's causal boundary
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if (c0 + c > row_pos) s0[c] = 0xff800000u;        // -inf
                    if (c0 + 32 + c > row_pos) s1[c] = 0xff800000u;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[c]), __uint_as_float(s1[c])));
            // the row's maximum over both halves
            float* xm = xchg + (size_t)(j & 1) * 2 * C::BM;
            xm[half * C::BM + r] = mx;
            mbar_arrive(&x_bar[quad]);
            if (!(ok = mbar_wait(&x_bar[quad], j & 1, a.status, 59))) break;
            mx = fmaxf(mx, xm[(half ^ 1) * C::BM + r]);
            const float m_cand = fmaxf(m, mx * sl2);    // the positive factor commutes with max; identical in both halves
            bool o_seen = j == 0;
            if (__any_sync(0xffffffffu, m_cand - m > C::RESCALE_STEP)) {   // always on the first step (m = -inf)
                const float alpha = ex2_approx(m - m_cand);
                m = m_cand;
                l *= alpha;
                if (j > 0) {
                    if (!(ok = mbar_wait(o_done, (j - 1) & 1, a.status, 60))) break;
                    o_seen = true;
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < HD / 64; ++ch) {
                        uint32_t v[32];
                        tmem_ld32(oa + ch * 32, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                        tmem_st32(oa + ch * 32, v);
                    }
                }
            }
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(s0[c]), sl2, -m));
                const float p1 = ex2_approx(fmaf(__uint_as_float(s1[c]), sl2, -m));
                s0[c] = __float_as_uint(p0);
                s1[c] = __float_as_uint(p1);
                sum0 += p0;
                sum1 += p1;
            }
            l += sum0 + sum1;
            tmem_st32(sa, s0);
            tmem_st32(sa + 32, s1);
            tmem_wait_st();
            if (!o_seen && !(ok = mbar_wait(o_done, (j - 1) & 1, a.status, 61))) break;
            // one arrival per warp: every lane's stores to tensor memory have completed and are fenced
            // before the warp meets, and lane 0 arrives after that
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(p_leader + 8u * (uint32_t)b);
        }
        if (ok && n > 0 && (ok = mbar_wait(o_done, (n - 1) & 1, a.status, 62))) {
            tc_fence_after();
            // the row's sum over both halves (same exchange, one more phase of the quadrant's barrier)
            float* xl = xchg + (size_t)(n & 1) * 2 * C::BM;
            xl[half * C::BM + r] = l;
            mbar_arrive(&x_bar[quad]);
            if (mbar_wait(&x_bar[quad], n & 1, a.status, 63)) {
                const float lt = l + xl[(half ^ 1) * C::BM + r];
                const float inv = PF_TRUNC_GAIN * PF_TRUNC_GAIN / lt;   // V and P are both truncated by the tensor core
                float* dst = a.out + ((size_t)(ti0 + r) * a.num_heads + head) * HD + half * (HD / 2);
#pragma unroll
                for (int ch = 0; ch < HD / 64; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(oa + ch * 32, v);
                    tmem_wait_ld();
                    if (r < trows) {
#pragma unroll
                        for (int d = 0; d < 32; d += 4)
                            *reinterpret_cast<float4*>(dst + ch * 32 + d) =
                                make_float4(__uint_as_float(v[d]) * inv, __uint_as_float(v[d + 1]) * inv,
                                            __uint_as_float(v[d + 2]) * inv, __uint_as_float(v[d + 3]) * inv);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA leaves while its shared and tensor memory may still be operands of the pair's MMAs
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// fp32 matrix [rows, cols] with row pitch `pitch_floats`; box = box_rows x 32 floats (128 bytes).
bool make_map(CUtensorMap* m, const float* base, uint64_t cols, uint64_t rows, uint64_t pitch_floats, uint32_t box_rows,
              CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_floats * sizeof(float)};
    cuuint32_t box[2] = {32, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
cudaError_t launch_pf(const AttnArgs& a, cudaStream_t s) {
    using C = PF2<HD>;
    static unsigned long long configured = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64 || !(configured >> dev & 1ull)) {
        e = cudaFuncSetAttribute(attn_prefill_tc2_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev < 64) configured |= 1ull << dev;
    }
    const SeqDesc& sd = a.seqs.one;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads;
    CUtensorMap tq, tk, tv;
    if (!make_map(&tq, a.q_rot, (uint64_t)H * HD, (uint64_t)a.T, (uint64_t)H * HD, C::BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map(&tk, sd.k, HD, (uint64_t)KV * sd.capacity, HD, C::BN, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map(&tv, sd.v, HD, (uint64_t)KV * sd.capacity, HD, C::BN, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
        return cudaErrorInvalidValue;
    Prefill2Args pa{};
    PrefillArgs& p = pa.p;
    p.out = a.out;
    p.T = a.T;
    p.start = sd.start;
    p.num_heads = H;
    p.num_kv_heads = KV;
    p.capacity = sd.capacity;
    p.scale = a.scale;
    p.status = a.status;
    const int row_tiles = (a.T + C::BM - 1) / C::BM;
    // two query heads of one kv head share a CTA when the group size is even,
    // otherwise two consecutive row tiles of one head
    pa.pair_heads = (H / KV) % 2 == 0 ? 1 : 0;
    dim3 grid = pa.pair_heads ? dim3(row_tiles, H / 2) : dim3((row_tiles + 1) / 2, H);
    attn_prefill_tc2_kernel<HD><<<grid, C::THREADS, C::SMEM_BYTES, s>>>(tq, tk, tv, pa);
    return cudaGetLastError();
}

template <int HD>
cudaError_t launch_pf_pair128(const AttnArgs& a, cudaStream_t s) {
    using C = PFP<HD>;
    static unsigned long long configured = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64 || !(configured >> dev & 1ull)) {
        e = cudaFuncSetAttribute(attn_prefill_pair_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev < 64) configured |= 1ull << dev;
    }
    const SeqDesc& sd = a.seqs.one;
    const int H = a.hs.num_heads, KV = a.hs.num_kv_heads;
    CUtensorMap tq, tk, tv;
    if (!make_map(&tq, a.q_rot, (uint64_t)H * HD, (uint64_t)a.T, (uint64_t)H * HD, C::BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map(&tk, sd.k, HD, (uint64_t)KV * sd.capacity, HD, C::K_ROWS, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map(&tv, sd.v, HD, (uint64_t)KV * sd.capacity, HD, C::BN, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
        return cudaErrorInvalidValue;
    PrefillArgs p{};
    p.out = a.out;
    p.T = a.T;
    p.start = sd.start;
    p.num_heads = H;
    p.num_kv_heads = KV;
    p.capacity = sd.capacity;
    p.scale = a.scale;
    p.status = a.status;
    const int row_tiles = (a.T + C::BM - 1) / C::BM;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * row_tiles, H / 2);   // clusters of two CTAs along x: two query heads of one kv head
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_prefill_pair_kernel<HD>, tq, tk, tv, p);
}

template <int HD>
cudaError_t launch_pf_any(const AttnArgs& a, cudaStream_t s) {
    // even group size and head_dim 128: two query heads of one kv head per pair of CTAs; otherwise the one-CTA kernel
    // (at head_dim 64 a step's exponentials take as long as its MMAs in either kernel and the pair's hand-over is pure
    // cost: 0.266 against 0.254 ms for 4096 tokens of the LLaMA-3.2-1B shape, 0.872 against 0.809 ms for 8192)
    if (HD == 128 && (a.hs.num_heads / a.hs.num_kv_heads) % 2 == 0 && !a.prefill_one_cta) return launch_pf_pair128<HD>(a, s);
    return launch_pf<HD>(a, s);
}

}  // namespace

bool prefill_tc_supported(const HeadShape& hs) { return hs.head_dim == 64 || hs.head_dim == 128; }

cudaError_t launch_attn_prefill_tc(const AttnArgs& a, cudaStream_t s) {
    if (a.batch != 1 || a.seqs.many != nullptr) return cudaErrorInvalidValue;
    if (a.T == 0) return cudaSuccess;
    if (a.hs.head_dim == 64) return launch_pf_any<64>(a, s);
    if (a.hs.head_dim == 128) return launch_pf_any<128>(a, s);
    return cudaErrorInvalidValue;
}

}  // namespace shainet
