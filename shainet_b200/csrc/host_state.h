// Host-side state of libshainet_attn shared by its translation units: the context and
// cache objects behind the opaque handles of include/shainet_attn.h, and the helpers that
// report errors, grow scratch buffers and run one attention call on device pointers.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>

#include <string>
#include <utility>
#include <vector>

#include "../../include/shainet_attn.h"
#include "kernels.h"

namespace shainet {

constexpr int SEQ_RING = 8;           // in-flight descriptor uploads of batched decode

struct DevBuf {
    float* p = nullptr;
    size_t cap = 0;  // floats
};

}  // namespace shainet

struct shainet_attn_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    shainet::DevBuf q_rot, part, part_words, dev_in, dev_out;
    shainet::DevBuf kv_f32;             // fp32 image of a bfloat16 cache's rows, for the kernels that read fp32 caches only
    shainet::DevBuf act[6];             // activations of the block / decoder entries (see decoder.cu)   // part_words: {value, epoch} partials of single-sequence decode
    float* pin_in = nullptr;
    size_t pin_in_cap = 0;
    float* pin_out = nullptr;
    size_t pin_out_cap = 0;
    shainet::AttnStatus* status_host = nullptr;  // mapped pinned; kernels write through status_dev
    shainet::AttnStatus* status_dev = nullptr;
    shainet::SeqDesc* seq_host = nullptr;        // [shainet::SEQ_RING][seq_cap] pinned
    shainet::SeqDesc* seq_dev = nullptr;         // [shainet::SEQ_RING][seq_cap]
    int seq_cap = 0;
    int seq_slot = 0;
    cudaEvent_t seq_ev[shainet::SEQ_RING] = {};
    int live_caches = 0;
    unsigned* tickets = nullptr;        // split-merge tickets of the fused decode kernel, zero between launches
    size_t tickets_cap = 0;
    unsigned epoch = 0;                 // tag of the newest word-merged decode launch
    bool last_fused = false;            // the newest launch on this context was a fused decode kernel
    bool after_chain_kernel = false;    // the newest launch was a kernel of the decoder chain (programmatic launch): a fused
                                        // decode kernel behind it may become resident while the chain's previous attention
                                        // kernel still appends its row
    bool rows_rewound = false;          // a cache was truncated or reset since: the next launch may rewrite rows the
                                        // previous one still reads, so it must not run ahead of it (F_INPUTS_READY is ignored once)
    unsigned long long peer_wait_ns = shainet::WAIT_LIMIT_NS;   // limit of the waits for other ranks' exchange words
    float* lse_out = nullptr;           // caller-owned device buffer for log-sum-exp values (nullable)
    // exchange buffer shared with the other ranks of the box (IPC): comm_data_floats
    // floats, then as many 8-byte {value, epoch} words
    unsigned char* comm_base = nullptr;
    size_t comm_data_floats = 0;
    int comm_world = 0, comm_rank = 0;
    unsigned char* comm_peer[shainet::MAX_PEERS] = {};
    bool gather_armed = false;          // the next fused decode call delivers to the peers
    long long gather_out_off = 0, gather_lse_off = -1;
    unsigned gather_epoch = 0;
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed;   // recorded, not yet read
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev_pool;  // reusable pairs
};

struct shainet_attn_kv {
    shainet_attn_ctx* ctx = nullptr;
    shainet::HeadShape hs{};
    float* k = nullptr;         // [num_kv_heads, cap, head_dim] elements of `es` bytes (bfloat16 behind a float pointer when es == 2)
    float* v = nullptr;
    int es = 4;                 // bytes per cache element: 4 = fp32, 2 = bfloat16
    // Reserved-address cache (kv_create_reserved): k and v are virtual address ranges of cap rows per kv head, reserved
    // once; physical pages are mapped behind the rows in use.  cap then never changes and rows never move.
    bool reserved = false;
    size_t page_bytes = 0;      // mapping granularity
    size_t pages_per_head = 0;  // pages mapped (and zeroed) behind every kv head of k and of v
    struct Mapping {
        unsigned long long at, bytes, handle;       // device address, size, CUmemGenericAllocationHandle
    };
    std::vector<Mapping> mappings;
    int cap = 0;
    int len = 0;
    float* inv_freq = nullptr;  // device, head_dim/2
    float* q_norm = nullptr;    // device, nullable
    float* k_norm = nullptr;
    float* b_q = nullptr;
    float* b_k = nullptr;
    float* b_v = nullptr;
    double eps = 1e-6;
};

namespace shainet {

// Sets the calling thread's last-error message and returns `code`.
int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);

#define CU(call)                                                        \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return shainet::fail_cuda(e__, #call);  \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// Grows a scratch buffer (doubling); synchronises `s` before freeing the old one.
int grow(DevBuf& b, size_t floats, cudaStream_t s);
// dst = device copy of host[n] (allocated on first use); host == null frees it.
int upload_vec(float*& dst, const float* host, size_t n);
bool aligned16(const void* p);
// Norm/RoPE/append + attention of T new tokens of one sequence, device pointers, stream s.
int forward_device(shainet_attn_ctx* ctx, shainet_attn_kv* kv, const float* q, const float* k_new, const float* v_new,
                   float* out, int T, float scale, unsigned flags, cudaStream_t s);

}  // namespace shainet
