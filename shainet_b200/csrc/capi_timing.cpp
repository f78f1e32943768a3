// Decode timing through the C ABI alone (no Python, no torch): dlopen the library,
// fill `layers` caches on the device, then time shainet_attn_forward_dev for one
// token per layer over 40 steps with CUDA events on the launching stream.
//
//   capi_timing <lib.so> [num_heads kv_heads head_dim context layers qk_norm flags]
//
// Prints device microseconds per launch, the GB/s of K/V streamed, and the host
// cost of one call.  Built by `python -m shainet_b200.build --harness`.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <vector>
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1);} } while (0)
typedef int (*ctx_create_t)(void**, int);
typedef int (*kv_create_t)(void*, void**, int, int, int, int);
typedef int (*kv_fill_t)(void*, int, unsigned long long);
typedef int (*kv_trunc_t)(void*, int);
typedef int (*kv_norm_t)(void*, const float*, const float*, double);
typedef int (*kv_theta_t)(void*, double);
typedef int (*fwd_t)(void*, void*, const float*, const float*, const float*, float*, int, float, unsigned, void*);
typedef const char* (*err_t)();
int main(int argc, char** argv) {
    const char* path = argc > 1 ? argv[1] : "shainet_b200/lib/libshainet_attn.so";
    int H = argc > 2 ? atoi(argv[2]) : 32, KV = argc > 3 ? atoi(argv[3]) : 4, HD = argc > 4 ? atoi(argv[4]) : 128;
    int L = argc > 5 ? atoi(argv[5]) : 32768, NL = argc > 6 ? atoi(argv[6]) : 12, norm = argc > 7 ? atoi(argv[7]) : 1; unsigned flags = argc > 8 ? atoi(argv[8]) : 0;
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { printf("dlopen failed: %s\n", dlerror()); return 1; }
    auto ctx_create = (ctx_create_t)dlsym(h, "shainet_attn_ctx_create");
    auto kv_create = (kv_create_t)dlsym(h, "shainet_attn_kv_create");
    auto kv_fill = (kv_fill_t)dlsym(h, "shainet_attn_kv_fill_normal");
    auto kv_trunc = (kv_trunc_t)dlsym(h, "shainet_attn_kv_truncate");
    auto kv_norm = (kv_norm_t)dlsym(h, "shainet_attn_kv_set_qk_norm");
    auto kv_theta = (kv_theta_t)dlsym(h, "shainet_attn_kv_set_rope_theta");
    auto fwd = (fwd_t)dlsym(h, "shainet_attn_forward_dev");
    auto lasterr = (err_t)dlsym(h, "shainet_attn_last_error");
    void* ctx; if (ctx_create(&ctx, 0)) { printf("ctx: %s\n", lasterr()); return 1; }
    std::vector<void*> kvs(NL);
    std::vector<float> w(HD, 1.0f);
    const int STEPS = 40;
    for (int l = 0; l < NL; ++l) {
        if (kv_create(ctx, &kvs[l], H, KV, HD, L + STEPS + 8)) { printf("kv: %s\n", lasterr()); return 1; }
        kv_theta(kvs[l], 1e6);
        if (norm) kv_norm(kvs[l], w.data(), w.data(), 1e-6);
        kv_fill(kvs[l], L, 100 + l);
    }
    float *q, *k, *v, *out;
    CK(cudaMalloc(&q, H * HD * 4)); CK(cudaMalloc(&k, KV * HD * 4)); CK(cudaMalloc(&v, KV * HD * 4)); CK(cudaMalloc(&out, (size_t)NL * H * HD * 4));
    CK(cudaMemset(q, 0x3c, H * HD * 4)); CK(cudaMemset(k, 0x3c, KV * HD * 4)); CK(cudaMemset(v, 0x3c, KV * HD * 4));
    cudaStream_t s; CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    double host_us = 0;
    for (int round = 0; round < 2; ++round) {
        for (int l = 0; l < NL; ++l) kv_trunc(kvs[l], L);
        CK(cudaDeviceSynchronize());
        CK(cudaEventRecord(e0, s));
        auto t0 = std::chrono::steady_clock::now();
        for (int st = 0; st < STEPS; ++st)
            for (int l = 0; l < NL; ++l)
                if (fwd(ctx, kvs[l], q, k, v, out + (size_t)l * H * HD, 1, 0.0883883f, flags, s)) { printf("fwd: %s\n", lasterr()); return 1; }
        auto t1 = std::chrono::steady_clock::now();
        CK(cudaEventRecord(e1, s));
        CK(cudaDeviceSynchronize());
        host_us = std::chrono::duration<double, std::micro>(t1 - t0).count() / (STEPS * NL);
    }
    float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
    double us = ms * 1e3 / (STEPS * NL);
    double bytes = 2.0 * KV * (L + STEPS / 2.0) * HD * 4;
    printf("%-36s flags=%u H=%d KV=%d hd=%d L=%d layers=%d : device %7.2f us/launch  %7.1f GB/s   host %5.2f us/call\n", path, flags, H, KV, HD, L, NL, us, bytes / us * 1e-3, host_us);
    {
        std::vector<float> ho((size_t)H * HD);
        CK(cudaMemcpy(ho.data(), out, ho.size() * 4, cudaMemcpyDeviceToHost));
        double cs = 0, ca = 0;
        for (size_t i = 0; i < ho.size(); ++i) { cs += ho[i] * (double)(i % 7 + 1); ca += ho[i] < 0 ? -ho[i] : ho[i]; }
        printf("    checksum %.12g  abs %.12g\n", cs, ca);
    }
    // Builds with -DSK_TIMELINE export per-CTA device timestamps of the fused kernel.
    typedef int (*tl_t)(unsigned long long*);
    auto tl = (tl_t)dlsym(h, "shainet_debug_timeline");
    if (tl) {
        const int NCTA = 320, NMARK = 16;
        std::vector<unsigned long long> buf((size_t)64 * NCTA * NMARK);
        if (tl(buf.data()) != 0) { printf("timeline read failed\n"); return 1; }
        // marks: 0 CTA resident, 2 consumers start, 3 first consumer warp done, 8 .. its state folded, 9 all warps done,
        // 10 states parked, 4 partial written, 7 merging CTAs start polling, 6 merged
        const char* names[] = {"CTA resident: mean", "CTA resident: last", "consumers start: mean", "consumers start: last",
                               "consumers done: first", "consumers done: mean", "consumers done: last",
                               "partial written: mean", "partial written: last", "merge starts: first", "merge starts: last",
                               "merged: first", "merged: last", "period", "warp 0 done -> all warps done: mean",
                               "all warps done -> parked: mean", "parked -> partial written: mean",
                               "warp 0 done -> all warps done: max"};
        double acc[18] = {0};
        int used = 0;
        unsigned long long prev_t0 = 0;
        for (int L = 8; L < 56; ++L) {
            const unsigned long long* t = buf.data() + (size_t)L * NCTA * NMARK;
            int n = 0;
            while (n < NCTA && t[n * NMARK] != 0) ++n;
            if (n == 0) { prev_t0 = 0; continue; }
            unsigned long long t0 = ~0ull;
            for (int c = 0; c < n; ++c) t0 = std::min(t0, t[c * NMARK]);
            double v[18] = {0, 0, 0, 0, 1e30, 0, 0, 0, 0, 1e30, 0, 1e30, 0, 0, 0, 0, 0, 0};
            for (int c = 0; c < n; ++c) {
                auto rel = [&](int k) { return (double)(long long)(t[c * NMARK + k] - t0) * 1e-3; };
                v[0] += rel(0) / n; v[1] = std::max(v[1], rel(0));
                v[2] += rel(2) / n; v[3] = std::max(v[3], rel(2));
                v[4] = std::min(v[4], rel(3)); v[5] += rel(3) / n; v[6] = std::max(v[6], rel(3));
                v[7] += rel(4) / n; v[8] = std::max(v[8], rel(4));
                if (t[c * NMARK + 7]) { v[9] = std::min(v[9], rel(7)); v[10] = std::max(v[10], rel(7)); }
                if (t[c * NMARK + 6]) { v[11] = std::min(v[11], rel(6)); v[12] = std::max(v[12], rel(6)); }
                v[14] += (rel(9) - rel(3)) / n; v[15] += (rel(10) - rel(9)) / n; v[16] += (rel(4) - rel(10)) / n;
                v[17] = std::max(v[17], rel(9) - rel(3));
            }
            if (prev_t0 == 0) { prev_t0 = t0; continue; }
            v[13] = (double)(long long)(t0 - prev_t0) * 1e-3;
            prev_t0 = t0;
            for (int k = 0; k < 18; ++k) acc[k] += v[k];
            ++used;
        }
        printf("device timeline, us after the first CTA of a launch became resident (mean over %d launches)\n", used);
        for (int k = 0; k < 18 && used; ++k) printf("  %-40s %7.2f\n", names[k], acc[k] / used);
    }
    return 0;
}
