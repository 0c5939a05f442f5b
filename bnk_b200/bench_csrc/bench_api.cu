// libbnkgpu_bench.so: the measurement helpers declared in include/bnk_gpu_bench.h.  They work on the
// handles of libbnkgpu.so (same struct layouts, same build) and use nothing of it but those layouts.
#include <atomic>
#include <chrono>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "../csrc/bnk_internal.cuh"
#include "../../include/bnk_gpu_bench.h"

cudaError_t launch_fill_random(uint8_t *dst, uint64_t bytes, uint64_t seed, int sm_count, cudaStream_t s);
cudaError_t probe_int_throughput(bnk_ctx *ctx, int mix, double *tops);
cudaError_t probe_coissue(bnk_ctx *ctx, int kind, int k, double *clk);

namespace {

int fail(bnk_ctx *ctx, int code, const char *what, cudaError_t e = cudaSuccess) {
    if (ctx) {
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->last_error = what;
        if (e != cudaSuccess) {
            ctx->last_error += ": ";
            ctx->last_error += cudaGetErrorString(e);
        }
    }
    return code;
}

#define CK(ctx, call)                                                   \
    do {                                                                \
        cudaError_t _e = (call);                                        \
        if (_e != cudaSuccess) return fail((ctx), BNK_ECUDA, #call, _e); \
    } while (0)

} // namespace

extern "C" {

int bnk_timer_start(bnk_ctx *ctx, bnk_batch *const *batches, uint32_t n) {
    if (!ctx || !batches || n == 0) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaEventRecord(ctx->timer_start, batches[0]->stream));
    for (uint32_t i = 1; i < n; i++) CK(ctx, cudaStreamWaitEvent(batches[i]->stream, ctx->timer_start, 0));
    return BNK_SUCCESS;
}

int bnk_timer_stop(bnk_ctx *ctx, bnk_batch *const *batches, uint32_t n, float *ms) {
    if (!ctx || !batches || n == 0 || !ms) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    for (uint32_t i = 0; i < n; i++) CK(ctx, cudaEventRecord(batches[i]->t_end, batches[i]->stream));
    float longest = 0.f;
    for (uint32_t i = 0; i < n; i++) {
        CK(ctx, cudaEventSynchronize(batches[i]->t_end));
        float t = 0.f;
        CK(ctx, cudaEventElapsedTime(&t, ctx->timer_start, batches[i]->t_end));
        if (t > longest) longest = t;
    }
    *ms = longest;
    return BNK_SUCCESS;
}

int bnk_probe_int_throughput(bnk_ctx *ctx, int mix, double *tera_ops_per_s) {
    if (!ctx || !tera_ops_per_s) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, probe_int_throughput(ctx, mix, tera_ops_per_s));
    return BNK_SUCCESS;
}

int bnk_probe_coissue(bnk_ctx *ctx, int kind, int k, double *cycles_per_double_round) {
    if (!ctx || !cycles_per_double_round) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, probe_coissue(ctx, kind, k, cycles_per_double_round));
    return BNK_SUCCESS;
}

int bnk_batch_fill_random(bnk_batch *b, uint64_t seed) {
    if (!b) return BNK_EINVAL;
    bnk_ctx *ctx = b->ctx;
    if (b->in_flight) return fail(ctx, BNK_EBUSY, "batch has work in flight");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, launch_fill_random(b->dev.ring, b->ring_bytes, seed, ctx->sm_count, b->stream));
    ++ctx->launches;
    CK(ctx, cudaStreamSynchronize(b->stream));
    return BNK_SUCCESS;
}

int bnk_batch_copy_only(bnk_batch *b, uint32_t npkts, int up, int down) {
    if (!b || npkts > b->max_pkts) return BNK_EINVAL;
    bnk_ctx *ctx = b->ctx;
    if (b->in_flight) return fail(ctx, BNK_EBUSY, "batch has work in flight");
    CK(ctx, cudaSetDevice(ctx->device));
    // the span a seal of these packets moves: header room + payload + padding + tag of the furthest packet
    uint64_t ext = 0;
    for (uint32_t i = 0; i < npkts; i++) {
        const uint64_t e = (uint64_t)b->host.off[i] + b->host.len[i] + 48u;
        if (e > ext) ext = e;
    }
    ext = (ext + 15) & ~15ull;
    if (ext > b->ring_bytes) ext = b->ring_bytes;
    const size_t np = b->npad, n = npkts;
    b->in_flight = true;
    if (up && n) {
        CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, b->stream));
        CK(ctx, cudaMemcpyAsync(b->d_desc, b->h_desc, 8 * np + 4 * n, cudaMemcpyHostToDevice, b->stream)); // off, len, slot
    }
    if (down && n) {
        CK(ctx, cudaMemcpyAsync(b->host.ring, b->dev.ring, ext, cudaMemcpyDeviceToHost, b->stream));
        CK(ctx, cudaMemcpyAsync(b->h_desc + 12 * np, b->d_desc + 12 * np, 12 * np + n, cudaMemcpyDeviceToHost,
                                b->stream)); // counter, out_len, status
    }
    return BNK_SUCCESS;
}

int bnk_probe_copy_rounds(bnk_ctx *ctx, uint32_t threads, uint64_t bytes, uint32_t rounds, int directions,
                          double *rounds_per_s) {
    if (!ctx || !rounds_per_s || threads == 0 || threads > 256 || bytes == 0 || rounds == 0 || !(directions & 3))
        return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    struct Lane {
        cudaStream_t s = nullptr;
        uint8_t *h = nullptr, *d = nullptr;
    };
    std::vector<Lane> lanes(threads);
    cudaError_t e = cudaSuccess;
    for (Lane &l : lanes) {
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&l.s, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaHostAlloc((void **)&l.h, bytes, cudaHostAllocDefault);
        if (e == cudaSuccess) e = cudaMalloc((void **)&l.d, bytes);
        if (e == cudaSuccess) memset(l.h, 0x5a, bytes);
    }
    std::atomic<int> failed{0};
    auto body = [&](Lane &l, uint32_t n) {
        cudaSetDevice(ctx->device);
        for (uint32_t r = 0; r < n; r++) {
            cudaError_t x = cudaSuccess;
            if (directions & 1) x = cudaMemcpyAsync(l.d, l.h, bytes, cudaMemcpyHostToDevice, l.s);
            if (x == cudaSuccess && (directions & 2)) x = cudaMemcpyAsync(l.h, l.d, bytes, cudaMemcpyDeviceToHost, l.s);
            if (x == cudaSuccess) x = cudaStreamSynchronize(l.s);
            if (x != cudaSuccess) {
                failed.store((int)x);
                return;
            }
        }
    };
    double secs = 0;
    if (e == cudaSuccess) {
        for (Lane &l : lanes) body(l, 20); // warm
        const auto t0 = std::chrono::steady_clock::now();
        std::vector<std::thread> pool;
        for (Lane &l : lanes) pool.emplace_back(body, std::ref(l), rounds);
        for (auto &t : pool) t.join();
        secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }
    for (Lane &l : lanes) {
        if (l.s) cudaStreamDestroy(l.s);
        if (l.h) cudaFreeHost(l.h);
        if (l.d) cudaFree(l.d);
    }
    if (e != cudaSuccess) return fail(ctx, BNK_ECUDA, "copy probe setup", e);
    if (failed.load()) return fail(ctx, BNK_ECUDA, "copy probe", (cudaError_t)failed.load());
    *rounds_per_s = (double)threads * rounds / secs;
    return BNK_SUCCESS;
}

} // extern "C"
