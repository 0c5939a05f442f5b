// libbnkgpu_bench.so: the measurement helpers declared in include/bnk_gpu_bench.h.  They work on the
// handles of libbnkgpu.so (same struct layouts, same build) and use nothing of it but those layouts.
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

} // extern "C"
