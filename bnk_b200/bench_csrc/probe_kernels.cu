// Measurement helpers for sm_100a: the 32-bit integer issue-rate probe that gives the
// seal/open kernels their ALU roofline denominator, and a seeded device-side fill for
// synthetic payloads.
#include "../csrc/bnk_internal.cuh"

namespace {

constexpr int kProbeIters = 4096;

// mix 0: add / xor chains, 8 independent chains per thread (ALU pipe only)
// mix 1: ChaCha20 quarter rounds on 16 registers (add, xor, byte-permute, funnel shift)
// mix 2: 32-bit multiply-add chains (FMA pipe only)
// mix 3: add/xor chains interleaved 1:1 with multiply-add chains (both pipes)
// mix 4: funnel-shift rotations by a run-time amount
// mix 5: byte permutes with a run-time selector
// mix 6: 32x32+64 -> 64-bit multiply-adds (the Poly1305 product form)
// mix 7: three-input adds and three-input logic ops
template <int MIX>
__global__ void __launch_bounds__(256) int_probe_kernel(uint32_t *sink, uint32_t seed, uint32_t mul) {
    uint32_t x[16];
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = seed * (i + 1) + threadIdx.x;
    const uint32_t y = seed ^ 0x9e3779b9u, z = seed + 0x7f4a7c15u;
    if (MIX == 0) {
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 4; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    x[i] += y;
                    x[i] ^= z;
                }
            }
        }
    } else if (MIX == 1) {
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t &a = x[i], &b = x[4 + i], &c = x[8 + i], &d = x[12 + i];
                a += b; d = __byte_perm(d ^ a, 0, 0x1032);
                c += d; b = __funnelshift_l(b ^ c, b ^ c, 12);
                a += b; d = __byte_perm(d ^ a, 0, 0x2103);
                c += d; b = __funnelshift_l(b ^ c, b ^ c, 7);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t &a = x[i], &b = x[4 + ((i + 1) & 3)], &c = x[8 + ((i + 2) & 3)], &d = x[12 + ((i + 3) & 3)];
                a += b; d = __byte_perm(d ^ a, 0, 0x1032);
                c += d; b = __funnelshift_l(b ^ c, b ^ c, 12);
                a += b; d = __byte_perm(d ^ a, 0, 0x2103);
                c += d; b = __funnelshift_l(b ^ c, b ^ c, 7);
            }
        }
    } else if (MIX == 2) {
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] = x[i] * mul + y;
            }
        }
    } else if (MIX == 3) {
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 4; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    x[i] += y;
                    x[8 + i] = x[8 + i] * mul + z;
                    x[i] ^= z;
                    x[8 + i] = x[8 + i] * mul + y;
                }
            }
        }
    } else if (MIX == 4) {
        const uint32_t sh = mul + 4; // 7 at run time: the compiler cannot fold consecutive rotations
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] = __funnelshift_l(x[i], x[i], sh);
            }
        }
    } else if (MIX == 5) {
        const uint32_t sel = 0x2100u + mul; // 0x2103 at run time
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] = __byte_perm(x[i], y, sel);
            }
        }
    } else if (MIX == 6) {
        uint64_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = ((uint64_t)x[i] << 32) | x[8 + i];
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) w[i] = (uint64_t)(uint32_t)w[i] * mul + w[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = (uint32_t)w[i] ^ (uint32_t)(w[i] >> 32);
    } else {
#pragma unroll 1
        for (int it = 0; it < kProbeIters; it++) {
#pragma unroll
            for (int r = 0; r < 4; r++) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    x[i] = x[i] + x[(i + 1) & 7] + y;
                    x[i] = x[i] ^ x[(i + 3) & 7] ^ z;
                }
            }
        }
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) acc ^= x[i];
    if (acc == 0x12345678u) sink[blockIdx.x * blockDim.x + threadIdx.x] = acc; // keeps the chains alive
}

constexpr double ops_per_iter(int mix) {
    return mix == 1 ? 96.0 : mix == 3 ? 128.0 : 64.0;
}

// SplitMix64: the k-th output (k = 0, 1, ...) of the stream seeded with `seed`
__device__ __forceinline__ uint64_t splitmix64_at(uint64_t seed, uint64_t k) {
    uint64_t z = seed + (k + 1) * 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

__global__ void fill_random_kernel(uint64_t *dst, uint64_t words, uint64_t seed) {
    for (uint64_t k = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; k < words; k += (uint64_t)gridDim.x * blockDim.x)
        dst[k] = splitmix64_at(seed, k);
}

} // namespace

cudaError_t launch_fill_random(uint8_t *dst, uint64_t bytes, uint64_t seed, int sm_count, cudaStream_t s) {
    const uint64_t words = bytes / 8; // ring sizes are multiples of 16
    if (words == 0) return cudaSuccess;
    fill_random_kernel<<<sm_count * 8, 256, 0, s>>>(reinterpret_cast<uint64_t *>(dst), words, seed);
    return cudaGetLastError();
}

// ---- what other work costs beside ChaCha20 rounds ----
// The seal/open kernels are ChaCha20 rounds (bound by the ALU pipe) plus Poly1305 and data movement.  This probe
// runs ChaCha20 double rounds, 4 warps per scheduler like the kernels, and adds K operations of one kind per
// double round from independent chains: 1 = 32x32+64 multiply-add (Poly1305's product form), 2 = FP64 fused
// multiply-add, 3 = 32-bit multiply-add, 4 = FP32 fused multiply-add, 5 = high half of a 32x32 product.  The
// result is scheduler cycles per double round per warp; the difference to K = 0 is what the extra work costs when
// it is interleaved as well as a compiler can interleave it, i.e. how much of it hides under the rounds.
constexpr int kCoIters = 2048;
__device__ __forceinline__ void probe_qr(uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    a += b; d = __byte_perm(d ^ a, 0, 0x1032);
    c += d; b = __funnelshift_l(b ^ c, b ^ c, 12);
    a += b; d = __byte_perm(d ^ a, 0, 0x2103);
    c += d; b = __funnelshift_l(b ^ c, b ^ c, 7);
}
template <int KIND, int K>
__device__ __forceinline__ void probe_extra(int first, int last, uint64_t (&w)[8], double (&f)[8], float (&g)[8], uint32_t (&y)[8],
                                            uint32_t mul, double dm) {
#pragma unroll
    for (int j = first; j < last; j++) {
        if (KIND == 1) w[j & 7] = (uint64_t)(uint32_t)w[j & 7] * mul + w[j & 7];
        if (KIND == 2) f[j & 7] = fma(f[j & 7], dm, f[(j + 1) & 7]);
        if (KIND == 3) y[j & 7] = y[j & 7] * mul + y[(j + 1) & 7];
        if (KIND == 4) g[j & 7] = fmaf(g[j & 7], (float)dm, g[(j + 1) & 7]);
        if (KIND == 5) y[j & 7] = __umulhi(y[j & 7], mul) + y[(j + 1) & 7];
    }
}
template <int KIND, int K>
__global__ void __launch_bounds__(128, 4) coissue_probe_kernel(uint32_t *sink, uint32_t seed, uint32_t mul, double dm) {
    uint32_t x[16], y[8];
    uint64_t w[8];
    double f[8];
    float g[8];
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = seed * (i + 1) + threadIdx.x;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        w[i] = seed * 77ull + i + threadIdx.x;
        f[i] = 1.0 + (double)(threadIdx.x + i) * 1e-3;
        g[i] = (float)f[i];
        y[i] = seed + i * 7 + threadIdx.x;
    }
#pragma unroll 1
    for (int it = 0; it < kCoIters; it++) {
        probe_qr(x[0], x[4], x[8], x[12]); probe_qr(x[1], x[5], x[9], x[13]);
        probe_qr(x[2], x[6], x[10], x[14]); probe_qr(x[3], x[7], x[11], x[15]);
        probe_extra<KIND, K>(0, K / 2, w, f, g, y, mul, dm);
        probe_qr(x[0], x[5], x[10], x[15]); probe_qr(x[1], x[6], x[11], x[12]);
        probe_qr(x[2], x[7], x[8], x[13]); probe_qr(x[3], x[4], x[9], x[14]);
        probe_extra<KIND, K>(K / 2, K, w, f, g, y, mul, dm);
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) acc ^= x[i];
#pragma unroll
    for (int i = 0; i < 8; i++) acc ^= (uint32_t)w[i] ^ (uint32_t)(w[i] >> 32) ^ (uint32_t)__double2loint(f[i]) ^ __float_as_uint(g[i]) ^ y[i];
    if (acc == 0x12345678u) sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

// Two ChaCha20 states per thread (twice the independent quarter rounds in flight per warp) at HALF the warps: what a
// seal/open kernel with two cipher blocks per thread would run at (its registers allow 2 CTAs per SM).  The CTAs ask
// for enough dynamic shared memory that only two fit an SM.
__global__ void __launch_bounds__(128, 2) coissue_two_blocks_kernel(uint32_t *sink, uint32_t seed) {
    uint32_t x[16], z[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        x[i] = seed * (i + 1) + threadIdx.x;
        z[i] = seed * (i + 33) + threadIdx.x * 3u;
    }
#pragma unroll 1
    for (int it = 0; it < kCoIters; it++) {
        probe_qr(x[0], x[4], x[8], x[12]); probe_qr(z[0], z[4], z[8], z[12]);
        probe_qr(x[1], x[5], x[9], x[13]); probe_qr(z[1], z[5], z[9], z[13]);
        probe_qr(x[2], x[6], x[10], x[14]); probe_qr(z[2], z[6], z[10], z[14]);
        probe_qr(x[3], x[7], x[11], x[15]); probe_qr(z[3], z[7], z[11], z[15]);
        probe_qr(x[0], x[5], x[10], x[15]); probe_qr(z[0], z[5], z[10], z[15]);
        probe_qr(x[1], x[6], x[11], x[12]); probe_qr(z[1], z[6], z[11], z[12]);
        probe_qr(x[2], x[7], x[8], x[13]); probe_qr(z[2], z[7], z[8], z[13]);
        probe_qr(x[3], x[4], x[9], x[14]); probe_qr(z[3], z[4], z[9], z[14]);
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) acc ^= x[i] ^ z[i];
    if (acc == 0x12345678u) sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
}
cudaError_t run_coissue_two_blocks(bnk_ctx *ctx, double sm_hz, double *clk) {
    const int waves = 4, ctas = ctx->sm_count * 2 * waves; // 2 CTAs of 4 warps per SM: 2 warps per scheduler
    const int smem = 100 << 10;
    cudaError_t e = cudaFuncSetAttribute(coissue_two_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    uint32_t *sink = nullptr;
    if ((e = cudaMalloc(&sink, (size_t)ctas * 128 * sizeof(uint32_t))) != cudaSuccess) return e;
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaStream_t s = ctx->admin_stream;
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(t0, s);
        coissue_two_blocks_kernel<<<ctas, 128, smem, s>>>(sink, 17u + rep);
        cudaEventRecord(t1, s);
        ctx->launches += 1;
        if ((e = cudaEventSynchronize(t1)) != cudaSuccess) break;
        float ms = 0;
        cudaEventElapsedTime(&ms, t0, t1);
        if (rep >= 1 && ms < best) best = ms;
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(sink);
    if (e != cudaSuccess) return e;
    // per double round of ONE cipher block, per scheduler: 2 warps x 2 blocks share a scheduler
    *clk = best * 1e-3 * sm_hz / kCoIters / waves / 4.0;
    return cudaSuccess;
}

template <int KIND, int K>
cudaError_t run_coissue(bnk_ctx *ctx, double sm_hz, double *clk) {
    const int waves = 4, ctas = ctx->sm_count * 4 * waves; // 4 CTAs of 4 warps per SM: 4 warps per scheduler
    uint32_t *sink = nullptr;
    cudaError_t e = cudaMalloc(&sink, (size_t)ctas * 128 * sizeof(uint32_t));
    if (e != cudaSuccess) return e;
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaStream_t s = ctx->admin_stream;
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(t0, s);
        coissue_probe_kernel<KIND, K><<<ctas, 128, 0, s>>>(sink, 17u + rep, 3u, 1.0000001);
        cudaEventRecord(t1, s);
        ctx->launches += 1;
        if ((e = cudaEventSynchronize(t1)) != cudaSuccess) break;
        float ms = 0;
        cudaEventElapsedTime(&ms, t0, t1);
        if (rep >= 1 && ms < best) best = ms;
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(sink);
    if (e != cudaSuccess) return e;
    *clk = best * 1e-3 * sm_hz / kCoIters / waves / 4.0; // per double round, per warp, in cycles of its scheduler
    return cudaSuccess;
}

cudaError_t probe_coissue(bnk_ctx *ctx, int kind, int k, double *clk) {
    int khz = 0;
    cudaError_t e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device);
    if (e != cudaSuccess) return e;
    const double hz = khz * 1e3;
    const int key = kind * 100 + k;
    switch (key) {
    case 0: return run_coissue<0, 0>(ctx, hz, clk);
    case 108: return run_coissue<1, 8>(ctx, hz, clk);
    case 116: return run_coissue<1, 16>(ctx, hz, clk);
    case 216: return run_coissue<2, 16>(ctx, hz, clk);
    case 232: return run_coissue<2, 32>(ctx, hz, clk);
    case 316: return run_coissue<3, 16>(ctx, hz, clk);
    case 332: return run_coissue<3, 32>(ctx, hz, clk);
    case 416: return run_coissue<4, 16>(ctx, hz, clk);
    case 432: return run_coissue<4, 32>(ctx, hz, clk);
    case 508: return run_coissue<5, 8>(ctx, hz, clk);
    case 516: return run_coissue<5, 16>(ctx, hz, clk);
    case 600: return run_coissue_two_blocks(ctx, hz, clk);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t probe_int_throughput(bnk_ctx *ctx, int mix, double *tops) {
    if (mix < 0 || mix > 7) return cudaErrorInvalidValue;
    const int ctas = ctx->sm_count * 8, threads = 256;
    uint32_t *sink = nullptr;
    cudaError_t e = cudaMalloc(&sink, (size_t)ctas * threads * sizeof(uint32_t));
    if (e != cudaSuccess) return e;
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaStream_t s = ctx->admin_stream;
    float best = 1e30f;
    for (int rep = 0; rep < 5; rep++) { // first repetitions warm the clocks up
        cudaEventRecord(t0, s);
        switch (mix) {
        case 0: int_probe_kernel<0><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 1: int_probe_kernel<1><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 2: int_probe_kernel<2><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 3: int_probe_kernel<3><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 4: int_probe_kernel<4><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 5: int_probe_kernel<5><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        case 6: int_probe_kernel<6><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        default: int_probe_kernel<7><<<ctas, threads, 0, s>>>(sink, 17u + rep, 3u); break;
        }
        cudaEventRecord(t1, s);
        ctx->launches += 1;
        e = cudaEventSynchronize(t1);
        if (e != cudaSuccess) break;
        float ms = 0;
        cudaEventElapsedTime(&ms, t0, t1);
        if (rep >= 1 && ms < best) best = ms;
    }
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(sink);
    if (e != cudaSuccess) return e;
    const double ops = ops_per_iter(mix) * kProbeIters * (double)ctas * threads;
    *tops = ops / (best * 1e-3) / 1e12;
    return cudaSuccess;
}
