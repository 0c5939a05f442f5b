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
