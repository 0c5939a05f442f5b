// Per-keypair ordering work for sm_100a: grouping a batch by keypair slot while
// keeping arrival order (a stable least-significant-digit radix sort whose ranking
// step uses warp match/ballot instead of per-element atomics), handing out send
// counters, and walking the anti-replay window.
//
// Why a stable grouping: both the send counter (packets of one peer get
// consecutive nonces in batch order) and the replay window (verdicts depend on
// the arrival order of a peer's authenticated packets) are defined by a
// sequential walk per peer.  Different peers are independent, so after grouping
// one thread walks one peer's packets and all peers proceed in parallel.
#include "bnk_internal.cuh"

namespace {

constexpr uint32_t kSortThreads = 256;                  // 8 warps per CTA
constexpr uint32_t kSortWarps = kSortThreads / 32;
constexpr uint32_t kTilesPerWarp = 32;                  // a lane keeps 32 keys in registers
constexpr uint32_t kWarpSpan = 32 * kTilesPerWarp;      // 1024 consecutive elements per warp
constexpr uint32_t kChunk = kSortWarps * kWarpSpan;     // 8192 elements per CTA
constexpr uint32_t kMaxDigitBits = 9;
constexpr uint32_t kMaxBins = 1u << kMaxDigitBits;

struct SortKeySrc {
    const uint32_t *slot;
    const uint8_t *status;
    uint32_t max_slots;
    int only_status_ok; // 1: packets whose status is not OK/KEEPALIVE do not take part
};

// Key of packet i: its keypair slot, or max_slots ("takes no part", sorts last).
__device__ __forceinline__ uint32_t slot_key(const SortKeySrc &k, uint32_t i) {
    const uint32_t s = k.slot[i];
    if (s >= k.max_slots) return k.max_slots;
    if (k.only_status_ok) {
        const uint8_t st = k.status[i];
        if (st != BNK_PKT_OK && st != BNK_PKT_KEEPALIVE) return k.max_slots;
    }
    return s;
}

// one shared-memory add per distinct digit in the warp instead of one per lane
__device__ __forceinline__ void warp_hist_add(uint32_t *cnt, uint32_t digit, bool have) {
    const uint32_t peers = __match_any_sync(0xffffffffu, have ? digit : 0xffffffffu);
    if (have && (__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&cnt[digit], __popc(peers));
}

// --- pass step 1: per-chunk digit histogram -------------------------------------------
// grid = chunks, block = 256.  hist is digit-major: hist[digit * chunks + chunk].
__global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(SortKeySrc src, const uint32_t *keys_in,
                                                                  uint32_t n, uint32_t shift, uint32_t bins,
                                                                  uint32_t chunks, uint32_t *hist) {
    __shared__ uint32_t cnt[kMaxBins];
    const uint32_t tid = threadIdx.x, chunk = blockIdx.x;
    for (uint32_t d = tid; d < bins; d += kSortThreads) cnt[d] = 0;
    __syncthreads();
    const uint32_t begin = chunk * kChunk;
    const uint32_t end = min(n, begin + kChunk);
    for (uint32_t base = begin; base < end; base += kSortThreads) { // uniform trip count per warp
        const uint32_t i = base + tid;
        const bool have = i < end;
        uint32_t digit = 0;
        if (have) digit = ((keys_in ? keys_in[i] : slot_key(src, i)) >> shift) & (bins - 1);
        warp_hist_add(cnt, digit, have);
    }
    __syncthreads();
    for (uint32_t d = tid; d < bins; d += kSortThreads) hist[d * chunks + chunk] = cnt[d];
}

// --- pass step 2: exclusive scan of the histogram (single CTA) -------------------------
// Tiles of 4096 values; each thread owns 4 consecutive ones, warps combine with shuffles
// and a running carry links the tiles.
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(uint32_t *data, uint32_t n) {
    __shared__ uint32_t warp_off[32];
    __shared__ uint32_t carry_s;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n; base += 4096) {
        const uint32_t i0 = base + tid * 4;
        uint32_t v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = (i0 + k < n) ? data[i0 + k] : 0u;
        const uint32_t mine = v[0] + v[1] + v[2] + v[3];
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += t;
        }
        if (lane == 31) warp_off[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const uint32_t ws = warp_off[lane];
            uint32_t wi = ws;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= (uint32_t)o) wi += t;
            }
            warp_off[lane] = wi - ws;
        }
        __syncthreads();
        uint32_t run = carry_s + warp_off[warp] + (incl - mine);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (i0 + k < n) data[i0 + k] = run;
            run += v[k];
        }
        __syncthreads();
        if (tid == 1023) carry_s = run; // carry + this tile's total
        __syncthreads();
    }
}

// --- pass step 3: stable scatter --------------------------------------------------------
// grid = chunks, block = 256.  Warp w owns the 1024 consecutive elements [w*1024, (w+1)*1024) of
// the chunk and keeps their keys in registers.  (A) every warp counts its digits, (B) the counts
// become start positions: global start of the digit for this chunk, plus the counts of the warps
// before, (C) every warp walks its elements in order, 32 at a time; lanes holding the same digit
// find each other with match_any and take consecutive positions, so equal digits keep their
// input order.  No per-element atomics on global memory.
__global__ void __launch_bounds__(kSortThreads) radix_scatter_kernel(SortKeySrc src, const uint32_t *keys_in,
                                                                     const uint32_t *vals_in, uint32_t n,
                                                                     uint32_t shift, uint32_t bins, uint32_t chunks,
                                                                     const uint32_t *hist, uint32_t *keys_out,
                                                                     uint32_t *vals_out) {
    __shared__ uint32_t cur[kSortWarps][kMaxBins];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, chunk = blockIdx.x;
    for (uint32_t d = tid; d < kSortWarps * kMaxBins; d += kSortThreads) (&cur[0][0])[d] = 0;
    __syncthreads();
    const uint32_t begin = chunk * kChunk + warp * kWarpSpan;
    const uint32_t end = min(n, chunk * kChunk + kChunk);
    uint32_t key[kTilesPerWarp];
#pragma unroll
    for (uint32_t t = 0; t < kTilesPerWarp; t++) {
        const uint32_t i = begin + t * 32 + lane;
        const bool have = i < end;
        key[t] = have ? (keys_in ? keys_in[i] : slot_key(src, i)) : 0xffffffffu;
        warp_hist_add(cur[warp], (key[t] >> shift) & (bins - 1), have);
    }
    __syncthreads();
    for (uint32_t d = tid; d < bins; d += kSortThreads) {
        uint32_t run = hist[d * chunks + chunk];
#pragma unroll
        for (uint32_t w = 0; w < kSortWarps; w++) {
            const uint32_t c = cur[w][d];
            cur[w][d] = run;
            run += c;
        }
    }
    __syncthreads();
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t *mine = cur[warp];
#pragma unroll
    for (uint32_t t = 0; t < kTilesPerWarp; t++) {
        const uint32_t i = begin + t * 32 + lane;
        const bool have = i < end;
        const uint32_t digit = have ? ((key[t] >> shift) & (bins - 1)) : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, digit);
        const uint32_t rank = __popc(peers & lt);
        uint32_t pos = 0;
        if (have) pos = mine[digit] + rank;
        __syncwarp();
        if (have && rank == 0) mine[digit] += __popc(peers);
        __syncwarp();
        if (have) {
            keys_out[pos] = key[t];
            vals_out[pos] = vals_in ? vals_in[i] : i;
        }
    }
}

// --- send counters ----------------------------------------------------------------------
// One thread per slot segment: packets of the slot get base, base+1, ... in batch order and
// the slot's counter moves past them, saturating at Reject-After-Messages (packets at or
// beyond it are refused by the seal kernel).
__global__ void assign_counters_kernel(const uint32_t *keys, const uint32_t *order, const uint32_t *head,
                                       uint32_t n, uint32_t max_slots, uint64_t *send_counter,
                                       uint64_t *counter_out) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const uint32_t slot = keys[j];
    if (head ? !head[j] : (j != 0 && keys[j - 1] == slot)) return; // only the first packet of a run walks it
    if (slot >= max_slots) return;
    const uint64_t base = send_counter[slot];
    uint32_t k = j;
    for (; k < n && keys[k] == slot; k++) {
        uint64_t c = base + (uint64_t)(k - j);
        if (c < base || c > BNK_REJECT_AFTER_MESSAGES) c = BNK_REJECT_AFTER_MESSAGES;
        counter_out[order[k]] = c;
    }
    uint64_t next = base + (uint64_t)(k - j);
    if (next < base || next > BNK_REJECT_AFTER_MESSAGES) next = BNK_REJECT_AFTER_MESSAGES;
    send_counter[slot] = next;
}

// --- anti-replay window, RFC 6479 -------------------------------------------------------
// One thread per slot segment walks the slot's packets in arrival order; only packets the open
// kernel authenticated (status OK or KEEPALIVE) reach the window, the others are stepped over.
__global__ void replay_kernel(const uint32_t *keys, const uint32_t *order, const uint32_t *head, uint32_t n,
                              uint32_t max_slots, uint32_t ring_blocks, uint64_t *replay_last,
                              uint64_t *replay_ring, const uint64_t *counter, uint8_t *status) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const uint32_t slot = keys[j];
    if (head ? !head[j] : (j != 0 && keys[j - 1] == slot)) return;
    if (slot >= max_slots) return;
    uint64_t *ring = replay_ring + (size_t)slot * ring_blocks;
    const uint64_t mask = ring_blocks - 1;
    const uint64_t window = (uint64_t)(ring_blocks - 1) * 64u;
    uint64_t last = replay_last[slot];
    for (uint32_t k = j; k < n && keys[k] == slot; k++) {
        const uint32_t pkt = order[k];
        const uint8_t st = status[pkt];
        if (st != BNK_PKT_OK && st != BNK_PKT_KEEPALIVE) continue;
        const uint64_t c = counter[pkt];
        bool ok = c < BNK_REJECT_AFTER_MESSAGES;
        if (ok) {
            const uint64_t block = c >> 6;
            if (c > last) {
                const uint64_t top = last >> 6;
                uint64_t steps = block - top;
                if (steps > ring_blocks) steps = ring_blocks;
                for (uint64_t s = 1; s <= steps; s++) ring[(top + s) & mask] = 0;
                last = c;
            } else if (last - c > window) {
                ok = false;
            }
            if (ok) {
                const uint64_t bit = 1ull << (c & 63u);
                const uint64_t w = ring[block & mask];
                if (w & bit) ok = false;
                else ring[block & mask] = w | bit;
            }
        }
        if (!ok) status[pkt] = BNK_PKT_REPLAY;
    }
    replay_last[slot] = last;
}

// --- scheduling order by length class (mixed packet sizes) ------------------------------
// Packets with the same number of 64-byte cipher blocks end up next to each other so that
// the lanes of a seal/open warp finish together.  Order inside a class does not matter.
constexpr uint32_t kLenBins = 1026;
__device__ __forceinline__ uint32_t len_bin(uint32_t len, bool open_side) {
    uint32_t body = open_side ? (len >= 32u ? len - 32u : 0u) : len;
    uint32_t blocks = (body + 63u) >> 6;
    return blocks > kLenBins - 1 ? kLenBins - 1 : blocks;
}
// Real traffic has a handful of sizes, so all lanes of a warp tend to hit the same few bins: lanes
// with equal bins elect a leader that does one atomic for the group.
__global__ void __launch_bounds__(256) len_hist_kernel(const uint32_t *len, uint32_t n, int open_side,
                                                       uint32_t *bins) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool have = i < n;
    const uint32_t bin = have ? len_bin(len[i], open_side) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, bin);
    if (have && (__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&bins[bin], __popc(peers));
}
__global__ void __launch_bounds__(256) len_scatter_kernel(const uint32_t *len, uint32_t n, int open_side,
                                                          uint32_t *bins, uint32_t *order) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31;
    const bool have = i < n;
    const uint32_t bin = have ? len_bin(len[i], open_side) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, bin);
    const int leader = __ffs(peers) - 1;
    uint32_t base = 0;
    if (have && leader == (int)lane) base = atomicAdd(&bins[bin], __popc(peers));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (have) order[base + __popc(peers & ((1u << lane) - 1u))] = i;
}

struct SortPlan {
    uint32_t passes, digit_bits;
};
SortPlan plan_for(uint32_t max_slots) {
    uint32_t bits = 1;
    while ((1ull << bits) <= (uint64_t)max_slots) bits++; // keys run 0..max_slots inclusive
    SortPlan p;
    p.passes = (bits + kMaxDigitBits - 1) / kMaxDigitBits;
    p.digit_bits = (bits + p.passes - 1) / p.passes;
    return p;
}

} // namespace

uint32_t group_sort_chunks(uint32_t max_pkts) { return (max_pkts + kChunk - 1) / kChunk; }

// Sorts packet indices 0..n-1 by keypair slot, stable.  Leaves the sorted keys in
// dev.keys_tmp (second half) and the packet indices in dev.order.
cudaError_t launch_group_by_slot(bnk_batch *b, uint32_t n, bool only_status_ok, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    bnk_ctx *ctx = b->ctx;
    DeviceBatch &d = b->dev;
    const SortPlan plan = plan_for(ctx->cfg.max_keypairs);
    const uint32_t bins = 1u << plan.digit_bits;
    const uint32_t chunks = (n + kChunk - 1) / kChunk;
    SortKeySrc src{d.slot, d.status, ctx->cfg.max_keypairs, only_status_ok ? 1 : 0};
    // ping-pong so that the last pass lands in (keys_tmp + max_pkts, order)
    uint32_t *kbuf[2] = {d.keys_tmp + b->max_pkts, d.keys_tmp};
    uint32_t *vbuf[2] = {d.order, d.order_tmp};
    const uint32_t *kin = nullptr, *vin = nullptr;
    for (uint32_t p = 0; p < plan.passes; p++) {
        const uint32_t shift = p * plan.digit_bits;
        const uint32_t o = (plan.passes - 1 - p) & 1u;
        radix_hist_kernel<<<chunks, kSortThreads, 0, s>>>(src, kin, n, shift, bins, chunks, d.hist);
        exclusive_scan_kernel<<<1, 1024, 0, s>>>(d.hist, bins * chunks);
        radix_scatter_kernel<<<chunks, kSortThreads, 0, s>>>(src, kin, vin, n, shift, bins, chunks, d.hist, kbuf[o],
                                                            vbuf[o]);
        ctx->launches += 3;
        kin = kbuf[o];
        vin = vbuf[o];
    }
    return cudaGetLastError();
}

cudaError_t launch_assign_counters(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    cudaError_t e = launch_group_by_slot(b, n, false, s);
    if (e != cudaSuccess) return e;
    DeviceBatch &d = b->dev;
    assign_counters_kernel<<<(n + 255) / 256, 256, 0, s>>>(d.keys_tmp + b->max_pkts, d.order, nullptr, n,
                                                          b->ctx->cfg.max_keypairs, b->ctx->kt.send_counter,
                                                          d.counter);
    b->ctx->launches += 1;
    return cudaGetLastError();
}

// Expects launch_group_by_slot(b, n, false, ...) to have completed before this point of stream s.
cudaError_t launch_replay(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    bnk_ctx *ctx = b->ctx;
    replay_kernel<<<(n + 255) / 256, 256, 0, s>>>(d.keys_tmp + b->max_pkts, d.order, nullptr, n,
                                                 ctx->cfg.max_keypairs, ctx->cfg.replay_ring_blocks,
                                                 ctx->kt.replay_last, ctx->kt.replay_ring, d.counter, d.status);
    ctx->launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_length_order(bnk_batch *b, uint32_t n, const uint32_t *len, bool open_side, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    cudaError_t e = cudaMemsetAsync(d.counters32, 0, kLenBins * sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    len_hist_kernel<<<(n + 255) / 256, 256, 0, s>>>(len, n, open_side ? 1 : 0, d.counters32);
    exclusive_scan_kernel<<<1, 1024, 0, s>>>(d.counters32, kLenBins);
    len_scatter_kernel<<<(n + 255) / 256, 256, 0, s>>>(len, n, open_side ? 1 : 0, d.counters32, d.len_order);
    b->ctx->launches += 3;
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Send-counter hand-out for callers that must not allocate.
//
// The packet loop of a forwarder cannot afford cudaMalloc/cudaFree: both serialise the
// whole device, so one allocation stalls every other batch in flight, and a caller that
// keeps packets in device buffers of its own (for instance buffers a NIC writes into
// directly) has no bnk_batch whose creation would have set the grouping scratch aside.
// For those callers the same grouping kernels run here on a fixed scratch area that is
// part of the library image: kNoAllocMaxPkts packets at most, 384 KiB held by every GPU
// that loads the library until the process exits.
//
// The area is shared by every call and keeps whatever the previous call left in it.  All
// regions are written before they are read within one call (the histogram kernel stores
// every bin of every chunk it later scans, the scatter kernel stores every element below
// npkts), so nothing needs clearing; calls that overlap on the GPU race on
// the area and must be ordered by the caller (same stream, or an event between them).
// ---------------------------------------------------------------------------------------
namespace {

constexpr uint32_t kNoAllocMaxPkts = BNK_NOALLOC_MAX_PKTS;
constexpr uint32_t kNoAllocChunks = (kNoAllocMaxPkts + kChunk - 1) / kChunk;
constexpr size_t kNoAllocWords = (size_t)5 * kNoAllocMaxPkts + 16384; // 384 KiB; the histogram needs kMaxBins * kNoAllocChunks words
static_assert((size_t)kMaxBins * kNoAllocChunks <= 16384, "histogram region too small");

static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocWords];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mu;
uint32_t *g_noalloc_ptr[kNoAllocMaxDevices] = {};

// Device address of the scratch area on the current device.  In host code the array's name
// is only a handle, so the address is asked for once per device and remembered.
cudaError_t noalloc_scratch(int device, uint32_t **out) {
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        g_noalloc_ptr[device] = static_cast<uint32_t *>(p);
    }
    *out = g_noalloc_ptr[device];
    return cudaSuccess;
}

int noalloc_fail(bnk_ctx *ctx, int code, const char *what, cudaError_t e = cudaSuccess) {
    std::lock_guard<std::mutex> g(ctx->mu);
    ctx->last_error = what;
    if (e != cudaSuccess) {
        ctx->last_error += ": ";
        ctx->last_error += cudaGetErrorString(e);
    }
    return code;
}

} // namespace

extern "C" int bnk_assign_counters_noalloc(bnk_ctx *ctx, void *stream, const uint32_t *dev_slot, uint32_t npkts,
                                           uint64_t *dev_counter) {
    if (!ctx) return BNK_EINVAL;
    if (!dev_slot || !dev_counter) return noalloc_fail(ctx, BNK_EINVAL, "bnk_assign_counters_noalloc: null buffer");
    if (npkts > kNoAllocMaxPkts)
        return noalloc_fail(ctx, BNK_EINVAL,
                            "bnk_assign_counters_noalloc: npkts exceeds BNK_NOALLOC_MAX_PKTS (16384); split the batch "
                            "or use bnk_seal_submit with BNK_F_ASSIGN_COUNTERS");
    if (ctx->device < 0 || ctx->device >= kNoAllocMaxDevices)
        return noalloc_fail(ctx, BNK_EINVAL, "bnk_assign_counters_noalloc: device ordinal above 63");
    if (npkts == 0) return BNK_SUCCESS;
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return noalloc_fail(ctx, BNK_ECUDA, "cudaSetDevice", e);
    uint32_t *base = nullptr;
    if ((e = noalloc_scratch(ctx->device, &base)) != cudaSuccess)
        return noalloc_fail(ctx, BNK_ECUDA, "cudaGetSymbolAddress(scratch)", e);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const uint32_t n = npkts, cap = kNoAllocMaxPkts;
    uint32_t *keys_a = base, *keys_b = base + cap, *vals_a = base + 2 * cap, *order = base + 3 * cap;
    uint32_t *hist = base + 5 * cap; // [4*cap, 5*cap) is spare
    const SortPlan plan = plan_for(ctx->cfg.max_keypairs);
    const uint32_t bins = 1u << plan.digit_bits;
    const uint32_t chunks = (n + kChunk - 1) / kChunk;
    SortKeySrc src{dev_slot, nullptr, ctx->cfg.max_keypairs, 0};
    uint32_t *kbuf[2] = {keys_b, keys_a};
    uint32_t *vbuf[2] = {order, vals_a};
    const uint32_t *kin = nullptr, *vin = nullptr;
    for (uint32_t p = 0; p < plan.passes; p++) {
        const uint32_t shift = p * plan.digit_bits;
        const uint32_t o = (plan.passes - 1 - p) & 1u;
        radix_hist_kernel<<<chunks, kSortThreads, 0, s>>>(src, kin, n, shift, bins, chunks, hist);
        exclusive_scan_kernel<<<1, 1024, 0, s>>>(hist, bins * chunks);
        radix_scatter_kernel<<<chunks, kSortThreads, 0, s>>>(src, kin, vin, n, shift, bins, chunks, hist, kbuf[o], vbuf[o]);
        kin = kbuf[o];
        vin = vbuf[o];
    }
    assign_counters_kernel<<<(n + 255) / 256, 256, 0, s>>>(keys_b, order, nullptr, n, ctx->cfg.max_keypairs,
                                                          ctx->kt.send_counter, dev_counter);
    ctx->launches += 3 * plan.passes + 1;
    if ((e = cudaGetLastError()) != cudaSuccess) return noalloc_fail(ctx, BNK_ECUDA, "kernel launch", e);
    return BNK_SUCCESS;
}
