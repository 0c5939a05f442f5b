// Per-keypair ordering work for sm_100a: grouping a batch by keypair slot while
// keeping arrival order (a stable least-significant-digit radix sort whose ranking
// step uses warp match/ballot instead of per-element atomics), handing out send
// counters, and walking the anti-replay window.
//
// Why a stable grouping: both the send counter (packets of one peer get
// consecutive nonces in batch order) and the replay window (verdicts depend on
// the arrival order of a peer's authenticated packets) are defined by a
// sequential walk per peer.  Different peers are independent, and inside a peer
// the walk has a parallel form: a packet's nonce is the peer's counter plus its
// rank in the peer's run, and the window's verdicts over a stretch of packets
// follow in closed form from the state at the start of the stretch.
#include "bnk_internal.cuh"

namespace {

constexpr uint32_t kSortThreads = 256; // 8 warps per CTA
constexpr uint32_t kSortWarps = kSortThreads / 32;
constexpr uint32_t kMaxTiles = 32;     // a lane keeps up to 32 keys in registers
constexpr uint32_t kMaxDigitBits = 9;
constexpr uint32_t kMaxBins = 1u << kMaxDigitBits;
#ifndef BNK_SORT_MAX_CHUNKS
#define BNK_SORT_MAX_CHUNKS 320
#endif
constexpr uint32_t kBatchMaxChunks = BNK_SORT_MAX_CHUNKS; // ~2 CTAs per SM: enough to fill the GPU, few enough to scan quickly

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

// A CTA owns a chunk of 256 * TILES consecutive elements; warp w owns the 32 * TILES consecutive
// elements [w * 32 * TILES, (w + 1) * 32 * TILES) of it.

// --- pass step 1: per-chunk digit histogram -------------------------------------------
// grid = chunks, block = 256.  hist is digit-major: hist[digit * chunks + chunk].
template <uint32_t TILES>
__global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(SortKeySrc src, const uint32_t *keys_in,
                                                                  uint32_t n, uint32_t shift, uint32_t bins,
                                                                  uint32_t chunks, uint32_t *hist) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ uint32_t cnt[kMaxBins];
    const uint32_t tid = threadIdx.x, chunk = blockIdx.x;
    for (uint32_t d = tid; d < bins; d += kSortThreads) cnt[d] = 0;
    __syncthreads();
    const uint32_t begin = chunk * (kSortThreads * TILES);
    const uint32_t end = min(n, begin + kSortThreads * TILES);
#pragma unroll
    for (uint32_t t = 0; t < TILES; t++) {
        const uint32_t i = begin + t * kSortThreads + tid;
        const bool have = i < end;
        uint32_t digit = 0;
        if (have) digit = ((keys_in ? keys_in[i] : slot_key(src, i)) >> shift) & (bins - 1);
        warp_hist_add(cnt, digit, have);
    }
    __syncthreads();
    for (uint32_t d = tid; d < bins; d += kSortThreads) hist[d * chunks + chunk] = cnt[d];
}

// --- pass step 2: per digit, exclusive prefix over the chunks -------------------------
// One warp per digit row (coalesced: the row is contiguous).  Row totals go to totals[digit]; the
// scatter kernel turns them into digit bases on its own.
__global__ void __launch_bounds__(kSortThreads) radix_rowscan_kernel(uint32_t *hist, uint32_t bins, uint32_t chunks,
                                                                     uint32_t *totals) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t d = (blockIdx.x * kSortThreads + threadIdx.x) >> 5;
    if (d >= bins) return;
    uint32_t *row = hist + (size_t)d * chunks;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < chunks; base += 32) {
        const uint32_t c = base + lane;
        const uint32_t v = c < chunks ? row[c] : 0u;
        uint32_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += t;
        }
        if (c < chunks) row[c] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[d] = carry;
}

// --- exclusive scan of a small array by one CTA (length-class bins) ---------------------
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(uint32_t *data, uint32_t n) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
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
// grid = chunks, block = 256.  (A) every warp counts the digits of its elements (kept in registers),
// (B) the counts become start positions: base of the digit (exclusive prefix of the row totals, done
// here per CTA) + the digit's elements in earlier chunks + the counts of the warps before,
// (C) every warp walks its elements in order, 32 at a time; lanes holding the same digit find each
// other with match_any and take consecutive positions, so equal digits keep their input order.
// No per-element atomics on global memory.
template <uint32_t TILES>
__global__ void __launch_bounds__(kSortThreads) radix_scatter_kernel(SortKeySrc src, const uint32_t *keys_in,
                                                                     const uint32_t *vals_in, uint32_t n,
                                                                     uint32_t shift, uint32_t bins, uint32_t chunks,
                                                                     const uint32_t *hist, const uint32_t *totals,
                                                                     uint32_t *keys_out, uint32_t *vals_out) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ uint32_t cur[kSortWarps][kMaxBins];
    __shared__ uint32_t base_of[kMaxBins];
    __shared__ uint32_t warp_sum[kSortWarps];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, chunk = blockIdx.x;
    for (uint32_t d = tid; d < kSortWarps * kMaxBins; d += kSortThreads) (&cur[0][0])[d] = 0;
    __syncthreads();
    const uint32_t begin = chunk * (kSortThreads * TILES) + warp * (32 * TILES);
    const uint32_t end = min(n, (chunk + 1) * (kSortThreads * TILES));
    uint32_t key[TILES];
#pragma unroll
    for (uint32_t t = 0; t < TILES; t++) {
        const uint32_t i = begin + t * 32 + lane;
        const bool have = i < end;
        key[t] = have ? (keys_in ? keys_in[i] : slot_key(src, i)) : 0xffffffffu;
        warp_hist_add(cur[warp], (key[t] >> shift) & (bins - 1), have);
    }
    // digit bases: exclusive prefix over totals[0..bins), two digits per thread (bins <= 512)
    {
        const uint32_t d0 = 2 * tid, d1 = 2 * tid + 1;
        const uint32_t v0 = d0 < bins ? totals[d0] : 0u, v1 = d1 < bins ? totals[d1] : 0u;
        uint32_t incl = v0 + v1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += t;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        uint32_t before = 0;
        for (uint32_t w = 0; w < warp; w++) before += warp_sum[w];
        const uint32_t excl = before + incl - (v0 + v1);
        if (d0 < bins) base_of[d0] = excl;
        if (d1 < bins) base_of[d1] = excl + v0;
    }
    __syncthreads();
    for (uint32_t d = tid; d < bins; d += kSortThreads) {
        uint32_t run = base_of[d] + hist[d * chunks + chunk];
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
    for (uint32_t t = 0; t < TILES; t++) {
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
// Packets of a slot get base, base+1, ... in batch order and the slot's counter moves past them, saturating
// at Reject-After-Messages (packets at or beyond it are refused by the seal kernel).  One thread per packet:
// in the sorted order a packet's rank inside its run is its position minus the start of the run, found by
// binary search, so a peer that owns most of a batch costs no more than any other.  The counters are read
// by the first kernel and advanced by the second, so no thread can see a counter that already moved.
__device__ __forceinline__ uint32_t run_start(const uint32_t *keys, uint32_t j) {
    const uint32_t key = keys[j];
    uint32_t lo = 0, hi = j; // first index in [0, j] whose key equals keys[j]
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (keys[mid] < key) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ uint64_t saturating_counter(uint64_t base, uint32_t k) {
    const uint64_t c = base + k;
    return (c < base || c > BNK_REJECT_AFTER_MESSAGES) ? BNK_REJECT_AFTER_MESSAGES : c;
}
__global__ void assign_counters_kernel(const uint32_t *keys, const uint32_t *order, uint32_t n, uint32_t max_slots,
                                       const uint64_t *send_counter, uint64_t *counter_out) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const uint32_t slot = keys[j];
    if (slot >= max_slots) return;
    counter_out[order[j]] = saturating_counter(send_counter[slot], j - run_start(keys, j));
}
__global__ void advance_counters_kernel(const uint32_t *keys, uint32_t n, uint32_t max_slots, uint64_t *send_counter) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const uint32_t slot = keys[j];
    if (slot >= max_slots || (j + 1 < n && keys[j + 1] == slot)) return; // the last packet of a run moves the counter
    send_counter[slot] = saturating_counter(send_counter[slot], j - run_start(keys, j) + 1);
}

// --- anti-replay window, RFC 6479 -------------------------------------------------------
// The window is defined by a sequential walk over a peer's authenticated packets in arrival order: a counter
// above `last` moves the window (clearing the ring words the top passes), one more than a window behind is
// refused, and one in between is accepted unless its bit is already marked.  A GPU cannot afford the walk: a
// peer that owns a large batch would hold the batch up for about a microsecond per 32 packets, and a small
// batch of many peers would pay one dependent chain of loads per peer.  The verdicts have a closed form in
// terms of the state (last, ring) at the start of the batch.  With M_j = max(last, counters of the peer's
// earlier packets of the batch), packet j is accepted iff its counter is below the message limit and either
// exceeds M_j, or lies within the window behind M_j, was not marked in the ring at the start (only counters
// <= last can be) and does not repeat the counter of an earlier packet.  (A ring word that the walk would have
// cleared before reaching j lies more than a window behind M_j; an earlier packet with the same counter that
// was itself refused was refused for a reason that still holds at j.)  Afterwards last = M at the end of the
// run, the words the top moved over are cleared, and the accepted packets within a ring of the new top are
// marked.  Every term is data-parallel over the grouped order:
//   M_j                         a segmented exclusive running maximum (a scan),
//   "marked at the start"       a read of the ring as it was before the batch,
//   "repeats an earlier one"    the lowest grouped position holding the same (peer, counter), found with a
//                               hash table of positions; built only when some packet of the batch lies behind
//                               its M_j inside the window, which in-order traffic never does.
// Up to 1024 packets all of this runs in the CTA that sorted them (group_small_kernel); beyond, as kernels in
// stream order: scan_tiles (also lays the counters out in grouped order), scan_carry, classify, advance (new
// last, clears), hash_clear, hash_insert, finish (duplicate look-up, verdicts, marks).
constexpr uint32_t kScanTile = 1024; // grouped positions per CTA: 256 threads x 4
constexpr uint64_t kReplayNoPart = ~0ull; // grouped-order counter of a packet that takes no part
constexpr uint32_t kHashEmpty = 0xffffffffu;
enum : uint8_t { RP_NOPART = 0, RP_ACCEPT = 1, RP_REJECT = 2, RP_PENDING = 3 };

struct ReplayArgs {
    const uint32_t *keys;  // [n] keypair slots in grouped order
    const uint32_t *order; // [n] packet index of each grouped position
    uint32_t n, max_slots, ring_blocks;
    uint64_t *replay_last, *replay_next, *replay_ring;
    const uint64_t *counter; // per packet, as the open kernel left it
    uint8_t *status;         // per packet
    uint64_t *sorted_counter; // [n] scratch
    uint8_t *state;           // [n] scratch
    uint32_t *table;          // hash table of positions, `mask` + 1 entries
    uint32_t mask;
};

struct SegMax { // running maximum that restarts at every run head
    uint32_t f; // a head lies inside the span
    uint64_t m; // maximum since the last head (or over the whole span)
};
__device__ __forceinline__ SegMax seg_combine(SegMax a, SegMax b) { // a: earlier span, b: the span after it
    return SegMax{a.f | b.f, (b.f || b.m > a.m) ? b.m : a.m};
}
__device__ __forceinline__ SegMax seg_shfl_up(SegMax v, int o) {
    return SegMax{__shfl_up_sync(0xffffffffu, v.f, o), __shfl_up_sync(0xffffffffu, v.m, o)};
}
// Inclusive scan of one value per thread over a CTA of NW warps; returns the exclusive prefix of the calling
// thread and the total of the CTA.  `part` is NW entries of shared memory.
template <int NW>
__device__ __forceinline__ SegMax seg_block_exclusive(SegMax mine, SegMax *part, SegMax &total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    SegMax inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const SegMax t = seg_shfl_up(inc, o);
        if (lane >= (uint32_t)o) inc = seg_combine(t, inc);
    }
    SegMax ex = seg_shfl_up(inc, 1);
    if (lane == 0) ex = SegMax{0u, 0ull};
    __syncthreads(); // `part` may still be read from an earlier call
    if (lane == 31) part[warp] = inc;
    __syncthreads();
    SegMax before{0u, 0ull};
    total = SegMax{0u, 0ull};
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        if ((uint32_t)w == warp) before = total;
        total = seg_combine(total, part[w]);
    }
    return seg_combine(before, ex);
}
// Four consecutive grouped positions per thread.  e[k] = maximum of the values of the same run that lie in
// front of item k (`carry` stands for what lies in front of the tile); total = the tile as one span.
__device__ __forceinline__ void tile_running_max(const bool head[4], const uint64_t v[4], uint64_t carry,
                                                 uint64_t e[4], SegMax *part, SegMax &total) {
    SegMax run{0u, 0ull};
    uint32_t headed = 0; // bit k: a head lies at or before item k inside this thread
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (head[k]) run = SegMax{1u, 0ull};
        e[k] = run.m;
        headed |= run.f << k;
        if (v[k] > run.m) run.m = v[k];
    }
    const SegMax ex = seg_block_exclusive<8>(run, part, total);
    const uint64_t front = ex.f ? ex.m : (carry > ex.m ? carry : ex.m);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (!((headed >> k) & 1u) && front > e[k]) e[k] = front;
}

// Counter of grouped position p, or kReplayNoPart.  Authenticated packets at or beyond the message limit are
// refused here: their verdict does not depend on the window and they leave no trace in it.
__device__ __forceinline__ uint64_t replay_gather(const ReplayArgs &a, uint32_t p, uint32_t slot) {
    uint64_t c = kReplayNoPart;
    if (slot < a.max_slots) {
        const uint32_t pkt = a.order[p];
        const uint8_t st = a.status[pkt];
        if (st == BNK_PKT_OK || st == BNK_PKT_KEEPALIVE) {
            c = a.counter[pkt];
            if (c >= BNK_REJECT_AFTER_MESSAGES) {
                a.status[pkt] = BNK_PKT_REPLAY;
                c = kReplayNoPart;
            }
        }
    }
    a.sorted_counter[p] = c;
    return c;
}
// Verdict of position p as far as it can be told without the duplicate search; the last packet of a run also
// leaves the peer's next `last`.  e = running maximum of the run in front of p.
__device__ __forceinline__ uint8_t replay_classify(const ReplayArgs &a, uint32_t p, uint32_t slot, uint64_t c, uint64_t e) {
    if (slot >= a.max_slots) return RP_NOPART;
    const uint64_t rmask = a.ring_blocks - 1, window = (uint64_t)(a.ring_blocks - 1) * 64u;
    const uint64_t last = a.replay_last[slot];
    const uint64_t M = e > last ? e : last;
    uint8_t st = RP_NOPART;
    uint64_t top = M;
    if (c != kReplayNoPart) {
        if (c > M) {
            st = RP_ACCEPT;
            top = c;
        } else if (M - c > window) st = RP_REJECT;
        else if (c <= last && ((a.replay_ring[(size_t)slot * a.ring_blocks + ((c >> 6) & rmask)] >> (c & 63u)) & 1ull))
            st = RP_REJECT;
        else st = RP_PENDING;
    }
    if (p + 1 == a.n || a.keys[p + 1] != slot) a.replay_next[slot] = top;
    return st;
}
// Warp-wide over 32 consecutive positions (p = this lane's): the peers whose run ends here move their window.
__device__ __forceinline__ void replay_advance_warp(const ReplayArgs &a, uint32_t p) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t key = p < a.n ? a.keys[p] : 0xffffffffu;
    const bool is_tail = p < a.n && key < a.max_slots && (p + 1 == a.n || a.keys[p + 1] != key);
    uint32_t tails = __ballot_sync(0xffffffffu, is_tail);
    const uint64_t rmask = a.ring_blocks - 1;
    while (tails) {
        const uint32_t src = __ffs(tails) - 1;
        tails &= tails - 1;
        const uint32_t slot = __shfl_sync(0xffffffffu, key, src);
        uint64_t *ring = a.replay_ring + (size_t)slot * a.ring_blocks;
        const uint64_t last = a.replay_last[slot], next = a.replay_next[slot];
        const uint64_t top = last >> 6;
        uint64_t steps = (next >> 6) - top;
        if (steps > a.ring_blocks) steps = a.ring_blocks;
        for (uint64_t i = lane; i < steps; i += 32) ring[(top + 1 + i) & rmask] = 0ull;
        __syncwarp();
        if (lane == 0) a.replay_last[slot] = next;
    }
}
__device__ __forceinline__ uint32_t replay_hash(uint32_t slot, uint64_t c) {
    uint64_t x = c * 0x9E3779B97F4A7C15ull + slot;
    x ^= x >> 29;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 32;
    return (uint32_t)x;
}
// table[h] = lowest grouped position that holds the key (peer, counter); the key of an entry is read through
// the position it holds and never changes, so a probe may compare against whatever position it sees.
// Warp-wide (32 consecutive positions, `active` per lane): of the lanes that hold the same key only the lowest,
// which has the lowest position, goes to the table, so a burst of copies of one packet costs one atomic per
// warp instead of one per copy.
__device__ __forceinline__ void replay_hash_insert_warp(const ReplayArgs &a, uint32_t p, bool active) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t slot = active ? a.keys[p] : 0u;
    const uint64_t c = active ? a.sorted_counter[p] : 0ull;
    const unsigned long long tag = active ? (c * 0x9E3779B97F4A7C15ull + slot) : ~0ull - lane;
    const uint32_t same_tag = __match_any_sync(0xffffffffu, tag);
    const uint32_t first = __ffs(same_tag) - 1;
    const uint32_t first_slot = __shfl_sync(0xffffffffu, slot, first);
    const uint64_t first_c = __shfl_sync(0xffffffffu, c, first);
    if (!active || (lane != first && first_slot == slot && first_c == c)) return; // a lower lane carries this key
    uint32_t h = replay_hash(slot, c) & a.mask;
    for (uint32_t probes = 0; probes <= a.mask; ++probes, h = (h + 1) & a.mask) {
        uint32_t cur = *(volatile uint32_t *)&a.table[h];
        if (cur == kHashEmpty) {
            cur = atomicCAS(&a.table[h], kHashEmpty, p);
            if (cur == kHashEmpty) return;
        }
        if (a.keys[cur] == slot && a.sorted_counter[cur] == c) {
            atomicMin(&a.table[h], p);
            return;
        }
    }
}
__device__ __forceinline__ bool replay_hash_has_earlier(const ReplayArgs &a, uint32_t p, uint32_t slot, uint64_t c) {
    uint32_t h = replay_hash(slot, c) & a.mask;
    for (uint32_t probes = 0; probes <= a.mask; ++probes, h = (h + 1) & a.mask) {
        const uint32_t cur = *(volatile uint32_t *)&a.table[h];
        if (cur == kHashEmpty) return false;
        if (a.keys[cur] == slot && a.sorted_counter[cur] == c) return cur < p;
    }
    return false;
}
// Warp-wide over 32 consecutive positions: settles the pending verdicts, writes the refusals and marks the
// ring.  Lanes that hit the same ring word hand their bits to the lowest of them.
__device__ __forceinline__ void replay_finish_warp(const ReplayArgs &a, uint32_t p) {
    const uint32_t lane = threadIdx.x & 31;
    uint8_t st = p < a.n ? a.state[p] : (uint8_t)RP_NOPART;
    uint32_t slot = 0;
    uint64_t c = 0;
    if (st != RP_NOPART) {
        slot = a.keys[p];
        c = a.sorted_counter[p];
    }
    if (st == RP_PENDING) st = replay_hash_has_earlier(a, p, slot, c) ? RP_REJECT : RP_ACCEPT;
    if (st == RP_REJECT) a.status[a.order[p]] = BNK_PKT_REPLAY;
    const uint64_t rmask = a.ring_blocks - 1;
    const bool mark = st == RP_ACCEPT && (a.replay_last[slot] >> 6) - (c >> 6) < a.ring_blocks;
    const unsigned long long word = mark ? (unsigned long long)slot * a.ring_blocks + ((c >> 6) & rmask) : ~0ull - lane;
    const uint32_t group = __match_any_sync(0xffffffffu, word);
    const bool leader = mark && (uint32_t)(__ffs(group) - 1) == lane;
    uint32_t leaders = __ballot_sync(0xffffffffu, leader);
    const uint32_t bit_lo = mark && (c & 32u) == 0 ? 1u << (c & 31u) : 0u;
    const uint32_t bit_hi = mark && (c & 32u) != 0 ? 1u << (c & 31u) : 0u;
    unsigned long long *ring = reinterpret_cast<unsigned long long *>(a.replay_ring);
    if (__popc(leaders) <= 4) {
        while (leaders) {
            const uint32_t src = __ffs(leaders) - 1;
            leaders &= leaders - 1;
            const uint32_t members = __shfl_sync(0xffffffffu, group, src);
            const bool in = (members >> lane) & 1u;
            const uint32_t lo = __reduce_or_sync(0xffffffffu, in ? bit_lo : 0u);
            const uint32_t hi = __reduce_or_sync(0xffffffffu, in ? bit_hi : 0u);
            if (lane == src) atomicOr(&ring[word], ((unsigned long long)hi << 32) | lo);
        }
    } else if (mark) {
        atomicOr(&ring[word], ((unsigned long long)bit_hi << 32) | bit_lo);
    }
}
// The tile of the calling CTA (thread t: positions base..base+3): counters gathered when GATHER, else read
// back; running maximum with `carry` in front; returns the tile as one span.
template <bool GATHER>
__device__ __forceinline__ SegMax replay_tile(const ReplayArgs &a, uint32_t base, uint64_t carry, uint32_t slot[4],
                                              uint64_t c[4], uint64_t e[4], SegMax *part) {
    bool head[4];
    uint64_t v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t p = base + k;
        head[k] = false;
        v[k] = 0;
        c[k] = kReplayNoPart;
        slot[k] = 0xffffffffu;
        if (p < a.n) {
            slot[k] = a.keys[p];
            head[k] = p == 0 || a.keys[p - 1] != slot[k];
            c[k] = GATHER ? replay_gather(a, p, slot[k]) : a.sorted_counter[p];
            if (c[k] != kReplayNoPart) v[k] = c[k];
        }
    }
    SegMax total;
    tile_running_max(head, v, carry, e, part, total);
    return total;
}

__global__ void __launch_bounds__(256) replay_scan_tiles_kernel(ReplayArgs a, uint32_t *tile_head, uint64_t *tile_max,
                                                                uint32_t *pending_flag) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ SegMax part[8];
    if (blockIdx.x == 0 && threadIdx.x == 0) *pending_flag = 0u;
    uint32_t slot[4];
    uint64_t c[4], e[4];
    const SegMax total = replay_tile<true>(a, blockIdx.x * kScanTile + threadIdx.x * 4u, 0ull, slot, c, e, part);
    if (threadIdx.x == 0) {
        tile_head[blockIdx.x] = total.f;
        tile_max[blockIdx.x] = total.m;
    }
}
// One CTA: carry[t] = running maximum that reaches tile t from the tiles in front of it.
__global__ void __launch_bounds__(1024) replay_scan_carry_kernel(const uint32_t *tile_head, const uint64_t *tile_max,
                                                                 uint32_t tiles, uint64_t *tile_carry) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ SegMax part[32];
    SegMax reached{0u, 0ull};
    for (uint32_t base = 0; base < tiles; base += 1024u) {
        const uint32_t t = base + threadIdx.x;
        SegMax mine{0u, 0ull};
        if (t < tiles) mine = SegMax{tile_head[t], tile_max[t]};
        SegMax total;
        const SegMax ex = seg_block_exclusive<32>(mine, part, total);
        if (t < tiles) tile_carry[t] = seg_combine(reached, ex).m;
        reached = seg_combine(reached, total);
    }
}
__global__ void __launch_bounds__(256) replay_classify_kernel(ReplayArgs a, const uint64_t *tile_carry,
                                                              uint32_t *pending_flag) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ SegMax part[8];
    const uint32_t base = blockIdx.x * kScanTile + threadIdx.x * 4u;
    uint32_t slot[4];
    uint64_t c[4], e[4];
    replay_tile<false>(a, base, tile_carry[blockIdx.x], slot, c, e, part);
    bool pending = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (base + k >= a.n) continue;
        const uint8_t st = replay_classify(a, base + k, slot[k], c[k], e[k]);
        a.state[base + k] = st;
        pending |= st == RP_PENDING;
    }
    if (__syncthreads_or(pending) && threadIdx.x == 0) *pending_flag = 1u;
}
__global__ void __launch_bounds__(256) replay_advance_kernel(ReplayArgs a) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    replay_advance_warp(a, blockIdx.x * blockDim.x + threadIdx.x);
}
__global__ void __launch_bounds__(256) replay_hash_clear_kernel(ReplayArgs a, const uint32_t *pending_flag) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    if (*pending_flag == 0u) return;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i <= a.mask; i += gridDim.x * blockDim.x) a.table[i] = kHashEmpty;
}
__global__ void __launch_bounds__(256) replay_hash_insert_kernel(ReplayArgs a, const uint32_t *pending_flag) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    if (*pending_flag == 0u) return;
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    replay_hash_insert_warp(a, p, p < a.n && a.state[p] != RP_NOPART);
}
__global__ void __launch_bounds__(256) replay_finish_kernel(ReplayArgs a) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    replay_finish_warp(a, blockIdx.x * blockDim.x + threadIdx.x);
}
// All of the above for one tile, by the CTA that holds it (n <= kScanTile, 256 threads).
__device__ __forceinline__ void replay_one_cta(const ReplayArgs &a, SegMax *part) {
    const uint32_t tid = threadIdx.x;
    uint32_t slot[4];
    uint64_t c[4], e[4];
    replay_tile<true>(a, tid * 4u, 0ull, slot, c, e, part);
    bool pending = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (tid * 4u + k >= a.n) continue;
        const uint8_t st = replay_classify(a, tid * 4u + k, slot[k], c[k], e[k]);
        a.state[tid * 4u + k] = st;
        pending |= st == RP_PENDING;
    }
    const bool any_pending = __syncthreads_or(pending); // also: every verdict and next `last` is written
    for (uint32_t p = tid; p < kScanTile; p += 256u) replay_advance_warp(a, p);
    if (any_pending) {
        for (uint32_t i = tid; i <= a.mask; i += 256u) a.table[i] = kHashEmpty;
        __syncthreads();
        for (uint32_t p = tid; p < kScanTile; p += 256u) replay_hash_insert_warp(a, p, p < a.n && a.state[p] != RP_NOPART);
    }
    __syncthreads(); // clears before marks, inserts before look-ups
    for (uint32_t p = tid; p < kScanTile; p += 256u) replay_finish_warp(a, p);
}

// --- the whole sort in one CTA, for batches of up to 1024 packets ----------------------
// Same three steps per digit as above, but keys and indices ping-pong between shared-memory buffers
// and all passes run inside one launch: a 128-packet batch pays one launch instead of six.
constexpr uint32_t kSmallMax = 1024;
// Send counters in the same launch (counter_out != nullptr): with one CTA a barrier separates the reads of
// the peers' counters from their advance, which takes two launches for larger batches.
// The replay window of a small batch can follow in the same launch as well (replay_last != nullptr).
struct SmallCounters {
    uint64_t *send_counter; // [max_slots]
    uint64_t *counter_out;  // per packet
    uint32_t max_slots;
};
__global__ void __launch_bounds__(kSortThreads) group_small_kernel(SortKeySrc src, uint32_t n, uint32_t passes,
                                                                   uint32_t digit_bits, uint32_t *keys_out,
                                                                   uint32_t *vals_out, SmallCounters sc, ReplayArgs rp) {
    let_next_kernel_start();    // seal side: the seal launch behind may take its place already
    wait_for_kernel_in_front(); // open side: statuses and counters come from the open launch in front
    constexpr uint32_t TILES = kSmallMax / kSortThreads; // 4
    __shared__ uint32_t kbuf[2][kSmallMax], vbuf[2][kSmallMax];
    __shared__ uint32_t cur[kSortWarps][kMaxBins];
    __shared__ uint32_t base_of[kMaxBins];
    __shared__ uint32_t warp_sum[kSortWarps];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bins = 1u << digit_bits;
    const uint32_t begin = warp * (32 * TILES);
    const uint32_t lt = (1u << lane) - 1u;
    if (n <= kSortThreads) {
        // One packet per thread at most (the upstream batch is 128): the place of a packet is the number of
        // packets with a lower key, or the same key and a lower index.  n broadcast reads from shared memory
        // instead of two radix passes with five barriers each.
        const uint32_t mine = tid < n ? slot_key(src, tid) : 0xffffffffu;
        kbuf[0][tid] = mine;
        __syncthreads();
        uint32_t place = 0;
        for (uint32_t j = 0; j < n; j++) {
            const uint32_t other = kbuf[0][j];
            place += (other < mine || (other == mine && j < tid)) ? 1u : 0u;
        }
        if (tid < n) {
            keys_out[place] = mine;
            vals_out[place] = tid;
        }
        __syncthreads();
        passes = 0;
    }
    for (uint32_t p = 0; p < passes; p++) {
        const uint32_t shift = p * digit_bits;
        const uint32_t *kin = kbuf[p & 1], *vin = vbuf[p & 1];
        uint32_t *kout = kbuf[(p + 1) & 1], *vout = vbuf[(p + 1) & 1];
        for (uint32_t d = tid; d < kSortWarps * kMaxBins; d += kSortThreads) (&cur[0][0])[d] = 0;
        __syncthreads();
        uint32_t key[TILES], val[TILES];
#pragma unroll
        for (uint32_t t = 0; t < TILES; t++) {
            const uint32_t i = begin + t * 32 + lane;
            const bool have = i < n;
            key[t] = have ? (p == 0 ? slot_key(src, i) : kin[i]) : 0xffffffffu;
            val[t] = have ? (p == 0 ? i : vin[i]) : 0u;
            warp_hist_add(cur[warp], (key[t] >> shift) & (bins - 1), have);
        }
        __syncthreads();
        {   // digit bases: exclusive prefix over the digit totals, two digits per thread
            const uint32_t d0 = 2 * tid, d1 = 2 * tid + 1;
            uint32_t v0 = 0, v1 = 0;
            for (uint32_t w = 0; w < kSortWarps; w++) {
                if (d0 < bins) v0 += cur[w][d0];
                if (d1 < bins) v1 += cur[w][d1];
            }
            uint32_t incl = v0 + v1;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= (uint32_t)o) incl += t;
            }
            if (lane == 31) warp_sum[warp] = incl;
            __syncthreads();
            uint32_t before = 0;
            for (uint32_t w = 0; w < warp; w++) before += warp_sum[w];
            const uint32_t excl = before + incl - (v0 + v1);
            if (d0 < bins) base_of[d0] = excl;
            if (d1 < bins) base_of[d1] = excl + v0;
        }
        __syncthreads();
        for (uint32_t d = tid; d < bins; d += kSortThreads) {
            uint32_t run = base_of[d];
#pragma unroll
            for (uint32_t w = 0; w < kSortWarps; w++) {
                const uint32_t c = cur[w][d];
                cur[w][d] = run;
                run += c;
            }
        }
        __syncthreads();
        const bool final_pass = p + 1 == passes;
        uint32_t *mine = cur[warp];
#pragma unroll
        for (uint32_t t = 0; t < TILES; t++) {
            const bool have = begin + t * 32 + lane < n;
            const uint32_t digit = have ? ((key[t] >> shift) & (bins - 1)) : 0xffffffffu;
            const uint32_t peers = __match_any_sync(0xffffffffu, digit);
            const uint32_t rank = __popc(peers & lt);
            uint32_t pos = 0;
            if (have) pos = mine[digit] + rank;
            __syncwarp();
            if (have && rank == 0) mine[digit] += __popc(peers);
            __syncwarp();
            if (have) {
                if (final_pass) {
                    keys_out[pos] = key[t];
                    vals_out[pos] = val[t];
                } else {
                    kout[pos] = key[t];
                    vout[pos] = val[t];
                }
            }
        }
        __syncthreads();
    }
    if (rp.replay_last != nullptr) { // the barrier that closed the last pass makes the sorted arrays visible
        __shared__ SegMax part[8];
        replay_one_cta(rp, part);
    }
    if (sc.counter_out == nullptr) return;
    uint64_t next[TILES];
    uint32_t tail_slot[TILES];
#pragma unroll
    for (uint32_t t = 0; t < TILES; t++) {
        const uint32_t j = t * kSortThreads + tid;
        tail_slot[t] = 0xffffffffu;
        if (j >= n) continue;
        const uint32_t slot = keys_out[j];
        if (slot >= sc.max_slots) continue;
        const uint32_t rank = j - run_start(keys_out, j);
        const uint64_t base = sc.send_counter[slot];
        sc.counter_out[vals_out[j]] = saturating_counter(base, rank);
        if (j + 1 == n || keys_out[j + 1] != slot) {
            tail_slot[t] = slot;
            next[t] = saturating_counter(base, rank + 1);
        }
    }
    __syncthreads();
#pragma unroll
    for (uint32_t t = 0; t < TILES; t++)
        if (tail_slot[t] != 0xffffffffu) sc.send_counter[tail_slot[t]] = next[t];
}

// --- scheduling order by length class (mixed packet sizes) ------------------------------
// Packets with the same number of 64-byte cipher blocks end up next to each other so that
// the lanes of a seal/open warp finish together; classes in falling order of length.  Order inside a class does
// not matter.
constexpr uint32_t kLenBins = 1026;
__device__ __forceinline__ uint32_t len_bin(uint32_t len, bool open_side) {
    uint32_t body = open_side ? (len >= 32u ? len - 32u : 0u) : len;
    uint32_t blocks = (body + 63u) >> 6;
    return blocks > kLenBins - 1 ? kLenBins - 1 : blocks;
}
// Real traffic has a handful of sizes, so nearly all packets fall into three or four bins: atomics straight on
// the global bins serialise there (100,000 warp-level atomics on three addresses took 50 us per million
// packets).  A CTA counts its tile of 2048 packets in shared memory first (lanes with equal bins elect a leader)
// and touches a global bin once per tile; the scatter reserves a range per (tile, bin) the same way and ranks
// inside the range with the shared counters.
constexpr uint32_t kLenItems = 8; // packets per thread
constexpr uint32_t kLenTile = 256 * kLenItems;
__device__ __forceinline__ uint32_t len_tile_count(const uint32_t *len, uint32_t n, int open_side, uint32_t *h,
                                                   uint32_t (&bin)[kLenItems], uint32_t (&rank)[kLenItems]) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t first = blockIdx.x * kLenTile + threadIdx.x;
    for (uint32_t d = threadIdx.x; d < kLenBins; d += 256) h[d] = 0;
    __syncthreads();
#pragma unroll
    for (uint32_t k = 0; k < kLenItems; k++) {
        const uint32_t i = first + k * 256u;
        const bool have = i < n;
        bin[k] = have ? len_bin(len[i], open_side) : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, bin[k]);
        const int leader = __ffs(peers) - 1;
        uint32_t at = 0;
        if (have && leader == (int)lane) at = atomicAdd(&h[bin[k]], __popc(peers));
        rank[k] = __shfl_sync(0xffffffffu, at, leader) + __popc(peers & ((1u << lane) - 1u)); // position inside the tile's bin
    }
    __syncthreads();
    return first;
}
__global__ void __launch_bounds__(256) len_hist_kernel(const uint32_t *len, uint32_t n, int open_side,
                                                       uint32_t *bins) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ uint32_t h[kLenBins];
    uint32_t bin[kLenItems], rank[kLenItems];
    len_tile_count(len, n, open_side, h, bin, rank);
    for (uint32_t d = threadIdx.x; d < kLenBins; d += 256)
        if (h[d]) atomicAdd(&bins[d], h[d]);
}
__global__ void __launch_bounds__(256) len_scatter_kernel(const uint32_t *len, uint32_t n, int open_side,
                                                          uint32_t *bins, uint32_t *order) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ uint32_t h[kLenBins];
    uint32_t bin[kLenItems], rank[kLenItems];
    const uint32_t first = len_tile_count(len, n, open_side, h, bin, rank);
    for (uint32_t d = threadIdx.x; d < kLenBins; d += 256)
        if (h[d]) h[d] = atomicAdd(&bins[d], h[d]); // the tile's range in bin d starts here
    __syncthreads();
#pragma unroll
    for (uint32_t k = 0; k < kLenItems; k++) {
        const uint32_t i = first + k * 256u;
        // longest class first: the launch then ends with the short packets, whose CTAs take a tenth of the time of
        // the long ones, instead of a last, half-empty wave of the longest
        if (i < n) order[n - 1u - (h[bin[k]] + rank[k])] = i;
    }
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

// elements per lane: the smallest power of two that keeps the chunk count at or below max_chunks
uint32_t tiles_for(uint32_t n, uint32_t max_chunks) {
    uint32_t tiles = 1;
    while (tiles < kMaxTiles && (n + kSortThreads * tiles - 1) / (kSortThreads * tiles) > max_chunks) tiles <<= 1;
    return tiles;
}
uint32_t chunks_for(uint32_t n, uint32_t tiles) { return (n + kSortThreads * tiles - 1) / (kSortThreads * tiles); }

struct SortBuffers {
    uint32_t *keys_a, *keys_b; // the sorted keys end up in keys_b
    uint32_t *vals_a, *order;  // the sorted packet indices end up in order
    uint32_t *hist;            // [bins * chunks]
    uint32_t *totals;          // [bins]
};

template <uint32_t TILES>
void sort_pass(const SortKeySrc &src, const uint32_t *kin, const uint32_t *vin, uint32_t n, uint32_t shift,
               uint32_t bins, uint32_t chunks, const SortBuffers &sb, uint32_t *kout, uint32_t *vout, cudaStream_t s) {
    launch_kernel(n <= dependent_launch_up_to(), radix_hist_kernel<TILES>, dim3(chunks), dim3(kSortThreads), s, src, kin,
        n, shift, bins, chunks, sb.hist);
    launch_kernel(n <= dependent_launch_up_to(), radix_rowscan_kernel,
        dim3((bins * 32 + kSortThreads - 1) / kSortThreads), dim3(kSortThreads), s, sb.hist, bins, chunks, sb.totals);
    launch_kernel(n <= dependent_launch_up_to(), radix_scatter_kernel<TILES>, dim3(chunks), dim3(kSortThreads), s, src,
        kin, vin, n, shift, bins, chunks, sb.hist, sb.totals, kout, vout);
}

// Stable sort of packet indices 0..n-1 by key.  Returns the number of kernel launches.
uint32_t group_sort(const SortKeySrc &src, uint32_t n, uint32_t max_chunks, const SortBuffers &sb, cudaStream_t s) {
    const SortPlan plan = plan_for(src.max_slots);
    if (n <= kSmallMax) {
        launch_after_kernel(group_small_kernel, dim3(1), dim3(kSortThreads), s, src, n, plan.passes, plan.digit_bits,
            sb.keys_b, sb.order, SmallCounters{nullptr, nullptr, 0}, ReplayArgs{});
        return 1;
    }
    const uint32_t bins = 1u << plan.digit_bits;
    const uint32_t tiles = tiles_for(n, max_chunks);
    const uint32_t chunks = chunks_for(n, tiles);
    // ping-pong so that the last pass lands in (keys_b, order)
    uint32_t *kbuf[2] = {sb.keys_b, sb.keys_a};
    uint32_t *vbuf[2] = {sb.order, sb.vals_a};
    const uint32_t *kin = nullptr, *vin = nullptr;
    for (uint32_t p = 0; p < plan.passes; p++) {
        const uint32_t shift = p * plan.digit_bits;
        const uint32_t o = (plan.passes - 1 - p) & 1u;
        switch (tiles) {
        case 1: sort_pass<1>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        case 2: sort_pass<2>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        case 4: sort_pass<4>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        case 8: sort_pass<8>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        case 16: sort_pass<16>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        default: sort_pass<32>(src, kin, vin, n, shift, bins, chunks, sb, kbuf[o], vbuf[o], s); break;
        }
        kin = kbuf[o];
        vin = vbuf[o];
    }
    return 3 * plan.passes;
}

} // namespace

// words of histogram scratch a batch of max_pkts packets needs
uint32_t group_sort_chunks(uint32_t max_pkts) {
    const uint32_t worst = chunks_for(max_pkts, kMaxTiles);
    return (worst > kBatchMaxChunks ? worst : kBatchMaxChunks) + 1; // + one row of digit totals
}

// Sorts packet indices 0..n-1 by keypair slot, stable.  Leaves the sorted keys in
// dev.keys_tmp (second half) and the packet indices in dev.order.
cudaError_t launch_group_by_slot(bnk_batch *b, uint32_t n, bool only_status_ok, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    bnk_ctx *ctx = b->ctx;
    DeviceBatch &d = b->dev;
    SortKeySrc src{d.slot, d.status, ctx->cfg.max_keypairs, only_status_ok ? 1 : 0};
    SortBuffers sb{d.keys_tmp, d.keys_tmp + b->max_pkts, d.order_tmp, d.order, d.hist + kMaxBins, d.hist};
    ctx->launches += group_sort(src, n, kBatchMaxChunks, sb, s);
    return cudaGetLastError();
}

cudaError_t launch_assign_counters(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    if (n <= kSmallMax) { // sort and counters in one launch
        bnk_ctx *ctx = b->ctx;
        DeviceBatch &d = b->dev;
        const SortPlan plan = plan_for(ctx->cfg.max_keypairs);
        launch_after_kernel(group_small_kernel, dim3(1), dim3(kSortThreads), s,
            SortKeySrc{d.slot, d.status, ctx->cfg.max_keypairs, 0}, n, plan.passes, plan.digit_bits,
            d.keys_tmp + b->max_pkts, d.order, SmallCounters{ctx->kt.send_counter, d.counter, ctx->cfg.max_keypairs},
            ReplayArgs{});
        ctx->launches += 1;
        return cudaGetLastError();
    }
    cudaError_t e = launch_group_by_slot(b, n, false, s);
    if (e != cudaSuccess) return e;
    DeviceBatch &d = b->dev;
    launch_kernel(n <= dependent_launch_up_to(), assign_counters_kernel, dim3((n + 255) / 256), dim3(256), s,
        d.keys_tmp + b->max_pkts, d.order, n, b->ctx->cfg.max_keypairs, b->ctx->kt.send_counter, d.counter);
    launch_kernel(n <= dependent_launch_up_to(), advance_counters_kernel, dim3((n + 255) / 256), dim3(256), s,
        d.keys_tmp + b->max_pkts, n, b->ctx->cfg.max_keypairs, b->ctx->kt.send_counter);
    b->ctx->launches += 2;
    return cudaGetLastError();
}

uint32_t replay_scan_tiles(uint32_t max_pkts) { return (max_pkts + kScanTile - 1) / kScanTile; }
uint32_t replay_hash_capacity(uint32_t max_pkts) {
    uint32_t cap = 1024;
    while (cap < 2u * max_pkts && cap < 0x80000000u) cap <<= 1;
    return cap;
}
static ReplayArgs replay_args(bnk_batch *b, uint32_t n) {
    bnk_ctx *ctx = b->ctx;
    DeviceBatch &d = b->dev;
    uint32_t cap = 1024;
    while (cap < 2u * n) cap <<= 1; // at most half full
    ReplayArgs a{};
    a.keys = d.keys_tmp + b->max_pkts;
    a.order = d.order;
    a.n = n;
    a.max_slots = ctx->cfg.max_keypairs;
    a.ring_blocks = ctx->cfg.replay_ring_blocks;
    a.replay_last = ctx->kt.replay_last;
    a.replay_next = ctx->kt.replay_next;
    a.replay_ring = ctx->kt.replay_ring;
    a.counter = d.counter;
    a.status = d.status;
    a.sorted_counter = d.sorted_counter;
    a.state = d.replay_state;
    a.table = d.replay_hash;
    a.mask = cap - 1;
    return a;
}
// Grouping and replay window of a small batch in one launch, for after the open kernel.
bool replay_is_one_launch(uint32_t n) { return n <= kSmallMax; }
cudaError_t launch_group_and_replay(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    bnk_ctx *ctx = b->ctx;
    DeviceBatch &d = b->dev;
    const SortPlan plan = plan_for(ctx->cfg.max_keypairs);
    launch_after_kernel(group_small_kernel, dim3(1), dim3(kSortThreads), s,
        SortKeySrc{d.slot, d.status, ctx->cfg.max_keypairs, 0}, n, plan.passes, plan.digit_bits,
        d.keys_tmp + b->max_pkts, d.order, SmallCounters{nullptr, nullptr, 0}, replay_args(b, n));
    ctx->launches += 1;
    return cudaGetLastError();
}
// Expects launch_group_by_slot(b, n, false, ...) to have completed before this point of stream s.
cudaError_t launch_replay(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    const ReplayArgs a = replay_args(b, n);
    const uint32_t tiles = (n + kScanTile - 1) / kScanTile, grid = (n + 255) / 256;
    uint32_t *flag = d.replay_tile_head + replay_scan_tiles(b->max_pkts);
    launch_kernel(n <= dependent_launch_up_to(), replay_scan_tiles_kernel, dim3(tiles), dim3(256), s, a,
        d.replay_tile_head, d.replay_tile_max, flag);
    launch_kernel(n <= dependent_launch_up_to(), replay_scan_carry_kernel, dim3(1), dim3(1024), s, d.replay_tile_head,
        d.replay_tile_max, tiles, d.replay_tile_carry);
    launch_kernel(n <= dependent_launch_up_to(), replay_classify_kernel, dim3(tiles), dim3(256), s, a,
        d.replay_tile_carry, flag);
    launch_kernel(n <= dependent_launch_up_to(), replay_advance_kernel, dim3(grid), dim3(256), s, a);
    launch_kernel(n <= dependent_launch_up_to(), replay_hash_clear_kernel, dim3(b->ctx->sm_count * 4), dim3(256), s, a, flag);
    launch_kernel(n <= dependent_launch_up_to(), replay_hash_insert_kernel, dim3(grid), dim3(256), s, a, flag);
    launch_kernel(n <= dependent_launch_up_to(), replay_finish_kernel, dim3(grid), dim3(256), s, a);
    b->ctx->launches += 7;
    return cudaGetLastError();
}

cudaError_t launch_length_order(bnk_batch *b, uint32_t n, const uint32_t *len, bool open_side, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    cudaError_t e = cudaMemsetAsync(d.counters32, 0, kLenBins * sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    launch_kernel(n <= dependent_launch_up_to(), len_hist_kernel, dim3((n + kLenTile - 1) / kLenTile), dim3(256), s, len,
        n, open_side ? 1 : 0, d.counters32);
    launch_kernel(n <= dependent_launch_up_to(), exclusive_scan_kernel, dim3(1), dim3(1024), s, d.counters32, kLenBins);
    launch_kernel(n <= dependent_launch_up_to(), len_scatter_kernel, dim3((n + kLenTile - 1) / kLenTile), dim3(256), s,
        len, n, open_side ? 1 : 0, d.counters32, d.len_order);
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
constexpr uint32_t kNoAllocMaxChunks = 31; // (31 chunk columns + 1 row of totals) * 512 bins = the 16384-word histogram region
constexpr size_t kNoAllocWords = (size_t)5 * kNoAllocMaxPkts + 16384; // 384 KiB
static_assert((size_t)kMaxBins * (kNoAllocMaxChunks + 1) <= 16384, "histogram region too small");

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
    SortKeySrc src{dev_slot, nullptr, ctx->cfg.max_keypairs, 0};
    SortBuffers sb{keys_a, keys_b, vals_a, order, hist + kMaxBins, hist};
    const uint32_t sort_launches = group_sort(src, n, kNoAllocMaxChunks, sb, s);
    launch_kernel(n <= dependent_launch_up_to(), assign_counters_kernel, dim3((n + 255) / 256), dim3(256), s, keys_b,
        order, n, ctx->cfg.max_keypairs, ctx->kt.send_counter, dev_counter);
    launch_kernel(n <= dependent_launch_up_to(), advance_counters_kernel, dim3((n + 255) / 256), dim3(256), s, keys_b, n,
        ctx->cfg.max_keypairs, ctx->kt.send_counter);
    ctx->launches += sort_launches + 2;
    if ((e = cudaGetLastError()) != cudaSuccess) return noalloc_fail(ctx, BNK_ECUDA, "kernel launch", e);
    return BNK_SUCCESS;
}
