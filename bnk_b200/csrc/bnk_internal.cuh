// Internal declarations shared by the translation units of libbnkgpu.so.
// Nothing here is part of the C ABI (that is include/bnk_gpu.h).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <vector>

#include "../../include/bnk_gpu.h"

// ---------------------------------------------------------------------------
// Device-resident tables of one context (one GPU).  All per-peer mutable state
// lives here, indexed by keypair slot, so that peers shard across GPUs with no
// exchange: keys, send counter, replay window.
// ---------------------------------------------------------------------------
struct KeypairTables {
    uint32_t *send_keys;    // [max_keypairs][8] little-endian words
    uint32_t *recv_keys;    // [max_keypairs][8]
    uint32_t *remote_index; // [max_keypairs] receiver index written into sealed headers
    uint64_t *send_counter; // [max_keypairs] next nonce to hand out
    uint64_t *replay_last;  // [max_keypairs] highest counter accepted
    uint64_t *replay_next;  // [max_keypairs] scratch: the value replay_last takes after the batch in flight
    uint64_t *replay_ring;  // [max_keypairs][ring_blocks] RFC 6479 bitmap ring
    uint32_t *allowed_ip;   // [max_keypairs] the peer's tunnel address, host order (0 = none)
    uint8_t *valid;         // [max_keypairs] 1 while the slot holds keys that bnk_keypair_set* put there
    // receiver index -> slot: open addressing, key = 1<<32 | index (0 = empty, 2<<32 = deleted)
    uint64_t *index_keys;   // [index_slots]
    uint32_t *index_vals;   // [index_slots]
    uint32_t index_slots;   // power of two
    // source address -> peer id (Bind.byAddr): open addressing over 32-byte entries
    struct AddrEntry {
        uint64_t hi, lo;   // the 16 address bytes as two little-endian words
        uint32_t port;     // port | 1<<16 when live, 2<<16 when deleted, 0 when empty
        uint32_t peer;
        uint64_t pad;
    };
    AddrEntry *addr_tab;    // [addr_slots]
    uint32_t addr_slots;    // power of two
};

// Flattened, indexed ACL and the reply-flow table (filter_kernels.cu).
struct FilterTables {
    // rule index: open-addressing table keyed by (prefix_len, masked address)
    uint64_t *rule_keys;   // [rule_slots] 0 = empty; else (1<<40 | len<<32 | masked addr)
    uint2 *rule_span;      // [rule_slots] (first entry, entry count) into rule_entries
    uint64_t *rule_entries; // packed (proto<<32 | first<<16 | last)
    uint32_t rule_slots;   // power of two (0 when no tuples)
    uint64_t len_mask;     // bit L set when some tuple has prefix length L (bits 0..32)
    int enforce;
    // flow table, one open-addressing region per protocol class (tcp, udp, icmp).  Every class has two
    // regions, [class][half][flow_capacity]; flow_half[class] says which one is in use, the other one is all
    // FLOW_EMPTY and receives the surviving entries when the class is compacted (filter_flows_compact).
    uint64_t *flow_keys;   // [3][2][flow_capacity] FLOW_EMPTY = all ones
    long long *flow_exp;   // [3][2][flow_capacity] expiry in unix ns; FLOW_DEAD = deleted
    uint32_t flow_capacity; // power of two
    uint8_t flow_half[3];
    unsigned long long *flow_live;  // device control block (FlowCtl): live entries (Go's len(f.flows)) and more
    long long *flow_special_exp;    // [3] entry for the one key that equals FLOW_EMPTY
    int *flow_error;       // counts the inserts that found no free slot
};
// region of protocol class `cls` that is in use
__host__ __device__ inline size_t flow_region(const FilterTables &ft, int cls) {
    return ((size_t)cls * 2 + ft.flow_half[cls]) * ft.flow_capacity;
}
// What a batch's filter work reports back to the host next to the packets (pinned, one per batch).
struct FlowReport {
    int error;            // inserts that found no free slot, since the table was last cleared
    uint32_t used[3];     // slots of the class's region that hold a key, live or deleted
    uint32_t dead[3];     // of those, deleted ones (reclaimed by compaction)
};

struct bnk_ctx {
    bnk_cfg cfg;
    int device;
    KeypairTables kt;
    FilterTables ft;
    cudaStream_t admin_stream;
    cudaEvent_t timer_start;
    int sm_count;
    uint64_t host_direct_bytes; // batches up to this ring extent run on the caller's pinned buffers (BNK_HOST_DIRECT_BYTES)
    std::atomic<int> direct_in_flight{0}; // batches whose last submit ran that way and has not been waited for
    int aead_mode; // 0 = choose by batch size, 1 = always thread per packet, 2 = always warp per packet (BNK_AEAD_KERNEL)
    uint32_t aead_side_stream_from; // batches of at least this many packets run seal/open on the low-priority stream (BNK_AEAD_SIDE_STREAM_FROM; 0 = never)
    int prio_low, prio_high;        // stream priority range of the device
    std::atomic<uint64_t> launches;
    std::mutex mu;
    std::string last_error;
    // Submits hold this shared while they queue their work; whoever changes what running kernels of other
    // batches could observe half-done (flow-table compaction) or swaps tables that launches capture by value
    // (rule table) holds it exclusively.
    std::shared_mutex submit_mu;
    std::vector<bnk_batch *> batches;       // every live batch of the context (guarded by mu)
    std::atomic<uint32_t> flow_dead_hint[3]; // deleted entries per class as last reported by the device
    std::atomic<int> flow_errors_seen;       // failed inserts already reported to a caller as BNK_EFULL
    // rule table: two device buffer sets, the one not in use receives the next upload
    struct RuleSet {
        uint64_t *keys = nullptr;
        uint2 *span = nullptr;
        uint64_t *entries = nullptr;
        size_t slots_cap = 0, entries_cap = 0;
        std::vector<cudaEvent_t> in_use; // recorded on every batch stream when the set was retired
    } rule_set[2];
    int rule_cur = 0;
    std::mutex acl_mu; // one bnk_acl_set at a time
    std::vector<KeypairTables::AddrEntry> addr_host; // host shadow of kt.addr_tab
    std::vector<uint64_t> index_keys_host; // host shadow of kt.index_keys (updates are rare: one per handshake)
    std::vector<uint32_t> index_vals_host; // host shadow of kt.index_vals
    uint32_t index_live, index_dead;       // entries of the receiver-index table in use / deleted but not yet reclaimed
    uint32_t addr_live, addr_dead;         // the same for the source-address table
};

struct DeviceBatch {
    uint8_t *ring;
    uint32_t *off, *len, *slot, *out_len;
    uint64_t *counter;
    uint8_t *status;
    uint8_t *src_addr;    // [max_pkts][BNK_SRC_ADDR_STRIDE]
    // scratch for grouping packets by keypair slot (group_kernels.cu)
    uint32_t *order;      // [max_pkts] packet indices, stable by slot
    uint32_t *order_tmp;  // [max_pkts]
    uint32_t *keys_tmp;   // [2][max_pkts] radix keys ping-pong
    // scratch of the replay window in its scan form (group_kernels.cu)
    uint64_t *sorted_counter;    // [max_pkts] counters in grouped order
    uint8_t *replay_state;       // [max_pkts] verdict per grouped position
    uint32_t *replay_hash;       // [replay_hash_capacity(max_pkts)] lowest position per (peer, counter)
    uint32_t *replay_tile_head;  // [tiles + 1] a run starts inside the tile; last entry: some packet needs the hash
    uint64_t *replay_tile_max;   // [tiles]
    uint64_t *replay_tile_carry; // [tiles]
    uint32_t *hist;       // [512 * chunks] digit-major histograms
    uint32_t *len_order;  // [max_pkts] packet indices ordered by length class
    uint32_t *counters32; // small scratch (bins)
    bnk_gso_super *gso;   // [max_pkts] super-packet descriptors of a GSO split
};

struct bnk_batch {
    bnk_ctx *ctx;
    uint32_t max_pkts;
    uint64_t ring_bytes;
    bnk_batch_view host; // pinned
    DeviceBatch dev;
    cudaStream_t stream;
    cudaStream_t aux_stream;   // grouping work that can run beside the open kernel
    // The seal/open launches of a large batch go to a stream of their own with the lowest priority, the short
    // kernels around them (grouping, counters, replay window, length classes) stay on `stream` / `aux_stream`
    // with the highest: a large seal/open launch fills every SM for hundreds of microseconds, and the short
    // kernels of the NEXT batch would otherwise get no SM until its last wave.  With priorities their CTAs take
    // the places seal/open CTAs leave as they retire, so the chain of one batch really runs beside the seal/open
    // kernel of another.
    cudaStream_t aead_stream;
    cudaEvent_t ev_aead_go, ev_aead_done;
    cudaEvent_t ev_fork, ev_join;
    cudaEvent_t k_begin, k_end, t_end, a_begin, a_end;
    bool in_flight;
    bool dev_stale; // a submit ran on the host arrays: the device copies of ring and descriptors are behind
    bool direct_counted; // this batch is one of ctx->direct_in_flight
    bool kernel_timed;
    bool aead_timed;
    bnk_gso_super *h_gso; // pinned staging for the super-packet descriptors
    uint8_t *h_desc, *d_desc; // one slab per side: off | len | slot | counter | out_len | status (npad entries each), then the ring
    uint32_t npad;
    size_t desc_room;  // bytes of the descriptor slab in front of the ring (same on both sides)
    bool joint_copy;   // descriptors and ring move as one copy
    FlowReport *h_flow; // pinned copy of the flow table's state after the batch's filter work
    bool stats_pending; // the last submit was made with BNK_F_STATS
    bool flow_reported; // the last submit queued a copy of the flow table's state into h_flow
    bnk_batch_stats *h_stats; // pinned; written by the tally kernel
    unsigned long long *d_stats; // device accumulators of the tally kernel (zero between launches)
    cudaEvent_t ev_fence; // orders this batch's stream against table maintenance on another stream
    // Set by the submit queue around one submit: the kernels of that submit start behind order_wait and
    // order_record is recorded behind the last of them (copies on either side stay free to overlap).
    cudaEvent_t order_wait, order_record;
};

// Small batches are two dependent launches with little work in each, so the gap between them counts.  A kernel
// launched through launch_after_kernel may be scheduled while the kernel in front of it on the stream is still
// running (programmatic dependent launch) and must call wait_for_kernel_in_front() before it touches anything
// that kernel writes: the wait ends when that kernel has finished and its writes are visible.  The kernel in front
// calls let_next_kernel_start() first thing, which allows the next one to be placed on the SMs (where it sits in
// its wait) as soon as all of this kernel's CTAs are resident; that hides the launch latency of the second kernel
// behind the first.  Launched the ordinary way, or with nothing of the kind behind it, both calls do nothing.
__device__ __forceinline__ void wait_for_kernel_in_front() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;"); }
// The chains of short kernels around a large batch (grouping, counters, replay window, length classes) are
// launched the same way while they are short: measured on 96,256 packets both sides of the pipeline got 7 % faster,
// on 1,048,576 packets 1 % slower.  With several large batches in flight it costs: CTAs that sit in their wait hold
// SM slots that the seal/open kernel of another batch could use (four batches of 262,144 mixed packets: 1.05 ms
// per step with dependent launches, 0.93 without).  Hence the limit.
inline uint32_t dependent_launch_up_to() {
    static const uint32_t v = [] {
        const char *m = getenv("BNK_DEPENDENT_LAUNCH_UP_TO"); // tuning aid
        return m ? (uint32_t)strtoul(m, nullptr, 0) : (1u << 17);
    }();
    return v;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_after_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// the same launch with the ordinary full dependency when `dependent` is false
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    if (dependent) return launch_after_kernel(kernel, grid, block, s, args...);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---------------------------------------------------------------------------
// Kernel launchers (each defined next to its kernels).  All are asynchronous on
// `s` and return the cudaError_t of the launch.
// ---------------------------------------------------------------------------
struct AeadArgs {
    uint8_t *ring;
    const uint32_t *off;
    const uint32_t *len;
    const uint32_t *slot;
    uint64_t *counter;
    uint32_t *out_len;
    uint8_t *status;
    const uint32_t *keys;         // send keys (seal) or receive keys (open)
    const uint32_t *remote_index; // seal only
    const uint8_t *valid;         // per keypair slot: keys present
    const uint32_t *order;        // optional scheduling permutation, may be null
    uint32_t n;
    uint32_t mtu;
    uint32_t max_slots;
    uint64_t ring_bytes;
};
cudaError_t launch_seal(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx);
cudaError_t launch_open(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx);

// group_kernels.cu
cudaError_t launch_group_by_slot(bnk_batch *b, uint32_t n, bool only_status_ok, cudaStream_t s);
cudaError_t launch_assign_counters(bnk_batch *b, uint32_t n, cudaStream_t s);
cudaError_t launch_replay(bnk_batch *b, uint32_t n, cudaStream_t s);
bool replay_is_one_launch(uint32_t n); // small batches: grouping and walk fit one CTA
cudaError_t launch_group_and_replay(bnk_batch *b, uint32_t n, cudaStream_t s); // after the open kernel
cudaError_t launch_length_order(bnk_batch *b, uint32_t n, const uint32_t *len, bool open_side, cudaStream_t s);
uint32_t group_sort_chunks(uint32_t max_pkts);
uint32_t replay_scan_tiles(uint32_t max_pkts);     // tiles of the running-maximum scan
uint32_t replay_hash_capacity(uint32_t max_pkts);  // entries of the duplicate-counter table

// filter_kernels.cu
cudaError_t launch_filter_note(bnk_batch *b, uint32_t n, long long now_ns, cudaStream_t s);
cudaError_t launch_filter_check(bnk_batch *b, uint32_t n, long long now_ns, bool only_status_ok, cudaStream_t s);
cudaError_t filter_tables_alloc(bnk_ctx *ctx);
void filter_tables_free(bnk_ctx *ctx);
int filter_acl_upload(bnk_ctx *ctx, int enforce, const bnk_acl_tuple *tuples, size_t n);
cudaError_t filter_flows_clear(bnk_ctx *ctx, cudaStream_t s);
cudaError_t filter_flow_stats(bnk_ctx *ctx, uint64_t *live, uint32_t used[3], uint32_t dead[3]);
int filter_flows_export(bnk_ctx *ctx, bnk_flow_entry *out, size_t capacity, size_t *count);
int filter_flows_import(bnk_ctx *ctx, const bnk_flow_entry *entries, size_t n);
cudaError_t launch_flow_report(bnk_batch *b, cudaStream_t s); // copies the flow table's control block to b->h_flow
// Rebuilds the regions whose deleted entries have piled up; called by a submit that feeds the flow table,
// before it takes submit_mu.  Returns without doing anything in the common case.
cudaError_t filter_flows_maintain(bnk_batch *b, cudaStream_t s);
// Per-status packet counts and byte total of the first n packets, into b->h_stats (one launch).
cudaError_t launch_tally(bnk_batch *b, uint32_t n, cudaStream_t s);

// inner_kernels.cu
constexpr uint32_t kSlotNoKeypair = 0xfffffffeu; // demux found no keypair for the receiver index
cudaError_t launch_demux_index(bnk_batch *b, uint32_t n, const uint32_t *len, cudaStream_t s);
cudaError_t launch_inner_check(bnk_batch *b, uint32_t n, cudaStream_t s);
cudaError_t launch_classify(bnk_batch *b, uint32_t n, cudaStream_t s);
__host__ __device__ inline uint32_t addr_hash(uint64_t hi, uint64_t lo, uint32_t port) {
    uint64_t z = hi * 0x9e3779b97f4a7c15ull ^ (lo + 0xbf58476d1ce4e5b9ull) * 0x94d049bb133111ebull ^ ((uint64_t)port << 40);
    z ^= z >> 29;
    z *= 0xbf58476d1ce4e5b9ull;
    return (uint32_t)(z >> 32);
}
__host__ __device__ inline uint32_t index_hash(uint32_t index) {
    uint32_t z = index * 0x9e3779b1u;
    z ^= z >> 15;
    z *= 0x85ebca6bu;
    return z ^ (z >> 13);
}

// gso_kernels.cu
cudaError_t launch_gso_split(bnk_batch *b, uint32_t n_super, uint32_t n_pkts, cudaStream_t s);
