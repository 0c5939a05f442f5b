// ACL packet filter for sm_100a: the per-packet work of filter.Filter
// (internal/filter/filter.go of the reference) and acl.CompiledRule.Match
// (internal/acl/acl.go:149-172), one thread per packet.
//
// Rules.  The reference scans every rule for every packet.  The verdict is an OR
// over rules, so scan order is free; here the flattened allowances
// (prefix, proto, port range) are grouped by prefix and the groups are put in an
// open-addressing table keyed by (prefix length, masked address).  A packet probes
// the table once per prefix length that occurs in the rule set (a 33-bit mask) and
// scans only the allowances of prefixes that contain its source address.
//
// Flows.  Go's map[flowKey]time.Time becomes three open-addressing tables (tcp,
// udp, icmp) keyed by remote address | remote port | local port, claimed with a
// 64-bit compare-and-swap.  A deleted entry keeps its key with expiry FLOW_DEAD,
// which behaves like an absent key for every later lookup.  The live-entry count
// is kept exactly because the reference's expiry sweep depends on len(flows) > 4096.
// Go deletes map entries (filter.go:144, 202-208), so its map is bounded by the live
// flows; here deleted entries are counted per class, and once they fill a quarter of
// a class's region the surviving entries are re-inserted into the class's second,
// empty region and the two swap roles (filter_flows_maintain), between two batches.
#include <algorithm>
#include <climits>
#include <vector>

#include "bnk_internal.cuh"

namespace {

constexpr unsigned long long FLOW_EMPTY = ~0ull;
constexpr long long FLOW_DEAD = LLONG_MIN;      // the key is there, the entry is deleted
constexpr long long FLOW_FRESH = LLONG_MIN + 1; // expiry of a slot no key has used yet
__device__ __forceinline__ bool flow_absent(long long exp) { return exp <= FLOW_FRESH; }
constexpr long long TTL_UDP = 30ll * 1000000000ll;  // filter.go:19
constexpr long long TTL_TCP = 120ll * 1000000000ll; // filter.go:20
constexpr long long TTL_ICMP = 30ll * 1000000000ll; // filter.go:21
constexpr unsigned long long SWEEP_THRESHOLD = 4096; // filter.go:202

// small device-side control block behind FilterTables::flow_live
struct FlowCtl {
    unsigned long long live;   // len(f.flows)
    long long swept_at;        // `now` of the last completed sweep
    int swept_valid;           // nothing was written at another `now` since that sweep
    int sweep_now;             // decision for the sweep kernel of this batch
    FlowReport rep;            // overflow flag and per-class slot counts; copied to the host after a batch
    uint32_t moved;            // entries a compaction has re-inserted so far
};

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Slot of a rule key: the key is a 32-bit address and a prefix length, so a 32-bit finaliser (two 32-bit
// multiplies) spreads it; the 64-bit mixer above costs three times the instructions on a machine without a 64-bit
// multiplier, and the check kernel hashes once per prefix length and packet.
__host__ __device__ __forceinline__ uint32_t rule_hash(uint64_t key) {
    uint32_t x = (uint32_t)key ^ ((uint32_t)(key >> 32) * 0x9e3779b1u);
    x ^= x >> 16;
    x *= 0x85ebca6bu;
    x ^= x >> 13;
    x *= 0xc2b2ae35u;
    return x ^ (x >> 16);
}

__host__ __device__ __forceinline__ uint64_t rule_key(uint32_t len, uint32_t addr) {
    const uint32_t mask = len == 0 ? 0u : 0xffffffffu << (32 - len);
    return (1ull << 40) | ((uint64_t)len << 32) | (addr & mask);
}

struct Parsed {
    uint32_t src, dst;
    uint16_t sport, dport;
    uint8_t proto;
};

// filter.go:71-106.  `p` is 16-byte aligned (packets start 16 bytes into a 16-aligned slot).
__device__ __forceinline__ bool parse_ipv4(const uint8_t *p, uint32_t len, Parsed &out) {
    if (len < 20) return false;
    const uint4 w = *reinterpret_cast<const uint4 *>(p); // bytes 0..15
    if (((w.x & 0xffu) >> 4) != 4u) return false;
    const uint32_t ihl = (w.x & 0x0fu) * 4u;
    if (ihl < 20u || len < ihl) return false;
    out.proto = (uint8_t)((w.z >> 8) & 0xffu); // byte 9
    out.src = __byte_perm(w.w, 0, 0x0123);     // bytes 12..15, big-endian
    out.dst = __byte_perm(*reinterpret_cast<const uint32_t *>(p + 16), 0, 0x0123);
    out.sport = 0;
    out.dport = 0;
    const uint32_t body = len - ihl;
    if (out.proto == 6 || out.proto == 17) {
        if (body < 4) return false;
        const uint32_t ports = *reinterpret_cast<const uint32_t *>(p + ihl); // ihl is a multiple of 4
        out.sport = (uint16_t)(((ports & 0xffu) << 8) | ((ports >> 8) & 0xffu));
        out.dport = (uint16_t)((((ports >> 16) & 0xffu) << 8) | (ports >> 24));
        return true;
    }
    if (out.proto == 1) return body >= 1;
    return false;
}

__device__ __forceinline__ int proto_class(uint8_t proto) { return proto == 6 ? 0 : (proto == 17 ? 1 : 2); }
__device__ __forceinline__ long long flow_ttl(uint8_t proto) { // filter.go:108-117
    return proto == 6 ? TTL_TCP : (proto == 1 ? TTL_ICMP : TTL_UDP);
}
__device__ __forceinline__ unsigned long long flow_key(uint32_t remote, uint16_t rport, uint16_t lport) {
    return ((unsigned long long)remote << 32) | ((unsigned long long)rport << 16) | lport;
}

// any allowance matches?  acl.go:149-172 over the indexed table
// (Fetching the first slot of four prefix lengths before looking at any of them, to overlap the round trips, was
// measured: 10 % slower on configuration 3, where nearly half the packets match at one of the first lengths.)
__device__ __forceinline__ bool rules_allow(const FilterTables &ft, const Parsed &p) {
    if (ft.rule_slots == 0) return false;
    // longest prefixes first: acl.Compile emits /32s (acl.go:98), so a packet that some rule admits is most often
    // admitted at the first probe; any match allows, the order changes no verdict
    uint64_t lens = ft.len_mask;
    while (lens) {
        const uint32_t len = 63u - (uint32_t)__clzll((long long)lens);
        lens &= ~(1ull << len);
        const uint64_t key = rule_key(len, p.src);
        uint32_t h = rule_hash(key) & (ft.rule_slots - 1);
        for (uint32_t probe = 0; probe < ft.rule_slots; probe++) {
            const uint64_t k = ft.rule_keys[h];
            if (k == 0) break;
            if (k == key) {
                const uint2 span = ft.rule_span[h];
                for (uint32_t e = 0; e < span.y; e++) {
                    const uint64_t ent = ft.rule_entries[span.x + e];
                    if ((uint8_t)(ent >> 32) != p.proto) continue;
                    if (p.proto == 1) return true;
                    const uint16_t first = (uint16_t)(ent >> 16), last = (uint16_t)ent;
                    if (p.dport >= first && p.dport <= last) return true;
                }
                break;
            }
            h = (h + 1) & (ft.rule_slots - 1);
        }
    }
    return false;
}

// One atomic per group of lanes that add to the same counter at the same point of the code, instead of one per
// lane: a batch of new flows otherwise sends a few hundred thousand atomics to two addresses (300,000 fresh flows
// took 0.7 ms that way).
template <typename T>
__device__ __forceinline__ void add_one_aggregated(T *counter) {
    const unsigned same = __match_any_sync(__activemask(), (unsigned long long)(uintptr_t)counter);
    if ((threadIdx.x & 31u) == (unsigned)(__ffs(same) - 1)) atomicAdd(counter, (T)__popc(same));
}

// ---- NoteOutbound, filter.go:189-209 ----------------------------------------------------
__global__ void filter_note_kernel(FilterTables ft, const uint8_t *ring, const uint32_t *off,
                                   const uint32_t *len, uint32_t n, uint64_t ring_bytes, long long now) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t o = off[i], l = len[i];
    if ((o & 15u) || (uint64_t)o + 16u + l > ring_bytes) return;
    Parsed p;
    if (!parse_ipv4(ring + o + 16, l, p)) return;
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    const long long exp = now + flow_ttl(p.proto);
    const int cls = proto_class(p.proto);
    const unsigned long long key = flow_key(p.dst, p.dport, p.sport);
    if (!(ctl->swept_valid && ctl->swept_at == now)) ctl->swept_valid = 0;
    if (key == FLOW_EMPTY) {
        const long long prev = (long long)atomicExch((unsigned long long *)&ft.flow_special_exp[cls],
                                                     (unsigned long long)exp);
        if (flow_absent(prev)) atomicAdd(&ctl->live, 1ull);
        return;
    }
    unsigned long long *keys = (unsigned long long *)ft.flow_keys + flow_region(ft, cls);
    long long *exps = ft.flow_exp + flow_region(ft, cls);
    uint32_t h = (uint32_t)mix64(key) & (ft.flow_capacity - 1);
    for (uint32_t probe = 0; probe < ft.flow_capacity; probe++) {
        const unsigned long long old = atomicCAS(&keys[h], FLOW_EMPTY, key);
        if (old == FLOW_EMPTY || old == key) {
            if (old == FLOW_EMPTY) add_one_aggregated(&ctl->rep.used[cls]);
            const long long prev = (long long)atomicExch((unsigned long long *)&exps[h], (unsigned long long)exp);
            if (flow_absent(prev)) add_one_aggregated(&ctl->live);
            if (prev == FLOW_DEAD) atomicSub(&ctl->rep.dead[cls], 1u); // a deleted entry is back
            return;
        }
        h = (h + 1) & (ft.flow_capacity - 1);
    }
    atomicAdd(ft.flow_error, 1); // table full: the flow is not recorded, the host reports BNK_EFULL
}

// The reference sweeps expired flows whenever the map holds more than 4096 entries after an
// insert.  Within one batch (one `now`) that equals: insert everything, then sweep once if
// the count exceeds the threshold.  A repeat sweep at an unchanged `now` finds nothing.
__global__ void filter_sweep_decide_kernel(FilterTables ft, long long now) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    ctl->sweep_now = (ctl->live > SWEEP_THRESHOLD && !(ctl->swept_valid && ctl->swept_at == now)) ? 1 : 0;
}
__global__ void filter_sweep_kernel(FilterTables ft, long long now) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    if (!ctl->sweep_now) return;
    // both regions of every class are walked; the one not in use holds nothing but fresh slots
    const size_t total = (size_t)6 * ft.flow_capacity;
    unsigned long long dropped = 0;
    uint32_t dead[3] = {0, 0, 0};
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < total + 3; k += (size_t)gridDim.x * blockDim.x) {
        long long *e = k < total ? &ft.flow_exp[k] : &ft.flow_special_exp[k - total];
        const long long exp = *e;
        if (!flow_absent(exp) && now > exp) {
            *e = FLOW_DEAD;
            dropped++;
            if (k < total) dead[k / ((size_t)2 * ft.flow_capacity)]++;
        }
    }
    if (dropped) atomicAdd(&ctl->live, 0ull - dropped);
#pragma unroll
    for (int c = 0; c < 3; c++)
        if (dead[c]) atomicAdd(&ctl->rep.dead[c], dead[c]);
}
__global__ void filter_sweep_finish_kernel(FilterTables ft, long long now) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    if (ctl->sweep_now) {
        ctl->swept_at = now;
        ctl->swept_valid = 1;
        ctl->sweep_now = 0;
    }
}

// ---- CheckInbound, filter.go:121-147 -----------------------------------------------------
// only_status_ok: packets whose status is not BNK_PKT_OK are left alone (open pipeline).
__global__ void filter_check_kernel(FilterTables ft, const uint8_t *ring, const uint32_t *off,
                                    const uint32_t *len, uint8_t *status, uint32_t n, uint64_t ring_bytes,
                                    long long now, int only_status_ok) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (only_status_ok) {
        if (status[i] != BNK_PKT_OK) return;
    }
    if (!ft.enforce) { // filter.go:124-126: allow-all passes even unparseable packets
        status[i] = BNK_PKT_OK;
        return;
    }
    const uint32_t o = off[i], l = len[i];
    Parsed p;
    if ((o & 15u) || (uint64_t)o + 16u + l > ring_bytes || !parse_ipv4(ring + o + 16, l, p)) {
        status[i] = BNK_PKT_FILTER_DENY;
        return;
    }
    if (rules_allow(ft, p)) {
        status[i] = BNK_PKT_OK;
        return;
    }
    // reply to a flow this node opened?  key mirrors NoteOutbound's
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    const int cls = proto_class(p.proto);
    const unsigned long long key = flow_key(p.src, p.sport, p.dport);
    long long *slot_exp = nullptr;
    if (ft.flow_capacity == 0) {
        status[i] = BNK_PKT_FILTER_DENY;
        return;
    }
    if (key == FLOW_EMPTY) {
        slot_exp = &ft.flow_special_exp[cls];
    } else {
        const unsigned long long *keys = (const unsigned long long *)ft.flow_keys + flow_region(ft, cls);
        uint32_t h = (uint32_t)mix64(key) & (ft.flow_capacity - 1);
        for (uint32_t probe = 0; probe < ft.flow_capacity; probe++) {
            const unsigned long long k = keys[h];
            if (k == FLOW_EMPTY) break;
            if (k == key) {
                slot_exp = ft.flow_exp + flow_region(ft, cls) + h;
                break;
            }
            h = (h + 1) & (ft.flow_capacity - 1);
        }
    }
    uint8_t verdict = BNK_PKT_FILTER_DENY;
    if (slot_exp) {
        const long long exp = *(volatile long long *)slot_exp;
        if (!flow_absent(exp)) {
            if (now < exp) { // strict: time.Before
                *(volatile long long *)slot_exp = now + flow_ttl(p.proto); // keep-alive on traffic
                if (!(ctl->swept_valid && ctl->swept_at == now)) ctl->swept_valid = 0;
                verdict = BNK_PKT_OK;
            } else {
                const long long prev = (long long)atomicExch((unsigned long long *)slot_exp, (unsigned long long)FLOW_DEAD);
                if (!flow_absent(prev)) {
                    atomicAdd(&ctl->live, 0ull - 1ull);
                    if (key != FLOW_EMPTY) atomicAdd(&ctl->rep.dead[cls], 1u);
                }
            }
        }
    }
    status[i] = verdict;
}

__global__ void flows_fill_kernel(FilterTables ft) {
    const size_t total = (size_t)6 * ft.flow_capacity;
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < total; k += (size_t)gridDim.x * blockDim.x) {
        ft.flow_keys[k] = FLOW_EMPTY;
        ft.flow_exp[k] = FLOW_FRESH;
    }
    if (blockIdx.x == 0 && threadIdx.x < 3) ft.flow_special_exp[threadIdx.x] = FLOW_FRESH;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
        *ctl = FlowCtl{};
    }
}

// ---- compaction: the entries of class `cls` that are not deleted move from the region in use to the class's
// other region, which is empty; the host then swaps the roles (filter_flows_maintain).  Expired entries that no
// sweep or lookup has deleted yet move along: they still count in len(f.flows), which decides the next sweep.
__global__ void flows_compact_kernel(FilterTables ft, int cls) {
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    const size_t from = flow_region(ft, cls), to = ((size_t)cls * 2 + (ft.flow_half[cls] ^ 1)) * ft.flow_capacity;
    unsigned long long *keys = (unsigned long long *)ft.flow_keys + to;
    long long *exps = ft.flow_exp + to;
    uint32_t moved = 0;
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < ft.flow_capacity; k += (size_t)gridDim.x * blockDim.x) {
        const unsigned long long key = ft.flow_keys[from + k];
        if (key == FLOW_EMPTY) continue;
        const long long exp = ft.flow_exp[from + k];
        if (flow_absent(exp)) continue;
        uint32_t h = (uint32_t)mix64(key) & (ft.flow_capacity - 1);
        bool placed = false; // the target region starts empty and takes fewer entries than it has slots
        for (uint32_t probe = 0; probe < ft.flow_capacity && !placed; probe++) {
            if (atomicCAS(&keys[h], FLOW_EMPTY, key) == FLOW_EMPTY) placed = true;
            else h = (h + 1) & (ft.flow_capacity - 1);
        }
        if (!placed) {
            atomicAdd(ft.flow_error, 1);
            continue;
        }
        exps[h] = exp;
        moved++;
    }
    if (moved) atomicAdd(&ctl->moved, moved);
}
// wipes the region the class has just left and books the move
__global__ void flows_compact_finish_kernel(FilterTables ft, int cls) {
    FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
    const size_t from = flow_region(ft, cls);
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < ft.flow_capacity; k += (size_t)gridDim.x * blockDim.x) {
        ft.flow_keys[from + k] = FLOW_EMPTY;
        ft.flow_exp[from + k] = FLOW_FRESH;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        ctl->rep.used[cls] = ctl->moved; // the kernel in front has finished: the count is final
        ctl->rep.dead[cls] = 0;
        ctl->moved = 0;
    }
}

// ---- per-batch counters (BNK_F_STATS): statuses and output bytes of the first n packets.  Every CTA adds its
// share to the device accumulators; the CTA that finishes last hands the totals to the host struct and leaves
// the accumulators zero for the next launch.
__global__ void __launch_bounds__(256) tally_kernel(const uint8_t *status, const uint32_t *out_len, uint32_t n,
                                                    unsigned long long *acc /* [16] statuses, [16] bytes, [17] ticket */,
                                                    bnk_batch_stats *host_out) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    __shared__ unsigned int cnt[16];
    __shared__ unsigned long long bytes_s;
    __shared__ bool last;
    if (threadIdx.x < 16) cnt[threadIdx.x] = 0;
    if (threadIdx.x == 0) bytes_s = 0;
    __syncthreads();
    unsigned long long bytes = 0;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint8_t st = status[i];
        add_one_aggregated(&cnt[st & 15u]); // nearly every lane hits the same bin
        if (st == BNK_PKT_OK) bytes += out_len[i];
    }
    for (int o = 16; o > 0; o >>= 1) bytes += __shfl_down_sync(0xffffffffu, bytes, o);
    if ((threadIdx.x & 31) == 0 && bytes) atomicAdd(&bytes_s, bytes);
    __syncthreads();
    if (threadIdx.x < 16 && cnt[threadIdx.x]) atomicAdd(&acc[threadIdx.x], (unsigned long long)cnt[threadIdx.x]);
    if (threadIdx.x == 0 && bytes_s) atomicAdd(&acc[16], bytes_s);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&acc[17], 1ull) + 1 == gridDim.x;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < 16) {
        host_out->by_status[threadIdx.x] = atomicExch(&acc[threadIdx.x], 0ull);
    } else if (threadIdx.x == 16) {
        host_out->bytes_out = atomicExch(&acc[16], 0ull);
        host_out->packets = n;
        acc[17] = 0;
    }
}

} // namespace

cudaError_t filter_tables_alloc(bnk_ctx *ctx) {
    FilterTables &ft = ctx->ft;
    ft = FilterTables{};
    const uint32_t cap = ctx->cfg.flow_capacity;
    ft.flow_capacity = cap;
    cudaError_t e;
    FlowCtl *ctl = nullptr;
    if ((e = cudaMalloc(&ctl, sizeof(FlowCtl))) != cudaSuccess) return e;
    ft.flow_live = reinterpret_cast<unsigned long long *>(ctl);
    ft.flow_error = &ctl->rep.error;
    if ((e = cudaMalloc(&ft.flow_special_exp, 3 * sizeof(long long))) != cudaSuccess) return e;
    if (cap) {
        if ((e = cudaMalloc(&ft.flow_keys, (size_t)6 * cap * sizeof(uint64_t))) != cudaSuccess) return e;
        if ((e = cudaMalloc(&ft.flow_exp, (size_t)6 * cap * sizeof(long long))) != cudaSuccess) return e;
    }
    // With a stated rule-table capacity both buffer sets are allocated here, and a rule swap allocates nothing.
    if (const size_t cap_t = ctx->cfg.max_acl_tuples) {
        size_t slots = 16;
        while (slots < cap_t * 8) slots <<= 1;
        for (bnk_ctx::RuleSet &rs : ctx->rule_set) {
            if ((e = cudaMalloc(&rs.keys, slots * sizeof(uint64_t))) != cudaSuccess) return e;
            if ((e = cudaMalloc(&rs.span, slots * sizeof(uint2))) != cudaSuccess) return e;
            if ((e = cudaMalloc(&rs.entries, cap_t * sizeof(uint64_t))) != cudaSuccess) return e;
            rs.slots_cap = slots;
            rs.entries_cap = cap_t;
        }
    }
    return filter_flows_clear(ctx, ctx->admin_stream);
}

void filter_tables_free(bnk_ctx *ctx) {
    FilterTables &ft = ctx->ft;
    cudaFree(ft.flow_live);
    cudaFree(ft.flow_special_exp);
    cudaFree(ft.flow_keys);
    cudaFree(ft.flow_exp);
    for (bnk_ctx::RuleSet &rs : ctx->rule_set) {
        cudaFree(rs.keys);
        cudaFree(rs.span);
        cudaFree(rs.entries);
        for (cudaEvent_t ev : rs.in_use) cudaEventDestroy(ev);
        rs = bnk_ctx::RuleSet{};
    }
    ft = FilterTables{};
}

cudaError_t filter_flows_clear(bnk_ctx *ctx, cudaStream_t s) {
    ctx->ft.flow_half[0] = ctx->ft.flow_half[1] = ctx->ft.flow_half[2] = 0;
    for (auto &h : ctx->flow_dead_hint) h = 0;
    ctx->flow_errors_seen = 0;
    flows_fill_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ctx->ft);
    ctx->launches += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return cudaStreamSynchronize(s);
}

cudaError_t filter_flow_stats(bnk_ctx *ctx, uint64_t *live, uint32_t used[3], uint32_t dead[3]) {
    FlowCtl ctl;
    cudaError_t e = cudaMemcpy(&ctl, ctx->ft.flow_live, sizeof ctl, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    *live = ctl.live;
    for (int c = 0; c < 3; c++) {
        used[c] = ctl.rep.used[c];
        dead[c] = ctl.rep.dead[c];
    }
    return cudaSuccess;
}

// Export and import work on host copies of the tables: they are for tests and state hand-over, not for the packet
// path, and the caller has quiesced the context.  The host applies the same hash and the same probing as the kernels.
namespace {
struct FlowTablesHost {
    std::vector<unsigned long long> keys;
    std::vector<long long> exp;
    long long special[3];
    FlowCtl ctl;
};
cudaError_t flows_download(bnk_ctx *ctx, FlowTablesHost &h) {
    const FilterTables &ft = ctx->ft;
    const size_t total = (size_t)6 * ft.flow_capacity;
    h.keys.resize(total);
    h.exp.resize(total);
    cudaError_t e = cudaSuccess;
    if (total) {
        e = cudaMemcpy(h.keys.data(), ft.flow_keys, total * sizeof(uint64_t), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(h.exp.data(), ft.flow_exp, total * sizeof(long long), cudaMemcpyDeviceToHost);
    }
    if (e == cudaSuccess) e = cudaMemcpy(h.special, ft.flow_special_exp, sizeof h.special, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(&h.ctl, ft.flow_live, sizeof h.ctl, cudaMemcpyDeviceToHost);
    return e;
}
int class_of(uint8_t proto) { return proto == 6 ? 0 : (proto == 17 ? 1 : 2); }
uint8_t proto_of(int cls) { return cls == 0 ? 6 : (cls == 1 ? 17 : 1); }
bool absent_host(long long exp) { return exp <= FLOW_FRESH; }
} // namespace

int filter_flows_export(bnk_ctx *ctx, bnk_flow_entry *out, size_t capacity, size_t *count) {
    FlowTablesHost h;
    if (flows_download(ctx, h) != cudaSuccess) return BNK_ECUDA;
    const FilterTables &ft = ctx->ft;
    size_t n = 0;
    auto emit = [&](int cls, unsigned long long key, long long exp) {
        if (n < capacity && out) {
            bnk_flow_entry e{};
            e.remote_addr = (uint32_t)(key >> 32);
            e.remote_port = (uint16_t)(key >> 16);
            e.local_port = (uint16_t)key;
            e.proto = proto_of(cls);
            e.expiry_unix_ns = exp;
            out[n] = e;
        }
        n++;
    };
    for (int cls = 0; cls < 3; cls++) {
        const size_t base = flow_region(ft, cls);
        for (size_t k = 0; k < ft.flow_capacity; k++)
            if (h.keys[base + k] != FLOW_EMPTY && !absent_host(h.exp[base + k])) emit(cls, h.keys[base + k], h.exp[base + k]);
        if (!absent_host(h.special[cls])) emit(cls, FLOW_EMPTY, h.special[cls]);
    }
    *count = n;
    return BNK_SUCCESS;
}

int filter_flows_import(bnk_ctx *ctx, const bnk_flow_entry *entries, size_t n) {
    FlowTablesHost h;
    if (flows_download(ctx, h) != cudaSuccess) return BNK_ECUDA;
    const FilterTables &ft = ctx->ft;
    const uint32_t cap = ft.flow_capacity;
    for (size_t i = 0; i < n; i++) {
        const bnk_flow_entry &e = entries[i];
        if (e.proto != 6 && e.proto != 17 && e.proto != 1) return BNK_EINVAL;
        if (absent_host(e.expiry_unix_ns)) return BNK_EINVAL;
        const int cls = class_of(e.proto);
        const unsigned long long key = ((unsigned long long)e.remote_addr << 32) | ((unsigned long long)e.remote_port << 16) | e.local_port;
        if (key == FLOW_EMPTY) {
            if (absent_host(h.special[cls])) h.ctl.live++;
            h.special[cls] = e.expiry_unix_ns;
            continue;
        }
        if (cap == 0) return BNK_EFULL;
        const size_t base = flow_region(ft, cls);
        uint32_t at = (uint32_t)mix64(key) & (cap - 1);
        bool placed = false;
        for (uint32_t probe = 0; probe < cap && !placed; probe++, at = (at + 1) & (cap - 1)) {
            unsigned long long &k = h.keys[base + at];
            if (k != FLOW_EMPTY && k != key) continue;
            if (k == FLOW_EMPTY) {
                k = key;
                h.ctl.rep.used[cls]++;
            }
            long long &x = h.exp[base + at];
            if (absent_host(x)) h.ctl.live++;
            if (x == FLOW_DEAD) h.ctl.rep.dead[cls]--;
            x = e.expiry_unix_ns;
            placed = true;
        }
        if (!placed) return BNK_EFULL;
    }
    h.ctl.swept_valid = 0;
    const size_t total = (size_t)6 * cap;
    cudaError_t e = cudaSuccess;
    if (total) {
        e = cudaMemcpy(ft.flow_keys, h.keys.data(), total * sizeof(uint64_t), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(ft.flow_exp, h.exp.data(), total * sizeof(long long), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaMemcpy(ft.flow_special_exp, h.special, sizeof h.special, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(ft.flow_live, &h.ctl, sizeof h.ctl, cudaMemcpyHostToDevice);
    return e == cudaSuccess ? BNK_SUCCESS : BNK_ECUDA;
}

cudaError_t launch_flow_report(bnk_batch *b, cudaStream_t s) {
    const FlowCtl *ctl = reinterpret_cast<const FlowCtl *>(b->ctx->ft.flow_live);
    b->flow_reported = true;
    return cudaMemcpyAsync(b->h_flow, &ctl->rep, sizeof(FlowReport), cudaMemcpyDeviceToHost, s);
}

// Deleted entries keep their slots, so a class whose flows come and go (every connection brings a new source
// port) would fill up although few flows are alive, and a lookup that misses would walk longer and longer
// chains.  The submit that is about to record flows calls this first: when the device last reported that
// deleted entries fill a quarter of a class's region, the class is compacted on this batch's stream.  Kernels
// of other batches must not see the table half-moved, so the move is fenced against every other stream of the
// context on both sides, and submits are held off while the fences are placed (submit_mu, exclusive).
cudaError_t filter_flows_maintain(bnk_batch *b, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    const uint32_t cap = ctx->ft.flow_capacity;
    if (cap == 0) return cudaSuccess;
    const uint32_t limit = cap / 4;
    if (ctx->flow_dead_hint[0] < limit && ctx->flow_dead_hint[1] < limit && ctx->flow_dead_hint[2] < limit)
        return cudaSuccess;
    std::unique_lock<std::shared_mutex> tables(ctx->submit_mu);
    cudaError_t e;
    for (bnk_batch *o : ctx->batches) { // everything submitted so far finishes before the move
        if (o == b) continue;
        if ((e = cudaEventRecord(o->ev_fence, o->stream)) != cudaSuccess) return e;
        if ((e = cudaStreamWaitEvent(s, o->ev_fence, 0)) != cudaSuccess) return e;
    }
    for (int cls = 0; cls < 3; cls++) {
        if (ctx->flow_dead_hint[cls] < limit) continue;
        flows_compact_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ctx->ft, cls);
        flows_compact_finish_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ctx->ft, cls);
        ctx->launches += 2;
        ctx->ft.flow_half[cls] ^= 1; // launches from here on use the other region
        ctx->flow_dead_hint[cls] = 0;
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if ((e = cudaEventRecord(b->ev_fence, s)) != cudaSuccess) return e;
    for (bnk_batch *o : ctx->batches) // and nothing submitted later starts before it is done
        if (o != b && (e = cudaStreamWaitEvent(o->stream, b->ev_fence, 0)) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_tally(bnk_batch *b, uint32_t n, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    uint32_t grid = (n + 1023) / 1024;
    if (grid == 0) grid = 1;
    if (grid > (uint32_t)ctx->sm_count * 4) grid = ctx->sm_count * 4;
    bnk_batch_stats *out = b->h_stats; // pinned memory has the same address on the device
    launch_kernel(n <= dependent_launch_up_to(), tally_kernel, dim3(grid), dim3(256), s, b->dev.status, b->dev.out_len, n,
                  b->d_stats, out);
    ctx->launches += 1;
    return cudaGetLastError();
}

// Builds the prefix-indexed rule table on the host and swaps it in.  Runs per policy change
// (Engine.ApplyNetmap, internal/dataplane/engine.go:279-283), never per packet, and may run while packets
// flow: the reference swaps the table under the filter's mutex between two packets (filter.go:46-51); here
// the new table is uploaded into the buffer set that is not in use, on the admin stream, and the context's
// FilterTables (which every launch captures by value) switch over between two submits.  A batch submitted
// before the switch is judged by the old rules as a whole, one submitted after it by the new ones.
int filter_acl_upload(bnk_ctx *ctx, int enforce, const bnk_acl_tuple *tuples, size_t n) {
    std::lock_guard<std::mutex> one_at_a_time(ctx->acl_mu);
    FilterTables &ft = ctx->ft;
    struct Item {
        uint64_t key, ent;
    };
    std::vector<Item> items;
    items.reserve(n);
    uint64_t len_mask = 0;
    for (size_t i = 0; i < n; i++) {
        const bnk_acl_tuple &t = tuples[i];
        if (t.prefix_len > 32) return BNK_EINVAL;
        if (t.proto != 6 && t.proto != 17 && t.proto != 1) continue; // can never equal a parsed protocol
        if (t.proto != 1 && t.port_first > t.port_last) continue;    // empty range
        items.push_back({rule_key(t.prefix_len, t.addr),
                         ((uint64_t)t.proto << 32) | ((uint64_t)t.port_first << 16) | t.port_last});
        len_mask |= 1ull << t.prefix_len;
    }
    std::sort(items.begin(), items.end(), [](const Item &a, const Item &b) {
        return a.key != b.key ? a.key < b.key : a.ent < b.ent;
    });
    items.erase(std::unique(items.begin(), items.end(),
                            [](const Item &a, const Item &b) { return a.key == b.key && a.ent == b.ent; }),
                items.end());
    size_t groups = 0;
    for (size_t i = 0; i < items.size(); i++)
        if (i == 0 || items[i].key != items[i - 1].key) groups++;
    uint32_t slots = 0;
    if (groups) {
        slots = 16;
        while ((size_t)slots < groups * 8) slots <<= 1; // a quarter full at most: misses end after 1.4 probes on average, and the lanes of a warp wait for the longest of their walks
    }
    std::vector<uint64_t> keys(slots, 0);
    std::vector<uint2> span(slots, make_uint2(0, 0));
    std::vector<uint64_t> ents(items.size());
    for (size_t i = 0; i < items.size();) {
        size_t j = i;
        while (j < items.size() && items[j].key == items[i].key) {
            ents[j] = items[j].ent;
            j++;
        }
        uint32_t h = rule_hash(items[i].key) & (slots - 1);
        while (keys[h]) h = (h + 1) & (slots - 1);
        keys[h] = items[i].key;
        span[h] = make_uint2((uint32_t)i, (uint32_t)(j - i));
        i = j;
    }
    bnk_ctx::RuleSet &spare = ctx->rule_set[ctx->rule_cur ^ 1];
    // Kernels launched before the previous switch may still be reading the spare set: wait for those (the events
    // were recorded on the batches' streams at that switch), not for the whole device.
    for (cudaEvent_t ev : spare.in_use) {
        cudaEventSynchronize(ev);
        cudaEventDestroy(ev);
    }
    spare.in_use.clear();
    // A context created without max_acl_tuples grows the spare set here when a larger table arrives
    // (an allocation can stall the device for a moment; state the capacity to avoid that).
    if (slots > spare.slots_cap) {
        cudaFree(spare.keys);
        cudaFree(spare.span);
        spare.keys = nullptr;
        spare.span = nullptr;
        spare.slots_cap = 0;
        if (cudaMalloc(&spare.keys, slots * sizeof(uint64_t)) != cudaSuccess) return BNK_ENOMEM;
        if (cudaMalloc(&spare.span, slots * sizeof(uint2)) != cudaSuccess) return BNK_ENOMEM;
        spare.slots_cap = slots;
    }
    if (ents.size() > spare.entries_cap) {
        cudaFree(spare.entries);
        spare.entries = nullptr;
        spare.entries_cap = 0;
        if (cudaMalloc(&spare.entries, ents.size() * sizeof(uint64_t)) != cudaSuccess) return BNK_ENOMEM;
        spare.entries_cap = ents.size();
    }
    cudaStream_t as = ctx->admin_stream;
    if (slots) {
        cudaMemcpyAsync(spare.keys, keys.data(), slots * sizeof(uint64_t), cudaMemcpyHostToDevice, as);
        cudaMemcpyAsync(spare.span, span.data(), slots * sizeof(uint2), cudaMemcpyHostToDevice, as);
        if (!ents.empty()) cudaMemcpyAsync(spare.entries, ents.data(), ents.size() * sizeof(uint64_t), cudaMemcpyHostToDevice, as);
    }
    if (cudaStreamSynchronize(as) != cudaSuccess) return BNK_ECUDA;
    {
        std::unique_lock<std::shared_mutex> tables(ctx->submit_mu); // between two submits
        bnk_ctx::RuleSet &old = ctx->rule_set[ctx->rule_cur];
        for (bnk_batch *b : ctx->batches) { // what has been launched with the old set, per stream
            cudaEvent_t ev;
            if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return BNK_ECUDA;
            cudaEventRecord(ev, b->stream);
            old.in_use.push_back(ev);
        }
        ft.rule_keys = spare.keys;
        ft.rule_span = spare.span;
        ft.rule_entries = spare.entries;
        ft.rule_slots = slots;
        ft.len_mask = len_mask;
        ft.enforce = enforce ? 1 : 0;
        ctx->rule_cur ^= 1;
    }
    return BNK_SUCCESS;
}

cudaError_t launch_filter_note(bnk_batch *b, uint32_t n, long long now_ns, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    if (n == 0 || !ctx->ft.enforce || ctx->ft.flow_capacity == 0) return cudaSuccess; // filter.go:192-194
    launch_kernel(n <= dependent_launch_up_to(), filter_note_kernel, dim3((n + 255) / 256), dim3(256), s, ctx->ft,
        b->dev.ring, b->dev.off, b->dev.len, n, b->ring_bytes, now_ns);
    launch_kernel(n <= dependent_launch_up_to(), filter_sweep_decide_kernel, dim3(1), dim3(1), s, ctx->ft, now_ns);
    launch_kernel(n <= dependent_launch_up_to(), filter_sweep_kernel, dim3(ctx->sm_count * 4), dim3(256), s, ctx->ft,
        now_ns);
    launch_kernel(n <= dependent_launch_up_to(), filter_sweep_finish_kernel, dim3(1), dim3(1), s, ctx->ft, now_ns);
    ctx->launches += 4;
    return cudaGetLastError();
}

cudaError_t launch_filter_check(bnk_batch *b, uint32_t n, long long now_ns, bool only_status_ok, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    if (n == 0) return cudaSuccess;
    // open pipeline: the packet handed to the filter is the decrypted payload of out_len bytes
    const uint32_t *lens = only_status_ok ? b->dev.out_len : b->dev.len;
    launch_kernel(n <= dependent_launch_up_to(), filter_check_kernel, dim3((n + 255) / 256), dim3(256), s, ctx->ft,
        b->dev.ring, b->dev.off, lens, b->dev.status, n, b->ring_bytes, now_ns, only_status_ok ? 1 : 0);
    ctx->launches += 1;
    return cudaGetLastError();
}
