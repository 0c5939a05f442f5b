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
#include <algorithm>
#include <climits>
#include <vector>

#include "bnk_internal.cuh"

namespace {

constexpr unsigned long long FLOW_EMPTY = ~0ull;
constexpr long long FLOW_DEAD = LLONG_MIN;
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
};

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
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
    uint64_t lens = ft.len_mask;
    while (lens) {
        const uint32_t len = __ffsll((long long)lens) - 1;
        lens &= lens - 1;
        const uint64_t key = rule_key(len, p.src);
        uint32_t h = (uint32_t)mix64(key) & (ft.rule_slots - 1);
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
        if (prev == FLOW_DEAD) atomicAdd(&ctl->live, 1ull);
        return;
    }
    unsigned long long *keys = (unsigned long long *)ft.flow_keys + (size_t)cls * ft.flow_capacity;
    long long *exps = ft.flow_exp + (size_t)cls * ft.flow_capacity;
    uint32_t h = (uint32_t)mix64(key) & (ft.flow_capacity - 1);
    for (uint32_t probe = 0; probe < ft.flow_capacity; probe++) {
        const unsigned long long old = atomicCAS(&keys[h], FLOW_EMPTY, key);
        if (old == FLOW_EMPTY || old == key) {
            const long long prev = (long long)atomicExch((unsigned long long *)&exps[h], (unsigned long long)exp);
            if (prev == FLOW_DEAD) atomicAdd(&ctl->live, 1ull);
            return;
        }
        h = (h + 1) & (ft.flow_capacity - 1);
    }
    *ft.flow_error = 1; // table full: the flow is not recorded, the host reports BNK_EFULL
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
    const size_t total = (size_t)3 * ft.flow_capacity;
    unsigned long long dropped = 0;
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < total + 3; k += (size_t)gridDim.x * blockDim.x) {
        long long *e = k < total ? &ft.flow_exp[k] : &ft.flow_special_exp[k - total];
        const long long exp = *e;
        if (exp != FLOW_DEAD && now > exp) {
            *e = FLOW_DEAD;
            dropped++;
        }
    }
    if (dropped) atomicAdd(&ctl->live, 0ull - dropped);
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
        const unsigned long long *keys = (const unsigned long long *)ft.flow_keys + (size_t)cls * ft.flow_capacity;
        uint32_t h = (uint32_t)mix64(key) & (ft.flow_capacity - 1);
        for (uint32_t probe = 0; probe < ft.flow_capacity; probe++) {
            const unsigned long long k = keys[h];
            if (k == FLOW_EMPTY) break;
            if (k == key) {
                slot_exp = ft.flow_exp + (size_t)cls * ft.flow_capacity + h;
                break;
            }
            h = (h + 1) & (ft.flow_capacity - 1);
        }
    }
    uint8_t verdict = BNK_PKT_FILTER_DENY;
    if (slot_exp) {
        const long long exp = *(volatile long long *)slot_exp;
        if (exp != FLOW_DEAD) {
            if (now < exp) { // strict: time.Before
                *(volatile long long *)slot_exp = now + flow_ttl(p.proto); // keep-alive on traffic
                if (!(ctl->swept_valid && ctl->swept_at == now)) ctl->swept_valid = 0;
                verdict = BNK_PKT_OK;
            } else {
                const long long prev = (long long)atomicExch((unsigned long long *)slot_exp, (unsigned long long)FLOW_DEAD);
                if (prev != FLOW_DEAD) atomicAdd(&ctl->live, 0ull - 1ull);
            }
        }
    }
    status[i] = verdict;
}

__global__ void flows_fill_kernel(FilterTables ft) {
    const size_t total = (size_t)3 * ft.flow_capacity;
    for (size_t k = blockIdx.x * (size_t)blockDim.x + threadIdx.x; k < total; k += (size_t)gridDim.x * blockDim.x) {
        ft.flow_keys[k] = FLOW_EMPTY;
        ft.flow_exp[k] = FLOW_DEAD;
    }
    if (blockIdx.x == 0 && threadIdx.x < 3) ft.flow_special_exp[threadIdx.x] = FLOW_DEAD;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        FlowCtl *ctl = reinterpret_cast<FlowCtl *>(ft.flow_live);
        ctl->live = 0;
        ctl->swept_at = 0;
        ctl->swept_valid = 0;
        ctl->sweep_now = 0;
        *ft.flow_error = 0;
    }
}

} // namespace

cudaError_t filter_tables_alloc(bnk_ctx *ctx) {
    FilterTables &ft = ctx->ft;
    ft = FilterTables{};
    const uint32_t cap = ctx->cfg.flow_capacity;
    ft.flow_capacity = cap;
    cudaError_t e;
    if ((e = cudaMalloc(&ft.flow_live, sizeof(FlowCtl))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&ft.flow_special_exp, 3 * sizeof(long long))) != cudaSuccess) return e;
    if ((e = cudaMalloc(&ft.flow_error, sizeof(int))) != cudaSuccess) return e;
    if (cap) {
        if ((e = cudaMalloc(&ft.flow_keys, (size_t)3 * cap * sizeof(uint64_t))) != cudaSuccess) return e;
        if ((e = cudaMalloc(&ft.flow_exp, (size_t)3 * cap * sizeof(long long))) != cudaSuccess) return e;
    }
    return filter_flows_clear(ctx, ctx->admin_stream);
}

void filter_tables_free(bnk_ctx *ctx) {
    FilterTables &ft = ctx->ft;
    cudaFree(ft.flow_live);
    cudaFree(ft.flow_special_exp);
    cudaFree(ft.flow_error);
    cudaFree(ft.flow_keys);
    cudaFree(ft.flow_exp);
    cudaFree(ft.rule_keys);
    cudaFree(ft.rule_span);
    cudaFree(ft.rule_entries);
    ft = FilterTables{};
}

cudaError_t filter_flows_clear(bnk_ctx *ctx, cudaStream_t s) {
    flows_fill_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ctx->ft);
    ctx->launches += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return cudaStreamSynchronize(s);
}

// Builds the prefix-indexed rule table on the host and swaps it in.  Runs per policy change
// (Engine.ApplyNetmap, internal/dataplane/engine.go:279-283), never per packet.
int filter_acl_upload(bnk_ctx *ctx, int enforce, const bnk_acl_tuple *tuples, size_t n) {
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
        while ((size_t)slots < groups * 2) slots <<= 1;
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
        uint32_t h = (uint32_t)mix64(items[i].key) & (slots - 1);
        while (keys[h]) h = (h + 1) & (slots - 1);
        keys[h] = items[i].key;
        span[h] = make_uint2((uint32_t)i, (uint32_t)(j - i));
        i = j;
    }
    uint64_t *d_keys = nullptr, *d_ents = nullptr;
    uint2 *d_span = nullptr;
    if (slots) {
        if (cudaMalloc(&d_keys, slots * sizeof(uint64_t)) != cudaSuccess) return BNK_ENOMEM;
        if (cudaMalloc(&d_span, slots * sizeof(uint2)) != cudaSuccess) { cudaFree(d_keys); return BNK_ENOMEM; }
        if (cudaMalloc(&d_ents, std::max<size_t>(ents.size(), 1) * sizeof(uint64_t)) != cudaSuccess) {
            cudaFree(d_keys);
            cudaFree(d_span);
            return BNK_ENOMEM;
        }
        cudaMemcpy(d_keys, keys.data(), slots * sizeof(uint64_t), cudaMemcpyHostToDevice);
        cudaMemcpy(d_span, span.data(), slots * sizeof(uint2), cudaMemcpyHostToDevice);
        if (!ents.empty()) cudaMemcpy(d_ents, ents.data(), ents.size() * sizeof(uint64_t), cudaMemcpyHostToDevice);
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return BNK_ECUDA;
    cudaFree(ft.rule_keys);
    cudaFree(ft.rule_span);
    cudaFree(ft.rule_entries);
    ft.rule_keys = d_keys;
    ft.rule_span = d_span;
    ft.rule_entries = d_ents;
    ft.rule_slots = slots;
    ft.len_mask = len_mask;
    ft.enforce = enforce ? 1 : 0;
    return BNK_SUCCESS;
}

cudaError_t launch_filter_note(bnk_batch *b, uint32_t n, long long now_ns, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    if (n == 0 || !ctx->ft.enforce || ctx->ft.flow_capacity == 0) return cudaSuccess; // filter.go:192-194
    launch_kernel(n <= kDependentLaunchUpTo, filter_note_kernel, dim3((n + 255) / 256), dim3(256), s, ctx->ft,
        b->dev.ring, b->dev.off, b->dev.len, n, b->ring_bytes, now_ns);
    launch_kernel(n <= kDependentLaunchUpTo, filter_sweep_decide_kernel, dim3(1), dim3(1), s, ctx->ft, now_ns);
    launch_kernel(n <= kDependentLaunchUpTo, filter_sweep_kernel, dim3(ctx->sm_count * 4), dim3(256), s, ctx->ft,
        now_ns);
    launch_kernel(n <= kDependentLaunchUpTo, filter_sweep_finish_kernel, dim3(1), dim3(1), s, ctx->ft, now_ns);
    ctx->launches += 4;
    return cudaGetLastError();
}

cudaError_t launch_filter_check(bnk_batch *b, uint32_t n, long long now_ns, bool only_status_ok, cudaStream_t s) {
    bnk_ctx *ctx = b->ctx;
    if (n == 0) return cudaSuccess;
    // open pipeline: the packet handed to the filter is the decrypted payload of out_len bytes
    const uint32_t *lens = only_status_ok ? b->dev.out_len : b->dev.len;
    launch_kernel(n <= kDependentLaunchUpTo, filter_check_kernel, dim3((n + 255) / 256), dim3(256), s, ctx->ft,
        b->dev.ring, b->dev.off, lens, b->dev.status, n, b->ring_bytes, now_ns, only_status_ok ? 1 : 0);
    ctx->launches += 1;
    return cudaGetLastError();
}
