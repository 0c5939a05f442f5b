// C ABI of libbnkgpu.so (declared in include/bnk_gpu.h): contexts, device tables,
// pinned packet rings with device mirrors, and the submit/wait pipeline that strings
// host->device copies, the kernels and device->host copies on one CUDA stream per batch.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <thread>

#include "bnk_internal.cuh"

namespace {

thread_local std::string g_last_error; // for failures that have no context to hang on

int fail(bnk_ctx *ctx, int code, const char *what, cudaError_t e = cudaSuccess) {
    char buf[512];
    if (e != cudaSuccess)
        snprintf(buf, sizeof buf, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    else
        snprintf(buf, sizeof buf, "%s", what);
    if (ctx) {
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->last_error = buf;
    }
    g_last_error = buf;
    return code;
}

#define CK(ctx, call)                                                  \
    do {                                                               \
        cudaError_t _e = (call);                                       \
        if (_e != cudaSuccess) return fail((ctx), BNK_ECUDA, #call, _e); \
    } while (0)

bool is_pow2(uint64_t v) { return v && !(v & (v - 1)); }

template <typename T>
cudaError_t dev_alloc_zero(T **p, size_t count) {
    cudaError_t e = cudaMalloc(p, count * sizeof(T));
    if (e != cudaSuccess) return e;
    return cudaMemset(*p, 0, count * sizeof(T));
}

// highest ring byte any of the first n packets can touch (input or output side)
uint64_t ring_extent(const bnk_batch *b, uint32_t n, uint32_t slack) {
    const uint32_t *off = b->host.off, *len = b->host.len;
    uint64_t ext = 0;
    for (uint32_t i = 0; i < n; i++) {
        const uint64_t e = (uint64_t)off[i] + len[i] + slack;
        if (e > ext) ext = e;
    }
    ext = (ext + 15) & ~15ull;
    return ext > b->ring_bytes ? b->ring_bytes : ext;
}

int begin_submit(bnk_batch *b, uint32_t npkts, bool touches_host = true) {
    if (!b) return BNK_EINVAL;
    if (npkts > b->max_pkts) return fail(b->ctx, BNK_EINVAL, "npkts exceeds the batch capacity");
    if (b->in_flight && (touches_host || b->dev_stale))
        return fail(b->ctx, BNK_EBUSY, "batch has work in flight; call bnk_wait first");
    CK(b->ctx, cudaSetDevice(b->ctx->device));
    return BNK_SUCCESS;
}

// Closes a submit on every path out of it: whatever was queued before an error is still on the batch's stream,
// so a later bnk_wait really waits for it before the host touches the ring.  (Completion is that of the stream:
// work on the side stream is always joined back before a submit returns, and no event is recorded per submit.)
struct SubmitScope {
    bnk_batch *b;
    std::shared_lock<std::shared_mutex> tables; // see bnk_ctx::submit_mu
    explicit SubmitScope(bnk_batch *batch) : b(batch), tables(batch->ctx->submit_mu) { b->stats_pending = false; }
    ~SubmitScope() { b->in_flight = true; }
};

// The counters of BNK_F_STATS: one launch behind the submit's last kernel, totals straight into pinned memory.
cudaError_t tally_if_asked(bnk_batch *b, uint32_t npkts, uint32_t flags, cudaStream_t s) {
    if (!(flags & BNK_F_STATS)) return cudaSuccess;
    b->stats_pending = true;
    return launch_tally(b, npkts, s);
}

// Small batches skip the copy engines: the kernels read the caller's pinned ring and descriptors through the
// bus and write the results straight back (pinned memory has the same address on the device).  For a batch of
// a few hundred KB the four copies and the engine hand-overs either side of the kernels cost more than the
// kernels themselves.  While a HostAlias lives, the launchers see the host arrays where the device copies
// would be; the device copies fall behind (dev_stale) until the next full upload.
// The seal/open kernel of such a batch (one warp per packet) moves its data in 512-byte stretches per load and store
// instruction; with 16-byte pieces 64 bytes apart every piece was a bus transaction of its own, reads came at
// ~10 GB/s and the mode stopped paying at a hundred KB and did not scale over threads.  Now, measured on 128 full-size
// packets: 35 us against 38 per seal, and eight / sixteen host threads with batches of their own move 140 / 144
// Gbit/s against 118 / 117 through the copy engines (256 packets: 154 / 170 against 155 / 137).  Beyond 256 packets
// the copy engines win again (512: 184 against 60), hence the two limits.  Serving only the descriptors this way and
// the ring by copy was measured too and gained nothing.
constexpr uint32_t kHostDirectMaxPkts = 256;
// With many such batches in flight at once the mode can collapse (sixteen threads with four 128-packet batches each:
// 51 Gbit/s in most runs, against 140-150 with two each or with eight threads), so at most kHostDirectInFlight
// batches of a context run this way at a time and the next ones are copied, which does not degrade.  With the cap,
// ten runs each: 8 threads x 2 batches median 140 Gbit/s (copies: 117), 16 x 2 152 (115), 16 x 4 127 (118); on a
// shared host both ways show slow runs now and then.
constexpr int kHostDirectInFlight = 16;
bool host_direct(bnk_batch *b, uint32_t npkts, uint32_t flags, uint64_t ext) {
    bnk_ctx *ctx = b->ctx;
    if (!(ctx->host_direct_bytes != 0 && npkts != 0 && npkts <= kHostDirectMaxPkts &&
          !(flags & (BNK_F_NO_H2D | BNK_F_NO_D2H | BNK_F_USE_OUT_LEN)) && ext <= ctx->host_direct_bytes))
        return false;
    if (b->direct_counted) return true; // a second submit on a batch that is already counted
    if (ctx->direct_in_flight.load(std::memory_order_relaxed) >= kHostDirectInFlight) return false;
    ctx->direct_in_flight.fetch_add(1, std::memory_order_relaxed);
    b->direct_counted = true;
    return true;
}
void direct_done(bnk_batch *b) {
    if (b->direct_counted) {
        b->direct_counted = false;
        b->ctx->direct_in_flight.fetch_sub(1, std::memory_order_relaxed);
    }
}
struct HostAlias {
    bnk_batch *b;
    DeviceBatch saved;
    bool on;
    HostAlias(bnk_batch *batch, bool enable) : b(batch), saved(batch->dev), on(enable) {
        if (!on) return;
        DeviceBatch &d = b->dev;
        const bnk_batch_view &h = b->host;
        d.ring = h.ring;
        d.off = h.off;
        d.len = h.len;
        d.slot = h.slot;
        d.counter = h.counter;
        d.out_len = h.out_len;
        d.status = h.status;
        b->dev_stale = true;
    }
    ~HostAlias() {
        if (on) b->dev = saved;
    }
};

// Descriptor fields in slab order.  A run of fields moves as one copy when that is cheap (a batch that is mostly
// full, or a slab prefix of a few KB); otherwise each field moves its first n entries.
enum { D_OFF = 0, D_LEN, D_SLOT, D_COUNTER, D_OUT_LEN, D_STATUS };
const uint32_t kDescOff[7] = {0, 4, 8, 12, 20, 24, 25};   // bytes per entry before each field
cudaError_t desc_copy(bnk_batch *b, size_t n, int first, int last, bool to_device, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    const size_t np = b->npad;
    const size_t lo = kDescOff[first] * np;
    const size_t hi = kDescOff[last] * np + (size_t)(kDescOff[last + 1] - kDescOff[last]) * n;
    const cudaMemcpyKind kind = to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
    if (first == last || hi - lo <= 65536 || 2 * n >= np) {
        return to_device ? cudaMemcpyAsync(b->d_desc + lo, b->h_desc + lo, hi - lo, kind, s)
                         : cudaMemcpyAsync(b->h_desc + lo, b->d_desc + lo, hi - lo, kind, s);
    }
    for (int f = first; f <= last; f++) {
        const size_t at = kDescOff[f] * np, bytes = (size_t)(kDescOff[f + 1] - kDescOff[f]) * n;
        cudaError_t e = to_device ? cudaMemcpyAsync(b->d_desc + at, b->h_desc + at, bytes, kind, s)
                                  : cudaMemcpyAsync(b->h_desc + at, b->d_desc + at, bytes, kind, s);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

AeadArgs aead_args(bnk_batch *b, uint32_t n, bool open, const uint32_t *order) {
    bnk_ctx *ctx = b->ctx;
    AeadArgs a{};
    a.ring = b->dev.ring;
    a.off = b->dev.off;
    a.len = b->dev.len;
    a.slot = b->dev.slot;
    a.counter = b->dev.counter;
    a.out_len = b->dev.out_len;
    a.status = b->dev.status;
    a.keys = open ? ctx->kt.recv_keys : ctx->kt.send_keys;
    a.remote_index = ctx->kt.remote_index;
    a.valid = ctx->kt.valid;
    a.order = order;
    a.n = n;
    a.mtu = ctx->cfg.mtu;
    a.max_slots = ctx->cfg.max_keypairs;
    a.ring_bytes = b->ring_bytes;
    return a;
}

} // namespace

extern "C" {

int bnk_abi_version(void) { return BNK_ABI_VERSION; }

const char *bnk_strerror(int code) {
    switch (code) {
    case BNK_SUCCESS: return "success";
    case BNK_EINVAL: return "invalid argument";
    case BNK_ENOMEM: return "out of memory";
    case BNK_ECUDA: return "CUDA error";
    case BNK_ETIMEDOUT: return "timed out";
    case BNK_EBUSY: return "batch busy";
    case BNK_EFULL: return "table full";
    default: return "unknown error";
    }
}

int bnk_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return fail(nullptr, BNK_ECUDA, "cudaGetDeviceCount", e);
    return n;
}

const char *bnk_last_error_string(bnk_ctx *ctx) {
    if (!ctx) return g_last_error.c_str();
    std::lock_guard<std::mutex> g(ctx->mu);
    g_last_error = ctx->last_error;
    return g_last_error.c_str();
}

int bnk_ctx_create(const bnk_cfg *cfg, bnk_ctx **out) {
    if (!cfg || !out || cfg->struct_size != sizeof(bnk_cfg)) return fail(nullptr, BNK_EINVAL, "bad bnk_cfg");
    if (cfg->max_keypairs == 0 || cfg->max_keypairs > (1u << 24)) return fail(nullptr, BNK_EINVAL, "max_keypairs out of range");
    if (!is_pow2(cfg->replay_ring_blocks) || cfg->replay_ring_blocks < 2 || cfg->replay_ring_blocks > 1024)
        return fail(nullptr, BNK_EINVAL, "replay_ring_blocks must be a power of two in 2..1024");
    if (cfg->flow_capacity && (!is_pow2(cfg->flow_capacity) || cfg->flow_capacity < 16))
        return fail(nullptr, BNK_EINVAL, "flow_capacity must be a power of two >= 16");
    *out = nullptr;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess) return fail(nullptr, BNK_ECUDA, "no usable CUDA device (there is no CPU fallback)", e);
    if (cfg->device_id < 0 || cfg->device_id >= ndev) return fail(nullptr, BNK_EINVAL, "device_id out of range");
    CK(nullptr, cudaSetDevice(cfg->device_id));
    cudaDeviceProp prop;
    CK(nullptr, cudaGetDeviceProperties(&prop, cfg->device_id));
    if (prop.major != 10) return fail(nullptr, BNK_ECUDA, "device is not sm_100: this library carries sm_100a code only");

    bnk_ctx *ctx = new (std::nothrow) bnk_ctx();
    if (!ctx) return fail(nullptr, BNK_ENOMEM, "host allocation failed");
    ctx->cfg = *cfg;
    ctx->device = cfg->device_id;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->launches = 0;
    ctx->aead_mode = 0;
    if (const char *m = getenv("BNK_AEAD_KERNEL")) // tuning and test aid: tpp | wpp
        ctx->aead_mode = !strcmp(m, "tpp") ? 1 : (!strcmp(m, "wpp") ? 2 : 0);
    ctx->host_direct_bytes = 384u << 10; // 256 slots of 1456 bytes and their headroom

    if (const char *m = getenv("BNK_HOST_DIRECT_BYTES")) // largest ring extent served without copies; 0 = never
        ctx->host_direct_bytes = strtoull(m, nullptr, 0);
    if (!prop.unifiedAddressing || !prop.canMapHostMemory) ctx->host_direct_bytes = 0; // pinned memory must have one address
    ctx->aead_side_stream_from = 1u << 18; // below, the seal/open launch is too short for the hand-over between streams to pay
    if (const char *m = getenv("BNK_AEAD_SIDE_STREAM_FROM")) // tuning aid: 0 = seal/open always on the batch's own stream
        ctx->aead_side_stream_from = (uint32_t)strtoul(m, nullptr, 0);
    ctx->prio_low = ctx->prio_high = 0;
    cudaDeviceGetStreamPriorityRange(&ctx->prio_low, &ctx->prio_high);
    ctx->kt = KeypairTables{};
    ctx->ft = FilterTables{};
    const size_t k = cfg->max_keypairs;
    auto bail = [&](const char *what, cudaError_t err) {
        int rc = fail(nullptr, BNK_ECUDA, what, err);
        bnk_ctx_destroy(ctx);
        return rc;
    };
    if ((e = cudaStreamCreateWithFlags(&ctx->admin_stream, cudaStreamNonBlocking)) != cudaSuccess) return bail("stream", e);
    if ((e = cudaEventCreate(&ctx->timer_start)) != cudaSuccess) return bail("event", e);
    if ((e = dev_alloc_zero(&ctx->kt.send_keys, k * 8)) != cudaSuccess) return bail("send_keys", e);
    if ((e = dev_alloc_zero(&ctx->kt.recv_keys, k * 8)) != cudaSuccess) return bail("recv_keys", e);
    if ((e = dev_alloc_zero(&ctx->kt.remote_index, k)) != cudaSuccess) return bail("remote_index", e);
    if ((e = dev_alloc_zero(&ctx->kt.send_counter, k)) != cudaSuccess) return bail("send_counter", e);
    if ((e = dev_alloc_zero(&ctx->kt.replay_last, k)) != cudaSuccess) return bail("replay_last", e);
    if ((e = dev_alloc_zero(&ctx->kt.replay_next, k)) != cudaSuccess) return bail("replay_next", e);
    if ((e = dev_alloc_zero(&ctx->kt.replay_ring, k * cfg->replay_ring_blocks)) != cudaSuccess) return bail("replay_ring", e);
    if ((e = dev_alloc_zero(&ctx->kt.allowed_ip, k)) != cudaSuccess) return bail("allowed_ip", e);
    if ((e = dev_alloc_zero(&ctx->kt.valid, k)) != cudaSuccess) return bail("valid", e);
    uint32_t islots = 16;
    while (islots < 2 * k) islots <<= 1;
    ctx->kt.index_slots = islots;
    ctx->index_keys_host.assign(islots, 0);
    ctx->index_vals_host.assign(islots, 0);
    ctx->index_live = ctx->index_dead = ctx->addr_live = ctx->addr_dead = 0;
    for (auto &h : ctx->flow_dead_hint) h = 0;
    ctx->flow_errors_seen = 0;
    if ((e = dev_alloc_zero(&ctx->kt.index_keys, (size_t)islots)) != cudaSuccess) return bail("index_keys", e);
    if ((e = dev_alloc_zero(&ctx->kt.index_vals, (size_t)islots)) != cudaSuccess) return bail("index_vals", e);
    ctx->kt.addr_slots = islots;
    ctx->addr_host.assign(islots, KeypairTables::AddrEntry{});
    if ((e = dev_alloc_zero(&ctx->kt.addr_tab, (size_t)islots)) != cudaSuccess) return bail("addr_tab", e);
    if ((e = filter_tables_alloc(ctx)) != cudaSuccess) return bail("filter tables", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return bail("sync", e);
    *out = ctx;
    return BNK_SUCCESS;
}

int bnk_ctx_destroy(bnk_ctx *ctx) {
    if (!ctx) return BNK_EINVAL;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    cudaFree(ctx->kt.send_keys);
    cudaFree(ctx->kt.recv_keys);
    cudaFree(ctx->kt.remote_index);
    cudaFree(ctx->kt.send_counter);
    cudaFree(ctx->kt.replay_last);
    cudaFree(ctx->kt.replay_next);
    cudaFree(ctx->kt.replay_ring);
    cudaFree(ctx->kt.allowed_ip);
    cudaFree(ctx->kt.valid);
    cudaFree(ctx->kt.index_keys);
    cudaFree(ctx->kt.index_vals);
    cudaFree(ctx->kt.addr_tab);
    filter_tables_free(ctx);
    if (ctx->timer_start) cudaEventDestroy(ctx->timer_start);
    if (ctx->admin_stream) cudaStreamDestroy(ctx->admin_stream);
    delete ctx;
    return BNK_SUCCESS;
}

int bnk_ctx_synchronize(bnk_ctx *ctx) {
    if (!ctx) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaDeviceSynchronize());
    return BNK_SUCCESS;
}

/* ---- keypairs ---- */
int bnk_keypair_set_many(bnk_ctx *ctx, uint32_t first_slot, uint32_t n, const uint8_t *send_keys,
                         const uint8_t *recv_keys, const uint32_t *remote_index) {
    if (!ctx || !send_keys || !recv_keys || !remote_index) return fail(ctx, BNK_EINVAL, "null argument");
    if ((uint64_t)first_slot + n > ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "keypair slot out of range");
    if (n == 0) return BNK_SUCCESS;
    CK(ctx, cudaSetDevice(ctx->device));
    const uint32_t rb = ctx->cfg.replay_ring_blocks;
    CK(ctx, cudaMemcpy(ctx->kt.send_keys + (size_t)first_slot * 8, send_keys, (size_t)n * 32, cudaMemcpyHostToDevice));
    CK(ctx, cudaMemcpy(ctx->kt.recv_keys + (size_t)first_slot * 8, recv_keys, (size_t)n * 32, cudaMemcpyHostToDevice));
    CK(ctx, cudaMemcpy(ctx->kt.remote_index + first_slot, remote_index, (size_t)n * 4, cudaMemcpyHostToDevice));
    CK(ctx, cudaMemset(ctx->kt.send_counter + first_slot, 0, (size_t)n * 8));
    CK(ctx, cudaMemset(ctx->kt.replay_last + first_slot, 0, (size_t)n * 8));
    CK(ctx, cudaMemset(ctx->kt.replay_ring + (size_t)first_slot * rb, 0, (size_t)n * rb * 8));
    CK(ctx, cudaMemset(ctx->kt.allowed_ip + first_slot, 0, (size_t)n * 4));
    CK(ctx, cudaMemset(ctx->kt.valid + first_slot, 1, (size_t)n));
    return BNK_SUCCESS;
}

int bnk_keypair_set(bnk_ctx *ctx, uint32_t slot, const uint8_t send_key[32], const uint8_t recv_key[32],
                    uint32_t remote_index) {
    return bnk_keypair_set_many(ctx, slot, 1, send_key, recv_key, &remote_index);
}

static int index_drop_slot(bnk_ctx *ctx, uint32_t slot);

int bnk_keypair_clear(bnk_ctx *ctx, uint32_t slot) {
    static const uint8_t zeros[32] = {0};
    int rc = bnk_keypair_set(ctx, slot, zeros, zeros, 0);
    if (rc != BNK_SUCCESS) return rc;
    // no keys: seal and open refuse the slot with BNK_PKT_NO_KEYPAIR, and no receiver index leads to it any more
    CK(ctx, cudaMemset(ctx->kt.valid + slot, 0, 1));
    return index_drop_slot(ctx, slot);
}

int bnk_send_counter_get(bnk_ctx *ctx, uint32_t slot, uint64_t *counter) {
    if (!ctx || !counter || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpy(counter, ctx->kt.send_counter + slot, 8, cudaMemcpyDeviceToHost));
    return BNK_SUCCESS;
}

int bnk_send_counter_set(bnk_ctx *ctx, uint32_t slot, uint64_t counter) {
    if (!ctx || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpy(ctx->kt.send_counter + slot, &counter, 8, cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}

int bnk_keypair_set_allowed_ip(bnk_ctx *ctx, uint32_t slot, uint32_t ipv4) {
    if (!ctx || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpy(ctx->kt.allowed_ip + slot, &ipv4, 4, cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}

// The index table is edited in a host shadow and the touched entry is copied over: updates happen once per
// handshake, lookups once per packet.  A deleted entry keeps its slot as a tombstone so that probe chains stay
// intact; every handshake brings a new random index, so tombstones pile up, and once a quarter of the table is
// tombstones the table is rebuilt without them (otherwise a lookup of an unknown index, which anyone can send,
// would end up walking the whole table).
constexpr uint64_t kIndexLive = 1ull << 32, kIndexDead = 2ull << 32;
static int index_rebuild(bnk_ctx *ctx) {
    const uint32_t slots = ctx->kt.index_slots, mask = slots - 1;
    std::vector<uint64_t> keys(slots, 0);
    std::vector<uint32_t> vals(slots, 0);
    for (uint32_t i = 0; i < slots; i++) {
        const uint64_t k = ctx->index_keys_host[i];
        if ((k >> 32) != 1) continue;
        uint32_t h = index_hash((uint32_t)k) & mask;
        while (keys[h]) h = (h + 1) & mask;
        keys[h] = k;
        vals[h] = ctx->index_vals_host[i];
    }
    ctx->index_keys_host.swap(keys);
    ctx->index_vals_host.swap(vals);
    ctx->index_dead = 0;
    CK(ctx, cudaDeviceSynchronize()); // the whole table moves: not under a running lookup
    CK(ctx, cudaMemcpy(ctx->kt.index_vals, ctx->index_vals_host.data(), (size_t)slots * 4, cudaMemcpyHostToDevice));
    CK(ctx, cudaMemcpy(ctx->kt.index_keys, ctx->index_keys_host.data(), (size_t)slots * 8, cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}
static int index_update(bnk_ctx *ctx, uint32_t local_index, bool insert, uint32_t slot) {
    const uint64_t key = kIndexLive | local_index;
    std::vector<uint64_t> &keys = ctx->index_keys_host;
    const uint32_t mask = ctx->kt.index_slots - 1;
    uint32_t h = index_hash(local_index) & mask;
    int64_t spare = -1, at = -1;
    for (uint32_t probe = 0; probe <= mask; probe++) {
        if (keys[h] == key) {
            at = h;
            break;
        }
        if (keys[h] == kIndexDead && spare < 0) spare = h;
        if (keys[h] == 0) {
            if (spare < 0) spare = h;
            break;
        }
        h = (h + 1) & mask;
    }
    if (!insert) {
        if (at < 0) return BNK_SUCCESS;
        keys[at] = kIndexDead;
        ctx->index_live--;
        ctx->index_dead++;
        CK(ctx, cudaMemcpy(ctx->kt.index_keys + at, &kIndexDead, 8, cudaMemcpyHostToDevice));
        if (ctx->index_dead >= ctx->kt.index_slots / 4) return index_rebuild(ctx);
        return BNK_SUCCESS;
    }
    const bool fresh = at < 0;
    if (at < 0) at = spare;
    if (at < 0) return fail(ctx, BNK_EFULL, "receiver index table full");
    if (fresh) {
        if (keys[at] == kIndexDead) ctx->index_dead--;
        ctx->index_live++;
    }
    // value first, then the key that makes the entry visible
    ctx->index_vals_host[at] = slot;
    CK(ctx, cudaMemcpy(ctx->kt.index_vals + at, &slot, 4, cudaMemcpyHostToDevice));
    keys[at] = key;
    CK(ctx, cudaMemcpy(ctx->kt.index_keys + at, &key, 8, cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}
// bnk_keypair_clear: the indices that led to the slot lead nowhere now
static int index_drop_slot(bnk_ctx *ctx, uint32_t slot) {
    bool any = false;
    for (uint32_t i = 0; i < ctx->kt.index_slots; i++) {
        if ((ctx->index_keys_host[i] >> 32) != 1 || ctx->index_vals_host[i] != slot) continue;
        ctx->index_keys_host[i] = kIndexDead;
        ctx->index_live--;
        ctx->index_dead++;
        any = true;
        CK(ctx, cudaMemcpy(ctx->kt.index_keys + i, &kIndexDead, 8, cudaMemcpyHostToDevice));
    }
    if (any && ctx->index_dead >= ctx->kt.index_slots / 4) return index_rebuild(ctx);
    return BNK_SUCCESS;
}

int bnk_index_set(bnk_ctx *ctx, uint32_t local_index, uint32_t slot) {
    if (!ctx || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    return index_update(ctx, local_index, true, slot);
}

int bnk_index_clear(bnk_ctx *ctx, uint32_t local_index) {
    if (!ctx) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    return index_update(ctx, local_index, false, 0);
}

// byAddr: same host-shadow scheme as the receiver-index table, tombstones reclaimed the same way
constexpr uint32_t kAddrLive = 1u << 16, kAddrDead = 2u << 16;
static int addr_rebuild(bnk_ctx *ctx) {
    const uint32_t slots = ctx->kt.addr_slots, mask = slots - 1;
    std::vector<KeypairTables::AddrEntry> tab(slots, KeypairTables::AddrEntry{});
    for (const KeypairTables::AddrEntry &e : ctx->addr_host) {
        if (!(e.port & kAddrLive)) continue;
        uint32_t h = addr_hash(e.hi, e.lo, e.port & 0xffffu) & mask;
        while (tab[h].port) h = (h + 1) & mask;
        tab[h] = e;
    }
    ctx->addr_host.swap(tab);
    ctx->addr_dead = 0;
    CK(ctx, cudaDeviceSynchronize());
    CK(ctx, cudaMemcpy(ctx->kt.addr_tab, ctx->addr_host.data(), (size_t)slots * sizeof(KeypairTables::AddrEntry),
                       cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}
static int addr_update(bnk_ctx *ctx, const uint8_t addr[16], uint16_t port, bool insert, uint32_t peer) {
    uint64_t hi, lo;
    memcpy(&hi, addr, 8);
    memcpy(&lo, addr + 8, 8);
    const uint32_t live = (uint32_t)port | kAddrLive, dead = kAddrDead;
    std::vector<KeypairTables::AddrEntry> &tab = ctx->addr_host;
    const uint32_t mask = ctx->kt.addr_slots - 1;
    uint32_t h = addr_hash(hi, lo, port) & mask;
    int64_t spare = -1, at = -1;
    for (uint32_t probe = 0; probe <= mask; probe++) {
        const KeypairTables::AddrEntry &e = tab[h];
        if (e.port == live && e.hi == hi && e.lo == lo) {
            at = h;
            break;
        }
        if (e.port == dead && spare < 0) spare = h;
        if (e.port == 0) {
            if (spare < 0) spare = h;
            break;
        }
        h = (h + 1) & mask;
    }
    if (!insert) {
        if (at < 0) return BNK_SUCCESS;
        tab[at].port = dead;
        ctx->addr_live--;
        ctx->addr_dead++;
    } else {
        if (at < 0) {
            at = spare;
            if (at < 0) return fail(ctx, BNK_EFULL, "source address table full");
            if (tab[at].port == dead) ctx->addr_dead--;
            ctx->addr_live++;
        }
        tab[at] = KeypairTables::AddrEntry{hi, lo, live, peer, 0};
    }
    CK(ctx, cudaDeviceSynchronize()); // entries are 32 bytes: never rewrite one under a running kernel
    CK(ctx, cudaMemcpy(ctx->kt.addr_tab + at, &tab[at], sizeof tab[at], cudaMemcpyHostToDevice));
    if (!insert && ctx->addr_dead >= ctx->kt.addr_slots / 4) return addr_rebuild(ctx);
    return BNK_SUCCESS;
}

int bnk_addr_set(bnk_ctx *ctx, const uint8_t addr[16], uint16_t port, uint32_t peer_id) {
    if (!ctx || !addr) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    return addr_update(ctx, addr, port, true, peer_id);
}

int bnk_addr_clear(bnk_ctx *ctx, const uint8_t addr[16], uint16_t port) {
    if (!ctx || !addr) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    return addr_update(ctx, addr, port, false, 0);
}

int bnk_replay_export(bnk_ctx *ctx, uint32_t slot, uint64_t *last, uint64_t *ring) {
    if (!ctx || !last || !ring || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    const uint32_t rb = ctx->cfg.replay_ring_blocks;
    CK(ctx, cudaMemcpy(last, ctx->kt.replay_last + slot, 8, cudaMemcpyDeviceToHost));
    CK(ctx, cudaMemcpy(ring, ctx->kt.replay_ring + (size_t)slot * rb, (size_t)rb * 8, cudaMemcpyDeviceToHost));
    return BNK_SUCCESS;
}

int bnk_replay_import(bnk_ctx *ctx, uint32_t slot, uint64_t last, const uint64_t *ring) {
    if (!ctx || !ring || slot >= ctx->cfg.max_keypairs) return fail(ctx, BNK_EINVAL, "bad slot");
    CK(ctx, cudaSetDevice(ctx->device));
    const uint32_t rb = ctx->cfg.replay_ring_blocks;
    CK(ctx, cudaMemcpy(ctx->kt.replay_last + slot, &last, 8, cudaMemcpyHostToDevice));
    CK(ctx, cudaMemcpy(ctx->kt.replay_ring + (size_t)slot * rb, ring, (size_t)rb * 8, cudaMemcpyHostToDevice));
    return BNK_SUCCESS;
}

/* ---- ACL ---- */
int bnk_acl_set(bnk_ctx *ctx, int enforce, const bnk_acl_tuple *tuples, size_t n) {
    if (!ctx || (n && !tuples)) return fail(ctx, BNK_EINVAL, "null tuples");
    if (ctx->cfg.max_acl_tuples && n > ctx->cfg.max_acl_tuples) return fail(ctx, BNK_EFULL, "more tuples than max_acl_tuples");
    CK(ctx, cudaSetDevice(ctx->device));
    const int rc = filter_acl_upload(ctx, enforce, tuples, n);
    if (rc != BNK_SUCCESS) return fail(ctx, rc, "rule table upload failed");
    return BNK_SUCCESS;
}

int bnk_flows_clear(bnk_ctx *ctx) {
    if (!ctx) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    std::unique_lock<std::shared_mutex> tables(ctx->submit_mu);
    CK(ctx, cudaDeviceSynchronize());
    CK(ctx, filter_flows_clear(ctx, ctx->admin_stream));
    return BNK_SUCCESS;
}

int bnk_flows_count(bnk_ctx *ctx, uint64_t *live) {
    if (!ctx || !live) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaDeviceSynchronize());
    unsigned long long v = 0;
    CK(ctx, cudaMemcpy(&v, ctx->ft.flow_live, sizeof v, cudaMemcpyDeviceToHost));
    *live = v;
    return BNK_SUCCESS;
}

int bnk_flows_export(bnk_ctx *ctx, bnk_flow_entry *out, size_t capacity, size_t *count) {
    if (!ctx || !count || (capacity && !out)) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    std::unique_lock<std::shared_mutex> tables(ctx->submit_mu);
    CK(ctx, cudaDeviceSynchronize());
    const int rc = filter_flows_export(ctx, out, capacity, count);
    return rc == BNK_SUCCESS ? rc : fail(ctx, rc, "flow table export failed");
}

int bnk_flows_import(bnk_ctx *ctx, const bnk_flow_entry *entries, size_t n) {
    if (!ctx || (n && !entries)) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    std::unique_lock<std::shared_mutex> tables(ctx->submit_mu);
    CK(ctx, cudaDeviceSynchronize());
    const int rc = filter_flows_import(ctx, entries, n);
    return rc == BNK_SUCCESS ? rc : fail(ctx, rc, rc == BNK_EFULL ? "flow table full" : "flow table import failed");
}

int bnk_table_stats_get(bnk_ctx *ctx, bnk_table_stats *out) {
    if (!ctx || !out) return BNK_EINVAL;
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaDeviceSynchronize());
    memset(out, 0, sizeof *out);
    CK(ctx, filter_flow_stats(ctx, &out->flow_live, out->flow_used, out->flow_dead));
    out->flow_capacity = ctx->ft.flow_capacity;
    out->index_live = ctx->index_live;
    out->index_dead = ctx->index_dead;
    out->index_slots = ctx->kt.index_slots;
    out->addr_live = ctx->addr_live;
    out->addr_dead = ctx->addr_dead;
    out->addr_slots = ctx->kt.addr_slots;
    return BNK_SUCCESS;
}

/* ---- batches ---- */
int bnk_batch_destroy(bnk_batch *b) {
    if (!b) return BNK_EINVAL;
    cudaSetDevice(b->ctx->device);
    direct_done(b);
    {
        std::unique_lock<std::shared_mutex> tables(b->ctx->submit_mu); // not while table maintenance walks the registry
        std::lock_guard<std::mutex> g(b->ctx->mu);
        std::vector<bnk_batch *> &all = b->ctx->batches;
        for (size_t i = 0; i < all.size(); i++)
            if (all[i] == b) {
                all.erase(all.begin() + i);
                break;
            }
    }
    if (b->stream) cudaStreamSynchronize(b->stream);
    cudaFreeHost(b->host.src_addr);
    cudaFreeHost(b->h_desc);
    cudaFree(b->d_desc);
    cudaFreeHost(b->h_flow);
    cudaFreeHost(b->h_stats);
    cudaFree(b->d_stats);
    cudaFreeHost(b->h_gso);
    DeviceBatch &d = b->dev;
    cudaFree(d.src_addr);
    cudaFree(d.order);
    cudaFree(d.order_tmp);
    cudaFree(d.keys_tmp);
    cudaFree(d.sorted_counter);
    cudaFree(d.replay_state);
    cudaFree(d.replay_hash);
    cudaFree(d.replay_tile_head);
    cudaFree(d.replay_tile_max);
    cudaFree(d.replay_tile_carry);
    cudaFree(d.hist);
    cudaFree(d.len_order);
    cudaFree(d.counters32);
    cudaFree(d.gso);
    if (b->k_begin) cudaEventDestroy(b->k_begin);
    if (b->k_end) cudaEventDestroy(b->k_end);
    if (b->a_begin) cudaEventDestroy(b->a_begin);
    if (b->a_end) cudaEventDestroy(b->a_end);
    if (b->t_end) cudaEventDestroy(b->t_end);
    if (b->ev_fork) cudaEventDestroy(b->ev_fork);
    if (b->ev_join) cudaEventDestroy(b->ev_join);
    if (b->ev_fence) cudaEventDestroy(b->ev_fence);
    if (b->ev_aead_go) cudaEventDestroy(b->ev_aead_go);
    if (b->ev_aead_done) cudaEventDestroy(b->ev_aead_done);
    if (b->aead_stream) cudaStreamDestroy(b->aead_stream);
    if (b->aux_stream) cudaStreamDestroy(b->aux_stream);
    if (b->stream) cudaStreamDestroy(b->stream);
    delete b;
    return BNK_SUCCESS;
}

int bnk_batch_create(bnk_ctx *ctx, uint32_t max_pkts, uint64_t ring_bytes, bnk_batch **out) {
    if (!ctx || !out || max_pkts == 0 || ring_bytes == 0) return fail(ctx, BNK_EINVAL, "bad batch size");
    if (ring_bytes > 0xffffffffull || (ring_bytes & 15)) return fail(ctx, BNK_EINVAL, "ring_bytes must be a multiple of 16 below 4 GiB");
    *out = nullptr;
    CK(ctx, cudaSetDevice(ctx->device));
    bnk_batch *b = new (std::nothrow) bnk_batch();
    if (!b) return fail(ctx, BNK_ENOMEM, "host allocation failed");
    memset(static_cast<void *>(b), 0, sizeof *b);
    b->ctx = ctx;
    b->max_pkts = max_pkts;
    b->ring_bytes = ring_bytes;
    const size_t n = max_pkts;
    cudaError_t e = cudaSuccess;
    auto H = [&](void **p, size_t bytes) {
        if (e == cudaSuccess) e = cudaHostAlloc(p, bytes, cudaHostAllocDefault);
        if (e == cudaSuccess) memset(*p, 0, bytes);
    };
    auto D = [&](void **p, size_t bytes) {
        if (e == cudaSuccess) e = cudaMalloc(p, bytes);
        if (e == cudaSuccess) e = cudaMemset(*p, 0, bytes);
    };
    // One slab per side: the descriptor arrays, then the ring.  A batch whose descriptor slab is small moves
    // descriptors and ring with one copy each way (joint_copy); otherwise the descriptor fields a call needs
    // move as one run or field by field (desc_copy).
    b->npad = (max_pkts + 15u) & ~15u;
    const size_t np = b->npad;
    b->desc_room = (25 * np + 255) & ~(size_t)255;
    b->joint_copy = b->desc_room <= 64u * 1024;
    H((void **)&b->h_desc, b->desc_room + ring_bytes);
    if (e == cudaSuccess) {
        b->host.ring = b->h_desc + b->desc_room;
        b->host.off = reinterpret_cast<uint32_t *>(b->h_desc);
        b->host.len = reinterpret_cast<uint32_t *>(b->h_desc + 4 * np);
        b->host.slot = reinterpret_cast<uint32_t *>(b->h_desc + 8 * np);
        b->host.counter = reinterpret_cast<uint64_t *>(b->h_desc + 12 * np);
        b->host.out_len = reinterpret_cast<uint32_t *>(b->h_desc + 20 * np);
        b->host.status = b->h_desc + 24 * np;
    }
    H((void **)&b->host.src_addr, n * BNK_SRC_ADDR_STRIDE);
    H((void **)&b->h_flow, sizeof(FlowReport));
    H((void **)&b->h_stats, sizeof(bnk_batch_stats));
    H((void **)&b->h_gso, n * sizeof(bnk_gso_super));
    b->host.ring_bytes = ring_bytes;
    b->host.max_pkts = max_pkts;
    DeviceBatch &d = b->dev;
    D((void **)&b->d_desc, b->desc_room + ring_bytes);
    if (e == cudaSuccess) {
        d.ring = b->d_desc + b->desc_room;
        d.off = reinterpret_cast<uint32_t *>(b->d_desc);
        d.len = reinterpret_cast<uint32_t *>(b->d_desc + 4 * np);
        d.slot = reinterpret_cast<uint32_t *>(b->d_desc + 8 * np);
        d.counter = reinterpret_cast<uint64_t *>(b->d_desc + 12 * np);
        d.out_len = reinterpret_cast<uint32_t *>(b->d_desc + 20 * np);
        d.status = b->d_desc + 24 * np;
    }
    D((void **)&d.src_addr, n * BNK_SRC_ADDR_STRIDE);
    D((void **)&d.order, n * 4);
    D((void **)&d.order_tmp, n * 4);
    D((void **)&d.keys_tmp, 2 * n * 4);
    D((void **)&d.sorted_counter, n * 8);
    D((void **)&d.replay_state, n);
    D((void **)&d.replay_hash, (size_t)replay_hash_capacity(max_pkts) * 4);
    D((void **)&d.replay_tile_head, ((size_t)replay_scan_tiles(max_pkts) + 1) * 4);
    D((void **)&d.replay_tile_max, (size_t)replay_scan_tiles(max_pkts) * 8);
    D((void **)&d.replay_tile_carry, (size_t)replay_scan_tiles(max_pkts) * 8);
    D((void **)&d.hist, (size_t)512 * group_sort_chunks(max_pkts) * 4); // histogram columns + one row of totals
    D((void **)&d.len_order, n * 4);
    D((void **)&d.counters32, 2048 * 4);
    D((void **)&d.gso, n * sizeof(bnk_gso_super));
    D((void **)&b->d_stats, 20 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&b->stream, cudaStreamNonBlocking, ctx->prio_high);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&b->aux_stream, cudaStreamNonBlocking, ctx->prio_high);
    if (e == cudaSuccess && ctx->aead_side_stream_from && max_pkts >= ctx->aead_side_stream_from && ctx->prio_low != ctx->prio_high) {
        e = cudaStreamCreateWithPriority(&b->aead_stream, cudaStreamNonBlocking, ctx->prio_low);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ev_aead_go, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ev_aead_done, cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ev_join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b->ev_fence, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&b->k_begin);
    if (e == cudaSuccess) e = cudaEventCreate(&b->k_end);
    if (e == cudaSuccess) e = cudaEventCreate(&b->t_end);
    if (e == cudaSuccess) e = cudaEventCreate(&b->a_begin);
    if (e == cudaSuccess) e = cudaEventCreate(&b->a_end);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        int rc = fail(ctx, e == cudaErrorMemoryAllocation ? BNK_ENOMEM : BNK_ECUDA, "batch allocation", e);
        bnk_batch_destroy(b);
        return rc;
    }
    {
        std::unique_lock<std::shared_mutex> tables(ctx->submit_mu);
        std::lock_guard<std::mutex> g(ctx->mu);
        ctx->batches.push_back(b);
    }
    *out = b;
    return BNK_SUCCESS;
}

int bnk_batch_view_get(bnk_batch *b, bnk_batch_view *out) {
    if (!b || !out) return BNK_EINVAL;
    *out = b->host;
    return BNK_SUCCESS;
}

int bnk_batch_upload(bnk_batch *b, uint32_t npkts) {
    int rc = begin_submit(b, npkts);
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    const size_t n = npkts;
    const uint64_t ext = ring_extent(b, npkts, 64);
    if (ext) CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, b->stream));
    if (n) {
        CK(ctx, desc_copy(b, n, D_OFF, b->dev_stale ? D_STATUS : D_COUNTER, true, b->stream));
    }
    b->dev_stale = false;
    return BNK_SUCCESS;
}

int bnk_batch_download(bnk_batch *b, uint32_t npkts) {
    int rc = begin_submit(b, npkts);
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    const size_t n = npkts;
    if (b->dev_stale) return BNK_SUCCESS; // the last submit already left its results in the host arrays
    const uint64_t ext = ring_extent(b, npkts, 64);
    if (ext) CK(ctx, cudaMemcpyAsync(b->host.ring, b->dev.ring, ext, cudaMemcpyDeviceToHost, b->stream));
    if (n) {
        CK(ctx, desc_copy(b, n, D_COUNTER, D_STATUS, false, b->stream));
    }
    return BNK_SUCCESS;
}

int bnk_seal_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns) {
    const bool device_only = (flags & BNK_F_NO_H2D) && (flags & BNK_F_NO_D2H);
    int rc = begin_submit(b, npkts, !device_only);
    if (rc) return rc;
    if (flags & BNK_F_NOTE_OUTBOUND) CK(b->ctx, filter_flows_maintain(b, b->stream));
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    const size_t n = npkts;
    // header room + payload + padding (< 16) + tag
    const bool refresh = b->dev_stale; // the device copies are behind the host arrays: upload whatever the flags say
    const uint64_t ext = (device_only && !refresh) ? 0 : ring_extent(b, npkts, 16 + 16 + 16);
    const bool direct = host_direct(b, npkts, flags, ext);
    HostAlias alias(b, direct);
    if (!direct && (!(flags & BNK_F_NO_H2D) || refresh) && n) {
        if (b->joint_copy) {
            CK(ctx, cudaMemcpyAsync(b->d_desc, b->h_desc, b->desc_room + ext, cudaMemcpyHostToDevice, s));
        } else {
            CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
            CK(ctx, desc_copy(b, n, D_OFF, refresh ? D_STATUS : (flags & BNK_F_ASSIGN_COUNTERS) ? D_SLOT : D_COUNTER, true, s));
        }
        b->dev_stale = false;
    }
    if (b->order_wait) CK(ctx, cudaStreamWaitEvent(s, b->order_wait, 0));
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    if (flags & BNK_F_NOTE_OUTBOUND) {
        CK(ctx, launch_filter_note(b, npkts, now_unix_ns, s));
        CK(ctx, launch_flow_report(b, s));
    }
    const uint32_t *order = nullptr;
    const bool side_order = (flags & BNK_F_SORT_BY_LENGTH) && (flags & BNK_F_ASSIGN_COUNTERS) && npkts > 4096;
    if (side_order) { // the length classes need only len[]: they are built beside the grouping for the counters
        CK(ctx, cudaEventRecord(b->ev_fork, s));
        CK(ctx, cudaStreamWaitEvent(b->aux_stream, b->ev_fork, 0));
        CK(ctx, launch_length_order(b, npkts, b->dev.len, false, b->aux_stream));
        CK(ctx, cudaEventRecord(b->ev_join, b->aux_stream));
        order = b->dev.len_order;
    }
    if (flags & BNK_F_ASSIGN_COUNTERS) CK(ctx, launch_assign_counters(b, npkts, s));
    if (side_order) {
        CK(ctx, cudaStreamWaitEvent(s, b->ev_join, 0));
    } else if (flags & BNK_F_SORT_BY_LENGTH) {
        CK(ctx, launch_length_order(b, npkts, b->dev.len, false, s));
        order = b->dev.len_order;
    }
    const bool side = b->aead_stream && npkts >= ctx->aead_side_stream_from;
    cudaStream_t as = side ? b->aead_stream : s;
    if (side) {
        CK(ctx, cudaEventRecord(b->ev_aead_go, s));
        CK(ctx, cudaStreamWaitEvent(as, b->ev_aead_go, 0));
    }
    if (timed) CK(ctx, cudaEventRecord(b->a_begin, as));
    CK(ctx, launch_seal(aead_args(b, npkts, false, order), as, ctx));
    if (timed) CK(ctx, cudaEventRecord(b->a_end, as));
    if (side) {
        CK(ctx, cudaEventRecord(b->ev_aead_done, as));
        CK(ctx, cudaStreamWaitEvent(s, b->ev_aead_done, 0));
    }
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    b->aead_timed = timed;
    CK(ctx, tally_if_asked(b, npkts, flags, s));
    if (b->order_record) CK(ctx, cudaEventRecord(b->order_record, s));
    if (!direct && !(flags & BNK_F_NO_D2H) && n) {
        if (b->joint_copy) {
            CK(ctx, cudaMemcpyAsync(b->h_desc, b->d_desc, b->desc_room + ext, cudaMemcpyDeviceToHost, s));
        } else {
            CK(ctx, cudaMemcpyAsync(b->host.ring, b->dev.ring, ext, cudaMemcpyDeviceToHost, s));
            CK(ctx, desc_copy(b, n, D_COUNTER, D_STATUS, false, s));
        }
    }
    return BNK_SUCCESS;
}

int bnk_open_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns) {
    const bool device_only = (flags & BNK_F_NO_H2D) && (flags & BNK_F_NO_D2H);
    int rc = begin_submit(b, npkts, !device_only);
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    const size_t n = npkts;
    const bool refresh = b->dev_stale;
    const uint64_t ext = (device_only && !refresh) ? 0 : ring_extent(b, npkts, (flags & BNK_F_USE_OUT_LEN) ? 48 : 0);
    const bool direct = host_direct(b, npkts, flags, ext);
    HostAlias alias(b, direct);
    // BNK_F_USE_OUT_LEN reads the lengths a seal left on the device: an upload beside it must not bring the
    // host's out_len along, so it moves the fields one by one instead of the whole slab.
    if (!direct && (!(flags & BNK_F_NO_H2D) || refresh) && n) {
        if (b->joint_copy && !((flags & BNK_F_USE_OUT_LEN) && !refresh)) {
            CK(ctx, cudaMemcpyAsync(b->d_desc, b->h_desc, b->desc_room + ext, cudaMemcpyHostToDevice, s));
        } else {
            CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
            CK(ctx, desc_copy(b, n, D_OFF, refresh ? D_STATUS : (flags & BNK_F_DEMUX_INDEX) ? D_LEN : D_SLOT, true, s));
        }
        b->dev_stale = false;
    }
    if (b->order_wait) CK(ctx, cudaStreamWaitEvent(s, b->order_wait, 0));
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    const uint32_t *order = nullptr;
    AeadArgs oa = aead_args(b, npkts, true, nullptr);
    if (flags & BNK_F_USE_OUT_LEN) oa.len = b->dev.out_len;
    if (flags & BNK_F_DEMUX_INDEX) CK(ctx, launch_demux_index(b, npkts, oa.len, s));
    if (flags & BNK_F_SORT_BY_LENGTH) {
        CK(ctx, launch_length_order(b, npkts, oa.len, true, s));
        order = b->dev.len_order;
    }
    oa.order = order;
    const bool replay_fused = (flags & BNK_F_REPLAY) && replay_is_one_launch(npkts);
    if ((flags & BNK_F_REPLAY) && !replay_fused) {
        // grouping by keypair needs only the descriptors: it runs on the side stream beside the open kernel
        CK(ctx, cudaEventRecord(b->ev_fork, s));
        CK(ctx, cudaStreamWaitEvent(b->aux_stream, b->ev_fork, 0));
        CK(ctx, launch_group_by_slot(b, npkts, false, b->aux_stream));
        CK(ctx, cudaEventRecord(b->ev_join, b->aux_stream));
    }
    const bool side = b->aead_stream && npkts >= ctx->aead_side_stream_from;
    cudaStream_t as = side ? b->aead_stream : s;
    if (side) {
        CK(ctx, cudaEventRecord(b->ev_aead_go, s));
        CK(ctx, cudaStreamWaitEvent(as, b->ev_aead_go, 0));
    }
    if (timed) CK(ctx, cudaEventRecord(b->a_begin, as));
    CK(ctx, launch_open(oa, as, ctx));
    if (timed) CK(ctx, cudaEventRecord(b->a_end, as));
    if (side) {
        CK(ctx, cudaEventRecord(b->ev_aead_done, as));
        CK(ctx, cudaStreamWaitEvent(s, b->ev_aead_done, 0));
    }
    b->aead_timed = timed;
    if (replay_fused) { // small batch: one launch sorts and walks; the stream hand-over would cost more than it hides
        CK(ctx, launch_group_and_replay(b, npkts, s));
    } else if (flags & BNK_F_REPLAY) {
        CK(ctx, cudaStreamWaitEvent(s, b->ev_join, 0));
        CK(ctx, launch_replay(b, npkts, s));
    }
    if (flags & BNK_F_INNER_CHECK) CK(ctx, launch_inner_check(b, npkts, s));
    if (flags & BNK_F_CHECK_INBOUND) CK(ctx, launch_filter_check(b, npkts, now_unix_ns, true, s));
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    CK(ctx, tally_if_asked(b, npkts, flags, s));
    if (b->order_record) CK(ctx, cudaEventRecord(b->order_record, s));
    if (!direct && !(flags & BNK_F_NO_D2H) && n) {
        if (b->joint_copy) {
            CK(ctx, cudaMemcpyAsync(b->h_desc, b->d_desc, b->desc_room + ext, cudaMemcpyDeviceToHost, s));
        } else {
            CK(ctx, cudaMemcpyAsync(b->host.ring, b->dev.ring, ext, cudaMemcpyDeviceToHost, s));
            CK(ctx, desc_copy(b, n, (flags & BNK_F_DEMUX_INDEX) ? D_SLOT : D_COUNTER, D_STATUS, false, s));
        }
    }
    return BNK_SUCCESS;
}

int bnk_filter_note_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns) {
    int rc = begin_submit(b, npkts);
    if (rc) return rc;
    CK(b->ctx, filter_flows_maintain(b, b->stream));
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    const size_t n = npkts;
    const bool refresh = b->dev_stale;
    const uint64_t ext = (!(flags & BNK_F_NO_H2D) || refresh) ? ring_extent(b, npkts, 16) : 0;
    // the filter reads at most 28 bytes of a packet: always cheaper through the bus than a copy of the ring
    const bool direct = host_direct(b, npkts, flags, 0);
    HostAlias alias(b, direct);
    if (!direct && (!(flags & BNK_F_NO_H2D) || refresh) && n) {
        CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
        if (refresh) {
            CK(ctx, desc_copy(b, n, D_OFF, D_STATUS, true, s));
            b->dev_stale = false;
        } else {
            CK(ctx, cudaMemcpyAsync(b->dev.off, b->host.off, n * 4, cudaMemcpyHostToDevice, s));
            CK(ctx, cudaMemcpyAsync(b->dev.len, b->host.len, n * 4, cudaMemcpyHostToDevice, s));
        }
    }
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    CK(ctx, launch_filter_note(b, npkts, now_unix_ns, s));
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    CK(ctx, launch_flow_report(b, s));
    return BNK_SUCCESS;
}

int bnk_filter_check_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns) {
    int rc = begin_submit(b, npkts);
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    const size_t n = npkts;
    const bool refresh = b->dev_stale;
    const uint64_t ext = (!(flags & BNK_F_NO_H2D) || refresh) ? ring_extent(b, npkts, 16) : 0;
    // the filter reads at most 28 bytes of a packet: always cheaper through the bus than a copy of the ring
    const bool direct = host_direct(b, npkts, flags, 0);
    HostAlias alias(b, direct);
    if (!direct && (!(flags & BNK_F_NO_H2D) || refresh) && n) {
        CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
        if (refresh) {
            CK(ctx, desc_copy(b, n, D_OFF, D_STATUS, true, s));
            b->dev_stale = false;
        } else {
            CK(ctx, cudaMemcpyAsync(b->dev.off, b->host.off, n * 4, cudaMemcpyHostToDevice, s));
            CK(ctx, cudaMemcpyAsync(b->dev.len, b->host.len, n * 4, cudaMemcpyHostToDevice, s));
        }
    }
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    CK(ctx, launch_filter_check(b, npkts, now_unix_ns, false, s));
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    CK(ctx, tally_if_asked(b, npkts, flags, s));
    if (!direct && !(flags & BNK_F_NO_D2H) && n)
        CK(ctx, cudaMemcpyAsync(b->host.status, b->dev.status, n, cudaMemcpyDeviceToHost, s));
    return BNK_SUCCESS;
}

int bnk_classify_submit(bnk_batch *b, uint32_t npkts, uint32_t flags) {
    int rc = begin_submit(b, npkts);
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    const size_t n = npkts;
    if ((!(flags & BNK_F_NO_H2D) || b->dev_stale) && n) {
        const uint64_t ext = ring_extent(b, npkts, 0);
        if (ext) CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
        if (b->dev_stale) { // a submit ran on the host arrays: every device descriptor field is behind
            CK(ctx, desc_copy(b, n, D_OFF, D_STATUS, true, s));
        } else {
            CK(ctx, cudaMemcpyAsync(b->dev.off, b->host.off, n * 4, cudaMemcpyHostToDevice, s));
            CK(ctx, cudaMemcpyAsync(b->dev.len, b->host.len, n * 4, cudaMemcpyHostToDevice, s));
        }
        b->dev_stale = false;
        CK(ctx, cudaMemcpyAsync(b->dev.src_addr, b->host.src_addr, n * BNK_SRC_ADDR_STRIDE, cudaMemcpyHostToDevice, s));
    }
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    CK(ctx, launch_classify(b, npkts, s));
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    CK(ctx, tally_if_asked(b, npkts, flags, s));
    if (!(flags & BNK_F_NO_D2H) && n) {
        CK(ctx, cudaMemcpyAsync(b->host.slot, b->dev.slot, n * 4, cudaMemcpyDeviceToHost, s));
        CK(ctx, cudaMemcpyAsync(b->host.status, b->dev.status, n, cudaMemcpyDeviceToHost, s));
    }
    return BNK_SUCCESS;
}

int bnk_gso_split_submit(bnk_batch *b, const bnk_gso_super *supers, uint32_t n_super, uint32_t n_pkts,
                         uint32_t flags) {
    int rc = begin_submit(b, n_pkts, true); // the descriptor staging area is host memory in any case
    if (rc) return rc;
    SubmitScope scope(b);
    bnk_ctx *ctx = b->ctx;
    cudaStream_t s = b->stream;
    const bool timed = (flags & BNK_F_TIMED) != 0;
    if (n_super > b->max_pkts || (n_super && !supers)) return fail(ctx, BNK_EINVAL, "bad super-packet list");
    const size_t n = n_pkts;
    if (!(flags & BNK_F_NO_H2D) || b->dev_stale) {
        const bool refresh = b->dev_stale;
        b->dev_stale = false;
        // the ring span holds the segments' slots and the super-packets
        uint64_t ext = ring_extent(b, n_pkts, 16 + 16 + 16);
        for (uint32_t j = 0; j < n_super; j++) {
            const uint64_t e = (uint64_t)supers[j].src_off + supers[j].src_len;
            if (e > b->ring_bytes) return fail(ctx, BNK_EINVAL, "super-packet lies outside the ring");
            if (e > ext) ext = e;
        }
        ext = (ext + 15) & ~15ull;
        if (ext > b->ring_bytes) ext = b->ring_bytes;
        if (ext) CK(ctx, cudaMemcpyAsync(b->dev.ring, b->host.ring, ext, cudaMemcpyHostToDevice, s));
        if (n && refresh) {
            CK(ctx, desc_copy(b, n, D_OFF, D_STATUS, true, s));
        } else if (n) {
            CK(ctx, cudaMemcpyAsync(b->dev.off, b->host.off, n * 4, cudaMemcpyHostToDevice, s));
            CK(ctx, cudaMemcpyAsync(b->dev.len, b->host.len, n * 4, cudaMemcpyHostToDevice, s));
            CK(ctx, cudaMemcpyAsync(b->dev.slot, b->host.slot, n * 4, cudaMemcpyHostToDevice, s));
        }
    }
    if (n_super) {
        memcpy(b->h_gso, supers, (size_t)n_super * sizeof(bnk_gso_super));
        CK(ctx, cudaMemcpyAsync(b->dev.gso, b->h_gso, (size_t)n_super * sizeof(bnk_gso_super), cudaMemcpyHostToDevice, s));
    }
    if (timed) CK(ctx, cudaEventRecord(b->k_begin, s));
    CK(ctx, launch_gso_split(b, n_super, n_pkts, s));
    if (timed) CK(ctx, cudaEventRecord(b->k_end, s));
    b->kernel_timed = timed;
    return BNK_SUCCESS;
}

int bnk_wait(bnk_batch *b, uint64_t timeout_ns) {
    if (!b) return BNK_EINVAL;
    if (!b->in_flight) return BNK_SUCCESS;
    bnk_ctx *ctx = b->ctx;
    CK(ctx, cudaSetDevice(ctx->device));
    if (timeout_ns == UINT64_MAX) {
        CK(ctx, cudaStreamSynchronize(b->stream));
    } else {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
        for (;;) {
            cudaError_t e = cudaStreamQuery(b->stream);
            if (e == cudaSuccess) break;
            if (e != cudaErrorNotReady) return fail(ctx, BNK_ECUDA, "cudaStreamQuery", e);
            if (std::chrono::steady_clock::now() >= deadline) return BNK_ETIMEDOUT;
            std::this_thread::yield();
        }
    }
    b->in_flight = false;
    direct_done(b);
    if (b->flow_reported) { // what the device said about the flow table after this batch: input of the next compaction
        b->flow_reported = false;
        for (int c = 0; c < 3; c++) ctx->flow_dead_hint[c] = b->h_flow->dead[c];
        int seen = ctx->flow_errors_seen.load();
        const int now_failed = b->h_flow->error;
        while (now_failed > seen && !ctx->flow_errors_seen.compare_exchange_weak(seen, now_failed)) {}
        if (now_failed > seen) return fail(ctx, BNK_EFULL, "flow table full: some outbound flows were not recorded");
    }
    return BNK_SUCCESS;
}

int bnk_batch_stats_get(bnk_batch *b, bnk_batch_stats *out) {
    if (!b || !out) return BNK_EINVAL;
    if (b->in_flight) return fail(b->ctx, BNK_EBUSY, "batch has work in flight; call bnk_wait first");
    if (!b->stats_pending) return fail(b->ctx, BNK_EINVAL, "the batch's last submit was not made with BNK_F_STATS");
    *out = *b->h_stats;
    return BNK_SUCCESS;
}

/* ---- stage timing ---- */
int bnk_batch_last_kernel_ms(bnk_batch *b, float *ms) {
    if (!b || !ms) return BNK_EINVAL;
    if (!b->kernel_timed) return fail(b->ctx, BNK_EINVAL, "no submit has been timed on this batch");
    CK(b->ctx, cudaSetDevice(b->ctx->device));
    CK(b->ctx, cudaEventSynchronize(b->k_end));
    CK(b->ctx, cudaEventElapsedTime(ms, b->k_begin, b->k_end));
    return BNK_SUCCESS;
}

int bnk_batch_last_aead_ms(bnk_batch *b, float *ms) {
    if (!b || !ms) return BNK_EINVAL;
    if (!b->aead_timed) return fail(b->ctx, BNK_EINVAL, "no seal/open has been submitted on this batch");
    CK(b->ctx, cudaSetDevice(b->ctx->device));
    CK(b->ctx, cudaEventSynchronize(b->a_end));
    CK(b->ctx, cudaEventElapsedTime(ms, b->a_begin, b->a_end));
    return BNK_SUCCESS;
}

int bnk_kernel_launch_count(bnk_ctx *ctx, uint64_t *count) {
    if (!ctx || !count) return BNK_EINVAL;
    *count = ctx->launches.load();
    return BNK_SUCCESS;
}

} // extern "C"
