// A submit queue below the C ABI (declared in include/bnk_gpu.h): callers hand in batches of the size the
// reference works with (conn.IdealBatchSize = 128 packets per tun.Device.Read / conn.ReceiveFunc call,
// internal/magicsock/bind.go:97,372-377), from as many threads as they like; the queue packs them into GPU
// batches that are worth a launch and gives every caller its own packets back.
//
// Why: one 128-packet submit costs the same handful of driver calls and the same two trips over the host link as
// a submit of a few thousand packets, and while such a small batch is on its way the GPU does nothing else.
// Here callers copy their packets into the pinned ring of the GPU batch that is filling.  When the device is idle
// the batch goes as it is (a lone caller waits for nobody); while something is in flight the batch keeps filling
// until it holds `min_fill` packets (by default one upstream batch of 128) and a slot on the device is free, or its
// first packet has waited kGatherNs, whichever comes first, and
// at the latest when it is full (under load batches grow by themselves).  Up to `depth` GPU batches are in flight, each
// on its own stream, so the upload of one runs beside the kernels of the one in front and the download of the
// one before; the KERNELS of consecutive batches are chained with events, which keeps what the library promises
// per keypair: nonces in submit order, replay verdicts in arrival order.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <new>
#include <thread>
#include <vector>

#include "bnk_internal.cuh"

namespace {

enum State : int { FREE, FILLING, CLOSED, IN_FLIGHT, DONE };

struct GpuBatch {
    bnk_batch *b = nullptr;
    bnk_batch_view v{};
    cudaEvent_t kernels_done = nullptr; // recorded behind the batch's last kernel
    std::atomic<int> state{FREE};       // written under the queue's lock; its callers watch it without
    uint32_t reserved = 0;              // packets handed out to callers
    std::atomic<uint32_t> filled{0};    // of those, copied in
    uint32_t users = 0;                 // caller batches whose results have not been collected
    uint32_t gen = 0;                   // how often the batch has been reused (part of the ticket)
    int64_t now = 0;
    int rc = BNK_SUCCESS;
    std::chrono::steady_clock::time_point first_at; // when the first caller arrived
};

constexpr uint32_t kMaxQueuePkts = 32768; // ticket fields are 16 bits
// How long the first packet of a GPU batch may wait for company while another batch is on the device.  A GPU
// batch costs ~40 us of driver calls on the submitting thread however small it is; a round trip of a batch takes
// ~100 us; so a few tens of microseconds of gathering cost little latency and are what makes batches worth a launch.
constexpr std::chrono::nanoseconds kGatherNs(40000);
constexpr uint32_t kRotationExtra = 6; // GPU batches beyond `depth`: filling, and done but not yet emptied by their callers

inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#else
    std::this_thread::yield();
#endif
}

// The critical sections below are a few dozen instructions and contain no system or driver call, and the threads
// that contend are callers that would otherwise sit in a driver wait loop: a lock that spins costs a fraction of a
// microsecond, a sleeping one costs a wake-up (tens of microseconds on a virtual machine) on every hand-over.
class SpinLock {
  public:
    void lock() {
        for (uint32_t spins = 0; flag_.exchange(true, std::memory_order_acquire); ++spins) {
            while (flag_.load(std::memory_order_relaxed)) {
                if (++spins & 0x3ffu) cpu_relax();
                else std::this_thread::yield(); // more threads than cores: let the holder run
            }
        }
    }
    void unlock() { flag_.store(false, std::memory_order_release); }

  private:
    std::atomic<bool> flag_{false};
};
struct Locked {
    explicit Locked(SpinLock &l) : l_(l) { l_.lock(); }
    ~Locked() { l_.unlock(); }
    SpinLock &l_;
};

// fixed-capacity first-in first-out list of batch indices (no allocation under the lock)
struct IndexFifo {
    std::vector<uint32_t> slot;
    uint32_t head = 0, count = 0;
    bool empty() const { return count == 0; }
    uint32_t front() const { return slot[head]; }
    void push(uint32_t v) { slot[(head + count++) % slot.size()] = v; }
    void pop() { head = (head + 1) % slot.size(); --count; }
};

} // namespace

// No thread of its own: the queue moves inside the calls of its users.  Whoever hands packets in or waits for a
// ticket also looks whether a GPU batch is ready to go (and submits it) and whether the oldest one in flight has
// come back (and marks it done); a caller that waits does so by watching its batch's state word and taking those
// two turns in between, the way it would otherwise spin inside the driver's own wait.
struct bnk_queue {
    bnk_ctx *ctx;
    bnk_queue_cfg cfg;
    uint32_t slot_bytes;
    std::vector<GpuBatch> gb;
    SpinLock mu;
    uint32_t cur = 0;    // the batch that is filling (or will be, once it is free)
    IndexFifo closed;    // full or cut off, waiting for the device, in order
    IndexFifo inflight;  // submitted, in order
    int last_submitted = -1;
    uint64_t n_gpu_batches = 0, n_packets = 0, n_caller_batches = 0;
    // mirrors that let a waiting caller decide without the lock whether a turn could do anything
    std::atomic<bool> submitting{false}; // somebody is inside bnk_seal_submit / bnk_open_submit
    std::atomic<bool> polling{false};    // somebody is asking the driver about the oldest batch in flight
    std::atomic<uint32_t> n_inflight{0}, n_pending{0}; // n_pending: closed batches + a filling one that holds packets
};

namespace {

// Under the lock: should the filling batch go now?
bool ripe(const bnk_queue *q) {
    const GpuBatch &c = q->gb[q->cur];
    if (c.state.load(std::memory_order_relaxed) != FILLING || c.reserved == 0 ||
        c.filled.load(std::memory_order_acquire) != c.reserved)
        return false;
    if (q->inflight.empty()) return true;                                   // the device is idle
    if (c.reserved >= q->cfg.min_fill) return true;                         // worth a launch
    return std::chrono::steady_clock::now() >= c.first_at + kGatherNs;      // waited long enough
}

// Submit whatever is ready while the device has a free slot.  One thread at a time is inside the library's
// submit call (the kernels of consecutive GPU batches are chained in that order); the others pass by.
void pump(bnk_queue *q) {
    for (;;) {
        if (q->n_pending.load(std::memory_order_relaxed) == 0 || q->submitting.load(std::memory_order_relaxed) ||
            q->n_inflight.load(std::memory_order_relaxed) >= q->cfg.depth)
            return;
        uint32_t idx, n;
        int prev;
        {
            Locked lk(q->mu);
            if (q->submitting.load(std::memory_order_relaxed) || q->inflight.count >= q->cfg.depth) return;
            if (!q->closed.empty()) {
                const GpuBatch &f = q->gb[q->closed.front()];
                if (f.filled.load(std::memory_order_acquire) != f.reserved) return; // a caller is still copying in
                idx = q->closed.front();
                q->closed.pop();
            } else if (ripe(q)) { // cut the filling batch off
                idx = q->cur;
                q->cur = (q->cur + 1) % q->gb.size();
            } else {
                return;
            }
            GpuBatch &g = q->gb[idx];
            n = g.reserved;
            prev = q->last_submitted;
            q->last_submitted = (int)idx;
            g.state.store(IN_FLIGHT, std::memory_order_relaxed);
            q->submitting.store(true, std::memory_order_relaxed);
            q->n_pending.fetch_sub(1, std::memory_order_relaxed);
            q->n_gpu_batches++;
            q->n_packets += n;
        }
        GpuBatch &g = q->gb[idx];
        // kernels of this batch start behind the kernels of the batch submitted before it
        g.b->order_wait = prev >= 0 ? q->gb[prev].kernels_done : nullptr;
        g.b->order_record = g.kernels_done;
        g.rc = q->cfg.open_side ? bnk_open_submit(g.b, n, q->cfg.flags, g.now) : bnk_seal_submit(g.b, n, q->cfg.flags, g.now);
        g.b->order_wait = nullptr;
        g.b->order_record = nullptr;
        {
            Locked lk(q->mu);
            q->inflight.push(idx); // only now may anybody ask the driver about it
            q->n_inflight.store(q->inflight.count, std::memory_order_relaxed);
            q->submitting.store(false, std::memory_order_release);
        }
    }
}

// Has the oldest batch in flight come back?  (In submit order: kernels are chained, and a caller's ticket can
// only be in a batch behind it if the caller came later.)
void poll(bnk_queue *q) {
    if (q->n_inflight.load(std::memory_order_relaxed) == 0 || q->polling.exchange(true, std::memory_order_acquire)) return;
    for (;;) {
        uint32_t idx;
        {
            Locked lk(q->mu);
            if (q->inflight.empty()) break;
            idx = q->inflight.front();
        }
        GpuBatch &g = q->gb[idx];
        const int rc = bnk_wait(g.b, 0);
        if (rc == BNK_ETIMEDOUT) break;
        Locked lk(q->mu);
        if (g.rc == BNK_SUCCESS) g.rc = rc;
        q->inflight.pop();
        q->n_inflight.store(q->inflight.count, std::memory_order_relaxed);
        g.state.store(DONE, std::memory_order_release);
    }
    q->polling.store(false, std::memory_order_release);
}

// One turn of a waiting caller.
inline void turn(bnk_queue *q, uint32_t &spins) {
    pump(q);
    poll(q);
    // A GPU batch is back within ~100 us: that long a waiting caller stays on its core; a longer wait means the
    // callers outnumber the cores (or the device is far behind), and the core goes to whoever has work.
    if (++spins < 64u) {
        for (int i = 0; i < 16; i++) cpu_relax();
    } else {
        std::this_thread::yield();
    }
}

uint64_t make_ticket(uint32_t idx, uint32_t gen, uint32_t first, uint32_t n) {
    return ((uint64_t)(idx & 0xff) << 56) | ((uint64_t)(gen & 0xffffff) << 32) | ((uint64_t)first << 16) | n;
}

} // namespace

extern "C" {

int bnk_queue_destroy(bnk_queue *q) {
    if (!q) return BNK_EINVAL;
    cudaSetDevice(q->ctx->device);
    for (GpuBatch &g : q->gb) {
        if (g.b) {
            bnk_wait(g.b, UINT64_MAX);
            bnk_batch_destroy(g.b);
        }
        if (g.kernels_done) cudaEventDestroy(g.kernels_done);
    }
    delete q;
    return BNK_SUCCESS;
}

int bnk_queue_create(bnk_ctx *ctx, const bnk_queue_cfg *cfg, bnk_queue **out) {
    if (!ctx || !cfg || !out || cfg->struct_size != sizeof(bnk_queue_cfg) || cfg->max_pkts == 0 ||
        cfg->max_pkts > kMaxQueuePkts || cfg->max_packet == 0 || cfg->depth == 0 || cfg->depth > 8)
        return BNK_EINVAL;
    *out = nullptr;
    bnk_queue *q = new (std::nothrow) bnk_queue();
    if (!q) return BNK_ENOMEM;
    q->ctx = ctx;
    q->cfg = *cfg;
    // the queue does the copies itself and hands out counters itself
    q->cfg.flags &= ~(BNK_F_NO_H2D | BNK_F_NO_D2H | BNK_F_USE_OUT_LEN | BNK_F_TIMED | BNK_F_STATS);
    if (!cfg->open_side) q->cfg.flags |= BNK_F_ASSIGN_COUNTERS;
    if (q->cfg.min_fill == 0) q->cfg.min_fill = std::min(128u, (cfg->max_pkts + 3) / 4); // one upstream batch
    q->slot_bytes = (16u + ((cfg->max_packet + 15u) & ~15u) + 16u + 15u) & ~15u;
    q->gb = std::vector<GpuBatch>(cfg->depth + kRotationExtra);
    q->closed.slot.resize(q->gb.size());
    q->inflight.slot.resize(q->gb.size());
    cudaSetDevice(ctx->device);
    for (GpuBatch &g : q->gb) {
        int rc = bnk_batch_create(ctx, cfg->max_pkts, (uint64_t)cfg->max_pkts * q->slot_bytes, &g.b);
        if (rc == BNK_SUCCESS) rc = bnk_batch_view_get(g.b, &g.v);
        if (rc == BNK_SUCCESS && cudaEventCreateWithFlags(&g.kernels_done, cudaEventDisableTiming) != cudaSuccess) rc = BNK_ECUDA;
        if (rc != BNK_SUCCESS) {
            bnk_queue_destroy(q);
            return rc;
        }
    }
    *out = q;
    return BNK_SUCCESS;
}

// Room for n packets in the GPU batch that is filling (under the lock); BNK_EBUSY when every batch is taken.
static int reserve(bnk_queue *q, uint32_t n, int64_t now_unix_ns, bnk_ticket *ticket, GpuBatch **gout, uint32_t *first_out) {
    Locked lk(q->mu);
    GpuBatch *g;
    for (;;) {
        g = &q->gb[q->cur];
        int st = g->state.load(std::memory_order_relaxed);
        if (st == FREE) {
            g->state.store(st = FILLING, std::memory_order_relaxed);
            g->reserved = g->users = 0;
            g->filled.store(0, std::memory_order_relaxed);
            g->gen++;
            g->now = now_unix_ns;
            g->rc = BNK_SUCCESS;
            g->first_at = std::chrono::steady_clock::now();
        }
        if (st == FILLING && g->reserved + n <= q->cfg.max_pkts) break;
        if (st == FILLING) { // no room for this caller's batch: the GPU batch is complete
            g->state.store(CLOSED, std::memory_order_relaxed);
            q->closed.push(q->cur);
            q->cur = (q->cur + 1) % q->gb.size();
            continue;
        }
        // The next batch in the rotation is still on the device or has not been emptied by its callers: the
        // callers are ahead of the device.  No waiting here: the caller may itself hold the tickets that keep
        // that batch from being reused.
        return BNK_EBUSY;
    }
    const uint32_t first = g->reserved;
    if (first == 0) q->n_pending.fetch_add(1, std::memory_order_relaxed);
    g->reserved += n;
    g->users++;
    if (now_unix_ns > g->now) g->now = now_unix_ns;
    q->n_caller_batches++;
    *ticket = make_ticket(q->cur, g->gen, first, n);
    *gout = g;
    *first_out = first;
    return BNK_SUCCESS;
}

// The GPU batch a ticket belongs to, if the ticket is out.
static GpuBatch *batch_of(bnk_queue *q, bnk_ticket ticket, uint32_t *first, uint32_t *n) {
    const uint32_t idx = (uint32_t)(ticket >> 56), gen = (uint32_t)(ticket >> 32) & 0xffffff;
    *first = (uint32_t)(ticket >> 16) & 0xffff;
    *n = (uint32_t)ticket & 0xffff;
    if (idx >= q->gb.size() || *first + *n > q->cfg.max_pkts) return nullptr;
    GpuBatch &g = q->gb[idx];
    Locked lk(q->mu);
    if ((g.gen & 0xffffff) != gen || g.state.load(std::memory_order_relaxed) == FREE || g.users == 0) return nullptr;
    return &g;
}

static void fill_span(const bnk_queue *q, const GpuBatch *g, uint32_t first, bnk_queue_span *span) {
    const bnk_batch_view &v = g->v;
    span->data = v.ring + (size_t)first * q->slot_bytes;
    span->stride = q->slot_bytes;
    span->len = v.len + first;
    span->slot = v.slot + first;
    span->out_len = v.out_len + first;
    span->counter = v.counter + first;
    span->status = v.status + first;
}

static void release(bnk_queue *q, GpuBatch *g) {
    Locked lk(q->mu);
    if (--g->users == 0) g->state.store(FREE, std::memory_order_release);
}

int bnk_queue_reserve(bnk_queue *q, uint32_t n, int64_t now_unix_ns, bnk_ticket *ticket, bnk_queue_span *span) {
    if (!q || !ticket || !span || n == 0 || n > q->cfg.max_pkts) return BNK_EINVAL;
    GpuBatch *g;
    uint32_t first;
    const int rc = reserve(q, n, now_unix_ns, ticket, &g, &first);
    if (rc != BNK_SUCCESS) return rc;
    for (uint32_t k = 0; k < n; k++) g->v.off[first + k] = (first + k) * q->slot_bytes;
    fill_span(q, g, first, span);
    return BNK_SUCCESS;
}

int bnk_queue_commit(bnk_queue *q, bnk_ticket ticket) {
    if (!q) return BNK_EINVAL;
    uint32_t first, n;
    GpuBatch *g = batch_of(q, ticket, &first, &n);
    if (!g) return BNK_EINVAL;
    const uint32_t room = q->cfg.open_side ? q->cfg.max_packet + 32u : q->cfg.max_packet;
    int rc = BNK_SUCCESS;
    for (uint32_t k = 0; k < n; k++)
        if (g->v.len[first + k] > room) { // would run into the next packet's slot: the packet is refused on the device
            g->v.len[first + k] = 0;                // (open: too short to be a message -> MALFORMED)
            g->v.slot[first + k] = 0xfffffffeu;     // (seal: no such keypair -> BAD_DESC)
            rc = BNK_EINVAL;
        }
    g->filled.fetch_add(n, std::memory_order_release);
    pump(q);
    return rc;
}

int bnk_queue_wait_span(bnk_queue *q, bnk_ticket ticket, bnk_queue_span *span) {
    if (!q) return BNK_EINVAL;
    uint32_t first, n;
    GpuBatch *g = batch_of(q, ticket, &first, &n);
    if (!g) return BNK_EINVAL;
    for (uint32_t spins = 0; g->state.load(std::memory_order_acquire) != DONE;) turn(q, spins);
    if (span) fill_span(q, g, first, span);
    return g->rc;
}

int bnk_queue_release(bnk_queue *q, bnk_ticket ticket) {
    if (!q) return BNK_EINVAL;
    uint32_t first, n;
    GpuBatch *g = batch_of(q, ticket, &first, &n);
    if (!g) return BNK_EINVAL;
    if (g->state.load(std::memory_order_acquire) != DONE) return BNK_EBUSY; // wait first: the batch may be on the device
    release(q, g);
    return BNK_SUCCESS;
}

int bnk_queue_submit(bnk_queue *q, const uint8_t *const *pkts, const uint32_t *len, const uint32_t *slot, uint32_t n,
                     int64_t now_unix_ns, bnk_ticket *ticket) {
    if (!q || !ticket || n == 0 || n > q->cfg.max_pkts || !pkts || !len) return BNK_EINVAL;
    const bool open_side = q->cfg.open_side != 0;
    if (!open_side && !slot) return BNK_EINVAL;
    if (open_side && !slot && !(q->cfg.flags & BNK_F_DEMUX_INDEX)) return BNK_EINVAL;
    const uint32_t room = open_side ? q->cfg.max_packet + 32u : q->cfg.max_packet;
    for (uint32_t i = 0; i < n; i++)
        if (len[i] > room) return BNK_EINVAL;
    GpuBatch *g;
    uint32_t first;
    const int rc = reserve(q, n, now_unix_ns, ticket, &g, &first);
    if (rc != BNK_SUCCESS) return rc;
    // copy in, outside the lock: callers fill their own stretches of the ring side by side
    const bnk_batch_view &v = g->v;
    const uint32_t head = open_side ? 0u : 16u;
    for (uint32_t k = 0; k < n; k++) {
        const uint32_t at = first + k;
        v.off[at] = at * q->slot_bytes;
        v.len[at] = len[k];
        v.slot[at] = slot ? slot[k] : 0u;
        if (len[k]) memcpy(v.ring + (size_t)at * q->slot_bytes + head, pkts[k], len[k]);
    }
    g->filled.fetch_add(n, std::memory_order_release);
    pump(q);
    return BNK_SUCCESS;
}

int bnk_queue_wait(bnk_queue *q, bnk_ticket ticket, uint8_t *const *out, uint32_t *out_len, uint64_t *counter,
                   uint32_t *slot_out, uint8_t *status) {
    if (!q || !out || !out_len || !status) return BNK_EINVAL;
    uint32_t first, n;
    GpuBatch *gp = batch_of(q, ticket, &first, &n);
    if (!gp) return BNK_EINVAL; // not a ticket that is out
    GpuBatch &g = *gp;
    for (uint32_t spins = 0; g.state.load(std::memory_order_acquire) != DONE;) turn(q, spins);
    const int rc = g.rc;
    const bnk_batch_view &v = g.v;
    const bool open_side = q->cfg.open_side != 0;
    for (uint32_t k = 0; k < n; k++) {
        const uint32_t at = first + k;
        // only what passed leaves the library: a replayed, filtered or otherwise refused packet yields no bytes
        const bool pass = v.status[at] == BNK_PKT_OK || v.status[at] == BNK_PKT_KEEPALIVE;
        status[k] = v.status[at];
        out_len[k] = pass ? v.out_len[at] : 0u;
        if (counter) counter[k] = v.counter[at];
        if (slot_out) slot_out[k] = v.slot[at];
        if (out_len[k]) memcpy(out[k], v.ring + (size_t)at * q->slot_bytes + (open_side ? 16u : 0u), out_len[k]);
    }
    release(q, &g);
    return rc;
}

int bnk_queue_wait_room(bnk_queue *q, uint64_t timeout_ns) {
    if (!q) return BNK_EINVAL;
    const auto deadline = std::chrono::steady_clock::now() +
                          std::chrono::nanoseconds(timeout_ns == UINT64_MAX ? (uint64_t)INT64_MAX / 2 : timeout_ns);
    for (uint32_t spins = 0;;) {
        int st;
        {
            Locked lk(q->mu);
            st = q->gb[q->cur].state.load(std::memory_order_relaxed);
        }
        if (st == FREE || st == FILLING) return BNK_SUCCESS;
        if (timeout_ns != UINT64_MAX && std::chrono::steady_clock::now() >= deadline) return BNK_ETIMEDOUT;
        turn(q, spins);
    }
}

int bnk_queue_stats_get(bnk_queue *q, uint64_t *gpu_batches, uint64_t *packets, uint64_t *caller_batches) {
    if (!q) return BNK_EINVAL;
    Locked lk(q->mu);
    if (gpu_batches) *gpu_batches = q->n_gpu_batches;
    if (packets) *packets = q->n_packets;
    if (caller_batches) *caller_batches = q->n_caller_batches;
    return BNK_SUCCESS;
}

} // extern "C"
