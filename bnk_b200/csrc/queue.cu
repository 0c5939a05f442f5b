// A submit queue below the C ABI (declared in include/bnk_gpu.h): callers hand in batches of the size the
// reference works with (conn.IdealBatchSize = 128 packets per tun.Device.Read / conn.ReceiveFunc call,
// internal/magicsock/bind.go:97,372-377), from as many threads as they like; the queue packs them into GPU
// batches that are worth a launch and gives every caller its own packets back.
//
// Why: one 128-packet submit costs the same handful of driver calls and the same two trips over the host link as
// a submit of a few thousand packets, and while such a small batch is on its way the GPU does nothing else.
// Here callers copy their packets into the pinned ring of the GPU batch that is filling.  When the device is idle
// the batch goes as it is (a lone caller waits for nobody); while something is in flight the batch keeps filling
// until it holds a quarter of its capacity or its first packet has waited kGatherNs, whichever comes first, and
// at the latest when it is full (under load batches grow by themselves).  Up to `depth` GPU batches are in flight, each
// on its own stream, so the upload of one runs beside the kernels of the one in front and the download of the
// one before; the KERNELS of consecutive batches are chained with events, which keeps what the library promises
// per keypair: nonces in submit order, replay verdicts in arrival order.
#include <chrono>
#include <condition_variable>
#include <deque>
#include <new>
#include <thread>

#include "bnk_internal.cuh"

namespace {

enum State { FREE, FILLING, CLOSED, IN_FLIGHT, DONE };

struct GpuBatch {
    bnk_batch *b = nullptr;
    bnk_batch_view v{};
    cudaEvent_t kernels_done = nullptr; // recorded behind the batch's last kernel
    State state = FREE;
    uint32_t reserved = 0; // packets handed out to callers
    uint32_t filled = 0;   // of those, copied in
    uint32_t users = 0;    // caller batches whose results have not been collected
    uint32_t gen = 0;      // how often the batch has been reused (part of the ticket)
    int64_t now = 0;
    int rc = BNK_SUCCESS;
    std::chrono::steady_clock::time_point first_at; // when the first caller arrived
    std::condition_variable done;                   // its callers wait here, nobody else is woken
};

constexpr uint32_t kMaxQueuePkts = 32768; // ticket fields are 16 bits
// How long the first packet of a GPU batch may wait for company while another batch is on the device.  A GPU
// batch costs ~40 us of driver calls on the submitting thread however small it is; a round trip of a batch takes
// ~100 us; so a few tens of microseconds of gathering cost little latency and are what makes batches worth a launch.
constexpr std::chrono::nanoseconds kGatherNs(40000);
constexpr uint32_t kRotationExtra = 6; // GPU batches beyond `depth`: filling, and done but not yet emptied by their callers

} // namespace

struct bnk_queue {
    bnk_ctx *ctx;
    bnk_queue_cfg cfg;
    uint32_t slot_bytes;
    std::deque<GpuBatch> gb; // (a deque: the entries hold condition variables and never move)
    uint32_t cur = 0;              // the batch that is filling (or will be, once it is free)
    std::deque<uint32_t> closed;   // full or cut off, waiting for the device, in order
    std::deque<uint32_t> inflight; // submitted, in order
    int last_submitted = -1;
    uint64_t n_gpu_batches = 0, n_packets = 0, n_caller_batches = 0;
    bool stop = false;
    std::mutex mu;
    uint32_t submitting = 0;       // 1 while the submitter is inside bnk_seal_submit / bnk_open_submit
    std::condition_variable cv_work, cv_complete, cv_room;
    std::thread submitter, completer;
};

namespace {

// true when the filling batch should go now; otherwise *until says when to look again (if it holds anything)
bool ripe(const bnk_queue *q, std::chrono::steady_clock::time_point *until, bool *timed) {
    *timed = false;
    const GpuBatch &c = q->gb[q->cur];
    if (c.state != FILLING || c.reserved == 0 || c.filled != c.reserved) return false;
    if (q->inflight.empty() && q->submitting == 0) return true;             // the device is idle
    if (c.reserved >= (q->cfg.max_pkts + 3) / 4) return true;               // worth a launch
    *until = c.first_at + kGatherNs;
    *timed = true;
    return std::chrono::steady_clock::now() >= *until;                      // waited long enough
}

void submitter_loop(bnk_queue *q) {
    std::unique_lock<std::mutex> lk(q->mu);
    for (;;) {
        // work: a closed batch, or a filling one that is ripe, while the device has a free slot
        for (;;) {
            if (q->stop) return;
            std::chrono::steady_clock::time_point until;
            bool timed = false;
            if (q->inflight.size() + q->submitting < q->cfg.depth) {
                if (!q->closed.empty()) {
                    const GpuBatch &f = q->gb[q->closed.front()];
                    if (f.filled == f.reserved) break;
                } else if (ripe(q, &until, &timed)) {
                    break;
                }
            }
            if (timed) q->cv_work.wait_until(lk, until);
            else q->cv_work.wait(lk);
        }
        if (q->closed.empty()) { // cut the filling batch off
            q->gb[q->cur].state = CLOSED;
            q->closed.push_back(q->cur);
            q->cur = (q->cur + 1) % q->gb.size();
            q->cv_room.notify_all();
        }
        const uint32_t idx = q->closed.front();
        q->closed.pop_front();
        GpuBatch &g = q->gb[idx];
        const uint32_t n = g.reserved;
        const int prev = q->last_submitted;
        q->last_submitted = (int)idx;
        g.state = IN_FLIGHT;
        q->submitting = 1;
        q->n_gpu_batches++;
        q->n_packets += n;
        lk.unlock();
        // kernels of this batch start behind the kernels of the batch submitted before it
        g.b->order_wait = prev >= 0 ? q->gb[prev].kernels_done : nullptr;
        g.b->order_record = g.kernels_done;
        g.rc = q->cfg.open_side ? bnk_open_submit(g.b, n, q->cfg.flags, g.now) : bnk_seal_submit(g.b, n, q->cfg.flags, g.now);
        g.b->order_wait = nullptr;
        g.b->order_record = nullptr;
        lk.lock();
        q->submitting = 0;
        q->inflight.push_back(idx); // only now may the completer wait for it
        q->cv_complete.notify_all();
    }
}

void completer_loop(bnk_queue *q) {
    std::unique_lock<std::mutex> lk(q->mu);
    for (;;) {
        q->cv_complete.wait(lk, [&] { return q->stop || !q->inflight.empty(); });
        if (q->inflight.empty()) return; // stop, and nothing left to wait for
        const uint32_t idx = q->inflight.front();
        GpuBatch &g = q->gb[idx];
        lk.unlock();
        const int rc = bnk_wait(g.b, UINT64_MAX);
        lk.lock();
        if (g.rc == BNK_SUCCESS) g.rc = rc;
        q->inflight.pop_front();
        g.state = DONE;
        g.done.notify_all();
        q->cv_work.notify_all(); // a slot on the device is free again
    }
}

uint64_t make_ticket(uint32_t idx, uint32_t gen, uint32_t first, uint32_t n) {
    return ((uint64_t)(idx & 0xff) << 56) | ((uint64_t)(gen & 0xffffff) << 32) | ((uint64_t)first << 16) | n;
}

} // namespace

extern "C" {

int bnk_queue_destroy(bnk_queue *q) {
    if (!q) return BNK_EINVAL;
    {
        std::lock_guard<std::mutex> g(q->mu);
        q->stop = true;
    }
    q->cv_work.notify_all();
    q->cv_complete.notify_all();
    if (q->submitter.joinable()) q->submitter.join();
    if (q->completer.joinable()) q->completer.join();
    cudaSetDevice(q->ctx->device);
    for (GpuBatch &g : q->gb) {
        if (g.b) bnk_batch_destroy(g.b);
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
    q->slot_bytes = (16u + ((cfg->max_packet + 15u) & ~15u) + 16u + 15u) & ~15u;
    q->gb.resize(cfg->depth + kRotationExtra);
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
    q->submitter = std::thread(submitter_loop, q);
    q->completer = std::thread(completer_loop, q);
    *out = q;
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
    std::unique_lock<std::mutex> lk(q->mu);
    GpuBatch *g;
    for (;;) {
        g = &q->gb[q->cur];
        if (g->state == FREE) {
            g->state = FILLING;
            g->reserved = g->filled = g->users = 0;
            g->gen++;
            g->now = now_unix_ns;
            g->rc = BNK_SUCCESS;
            g->first_at = std::chrono::steady_clock::now();
        }
        if (g->state == FILLING && g->reserved + n <= q->cfg.max_pkts) break;
        if (g->state == FILLING) { // no room for this caller's batch: the GPU batch is complete
            g->state = CLOSED;
            q->closed.push_back(q->cur);
            q->cur = (q->cur + 1) % q->gb.size();
            q->cv_work.notify_all();
            continue;
        }
        // The next batch in the rotation is still on the device or has not been emptied by its callers: the
        // callers are ahead of the device.  No waiting here: the caller may itself hold the tickets that keep
        // that batch from being reused.
        return BNK_EBUSY;
    }
    const uint32_t first = g->reserved, idx = q->cur;
    g->reserved += n;
    g->users++;
    if (now_unix_ns > g->now) g->now = now_unix_ns;
    q->n_caller_batches++;
    *ticket = make_ticket(idx, g->gen, first, n);
    lk.unlock();
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
    lk.lock();
    g->filled += n;
    q->cv_work.notify_all();
    return BNK_SUCCESS;
}

int bnk_queue_wait(bnk_queue *q, bnk_ticket ticket, uint8_t *const *out, uint32_t *out_len, uint64_t *counter,
                   uint32_t *slot_out, uint8_t *status) {
    if (!q || !out || !out_len || !status) return BNK_EINVAL;
    const uint32_t idx = (uint32_t)(ticket >> 56), gen = (uint32_t)(ticket >> 32) & 0xffffff;
    const uint32_t first = (uint32_t)(ticket >> 16) & 0xffff, n = (uint32_t)ticket & 0xffff;
    if (idx >= q->gb.size() || first + n > q->cfg.max_pkts) return BNK_EINVAL;
    GpuBatch &g = q->gb[idx];
    std::unique_lock<std::mutex> lk(q->mu);
    if ((g.gen & 0xffffff) != gen || g.state == FREE || g.users == 0) return BNK_EINVAL; // not a ticket that is out
    g.done.wait(lk, [&] { return g.state == DONE; });
    const int rc = g.rc;
    lk.unlock();
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
    lk.lock();
    if (--g.users == 0) {
        g.state = FREE;
        q->cv_room.notify_all();
    }
    return rc;
}

int bnk_queue_wait_room(bnk_queue *q, uint64_t timeout_ns) {
    if (!q) return BNK_EINVAL;
    std::unique_lock<std::mutex> lk(q->mu);
    auto room = [&] { return q->gb[q->cur].state == FREE || q->gb[q->cur].state == FILLING; };
    if (timeout_ns == UINT64_MAX) {
        q->cv_room.wait(lk, room);
        return BNK_SUCCESS;
    }
    return q->cv_room.wait_for(lk, std::chrono::nanoseconds(timeout_ns), room) ? BNK_SUCCESS : BNK_ETIMEDOUT;
}

int bnk_queue_stats_get(bnk_queue *q, uint64_t *gpu_batches, uint64_t *packets, uint64_t *caller_batches) {
    if (!q) return BNK_EINVAL;
    std::lock_guard<std::mutex> g(q->mu);
    if (gpu_batches) *gpu_batches = q->n_gpu_batches;
    if (packets) *packets = q->n_packets;
    if (caller_batches) *caller_batches = q->n_caller_batches;
    return BNK_SUCCESS;
}

} // extern "C"
