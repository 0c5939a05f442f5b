// Several GPUs behind one entry point: placement of peers by measured load and a dispatcher that routes mixed
// batches to per-GPU contexts (declared in include/bnk_gpu.h).  Host code only; every packet decision is made by
// the kernels behind bnk_seal_submit / bnk_open_submit of the GPU a packet is routed to.
//
// Why peers and nothing finer: the send counter hands out consecutive nonces per peer in batch order and the
// replay window is a sequential walk per peer, so a peer's packets must meet in one context; flows are keyed by
// the peer's tunnel address (one /32 per peer, internal/dataplane/engine.go:294 of the reference) and stay with
// it.  The rule table is read-only per packet and is replicated.  GPUs therefore never exchange packet data.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <new>
#include <queue>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/bnk_gpu.h"

extern "C" int bnk_place_peers(const uint64_t *load, uint32_t n_peers, uint32_t n_gpus, uint32_t max_per_gpu,
                               uint32_t *gpu_of, uint32_t *slot_of, uint64_t *load_per_gpu) {
    if (!gpu_of || !slot_of || n_gpus == 0) return BNK_EINVAL;
    if ((uint64_t)n_gpus * max_per_gpu < n_peers) return BNK_EFULL;
    std::vector<uint32_t> order(n_peers);
    for (uint32_t p = 0; p < n_peers; p++) order[p] = p;
    if (load)
        std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return load[a] > load[b]; });
    // Longest processing time first.  Every peer weighs its load plus one, so that the many peers that carried
    // nothing in the measured period still spread evenly instead of piling onto the lightest GPU.
    struct Gpu {
        uint64_t weight;
        uint32_t count, id;
    };
    auto heavier = [](const Gpu &a, const Gpu &b) { // priority_queue keeps the largest on top: invert
        if (a.weight != b.weight) return a.weight > b.weight;
        if (a.count != b.count) return a.count > b.count;
        return a.id > b.id;
    };
    std::priority_queue<Gpu, std::vector<Gpu>, decltype(heavier)> heap(heavier);
    for (uint32_t g = 0; g < n_gpus; g++) heap.push(Gpu{0, 0, g});
    std::vector<uint64_t> carried(n_gpus, 0);
    for (uint32_t p : order) {
        Gpu g = heap.top();
        heap.pop();
        gpu_of[p] = g.id;
        slot_of[p] = g.count;
        const uint64_t l = load ? load[p] : 0;
        carried[g.id] += l;
        g.weight += l + 1;
        g.count++;
        if (g.count < max_per_gpu) heap.push(g); // a full GPU takes no more peers
    }
    if (load_per_gpu)
        for (uint32_t g = 0; g < n_gpus; g++) load_per_gpu[g] = carried[g];
    return BNK_SUCCESS;
}

namespace {

constexpr uint32_t kNoPeer = 0xffffffffu;

// One host thread per GPU: runs the jobs posted to it in order.
class Worker {
  public:
    Worker() : thread_([this] { Run(); }) {}
    ~Worker() {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        thread_.join();
    }
    void Post(std::function<void()> job) {
        {
            std::lock_guard<std::mutex> g(mu_);
            jobs_.push(std::move(job));
        }
        cv_.notify_all();
    }

  private:
    void Run() {
        for (;;) {
            std::function<void()> job;
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [this] { return stop_ || !jobs_.empty(); });
                if (jobs_.empty()) return;
                job = std::move(jobs_.front());
                jobs_.pop();
            }
            job();
        }
    }
    std::mutex mu_;
    std::condition_variable cv_;
    std::queue<std::function<void()>> jobs_;
    bool stop_ = false;
    std::thread thread_;
};

// counts the per-GPU jobs of one call down
class Latch {
  public:
    explicit Latch(int n) : left_(n) {}
    void Done() {
        std::lock_guard<std::mutex> g(mu_);
        if (--left_ == 0) cv_.notify_all();
    }
    void Wait() {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [this] { return left_ <= 0; });
    }

  private:
    std::mutex mu_;
    std::condition_variable cv_;
    int left_;
};

struct PeerInfo {
    bool set = false;
    uint32_t local_index = 0;
};

} // namespace

struct bnk_mgpu {
    bnk_mgpu_cfg cfg;
    uint32_t slot_bytes;
    std::vector<bnk_ctx *> ctx;
    std::vector<bnk_batch *> batch;
    std::vector<bnk_batch_view> view;
    std::vector<std::unique_ptr<Worker>> worker;
    std::vector<uint32_t> gpu_of, slot_of;
    std::vector<PeerInfo> peer;
    std::unordered_map<uint32_t, uint32_t> peer_of_index; // receiver index -> peer
    std::vector<uint64_t> pkts_per_peer, bytes_per_peer, pkts_per_gpu;
    uint32_t peers_set = 0;
    std::mutex mu; // one call at a time: per-peer order is the order of the calls
    std::string last_error;
};

namespace {

int mfail(bnk_mgpu *m, int code, const std::string &what) {
    if (m) m->last_error = what;
    return code;
}

// Per-GPU lists of packet numbers in batch order (stable: a peer's packets keep their order).
void route(const bnk_mgpu *m, const std::vector<uint32_t> &gpu_of_pkt, std::vector<std::vector<uint32_t>> &lists) {
    const uint32_t ng = (uint32_t)m->ctx.size();
    std::vector<uint32_t> count(ng, 0);
    for (uint32_t g : gpu_of_pkt)
        if (g != kNoPeer) count[g]++;
    lists.assign(ng, {});
    for (uint32_t g = 0; g < ng; g++) lists[g].reserve(count[g]);
    for (uint32_t i = 0; i < gpu_of_pkt.size(); i++)
        if (gpu_of_pkt[i] != kNoPeer) lists[gpu_of_pkt[i]].push_back(i);
}

} // namespace

extern "C" {

const char *bnk_mgpu_last_error_string(bnk_mgpu *m) { return m ? m->last_error.c_str() : "null dispatcher"; }

int bnk_mgpu_destroy(bnk_mgpu *m) {
    if (!m) return BNK_EINVAL;
    m->worker.clear(); // joins the threads
    for (bnk_batch *b : m->batch)
        if (b) bnk_batch_destroy(b);
    for (bnk_ctx *c : m->ctx)
        if (c) bnk_ctx_destroy(c);
    delete m;
    return BNK_SUCCESS;
}

int bnk_mgpu_create(const bnk_mgpu_cfg *cfg, bnk_mgpu **out) {
    if (!cfg || !out || cfg->struct_size != sizeof(bnk_mgpu_cfg) || cfg->n_devices == 0 || !cfg->devices ||
        cfg->max_pkts_per_gpu == 0 || cfg->max_peers == 0 || cfg->max_packet == 0)
        return BNK_EINVAL;
    *out = nullptr;
    if ((uint64_t)cfg->n_devices * cfg->ctx.max_keypairs < cfg->max_peers) return BNK_EINVAL;
    bnk_mgpu *m = new (std::nothrow) bnk_mgpu();
    if (!m) return BNK_ENOMEM;
    m->cfg = *cfg;
    m->cfg.devices = nullptr;
    m->slot_bytes = (16u + ((cfg->max_packet + 15u) & ~15u) + 16u + 15u) & ~15u;
    const uint32_t ng = cfg->n_devices;
    m->ctx.assign(ng, nullptr);
    m->batch.assign(ng, nullptr);
    m->view.assign(ng, bnk_batch_view{});
    m->pkts_per_gpu.assign(ng, 0);
    for (uint32_t g = 0; g < ng; g++) {
        bnk_cfg c = cfg->ctx;
        c.struct_size = sizeof c;
        c.device_id = cfg->devices[g];
        int rc = bnk_ctx_create(&c, &m->ctx[g]);
        if (rc == BNK_SUCCESS) rc = bnk_batch_create(m->ctx[g], cfg->max_pkts_per_gpu, (uint64_t)cfg->max_pkts_per_gpu * m->slot_bytes, &m->batch[g]);
        if (rc == BNK_SUCCESS) rc = bnk_batch_view_get(m->batch[g], &m->view[g]);
        if (rc != BNK_SUCCESS) {
            bnk_mgpu_destroy(m);
            return rc;
        }
        m->worker.emplace_back(new Worker());
    }
    m->gpu_of.assign(cfg->max_peers, 0);
    m->slot_of.assign(cfg->max_peers, 0);
    m->peer.assign(cfg->max_peers, PeerInfo{});
    m->pkts_per_peer.assign(cfg->max_peers, 0);
    m->bytes_per_peer.assign(cfg->max_peers, 0);
    const int rc = bnk_place_peers(nullptr, cfg->max_peers, ng, cfg->ctx.max_keypairs, m->gpu_of.data(), m->slot_of.data(), nullptr);
    if (rc != BNK_SUCCESS) {
        bnk_mgpu_destroy(m);
        return rc;
    }
    *out = m;
    return BNK_SUCCESS;
}

bnk_ctx *bnk_mgpu_ctx(bnk_mgpu *m, uint32_t g) { return (m && g < m->ctx.size()) ? m->ctx[g] : nullptr; }

int bnk_mgpu_place(bnk_mgpu *m, const uint64_t *load) {
    if (!m) return BNK_EINVAL;
    std::lock_guard<std::mutex> g(m->mu);
    if (m->peers_set) return mfail(m, BNK_EBUSY, "peers are set: remove them before placing anew (a live peer moves with its next keypair)");
    return bnk_place_peers(load, m->cfg.max_peers, (uint32_t)m->ctx.size(), m->cfg.ctx.max_keypairs, m->gpu_of.data(),
                           m->slot_of.data(), nullptr);
}

int bnk_mgpu_locate(bnk_mgpu *m, uint32_t peer, uint32_t *gpu, uint32_t *slot) {
    if (!m || peer >= m->cfg.max_peers) return BNK_EINVAL;
    if (gpu) *gpu = m->gpu_of[peer];
    if (slot) *slot = m->slot_of[peer];
    return BNK_SUCCESS;
}

int bnk_mgpu_peer_clear(bnk_mgpu *m, uint32_t peer) {
    if (!m || peer >= m->cfg.max_peers) return BNK_EINVAL;
    std::lock_guard<std::mutex> g(m->mu);
    PeerInfo &pi = m->peer[peer];
    if (!pi.set) return BNK_SUCCESS;
    bnk_ctx *c = m->ctx[m->gpu_of[peer]];
    int rc = bnk_index_clear(c, pi.local_index);
    if (rc == BNK_SUCCESS) rc = bnk_keypair_clear(c, m->slot_of[peer]);
    if (rc != BNK_SUCCESS) return mfail(m, rc, bnk_last_error_string(c));
    m->peer_of_index.erase(pi.local_index);
    pi.set = false;
    m->peers_set--;
    return BNK_SUCCESS;
}

int bnk_mgpu_peer_set(bnk_mgpu *m, uint32_t peer, const uint8_t send_key[32], const uint8_t recv_key[32],
                      uint32_t remote_index, uint32_t local_index, uint32_t allowed_ipv4) {
    if (!m || peer >= m->cfg.max_peers || !send_key || !recv_key) return BNK_EINVAL;
    int rc = bnk_mgpu_peer_clear(m, peer);
    if (rc != BNK_SUCCESS) return rc;
    std::lock_guard<std::mutex> g(m->mu);
    auto taken = m->peer_of_index.find(local_index);
    if (taken != m->peer_of_index.end()) return mfail(m, BNK_EINVAL, "receiver index already belongs to another peer");
    bnk_ctx *c = m->ctx[m->gpu_of[peer]];
    const uint32_t slot = m->slot_of[peer];
    rc = bnk_keypair_set(c, slot, send_key, recv_key, remote_index);
    if (rc == BNK_SUCCESS) rc = bnk_keypair_set_allowed_ip(c, slot, allowed_ipv4);
    if (rc == BNK_SUCCESS) rc = bnk_index_set(c, local_index, slot);
    if (rc != BNK_SUCCESS) return mfail(m, rc, bnk_last_error_string(c));
    m->peer[peer].set = true;
    m->peer[peer].local_index = local_index;
    m->peer_of_index[local_index] = peer;
    m->peers_set++;
    return BNK_SUCCESS;
}

int bnk_mgpu_acl_set(bnk_mgpu *m, int enforce, const bnk_acl_tuple *tuples, size_t n) {
    if (!m) return BNK_EINVAL;
    for (bnk_ctx *c : m->ctx) {
        const int rc = bnk_acl_set(c, enforce, tuples, n);
        if (rc != BNK_SUCCESS) return mfail(m, rc, bnk_last_error_string(c));
    }
    return BNK_SUCCESS;
}

int bnk_mgpu_loads_get(bnk_mgpu *m, uint64_t *packets_per_peer, uint64_t *bytes_per_peer, uint64_t *packets_per_gpu,
                       int reset) {
    if (!m) return BNK_EINVAL;
    std::lock_guard<std::mutex> g(m->mu);
    if (packets_per_peer) memcpy(packets_per_peer, m->pkts_per_peer.data(), m->pkts_per_peer.size() * 8);
    if (bytes_per_peer) memcpy(bytes_per_peer, m->bytes_per_peer.data(), m->bytes_per_peer.size() * 8);
    if (packets_per_gpu) memcpy(packets_per_gpu, m->pkts_per_gpu.data(), m->pkts_per_gpu.size() * 8);
    if (reset) {
        std::fill(m->pkts_per_peer.begin(), m->pkts_per_peer.end(), 0);
        std::fill(m->bytes_per_peer.begin(), m->bytes_per_peer.end(), 0);
    }
    return BNK_SUCCESS;
}

// The two data calls share their shape: route, one job per GPU (fill the pinned ring, submit, wait, copy out,
// in rounds of max_pkts_per_gpu), wait for all jobs.
static int run_jobs(bnk_mgpu *m, const std::vector<std::vector<uint32_t>> &lists,
                    const std::function<int(uint32_t g, const uint32_t *idx, uint32_t cnt)> &round) {
    const uint32_t ng = (uint32_t)m->ctx.size();
    int busy = 0;
    for (uint32_t g = 0; g < ng; g++) busy += !lists[g].empty();
    if (busy == 0) return BNK_SUCCESS;
    // The calling thread takes the last busy GPU itself: with one busy GPU (a small batch, a single-GPU box)
    // nothing is handed to another thread at all, and otherwise the caller works instead of sleeping.
    uint32_t own = 0;
    for (uint32_t g = 0; g < ng; g++)
        if (!lists[g].empty()) own = g;
    Latch latch(busy - 1);
    std::vector<int> rcs(ng, BNK_SUCCESS);
    auto job = [&](uint32_t g) {
        const std::vector<uint32_t> &l = lists[g];
        const uint32_t cap = m->cfg.max_pkts_per_gpu;
        for (size_t first = 0; first < l.size() && rcs[g] == BNK_SUCCESS; first += cap)
            rcs[g] = round(g, l.data() + first, (uint32_t)std::min<size_t>(cap, l.size() - first));
    };
    for (uint32_t g = 0; g < ng; g++) {
        if (lists[g].empty()) continue;
        m->pkts_per_gpu[g] += lists[g].size();
        if (g == own) continue;
        m->worker[g]->Post([&, g] {
            job(g);
            latch.Done();
        });
    }
    job(own);
    latch.Wait();
    for (uint32_t g = 0; g < ng; g++)
        if (rcs[g] != BNK_SUCCESS) return mfail(m, rcs[g], bnk_last_error_string(m->ctx[g]));
    return BNK_SUCCESS;
}

int bnk_mgpu_seal(bnk_mgpu *m, const uint8_t *const *pkts, const uint32_t *len, const uint32_t *peer, uint32_t n,
                  uint32_t flags, int64_t now_unix_ns, uint8_t *const *out, uint32_t *out_len, uint64_t *counter,
                  uint8_t *status) {
    if (!m || (n && (!pkts || !len || !peer || !out || !out_len || !status))) return BNK_EINVAL;
    std::lock_guard<std::mutex> guard(m->mu);
    std::vector<uint32_t> gpu_of_pkt(n);
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t p = peer[i];
        if (p >= m->cfg.max_peers || !m->peer[p].set || len[i] > m->cfg.max_packet) {
            gpu_of_pkt[i] = kNoPeer;
            status[i] = (p < m->cfg.max_peers && m->peer[p].set) ? BNK_PKT_BAD_DESC : BNK_PKT_NO_KEYPAIR;
            out_len[i] = 0;
            continue;
        }
        gpu_of_pkt[i] = m->gpu_of[p];
        m->pkts_per_peer[p]++;
        m->bytes_per_peer[p] += len[i];
    }
    std::vector<std::vector<uint32_t>> lists;
    route(m, gpu_of_pkt, lists);
    const uint32_t f = (flags | BNK_F_ASSIGN_COUNTERS) & ~(BNK_F_NO_H2D | BNK_F_NO_D2H | BNK_F_USE_OUT_LEN);
    return run_jobs(m, lists, [&](uint32_t g, const uint32_t *idx, uint32_t cnt) {
        const bnk_batch_view &v = m->view[g];
        for (uint32_t k = 0; k < cnt; k++) {
            const uint32_t i = idx[k];
            v.off[k] = k * m->slot_bytes;
            v.len[k] = len[i];
            v.slot[k] = m->slot_of[peer[i]];
            if (len[i]) memcpy(v.ring + (size_t)k * m->slot_bytes + 16, pkts[i], len[i]);
        }
        int rc = bnk_seal_submit(m->batch[g], cnt, f, now_unix_ns);
        if (rc == BNK_SUCCESS) rc = bnk_wait(m->batch[g], UINT64_MAX);
        if (rc != BNK_SUCCESS && rc != BNK_EFULL) return rc;
        for (uint32_t k = 0; k < cnt; k++) {
            const uint32_t i = idx[k];
            status[i] = v.status[k];
            out_len[i] = v.out_len[k];
            if (counter) counter[i] = v.counter[k];
            if (v.out_len[k]) memcpy(out[i], v.ring + (size_t)k * m->slot_bytes, v.out_len[k]);
        }
        return rc;
    });
}

int bnk_mgpu_open(bnk_mgpu *m, const uint8_t *const *msgs, const uint32_t *len, uint32_t n, uint32_t flags,
                  int64_t now_unix_ns, uint8_t *const *out, uint32_t *out_len, uint64_t *counter, uint32_t *peer_out,
                  uint8_t *status) {
    if (!m || (n && (!msgs || !len || !out || !out_len || !status))) return BNK_EINVAL;
    std::lock_guard<std::mutex> guard(m->mu);
    std::vector<uint32_t> gpu_of_pkt(n), peer_of_pkt(n, kNoPeer);
    for (uint32_t i = 0; i < n; i++) {
        gpu_of_pkt[i] = kNoPeer;
        out_len[i] = 0;
        if (peer_out) peer_out[i] = kNoPeer;
        if (len[i] < BNK_WG_HEADER + BNK_WG_TAG || (uint64_t)len[i] > (uint64_t)m->cfg.max_packet + 32u) {
            status[i] = BNK_PKT_MALFORMED;
            continue;
        }
        uint32_t type, index;
        memcpy(&type, msgs[i], 4);
        memcpy(&index, msgs[i] + 4, 4); // little-endian hosts only, like the rest of the library
        if (type != 4u) {
            status[i] = BNK_PKT_MALFORMED;
            continue;
        }
        auto it = m->peer_of_index.find(index);
        if (it == m->peer_of_index.end()) {
            status[i] = BNK_PKT_NO_KEYPAIR;
            continue;
        }
        peer_of_pkt[i] = it->second;
        gpu_of_pkt[i] = m->gpu_of[it->second];
        if (peer_out) peer_out[i] = it->second;
        m->pkts_per_peer[it->second]++;
        m->bytes_per_peer[it->second] += len[i];
    }
    std::vector<std::vector<uint32_t>> lists;
    route(m, gpu_of_pkt, lists);
    const uint32_t f = flags & ~(BNK_F_NO_H2D | BNK_F_NO_D2H | BNK_F_USE_OUT_LEN | BNK_F_DEMUX_INDEX);
    return run_jobs(m, lists, [&](uint32_t g, const uint32_t *idx, uint32_t cnt) {
        const bnk_batch_view &v = m->view[g];
        for (uint32_t k = 0; k < cnt; k++) {
            const uint32_t i = idx[k];
            v.off[k] = k * m->slot_bytes;
            v.len[k] = len[i];
            v.slot[k] = m->slot_of[peer_of_pkt[i]];
            memcpy(v.ring + (size_t)k * m->slot_bytes, msgs[i], len[i]);
        }
        int rc = bnk_open_submit(m->batch[g], cnt, f, now_unix_ns);
        if (rc == BNK_SUCCESS) rc = bnk_wait(m->batch[g], UINT64_MAX);
        if (rc != BNK_SUCCESS) return rc;
        for (uint32_t k = 0; k < cnt; k++) {
            const uint32_t i = idx[k];
            // only what passed leaves the library: a replayed, filtered or otherwise refused packet yields no bytes
            const bool pass = v.status[k] == BNK_PKT_OK || v.status[k] == BNK_PKT_KEEPALIVE;
            status[i] = v.status[k];
            out_len[i] = pass ? v.out_len[k] : 0u;
            if (counter) counter[i] = v.counter[k];
            if (out_len[i]) memcpy(out[i], v.ring + (size_t)k * m->slot_bytes + 16, out_len[i]);
        }
        return rc;
    });
}

} // extern "C"
