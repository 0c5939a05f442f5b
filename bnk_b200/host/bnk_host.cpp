// Host side above the C ABI (see bnk_host.hpp).  Byte shuffling only: every verdict, ciphertext byte and
// counter comes back from libbnkgpu's kernels.
#include "bnk_host.hpp"

#include <algorithm>
#include <chrono>
#include <cstring>

namespace bnk {

TimeNs Now() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

// ---- acl ----
namespace {

// netip.ParsePrefix restricted to what can contain an IPv4 address; anything else "never contains"
bool parse_prefix(const std::string &s, uint32_t &addr, int &bits) {
    const size_t slash = s.find('/');
    if (slash == std::string::npos) return false;
    unsigned a[4];
    char extra;
    if (sscanf(s.substr(0, slash).c_str(), "%u.%u.%u.%u%c", &a[0], &a[1], &a[2], &a[3], &extra) != 4) return false;
    for (unsigned v : a)
        if (v > 255) return false;
    int b = -1;
    if (sscanf(s.c_str() + slash + 1, "%d%c", &b, &extra) != 1 || b < 0 || b > 32) return false;
    addr = (a[0] << 24) | (a[1] << 16) | (a[2] << 8) | a[3];
    bits = b;
    return true;
}

} // namespace

std::vector<bnk_acl_tuple> FlattenRules(const std::vector<CompiledRule> &rules) {
    std::vector<bnk_acl_tuple> out;
    for (const CompiledRule &r : rules) {
        uint8_t proto = r.Proto == "tcp" ? 6 : r.Proto == "udp" ? 17 : r.Proto == "icmp" ? 1 : 0;
        if (!proto) continue; // can never equal a parsed packet's protocol name (acl.go:150)
        for (const std::string &s : r.Srcs) {
            uint32_t addr;
            int bits;
            if (!parse_prefix(s, addr, bits)) continue;
            if (proto == 1) {
                out.push_back(bnk_acl_tuple{addr, (uint8_t)bits, proto, 0, 0, 0}); // icmp ignores ports (acl.go:163)
            } else {
                for (const PortRange &p : r.Ports)
                    if (p.First <= p.Last) out.push_back(bnk_acl_tuple{addr, (uint8_t)bits, proto, p.First, p.Last, 0});
            }
        }
    }
    return out;
}

// ---- Context / Batch ----
Context::Context(int device, uint32_t max_keypairs, uint32_t mtu, uint32_t flow_capacity, uint32_t replay_ring_blocks)
    : mtu_(mtu) {
    bnk_cfg cfg{};
    cfg.struct_size = sizeof cfg;
    cfg.device_id = device;
    cfg.max_keypairs = max_keypairs;
    cfg.replay_ring_blocks = replay_ring_blocks;
    cfg.mtu = mtu;
    cfg.flow_capacity = flow_capacity;
    const int rc = bnk_ctx_create(&cfg, &ctx_);
    if (rc != BNK_SUCCESS) throw Error(rc, std::string("bnk_ctx_create: ") + bnk_last_error_string(nullptr));
}

Context::~Context() {
    if (ctx_) bnk_ctx_destroy(ctx_);
}

void Context::Check(int rc) const {
    if (rc < 0) throw Error(rc, std::string(bnk_strerror(rc)) + ": " + bnk_last_error_string(ctx_));
}

uint64_t Context::LaunchCount() const {
    uint64_t n = 0;
    Check(bnk_kernel_launch_count(ctx_, &n));
    return n;
}

Batch::Batch(Context &ctx, uint32_t max_pkts, uint32_t slot_bytes) : ctx_(ctx), slot_((slot_bytes + 15u) & ~15u) {
    ctx_.Check(bnk_batch_create(ctx_.raw(), max_pkts, (uint64_t)max_pkts * slot_, &b_));
    ctx_.Check(bnk_batch_view_get(b_, &v_));
}

Batch::~Batch() {
    if (b_) bnk_batch_destroy(b_);
}

void Batch::Put(uint32_t i, const uint8_t *data, size_t len, uint32_t headroom, uint32_t keypair_slot) {
    if (i >= v_.max_pkts || headroom + len + 32 > slot_) throw Error(BNK_EINVAL, "packet does not fit its slot");
    v_.off[i] = i * slot_;
    v_.len[i] = (uint32_t)len;
    v_.slot[i] = keypair_slot;
    if (len) memcpy(slot(i) + headroom, data, len);
}

void Batch::Wait(uint64_t timeout_ns) { ctx_.Check(bnk_wait(b_, timeout_ns)); }

// ---- Filter ----
Filter::Filter(Context &ctx, uint32_t batch_pkts, uint32_t max_packet)
    : ctx_(ctx), batch_(ctx, batch_pkts, 16 + max_packet + 32) {
    ctx_.Check(bnk_acl_set(ctx_.raw(), 0, nullptr, 0)); // allow-all until rules are pushed (filter.go:41-43)
}

std::unique_ptr<Filter> Filter::New(Context &ctx, uint32_t batch_pkts, uint32_t max_packet) {
    return std::unique_ptr<Filter>(new Filter(ctx, batch_pkts, max_packet));
}

void Filter::SetRules(const std::vector<CompiledRule> &rules) {
    const std::vector<bnk_acl_tuple> t = FlattenRules(rules);
    ctx_.Check(bnk_acl_set(ctx_.raw(), 1, t.empty() ? nullptr : t.data(), t.size()));
}

void Filter::SetAllowAll() { ctx_.Check(bnk_acl_set(ctx_.raw(), 0, nullptr, 0)); }

uint32_t Filter::Load(const std::vector<Span> &pkts, size_t first) {
    const uint32_t n = (uint32_t)std::min<size_t>(batch_.capacity(), pkts.size() - first);
    for (uint32_t i = 0; i < n; i++) batch_.Put(i, pkts[first + i].data, pkts[first + i].len, 16);
    return n;
}

std::vector<uint8_t> Filter::CheckInboundBatch(const std::vector<Span> &pkts, TimeNs now) {
    std::vector<uint8_t> verdict(pkts.size(), 0);
    for (size_t first = 0; first < pkts.size(); first += batch_.capacity()) {
        const uint32_t n = Load(pkts, first);
        ctx_.Check(bnk_filter_check_submit(batch_.raw(), n, 0, now));
        batch_.Wait();
        for (uint32_t i = 0; i < n; i++) verdict[first + i] = batch_.view().status[i] == BNK_PKT_OK;
    }
    return verdict;
}

void Filter::NoteOutboundBatch(const std::vector<Span> &pkts, TimeNs now) {
    for (size_t first = 0; first < pkts.size(); first += batch_.capacity()) {
        const uint32_t n = Load(pkts, first);
        ctx_.Check(bnk_filter_note_submit(batch_.raw(), n, 0, now));
        batch_.Wait();
    }
}

bool Filter::CheckInbound(const uint8_t *pkt, size_t len, TimeNs now) {
    return CheckInboundBatch({Span{pkt, len}}, now)[0] != 0;
}

void Filter::NoteOutbound(const uint8_t *pkt, size_t len, TimeNs now) { NoteOutboundBatch({Span{pkt, len}}, now); }

uint64_t Filter::FlowCount() const {
    uint64_t live = 0;
    ctx_.Check(bnk_flows_count(ctx_.raw(), &live));
    return live;
}

// ---- WrapTUN ----
namespace {

class FilteredTUN final : public TunDevice { // filteredTUN, filter.go:155-186
  public:
    FilteredTUN(TunDevice *inner, Filter *f, std::function<TimeNs()> clock)
        : inner_(inner), f_(f), clock_(std::move(clock)) {}

    int Read(std::vector<Packet> &bufs, std::vector<int> &sizes, int offset) override {
        const int n = inner_->Read(bufs, sizes, offset);
        const TimeNs now = clock_(); // one clock sample per batch (filter.go:162)
        std::vector<Filter::Span> spans;
        for (int i = 0; i < n; i++) spans.push_back({bufs[i].data() + offset, (size_t)sizes[i]});
        f_->NoteOutboundBatch(spans, now);
        return n;
    }

    // Drops denied packets in place but still reports them written (filter.go:169-186).
    int Write(std::vector<Packet> &bufs, int offset) override {
        const TimeNs now = clock_();
        std::vector<Filter::Span> spans;
        for (const Packet &b : bufs)
            spans.push_back({b.data() + std::min<size_t>(offset, b.size()), b.size() > (size_t)offset ? b.size() - offset : 0});
        const std::vector<uint8_t> ok = f_->CheckInboundBatch(spans, now);
        std::vector<Packet> kept;
        for (size_t i = 0; i < bufs.size(); i++)
            if (ok[i]) kept.push_back(bufs[i]);
        if (kept.empty()) return (int)bufs.size();
        inner_->Write(kept, offset); // an inner failure propagates as the exception it throws
        return (int)bufs.size();
    }

    int MTU() override { return inner_->MTU(); }
    std::string Name() override { return inner_->Name(); }
    int BatchSize() override { return inner_->BatchSize(); }
    void Close() override { inner_->Close(); }

  private:
    TunDevice *inner_;
    Filter *f_;
    std::function<TimeNs()> clock_;
};

} // namespace

std::unique_ptr<TunDevice> WrapTUN(TunDevice *inner, Filter *f, std::function<TimeNs()> clock) {
    return std::unique_ptr<TunDevice>(new FilteredTUN(inner, f, std::move(clock)));
}

// ---- Device ----
Device::Device(Context &ctx, TunDevice *tun, Bind *bind, uint32_t batch_pkts, uint32_t coalesce)
    : ctx_(ctx), tun_(tun), bind_(bind),
      batch_(ctx, batch_pkts * std::max(1u, coalesce), 16 + ((ctx.mtu() ? ctx.mtu() : 1500) + 15) / 16 * 16 + 32),
      read_pkts_(batch_pkts), coalesce_(std::max(1u, coalesce)) {}

void Device::SetPeer(uint32_t slot, const uint8_t send_key[32], const uint8_t recv_key[32], uint32_t remote_index,
                     uint32_t local_index, uint32_t allowed_ip) {
    RemovePeer(slot);
    ctx_.Check(bnk_keypair_set(ctx_.raw(), slot, send_key, recv_key, remote_index));
    ctx_.Check(bnk_keypair_set_allowed_ip(ctx_.raw(), slot, allowed_ip));
    ctx_.Check(bnk_index_set(ctx_.raw(), local_index, slot));
    route_[allowed_ip] = slot;
    by_index_[slot] = local_index;
    src_of_[slot] = allowed_ip;
}

void Device::RemovePeer(uint32_t slot) {
    auto it = by_index_.find(slot);
    if (it == by_index_.end()) return;
    ctx_.Check(bnk_index_clear(ctx_.raw(), it->second));
    ctx_.Check(bnk_keypair_clear(ctx_.raw(), slot));
    route_.erase(src_of_[slot]);
    src_of_.erase(slot);
    by_index_.erase(it);
}

void Device::AttachFilter(Filter *f, std::function<TimeNs()> clock) {
    filter_ = f;
    clock_ = std::move(clock);
}

int Device::PumpOutbound() {
    // One GPU submit per pump: up to `coalesce` reads of the TUN, as long as each comes back full, go into the
    // same batch (packets of different reads are as independent as packets of one read; order is kept).
    const int cap = std::min<int>(read_pkts_, std::max(1, tun_->BatchSize()));
    const size_t room = (size_t)kOffset + (ctx_.mtu() ? ctx_.mtu() : 1500) + 32;
    if ((int)tx_bufs_.size() != cap) {
        tx_bufs_.assign(cap, Packet(room));
        tx_sizes_.assign(cap, 0);
    }
    uint32_t m = 0;
    std::vector<uint32_t> peer_of;
    for (uint32_t r = 0; r < coalesce_ && m + cap <= batch_.capacity(); r++) {
        const int n = tun_->Read(tx_bufs_, tx_sizes_, kOffset);
        for (int i = 0; i < n; i++) {
            const uint8_t *p = tx_bufs_[i].data() + kOffset;
            // outbound routing: destination address -> peer (allowed-IPs, one /32 per peer)
            if (tx_sizes_[i] < 20 || (p[0] >> 4) != 4) {
                stats_.no_route++;
                continue;
            }
            const uint32_t dst = ((uint32_t)p[16] << 24) | ((uint32_t)p[17] << 16) | ((uint32_t)p[18] << 8) | p[19];
            auto it = route_.find(dst);
            if (it == route_.end()) {
                stats_.no_route++;
                continue;
            }
            batch_.Put(m++, p, (size_t)tx_sizes_[i], kOffset, it->second);
            peer_of.push_back(it->second);
        }
        if (n < cap) break; // the TUN ran dry
    }
    if (m == 0) return 0;
    uint32_t flags = BNK_F_ASSIGN_COUNTERS;
    if (filter_) flags |= BNK_F_NOTE_OUTBOUND;
    ctx_.Check(bnk_seal_submit(batch_.raw(), m, flags, clock_()));
    batch_.Wait();
    // per-peer sends, batch order kept inside each peer (bind.go:296, called once per peer by the device);
    // peers in the order of their first packet
    int sent = 0;
    std::unordered_map<uint32_t, size_t> group_of;
    std::vector<std::pair<uint32_t, std::vector<Packet>>> groups;
    for (uint32_t j = 0; j < m; j++) {
        if (batch_.view().status[j] != BNK_PKT_OK) continue; // counter exhausted: dropped, a rekey is due
        auto it = group_of.find(peer_of[j]);
        if (it == group_of.end()) {
            it = group_of.emplace(peer_of[j], groups.size()).first;
            groups.emplace_back(peer_of[j], std::vector<Packet>());
        }
        const uint8_t *msg = batch_.slot(j);
        groups[it->second].second.emplace_back(msg, msg + batch_.view().out_len[j]);
        stats_.sealed++;
    }
    for (auto &g : groups) {
        bind_->Send(g.second, Endpoint{g.first});
        sent += (int)g.second.size();
    }
    return sent;
}

int Device::PumpInbound() {
    const int cap = std::min<int>(read_pkts_, std::max(1, bind_->BatchSize()));
    if ((int)rx_bufs_.size() != cap) {
        rx_bufs_.assign(cap, Packet(batch_.slot_bytes()));
        rx_sizes_.assign(cap, 0);
        rx_eps_.assign(cap, Endpoint{});
    }
    uint32_t m = 0;
    for (uint32_t r = 0; r < coalesce_ && m + cap <= batch_.capacity(); r++) {
        const int n = bind_->Receive(rx_bufs_, rx_sizes_, rx_eps_);
        for (int i = 0; i < n; i++) {
            if ((size_t)rx_sizes_[i] + 32 > batch_.slot_bytes()) {
                stats_.malformed++;
                continue;
            }
            batch_.Put(m++, rx_bufs_[i].data(), (size_t)rx_sizes_[i], 0, 0);
        }
        if (n < cap) break; // nothing more pending
    }
    if (m == 0) return 0;
    uint32_t flags = BNK_F_DEMUX_INDEX | BNK_F_REPLAY | BNK_F_INNER_CHECK;
    if (filter_) flags |= BNK_F_CHECK_INBOUND;
    ctx_.Check(bnk_open_submit(batch_.raw(), m, flags, clock_()));
    batch_.Wait();
    std::vector<Packet> up;
    for (uint32_t j = 0; j < m; j++) {
        switch (batch_.view().status[j]) {
        case BNK_PKT_OK: {
            Packet b((size_t)kOffset + batch_.view().out_len[j]);
            memcpy(b.data() + kOffset, batch_.slot(j) + 16, batch_.view().out_len[j]);
            up.push_back(std::move(b));
            stats_.opened++;
            break;
        }
        case BNK_PKT_KEEPALIVE: stats_.keepalive++; break;
        case BNK_PKT_AUTH_FAIL: stats_.auth_fail++; break;
        case BNK_PKT_REPLAY: stats_.replay++; break;
        case BNK_PKT_FILTER_DENY: stats_.filter_deny++; break;
        case BNK_PKT_BAD_INNER: stats_.bad_source++; break;
        default: stats_.malformed++; break;
        }
    }
    if (!up.empty()) tun_->Write(up, kOffset);
    return (int)up.size();
}

// ---- Dispatcher ----
Dispatcher::Dispatcher(const std::vector<int32_t> &devices, uint32_t max_peers, uint32_t max_pkts_per_gpu,
                       uint32_t max_packet, uint32_t flow_capacity)
    : max_peers_(max_peers), max_packet_(max_packet) {
    bnk_mgpu_cfg cfg{};
    cfg.struct_size = sizeof cfg;
    cfg.n_devices = (uint32_t)devices.size();
    cfg.devices = devices.data();
    cfg.max_pkts_per_gpu = max_pkts_per_gpu;
    cfg.max_packet = max_packet;
    cfg.max_peers = max_peers;
    cfg.ctx.struct_size = sizeof cfg.ctx;
    cfg.ctx.max_keypairs = max_peers;
    cfg.ctx.replay_ring_blocks = 128;
    cfg.ctx.mtu = max_packet;
    cfg.ctx.flow_capacity = flow_capacity;
    const int rc = bnk_mgpu_create(&cfg, &m_);
    if (rc != BNK_SUCCESS) throw Error(rc, std::string("bnk_mgpu_create: ") + bnk_last_error_string(nullptr));
}

Dispatcher::~Dispatcher() {
    if (m_) bnk_mgpu_destroy(m_);
}

void Dispatcher::Check(int rc) const {
    if (rc < 0) throw Error(rc, std::string(bnk_strerror(rc)) + ": " + bnk_mgpu_last_error_string(m_));
}

void Dispatcher::Place(const std::vector<uint64_t> &load) {
    if (!load.empty() && load.size() != max_peers_) throw Error(BNK_EINVAL, "one load per peer");
    Check(bnk_mgpu_place(m_, load.empty() ? nullptr : load.data()));
}

void Dispatcher::SetPeer(uint32_t peer, const uint8_t send_key[32], const uint8_t recv_key[32], uint32_t remote_index,
                         uint32_t local_index, uint32_t allowed_ip) {
    Check(bnk_mgpu_peer_set(m_, peer, send_key, recv_key, remote_index, local_index, allowed_ip));
}

void Dispatcher::RemovePeer(uint32_t peer) { Check(bnk_mgpu_peer_clear(m_, peer)); }

void Dispatcher::SetRules(const std::vector<CompiledRule> &rules) {
    const std::vector<bnk_acl_tuple> t = FlattenRules(rules);
    Check(bnk_mgpu_acl_set(m_, 1, t.empty() ? nullptr : t.data(), t.size()));
}

Dispatcher::Result Dispatcher::Seal(const std::vector<Packet> &pkts, const std::vector<uint32_t> &peers, uint32_t flags,
                                    TimeNs now) {
    const uint32_t n = (uint32_t)pkts.size();
    if (peers.size() != n) throw Error(BNK_EINVAL, "one peer per packet");
    Result r;
    r.out.assign(n, Packet(max_packet_ + 64));
    r.status.assign(n, 0);
    r.counter.assign(n, 0);
    std::vector<const uint8_t *> in(n);
    std::vector<uint8_t *> out(n);
    std::vector<uint32_t> len(n), out_len(n);
    for (uint32_t i = 0; i < n; i++) {
        in[i] = pkts[i].data();
        len[i] = (uint32_t)pkts[i].size();
        out[i] = r.out[i].data();
    }
    Check(bnk_mgpu_seal(m_, in.data(), len.data(), peers.data(), n, flags, now, out.data(), out_len.data(), r.counter.data(),
                        r.status.data()));
    for (uint32_t i = 0; i < n; i++) r.out[i].resize(out_len[i]);
    return r;
}

Dispatcher::Result Dispatcher::Open(const std::vector<Packet> &msgs, uint32_t flags, TimeNs now) {
    const uint32_t n = (uint32_t)msgs.size();
    Result r;
    r.out.assign(n, Packet(max_packet_ + 64));
    r.status.assign(n, 0);
    r.counter.assign(n, 0);
    r.peer.assign(n, 0);
    std::vector<const uint8_t *> in(n);
    std::vector<uint8_t *> out(n);
    std::vector<uint32_t> len(n), out_len(n);
    for (uint32_t i = 0; i < n; i++) {
        in[i] = msgs[i].data();
        len[i] = (uint32_t)msgs[i].size();
        out[i] = r.out[i].data();
    }
    Check(bnk_mgpu_open(m_, in.data(), len.data(), n, flags, now, out.data(), out_len.data(), r.counter.data(), r.peer.data(),
                        r.status.data()));
    for (uint32_t i = 0; i < n; i++) r.out[i].resize(out_len[i]);
    return r;
}

// ---- Queue ----
Queue::Queue(Context &ctx, bool open_side, uint32_t flags, uint32_t max_pkts, uint32_t max_packet, uint32_t depth)
    : ctx_(ctx), open_side_(open_side), max_packet_(max_packet) {
    bnk_queue_cfg cfg{};
    cfg.struct_size = sizeof cfg;
    cfg.max_pkts = max_pkts;
    cfg.max_packet = max_packet;
    cfg.depth = depth;
    cfg.open_side = open_side ? 1u : 0u;
    cfg.flags = flags;
    ctx_.Check(bnk_queue_create(ctx.raw(), &cfg, &q_));
}

Queue::~Queue() {
    if (q_) bnk_queue_destroy(q_);
}

Queue::Result Queue::Run(const std::vector<Packet> &pkts, const std::vector<uint32_t> &slots, TimeNs now) {
    const uint32_t n = (uint32_t)pkts.size();
    Result r;
    if (n == 0) return r;
    std::vector<const uint8_t *> in(n);
    std::vector<uint32_t> len(n);
    static const uint8_t none = 0;
    for (uint32_t i = 0; i < n; i++) {
        in[i] = pkts[i].empty() ? &none : pkts[i].data();
        len[i] = (uint32_t)pkts[i].size();
    }
    bnk_ticket t = 0;
    for (;;) {
        const int rc = bnk_queue_submit(q_, in.data(), len.data(), slots.empty() ? nullptr : slots.data(), n, now, &t);
        if (rc == BNK_SUCCESS) break;
        if (rc != BNK_EBUSY) ctx_.Check(rc);
        bnk_queue_wait_room(q_, 1000000);
    }
    const uint32_t room = max_packet_ + 64;
    std::vector<uint8_t> flat((size_t)n * room);
    std::vector<uint8_t *> out(n);
    std::vector<uint32_t> out_len(n);
    for (uint32_t i = 0; i < n; i++) out[i] = flat.data() + (size_t)i * room;
    r.status.resize(n);
    r.counter.resize(n);
    r.slot.resize(n);
    ctx_.Check(bnk_queue_wait(q_, t, out.data(), out_len.data(), r.counter.data(), r.slot.data(), r.status.data()));
    r.out.resize(n);
    for (uint32_t i = 0; i < n; i++) r.out[i].assign(out[i], out[i] + out_len[i]);
    return r;
}

Queue::Span Queue::Reserve(uint32_t n, TimeNs now) {
    Span sp;
    sp.n = n;
    for (;;) {
        const int rc = bnk_queue_reserve(q_, n, now, &sp.ticket, &sp.s);
        if (rc == BNK_SUCCESS) return sp;
        if (rc != BNK_EBUSY) ctx_.Check(rc);
        bnk_queue_wait_room(q_, 1000000);
    }
}

void Queue::Commit(const Span &sp) { ctx_.Check(bnk_queue_commit(q_, sp.ticket)); }
void Queue::Wait(Span &sp) { ctx_.Check(bnk_queue_wait_span(q_, sp.ticket, &sp.s)); }
void Queue::Release(const Span &sp) { ctx_.Check(bnk_queue_release(q_, sp.ticket)); }

} // namespace bnk
