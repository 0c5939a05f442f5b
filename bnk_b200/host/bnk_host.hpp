// C++ host side above the C ABI: the reference's Go interfaces for the hot path, name for name.
//
//   bnk::Filter            filter.Filter            internal/filter/filter.go:33-59, :121-147, :189-209
//   bnk::CompiledRule      acl.CompiledRule         internal/acl/acl.go:33-42
//   bnk::TunDevice         tun.Device (wireguard-go) as the reference uses it, internal/filter/tun_test.go:19-41
//   bnk::WrapTUN           filter.WrapTUN           internal/filter/filter.go:151-186
//   bnk::Bind, Endpoint    conn.Bind / conn.Endpoint, internal/magicsock/bind.go:72, :296, :111
//   bnk::Device            the packet path of device.NewDevice(tun, bind, logger), internal/dataplane/engine.go:51
//
// Every packet decision is made by the CUDA kernels behind include/bnk_gpu.h; this layer moves bytes
// between the caller's buffers and the pinned rings and keeps the Go calling conventions: Write reports
// len(bufs) even when the filter dropped packets, inner errors propagate (here: as exceptions), one clock
// sample per batch.  Go's (value, error) returns become return values plus bnk::Error.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/bnk_gpu.h"

namespace bnk {

using TimeNs = int64_t; // time.Time as unix nanoseconds
using Packet = std::vector<uint8_t>;

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &what) : std::runtime_error(what), code(c) {}
};

TimeNs Now(); // time.Now()

// ---- acl ----
struct PortRange { // acl.PortRange
    uint16_t First, Last;
};
struct CompiledRule { // acl.CompiledRule; Srcs are CIDR strings as in the JSON the server pushes
    std::vector<std::string> Srcs;
    std::string Proto; // "tcp" | "udp" | "icmp"
    std::vector<PortRange> Ports;
};
// Expands rules to the device's allowance tuples (the cross product acl.CompiledRule.Match walks, acl.go:149-172).
std::vector<bnk_acl_tuple> FlattenRules(const std::vector<CompiledRule> &rules);

// ---- one GPU ----
class Context {
  public:
    explicit Context(int device = 0, uint32_t max_keypairs = 1024, uint32_t mtu = 1420, uint32_t flow_capacity = 1u << 16,
                     uint32_t replay_ring_blocks = 128);
    ~Context();
    Context(const Context &) = delete;
    Context &operator=(const Context &) = delete;
    bnk_ctx *raw() const { return ctx_; }
    uint32_t mtu() const { return mtu_; }
    void Check(int rc) const; // throws bnk::Error with the library's message
    uint64_t LaunchCount() const; // kernels launched through this context so far

  private:
    bnk_ctx *ctx_ = nullptr;
    uint32_t mtu_;
};

// A pinned ring with fixed-stride slots; thin RAII over bnk_batch.
class Batch {
  public:
    Batch(Context &ctx, uint32_t max_pkts, uint32_t slot_bytes);
    ~Batch();
    Batch(const Batch &) = delete;
    Batch &operator=(const Batch &) = delete;
    bnk_batch *raw() const { return b_; }
    const bnk_batch_view &view() const { return v_; }
    uint32_t capacity() const { return v_.max_pkts; }
    uint32_t slot_bytes() const { return slot_; }
    uint8_t *slot(uint32_t i) const { return v_.ring + (size_t)i * slot_; }
    // lays `len` bytes at slot i + headroom and fills the descriptor
    void Put(uint32_t i, const uint8_t *data, size_t len, uint32_t headroom, uint32_t keypair_slot = 0);
    void Wait(uint64_t timeout_ns = UINT64_MAX);

  private:
    Context &ctx_;
    bnk_batch *b_ = nullptr;
    bnk_batch_view v_{};
    uint32_t slot_;
};

// ---- filter.Filter ----
class Filter {
  public:
    static std::unique_ptr<Filter> New(Context &ctx, uint32_t batch_pkts = 128, uint32_t max_packet = 2048); // filter.New
    void SetRules(const std::vector<CompiledRule> &rules);                                                  // filter.go:46
    void SetAllowAll();                                                                                     // filter.go:54
    bool CheckInbound(const uint8_t *pkt, size_t len, TimeNs now);                                          // filter.go:121
    bool CheckInbound(const Packet &pkt, TimeNs now) { return CheckInbound(pkt.data(), pkt.size(), now); }
    void NoteOutbound(const uint8_t *pkt, size_t len, TimeNs now);                                          // filter.go:189
    void NoteOutbound(const Packet &pkt, TimeNs now) { NoteOutbound(pkt.data(), pkt.size(), now); }
    // the loops of filteredTUN.Read / Write as one GPU batch each (one `now` per batch, as in the reference)
    struct Span {
        const uint8_t *data;
        size_t len;
    };
    std::vector<uint8_t> CheckInboundBatch(const std::vector<Span> &pkts, TimeNs now); // 1 = allowed
    void NoteOutboundBatch(const std::vector<Span> &pkts, TimeNs now);
    uint64_t FlowCount() const; // len(f.flows)
    Context &context() const { return ctx_; }

  private:
    Filter(Context &ctx, uint32_t batch_pkts, uint32_t max_packet);
    uint32_t Load(const std::vector<Span> &pkts, size_t first);
    Context &ctx_;
    Batch batch_;
};

// ---- tun.Device ----
// Packet i of a batch lives at bufs[i][offset : offset+sizes[i]]; the headroom in front is the caller's.
class TunDevice {
  public:
    virtual ~TunDevice() = default;
    virtual int Read(std::vector<Packet> &bufs, std::vector<int> &sizes, int offset) = 0;
    virtual int Write(std::vector<Packet> &bufs, int offset) = 0;
    virtual int MTU() = 0;
    virtual std::string Name() = 0;
    virtual int BatchSize() = 0;
    virtual void Close() {}
};

// filter.WrapTUN: inbound Writes are checked, outbound Reads feed the flow table.
std::unique_ptr<TunDevice> WrapTUN(TunDevice *inner, Filter *f, std::function<TimeNs()> clock = Now);

// ---- conn.Bind ----
struct Endpoint { // conn.Endpoint: which peer path a datagram belongs to
    uint32_t peer = 0;
};
class Bind {
  public:
    virtual ~Bind() = default;
    virtual void Send(std::vector<Packet> &bufs, const Endpoint &ep) = 0; // bind.go:296
    // conn.ReceiveFunc, bind.go:111,153: fills packets/sizes/eps, returns the count (0 = nothing pending)
    virtual int Receive(std::vector<Packet> &packets, std::vector<int> &sizes, std::vector<Endpoint> &eps) = 0;
    virtual int BatchSize() = 0; // bind.go:372
};

// ---- the device ----
// Stands where device.NewDevice(tun, bind, logger) stands: reads plaintext batches from the TUN, seals them on
// the GPU and hands them to the Bind; takes datagram batches from the Bind, opens them on the GPU (replay window
// included) and writes the survivors to the TUN.  Handshakes, timers and roaming stay outside: keys arrive
// through SetPeer, as they would after a completed handshake.
class Device {
  public:
    static constexpr int kOffset = 16; // transport header room kept in front of every TUN packet

    // `coalesce`: how many full reads of the TUN (or receive calls of the Bind) one pump may put into a single
    // GPU submit.  1 keeps the reference's batch size; the GPU pays off from about a thousand packets per submit.
    Device(Context &ctx, TunDevice *tun, Bind *bind, uint32_t batch_pkts = 128, uint32_t coalesce = 1);
    // keypair slot `slot`; `local_index` is the receiver index peers put in messages for us, `remote_index` the one
    // we put in messages for them; `allowed_ip` the peer's tunnel address (one /32 per peer, engine.go:294)
    void SetPeer(uint32_t slot, const uint8_t send_key[32], const uint8_t recv_key[32], uint32_t remote_index,
                 uint32_t local_index, uint32_t allowed_ip);
    void RemovePeer(uint32_t slot);
    // When a filter is attached the device runs NoteOutbound / CheckInbound inside the seal / open submits;
    // pass the raw TUN in that case, not a WrapTUN'd one.
    void AttachFilter(Filter *f, std::function<TimeNs()> clock = Now);
    int PumpOutbound(); // one TUN read batch -> seal -> Bind.Send per peer; returns datagrams sent
    int PumpInbound();  // one receive batch -> open -> TUN write; returns packets written
    struct Counters {
        uint64_t sealed = 0, opened = 0, auth_fail = 0, replay = 0, filter_deny = 0, malformed = 0, keepalive = 0,
                 no_route = 0, bad_source = 0;
    };
    const Counters &counters() const { return stats_; }

  private:
    Context &ctx_;
    TunDevice *tun_;
    Bind *bind_;
    Batch batch_;
    uint32_t read_pkts_, coalesce_;
    std::vector<Packet> tx_bufs_, rx_bufs_; // reused between pumps
    std::vector<int> tx_sizes_, rx_sizes_;
    std::vector<Endpoint> rx_eps_;
    Filter *filter_ = nullptr;
    std::function<TimeNs()> clock_ = Now;
    std::unordered_map<uint32_t, uint32_t> route_;    // allowed ip -> keypair slot
    std::unordered_map<uint32_t, uint32_t> by_index_; // local receiver index -> keypair slot
    std::unordered_map<uint32_t, uint32_t> src_of_;   // keypair slot -> allowed ip
    Counters stats_;
};

// ---- several GPUs ----
// RAII over bnk_mgpu: one context per listed device, peers placed by measured load, mixed batches routed by
// peer (see include/bnk_gpu.h).  Stands where Device stands when a box has more than one GPU; a peer's packets
// always meet on one GPU, as the reference gives each peer one sequential worker (bind.go:325-328).
class Dispatcher {
  public:
    Dispatcher(const std::vector<int32_t> &devices, uint32_t max_peers, uint32_t max_pkts_per_gpu = 4096,
               uint32_t max_packet = 1420, uint32_t flow_capacity = 1u << 16);
    ~Dispatcher();
    Dispatcher(const Dispatcher &) = delete;
    Dispatcher &operator=(const Dispatcher &) = delete;
    bnk_mgpu *raw() const { return m_; }
    void Check(int rc) const;
    void Place(const std::vector<uint64_t> &load); // empty = equal loads
    void SetPeer(uint32_t peer, const uint8_t send_key[32], const uint8_t recv_key[32], uint32_t remote_index,
                 uint32_t local_index, uint32_t allowed_ip);
    void RemovePeer(uint32_t peer);
    void SetRules(const std::vector<CompiledRule> &rules); // on every GPU
    struct Result {
        std::vector<Packet> out;      // sealed messages, or opened plaintexts
        std::vector<uint8_t> status;  // BNK_PKT_*
        std::vector<uint64_t> counter;
        std::vector<uint32_t> peer;   // open: the peer each message belongs to
    };
    Result Seal(const std::vector<Packet> &pkts, const std::vector<uint32_t> &peers, uint32_t flags = 0, TimeNs now = 0);
    Result Open(const std::vector<Packet> &msgs, uint32_t flags = BNK_F_REPLAY, TimeNs now = 0);

  private:
    bnk_mgpu *m_ = nullptr;
    uint32_t max_peers_, max_packet_;
};

// RAII over bnk_queue: the workers of one direction hand their upstream-sized batches (conn.IdealBatchSize = 128,
// bind.go:97) to one queue, which packs them into GPU batches (see include/bnk_gpu.h).  Thread-safe; one Queue per
// direction and set of flags.
class Queue {
  public:
    Queue(Context &ctx, bool open_side, uint32_t flags, uint32_t max_pkts = 1024, uint32_t max_packet = 1420, uint32_t depth = 3);
    ~Queue();
    Queue(const Queue &) = delete;
    Queue &operator=(const Queue &) = delete;
    bnk_queue *raw() const { return q_; }
    struct Result {
        std::vector<Packet> out;     // sealed messages, or opened plaintexts; empty where the packet was refused
        std::vector<uint8_t> status; // BNK_PKT_*
        std::vector<uint64_t> counter;
        std::vector<uint32_t> slot;
    };
    // Copying form: hand in, wait, get everything back (blocks; collects room by itself when the queue is full).
    Result Run(const std::vector<Packet> &pkts, const std::vector<uint32_t> &slots, TimeNs now = 0);
    // Span form: write into / read from the GPU batch's pinned ring.  Reserve blocks until there is room.
    struct Span {
        bnk_ticket ticket = 0;
        uint32_t n = 0;
        bnk_queue_span s{};
        uint8_t *packet(uint32_t k) const { return s.data + (size_t)k * s.stride; }
    };
    Span Reserve(uint32_t n, TimeNs now = 0);
    void Commit(const Span &sp);
    void Wait(Span &sp);   // results of the span are valid from here until Release
    void Release(const Span &sp);

  private:
    Context &ctx_;
    bnk_queue *q_ = nullptr;
    bool open_side_;
    uint32_t max_packet_;
};

} // namespace bnk
