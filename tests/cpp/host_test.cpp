// The reference's Go tests for the hot path, restated against the C++ host mirror (bnk_b200/host/bnk_host.hpp):
//   internal/filter/filter_test.go:56-170, internal/filter/tun_test.go:43-94, internal/acl/acl_test.go:83-114,
// plus the functional round trip the reference's device tests make (internal/dataplane/device_test.go:85-91):
// two devices joined by an in-memory bind, packets written into one TUN come out of the other.
// Needs a B200: every verdict and every ciphertext byte is produced by libbnkgpu.so.
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <deque>
#include <thread>
#include <string>

#include "../../bnk_b200/host/bnk_host.hpp"

using namespace bnk;

static int g_failed = 0, g_checks = 0;
static const char *g_test = "";
#define CHECK(cond, msg)                                                      \
    do {                                                                      \
        g_checks++;                                                           \
        if (!(cond)) {                                                        \
            g_failed++;                                                       \
            printf("FAIL %s: %s (%s:%d)\n", g_test, msg, __FILE__, __LINE__); \
        }                                                                     \
    } while (0)

// ---- packet builders, filter_test.go:13-54 ----
static uint32_t ip(int a, int b, int c, int d) { return ((uint32_t)a << 24) | (b << 16) | (c << 8) | d; }
static void put16(Packet &p, size_t at, uint16_t v) { p[at] = v >> 8; p[at + 1] = v & 0xff; }
static void put32(Packet &p, size_t at, uint32_t v) { put16(p, at, v >> 16); put16(p, at + 2, v & 0xffff); }
static Packet ipv4(uint8_t proto, uint32_t src, uint32_t dst, const Packet &payload) {
    Packet pkt(20 + payload.size());
    pkt[0] = 0x45;
    put16(pkt, 2, (uint16_t)pkt.size());
    pkt[8] = 64;
    pkt[9] = proto;
    put32(pkt, 12, src);
    put32(pkt, 16, dst);
    std::copy(payload.begin(), payload.end(), pkt.begin() + 20);
    return pkt;
}
static Packet tcp(uint32_t src, uint32_t dst, uint16_t sport, uint16_t dport, bool syn) {
    Packet h(20);
    put16(h, 0, sport);
    put16(h, 2, dport);
    h[12] = 5 << 4;
    h[13] = syn ? 0x02 : 0x10;
    return ipv4(6, src, dst, h);
}
static Packet udp(uint32_t src, uint32_t dst, uint16_t sport, uint16_t dport) {
    Packet h(8);
    put16(h, 0, sport);
    put16(h, 2, dport);
    put16(h, 4, 8);
    return ipv4(17, src, dst, h);
}
static Packet icmpEcho(uint32_t src, uint32_t dst, bool reply) {
    Packet h(8);
    h[0] = reply ? 0 : 8;
    return ipv4(1, src, dst, h);
}

static const uint32_t peer = ip(100, 64, 0, 9), other = ip(100, 64, 0, 7), self = ip(100, 64, 0, 1);
static const TimeNs SEC = 1000000000ll, MIN = 60 * SEC, t0 = 1700000000ll * SEC; // filter_test.go:57-60

static std::unique_ptr<Filter> sshOnlyFilter(Context &ctx) { // filter_test.go:63-71
    bnk_flows_clear(ctx.raw());
    auto f = Filter::New(ctx);
    f->SetRules({CompiledRule{{"100.64.0.9/32"}, "tcp", {PortRange{22, 22}}}});
    return f;
}
static std::unique_ptr<Filter> fresh(Context &ctx) {
    bnk_flows_clear(ctx.raw());
    return Filter::New(ctx);
}

static void TestAllowAllModePassesEverything(Context &ctx) {
    auto f = fresh(ctx);
    CHECK(f->CheckInbound(tcp(peer, self, 5555, 23, true), t0), "allow-all dropped a packet");
}
static void TestRuleAllowsMatchingInbound(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    CHECK(f->CheckInbound(tcp(peer, self, 5555, 22, true), t0), "rule-allowed tcp/22 dropped");
}
static void TestDefaultDenyDropsNonMatching(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    CHECK(!f->CheckInbound(tcp(peer, self, 5555, 23, true), t0), "tcp/23 passed despite ssh-only policy");
    CHECK(!f->CheckInbound(tcp(other, self, 5555, 22, true), t0), "tcp/22 from disallowed source passed");
    CHECK(!f->CheckInbound(udp(peer, self, 53, 22), t0), "udp passed a tcp-only rule");
}
static void TestReturnTrafficAllowedViaFlowTable(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    f->NoteOutbound(udp(self, peer, 40000, 9999), t0);
    CHECK(f->CheckInbound(udp(peer, self, 9999, 40000), t0 + 2 * SEC), "UDP reply to our own outbound flow was dropped");
    CHECK(!f->CheckInbound(udp(peer, self, 9999, 40000), t0 + 5 * MIN), "UDP reply passed long after the flow expired");
    CHECK(!f->CheckInbound(udp(peer, self, 9998, 40000), t0 + SEC), "UDP from a different source port matched the flow");
}
static void TestTCPReturnFlowAllowed(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    f->NoteOutbound(tcp(self, peer, 40000, 8080, true), t0);
    CHECK(f->CheckInbound(tcp(peer, self, 8080, 40000, false), t0 + SEC), "TCP reply to our outbound connection was dropped");
    CHECK(!f->CheckInbound(tcp(peer, self, 8081, 40000, false), t0 + SEC), "TCP from wrong port matched the flow");
}
static void TestICMPEchoReplyViaFlow(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    f->NoteOutbound(icmpEcho(self, peer, false), t0);
    CHECK(f->CheckInbound(icmpEcho(peer, self, true), t0 + SEC), "ICMP echo reply to our ping was dropped");
    CHECK(!f->CheckInbound(icmpEcho(other, self, true), t0 + SEC), "ICMP reply from a host we never pinged passed");
}
static void TestICMPRuleAllowsInboundPing(Context &ctx) {
    auto f = fresh(ctx);
    f->SetRules({CompiledRule{{"100.64.0.9/32"}, "icmp", {}}});
    CHECK(f->CheckInbound(icmpEcho(peer, self, false), t0), "icmp rule did not allow inbound ping");
}
static void TestMalformedAndNonIPv4Dropped(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    CHECK(!f->CheckInbound(Packet{0x60, 0x00, 0x00}, t0), "IPv6/short packet passed while enforcing");
    CHECK(!f->CheckInbound(nullptr, 0, t0), "nil packet passed");
    Packet truncated = tcp(peer, self, 1, 22, true);
    truncated.resize(22);
    CHECK(!f->CheckInbound(truncated, t0), "truncated transport header passed");
}
static void TestSetAllowAllDisablesEnforcement(Context &ctx) {
    auto f = sshOnlyFilter(ctx);
    f->SetAllowAll();
    CHECK(f->CheckInbound(tcp(other, self, 5555, 23, true), t0), "allow-all after rules still dropped");
}
static void TestCompiledRuleMatch(Context &ctx) { // acl_test.go:83-107 through the filter
    auto f = fresh(ctx);
    f->SetRules({CompiledRule{{"100.64.0.1/32"}, "tcp", {PortRange{22, 22}, PortRange{8000, 9000}}}});
    const uint32_t a = ip(100, 64, 0, 1), b = ip(100, 64, 0, 9);
    CHECK(f->CheckInbound(tcp(a, self, 1, 22, true), t0), "tcp/22");
    CHECK(f->CheckInbound(tcp(a, self, 1, 8500, true), t0), "tcp/8500");
    CHECK(!f->CheckInbound(tcp(a, self, 1, 23, true), t0), "tcp/23");
    CHECK(!f->CheckInbound(udp(a, self, 1, 22), t0), "udp/22");
    CHECK(!f->CheckInbound(tcp(b, self, 1, 22, true), t0), "other source");
}
static void TestICMPRuleIgnoresPorts(Context &ctx) { // acl_test.go:109-114
    auto f = fresh(ctx);
    f->SetRules({CompiledRule{{"100.64.0.0/10"}, "icmp", {}}});
    CHECK(f->CheckInbound(icmpEcho(ip(100, 64, 0, 1), self, false), t0), "icmp rule did not match");
    CHECK(!f->CheckInbound(icmpEcho(ip(100, 128, 0, 1), self, false), t0), "address outside the /10 matched");
}

// ---- fakeTUN, tun_test.go:13-41 ----
struct FakeTUN : TunDevice {
    std::vector<Packet> written;
    std::deque<Packet> pending;
    int Read(std::vector<Packet> &bufs, std::vector<int> &sizes, int offset) override {
        int n = 0;
        while (n < (int)bufs.size() && !pending.empty()) {
            const Packet &pkt = pending.front();
            if (bufs[n].size() < offset + pkt.size()) bufs[n].resize(offset + pkt.size());
            std::copy(pkt.begin(), pkt.end(), bufs[n].begin() + offset);
            sizes[n] = (int)pkt.size();
            pending.pop_front();
            n++;
        }
        return n;
    }
    int Write(std::vector<Packet> &bufs, int offset) override {
        for (const Packet &b : bufs) written.emplace_back(b.begin() + offset, b.end());
        return (int)bufs.size();
    }
    int MTU() override { return 1280; }
    std::string Name() override { return "fake0"; }
    int BatchSize() override { return 4; }
};
static Packet pad(const Packet &p, int offset) {
    Packet out(offset);
    out.insert(out.end(), p.begin(), p.end());
    return out;
}
static void TestWrapTUNDropsDeniedInboundWrites(Context &ctx) { // tun_test.go:43-66
    FakeTUN inner;
    auto f = sshOnlyFilter(ctx);
    auto wrapped = WrapTUN(&inner, f.get(), [] { return t0; });
    const Packet allowed = tcp(peer, self, 5555, 22, true), denied = tcp(peer, self, 5555, 23, true);
    std::vector<Packet> bufs{pad(allowed, 16), pad(denied, 16)};
    const int n = wrapped->Write(bufs, 16);
    CHECK(n == 2, "Write must report 2: denied packets are silently dropped");
    CHECK(inner.written.size() == 1, "inner TUN must get only the allowed packet");
    CHECK(!inner.written.empty() && inner.written[0] == allowed, "the surviving packet is not the allowed one");
    std::vector<Packet> all_denied{pad(denied, 16)};
    CHECK(wrapped->Write(all_denied, 16) == 1 && inner.written.size() == 1, "all-denied batch still reports its length");
}
static void TestWrapTUNReadRecordsOutboundFlows(Context &ctx) { // tun_test.go:68-94
    FakeTUN inner;
    auto f = fresh(ctx);
    f->SetRules({}); // deny-all policy: only flows admit traffic
    auto wrapped = WrapTUN(&inner, f.get(), [] { return t0; });
    inner.pending.push_back(udp(self, peer, 40000, 9999));
    std::vector<Packet> bufs{Packet(2048)};
    std::vector<int> sizes(1);
    CHECK(wrapped->Read(bufs, sizes, 16) == 1, "read one packet");
    const Packet reply = udp(peer, self, 9999, 40000), unrelated = udp(peer, self, 9999, 40001);
    std::vector<Packet> in{pad(reply, 16), pad(unrelated, 16)};
    wrapped->Write(in, 16);
    CHECK(inner.written.size() == 1 && inner.written[0] == reply, "inner must get just the reply");
}

// ---- two devices over an in-memory bind ----
struct WireBind : Bind {
    std::deque<Packet> *tx = nullptr, *rx = nullptr;
    void Send(std::vector<Packet> &bufs, const Endpoint &) override {
        for (Packet &b : bufs) tx->push_back(b);
    }
    int Receive(std::vector<Packet> &packets, std::vector<int> &sizes, std::vector<Endpoint> &) override {
        int n = 0;
        while (n < (int)packets.size() && !rx->empty()) {
            packets[n].assign(rx->front().begin(), rx->front().end());
            sizes[n] = (int)rx->front().size();
            rx->pop_front();
            n++;
        }
        return n;
    }
    int BatchSize() override { return 128; }
};

static void TestTwoDevicesRoundTrip(Context &) {
    // two nodes, each with its own tables (keypairs, rules, flows), here on the same GPU
    Context ctxA(0, 16, 1420, 1u << 12), ctxB(0, 16, 1420, 1u << 12);
    std::deque<Packet> a2b, b2a;
    WireBind bindA, bindB;
    bindA.tx = &a2b; bindA.rx = &b2a;
    bindB.tx = &b2a; bindB.rx = &a2b;
    FakeTUN tunA, tunB;
    Device A(ctxA, &tunA, &bindA), B(ctxB, &tunB, &bindB);
    uint8_t kAB[32], kBA[32];
    for (int i = 0; i < 32; i++) { kAB[i] = (uint8_t)(i * 7 + 1); kBA[i] = (uint8_t)(200 - i); }
    const uint32_t ipA = ip(100, 64, 0, 1), ipB = ip(100, 64, 0, 2);
    A.SetPeer(0, kAB, kBA, /*remote_index=*/0xB0B0B0B0u, /*local_index=*/0xA0A0A0A0u, ipB);
    B.SetPeer(1, kBA, kAB, /*remote_index=*/0xA0A0A0A0u, /*local_index=*/0xB0B0B0B0u, ipA);
    auto fB = Filter::New(ctxB);
    fB->SetRules({CompiledRule{{"100.64.0.1/32"}, "tcp", {PortRange{7777, 7777}}}}); // acl_integration_test.go:20-80
    B.AttachFilter(fB.get(), [] { return t0; });

    std::vector<Packet> sent;
    for (int i = 0; i < 4; i++) sent.push_back(tcp(ipA, ipB, 40000 + i, 7777, true));
    sent.push_back(tcp(ipA, ipB, 40010, 8888, true));       // blocked port
    sent.push_back(tcp(ip(100, 64, 0, 3), ipB, 1, 7777, true)); // spoofed source: not A's allowed address
    sent.push_back(udp(ipA, ip(100, 64, 0, 99), 1, 2));      // no peer owns that address: never leaves A
    for (const Packet &p : sent) tunA.pending.push_back(p);
    int out = 0, rounds = 0;
    while (!tunA.pending.empty() && rounds++ < 8) out += A.PumpOutbound();
    CHECK(out == 6, "six packets have a route");
    CHECK(A.counters().no_route == 1, "one packet has no route");
    CHECK(a2b.size() == 6, "six datagrams on the wire");
    const std::deque<Packet> wire = a2b; // keep the ciphertext for the replay below
    bool headers_ok = true;
    uint64_t ctr = 0;
    for (const Packet &m : wire) {
        headers_ok = headers_ok && m.size() == 16 + 48 + 16 && m[0] == 4 && m[1] == 0 && m[4] == 0xB0;
        uint64_t c = 0;
        memcpy(&c, m.data() + 8, 8);
        headers_ok = headers_ok && c == ctr++;
    }
    CHECK(headers_ok, "transport headers: type 4, receiver index of B, counters 0..5 in send order");
    int in = 0;
    while (!a2b.empty()) in += B.PumpInbound();
    CHECK(in == 4 && tunB.written.size() == 4, "four packets reach B's TUN");
    bool same = tunB.written.size() == 4;
    for (int i = 0; same && i < 4; i++) same = tunB.written[i] == sent[i];
    CHECK(same, "plaintext arrives byte for byte, in order");
    CHECK(B.counters().filter_deny == 1, "tcp/8888 is blocked by B's filter");
    CHECK(B.counters().bad_source == 1, "spoofed inner source is dropped");
    // replay the same ciphertext: every datagram is refused by the window
    a2b = wire;
    while (!a2b.empty()) B.PumpInbound();
    CHECK(B.counters().replay == 6 && tunB.written.size() == 4, "replayed datagrams are dropped");
    // a flipped bit fails authentication; a datagram for an unknown receiver index is ignored
    Packet bad = wire.front();
    bad[20] ^= 1;
    Packet stranger = wire.front();
    stranger[5] ^= 0x55;
    a2b.push_back(bad);
    a2b.push_back(stranger);
    B.PumpInbound();
    CHECK(B.counters().auth_fail == 1 && B.counters().malformed == 1, "forged and stranger datagrams are dropped");
    // B answers on the flow A opened: A has no rule for it, only the reply-flow entry (A's filter sees its own sends)
    auto fA = Filter::New(ctxA);
    fA->SetRules({});
    A.AttachFilter(fA.get(), [] { return t0 + SEC; });
    tunA.pending.push_back(tcp(ipA, ipB, 41000, 7777, true));
    A.PumpOutbound();
    while (!a2b.empty()) B.PumpInbound();
    tunB.pending.push_back(tcp(ipB, ipA, 7777, 41000, false)); // reply
    tunB.pending.push_back(tcp(ipB, ipA, 7777, 41001, false)); // not a reply to anything
    B.PumpOutbound();
    while (!b2a.empty()) A.PumpInbound();
    CHECK(tunA.written.size() == 1 && tunA.written[0] == tcp(ipB, ipA, 7777, 41000, false), "only the reply reaches A's TUN");
}

// One pump, several reads: 40 packets for three peers wait in a TUN that hands out 4 per read; a device that may
// coalesce 16 reads seals them in one submit, counters still run in TUN order per peer, and the receiving device
// (which coalesces its receive calls the same way) writes them to its TUN in order.
static void TestCoalescedPumps(Context &) {
    Context ctxA(0, 16, 1420, 1u << 12), ctxB(0, 16, 1420, 1u << 12);
    std::deque<Packet> a2b, b2a;
    WireBind bindA, bindB;
    bindA.tx = &a2b; bindA.rx = &b2a;
    bindB.tx = &b2a; bindB.rx = &a2b;
    FakeTUN tunA, tunB;
    Device A(ctxA, &tunA, &bindA, 4, 16), B(ctxB, &tunB, &bindB, 4, 16);
    const uint32_t ipA = ip(100, 64, 0, 1);
    uint8_t key[3][32];
    for (int p = 0; p < 3; p++) {
        for (int i = 0; i < 32; i++) key[p][i] = (uint8_t)(p * 50 + i);
        A.SetPeer(p, key[p], key[p], 0x500 + p, 0x600 + p, ip(100, 64, 1, 1 + p));
        B.SetPeer(p, key[p], key[p], 0x600 + p, 0x500 + p, ipA); // B plays all three peers of A
    }
    std::vector<Packet> sent;
    for (int i = 0; i < 40; i++) sent.push_back(udp(ipA, ip(100, 64, 1, 1 + i % 3), 1000 + i, 53));
    for (const Packet &p : sent) tunA.pending.push_back(p);
    const uint64_t before = ctxA.LaunchCount();
    CHECK(A.PumpOutbound() == 40 && tunA.pending.empty(), "one pump takes all ten reads");
    CHECK(ctxA.LaunchCount() - before <= 3, "and seals them with one submit");
    CHECK(a2b.size() == 40, "forty datagrams on the wire");
    // per peer, the counters follow the order the packets had in the TUN
    bool ordered = true;
    uint64_t next[3] = {0, 0, 0};
    for (const Packet &m : a2b) {
        uint32_t idx;
        uint64_t c;
        memcpy(&idx, m.data() + 4, 4);
        memcpy(&c, m.data() + 8, 8);
        ordered = ordered && idx >= 0x500 && idx < 0x503 && c == next[idx - 0x500]++;
    }
    CHECK(ordered && next[0] == 14 && next[1] == 13 && next[2] == 13, "consecutive counters per peer");
    CHECK(B.PumpInbound() == 40 && a2b.empty(), "one pump opens all of them");
    // Send groups by peer, so B sees peer 0's packets first, then peer 1's, then peer 2's
    std::vector<Packet> want;
    for (int p = 0; p < 3; p++)
        for (int i = p; i < 40; i += 3) want.push_back(sent[i]);
    CHECK(tunB.written == want, "every plaintext arrives, in send order per peer");
}

// Two dispatchers (each with two contexts on this GPU) joined back to back: packets for twelve peers sealed by one
// come out of the other in order per peer, the nonces run per peer across the GPUs, and a second delivery of the
// same messages is refused by the replay window of the GPU each peer lives on.
static void TestDispatcherRoundTrip(Context &) {
    const uint32_t n_peers = 12;
    Dispatcher A({0, 0}, n_peers, 64, 1420, 1u << 10), B({0, 0}, n_peers, 64, 1420, 1u << 10);
    std::vector<uint64_t> load(n_peers, 1);
    load[3] = 500;
    load[4] = 400;
    A.Place(load);
    uint32_t g3 = 0, g4 = 0;
    bnk_mgpu_locate(A.raw(), 3, &g3, nullptr);
    bnk_mgpu_locate(A.raw(), 4, &g4, nullptr);
    CHECK(g3 != g4, "the two heaviest peers are placed on different GPUs");
    for (uint32_t p = 0; p < n_peers; p++) {
        uint8_t key[32];
        for (int i = 0; i < 32; i++) key[i] = (uint8_t)(p * 7 + i);
        A.SetPeer(p, key, key, 0x900 + p, 0x800 + p, ip(100, 64, 2, 1 + p));
        B.SetPeer(p, key, key, 0x800 + p, 0x900 + p, ip(100, 64, 0, 1));
    }
    std::vector<Packet> sent;
    std::vector<uint32_t> peers;
    for (int i = 0; i < 200; i++) {
        peers.push_back(i % 3 == 0 ? 3 : (uint32_t)(i % n_peers));
        sent.push_back(udp(ip(100, 64, 0, 1), ip(100, 64, 2, 1 + peers.back()), 2000 + i, 53));
    }
    Dispatcher::Result sealed = A.Seal(sent, peers);
    bool ok = true;
    std::vector<uint64_t> next(n_peers, 0);
    for (size_t i = 0; i < sent.size(); i++) ok = ok && sealed.status[i] == BNK_PKT_OK && sealed.counter[i] == next[peers[i]]++;
    CHECK(ok, "consecutive nonces per peer in batch order, whichever GPU holds the peer");
    Dispatcher::Result opened = B.Open(sealed.out, BNK_F_REPLAY | BNK_F_INNER_CHECK);
    ok = true;
    for (size_t i = 0; i < sent.size(); i++) ok = ok && opened.status[i] == BNK_PKT_OK && opened.out[i] == sent[i] && opened.peer[i] == peers[i];
    CHECK(ok, "every plaintext comes back, attributed to its peer");
    Dispatcher::Result again = B.Open(sealed.out, BNK_F_REPLAY | BNK_F_INNER_CHECK);
    ok = true;
    for (size_t i = 0; i < sent.size(); i++) ok = ok && again.status[i] == BNK_PKT_REPLAY && again.out[i].empty();
    CHECK(ok, "the same messages again are replays on every GPU");
}

// Workers of both directions share one queue each (the reference's workers move conn.IdealBatchSize packets per
// call, bind.go:97): four threads, copying calls and span calls mixed; nonces per peer in call order, every
// plaintext back, a second delivery refused.
static void TestWorkersShareQueues(Context &) {
    Context ctx(0, 64, 1420, 0);
    for (uint32_t p = 0; p < 64; p++) {
        uint8_t key[32];
        for (int i = 0; i < 32; i++) key[i] = (uint8_t)(p * 5 + i);
        ctx.Check(bnk_keypair_set(ctx.raw(), p, key, key, 0x700 + p));
    }
    Queue sealq(ctx, false, 0, 512, 1420, 2), openq(ctx, true, BNK_F_REPLAY, 512, 1420, 2);
    std::atomic<int> bad{0};
    auto worker = [&](int t) {
        std::vector<uint64_t> next(64, 0);
        for (int round = 0; round < 8; round++) {
            const uint32_t n = 20 + 13 * (uint32_t)t + (uint32_t)round;
            std::vector<Packet> plain(n);
            std::vector<uint32_t> slots(n);
            for (uint32_t i = 0; i < n; i++) {
                slots[i] = (uint32_t)t * 16 + (i * 7 + (uint32_t)round) % 16; // sixteen peers per worker
                plain[i] = udp(ip(100, 64, 0, 1), ip(100, 64, 2, 1 + slots[i]), 3000 + i, 53);
                plain[i].resize(28 + (i * 97) % 1300, (uint8_t)i);
            }
            std::vector<Packet> msgs(n);
            if (t % 2 == 0) { // copying calls
                Queue::Result r = sealq.Run(plain, slots);
                for (uint32_t i = 0; i < n; i++) {
                    if (r.status[i] != BNK_PKT_OK || r.counter[i] != next[slots[i]]++) bad++;
                    msgs[i] = r.out[i];
                }
                Queue::Result o = openq.Run(msgs, slots);
                for (uint32_t i = 0; i < n; i++)
                    if (o.status[i] != BNK_PKT_OK || o.out[i].size() < plain[i].size() ||
                        !std::equal(plain[i].begin(), plain[i].end(), o.out[i].begin()))
                        bad++;
                Queue::Result again = openq.Run(msgs, slots);
                for (uint32_t i = 0; i < n; i++)
                    if (again.status[i] != BNK_PKT_REPLAY || !again.out[i].empty()) bad++;
            } else { // spans: written and read in the pinned ring
                Queue::Span sp = sealq.Reserve(n);
                for (uint32_t i = 0; i < n; i++) {
                    std::copy(plain[i].begin(), plain[i].end(), sp.packet(i) + 16);
                    sp.s.len[i] = (uint32_t)plain[i].size();
                    sp.s.slot[i] = slots[i];
                }
                sealq.Commit(sp);
                sealq.Wait(sp);
                for (uint32_t i = 0; i < n; i++) {
                    if (sp.s.status[i] != BNK_PKT_OK || sp.s.counter[i] != next[slots[i]]++) bad++;
                    msgs[i].assign(sp.packet(i), sp.packet(i) + sp.s.out_len[i]);
                }
                sealq.Release(sp);
                for (int pass = 0; pass < 2; pass++) {
                    Queue::Span op = openq.Reserve(n);
                    for (uint32_t i = 0; i < n; i++) {
                        std::copy(msgs[i].begin(), msgs[i].end(), op.packet(i));
                        op.s.len[i] = (uint32_t)msgs[i].size();
                        op.s.slot[i] = slots[i];
                    }
                    openq.Commit(op);
                    openq.Wait(op);
                    for (uint32_t i = 0; i < n; i++) {
                        if (pass == 0) {
                            if (op.s.status[i] != BNK_PKT_OK || !std::equal(plain[i].begin(), plain[i].end(), op.packet(i) + 16)) bad++;
                        } else if (op.s.status[i] != BNK_PKT_REPLAY) {
                            bad++;
                        }
                    }
                    openq.Release(op);
                }
            }
        }
    };
    std::vector<std::thread> pool;
    for (int t = 0; t < 4; t++) pool.emplace_back(worker, t);
    for (auto &th : pool) th.join();
    CHECK(bad.load() == 0, "four workers through two shared queues: nonces in call order, plaintext back, replays refused");
}

int main() {
    try {
        Context ctx(0, /*max_keypairs=*/16, /*mtu=*/1420, /*flow_capacity=*/1u << 12);
#define RUN(t)      \
    g_test = #t;    \
    t(ctx);         \
    printf("ran %s\n", #t);
        RUN(TestAllowAllModePassesEverything)
        RUN(TestRuleAllowsMatchingInbound)
        RUN(TestDefaultDenyDropsNonMatching)
        RUN(TestReturnTrafficAllowedViaFlowTable)
        RUN(TestTCPReturnFlowAllowed)
        RUN(TestICMPEchoReplyViaFlow)
        RUN(TestICMPRuleAllowsInboundPing)
        RUN(TestMalformedAndNonIPv4Dropped)
        RUN(TestSetAllowAllDisablesEnforcement)
        RUN(TestCompiledRuleMatch)
        RUN(TestICMPRuleIgnoresPorts)
        RUN(TestWrapTUNDropsDeniedInboundWrites)
        RUN(TestWrapTUNReadRecordsOutboundFlows)
        RUN(TestTwoDevicesRoundTrip)
        RUN(TestCoalescedPumps)
        RUN(TestDispatcherRoundTrip)
        RUN(TestWorkersShareQueues)
    } catch (const Error &e) {
        printf("FAIL %s: exception %d %s\n", g_test, e.code, e.what());
        return 2;
    }
    printf("%d checks, %d failed\n", g_checks, g_failed);
    return g_failed ? 1 : 0;
}
