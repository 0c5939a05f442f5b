// Several host threads drive one context, each through batches of its own: the calling pattern of the
// reference, where wireguard-go runs one encryption/decryption worker per core and Bind.Send is entered from
// per-peer goroutines (internal/magicsock/bind.go:327-328).  Every thread seals upstream-sized batches
// (128 packets) for its own peers with counters handed out by the library, opens them again with the replay
// window on, and checks that the plaintext came back and that a second open of the same messages is refused.
// Prints the aggregate rate; exits non-zero on any mismatch.
//
// With a sixth argument of 1 the threads do the same through two shared submit queues (bnk_queue, one per
// direction) instead of batches of their own: their 128-packet calls are packed into GPU batches by the library.
//
//   mt_stress [threads] [rounds] [packets per batch] [payload bytes] [batches per thread] [0 = own batches | 1 = queue | 2 = queue, spans]
//             [queue: packets per GPU batch] [queue: GPU batches in flight] [queue: min_fill]
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "../../../include/bnk_gpu.h"

static std::atomic<int> failures{0};
#define CHECK(cond, ...)                                                                                              \
    do {                                                                                                              \
        if (!(cond)) {                                                                                                \
            if (failures.fetch_add(1) < 10) {                                                                         \
                std::fprintf(stderr, "FAIL %s:%d: ", __FILE__, __LINE__);                                             \
                std::fprintf(stderr, __VA_ARGS__);                                                                    \
                std::fprintf(stderr, "\n");                                                                           \
            }                                                                                                         \
        }                                                                                                             \
    } while (0)

static uint64_t mix(uint64_t &s) {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct Lane { // one batch and what was put into it
    bnk_batch *b = nullptr;
    bnk_batch_view v{};
    std::vector<uint8_t> plain;
};

int main(int argc, char **argv) {
    const int threads = argc > 1 ? std::atoi(argv[1]) : 8;
    const int rounds = argc > 2 ? std::atoi(argv[2]) : 100;
    const uint32_t n = argc > 3 ? (uint32_t)std::atoi(argv[3]) : 128;
    const uint32_t size = argc > 4 ? (uint32_t)std::atoi(argv[4]) : 1420;
    const int lanes = argc > 5 ? std::atoi(argv[5]) : 2;
    const uint32_t peers_per_lane = 8, stride = (16 + ((size + 15) & ~15u) + 16 + 15) & ~15u;
    const uint32_t max_peers = (uint32_t)threads * lanes * peers_per_lane;

    bnk_cfg cfg{};
    cfg.struct_size = sizeof(cfg);
    cfg.device_id = 0;
    cfg.max_keypairs = max_peers;
    cfg.replay_ring_blocks = 128;
    cfg.mtu = 1420;
    cfg.flow_capacity = 0;
    bnk_ctx *ctx = nullptr;
    if (bnk_ctx_create(&cfg, &ctx) != BNK_SUCCESS) {
        std::fprintf(stderr, "no context: %s\n", bnk_last_error_string(nullptr));
        return 2;
    }
    uint64_t ks = 42;
    for (uint32_t p = 0; p < max_peers; p++) {
        uint8_t key[32];
        for (int i = 0; i < 32; i += 8) {
            const uint64_t w = mix(ks);
            std::memcpy(key + i, &w, 8);
        }
        if (bnk_keypair_set(ctx, p, key, key, 0x100 + p) != BNK_SUCCESS) return 2;
    }

    std::atomic<int> ready{0};
    std::atomic<bool> go{false};
    std::atomic<uint64_t> packets{0};
    const int queue_mode = argc > 6 ? std::atoi(argv[6]) : 0; // 1: copying calls, 2: spans (no host copies inside the library)
    const bool use_queue = queue_mode == 1 || queue_mode == 2;
    const bool use_spans = queue_mode == 2;
    bnk_queue *sealq = nullptr, *openq = nullptr;
    if (use_queue) {
        bnk_queue_cfg qc{};
        qc.struct_size = sizeof qc;
        // GPU batches of up to 1024 packets stay on the library's short path (one grouping launch, one seal or open
        // launch, one copy each way); three of them in flight keep the copy engines and the SMs busy together
        qc.max_pkts = argc > 7 ? (uint32_t)std::atoi(argv[7]) : 1024;
        qc.max_packet = size ? size : 16;
        qc.depth = argc > 8 ? (uint32_t)std::atoi(argv[8]) : 3;
        qc.min_fill = argc > 9 ? (uint32_t)std::atoi(argv[9]) : 0;
        qc.open_side = 0;
        qc.flags = 0;
        if (bnk_queue_create(ctx, &qc, &sealq) != BNK_SUCCESS) return 2;
        qc.open_side = 1;
        qc.flags = BNK_F_REPLAY;
        if (bnk_queue_create(ctx, &qc, &openq) != BNK_SUCCESS) return 2;
    }
    // The same work through the queues.  A lane is one caller batch in flight: its plaintext, the sealed messages
    // that came back, the opened packets; `lanes` tickets per thread are out at any time.
    auto queue_worker = [&](int t) {
        struct QLane {
            std::vector<uint8_t> plain, sealed, opened;
            std::vector<const uint8_t *> in;
            std::vector<uint8_t *> out;
            std::vector<uint32_t> len, slot, out_len;
            std::vector<uint64_t> counter;
            std::vector<uint8_t> status;
            bnk_ticket ticket = 0;
        };
        const uint32_t msg_room = stride;
        std::vector<QLane> ls(lanes);
        uint64_t rs = 1000 + t;
        for (QLane &L : ls) {
            L.plain.resize((size_t)n * (size ? size : 1));
            for (auto &x : L.plain) x = (uint8_t)mix(rs);
            L.sealed.resize((size_t)n * msg_room);
            L.opened.resize((size_t)n * msg_room);
            L.in.resize(n); L.out.resize(n); L.len.resize(n); L.slot.resize(n); L.out_len.resize(n);
            L.counter.resize(n); L.status.resize(n);
        }
        std::vector<uint64_t> next_counter(max_peers, 0);
        // A submit that finds every GPU batch taken returns BNK_EBUSY; the caller then collects its oldest ticket
        // (which may be what keeps a batch from being reused) and tries again.
        int r = 0;
        auto collect_sealed = [&](QLane &L) {
            if (use_spans) { // results are read where they lie; the copy below stands for Bind.Send + the peer's receive
                bnk_queue_span sp{};
                CHECK(bnk_queue_wait_span(sealq, L.ticket, &sp) == BNK_SUCCESS, "queue_wait_span after seal");
                for (uint32_t i = 0; i < n; i++) {
                    L.status[i] = sp.status[i];
                    L.counter[i] = sp.counter[i];
                    L.out_len[i] = sp.out_len[i];
                    std::memcpy(L.sealed.data() + (size_t)i * msg_room, sp.data + (size_t)i * sp.stride, sp.out_len[i]);
                }
                CHECK(bnk_queue_release(sealq, L.ticket) == BNK_SUCCESS, "queue_release after seal");
            } else
            CHECK(bnk_queue_wait(sealq, L.ticket, L.out.data(), L.out_len.data(), L.counter.data(), nullptr, L.status.data()) == BNK_SUCCESS,
                  "queue_wait after seal");
            for (uint32_t i = 0; i < n; i++) {
                CHECK(L.status[i] == BNK_PKT_OK, "seal status %u", L.status[i]);
                CHECK(L.counter[i] == next_counter[L.slot[i]]++, "thread %d round %d packet %u: nonce out of order", t, r, i);
                L.in[i] = L.sealed.data() + (size_t)i * msg_room;
                L.len[i] = L.out_len[i];
                L.out[i] = L.opened.data() + (size_t)i * msg_room;
            }
        };
        auto collect_opened = [&](QLane &L) {
            if (use_spans) { // compared in place, as tun.Device.Write would read it in place
                bnk_queue_span sp{};
                CHECK(bnk_queue_wait_span(openq, L.ticket, &sp) == BNK_SUCCESS, "queue_wait_span after open");
                for (uint32_t i = 0; i < n; i++) {
                    CHECK(sp.status[i] == (size ? BNK_PKT_OK : BNK_PKT_KEEPALIVE), "thread %d round %d packet %u: open status %u", t, r, i, sp.status[i]);
                    CHECK(std::memcmp(sp.data + (size_t)i * sp.stride + 16, L.plain.data() + (size_t)i * size, size) == 0,
                          "thread %d round %d packet %u: plaintext differs", t, r, i);
                }
                CHECK(bnk_queue_release(openq, L.ticket) == BNK_SUCCESS, "queue_release after open");
                return;
            }
            CHECK(bnk_queue_wait(openq, L.ticket, L.out.data(), L.out_len.data(), nullptr, nullptr, L.status.data()) == BNK_SUCCESS,
                  "queue_wait after open");
            for (uint32_t i = 0; i < n; i++) {
                CHECK(L.status[i] == (size ? BNK_PKT_OK : BNK_PKT_KEEPALIVE), "thread %d round %d packet %u: open status %u", t, r, i, L.status[i]);
                CHECK(std::memcmp(L.opened.data() + (size_t)i * msg_room, L.plain.data() + (size_t)i * size, size) == 0,
                      "thread %d round %d packet %u: plaintext differs", t, r, i);
            }
        };
        // hand lane L's packets (L.in / L.len / L.slot) to q: copying call, or reserve + write in place + commit
        auto hand_in = [&](bnk_queue *q, QLane &L, bool seal_side) -> int {
            if (!use_spans) return bnk_queue_submit(q, L.in.data(), L.len.data(), L.slot.data(), n, 0, &L.ticket);
            bnk_queue_span sp{};
            const int rc = bnk_queue_reserve(q, n, 0, &L.ticket, &sp);
            if (rc != BNK_SUCCESS) return rc;
            for (uint32_t i = 0; i < n; i++) { // stands for tun.Device.Read / the receive call landing in the ring
                sp.len[i] = L.len[i];
                sp.slot[i] = L.slot[i];
                if (L.len[i]) std::memcpy(sp.data + (size_t)i * sp.stride + (seal_side ? 16 : 0), L.in[i], L.len[i]);
            }
            return bnk_queue_commit(q, L.ticket);
        };
        // one phase: submit every lane, collecting the oldest outstanding one whenever the queue is full
        auto phase = [&](bnk_queue *q, const std::function<void(QLane &)> &prepare, const std::function<void(QLane &)> &collect) {
            int collected = 0;
            for (int l = 0; l < lanes; l++) {
                prepare(ls[l]);
                for (;;) {
                    const int rc = hand_in(q, ls[l], q == sealq);
                    if (rc == BNK_SUCCESS) break;
                    CHECK(rc == BNK_EBUSY, "queue_submit: %d %s", rc, bnk_last_error_string(ctx));
                    if (rc != BNK_EBUSY) return;
                    if (collected < l) collect(ls[collected++]);
                    else bnk_queue_wait_room(q, 1000000); // nothing of this thread is outstanding: others are ahead
                }
            }
            while (collected < lanes) collect(ls[collected++]);
        };
        const int warm = rounds / 10 + 1;
        int lane_no = 0;
        for (r = -warm; r < rounds; r++) {
            if (r == 0) {
                ready.fetch_add(1);
                while (!go.load()) std::this_thread::yield();
            }
            lane_no = 0;
            phase(sealq, [&](QLane &L) {
                const uint32_t first_peer = (uint32_t)(t * lanes + lane_no++) * peers_per_lane;
                for (uint32_t i = 0; i < n; i++) {
                    L.in[i] = L.plain.data() + (size_t)i * size;
                    L.len[i] = size;
                    L.slot[i] = first_peer + (uint32_t)(mix(rs) % peers_per_lane);
                    L.out[i] = L.sealed.data() + (size_t)i * msg_room;
                }
            }, collect_sealed);
            phase(openq, [](QLane &) {}, collect_opened);
            if (r >= 0) packets.fetch_add((uint64_t)n * lanes);
        }
        // the last sealed messages once more: all replays
        QLane &L = ls[0];
        while (hand_in(openq, L, false) == BNK_EBUSY) bnk_queue_wait_room(openq, 1000000);
        if (use_spans) {
            bnk_queue_span sp{};
            CHECK(bnk_queue_wait_span(openq, L.ticket, &sp) == BNK_SUCCESS, "queue_wait_span");
            for (uint32_t i = 0; i < n; i++) L.status[i] = sp.status[i];
            CHECK(bnk_queue_release(openq, L.ticket) == BNK_SUCCESS, "queue_release");
        } else
        CHECK(bnk_queue_wait(openq, L.ticket, L.out.data(), L.out_len.data(), nullptr, nullptr, L.status.data()) == BNK_SUCCESS, "queue_wait");
        for (uint32_t i = 0; i < n; i++) CHECK(L.status[i] == BNK_PKT_REPLAY, "thread %d: replayed packet %u has status %u", t, i, L.status[i]);
    };
    auto worker = [&](int t) {
        if (use_queue) {
            queue_worker(t);
            return;
        }
        std::vector<Lane> ls(lanes);
        uint64_t rs = 1000 + t;
        for (int l = 0; l < lanes; l++) {
            Lane &L = ls[l];
            CHECK(bnk_batch_create(ctx, n, (uint64_t)n * stride + 64, &L.b) == BNK_SUCCESS, "batch_create");
            if (!L.b) {
                ready.fetch_add(1);
                return;
            }
            bnk_batch_view_get(L.b, &L.v);
            L.plain.resize((size_t)n * size);
            for (auto &x : L.plain) x = (uint8_t)mix(rs);
        }
        const int warm = rounds / 10 + 1; // untimed: clocks come up, pages and caches get touched
        for (int r = -warm; r < rounds; r++) {
            if (r == 0) {
                ready.fetch_add(1);
                while (!go.load()) std::this_thread::yield();
            }
            // seal on every lane, then collect: two batches of the thread are in flight together
            for (int l = 0; l < lanes; l++) {
                Lane &L = ls[l];
                const uint32_t first_peer = (uint32_t)(t * lanes + l) * peers_per_lane;
                for (uint32_t i = 0; i < n; i++) {
                    L.v.off[i] = i * stride;
                    L.v.len[i] = size;
                    L.v.slot[i] = first_peer + (uint32_t)(mix(rs) % peers_per_lane);
                    std::memcpy(L.v.ring + (size_t)i * stride + 16, L.plain.data() + (size_t)i * size, size);
                }
                CHECK(bnk_seal_submit(L.b, n, BNK_F_ASSIGN_COUNTERS, 0) == BNK_SUCCESS, "seal_submit: %s", bnk_last_error_string(ctx));
            }
            for (int l = 0; l < lanes; l++) {
                Lane &L = ls[l];
                CHECK(bnk_wait(L.b, 10ull * 1000 * 1000 * 1000) == BNK_SUCCESS, "wait after seal");
                for (uint32_t i = 0; i < n; i++) {
                    CHECK(L.v.status[i] == BNK_PKT_OK, "seal status %u", L.v.status[i]);
                    L.v.len[i] = L.v.out_len[i];
                }
                CHECK(bnk_open_submit(L.b, n, BNK_F_REPLAY, 0) == BNK_SUCCESS, "open_submit: %s", bnk_last_error_string(ctx));
            }
            for (int l = 0; l < lanes; l++) {
                Lane &L = ls[l];
                CHECK(bnk_wait(L.b, 10ull * 1000 * 1000 * 1000) == BNK_SUCCESS, "wait after open");
                for (uint32_t i = 0; i < n; i++) {
                    const uint8_t want = size ? BNK_PKT_OK : BNK_PKT_KEEPALIVE;
                    CHECK(L.v.status[i] == want, "thread %d round %d packet %u: open status %u", t, r, i, L.v.status[i]);
                    CHECK(std::memcmp(L.v.ring + (size_t)i * stride + 16, L.plain.data() + (size_t)i * size, size) == 0,
                          "thread %d round %d packet %u: plaintext differs", t, r, i);
                }
            }
            if (r >= 0) packets.fetch_add((uint64_t)n * lanes);
        }
        // the same counters again must all be refused: seal once more, open twice
        Lane &L = ls[0];
        for (uint32_t i = 0; i < n; i++) {
            L.v.len[i] = size;
            std::memcpy(L.v.ring + (size_t)i * stride + 16, L.plain.data() + (size_t)i * size, size);
        }
        CHECK(bnk_seal_submit(L.b, n, BNK_F_ASSIGN_COUNTERS, 0) == BNK_SUCCESS, "seal_submit");
        CHECK(bnk_wait(L.b, 10ull * 1000 * 1000 * 1000) == BNK_SUCCESS, "wait");
        std::vector<uint8_t> sealed(L.v.ring, L.v.ring + (size_t)n * stride);
        std::vector<uint32_t> message_len(L.v.out_len, L.v.out_len + n);
        for (int pass = 0; pass < 2; pass++) {
            std::memcpy(L.v.ring, sealed.data(), sealed.size());
            for (uint32_t i = 0; i < n; i++) L.v.len[i] = message_len[i];
            CHECK(bnk_open_submit(L.b, n, BNK_F_REPLAY, 0) == BNK_SUCCESS, "open_submit");
            CHECK(bnk_wait(L.b, 10ull * 1000 * 1000 * 1000) == BNK_SUCCESS, "wait");
            for (uint32_t i = 0; i < n; i++)
                CHECK(L.v.status[i] == (pass == 0 ? (size ? BNK_PKT_OK : BNK_PKT_KEEPALIVE) : BNK_PKT_REPLAY),
                      "thread %d pass %d packet %u: status %u", t, pass, i, L.v.status[i]);
        }
        for (auto &x : ls) bnk_batch_destroy(x.b);
    };

    std::vector<std::thread> pool;
    for (int t = 0; t < threads; t++) pool.emplace_back(worker, t);
    while (ready.load() < threads) std::this_thread::yield();
    const auto t0 = std::chrono::steady_clock::now();
    go.store(true);
    for (auto &th : pool) th.join();
    const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (use_queue) {
        uint64_t gb = 0, pk = 0, cb = 0;
        bnk_queue_stats_get(sealq, &gb, &pk, &cb);
        std::printf("seal queue: %llu caller batches in %llu gpu batches (%.1f packets per gpu batch)\n", (unsigned long long)cb,
                    (unsigned long long)gb, gb ? (double)pk / (double)gb : 0.0);
        bnk_queue_destroy(sealq);
        bnk_queue_destroy(openq);
    }
    bnk_ctx_destroy(ctx);
    const double gbps = 2.0 * (double)packets.load() * size * 8 / secs / 1e9; // sealed + opened payload bits
    std::printf("%s mode=%s threads=%d lanes=%d packets_per_batch=%u payload=%u rounds=%d seconds=%.3f mpps=%.3f gbps=%.2f failures=%d\n",
                failures.load() ? "FAILED" : "OK", use_spans ? "queue-spans" : use_queue ? "queue" : "batches", threads, lanes, n, size, rounds, secs,
                2.0 * packets.load() / secs / 1e6, gbps, failures.load());
    return failures.load() ? 1 : 0;
}
