// Several host threads drive one context, each through batches of its own: the calling pattern of the
// reference, where wireguard-go runs one encryption/decryption worker per core and Bind.Send is entered from
// per-peer goroutines (internal/magicsock/bind.go:327-328).  Every thread seals upstream-sized batches
// (128 packets) for its own peers with counters handed out by the library, opens them again with the replay
// window on, and checks that the plaintext came back and that a second open of the same messages is refused.
// Prints the aggregate rate; exits non-zero on any mismatch.
//
//   mt_stress [threads] [rounds] [packets per batch] [payload bytes] [batches per thread]
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
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
    auto worker = [&](int t) {
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
    bnk_ctx_destroy(ctx);
    const double gbps = 2.0 * (double)packets.load() * size * 8 / secs / 1e9; // sealed + opened payload bits
    std::printf("%s threads=%d lanes=%d packets_per_batch=%u payload=%u rounds=%d seconds=%.3f mpps=%.3f gbps=%.2f failures=%d\n",
                failures.load() ? "FAILED" : "OK", threads, lanes, n, size, rounds, secs,
                2.0 * packets.load() / secs / 1e6, gbps, failures.load());
    return failures.load() ? 1 : 0;
}
