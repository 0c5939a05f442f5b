/* What cgo hands to the C compiler for the shim shown in INTEGRATION.md: the same calls with the same argument
 * types, in plain C (cgo compiles the header as C, not C++).  Compiled with -std=c11 -Wall -Wextra -Werror and
 * linked against libbnkgpu.so by tests/test_abi.py; never run there (the calls need a GPU).  The function names
 * follow the Go methods they stand for. */
#include <stddef.h>
#include <string.h>

#include "bnk_gpu.h"

struct device {
    bnk_ctx *ctx;
    bnk_batch *batch;
    bnk_batch_view view;
    uint32_t slot; /* bytes per packet slot */
};

int gpudev_new(struct device *d, int gpu, uint32_t max_peers, uint32_t mtu) {
    bnk_cfg cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.struct_size = (uint32_t)sizeof cfg;
    cfg.device_id = gpu;
    cfg.max_keypairs = max_peers;
    cfg.replay_ring_blocks = 128;
    cfg.mtu = mtu;
    cfg.flow_capacity = 1u << 20;
    d->slot = (16u + ((mtu + 15u) & ~15u) + 16u + 15u) & ~15u;
    int rc = bnk_ctx_create(&cfg, &d->ctx);
    if (rc != BNK_SUCCESS) return rc;
    rc = bnk_batch_create(d->ctx, 128, (uint64_t)128 * d->slot, &d->batch);
    if (rc != BNK_SUCCESS) return rc;
    return bnk_batch_view_get(d->batch, &d->view);
}

int gpudev_set_peer(struct device *d, uint32_t slot, const uint8_t send_key[32], const uint8_t recv_key[32],
                    uint32_t remote_index, uint32_t local_index, uint32_t allowed_ip) {
    int rc = bnk_keypair_set(d->ctx, slot, send_key, recv_key, remote_index);
    if (rc != BNK_SUCCESS) return rc;
    rc = bnk_keypair_set_allowed_ip(d->ctx, slot, allowed_ip);
    if (rc != BNK_SUCCESS) return rc;
    return bnk_index_set(d->ctx, local_index, slot);
}

int gpudev_remove_peer(struct device *d, uint32_t slot) { return bnk_keypair_clear(d->ctx, slot); }

int gpudev_set_rules(struct device *d, int enforce, const bnk_acl_tuple *tuples, size_t n) {
    return bnk_acl_set(d->ctx, enforce, tuples, n);
}

/* SealBatch: packet i at bufs[i] + offset, sizes[i] bytes; message i comes back at bufs[i] + offset - 16 */
int gpudev_seal_batch(struct device *d, uint8_t *const *bufs, const int *sizes, const uint32_t *peer_slot, int n,
                      int offset, int64_t now_unix_ns) {
    for (int i = 0; i < n; i++) {
        d->view.off[i] = (uint32_t)i * d->slot;
        d->view.len[i] = (uint32_t)sizes[i];
        d->view.slot[i] = peer_slot[i];
        memcpy(d->view.ring + (size_t)i * d->slot + 16, bufs[i] + offset, (size_t)sizes[i]);
    }
    int rc = bnk_seal_submit(d->batch, (uint32_t)n, BNK_F_NOTE_OUTBOUND | BNK_F_ASSIGN_COUNTERS, now_unix_ns);
    if (rc != BNK_SUCCESS) return rc;
    rc = bnk_wait(d->batch, 5000000000ull);
    if (rc != BNK_SUCCESS) return rc;
    for (int i = 0; i < n; i++)
        if (d->view.status[i] == BNK_PKT_OK)
            memcpy(bufs[i] + offset - 16, d->view.ring + (size_t)i * d->slot, d->view.out_len[i]);
    return BNK_SUCCESS;
}

/* OpenBatch: message i = packets[i][:sizes[i]]; plaintext of accepted packets to bufs[i] + offset */
int gpudev_open_batch(struct device *d, const uint8_t *const *packets, const int *sizes, uint8_t *const *bufs, int n,
                      int offset, int64_t now_unix_ns) {
    for (int i = 0; i < n; i++) {
        d->view.off[i] = (uint32_t)i * d->slot;
        d->view.len[i] = (uint32_t)sizes[i];
        memcpy(d->view.ring + (size_t)i * d->slot, packets[i], (size_t)sizes[i]);
    }
    int rc = bnk_open_submit(d->batch, (uint32_t)n,
                             BNK_F_DEMUX_INDEX | BNK_F_REPLAY | BNK_F_INNER_CHECK | BNK_F_CHECK_INBOUND, now_unix_ns);
    if (rc != BNK_SUCCESS) return rc;
    rc = bnk_wait(d->batch, 5000000000ull);
    if (rc != BNK_SUCCESS) return rc;
    for (int i = 0; i < n; i++)
        if (d->view.status[i] == BNK_PKT_OK)
            memcpy(bufs[i] + offset, d->view.ring + (size_t)i * d->slot + 16, d->view.out_len[i]);
    return BNK_SUCCESS;
}

/* the workers' shared queue: reserve, fill in place, commit, wait, read in place, release */
int gpudev_queue_round(bnk_queue *q, uint32_t n, int64_t now_unix_ns) {
    bnk_ticket ticket;
    bnk_queue_span sp;
    int rc;
    while ((rc = bnk_queue_reserve(q, n, now_unix_ns, &ticket, &sp)) == BNK_EBUSY) bnk_queue_wait_room(q, 1000000ull);
    if (rc != BNK_SUCCESS) return rc;
    for (uint32_t i = 0; i < n; i++) {
        sp.len[i] = 0;
        sp.slot[i] = 0xffffffffu;
        sp.data[(size_t)i * sp.stride + 16] = 0;
    }
    rc = bnk_queue_commit(q, ticket);
    if (rc != BNK_SUCCESS && rc != BNK_EINVAL) return rc;
    rc = bnk_queue_wait_span(q, ticket, &sp);
    if (rc != BNK_SUCCESS) return rc;
    uint32_t ok = 0;
    for (uint32_t i = 0; i < n; i++) ok += sp.status[i] == BNK_PKT_OK && sp.out_len[i] > 0 && sp.counter[i] < UINT64_MAX;
    (void)ok;
    return bnk_queue_release(q, ticket);
}

int gpudev_new_queue(struct device *d, int open_side, uint32_t flags, bnk_queue **out) {
    bnk_queue_cfg qc;
    memset(&qc, 0, sizeof qc);
    qc.struct_size = (uint32_t)sizeof qc;
    qc.max_pkts = 1024;
    qc.max_packet = 1420;
    qc.depth = 3;
    qc.open_side = (uint32_t)open_side;
    qc.flags = flags;
    return bnk_queue_create(d->ctx, &qc, out);
}

void gpudev_close(struct device *d) {
    bnk_batch_destroy(d->batch);
    bnk_ctx_destroy(d->ctx);
}

const char *gpudev_error(struct device *d) { return bnk_last_error_string(d ? d->ctx : NULL); }
