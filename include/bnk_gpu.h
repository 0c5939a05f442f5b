/*
 * bnk_gpu.h -- C ABI of libbnkgpu.so, the B200 (sm_100a) implementation of the
 * bnk dataplane hot path: batched WireGuard transport-data seal/open
 * (ChaCha20-Poly1305), per-keypair send counters, the anti-replay window and
 * the ACL packet filter with reply-flow tracking.
 *
 * The reference (a Go program) has no FFI.  Each entry point below names the
 * reference interface whose per-packet work it takes over (a cgo binding for
 * them ships with the integration notes of this repository).  Paths are
 * relative to the reference tree;
 * "wireguard-go" is golang.zx2c4.com/wireguard (go.mod:10) and "x/crypto" is
 * golang.org/x/crypto (go.mod:7), both entered through device.NewDevice at
 * internal/dataplane/engine.go:51.
 *
 * Conventions
 *   - Every call returns an int: BNK_SUCCESS or a negative BNK_E* code.  No call
 *     aborts the process.  bnk_last_error_string() describes the last failure.
 *   - Per-packet outcomes are data (the status[] array), not errors.
 *   - One bnk_ctx per GPU.  A bnk_batch owns one CUDA stream; calls on one batch
 *     are single-producer, different batches may be driven from different
 *     threads.  Table updates (keypairs, ACL) must not overlap submitted work.
 *   - A submit that copies to or from the pinned ring needs the previous submit
 *     of that batch to have been waited for (BNK_EBUSY otherwise).  Submits with
 *     both BNK_F_NO_H2D and BNK_F_NO_D2H only queue kernels on the batch's stream
 *     and may be issued back to back.
 *   - Between a submit and its bnk_wait the batch's host arrays belong to the
 *     library.  Small batches (up to 256 packets and a ring extent of 384 KiB,
 *     environment BNK_HOST_DIRECT_BYTES, 0 = never) are not copied: the kernels
 *     read and write the pinned arrays in place.  The results are the same bytes.
 *   - Send counters and replay windows are per keypair and ordered: batches that
 *     are in flight at the same time must not carry packets of the same keypair
 *     slot when BNK_F_ASSIGN_COUNTERS or BNK_F_REPLAY is used (give each peer's
 *     traffic to one batch at a time, as wireguard-go gives it to one sequential
 *     worker per peer).
 *   - There is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails with BNK_ECUDA.
 */
#ifndef BNK_GPU_H
#define BNK_GPU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BNK_ABI_VERSION 1

/* ---- return codes ---- */
#define BNK_SUCCESS 0
#define BNK_EINVAL (-1)    /* bad argument */
#define BNK_ENOMEM (-2)    /* host or device allocation failed */
#define BNK_ECUDA (-3)     /* CUDA runtime error, see bnk_last_error_string */
#define BNK_ETIMEDOUT (-4) /* bnk_wait ran out of time; the batch is still in flight */
#define BNK_EBUSY (-5)     /* batch already has work in flight */
#define BNK_EFULL (-6)     /* flow table or rule table capacity exceeded */

/* ---- per-packet status ---- */
#define BNK_PKT_OK 0
#define BNK_PKT_AUTH_FAIL 1         /* tag mismatch: plaintext zeroed, packet to be dropped */
#define BNK_PKT_REPLAY 2            /* rejected by the anti-replay window */
#define BNK_PKT_FILTER_DENY 3       /* ACL filter verdict: drop */
#define BNK_PKT_MALFORMED 4         /* not a transport-data message (type != 4 or shorter than 32) */
#define BNK_PKT_KEEPALIVE 5         /* authenticated zero-length payload */
#define BNK_PKT_COUNTER_EXHAUSTED 6 /* send counter reached Reject-After-Messages */
#define BNK_PKT_BAD_DESC 7          /* descriptor out of range (offset, length or keypair slot) */
#define BNK_PKT_NO_KEYPAIR 8        /* the keypair slot holds no keys (never set, or cleared), or with
                                       BNK_F_DEMUX_INDEX the receiver index in the header maps to no keypair */
#define BNK_PKT_BAD_INNER 9         /* BNK_F_INNER_CHECK: decrypted packet is not IPv4, lies about its length,
                                       or does not come from the peer's allowed address */

#define BNK_WG_HEADER 16u
#define BNK_WG_TAG 16u
#define BNK_REJECT_AFTER_MESSAGES 0xFFFFFFFFFFFFDFFFull /* 2^64 - 2^13 - 1 */

/* ---- submit flags ---- */
#define BNK_F_NO_H2D (1u << 0)          /* inputs are already in the batch's device mirror */
#define BNK_F_NO_D2H (1u << 1)          /* leave results on the device */
#define BNK_F_ASSIGN_COUNTERS (1u << 2) /* seal: take counters from the keypair's send counter */
#define BNK_F_NOTE_OUTBOUND (1u << 3)   /* seal: feed plaintext headers to the flow table first */
#define BNK_F_REPLAY (1u << 4)          /* open: run the anti-replay window on authenticated packets */
#define BNK_F_CHECK_INBOUND (1u << 5)   /* open: run the ACL filter on accepted packets */
#define BNK_F_SORT_BY_LENGTH (1u << 6)  /* schedule packets of similar length together (mixed sizes) */
#define BNK_F_USE_OUT_LEN (1u << 7)     /* open: message lengths are the out_len[] a seal left on the device */
#define BNK_F_DEMUX_INDEX (1u << 8)     /* open: slot[] is an output, looked up from each header's receiver index */
#define BNK_F_INNER_CHECK (1u << 9)     /* open: cut the plaintext to its IPv4 total length and check its source */
#define BNK_F_TIMED (1u << 10)          /* record the CUDA events bnk_batch_last_kernel_ms / _aead_ms read */
#define BNK_F_STATS (1u << 11)          /* count the batch's outcomes on the device for bnk_batch_stats_get */

typedef struct bnk_ctx bnk_ctx;
typedef struct bnk_batch bnk_batch;

typedef struct bnk_cfg {
    uint32_t struct_size;        /* sizeof(bnk_cfg), for ABI growth */
    int32_t device_id;           /* CUDA device ordinal */
    uint32_t max_keypairs;       /* keypair slots (one per peer direction pair) */
    uint32_t replay_ring_blocks; /* 64-bit blocks per replay ring: power of two, 2..1024 (32 or 128 upstream) */
    uint32_t mtu;                /* padding cap of the seal path; 0 = pad to 16 with no cap */
    uint32_t flow_capacity;      /* flow-table slots, power of two; 0 = no flow table */
    uint32_t max_acl_tuples;     /* capacity of the flattened rule table; 0 = no rule table */
    uint32_t reserved;
} bnk_cfg;

/* One flattened ACL allowance: acl.CompiledRule (internal/acl/acl.go:33-42) expanded to
 * the cross product of its Srcs and Ports.  addr is host-order IPv4 (a<<24|b<<16|c<<8|d). */
typedef struct bnk_acl_tuple {
    uint32_t addr;
    uint8_t prefix_len; /* 0..32 */
    uint8_t proto;      /* 6 tcp, 17 udp, 1 icmp */
    uint16_t port_first;
    uint16_t port_last; /* ignored for icmp */
    uint16_t reserved;
} bnk_acl_tuple;

/* Pinned host memory of a batch.  Packet i occupies ring[off[i] ...]:
 *   seal: 16 bytes of header room, then len[i] payload bytes, then room for padding + 16-byte tag;
 *         on completion ring[off[i]] holds header|ciphertext|tag and out_len[i] its length.
 *   open: the received message (len[i] bytes) at ring[off[i]]; on completion the plaintext is at
 *         ring[off[i]+16], out_len[i] its length, counter[i] the counter parsed from the header.
 * off[i] must be a multiple of 16 and the packet's span must lie inside the ring. */
typedef struct bnk_batch_view {
    uint8_t *ring;
    uint32_t *off;
    uint32_t *len;
    uint32_t *slot;    /* keypair slot of the packet */
    uint64_t *counter; /* seal without ASSIGN_COUNTERS: input; otherwise output */
    uint32_t *out_len;
    uint8_t *status;
    uint64_t ring_bytes;
    uint32_t max_pkts;
    uint32_t reserved;
    uint8_t *src_addr; /* [max_pkts][BNK_SRC_ADDR_STRIDE], bnk_classify_submit only: the datagram's source,
                          16 address bytes (IPv4 as ::ffff:a.b.c.d) then the port, big-endian */
} bnk_batch_view;
#define BNK_SRC_ADDR_STRIDE 20u

/* ---- library / context ---- */
int bnk_abi_version(void);
const char *bnk_strerror(int code);
/* Number of CUDA devices visible, or a negative code. */
int bnk_device_count(void);
/* Replaces the construction seam device.NewDevice(tun, bind, logger), internal/dataplane/engine.go:51. */
int bnk_ctx_create(const bnk_cfg *cfg, bnk_ctx **out);
int bnk_ctx_destroy(bnk_ctx *ctx);
const char *bnk_last_error_string(bnk_ctx *ctx);
/* Blocks until all work submitted on any batch of the context has finished. */
int bnk_ctx_synchronize(bnk_ctx *ctx);

/* ---- keypair table ----
 * Replaces the keypair state wireguard-go builds from the UAPI text the reference sends with
 * IpcSet (internal/dataplane/engine.go:292-299,334,341).  Setting a slot zeroes its send counter
 * and replay window; clearing also wipes the keys. */
int bnk_keypair_set(bnk_ctx *ctx, uint32_t slot, const uint8_t send_key[32], const uint8_t recv_key[32],
                    uint32_t remote_index);
int bnk_keypair_set_many(bnk_ctx *ctx, uint32_t first_slot, uint32_t n, const uint8_t *send_keys,
                         const uint8_t *recv_keys, const uint32_t *remote_index);
int bnk_keypair_clear(bnk_ctx *ctx, uint32_t slot);
int bnk_send_counter_get(bnk_ctx *ctx, uint32_t slot, uint64_t *counter);
int bnk_send_counter_set(bnk_ctx *ctx, uint32_t slot, uint64_t counter);
/* Receive-side demultiplexing, the type/index lookup wireguard-go's receive routine does before it
 * queues a message for decryption: local receiver index -> keypair slot.  With BNK_F_DEMUX_INDEX the open
 * path fills slot[] from the header (bytes 4..7); an unknown index yields BNK_PKT_NO_KEYPAIR. */
int bnk_index_set(bnk_ctx *ctx, uint32_t local_index, uint32_t slot);
int bnk_index_clear(bnk_ctx *ctx, uint32_t local_index);
/* The peer's tunnel address (the reference gives every peer exactly one /32, internal/dataplane/engine.go:294).
 * With BNK_F_INNER_CHECK the open path does what wireguard-go's sequential receiver does after the replay
 * check: the plaintext must be IPv4 with 20 <= total length <= decrypted length (out_len becomes the total
 * length) and its source address must be this one; otherwise BNK_PKT_BAD_INNER.  ipv4 is host order. */
int bnk_keypair_set_allowed_ip(bnk_ctx *ctx, uint32_t slot, uint32_t ipv4);
/* Replay-window state, for tests and state hand-over: ring has replay_ring_blocks words. */
int bnk_replay_export(bnk_ctx *ctx, uint32_t slot, uint64_t *last, uint64_t *ring);
int bnk_replay_import(bnk_ctx *ctx, uint32_t slot, uint64_t last, const uint64_t *ring);

/* ---- ACL filter tables ----
 * bnk_acl_set replaces Filter.SetRules / Filter.SetAllowAll (internal/filter/filter.go:46-59):
 * enforce=0 is allow-all mode, enforce=1 with n=0 is deny-all-but-flows.  The flow table is kept. */
int bnk_acl_set(bnk_ctx *ctx, int enforce, const bnk_acl_tuple *tuples, size_t n);
int bnk_flows_clear(bnk_ctx *ctx);
int bnk_flows_count(bnk_ctx *ctx, uint64_t *live);
/* The flow table's contents, for tests and for handing state over (the reference never persists it: it is rebuilt
 * by traffic).  One entry = one key of Go's map f.flows (internal/filter/filter.go:26-31) with its expiry.
 * bnk_flows_export writes up to `capacity` live entries in no particular order and always stores the number of
 * live entries in *count; bnk_flows_import adds entries (an existing key gets the new expiry), BNK_EFULL when a
 * class's region has no room.  Both wait for submitted work and must not run beside submits. */
typedef struct bnk_flow_entry {
    uint32_t remote_addr;   /* host order */
    uint16_t remote_port, local_port;
    uint8_t proto;          /* 6 tcp, 17 udp, 1 icmp */
    uint8_t reserved[7];
    int64_t expiry_unix_ns;
} bnk_flow_entry;
int bnk_flows_export(bnk_ctx *ctx, bnk_flow_entry *out, size_t capacity, size_t *count);
int bnk_flows_import(bnk_ctx *ctx, const bnk_flow_entry *entries, size_t n);
/* Occupancy of the context's hash tables, for monitoring: entries in use, entries deleted but not yet
 * reclaimed, and slots.  Deleted entries are reclaimed by the library itself (the flow table is compacted
 * between batches once a quarter of a class's slots are deleted entries, the two host-maintained tables are
 * rebuilt on update), so `dead` stays below a fraction of `slots`.  Waits for submitted work like
 * bnk_flows_count. */
typedef struct bnk_table_stats {
    uint64_t flow_live;        /* Go's len(f.flows) */
    uint32_t flow_used[3];     /* slots holding a key, per protocol class (tcp, udp, icmp) */
    uint32_t flow_dead[3];
    uint32_t flow_capacity;    /* slots per class */
    uint32_t index_live, index_dead, index_slots; /* receiver index -> keypair slot */
    uint32_t addr_live, addr_dead, addr_slots;    /* source address -> peer */
    uint32_t reserved;
} bnk_table_stats;
int bnk_table_stats_get(bnk_ctx *ctx, bnk_table_stats *out);

/* ---- batches ---- */
int bnk_batch_create(bnk_ctx *ctx, uint32_t max_pkts, uint64_t ring_bytes, bnk_batch **out);
int bnk_batch_destroy(bnk_batch *b);
int bnk_batch_view_get(bnk_batch *b, bnk_batch_view *out);

/* Replaces the per-packet work of wireguard-go's encryption worker (header, padding, x/crypto
 * chacha20poly1305 Seal, nonce from the keypair's send counter) for one tun.Device.Read batch;
 * with BNK_F_NOTE_OUTBOUND also filteredTUN.Read's NoteOutbound loop (internal/filter/filter.go:160-167). */
int bnk_seal_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns);
/* Replaces wireguard-go's decryption worker (x/crypto Open), the sequential replay-window check, and
 * with BNK_F_CHECK_INBOUND filteredTUN.Write's CheckInbound loop (internal/filter/filter.go:171-186)
 * for one conn.ReceiveFunc batch. */
int bnk_open_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns);
/* Filter-only batches.  Packet i is the IP packet of len[i] bytes at ring[off[i]+16].
 * Replaces Filter.NoteOutbound (filter.go:189-209) / Filter.CheckInbound (filter.go:121-147)
 * called once per packet with one `now` per batch; status[i] is BNK_PKT_OK or BNK_PKT_FILTER_DENY. */
int bnk_filter_note_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns);
int bnk_filter_check_submit(bnk_batch *b, uint32_t npkts, uint32_t flags, int64_t now_unix_ns);
/* Waits for the batch's submitted work.  timeout_ns = 0 polls once; UINT64_MAX waits without limit. */
int bnk_wait(bnk_batch *b, uint64_t timeout_ns);
/* Per-batch counters, the analogue of the per-bind send/receive counters the reference keeps
 * (internal/magicsock/bind.go:68-69,469-473).  A submit made with BNK_F_STATS counts the statuses of its
 * packets on the device, after its last kernel, and the totals come back with the batch's results:
 * bnk_batch_stats_get is valid after the bnk_wait that follows such a submit.
 *   by_status[s]  packets whose status[] is s (BNK_PKT_* for seal, open and filter submits;
 *                 BNK_CLASS_* for bnk_classify_submit)
 *   bytes_out     sum of out_len[] over packets with status BNK_PKT_OK (sealed message bytes, or
 *                 opened plaintext bytes) */
typedef struct bnk_batch_stats {
    uint64_t packets;
    uint64_t bytes_out;
    uint64_t by_status[16];
} bnk_batch_stats;
int bnk_batch_stats_get(bnk_batch *b, bnk_batch_stats *out);
/* Explicit transfers between the pinned ring/descriptors and the device mirror (asynchronous). */
int bnk_batch_upload(bnk_batch *b, uint32_t npkts);
int bnk_batch_download(bnk_batch *b, uint32_t npkts);

/* ---- receive classification ----
 * Replaces Bind.classify (internal/magicsock/bind.go:207-228) for one ReadBatch: disco.IsDisco
 * (internal/disco/disco.go:20,177-179: the datagram starts with "bnk\0disco\0"), then isSTUN
 * (bind.go:250-253: at least 20 bytes, top two bits zero, magic cookie 21 12 A4 42 at bytes 4..7), then
 * the byAddr lookup of the normalised source address (bind.go:263-274).  status[i] becomes one of the
 * classes below; for BNK_CLASS_WIREGUARD slot[i] is the peer id registered for the source address.
 * Addresses are 16 bytes, IPv4 in its ::ffff:a.b.c.d form (what normalize()'s Unmap makes equal). */
#define BNK_CLASS_WIREGUARD 0
#define BNK_CLASS_DISCO 10
#define BNK_CLASS_STUN 11
#define BNK_CLASS_STRANGER 12 /* unknown source: dropped by the reference */
int bnk_addr_set(bnk_ctx *ctx, const uint8_t addr[16], uint16_t port, uint32_t peer_id);
int bnk_addr_clear(bnk_ctx *ctx, const uint8_t addr[16], uint16_t port);
int bnk_classify_submit(bnk_batch *b, uint32_t npkts, uint32_t flags);

/* ---- segmentation offload (GSO) ----
 * Replaces the split wireguard-go's Linux TUN code performs on a super-packet read with a virtio-net
 * header (TCP or UDP over IPv4) before the packets reach the encryption workers: every segment gets
 * the IP and transport headers, its IPv4 total length, identification (first id + segment number) and
 * header checksum, its TCP sequence number (first + segment number * gso_size) with FIN/PSH kept only
 * on the last segment, or its UDP length, and a freshly computed transport checksum.
 * Super-packet j is ring[src_off .. src_off+src_len); its segments are packets first_pkt .. first_pkt +
 * n_pkts - 1 of the batch, whose off[], len[] (= hdr_len + segment payload) and slot[] the caller has
 * filled; each segment is written at ring[off+16], ready for bnk_seal_submit(... BNK_F_NO_H2D ...).
 * The submit copies ring, descriptors and `supers` to the device unless BNK_F_NO_H2D is given, and
 * copies nothing back.  A segment whose descriptor does not match the split (wrong len, out of range,
 * unsupported header layout) has its device-side slot[] set to an invalid keypair, so the seal that
 * follows reports BNK_PKT_BAD_DESC for it. */
typedef struct bnk_gso_super {
    uint32_t src_off;     /* 4-byte aligned */
    uint32_t src_len;
    uint32_t first_pkt;
    uint32_t n_pkts;
    uint16_t hdr_len;     /* IP + transport header bytes (virtio hdr_len) */
    uint16_t gso_size;    /* payload bytes per segment */
    uint16_t csum_start;  /* IP header bytes (virtio csum_start) */
    uint16_t csum_offset; /* 16 for TCP, 6 for UDP */
    uint8_t proto;        /* 6 tcp, 17 udp */
    uint8_t reserved[3];
} bnk_gso_super;
int bnk_gso_split_submit(bnk_batch *b, const bnk_gso_super *supers, uint32_t n_super, uint32_t n_pkts,
                         uint32_t flags);

/* ---- for callers that must not allocate ----
 * No counterpart in the reference.  A packet loop cannot call cudaMalloc or cudaFree (either one
 * stalls every stream of the device), and a caller that keeps packets in device buffers of its own,
 * such as buffers a NIC writes into directly, has no bnk_batch to lend it grouping scratch.  This
 * entry point does the send-counter stage of bnk_seal_submit(BNK_F_ASSIGN_COUNTERS) on the caller's
 * buffers and allocates nothing: its scratch is a fixed 384 KiB area inside the library image,
 * present on every GPU that loads the library, which limits a call to BNK_NOALLOC_MAX_PKTS packets
 * (more is refused with BNK_EINVAL).
 *   dev_slot[i]    (device memory, in)  keypair slot of packet i
 *   dev_counter[i] (device memory, out) the nonce handed to packet i: packets of one slot get
 *                  consecutive values in batch order and the slot's send counter moves past them,
 *                  saturating at BNK_REJECT_AFTER_MESSAGES; packets whose slot is not below
 *                  max_keypairs are left untouched
 *   stream         a cudaStream_t of ctx's device, or NULL for the default stream; the work is
 *                  queued on it and the call returns without waiting.
 * The first call on each device looks up the address of the scratch area (the device must be usable
 * at that moment); make that first call before any stream capture begins.  The scratch is shared by
 * all calls and keeps the previous call's contents; each call overwrites what it reads, so nothing
 * has to be cleared, but two calls whose work overlaps on the GPU would corrupt each other: order
 * them on one stream or with an event.  The same holds against batches in flight that hand out
 * counters for the same keypair slots. */
#define BNK_NOALLOC_MAX_PKTS 16384u
int bnk_assign_counters_noalloc(bnk_ctx *ctx, void *stream, const uint32_t *dev_slot, uint32_t npkts,
                                uint64_t *dev_counter);

/* ---- submit queue: many small caller batches, few large GPU batches ----
 * The reference moves packets in batches of conn.IdealBatchSize = 128 (internal/magicsock/bind.go:97,372-377),
 * from one goroutine per receive function and one per peer (bind.go:152,327-328).  A 128-packet submit does not
 * fill a GPU; a queue takes such batches from any number of threads, packs them into GPU batches of up to
 * max_pkts packets (a batch goes as soon as the device has a free slot, so a lone caller is not held up, and
 * grows by itself while the device is busy), keeps up to `depth` GPU batches in flight with their copies
 * overlapping each other's kernels, and hands every caller its own results.  One queue works in one direction
 * with one set of flags.  Per keypair, nonces follow the order of the bnk_queue_submit calls and replay
 * verdicts the order of arrival, across GPU batches too (their kernels are chained); the packets of one
 * keypair should come through one queue at a time.
 *   bnk_queue_submit  copies the caller's packets in (the caller's buffers are free again on return) and
 *                     returns a ticket; BNK_EBUSY when every GPU batch is taken: collect a ticket, then retry.
 *                     slot[] names the keypair of each packet (open side: may be NULL with BNK_F_DEMUX_INDEX).
 *   bnk_queue_wait    blocks until the ticket's GPU batch is done and copies the caller's results out:
 *                     sealed messages (room for len + 48 bytes each) or opened plaintexts, out_len[], status[],
 *                     and if not NULL counter[] and slot_out[].  Every ticket must be collected exactly once.
 * Seal queues always take counters from the keypairs' send counters.
 * A queue has no thread of its own: GPU batches are submitted and collected inside these calls, by whichever
 * caller comes by first.  A caller that waits watches its batch and takes those turns in between; after ~100 us
 * it gives its core away between turns (sched_yield), so callers may outnumber the cores.  Packets handed in are
 * therefore on their way at the latest when some caller of the queue submits again or waits. */
typedef struct bnk_queue bnk_queue;
typedef uint64_t bnk_ticket;
typedef struct bnk_queue_cfg {
    uint32_t struct_size; /* sizeof(bnk_queue_cfg) */
    uint32_t max_pkts;    /* packets per GPU batch, up to 32768 */
    uint32_t max_packet;  /* longest plaintext packet */
    uint32_t depth;       /* GPU batches in flight at once, 1..8 (2 or 3 keeps copies and kernels overlapped) */
    uint32_t open_side;   /* 0 = seal queue, 1 = open queue */
    uint32_t flags;       /* BNK_F_* of every submit (BNK_F_NOTE_OUTBOUND, BNK_F_REPLAY, BNK_F_CHECK_INBOUND ...) */
    uint32_t min_fill;    /* while the device is busy a GPU batch goes once it holds this many packets and a slot is
                             free (0 = 128, one upstream batch, or max_pkts / 4 if that is less); it always goes when the
                             device is idle, after 40 us, or full */
    uint32_t reserved;
} bnk_queue_cfg;
int bnk_queue_create(bnk_ctx *ctx, const bnk_queue_cfg *cfg, bnk_queue **out);
int bnk_queue_destroy(bnk_queue *q);
int bnk_queue_submit(bnk_queue *q, const uint8_t *const *pkts, const uint32_t *len, const uint32_t *slot, uint32_t n,
                     int64_t now_unix_ns, bnk_ticket *ticket);
int bnk_queue_wait(bnk_queue *q, bnk_ticket ticket, uint8_t *const *out, uint32_t *out_len, uint64_t *counter,
                   uint32_t *slot_out, uint8_t *status);
/* The same without the two host copies: the caller writes its packets straight into the pinned ring of the GPU
 * batch that is filling and reads the results there (a tun.Device.Read or ReceiveFunc can be pointed at the span's
 * slots, and Bind.Send / tun.Device.Write at the results).
 *   bnk_queue_reserve    room for n packets: packet k of the span lives at data + k * stride; a seal queue wants the
 *                        plaintext at +16 (the message is built in place from +0), an open queue the message at +0
 *                        (the plaintext comes back at +16); the caller sets len[k] and slot[k].  BNK_EBUSY as above.
 *   bnk_queue_commit     the packets are in: the GPU batch may go.  Must follow the reserve promptly (the GPU batch,
 *                        with other callers' packets, waits for it).  A packet whose len[] exceeds max_packet
 *                        is refused (BNK_EINVAL; its status comes back BAD_DESC or MALFORMED).
 *   bnk_queue_wait_span  blocks until the ticket's GPU batch is done; status[], out_len[], counter[] (and slot[] of
 *                        an open queue with BNK_F_DEMUX_INDEX) of the span are then valid, and the bytes stay where
 *                        they are until the release.  Look at status[k] before using packet k.
 *   bnk_queue_release    the caller is done with the span (once per ticket, after the wait). */
typedef struct bnk_queue_span {
    uint8_t *data;
    uint32_t stride;
    uint32_t reserved;
    uint32_t *len;
    uint32_t *slot;
    const uint32_t *out_len;
    const uint64_t *counter;
    const uint8_t *status;
} bnk_queue_span;
int bnk_queue_reserve(bnk_queue *q, uint32_t n, int64_t now_unix_ns, bnk_ticket *ticket, bnk_queue_span *span);
int bnk_queue_commit(bnk_queue *q, bnk_ticket ticket);
int bnk_queue_wait_span(bnk_queue *q, bnk_ticket ticket, bnk_queue_span *span);
int bnk_queue_release(bnk_queue *q, bnk_ticket ticket);
/* Blocks until bnk_queue_submit has room again (some GPU batch has been emptied by its callers), at most
 * timeout_ns (UINT64_MAX = no limit; BNK_ETIMEDOUT otherwise).  For callers that hold no ticket they could
 * collect instead. */
int bnk_queue_wait_room(bnk_queue *q, uint64_t timeout_ns);
/* GPU batches submitted, packets in them, and caller batches taken so far (packets / GPU batches = how well the
 * queue packs). */
int bnk_queue_stats_get(bnk_queue *q, uint64_t *gpu_batches, uint64_t *packets, uint64_t *caller_batches);

/* ---- several GPUs: placement of peers and a dispatcher that routes mixed batches ----
 * All per-peer state (keys, send counter, replay window, the flows of the peer's /32) lives in one context, so
 * peers shard over GPUs with no traffic between the GPUs; the reference likewise gives each peer one /32
 * (internal/dataplane/engine.go:294) and one sequential worker (internal/magicsock/bind.go:325-328).  A peer is
 * never split over two GPUs (its nonce order and its replay window are sequential).
 *
 * bnk_place_peers decides where peers go from a measured load per peer (packets or bytes of a past period):
 * peers in order of falling load, each to the GPU that carries the least so far (ties: the GPU with fewer
 * peers, then the lower ordinal), at most max_per_gpu peers per GPU.  With equal loads that is round robin;
 * with skewed loads (a few heavy peers) the heavy ones end up on different GPUs.  Pure host arithmetic, the
 * same on every caller that passes the same loads: processes that each drive one GPU agree on the placement
 * without talking to each other.  Outputs: gpu_of[p] and slot_of[p] (the peer's keypair slot in that GPU's
 * context, handed out in placement order), load_per_gpu[g] (may be NULL).  Returns BNK_EFULL when
 * n_gpus * max_per_gpu < n_peers. */
int bnk_place_peers(const uint64_t *load, uint32_t n_peers, uint32_t n_gpus, uint32_t max_per_gpu, uint32_t *gpu_of,
                    uint32_t *slot_of, uint64_t *load_per_gpu);

/* The dispatcher: one context per listed device, driven by one host thread each.  It stands where the
 * reference's device.NewDevice stands when a box has several GPUs: bnk_mgpu_seal / bnk_mgpu_open take one
 * mixed batch in the caller's buffers (a tun.Device.Read or conn.ReceiveFunc batch, or many of them), route
 * every packet to its peer's GPU, keep batch order inside each peer, run the per-GPU submits side by side and
 * hand the results back in the caller's order.  Plain cudaMemcpyAsync per GPU; no peer access, no collective. */
typedef struct bnk_mgpu bnk_mgpu;
typedef struct bnk_mgpu_cfg {
    uint32_t struct_size;       /* sizeof(bnk_mgpu_cfg) */
    uint32_t n_devices;
    const int32_t *devices;     /* CUDA ordinals; one listed twice gets two contexts (for tests on one GPU) */
    uint32_t max_pkts_per_gpu;  /* packets one submit of one GPU carries; longer batches go in rounds */
    uint32_t max_packet;        /* longest plaintext packet */
    uint32_t max_peers;         /* peers numbered 0 .. max_peers-1 */
    uint32_t reserved;
    bnk_cfg ctx;                /* per-GPU context settings; device_id is ignored, max_keypairs is per GPU */
} bnk_mgpu_cfg;
int bnk_mgpu_create(const bnk_mgpu_cfg *cfg, bnk_mgpu **out);
int bnk_mgpu_destroy(bnk_mgpu *m);
const char *bnk_mgpu_last_error_string(bnk_mgpu *m);
/* The context of GPU g (0 .. n_devices-1), for table calls the dispatcher does not wrap. */
bnk_ctx *bnk_mgpu_ctx(bnk_mgpu *m, uint32_t g);
/* Places all peers from `load` (NULL = equal loads) with bnk_place_peers.  Allowed while no peer is set:
 * a live peer moves with its next keypair (remove it, place, set it again), as a rekey would bring it. */
int bnk_mgpu_place(bnk_mgpu *m, const uint64_t *load);
int bnk_mgpu_locate(bnk_mgpu *m, uint32_t peer, uint32_t *gpu, uint32_t *slot);
/* What bnk_keypair_set + bnk_index_set + bnk_keypair_set_allowed_ip do, on the peer's GPU. */
int bnk_mgpu_peer_set(bnk_mgpu *m, uint32_t peer, const uint8_t send_key[32], const uint8_t recv_key[32],
                      uint32_t remote_index, uint32_t local_index, uint32_t allowed_ipv4);
int bnk_mgpu_peer_clear(bnk_mgpu *m, uint32_t peer);
/* bnk_acl_set on every GPU (the rule table is replicated, flows stay with their peer's GPU). */
int bnk_mgpu_acl_set(bnk_mgpu *m, int enforce, const bnk_acl_tuple *tuples, size_t n);
/* Seals packets pkts[i][0 .. len[i]) of peer peer[i]; the message goes to out[i] (room for len + 48 bytes),
 * its length to out_len[i], the nonce used to counter[i] (may be NULL), the outcome to status[i].  flags as for
 * bnk_seal_submit; counters are always taken from the peers' send counters.  A peer that is not set yields
 * BNK_PKT_NO_KEYPAIR.  Blocks until every GPU has finished.  One GPU's share is worked on by the calling thread
 * itself (with a single busy GPU nothing is handed to another thread); like the other calls of the library this
 * leaves the thread's current CUDA device set to a GPU of the dispatcher. */
int bnk_mgpu_seal(bnk_mgpu *m, const uint8_t *const *pkts, const uint32_t *len, const uint32_t *peer, uint32_t n,
                  uint32_t flags, int64_t now_unix_ns, uint8_t *const *out, uint32_t *out_len, uint64_t *counter,
                  uint8_t *status);
/* Opens messages msgs[i][0 .. len[i]); the GPU is chosen by the receiver index in each header (bytes 4..7)
 * through the indices given to bnk_mgpu_peer_set, the peer found goes to peer_out[i] (may be NULL), the
 * plaintext to out[i] (room for len bytes), its length to out_len[i].  flags as for bnk_open_submit
 * (BNK_F_REPLAY, BNK_F_INNER_CHECK, BNK_F_CHECK_INBOUND ...). */
int bnk_mgpu_open(bnk_mgpu *m, const uint8_t *const *msgs, const uint32_t *len, uint32_t n, uint32_t flags,
                  int64_t now_unix_ns, uint8_t *const *out, uint32_t *out_len, uint64_t *counter, uint32_t *peer_out,
                  uint8_t *status);
/* Packets and bytes the dispatcher has routed per peer since the last call with reset != 0: the measured load
 * for the next placement.  Packets handed to each GPU since creation go to per_gpu (may be NULL). */
int bnk_mgpu_loads_get(bnk_mgpu *m, uint64_t *packets_per_peer, uint64_t *bytes_per_peer, uint64_t *packets_per_gpu,
                       int reset);

/* ---- stage timing (tracing) ----
 * A submit made with BNK_F_TIMED brackets its kernels with CUDA events on the batch's stream. */
/* Duration of the kernels of the batch's most recent submit made with BNK_F_TIMED (excluding copies), milliseconds. */
int bnk_batch_last_kernel_ms(bnk_batch *b, float *ms);
/* Duration of the seal or open kernel alone in the batch's most recent seal/open submit, milliseconds. */
int bnk_batch_last_aead_ms(bnk_batch *b, float *ms);
/* Number of kernels this library has launched on the context since creation. */
int bnk_kernel_launch_count(bnk_ctx *ctx, uint64_t *count);

#ifdef __cplusplus
}
#endif
#endif
