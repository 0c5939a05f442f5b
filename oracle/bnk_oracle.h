/*
 * bnk_oracle.h -- CPU restatement of the bnk dataplane hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker that the CUDA path is
 * compared against (tests, the smoke check, and the CPU-baseline leg of the
 * benchmark).  Nothing in the product package may call it.
 *
 * What it restates, and from where:
 *   - ChaCha20-Poly1305 AEAD: RFC 8439 (the algorithm behind
 *     golang.org/x/crypto v0.55.0 chacha20poly1305, a go.mod:7 dependency
 *     whose source is not in the reference tree).
 *   - WireGuard transport-data framing, padding, nonce and the anti-replay
 *     window: WireGuard whitepaper section 5.4.6 and RFC 6479 (implemented
 *     upstream by golang.zx2c4.com/wireguard v0.0.0-20260522210424-ecfc5a8d5446,
 *     go.mod:10; reached by the reference only through device.NewDevice,
 *     internal/dataplane/engine.go:51).
 *   - The ACL packet filter: internal/filter/filter.go and
 *     internal/acl/acl.go:149-172 of the reference, function by function.
 *
 * Parity pin: the reference holds no known-answer bytes for the AEAD, nonce or
 * replay window ("parity unpinned" by the reference itself); the AEAD is pinned
 * here against three independent RFC 8439 implementations (OpenSSL, the
 * `cryptography` package, libsodium via PyNaCl) and against committed golden
 * vectors generated from them.  The filter is pinned against every case of the
 * reference's own filter_test.go / tun_test.go / acl_test.go.
 */
#ifndef BNK_ORACLE_H
#define BNK_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* per-packet outcome codes; the numeric values are shared with include/bnk_gpu.h */
enum {
    BNKO_OK = 0,
    BNKO_AUTH_FAIL = 1,
    BNKO_REPLAY = 2,
    BNKO_FILTER_DENY = 3,
    BNKO_MALFORMED = 4,
    BNKO_KEEPALIVE = 5,
    BNKO_COUNTER_EXHAUSTED = 6,
    BNKO_BAD_DESC = 7
};

#define BNKO_WG_HEADER 16u
#define BNKO_WG_TAG 16u
/* whitepaper: Reject-After-Messages = 2^64 - 2^13 - 1 */
#define BNKO_REJECT_AFTER_MESSAGES 0xFFFFFFFFFFFFDFFFull

/* ---- RFC 8439 ---- */
void bnko_chacha20_block(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], uint8_t out[64]);
void bnko_chacha20_xor(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], const uint8_t *in,
                       uint8_t *out, size_t len);
void bnko_poly1305(const uint8_t key[32], const uint8_t *msg, size_t len, uint8_t tag[16]);
void bnko_aead_seal(const uint8_t key[32], const uint8_t nonce[12], const uint8_t *aad, size_t aad_len,
                    const uint8_t *pt, size_t len, uint8_t *out /* len + 16 */);
/* returns 1 on success; on failure returns 0 and zeroes out[0..ct_len-16) */
int bnko_aead_open(const uint8_t key[32], const uint8_t nonce[12], const uint8_t *aad, size_t aad_len,
                   const uint8_t *ct, size_t ct_len /* incl. tag */, uint8_t *out);

/* ---- WireGuard transport data ---- */
size_t bnko_wg_padded_len(size_t len, size_t mtu);
/* writes header | ciphertext | tag into out, returns message length (0 if the counter is exhausted) */
size_t bnko_wg_seal(const uint8_t key[32], uint32_t receiver_index, uint64_t counter, const uint8_t *pt,
                    size_t len, size_t mtu, uint8_t *out);
/* returns BNKO_OK / BNKO_KEEPALIVE / BNKO_AUTH_FAIL / BNKO_MALFORMED; no replay check here */
int bnko_wg_open(const uint8_t key[32], const uint8_t *msg, size_t msg_len, uint8_t *out_pt, size_t *pt_len,
                 uint64_t *counter, uint32_t *receiver_index);

/* What the upstream sequential receiver does with an authenticated, fresh plaintext before the TUN write
 * (restated from its documented behaviour): IPv4 only, 20 <= total-length field <= len, the packet is cut to the
 * total length, and its source address must be the sending peer's allowed address (the reference gives each peer
 * one /32, internal/dataplane/engine.go:294).  Returns 1 and the new length, or 0 = drop. */
int bnko_inner_check(const uint8_t *pt, size_t len, uint32_t allowed_ip, size_t *new_len);

/* Segmentation of an IPv4 TCP/UDP super-packet the way the upstream Linux TUN offload code splits a read that
 * carries a virtio-net header (restated from its documented behaviour; the module is not in the reference tree):
 * per segment the headers are copied, IPv4 id += segment number, total length and header checksum are rewritten,
 * TCP sequence += segment number * gso_size with FIN/PSH only on the last segment, UDP length is rewritten, and
 * the transport checksum is recomputed.  Segment i is written at out + i*out_stride, its length to sizes[i].
 * Returns the number of segments, or -1 when the headers are inconsistent or max_segs is too small. */
int bnko_gso_split(const uint8_t *in, size_t in_len, unsigned hdr_len, unsigned gso_size, unsigned csum_start,
                   unsigned csum_offset, unsigned proto, uint8_t *out, size_t out_stride, uint32_t *sizes,
                   size_t max_segs);
/* RFC 1071 checksum helpers, for tests */
uint16_t bnko_inet_checksum(const uint8_t *p, size_t len, uint32_t initial);

/* Shape tests of Bind.classify (internal/magicsock/bind.go:207-228): 10 = disco.IsDisco
 * (internal/disco/disco.go:20,177-179), 11 = isSTUN (bind.go:250-253), 0 = neither (goes to the byAddr lookup). */
int bnko_classify_shape(const uint8_t *pkt, size_t len);

/* batch forms over a packet ring (same descriptor layout as the GPU library) */
void bnko_wg_seal_batch(const uint8_t *keys /* n_keys*32 */, const uint32_t *remote_index /* n_keys */,
                        size_t mtu, uint8_t *ring, const uint32_t *off, const uint32_t *len,
                        const uint32_t *slot, const uint64_t *counter, uint8_t *status, uint32_t *out_len,
                        size_t n);
void bnko_wg_open_batch(const uint8_t *keys, uint8_t *ring, const uint32_t *off, const uint32_t *len,
                        const uint32_t *slot, uint64_t *counter, uint8_t *status, uint32_t *out_len, size_t n);

/* ---- RFC 6479 anti-replay window ---- */
typedef struct bnko_replay bnko_replay;
bnko_replay *bnko_replay_new(uint32_t ring_blocks /* power of two, e.g. 32 or 128 */);
void bnko_replay_free(bnko_replay *r);
void bnko_replay_reset(bnko_replay *r);
int bnko_replay_validate(bnko_replay *r, uint64_t counter, uint64_t limit); /* 1 accept, 0 reject */
uint64_t bnko_replay_last(const bnko_replay *r);
void bnko_replay_ring(const bnko_replay *r, uint64_t *out /* ring_blocks words */);
void bnko_replay_load(bnko_replay *r, uint64_t last, const uint64_t *ring);

/* ---- ACL filter (internal/filter + acl.Match) ---- */
typedef struct {
    uint32_t addr;   /* IPv4 prefix address, host order (a.b.c.d -> a<<24|...) */
    int32_t bits;    /* prefix length 0..32; <0 = invalid / non-IPv4 prefix (never contains) */
} bnko_prefix;
typedef struct {
    uint16_t first, last;
} bnko_port_range;
typedef struct {
    uint8_t proto;        /* 6 "tcp", 17 "udp", 1 "icmp", 0 = any other string (never equal) */
    uint32_t src_begin, src_end;   /* range in the srcs array */
    uint32_t port_begin, port_end; /* range in the ports array */
} bnko_rule;

typedef struct bnko_filter bnko_filter;
bnko_filter *bnko_filter_new(void);
void bnko_filter_free(bnko_filter *f);
void bnko_filter_set_rules(bnko_filter *f, const bnko_rule *rules, size_t n_rules, const bnko_prefix *srcs,
                           size_t n_srcs, const bnko_port_range *ports, size_t n_ports);
void bnko_filter_set_allow_all(bnko_filter *f);
int bnko_filter_check_inbound(bnko_filter *f, const uint8_t *pkt, size_t len, int64_t now_ns);
void bnko_filter_note_outbound(bnko_filter *f, const uint8_t *pkt, size_t len, int64_t now_ns);
size_t bnko_filter_flow_count(const bnko_filter *f);
/* one entry of the flow map: key {remote, remote port, local port, proto} -> expiry (unix ns); same layout as
 * bnk_flow_entry of the GPU library */
typedef struct {
    uint32_t remote;
    uint16_t rport, lport;
    uint8_t proto;
    uint8_t reserved[7];
    int64_t exp;
} bnko_flow;
/* writes up to cap entries, returns how many the map holds */
size_t bnko_filter_flows_export(const bnko_filter *f, bnko_flow *out, size_t cap);
/* header-array forms: packet i is hdr + i*stride, length len[i] */
void bnko_filter_check_batch(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                             int64_t now_ns, uint8_t *verdict);
void bnko_filter_note_batch(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                            int64_t now_ns);
/* bnko_filter_check_batch with the rule walk spread over `threads` host threads; same verdicts, same table */
void bnko_filter_check_batch_mt(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                                int64_t now_ns, uint8_t *verdict, int threads);
int bnko_rule_match(const bnko_rule *r, const bnko_prefix *srcs, const bnko_port_range *ports, uint32_t src,
                    uint8_t proto, uint16_t dport);
/* parse; returns 1 ok.  out[0]=proto out[1]=src out[2]=dst out[3]=sport out[4]=dport out[5]=icmp type */
int bnko_filter_parse(const uint8_t *pkt, size_t len, uint32_t out[6]);

#ifdef __cplusplus
}
#endif
#endif
