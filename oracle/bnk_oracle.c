/*
 * bnk_oracle.c -- CPU restatement of the bnk dataplane hot path (see bnk_oracle.h).
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path, never the product.
 * Scalar, portable C; written for clarity, not speed.  The arithmetic is laid
 * out differently from the CUDA kernels on purpose (64-bit limbs and
 * unsigned __int128 here, 32-bit limbs there) so the two cannot share a bug.
 */
#include "bnk_oracle.h"

#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* little helpers                                                             */
/* ------------------------------------------------------------------------- */
static uint32_t ld32le(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static uint64_t ld64le(const uint8_t *p) { return (uint64_t)ld32le(p) | ((uint64_t)ld32le(p + 4) << 32); }
static void st32le(uint8_t *p, uint32_t v) {
    p[0] = (uint8_t)v;
    p[1] = (uint8_t)(v >> 8);
    p[2] = (uint8_t)(v >> 16);
    p[3] = (uint8_t)(v >> 24);
}
static void st64le(uint8_t *p, uint64_t v) {
    st32le(p, (uint32_t)v);
    st32le(p + 4, (uint32_t)(v >> 32));
}
static uint32_t rotl32(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }

/* ------------------------------------------------------------------------- */
/* ChaCha20 block function, RFC 8439 section 2.3                              */
/* ------------------------------------------------------------------------- */
#define QR(a, b, c, d)          \
    do {                        \
        a += b;                 \
        d ^= a;                 \
        d = rotl32(d, 16);      \
        c += d;                 \
        b ^= c;                 \
        b = rotl32(b, 12);      \
        a += b;                 \
        d ^= a;                 \
        d = rotl32(d, 8);       \
        c += d;                 \
        b ^= c;                 \
        b = rotl32(b, 7);       \
    } while (0)

void bnko_chacha20_block(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], uint8_t out[64]) {
    uint32_t init[16], x[16];
    init[0] = 0x61707865u; /* "expa" */
    init[1] = 0x3320646eu; /* "nd 3" */
    init[2] = 0x79622d32u; /* "2-by" */
    init[3] = 0x6b206574u; /* "te k" */
    for (int i = 0; i < 8; i++) init[4 + i] = ld32le(key + 4 * i);
    init[12] = counter;
    for (int i = 0; i < 3; i++) init[13 + i] = ld32le(nonce + 4 * i);
    memcpy(x, init, sizeof x);
    for (int round = 0; round < 10; round++) {
        QR(x[0], x[4], x[8], x[12]);
        QR(x[1], x[5], x[9], x[13]);
        QR(x[2], x[6], x[10], x[14]);
        QR(x[3], x[7], x[11], x[15]);
        QR(x[0], x[5], x[10], x[15]);
        QR(x[1], x[6], x[11], x[12]);
        QR(x[2], x[7], x[8], x[13]);
        QR(x[3], x[4], x[9], x[14]);
    }
    for (int i = 0; i < 16; i++) st32le(out + 4 * i, x[i] + init[i]);
}

/* RFC 8439 section 2.4: keystream XOR, block counter starting at `counter` */
void bnko_chacha20_xor(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], const uint8_t *in,
                       uint8_t *out, size_t len) {
    uint8_t ks[64];
    size_t done = 0;
    while (done < len) {
        size_t n = len - done < 64 ? len - done : 64;
        bnko_chacha20_block(key, counter++, nonce, ks);
        for (size_t i = 0; i < n; i++) out[done + i] = in[done + i] ^ ks[i];
        done += n;
    }
}

/* ------------------------------------------------------------------------- */
/* Poly1305, RFC 8439 section 2.5, on 64-bit limbs                            */
/* h = h0 + h1*2^64 + h2*2^128, r = r0 + r1*2^64 (clamped, so r1 % 4 == 0).   */
/* 2^130 = 5 (mod p) gives 2^128 * r1 = 5*(r1/4) = r1 + r1/4 =: s1.           */
/* ------------------------------------------------------------------------- */
typedef unsigned __int128 u128;

typedef struct {
    uint64_t h0, h1, h2;
    uint64_t r0, r1, s1;
    uint64_t pad0, pad1;
} poly_state;

static void poly_init(poly_state *st, const uint8_t key[32]) {
    st->h0 = st->h1 = st->h2 = 0;
    st->r0 = ld64le(key) & 0x0ffffffc0fffffffull;
    st->r1 = ld64le(key + 8) & 0x0ffffffc0ffffffcull;
    st->s1 = st->r1 + (st->r1 >> 2);
    st->pad0 = ld64le(key + 16);
    st->pad1 = ld64le(key + 24);
}

/* absorb one 16-byte block whose value is m0 + m1*2^64 + hibit*2^128 */
static void poly_block(poly_state *st, uint64_t m0, uint64_t m1, uint64_t hibit) {
    u128 t = (u128)st->h0 + m0;
    uint64_t h0 = (uint64_t)t;
    t = (u128)st->h1 + m1 + (uint64_t)(t >> 64);
    uint64_t h1 = (uint64_t)t;
    uint64_t h2 = st->h2 + hibit + (uint64_t)(t >> 64);

    u128 d0 = (u128)h0 * st->r0 + (u128)h1 * st->s1;
    u128 d1 = (u128)h0 * st->r1 + (u128)h1 * st->r0 + (u128)h2 * st->s1;
    uint64_t d2 = h2 * st->r0;

    h0 = (uint64_t)d0;
    d1 += (uint64_t)(d0 >> 64);
    h1 = (uint64_t)d1;
    h2 = d2 + (uint64_t)(d1 >> 64);

    /* fold everything above bit 130 back in: x*2^130 = 5x */
    uint64_t c = (h2 >> 2) * 5;
    h2 &= 3;
    t = (u128)h0 + c;
    h0 = (uint64_t)t;
    t = (u128)h1 + (uint64_t)(t >> 64);
    h1 = (uint64_t)t;
    h2 += (uint64_t)(t >> 64);
    st->h0 = h0;
    st->h1 = h1;
    st->h2 = h2;
}

static void poly_update(poly_state *st, const uint8_t *msg, size_t len) {
    while (len >= 16) {
        poly_block(st, ld64le(msg), ld64le(msg + 8), 1);
        msg += 16;
        len -= 16;
    }
    if (len) { /* short final block: append 0x01 then zeros, no 2^128 bit */
        uint8_t buf[16] = {0};
        memcpy(buf, msg, len);
        buf[len] = 1;
        poly_block(st, ld64le(buf), ld64le(buf + 8), 0);
    }
}

static void poly_finish(poly_state *st, uint8_t tag[16]) {
    uint64_t h0 = st->h0, h1 = st->h1, h2 = st->h2;
    /* one more fold so that h < 2^130 + small, then the conditional subtract of p */
    uint64_t c = (h2 >> 2) * 5;
    h2 &= 3;
    u128 t = (u128)h0 + c;
    h0 = (uint64_t)t;
    t = (u128)h1 + (uint64_t)(t >> 64);
    h1 = (uint64_t)t;
    h2 += (uint64_t)(t >> 64);
    /* g = h + 5; if g >= 2^130 then h >= p and the result is g - 2^130 */
    t = (u128)h0 + 5;
    uint64_t g0 = (uint64_t)t;
    t = (u128)h1 + (uint64_t)(t >> 64);
    uint64_t g1 = (uint64_t)t;
    uint64_t g2 = h2 + (uint64_t)(t >> 64);
    if (g2 >> 2) {
        h0 = g0;
        h1 = g1;
    }
    /* tag = (h + s) mod 2^128 */
    t = (u128)h0 + st->pad0;
    st64le(tag, (uint64_t)t);
    t = (u128)h1 + st->pad1 + (uint64_t)(t >> 64);
    st64le(tag + 8, (uint64_t)t);
}

void bnko_poly1305(const uint8_t key[32], const uint8_t *msg, size_t len, uint8_t tag[16]) {
    poly_state st;
    poly_init(&st, key);
    poly_update(&st, msg, len);
    poly_finish(&st, tag);
}

/* ------------------------------------------------------------------------- */
/* AEAD_CHACHA20_POLY1305, RFC 8439 section 2.8                               */
/* mac input = aad | pad16 | ciphertext | pad16 | le64(aad_len) | le64(ct_len)*/
/* ------------------------------------------------------------------------- */
static void aead_tag(const uint8_t key[32], const uint8_t nonce[12], const uint8_t *aad, size_t aad_len,
                     const uint8_t *ct, size_t len, uint8_t tag[16]) {
    uint8_t block0[64];
    poly_state st;
    bnko_chacha20_block(key, 0, nonce, block0);
    poly_init(&st, block0);
    /* every padded piece is a whole number of 16-byte blocks, all with the 2^128 bit */
    size_t full = aad_len & ~(size_t)15;
    poly_update(&st, aad, full);
    if (aad_len & 15) {
        uint8_t buf[16] = {0};
        memcpy(buf, aad + full, aad_len & 15);
        poly_update(&st, buf, 16);
    }
    full = len & ~(size_t)15;
    poly_update(&st, ct, full);
    if (len & 15) {
        uint8_t buf[16] = {0};
        memcpy(buf, ct + full, len & 15);
        poly_update(&st, buf, 16);
    }
    uint8_t lens[16];
    st64le(lens, (uint64_t)aad_len);
    st64le(lens + 8, (uint64_t)len);
    poly_update(&st, lens, 16);
    poly_finish(&st, tag);
}

void bnko_aead_seal(const uint8_t key[32], const uint8_t nonce[12], const uint8_t *aad, size_t aad_len,
                    const uint8_t *pt, size_t len, uint8_t *out) {
    bnko_chacha20_xor(key, 1, nonce, pt, out, len);
    aead_tag(key, nonce, aad, aad_len, out, len, out + len);
}

int bnko_aead_open(const uint8_t key[32], const uint8_t nonce[12], const uint8_t *aad, size_t aad_len,
                   const uint8_t *ct, size_t ct_len, uint8_t *out) {
    if (ct_len < 16) return 0;
    size_t len = ct_len - 16;
    uint8_t tag[16];
    aead_tag(key, nonce, aad, aad_len, ct, len, tag);
    uint8_t diff = 0;
    for (int i = 0; i < 16; i++) diff |= (uint8_t)(tag[i] ^ ct[len + i]);
    if (diff) {
        memset(out, 0, len);
        return 0;
    }
    bnko_chacha20_xor(key, 1, nonce, ct, out, len);
    return 1;
}

/* ------------------------------------------------------------------------- */
/* WireGuard transport data message (whitepaper 5.4.6)                        */
/*   u32le type=4 | u32le receiver index | u64le counter | AEAD(pt|pad) | tag */
/*   nonce = 4 zero bytes | u64le counter, empty AAD                          */
/* ------------------------------------------------------------------------- */

/* Padding: round the packet up to a multiple of 16, never beyond the MTU.
 * A packet longer than the MTU is padded as if only its last MTU-sized unit
 * counted; mtu == 0 means "no cap".  (Behaviour of the upstream device's send
 * path, restated from its documented rule.) */
size_t bnko_wg_padded_len(size_t len, size_t mtu) {
    size_t last_unit = len;
    if (mtu == 0) return (len + 15) & ~(size_t)15;
    if (last_unit > mtu) last_unit %= mtu;
    size_t padded = (last_unit + 15) & ~(size_t)15;
    if (padded > mtu) padded = mtu;
    return len + (padded - last_unit);
}

static void wg_nonce(uint64_t counter, uint8_t nonce[12]) {
    memset(nonce, 0, 4);
    st64le(nonce + 4, counter);
}

size_t bnko_wg_seal(const uint8_t key[32], uint32_t receiver_index, uint64_t counter, const uint8_t *pt,
                    size_t len, size_t mtu, uint8_t *out) {
    if (counter >= BNKO_REJECT_AFTER_MESSAGES) return 0;
    size_t padded = bnko_wg_padded_len(len, mtu);
    uint8_t *tmp = (uint8_t *)calloc(padded ? padded : 1, 1);
    memcpy(tmp, pt, len);
    st32le(out, 4);
    st32le(out + 4, receiver_index);
    st64le(out + 8, counter);
    uint8_t nonce[12];
    wg_nonce(counter, nonce);
    bnko_aead_seal(key, nonce, NULL, 0, tmp, padded, out + BNKO_WG_HEADER);
    free(tmp);
    return BNKO_WG_HEADER + padded + BNKO_WG_TAG;
}

int bnko_wg_open(const uint8_t key[32], const uint8_t *msg, size_t msg_len, uint8_t *out_pt, size_t *pt_len,
                 uint64_t *counter, uint32_t *receiver_index) {
    if (pt_len) *pt_len = 0;
    if (msg_len < BNKO_WG_HEADER + BNKO_WG_TAG || ld32le(msg) != 4) return BNKO_MALFORMED;
    uint64_t ctr = ld64le(msg + 8);
    if (counter) *counter = ctr;
    if (receiver_index) *receiver_index = ld32le(msg + 4);
    uint8_t nonce[12];
    wg_nonce(ctr, nonce);
    size_t len = msg_len - BNKO_WG_HEADER - BNKO_WG_TAG;
    if (!bnko_aead_open(key, nonce, NULL, 0, msg + BNKO_WG_HEADER, len + BNKO_WG_TAG, out_pt))
        return BNKO_AUTH_FAIL;
    if (pt_len) *pt_len = len;
    return len == 0 ? BNKO_KEEPALIVE : BNKO_OK;
}

int bnko_inner_check(const uint8_t *pt, size_t len, uint32_t allowed_ip, size_t *new_len) {
    if (len < 20 || (pt[0] >> 4) != 4) return 0;
    size_t total = ((size_t)pt[2] << 8) | pt[3];
    if (total > len || total < 20) return 0;
    uint32_t src = ((uint32_t)pt[12] << 24) | ((uint32_t)pt[13] << 16) | ((uint32_t)pt[14] << 8) | pt[15];
    if (allowed_ip == 0 || src != allowed_ip) return 0;
    if (new_len) *new_len = total;
    return 1;
}

int bnko_classify_shape(const uint8_t *pkt, size_t len) {
    static const uint8_t magic[10] = {'b', 'n', 'k', 0, 'd', 'i', 's', 'c', 'o', 0}; /* disco.go:20 */
    if (len >= sizeof magic && memcmp(pkt, magic, sizeof magic) == 0) return 10;
    if (len >= 20 && (pkt[0] >> 6) == 0 && pkt[4] == 0x21 && pkt[5] == 0x12 && pkt[6] == 0xA4 && pkt[7] == 0x42) return 11;
    return 0;
}

/* one's-complement sum of big-endian 16-bit words (RFC 1071), odd tail padded with a zero byte; NOT inverted */
static uint32_t csum_add(const uint8_t *p, size_t len, uint32_t acc) {
    uint64_t s = acc;
    size_t i = 0;
    for (; i + 1 < len; i += 2) s += ((uint32_t)p[i] << 8) | p[i + 1];
    if (i < len) s += (uint32_t)p[i] << 8;
    while (s >> 16) s = (s & 0xffff) + (s >> 16);
    return (uint32_t)s;
}

uint16_t bnko_inet_checksum(const uint8_t *p, size_t len, uint32_t initial) {
    return (uint16_t)~csum_add(p, len, initial);
}

int bnko_gso_split(const uint8_t *in, size_t in_len, unsigned hdr_len, unsigned gso_size, unsigned csum_start,
                   unsigned csum_offset, unsigned proto, uint8_t *out, size_t out_stride, uint32_t *sizes,
                   size_t max_segs) {
    if ((proto != 6 && proto != 17) || csum_start < 20 || hdr_len <= csum_start || gso_size == 0 || in_len <= hdr_len ||
        csum_offset + 2 > hdr_len - csum_start || (in[0] >> 4) != 4)
        return -1;
    const unsigned th = hdr_len - csum_start;
    const uint32_t first_seq = proto == 6 ? (((uint32_t)in[csum_start + 4] << 24) | ((uint32_t)in[csum_start + 5] << 16) |
                                             ((uint32_t)in[csum_start + 6] << 8) | in[csum_start + 7])
                                          : 0;
    const unsigned first_id = ((unsigned)in[4] << 8) | in[5];
    size_t at = hdr_len, i = 0;
    for (; at < in_len; i++, at += gso_size) {
        if (i == max_segs) return -1;
        size_t seg = in_len - at < gso_size ? in_len - at : gso_size;
        size_t total = hdr_len + seg;
        uint8_t *o = out + i * out_stride;
        sizes[i] = (uint32_t)total;
        memcpy(o, in, hdr_len);
        unsigned id = (first_id + (unsigned)i) & 0xffff;
        o[4] = (uint8_t)(id >> 8);
        o[5] = (uint8_t)id;
        o[2] = (uint8_t)(total >> 8);
        o[3] = (uint8_t)total;
        o[10] = o[11] = 0;
        uint16_t ipc = bnko_inet_checksum(o, csum_start, 0);
        o[10] = (uint8_t)(ipc >> 8);
        o[11] = (uint8_t)ipc;
        uint8_t *t = o + csum_start;
        if (proto == 6) {
            uint32_t seq = first_seq + (uint32_t)(i * gso_size);
            t[4] = (uint8_t)(seq >> 24);
            t[5] = (uint8_t)(seq >> 16);
            t[6] = (uint8_t)(seq >> 8);
            t[7] = (uint8_t)seq;
            if (at + seg != in_len) t[13] &= (uint8_t)~0x09; /* FIN | PSH only on the last segment */
        } else {
            unsigned ulen = th + (unsigned)seg;
            t[4] = (uint8_t)(ulen >> 8);
            t[5] = (uint8_t)ulen;
        }
        t[csum_offset] = t[csum_offset + 1] = 0;
        memcpy(o + hdr_len, in + at, seg);
        /* pseudo header: src, dst, zero+proto, transport length */
        uint32_t acc = csum_add(o + 12, 8, 0);
        acc += proto;
        acc += (uint32_t)(th + seg);
        uint16_t tc = bnko_inet_checksum(t, th + seg, acc);
        t[csum_offset] = (uint8_t)(tc >> 8);
        t[csum_offset + 1] = (uint8_t)tc;
    }
    return (int)i;
}

/* Batch forms.  Packet i occupies ring[off[i] ...]: 16 bytes of header room, then
 * the payload.  Seal works in place (payload -> header|ciphertext|tag at off[i]);
 * open reads the message at off[i] and leaves the plaintext at off[i]+16. */
void bnko_wg_seal_batch(const uint8_t *keys, const uint32_t *remote_index, size_t mtu, uint8_t *ring,
                        const uint32_t *off, const uint32_t *len, const uint32_t *slot,
                        const uint64_t *counter, uint8_t *status, uint32_t *out_len, size_t n) {
    uint8_t *tmp = (uint8_t *)malloc(65536 + 64);
    for (size_t i = 0; i < n; i++) {
        uint8_t *p = ring + off[i];
        size_t m = bnko_wg_seal(keys + 32u * slot[i], remote_index[slot[i]], counter[i], p + BNKO_WG_HEADER,
                                len[i], mtu, tmp);
        if (m == 0) {
            status[i] = BNKO_COUNTER_EXHAUSTED;
            if (out_len) out_len[i] = 0;
            continue;
        }
        memcpy(p, tmp, m);
        status[i] = BNKO_OK;
        if (out_len) out_len[i] = (uint32_t)m;
    }
    free(tmp);
}

void bnko_wg_open_batch(const uint8_t *keys, uint8_t *ring, const uint32_t *off, const uint32_t *len,
                        const uint32_t *slot, uint64_t *counter, uint8_t *status, uint32_t *out_len, size_t n) {
    uint8_t *tmp = (uint8_t *)malloc(65536 + 64);
    for (size_t i = 0; i < n; i++) {
        uint8_t *p = ring + off[i];
        size_t pl = 0;
        uint64_t ctr = 0;
        int st = bnko_wg_open(keys + 32u * slot[i], p, len[i], tmp, &pl, &ctr, NULL);
        status[i] = (uint8_t)st;
        counter[i] = ctr;
        if (st == BNKO_OK || st == BNKO_KEEPALIVE) {
            memcpy(p + BNKO_WG_HEADER, tmp, pl);
        } else if (st == BNKO_AUTH_FAIL) {
            memset(p + BNKO_WG_HEADER, 0, len[i] - BNKO_WG_HEADER - BNKO_WG_TAG);
        }
        if (out_len) out_len[i] = (uint32_t)pl;
    }
    free(tmp);
}

/* ------------------------------------------------------------------------- */
/* Anti-replay window, RFC 6479 (ring of 64-bit blocks)                       */
/* window = (ring_blocks - 1) * 64 counters behind the highest one seen.      */
/* ------------------------------------------------------------------------- */
struct bnko_replay {
    uint64_t last;
    uint32_t ring_blocks;
    uint64_t *ring;
};

bnko_replay *bnko_replay_new(uint32_t ring_blocks) {
    if (ring_blocks == 0 || (ring_blocks & (ring_blocks - 1))) return NULL;
    bnko_replay *r = (bnko_replay *)calloc(1, sizeof *r);
    r->ring_blocks = ring_blocks;
    r->ring = (uint64_t *)calloc(ring_blocks, sizeof(uint64_t));
    return r;
}
void bnko_replay_free(bnko_replay *r) {
    if (!r) return;
    free(r->ring);
    free(r);
}
void bnko_replay_reset(bnko_replay *r) {
    r->last = 0;
    memset(r->ring, 0, r->ring_blocks * sizeof(uint64_t));
}
uint64_t bnko_replay_last(const bnko_replay *r) { return r->last; }
void bnko_replay_ring(const bnko_replay *r, uint64_t *out) { memcpy(out, r->ring, r->ring_blocks * 8u); }
void bnko_replay_load(bnko_replay *r, uint64_t last, const uint64_t *ring) {
    r->last = last;
    memcpy(r->ring, ring, r->ring_blocks * 8u);
}

int bnko_replay_validate(bnko_replay *r, uint64_t counter, uint64_t limit) {
    const uint64_t blocks = r->ring_blocks;
    const uint64_t window = (blocks - 1) * 64;
    if (counter >= limit) return 0;
    uint64_t block = counter >> 6;
    if (counter > r->last) {
        /* slide forward: every block entered since the old top starts empty */
        uint64_t top = r->last >> 6;
        uint64_t steps = block - top;
        if (steps > blocks) steps = blocks;
        for (uint64_t i = 1; i <= steps; i++) r->ring[(top + i) & (blocks - 1)] = 0;
        r->last = counter;
    } else if (r->last - counter > window) {
        return 0; /* fell off the back of the window */
    }
    uint64_t *word = &r->ring[block & (blocks - 1)];
    uint64_t bit = 1ull << (counter & 63);
    if (*word & bit) return 0; /* seen before */
    *word |= bit;
    return 1;
}

/* ------------------------------------------------------------------------- */
/* ACL filter: internal/filter/filter.go + internal/acl/acl.go:149-172        */
/* ------------------------------------------------------------------------- */
#define TTL_UDP_NS (30ll * 1000000000ll)  /* filter.go:19 */
#define TTL_TCP_NS (120ll * 1000000000ll) /* filter.go:20 */
#define TTL_ICMP_NS (30ll * 1000000000ll) /* filter.go:21 */
#define SWEEP_THRESHOLD 4096u             /* filter.go:202 */

typedef struct {
    uint8_t proto;
    uint32_t src, dst;
    uint16_t sport, dport;
    uint8_t icmp_type;
} parsed_t;

/* filter.go:71-106 */
static int parse_pkt(const uint8_t *pkt, size_t len, parsed_t *p) {
    if (len < 20 || (pkt[0] >> 4) != 4) return 0;
    size_t ihl = (size_t)(pkt[0] & 0x0f) * 4;
    if (ihl < 20 || len < ihl) return 0;
    memset(p, 0, sizeof *p);
    p->proto = pkt[9];
    p->src = ((uint32_t)pkt[12] << 24) | ((uint32_t)pkt[13] << 16) | ((uint32_t)pkt[14] << 8) | pkt[15];
    p->dst = ((uint32_t)pkt[16] << 24) | ((uint32_t)pkt[17] << 16) | ((uint32_t)pkt[18] << 8) | pkt[19];
    const uint8_t *body = pkt + ihl;
    size_t blen = len - ihl;
    switch (p->proto) {
    case 6:
    case 17:
        if (blen < 4) return 0;
        p->sport = (uint16_t)((body[0] << 8) | body[1]);
        p->dport = (uint16_t)((body[2] << 8) | body[3]);
        break;
    case 1:
        if (blen < 1) return 0;
        p->icmp_type = body[0];
        break;
    default:
        return 0;
    }
    return 1;
}

int bnko_filter_parse(const uint8_t *pkt, size_t len, uint32_t out[6]) {
    parsed_t p;
    if (!parse_pkt(pkt, len, &p)) return 0;
    out[0] = p.proto;
    out[1] = p.src;
    out[2] = p.dst;
    out[3] = p.sport;
    out[4] = p.dport;
    out[5] = p.icmp_type;
    return 1;
}

/* filter.go:108-117 */
static int64_t flow_ttl(uint8_t proto) {
    switch (proto) {
    case 6:
        return TTL_TCP_NS;
    case 1:
        return TTL_ICMP_NS;
    default:
        return TTL_UDP_NS;
    }
}

/* netip.Prefix.Contains for an IPv4 address: equal on the top `bits` bits */
static int prefix_contains(const bnko_prefix *p, uint32_t addr) {
    if (p->bits < 0 || p->bits > 32) return 0;
    if (p->bits == 0) return 1;
    uint32_t mask = 0xffffffffu << (32 - p->bits);
    return ((addr ^ p->addr) & mask) == 0;
}

/* acl.go:149-172 */
int bnko_rule_match(const bnko_rule *r, const bnko_prefix *srcs, const bnko_port_range *ports, uint32_t src,
                    uint8_t proto, uint16_t dport) {
    if (r->proto == 0 || proto != r->proto) return 0;
    int in_src = 0;
    for (uint32_t i = r->src_begin; i < r->src_end; i++) {
        if (prefix_contains(&srcs[i], src)) {
            in_src = 1;
            break;
        }
    }
    if (!in_src) return 0;
    if (r->proto == 1) return 1;
    for (uint32_t i = r->port_begin; i < r->port_end; i++)
        if (dport >= ports[i].first && dport <= ports[i].last) return 1;
    return 0;
}

/* flow table: Go map[flowKey]time.Time restated as open addressing with tombstones */
typedef struct {
    uint32_t remote;
    uint16_t rport, lport;
    uint8_t proto;
    uint8_t state; /* 0 empty, 1 live, 2 tombstone */
    int64_t exp;
} flow_ent;

struct bnko_filter {
    int enforce;
    bnko_rule *rules;
    size_t n_rules;
    bnko_prefix *srcs;
    bnko_port_range *ports;
    flow_ent *tab;
    size_t cap;  /* power of two */
    size_t live; /* len(f.flows) */
    size_t used; /* live + tombstones */
    /* The reference sweeps the whole map on every NoteOutbound once it holds more
     * than 4096 flows (filter.go:202-208).  A sweep at time T leaves nothing with
     * exp < T, and whatever is written afterwards by calls that also run at T gets
     * exp > T, so a repeat sweep at the same T finds nothing: it is skipped. */
    int64_t swept_at;
    int swept_valid;
};

static uint64_t flow_hash(uint32_t remote, uint16_t rport, uint16_t lport, uint8_t proto) {
    uint64_t z = ((uint64_t)remote << 32) | ((uint64_t)rport << 16) | lport;
    z ^= (uint64_t)proto << 59;
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

static flow_ent *flow_find(bnko_filter *f, uint32_t remote, uint16_t rport, uint16_t lport, uint8_t proto) {
    size_t i = flow_hash(remote, rport, lport, proto) & (f->cap - 1);
    for (;;) {
        flow_ent *e = &f->tab[i];
        if (e->state == 0) return NULL;
        if (e->state == 1 && e->remote == remote && e->rport == rport && e->lport == lport && e->proto == proto)
            return e;
        i = (i + 1) & (f->cap - 1);
    }
}

static void flow_rehash(bnko_filter *f, size_t new_cap) {
    flow_ent *old = f->tab;
    size_t old_cap = f->cap;
    f->tab = (flow_ent *)calloc(new_cap, sizeof(flow_ent));
    f->cap = new_cap;
    f->used = f->live;
    for (size_t k = 0; k < old_cap; k++) {
        if (old[k].state != 1) continue;
        size_t i = flow_hash(old[k].remote, old[k].rport, old[k].lport, old[k].proto) & (new_cap - 1);
        while (f->tab[i].state) i = (i + 1) & (new_cap - 1);
        f->tab[i] = old[k];
    }
    free(old);
}

static void flow_put(bnko_filter *f, uint32_t remote, uint16_t rport, uint16_t lport, uint8_t proto, int64_t exp) {
    flow_ent *e = flow_find(f, remote, rport, lport, proto);
    if (e) {
        e->exp = exp;
        return;
    }
    if ((f->used + 1) * 2 > f->cap) flow_rehash(f, f->live * 4 + 16 > f->cap ? f->cap * 2 : f->cap);
    size_t i = flow_hash(remote, rport, lport, proto) & (f->cap - 1);
    while (f->tab[i].state == 1) i = (i + 1) & (f->cap - 1);
    if (f->tab[i].state == 0) f->used++;
    f->tab[i].remote = remote;
    f->tab[i].rport = rport;
    f->tab[i].lport = lport;
    f->tab[i].proto = proto;
    f->tab[i].state = 1;
    f->tab[i].exp = exp;
    f->live++;
}

bnko_filter *bnko_filter_new(void) { /* filter.go:41-43: allow-all until rules are pushed */
    bnko_filter *f = (bnko_filter *)calloc(1, sizeof *f);
    f->cap = 1024;
    f->tab = (flow_ent *)calloc(f->cap, sizeof(flow_ent));
    return f;
}

static void drop_rules(bnko_filter *f) {
    free(f->rules);
    free(f->srcs);
    free(f->ports);
    f->rules = NULL;
    f->srcs = NULL;
    f->ports = NULL;
    f->n_rules = 0;
}

void bnko_filter_free(bnko_filter *f) {
    if (!f) return;
    drop_rules(f);
    free(f->tab);
    free(f);
}

/* filter.go:46-51 -- the flow table is kept across rule changes */
void bnko_filter_set_rules(bnko_filter *f, const bnko_rule *rules, size_t n_rules, const bnko_prefix *srcs,
                           size_t n_srcs, const bnko_port_range *ports, size_t n_ports) {
    drop_rules(f);
    f->enforce = 1;
    f->n_rules = n_rules;
    f->rules = (bnko_rule *)malloc((n_rules ? n_rules : 1) * sizeof *rules);
    f->srcs = (bnko_prefix *)malloc((n_srcs ? n_srcs : 1) * sizeof *srcs);
    f->ports = (bnko_port_range *)malloc((n_ports ? n_ports : 1) * sizeof *ports);
    if (n_rules) memcpy(f->rules, rules, n_rules * sizeof *rules);
    if (n_srcs) memcpy(f->srcs, srcs, n_srcs * sizeof *srcs);
    if (n_ports) memcpy(f->ports, ports, n_ports * sizeof *ports);
}

/* filter.go:54-59 */
void bnko_filter_set_allow_all(bnko_filter *f) {
    drop_rules(f);
    f->enforce = 0;
}

size_t bnko_filter_flow_count(const bnko_filter *f) { return f->live; }

/* the map's contents, in no particular order: Go's f.flows as (key, expiry) pairs */
size_t bnko_filter_flows_export(const bnko_filter *f, bnko_flow *out, size_t cap) {
    size_t n = 0;
    for (size_t k = 0; k < f->cap; k++) {
        if (f->tab[k].state != 1) continue;
        if (n < cap) {
            out[n].remote = f->tab[k].remote;
            out[n].rport = f->tab[k].rport;
            out[n].lport = f->tab[k].lport;
            out[n].proto = f->tab[k].proto;
            memset(out[n].reserved, 0, sizeof out[n].reserved);
            out[n].exp = f->tab[k].exp;
        }
        n++;
    }
    return n;
}

/* filter.go:121-147 */
int bnko_filter_check_inbound(bnko_filter *f, const uint8_t *pkt, size_t len, int64_t now_ns) {
    if (!f->enforce) return 1;
    parsed_t p;
    if (!parse_pkt(pkt, len, &p)) return 0;
    for (size_t i = 0; i < f->n_rules; i++)
        if (bnko_rule_match(&f->rules[i], f->srcs, f->ports, p.src, p.proto, p.dport)) return 1;
    flow_ent *e = flow_find(f, p.src, p.sport, p.dport, p.proto);
    if (e) {
        if (now_ns < e->exp) {
            e->exp = now_ns + flow_ttl(p.proto);
            if (!f->swept_valid || f->swept_at != now_ns) f->swept_valid = 0;
            return 1;
        }
        e->state = 2;
        f->live--;
    }
    return 0;
}

/* filter.go:189-209 */
void bnko_filter_note_outbound(bnko_filter *f, const uint8_t *pkt, size_t len, int64_t now_ns) {
    if (!f->enforce) return;
    parsed_t p;
    if (!parse_pkt(pkt, len, &p)) return;
    flow_put(f, p.dst, p.dport, p.sport, p.proto, now_ns + flow_ttl(p.proto));
    if (!f->swept_valid || f->swept_at != now_ns) f->swept_valid = 0;
    if (f->live > SWEEP_THRESHOLD && !f->swept_valid) {
        for (size_t k = 0; k < f->cap; k++) {
            if (f->tab[k].state == 1 && now_ns > f->tab[k].exp) {
                f->tab[k].state = 2;
                f->live--;
            }
        }
        f->swept_at = now_ns;
        f->swept_valid = 1;
    }
}

void bnko_filter_check_batch(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                             int64_t now_ns, uint8_t *verdict) {
    for (size_t i = 0; i < n; i++)
        verdict[i] = (uint8_t)bnko_filter_check_inbound(f, hdr + i * stride, len[i], now_ns);
}

/* The same batch on several host cores, for full-size comparisons.  CheckInbound (filter.go:121-147) first
 * walks the rules (filter.go:131-135), which reads nothing a packet can change, and only then touches the flow
 * table.  So the rule walk of every header runs in parallel here (phase 1), and the rest of CheckInbound runs
 * header by header in batch order exactly as above (phase 2): the verdicts and the table afterwards are those
 * of bnko_filter_check_batch. */
typedef struct {
    const bnko_filter *f;
    const uint8_t *hdr;
    size_t stride, begin, end;
    const uint32_t *len;
    uint8_t *pre; /* 0 = does not parse, 1 = a rule matches, 2 = goes on to the flow table */
} rule_job;

static void *rule_walk_worker(void *arg) {
    rule_job *j = (rule_job *)arg;
    const bnko_filter *f = j->f;
    for (size_t i = j->begin; i < j->end; i++) {
        parsed_t p;
        uint8_t r = 2;
        if (!parse_pkt(j->hdr + i * j->stride, j->len[i], &p)) r = 0;
        else
            for (size_t k = 0; k < f->n_rules; k++)
                if (bnko_rule_match(&f->rules[k], f->srcs, f->ports, p.src, p.proto, p.dport)) {
                    r = 1;
                    break;
                }
        j->pre[i] = r;
    }
    return NULL;
}

void bnko_filter_check_batch_mt(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                                int64_t now_ns, uint8_t *verdict, int threads) {
    if (!f->enforce) {
        memset(verdict, 1, n);
        return;
    }
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    uint8_t *pre = (uint8_t *)malloc(n ? n : 1);
    pthread_t tid[256];
    rule_job job[256];
    for (int t = 0; t < threads; t++) {
        job[t] = (rule_job){f, hdr, stride, n * (size_t)t / (size_t)threads, n * (size_t)(t + 1) / (size_t)threads, len, pre};
        pthread_create(&tid[t], NULL, rule_walk_worker, &job[t]);
    }
    for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    for (size_t i = 0; i < n; i++) {
        if (pre[i] != 2) {
            verdict[i] = pre[i];
            continue;
        }
        parsed_t p;
        parse_pkt(hdr + i * stride, len[i], &p);
        uint8_t v = 0;
        flow_ent *e = flow_find(f, p.src, p.sport, p.dport, p.proto);
        if (e) {
            if (now_ns < e->exp) {
                e->exp = now_ns + flow_ttl(p.proto);
                if (!f->swept_valid || f->swept_at != now_ns) f->swept_valid = 0;
                v = 1;
            } else {
                e->state = 2;
                f->live--;
            }
        }
        verdict[i] = v;
    }
    free(pre);
}

void bnko_filter_note_batch(bnko_filter *f, const uint8_t *hdr, size_t stride, const uint32_t *len, size_t n,
                            int64_t now_ns) {
    for (size_t i = 0; i < n; i++) bnko_filter_note_outbound(f, hdr + i * stride, len[i], now_ns);
}
