// Batched WireGuard transport-data seal / open for sm_100a.
//
// Work mapping: one thread owns one packet from the first ChaCha20 block to the
// Poly1305 tag, so every lane of a warp does useful 32-bit integer work on every
// instruction.  The path is bound by instruction issue on the integer pipes, not
// by HBM: ~19 integer operations per payload byte against ~2 bytes of traffic
// per payload byte, and the rotations of ChaCha20 issue at half rate on sm_100.
//
// Data movement is therefore kept to the fewest instructions: per 64-byte step a
// lane issues four 16-byte loads of its own packet ahead of the step's 80 quarter
// rounds (the rounds hide the latency; the two loads that share a 32-byte sector
// meet in L1) and four 16-byte stores after them (L2 merges the half sectors
// before they reach HBM).  No shared memory, no barriers, no cross-lane traffic:
// staging the 32 packets of a warp through shared memory so that global accesses
// are 512-byte wavefronts was measured and is 6 % slower, because its address
// arithmetic, shuffles and barriers cost issue slots that the rounds need.
//
// Arithmetic: ChaCha20 is RFC 8439 section 2.3 on 16 registers (rotations by 16
// and 8 are byte permutes, by 12 and 7 funnel shifts).  Poly1305 keeps h in five
// 32-bit limbs (radix 2^32) and multiplies with 32x32->64 multiply-adds on the
// FMA pipe.  The MAC input is ciphertext | zero pad to 16 | le64(0) | le64(ct_len),
// RFC 8439 section 2.8 with empty AAD; nonce = 32 zero bits | le64(counter) and the
// header is le32(4) | le32(receiver index) | le64(counter) (WireGuard whitepaper 5.4.6).
#include "bnk_internal.cuh"

namespace {

// Occupancy target for the register allocator: 4 CTAs of 128 threads per SM (up to 128 registers, no
// spills).  Measured within 2 % of each other: 3..6 CTAs of 128 threads, 3 CTAs of 256, 10 CTAs of 64.
#ifndef BNK_MIN_CTAS
#define BNK_MIN_CTAS 4
#endif
#ifndef BNK_WARPS_PER_CTA
#define BNK_WARPS_PER_CTA 4
#endif
constexpr int kWarpsPerCta = BNK_WARPS_PER_CTA;
constexpr int kThreads = kWarpsPerCta * 32;

// ---------------------------------------------------------------------------
// ChaCha20
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t rotl16(uint32_t x) { return __byte_perm(x, 0, 0x1032); }
__device__ __forceinline__ uint32_t rotl8(uint32_t x) { return __byte_perm(x, 0, 0x2103); }
__device__ __forceinline__ uint32_t rotl12(uint32_t x) { return __funnelshift_l(x, x, 12); }
__device__ __forceinline__ uint32_t rotl7(uint32_t x) { return __funnelshift_l(x, x, 7); }

// 12 instructions.  Exclusive-or, funnel shift and byte permute run on the ALU pipe only, at 64 lanes/clk/SM
// (two cycles per warp instruction per scheduler): 8 of them make a quarter round cost 16-17 cycles per warp,
// with the four additions riding along on the FMA pipe (the compiler already issues them there, so writing
// them as multiply-adds changes nothing).  The profiler agrees: issue slots 66 % busy, ALU pipe 75 %, top stall
// "math pipe throttle".  Moving a rotation to the multiplier (x * 2^n as a 64-bit product, low + high word) was
// measured too: each of the four rotations moved costs 9 % more time, the wide multiply being slower still.
#define BNK_QR(a, b, c, d) \
    a += b;                \
    d = rotl16(d ^ a);     \
    c += d;                \
    b = rotl12(b ^ c);     \
    a += b;                \
    d = rotl8(d ^ a);      \
    c += d;                \
    b = rotl7(b ^ c);

// One block: state = constants | key | block counter | 0 | counter lo | counter hi.
// (The first column round of columns 1, 2 and 3 reads constants, key and nonce only, so it is the same for every
// block of a packet.  Written out as a per-packet precomputation it compiles to the same register count as this
// form: the compiler already moves those 37 instructions out of the block loop.)
__device__ __forceinline__ void chacha20_block(uint32_t (&x)[16], const uint32_t (&k)[8], uint32_t blk,
                                               uint32_t n_lo, uint32_t n_hi) {
    x[0] = 0x61707865u;
    x[1] = 0x3320646eu;
    x[2] = 0x79622d32u;
    x[3] = 0x6b206574u;
#pragma unroll
    for (int i = 0; i < 8; i++) x[4 + i] = k[i];
    x[12] = blk;
    x[13] = 0u;
    x[14] = n_lo;
    x[15] = n_hi;
#pragma unroll
    for (int r = 0; r < 10; r++) {
        BNK_QR(x[0], x[4], x[8], x[12])
        BNK_QR(x[1], x[5], x[9], x[13])
        BNK_QR(x[2], x[6], x[10], x[14])
        BNK_QR(x[3], x[7], x[11], x[15])
        BNK_QR(x[0], x[5], x[10], x[15])
        BNK_QR(x[1], x[6], x[11], x[12])
        BNK_QR(x[2], x[7], x[8], x[13])
        BNK_QR(x[3], x[4], x[9], x[14])
    }
    x[0] += 0x61707865u;
    x[1] += 0x3320646eu;
    x[2] += 0x79622d32u;
    x[3] += 0x6b206574u;
#pragma unroll
    for (int i = 0; i < 8; i++) x[4 + i] += k[i];
    x[12] += blk;
    x[14] += n_lo;
    x[15] += n_hi;
}

// ---------------------------------------------------------------------------
// Poly1305, radix 2^32.  r is clamped so r1..r3 are multiples of 4 and
// s_i = r_i + r_i/4 = 5*r_i/4 folds the 2^128-and-above partial products back
// (2^130 = 5 mod p).  h4 stays below 8 between blocks.
// ---------------------------------------------------------------------------
struct Poly {
    uint32_t h0, h1, h2, h3, h4;
    uint32_t r0, r1, r2, r3;
    uint32_t s1, s2, s3;
};

__device__ __forceinline__ void poly_init(Poly &p, uint32_t k0, uint32_t k1, uint32_t k2, uint32_t k3) {
    p.h0 = p.h1 = p.h2 = p.h3 = p.h4 = 0;
    p.r0 = k0 & 0x0fffffffu;
    p.r1 = k1 & 0x0ffffffcu;
    p.r2 = k2 & 0x0ffffffcu;
    p.r3 = k3 & 0x0ffffffcu;
    p.s1 = p.r1 + (p.r1 >> 2);
    p.s2 = p.r2 + (p.r2 >> 2);
    p.s3 = p.r3 + (p.r3 >> 2);
}

// h = (h + m + 2^128) * r, partially reduced.
__device__ __forceinline__ void poly_block(Poly &p, uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
    uint32_t h0 = p.h0, h1 = p.h1, h2 = p.h2, h3 = p.h3, h4 = p.h4;
    asm("add.cc.u32 %0, %0, %5;\n\t"
        "addc.cc.u32 %1, %1, %6;\n\t"
        "addc.cc.u32 %2, %2, %7;\n\t"
        "addc.cc.u32 %3, %3, %8;\n\t"
        "addc.u32 %4, %4, 1;"
        : "+r"(h0), "+r"(h1), "+r"(h2), "+r"(h3), "+r"(h4)
        : "r"(m0), "r"(m1), "r"(m2), "r"(m3));
    uint64_t d0 = (uint64_t)h0 * p.r0 + (uint64_t)h1 * p.s3 + (uint64_t)h2 * p.s2 + (uint64_t)h3 * p.s1;
    uint64_t d1 = (uint64_t)h0 * p.r1 + (uint64_t)h1 * p.r0 + (uint64_t)h2 * p.s3 + (uint64_t)h3 * p.s2 +
                  (uint64_t)h4 * p.s1;
    uint64_t d2 = (uint64_t)h0 * p.r2 + (uint64_t)h1 * p.r1 + (uint64_t)h2 * p.r0 + (uint64_t)h3 * p.s3 +
                  (uint64_t)h4 * p.s2;
    uint64_t d3 = (uint64_t)h0 * p.r3 + (uint64_t)h1 * p.r2 + (uint64_t)h2 * p.r1 + (uint64_t)h3 * p.r0 +
                  (uint64_t)h4 * p.s3;
    uint32_t top = h4 * p.r0;
    d1 += d0 >> 32;
    d2 += d1 >> 32;
    d3 += d2 >> 32;
    top += (uint32_t)(d3 >> 32);
    // everything at or above 2^130 comes back multiplied by 5
    uint32_t c = (top >> 2) + (top & ~3u);
    h0 = (uint32_t)d0;
    h1 = (uint32_t)d1;
    h2 = (uint32_t)d2;
    h3 = (uint32_t)d3;
    h4 = top & 3u;
    asm("add.cc.u32 %0, %0, %5;\n\t"
        "addc.cc.u32 %1, %1, 0;\n\t"
        "addc.cc.u32 %2, %2, 0;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;"
        : "+r"(h0), "+r"(h1), "+r"(h2), "+r"(h3), "+r"(h4)
        : "r"(c));
    p.h0 = h0;
    p.h1 = h1;
    p.h2 = h2;
    p.h3 = h3;
    p.h4 = h4;
}

// tag = ((h mod p) + pad) mod 2^128
__device__ __forceinline__ void poly_finish(const Poly &p, const uint32_t (&pad)[4], uint32_t (&tag)[4]) {
    uint32_t h0 = p.h0, h1 = p.h1, h2 = p.h2, h3 = p.h3, h4 = p.h4;
    uint32_t c = (h4 >> 2) * 5u;
    h4 &= 3u;
    asm("add.cc.u32 %0, %0, %5;\n\t"
        "addc.cc.u32 %1, %1, 0;\n\t"
        "addc.cc.u32 %2, %2, 0;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;"
        : "+r"(h0), "+r"(h1), "+r"(h2), "+r"(h3), "+r"(h4)
        : "r"(c));
    // g = h + 5; h >= p exactly when g reaches 2^130, and then h mod p = g - 2^130
    uint32_t g0, g1, g2, g3, g4;
    asm("add.cc.u32 %0, %5, 5;\n\t"
        "addc.cc.u32 %1, %6, 0;\n\t"
        "addc.cc.u32 %2, %7, 0;\n\t"
        "addc.cc.u32 %3, %8, 0;\n\t"
        "addc.u32 %4, %9, 0;"
        : "=r"(g0), "=r"(g1), "=r"(g2), "=r"(g3), "=r"(g4)
        : "r"(h0), "r"(h1), "r"(h2), "r"(h3), "r"(h4));
    if (g4 >> 2) {
        h0 = g0;
        h1 = g1;
        h2 = g2;
        h3 = g3;
    }
    asm("add.cc.u32 %0, %4, %8;\n\t"
        "addc.cc.u32 %1, %5, %9;\n\t"
        "addc.cc.u32 %2, %6, %10;\n\t"
        "addc.u32 %3, %7, %11;"
        : "=r"(tag[0]), "=r"(tag[1]), "=r"(tag[2]), "=r"(tag[3])
        : "r"(h0), "r"(h1), "r"(h2), "r"(h3), "r"(pad[0]), "r"(pad[1]), "r"(pad[2]), "r"(pad[3]));
}

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------
// keep the first k bytes (little-endian) of a word; k may be <= 0 or >= 4
__device__ __forceinline__ uint32_t keep_bytes(uint32_t w, int k) {
    if (k >= 4) return w;
    if (k <= 0) return 0u;
    return w & ((1u << (8 * k)) - 1u);
}

// WireGuard padding: up to a multiple of 16, never beyond the MTU; a packet
// longer than the MTU is padded as if only its last MTU-sized unit counted.
__device__ __forceinline__ uint32_t wg_padded_len(uint32_t len, uint32_t mtu) {
    if (mtu == 0) return (len + 15u) & ~15u;
    uint32_t last = len > mtu ? len % mtu : len;
    uint32_t padded = (last + 15u) & ~15u;
    if (padded > mtu) padded = mtu;
    return len + (padded - last);
}

// ---------------------------------------------------------------------------
// Descriptor of one packet, validated.  `writer` says whether this thread records the
// outcome of a refused packet (one thread per packet does).
// ---------------------------------------------------------------------------
struct Desc {
    uint32_t off, body /* bytes under the cipher */, in_len /* bytes to fetch */, n_lo, n_hi, slot;
    bool live;
};

template <bool OPEN>
__device__ __forceinline__ Desc load_desc(const AeadArgs &a, uint32_t pkt, bool have, bool writer) {
    Desc d{0, 0, 0, 0, 0, 0, false};
    if (!have) return d;
    uint8_t st = BNK_PKT_OK;
    d.off = a.off[pkt];
    const uint32_t len = a.len[pkt];
    d.slot = a.slot[pkt];
    d.live = true;
    if ((d.off & 15u) || d.slot >= a.max_slots) {
        st = (OPEN && d.slot == kSlotNoKeypair) ? BNK_PKT_NO_KEYPAIR : BNK_PKT_BAD_DESC;
        d.live = false;
    } else if (!a.valid[d.slot]) {
        // never set, or cleared: the zeroed key of such a slot is public knowledge, so nothing is sealed
        // under it and nothing "authenticates" against it (wireguard-go drops traffic that has no keypair)
        st = BNK_PKT_NO_KEYPAIR;
        d.live = false;
    } else if (!OPEN) {
        d.body = wg_padded_len(len, a.mtu);
        d.in_len = len;
        const uint64_t ctr = a.counter[pkt];
        d.n_lo = (uint32_t)ctr;
        d.n_hi = (uint32_t)(ctr >> 32);
        if ((uint64_t)d.off + BNK_WG_HEADER + d.body + BNK_WG_TAG > a.ring_bytes || d.body < len) {
            st = BNK_PKT_BAD_DESC;
            d.live = false;
        } else if (ctr >= BNK_REJECT_AFTER_MESSAGES) {
            st = BNK_PKT_COUNTER_EXHAUSTED;
            d.live = false;
        }
    } else {
        if ((uint64_t)d.off + len > a.ring_bytes) {
            st = BNK_PKT_BAD_DESC;
            d.live = false;
        } else if (len < BNK_WG_HEADER + BNK_WG_TAG) {
            st = BNK_PKT_MALFORMED;
            d.live = false;
        } else {
            const uint4 hdr = *reinterpret_cast<const uint4 *>(a.ring + d.off);
            d.n_lo = hdr.z;
            d.n_hi = hdr.w;
            if (writer) a.counter[pkt] = ((uint64_t)hdr.w << 32) | hdr.z;
            if (hdr.x != 4u) {
                st = BNK_PKT_MALFORMED;
                d.live = false;
            } else {
                d.body = len - (BNK_WG_HEADER + BNK_WG_TAG);
                d.in_len = d.body;
            }
        }
    }
    if (!d.live) {
        if (writer) {
            a.status[pkt] = st;
            a.out_len[pkt] = 0;
        }
        d.body = 0;
        d.in_len = 0;
    }
    return d;
}

// ---------------------------------------------------------------------------
// Kernel 1, thread per packet.  OPEN=false: seal in place.  OPEN=true: authenticate + decrypt in place.
// The throughput kernel: used when the batch is large enough to fill the GPU with one packet per thread.
// ---------------------------------------------------------------------------
template <bool OPEN>
__global__ void __launch_bounds__(kThreads, BNK_MIN_CTAS) aead_kernel(const AeadArgs a) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t idx = blockIdx.x * kThreads + threadIdx.x;
    const bool have = idx < a.n;
    const uint32_t pkt = have ? (a.order ? a.order[idx] : idx) : 0u;
    const Desc dsc = load_desc<OPEN>(a, pkt, have, true);
    const uint32_t off = dsc.off, body = dsc.body, in_len = dsc.in_len, n_lo = dsc.n_lo, n_hi = dsc.n_hi, slot = dsc.slot;
    const bool live = dsc.live;
    const uint32_t nblk = (body + 63u) >> 6;
    uint8_t *const data = a.ring + (size_t)off + BNK_WG_HEADER; // 16-byte aligned

    uint32_t key[8];
    Poly poly;
    uint32_t pad[4] = {0, 0, 0, 0};
    if (live) {
        const uint4 *kp = reinterpret_cast<const uint4 *>(a.keys + (size_t)slot * 8);
        const uint4 ka = kp[0], kb = kp[1];
        key[0] = ka.x; key[1] = ka.y; key[2] = ka.z; key[3] = ka.w;
        key[4] = kb.x; key[5] = kb.y; key[6] = kb.z; key[7] = kb.w;
        uint32_t x[16];
        chacha20_block(x, key, 0u, n_lo, n_hi); // block 0 = one-time Poly1305 key
        poly_init(poly, x[0], x[1], x[2], x[3]);
        pad[0] = x[4]; pad[1] = x[5]; pad[2] = x[6]; pad[3] = x[7];
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) key[i] = 0;
        poly_init(poly, 0, 0, 0, 0);
    }

    // (Splitting off a branch-free loop over the whole blocks so that the Poly1305 multiplies can be scheduled
    // into the ChaCha20 rounds of the same thread, with the seal side absorbing the previous block's ciphertext,
    // was measured: no gain for seal, 10 % slower for open.  The warps of an SM already overlap the two phases.
    // Measured again on 1,048,576 x 1420 B with the comparisons peeled off the whole-block loop: seal 1.279 ms
    // against 1.276, open 1.383 against 1.261.  Feeding each Poly1305 column's carry into the next column's
    // first multiply-add instead of three 64-bit additions: seal 1.256, open 1.276: within the run-to-run spread.)
    for (uint32_t b = 0; b < nblk; b++) {
        const uint32_t base = b * 64u;
        uint32_t d[16];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint4 v = make_uint4(0, 0, 0, 0);
            // a chunk that starts inside the input is read whole: the bytes past in_len lie in the packet's own
            // padding / tag room and are masked below
            if (base + 16u * c < in_len) v = *reinterpret_cast<const uint4 *>(data + base + 16u * c);
            d[4 * c + 0] = v.x; d[4 * c + 1] = v.y; d[4 * c + 2] = v.z; d[4 * c + 3] = v.w;
        }
        uint32_t x[16];
        chacha20_block(x, key, b + 1u, n_lo, n_hi);
        if (base + 64u <= in_len) {
            // whole block of real bytes
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t o0 = d[4 * c + 0] ^ x[4 * c + 0], o1 = d[4 * c + 1] ^ x[4 * c + 1];
                const uint32_t o2 = d[4 * c + 2] ^ x[4 * c + 2], o3 = d[4 * c + 3] ^ x[4 * c + 3];
                if (OPEN) poly_block(poly, d[4 * c + 0], d[4 * c + 1], d[4 * c + 2], d[4 * c + 3]);
                else poly_block(poly, o0, o1, o2, o3);
                *reinterpret_cast<uint4 *>(data + base + 16u * c) = make_uint4(o0, o1, o2, o3);
            }
        } else {
            // ragged end: bytes past in_len are zero padding (seal) and bytes past body do not exist
            const int in_left = (int)in_len - (int)base;
            const int body_left = (int)body - (int)base;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[4], m[4];
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const int k = 16 * c + 4 * w;
                    const uint32_t in_w = keep_bytes(d[4 * c + w], in_left - k);
                    o[w] = keep_bytes(in_w ^ x[4 * c + w], body_left - k);
                    m[w] = OPEN ? in_w : o[w];
                }
                if (16 * c < body_left) poly_block(poly, m[0], m[1], m[2], m[3]);
                if (16 * c + 16 <= body_left) {
                    *reinterpret_cast<uint4 *>(data + base + 16u * c) = make_uint4(o[0], o[1], o[2], o[3]);
                } else if (16 * c < body_left) {
                    // last, partial chunk: byte stores
                    uint8_t *dst = data + base + 16u * c;
                    const int tail = body_left - 16 * c;
#pragma unroll
                    for (int k = 0; k < 15; k++)
                        if (k < tail) dst[k] = (uint8_t)(o[k >> 2] >> (8 * (k & 3)));
                }
            }
        }
    }

    if (!live) return;

    // ---- length block and tag ----
    // le64(aad_len = 0) | le64(body), with the 2^128 bit like every other block
    poly_block(poly, 0u, 0u, body, 0u);
    uint32_t tag[4];
    poly_finish(poly, pad, tag);
    uint8_t *tagp = data + body;

    if (!OPEN) {
        *reinterpret_cast<uint4 *>(a.ring + off) = make_uint4(4u, a.remote_index[slot], n_lo, n_hi);
        if ((body & 3u) == 0) {
            uint32_t *t32 = reinterpret_cast<uint32_t *>(tagp);
            t32[0] = tag[0]; t32[1] = tag[1]; t32[2] = tag[2]; t32[3] = tag[3];
        } else {
#pragma unroll
            for (int w = 0; w < 4; w++)
#pragma unroll
                for (int k = 0; k < 4; k++) tagp[4 * w + k] = (uint8_t)(tag[w] >> (8 * k));
        }
        a.status[pkt] = BNK_PKT_OK;
        a.out_len[pkt] = BNK_WG_HEADER + body + BNK_WG_TAG;
    } else {
        uint32_t diff = 0;
        if ((body & 3u) == 0) {
            const uint32_t *t32 = reinterpret_cast<const uint32_t *>(tagp);
            diff = (t32[0] ^ tag[0]) | (t32[1] ^ tag[1]) | (t32[2] ^ tag[2]) | (t32[3] ^ tag[3]);
        } else {
#pragma unroll
            for (int w = 0; w < 4; w++)
#pragma unroll
                for (int k = 0; k < 4; k++) diff |= (uint32_t)(tagp[4 * w + k] ^ (uint8_t)(tag[w] >> (8 * k)));
        }
        if (diff == 0) {
            a.status[pkt] = body ? BNK_PKT_OK : BNK_PKT_KEEPALIVE;
            a.out_len[pkt] = body;
        } else {
            // forged or damaged: no plaintext may leave, wipe what the fused pass wrote
            uint8_t *dst = data;
            uint32_t k = 0;
            for (; k + 16u <= body; k += 16u) *reinterpret_cast<uint4 *>(dst + k) = make_uint4(0, 0, 0, 0);
            for (; k < body; k++) dst[k] = 0;
            a.status[pkt] = BNK_PKT_AUTH_FAIL;
            a.out_len[pkt] = 0;
        }
    }
}

// ---------------------------------------------------------------------------
// Poly1305 in radix 2^26 with both factors arbitrary: the warp-per-packet kernel multiplies by powers
// of r, which are not clamped, so the 5/4 trick of the radix-2^32 code above does not apply.
// Limbs of a product are below 2^26 (limb 1 may carry a few extra units); sums of two such values are
// valid left factors.
// ---------------------------------------------------------------------------
struct P26 {
    uint32_t v[5];
};
constexpr uint32_t kM26 = 0x3ffffffu;

__device__ __forceinline__ P26 p26_zero() { return P26{{0, 0, 0, 0, 0}}; }
__device__ __forceinline__ P26 p26_words(uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3, uint32_t hibit) {
    P26 m;
    m.v[0] = t0 & kM26;
    m.v[1] = ((t0 >> 26) | (t1 << 6)) & kM26;
    m.v[2] = ((t1 >> 20) | (t2 << 12)) & kM26;
    m.v[3] = ((t2 >> 14) | (t3 << 18)) & kM26;
    m.v[4] = (t3 >> 8) | (hibit << 24);
    return m;
}
__device__ __forceinline__ P26 p26_add(const P26 &x, const P26 &y) {
    P26 o;
#pragma unroll
    for (int i = 0; i < 5; i++) o.v[i] = x.v[i] + y.v[i];
    return o;
}
__device__ __forceinline__ P26 p26_mul(const P26 &x, const P26 &y) {
    const uint32_t s1 = y.v[1] * 5u, s2 = y.v[2] * 5u, s3 = y.v[3] * 5u, s4 = y.v[4] * 5u; // 2^130 = 5 (mod p)
    uint64_t d0 = (uint64_t)x.v[0] * y.v[0] + (uint64_t)x.v[1] * s4 + (uint64_t)x.v[2] * s3 + (uint64_t)x.v[3] * s2 +
                  (uint64_t)x.v[4] * s1;
    uint64_t d1 = (uint64_t)x.v[0] * y.v[1] + (uint64_t)x.v[1] * y.v[0] + (uint64_t)x.v[2] * s4 + (uint64_t)x.v[3] * s3 +
                  (uint64_t)x.v[4] * s2;
    uint64_t d2 = (uint64_t)x.v[0] * y.v[2] + (uint64_t)x.v[1] * y.v[1] + (uint64_t)x.v[2] * y.v[0] + (uint64_t)x.v[3] * s4 +
                  (uint64_t)x.v[4] * s3;
    uint64_t d3 = (uint64_t)x.v[0] * y.v[3] + (uint64_t)x.v[1] * y.v[2] + (uint64_t)x.v[2] * y.v[1] + (uint64_t)x.v[3] * y.v[0] +
                  (uint64_t)x.v[4] * s4;
    uint64_t d4 = (uint64_t)x.v[0] * y.v[4] + (uint64_t)x.v[1] * y.v[3] + (uint64_t)x.v[2] * y.v[2] + (uint64_t)x.v[3] * y.v[1] +
                  (uint64_t)x.v[4] * y.v[0];
    P26 o;
    d1 += d0 >> 26;
    d2 += d1 >> 26;
    d3 += d2 >> 26;
    d4 += d3 >> 26;
    const uint64_t t = (d0 & kM26) + (d4 >> 26) * 5u;
    o.v[0] = (uint32_t)t & kM26;
    o.v[1] = ((uint32_t)d1 & kM26) + (uint32_t)(t >> 26);
    o.v[2] = (uint32_t)d2 & kM26;
    o.v[3] = (uint32_t)d3 & kM26;
    o.v[4] = (uint32_t)d4 & kM26;
    return o;
}
__device__ __forceinline__ P26 p26_shfl(const P26 &x, int src) {
    P26 o;
#pragma unroll
    for (int i = 0; i < 5; i++) o.v[i] = __shfl_sync(0xffffffffu, x.v[i], src);
    return o;
}
__device__ __forceinline__ P26 p26_shfl_up(const P26 &x, int delta) {
    P26 o;
#pragma unroll
    for (int i = 0; i < 5; i++) o.v[i] = __shfl_up_sync(0xffffffffu, x.v[i], delta);
    return o;
}
// tag = ((h mod p) + pad) mod 2^128
__device__ __forceinline__ void p26_finish(const P26 &x, const uint32_t (&pad)[4], uint32_t (&tag)[4]) {
    uint32_t h0 = x.v[0], h1 = x.v[1], h2 = x.v[2], h3 = x.v[3], h4 = x.v[4], c;
    c = h1 >> 26; h1 &= kM26; h2 += c;
    c = h2 >> 26; h2 &= kM26; h3 += c;
    c = h3 >> 26; h3 &= kM26; h4 += c;
    c = h4 >> 26; h4 &= kM26; h0 += c * 5u;
    c = h0 >> 26; h0 &= kM26; h1 += c;
    // g = h + 5 - 2^130; g is non-negative exactly when h >= p
    uint32_t g0 = h0 + 5u; c = g0 >> 26; g0 &= kM26;
    uint32_t g1 = h1 + c;  c = g1 >> 26; g1 &= kM26;
    uint32_t g2 = h2 + c;  c = g2 >> 26; g2 &= kM26;
    uint32_t g3 = h3 + c;  c = g3 >> 26; g3 &= kM26;
    const uint32_t g4 = h4 + c - (1u << 26);
    if (!(g4 >> 31)) {
        h0 = g0; h1 = g1; h2 = g2; h3 = g3; h4 = g4;
    }
    const uint32_t w0 = h0 | (h1 << 26), w1 = (h1 >> 6) | (h2 << 20), w2 = (h2 >> 12) | (h3 << 14),
                   w3 = (h3 >> 18) | (h4 << 8);
    asm("add.cc.u32 %0, %4, %8;\n\t"
        "addc.cc.u32 %1, %5, %9;\n\t"
        "addc.cc.u32 %2, %6, %10;\n\t"
        "addc.u32 %3, %7, %11;"
        : "=r"(tag[0]), "=r"(tag[1]), "=r"(tag[2]), "=r"(tag[3])
        : "r"(w0), "r"(w1), "r"(w2), "r"(w3), "r"(pad[0]), "r"(pad[1]), "r"(pad[2]), "r"(pad[3]));
}

// ---------------------------------------------------------------------------
// Kernel 2, warp per packet: the latency kernel for batches too small to fill the GPU with one
// packet per thread (a 128-packet batch takes ~24 sequential cipher blocks per thread there).
// Lane j of a round takes one 64-byte chunk: its ChaCha20 block and the Poly1305 Horner steps over
// its four 16-byte blocks starting from zero, Q_j = sum_s b_s r^(5-s).  The chunks of a round, up
// to 30, sit right-aligned in lanes 31-F..30; lane 30-F carries the running state in; a binary
// tree over the warp (five shuffle + multiply steps with r^4, r^8, ... r^64) folds them to
//   state' = state * r^(4F) + sum_j Q_j * r^(4(F-1-j))
// on lane 30.  Lane 31 then continues sequentially over what is left of the packet (up to three whole
// blocks and a ragged one) and the length block, and makes the tag.  Block 0 of the keystream (the
// one-time Poly1305 key) is computed by the carry lane of the first round in the same pass as the data
// blocks.  Accesses are coalesced by construction: consecutive lanes hold consecutive 64 bytes.
// ---------------------------------------------------------------------------
constexpr uint32_t kWppFull = 30;

template <bool OPEN>
__global__ void __launch_bounds__(128) aead_wpp_kernel(const AeadArgs a) {
    let_next_kernel_start();    // open side: the grouping + replay launch behind may take its place already
    wait_for_kernel_in_front(); // seal side: the counters come from the grouping launch in front
    __shared__ uint4 stage_all[4][128]; // per warp: the 16-byte pieces of one round (up to 30 chunks of 64 bytes)
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (idx >= a.n) return; // a whole warp at a time
    const uint32_t pkt = a.order ? a.order[idx] : idx;
    const Desc dsc = load_desc<OPEN>(a, pkt, true, lane == 0);
    if (!dsc.live) return;
    const uint32_t body = dsc.body, in_len = dsc.in_len;
    uint8_t *const data = a.ring + (size_t)dsc.off + BNK_WG_HEADER;

    uint32_t key[8];
    {
        const uint4 *kp = reinterpret_cast<const uint4 *>(a.keys + (size_t)dsc.slot * 8);
        const uint4 ka = kp[0], kb = kp[1];
        key[0] = ka.x; key[1] = ka.y; key[2] = ka.z; key[3] = ka.w;
        key[4] = kb.x; key[5] = kb.y; key[6] = kb.z; key[7] = kb.w;
    }
    const uint32_t full_total = body >> 6, tail_bytes = body & 63u;
    P26 r = p26_zero(), state = p26_zero();
    uint32_t pad[4] = {0, 0, 0, 0};
    uint32_t ct[16]; // the lane's ciphertext words of the current round (lane 31: the ragged tail)
#pragma unroll
    for (int i = 0; i < 16; i++) ct[i] = 0;

    uint32_t done = 0;
    bool first = true, last_round;
    do {
        const uint32_t remaining = full_total - done;
        last_round = remaining <= kWppFull;
        const uint32_t F = last_round ? remaining : kWppFull;
        const bool is_chunk = lane + F >= 31u && lane <= 30u;
        const bool is_carry = lane + F == 30u;
        const bool is_tail = last_round && lane == 31u && tail_bytes != 0;
        const bool works = is_chunk || is_tail;
        const uint32_t chunk = is_tail ? full_total : done + (lane + F - 31u);
        const uint32_t base = chunk * 64u;

        // The round's F chunks are 64 F consecutive bytes.  The warp fetches them as 16-byte pieces in piece order
        // (lane l takes pieces l, 32 + l, ...: every load instruction covers 512 consecutive bytes) and hands each
        // chunk lane its four pieces through shared memory.  Fetched chunk by chunk instead, a load instruction
        // touches thirty-two separate 16-byte pieces 64 bytes apart: the same bytes from device memory, but when the
        // ring is the caller's pinned host memory (small batches run there, no copies) every piece is a PCIe read
        // of its own, and few of those can be in flight.
        const uint32_t round_base = done * 64u;
        uint4 *const stage = stage_all[threadIdx.x >> 5];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint32_t q = 32u * c + lane;
            if (q < 4u * F) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (round_base + 16u * q < in_len) v = *reinterpret_cast<const uint4 *>(data + round_base + 16u * q);
                stage[q] = v;
            }
        }
        __syncwarp();
        uint32_t d[16];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (is_chunk) v = stage[4u * (chunk - done) + c];
            else if (is_tail && base + 16u * c < in_len) v = *reinterpret_cast<const uint4 *>(data + base + 16u * c);
            d[4 * c + 0] = v.x; d[4 * c + 1] = v.y; d[4 * c + 2] = v.z; d[4 * c + 3] = v.w;
        }
        __syncwarp(); // the pieces are read: the stage may take the output
        uint32_t x[16];
        chacha20_block(x, key, works ? chunk + 1u : 0u, dsc.n_lo, dsc.n_hi); // idle lanes and the carry lane: block 0
        if (first) {
            const int src = 30 - (int)F; // the carry lane holds block 0
            const uint32_t k0 = __shfl_sync(0xffffffffu, x[0], src), k1 = __shfl_sync(0xffffffffu, x[1], src);
            const uint32_t k2 = __shfl_sync(0xffffffffu, x[2], src), k3 = __shfl_sync(0xffffffffu, x[3], src);
            r = p26_words(k0 & 0x0fffffffu, k1 & 0x0ffffffcu, k2 & 0x0ffffffcu, k3 & 0x0ffffffcu, 0u);
#pragma unroll
            for (int i = 0; i < 4; i++) pad[i] = __shfl_sync(0xffffffffu, x[4 + i], src);
        }
        if (works) {
            const int in_left = (int)in_len - (int)base;
            const int body_left = (int)body - (int)base;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[4];
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const int k = 16 * c + 4 * w;
                    const uint32_t in_w = keep_bytes(d[4 * c + w], in_left - k);
                    o[w] = keep_bytes(in_w ^ x[4 * c + w], body_left - k);
                    ct[4 * c + w] = OPEN ? in_w : o[w];
                }
                if (is_chunk) { // a whole chunk lies inside the body: out through the stage, in piece order
                    stage[4u * (chunk - done) + c] = make_uint4(o[0], o[1], o[2], o[3]);
                } else if (16 * c + 16 <= body_left) {
                    *reinterpret_cast<uint4 *>(data + base + 16u * c) = make_uint4(o[0], o[1], o[2], o[3]);
                } else if (16 * c < body_left) {
                    uint8_t *dst = data + base + 16u * c;
                    const int tail = body_left - 16 * c;
#pragma unroll
                    for (int k = 0; k < 15; k++)
                        if (k < tail) dst[k] = (uint8_t)(o[k >> 2] >> (8 * (k & 3)));
                }
            }
        }
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint32_t q = 32u * c + lane;
            if (q < 4u * F) *reinterpret_cast<uint4 *>(data + round_base + 16u * q) = stage[q];
        }
        __syncwarp(); // before the next round writes the stage
        // Horner over the lane's own four blocks (chunk lanes), or the state carried in (carry lane)
        P26 V = p26_zero();
        if (is_chunk) {
#pragma unroll
            for (int c = 0; c < 4; c++)
                V = p26_mul(p26_add(V, p26_words(ct[4 * c], ct[4 * c + 1], ct[4 * c + 2], ct[4 * c + 3], 1u)), r);
        }
        if (is_carry) V = state;
        // fold lanes 0..30 (tree positions 1..31) with r^4, r^8, ..., r^64
        P26 pw = p26_mul(r, r);
        pw = p26_mul(pw, pw);
#pragma unroll
        for (int k = 0; k < 5; k++) {
            P26 left = p26_shfl_up(V, 1 << k);
            if (lane < (1u << k)) left = p26_zero();
            const P26 t = p26_add(p26_mul(left, pw), V);
            const uint32_t mask = (2u << k) - 1u;
            if (((lane + 1u) & mask) == mask && lane != 31u) V = t;
            if (k < 4) pw = p26_mul(pw, pw);
        }
        state = p26_shfl(V, 30);
        done += F;
        first = false;
    } while (!last_round);

    // lane 31: the blocks behind the last whole chunk, the length block, the tag
    uint32_t verdict = 0; // open: 1 = tag mismatch
    if (lane == 31u) {
        P26 h = state;
        const uint32_t nb = (tail_bytes + 15u) >> 4;
#pragma unroll
        for (int c = 0; c < 4; c++)
            if ((uint32_t)c < nb) h = p26_mul(p26_add(h, p26_words(ct[4 * c], ct[4 * c + 1], ct[4 * c + 2], ct[4 * c + 3], 1u)), r);
        h = p26_mul(p26_add(h, p26_words(0u, 0u, body, 0u, 1u)), r); // le64(0) | le64(body)
        uint32_t tag[4];
        p26_finish(h, pad, tag);
        uint8_t *tagp = data + body;
        if (!OPEN) {
#pragma unroll
            for (int w = 0; w < 4; w++)
#pragma unroll
                for (int k = 0; k < 4; k++) tagp[4 * w + k] = (uint8_t)(tag[w] >> (8 * k));
        } else {
            uint32_t diff = 0;
#pragma unroll
            for (int w = 0; w < 4; w++)
#pragma unroll
                for (int k = 0; k < 4; k++) diff |= (uint32_t)(tagp[4 * w + k] ^ (uint8_t)(tag[w] >> (8 * k)));
            verdict = diff != 0;
        }
    }
    if (!OPEN) {
        if (lane == 0) {
            *reinterpret_cast<uint4 *>(a.ring + dsc.off) = make_uint4(4u, a.remote_index[dsc.slot], dsc.n_lo, dsc.n_hi);
            a.status[pkt] = BNK_PKT_OK;
            a.out_len[pkt] = BNK_WG_HEADER + body + BNK_WG_TAG;
        }
    } else {
        verdict = __shfl_sync(0xffffffffu, verdict, 31);
        if (verdict) { // forged or damaged: wipe what the fused pass wrote
            for (uint32_t k = lane * 16u; k + 16u <= body; k += 512u) *reinterpret_cast<uint4 *>(data + k) = make_uint4(0, 0, 0, 0);
            if (lane == 0)
                for (uint32_t k = body & ~15u; k < body; k++) data[k] = 0;
        }
        if (lane == 0) {
            a.status[pkt] = verdict ? BNK_PKT_AUTH_FAIL : (body ? BNK_PKT_OK : BNK_PKT_KEEPALIVE);
            a.out_len[pkt] = verdict ? 0u : body;
        }
    }
}

// Below this many packets one-packet-per-thread leaves most of the GPU idle and its run time is that of one thread
// walking one packet (~39 us for 1420 B) whatever the batch size; one warp per packet takes ~13 us up to 2,400
// packets and then grows by ~14 us per 2,400 more.  Measured crossover on B200: between 6,000 and 7,000 packets.
#ifndef BNK_WPP_MAX_PACKETS
#define BNK_WPP_MAX_PACKETS 6144u
#endif

template <bool OPEN>
cudaError_t launch_aead(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) {
    if (a.n == 0) return cudaSuccess;
    const bool wpp = ctx->aead_mode == 2 || (ctx->aead_mode == 0 && a.n <= BNK_WPP_MAX_PACKETS);
    if (wpp) {
        const uint32_t ctas = (a.n + 3) / 4; // 4 warps = 4 packets per CTA
        cudaError_t e = launch_after_kernel(aead_wpp_kernel<OPEN>, dim3(ctas), dim3(128), s, a);
        if (e != cudaSuccess) return e;
    } else {
        // one CTA per 128 packets; the hardware hands CTAs to SMs as slots free up, which measured faster
        // than persistent warps with an even static share of the packets
        const uint32_t ctas = (a.n + kThreads - 1) / kThreads;
        launch_kernel(a.n <= dependent_launch_up_to(), aead_kernel<OPEN>, dim3(ctas), dim3(kThreads), s, a);
    }
    ++ctx->launches;
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_seal(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) { return launch_aead<false>(a, s, ctx); }
cudaError_t launch_open(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) { return launch_aead<true>(a, s, ctx); }
