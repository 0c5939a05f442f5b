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

// 12 instructions; the four rotations issue at half rate on sm_100 (byte permute and funnel shift
// both measure 64 lanes/clk/SM), which makes a quarter round cost ~17 issue cycles per warp.
// Issuing the additions as multiply-adds on the FMA pipe was measured and does not help: the
// issue slots, not the ALU pipe, are what runs out.
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
// The kernel.  OPEN=false: seal in place.  OPEN=true: authenticate + decrypt in place.
// ---------------------------------------------------------------------------
template <bool OPEN>
__global__ void __launch_bounds__(kThreads, BNK_MIN_CTAS) aead_kernel(const AeadArgs a) {
    const uint32_t idx = blockIdx.x * kThreads + threadIdx.x;
    const bool have = idx < a.n;
    const uint32_t pkt = have ? (a.order ? a.order[idx] : idx) : 0u;

    // ---- descriptor ----
    uint32_t off = 0, body = 0 /* bytes under the cipher */, in_len = 0 /* bytes to fetch */;
    uint32_t n_lo = 0, n_hi = 0, slot = 0;
    uint8_t st = BNK_PKT_OK;
    bool live = false;
    if (have) {
        off = a.off[pkt];
        const uint32_t len = a.len[pkt];
        slot = a.slot[pkt];
        live = true;
        if ((off & 15u) || slot >= a.max_slots) {
            st = (OPEN && slot == kSlotNoKeypair) ? BNK_PKT_NO_KEYPAIR : BNK_PKT_BAD_DESC;
            live = false;
        } else if (!OPEN) {
            body = wg_padded_len(len, a.mtu);
            in_len = len;
            const uint64_t ctr = a.counter[pkt];
            n_lo = (uint32_t)ctr;
            n_hi = (uint32_t)(ctr >> 32);
            if ((uint64_t)off + BNK_WG_HEADER + body + BNK_WG_TAG > a.ring_bytes || body < len) {
                st = BNK_PKT_BAD_DESC;
                live = false;
            } else if (ctr >= BNK_REJECT_AFTER_MESSAGES) {
                st = BNK_PKT_COUNTER_EXHAUSTED;
                live = false;
            }
        } else {
            if ((uint64_t)off + len > a.ring_bytes) {
                st = BNK_PKT_BAD_DESC;
                live = false;
            } else if (len < BNK_WG_HEADER + BNK_WG_TAG) {
                st = BNK_PKT_MALFORMED;
                live = false;
            } else {
                const uint4 hdr = *reinterpret_cast<const uint4 *>(a.ring + off);
                n_lo = hdr.z;
                n_hi = hdr.w;
                a.counter[pkt] = ((uint64_t)hdr.w << 32) | hdr.z;
                if (hdr.x != 4u) {
                    st = BNK_PKT_MALFORMED;
                    live = false;
                } else {
                    body = len - (BNK_WG_HEADER + BNK_WG_TAG);
                    in_len = body;
                }
            }
        }
        if (!live) {
            a.status[pkt] = st;
            a.out_len[pkt] = 0;
            body = 0;
            in_len = 0;
        }
    }
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

// One warp per 32 packets, one CTA per 128.  The hardware hands CTAs to SMs as slots free up, which
// measured faster here than persistent warps with an even static share of the packets.
template <bool OPEN>
cudaError_t launch_aead(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) {
    if (a.n == 0) return cudaSuccess;
    const uint32_t ctas = (a.n + kThreads - 1) / kThreads;
    aead_kernel<OPEN><<<ctas, kThreads, 0, s>>>(a);
    ++ctx->launches;
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_seal(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) { return launch_aead<false>(a, s, ctx); }
cudaError_t launch_open(const AeadArgs &a, cudaStream_t s, bnk_ctx *ctx) { return launch_aead<true>(a, s, ctx); }
