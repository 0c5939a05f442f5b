// Segmentation of TCP / UDP super-packets (IPv4) into MTU-sized packets, one warp per segment.
//
// Behaviour follows the split wireguard-go's Linux TUN code applies to a read that carries a virtio-net
// header (restated from its documented behaviour, golang.zx2c4.com/wireguard is not in the reference tree):
//   - every segment starts with the super-packet's IP header and transport header;
//   - IPv4: identification = first id + segment number, total length = header + segment payload,
//     header checksum recomputed;
//   - TCP: sequence number = first + segment number * gso_size, FIN and PSH survive on the last segment only;
//   - UDP: length = transport header + segment payload;
//   - transport checksum recomputed over pseudo header + transport header + payload.
// The work is a copy with a running one's-complement sum: HBM-bound, ~2 x segment bytes of traffic.
#include "bnk_internal.cuh"

namespace {

__device__ __forceinline__ uint32_t be16(const uint8_t *p) { return ((uint32_t)p[0] << 8) | p[1]; }

// one's-complement sum of big-endian 16-bit words, folded to 16 bits
__device__ __forceinline__ uint32_t fold16(uint64_t s) {
    s = (s & 0xffffffffull) + (s >> 32);
    s = (s & 0xffffffffull) + (s >> 32);
    uint32_t t = (uint32_t)s;
    t = (t & 0xffffu) + (t >> 16);
    t = (t & 0xffffu) + (t >> 16);
    return t;
}

__global__ void __launch_bounds__(256) gso_split_kernel(const bnk_gso_super *supers, uint32_t n_super, uint8_t *ring,
                                                        const uint32_t *off, const uint32_t *len, uint32_t *slot,
                                                        uint32_t n_pkts, uint64_t ring_bytes, const uint32_t *seg_super) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_pkts) return;
    const uint32_t pkt = warp;
    const uint32_t j = seg_super[pkt];
    if (j >= n_super) return; // not a segment of any super-packet: left alone
    const bnk_gso_super sp = supers[j];
    const uint32_t k = pkt - sp.first_pkt;
    const uint32_t hdr = sp.hdr_len, iph = sp.csum_start;
    const uint32_t data_at = hdr + k * sp.gso_size;
    bool ok = (sp.proto == 6 || sp.proto == 17) && iph >= 20 && hdr > iph && sp.gso_size > 0 && data_at < sp.src_len &&
              (sp.src_off & 3u) == 0 && (uint64_t)sp.src_off + sp.src_len <= ring_bytes &&
              sp.csum_offset + 2u <= hdr - iph && hdr - iph >= (sp.proto == 6 ? 20u : 8u) && ((hdr | iph) & 3u) == 0 &&
              (sp.csum_offset & 1u) == 0 && hdr <= 128u; // one header word per lane
    uint32_t seg_len = 0, total = 0;
    const uint32_t o = off[pkt];
    if (ok) {
        seg_len = min((uint32_t)sp.gso_size, sp.src_len - data_at);
        total = hdr + seg_len;
        ok = len[pkt] == total && (o & 15u) == 0 && (uint64_t)o + 16 + total + 32 <= ring_bytes && total <= 65535u;
    }
    if (!ok) {
        if (lane == 0) slot[pkt] = 0xffffffffu; // the seal that follows reports BNK_PKT_BAD_DESC for it
        return;
    }
    const uint8_t *in = ring + sp.src_off;
    uint8_t *out = ring + o + BNK_WG_HEADER;
    const bool last = data_at + seg_len == sp.src_len;

    // Headers: lane i takes header word i (IPv4 header and transport header are multiples of 4 bytes and together
    // at most 30 words), patches the field it holds and contributes its word to the IPv4 sum or to the transport
    // sum (source and destination address count for both: pseudo header).  The sums meet in the reductions below.
    const uint32_t ipw = iph >> 2, hw = hdr >> 2;
    uint64_t ip_sum = 0;  // IPv4 header, checksum field zero
    uint64_t hdr_sum = 0; // transport header + pseudo header, checksum field zero
    if (lane < hw) {
        uint32_t w = reinterpret_cast<const uint32_t *>(in)[lane];
        if (lane < ipw) {
            // words 0 (ver/ihl/tos/total length), 1 (id/flags/frag), 2 (ttl/proto/checksum), 3 src, 4 dst, options
            if (lane == 0) w = (w & 0x0000ffffu) | ((total >> 8) << 16) | ((total & 0xffu) << 24);
            else if (lane == 1) {
                const uint32_t id = (((w & 0xffu) << 8) | ((w >> 8) & 0xffu)) + k; // big-endian field in a little-endian word
                w = (w & 0xffff0000u) | ((id >> 8) & 0xffu) | ((id & 0xffu) << 8);
            } else if (lane == 2) w &= 0x0000ffffu; // checksum field cleared; lane 0 fills it in below
            ip_sum = (uint64_t)__byte_perm(w, 0, 0x4401) + (uint64_t)__byte_perm(w, 0, 0x4423);
            if (lane == 3 || lane == 4) hdr_sum = ip_sum;
        } else {
            const uint32_t t = lane - ipw;
            if (sp.proto == 6) {
                if (t == 1) {
                    const uint32_t seq = __byte_perm(w, 0, 0x0123) + k * sp.gso_size;
                    w = __byte_perm(seq, 0, 0x0123);
                } else if (t == 3 && !last) {
                    w &= ~(0x09u << 8); // flags are byte 13: FIN | PSH survive on the last segment only
                }
            } else if (t == 1) {
                const uint32_t ulen = hdr - iph + seg_len;
                w = (w & 0xffff0000u) | (ulen >> 8) | ((ulen & 0xffu) << 8);
            }
            if (t == (sp.csum_offset >> 2)) w &= (sp.csum_offset & 2u) ? 0x0000ffffu : 0xffff0000u; // checksum field cleared
            hdr_sum = (uint64_t)__byte_perm(w, 0, 0x4401) + (uint64_t)__byte_perm(w, 0, 0x4423);
        }
        reinterpret_cast<uint32_t *>(out)[lane] = w;
    }
    if (lane == 0) hdr_sum += sp.proto + (hdr - iph + seg_len);

    // payload copy + sum.  Payload byte i sits at transport offset (hdr - iph + i): when that is odd the
    // 16-bit words straddle, so sum bytes with their parity weight instead.
    const uint8_t *src = in + data_at;
    uint8_t *dst = out + hdr;
    const uint32_t parity = (hdr - iph) & 1u;
    uint64_t sum = 0;    // of big-endian 16-bit words
    uint64_t le_sum = 0; // of the payload words as loaded (little-endian): the one's-complement sum commutes with the
                         // byte swap (RFC 1071, 2(B)), so the words are added raw and the folded sum is swapped once
    if ((((uintptr_t)src | (uintptr_t)dst) & 3u) == 0 && parity == 0) {
        const uint32_t words = seg_len >> 2;
        const uint32_t *s32 = reinterpret_cast<const uint32_t *>(src);
        uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
        // several loads in flight per lane: the copy is latency-bound otherwise.  (Writing the destination in
        // aligned 16-byte chunks assembled from two aligned source lines was measured: 17 % slower.)
        constexpr uint32_t kInFlight = 4; // 2, 4 and 11 measure the same within noise
        uint32_t i = lane;
        for (; i + 32u * (kInFlight - 1) < words; i += 32u * kInFlight) {
            uint32_t w[kInFlight];
#pragma unroll
            for (uint32_t u = 0; u < kInFlight; u++) w[u] = s32[i + 32u * u];
#pragma unroll
            for (uint32_t u = 0; u < kInFlight; u++) {
                d32[i + 32u * u] = w[u];
                le_sum += w[u];
            }
        }
        for (; i < words; i += 32) {
            const uint32_t w = s32[i];
            d32[i] = w;
            le_sum += w;
        }
        for (uint32_t i = (words << 2) + lane; i < seg_len; i += 32) {
            const uint8_t v = src[i];
            dst[i] = v;
            sum += (i & 1u) ? v : ((uint32_t)v << 8);
        }
    } else {
        for (uint32_t i = lane; i < seg_len; i += 32) {
            const uint8_t v = src[i];
            dst[i] = v;
            sum += ((i + parity) & 1u) ? v : ((uint32_t)v << 8);
        }
    }
    le_sum = (le_sum & 0xffffffffull) + (le_sum >> 32); // 33 bits: 32 lanes of them still fit
    sum += hdr_sum; // both in 16-bit big-endian words
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, d);
        le_sum += __shfl_xor_sync(0xffffffffu, le_sum, d);
        ip_sum += __shfl_xor_sync(0xffffffffu, ip_sum, d);
    }
    __syncwarp(); // the header words are in place before lane 0 writes the checksum bytes into them
    if (lane == 0) {
        const uint32_t ipc = ~fold16(ip_sum) & 0xffffu;
        out[10] = (uint8_t)(ipc >> 8);
        out[11] = (uint8_t)ipc;
        const uint32_t le = fold16(le_sum);
        const uint32_t c = ~fold16(sum + (((le & 0xffu) << 8) | (le >> 8))) & 0xffffu;
        out[iph + sp.csum_offset] = (uint8_t)(c >> 8);
        out[iph + sp.csum_offset + 1] = (uint8_t)c;
    }
}

// segment -> super-packet index (n_super for packets that belong to none)
__global__ void gso_map_kernel(const bnk_gso_super *supers, uint32_t n_super, uint32_t n_pkts, uint32_t *seg_super) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_super) return;
    const bnk_gso_super sp = supers[j];
    for (uint32_t k = 0; k < sp.n_pkts; k++)
        if (sp.first_pkt + k < n_pkts) seg_super[sp.first_pkt + k] = j;
}

__global__ void fill_u32_kernel(uint32_t *p, uint32_t n, uint32_t v) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

} // namespace

cudaError_t launch_gso_split(bnk_batch *b, uint32_t n_super, uint32_t n_pkts, cudaStream_t s) {
    if (n_pkts == 0 || n_super == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    uint32_t *seg_super = d.order_tmp; // grouping scratch is idle here
    launch_kernel(n_pkts <= dependent_launch_up_to(), fill_u32_kernel, dim3((n_pkts + 255) / 256), dim3(256), s,
        seg_super, n_pkts, n_super);
    launch_kernel(n_pkts <= dependent_launch_up_to(), gso_map_kernel, dim3((n_super + 127) / 128), dim3(128), s, d.gso,
        n_super, n_pkts, seg_super);
    launch_kernel(n_pkts <= dependent_launch_up_to(), gso_split_kernel, dim3((n_pkts + 7) / 8), dim3(256), s, d.gso,
        n_super, d.ring, d.off, d.len, d.slot, n_pkts, b->ring_bytes, seg_super);
    b->ctx->launches += 3;
    return cudaGetLastError();
}
