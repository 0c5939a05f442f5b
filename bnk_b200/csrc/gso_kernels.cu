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
              sp.csum_offset + 2u <= hdr - iph && hdr - iph >= (sp.proto == 6 ? 20u : 8u);
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

    // headers: copied and patched by lane 0 (at most 120 bytes), payload by the whole warp
    if (lane == 0) {
        for (uint32_t i = 0; i < hdr; i++) out[i] = in[i];
        uint32_t id = be16(in + 4) + k;
        out[4] = (uint8_t)(id >> 8);
        out[5] = (uint8_t)id;
        out[2] = (uint8_t)(total >> 8);
        out[3] = (uint8_t)total;
        out[10] = 0;
        out[11] = 0;
        uint64_t s = 0;
        for (uint32_t i = 0; i < iph; i += 2) s += be16(out + i);
        const uint32_t c = ~fold16(s) & 0xffffu;
        out[10] = (uint8_t)(c >> 8);
        out[11] = (uint8_t)c;
        uint8_t *t = out + iph;
        if (sp.proto == 6) {
            const uint32_t seq = (((uint32_t)in[iph + 4] << 24) | ((uint32_t)in[iph + 5] << 16) | ((uint32_t)in[iph + 6] << 8) |
                                  in[iph + 7]) + k * sp.gso_size;
            t[4] = (uint8_t)(seq >> 24);
            t[5] = (uint8_t)(seq >> 16);
            t[6] = (uint8_t)(seq >> 8);
            t[7] = (uint8_t)seq;
            if (!last) t[13] &= (uint8_t)~(0x01u | 0x08u); // FIN, PSH
        } else {
            const uint32_t ulen = hdr - iph + seg_len;
            t[4] = (uint8_t)(ulen >> 8);
            t[5] = (uint8_t)ulen;
        }
        t[sp.csum_offset] = 0;
        t[sp.csum_offset + 1] = 0;
    }
    __syncwarp();

    // payload copy + sum.  Payload byte i sits at transport offset (hdr - iph + i): when that is odd the
    // 16-bit words straddle, so sum bytes with their parity weight instead.
    const uint8_t *src = in + data_at;
    uint8_t *dst = out + hdr;
    const uint32_t parity = (hdr - iph) & 1u;
    uint64_t sum = 0;
    if ((((uintptr_t)src | (uintptr_t)dst) & 3u) == 0 && parity == 0) {
        const uint32_t words = seg_len >> 2;
        const uint32_t *s32 = reinterpret_cast<const uint32_t *>(src);
        uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
        for (uint32_t i = lane; i < words; i += 32) {
            const uint32_t w = s32[i];
            d32[i] = w;
            // little-endian load of bytes b0 b1 b2 b3 -> big-endian words b0b1 + b2b3
            sum += (uint64_t)__byte_perm(w, 0, 0x4401) + (uint64_t)__byte_perm(w, 0, 0x4423);
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
#pragma unroll
    for (int d = 16; d; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0) {
        const uint8_t *t = out + iph;
        const uint32_t tlen = hdr - iph + seg_len;
        // pseudo header: source, destination, protocol, transport length
        uint64_t s = sum + be16(out + 12) + be16(out + 14) + be16(out + 16) + be16(out + 18) + sp.proto + tlen;
        const uint32_t th = hdr - iph;
        for (uint32_t i = 0; i + 1 < th; i += 2) s += be16(t + i);
        if (th & 1u) s += (uint32_t)t[th - 1] << 8;
        const uint32_t c = ~fold16(s) & 0xffffu;
        out[iph + sp.csum_offset] = (uint8_t)(c >> 8);
        out[iph + sp.csum_offset + 1] = (uint8_t)c;
    }
}

// segment -> super-packet index (n_super for packets that belong to none)
__global__ void gso_map_kernel(const bnk_gso_super *supers, uint32_t n_super, uint32_t n_pkts, uint32_t *seg_super) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_super) return;
    const bnk_gso_super sp = supers[j];
    for (uint32_t k = 0; k < sp.n_pkts; k++)
        if (sp.first_pkt + k < n_pkts) seg_super[sp.first_pkt + k] = j;
}

__global__ void fill_u32_kernel(uint32_t *p, uint32_t n, uint32_t v) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

} // namespace

cudaError_t launch_gso_split(bnk_batch *b, uint32_t n_super, uint32_t n_pkts, cudaStream_t s) {
    if (n_pkts == 0 || n_super == 0) return cudaSuccess;
    DeviceBatch &d = b->dev;
    uint32_t *seg_super = d.order_tmp; // grouping scratch is idle here
    fill_u32_kernel<<<(n_pkts + 255) / 256, 256, 0, s>>>(seg_super, n_pkts, n_super);
    gso_map_kernel<<<(n_super + 127) / 128, 128, 0, s>>>(d.gso, n_super, n_pkts, seg_super);
    gso_split_kernel<<<(n_pkts + 7) / 8, 256, 0, s>>>(d.gso, n_super, d.ring, d.off, d.len, d.slot, n_pkts, b->ring_bytes,
                                                     seg_super);
    b->ctx->launches += 3;
    return cudaGetLastError();
}
