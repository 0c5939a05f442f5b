// Receive-side bookkeeping around the open kernel, one thread per packet:
//  - demux: receiver index in the transport header -> keypair slot (the lookup wireguard-go's receive
//    routine does in its index table before it hands a message to a decryption worker);
//  - inner check: what its sequential receiver does with an authenticated, fresh plaintext before the
//    TUN write: IPv4 only here (the reference gives peers one IPv4 /32 each, internal/dataplane/engine.go:294),
//    20 <= total-length field <= decrypted length, cut to the total length, source address must be the
//    sending peer's allowed address.
#include "bnk_internal.cuh"

namespace {

__global__ void demux_index_kernel(KeypairTables kt, const uint8_t *ring, const uint32_t *off, const uint32_t *len,
                                   uint32_t *slot, uint32_t n, uint64_t ring_bytes) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t o = off[i], l = len[i];
    if ((o & 15u) || (uint64_t)o + l > ring_bytes || l < BNK_WG_HEADER + BNK_WG_TAG) {
        slot[i] = 0; // the open kernel reports BAD_DESC / MALFORMED for these on its own
        return;
    }
    const uint32_t index = *reinterpret_cast<const uint32_t *>(ring + o + 4);
    const uint64_t key = (1ull << 32) | index;
    uint32_t found = kSlotNoKeypair;
    if (kt.index_slots) {
        uint32_t h = index_hash(index) & (kt.index_slots - 1);
        for (uint32_t probe = 0; probe < kt.index_slots; probe++) {
            const uint64_t k = kt.index_keys[h];
            if (k == 0) break;
            if (k == key) {
                found = kt.index_vals[h];
                break;
            }
            h = (h + 1) & (kt.index_slots - 1);
        }
    }
    slot[i] = found;
}

__global__ void inner_check_kernel(KeypairTables kt, const uint8_t *ring, const uint32_t *off, const uint32_t *slot,
                                   uint32_t *out_len, uint8_t *status, uint32_t n) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n || status[i] != BNK_PKT_OK) return;
    const uint8_t *p = ring + off[i] + BNK_WG_HEADER; // 16-byte aligned
    const uint32_t l = out_len[i];
    bool ok = false;
    if (l >= 20) {
        const uint4 w = *reinterpret_cast<const uint4 *>(p);
        if (((w.x & 0xffu) >> 4) == 4u) {
            const uint32_t total = ((w.x >> 8) & 0xff00u) | (w.x >> 24); // bytes 2,3 big-endian
            const uint32_t src = __byte_perm(w.w, 0, 0x0123);
            if (total >= 20 && total <= l && src == kt.allowed_ip[slot[i]] && src != 0) {
                out_len[i] = total;
                ok = true;
            }
        }
    }
    if (!ok) status[i] = BNK_PKT_BAD_INNER;
}

// Bind.classify, internal/magicsock/bind.go:207-228
__global__ void classify_kernel(KeypairTables kt, const uint8_t *ring, const uint32_t *off, const uint32_t *len,
                                const uint8_t *src_addr, uint32_t *slot, uint8_t *status, uint32_t n,
                                uint64_t ring_bytes) {
    let_next_kernel_start();
    wait_for_kernel_in_front();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t o = off[i], l = len[i];
    if ((o & 15u) || (uint64_t)o + l > ring_bytes) {
        status[i] = BNK_PKT_BAD_DESC;
        return;
    }
    const uint8_t *p = ring + o;
    uint4 w = make_uint4(0, 0, 0, 0);
    if (l >= 16) {
        w = *reinterpret_cast<const uint4 *>(p);
    } else { // short datagram: whole words as far as they go, the rest zero
        const uint32_t *p32 = reinterpret_cast<const uint32_t *>(p);
        if (l >= 4) w.x = p32[0];
        if (l >= 8) w.y = p32[1];
        if (l >= 12) w.z = p32[2];
        else if (l >= 10) w.z = (uint32_t)p[8] | ((uint32_t)p[9] << 8);
    }
    // disco.IsDisco: "bnk\0disco\0", 10 bytes
    if (l >= 10 && w.x == 0x006b6e62u /* b n k \0 */ && w.y == 0x63736964u /* d i s c */ &&
        (w.z & 0xffffu) == 0x006fu /* o \0 */) {
        status[i] = BNK_CLASS_DISCO;
        return;
    }
    // isSTUN: RFC 5389 shape
    if (l >= 20 && ((w.x & 0xffu) >> 6) == 0 && w.y == 0x42a41221u) {
        status[i] = BNK_CLASS_STUN;
        return;
    }
    // byAddr[normalize(src)]
    const uint8_t *sa = src_addr + (size_t)i * BNK_SRC_ADDR_STRIDE;
    const uint32_t *s32 = reinterpret_cast<const uint32_t *>(sa); // stride 20 keeps 4-byte alignment
    const uint64_t hi = (uint64_t)s32[0] | ((uint64_t)s32[1] << 32), lo = (uint64_t)s32[2] | ((uint64_t)s32[3] << 32);
    const uint32_t port = ((uint32_t)sa[16] << 8) | sa[17];
    uint8_t cls = BNK_CLASS_STRANGER;
    if (kt.addr_slots) {
        uint32_t h = addr_hash(hi, lo, port) & (kt.addr_slots - 1);
        for (uint32_t probe = 0; probe < kt.addr_slots; probe++) {
            const KeypairTables::AddrEntry e = kt.addr_tab[h];
            if (e.port == 0) break;
            if (e.port == (port | (1u << 16)) && e.hi == hi && e.lo == lo) {
                slot[i] = e.peer;
                cls = BNK_CLASS_WIREGUARD;
                break;
            }
            h = (h + 1) & (kt.addr_slots - 1);
        }
    }
    status[i] = cls;
}

} // namespace

cudaError_t launch_classify(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_kernel(n <= dependent_launch_up_to(), classify_kernel, dim3((n + 255) / 256), dim3(256), s, b->ctx->kt,
        b->dev.ring, b->dev.off, b->dev.len, b->dev.src_addr, b->dev.slot, b->dev.status, n, b->ring_bytes);
    ++b->ctx->launches;
    return cudaGetLastError();
}

cudaError_t launch_demux_index(bnk_batch *b, uint32_t n, const uint32_t *len, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_kernel(n <= dependent_launch_up_to(), demux_index_kernel, dim3((n + 255) / 256), dim3(256), s, b->ctx->kt,
        b->dev.ring, b->dev.off, len, b->dev.slot, n, b->ring_bytes);
    ++b->ctx->launches;
    return cudaGetLastError();
}

cudaError_t launch_inner_check(bnk_batch *b, uint32_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    launch_kernel(n <= dependent_launch_up_to(), inner_check_kernel, dim3((n + 255) / 256), dim3(256), s, b->ctx->kt,
        b->dev.ring, b->dev.off, b->dev.slot, b->dev.out_len, b->dev.status, n);
    ++b->ctx->launches;
    return cudaGetLastError();
}
