"""Generates the golden vectors under tests/golden/.  The AEAD vectors and the sealed messages of
configurations 1, 2 and 5 come from implementations that are independent of this repository: OpenSSL
(through the `cryptography` package) and libsodium (through PyNaCl).  Configuration 3 (filter verdicts) and
the segment bytes of configuration 5 have no independent implementation in this container: their digests are
taken from the CPU checker under oracle/ (itself pinned to the reference's own test cases) and serve as a
regression pin for checker and generator together.

Run from the repository root:  python tests/golden/make_golden.py
The output is committed; the tests only read it.  Inputs come from the seeded generators in
bnk_b200/gen.py, so the file is reproducible bit for bit.
"""
import hashlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import nacl.bindings as sodium  # noqa: E402
from cryptography.hazmat.primitives.ciphers.aead import ChaCha20Poly1305  # noqa: E402

from bnk_b200 import gen  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def wg_message(key: bytes, receiver: int, counter: int, pt: bytes, padded_len: int) -> bytes:
    """WireGuard transport-data message built from a library AEAD (whitepaper 5.4.6)."""
    nonce = bytes(4) + counter.to_bytes(8, "little")
    body = pt + bytes(padded_len - len(pt))
    a = ChaCha20Poly1305(key).encrypt(nonce, body, b"")
    b = sodium.crypto_aead_chacha20poly1305_ietf_encrypt(body, b"", nonce, key)
    assert a == b, "OpenSSL and libsodium disagree"
    return (4).to_bytes(4, "little") + receiver.to_bytes(4, "little") + counter.to_bytes(8, "little") + a


def padded(n: int, mtu: int) -> int:
    if mtu == 0:
        return (n + 15) & ~15
    last = n % mtu if n > mtu else n
    p = min((last + 15) & ~15, mtu)
    return n + (p - last)


SEC = 1_000_000_000


def filter_and_gso_digests():
    import numpy as np

    from oracle import oracle as O

    out = {}
    # (d) configuration 3 at a size the scalar checker walks in a second: digests of the generated tables and
    # headers, and of the checker's verdicts at t0 + 1 s, of the late replies at t0 + 10 min and again at t0 + 2 s
    w = gen.config3(500, 2000, 6000, 20000)
    f = O.Filter()
    f.set_rules_arrays(w.rules.astype(O.RULE_DTYPE), w.srcs.astype(O.PREFIX_DTYPE), w.ports.astype(O.PORT_DTYPE))
    f.note_batch(np.ascontiguousarray(w.outbound), 28, w.outbound_len, w.t0_ns)
    v1 = f.check_batch(np.ascontiguousarray(w.inbound), 28, np.ascontiguousarray(w.inbound_len), w.t0_ns + SEC)
    v2 = f.check_batch(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 600 * SEC)
    v3 = f.check_batch(np.ascontiguousarray(w.late), 28, w.late_len, w.t0_ns + 2 * SEC)
    sha = lambda *arrays: hashlib.sha256(b"".join(np.ascontiguousarray(a).tobytes() for a in arrays)).hexdigest()
    out["config3"] = {"sizes": [500, 2000, 6000, 20000],
                      "tables_sha256": sha(w.rules, w.srcs, w.ports),
                      "headers_sha256": sha(w.outbound, w.outbound_len, w.inbound, w.inbound_len, w.late, w.late_len),
                      "verdicts_sha256": sha(v1.astype(np.uint8), v2.astype(np.uint8), v3.astype(np.uint8)),
                      "allowed": [int(v1.sum()), int(v2.sum()), int(v3.sum())], "flows": int(f.flow_count),
                      "source": "oracle/ (CPU checker)"}
    # (e) configuration 5, eight super-packets: the checker's segments, each then sealed by the library AEAD with
    # the peer's key and consecutive counters per peer in batch order
    w5 = gen.config5(n_super=8)
    segs, msgs, nxt = [], [], {}
    for j, sp in enumerate(w5.supers):
        parts = O.gso_split(sp, w5.hdr_len, w5.mss, w5.csum_start, w5.csum_offset, 6)
        assert parts is not None and len(parts) == 47
        p = int(w5.peer[j])
        for seg in parts:
            c = nxt.get(p, 0)
            nxt[p] = c + 1
            segs.append(seg)
            msgs.append(wg_message(w5.keys[p].tobytes(), p + 1, c, seg, padded(len(seg), 1420)))
    out["config5"] = {"n_super": 8, "supers_sha256": hashlib.sha256(b"".join(w5.supers)).hexdigest(),
                      "segments_sha256": hashlib.sha256(b"".join(segs)).hexdigest(),
                      "sealed_sha256": hashlib.sha256(b"".join(msgs)).hexdigest(),
                      "peers": [int(x) for x in w5.peer],
                      "source": "segments: oracle/ (CPU checker); sealing: cryptography + PyNaCl; remote index = peer + 1"}
    out.update(full_size_digests())
    return out


def full_size_digests():
    """Configurations 4 and 5 at the sizes BASELINE.json states.  Too large for per-message Python calls into two
    libraries, so the sealing is done by OpenSSL's EVP_chacha20_poly1305 called from C on every core
    (oracle/cpu_baseline.c, independent of the scalar checker and of the CUDA path); configuration 5's segments
    come from the checker's split as above."""
    import numpy as np

    from oracle import oracle as O

    out = {}
    threads = O.host_cores()
    # configuration 4: 1,048,576 x 1420 B over 65,536 peers, 16 sequential counters per peer, remote index = peer
    n, peers, size = 1 << 20, 1 << 16, 1420
    plan = gen.config4(n, peers, size)
    stride = plan.stride
    ring = gen.splitmix_fill(plan.payload_seed, n * stride)
    i = np.arange(n, dtype=np.uint64)
    off = (i * np.uint64(stride)).astype(np.uint32)
    keys = gen.bulk_keys(plan)
    _, st, ol = O.cpu_aead_batch(False, threads, keys, np.arange(peers, dtype=np.uint32), size, ring, off,
                                 np.full(n, size, np.uint32), (i % np.uint64(peers)).astype(np.uint32), i // np.uint64(peers))
    assert (st == 0).all() and (ol == size + 32).all()
    msgs = np.ascontiguousarray(ring.reshape(n, stride)[:, :size + 32])
    out["config4_full"] = {"packets": n, "peers": peers, "payload": size,
                           "sealed_sha256": hashlib.sha256(msgs).hexdigest(),
                           "source": "OpenSSL EVP_chacha20_poly1305 from C (oracle/cpu_baseline.c); messages concatenated "
                                     "in packet order, remote index = peer, counter = packet // peers"}
    del ring, msgs
    # configuration 5: 2,048 super-packets -> 96,256 segments, Zipf(1.1) over 10,000 peers, remote index = 0x1000 + peer
    w5 = gen.config5(n_super=2048)
    segs, seg_peer = [], []
    for j, sp in enumerate(w5.supers):
        parts = O.gso_split(sp, w5.hdr_len, w5.mss, w5.csum_start, w5.csum_offset, 6)
        assert parts is not None and len(parts) == 47
        segs.extend(parts)
        seg_peer.extend([int(w5.peer[j])] * 47)
    m = len(segs)
    stride = 1456
    ring = np.zeros(m * stride, np.uint8)
    view = ring.reshape(m, stride)
    view[:, 16:16 + 1420] = np.frombuffer(b"".join(segs), np.uint8).reshape(m, 1420)
    seg_peer = np.array(seg_peer, np.uint32)
    counter = np.zeros(m, np.uint64)
    nxt = {}
    for k, pr in enumerate(seg_peer.tolist()):
        counter[k] = nxt.get(pr, 0)
        nxt[pr] = int(counter[k]) + 1
    _, st, ol = O.cpu_aead_batch(False, threads, w5.keys, (0x1000 + np.arange(len(w5.keys))).astype(np.uint32), 1420, ring,
                                 (np.arange(m, dtype=np.uint64) * stride).astype(np.uint32), np.full(m, 1420, np.uint32),
                                 seg_peer, counter)
    assert (st == 0).all() and (ol == 1452).all()
    out["config5_full"] = {"n_super": 2048, "segments": m,
                           "supers_sha256": hashlib.sha256(b"".join(w5.supers)).hexdigest(),
                           "segments_sha256": hashlib.sha256(b"".join(segs)).hexdigest(),
                           "sealed_sha256": hashlib.sha256(np.ascontiguousarray(view[:, :1452])).hexdigest(),
                           "source": "segments: oracle/ (CPU checker); sealing: OpenSSL EVP from C (oracle/cpu_baseline.c); "
                                     "remote index = 0x1000 + peer, counters consecutive per peer in batch order"}
    return out


def main():
    out = {"source": "cryptography (OpenSSL) cross-checked with PyNaCl (libsodium)", "aead": [], "config1": {},
           "config2": {}}
    # (a) small known-answer vectors, WireGuard nonce layout, lengths around every boundary
    g = gen.SplitMix64(0xB2000000 + 0xA)
    for length in [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 576, 1280, 1420]:
        key = g.bytes(32).tobytes()
        counter = int(g.u64(1)[0])
        aad = g.bytes(int(g.one_below(3)) * 7).tobytes()
        pt = g.bytes(length).tobytes()
        nonce = bytes(4) + counter.to_bytes(8, "little")
        ct = ChaCha20Poly1305(key).encrypt(nonce, pt, aad)
        assert ct == sodium.crypto_aead_chacha20poly1305_ietf_encrypt(pt, aad, nonce, key)
        out["aead"].append({"key": key.hex(), "nonce": nonce.hex(), "aad": aad.hex(), "pt": pt.hex(), "ct": ct.hex()})
    # (b) configuration 1: digest of all 128 sealed messages + the first and last in full
    w = gen.config1()
    msgs = [wg_message(w.keys[0].tobytes(), 1, int(w.counter[i]), w.payloads[i], padded(1420, 1420)) for i in range(128)]
    out["config1"] = {"sha256": hashlib.sha256(b"".join(msgs)).hexdigest(), "first": msgs[0].hex(), "last": msgs[-1].hex(),
                      "plaintext_sha256": hashlib.sha256(b"".join(w.payloads)).hexdigest()}
    # (c) configuration 2: digest of the distinct sealed messages in send order
    w2 = gen.config2()
    b = w2.base
    msgs2 = [wg_message(b.keys[int(b.peer[i])].tobytes(), int(b.remote_index[int(b.peer[i])]), int(b.counter[i]),
                        b.payloads[i], padded(int(b.length[i]), 1420)) for i in range(len(b.payloads))]
    out["config2"] = {"sha256": hashlib.sha256(b"".join(msgs2)).hexdigest(), "n_base": len(msgs2),
                      "n_arrivals": int(len(w2.arrival)),
                      "arrival_sha256": hashlib.sha256(w2.arrival.astype("<i8").tobytes()).hexdigest()}
    out.update(filter_and_gso_digests())
    with open(os.path.join(HERE, "aead_golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote aead_golden.json:", len(out["aead"]), "vectors")


if __name__ == "__main__":
    main()
