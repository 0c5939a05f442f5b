"""Pins the CPU checker's AEAD and transport framing against independent RFC 8439 implementations
(OpenSSL via `cryptography`, libsodium via PyNaCl) and against the committed golden vectors."""
import hashlib
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "aead_golden.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def test_golden_aead_vectors(oracle, golden):
    for v in golden["aead"]:
        key, nonce, aad = bytes.fromhex(v["key"]), bytes.fromhex(v["nonce"]), bytes.fromhex(v["aad"])
        pt, ct = bytes.fromhex(v["pt"]), bytes.fromhex(v["ct"])
        assert oracle.aead_seal(key, nonce, pt, aad) == ct
        assert oracle.aead_open(key, nonce, ct, aad) == pt
        if ct:
            bad = bytearray(ct)
            bad[len(bad) // 2] ^= 0x10
            assert oracle.aead_open(key, nonce, bytes(bad), aad) is None


def test_against_openssl_and_libsodium_live(oracle):
    nacl = pytest.importorskip("nacl.bindings")
    aead = pytest.importorskip("cryptography.hazmat.primitives.ciphers.aead")
    rng = np.random.default_rng(2024)
    for length in list(range(0, 70)) + [127, 128, 129, 575, 576, 1419, 1420, 1424, 4097, 65503]:
        key = rng.integers(0, 256, 32, dtype=np.uint8).tobytes()
        nonce = bytes(4) + rng.integers(0, 256, 8, dtype=np.uint8).tobytes()
        pt = rng.integers(0, 256, length, dtype=np.uint8).tobytes()
        want = aead.ChaCha20Poly1305(key).encrypt(nonce, pt, b"")
        assert want == nacl.crypto_aead_chacha20poly1305_ietf_encrypt(pt, b"", nonce, key)
        assert oracle.aead_seal(key, nonce, pt) == want


def test_poly1305_carry_edge_cases(oracle):
    """Inputs that force the wrap-around paths of the MAC: all-ones blocks and an r that is all ones after clamping."""
    aead = pytest.importorskip("cryptography.hazmat.primitives.poly1305")
    for key in [bytes([0xFF] * 32), bytes([0xFF] * 16) + bytes(16), bytes(16) + bytes([0xFF] * 16),
                bytes([2] + [0] * 15 + [0xFF] * 16)]:
        for msg in [bytes([0xFF] * n) for n in (16, 32, 48, 64, 15, 17, 160)] + [bytes(64), b""]:
            want = aead.Poly1305.generate_tag(key, msg)
            assert oracle.poly1305(key, msg) == want


def test_config1_messages_match_golden(oracle, golden):
    from bnk_b200 import gen

    w = gen.config1()
    assert hashlib.sha256(b"".join(w.payloads)).hexdigest() == golden["config1"]["plaintext_sha256"]
    msgs = [oracle.wg_seal(w.keys[0].tobytes(), 1, int(w.counter[i]), w.payloads[i], 1420) for i in range(128)]
    assert all(len(m) == 1452 for m in msgs)
    assert msgs[0].hex() == golden["config1"]["first"]
    assert msgs[-1].hex() == golden["config1"]["last"]
    assert hashlib.sha256(b"".join(msgs)).hexdigest() == golden["config1"]["sha256"]
    st, pt, ctr, rx = oracle.wg_open(w.keys[0].tobytes(), msgs[5])
    assert (st, pt, ctr, rx) == (oracle.OK, w.payloads[5], 5, 1)


def test_config2_messages_match_golden(oracle, golden):
    from bnk_b200 import gen

    w = gen.config2()
    b = w.base
    assert len(b.payloads) == golden["config2"]["n_base"] and len(w.arrival) == golden["config2"]["n_arrivals"] == 4096
    assert hashlib.sha256(w.arrival.astype("<i8").tobytes()).hexdigest() == golden["config2"]["arrival_sha256"]
    msgs = [oracle.wg_seal(b.keys[int(b.peer[i])].tobytes(), int(b.remote_index[int(b.peer[i])]), int(b.counter[i]),
                           b.payloads[i], 1420) for i in range(len(b.payloads))]
    assert hashlib.sha256(b"".join(msgs)).hexdigest() == golden["config2"]["sha256"]


def test_transport_framing_and_padding(oracle):
    key = bytes(range(32))
    m = oracle.wg_seal(key, 0xAABBCCDD, 0x0102030405060708, b"hello", 1420)
    assert m[:4] == b"\x04\x00\x00\x00" and m[4:8] == bytes.fromhex("ddccbbaa") and m[8:16] == bytes.fromhex("0807060504030201")
    assert len(m) == 16 + 16 + 16  # 5 bytes padded to 16
    st, pt, ctr, rx = oracle.wg_open(key, m)
    assert st == oracle.OK and pt == b"hello" + bytes(11) and ctr == 0x0102030405060708 and rx == 0xAABBCCDD
    # keepalive: empty payload, authenticated
    k = oracle.wg_seal(key, 1, 9, b"", 1420)
    assert len(k) == 32 and oracle.wg_open(key, k)[0] == oracle.KEEPALIVE
    # padding never goes beyond the MTU; beyond-MTU packets pad their last MTU-sized unit only
    assert [oracle.wg_padded_len(n, 1420) for n in (0, 1, 16, 17, 1408, 1409, 1419, 1420)] == [0, 16, 16, 32, 1408, 1420, 1420, 1420]
    assert oracle.wg_padded_len(1421, 1420) == 1436 and oracle.wg_padded_len(2840, 1420) == 2840
    assert oracle.wg_padded_len(1419, 0) == 1424
    # malformed: wrong type, too short; exhausted counter refuses to seal
    assert oracle.wg_open(key, b"\x01" + m[1:])[0] == oracle.MALFORMED
    assert oracle.wg_open(key, m[:31])[0] == oracle.MALFORMED
    assert oracle.wg_seal(key, 1, oracle.REJECT_AFTER_MESSAGES, b"x", 1420) == b""
    assert len(oracle.wg_seal(key, 1, oracle.REJECT_AFTER_MESSAGES - 1, b"x", 1420)) == 48


def test_inner_check_rules(oracle):
    from bnk_b200 import gen

    ip = gen.ip4(100, 64, 0, 9)
    pkt = bytes(gen.ipv4_header(6, ip, gen.ip4(100, 64, 0, 1), 40)) + bytes(20) + bytes(8)  # 8 bytes of padding behind it
    assert oracle.inner_check(pkt, ip) == 40                      # cut to the total-length field
    assert oracle.inner_check(pkt[:40], ip) == 40
    assert oracle.inner_check(pkt[:39], ip) is None               # claims more than there is
    assert oracle.inner_check(pkt, ip + 1) is None                # not this peer's address
    assert oracle.inner_check(pkt, 0) is None                     # peer without an allowed address
    assert oracle.inner_check(bytes([0x60]) + pkt[1:], ip) is None  # IPv6 nibble: the reference hands out IPv4 only
    short = bytearray(pkt)
    short[2:4] = (19).to_bytes(2, "big")
    assert oracle.inner_check(bytes(short), ip) is None           # shorter than an IPv4 header
    assert oracle.inner_check(pkt[:19], ip) is None
