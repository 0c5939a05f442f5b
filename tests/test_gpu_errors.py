"""Error behaviour of the C ABI: bad arguments come back as codes with a message, nothing aborts, and without a
GPU there is nothing to fall back to."""
import ctypes as C

import numpy as np
import pytest


def test_without_a_gpu_context_creation_fails_loudly():
    """No CPU fallback: on a machine without a usable CUDA device the library refuses to create a context."""
    from bnk_b200 import _lib

    L = _lib.lib()
    if L.bnk_device_count() > 0:
        pytest.skip("a GPU is present")
    cfg = _lib.Cfg(C.sizeof(_lib.Cfg), 0, 16, 128, 1420, 0, 0, 0)
    h = C.c_void_p()
    assert L.bnk_ctx_create(C.byref(cfg), C.byref(h)) == _lib.ECUDA
    assert not h.value
    assert b"no usable CUDA device" in L.bnk_last_error_string(None)
    with pytest.raises(_lib.BnkError):
        from bnk_b200 import Context

        Context()


@pytest.mark.gpu
def test_bad_arguments_are_codes_not_crashes(gpu_lib):
    from bnk_b200 import Context, _lib
    from bnk_b200.device import ACL_TUPLE_DTYPE

    L = gpu_lib
    h = C.c_void_p()

    def create(**kw):
        base = dict(struct_size=C.sizeof(_lib.Cfg), device_id=0, max_keypairs=16, replay_ring_blocks=128, mtu=1420,
                    flow_capacity=1 << 10, max_acl_tuples=0, reserved=0)
        base.update(kw)
        cfg = _lib.Cfg(*[base[f] for f, _ in _lib.Cfg._fields_])
        return L.bnk_ctx_create(C.byref(cfg), C.byref(h))

    assert create(struct_size=8) == _lib.EINVAL
    assert create(replay_ring_blocks=100) == _lib.EINVAL      # not a power of two
    assert create(replay_ring_blocks=1) == _lib.EINVAL
    assert create(flow_capacity=1000) == _lib.EINVAL
    assert create(max_keypairs=0) == _lib.EINVAL
    assert create(device_id=99) == _lib.EINVAL
    assert L.bnk_ctx_create(None, C.byref(h)) == _lib.EINVAL
    assert L.bnk_strerror(_lib.EBUSY) == b"batch busy" and L.bnk_strerror(-99) == b"unknown error"

    with Context(max_keypairs=16, flow_capacity=1 << 10, max_acl_tuples=4) as c:
        bh = C.c_void_p()
        assert L.bnk_batch_create(c._h, 8, 1000, C.byref(bh)) == _lib.EINVAL       # ring not a multiple of 16
        assert L.bnk_batch_create(c._h, 0, 1024, C.byref(bh)) == _lib.EINVAL
        assert L.bnk_batch_create(c._h, 8, 1 << 33, C.byref(bh)) == _lib.EINVAL    # above 4 GiB
        assert b"4 GiB" in L.bnk_last_error_string(c._h)
        key = bytes(32)
        assert L.bnk_keypair_set(c._h, 16, key, key, 0) == _lib.EINVAL             # slot out of range
        assert L.bnk_keypair_set(c._h, 0, None, key, 0) == _lib.EINVAL
        assert L.bnk_keypair_set_allowed_ip(c._h, 99, 1) == _lib.EINVAL
        assert L.bnk_index_set(c._h, 5, 99) == _lib.EINVAL
        v = C.c_uint64()
        assert L.bnk_send_counter_get(c._h, 16, C.byref(v)) == _lib.EINVAL
        t = np.zeros(5, ACL_TUPLE_DTYPE)
        assert L.bnk_acl_set(c._h, 1, t.ctypes.data, 5) == _lib.EFULL              # more than max_acl_tuples
        t = np.zeros(1, ACL_TUPLE_DTYPE)
        t["prefix_len"] = 33
        assert L.bnk_acl_set(c._h, 1, t.ctypes.data, 1) == _lib.EINVAL
        assert L.bnk_acl_set(c._h, 1, None, 3) == _lib.EINVAL
        b = c.batch(8, 8 * 128)
        assert L.bnk_seal_submit(b._h, 9, 0, 0) == _lib.EINVAL                     # more packets than the batch holds
        assert L.bnk_open_submit(b._h, 9, 0, 0) == _lib.EINVAL
        ms = C.c_float()
        b.seal(1)
        assert L.bnk_batch_last_kernel_ms(b._h, C.byref(ms)) == _lib.EINVAL        # that submit was not timed
        assert L.bnk_batch_last_aead_ms(b._h, C.byref(ms)) == _lib.EINVAL
        b.seal(1, _lib.F_TIMED)
        assert L.bnk_batch_last_kernel_ms(b._h, C.byref(ms)) == 0 and ms.value > 0
        assert L.bnk_wait(None, 0) == _lib.EINVAL
        assert L.bnk_wait(b._h, 0) == 0                                            # nothing in flight: done
        big = np.zeros(1, np.dtype(_lib.GsoSuper))
        big["src_off"], big["src_len"] = 8 * 128, 64                               # outside the ring
        assert L.bnk_gso_split_submit(b._h, big.ctypes.data, 1, 1, 0) == _lib.EINVAL
        b.wait()
        # the context is still fine after all that
        b.off[0], b.len[0], b.slot[0], b.counter[0] = 0, 16, 0, 1
        c.set_keypair(0, key, key, 7)
        b.seal(1)
        assert b.status[0] == 0 and b.out_len[0] == 48
        b.close()
