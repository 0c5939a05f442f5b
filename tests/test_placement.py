"""Placement of peers on GPUs (bnk_place_peers) and the benchmark's share rule, on CPU: a peer is never split,
every peer lands somewhere, heavy peers end up apart, and ranks that compute the placement on their own agree."""
import os
import socket

import numpy as np
import pytest


def test_equal_loads_are_round_robin_and_capacity_is_kept():
    from bnk_b200.mgpu import place_peers

    gpu_of, slot_of, per = place_peers(None, 1000, 8)
    assert np.bincount(gpu_of, minlength=8).tolist() == [125] * 8
    assert gpu_of[:16].tolist() == list(range(8)) * 2
    for g in range(8):
        assert sorted(slot_of[gpu_of == g].tolist()) == list(range(125))   # slots are dense per GPU
    # a cap per GPU is honoured even when the loads would pile peers up
    load = np.zeros(10, np.uint64)
    gpu_of, slot_of, _ = place_peers(load, 10, 3, max_per_gpu=4)
    assert np.bincount(gpu_of, minlength=3).max() <= 4
    from bnk_b200 import _lib

    with pytest.raises(_lib.BnkError):
        place_peers(load, 10, 3, max_per_gpu=3)                              # 9 slots for 10 peers


def test_skewed_loads_spread_the_heavy_peers():
    from bnk_b200 import gen
    from bnk_b200.mgpu import place_peers

    n_peers = 10_000
    for world in (2, 4, 8):
        draws = gen.config5_peers(2048 * world, n_peers)
        load = np.bincount(draws, minlength=n_peers).astype(np.uint64)
        gpu_of, slot_of, per = place_peers(load, n_peers, world)
        assert per.sum() == load.sum()
        assert np.array_equal(per, np.bincount(gpu_of, weights=load.astype(np.float64), minlength=world).astype(np.uint64))
        # the greedy rule's guarantee: no GPU carries more than the mean plus the heaviest single peer
        assert per.max() <= load.sum() / world + load.max()
        # the eight heaviest peers sit on different GPUs (as far as there are GPUs)
        top = np.argsort(-load.astype(np.int64), kind="stable")[:world]
        assert len(set(gpu_of[top].tolist())) == world
        # far better than peer index modulo the number of GPUs
        mod = np.bincount(np.arange(n_peers) % world, weights=load.astype(np.float64), minlength=world)
        assert per.max() / per.mean() <= mod.max() / mod.mean() + 1e-9
        # peers without traffic do not pile onto one GPU (keypair slots are a per-GPU resource); the GPU that
        # carries the heaviest peer gets fewer of them, the others share the rest evenly
        counts = np.bincount(gpu_of, minlength=world)
        assert counts.max() <= 1.1 * counts.mean()
        # deterministic
        again = place_peers(load, n_peers, world)
        assert np.array_equal(again[0], gpu_of) and np.array_equal(again[1], slot_of)


def test_benchmark_shares_are_disjoint_and_complete():
    import bench

    for world in (1, 2, 4):
        seen = set()
        for rank in range(world):
            w5, mine, gpu_of, slot_of, per_gpu = bench.pipeline5_share(rank, world, supers_per_gpu=96)
            assert not seen & set(mine.tolist())
            seen |= set(mine.tolist())
            assert (gpu_of[w5.peer[mine]] == rank).all()                     # only peers placed on this rank
            assert len(mine) * bench.PIPE5_SEGS == per_gpu[rank]
        assert seen == set(range(96 * world))                               # every super-packet has exactly one owner


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import bench

    d = bench.Dist(rank, world, rank, backend="gloo")
    w5, mine, gpu_of, slot_of, per_gpu = bench.pipeline5_share(rank, world, supers_per_gpu=128)
    d.barrier()
    total = d.sum(float(len(mine)))
    slowest = d.max(float(len(mine)))
    np.save(os.path.join(out_dir, f"mine{rank}.npy"), mine)
    np.save(os.path.join(out_dir, f"gpu_of{rank}.npy"), gpu_of)
    with open(os.path.join(out_dir, f"res{rank}.txt"), "w") as f:
        f.write(f"{total} {slowest}")
    d.close()


@pytest.mark.timeout(180)
def test_two_gloo_ranks_agree_on_the_placement(tmp_path):
    mp = pytest.importorskip("torch.multiprocessing")
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    g0, g1 = np.load(tmp_path / "gpu_of0.npy"), np.load(tmp_path / "gpu_of1.npy")
    assert np.array_equal(g0, g1)                                            # nobody had to be told
    m0, m1 = np.load(tmp_path / "mine0.npy"), np.load(tmp_path / "mine1.npy")
    assert not set(m0) & set(m1) and len(m0) + len(m1) == 256
    res = [open(tmp_path / f"res{r}.txt").read().split() for r in range(world)]
    assert [float(r[0]) for r in res] == [256.0, 256.0]
    assert float(res[0][1]) == max(len(m0), len(m1))
