"""Host-side multi-GPU logic on CPU: two gloo ranks partition the peers, build their shards and
agree on the slowest rank's time -- the only things ranks ever exchange."""
import os
import socket

import numpy as np
import pytest


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
    from bnk_b200 import gen

    d = bench.Dist(rank, world, rank, backend="gloo")
    n_global = 1000
    mine = [p for p in range(n_global) if gen.shard_of_peer(p, world) == rank]
    plan = gen.config4(4096, 256, 1420, rank, world)
    keys = gen.bulk_keys(plan)
    d.barrier()
    slowest = d.max(10.0 + rank)              # rank r "took" 10 + r ms
    all_ok = d.all_true(rank != 1)            # rank 1 reports a failed verification
    np.save(os.path.join(out_dir, f"peers{rank}.npy"), np.array(mine))
    np.save(os.path.join(out_dir, f"keys{rank}.npy"), keys)
    with open(os.path.join(out_dir, f"res{rank}.txt"), "w") as f:
        f.write(f"{slowest} {all_ok} {plan.key_seed} {plan.payload_seed}")
    d.close()


@pytest.mark.timeout(180)
def test_two_gloo_ranks_partition_and_agree(tmp_path):
    mp = pytest.importorskip("torch.multiprocessing")
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    peers = [np.load(tmp_path / f"peers{r}.npy") for r in range(world)]
    assert sorted(np.concatenate(peers).tolist()) == list(range(1000))      # complete
    assert not set(peers[0]) & set(peers[1])                                 # disjoint: no shared peer state
    res = [open(tmp_path / f"res{r}.txt").read().split() for r in range(world)]
    assert [float(r[0]) for r in res] == [11.0, 11.0]                        # max over ranks
    assert [r[1] for r in res] == ["False", "False"]                         # one failed rank fails the job
    assert len({r[2] for r in res}) == 2 and len({r[3] for r in res}) == 2   # shards draw from distinct streams
    k0, k1 = np.load(tmp_path / "keys0.npy"), np.load(tmp_path / "keys1.npy")
    assert k0.shape == (256, 32) and not np.array_equal(k0, k1)


def test_shard_rule_and_weak_scaling_plan():
    from bnk_b200 import gen

    for world in (1, 2, 4, 8):
        owners = [gen.shard_of_peer(p, world) for p in range(64)]
        assert all(0 <= o < world for o in owners)
        assert owners[:world] == list(range(world))
        plans = [gen.config4(rank=r, world=world) for r in range(world)]
        assert all(p.n_packets == 1 << 20 and p.n_peers == 1 << 16 and p.stride % 16 == 0 for p in plans)  # per-GPU work fixed
        assert len({p.key_seed for p in plans}) == world
