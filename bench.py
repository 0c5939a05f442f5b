#!/usr/bin/env python
"""Benchmark of the bnk dataplane hot path on B200.

One "step" = one pass of the hot path over one batch of synthetic packets: the per-keypair
send counters are handed out and 1,048,576 packets of 1420 B (65,536 peers, 16 packets each)
are sealed, then the sealed messages are opened and run through the anti-replay window.
`value` is payload bits sealed plus payload bits opened per second with everything resident in
HBM; `e2e` is the same work through the C ABI with pinned host rings, host->device and
device->host copies inside the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 it is launched by torchrun, one rank per GPU; ranks own disjoint peers (peer index
mod N) and never exchange packet data, so the only collectives are the barrier around the
timed region and the max over ranks of the measured time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_PACKETS = 1 << 20
N_PEERS = 1 << 16
SIZE = 1420
HBM_BYTES_PER_PACKET = 2 * SIZE + 32          # seal: read 1420 + write 1452; open: the mirror
# 32-bit integer operations per 1420-byte packet: (23 + 1) ChaCha20 blocks x 992 + 90 Poly1305 blocks x 40
INT_OPS_PER_PACKET = 24 * 992 + 90 * 40
E2E_BATCHES = 8
DEVICE_BATCHES = 2  # device-resident legs: batches in flight, each with half of the step's packets
IMIX_BATCHES = 3    # the mixed-size leg (--device-batches overrides both)
REGIONS = 5  # timed regions of K steps each; the median one is reported
# dram__bytes_read.sum + dram__bytes_write.sum of one seal launch, from the ncu captures summarised in profiles/:
# (packets of the captured launch, bytes).  The figure is a LOWER bound of what a launch moves: whatever part of
# the output is still dirty in the 126 MB L2 when the launch ends has not reached DRAM yet (about 50 MB, so the
# larger the launch the smaller the share).  The capture closest in size to the benchmark's launch is used and
# scaled by the packet count.
NCU_DRAM_CAPTURES = [(131072, 131072 * 2569), (524288, 780716032 + 718754304)]


# ----------------------------------------------------------------------------------------------
# plumbing
# ----------------------------------------------------------------------------------------------
def env_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


class Dist:
    """Barrier and max-over-ranks; a no-op for one rank (torch is only imported for N > 1)."""

    def __init__(self, rank, world, local_rank, backend="nccl"):
        self.rank, self.world, self.backend = rank, world, backend
        self.torch = None
        if world > 1:
            import torch
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if backend == "nccl":
                torch.cuda.set_device(local_rank)
                dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            else:  # gloo: the CPU tests of this plumbing
                dist.init_process_group(backend, rank=rank, world_size=world)
            self.torch, self.dist = torch, dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
            if self.backend == "nccl":
                self.torch.cuda.synchronize()

    def max(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda" if self.backend == "nccl" else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda" if self.backend == "nccl" else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        return self.max(0.0 if ok else 1.0) == 0.0

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        """windows: [(t_begin, t_end)] wall-clock spans of the timed regions."""
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.lines:
            if not any(a - 0.05 <= t <= b + 0.15 for a, b in windows):
                continue
            p = [x.strip() for x in line.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                smax.append(float(p[1]))
                power.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


def bind_to_gpu_numa_node(local_rank: int) -> str:
    """Pins this rank to the CPUs of the NUMA node its GPU hangs off, so that the pinned packet rings are
    allocated in that node's memory and the host<->device copies do not cross sockets.  Best effort."""
    try:
        bus = subprocess.run(["nvidia-smi", "-i", str(local_rank), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if not bus:
            return "no bus id"
        if bus.startswith("00000000:"):
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read().strip())
        if node < 0:
            return f"gpu {bus}: no numa node"
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return f"gpu {bus}: node {node} has no allowed cpu"
        os.sched_setaffinity(0, allowed)
        return f"gpu {bus}: numa node {node}, {len(allowed)} cpus"
    except Exception as e:  # noqa: BLE001 - placement is an optimisation, never a failure
        return f"not bound ({type(e).__name__})"


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ----------------------------------------------------------------------------------------------
# the CPU arm: OpenSSL ChaCha20-Poly1305 on every host core, same packets, same framing
# ----------------------------------------------------------------------------------------------
def cpu_sample(n: int, peers: int, seed: int):
    from bnk_b200 import gen
    from bnk_b200.device import slot_size

    stride = slot_size(SIZE)
    ring = gen.splitmix_fill(seed, n * stride)
    i = np.arange(n, dtype=np.uint64)
    off = (i * stride).astype(np.uint32)
    length = np.full(n, SIZE, np.uint32)
    slot = (i % peers).astype(np.uint32)
    counter = i // np.uint64(peers)
    keys = gen.SplitMix64(seed + 1).bytes(peers * 32)
    ridx = np.arange(peers, dtype=np.uint32)
    return ring, off, length, slot, counter, keys, ridx


class CpuArm:
    """The CPU arm's ring: built once, then sealed and opened in place over and over, as a forwarder's packet
    buffers are.  One pass = seal all packets, then open them (which restores the plaintext)."""

    def __init__(self, threads: int, n: int):
        self.threads, self.n = threads, n
        self.peers = min(N_PEERS, max(1, n // 16))
        (self.ring, self.off, self.length, self.slot, self.counter, self.keys, self.ridx) = cpu_sample(n, self.peers, 0xB2000004)
        self.first = self.ring[16:16 + SIZE].copy()

    def passes(self, count: int) -> float:
        """-> seconds the worker threads took for `count` passes (checked against the round trip)."""
        from oracle import oracle as O

        total = 0.0
        for _ in range(count):
            s1, st, out_len = O.cpu_aead_batch(False, self.threads, self.keys, self.ridx, SIZE, self.ring, self.off,
                                               self.length, self.slot, self.counter)
            ctr = np.zeros(self.n, np.uint64)
            s2, st2, _ = O.cpu_aead_batch(True, self.threads, self.keys, self.ridx, SIZE, self.ring, self.off, out_len,
                                          self.slot, ctr)
            assert (st == 0).all() and (st2 == 0).all() and np.array_equal(ctr, self.counter)
            assert np.array_equal(self.ring[16:16 + SIZE], self.first)
            total += s1 + s2
        return total

    def gbps(self, count: int, secs: float) -> float:
        return 2.0 * self.n * SIZE * 8 * count / secs / 1e9


REFERENCE_PASSES_PER_STEP = 3


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = host_threads()
    # a bounded sample of the same workload: 16 packets per peer, 1420 B; every step walks the same ring three
    # times (the ring is warm, as in the GPU arm, where every step reuses its rings)
    n = 1 << 18
    arm = CpuArm(threads, n)
    for _ in range(max(1, args.warmup)):
        arm.passes(1)
    t0 = time.time()
    per_step = [arm.passes(REFERENCE_PASSES_PER_STEP) for _ in range(args.steps)]
    secs = sum(per_step)
    gbps = arm.gbps(REFERENCE_PASSES_PER_STEP * args.steps, secs)
    sample = (f"{n} packets x {SIZE} B sealed then opened, {REFERENCE_PASSES_PER_STEP} passes per step over one warm ring "
              f"(a quarter of the GPU arm's batch)")
    line = {
        "impl": "reference", "metric": "aead_seal_open_gbps_1420B", "value": gbps, "unit": "Gbit/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gbps, "unit": "Gbit/s", "cores": threads, "kind": "port", "sample": sample,
                         "step_gbps_min_max": [arm.gbps(REFERENCE_PASSES_PER_STEP, max(per_step)),
                                               arm.gbps(REFERENCE_PASSES_PER_STEP, min(per_step))],
                         "note": "OpenSSL EVP_chacha20_poly1305 (AVX2/AVX-512 assembly) standing in for x/crypto's "
                                 "assembly: the Go reference path cannot be built here (no Go toolchain or module cache)"},
        "e2e": {"value": gbps, "unit": "Gbit/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.time() - t0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, device_batches: int = DEVICE_BATCHES):
    return {
        "workload": "bulk seal+open at scale (BASELINE configs[3]): 1,048,576 packets x 1420 B over 65,536 peers per GPU, "
                    "16 sequential counters per peer, MTU 1420, replay ring 128 blocks",
        "packets_per_gpu": N_PACKETS, "peers_per_gpu": N_PEERS, "payload_bytes": SIZE,
        "sharding": f"peer index mod {n_gpus}, no inter-GPU traffic",
        "bits_counted": "payload bits sealed + payload bits opened",
        "l2": "inputs (1.5 GB per pass) are larger than L2, no flush needed",
        "device_batches_in_flight": device_batches,
    }


# ----------------------------------------------------------------------------------------------
# the GPU arm
# ----------------------------------------------------------------------------------------------
def setup_batch(ctx, n, stride, peers, first_peer=0):
    b = ctx.batch(n, n * stride)
    i = np.arange(n, dtype=np.uint64)
    b.off[:] = (i * np.uint64(stride)).astype(np.uint32)
    b.len[:] = SIZE
    b.slot[:] = (first_peer + (i % np.uint64(peers))).astype(np.uint32)
    b.counter[:] = 0
    return b


PIPE5_SUPERS_PER_GPU, PIPE5_SEGS, PIPE5_MSS, PIPE5_PEERS = 2048, 47, 1380, 10_000


def pipeline5_share(rank: int, world: int, supers_per_gpu: int = PIPE5_SUPERS_PER_GPU, n_peers: int = PIPE5_PEERS):
    """Which super-packets of configuration 5's batch this rank works on.  Every rank computes the same placement
    from the same measured loads (the peer draws of an earlier period of the same traffic), so no rank has to be
    told.  -> (workload, indices of this rank's super-packets, gpu_of, slot_of, segments per GPU)"""
    from bnk_b200 import gen
    from bnk_b200.mgpu import place_peers

    n_super = supers_per_gpu * world
    earlier = gen.config5_peers(n_super, n_peers, seed=gen.seed_for(5) + 1000)
    load = np.bincount(earlier, minlength=n_peers).astype(np.uint64)
    gpu_of, slot_of, _ = place_peers(load, n_peers, world)
    w5 = gen.config5(n_super=n_super, n_peers=n_peers)
    per_gpu = np.bincount(gpu_of[w5.peer], minlength=world) * PIPE5_SEGS
    mine = np.flatnonzero(gpu_of[w5.peer] == rank)
    return w5, mine, gpu_of, slot_of, per_gpu


def run_pipeline5(rank, world, local_rank, dist, W, K, windows):
    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_ASSIGN_COUNTERS, F_CHECK_INBOUND, F_DEMUX_INDEX, F_INNER_CHECK, F_NO_D2H, F_NO_H2D,
                                 F_NOTE_OUTBOUND, F_REPLAY, F_TIMED, F_USE_OUT_LEN, GSO_SUPER_DTYPE, PKT_FILTER_DENY, PKT_OK,
                                 slot_size)
    from bnk_b200.filter import flatten_rule_arrays

    n_seg, mss, p_peers, stride = PIPE5_SEGS, PIPE5_MSS, PIPE5_PEERS, slot_size(SIZE)
    w5, mine, gpu_of, slot_of, per_gpu = pipeline5_share(rank, world)
    f5 = gen.config3(n_rules=2000, n_nodes=5000, n_out=16, n_in=16, seed=gen.seed_for(5) + 1)
    hit = np.flatnonzero(f5.rules["proto"] == 6)[:3]
    for rr in hit:
        f5.srcs["addr"][f5.rules["src_begin"][rr]] = w5.self_ip
    my_peers = np.flatnonzero(gpu_of == rank)
    n_slots = max(1, int(slot_of[my_peers].max()) + 1) if len(my_peers) else 1
    pctx = Context(device_id=local_rank, max_keypairs=n_slots, mtu=SIZE, flow_capacity=1 << 16)
    # a peer's keypair slot on its GPU is the one the placement handed out
    keys = np.zeros((n_slots, 32), np.uint8)
    keys[slot_of[my_peers]] = w5.keys[my_peers]
    ridx = np.zeros(n_slots, np.uint32)
    ridx[slot_of[my_peers]] = (0x1000 + my_peers).astype(np.uint32)
    pctx.set_keypairs(0, keys, keys, ridx)
    for p_ in sorted(set(w5.peer[mine].tolist())):
        pctx.index_set(0x1000 + p_, int(slot_of[p_]))
        pctx.set_allowed_ip(int(slot_of[p_]), w5.self_ip)
    pctx.acl_set(True, flatten_rule_arrays(f5.rules, f5.srcs, f5.ports))
    n_super = len(mine)
    n_pkts = n_super * n_seg
    split_ms, seal5_ms, open5_ms = [], [], []
    st5 = np.zeros(0, np.uint8)
    if n_super:
        sup = np.zeros(n_super, GSO_SUPER_DTYPE)
        sup_stride = (len(w5.supers[0]) + 15) & ~15
        pb = pctx.batch(n_pkts, n_pkts * stride + n_super * sup_stride)
        for k, j in enumerate(mine.tolist()):
            pkt = w5.supers[j]
            o = n_pkts * stride + k * sup_stride
            pb.ring[o:o + len(pkt)] = np.frombuffer(pkt, np.uint8)
            sup[k] = (o, len(pkt), k * n_seg, n_seg, 40, mss, 20, 16, 6, (0, 0, 0))
        pb.off[:n_pkts] = (np.arange(n_pkts, dtype=np.uint64) * np.uint64(stride)).astype(np.uint32)
        pb.len[:n_pkts] = 40 + mss
        pb.slot[:n_pkts] = np.repeat(slot_of[w5.peer[mine]], n_seg)
        pb.gso_split(sup, n_pkts)  # uploads the ring once
    now = 1_700_000_000 * 10**9
    dist.barrier()
    t_begin = time.time()
    for it in range(W + K):
        if not n_super:
            break
        pb.gso_split(sup, n_pkts, F_NO_H2D | F_TIMED)
        split_ms.append(pb.last_kernel_ms())
        pb.seal(n_pkts, F_NO_H2D | F_NO_D2H | F_NOTE_OUTBOUND | F_ASSIGN_COUNTERS | F_TIMED, now_ns=now + it)
        seal5_ms.append(pb.last_kernel_ms())
        pb.open(n_pkts, F_NO_H2D | F_NO_D2H | F_USE_OUT_LEN | F_DEMUX_INDEX | F_REPLAY | F_INNER_CHECK | F_CHECK_INBOUND | F_TIMED,
                now_ns=now + it)
        open5_ms.append(pb.last_kernel_ms())
    windows.append((t_begin, time.time()))
    mean = lambda v: statistics.mean(v[W:]) if len(v) > W else 0.0
    t_local = mean(split_ms) + mean(seal5_ms) + mean(open5_ms)
    if n_super:
        pb.download(n_pkts)
        st5 = np.array(pb.status[:n_pkts])
        pb.close()
    pctx.close()
    ok_local = bool(((st5 == PKT_OK) | (st5 == PKT_FILTER_DENY)).all())
    t5 = dist.max(t_local)  # the slowest rank decides
    ok = dist.all_true(ok_local)
    total_pkts = int(per_gpu.sum())
    allowed = dist.sum(float((st5 == PKT_OK).sum()))
    denied = dist.sum(float((st5 == PKT_FILTER_DENY).sum()))
    return {"segments": total_pkts, "super_packets": PIPE5_SUPERS_PER_GPU * world, "peers": p_peers, "rules": 2000, "n_gpus": world,
            "segments_per_gpu": [int(x) for x in per_gpu],
            "load_imbalance": float(per_gpu.max() / per_gpu.mean()),
            "load_imbalance_peer_mod_n": float((lambda c: c.max() / c.mean())(np.bincount(w5.peer % world, minlength=world))),
            "heaviest_peer_share": float(np.bincount(w5.peer).max() / len(w5.peer)),
            "placement": "bnk_place_peers on the per-peer load of an earlier period (heaviest first, least-loaded GPU); "
                         "a peer is never split",
            "split_ms": mean(split_ms), "seal_side_ms": mean(seal5_ms), "open_side_ms": mean(open5_ms),
            "slowest_rank_ms": t5,
            "gbps": 2.0 * total_pkts * (40 + mss) * 8 / (t5 * 1e-3) / 1e9 if t5 else None,
            "mpps": 2.0 * total_pkts / (t5 * 1e-3) / 1e6 if t5 else None,
            "allowed": int(allowed), "filter_deny": int(denied), "verified": ok,
            "note": "every context plays sender and receiver of its peers (loopback); Zipf(1.1) peers, 47 x 1420 B per "
                    "super-packet; split/seal/open times are rank 0's, the rate uses the slowest rank's total"}


def run_ours(args, rank, world, local_rank):
    from bnk_b200 import Context, gen
    from bnk_b200.device import (F_ASSIGN_COUNTERS, F_NO_D2H, F_NO_H2D, F_REPLAY, F_SORT_BY_LENGTH, F_TIMED, F_USE_OUT_LEN,
                                 slot_size)

    placement = bind_to_gpu_numa_node(local_rank) if world > 1 else "single rank: not bound"
    dist = Dist(rank, world, local_rank)
    K, W = args.steps, args.warmup
    n, peers = args.packets, min(N_PEERS, max(1, args.packets // 16))
    plan = gen.config4(n, peers, SIZE, rank, world)
    stride = plan.stride
    ctx = Context(device_id=local_rank, max_keypairs=2 * peers, replay_ring_blocks=128, mtu=SIZE, flow_capacity=0)
    keys = gen.bulk_keys(plan)
    # slots [0, peers) serve the device-resident run, [peers, 2*peers) the host-ring run
    ctx.set_keypairs(0, np.concatenate([keys, keys]), np.concatenate([keys, keys]),
                     np.arange(2 * peers, dtype=np.uint32))
    sampler = ClockSampler(local_rank)
    sampler.start()
    windows = []

    # ---- device-resident: value + roofline ----
    # The step's 1,048,576 packets sit in DEVICE_BATCHES batches with disjoint peers, each on its own stream, as a
    # forwarder keeps several batches in flight: the grouping, counter and replay kernels of one batch run beside
    # the seal/open kernels of the other.  The work per step is the same whatever the number.
    nbd = max(1, args.device_batches)
    per_d, peers_d = n // nbd, max(1, peers // nbd)
    devs = [setup_batch(ctx, per_d, stride, peers_d, first_peer=j * peers_d) for j in range(nbd)]
    for j, d in enumerate(devs):
        d.upload(per_d)
        d.fill_random(plan.payload_seed + 101 * j)
    dev = devs[0]
    SEAL = F_NO_H2D | F_NO_D2H | F_ASSIGN_COUNTERS
    OPEN = F_NO_H2D | F_NO_D2H | F_REPLAY | F_USE_OUT_LEN

    def step_dev():
        for d in devs:
            d.seal(per_d, SEAL, wait=False)
        for d in devs:
            d.open(per_d, OPEN, wait=False)

    for _ in range(W):
        step_dev()
    ctx.synchronize()
    # The timed region of exactly K steps is taken REGIONS times and the median region is reported (with the
    # fastest and the slowest), so that one clock blip cannot decide the number; every region is bracketed by a
    # barrier and timed on the device, the maximum over ranks counts.
    region_ms = []
    launches = 0
    for _ in range(REGIONS):
        dist.barrier()
        launches0 = ctx.launch_count()
        t_begin = time.time()
        ctx.timer_start(devs)
        for _ in range(K):
            step_dev()
        ms_local = ctx.timer_stop(devs)
        ctx.synchronize()
        dist.barrier()
        windows.append((t_begin, time.time()))
        launches = ctx.launch_count() - launches0
        region_ms.append(dist.max(ms_local))
    ms = statistics.median(region_ms)
    verified = True
    for d in devs:
        d.wait()
        d.download(per_d)
        verified = verified and bool((d.status[:per_d] == 0).all() and (d.out_len[:per_d] == SIZE).all()
                                     and (int(d.counter[:per_d].max()) == (per_d // peers_d) * (W + REGIONS * K) - 1
                                          if per_d >= 16 * peers_d else True))
    bits_per_step = 2.0 * n * SIZE * 8
    value = world * bits_per_step * K / (ms * 1e-3) / 1e9
    value_spread = [world * bits_per_step * K / (t * 1e-3) / 1e9 for t in (max(region_ms), min(region_ms))]
    for d in devs[1:]:
        d.close()
    n_launch = per_d  # packets per seal/open launch from here on (one batch alone on the device)

    # per-launch duration of the dominant kernels (CUDA events around the seal / open kernel alone)
    seal_ms, open_ms = [], []
    t_begin = time.time()
    for _ in range(max(K, 3)):
        dev.seal(n_launch, SEAL | F_TIMED, wait=False)
        seal_ms.append(dev.last_aead_ms())
        dev.open(n_launch, OPEN | F_TIMED, wait=False)
        open_ms.append(dev.last_aead_ms())
    dev.wait()
    windows.append((t_begin, time.time()))
    seal_avg, open_avg = statistics.mean(seal_ms), statistics.mean(open_ms)
    aead_avg = 0.5 * (seal_avg + open_avg)
    peak, peak_src = measured_hbm_peak()
    achieved = n_launch * HBM_BYTES_PER_PACKET / (aead_avg * 1e-3) / 1e9
    cap_n, cap_bytes = min(NCU_DRAM_CAPTURES, key=lambda c: abs(c[0] - n_launch))
    traffic = cap_bytes * n_launch // cap_n
    traffic_note = (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of a {cap_n}-packet seal launch, scaled by packet "
                    f"count; a lower bound (output still dirty in L2 at kernel end is not counted: "
                    f"~{42e6 / (cap_n * HBM_BYTES_PER_PACKET) * 100:.0f} % of that launch)")
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": traffic, "traffic_note": traffic_note,
        "kernel": "aead_kernel<seal> / aead_kernel<open> (2872 algorithmic bytes per packet)", "packets_per_launch": n_launch,
        "launch_note": "timed with one batch alone on the device; a step runs this launch once per batch and direction",
        "peak_source": peak_src, "seal_ms": seal_avg, "open_ms": open_avg,
        "note": "the path is bound by the 32-bit integer pipes, not by HBM: see `alu`",
    }
    alu = None
    ctx_sm_count = 148  # B200; only used to turn the measured kernel time into cycles per block
    if rank == 0 and not args.no_probe:
        probes = {name: ctx.probe_int_throughput(mix) for mix, name in
                  enumerate(["add_xor", "chacha_rounds", "imad", "add_xor_plus_imad"])}
        int_peak = max(probes.values())
        ops = n_launch * INT_OPS_PER_PACKET / (aead_avg * 1e-3) / 1e12
        # what Poly1305's multiplies (or any stand-in for them) cost beside the rounds: scheduler cycles per ChaCha20
        # double round per warp with k extra operations interleaved; 128 is the ALU-pipe bound of the rounds alone
        co = {name: ctx.probe_coissue(kind, k) for name, kind, k in
              [("rounds_alone", 0, 0), ("mad_wide_x8", 1, 8), ("mad_wide_x16", 1, 16), ("fp64_fma_x16", 2, 16),
               ("fp64_fma_x32", 2, 32), ("mad_lo_x16", 3, 16), ("mad_lo_x32", 3, 32), ("fp32_fma_x16", 4, 16),
               ("fp32_fma_x32", 4, 32), ("mul_hi_x8", 5, 8), ("mul_hi_x16", 5, 16),
               # two cipher blocks per thread at half the warps (what doubling the state registers would allow)
               ("two_blocks_per_thread_half_the_warps", 6, 0)]}
        # per 64-byte block: 10 double rounds + 85 wide multiply-adds (4 Poly1305 blocks) at their interleaved cost,
        # + the ~100 ALU-pipe instructions of Poly1305's carries and the data exclusive-ors at 2 cycles each
        wide_each = (co["mad_wide_x8"] - co["rounds_alone"]) / 8.0
        floor_cycles = 10 * co["rounds_alone"] + 85 * wide_each + 100 * 2
        cycles_now = aead_avg * 1e-3 * 1.965e9 * 4 * ctx_sm_count / (n_launch / 32.0) / 24.0  # 4 schedulers per SM, 24 blocks per packet
        alu = {"bound": "int32 issue", "achieved": ops, "peak": int_peak, "unit": "Tops/s", "frac": ops / int_peak,
               "ops_per_packet": INT_OPS_PER_PACKET, "probes_tops": probes,
               "peak_source": "measured live by bnk_probe_int_throughput (best of the instruction mixes)",
               "coissue_cycles_per_double_round": co,
               "cycles_per_64B_block_per_warp": {"kernel_now": cycles_now, "floor_from_probes": floor_cycles,
                                                  "kernel_over_floor": cycles_now / floor_cycles,
                                                  "alu_pipe_bound_of_the_rounds_alone": 1280.0}}
    dev.close()

    # ---- IMIX, device-resident, the same number of batches in flight ----
    imix = None
    if not args.no_imix:
        g = gen.SplitMix64(gen.seed_for(2) + 7919 * rank)
        # Three batches in flight here (the sizes differ by at most one packet, the peers of the batches are
        # disjoint): with packets this short the grouping, counter and replay kernels are a third of a batch's own
        # time, and a third batch gives them more seal/open work of other batches to run beside.
        nbi = IMIX_BATCHES if args.device_batches == DEVICE_BATCHES else nbd
        per_i = [n // nbi + (1 if j < n % nbi else 0) for j in range(nbi)]
        peers_i = max(1, peers // nbi)
        ibs, size_sum = [], 0.0
        for j in range(nbi):
            sizes = gen.imix_sizes(g, per_i[j])
            size_sum += float(sizes.sum())
            slots_sz = ((sizes.astype(np.uint64) + np.uint64(48 + 15)) // np.uint64(16)) * np.uint64(16)
            offs = np.concatenate([[0], np.cumsum(slots_sz)[:-1]]).astype(np.uint64)
            ib = ctx.batch(per_i[j], int(offs[-1] + slots_sz[-1]))
            ib.off[:] = offs.astype(np.uint32)
            ib.len[:] = sizes
            ib.slot[:] = (j * peers_i + np.arange(per_i[j], dtype=np.uint64) % np.uint64(peers_i)).astype(np.uint32)
            ib.upload(per_i[j])
            ib.fill_random(plan.payload_seed + 5 + j)
            ibs.append(ib)

        def step_imix():
            for ib, m_ in zip(ibs, per_i):
                ib.seal(m_, SEAL | F_SORT_BY_LENGTH, wait=False)
            for ib, m_ in zip(ibs, per_i):
                ib.open(m_, OPEN | F_SORT_BY_LENGTH, wait=False)

        for _ in range(W):
            step_imix()
        ctx.synchronize()
        dist.barrier()
        t_begin = time.time()
        ctx.timer_start(ibs)
        for _ in range(K):
            step_imix()
        ims = dist.max(ctx.timer_stop(ibs))
        dist.barrier()
        windows.append((t_begin, time.time()))
        for ib in ibs:
            ib.wait()
        # one more pass over one batch alone with events around its two AEAD launches
        ibs[0].seal(per_i[0], SEAL | F_SORT_BY_LENGTH | F_TIMED)
        imix_seal_ms = ibs[0].last_aead_ms()
        ibs[0].open(per_i[0], OPEN | F_SORT_BY_LENGTH | F_TIMED)
        imix_open_ms = ibs[0].last_aead_ms()
        imix_ok = True
        for ib, m_ in zip(ibs, per_i):
            ib.download(m_)
            imix_ok = imix_ok and bool((ib.status[:m_] == 0).all())
        imix = {"mpps": world * 2.0 * n * K / (ims * 1e-3) / 1e6, "unit": "Mpps",
                "packets_counted": "packets sealed + packets opened", "sizes": "64/576/1420 B at 7:4:1",
                "gbps": world * 2.0 * size_sum * 8 * K / (ims * 1e-3) / 1e9, "verified": imix_ok,
                "ms_per_step": ims / K, "batches_in_flight": nbi, "packets_per_launch": per_i[0],
                "seal_kernel_ms": imix_seal_ms, "open_kernel_ms": imix_open_ms}
        for ib in ibs:
            ib.close()

    e2e_value = e2e_ms = e2e_roofline = None
    e2e_ok = True
    h2d = d2h = 0
    nb = E2E_BATCHES
    if not args.no_e2e:
        # ---- end to end: pinned host rings, H2D and D2H inside the timed region ----
        nb = max(1, args.e2e_batches)
        per = n // nb
        batches = [setup_batch(ctx, per, stride, peers, first_peer=peers) for _ in range(nb)]
        ppb = max(1, peers // nb)  # batches in flight together own disjoint peers: nonce and replay order is per peer
        for j, b in enumerate(batches):
            b.slot[:] = (peers + j * ppb + (np.arange(per, dtype=np.uint64) % np.uint64(ppb))).astype(np.uint32)
            b.upload(per)
            b.fill_random(plan.payload_seed + 11 + j)
            b.download(per)  # the pinned host ring now holds the synthetic plaintext

        # Each batch alternates seal and open; the host walks the batches round-robin, waits for a batch's previous
        # operation and queues its next one, so the copy engines never drain between steps.
        def run_e2e(steps):
            phase = [0] * nb  # operations queued so far per batch: even = next is a seal, odd = next is an open
            for _ in range(2 * steps):
                for j, b in enumerate(batches):
                    b.wait()
                    if phase[j] % 2 == 0:
                        b.len[:per] = SIZE
                        b.seal(per, F_ASSIGN_COUNTERS, wait=False)
                    else:
                        b.len[:per] = b.out_len[:per]
                        b.open(per, F_REPLAY, wait=False)
                    phase[j] += 1
            for b in batches:
                b.wait()

        run_e2e(W)
        ctx.synchronize()
        dist.barrier()
        t_begin = time.time()
        ctx.timer_start(batches)
        run_e2e(K)
        e2e_ms = dist.max(ctx.timer_stop(batches))
        dist.barrier()
        windows.append((t_begin, time.time()))
        e2e_ok = all(bool((b.status[:per] == 0).all() and (b.out_len[:per] == SIZE).all()) for b in batches)
        ring_span = per * stride
        h2d = nb * ((ring_span + 3 * 4 * per) + (ring_span + 3 * 4 * per))
        d2h = nb * 2 * (ring_span + (8 + 4 + 1) * per)
        e2e_value = world * bits_per_step * K / (e2e_ms * 1e-3) / 1e9

        # The ceiling of this leg: the same pinned rings, the same streams, the same copies in the same order,
        # and no kernel in between.  What the host link carries at this N, with every rank copying at once.
        def run_copy_only(steps):
            for _ in range(2 * steps):
                for b in batches:
                    b.wait()
                    b.copy_only(per, True, True, wait=False)
            for b in batches:
                b.wait()

        run_copy_only(W)
        ctx.synchronize()
        dist.barrier()
        t_begin = time.time()
        ctx.timer_start(batches)
        run_copy_only(K)
        copy_ms = dist.max(ctx.timer_stop(batches))
        dist.barrier()
        windows.append((t_begin, time.time()))
        e2e_roofline = {
            "bound": "pcie", "unit": "GB/s each way",
            "achieved": (h2d + d2h) / 2 / (e2e_ms / K * 1e-3) / 1e9,
            "peak": (h2d + d2h) / 2 / (copy_ms / K * 1e-3) / 1e9,
            "frac": copy_ms / e2e_ms,
            "peak_source": f"measured in this run at this N: the leg's own copies without its kernels, all {world} "
                           f"rank(s) copying at once ({copy_ms / K:.2f} ms per step against {e2e_ms / K:.2f} ms with kernels)",
            "aggregate_gbs_each_way": world * (h2d + d2h) / 2 / (copy_ms / K * 1e-3) / 1e9,
        }
        for b in batches:
            b.close()

    # ---- ACL filter, configuration 3: 10,000 rules, 300,000 noted flows, 1,000,000 inbound headers, device resident ----
    filt = None
    if rank == 0 and not args.no_filter:
        from bnk_b200.filter import flatten_rule_arrays

        w3 = gen.config3()
        fctx = Context(device_id=local_rank, max_keypairs=4, flow_capacity=1 << 20)
        tuples = flatten_rule_arrays(w3.rules, w3.srcs, w3.ports)
        fctx.acl_set(True, tuples)
        n_out, n_in = len(w3.outbound_len), len(w3.inbound_len)
        fb = fctx.batch(n_in, n_in * gen.HDR_STRIDE)

        def load(hdr, lens):
            m = len(lens)
            view = fb.ring[:m * gen.HDR_STRIDE].reshape(m, gen.HDR_STRIDE)
            view[:, 16:16 + hdr.shape[1]] = hdr
            fb.off[:m] = (np.arange(m, dtype=np.uint64) * gen.HDR_STRIDE).astype(np.uint32)
            fb.len[:m] = lens
            fb.upload(m)

        load(w3.outbound, w3.outbound_len)
        fb.filter_note(n_out, w3.t0_ns, F_NO_H2D | F_TIMED)
        note_ms = fb.last_kernel_ms()
        load(w3.inbound, w3.inbound_len)
        check_ms = []
        for _ in range(W + K):
            fb.filter_check(n_in, w3.t0_ns + 10**9, F_NO_H2D | F_NO_D2H | F_TIMED)
            check_ms.append(fb.last_kernel_ms())
        fb.download(n_in)
        allowed = int((fb.status[:n_in] == 0).sum())
        cms = statistics.mean(check_ms[W:])
        filt = {"mverdicts_per_s": n_in / (cms * 1e-3) / 1e6, "check_ms": cms, "headers": n_in, "rules": len(w3.rules),
                "allowances": int(len(tuples)), "noted_flows": n_out, "note_ms": note_ms, "allowed": allowed,
                "hbm_gbs": n_in * 29 / (cms * 1e-3) / 1e9,
                "note": "29 algorithmic bytes per header: latency-bound hash probes, HBM-trivial"}
        if not args.no_cpu:
            # the reference walks every rule for every packet under one mutex: one host thread, a sample of the headers
            from oracle import oracle as O

            of = O.Filter()
            of.set_rules_arrays(w3.rules.astype(O.RULE_DTYPE), w3.srcs.astype(O.PREFIX_DTYPE), w3.ports.astype(O.PORT_DTYPE))
            of.note_batch(np.ascontiguousarray(w3.outbound), 28, w3.outbound_len, w3.t0_ns)
            sample = 20000
            t0 = time.perf_counter()
            ov = of.check_batch(np.ascontiguousarray(w3.inbound[:sample]), 28, np.ascontiguousarray(w3.inbound_len[:sample]),
                                w3.t0_ns + 10**9)
            dt = time.perf_counter() - t0
            same = bool(np.array_equal(ov, (fb.status[:sample] == 0).astype(np.uint8)))
            filt["cpu_baseline"] = {"mverdicts_per_s": sample / dt / 1e6, "cores": 1, "kind": "port", "sample": f"{sample} headers",
                                    "verdicts_equal_gpu": same}
        fb.close()
        fctx.close()

    # ---- configuration 5 over all ranks, device resident.  The offered batch (2,048 super-packets per GPU, Zipf(1.1)
    #      over 10,000 peers) is the same on every rank; peers are placed on GPUs by the load measured over an earlier
    #      period (bnk_place_peers, never splitting a peer) and every rank works on the super-packets of its peers:
    #      GSO split -> NoteOutbound -> counters -> seal, then demux -> open -> replay -> inner check -> CheckInbound ----
    pipe = None
    if not args.no_pipeline:
        pipe = run_pipeline5(rank, world, local_rank, dist, W, K, windows)

    # ---- one upstream-sized batch (128 packets, the reference's conn.IdealBatchSize): latency through the C ABI ----
    small = None
    if rank == 0 and not args.no_small:
        def small_latency(sn):
            sb = setup_batch(ctx, sn, stride, 32, first_peer=0)
            sb.ring[:] = 0x5A
            for _ in range(min(30, args.small_rounds)):
                sb.len[:sn] = SIZE
                sb.seal(sn, F_ASSIGN_COUNTERS)
                sb.len[:sn] = sb.out_len[:sn]
                sb.open(sn, F_REPLAY)
            seal_t, open_t = [], []
            for _ in range(args.small_rounds):
                sb.len[:sn] = SIZE
                t0 = time.perf_counter()
                sb.seal(sn, F_ASSIGN_COUNTERS)
                t1 = time.perf_counter()
                sb.len[:sn] = sb.out_len[:sn]
                t2 = time.perf_counter()
                sb.open(sn, F_REPLAY)
                t3 = time.perf_counter()
                seal_t.append(t1 - t0)
                open_t.append(t3 - t2)
            ok = bool((sb.status[:sn] == 0).all())
            sb.close()
            return statistics.median(seal_t) * 1e6, statistics.median(open_t) * 1e6, ok

        def small_pipelined(sn, nb, rounds=max(1, args.small_rounds // 3)):
            """nb batches of sn packets in flight from this one host thread, each with its own peers."""
            bs = [setup_batch(ctx, sn, stride, 32, first_peer=64 * k) for k in range(nb)]
            for x in bs:
                x.ring[:] = 0x5A
            def one_round():
                for x in bs:
                    x.len[:sn] = SIZE
                    x.seal(sn, F_ASSIGN_COUNTERS, wait=False)
                for x in bs:
                    x.wait()
                    x.len[:sn] = x.out_len[:sn]
                    x.open(sn, F_REPLAY, wait=False)
                for x in bs:
                    x.wait()
            for _ in range(min(10, rounds)):
                one_round()
            t0 = time.perf_counter()
            for _ in range(rounds):
                one_round()
            dt = time.perf_counter() - t0
            ok = all(bool((x.status[:sn] == 0).all()) for x in bs)
            for x in bs:
                x.close()
            return 2.0 * sn * nb * rounds * SIZE * 8 / dt / 1e9, ok

        def threaded(threads, packets, rounds, lanes=2, queue=False):
            """bnk_b200/host/apps/mt_stress: host threads with two batches in flight each, one context, through the
            C ABI; it checks statuses, plaintext and replay verdicts itself.  -> Gbit/s or None"""
            import re
            import subprocess
            from bnk_b200 import _build
            exe = os.path.join(_build.HOST, "apps", "mt_stress")
            if not os.path.exists(exe):
                return None
            rates = []
            for _ in range(5):  # the rate is bimodal on shared hosts (some runs are several times slower): median of five
                res = subprocess.run([exe, str(threads), str(rounds), str(packets), str(SIZE), str(lanes), str(int(queue))],
                                     capture_output=True, text=True, timeout=300)
                m = re.search(r"gbps=([0-9.]+)", res.stdout)
                if res.returncode != 0 or "\nOK" not in "\n" + res.stdout or not m:
                    return None
                rates.append(float(m.group(1)))
            return statistics.median(rates)

        # what the host link gives copies of one 128-packet batch (186 KB each way), kernels or not
        one_batch_bytes = 128 * (16 + ((SIZE + 15) & ~15) + 16 + 24)
        copy_rounds = ctx.probe_copy_rounds(8, one_batch_bytes, max(200, 5 * args.small_rounds))
        copy_rounds_8x = ctx.probe_copy_rounds(8, 8 * one_batch_bytes, max(100, 2 * args.small_rounds))
        s128, o128, ok128 = small_latency(128)
        pipe_gbps, pipe_ok = small_pipelined(128, 16)
        s16, o16, ok16 = small_latency(16)
        small = {"packets": 128, "payload_bytes": SIZE, "seal_us": s128, "open_us": o128,
                 "seal_us_16_packets": s16, "open_us_16_packets": o16, "verified": ok128 and ok16 and pipe_ok,
                 "gbps_16_batches_in_flight": pipe_gbps,
                 # seal + open of one batch = two copy rounds; the rate a batch per worker cannot exceed on this host
                 "copy_only_ceiling_gbps_128_packet_copies": copy_rounds / 2 * 2 * 128 * SIZE * 8 / 1e9,
                 "copy_only_ceiling_gbps_1024_packet_copies": copy_rounds_8x / 2 * 2 * 1024 * SIZE * 8 / 1e9,
                 # (a second process on this GPU: only in single-GPU runs, like the CPU baseline)
                 "gbps_8_threads_128_packets": threaded(8, 128, max(20, args.small_rounds)) if world == 1 else None,
                 "gbps_8_threads_1024_packets": threaded(8, 1024, max(10, args.small_rounds // 2)) if world == 1 else None,
                 # every host core drives the GPU, as every host core runs the CPU baseline
                 "gbps_all_cores_128_packets": threaded(host_threads(), 128, max(20, args.small_rounds)) if world == 1 else None,
                 "host_cores": host_threads(),
                 # the same 128-packet calls handed to the library's submit queue (bnk_queue), which packs them into
                 # GPU batches of up to 1024 packets; 2 and 4 caller batches outstanding per thread; the queue has no
                 # thread of its own, so its callers may outnumber the cores (a waiting caller gives its core away)
                 "gbps_8_threads_128_packets_queue": threaded(8, 128, max(20, args.small_rounds), 2, True) if world == 1 else None,
                 "gbps_8_threads_128_packets_queue_4_outstanding": threaded(8, 128, max(20, args.small_rounds), 4, True) if world == 1 else None,
                 "gbps_all_cores_128_packets_queue": threaded(host_threads(), 128, max(20, args.small_rounds), 2, True) if world == 1 else None,
                 "gbps_all_cores_128_packets_queue_4_outstanding": threaded(host_threads(), 128, max(20, args.small_rounds), 4, True) if world == 1 else None,
                 "gbps_2x_cores_128_packets_queue_4_outstanding": threaded(2 * host_threads(), 128, max(20, args.small_rounds), 4, True) if world == 1 else None,
                 # the queue's calls without host copies inside the library (bnk_queue_reserve / commit / wait_span /
                 # release): the caller's reads and writes land in the GPU batch's pinned ring
                 "gbps_8_threads_128_packets_queue_spans": threaded(8, 128, max(20, args.small_rounds), 2, 2) if world == 1 else None,
                 "gbps_8_threads_128_packets_queue_spans_4_outstanding": threaded(8, 128, max(20, args.small_rounds), 4, 2) if world == 1 else None,
                 "gbps_all_cores_128_packets_queue_spans_4_outstanding": threaded(host_threads(), 128, max(20, args.small_rounds), 4, 2) if world == 1 else None,
                 "note": "host wall clock per submit+wait; seal = group+counters launch, seal launch; open = open "
                         "launch, group+replay launch; batches of up to 256 packets and 384 KiB run on the pinned host arrays "
                         "without copies (BNK_HOST_DIRECT_BYTES), larger ones go through the copy engines; gbps_16_batches_in_flight: sixteen "
                         "128-packet batches submitted round-robin by this one Python thread, seal then open; "
                         "gbps_8_threads_*: eight C++ host threads, two batches in flight each, same context "
                         "(bnk_b200/host/apps/mt_stress.cpp), median of five runs; copy_only_ceiling_*: eight threads and streams "
                         "copying one batch's bytes up and down with no kernel between (bnk_probe_copy_rounds), as "
                         "payload Gbit/s sealed + opened; *_queue: the same threads hand "
                         "their 128-packet calls (pageable buffers, copied in and out by the library) to bnk_queue"}

    sampler.stop()
    clocks = sampler.summary(windows)
    ok = dist.all_true(verified and e2e_ok and (imix is None or imix["verified"]) and (pipe is None or pipe["verified"]))

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = host_threads()
        sample_n = 1 << 18
        passes = 24  # about 20 core-seconds on a 16-thread host
        arm = CpuArm(threads, sample_n)
        arm.passes(1)
        secs = arm.passes(passes)
        gbps = arm.gbps(passes, secs)
        cpu = {"value": gbps, "unit": "Gbit/s", "cores": threads, "kind": "port",
               "sample": f"{sample_n} packets x {SIZE} B sealed then opened, {passes} passes "
                         f"({secs:.2f} s wall, {secs * threads:.0f} core-seconds)",
               "note": "OpenSSL EVP_chacha20_poly1305 stand-in for x/crypto's assembly (no Go toolchain on this box)"}

    if rank == 0:
        line = {
            "metric": "aead_seal_open_gbps_1420B", "value": value, "unit": "Gbit/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic", "config": workload_config(world, nbd),
            "mpps": world * 2.0 * n * K / (ms * 1e-3) / 1e6,
            "timed_regions": {"count": REGIONS, "steps_each": K, "value_is": "median region", "value_min_max": value_spread,
                              "ms": region_ms},
            "e2e": None if e2e_value is None else {
                "value": e2e_value, "unit": "Gbit/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / K, "batches_in_flight": nb, "mpps": world * 2.0 * n * K / (e2e_ms * 1e-3) / 1e6,
                "pcie_gbs_each_way": (h2d + d2h) / 2 / (e2e_ms / K * 1e-3) / 1e9, "roofline": e2e_roofline},
            "gpu_launches": int(launches), "roofline": roofline, "alu": alu, "imix": imix, "filter": filt, "pipeline5": pipe, "small_batch": small, "cpu_baseline": cpu,
            "clocks": clocks, "verified": ok, "placement": placement,
        }
        print(json.dumps(line), flush=True)
    ctx.close()
    dist.close()
    if not ok:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--packets", type=int, default=N_PACKETS, help="packets per GPU (smaller only for profiling)")
    ap.add_argument("--device-batches", type=int, default=DEVICE_BATCHES,
                    help="batches (streams) the device-resident step spreads its packets over")
    ap.add_argument("--e2e-batches", type=int, default=E2E_BATCHES, help="pinned rings in flight in the host-ring leg")
    ap.add_argument("--no-imix", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-probe", action="store_true")
    ap.add_argument("--no-filter", action="store_true")
    ap.add_argument("--no-pipeline", action="store_true")
    ap.add_argument("--no-small", action="store_true", help="skip the small-batch latency section (thousands of launches)")
    ap.add_argument("--small-rounds", type=int, default=200, help="timed rounds of the small-batch section (few, for profiling)")
    ap.add_argument("--no-e2e", action="store_true", help="profiling only: skip the host-ring leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and args.packets == N_PACKETS else args.warmup
    rank, world, local_rank = env_world()
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
