"""Two processes over gloo on the CPU: the host-side logic of the one-process-per-GPU mode.

What crosses NVLink on the GPUs (rows pushed into the peers' receive buffers) is emulated here
with torch.distributed.all_to_all over the same per-rank slices and the same slot layout, and
checked against the oracle's all-to-all on the whole batch."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    sys.path[:0] = [str(ROOT), str(ROOT / "tests")]
    import bench
    from oracle.step_oracle import all_to_all

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_shard, rows, batch, a2a, steps = 4, 2001, 32, 12, 2
        n_local = n_shard // world
        pool = bench.TriplePool(n_shard, rows, 8, 20_000)
        full = pool.sample(steps, batch, a2a, seed=5)
        mine = bench.local_slice(full, rank, world)

        # every rank derives the same global batch from the seed: compare checksums
        digest = torch.tensor([int(v.astype(np.uint64).sum() % (1 << 40)) for v in full.values()], dtype=torch.int64)
        gathered = [torch.zeros_like(digest) for _ in range(world)]
        dist.all_gather(gathered, digest)
        assert all(torch.equal(g, digest) for g in gathered)

        # connection handles travel in rank order
        blob = bytes([rank]) * 80
        joined = bench.exchange_handles(blob, world)
        assert joined == b"".join(bytes([r]) * 80 for r in range(world))

        # the exchange: local shard l (global s) sends block d to shard d's slot s
        for step in range(steps):
            send = np.stack([mine["remote"][l, step][mine["a2a"][l, step]] for l in range(n_local)])  # [l, dst, a2a]
            out_parts = [torch.tensor(np.ascontiguousarray(send[:, p * n_local:(p + 1) * n_local]).astype(np.int64))
                         for p in range(world)]  # to process p: [l_src, l_dst, a2a]
            in_parts = [torch.zeros_like(out_parts[0]) for _ in range(world)]
            dist.all_to_all(in_parts, out_parts) if dist.get_backend() != "gloo" else _gloo_all_to_all(in_parts, out_parts, rank, world)
            received = np.zeros((n_local, n_shard, a2a), np.int64)  # [l_dst, src, a2a]
            for p in range(world):
                block = in_parts[p].numpy()  # [l_src (of p), l_dst, a2a]
                for ls in range(n_local):
                    received[:, p * n_local + ls] = block[ls]
            sent_all = np.stack([full["remote"][s, step][full["a2a"][s, step]] for s in range(n_shard)]).astype(np.int64)
            expect = all_to_all(sent_all)[rank * n_local:(rank + 1) * n_local]
            np.testing.assert_array_equal(received, expect)
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def _gloo_all_to_all(in_parts, out_parts, rank, world):
    """gloo has no all_to_all: do it with paired send / recv."""
    import torch.distributed as dist

    in_parts[rank].copy_(out_parts[rank])
    for peer in range(world):
        if peer == rank:
            continue
        if rank < peer:
            dist.send(out_parts[peer], peer)
            dist.recv(in_parts[peer], peer)
        else:
            dist.recv(in_parts[peer], peer)
            dist.send(out_parts[peer], peer)


def test_two_ranks_agree_on_batches_and_routing(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["ok0", "ok1"]
