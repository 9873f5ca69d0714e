"""Multi-rank host logic on CPU (gloo, world size 2): the (batch, head) partition of ahpc_shard_range,
each rank working on its own shard with no data-path collective, and the optional gather of the
output onto one rank.  The per-shard arithmetic here is the CPU oracle (there is no GPU in this tier);
what is under test is the partition / reassembly, and the timing reduction bench.py uses."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from attention_b200 import abi


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import cpu_oracle as o
    B, H, S, D = 2, 3, 40, 16                       # 6 (batch, head) units over 2 ranks
    rng = np.random.default_rng(5)                  # same tensors on every rank
    q, k, v = (rng.standard_normal((B, H, S, D)).astype(np.float32) for _ in range(3))
    begin, end = abi.shard_range(B * H, world, rank)
    flat = lambda x: x.reshape(B * H, 1, S, D)      # noqa: E731  a (b,h) unit is one [1,1,S,D] problem
    mine = np.concatenate([o.attention_fwd(flat(q)[u:u + 1], flat(k)[u:u + 1], flat(v)[u:u + 1], 0.25, True) for u in range(begin, end)])
    # gather onto rank 0 (ranks may hold different unit counts: pad to the longest shard)
    longest = max(abi.shard_range(B * H, world, r)[1] - abi.shard_range(B * H, world, r)[0] for r in range(world))
    padded = np.zeros((longest, 1, S, D), np.float32)
    padded[: end - begin] = mine
    bucket = [torch.zeros(padded.shape) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.from_numpy(padded), bucket, dst=0)
    # the max-over-ranks reduction of the step time
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == 10.0 + world - 1
    if rank == 0:
        parts = []
        for r in range(world):
            b, e = abi.shard_range(B * H, world, r)
            parts.append(bucket[r].numpy()[: e - b])
        full = np.concatenate(parts).reshape(B, H, S, D)
        want = o.attention_fwd(q, k, v, 0.25, True)
        np.save(os.path.join(tmpdir, "ok.npy"), np.array([np.abs(full - want).max()]))
    dist.barrier()
    dist.destroy_process_group()


def test_head_shards_reassemble_to_the_full_output(tmp_path, native_lib):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    err = np.load(tmp_path / "ok.npy")[0]
    assert err == 0.0


def test_decode_head_shards_cover_all_heads(native_lib):
    """Decode shards heads: every GPU holds [page, H/g, slot, D] of every page and the same block table."""
    for heads, world in [(32, 1), (32, 2), (32, 4), (32, 8), (16, 8), (6, 4)]:
        got = []
        for r in range(world):
            b, e = abi.shard_range(heads, world, r)
            got += list(range(b, e))
        assert got == list(range(heads))
