"""The N > 1 path on CPU: two gloo ranks cut one global batch with the library's
partitioner, each processes its shard with a stand-in for the device model, rank 0 gathers
the rows on the host, and the result equals the single-process result bit for bit."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def fake_rows(seqs, dim):
    """Deterministic per-sequence function (depends only on the sequence's own tokens)."""
    out = np.zeros((len(seqs), dim), dtype=np.float32)
    for i, s in enumerate(seqs):
        out[i, 0] = len(s)
        out[i, 1] = float(np.asarray(s, dtype=np.int64).sum() % 9973)
        out[i, 2] = float(s[-1])
    return out


def _worker(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from infinity_b200 import configs as cf
    from infinity_b200.sharding import scatter_rows, shard_indices
    spec = cf.BERT_LARGE
    seqs = []
    for r in range(world):
        seqs.extend(cf.synth_batch("c2", 64, seed_offset=r).sequences())
    lens = [len(s) for s in seqs]
    shards = shard_indices(lens, world, spec)
    mine = shards[rank]
    rows = fake_rows([seqs[i] for i in mine], 8)
    gathered = [None] * world
    dist.all_gather_object(gathered, (mine, rows))  # host gather; the data path has no collective
    max_tokens = torch.tensor([float(sum(lens[i] for i in mine))])
    dist.all_reduce(max_tokens, op=dist.ReduceOp.MAX)
    if rank == 0:
        out = np.zeros((len(seqs), 8), dtype=np.float32)
        for idx, r in gathered:
            scatter_rows(out, r, idx)
        np.savez(result_path, out=out, max_tokens=max_tokens.numpy(), total=np.array([sum(lens)]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_equal_one(tmp_path, world):
    from infinity_b200 import configs as cf
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = tmp_path / "res.npz"
    mp.spawn(_worker, args=(world, port, str(result)), nprocs=world, join=True)
    got = np.load(result)
    seqs = []
    for r in range(world):
        seqs.extend(cf.synth_batch("c2", 64, seed_offset=r).sequences())
    want = fake_rows(seqs, 8)
    assert np.array_equal(got["out"], want)
    # token balance: the busiest rank holds at most one longest sequence more than its share
    assert got["max_tokens"][0] <= got["total"][0] / world + 512


def test_shards_cover_the_batch_once():
    from infinity_b200 import configs as cf
    from infinity_b200.sharding import shard_indices
    lens = cf.synth_batch("c2", 256).lengths
    for g in (1, 2, 4, 8):
        shards = shard_indices(lens, g, cf.BERT_LARGE)
        allidx = np.sort(np.concatenate(shards))
        assert np.array_equal(allidx, np.arange(len(lens)))
        assert all(np.all(np.diff(s) > 0) for s in shards if len(s) > 1)
