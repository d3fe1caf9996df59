"""Host logic of the row sharding (ao_b200/sharding.py) on CPU: shard bounds, and two gloo ranks whose gathered
outputs equal the unsharded layer.  The quantized kernels are not involved (they need a GPU); the shards stay dense."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ao_b200.sharding import RowShardedLinear, all_gather_rows, row_shard_bounds


def test_bounds_cover_all_rows_in_blocks():
    for n, world, mult in [(4096, 8, 8), (28672, 8, 64), (1032, 4, 8), (64, 8, 8), (10240, 8, 64), (57344, 8, 64)]:
        pieces = [row_shard_bounds(n, world, r, mult) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        for (lo, hi), (lo2, _) in zip(pieces, pieces[1:]):
            assert hi == lo2
        assert all((hi - lo) % mult == 0 for lo, hi in pieces)
        sizes = [hi - lo for lo, hi in pieces]
        assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        row_shard_bounds(100, 2, 0, 8)
    with pytest.raises(ValueError):
        row_shard_bounds(128, 2, 2, 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_out, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(7)  # every rank builds the same full layer
        full = torch.nn.Linear(96, n_out, bias=True)
        x = torch.randn(3, 5, 96)
        sharded = RowShardedLinear.from_linear(full, multiple=8)
        lo, hi = row_shard_bounds(n_out, world, rank, 8)
        assert sharded.shard.out_features == hi - lo
        y = sharded(x)
        ok = torch.allclose(y, full(x), atol=1e-6) and y.shape == (3, 5, n_out)
        # the gather alone, with rank-dependent content
        mine = torch.full((2, hi - lo), float(rank))
        g = all_gather_rows(mine, n_out, 8)
        for r in range(world):
            a, b = row_shard_bounds(n_out, world, r, 8)
            ok = ok and bool((g[:, a:b] == r).all())
        torch.save(ok, f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_out", [64, 40])  # equal shards; uneven shards (3 + 2 blocks of 8)
def test_two_gloo_ranks_match_the_full_layer(tmp_path, n_out):
    world, port = 2, _free_port()
    out = str(tmp_path / "ok")
    mp.spawn(_worker, args=(world, port, n_out, out), nprocs=world, join=True)
    assert all(torch.load(f"{out}.{r}") for r in range(world))
