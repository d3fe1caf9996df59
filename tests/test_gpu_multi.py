"""Two-GPU test of the fused output exchange (ao_int4_gemv_gather): every rank's gathered buffer must equal the
concatenation of all ranks' single-GPU results, over repeated calls.  Skipped unless two GPUs are visible.
Ranks are child processes; they leave only after a barrier, with nothing in flight."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    import datetime

    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    ok, why = True, ""
    try:
        from ao_b200 import _cabi, ops
        from ao_b200.comm import PeerExchange
        from tests import gpu_util as tu
        g = 64
        shapes = [(1, 1024, 4096), (4, 2048, 4096), (1, 14336 // 2, 4096)]
        slot = 0
        exch = PeerExchange(sum(ops.gather_slot_bytes(world, M, N) for M, N, K in shapes))
        for it, (M, N, K) in enumerate(shapes):
            w = tu.make_weight((N, K), seed=100 * rank + it).to(dev)      # every rank has its own rows
            packed, sz = ops.int4_quantize_pack(w, g, 8)
            x = torch.randn(M, K, generator=torch.Generator().manual_seed(it)).bfloat16().to(dev)   # replicated
            y_local = ops.weight_int4pack_mm(x, packed, g, sz)
            ref = [torch.empty_like(y_local) for _ in range(world)]
            dist.all_gather(ref, y_local)
            for rep in range(3):
                out = ops.weight_int4pack_mm_gather(x, packed, g, sz, exch, slot_offset_bytes=slot)
                torch.cuda.synchronize()
                for r in range(world):
                    if not torch.equal(out[r], ref[r]):
                        ok, why = False, f"shape {(M, N, K)} rep {rep}: block {r} differs on rank {rank}"
                dist.barrier()
            slot += ops.gather_slot_bytes(world, M, N)
        if _cabi.workspace_status(dev) != 0:
            ok, why = False, "status word set"
        exch.close()
    except Exception as e:  # report instead of leaving the other rank waiting
        ok, why = False, f"{type(e).__name__}: {e}"
    torch.save((ok, why), f"{out_path}.{rank}")
    torch.cuda.synchronize()
    try:
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gather_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        ok, why = torch.load(f"{out}.{r}")
        assert ok, why
