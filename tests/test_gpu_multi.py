"""Multi-GPU tests of the output exchange over peer memory (ao_int4_gemv_push / ao_gather_exchange): every rank's
gathered buffer must equal the concatenation of all ranks' single-GPU results, bit for bit, over repeated calls that are
NOT separated by host barriers: as push + wait per layer, as several GEMV pushes followed by one wait for all of them,
as plain GEMVs followed by one exchange kernel that pushes and waits, and as a 32-row batch (tcgen05 kernel) followed by
the exchange kernel.
Runs for every world size in {2, 4, 8} that the box has GPUs for; skipped on a single GPU.
Ranks are child processes; they leave only after a barrier, with nothing in flight.  NVLS is switched off in NCCL
(the test's collectives are only the reference all-gather and the handle exchange)."""
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
        shapes = [(1, 1024, 4096), (4, 2048, 4096), (1, 14336 // 2, 4096), (8, 512, 2048)]
        big = (32, 1024, 2048)    # a batch of the tcgen05 kernel: exchanged by the exchange kernel alone (mode 3)
        exch = PeerExchange(sum(ops.gather_slot_bytes(world, M, N) for M, N, K in shapes + [big]))
        layers = []
        for it, (M, N, K) in enumerate(shapes):
            w = tu.make_weight((N, K), seed=100 * rank + it).to(dev)      # every rank has its own rows
            packed, sz = ops.int4_quantize_pack(w, g, 8)
            site = exch.reserve(M, N)
            xs, refs = [], []
            for rep in range(3):                                          # different activations per repetition
                x = torch.randn(M, K, generator=torch.Generator().manual_seed(10 * it + rep)).bfloat16().to(dev)   # replicated
                y_local = ops.weight_int4pack_mm(x, packed, g, sz, decode_kernel=True)   # the kernel the exchange path runs
                ref = [torch.empty_like(y_local) for _ in range(world)]
                dist.all_gather(ref, y_local)
                xs.append(x)
                refs.append(torch.stack(ref))
            layers.append((packed, sz, site, xs, refs))
        torch.cuda.synchronize()
        dist.barrier()
        # (1) push + wait per call, repetitions back to back with no host synchronisation in between: a fast rank runs
        # ahead of a slow one by up to one call per site
        outs = []
        for rep in range(3):
            for packed, sz, site, xs, refs in layers:
                out = ops.weight_int4pack_mm_gather(xs[rep], packed, g, sz, exch, site=site)
                outs.append((out.clone(), refs[rep], f"push+wait rep {rep} shape {tuple(refs[rep].shape)}"))
        # (2) all layers pushed, then one wait for all of them
        for rep in range(3):
            for packed, sz, site, xs, refs in layers:
                ops.weight_int4pack_mm_gather(xs[rep], packed, g, sz, exch, site=site, wait=False)
            ops.gather_wait(exch, [ly[2] for ly in layers])
            for packed, sz, site, xs, refs in layers:
                outs.append((site.y.clone(), refs[rep], f"push..push wait rep {rep} shape {tuple(refs[rep].shape)}"))
        # (3) plain GEMV into this rank's block, then one exchange kernel that pushes and waits for all layers
        for rep in range(3):
            for packed, sz, site, xs, refs in layers:
                ops.weight_int4pack_mm(xs[rep], packed, g, sz, out=site.y[rank], decode_kernel=True)
            ops.gather_exchange(exch, [ly[2] for ly in layers], push=True)
            for packed, sz, site, xs, refs in layers:
                outs.append((site.y.clone(), refs[rep], f"gemv.. exchange rep {rep} shape {tuple(refs[rep].shape)}"))
        # (4) a 32-row batch: the local product by whatever kernel the dispatcher picks, straight into this rank's block,
        # then the exchange kernel; twice, so that both landing buffers are used
        M, N, K = big
        wb = tu.make_weight((N, K), seed=977 + rank).to(dev)
        packed_b, sz_b = ops.int4_quantize_pack(wb, g, 8)
        site_b = exch.reserve(M, N)
        for rep in range(2):
            xb = torch.randn(M, K, generator=torch.Generator().manual_seed(500 + rep)).bfloat16().to(dev)
            y_local = ops.weight_int4pack_mm(xb, packed_b, g, sz_b)
            ref = [torch.empty_like(y_local) for _ in range(world)]
            dist.all_gather(ref, y_local)
            ops.weight_int4pack_mm(xb, packed_b, g, sz_b, out=site_b.y[rank])
            ops.gather_exchange(exch, [site_b], push=True)
            outs.append((site_b.y.clone(), torch.stack(ref), f"32-row batch + exchange rep {rep}"))
        torch.cuda.synchronize()
        for out, ref, what in outs:
            if not torch.equal(out, ref):
                ok, why = False, f"{what}: gathered output differs on rank {rank}"
                break
        if _cabi.workspace_status(dev) != 0:
            ok, why = False, "status word set"
        dist.barrier()
        exch.close()
    except Exception as e:  # report instead of leaving the other ranks waiting
        ok, why = False, f"{type(e).__name__}: {e}"
    torch.save((ok, why), f"{out_path}.{rank}")
    torch.cuda.synchronize()
    try:
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        pass


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gather(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        ok, why = torch.load(f"{out}.{r}")
        assert ok, why
