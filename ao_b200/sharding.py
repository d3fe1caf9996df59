"""Row sharding of a weight-only quantized linear across the GPUs of one node.

The quantization groups run along K, so the output rows (N) of a weight split cleanly: rank r of p keeps
W[r*N/p : (r+1)*N/p, :] (a multiple of 8 rows for the int4 tensor_core_tiled layout, of 64 for fp6), quantizes it on
its own device, computes y_r = x @ W_r^T from the replicated activation and one all-gather of the outputs assembles y
on every rank.  There is no K sharding (it would need an all-reduce).  One process per GPU; the collective is
torch.distributed's (NCCL over NVLink on GPUs, gloo in the CPU tests of this host logic).
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def row_shard_bounds(n_rows: int, world_size: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """[lo, hi) of rank's rows: blocks of `multiple` rows dealt out as evenly as possible, lower ranks first."""
    if n_rows % multiple != 0:
        raise ValueError(f"{n_rows} rows are not a multiple of {multiple}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    blocks = n_rows // multiple
    base, extra = divmod(blocks, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


def all_gather_rows(y_local: torch.Tensor, n_rows: int, multiple: int = 8, group=None) -> torch.Tensor:
    """Outputs [..., n_local] of every rank -> [..., n_rows] in rank order, on every rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    y_local = y_local.detach()   # inference path: the gather is not differentiated
    sizes = [hi - lo for lo, hi in (row_shard_bounds(n_rows, world, r, multiple) for r in range(world))]
    lead = y_local.shape[:-1]
    if len(set(sizes)) == 1:
        flat = torch.empty(world * y_local.numel(), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(flat, y_local.contiguous().view(-1), group=group)
        out = flat.view((world,) + tuple(lead) + (sizes[0],))
        return out.movedim(0, -2).reshape(*lead, n_rows)
    widest = max(sizes)
    padded = torch.zeros(tuple(lead) + (widest,), dtype=y_local.dtype, device=y_local.device)
    padded[..., : y_local.shape[-1]] = y_local
    flat = torch.empty(world * padded.numel(), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, padded.view(-1), group=group)
    out = flat.view((world,) + tuple(lead) + (widest,))
    return torch.cat([out[r][..., : sizes[r]] for r in range(world)], dim=-1)


class RowShardedLinear(torch.nn.Module):
    """This rank's row shard of a linear layer plus the output all-gather.

    `from_linear` slices the full layer (every rank holds or can build the full weight once), applies
    `quantize_fn(shard)` (e.g. lambda m: quantize(m, int4_weight_only(128))) on the shard only, and forward returns the
    full-width output on every rank."""

    def __init__(self, shard: torch.nn.Linear, out_features: int, multiple: int, group=None, exchange=None,
                 slot_offset_bytes: Optional[int] = None):
        super().__init__()
        self.shard = shard
        self.out_features = out_features
        self.multiple = multiple
        self.group = group
        # optional peer-memory exchange (ao_b200.comm.PeerExchange): decode batches of an int4 tensor_core_tiled shard
        # write their rows into this rank's block of the gathered output and a small kernel stores them into every
        # peer's memory and collects the peers' rows (no NCCL call on the decode path).  Every instance uses call
        # sites of its own (one per batch size): the site at slot_offset_bytes if one is given, else sites reserved
        # from the exchange on first use (every rank then has to run its layers in the same order the first time).
        # The returned tensor is a view of the site's output buffer and is overwritten by this layer's next forward.
        self.exchange = exchange
        self.slot_offset_bytes = slot_offset_bytes
        self._sites = {}

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, multiple: int = 8, group=None,
                    quantize_fn: Optional[Callable[[torch.nn.Module], object]] = None, exchange=None,
                    slot_offset_bytes: Optional[int] = None) -> "RowShardedLinear":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        lo, hi = row_shard_bounds(linear.out_features, world, rank, multiple)
        shard = torch.nn.Linear(linear.in_features, hi - lo, bias=linear.bias is not None, device=linear.weight.device,
                                dtype=linear.weight.dtype)
        with torch.no_grad():
            shard.weight.copy_(linear.weight[lo:hi])
            if linear.bias is not None:
                shard.bias.copy_(linear.bias[lo:hi])
        if quantize_fn is not None:
            quantize_fn(shard)
        return cls(shard, linear.out_features, multiple, group, exchange, slot_offset_bytes)

    def _fused(self, x: torch.Tensor):
        """The fused path, or None when it does not apply (then forward uses the collective)."""
        if self.exchange is None or self.shard.bias is not None or x.dtype != torch.bfloat16 or not x.is_cuda:
            return None
        w = self.shard.weight
        lt = getattr(w, "layout_tensor", None)
        packed = getattr(lt, "packed_weight", None)
        world = self.exchange.world
        if packed is None or self.out_features % world != 0 or self.out_features // world != w.shape[0]:
            return None
        x2 = x.reshape(-1, x.shape[-1])
        if x2.shape[0] > 8 or packed.shape[0] * 8 != w.shape[0] or x2.stride(1) != 1:
            return None
        from . import ops
        M, n_local = x2.shape[0], packed.shape[0] * 8
        site = self._sites.get(M)
        if site is None:
            site = (self.exchange.reserve(M, n_local) if self.slot_offset_bytes is None
                    else self.exchange.site(self.slot_offset_bytes, M, n_local))
            self._sites[M] = site
        # this rank's rows go straight into its block of the gathered output; one small kernel exchanges the blocks
        ops.weight_int4pack_mm(x2, packed, int(w.block_size[1]), lt.scale_and_zero, out=site.y[self.exchange.rank])
        ops.gather_exchange(self.exchange, [site], push=True)
        out = site.y                                                           # [world][M][N / world]
        y = out.reshape(-1) if M == 1 else out.permute(1, 0, 2).reshape(M, -1)
        return y.reshape(*x.shape[:-1], self.out_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._fused(x)
        if y is not None:
            return y
        return all_gather_rows(self.shard(x), self.out_features, self.multiple, self.group)
