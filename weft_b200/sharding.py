"""Row sharding of a weight matrix across the GPUs of one node.

The path shards naturally: every output column n depends on weight row n only
(``for column in range(N): Y[row, column] = vec_dot(W[column], Xq[row])``,
examples/kernels/mul_mat/q4_k_decode.py:17-20 of the reference), and K is never split, so each output
element is computed wholly on one GPU and results are bit-identical for any number of GPUs.

Rank r of g holds the contiguous row block [N*r/g, N*(r+1)/g) of W -- a contiguous byte range of the
record array, i.e. a view, not a repack -- and a replica of the (small) activations.  After the local
mul_mat the fp32 outputs are all-gathered: here with ``torch.distributed.all_gather_into_tensor`` (NCCL over
NVLink on GPUs, gloo in the CPU tests); ``weft_b200.peers`` + ``weft_b200_mul_mat_shard_gather`` do the same
gather inside the library's own kernels over peer memory, which is what ``bench.py`` times by default.
One process per GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .formats import row_bytes


@dataclass(frozen=True)
class RowShard:
    """Rows [begin, end) of an (n, k) matrix of ``encoding`` records, owned by ``rank`` of ``world``."""
    rank: int
    world: int
    n: int
    k: int
    encoding: str
    begin: int
    end: int

    @property
    def rows(self) -> int:
        return self.end - self.begin

    @property
    def byte_range(self) -> tuple[int, int]:
        pitch = row_bytes(self.encoding, self.k)
        return self.begin * pitch, self.end * pitch


def plan(n: int, k: int, encoding: str, world: int) -> list[RowShard]:
    """Contiguous, near-equal row blocks; every rank gets floor or ceil of n / world rows."""
    if world < 1:
        raise ValueError("world size must be positive")
    row_bytes(encoding, k)      # validates K against the record size
    return [RowShard(r, world, n, k, encoding, n * r // world, n * (r + 1) // world) for r in range(world)]


def shard_of(n: int, k: int, encoding: str, rank: int, world: int) -> RowShard:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    return plan(n, k, encoding, world)[rank]


def sharded_mul_mat(shard: RowShard, m: int, local_mul_mat: Callable, *, group=None):
    """Run ``local_mul_mat(y_local)`` (which must fill the (m, shard.rows) tensor it is handed with this
    rank's output columns) and assemble the full (m, n) result on every rank.

    Returns the (m, n) tensor.  Ranks with unequal row counts are padded to the largest block for the
    collective and trimmed afterwards, so any n works with any world size.
    """
    import torch
    import torch.distributed as dist

    plans = plan(shard.n, shard.k, shard.encoding, shard.world)
    widest = max(p.rows for p in plans)
    device = _device_for(group)
    y_local = torch.zeros((m, widest), dtype=torch.float32, device=device)
    local_mul_mat(y_local[:, : shard.rows] if shard.rows == widest else y_local.narrow(1, 0, shard.rows))
    if shard.world == 1:
        return y_local[:, : shard.rows]
    flat = torch.empty((shard.world * m, widest), dtype=torch.float32, device=device)   # rank-major concatenation
    dist.all_gather_into_tensor(flat, y_local, group=group)
    gathered = flat.view(shard.world, m, widest)
    return torch.cat([gathered[p.rank, :, : p.rows] for p in plans], dim=1)


def _device_for(group):
    import torch
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_backend(group) == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")
