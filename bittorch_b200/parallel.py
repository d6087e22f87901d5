"""Column-parallel sharding of a packed ternary linear layer across the GPUs of one box.

The reference has no distributed code; this is the multi-GPU form of its packed inference
layer (bittorch/nn/ternary_linear_infer.py): output columns are independent, so rank r of p
owns columns [r*N/p, (r+1)*N/p) of the weight as its own contiguous packed buffer
[ceil(K/4), N/p] plus the matching scale / bias slices, the activations are replicated,
and one all-gather of the [M, N/p] outputs (NCCL over NVLink) rebuilds [M, N].  It pays off
only where the weight stream dominates the gather, i.e. decode-sized batches
(ceil(K/4)*N/p bytes of weights against 2*M*N bytes gathered).
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor


def column_range(out_features: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Columns owned by ``rank``; ``out_features`` must divide evenly so that the
    all-gather moves equal pieces."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if out_features % world_size != 0:
        raise ValueError(f"out_features={out_features} is not divisible by world_size={world_size}")
    per = out_features // world_size
    return rank * per, (rank + 1) * per


def shard_packed_columns(weight_packed: Tensor, scale: Tensor, bias: Optional[Tensor], rank: int, world_size: int):
    """Materialises rank's column shard of the public packed buffer (a column slice of
    [ceil(K/4), N] is strided, so it is copied once at load) and of scale / bias."""
    n = weight_packed.shape[1]
    n0, n1 = column_range(n, rank, world_size)
    return (weight_packed[:, n0:n1].contiguous(), scale[n0:n1].contiguous(),
            None if bias is None else bias[n0:n1].contiguous())


class ColumnParallelTernaryLinear(nn.Module):
    """One rank's shard of a packed ternary linear layer + the output all-gather.

    ``local_linear(x2d) -> [M, N/p]`` computes the shard; by default it is a
    ``TernaryLinearInference`` on the shard's buffers (CUDA kernels).  Tests of the host
    logic on CPU ranks inject their own callable.
    """

    def __init__(self, in_features: int, out_features: int, weight_packed_shard: Tensor, scale_shard: Tensor,
                 bias_shard: Optional[Tensor] = None, group: Optional[dist.ProcessGroup] = None,
                 local_linear: Optional[Callable[[Tensor], Tensor]] = None) -> None:
        super().__init__()
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features = in_features
        self.out_features = out_features
        n0, n1 = column_range(out_features, self.rank, self.world_size)
        if weight_packed_shard.shape != ((in_features + 3) // 4, n1 - n0):
            raise ValueError(f"shard has shape {tuple(weight_packed_shard.shape)}, expected "
                             f"{((in_features + 3) // 4, n1 - n0)}")
        if local_linear is None:
            from .nn import TernaryLinearInference
            self.local = TernaryLinearInference(in_features, n1 - n0, weight_packed_shard, scale_shard, bias_shard)
            self._local_fn = self.local
        else:
            self.register_buffer("weight_packed", weight_packed_shard)
            self.register_buffer("scale", scale_shard)
            self.register_buffer("bias", bias_shard)
            self._local_fn = local_linear

    @classmethod
    def from_full(cls, in_features: int, weight_packed: Tensor, scale: Tensor, bias: Optional[Tensor] = None,
                  group: Optional[dist.ProcessGroup] = None, local_linear=None) -> "ColumnParallelTernaryLinear":
        """Every rank holds (or loads) the full buffers and keeps only its columns."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        wp, sc, b = shard_packed_columns(weight_packed, scale, bias, rank, world)
        return cls(in_features, weight_packed.shape[1], wp, sc, b, group, local_linear)

    def forward(self, x: Tensor) -> Tensor:
        """x: (*, in_features), identical on every rank -> (*, out_features) on every rank."""
        x2d = x.reshape(-1, self.in_features)
        y_local = self._local_fn(x2d).contiguous()
        if self.world_size == 1:
            return y_local.reshape(*x.shape[:-1], self.out_features)
        m, per = y_local.shape
        gathered = torch.empty((self.world_size * m, per), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, y_local, group=self.group)      # rank-major: [p][m][N/p]
        y = gathered.view(self.world_size, m, per).permute(1, 0, 2).reshape(m, self.out_features)
        return y.reshape(*x.shape[:-1], self.out_features)
