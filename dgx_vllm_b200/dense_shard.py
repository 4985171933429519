"""Dense NVFP4 linear layer split by output columns over the ranks of a process group.

Rank r keeps rows [r*N/G, (r+1)*N/G) of the weight (packed codes and their block-scale rows); the
activation is replicated and every rank quantizes it itself (the quantizer is cheaper than moving
codes and scales), so the matmul needs no exchange.  `gather=True` appends one all-gather of the
output column blocks over NCCL.  N/G must be a multiple of 128 so that no 128-row tile of the
swizzled scale-factor layout straddles two shards.

The reference has no multi-GPU code of its own (it serves through vLLM's tensor parallelism,
entrypoint.sh:100-116); this is the column-parallel layout vLLM uses for such a layer.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the weight rows (= output columns) rank `rank` owns."""
    if N % world != 0 or (N // world) % 128 != 0:
        raise RuntimeError("N / world must be a multiple of 128")
    per = N // world
    return rank * per, (rank + 1) * per


class ColumnShardedNvfp4Linear:
    """y[:, shard] = x @ W[shard]^T with W[shard] in NVFP4.

    `weight_bf16` is this rank's [N/G, K] slice (quantized here with `weight_global_scale`, which
    must be the scale of the WHOLE weight so that all shards decode alike), or pass pre-quantized
    `codes`/`sf`.  `local_fn(x, self) -> [M, N/G]`, when given, replaces the CUDA ops (CPU ranks in tests)."""

    def __init__(self, N: int, weight_global_scale: torch.Tensor, weight_bf16: Optional[torch.Tensor] = None,
                 codes: Optional[torch.Tensor] = None, sf: Optional[torch.Tensor] = None, group=None,
                 local_fn: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = N
        self.begin, self.end = shard_rows(N, self.world, self.rank)
        self.gw = weight_global_scale
        self._fn = local_fn
        self._alpha = None          # (x_global_scale tensor, its version, alpha) of the last call
        if local_fn is None:
            from .ops import scaled_fp4_quant
            if codes is None:
                if weight_bf16 is None or weight_bf16.shape[0] != self.end - self.begin:
                    raise RuntimeError("weight_bf16 must be this rank's [N/G, K] slice")
                codes, sf = scaled_fp4_quant(weight_bf16, weight_global_scale)
            self.codes, self.sf = codes, sf
        else:
            self.codes, self.sf = codes, sf

    def forward(self, x: torch.Tensor, x_global_scale: torch.Tensor, gather: bool = False) -> torch.Tensor:
        if self._fn is not None:
            y = self._fn(x, self)
        else:
            from .ops import nvfp4_linear
            a = self._alpha
            if a is None or a[0] is not x_global_scale or a[1] != x_global_scale._version:
                a = (x_global_scale, x_global_scale._version, (1.0 / (x_global_scale * self.gw)).to(torch.float32))
                self._alpha = a
            alpha = a[2]
            y = nvfp4_linear(x, x_global_scale, self.codes, self.sf, alpha)      # quantizer + GEMM in one library call
        if not gather or self.world == 1:
            return y
        parts = [torch.empty_like(y) for _ in range(self.world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)
