"""Head-sharded (tensor-parallel style) decode attention on the GPUs of one node.

Every (sequence, head) pair is independent in this op, so rank r of g owns the heads
[r*H/g, (r+1)*H/g) together with their latent caches and U_k/U_v slices; nothing moves
during attention.  The one exchange is an all-gather of the per-rank outputs
[B, H/g, D] into [B, H, D].  One process per GPU, torch.distributed (NCCL on GPUs; the
host-side logic is backend-agnostic and is tested with gloo on CPU)."""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def head_shard(n_heads: int, rank: int, world: int) -> slice:
    """Contiguous slice of heads owned by `rank`; heads must divide evenly."""
    if n_heads % world != 0:
        raise ValueError(f"{n_heads} heads do not divide over {world} ranks")
    per = n_heads // world
    return slice(rank * per, (rank + 1) * per)


def gather_heads(out_local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather [B, H_local, D] shards (rank-major head order) into [B, H, D].

    The gather dimension is not outermost, so ranks are gathered into [g, B, H_local, D]
    and viewed as [B, g*H_local, D] with one permute+copy."""
    world = dist.get_world_size(group)
    B, Hl, D = out_local.shape
    stage = torch.empty(world, B, Hl, D, dtype=out_local.dtype, device=out_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(stage, out_local.contiguous(), group=group)
    else:  # gloo (CPU tests) gathers into per-rank views of the same staging tensor
        dist.all_gather([stage[r] for r in range(world)], out_local.contiguous(), group=group)
    full = stage.permute(1, 0, 2, 3).reshape(B, world * Hl, D)
    if out is not None:
        out.copy_(full)
        return out
    return full


def sharded_decode(op: Callable[..., torch.Tensor], *op_args, group=None, **op_kwargs) -> torch.Tensor:
    """Run `op` (one of the decode-attention ops of this package, called with this rank's
    head shard) and all-gather the heads."""
    return gather_heads(op(*op_args, **op_kwargs), group=group)
