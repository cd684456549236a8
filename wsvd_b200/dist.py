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


class _DeviceArray:
    """Raw device memory as something torch.as_tensor can wrap (CUDA array interface)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


class PeerGather:
    """Head-sharded decode whose all-gather is fused into the op's own kernels.

    Every rank owns two gathered output buffers [B, H_total, D] f16 (used alternately, by step
    parity), a flag array and a block counter in memory that the other ranks map through
    CUDA IPC.  `decode(...)` runs this rank's shard; the kernel that finishes a row stores it into
    all ranks' buffers over NVLink and runs the group barrier in its last block, so when
    the returned tensor is read on the same stream it holds every rank's heads.  No NCCL
    call is made per step; torch.distributed is used once, to exchange the handles.

    `device_epoch=True` keeps the step count on the device and always uses the first buffer, so
    the argument block never changes and `decode` can be captured in a CUDA graph.  With one
    buffer the caller has to keep a group synchronisation between consecutive steps (in the
    decoder backbone the all-reduce of the FFN output is one): otherwise a fast rank could
    overwrite rows that a slow rank has not read yet.
    """

    def __init__(self, batch: int, heads_total: int, head_dim: int, group=None, device=None, timeout_ms: int = 0,
                 device_epoch: bool = False):
        import ctypes

        from . import _lib

        self._lib, self._ct = _lib, ctypes
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks")
        self.shard = head_shard(heads_total, self.rank, self.world)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shape = (int(batch), int(heads_total), int(head_dim))
        self.timeout_ms = int(timeout_ms)
        self.device_epoch = bool(device_epoch)
        out_bytes = batch * heads_total * head_dim * 2
        self._out_bytes = (out_bytes + 255) // 256 * 256
        total = 2 * self._out_bytes + 256  # two buffers | flags (MAX_PEERS u32) | counter
        lib = _lib.lib()
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _lib.check(lib.wsvd_peer_alloc(total, ctypes.byref(base)), "wsvd_peer_alloc")
            self._base = base.value
            handle = ctypes.create_string_buffer(_lib.PEER_HANDLE_BYTES)
            _lib.check(lib.wsvd_peer_export(ctypes.c_void_p(self._base), handle), "wsvd_peer_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self._bases = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._bases.append(self._base)
                    continue
                mapped = ctypes.c_void_p()
                _lib.check(lib.wsvd_peer_import(h, ctypes.byref(mapped)), "wsvd_peer_import")
                self._bases.append(mapped.value)
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone stores
        self.epoch = 0

    def buffer(self, parity: int) -> torch.Tensor:
        """This rank's gathered buffer [B, H_total, D] of the given step parity."""
        arr = _DeviceArray(self._base + parity * self._out_bytes, self.shape, "<f2")
        return torch.as_tensor(arr, device=self.device)

    def peer_set(self):
        """The argument block of the next step (advances the epoch)."""
        if self.device_epoch:
            parity = 0
        else:
            self.epoch += 1
            parity = self.epoch & 1
        ps = self._lib.PeerSet()
        for r, b in enumerate(self._bases):
            ps.out[r] = b + parity * self._out_bytes
            ps.flags[r] = b + 2 * self._out_bytes
        ps.counter = self._base + 2 * self._out_bytes + 128
        ps.n_peers, ps.rank, ps.head_offset = self.world, self.rank, self.shard.start
        ps.epoch = self.epoch
        if self.device_epoch:
            ps.epoch_counter = self._base + 2 * self._out_bytes + 192
        B, H, D = self.shape
        ps.out_stride_b, ps.out_stride_h = H * D, D
        ps.timeout_ms = self.timeout_ms
        return ps, parity

    def decode(self, q_local, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale=None, *, wv=None,
               **kw) -> torch.Tensor:
        """One step on this rank's heads; returns the gathered [B, H_total, D] buffer (valid in
        stream order; it is overwritten two steps later)."""
        from . import ops

        if wv is None and self.shape[2] != latent_v.shape[-1]:
            raise ValueError("without wv the gathered width must be rank_v")
        ps, parity = self.peer_set()
        ops.latent_decode_gather(q_local, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, ps, wv=wv,
                                 **kw)
        return self.buffer(parity)

    def close(self):
        if getattr(self, "_base", None) is None:
            return
        lib = self._lib.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody still stores into a buffer that is about to go
        with torch.cuda.device(self.device):
            for r, b in enumerate(self._bases):
                if r != self.rank:
                    lib.wsvd_peer_release(self._ct.c_void_p(b))
            lib.wsvd_peer_free(self._ct.c_void_p(self._base))
        self._base = None
