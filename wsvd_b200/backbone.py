"""A decode step of a Llama-2-architecture backbone with per-head low-rank K/V, head-sharded.

Per layer, for one new token per sequence (the accuracy pipeline's forward,
fake_quant/svd_utils.py:1628-1674, with the latent cache of the efficiency path):

    xn = RMSNorm(x)
    q  = RoPE(xn @ Wq)                      full-rank query, rotated at the new position
    xk, xv = xn @ A_k, xn @ A_v             down-projection to the per-head latents
    cache <- int8(xk), int8(xv)             quantise-and-append (wsvd_latent_quant_append_i8)
    o  = latent decode attention over len+1 tokens, U_v applied   (the op of this package)
    x  = x + gather_heads(o) @ Wo           heads gathered across ranks, then the o-projection
                                            (o_proj="row": x + all_reduce(o_local @ Wo[rows of the shard]))
    x  = x + SwiGLU FFN(RMSNorm(x))         FFN sharded by columns/rows, all-reduced

Random-init weights and caches; dense projections are torch matmuls (cuBLAS), everything
on the attention path and the element-wise chains (RMSNorm, RoPE, SiLU*up: one kernel each,
`fused_elementwise=False` runs them as the torch chains below instead) are this package's CUDA.  Rank r of g owns heads [r*H/g, (r+1)*H/g),
their A_k/A_v/U_k/U_v/Wq columns and their cache shard.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import ops
from .infer_state import InferState


@dataclass
class BackboneSpec:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    rank_k: int = 64
    rank_v: int = 64
    theta: float = 10000.0


def _rms_norm(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(x.dtype)


def rope_half(q: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotary embedding of q [B, H, D] at per-sequence positions pos [B]."""
    D = q.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, device=q.device, dtype=torch.float32) / D)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    qf = q.float()
    a, b = qf[..., : D // 2], qf[..., D // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(q.dtype)


class _Layer:
    pass


class LatentDecoder:
    """Weights, latent caches and the decode step for this rank's shard."""

    def __init__(self, spec: BackboneSpec, batch: int, context: int, capacity: int, rank: int = 0, world: int = 1,
                 device="cuda", seed: int = 0, peer_gather=None, group=None, o_proj: str = "gather",
                 fused_elementwise: bool = True):
        assert spec.heads % world == 0 and spec.ffn % world == 0
        assert o_proj in ("gather", "row")
        # "gather": all ranks hold Wo and apply it to the gathered heads; "row": every rank applies its
        # heads' rows of Wo to its own heads and the partial products are all-reduced
        self.o_proj = o_proj if world > 1 else "gather"
        self.fused_elementwise = fused_elementwise
        self.spec, self.batch, self.rank, self.world = spec, batch, rank, world
        self.device = torch.device(device)
        self.group, self.pg = group, peer_gather
        Hl = spec.heads // world
        self.local_heads = Hl
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + rank)
        dt = torch.float16
        dev = self.device

        def gauss(rows, cols, std):
            return (torch.randn(rows, cols, generator=gen, device=dev, dtype=torch.float32) * std).to(dt)

        def ortho(rank_r):
            a = torch.randn(Hl, spec.head_dim, rank_r, generator=gen, device=dev, dtype=torch.float32)
            qf, _ = torch.linalg.qr(a)
            return qf.permute(2, 0, 1).reshape(rank_r, Hl * spec.head_dim).to(dt).contiguous()

        s = 1.0 / math.sqrt(spec.hidden)
        self.layers: List[_Layer] = []
        S = capacity
        for _ in range(spec.layers):
            L = _Layer()
            L.Wq = gauss(spec.hidden, Hl * spec.head_dim, s)
            L.A_k = gauss(spec.hidden, Hl * spec.rank_k, s)
            L.A_v = gauss(spec.hidden, Hl * spec.rank_v, s)
            L.wk, L.wv = ortho(spec.rank_k), ortho(spec.rank_v)
            L.Wo = gauss(spec.heads * spec.head_dim, spec.hidden, s)  # replicated: applied to the gathered heads
            if self.o_proj == "row":  # keep only this rank's rows
                L.Wo = L.Wo[rank * Hl * spec.head_dim:(rank + 1) * Hl * spec.head_dim].contiguous()
            L.Wup = gauss(spec.hidden, spec.ffn // world, s)
            L.Wgate = gauss(spec.hidden, spec.ffn // world, s)
            # one GEMM for the three projections of the normalised input, one for up | gate: the
            # weights live concatenated and the separate names are column slices of them
            L.Wqkv = torch.cat([L.Wq, L.A_k, L.A_v], dim=1).contiguous()
            L.Wug = torch.cat([L.Wup, L.Wgate], dim=1).contiguous()
            nq, nk, nf = L.Wq.shape[1], L.A_k.shape[1], L.Wup.shape[1]
            L.Wq, L.A_k, L.A_v = L.Wqkv[:, :nq], L.Wqkv[:, nq:nq + nk], L.Wqkv[:, nq + nk:]
            L.Wup, L.Wgate = L.Wug[:, :nf], L.Wug[:, nf:]
            L.Wdown = gauss(spec.ffn // world, spec.hidden, 1.0 / math.sqrt(spec.ffn))
            # head-major latent cache [B, Hl, S, R] seen as the token-major strided view the op takes
            L.k_store = torch.randint(-127, 128, (batch, Hl, S, spec.rank_k), generator=gen, device=dev,
                                      dtype=torch.int8)
            L.v_store = torch.randint(-127, 128, (batch, Hl, S, spec.rank_v), generator=gen, device=dev,
                                      dtype=torch.int8)
            L.ks_store = (torch.rand(batch, Hl, S, generator=gen, device=dev) * 0.02 + 0.02).to(dt)
            L.vs_store = (torch.rand(batch, Hl, S, generator=gen, device=dev) * 0.02 + 0.02).to(dt)
            T = (batch - 1) * Hl * S + S
            L.lk = L.k_store.as_strided((T, Hl, spec.rank_k), (spec.rank_k, S * spec.rank_k, 1))
            L.lv = L.v_store.as_strided((T, Hl, spec.rank_v), (spec.rank_v, S * spec.rank_v, 1))
            L.ks = L.ks_store.as_strided((T, Hl), (1, S))
            L.vs = L.vs_store.as_strided((T, Hl), (1, S))
            self.layers.append(L)
        table = (torch.arange(batch, dtype=torch.int64)[:, None] * (Hl * S) + torch.arange(S, dtype=torch.int64)[None, :])
        assert int(table.max()) < 2 ** 31
        self.before = InferState(batch, capacity, [context] * batch, device=dev, req_to_token=table.to(torch.int32))
        self.after = InferState(batch, capacity, [context + 1] * batch, device=dev,
                                req_to_token=self.before.req_manager.req_to_token_indexs)
        self.after.max_len_in_batch = context + 1
        self.before.max_len_in_batch = context
        self.context, self.capacity = context, capacity
        self.out_local = torch.empty(batch, Hl, spec.head_dim, dtype=dt, device=dev)
        self.gathered = (torch.empty(world, batch, Hl, spec.head_dim, dtype=dt, device=dev)
                         if world > 1 and peer_gather is None and self.o_proj == "gather" else None)
        self.workspace = None
        self.inv_freq = spec.theta ** (-torch.arange(0, spec.head_dim, 2, device=dev, dtype=torch.float32)
                                       / spec.head_dim)

    def attention_bytes(self) -> int:
        """Algorithmic latent+scale bytes one step reads on this rank (all layers)."""
        sp = self.spec
        return self.spec.layers * self.batch * self.local_heads * (self.context + 1) * (sp.rank_k + sp.rank_v + 4)

    def weight_bytes(self) -> int:
        n = 0
        for L in self.layers[:1]:
            for w in (L.Wq, L.A_k, L.A_v, L.wk, L.wv, L.Wo, L.Wup, L.Wgate, L.Wdown):
                n += w.numel() * 2
        return n * self.spec.layers

    def _attend(self, L, q):
        sp = self.spec
        if self.o_proj == "row":
            o = ops.latent_decode(q, self.after, L.lk, L.ks, L.lv, L.vs, L.wk, None, wv=L.wv, out=self.out_local,
                                  workspace=self.workspace)
            return o.reshape(self.batch, self.local_heads * sp.head_dim)
        if self.pg is not None:
            full = self.pg.decode(q, self.after, L.lk, L.ks, L.lv, L.vs, L.wk, None, wv=L.wv,
                                  workspace=self.workspace)
            return full.reshape(self.batch, sp.heads * sp.head_dim)
        o = ops.latent_decode(q, self.after, L.lk, L.ks, L.lv, L.vs, L.wk, None, wv=L.wv, out=self.out_local,
                              workspace=self.workspace)
        if self.world == 1:
            return o.reshape(self.batch, sp.heads * sp.head_dim)
        import torch.distributed as dist

        dist.all_gather_into_tensor(self.gathered, o, group=self.group)
        return self.gathered.permute(1, 0, 2, 3).reshape(self.batch, sp.heads * sp.head_dim)

    @torch.no_grad()
    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x [B, hidden] f16 -> [B, hidden]; appends one token per sequence to every layer's cache
        at position `context` (the caller advances the lengths with `advance()`)."""
        sp = self.spec
        B, Hl = self.batch, self.local_heads
        if self.workspace is None:
            L0 = self.layers[0]
            q0 = torch.zeros(B, Hl, sp.head_dim, dtype=torch.float16, device=self.device)
            p, _ = ops.build_params(q0, self.after.b_seq_len, self.after.b_req_idx,
                                    self.after.req_manager.req_to_token_indexs, self.capacity, L0.lk, L0.ks, L0.lv,
                                    L0.vs, L0.wk, None, wv=L0.wv)
            # the split plan (where one is used) depends on max_len: take the largest request over the
            # lengths this decoder can run at
            need = 0
            for max_len in sorted({self.capacity, *range(max(1, self.context), self.capacity + 1, 128)}):
                p.max_len = max_len
                need = max(need, ops.workspace_bytes(p))
            self.workspace = torch.empty((need + 3) // 4, dtype=torch.float32, device=self.device)
        pos = self.before.b_seq_len
        fe = self.fused_elementwise
        if self.world > 1:
            import torch.distributed as dist
        xn = ops.rms_norm(x) if fe else None  # later layers get theirs from the residual add of the FFN
        for L in self.layers:
            if fe:
                qkv = xn @ L.Wqkv  # [B, Hl*D | Hl*Rk | Hl*Rv]: the three outputs are column slices
                nq, nk = Hl * sp.head_dim, Hl * sp.rank_k
                q = ops.rope_half_(qkv[:, :nq].unflatten(1, (Hl, sp.head_dim)), pos, self.inv_freq)
                xk = qkv[:, nq:nq + nk].unflatten(1, (Hl, sp.rank_k))
                xv = qkv[:, nq + nk:].unflatten(1, (Hl, sp.rank_v))
            else:
                xn = _rms_norm(x)
                q = rope_half((xn @ L.Wq).view(B, Hl, sp.head_dim), pos, sp.theta)
                xk = (xn @ L.A_k).view(B, Hl, sp.rank_k)
                xv = (xn @ L.A_v).view(B, Hl, sp.rank_v)
            ops.latent_quant_append(xk, xv, self.before, L.lk, L.ks, L.lv, L.vs)
            o = self._attend(L, q)
            a = o @ L.Wo
            if self.o_proj == "row":
                dist.all_reduce(a, group=self.group)
            if fe:
                x, h = ops.add_rms_norm(x, a)  # residual add + the FFN's normalisation
                ug = h @ L.Wug
                nf = L.Wup.shape[1]
                f = ops.silu_mul(ug[:, :nf], ug[:, nf:]) @ L.Wdown
            else:
                x = x + a
                h = _rms_norm(x)
                f = ((h @ L.Wup) * torch.nn.functional.silu(h @ L.Wgate)) @ L.Wdown
            if self.world > 1:
                dist.all_reduce(f, group=self.group)
            if fe:
                x, xn = ops.add_rms_norm(x, f)  # residual add + the next layer's normalisation
            else:
                x = x + f
        return x

    def capture(self, x: torch.Tensor):
        """Capture `step(x)` followed by the length update in a CUDA graph.  The split plan is
        made for the cache capacity, so one graph serves every later step.  With several ranks
        the head gather has to be the fused one with its epoch on the device
        (`PeerGather(device_epoch=True)`); the FFN's NCCL all-reduce is captured as it is.  Returns (graph, output tensor); replay
        with graph.replay() after writing the new input into x."""
        assert self.world == 1 or self.o_proj == "row" or (self.pg is not None and self.pg.device_epoch)
        self.before.max_len_in_batch = self.capacity
        self.after.max_len_in_batch = self.capacity
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm-up: workspace, position table, cuBLAS handles
            self.step(x)
            self._advance_device()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y = self.step(x)
            self._advance_device(host=False)  # recorded, not run: the caller counts replays in self.context
        return graph, y

    def _advance_device(self, host: bool = True):
        if host:
            self.context += 1
        self.before.b_seq_len += 1
        self.after.b_seq_len += 1

    def advance(self):
        """Make the appended token part of the context (needs capacity for the next one)."""
        self.context += 1
        assert self.context + 1 <= self.capacity
        self.before.b_seq_len += 1
        self.after.b_seq_len += 1
        self.before.max_len_in_batch = self.context
        self.after.max_len_in_batch = self.context + 1
