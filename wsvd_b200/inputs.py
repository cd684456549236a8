"""Seeded synthetic inputs for the latent decode-attention op.

The decode-attention workloads are defined by shapes and value distributions only
(image and text tokens are indistinguishable to decode attention), so seeded synthetic
tensors stand in for LLaVA prompts: pre-quantisation latents ~ N(0,1), symmetric int8
per (token, head) with an f16 scale = max|x|/127 (fake_quant/quant_utils.py:30-33,
179-184), U_k/U_v = orthonormal columns from the QR of a seeded Gaussian, q ~ N(0,1).

Storage is head-major [B, H, S, R] (each (b, h) stream contiguous); the op sees it through
the reference's token-major interface [T, Hkv, R] + page table as a strided view:
stride_t = R, stride_h = S*R, req_to_token[b][s] = b*H*S + s.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .infer_state import InferState


@dataclass
class WorkloadSpec:
    name: str
    batch: int
    heads: int
    head_dim: int
    rank_k: int
    rank_v: int
    max_len: int
    len_lo: int  # per-sequence length ~ U[len_lo, len_hi] (seeded); equal => fixed
    len_hi: int
    seed: int
    note: str = ""


# The single-layer decode-attention workloads (shapes of LLaVA-1.5-7B/13B, LLaVA-Next-7B
# and a long-context 13B case).
WORKLOADS = {
    "c1_7b_b1_s2048": WorkloadSpec("c1_7b_b1_s2048", 1, 32, 128, 64, 64, 2048, 2048, 2048, 101,
                                   "LLaVA-1.5-7B shape, 576 image + 1472 text tokens"),
    "c2_13b_b16_s8192": WorkloadSpec("c2_13b_b16_s8192", 16, 40, 128, 64, 64, 8192, 8192, 8192, 102,
                                     "LLaVA-1.5-13B shape"),
    "c3_next7b_b32_ragged4096": WorkloadSpec("c3_next7b_b32_ragged4096", 32, 32, 128, 64, 64, 4096, 3000, 4096, 103,
                                             "LLaVA-Next-7B shape, ragged"),
    "c4_13b_b64_ragged32k": WorkloadSpec("c4_13b_b64_ragged32k", 64, 40, 128, 64, 48, 32768, 1024, 32768, 104,
                                         "long-context 13B shape, rank_v 48, ragged"),
}


def seq_lens_for(spec: WorkloadSpec) -> List[int]:
    if spec.len_lo == spec.len_hi:
        return [spec.len_hi] * spec.batch
    g = torch.Generator().manual_seed(spec.seed)
    return torch.randint(spec.len_lo, spec.len_hi + 1, (spec.batch,), generator=g).tolist()


def algorithmic_bytes(seq_lens: Sequence[int], heads: int, rank_k: int, rank_v: int, latent_bytes: int = 1) -> int:
    """Latent + scale bytes the op must read: sum_b len_b * H * (Rk + Rv + 2 + 2) for int8."""
    per = (rank_k + rank_v) * latent_bytes + (4 if latent_bytes == 1 else 0)
    return int(sum(seq_lens)) * heads * per


@dataclass
class DecodeCase:
    q: torch.Tensor                 # [B, Hq, D] f16
    latent_k: torch.Tensor          # view [T, Hkv, Rk] int8 (or f16)
    k_scale: Optional[torch.Tensor]  # view [T, Hkv] f16
    latent_v: torch.Tensor
    v_scale: Optional[torch.Tensor]
    wk: torch.Tensor                # [Rk, Hkv*D] f16
    wv: torch.Tensor                # [Rv, Hkv*D] f16
    infer_state: InferState
    seq_lens: List[int]
    storage: dict = field(default_factory=dict)  # the head-major tensors the views alias

    def to(self, device) -> "DecodeCase":
        """Copy to `device`, re-deriving the strided views over the copied storage."""
        if not self.storage:  # token-major copy: plain tensors, no aliasing views
            s = self.infer_state
            state = InferState(s.batch_size, s.max_len_in_batch, self.seq_lens, device=device,
                               req_to_token=s.req_manager.req_to_token_indexs, b_req_idx=s.b_req_idx)
            mv = lambda t: None if t is None else t.to(device)
            return DecodeCase(self.q.to(device), mv(self.latent_k), mv(self.k_scale), mv(self.latent_v),
                              mv(self.v_scale), self.wk.to(device), self.wv.to(device), state, self.seq_lens, {})
        st = {k: v.to(device) for k, v in self.storage.items()}
        return _assemble(st, self.q.to(device), self.wk.to(device), self.wv.to(device), self.seq_lens,
                         self.infer_state.max_len_in_batch, device)

    def oracle_args(self):
        s = self.infer_state
        return (self.q, s.b_seq_len, s.b_req_idx, s.req_manager.req_to_token_indexs, self.latent_k, self.k_scale,
                self.latent_v, self.v_scale, self.wk)


def _token_view(x: torch.Tensor) -> torch.Tensor:
    """[B, H, S, R] head-major storage -> [T, H, R] token-major strided view, T=(B-1)*H*S+S."""
    B, H, S, R = x.shape
    return x.as_strided(((B - 1) * H * S + S, H, R), (R, S * R, 1))


def _scale_view(x: torch.Tensor) -> torch.Tensor:
    B, H, S = x.shape
    return x.as_strided(((B - 1) * H * S + S, H), (1, S))


def _assemble(st, q, wk, wv, seq_lens, max_len, device) -> DecodeCase:
    B, H, S, _ = st["latent_k"].shape
    table = (torch.arange(B, dtype=torch.int64)[:, None] * (H * S) + torch.arange(S, dtype=torch.int64)[None, :])
    assert int(table.max()) < 2 ** 31
    state = InferState(B, max_len, seq_lens, device=device, req_to_token=table.to(torch.int32))
    ks = st.get("k_scale")
    vs = st.get("v_scale")
    return DecodeCase(
        q=q, latent_k=_token_view(st["latent_k"]), k_scale=None if ks is None else _scale_view(ks),
        latent_v=_token_view(st["latent_v"]), v_scale=None if vs is None else _scale_view(vs),
        wk=wk, wv=wv, infer_state=state, seq_lens=list(seq_lens), storage=st)


def _quantize(x: torch.Tensor):
    """scale = amax/127 stored f16 (1 where the row is zero); q = clamp(round(x/scale_f16))."""
    amax = x.abs().amax(dim=-1)
    scale = torch.where(amax == 0, torch.ones_like(amax), amax / 127.0).to(torch.float16)
    q = torch.clamp(torch.round(x / scale.float().unsqueeze(-1)), -128, 127).to(torch.int8)
    return q, scale


def _orthonormal(gen, heads, head_dim, rank, device):
    a = torch.randn(heads, head_dim, rank, generator=gen, device=device, dtype=torch.float32)
    qf, _ = torch.linalg.qr(a)  # [H, D, R], orthonormal columns
    # reference weight layout: w[r, h*D + d] = U[h, d, r]
    return qf.permute(2, 0, 1).reshape(rank, heads * head_dim).to(torch.float16).contiguous()


def make_case(batch, heads, head_dim, rank_k, rank_v, seq_lens: Sequence[int], max_len: int, seed: int,
              device="cpu", latent_dtype=torch.int8, poison: bool = True) -> DecodeCase:
    """Build one seeded case.  Generation happens on `device` with a generator seeded
    there (CPU generation is device-independent and is what the parity tests use; large
    benchmark workloads generate directly on the GPU, one sequence at a time)."""
    assert len(seq_lens) == batch and max(seq_lens, default=0) <= max_len
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(batch, heads, head_dim, generator=gen, device=dev).to(torch.float16)
    wk = _orthonormal(gen, heads, head_dim, rank_k, dev)
    wv = _orthonormal(gen, heads, head_dim, rank_v, dev)
    S = max_len
    st = {}
    if latent_dtype == torch.int8:
        st["latent_k"] = torch.empty(batch, heads, S, rank_k, dtype=torch.int8, device=dev)
        st["latent_v"] = torch.empty(batch, heads, S, rank_v, dtype=torch.int8, device=dev)
        st["k_scale"] = torch.empty(batch, heads, S, dtype=torch.float16, device=dev)
        st["v_scale"] = torch.empty(batch, heads, S, dtype=torch.float16, device=dev)
    else:
        st["latent_k"] = torch.empty(batch, heads, S, rank_k, dtype=torch.float16, device=dev)
        st["latent_v"] = torch.empty(batch, heads, S, rank_v, dtype=torch.float16, device=dev)
    for b in range(batch):
        n = int(seq_lens[b])
        for name, rank in (("k", rank_k), ("v", rank_v)):
            x = torch.randn(heads, n, rank, generator=gen, device=dev, dtype=torch.float32)
            lat = st["latent_" + name]
            if latent_dtype == torch.int8:
                qx, sc = _quantize(x)
                lat[b, :, :n] = qx
                st[name + "_scale"][b, :, :n] = sc
                if poison:  # padding slots must never be read
                    lat[b, :, n:] = -128
                    st[name + "_scale"][b, :, n:] = float("nan")
            else:
                lat[b, :, :n] = x.to(torch.float16)
                if poison:
                    lat[b, :, n:] = float("nan")
    return _assemble(st, q, wk, wv, seq_lens, max_len, dev)


def make_workload(spec: WorkloadSpec, device="cuda", heads: Optional[slice] = None) -> DecodeCase:
    """A named workload; `heads` selects a head shard (rank r of g owns a contiguous
    slice of heads) without generating the other heads' caches."""
    lens = seq_lens_for(spec)
    if heads is None:
        return make_case(spec.batch, spec.heads, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len,
                         spec.seed, device)
    n_local = len(range(*heads.indices(spec.heads)))
    # a shard is generated with its own seed stream; shards are independent workloads
    return make_case(spec.batch, n_local, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len,
                     spec.seed * 1000 + heads.indices(spec.heads)[0], device)


def padded_rank_copy(case: DecodeCase, rank_k: int, rank_v: int) -> DecodeCase:
    """The same case with its latents and up-projection factors zero-padded to (rank_k, rank_v):
    how a cache of rank 62 (the accuracy pipeline's uniform rank) is stored to reach the
    tensor-core path, which takes ranks that are multiples of 16.  The padded ranks contribute
    exact zeros, so the result is unchanged."""
    st = case.storage
    assert st, "needs the head-major storage of make_case"
    B, H, S, Rk = st["latent_k"].shape
    Rv = st["latent_v"].shape[3]
    assert rank_k >= Rk and rank_v >= Rv
    pad = torch.nn.functional.pad
    st2 = dict(st)
    st2["latent_k"] = pad(st["latent_k"], (0, rank_k - Rk)).contiguous()
    st2["latent_v"] = pad(st["latent_v"], (0, rank_v - Rv)).contiguous()
    wk = pad(case.wk, (0, 0, 0, rank_k - Rk)).contiguous()
    wv = pad(case.wv, (0, 0, 0, rank_v - Rv)).contiguous()
    return _assemble(st2, case.q, wk, wv, case.seq_lens, case.infer_state.max_len_in_batch, st["latent_k"].device)


def token_major_copy(case: DecodeCase, shuffle_seed: Optional[int] = None, page_size: int = 1) -> DecodeCase:
    """Re-lay a case out in the reference's native token-major form [T, Hkv, R] with a
    (optionally shuffled) page table; contents are identical.  `page_size` > 1 shuffles whole
    pages of that many consecutive token slots (a paged cache) instead of single slots."""
    st = case.storage
    B, H, S, Rk = st["latent_k"].shape
    dev = st["latent_k"].device
    T = B * S
    perm = torch.arange(T)
    if shuffle_seed is not None and page_size > 1:
        assert T % page_size == 0
        pages = torch.randperm(T // page_size, generator=torch.Generator().manual_seed(shuffle_seed))
        perm = (pages[:, None] * page_size + torch.arange(page_size)[None, :]).reshape(T)
    elif shuffle_seed is not None:
        perm = torch.randperm(T, generator=torch.Generator().manual_seed(shuffle_seed))
    table = perm.view(B, S).to(torch.int32)
    idx = table.long().to(dev)

    def relay(x):  # [B,H,S,...] -> [T,H,...]
        y = torch.empty((T, H) + tuple(x.shape[3:]), dtype=x.dtype, device=dev)
        y[idx.reshape(-1)] = x.permute(0, 2, 1, *range(3, x.dim())).reshape((T, H) + tuple(x.shape[3:]))
        return y

    state = InferState(B, case.infer_state.max_len_in_batch, case.seq_lens, device=dev, req_to_token=table)
    return DecodeCase(
        q=case.q, latent_k=relay(st["latent_k"]), k_scale=relay(st["k_scale"]) if "k_scale" in st else None,
        latent_v=relay(st["latent_v"]), v_scale=relay(st["v_scale"]) if "v_scale" in st else None,
        wk=case.wk, wv=case.wv, infer_state=state, seq_lens=case.seq_lens, storage={})
