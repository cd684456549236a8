"""Head sharding + all-gather with two gloo ranks on CPU: shard bounds and the gathered
layout, with the CPU oracle standing in for the per-rank op."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from wsvd_b200 import dist as wdist


def test_head_shard_bounds():
    assert wdist.head_shard(40, 0, 8) == slice(0, 5)
    assert wdist.head_shard(40, 7, 8) == slice(35, 40)
    assert wdist.head_shard(32, 1, 2) == slice(16, 32)
    with pytest.raises(ValueError):
        wdist.head_shard(40, 0, 3)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import latent_decode_oracle as orc
    from wsvd_b200 import inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, D = 8, 128
        case = inputs.make_case(3, H, D, 64, 48, [200, 0, 77], 200, seed=42)  # same on every rank
        full_lat, full = orc.latent_decode_oracle(*case.oracle_args(), wv=case.wv)
        sl = wdist.head_shard(H, rank, world)
        cols = slice(sl.start * D, sl.stop * D)
        st = case.infer_state
        _, local = orc.latent_decode_oracle(
            case.q[:, sl], st.b_seq_len, st.b_req_idx, st.req_manager.req_to_token_indexs,
            case.latent_k[:, sl], case.k_scale[:, sl], case.latent_v[:, sl], case.v_scale[:, sl],
            case.wk[:, cols], wv=case.wv[:, cols])
        got = wdist.sharded_decode(lambda: local.half())
        ok = torch.allclose(got.float(), full.half().float(), atol=1e-6)
        ret[rank] = bool(ok) and tuple(got.shape) == (3, H, D)
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_matches_unsharded_oracle():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
