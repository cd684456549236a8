"""The merge kernel with the head all-gather fused in (wsvd_latent_decode_gather).

One GPU: the ranks of a group are emulated one after the other with local buffers standing
in for the peers' (no launch waits on a flag that another launch writes: the flags a rank
waits for are set from the host beforehand).  Two GPUs: two real processes, CUDA IPC
mappings, against the single-GPU op and the oracle.
"""
import ctypes
import os
import socket

import pytest
import torch

from tests.helpers import assert_close, oracle_for
from wsvd_b200 import inputs

pytestmark = pytest.mark.gpu


def _shard_case(case, sl):
    """Views of one head shard of a CUDA case (head-major storage: slicing the head axis)."""
    return (case.q[:, sl], case.latent_k[:, sl], case.k_scale[:, sl], case.latent_v[:, sl], case.v_scale[:, sl],
            case.wk.view(case.wk.shape[0], -1, 128)[:, sl].reshape(case.wk.shape[0], -1),
            case.wv.view(case.wv.shape[0], -1, 128)[:, sl].reshape(case.wv.shape[0], -1))


def _peer_set(lib_mod, outs, flags, counter, rank, head_offset, epoch, H, D, timeout_ms=0):
    ps = lib_mod.PeerSet()
    for i, (o, f) in enumerate(zip(outs, flags)):
        ps.out[i], ps.flags[i] = o.data_ptr(), f.data_ptr()
    ps.counter = counter.data_ptr()
    ps.n_peers, ps.rank, ps.head_offset, ps.epoch = len(outs), rank, head_offset, epoch
    ps.out_stride_b, ps.out_stride_h, ps.timeout_ms = H * D, D, timeout_ms
    return ps


@pytest.mark.parametrize("with_wv", [True, False])
def test_emulated_ranks_fill_every_buffer(with_wv):
    from wsvd_b200 import _lib, ops

    world, H, B = 3, 12, 4
    case = inputs.make_case(B, H, 128, 64, 64, [700, 1, 333, 512], 704, seed=21).to("cuda")
    D = 128 if with_wv else 64
    outs = [torch.full((B, H, D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(_lib.MAX_PEERS, dtype=torch.int32, device="cuda") for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    epoch = 7
    for r in range(world):
        sl = slice(r * H // world, (r + 1) * H // world)
        q, lk, ks, lv, vs, wk, wv = _shard_case(case, sl)
        for f in flags:
            f.zero_()
        flags[r].fill_(epoch)  # what the peers would have signalled
        ps = _peer_set(_lib, outs, flags, counter, r, sl.start, epoch, H, D)
        ops.latent_decode_gather(q, case.infer_state, lk, ks, lv, vs, wk, None, ps, wv=wv if with_wv else None)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        assert int(counter.item()) == 0, "the block counter must be back at zero"
        for i in range(world):
            assert int(flags[i][r].item()) == epoch, f"rank {r} did not signal peer {i}"
    want = oracle_for(case.to("cpu"), wv=with_wv)
    for i, o in enumerate(outs):
        assert_close(o, want, f"buffer of rank {i}")


def test_barrier_wait_is_bounded():
    """A flag that nothing sets: the wait runs out, status 6 is recorded, the context lives."""
    from wsvd_b200 import _lib, ops

    H, B = 4, 2
    case = inputs.make_case(B, H, 128, 64, 64, [300, 200], 320, seed=3).to("cuda")
    outs = [torch.zeros(B, H, 64, dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(_lib.MAX_PEERS, dtype=torch.int32, device="cuda") for _ in range(2)]
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    sl = slice(0, 2)
    q, lk, ks, lv, vs, wk, wv = _shard_case(case, sl)
    ps = _peer_set(_lib, outs, flags, counter, 0, 0, 1, H, 64, timeout_ms=50)
    ops.latent_decode_gather(q, case.infer_state, lk, ks, lv, vs, wk, None, ps)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 6
    _lib.check(_lib.lib().wsvd_kernel_status_reset(), "reset")
    assert ops.kernel_status() == 0
    # the rows were delivered all the same, and the library still works
    assert_close(outs[1][:, sl], oracle_for(case.to("cpu"))[:, sl], "rows stored before the wait")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank, world, port, ret):
    import torch.distributed as dist

    from wsvd_b200 import ops
    from wsvd_b200.dist import PeerGather
    from wsvd_b200.kernel.flash_decoding import (
        token_decode_attention_flash_int8_latent_per_head_decoding_rope as op_i8,
    )

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        H, B = 8, 3
        cpu_case = inputs.make_case(B, H, 128, 64, 64, [900, 130, 512], 960, seed=5)
        case = cpu_case.to("cuda")
        pg = PeerGather(B, H, 128, timeout_ms=5000)
        q, lk, ks, lv, vs, wk, wv = _shard_case(case, pg.shard)
        want = oracle_for(cpu_case, wv=True)
        for step in range(4):  # both buffer parities, twice
            got = pg.decode(q, case.infer_state, lk, ks, lv, vs, wk, None, wv=wv)
            torch.cuda.synchronize()
            assert ops.kernel_status() == 0, "barrier wait timed out"
            assert_close(got, want, f"rank {rank} step {step}")
            got.fill_(float("nan"))  # so that the next use of this buffer has to be rewritten
            torch.cuda.synchronize()
            dist.barrier()
        full = op_i8(case.q, case.infer_state, H, 128, case.latent_k, case.k_scale, case.latent_v, case.v_scale,
                     case.wk, None, wv=case.wv)
        got = pg.decode(q, case.infer_state, lk, ks, lv, vs, wk, None, wv=wv)
        torch.cuda.synchronize()
        assert torch.equal(got, full), "gathered result differs from the single-GPU op"
        pg.close()
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_peer_stores():
    import torch.multiprocessing as mp

    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_two_gpu_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def test_device_side_epoch_counts_the_steps():
    """epoch_counter mode: the kernel takes the step number from device memory, so the same
    argument block serves step after step (what a captured CUDA graph replays)."""
    from wsvd_b200 import _lib, ops

    H, B = 4, 2
    case = inputs.make_case(B, H, 128, 64, 64, [300, 200], 320, seed=3).to("cuda")
    out = torch.zeros(B, H, 64, dtype=torch.float16, device="cuda")
    flags = torch.zeros(_lib.MAX_PEERS, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    epoch_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    q, lk, ks, lv, vs, wk, wv = _shard_case(case, slice(0, H))
    ps = _peer_set(_lib, [out], [flags], counter, 0, 0, 0, H, 64)   # epoch 0: taken from the device
    ps.epoch_counter = epoch_dev.data_ptr()
    for step in range(1, 4):
        out.zero_()
        ops.latent_decode_gather(q, case.infer_state, lk, ks, lv, vs, wk, None, ps)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        assert int(epoch_dev.item()) == step and int(flags[0].item()) == step
        assert_close(out, oracle_for(case.to("cpu")), f"step {step}")
