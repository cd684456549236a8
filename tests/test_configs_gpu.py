"""Parity at the shapes of the benchmark workloads (c1..c4), through the public op and the raw
C ABI, against the CPU oracle on identical seeded inputs.

The other GPU parity tests use a handful of heads and short sequences; here the head
counts (32 / 40), the rank pairs (64/64 and 64/48), the context lengths (2k..32k) and the
split plan the library makes by itself are the ones the benchmark runs with.  c1 runs in
full; c2..c4 run a sub-batch that contains the workload's shortest and longest sequences,
once with the plan the library makes for the sub-batch and once with the split length it
makes for the full batch.  The reference's only check of this kind is
efficiency/test_functional_layer.py:347-399 (fp16 path, S = 256).
"""
import ctypes

import pytest
import torch

from tests.helpers import assert_close, oracle_for
from wsvd_b200 import _lib, inputs, ops
from wsvd_b200.kernel.flash_decoding import (
    token_decode_attention_flash_int8_latent_per_head_decoding_rope as op_i8,
)

pytestmark = pytest.mark.gpu

KERNELS = ["tc", "generic"]


def _sub_batch(name, pick):
    """(spec, lengths of the picked sequences); `pick` maps the workload's lengths to indices."""
    spec = inputs.WORKLOADS[name]
    lens = inputs.seq_lens_for(spec)
    idx = pick(lens)
    return spec, [lens[i] for i in idx]


def _full_batch_split_len(spec, case_cuda, kernel):
    """Split length the library plans for the whole workload (its batch size and max_len)."""
    s = case_cuda.infer_state
    p, _keep = ops.build_params(case_cuda.q, s.b_seq_len, s.b_req_idx, s.req_manager.req_to_token_indexs,
                                spec.max_len, case_cuda.latent_k, case_cuda.k_scale, case_cuda.latent_v,
                                case_cuda.v_scale, case_cuda.wk, None, kernel=kernel)
    p.batch = spec.batch
    return ops.plan(p)[0]


_ORACLE = {}  # workload -> (O_lat, O): the 32k-token oracle takes seconds, both kernels share it


def _run_both_outputs(case, kernel, max_len, split_len, what):
    from oracle import latent_decode_oracle as orc

    c = case.to("cuda")
    s = c.infer_state
    s.max_len_in_batch = max_len  # the full workload's max_len: empty splits are part of the test
    H, D = c.q.shape[1], c.q.shape[2]
    if what not in _ORACLE:
        _ORACLE[what] = orc.latent_decode_oracle(*case.oracle_args(), wv=case.wv)
    want_lat, want = _ORACLE[what]
    for sl in sorted({0, split_len}):
        got_lat = op_i8(c.q, s, H, D, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, kernel=kernel,
                        split_len=sl)
        got = op_i8(c.q, s, H, D, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, wv=c.wv, kernel=kernel,
                    split_len=sl)
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0, "a bounded wait timed out"
        assert_close(got_lat, want_lat, f"{what} O_lat kernel={kernel} split_len={sl}")
        assert_close(got, want, f"{what} O kernel={kernel} split_len={sl}")


@pytest.mark.parametrize("kernel", KERNELS)
def test_c1_in_full(kernel):
    spec = inputs.WORKLOADS["c1_7b_b1_s2048"]
    case = inputs.make_workload(spec, device="cpu")
    c = case.to("cuda")
    _run_both_outputs(case, kernel, spec.max_len, _full_batch_split_len(spec, c, kernel), "c1")


@pytest.mark.parametrize("kernel", KERNELS)
def test_c2_two_sequences_40_heads_8k(kernel):
    spec = inputs.WORKLOADS["c2_13b_b16_s8192"]
    lens = [spec.max_len, spec.max_len]
    case = inputs.make_case(2, spec.heads, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len, spec.seed)
    c = case.to("cuda")
    _run_both_outputs(case, kernel, spec.max_len, _full_batch_split_len(spec, c, kernel), "c2")


@pytest.mark.parametrize("kernel", KERNELS)
def test_c3_shortest_longest_and_one_more_32_heads(kernel):
    spec, lens = _sub_batch("c3_next7b_b32_ragged4096",
                            lambda l: [l.index(min(l)), l.index(max(l)), len(l) // 2])
    case = inputs.make_case(3, spec.heads, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len, spec.seed)
    c = case.to("cuda")
    _run_both_outputs(case, kernel, spec.max_len, _full_batch_split_len(spec, c, kernel), "c3")


@pytest.mark.parametrize("kernel", KERNELS)
def test_c4_shortest_longest_and_one_more_40_heads_rank_64_48(kernel):
    spec, lens = _sub_batch("c4_13b_b64_ragged32k",
                            lambda l: [l.index(max(l)), l.index(min(l)), len(l) // 2])
    assert max(lens) > 30000 and spec.rank_v == 48
    case = inputs.make_case(3, spec.heads, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len, spec.seed)
    c = case.to("cuda")
    _run_both_outputs(case, kernel, spec.max_len, _full_batch_split_len(spec, c, kernel), "c4")


# ---- equal shares of tiles over persistent CTAs (what the op does when no split length is given) ----

@pytest.mark.parametrize("heads,lens", [
    (6, [1500, 0, 257, 0, 2049]),              # a last group of 2 heads; sequences without tokens
    (8, [0, 0, 129, 128, 1, 0, 4000, 127]),    # leading/trailing empty sequences, one-token sequence
    (40, [3000, 17]),                          # more tiles than CTAs: several items per share
    (4, [128] * 200),                          # more sequences than CTAs: many one-tile items per share
], ids=["h6-zero-lengths", "h8-edges", "h40-long", "b200-one-tile"])
def test_balanced_shares_on_ragged_batches(heads, lens):
    case = inputs.make_case(len(lens), heads, 128, 64, 48, lens, max(lens), seed=61)
    c = case.to("cuda")
    want_lat, want = oracle_for(case), oracle_for(case, wv=True)
    for _ in range(2):  # the second call reuses the workspace the first one left behind
        got_lat = op_i8(c.q, c.infer_state, heads, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                        kernel="tc")
        got = op_i8(c.q, c.infer_state, heads, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, wv=c.wv,
                    kernel="tc")
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0, "a bounded wait timed out"
        assert_close(got_lat, want_lat, "balanced O_lat")
        assert_close(got, want, "balanced O")


def test_balanced_shares_with_more_sequences_than_threads():
    """700 sequences: the in-kernel prefix sum over the lengths runs in two chunks of 640."""
    g = torch.Generator().manual_seed(5)
    lens = [int(x) for x in torch.randint(0, 260, (700,), generator=g)]
    lens[3], lens[650], lens[699] = 0, 513, 129
    case = inputs.make_case(len(lens), 4, 128, 16, 16, lens, max(lens), seed=63)
    c = case.to("cuda")
    got = op_i8(c.q, c.infer_state, 4, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, wv=c.wv, kernel="tc")
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0, "a bounded wait timed out"
    assert_close(got, oracle_for(case, wv=True), "700 sequences")


def test_rank_62_reaches_the_tensor_core_path_by_zero_padding():
    """The accuracy pipeline's uniform rank is 62 (fake_quant/local_ft_grad_utils.py:2475-2478): not a
    multiple of 16, so the unpadded cache runs on the generic kernel; stored zero-padded to 64 it runs on
    the tensor-core kernel, with the same result."""
    lens = [1300, 40, 777]
    case = inputs.make_case(len(lens), 8, 128, 62, 62, lens, 1300, seed=67)
    want = oracle_for(case, wv=True)
    c = case.to("cuda")
    got_generic = op_i8(c.q, c.infer_state, 8, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, wv=c.wv)
    padded = inputs.padded_rank_copy(case, 64, 64).to("cuda")
    got_tc = op_i8(padded.q, padded.infer_state, 8, 128, padded.latent_k, padded.k_scale, padded.latent_v,
                   padded.v_scale, padded.wk, None, wv=padded.wv, kernel="tc")
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(got_generic, want, "rank 62, generic kernel")
    assert_close(got_tc, want, "rank 62 padded to 64, tensor-core kernel")


def test_all_sequences_empty():
    case = inputs.make_case(3, 4, 128, 64, 64, [0, 0, 0], 1, seed=62)
    c = case.to("cuda")
    got = op_i8(c.q, c.infer_state, 4, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None, kernel="tc")
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.count_nonzero(got).item() == 0


# ---- the raw C entry points on paths the Python op never takes ----

def _raw_params(c, out, **kw):
    s = c.infer_state
    p, keep = ops.build_params(c.q, s.b_seq_len, s.b_req_idx, s.req_manager.req_to_token_indexs,
                               s.max_len_in_batch, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                               wv=c.wv, out=out, **kw)
    return p, keep


@pytest.mark.parametrize("entry", ["workspace", "static"])
def test_position_table_built_by_the_library_when_none_is_passed(entry):
    """rope_table = NULL: the tensor-core kernel's cos/sin table is built in the workspace
    (or in the static scratch) by the call itself — what a bare C host gets."""
    lib = _lib.lib()
    lens = [1500, 257, 0, 2049]
    case = inputs.make_case(len(lens), 8, 128, 64, 48, lens, 2049, seed=41)
    c = case.to("cuda")
    out = torch.full((len(lens), 8, 128), float("nan"), dtype=torch.float16, device="cuda")
    p, keep = _raw_params(c, out, kernel="tc")
    p.rope_table, p.rope_table_rows = None, 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
    p_with, _k = _raw_params(c, out, kernel="tc")
    assert need > lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p_with)), "the table must be part of the workspace"
    if entry == "workspace":
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        _lib.check(lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), need, stream), "decode")
    else:
        _lib.check(lib.wsvd_latent_decode_static(ctypes.byref(p), stream), "decode_static")
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(out, oracle_for(case, wv=True), f"rope_table=NULL via {entry}")


def test_unknown_token_slot_count_takes_the_gather_path():
    """n_token_slots = 0 ("extent of the cache unknown"): rows are gathered through the page
    table instead of being fetched with tensor-map copies; same result."""
    lib = _lib.lib()
    lens = [700, 1025, 130]
    case = inputs.make_case(len(lens), 8, 128, 64, 64, lens, 1025, seed=43)
    c = case.to("cuda")
    out = torch.full((len(lens), 8, 128), float("nan"), dtype=torch.float16, device="cuda")
    p, keep = _raw_params(c, out, kernel="tc")
    p.n_token_slots = 0
    need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), need, stream), "decode")
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(out, oracle_for(case, wv=True), "n_token_slots=0")


@pytest.mark.parametrize("kernel", ["generic", "tc", "mma"])
def test_position_offsets(kernel):
    """pos_offset[b] shifts the RoPE position of every token of sequence b."""
    lens = [300, 1, 513]
    case = inputs.make_case(len(lens), 4, 128, 64, 64, lens, 513, seed=47)
    off = torch.tensor([0, 4095, 1234], dtype=torch.int32)
    c = case.to("cuda")
    got = op_i8(c.q, c.infer_state, 4, 128, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                pos_offset=off.cuda(), kernel=kernel)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(got, oracle_for(case, pos_offset=off), f"pos_offset kernel={kernel}")


def test_cached_argument_block_survives_a_growing_position_table():
    """A call signature seen before a longer context arrived must still read a valid table:
    the table grows (and its buffer changes) between the first call and its repeat."""
    short = inputs.make_case(2, 4, 128, 64, 64, [300, 77], 300, seed=51)
    cs = short.to("cuda")
    s = cs.infer_state
    want = oracle_for(short)
    first = op_i8(cs.q, s, 4, 128, cs.latent_k, cs.k_scale, cs.latent_v, cs.v_scale, cs.wk, None, kernel="tc")
    torch.cuda.synchronize()
    assert_close(first, want, "first call")
    n_long = 40000  # beyond any table built so far in this process: forces a new, larger buffer
    long = inputs.make_case(1, 1, 128, 64, 64, [n_long], n_long, seed=52).to("cuda")
    op_i8(long.q, long.infer_state, 1, 128, long.latent_k, long.k_scale, long.latent_v, long.v_scale, long.wk, None,
          kernel="tc")
    # fill whatever the allocator may have recycled
    junk = [torch.full((1 << 20,), 0x7F, dtype=torch.uint8, device="cuda") for _ in range(24)]
    torch.cuda.synchronize()
    again = op_i8(cs.q, s, 4, 128, cs.latent_k, cs.k_scale, cs.latent_v, cs.v_scale, cs.wk, None, kernel="tc")
    torch.cuda.synchronize()
    del junk
    assert ops.kernel_status() == 0
    assert_close(again, want, "repeat of the first call after the table grew")
