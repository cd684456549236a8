"""Batch metadata object the decode op reads, with the attribute names of the
reference's LightLLM-style `infer_state` (efficiency/test_utils.py:9-22):
batch_size, max_len_in_batch, b_seq_len, b_req_idx, req_manager.req_to_token_indexs."""
from __future__ import annotations

from typing import Optional, Sequence

import torch


class ReqManager:
    def __init__(self, req_to_token_indexs: torch.Tensor):
        self.req_to_token_indexs = req_to_token_indexs


class InferState:
    """Any object with these attributes works; this one also accepts ragged lengths and
    a caller-supplied page table, which the reference's mock does not."""

    def __init__(self, batch_size: int, max_len_in_batch: int, seq_lens: Sequence[int],
                 device="cuda", req_to_token: Optional[torch.Tensor] = None,
                 b_req_idx: Optional[torch.Tensor] = None):
        self.batch_size = int(batch_size)
        self.max_len_in_batch = int(max_len_in_batch)
        self.b_seq_len = torch.as_tensor(list(seq_lens), dtype=torch.int32).to(device)
        if b_req_idx is None:
            b_req_idx = torch.arange(batch_size, dtype=torch.int32)
        self.b_req_idx = b_req_idx.to(device=device, dtype=torch.int32)
        if req_to_token is None:
            # contiguous slots, one row of max_len per request (test_utils.py:20)
            req_to_token = torch.arange(batch_size * max_len_in_batch, dtype=torch.int32).view(
                batch_size, max_len_in_batch)
        self.req_manager = ReqManager(req_to_token.to(device=device, dtype=torch.int32))


# the reference's name for it
MockInferState = InferState
