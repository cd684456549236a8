"""wsvd_b200 — B200 (sm_100a) latent flash-decoding for WSVD-style low-rank KV caches.

Public surface (names follow the reference's efficiency/ package):
  wsvd_b200.kernel.flash_decoding.token_decode_attention_flash_int8_latent_per_head_decoding_rope
  wsvd_b200.kernel.flash_decoding.token_decode_attention_flash_latent_per_head_decoding_rope
  wsvd_b200.layer_utils.run_flash_int8_latent_per_head_decoding_rope_layer
  wsvd_b200.layer_utils.run_flash_latent_per_head_decoding_rope_layer
  wsvd_b200.infer_state.InferState
The compute lives in libwsvd_b200.so (C ABI: include/wsvd_b200.h).
"""
from ._lib import build, lib, WsvdError  # noqa: F401
from .infer_state import InferState, MockInferState  # noqa: F401

__version__ = "0.1.0"
