"""Build and load the CUDA library (libwsvd_b200.so) and describe its C ABI to ctypes.

The library is compiled in-tree with nvcc for sm_100a only.  There is no fallback: if
the shared object cannot be built or loaded, importing an op raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_CSRC = os.path.join(_PKG, "csrc")
_INCLUDE = os.path.join(_ROOT, "include")
LIB_PATH = os.path.join(_PKG, "libwsvd_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]

_lock = threading.Lock()
_lib = None


def sources():
    return sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith(".cu"))


def _deps():
    hdr = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".cuh", ".h"))]
    return sources() + hdr + [os.path.join(_INCLUDE, "wsvd_b200.h")]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > t for f in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into one shared object for sm_100a.

    Safe when several processes start at once (one rank per GPU under torchrun): the
    staleness check, the compile and the rename happen under an inter-process file lock, the
    compiler writes to a per-process temporary name, and a process that gets the lock after
    another one has built finds the library fresh and returns."""
    import fcntl

    with _lock:
        if not force and not _stale():
            return LIB_PATH
        with open(LIB_PATH + ".lock", "w") as lockfile:
            fcntl.flock(lockfile, fcntl.LOCK_EX)
            try:
                if not force and not _stale():
                    return LIB_PATH
                nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
                if not os.path.exists(nvcc):
                    raise RuntimeError("nvcc not found: cannot build libwsvd_b200.so")
                tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
                cmd = [nvcc, *NVCC_FLAGS, "-I", _INCLUDE, "-I", _CSRC, *sources(), "-o", tmp, "-lcuda"]
                if verbose:
                    cmd.insert(1, "-Xptxas=-v")
                res = subprocess.run(cmd, capture_output=True, text=True)
                if res.returncode != 0:
                    if os.path.exists(tmp):
                        os.remove(tmp)
                    raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
                if verbose:
                    print(res.stderr)
                os.replace(tmp, LIB_PATH)
            finally:
                fcntl.flock(lockfile, fcntl.LOCK_UN)
        return LIB_PATH


class LatentDecodeParams(ctypes.Structure):
    """ctypes mirror of WsvdLatentDecodeParams (include/wsvd_b200.h)."""

    _fields_ = [
        ("q", ctypes.c_void_p), ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64),
        ("latent_k", ctypes.c_void_p), ("k_stride_t", ctypes.c_int64), ("k_stride_h", ctypes.c_int64),
        ("k_scale", ctypes.c_void_p), ("ks_stride_t", ctypes.c_int64), ("ks_stride_h", ctypes.c_int64),
        ("latent_v", ctypes.c_void_p), ("v_stride_t", ctypes.c_int64), ("v_stride_h", ctypes.c_int64),
        ("v_scale", ctypes.c_void_p), ("vs_stride_t", ctypes.c_int64), ("vs_stride_h", ctypes.c_int64),
        ("wk", ctypes.c_void_p), ("wk_stride_r", ctypes.c_int64),
        ("wk_scale", ctypes.c_void_p),
        ("wv", ctypes.c_void_p), ("wv_stride_r", ctypes.c_int64),
        ("req_to_token", ctypes.c_void_p), ("rtt_stride", ctypes.c_int64),
        ("b_req_idx", ctypes.c_void_p),
        ("b_seq_len", ctypes.c_void_p),
        ("pos_offset", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("out_stride_b", ctypes.c_int64), ("out_stride_h", ctypes.c_int64),
        ("batch", ctypes.c_int32), ("n_q_heads", ctypes.c_int32), ("n_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("rank_k", ctypes.c_int32), ("rank_v", ctypes.c_int32),
        ("max_len", ctypes.c_int32),
        ("latent_dtype", ctypes.c_int32), ("wk_dtype", ctypes.c_int32), ("rope_layout", ctypes.c_int32),
        ("split_len", ctypes.c_int32), ("kernel", ctypes.c_int32),
        ("theta", ctypes.c_float), ("sm_scale", ctypes.c_float),
        ("rope_table", ctypes.c_void_p), ("rope_table_rows", ctypes.c_int32),
        ("n_token_slots", ctypes.c_int64),
    ]


class DenseDecodeParams(ctypes.Structure):
    """ctypes mirror of WsvdDenseDecodeParams."""

    _fields_ = [
        ("q", ctypes.c_void_p), ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64),
        ("k", ctypes.c_void_p), ("k_stride_t", ctypes.c_int64), ("k_stride_h", ctypes.c_int64),
        ("v", ctypes.c_void_p), ("v_stride_t", ctypes.c_int64), ("v_stride_h", ctypes.c_int64),
        ("req_to_token", ctypes.c_void_p), ("rtt_stride", ctypes.c_int64),
        ("b_req_idx", ctypes.c_void_p), ("b_seq_len", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("out_stride_b", ctypes.c_int64), ("out_stride_h", ctypes.c_int64),
        ("batch", ctypes.c_int32), ("n_q_heads", ctypes.c_int32), ("n_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("max_len", ctypes.c_int32), ("split_len", ctypes.c_int32),
        ("sm_scale", ctypes.c_float),
    ]


class QuantAppendParams(ctypes.Structure):
    """ctypes mirror of WsvdQuantAppendParams."""

    _fields_ = [
        ("x_k", ctypes.c_void_p), ("xk_stride_b", ctypes.c_int64), ("xk_stride_h", ctypes.c_int64),
        ("x_v", ctypes.c_void_p), ("xv_stride_b", ctypes.c_int64), ("xv_stride_h", ctypes.c_int64),
        ("latent_k", ctypes.c_void_p), ("k_stride_t", ctypes.c_int64), ("k_stride_h", ctypes.c_int64),
        ("k_scale", ctypes.c_void_p), ("ks_stride_t", ctypes.c_int64), ("ks_stride_h", ctypes.c_int64),
        ("latent_v", ctypes.c_void_p), ("v_stride_t", ctypes.c_int64), ("v_stride_h", ctypes.c_int64),
        ("v_scale", ctypes.c_void_p), ("vs_stride_t", ctypes.c_int64), ("vs_stride_h", ctypes.c_int64),
        ("req_to_token", ctypes.c_void_p), ("rtt_stride", ctypes.c_int64),
        ("b_req_idx", ctypes.c_void_p), ("b_seq_len", ctypes.c_void_p),
        ("batch", ctypes.c_int32), ("n_kv_heads", ctypes.c_int32), ("rank_k", ctypes.c_int32),
        ("rank_v", ctypes.c_int32), ("max_len", ctypes.c_int32), ("x_dtype", ctypes.c_int32),
    ]


MAX_PEERS = 8
PEER_HANDLE_BYTES = 64


class PeerSet(ctypes.Structure):
    """ctypes mirror of WsvdPeerSet."""

    _fields_ = [
        ("out", ctypes.c_void_p * MAX_PEERS), ("flags", ctypes.c_void_p * MAX_PEERS), ("counter", ctypes.c_void_p),
        ("n_peers", ctypes.c_int32), ("rank", ctypes.c_int32), ("head_offset", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("out_stride_b", ctypes.c_int64), ("out_stride_h", ctypes.c_int64),
        ("timeout_ms", ctypes.c_int32), ("epoch_counter", ctypes.c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/wsvd_b200.h declares
_P = ctypes.POINTER(LatentDecodeParams)
SYMBOLS = {
    "wsvd_abi_version": (ctypes.c_int, []),
    "wsvd_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "wsvd_last_cuda_error": (ctypes.c_int, []),
    "wsvd_rope_table_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32]),
    "wsvd_rope_table_init": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int32, ctypes.c_int32,
                                            ctypes.c_float, ctypes.c_void_p]),
    "wsvd_kernel_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "wsvd_kernel_status_reset": (ctypes.c_int, []),
    "wsvd_latent_decode_plan": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
    "wsvd_latent_decode_workspace_bytes": (ctypes.c_size_t, [_P]),
    "wsvd_latent_decode": (ctypes.c_int, [_P, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "wsvd_share_begin": (ctypes.c_int64, [ctypes.c_int32, ctypes.c_int64, ctypes.c_int32]),
    "wsvd_share_owner": (ctypes.c_int32, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int32]),
    "wsvd_latent_decode_partials": (ctypes.c_int, [_P, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "wsvd_dense_decode_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(DenseDecodeParams)]),
    "wsvd_dense_decode_f16": (ctypes.c_int, [ctypes.POINTER(DenseDecodeParams), ctypes.c_void_p, ctypes.c_size_t,
                                             ctypes.c_void_p]),
    "wsvd_latent_decode_static": (ctypes.c_int, [_P, ctypes.c_void_p]),
    "wsvd_latent_decode_gather": (ctypes.c_int, [_P, ctypes.POINTER(PeerSet), ctypes.c_void_p, ctypes.c_size_t,
                                                 ctypes.c_void_p]),
    "wsvd_peer_alloc": (ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]),
    "wsvd_peer_free": (ctypes.c_int, [ctypes.c_void_p]),
    "wsvd_peer_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "wsvd_peer_import": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "wsvd_peer_release": (ctypes.c_int, [ctypes.c_void_p]),
    "wsvd_latent_quant_append_i8": (ctypes.c_int, [ctypes.POINTER(QuantAppendParams), ctypes.c_void_p]),
    "wsvd_rms_norm_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                         ctypes.c_float, ctypes.c_void_p]),
    "wsvd_add_rms_norm_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_int32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p]),
    "wsvd_rope_half_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]),
    "wsvd_silu_mul_f16": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]),
    "wsvd_latent_decode_stage1": (ctypes.c_int, [_P, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]),
    "wsvd_decode_stage2": (ctypes.c_int, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
        ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]),
}


def lib() -> ctypes.CDLL:
    """The loaded library; builds it first if the shared object is missing or stale."""
    global _lib
    if _lib is None:
        build()
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class WsvdError(RuntimeError):
    """A C entry point returned a nonzero status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().wsvd_status_string(status).decode()
        if status == 6:
            msg += f" [cudaError {lib().wsvd_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (status {status})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise WsvdError(status, where)
