"""ctypes binding of libemmyq.so: the same calls a C host would make.

The library is loaded on first use.  If it has not been built the loader
raises: there is no fallback path.
"""

from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libemmyq.so"
HEADER = PKG.parent / "include" / "emmyq.h"

# status codes and enums of include/emmyq.h
EQ_OK = 0
EQ_ERR_BAD_ARG, EQ_ERR_BAD_ALIGN, EQ_ERR_UNSUPPORTED, EQ_ERR_CUDA = -1, -2, -3, -4
EQ_ERR_NCCL, EQ_ERR_TIMEOUT, EQ_ERR_WORKSPACE = -5, -6, -7
EQ_W4_AWQ, EQ_W4_GPTQ, EQ_W4_CT = 0, 1, 2
EQ_F16, EQ_BF16, EQ_F32 = 0, 1, 2


EQ_EP_MAX_RANKS = 8


class EpPeers(C.Structure):
    """struct eq_ep_peers of include/emmyq.h."""

    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("cap", C.c_int64),
        ("recv_x", C.c_void_p * EQ_EP_MAX_RANKS),
        ("recv_meta", C.c_void_p * EQ_EP_MAX_RANKS),
        ("recv_count", C.c_void_p * EQ_EP_MAX_RANKS),
        ("back", C.c_void_p * EQ_EP_MAX_RANKS),
        ("flags", C.c_void_p * EQ_EP_MAX_RANKS),
    ]


class ArPeers(C.Structure):
    """struct eq_ar_peers of include/emmyq.h."""

    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("cap", C.c_int64),
        ("max_blocks", C.c_int64),
        ("recv", C.c_void_p * EQ_EP_MAX_RANKS),
        ("flags", C.c_void_p * EQ_EP_MAX_RANKS),
    ]


class EmmyqError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"{name} ({status}): {message}")
        self.status = status
        self.status_name = name


_lib = None


def declared_symbols() -> list[str]:
    """Every function name include/emmyq.h declares."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(eq_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m emmy_b200.build` (needs nvcc). "
            "The quantized-linear operators have no CPU path."
        )
    lib = C.CDLL(str(LIB_PATH))
    p, i, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
    szp, ip = C.POINTER(C.c_size_t), C.POINTER(C.c_int)
    sig = {
        "eq_version": (i, []),
        "eq_last_error": (C.c_char_p, []),
        "eq_status_name": (C.c_char_p, [i]),
        "eq_unpack_int4": (i, [i, i, p, i64, i64, p, p]),
        "eq_dequant_w4": (i, [i, p, p, p, i, p, i64, i64, i64, i, i, p, p]),
        "eq_dequant_fp8": (i, [p, p, i64, i64, i64, i64, i, p, p]),
        "eq_dequant_nvfp4": (i, [p, p, p, i64, i64, i, p, p]),
        "eq_dequant_mxfp4": (i, [p, p, i64, i64, i, p, p]),
        "eq_w4_repack_sizes": (i, [i64, i64, i64, szp, szp]),
        "eq_w4_repack": (i, [i, p, p, p, p, i64, i64, i64, p, p, ip, p]),
        "eq_w4_repack_stack": (i, [i, p, p, p, i64, i64, i64, i64, p, p]),
        "eq_w4_unpack_repacked": (i, [p, i64, i64, p, p]),
        "eq_w4a16_workspace_bytes": (sz, [i64, i64, i64]),
        "eq_w4a16_linear": (i, [p, i, p, i64, i64, i64, p, i64, i, p, p, sz, p]),
        "eq_w4a16_status": (i, [p, i64, i64, p]),
        "eq_w4a16_gate_up_workspace_bytes": (sz, [i64, i64, i64]),
        "eq_w4a16_gate_up_swiglu": (i, [p, i, p, i64, i64, i64, p, i64, i, p, p, sz, p]),
        "eq_quant_fp8_per_token": (i, [p, i64, i64, i, p, p, p]),
        "eq_fp8_workspace_bytes": (sz, [i64, i64]),
        "eq_fp8_linear": (i, [p, p, i64, i64, p, i64, i, p, p, sz, p]),
        "eq_fp8_linear_static": (i, [p, p, i64, i64, p, p, i64, i, p, p, sz, p]),
        "eq_fp8_linear_rmsnorm": (i, [p, p, i64, i64, p, p, C.c_float, i64, i, p, p, sz, p]),
        "eq_fp8_status": (i, [p, i64, i64, p]),
        "eq_quant_fp8_per_group": (i, [p, i64, i64, i, p, p, p]),
        "eq_fp8_block_workspace_bytes": (sz, [i64, i64]),
        "eq_fp8_block_linear": (i, [p, p, i64, i64, p, i64, i, p, p, sz, p]),
        "eq_fp8_block_status": (i, [p, i64, i64, p]),
        "eq_nvfp4_global_scale": (i, [p, i64, i64, i, p, p, p]),
        "eq_quant_nvfp4_act": (i, [p, i64, i64, i, p, p, p, p, p]),
        "eq_quant_nvfp4_weight": (i, [p, i64, i64, i, p, p, p, p, p]),
        "eq_nvfp4_tiled_scale_bytes": (sz, [i64, i64]),
        "eq_nvfp4_tile_scales": (i, [p, i64, i64, p, p]),
        "eq_nvfp4_weight_scale_bytes": (sz, [i64, i64]),
        "eq_nvfp4_tile_weight_scales": (i, [p, i64, i64, p, p]),
        "eq_nvfp4_workspace_bytes": (sz, [i64, i64]),
        "eq_nvfp4_linear": (i, [p, p, p, i64, i64, p, p, i64, i, p, p, sz, p]),
        "eq_nvfp4_linear_rmsnorm": (i, [p, p, p, i64, i64, p, p, C.c_float, p, i64, i, p, p, sz, p]),
        "eq_nvfp4_status": (i, [p, i64, i64, p]),
        "eq_moe_route": (i, [p, i64, i64, i64, i, p, p, p]),
        "eq_moe_workspace_bytes": (sz, [i64, i64, i64, i64, i64]),
        "eq_moe_experts_w4a16": (i, [p, p, i, i64, i64, i64, i64, p, p, p, i64, i, p, p, sz, p]),
        "eq_moe_combine": (i, [p, p, i64, i64, i64, i, p, p]),
        "eq_moe_w4a16": (i, [p, p, i, i64, i64, i64, i64, i64, p, p, i64, i, p, p, sz, p]),
        "eq_moe_status": (i, [p, i64, i64, i64, i64, i64, p]),
        "eq_w4a16_linear_noalloc": (i, [p, i, p, i64, i64, i64, p, i64, i, p, p]),
        "eq_w4a16_noalloc_status": (i, [p]),
        "eq_ep_moe_workspace_bytes": (sz, [i64, i64, i64, i64, i64]),
        "eq_ep_moe_w4a16": (i, [p, p, i, i64, i64, i64, i64, i64, p, p, p, i64, i, p, C.POINTER(EpPeers), C.c_uint32, p, sz, p]),
        "eq_ep_moe_status": (i, [p, i64, i64, i64, i64, i64, p]),
        "eq_peer_allreduce_recv_bytes": (sz, [i64, i64]),
        "eq_peer_allreduce_flag_bytes": (sz, [i64, i64]),
        "eq_peer_allreduce_state_bytes": (sz, []),
        "eq_peer_allreduce": (i, [C.POINTER(ArPeers), p, i64, i, p, p, p]),
        "eq_peer_allreduce_status": (i, [p, p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib._eq_signatures = sig
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != EQ_OK:
        lib = load()
        raise EmmyqError(status, lib.eq_status_name(status).decode(), lib.eq_last_error().decode())
