"""ctypes binding of libnqb200.so (the C ABI declared in include/nqb200.h).

There is no fallback: if the shared library is missing, or a call returns a
nonzero status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libnqb200.so")

F16, BF16 = 0, 1
_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t

class DecodeFusion(ctypes.Structure):
    """nqb200_decode_fusion of include/nqb200.h."""
    _fields_ = [("norm_ssq", ctypes.c_void_p), ("norm_tiles", ctypes.c_int64), ("norm_weight", ctypes.c_void_p),
                ("norm_eps", ctypes.c_float), ("silu_mul", ctypes.c_int), ("residual_in", ctypes.c_void_p),
                ("ssq_out", ctypes.c_void_p)]


FUSE_RMSNORM, FUSE_RESIDUAL, FUSE_SILU_MUL, FUSE_ALLREDUCE = 1, 2, 4, 8

# name -> (restype, argtypes); mirrors include/nqb200.h one to one
SIGNATURES = {
    "nqb200_version": (_int, []),
    "nqb200_status_string": (ctypes.c_char_p, [_int]),
    "nqb200_device_supported": (_int, [_int]),
    "nqb200_unpack_int4": (_int, [_vp, _vp, _i64, _i64, _vp]),
    "nqb200_dequant": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nqb200_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _int]),
    "nqb200_gemm": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "nqb200_decode_tile_columns": (_int, []),
    "nqb200_gemm_gate_up_silu_supported": (_int, [_i64, _i64, _i64, _i64, _int]),
    "nqb200_gemm_gate_up_silu": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "nqb200_gemm_decode_fused_supported": (_int, [_i64, _i64, _i64, _i64, _int, _int, _int, _sz]),
    "nqb200_gemm_decode_fused": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz,
                                 ctypes.POINTER(DecodeFusion), ctypes.POINTER(_vp), _int, _int, _sz, _sz, _vp]),
    "nqb200_gemm_decode_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp]),
    "nqb200_quantize_pack": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "nqb200_add_rmsnorm": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, _int, _vp]),
    "nqb200_qknorm_rope": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _int, _vp]),
    "nqb200_qknorm_rope_kv": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _int, _vp]),
    "nqb200_silu_mul": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "nqb200_comm_alloc": (_int, [ctypes.POINTER(_vp), _sz]),
    "nqb200_comm_free": (_int, [_vp]),
    "nqb200_comm_export": (_int, [_vp, _vp]),
    "nqb200_comm_import": (_int, [_vp, ctypes.POINTER(_vp)]),
    "nqb200_comm_unimport": (_int, [_vp]),
    "nqb200_comm_data_offset": (_sz, []),
    "nqb200_comm_set_wait_limit": (_int, [_vp, ctypes.c_uint64]),
    "nqb200_comm_status": (_int, [_vp, _vp]),
    "nqb200_gemm_allreduce_supported": (_int, [_i64, _i64, _i64, _i64, _int, _int, _sz]),
    "nqb200_gemm_allreduce": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz, ctypes.POINTER(_vp), _int, _int, _sz, _sz, _vp]),
    "nqb200_peer_allreduce": (_int, [ctypes.POINTER(_vp), _int, _int, _sz, _vp, _vp, _int, _i64, _i64, _int, _vp]),
    "nqb200_peer_allreduce_large": (_int, [ctypes.POINTER(_vp), _int, _int, _sz, _sz, _vp, _vp, _int, _i64, _i64, _int, _vp]),
    "nqb200_workspace_status": (_int, [_vp, _sz, _vp]),
    "nqb200_gemm_kernel_name": (ctypes.c_char_p, [_i64, _i64, _i64, _i64, _int]),
    "nqb200_gemm_launch_count": (_int, [_i64, _i64, _i64, _i64, _int]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with "
                    "`python -m nanoquantization_b200.csrc.build` (needs nvcc). "
                    "There is no CPU or PyTorch fallback for the W4A16 kernels.")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(f"nqb200: {load().nqb200_status_string(status).decode()} (status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return F16
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"W4A16 kernels take float16 or bfloat16, got {dtype}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t.device.type != "cuda":
            raise RuntimeError("nanoquantization_b200 runs on CUDA tensors only (no CPU fallback); "
                               f"got a tensor on {t.device}")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


_supported: dict[int, bool] = {}


def require_b200(dev: torch.device) -> None:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    ok = _supported.get(idx)
    if ok is None:
        ok = load().nqb200_device_supported(idx) == 1
        _supported[idx] = ok
    if not ok:
        check(6)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def workspace(dev: torch.device, nbytes: int) -> torch.Tensor | None:
    """Zero-filled scratch, one per (device, stream), grown on demand.  The
    kernels leave it zero-filled again, so it is only cleared when created."""
    if nbytes == 0:
        return None
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), stream_ptr())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def check_workspaces() -> None:
    """Synchronise and raise if any kernel recorded a give-up (a bounded wait that ran out)."""
    lib = load()
    for (_dev, stream), ws in list(_workspaces.items()):
        check(lib.nqb200_workspace_status(ws.data_ptr(), ws.numel(), stream))
