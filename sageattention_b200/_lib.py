"""ctypes binding of ``libsage3_b200.so`` (C ABI declared in ``include/sage3_b200.h``).

There is no fallback: if the shared library is missing the import fails with instructions to
build it, and every call checks the returned status.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
# SAGE3_B200_LIB points at another build of the same library (A/B timing of kernel variants); it must export the same C ABI
LIB_PATH = Path(os.environ.get("SAGE3_B200_LIB") or (_HERE / "libsage3_b200.so"))

OK, ERR_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_WAIT, ERR_TOO_LARGE = range(6)


class Shape(C.Structure):
    _fields_ = [("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32),
                ("Nq", C.c_int32), ("Nk", C.c_int32), ("D", C.c_int32)]


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_n", C.c_int64)]


class Sizes(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in
                ("q_codes", "q_sf", "k_codes", "k_sf", "vt_codes", "vt_sf", "qm", "km",
                 "delta_s", "q_dot_km", "scratch", "status", "workspace")]


class QuantArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", Tensor), ("k", Tensor), ("v", Tensor),
                ("per_block_mean", C.c_int32), ("smooth_k", C.c_int32),
                ("km_in", C.c_void_p), ("qm_in", C.c_void_p),
                ("q_codes", C.c_void_p), ("q_sf", C.c_void_p), ("k_codes", C.c_void_p), ("k_sf", C.c_void_p),
                ("vt_codes", C.c_void_p), ("vt_sf", C.c_void_p),
                ("qm", C.c_void_p), ("km", C.c_void_p), ("delta_s", C.c_void_p),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("device_status", C.c_void_p),
                ("q_dot_km", C.c_void_p), ("head_dim_in", C.c_int32)]


class AttnArgs(C.Structure):
    _fields_ = [("shape", Shape),
                ("q_codes", C.c_void_p), ("q_sf", C.c_void_p), ("k_codes", C.c_void_p), ("k_sf", C.c_void_p),
                ("vt_codes", C.c_void_p), ("vt_sf", C.c_void_p),
                ("delta_s", C.c_void_p), ("delta_s_rows", C.c_int32),
                ("out", C.c_void_p), ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
                ("out_stride_n", C.c_int64),
                ("lse", C.c_void_p), ("sm_scale", C.c_float), ("is_causal", C.c_int32),
                ("device_status", C.c_void_p), ("lse_add", C.c_void_p), ("out_head_dim", C.c_int32),
                ("sm_margin", C.c_int32)]


class FwdArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", Tensor), ("k", Tensor), ("v", Tensor),
                ("out", C.c_void_p), ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
                ("out_stride_n", C.c_int64),
                ("lse", C.c_void_p), ("km_out", C.c_void_p), ("sm_scale", C.c_float), ("is_causal", C.c_int32),
                ("per_block_mean", C.c_int32), ("smooth_k", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("device_status", C.c_void_p),
                ("head_dim", C.c_int32), ("sm_margin", C.c_int32)]


class PackArgs(C.Structure):
    _fields_ = [("shape", Shape), ("k", Tensor), ("v", Tensor), ("smooth_k", C.c_int32),
                ("km_in", C.c_void_p), ("km", C.c_void_p), ("k_packed", C.c_void_p), ("v_packed", C.c_void_p),
                ("k_lambda", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
                ("split_first", C.c_int32)]


class VarlenArgs(C.Structure):
    _fields_ = [("shape", Shape), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
                ("q_stride_n", C.c_int64), ("q_stride_h", C.c_int64), ("k_stride_n", C.c_int64),
                ("k_stride_h", C.c_int64), ("v_stride_n", C.c_int64), ("v_stride_h", C.c_int64),
                ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
                ("out", C.c_void_p), ("out_stride_n", C.c_int64), ("out_stride_h", C.c_int64),
                ("sm_scale", C.c_float), ("is_causal", C.c_int32), ("smooth_k", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("device_status", C.c_void_p)]


EXPORTS = ("sage3_version", "sage3_status_string", "sage3_last_cuda_error", "sage3_buffer_sizes",
           "sage3_quant_qkv", "sage3_attn_fwd", "sage3_attention", "sage3_read_device_status",
           "sage3_k_mean_static", "sage3_packed_rows", "sage3_packed_len", "sage3_pack_kv",
           "sage3_attn_fwd_packed", "sage3_attention_varlen", "sage3_fp4_mma_peak", "sage3_selftest_bounded_wait")

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sageattention_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    lib.sage3_version.restype = C.c_int
    lib.sage3_status_string.restype = C.c_char_p
    lib.sage3_status_string.argtypes = [C.c_int]
    lib.sage3_last_cuda_error.restype = C.c_int
    lib.sage3_buffer_sizes.argtypes = [C.POINTER(Shape), C.c_int, C.POINTER(Sizes)]
    lib.sage3_quant_qkv.argtypes = [C.POINTER(QuantArgs), C.c_void_p]
    lib.sage3_attn_fwd.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
    lib.sage3_attention.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.sage3_read_device_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    lib.sage3_k_mean_static.argtypes = [C.POINTER(Shape), C.POINTER(Tensor), C.c_void_p, C.c_void_p]
    lib.sage3_packed_rows.argtypes = [C.c_int]
    lib.sage3_packed_len.argtypes = [C.c_int]
    lib.sage3_pack_kv.argtypes = [C.POINTER(PackArgs), C.c_void_p]
    lib.sage3_attn_fwd_packed.argtypes = [C.POINTER(AttnArgs), C.c_void_p, C.c_int32, C.c_void_p]
    lib.sage3_attention_varlen.argtypes = [C.POINTER(VarlenArgs), C.c_void_p]
    lib.sage3_fp4_mma_peak.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_double)]
    lib.sage3_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_void_p]
    for name in EXPORTS:
        getattr(lib, name)            # raises AttributeError if an export is missing
    _lib = lib
    return lib


class Sage3Error(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.sage3_status_string(status).decode()
        if status == ERR_CUDA:
            msg += f" [cudaError {lib.sage3_last_cuda_error()}]"
        super().__init__(f"{where}: {msg}")
        self.status = status


def check(status: int, where: str) -> None:
    if status != OK:
        raise Sage3Error(status, where)
