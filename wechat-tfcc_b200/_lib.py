"""ctypes binding of libtfcc_b200.so.  Loading fails loudly: no fallback exists."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import exceptions

_HERE = Path(__file__).resolve().parent

# int barrier(void* ctx, void* stream): see tfccb200_barrier_fn in include/tfcc_b200.h
BARRIER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p)


def library_path() -> Path:
    return _HERE / "libtfcc_b200.so"


class _Lib:
    """Lazy handle: the library is opened on first use so that importing the
    package on a machine without the build does not fail until an op is called."""

    def __init__(self):
        self._dll = None

    def _load(self):
        path = library_path()
        if not path.exists():
            raise ImportError(
                f"{path} is missing: build it with `python {_HERE / 'build.py'}`; "
                "this package has no CPU or eager fallback")
        dll = C.CDLL(str(path))
        vp, u, i, sz = C.c_void_p, C.c_uint, C.c_int, C.c_size_t
        i32, f = C.c_int32, C.c_float
        sig = {
            "tfccb200_strerror": (C.c_char_p, [i]),
            "tfccb200_version": (i, []),
            "tfccb200_launch_count": (C.c_ulonglong, []),
            "tfccb200_test_flag_wait": (None, [C.c_ulonglong, u]),
            "tfccb200_sgemm": (i, [vp, vp, u, vp, u, vp, u, vp, u, u, u, u, i, vp, sz, vp]),
            "tfccb200_sgemm_ex": (i, [vp, vp, u, vp, u, vp, u, vp, u, u, u, u, i, i, vp, sz, vp]),
            "tfccb200_sgemm_workspace": (sz, [u, u, u, u, i]),
            "tfccb200_sgemm_path": (i, [u, u, u, u, u, u, i]),
            "tfccb200_qgemm_u8s8s32": (i, [vp, vp, u, vp, u, i32, vp, u, vp, u, i32, vp, u, u, u, u, u, vp]),
            "tfccb200_qgemm_u8s8s32_ex": (i, [vp, vp, u, vp, u, i32, vp, u, vp, u, i32, vp, u, u, u, u, u, i, vp]),
            "tfccb200_qgemm_u8s8s32_dev": (i, [vp, vp, u, vp, u, vp, vp, vp, u, vp, u, vp, vp, vp, u,
                                               vp, vp, vp, u, u, u, u, i, vp]),
            "tfccb200_quantized_matmul_params": (i, [f, f, f, f, C.POINTER(i32), C.POINTER(i32),
                                                     C.POINTER(f), C.POINTER(f)]),
            "tfccb200_reduce_sum_u8": (i, [vp, vp, u, u, u, i, vp]),
            "tfccb200_reduce_sum_s8": (i, [vp, vp, u, u, u, i, vp]),
            "tfccb200_reduce_sum_s16": (i, [vp, vp, u, u, u, i, vp]),
            "tfccb200_sgemm_act": (i, [vp, vp, u, vp, u, vp, u, vp, u, u, u, u, i, i, i, vp, sz, vp]),
            "tfccb200_attention_f32": (i, [vp, vp, vp, vp, vp, u, u, u, u, u, u, f, vp]),
            "tfccb200_softmax_f32": (i, [vp, vp, u, u, f, vp]),
            "tfccb200_layer_norm_f32": (i, [vp, vp, vp, vp, vp, f, u, u, vp]),
            "tfccb200_gelu_f32": (i, [vp, vp, sz, vp]),
            "tfccb200_permute_0213_f32": (i, [vp, vp, u, u, u, u, vp]),
            "tfccb200_transpose_last2_f32": (i, [vp, vp, u, u, u, vp]),
            "tfccb200_minmax_f32": (i, [vp, vp, sz, vp]),
            "tfccb200_quantize_f32": (i, [vp, vp, sz, vp, vp, vp, i]),
            "tfccb200_quantize_rowsum_f32": (i, [vp, vp, u, u, vp, vp, vp, i, vp]),
            "tfccb200_dequantize_f32": (i, [vp, vp, i, sz, vp, vp, vp]),
            "tfccb200_requantize": (i, [vp, vp, i, sz, vp, vp, vp, vp, vp, i]),
            "tfccb200_sgemm_nsplit_push": (i, [vp, vp, vp, C.POINTER(C.c_void_p), u, u, vp, u, u, u, i, vp, vp, C.c_size_t, vp]),
            "tfccb200_sgemm_nsplit_push_ex": (i, [vp, vp, vp, C.POINTER(C.c_void_p), u, u, vp, u, u, u, i, vp, vp, C.c_size_t, u, vp]),
            "tfccb200_qgemm_nsplit_push": (i, [vp, vp, vp, i32, vp, vp, i32, C.POINTER(C.c_void_p), u, u, u, u, u, vp, vp]),
            "tfccb200_sgemm_nsplit_host": (i, [vp, vp, vp, u, vp, C.POINTER(C.c_void_p), vp, vp,
                                               C.POINTER(C.c_void_p), vp, u, u, u, u, u, i, vp, sz,
                                               BARRIER_FN, vp, vp]),
            "tfccb200_group_create": (i, [i, C.POINTER(i), C.POINTER(vp)]),
            "tfccb200_group_destroy": (i, [vp]),
            "tfccb200_group_size": (i, [vp]),
            "tfccb200_group_device": (i, [vp, i]),
            "tfccb200_group_stream": (vp, [vp, i]),
            "tfccb200_group_sync": (i, [vp]),
            "tfccb200_group_sgemm_nsplit": (i, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                                C.POINTER(vp), u, u, u, i]),
            "tfccb200_group_qgemm_nsplit": (i, [vp, C.POINTER(vp), C.POINTER(vp), i32, C.POINTER(vp),
                                                C.POINTER(vp), i32, C.POINTER(vp), u, u, u]),
            "tfccb200_group_sgemm_nsplit_host": (i, [vp, vp, vp, vp, u, u, u, i]),
            "tfccb200_sgemm_skinny_static": (i, [vp, vp, vp, vp, vp, u, u, u]),
            "tfccb200_sgemm_skinny_static_capacity": (sz, []),
            "tfccb200_sgemm_skinny_static_need": (sz, [u, u, u]),
            "tfccb200_interleave_panels_f32": (i, [vp, vp, vp, u, u, u]),
            "tfccb200_sgemm_host": (i, [vp, vp, u, vp, u, vp, u, vp, u, u, u, u, i]),
            "tfccb200_qgemm_u8s8s32_host": (i, [vp, vp, u, vp, u, f, f, f, f, vp, u,
                                                C.POINTER(f), C.POINTER(f), u, u, u, u]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(dll, name)
            fn.restype = res
            fn.argtypes = args
        self._dll = dll

    def __getattr__(self, name):
        if self._dll is None:
            self._load()
        return getattr(self._dll, name)


lib = _Lib()

EXPORTED_SYMBOLS = (
    "tfccb200_strerror", "tfccb200_version", "tfccb200_launch_count", "tfccb200_test_flag_wait",
    "tfccb200_sgemm",
    "tfccb200_sgemm_ex", "tfccb200_sgemm_workspace", "tfccb200_sgemm_path",
    "tfccb200_qgemm_u8s8s32", "tfccb200_qgemm_u8s8s32_ex", "tfccb200_qgemm_u8s8s32_dev",
    "tfccb200_quantized_matmul_params",
    "tfccb200_reduce_sum_u8", "tfccb200_reduce_sum_s8", "tfccb200_reduce_sum_s16",
    "tfccb200_sgemm_act", "tfccb200_attention_f32", "tfccb200_softmax_f32", "tfccb200_layer_norm_f32", "tfccb200_gelu_f32",
    "tfccb200_permute_0213_f32", "tfccb200_transpose_last2_f32",
    "tfccb200_minmax_f32", "tfccb200_quantize_f32", "tfccb200_quantize_rowsum_f32", "tfccb200_dequantize_f32", "tfccb200_requantize",
    "tfccb200_sgemm_nsplit_push", "tfccb200_sgemm_nsplit_push_ex", "tfccb200_qgemm_nsplit_push",
    "tfccb200_sgemm_nsplit_host", "tfccb200_group_create", "tfccb200_group_destroy",
    "tfccb200_group_size", "tfccb200_group_device", "tfccb200_group_stream", "tfccb200_group_sync",
    "tfccb200_group_sgemm_nsplit", "tfccb200_group_qgemm_nsplit",
    "tfccb200_group_sgemm_nsplit_host", "tfccb200_sgemm_skinny_static",
    "tfccb200_sgemm_skinny_static_capacity", "tfccb200_sgemm_skinny_static_need",
    "tfccb200_interleave_panels_f32", "tfccb200_sgemm_host", "tfccb200_qgemm_u8s8s32_host",
)

PATHS = {"auto": 0, "simt": 1, "skinny": 2, "umma": 3, "umma2": 4, "cluster_simt": 5}
PRECISIONS = {"fp32": 0, "tf32": 1, "bf16": 2}
ACTIVATIONS = {None: 0, "none": 0, "gelu": 1}


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.tfccb200_launch_count())


def check(status: int) -> None:
    """Turn a C-ABI status into the matching exception."""
    if status == 0:
        return
    msg = lib.tfccb200_strerror(status).decode()
    if status in (-1, -2, -4, -5, -7):
        raise exceptions.InvalidArgumentError(f"tfcc_b200 status {status}: {msg}")
    if status == -3:
        raise exceptions.ResourceExhaustedError(f"tfcc_b200 status {status}: {msg}")
    raise exceptions.RuntimeError(status, msg)
