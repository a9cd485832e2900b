"""ctypes binding of ``libechokv_b200.so`` (the C ABI declared in ``include/echokv_b200.h``).

There is no fallback: if the library is missing it is built with nvcc, and if
that fails importing this module raises.  Every wrapper takes torch CUDA
tensors, passes raw pointers / strides and the current CUDA stream, and raises
``RuntimeError`` with the library's message on a non-zero status.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
# ECHOKV_B200_LIB names another build of the same sources to load instead (e.g. an instrumented one).
LIB_PATH = Path(os.environ["ECHOKV_B200_LIB"]) if os.environ.get("ECHOKV_B200_LIB") else _HERE / "libechokv_b200.so"

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}


class Layout(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("num_kv_heads", "head_size", "block_size", "mem_bits", "k_group", "v_group")]


class LayoutInfo(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("o_v_scale", "o_v_min", "o_k_scale", "o_k_min", "o_data", "page_bytes",
                                         "chunk_bytes", "per_token_bytes")] + \
               [(n, C.c_int32) for n in ("chunks_per_page", "k_groups_per_block", "v_groups", "reserved")]


class Pages(C.Structure):
    _fields_ = [("base", C.c_void_p), ("page_stride_bytes", C.c_int64), ("num_blocks", C.c_int64),
                ("max_tier", C.c_int32), ("reserved", C.c_int32)]


class Residual(C.Structure):
    _fields_ = [("base", C.c_void_p), ("dtype", C.c_int32), ("reserved", C.c_int32),
                ("s_slot", C.c_int64), ("s_pos", C.c_int64), ("s_head", C.c_int64),
                ("block_res", C.c_void_p), ("res_group", C.c_void_p)]


def _load() -> C.CDLL:
    if not LIB_PATH.exists() or os.environ.get("ECHOKV_B200_REBUILD") == "1":
        from echokv_b200.build import build

        build(force=os.environ.get("ECHOKV_B200_REBUILD") == "1")
    lib = C.CDLL(str(LIB_PATH))
    if lib.echokv_abi_version() != 1:
        raise RuntimeError("libechokv_b200.so has an unexpected ABI version; rebuild it")
    return lib


lib = _load()
lib.echokv_last_error.restype = C.c_char_p
lib.echokv_decode_scratch_bytes.restype = C.c_int64
lib.echokv_decode_scratch_bytes.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32]
lib.echokv_decode_static_scratch_bytes.restype = C.c_int64
lib.echokv_decode_static_scratch_bytes.argtypes = []
lib.echokv_demote_scratch_bytes.restype = C.c_int64
lib.echokv_demote_scratch_bytes.argtypes = [C.POINTER(Layout), C.c_int64]

_P, _I64, _I32, _F = C.c_void_p, C.c_int64, C.c_int32, C.c_float
_LP, _PP, _RP = C.POINTER(Layout), C.POINTER(Pages), C.POINTER(Residual)
_SIGS = {
    "echokv_layout_describe": [_LP, C.POINTER(LayoutInfo)],
    "echokv_write_headers": [_PP, _P, _P, _I64, _P],
    "echokv_scatter_i64": [_P, _P, _P, _I64, _P],
    "echokv_write_tokens": [_LP, _PP, _P, _I64, _I64, _P, _I64, _I64, _I32, _P, _I64, _RP, _P, _I64, _I64, _I64, _P],
    "echokv_finalize_k": [_LP, _PP, _P, _I64, _I64, _I32, _P, _P, _RP, _I64, _P],
    "echokv_write_step": [_LP, _PP, _P, _I64, _I64, _P, _I64, _I64, _I32, _P, _I64, _RP, _P, _I64, _I64, _I64, _P, _P, _I64,
                          _P, _I64, _P, _I64, _P, _I64, _P],
    "echokv_seal_group": [_LP, _PP, _RP, _I64, _I64, _I32, _I32, _I32, _I32, _P],
    "echokv_demote_blocks": [_LP, _PP, _RP, _P, _I64, _P, _I64, _P],
    "echokv_gather": [_LP, _PP, _RP, _P, _P, _I64, _P, _P, _P],
    "echokv_decode": [_LP, _PP, _RP, _P, _I64, _I64, _I32, _P, _P, _I64, _P, _P, _P, _I64, _P, _I64, _I64, _I32,
                      _F, _I32, _I32, _I64, _I32, _P],
    "echokv_decode_ex": [_LP, _PP, _RP, _P, _I64, _I64, _I32, _P, _P, _I64, _P, _P, _P, _I64, _P, _I64, _I64, _I32,
                         _F, _I32, _I32, _P, _I64, _I32, _P],
    "echokv_decode_static": [_LP, _PP, _RP, _P, _I64, _I64, _I32, _P, _P, _I64, _P, _P, _P, _I64, _I64, _I32,
                             _F, _I32, _I32, _I64, _I32, _P],
    "echokv_dequant_dense": [_LP, _PP, _RP, _P, _I64, _P, _I64, _P, _P, _I64, _I64, _I32, _P],
    "echokv_prefill": [_P, _I64, _I64, _P, _P, _I64, _I64, _I64, _I32, _P, _I64, _I32, _P, _I64, _I64, _I32, _F, _I32,
                       _I32, _I32, _P],
    "echokv_set_decode_events": [_P, _P],
    "echokv_gather_rows": [_P, _I64, _P, _I64, _P, _I64, _P],
    "echokv_canary_kl": [_P, _I32, _I64, _I64, _I64, _P, _I64, _I64, _I64, _I32, _I32, _I32, _I32, _I32, _I32, _I32,
                         _I32, _I32, _F, _P, _P],
}
for _name, _args in _SIGS.items():
    fn = getattr(lib, _name)
    fn.argtypes = _args
    fn.restype = C.c_int

lib.echokv_set_decode_path.argtypes = [C.c_int]
lib.echokv_set_decode_path.restype = C.c_int
lib.echokv_set_decode_wait_limit.argtypes = [C.c_int64, C.c_int]
lib.echokv_set_decode_wait_limit.restype = C.c_int
lib.echokv_planner_create.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
lib.echokv_planner_create.restype = C.c_void_p
lib.echokv_planner_destroy.argtypes = [C.c_void_p]
lib.echokv_planner_destroy.restype = None
lib.echokv_planner_get.argtypes = [C.c_void_p, C.c_int32]
lib.echokv_planner_get.restype = C.c_int64
lib.echokv_planner_sealed_mask.argtypes = [C.c_void_p, C.c_int64, C.c_int64]
lib.echokv_planner_sealed_mask.restype = C.c_int64
lib.echokv_planner_plan.argtypes = [C.c_void_p, C.c_void_p, C.c_int64] + [C.c_void_p] * 12
lib.echokv_planner_plan.restype = C.c_int
lib.echokv_decode_parallelism.argtypes = [_LP, C.c_int32]
lib.echokv_decode_parallelism.restype = C.c_int32
lib.echokv_kernel_status.argtypes = [C.c_int]
lib.echokv_kernel_status.restype = C.c_int

EXPORTS = sorted(list(_SIGS) + ["echokv_set_decode_path", "echokv_set_decode_wait_limit", "echokv_kernel_status", "echokv_set_prefill_path", "echokv_decode_static_scratch_bytes", "echokv_decode_parallelism", "echokv_planner_create", "echokv_planner_destroy", "echokv_planner_get",
                                "echokv_planner_sealed_mask", "echokv_planner_plan", "echokv_abi_version", "echokv_last_error", "echokv_decode_scratch_bytes",
                                "echokv_demote_scratch_bytes"])


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"echokv_b200 [{rc}]: {lib.echokv_last_error().decode()}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("echokv_b200 kernels need CUDA tensors; there is no CPU path")


def describe(num_kv_heads, head_size, block_size, mem_bits, k_group, v_group) -> LayoutInfo:
    info = LayoutInfo()
    lay = Layout(num_kv_heads, head_size, block_size, mem_bits, k_group, v_group)
    rc = lib.echokv_layout_describe(C.byref(lay), C.byref(info))
    if rc != 0:
        raise ValueError(lib.echokv_last_error().decode())
    return info
