"""ctypes binding of the C-ABI library (include/void_b200.h).

The library is the only compute path of this package: there is no CPU or PyTorch fallback.
Loading fails loudly when the shared object is missing and cannot be built.
"""
import ctypes
import os
import threading

import torch

from . import build as _build

_LOCK = threading.Lock()
_LIB = None

ABI_VERSION = 5
c_i32, c_i64, c_f32, c_vp, c_sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

# enums of include/void_b200.h
KIND_I8, KIND_F8E4M3, KIND_F16, KIND_BF16, KIND_TF32 = 0, 1, 2, 3, 4
FP_KIND = {torch.float16: KIND_F16, torch.bfloat16: KIND_BF16, torch.float32: KIND_TF32}
KIND_ELEM_BYTES = {KIND_I8: 1, KIND_F8E4M3: 1, KIND_F16: 2, KIND_BF16: 2, KIND_TF32: 4}
OUT_F32, OUT_F16, OUT_BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3
SCALE_ROW_MEAN, SCALE_PER_TILE = 0, 1

OUT_DTYPE_CODE = {torch.float32: OUT_F32, torch.float16: OUT_F16, torch.bfloat16: OUT_BF16}
ELEM_CODE = OUT_DTYPE_CODE   # VOID_ELEM_* uses the same numbering


class SpmmArgs(ctypes.Structure):
    """Mirror of ``struct void_spmm_args``."""
    _fields_ = [
        ("tiles", c_vp), ("tile_cols", c_vp), ("tile_scales", c_vp), ("row_ptr", c_vp), ("row_scale", c_vp),
        ("nbr", c_i32), ("nbc", c_i32), ("nnz", c_i64),
        ("b", c_vp), ("ldb", c_i64), ("K", c_i32), ("N", c_i32),
        ("col_scale", c_vp), ("b_scale", c_f32), ("bias", c_vp),
        ("out", c_vp), ("ldc", c_i64), ("M", c_i32), ("out_dtype", c_i32), ("act", c_i32), ("scale_mode", c_i32),
        ("acc_out", c_vp),
        ("segs", c_vp), ("cta_seg_ptr", c_vp), ("n_cta", c_i32),
        ("partials", c_vp), ("partials_bytes", c_i64), ("counters", c_vp), ("worker_partials", c_vp),
        ("status", c_vp),
        ("panels_per_item", c_i32), ("stages", c_i32), ("grid", c_i32), ("tiles_per_stage", c_i32),
        ("trace", c_vp), ("cta_shape", c_i32), ("flags", c_i32), ("row_bias", c_vp), ("transposed", c_i32), ("test_hooks", c_i32), ("tile_terms", c_i32), ("reserved", c_i32), ("n_peers", c_i32), ("peer_slots", c_i32),
        ("peer_partials", c_vp * 8), ("peer_counters", c_vp * 8), ("peer_out", c_vp * 8),
        ("row_order", c_vp),
    ]


_PROTOTYPES = {
    "void_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "void_b200_abi_version": (ctypes.c_int, []),
    "void_device_sm_count": (ctypes.c_int, []),
    "void_launch_floor": (ctypes.c_int, [c_i32, c_i32, c_i32, c_vp]),
    "void_tile_index_ws_bytes": (c_sz, [c_i32, c_i32]),
    "void_build_tile_index": (ctypes.c_int, [c_vp, c_vp, c_i64, c_i32, c_i32, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "void_format_ws_bytes": (c_sz, [c_i32, c_i32]),
    "void_dense_mark": (ctypes.c_int, [c_vp, c_i32, c_i64, c_i32, c_i32, c_f32, c_vp, c_sz, c_vp, c_vp]),
    "void_csr_mark": (ctypes.c_int, [c_vp, c_vp, c_i32, c_i32, c_vp, c_sz, c_vp, c_vp]),
    "void_morton_emit": (ctypes.c_int, [c_vp, c_i32, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "void_dense_gather": (ctypes.c_int, [c_vp, c_i32, c_i64, c_i32, c_i32, c_vp, c_vp, c_i64, c_vp, c_vp]),
    "void_csr_scatter": (ctypes.c_int, [c_vp, c_vp, c_vp, c_i32, c_i32, c_vp, c_i64, c_vp, c_vp]),
    "void_pack_tiles": (ctypes.c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_i64, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "void_pack_tiles_f8_split": (ctypes.c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "void_reduce_slots": (ctypes.c_int, [c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp, c_f32, c_vp, c_i32, c_vp, c_i64,
                                         c_i32, c_i32, c_i32, c_vp]),
    "void_pack_tiles_fp": (ctypes.c_int, [c_vp, c_i32, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "void_quant_i8_tiles": (ctypes.c_int, [c_vp, c_i64, c_vp, c_vp, c_vp]),
    "void_quant_fp8_tiles": (ctypes.c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "void_quant_cols": (ctypes.c_int, [c_vp, c_i64, c_i32, c_i32, c_i32, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "void_quant_i8_tensor": (ctypes.c_int, [c_vp, c_i64, c_i32, c_i32, c_vp, c_i64, c_vp, c_vp]),
    "void_streamk_table_capacity": (c_i64, [c_i64, c_i32]),
    "void_streamk_target": (c_i32, [c_i64, c_i32, c_i32]),
    "void_streamk_table": (ctypes.c_int, [c_vp, c_i32, c_i64, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "void_plan_capacity": (c_i64, [c_i64, c_i32, c_i32, c_i32, c_i32, c_i32]),
    "void_plan_ws_bytes": (c_sz, [c_i32, c_i32]),
    "void_plan_segments": (ctypes.c_int, [c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "void_plan_segments_host": (ctypes.c_int, [c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp, c_i64, c_vp, c_vp]),
    "void_spmm_i8": (ctypes.c_int, [ctypes.POINTER(SpmmArgs), c_vp]),
    "void_spmm_f8": (ctypes.c_int, [ctypes.POINTER(SpmmArgs), c_vp]),
    "void_spmm_fp": (ctypes.c_int, [ctypes.POINTER(SpmmArgs), c_i32, c_vp]),
    "void_spmm_tile_grad": (ctypes.c_int, [c_vp, c_i64, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp, c_i32, c_vp, c_vp,
                                           c_vp, c_i32, c_vp, c_vp]),
    "void_spmm_i8_static_scratch": (ctypes.c_int, [ctypes.POINTER(SpmmArgs), c_i32, c_vp]),
}

EXPORTED_SYMBOLS = tuple(_PROTOTYPES)


class VoidB200Error(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""


def lib_path():
    return _build.LIB_PATH


def load():
    """Load (building first when the sources are newer) and return the ctypes library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = _build.LIB_PATH
        if not os.path.exists(path) or (_build.needs_build() and _build.have_nvcc()):
            path = _build.build()
        if not os.path.exists(path):
            raise VoidB200Error(
                "void_b200: the CUDA library %s is missing and could not be built; "
                "this package has no CPU fallback" % path)
        lib = ctypes.CDLL(path)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        if lib.void_b200_abi_version() != ABI_VERSION:
            raise VoidB200Error("void_b200: ABI version mismatch, rebuild with python -m void_b200.build --force")
        _LIB = lib
    return _LIB


def check(status, what=""):
    if status != 0:
        msg = load().void_strerror(status).decode()
        raise VoidB200Error("void_b200 %s failed: %s (status %d)" % (what, msg, status))


def ptr(t):
    """Device pointer of a tensor as a ctypes void pointer (None -> NULL)."""
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise VoidB200Error(
                "void_b200 runs on a B200 GPU only: got a tensor on %s (there is no CPU path)" % t.device)


_STATUS = {}


def status_word(device):
    """Per-device int32 status word the kernels write when a bounded wait gives up."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    w = _STATUS.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _STATUS[key] = w
    return w


STATUS_TEXT = {1: "a device-side wait gave up", 2: "a split row of the work plan does not fit the scratch it was given"}


def check_device_status(device=None):
    """Synchronise and raise if a kernel on ``device`` recorded a failure in the status word.  The word is
    cleared, and so is the split-row scratch of every live work plan on the device (a launch that gave up may
    have left partial sums in it), so that the next launch starts clean."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    w = status_word(dev)
    code = int(w.item())
    if code != 0:
        w.zero_()
        from . import _spmm
        _spmm.reset_plan_scratch(dev)
        raise VoidB200Error("void_b200: %s (status word %d); the output is invalid"
                            % (STATUS_TEXT.get(code, "a kernel reported a failure"), code))
