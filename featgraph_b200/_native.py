"""ctypes binding of libfeatgraph_b200.so (the C ABI declared in include/featgraph_b200.h).

There is no CPU fallback: if the library is missing and cannot be built, or a call
fails, an exception is raised.
"""
import ctypes
import os

from . import build as _build

_i32, _i64, _vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p

FG_OK = 0
ERROR_NAMES = {1: "invalid argument", 2: "CUDA error", 3: "out of device memory", 4: "bad index"}

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "fg_version": (ctypes.c_int, []),
    "fg_last_error": (ctypes.c_char_p, []),
    "fg_kernel_signature": (ctypes.c_char_p, []),
    "fg_kernel_launch_count": (_i64, []),
    "fg_device_info": (ctypes.c_int, [_vp, _vp, _vp, _vp]),
    "fg_row_schedule_create": (ctypes.c_int, [_vp, _i64, _i32, _vp, _vp]),
    "fg_row_schedule_order": (_vp, [_vp]),
    "fg_row_schedule_num_rows": (_i64, [_vp]),
    "fg_row_schedule_rows_at_least": (_i64, [_vp, _i64]),
    "fg_row_schedule_destroy": (None, [_vp]),
    "fg_spmm_csr_f32": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_spmm_sddmm_fused_f32": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64,
                                               _i32, _vp]),
    "fg_spmm_csr_f32_static": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_spmm_dds_f32": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "fg_sddmm_coo_f32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp]),
    "fg_sddmm_auto_partitions": (_i32, [_i64, _i64, _i64, _i32]),
    "fg_sddmm_plan_create": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "fg_sddmm_plan_partitions": (_i32, [_vp]),
    "fg_sddmm_plan_batches": (_i64, [_vp]),
    "fg_sddmm_plan_destroy": (None, [_vp]),
    "fg_sddmm_coo_f32_planned": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_sddmm_coo_f32_exact": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_spmm_csr_f32_host": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "fg_sddmm_coo_f32_host": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp]),
    "fg_sddmm_coo_f32_planned_host": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_host_sync": (ctypes.c_int, [_vp]),
    "fg_spmm_csr_reduce_f32": (ctypes.c_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_edge_binary_f32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fg_gather_rows_f32": (ctypes.c_int, [_vp, _i64, _vp, _i64, _i32, _vp, _i64, _vp]),
    "fg_csr_validate": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    "fg_coo_validate": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
}

_lib = None


class FeatGraphError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, text):
        super().__init__("featgraph_b200: %s: %s" % (ERROR_NAMES.get(code, "error %d" % code), text))
        self.code = code


def library_path():
    return _build.CUDA_LIB


def lib():
    """Load and return the ctypes library.  Where nvcc is present the library is first brought up
    to date with its sources (``build.build_cuda()`` compiles only what is older than a source or
    header and does nothing otherwise), so an edited kernel can never be tested against a stale
    binary.  Without nvcc an existing library is loaded as it is; with neither, this raises.
    ``FEATGRAPH_B200_LIB=/path/to/lib.so`` loads that file instead, without building."""
    global _lib
    if _lib is None:
        path = _build.CUDA_LIB
        override = os.environ.get("FEATGRAPH_B200_LIB")  # a prebuilt library to load as it is
        try:
            _build._nvcc()
            have_nvcc = True
        except RuntimeError:
            have_nvcc = False
        if override:
            path = override
        elif have_nvcc:
            path = _build.build_cuda(force=bool(os.environ.get("FEATGRAPH_B200_REBUILD")))
        elif not os.path.exists(path):
            raise RuntimeError("featgraph_b200: %s is missing and nvcc is not available to build it "
                               "(there is no CPU fallback)" % path)
        L = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)  # AttributeError here = header and library out of step
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != FG_OK:
        raise FeatGraphError(rc, lib().fg_last_error().decode("utf-8", "replace"))


def device_info():
    sm, ma, mi = _i32(), _i32(), _i32()
    l2 = _i64()
    check(lib().fg_device_info(ctypes.byref(sm), ctypes.byref(ma), ctypes.byref(mi), ctypes.byref(l2)))
    return {"sm_count": sm.value, "cc": (ma.value, mi.value), "l2_bytes": l2.value}
