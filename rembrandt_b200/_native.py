"""ctypes bindings of the two in-tree native libraries.

``cuda()`` returns ``librembrandt_cuda.so`` (sm_100a kernels), ``host()`` returns ``librembrandt_host.so``
(CPU runtime). Both are built on demand by ``_build.py``. Every kernel launcher returns an ``int`` status
(0 = launched); ``check()`` turns a non-zero code into an exception so a missing or broken native path is
loud, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

_LOCK = threading.Lock()
_CUDA = None
_HOST = None

vp = C.c_void_p
i32 = C.c_int
i64 = C.c_longlong
u32 = C.c_uint
u64 = C.c_ulonglong
f32 = C.c_float

_CUDA_SIGS = {
    # gemm_tc.cu
    "rb_gemm_tc": [vp, i32, i64, vp, i32, i64, i32, i32, i32, vp, i64, i32, vp, i32, vp, i32, i32, i32, i32, vp, i64,
                   vp, vp],
    "rb_conv_fprop_tc": [vp, i32, i32, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, i64, vp, i32, vp,
                         i32, i32, vp, i64, vp, vp],
    "rb_gemm_set_option": [vp, i32],
    "rb_gemm_get_option": [vp, vp],
    "rb_gemm_tune_mode": [i32],
    "rb_gemm_clear_plans": [],
    "rb_conv_wgrad_tc": [vp, i32, i32, i32, i32, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp, vp],
    "rb_num_sms": [],
    "rb_gemm_role_profile": [vp],
    "rb_gemm_last_launch": [vp],
    "rb_gemm_last_cuda_error": [],
    # conv_direct.cu
    "rb_conv_direct_fwd": [vp, vp, vp, vp] + [i32] * 14 + [vp],
    "rb_conv_direct_dgrad": [vp, vp, vp, vp] + [i32] * 13 + [vp],
    "rb_conv_direct_wgrad": [vp, vp, vp] + [i32] * 13 + [vp],
    # pool.cu
    "rb_pool_fwd": [vp, vp, vp] + [i32] * 11 + [vp],
    "rb_pool_bwd": [vp, vp, vp, vp, vp] + [i32] * 10 + [vp],
    # lrn.cu
    "rb_lrn_fwd": [vp, vp, i64, i32, i32, f32, f32, f32, vp],
    "rb_lrn_bwd": [vp, vp, vp, vp, i64, i32, i32, f32, f32, f32, vp],
    # elementwise.cu
    "rb_colsum": [vp, i64, i32, i32, vp, vp],
    "rb_gemv_sparse": [vp, i32, i32, i32, vp, vp, i32, f32, f32, vp, vp],
    "rb_bias_act": [vp, i64, i32, i32, vp, i32, vp, vp, i32, vp],
    "rb_dropout": [vp, vp, vp, i64, f32, u64, u32, vp, vp],
    "rb_relu_mask": [vp, vp, i64, vp],
    "rb_add_bf16": [vp, vp, i64, vp],
    "rb_f32_to_bf16": [vp, vp, i64, vp],
    "rb_pack_dgrad_filters": [vp, vp, i32, i32, i32, i32, vp],
    "rb_zero_s2d_structural": [vp, i32, i32, i32, i32, i32, i32, vp],
    # activations.cu
    "rb_act_fwd": [vp, i64, i32, i32, i32, f32, vp],
    "rb_act_bwd": [vp, vp, i64, i32, i32, i32, f32, vp],
    "rb_count_above": [vp, i64, i32, f32, vp, vp],
    # softmax_ce.cu
    "rb_pointwise_loss": [vp, i32, i32, i32, vp, vp, f32, vp, vp, vp, i32, vp],
    "rb_sample_categories": [vp, i32, i32, i32, vp, f32, u64, u32, vp, vp],
    "rb_categorical_loss": [vp, i32, i32, i32, vp, vp, f32, vp, vp, vp, vp, vp, vp, vp, i32, vp],
    "rb_softmax_ce": [vp, i32, i32, i32, i32, vp, vp, f32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp],
    # sgd_fused.cu
    "rb_sgd_fused": [vp, vp, vp, vp, i64, f32, f32, f32, f32, i32, i32, vp],
    "rb_sgd_fused_grid": [vp, vp, vp, vp, i64, f32, f32, f32, f32, i32, i32, i32, i32, vp],
    "rb_axpy_shadow": [vp, vp, vp, i64, f32, vp],
    "rb_axpby": [vp, vp, i64, f32, f32, vp],
    # input_pipeline.cu
    "rb_input_u8": [vp, vp, vp] + [i32] * 17 + [f32, f32, f32, vp, vp, u64, u32, vp, vp],
    "rb_var_input_u8": [vp, vp, vp, vp, i64] + [i32] * 14 + [f32, vp, f32, vp, vp, u64, u32, vp, vp],
    "rb_synth_normal": [vp, i64, i32, i32, u64, u32, vp],
    "rb_synth_labels": [vp, i32, i32, u64, u32, vp],
    # bn.cu
    "rb_bn_fwd_train": [vp, i64, i32, i32, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, vp],
    "rb_bn_fwd_infer": [vp, i64, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp, i32, vp],
    "rb_bn_bwd": [vp, vp, vp, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp],
}


class BlobRecord(C.Structure):
    _fields_ = [("tag", C.c_uint8 * 2), ("ndim", C.c_uint32), ("dims", C.c_uint64 * 8),
                ("data_offset", C.c_uint64), ("num_elems", C.c_uint64), ("next_offset", C.c_uint64)]


class Datum(C.Structure):
    _fields_ = [("channels", C.c_int32), ("height", C.c_int32), ("width", C.c_int32), ("label", C.c_int32),
                ("encoded", C.c_int32), ("data_offset", C.c_uint64), ("data_len", C.c_uint64),
                ("float_count", C.c_uint64)]


class XorShift(C.Structure):
    _fields_ = [("s", C.c_uint64 * 2)]


def _libdir() -> Path:
    return Path(__file__).resolve().parent / "lib"


def host():
    """The CPU runtime library (built on first use)."""
    global _HOST
    with _LOCK:
        if _HOST is None:
            path = _libdir() / "librembrandt_host.so"
            if not path.exists():
                from . import _build
                _build.build_host()
            lib = C.CDLL(str(path))
            lib.rb_blob_parse.argtypes = [vp, u64, u64, C.c_uint32, C.POINTER(BlobRecord)]
            lib.rb_blob_parse.restype = i32
            lib.rb_blob_record_size.argtypes = [C.c_uint32, C.POINTER(C.c_uint64), C.c_uint32]
            lib.rb_blob_record_size.restype = u64
            lib.rb_blob_write.argtypes = [vp, u64, C.POINTER(C.c_uint8), C.c_uint32, C.POINTER(C.c_uint64), vp,
                                          C.c_uint32]
            lib.rb_blob_write.restype = u64
            lib.rb_lmdb_open.argtypes = [C.c_char_p]
            lib.rb_lmdb_open.restype = vp
            for name, res in (("rb_lmdb_entries", u64), ("rb_lmdb_depth", C.c_uint32), ("rb_lmdb_page_size", C.c_uint32)):
                getattr(lib, name).argtypes = [vp]
                getattr(lib, name).restype = res
            lib.rb_lmdb_seek.argtypes = [vp, vp, C.c_uint32]
            lib.rb_lmdb_seek.restype = i32
            lib.rb_lmdb_next.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_uint32), C.POINTER(vp), C.POINTER(u64)]
            lib.rb_lmdb_next.restype = i32
            lib.rb_lmdb_close.argtypes = [vp]
            lib.rb_lmdb_close.restype = None
            lib.rb_datum_parse.argtypes = [vp, u64, C.POINTER(Datum)]
            lib.rb_datum_parse.restype = i32
            lib.rb_datum_floats.argtypes = [vp, u64, vp, u64]
            lib.rb_datum_floats.restype = u64
            lib.rb_bits_unpack.argtypes = [vp, u64, u64, C.c_uint8, vp]
            lib.rb_bits_unpack.restype = i32
            lib.rb_loader_create.argtypes = [vp, vp, u64, u64, u64, C.c_uint32, C.c_uint32, u64, C.c_uint32,
                                             C.c_uint32, C.POINTER(vp), C.POINTER(vp)]
            lib.rb_loader_create.restype = vp
            lib.rb_loader_create_lmdb.argtypes = [C.c_char_p, u64, u64, u64, C.c_uint32, C.c_uint32, u64, C.c_uint32,
                                                  C.c_uint32, C.POINTER(vp), C.POINTER(vp), C.POINTER(C.c_int32)]
            lib.rb_loader_create_lmdb.restype = vp
            lib.rb_loader_acquire.argtypes = [vp, C.POINTER(C.c_uint64)]
            lib.rb_loader_acquire.restype = i32
            lib.rb_loader_release.argtypes = [vp, i32]
            lib.rb_loader_release.restype = None
            lib.rb_loader_destroy.argtypes = [vp]
            lib.rb_loader_destroy.restype = None
            lib.rb_loader_sample_index.argtypes = [u64, u64, C.c_uint32, u64, u64]
            lib.rb_loader_sample_index.restype = u64
            lib.rb_xs_seed.argtypes = [C.POINTER(XorShift), u64, u64]
            lib.rb_xs_seed.restype = None
            lib.rb_xs_next.argtypes = [C.POINTER(XorShift)]
            lib.rb_xs_next.restype = u64
            lib.rb_xs_unit.argtypes = [C.POINTER(XorShift)]
            lib.rb_xs_unit.restype = C.c_double
            lib.rb_xs_below.argtypes = [C.POINTER(XorShift), C.c_uint32]
            lib.rb_xs_below.restype = C.c_uint32
            lib.rb_xs_fill_uniform.argtypes = [C.POINTER(XorShift), vp, u64, f32, f32]
            lib.rb_xs_fill_uniform.restype = None
            lib.rb_xs_fill_normal.argtypes = [C.POINTER(XorShift), vp, u64, f32, f32]
            lib.rb_xs_fill_normal.restype = None
            lib.rb_xs_permutation.argtypes = [C.POINTER(XorShift), vp, C.c_int32]
            lib.rb_xs_permutation.restype = None
            lib.rb_partition_range.argtypes = [u64, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64),
                                               C.POINTER(C.c_uint64)]
            lib.rb_partition_range.restype = None
            lib.rb_idx_header.argtypes = [vp, u64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                          C.POINTER(C.c_uint32 * 4), C.POINTER(C.c_uint64)]
            lib.rb_idx_header.restype = i32
            lib.rb_cifar_split.argtypes = [vp, u64, u64, u64, vp, vp]
            lib.rb_cifar_split.restype = i32
            lib.rb_mean_u8.argtypes = [vp, u64, u64, vp]
            lib.rb_mean_u8.restype = None
            _HOST = lib
    return _HOST


def cuda():
    """The sm_100a kernel library (built on first use). Loading it needs no GPU; launching does."""
    global _CUDA
    with _LOCK:
        if _CUDA is None:
            path = _libdir() / "librembrandt_cuda.so"
            if not path.exists():
                from . import _build
                _build.build_cuda()
            lib = C.CDLL(str(path))
            for name, sig in _CUDA_SIGS.items():
                fn = getattr(lib, name)
                fn.argtypes = sig
                fn.restype = i32
            _CUDA = lib
    return _CUDA


def cuda_lib_path() -> Path:
    return _libdir() / "librembrandt_cuda.so"


def register(name: str, argtypes, restype=i32):
    """Declare the signature of an additional exported launcher (used by the comm modules)."""
    fn = getattr(cuda(), name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


class NativeError(RuntimeError):
    pass


LAUNCH_COUNT = [0]   # launcher calls made through check(); the benchmark reports it per step


def check(rc: int, what: str) -> None:
    LAUNCH_COUNT[0] += 1
    if rc != 0:
        detail = ""
        if rc == -4 and _CUDA is not None:
            code = _CUDA.rb_gemm_last_cuda_error()
            if code:
                detail = f" (CUDA error {code})"
                try:
                    import torch
                    detail = f" (CUDA error {code}: {torch.cuda.cudart().cudaGetErrorString(code)})"
                except Exception:
                    pass
        raise NativeError(f"{what}: native launcher returned {rc}{detail}")


def ptr(t):
    """Device/host address of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_handle():
    import torch
    return torch.cuda.current_stream().cuda_stream
