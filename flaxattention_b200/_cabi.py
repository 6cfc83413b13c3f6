"""ctypes binding of the C ABI declared in include/flaxattn.h.

This is the stand-in for the ``jax.ffi`` custom-call layer on machines without JAX: the
same entry points, driven with raw device pointers (taken from torch CUDA tensors by the
callers in this package).  There is no CPU implementation behind it.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflaxattn.so")

FA_F16, FA_BF16, FA_F32 = 0, 1, 2
FLAG_ROUND_SCORES = 1
FLAG_GENERAL_KERNELS = 16
KIND_FWD, KIND_BWD, KIND_DECODE, KIND_BLOCKMASK = 0, 1, 2, 3


class FaTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class FaBlockTables(C.Structure):
    _fields_ = [
        ("kv_num_blocks", C.c_void_p), ("kv_indices", C.c_void_p),
        ("full_kv_num_blocks", C.c_void_p), ("full_kv_indices", C.c_void_p),
        ("q_num_blocks", C.c_void_p), ("q_indices", C.c_void_p),
        ("full_q_num_blocks", C.c_void_p), ("full_q_indices", C.c_void_p),
        ("mask_B", C.c_int32), ("mask_H", C.c_int32),
        ("num_q_blocks", C.c_int32), ("num_kv_blocks", C.c_int32),
        ("q_block_size", C.c_int32), ("kv_block_size", C.c_int32),
        ("mask_bits", C.c_void_p), ("mask_bits_stride", C.c_int64), ("mask_bits_rows", C.c_int32),
        ("mask_bits_B", C.c_int32), ("mask_bits_H", C.c_int32),
    ]


class FaAttnParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32), ("Dv", C.c_int32),
        ("scale", C.c_float),
        ("b_offset", C.c_int32), ("h_offset", C.c_int32),
        ("q", FaTensor), ("k", FaTensor), ("v", FaTensor), ("o", FaTensor),
        ("lse", C.c_void_p),
        ("tables", FaBlockTables),
        ("flags", C.c_int32),
        ("status", C.c_void_p),
    ]


class FlaxAttnError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"flaxattn error {code}: {msg}")
        self.code = code


_lib: Optional[C.CDLL] = None

# every symbol include/flaxattn.h declares
EXPORTS = [
    "fa_last_error", "fa_version", "fa_set_kernel_dir", "fa_set_cache_dir", "fa_module_create",
    "fa_module_set_buffers", "fa_module_destroy", "fa_module_prepare", "fa_compile_count", "fa_fwd", "fa_bwd_workspace_bytes",
    "fa_bwd", "fa_decode_num_splits", "fa_decode_workspace_bytes", "fa_decode",
    "fa_block_mask_workspace_bytes", "fa_block_mask", "fa_decode_static_capacity", "fa_decode_static",
    "fa_profile_enable", "fa_profile_read", "fa_decode_packs_heads", "fa_selftest_bounded_wait",
    "fa_mask_bits_row_words", "fa_mask_bits",
]


def lib() -> C.CDLL:
    """Loads libflaxattn.so.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FlaxAttnError(
            -3, f"{LIB_PATH} is missing; build it with `python -m flaxattention_b200.csrc.build` "
                "(the CUDA extension is required, there is no CPU path)")
    from .csrc.build import is_current

    if not is_current():
        raise FlaxAttnError(
            -3, f"{LIB_PATH} was built from other sources than the ones beside it (its launch parameters have to "
                "match the kernel templates); rebuild it with `python -m flaxattention_b200.csrc.build`")
    L = C.CDLL(LIB_PATH)
    L.fa_last_error.restype = C.c_char_p
    L.fa_module_create.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.fa_module_destroy.argtypes = [C.c_void_p]
    L.fa_module_set_buffers.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int]
    L.fa_module_destroy.restype = None
    L.fa_module_prepare.argtypes = [C.c_void_p] + [C.c_int] * 6
    L.fa_set_kernel_dir.argtypes = [C.c_char_p]
    L.fa_set_cache_dir.argtypes = [C.c_char_p]
    L.fa_fwd.argtypes = [C.c_void_p, C.POINTER(FaAttnParams), C.c_void_p]
    L.fa_block_mask_workspace_bytes.restype = C.c_size_t
    L.fa_block_mask_workspace_bytes.argtypes = [C.c_int] * 6
    L.fa_block_mask.argtypes = [C.c_void_p] + [C.c_int] * 8 + [C.c_void_p] * 8 + [C.c_void_p, C.c_size_t, C.c_void_p]
    if hasattr(L, "fa_bwd"):
        L.fa_bwd_workspace_bytes.restype = C.c_size_t
        L.fa_bwd_workspace_bytes.argtypes = [C.POINTER(FaAttnParams)]
        L.fa_bwd.argtypes = [C.c_void_p, C.POINTER(FaAttnParams)] + [C.POINTER(FaTensor)] * 4 + [
            C.c_void_p, C.c_size_t, C.c_void_p]
    if hasattr(L, "fa_decode"):
        L.fa_decode_num_splits.argtypes = [C.POINTER(FaAttnParams), C.c_int]
        L.fa_decode_packs_heads.argtypes = [C.POINTER(FaAttnParams)]
        L.fa_decode_workspace_bytes.restype = C.c_size_t
        L.fa_decode_workspace_bytes.argtypes = [C.POINTER(FaAttnParams), C.c_int]
        L.fa_decode.argtypes = [C.c_void_p, C.POINTER(FaAttnParams), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    if hasattr(L, "fa_decode_static"):
        L.fa_decode_static_capacity.restype = C.c_size_t
        L.fa_decode_static.argtypes = [C.c_void_p, C.POINTER(FaAttnParams), C.c_int, C.c_void_p]
    L.fa_profile_enable.argtypes = [C.c_int]
    L.fa_profile_read.argtypes = [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_char_p)]
    L.fa_selftest_bounded_wait.argtypes = [C.c_ulonglong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.fa_mask_bits_row_words.restype = C.c_int64
    L.fa_mask_bits_row_words.argtypes = [C.c_int]
    L.fa_mask_bits.argtypes = [C.c_void_p] + [C.c_int] * 6 + [C.c_void_p, C.c_void_p]
    L.fa_set_kernel_dir(os.path.join(_HERE, "csrc", "kernels").encode())
    cache = os.environ.get("FLAXATTN_CACHE_DIR")
    if cache is None:
        # keep compiled kernels beside the package when it is writable, so that a checkout
        # carries its kernel cache with it
        local = os.path.join(_HERE, "_kernel_cache")
        try:
            os.makedirs(local, exist_ok=True)
            if os.access(local, os.W_OK):
                L.fa_set_cache_dir(local.encode())
        except OSError:
            pass
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != 0:
        raise FlaxAttnError(rc, lib().fa_last_error().decode(errors="replace"))


class Module:
    """Owns one ``fa_module`` (a lowered score_mod / mask_mod pair)."""

    def __init__(self, mod_source: Optional[str]):
        L = lib()
        h = C.c_void_p()
        check(L.fa_module_create(mod_source.encode() if mod_source else None, C.byref(h)))
        self.handle = h

    def set_buffers(self, ptrs) -> None:
        """Device addresses of the tensors the mods index (``fa_module_set_buffers``)."""
        arr = (C.c_void_p * max(len(ptrs), 1))(*ptrs)
        check(lib().fa_module_set_buffers(self.handle, arr, len(ptrs)))

    def prepare(self, kind: int, dtype: int, D: int, Dv: int, sq_hint: int = 1024, skv_hint: int = 1024) -> None:
        check(lib().fa_module_prepare(self.handle, kind, dtype, D, Dv, sq_hint, skv_hint))

    def __del__(self):
        try:
            if self.handle and _lib is not None:
                _lib.fa_module_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def profile_enable(on: bool) -> None:
    """Switches the per-kernel event timing of fa_fwd / fa_bwd / fa_decode on or off."""
    check(lib().fa_profile_enable(1 if on else 0))


def selftest_bounded_wait(limit_ns: int, status_ptr: int, gave_up_ptr: int, waited_ns_ptr: int, stream: int = 0) -> None:
    """Launches the kernel whose only job is to let a bounded mbarrier wait run out (see
    include/flaxattn.h); the three pointers are device-accessible, zeroed words."""
    check(lib().fa_selftest_bounded_wait(limit_ns, status_ptr, gave_up_ptr, waited_ns_ptr, stream))


def profile_read(max_kernels: int = 16):
    """[(kernel name, milliseconds)] of this thread's most recent timed call, in launch order."""
    ms = (C.c_float * max_kernels)()
    names = (C.c_char_p * max_kernels)()
    n = lib().fa_profile_read(max_kernels, ms, names)
    if n < 0:
        check(n)
    return [(names[i].decode(), float(ms[i])) for i in range(min(n, max_kernels))]
