"""ctypes binding of libmuse_proj.so (declarations: include/muse_proj.h).

The library is the only compute path: if it is missing and cannot be built, loading raises and so
does every call that needs it. There is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

_LIB = None

# name -> (restype, argtypes); kept in one place so that the symbol-export test can walk it.
SIGNATURES = {
    "muse_abi_version": (C.c_int, []),
    "muse_set_programmatic_launch": (C.c_int, [C.c_int]),
    "muse_query": (C.c_int, [C.c_int]),
    "muse_gemv1": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                             C.c_void_p, C.c_void_p, C.c_void_p]),
    "muse_tmap_encode_2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int]),
    "muse_skinny_ws_floats": (C.c_longlong, [C.c_int, C.c_int, C.c_int]),
    "muse_skinny_tiles": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "muse_skinny_stage_bytes": (C.c_int, [C.c_int, C.c_int]),
    "muse_skinny_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                 C.c_void_p, C.c_void_p]),
    "muse_skinny_smem_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_skinny_max_clusters": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_nop": (C.c_int, [C.c_void_p]),
    "muse_copy_h2d_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "muse_copy_d2h_sync": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "muse_fetch_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "muse_fewtok_mma_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "muse_fewtok_mma": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "muse_fewtok_rowpar": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "muse_fewtok_smem_bytes": (C.c_longlong, [C.c_int, C.c_int, C.c_int]),
    "muse_fewtok_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_int, C.c_void_p]),
    "muse_attn_boundary": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "muse_fewtok_boundary": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p]),
    "muse_boundary_pooler_router": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_void_p]),
    "muse_fewtok_zip": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "muse_ffn_boundary": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "muse_unpooler_ffn_boundary": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                             C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "muse_gemm_tc_smem_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_gemm_tc_max_clusters": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_gemm_tc_ws_floats": (C.c_longlong, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_gemm_tc_cnt_ints": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "muse_gemm_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_void_p, C.c_void_p]),
    "muse_static_scratch_floats": (C.c_longlong, []),
    "muse_static_scratch_tiles": (C.c_int, []),
    "muse_skinny_tc_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p]),
}

ABI_VERSION = 18


class MuseError(RuntimeError):
    """A C-ABI call returned non-zero (negative: rejected argument; positive: CUDA error)."""


def lib_path() -> Path:
    return _build.LIB_PATH


def load(build_if_missing: bool = True):
    """Load (building first if needed) and type the library. Raises if that is impossible."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        if not build_if_missing:
            raise MuseError(f"{path} is missing: run `python -m llm_inference_engine_b200.build`")
        _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export the symbol
        fn.restype = res
        fn.argtypes = args
    if lib.muse_abi_version() != ABI_VERSION:
        raise MuseError(f"{path}: ABI {lib.muse_abi_version()} != expected {ABI_VERSION}; rebuild")
    _LIB = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        kind = "rejected argument" if rc < 0 else "CUDA error"
        raise MuseError(f"{what}: {kind} {rc}")


MAX_WORLD = 8
LL_TOKENS = 32   # MUSE_LL_TOKENS: most tokens of a column-parallel muse_fewtok_mma call
RP_TOKENS = 8    # MUSE_RP_TOKENS: most tokens of a row-parallel muse_fewtok_rowpar call


class PeerSync(C.Structure):
    """muse_peer_sync_t: where a column-parallel kernel writes its slice on every rank (muse_proj.h)."""

    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("col0", C.c_int), ("reserved", C.c_int),
                ("out", C.c_void_p * MAX_WORLD), ("flags", C.c_void_p * MAX_WORLD), ("ll", C.c_void_p * MAX_WORLD)]


class Boundary(C.Structure):
    """muse_boundary_t: the operands of the post-attention boundary (muse_proj.h)."""

    _fields_ = [("stream", C.c_void_p), ("attn_out", C.c_void_p), ("alpha", C.c_void_p), ("beta", C.c_void_p),
                ("norm_w", C.c_void_p), ("stream1", C.c_void_p), ("h", C.c_void_p), ("h_f32", C.c_void_p)]


class FfnBoundary(C.Structure):
    """muse_ffn_boundary_t: the operands of the post-FFN boundary (muse_proj.h)."""

    _fields_ = [("stream1", C.c_void_p), ("alpha", C.c_void_p), ("beta", C.c_void_p), ("post_w", C.c_void_p),
                ("next_w", C.c_void_p), ("stream2", C.c_void_p), ("hidden", C.c_void_p)]


class TensorMap:
    """A 128-byte CUtensorMap blob in host memory, 64-byte aligned as the driver requires."""

    def __init__(self):
        self._raw = C.create_string_buffer(128 + 64)
        base = C.addressof(self._raw)
        self.ptr = (base + 63) & ~63

    @classmethod
    def for_matrix(cls, data_ptr: int, rows: int, cols: int, row_stride_bytes: int, box_rows: int) -> "TensorMap":
        tm = cls()
        check(load().muse_tmap_encode_2d(tm.ptr, data_ptr, rows, cols, row_stride_bytes, box_rows),
              f"muse_tmap_encode_2d(rows={rows}, cols={cols}, box_rows={box_rows})")
        return tm
