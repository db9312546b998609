"""ctypes prototypes for every symbol declared in include/strata_masonry_b200.h.

``lib()`` loads the shared library built by build.py (and fails loudly if it is missing:
there is no fallback implementation).  ``DECLARED`` lists (name, restype, argtypes) for each
exported function; the CPU test suite checks that the library exports all of them.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "lib" / "libstrata_masonry_b200.so"

SMB_OK = 0
SMB_ERR_INVALID = -1
SMB_ERR_UNSUPPORTED = -2
SMB_ERR_CUDA = -3
SMB_ERR_DEVICE = -4
SMB_ERR_IO = -5
SMB_ERR_NOMEM = -6

FLAG_NONE = 0
FLAG_FORCE_PLAIN_STORE = 1
FLAG_TILE_N_128 = 2
FLAG_TILE_N_64 = 4
FLAG_TILE_N_256 = 8
FLAG_TILE_N_512 = 16
FLAG_TILE_N_384 = 32
FLAG_NO_DECODE = 64
FLAG_NO_LAUNCH_OVERLAP = 128
FLAG_DYNAMIC_TILES = 256
FLAG_OPERANDS_STATIC = 1024
FLAG_DECODE_DUAL = 512
FLAG_DECODE_SINGLE = 2048
FLAG_LAUNCH_INDEPENDENT = 4096
FLAG_EPILOGUE_SWIGLU = 8192
FLAG_SCALE_BLOCK16 = 16384
FLAG_ACT_QUANT_PER_CTA = 32768
FLAG_ACT_QUANT_CHAINED = 65536
FLAG_ACT_QUANT_SHARED = 131072
FLAG_TILE_N_192 = 262144
FLAG_STREAM_K = 524288

_vp = C.c_void_p
_i = C.c_int
_i64 = C.c_int64
_u64 = C.c_uint64
_u32 = C.c_uint32

DECLARED = [
    ("smb_version", _i, []),
    ("smb_last_error", C.c_char_p, []),
    ("smb_fill_bf16_device", _i, [_vp, _i64, _i64, _i64, _u64, _u64, _u64, _i, _u32, _vp]),
    ("smb_fill_bf16_host", _i, [_vp, _i64, _i64, _i64, _u64, _u64, _u64, _i, _u32]),
    ("smb_fill_fp4_device", _i, [_vp, _i64, _vp, _vp, _i64, _i64, _u64, _i, _i, _vp]),
    ("smb_fill_fp4_host", _i, [_vp, _i64, _vp, _vp, _i64, _i64, _u64, _i, _i]),
    ("smb_quantize_mx_device", _i, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _vp]),
    ("smb_quantize_mx_host", _i, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64]),
    ("smb_quantize_nvf4_device", _i, [_vp, _i64, C.c_float, _vp, _i64, _vp, _vp, _i64, _i64, _vp]),
    ("smb_quantize_nvf4_host", _i, [_vp, _i64, C.c_float, _vp, _i64, _vp, _vp, _i64, _i64]),
    ("smb_quantize_mx_bf16_device", _i, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _vp]),
    ("smb_sf_packed_bytes", C.c_size_t, [_i64, _i64]),
    ("smb_sf_pack_host", _i, [_vp, _i64, _i64, _vp]),
    ("smb_debug_smem_desc", _u64, [_u32, _u32, _u32, _u32]),
    ("smb_debug_idesc_bf16", _u32, [_i, _i]),
    ("smb_debug_idesc_mxf4", _u32, [_i, _i, _u32, _u32, _i]),
    ("smb_debug_tile_coords", None, [_i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    ("smb_debug_sf_offset", _u64, [_u32, _u32, _u32]),
    ("smb_debug_fp4_phases", None, [_i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    ("smb_debug_fp4_tile", None, [_i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    ("smb_debug_fp4_arun_split", _i, [_i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    ("smb_debug_bf16_streamk_plan", _i, [C.c_longlong, _i, _i, C.POINTER(_i)]),
    ("smb_bf16_plan_create", _i, [C.POINTER(_vp), _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, C.c_uint]),
    ("smb_bf16_grouped_plan_create", _i, [C.POINTER(_vp), _vp, _vp, _vp, _i, _i, _i, _i, _vp, C.c_uint]),
    ("smb_bf16_grouped_plan_create_offsets", _i, [C.POINTER(_vp), _vp, _vp, _vp, _i, _i, _i, C.POINTER(_i), C.c_uint]),
    ("smb_fp4_grouped_plan_create_offsets", _i,
     [C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _i, _i, _i, C.POINTER(_i), C.c_uint]),
    ("smb_bf16_plan_run", _i, [_vp, _vp]),
    ("smb_bf16_plan_check", _i, [_vp, _vp]),
    ("smb_bf16_plan_destroy", _i, [_vp]),
    ("smb_bf16_plan_describe", _i, [_vp, C.c_char_p, C.c_size_t]),
    ("smb_fp4_plan_describe", _i, [_vp, C.c_char_p, C.c_size_t]),
    ("smb_bf16_plan_wait_probe", _i, [_vp, C.c_longlong, _vp]),
    ("smb_bf16_plan_tune", _i, [_vp, _i, _i]),
    ("smb_bf16_plan_set_profile", _i, [_vp, _vp]),
    ("smb_dense_gemm_bf16", _i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    ("smb_dense_gemm_bf16_host", _i, [_vp, _vp, _vp, _i, _i, _i]),
    ("smb_bf16_host_ctx_create", _i, [C.POINTER(_vp), _i, _i, _i]),
    ("smb_bf16_host_ctx_run", _i, [_vp, _vp, _vp, _vp]),
    ("smb_bf16_host_ctx_destroy", _i, [_vp]),
    ("smb_fp4_plan_create", _i, [C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, C.c_uint]),
    ("smb_fp4_plan_create_bf16_activations", _i,
     [C.POINTER(_vp), _vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, C.c_uint]),
    ("smb_fp4_plan_set_alpha", _i, [_vp, C.c_float]),
    ("smb_fp4_grouped_plan_create", _i,
     [C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, C.c_uint]),
    ("smb_fp4_plan_run", _i, [_vp, _vp]),
    ("smb_fp4_plan_check", _i, [_vp, _vp]),
    ("smb_fp4_plan_destroy", _i, [_vp]),
    ("smb_fp4_plan_wait_probe", _i, [_vp, C.c_longlong, _vp]),
    ("smb_fp4_plan_tune", _i, [_vp, _i, _i, _i]),
    ("smb_fp4_plan_set_profile", _i, [_vp, _vp]),
    ("smb_dense_gemm_nvfp4", _i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    ("smb_dense_gemm_nvfp4_host", _i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    ("smb_fp4_host_ctx_create", _i, [C.POINTER(_vp), _i, _i, _i]),
    ("smb_fp4_host_ctx_run", _i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    ("smb_fp4_host_ctx_destroy", _i, [_vp]),
    ("smb_dense_gemm_nvfp4_decode_noalloc", _i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    ("smb_decode_noalloc_set_split", _i, [_i]),
    ("smb_decode_noalloc_check", _i, [_vp]),
    ("smb_decode_noalloc_scratch_limit", C.c_size_t, []),
    ("smb_bf16_plan_set_peer_copies", _i, [_vp, _i, C.POINTER(_vp), _i64]),
    ("smb_fp4_plan_set_peer_copies", _i, [_vp, _i, C.POINTER(_vp), _i64]),
    ("smb_bf16_plan_set_row_route", _i, [_vp, _i, C.POINTER(_vp), _i, _i64, _i]),
    ("smb_fp4_plan_set_row_route", _i, [_vp, _i, C.POINTER(_vp), _i, _i64, _i]),
    ("smb_sum_slots_bf16_device", _i, [_vp, _vp, _i, _i64, _vp]),
    ("smb_peer_alloc", _i, [C.POINTER(_vp), C.c_size_t]),
    ("smb_peer_export", _i, [_vp, C.c_char_p]),
    ("smb_peer_open", _i, [C.c_char_p, C.POINTER(_vp)]),
    ("smb_peer_close", _i, [_vp]),
    ("smb_peer_free", _i, [_vp]),
    ("smb_device_synchronize", _i, []),
    ("smb_column_shard", C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    ("smb_unshard_columns_device", _i, [_vp, _vp, _i, _i, _i, _i64, _vp]),
    ("smb_comm_unique_id", _i, [C.c_char_p]),
    ("smb_comm_create", _i, [C.POINTER(_vp), C.c_char_p, _i, _i]),
    ("smb_comm_create_all", _i, [C.POINTER(_vp), _i, C.POINTER(_i)]),
    ("smb_comm_destroy", _i, [_vp]),
    ("smb_bf16_host_ctx_create_sharded", _i, [C.POINTER(_vp), _i, _i, _i, _vp]),
    ("smb_fp4_host_ctx_create_sharded", _i, [C.POINTER(_vp), _i, _i, _i, _vp]),
    ("smb_allgather_check", _i, [_i, _i, _i, _i64]),
    ("smb_allgather_columns", _i, [_vp, _vp, _vp, _vp, _i, _i, _i64, _vp]),
    ("smb_allgather_columns_multi", _i,
     [C.POINTER(_vp), _i, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _i, _i, _i64, C.POINTER(_vp)]),
]

PEER_HANDLE_BYTES = 64
COMM_ID_BYTES = 128
MAX_PEER_COPIES = 7
MAX_ROUTE_BLOCKS = 8


class SmbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"strata_masonry_b200 error {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def lib() -> C.CDLL:
    """Load the library once and attach prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python strata-masonry_b200/build.py` "
            "(there is no CPU fallback for this path)")
    handle = C.CDLL(str(LIB_PATH))
    for name, restype, argtypes in DECLARED:
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return handle


def last_error() -> str:
    return lib().smb_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != SMB_OK:
        raise SmbError(code, last_error())
