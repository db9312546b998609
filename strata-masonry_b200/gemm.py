"""Python face of the C ABI for the two GEMMs.

Host-array helpers (`*_host`) take and return NumPy arrays and go through the library's
host-buffer entry points (upload, run, download).  Plan classes wrap device pointers (any
object with ``data_ptr()``, e.g. a torch CUDA tensor, or a raw integer address) and are what
timing loops use.  Nothing in here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if isinstance(x, np.ndarray):
        return int(x.ctypes.data)
    raise TypeError(f"cannot take the address of {type(x)!r}")


def _stream_ptr(stream) -> int:
    if stream is None:
        return 0
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


# ------------------------------------------------------------------------------- BF16
def dense_gemm_bf16_host(a_bits: np.ndarray, bt_bits: np.ndarray) -> np.ndarray:
    """D = bf16(A . BT^T) for host arrays of bf16 bit patterns: A [M,K], BT [N,K] -> D [M,N]."""
    a = np.ascontiguousarray(a_bits, dtype=np.uint16)
    bt = np.ascontiguousarray(bt_bits, dtype=np.uint16)
    if a.ndim != 2 or bt.ndim != 2 or a.shape[1] != bt.shape[1]:
        raise ValueError("A must be [M,K] and BT [N,K]")
    m, k = a.shape
    n = bt.shape[0]
    d = np.empty((m, n), dtype=np.uint16)
    capi.check(capi.lib().smb_dense_gemm_bf16_host(a.ctypes.data, bt.ctypes.data, d.ctypes.data, m, n, k))
    return d



def _peer_array(dst):
    """List of destination addresses (ints, tensors, arrays) -> (count, ctypes array)."""
    addrs = [_ptr(x) if not isinstance(x, int) else x for x in dst]
    arr = (C.c_void_p * max(1, len(addrs)))(*addrs)
    return len(addrs), arr


class Bf16Plan:
    """Tensor maps + tile choice for one (A, BT, D) device buffer set."""

    def __init__(self, a, bt, d, m: int, n: int, k: int, lda: int | None = None,
                 ldb: int | None = None, ldd: int | None = None, flags: int = 0):
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m, n, k)
        self._keep = (a, bt, d)
        capi.check(self._lib.smb_bf16_plan_create(
            C.byref(self._h), _ptr(a), _ptr(bt), _ptr(d), m, n, k,
            k if lda is None else lda, k if ldb is None else ldb, n if ldd is None else ldd, flags))

    @classmethod
    def grouped(cls, a, bt_stacked, d, m_total: int, n: int, k: int, groups: int, mtile_group, flags: int = 0):
        """Grouped (mixture-of-experts) GEMM: rows of A sorted by group, every group padded to a
        multiple of 256 rows; `mtile_group` is a device int32 array with the group of every
        256-row tile."""
        self = cls.__new__(cls)
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m_total, n, k)
        self._keep = (a, bt_stacked, d, mtile_group)
        capi.check(self._lib.smb_bf16_grouped_plan_create(
            C.byref(self._h), _ptr(a), _ptr(bt_stacked), _ptr(d), m_total, n, k, groups, _ptr(mtile_group), flags))
        return self

    @classmethod
    def grouped_offsets(cls, a, bt_stacked, d, n: int, k: int, offsets, flags: int = 0):
        """Grouped GEMM over groups of any row count: `offsets` = groups + 1 row offsets into A / D."""
        self = cls.__new__(cls)
        self._lib = capi.lib()
        self._h = C.c_void_p()
        offs = [int(x) for x in offsets]
        self.shape = (offs[-1], n, k)
        self._keep = (a, bt_stacked, d)
        arr = (C.c_int * len(offs))(*offs)
        capi.check(self._lib.smb_bf16_grouped_plan_create_offsets(
            C.byref(self._h), _ptr(a), _ptr(bt_stacked), _ptr(d), n, k, len(offs) - 1, arr, flags))
        return self

    def tune(self, group_m: int = 0, max_clusters: int = 0) -> None:
        capi.check(self._lib.smb_bf16_plan_tune(self._h, group_m, max_clusters))

    def set_profile(self, counters) -> None:
        capi.check(self._lib.smb_bf16_plan_set_profile(self._h, _ptr(counters)))

    def set_peer_copies(self, dst, ld: int) -> None:
        """Every stored box of D also goes to dst[i] + row * ld (elements): the fused all-gather."""
        count, arr = _peer_array(dst)
        self._peer_keep = dst
        capi.check(self._lib.smb_bf16_plan_set_peer_copies(self._h, count, arr, ld))

    def set_row_route(self, dst, rows_per_block: int, ld: int, first_block: int = 0) -> None:
        """Rows of block b go to dst[b] only (D itself is not written): the fused scatter.  The tile
        walk starts at `first_block`; give every rank a different one."""
        count, arr = _peer_array(dst)
        self._peer_keep = dst
        capi.check(self._lib.smb_bf16_plan_set_row_route(self._h, count, arr, rows_per_block, ld, first_block))

    def run(self, stream=None) -> None:
        capi.check(self._lib.smb_bf16_plan_run(self._h, _stream_ptr(stream)))

    def describe(self) -> str:
        buf = C.create_string_buffer(160)
        capi.check(self._lib.smb_bf16_plan_describe(self._h, buf, 160))
        return buf.value.decode()

    def wait_probe(self, budget_cycles: int = 200_000, stream=None) -> None:
        """Self test of the bounded device waits: the next check() raises SMB_ERR_DEVICE."""
        capi.check(self._lib.smb_bf16_plan_wait_probe(self._h, budget_cycles, _stream_ptr(stream)))

    def check(self, stream=None) -> None:
        capi.check(self._lib.smb_bf16_plan_check(self._h, _stream_ptr(stream)))

    def close(self) -> None:
        if self._h:
            self._lib.smb_bf16_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Bf16HostContext:
    """Host-buffer GEMM with device buffers, plan and stream kept between calls."""

    def __init__(self, m: int, n: int, k: int, comm=None):
        """With `comm` (a Comm): the sharded form, n = this rank's columns, run() takes this
        rank's M / world rows of A and all ranks call it together."""
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m, n, k)
        self._comm = comm
        if comm is None:
            capi.check(self._lib.smb_bf16_host_ctx_create(C.byref(self._h), m, n, k))
        else:
            capi.check(self._lib.smb_bf16_host_ctx_create_sharded(C.byref(self._h), m, n, k, comm._h))

    def run(self, a, bt, d) -> None:
        """a [M,K], bt [N,K], d [M,N]: host buffers of bf16 bit patterns (NumPy arrays, pinned
        torch tensors or raw addresses)."""
        capi.check(self._lib.smb_bf16_host_ctx_run(self._h, _ptr(a), _ptr(bt), _ptr(d)))

    def close(self) -> None:
        if self._h:
            self._lib.smb_bf16_host_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------- fills
def fill_bf16_device(out, rows: int, cols: int, fill: int, seed: int, index0: int = 0,
                     row_stride: int | None = None, col_stride: int = 1, ld: int | None = None,
                     stream=None) -> None:
    capi.check(capi.lib().smb_fill_bf16_device(
        _ptr(out), rows, cols, cols if ld is None else ld, index0,
        cols if row_stride is None else row_stride, col_stride, fill, seed, _stream_ptr(stream)))


def fill_bf16_host(rows: int, cols: int, fill: int, seed: int, index0: int = 0,
                   row_stride: int | None = None, col_stride: int = 1) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.uint16)
    capi.check(capi.lib().smb_fill_bf16_host(
        out.ctypes.data, rows, cols, cols, index0, cols if row_stride is None else row_stride,
        col_stride, fill, seed))
    return out


def bf16_operands_device(a, bt, m: int, n: int, k: int, fill: int, n0: int = 0,
                         n_total: int | None = None, stream=None) -> None:
    """Fill A [m,k] and BT [n,k] on the device as the reference driver would on the host
    (A index m*K+k seed 1; B index k*N+n seed 2, stored transposed)."""
    n_total = n if n_total is None else n_total
    fill_bf16_device(a, m, k, fill, 1, 0, k, 1, stream=stream)
    fill_bf16_device(bt, n, k, fill, 2, n0, 1, n_total, stream=stream)


def fill_fp4_host(rows: int, k: int, fill: int, which: int, row0: int = 0):
    """Returns (data [rows, k/2] u8, packed scales u8, row-major scales [rows, k/32] u8)."""
    lib = capi.lib()
    data = np.empty((rows, k // 2), dtype=np.uint8)
    sf_rm = np.empty((rows, k // 32), dtype=np.uint8)
    sf_packed = np.empty(lib.smb_sf_packed_bytes(rows, k // 32), dtype=np.uint8)
    capi.check(lib.smb_fill_fp4_host(data.ctypes.data, k // 2, sf_packed.ctypes.data,
                                     sf_rm.ctypes.data, rows, k, row0, fill, which))
    return data, sf_packed, sf_rm


def quantize_mx_host(src: np.ndarray):
    """FP32 [rows, K] -> (data [rows, K/2] u8, packed scales, row-major scales)."""
    lib = capi.lib()
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows, k = src.shape
    data = np.empty((rows, k // 2), dtype=np.uint8)
    sf_rm = np.empty((rows, k // 32), dtype=np.uint8)
    sf_packed = np.empty(lib.smb_sf_packed_bytes(rows, k // 32), dtype=np.uint8)
    capi.check(lib.smb_quantize_mx_host(src.ctypes.data, k, data.ctypes.data, k // 2,
                                        sf_packed.ctypes.data, sf_rm.ctypes.data, rows, k))
    return data, sf_packed, sf_rm


def sf_pack_host(sf_rowmajor: np.ndarray) -> np.ndarray:
    lib = capi.lib()
    sf = np.ascontiguousarray(sf_rowmajor, dtype=np.uint8)
    rows, kb = sf.shape
    out = np.empty(lib.smb_sf_packed_bytes(rows, kb), dtype=np.uint8)
    capi.check(lib.smb_sf_pack_host(sf.ctypes.data, rows, kb, out.ctypes.data))
    return out


# ------------------------------------------------------------------------------- block-scaled FP4
def dense_gemm_nvfp4_host(a_packed: np.ndarray, a_sf: np.ndarray, b_packed: np.ndarray,
                          b_sf: np.ndarray) -> np.ndarray:
    """Host arrays: A [M,K/2] u8, SFA [M,K/32] u8 (row-major), B [N,K/2] u8, SFB [N,K/32] u8
    -> D [M,N] bf16 bit patterns."""
    a = np.ascontiguousarray(a_packed, dtype=np.uint8)
    b = np.ascontiguousarray(b_packed, dtype=np.uint8)
    sa = np.ascontiguousarray(a_sf, dtype=np.uint8)
    sb = np.ascontiguousarray(b_sf, dtype=np.uint8)
    m, kh = a.shape
    n = b.shape[0]
    k = kh * 2
    if b.shape[1] != kh or sa.shape != (m, k // 32) or sb.shape != (n, k // 32):
        raise ValueError("operand shapes do not agree")
    d = np.empty((m, n), dtype=np.uint16)
    capi.check(capi.lib().smb_dense_gemm_nvfp4_host(a.ctypes.data, sa.ctypes.data, b.ctypes.data,
                                                    sb.ctypes.data, d.ctypes.data, m, n, k))
    return d


class Fp4Plan:
    """Tensor maps + tile choice for one (A, SFA, B, SFB, D) device buffer set (packed scales)."""

    def __init__(self, a, sfa, b, sfb, d, m: int, n: int, k: int, lda_bytes: int | None = None,
                 ldb_bytes: int | None = None, ldd: int | None = None, flags: int = 0):
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m, n, k)
        self._keep = (a, sfa, b, sfb, d)
        capi.check(self._lib.smb_fp4_plan_create(
            C.byref(self._h), _ptr(a), _ptr(sfa), _ptr(b), _ptr(sfb), _ptr(d), m, n, k,
            k // 2 if lda_bytes is None else lda_bytes, k // 2 if ldb_bytes is None else ldb_bytes,
            n if ldd is None else ldd, flags))

    @classmethod
    def grouped(cls, a, sfa, b_stacked, sfb_stacked, d, m_total: int, n: int, k: int, groups: int, mtile_group,
                flags: int = 0):
        """Grouped (mixture-of-experts) FP4 GEMM; see Bf16Plan.grouped."""
        self = cls.__new__(cls)
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m_total, n, k)
        self._keep = (a, sfa, b_stacked, sfb_stacked, d, mtile_group)
        capi.check(self._lib.smb_fp4_grouped_plan_create(
            C.byref(self._h), _ptr(a), _ptr(sfa), _ptr(b_stacked), _ptr(sfb_stacked), _ptr(d), m_total, n, k,
            groups, _ptr(mtile_group), flags))
        return self

    @classmethod
    def grouped_offsets(cls, a, sfa, b_stacked, sfb_stacked, d, n: int, k: int, offsets, flags: int = 0):
        """Grouped FP4 GEMM over groups that start on multiples of 128 rows; see Bf16Plan.grouped_offsets."""
        self = cls.__new__(cls)
        self._lib = capi.lib()
        self._h = C.c_void_p()
        offs = [int(x) for x in offsets]
        self.shape = (offs[-1], n, k)
        self._keep = (a, sfa, b_stacked, sfb_stacked, d)
        arr = (C.c_int * len(offs))(*offs)
        capi.check(self._lib.smb_fp4_grouped_plan_create_offsets(
            C.byref(self._h), _ptr(a), _ptr(sfa), _ptr(b_stacked), _ptr(sfb_stacked), _ptr(d), n, k,
            len(offs) - 1, arr, flags))
        return self

    @classmethod
    def from_bf16_activations(cls, x, b, sfb, d, m: int, n: int, k: int, ldx: int | None = None,
                              ldb_bytes: int | None = None, ldd: int | None = None, flags: int = 0):
        """Plan whose every run first quantises the BF16 activations `x` [M, K] on the device."""
        self = cls.__new__(cls)
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m, n, k)
        self._keep = (x, b, sfb, d)
        capi.check(self._lib.smb_fp4_plan_create_bf16_activations(
            C.byref(self._h), _ptr(x), k if ldx is None else ldx, _ptr(b), _ptr(sfb), _ptr(d), m, n, k,
            k // 2 if ldb_bytes is None else ldb_bytes, n if ldd is None else ldd, flags))
        return self

    def tune(self, group_m: int = 0, max_clusters: int = 0, prefetch: int = -1) -> None:
        capi.check(self._lib.smb_fp4_plan_tune(self._h, group_m, max_clusters, prefetch))

    def set_profile(self, counters) -> None:
        capi.check(self._lib.smb_fp4_plan_set_profile(self._h, _ptr(counters)))

    def set_peer_copies(self, dst, ld: int) -> None:
        count, arr = _peer_array(dst)
        self._peer_keep = dst
        capi.check(self._lib.smb_fp4_plan_set_peer_copies(self._h, count, arr, ld))

    def set_row_route(self, dst, rows_per_block: int, ld: int, first_block: int = 0) -> None:
        count, arr = _peer_array(dst)
        self._peer_keep = dst
        capi.check(self._lib.smb_fp4_plan_set_row_route(self._h, count, arr, rows_per_block, ld, first_block))

    def set_alpha(self, alpha: float) -> None:
        """Output factor of a FLAG_SCALE_BLOCK16 plan: 1 / (global scale of A x global scale of B)."""
        capi.check(self._lib.smb_fp4_plan_set_alpha(self._h, alpha))

    def run(self, stream=None) -> None:
        capi.check(self._lib.smb_fp4_plan_run(self._h, _stream_ptr(stream)))

    def describe(self) -> str:
        buf = C.create_string_buffer(160)
        capi.check(self._lib.smb_fp4_plan_describe(self._h, buf, 160))
        return buf.value.decode()

    def wait_probe(self, budget_cycles: int = 200_000, stream=None) -> None:
        """Self test of the bounded device waits: the next check() raises SMB_ERR_DEVICE."""
        capi.check(self._lib.smb_fp4_plan_wait_probe(self._h, budget_cycles, _stream_ptr(stream)))

    def check(self, stream=None) -> None:
        capi.check(self._lib.smb_fp4_plan_check(self._h, _stream_ptr(stream)))

    def close(self) -> None:
        if self._h:
            self._lib.smb_fp4_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Fp4HostContext:
    """Host-buffer FP4 GEMM with device buffers, plans and streams kept between calls: codes and
    row-major scale bytes go up, the scales are packed on the device, D comes back."""

    def __init__(self, m: int, n: int, k: int, comm=None):
        """With `comm` (a Comm): the sharded form, n = this rank's columns, run() takes this
        rank's M / world rows of A and of its scales, and all ranks call it together."""
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.shape = (m, n, k)
        self._comm = comm
        if comm is None:
            capi.check(self._lib.smb_fp4_host_ctx_create(C.byref(self._h), m, n, k))
        else:
            capi.check(self._lib.smb_fp4_host_ctx_create_sharded(C.byref(self._h), m, n, k, comm._h))

    def run(self, a, sfa, b, sfb, d) -> None:
        """a [M,K/2] u8, sfa [M,K/32] u8, b [N,K/2] u8, sfb [N,K/32] u8, d [M,N] bf16 bits: host
        buffers (NumPy arrays, pinned torch tensors or raw addresses).  b = sfb = None keeps the
        weights of the previous run on the device."""
        capi.check(self._lib.smb_fp4_host_ctx_run(self._h, _ptr(a), _ptr(sfa), _ptr(b), _ptr(sfb), _ptr(d)))

    def close(self) -> None:
        if self._h:
            self._lib.smb_fp4_host_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Comm:
    """One rank's NCCL communicator behind the C ABI (one process per GPU)."""

    def __init__(self, comm_id: bytes, world: int, rank: int):
        self._lib = capi.lib()
        self._h = C.c_void_p()
        self.world, self.rank = world, rank
        capi.check(self._lib.smb_comm_create(C.byref(self._h), comm_id, world, rank))

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(capi.COMM_ID_BYTES)
        capi.check(capi.lib().smb_comm_unique_id(buf))
        return buf.raw

    def allgather_columns(self, slab, gathered, d_full, m: int, n_local: int, ldd: int | None = None,
                          stream=None) -> None:
        """[M, n_local] slabs of all ranks -> `gathered` [world, M, n_local]; with d_full also the
        row-major [M, world * n_local] copy."""
        capi.check(self._lib.smb_allgather_columns(
            self._h, _ptr(slab), _ptr(gathered), _ptr(d_full), m, n_local,
            self.world * n_local if ldd is None else ldd, _stream_ptr(stream)))

    def close(self) -> None:
        if self._h:
            self._lib.smb_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sum_slots_bf16_device(slots, d, count: int, elems: int, stream=None) -> None:
    """d[i] = bf16(sum over `count` consecutive slots of `elems` bf16 each), fp32 accumulation."""
    capi.check(capi.lib().smb_sum_slots_bf16_device(_ptr(slots), _ptr(d), count, elems, _stream_ptr(stream)))


def unshard_columns_device(gathered, d, g: int, m: int, n_local: int, ldd: int | None = None,
                           stream=None) -> None:
    """[g, M, N/g] (all-gathered slabs) -> row-major [M, N] on the device."""
    capi.check(capi.lib().smb_unshard_columns_device(
        _ptr(gathered), _ptr(d), g, m, n_local, g * n_local if ldd is None else ldd, _stream_ptr(stream)))


def fill_fp4_device(data, sf_packed, sf_rowmajor, rows: int, k: int, fill: int, which: int,
                    row0: int = 0, ld_bytes: int | None = None, stream=None) -> None:
    capi.check(capi.lib().smb_fill_fp4_device(
        _ptr(data), k // 2 if ld_bytes is None else ld_bytes, _ptr(sf_packed), _ptr(sf_rowmajor),
        rows, k, row0, fill, which, _stream_ptr(stream)))


def sf_packed_bytes(rows: int, k: int) -> int:
    return int(capi.lib().smb_sf_packed_bytes(rows, k // 32))
