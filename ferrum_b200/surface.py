"""Host-side mirror of the reference's quantized-linear op surface, over the C ABI.

Names, argument order and error behaviour follow ``HybridModel::project / project_id /
project_mm_id(_in) / get_rows / moe_ffn / dense_ffn`` (src/hybrid/engine.rs:2881-3500) and
``Matrix::from_packed`` (src/hybrid/weights.rs:1301-1330).  Tensors are ``torch`` CUDA tensors, used
only as device memory: every computation happens inside ``libferrum_b200.so``.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import BF16, F32, Q4_K, Q6_K, Q8_0  # noqa: F401  (re-exported)


class FerrumError(RuntimeError):
    """Base of the errors below; ``status`` is the C ABI status code."""
    status = -1


class ShapeError(FerrumError):  # Error::Shape
    status = _lib.ERR_SHAPE


class RangeError(FerrumError):  # Error::Range
    status = _lib.ERR_RANGE


class DeviceMismatch(FerrumError):  # Error::DeviceMismatch
    status = _lib.ERR_DEVICE


class AliasError(FerrumError):  # Error::Dispatch("... alias")
    status = _lib.ERR_ALIAS


class WeightError(FerrumError):  # Error::Weight / Error::Gguf
    status = _lib.ERR_WEIGHT


class SynchronizationError(FerrumError):  # Error::Synchronization
    status = _lib.ERR_SYNC


class TimeoutError_(FerrumError):
    status = _lib.ERR_TIMEOUT


class CudaError(FerrumError):
    status = _lib.ERR_CUDA


class ParameterError(FerrumError):  # Error::Parameter
    status = _lib.ERR_PARAM


class Unsupported(FerrumError):
    status = _lib.ERR_UNSUPPORTED


class GgufError(FerrumError):
    """``Error::Gguf``: a malformed or truncated file, a missing tensor or metadata entry."""
    status = _lib.ERR_GGUF


_BY_STATUS = {c.status: c for c in (ShapeError, RangeError, DeviceMismatch, AliasError, WeightError,
                                    SynchronizationError, TimeoutError_, CudaError, ParameterError, Unsupported, GgufError)}


def _dtype_id(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise Unsupported(f"tensor dtype {t.dtype}")


class Device:
    """``MetalDevice`` counterpart: one CUDA device, one stream, fixed scratch."""

    def __init__(self, ordinal: int = 0, use_torch_stream: bool = True):
        self._L = _lib.load()
        h = C.c_void_p()
        rc = self._L.fq_device_create(ordinal, C.byref(h))
        if rc != _lib.OK:
            raise _BY_STATUS.get(rc, FerrumError)(f"fq_device_create({ordinal}) -> {self._L.fq_status_name(rc).decode()}")
        self.handle = h
        self.ordinal = ordinal
        self.torch_device = torch.device("cuda", ordinal)
        if use_torch_stream:
            # Share torch's current stream so tensors produced by torch are ordered with the kernels.
            self.set_stream(torch.cuda.current_stream(self.torch_device).cuda_stream)

    def check(self, rc: int) -> None:
        if rc != _lib.OK:
            msg = self._L.fq_last_error(self.handle).decode()
            raise _BY_STATUS.get(rc, FerrumError)(msg or self._L.fq_status_name(rc).decode())

    def set_stream(self, cuda_stream: Optional[int]) -> None:
        self.check(self._L.fq_device_set_stream(self.handle, C.c_void_p(cuda_stream or 0)))

    def stream_ptr(self) -> int:
        """The ``cudaStream_t`` enqueues currently go to."""
        return int(self._L.fq_device_stream(self.handle) or 0)

    def synchronize(self) -> None:
        self.check(self._L.fq_synchronize(self.handle))

    def recover(self) -> None:
        self.check(self._L.fq_device_recover(self.handle))

    def set_exact(self, on: bool) -> None:
        self.check(self._L.fq_set_exact(self.handle, int(on)))

    def counters(self) -> _lib.Counters:
        c = _lib.Counters()
        self.check(self._L.fq_get_counters(self.handle, C.byref(c)))
        return c

    def fail_after(self, n: int) -> None:
        self.check(self._L.fq_test_fail_after(self.handle, n))

    def fail_completion(self) -> None:
        self.check(self._L.fq_test_fail_completion(self.handle))

    def set_profiling(self, enabled: bool) -> None:
        """`MetalDevice::set_profiling` (src/metal/mod.rs:636-639): per-operation table on / off, cleared either way."""
        self.check(self._L.fq_set_profiling(self.handle, 1 if enabled else 0))

    def take_profile(self) -> dict:
        """`MetalDevice::take_profile` (src/metal/mod.rs:649-651): waits, then returns and clears the table:
        ``{name: {"calls", "kernels", "wall_ns", "gpu_ns", "gpu_samples"}}`` in name order."""
        cap = 256
        buf = (_lib.ProfileEntry * cap)()
        n = C.c_size_t(0)
        self.check(self._L.fq_take_profile(self.handle, buf, cap, C.byref(n)))
        return {buf[i].name.decode(): {k: int(getattr(buf[i], k)) for k in ("calls", "kernels", "wall_ns", "gpu_ns", "gpu_samples")}
                for i in range(min(n.value, cap))}

    def probe_read_stream(self, data: torch.Tensor, blocks_per_sm: int = 8) -> None:
        """Enqueue a kernel that only reads ``data`` (the device's read-only streaming ceiling, timed by the caller)."""
        self.check(self._L.fq_probe_read_stream(self.handle, C.c_void_p(data.data_ptr()), data.numel() * data.element_size(), blocks_per_sm))

    def capture_begin(self) -> None:
        """Start recording enqueues (the handle must be on its own stream: ``set_stream(None)``)."""
        self.check(self._L.fq_capture_begin(self.handle))

    def capture_end(self) -> "Graph":
        g = C.c_void_p()
        self.check(self._L.fq_capture_end(self.handle, C.byref(g)))
        return Graph(self, g)

    def upload(self, dst: torch.Tensor, host: np.ndarray) -> None:
        """Enqueue a host-to-device copy (asynchronous when ``host`` is pinned memory)."""
        self.check(self._L.fq_upload(self.handle, C.c_void_p(dst.data_ptr()), C.c_void_p(host.ctypes.data), host.nbytes))

    def download_async(self, host: np.ndarray, src: torch.Tensor) -> None:
        """Enqueue a device-to-host copy; valid after the next ``synchronize``."""
        self.check(self._L.fq_download_async(self.handle, C.c_void_p(host.ctypes.data), C.c_void_p(src.data_ptr()), host.nbytes))

    def close(self) -> None:
        if self.handle:
            self._L.fq_device_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Comm:
    """Tensor-parallel exchange over NVLink peer memory: this rank's symmetric buffer plus every peer's,
    mapped through CUDA IPC.  The 64-byte handles travel through ``torch.distributed`` (plumbing only)."""

    def __init__(self, device: Device, rank: int, world: int, nbytes: int, group=None, local_peer: bool = False):
        """``local_peer`` (tests only, world 2): the peer is a second buffer on this GPU that nothing writes,
        so every wait for it runs out."""
        import torch.distributed as dist
        self.device, self.rank, self.world = device, rank, world
        self.nbytes = (nbytes + 255) // 256 * 256
        h = C.c_void_p()
        device.check(device._L.fq_comm_create(device.handle, rank, world, self.nbytes, C.byref(h)))
        self.handle = h
        if local_peer:
            device.check(device._L.fq_comm_open_local(h))
        elif world > 1:
            mine = (C.c_ubyte * 64)()
            device.check(device._L.fq_comm_handle(h, mine))
            every = [None] * world
            dist.all_gather_object(every, bytes(mine), group=group)  # works on gloo and nccl groups alike
            raw = b"".join(every)
            device.check(device._L.fq_comm_open(h, raw))
            dist.barrier(group=group)
        self.base = int(device._L.fq_comm_buffer(h))

    def view(self, offset_bytes: int, numel: int, dtype=torch.float32) -> torch.Tensor:
        """A torch view of ``numel`` elements of the local buffer (no copy)."""
        item = torch.empty((), dtype=dtype).element_size()
        assert offset_bytes % 16 == 0 and offset_bytes + numel * item <= self.nbytes

        class _Ptr:
            pass
        holder = _Ptr()
        holder.__cuda_array_interface__ = {"shape": (numel,), "typestr": {4: "<f4", 2: "<u2", 1: "|u1"}[item],
                                           "data": (self.base + offset_bytes, False), "version": 2}
        t = torch.as_tensor(holder, device=self.device.torch_device)
        return t.view(dtype) if t.dtype != dtype else t

    def set_wait_ns(self, ns: int) -> None:
        """Wall-time limit of the device-side waits for a peer."""
        self.device.check(self.device._L.fq_comm_set_wait_ns(self.handle, ns))

    def all_gather(self, offset_bytes: int, shard_bytes: int) -> None:
        """Rank r's slice is ``[offset + r * shard, + shard)``; afterwards (in stream order) all are local."""
        self.device.check(self.device._L.fq_comm_all_gather(self.device.handle, self.handle, offset_bytes, shard_bytes))

    def all_gather_rows(self, offset_bytes: int, row_bytes: int, bounds, stride: int, total_rows: int) -> None:
        """Runs of rows of unequal length: rank r owns rows ``bounds[r * stride] .. bounds[(r + 1) * stride]``
        (``bounds``: a device tensor of uint32/int32)."""
        self.device.check(self.device._L.fq_comm_all_gather_rows(self.device.handle, self.handle, offset_bytes, row_bytes,
                                                                  _ptr(bounds), stride, total_rows))

    def close(self) -> None:
        if self.handle and self.device.handle:
            self.device._L.fq_comm_destroy(self.handle)
        self.handle = None


class Graph:
    """A recorded batch of enqueues (the counterpart of one command epoch of the reference)."""

    def __init__(self, device: Device, handle: C.c_void_p):
        self.device, self.handle = device, handle

    def launch(self) -> None:
        self.device.check(self.device._L.fq_graph_launch(self.device.handle, self.handle))

    def close(self) -> None:
        if self.handle and self.device.handle:
            self.device._L.fq_graph_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GgufFile:
    """``GgufFile`` (src/loader/gguf.rs:162-530): the checked index of a GGUF file; payloads are read on demand.
    Needs no GPU."""

    def __init__(self, path: str, require_architecture: bool = True, skip_arrays_over: int = 0):
        self._L = _lib.load()
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        rc = self._L.fq_gguf_open(os.fsencode(path), int(require_architecture), skip_arrays_over, C.byref(h), err, len(err))
        if rc != _lib.OK:
            raise _BY_STATUS.get(rc, FerrumError)(err.value.decode() or self._L.fq_status_name(rc).decode())
        self.handle = h
        info = _lib.GgufInfo()
        self._check(self._L.fq_gguf_info(h, C.byref(info)))
        self.version, self.alignment = int(info.version), int(info.alignment)
        self.file_len, self.tensor_data_offset = int(info.file_len), int(info.tensor_data_offset)
        self.tensor_count, self.metadata_count = int(info.tensor_count), int(info.metadata_count)

    def _check(self, rc: int) -> None:
        if rc != _lib.OK:
            raise _BY_STATUS.get(rc, FerrumError)(self._L.fq_gguf_last_error(self.handle).decode())

    @staticmethod
    def _info(t: "_lib.GgufTensor") -> dict:
        return {"name": t.name.decode(), "dimensions": [int(t.dims[i]) for i in range(t.n_dims)], "type_id": int(t.type_id),
                "offset": int(t.offset), "byte_len": int(t.byte_len)}

    def tensor(self, name: str) -> dict:
        t = _lib.GgufTensor()
        self._check(self._L.fq_gguf_tensor_by_name(self.handle, name.encode(), C.byref(t)))
        return self._info(t)

    def tensors(self) -> list:
        out = []
        for i in range(self.tensor_count):
            t = _lib.GgufTensor()
            self._check(self._L.fq_gguf_tensor_by_index(self.handle, i, C.byref(t)))
            out.append(self._info(t))
        return out

    def read_tensor(self, name: str) -> np.ndarray:
        n = self.tensor(name)["byte_len"]
        out = np.empty(n, dtype=np.uint8)
        self._check(self._L.fq_gguf_read_tensor(self.handle, name.encode(), C.c_void_p(out.ctypes.data), n))
        return out

    def metadata_u64(self, key: str) -> int:
        v = C.c_uint64()
        self._check(self._L.fq_gguf_metadata_u64(self.handle, key.encode(), C.byref(v)))
        return int(v.value)

    def metadata_f64(self, key: str) -> float:
        v = C.c_double()
        self._check(self._L.fq_gguf_metadata_f64(self.handle, key.encode(), C.byref(v)))
        return float(v.value)

    def metadata_string(self, key: str) -> str:
        buf = C.create_string_buffer(1 << 16)
        self._check(self._L.fq_gguf_metadata_string(self.handle, key.encode(), buf, len(buf)))
        return buf.value.decode()

    def metadata_array(self, key: str) -> tuple:
        """(element type, elements in the file, elements kept)."""
        et, n, kept = C.c_uint32(), C.c_uint64(), C.c_uint64()
        self._check(self._L.fq_gguf_metadata_array(self.handle, key.encode(), C.byref(et), C.byref(n), C.byref(kept)))
        return int(et.value), int(n.value), int(kept.value)

    def close(self) -> None:
        if self.handle:
            self._L.fq_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def q3k_to_q6k(q3: np.ndarray) -> np.ndarray:
    """``q3k_to_q6k`` (src/hybrid/weights.rs:761-805) on host bytes."""
    q3 = np.ascontiguousarray(q3, dtype=np.uint8)
    blocks = q3.size // 110
    out = np.empty(blocks * 210, dtype=np.uint8)
    rc = _lib.load().fq_q3k_to_q6k(C.c_void_p(q3.ctypes.data), blocks, C.c_void_p(out.ctypes.data))
    if rc != _lib.OK:
        raise ParameterError("q3k_to_q6k")
    return out


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """ggml's reference Q8_0 row quantisation (``quantize_row``, src/hybrid/weights.rs:1397-1415) on host floats."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    rc = _lib.load().fq_quantize_q8_0(C.c_void_p(x.ctypes.data), x.size, C.c_void_p(out.ctypes.data))
    if rc != _lib.OK:
        raise ParameterError("quantize_q8_0: the length must be a multiple of 32")
    return out


class Matrix:
    """``Matrix`` counterpart (src/hybrid/weights.rs:107-143): immutable packed blocks on the device."""

    def __init__(self, device: Device, handle: C.c_void_p):
        self.device = device
        self.handle = handle
        info = _lib.MatrixInfo()
        device.check(device._L.fq_matrix_get_info(handle, C.byref(info)))
        self.rows, self.cols, self.experts = int(info.rows), int(info.cols), int(info.experts)
        self.row_bytes, self.format = int(info.row_bytes), int(info.format)
        self._byte_size = int(info.byte_size)

    @classmethod
    def from_packed(cls, device: Device, rows: int, cols: int, experts: int, fmt: int, packed) -> "Matrix":
        buf = np.ascontiguousarray(np.frombuffer(packed, dtype=np.uint8) if not isinstance(packed, np.ndarray) else packed,
                                   dtype=np.uint8)
        h = C.c_void_p()
        device.check(device._L.fq_matrix_create(device.handle, fmt, rows, cols, experts,
                                                C.c_void_p(buf.ctypes.data), buf.size, C.byref(h)))
        return cls(device, h)

    @classmethod
    def from_gguf(cls, device: Device, file: "GgufFile", name: str, experts: int, rows: int, cols: int, q3k_as_q6k: bool = False) -> "Matrix":
        """``gguf_matrix`` (src/hybrid/weights.rs:671-736)."""
        h = C.c_void_p()
        device.check(device._L.fq_matrix_from_gguf(device.handle, file.handle, name.encode(), experts, rows, cols, int(q3k_as_q6k), C.byref(h)))
        return cls(device, h)

    def byte_size(self) -> int:
        return self._byte_size

    def expert_rows(self) -> int:
        return self.rows // self.experts

    def close(self) -> None:
        if self.handle and self.device.handle:
            self.device._L.fq_matrix_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _need(d: Device, *tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.device != d.torch_device:
            raise DeviceMismatch(f"tensor on {t.device}, device handle on {d.torch_device}")
        if not t.is_contiguous():
            raise ShapeError("tensor is not contiguous")


def project(d: Device, w: Matrix, x: torch.Tensor, m: int, y: torch.Tensor) -> None:
    """``HybridModel::project(d, w, x, m, y)``: y[m, rows] = x[m, cols] . W^T."""
    _need(d, x, y)
    d.check(d._L.fq_project(d.handle, w.handle, _ptr(x), _dtype_id(x), x.numel(), m, _ptr(y), _dtype_id(y), y.numel()))


def project_many(d: Device, ws: Sequence[Matrix], x: torch.Tensor, m: int, ys: Sequence[torch.Tensor]) -> None:
    """Projections sharing x and m (q|k|v, gate|up): one launch when the matrices share format and width."""
    _need(d, x, *ys)
    n = len(ws)
    wa = (C.c_void_p * n)(*[w.handle.value for w in ws])
    ya = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    for w, y in zip(ws, ys):
        if y.numel() != m * w.rows:
            raise ShapeError(f"output of {y.numel()} values for [{m}, {w.rows}]")
    d.check(d._L.fq_project_many(d.handle, wa, n, _ptr(x), _dtype_id(x), x.numel(), m, ya, _dtype_id(ys[0])))


def project_many_gather(d: Device, comm: "Comm", offset_bytes: int, shard_bytes: int, ws: Sequence[Matrix], x: torch.Tensor, m: int,
                        ys: Sequence[torch.Tensor]) -> None:
    """Row-sharded ``project_many`` whose outputs (views of ``comm``'s buffer inside this rank's slice of the
    region) are exchanged by the projection kernel itself at decode widths, else by ``comm.all_gather``."""
    _need(d, x, *ys)
    n = len(ws)
    wa = (C.c_void_p * n)(*[w.handle.value for w in ws])
    ya = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    d.check(d._L.fq_project_many_gather(d.handle, comm.handle, offset_bytes, shard_bytes, wa, n, _ptr(x), _dtype_id(x), x.numel(), m,
                                        ya, _dtype_id(ys[0])))


def rmsnorm(d: Device, x: torch.Tensor, w: torch.Tensor, eps: float, rows: int, y: torch.Tensor) -> None:
    """``HybridModel::rmsnorm``: y = rmsnorm(x) * w over ``rows`` rows."""
    _need(d, x, w, y)
    d.check(d._L.fq_rmsnorm(d.handle, _ptr(x), _ptr(w), w.numel(), eps, rows, _ptr(y)))


def add_rmsnorm(d: Device, x, r, w, eps: float, rows: int, h, y) -> None:
    """``HybridModel::add_rmsnorm``: h = x + r, y = rmsnorm(h) * w."""
    _need(d, x, r, w, h, y)
    d.check(d._L.fq_add_rmsnorm(d.handle, _ptr(x), _ptr(r), _ptr(w), w.numel(), eps, rows, _ptr(h), _ptr(y)))


def rmsnorm_project_many(d: Device, ws: Sequence[Matrix], x: torch.Tensor, norm_w: torch.Tensor, eps: float, m: int,
                         ys: Sequence[torch.Tensor], scratch: Optional[torch.Tensor] = None) -> None:
    """``project_many`` on rmsnorm(x) * norm_w, the normalisation inside the activation preparation where it can be."""
    _need(d, x, norm_w, scratch, *ys)
    n = len(ws)
    wa = (C.c_void_p * n)(*[w.handle for w in ws])
    ya = (C.c_void_p * n)(*[_ptr(y) for y in ys])
    d.check(d._L.fq_rmsnorm_project_many(d.handle, wa, n, _ptr(x), _ptr(norm_w), eps, x.numel(), m, _ptr(scratch), ya))


def argmax(d: Device, x: torch.Tensor, n: int, rows: int, out: torch.Tensor) -> None:
    """``h_argmax``: the index of the first maximum of every row."""
    _need(d, x, out)
    d.check(d._L.fq_argmax(d.handle, _ptr(x), n, rows, _ptr(out)))


def topk_blocks(d: Device, x: torch.Tensor, n: int, rows: int, out: torch.Tensor) -> None:
    """``h_topk_blocks``: per 1024-value block the 32 largest (value, index) pairs, descending."""
    _need(d, x, out)
    d.check(d._L.fq_topk_blocks(d.handle, _ptr(x), n, rows, _ptr(out)))


def project_id(d: Device, w: Matrix, x: torch.Tensor, ids: torch.Tensor, routes: int, x_div: int, y: torch.Tensor) -> None:
    """``HybridModel::project_id``: route r uses expert ids[r] on activation row r // x_div."""
    _need(d, x, ids, y)
    if x.dtype != torch.float32 or y.dtype != torch.float32:
        raise Unsupported("expert GEMV is F32 in, F32 out")
    d.check(d._L.fq_project_id(d.handle, w.handle, _ptr(x), x.numel(), _ptr(ids), routes, x_div, _ptr(y), y.numel()))


def project_mm_id_in(d: Device, w: Matrix, x: torch.Tensor, offsets: torch.Tensor,
                     slots: Optional[tuple], max_rows: int, y: torch.Tensor) -> None:
    """``HybridModel::project_mm_id_in``: ``slots`` is ``None`` or ``(table, k)``."""
    table, groups = (slots if slots is not None else (None, w.experts))
    _need(d, x, offsets, table, y)
    d.check(d._L.fq_project_mm_id(d.handle, w.handle, _ptr(x), _dtype_id(x), x.numel(), _ptr(offsets), _ptr(table),
                                  groups, max_rows, _ptr(y), _dtype_id(y), y.numel()))


def project_mm_id(d: Device, w: Matrix, x: torch.Tensor, offsets: torch.Tensor, max_rows: int, y: torch.Tensor) -> None:
    project_mm_id_in(d, w, x, offsets, None, max_rows, y)


def get_rows(d: Device, w: Matrix, ids: torch.Tensor, y: torch.Tensor) -> None:
    """``HybridModel::get_rows``: y[t] = exact decode of row ids[t]."""
    _need(d, ids, y)
    d.check(d._L.fq_get_rows(d.handle, w.handle, _ptr(ids), ids.numel(), _ptr(y), _dtype_id(y), y.numel()))


def moe_route(d, logits, x, shared_w, experts, used, hidden, tokens, sigmoid, norm, shared_gate, ids, weights, gate):
    _need(d, logits, x, shared_w, ids, weights, gate)
    d.check(d._L.fq_moe_route(d.handle, _ptr(logits), _ptr(x), _ptr(shared_w), experts, used, hidden, tokens,
                              int(sigmoid), int(norm), int(shared_gate), _ptr(ids), _ptr(weights), _ptr(gate)))


def moe_map(d, ids, experts, routes, offsets, sorted_, position):
    _need(d, ids, offsets, sorted_, position)
    d.check(d._L.fq_moe_map(d.handle, _ptr(ids), experts, routes, _ptr(offsets), _ptr(sorted_), _ptr(position)))


def moe_gather(d, x, sorted_, hidden, used, routes, xg):
    _need(d, x, sorted_, xg)
    d.check(d._L.fq_moe_gather(d.handle, _ptr(x), _ptr(sorted_), hidden, used, routes, _ptr(xg)))


def moe_combine(d, down, weights, position, shared, gate, hidden, used, tokens, identity, out):
    _need(d, down, weights, position, shared, gate, out)
    d.check(d._L.fq_moe_combine(d.handle, _ptr(down), _ptr(weights), _ptr(position), _ptr(shared), _ptr(gate),
                                hidden, used, tokens, int(identity), _ptr(out)))


def glu(d, gate, up, out):
    _need(d, gate, up, out)
    d.check(d._L.fq_glu(d.handle, _ptr(gate), _ptr(up), gate.numel(), _ptr(out)))


def dense_ffn(d, gate: Matrix, up: Matrix, down: Matrix, x, m, scratch, out):
    _need(d, x, scratch, out)
    d.check(d._L.fq_dense_ffn(d.handle, gate.handle, up.handle, down.handle, _ptr(x), m, _ptr(scratch),
                              scratch.numel(), _ptr(out)))


@dataclass
class MoeFfn:
    """``MoeFfn`` of the reference (src/hybrid/engine.rs:2881-2906) plus its geometry."""
    router: Matrix
    gate_exps: Matrix
    up_exps: Matrix
    down_exps: Matrix
    shared_gate: Matrix
    shared_up: Matrix
    shared_down: Matrix
    shared_gate_inp: Optional[torch.Tensor]
    experts: int
    used: int
    hidden: int
    expert_ffn: int
    shared_ffn: int
    sigmoid: bool = False
    norm_weights: bool = True

    def desc(self) -> _lib.MoeFfnDesc:
        return _lib.MoeFfnDesc(
            self.router.handle, self.gate_exps.handle, self.up_exps.handle, self.down_exps.handle,
            self.shared_gate.handle, self.shared_up.handle, self.shared_down.handle,
            C.c_void_p(0 if self.shared_gate_inp is None else self.shared_gate_inp.data_ptr()),
            self.experts, self.used, self.hidden, self.expert_ffn, self.shared_ffn,
            int(self.sigmoid), int(self.norm_weights))


def moe_ffn_scratch_elems(d: Device, f: MoeFfn, m: int) -> int:
    desc = f.desc()
    return int(d._L.fq_moe_ffn_scratch_elems(C.byref(desc), m))


def moe_ffn(d: Device, f: MoeFfn, x, m, scratch, out):
    _need(d, x, scratch, out)
    desc = f.desc()
    d.check(d._L.fq_moe_ffn(d.handle, C.byref(desc), _ptr(x), m, _ptr(scratch), scratch.numel(), _ptr(out)))


def moe_ffn_ep(d: Device, comm: Comm, offset_bytes: int, f: MoeFfn, expert_first: int, x, m, scratch, out):
    """Expert-parallel ``moe_ffn``: the expert matrices of ``f`` hold this rank's experts
    ``[expert_first, expert_first + E / world)``; the expert rows are exchanged through ``comm``'s buffer at
    ``offset_bytes``.  ``out`` is complete on every rank."""
    _need(d, x, scratch, out)
    desc = f.desc()
    d.check(d._L.fq_moe_ffn_ep(d.handle, comm.handle, offset_bytes, C.byref(desc), expert_first, _ptr(x), m, _ptr(scratch),
                               scratch.numel(), _ptr(out)))


def project_host(d: Device, w: Matrix, x_host: np.ndarray, m: int, y_host: np.ndarray) -> None:
    """Host-buffer projection: upload x, project, download y, wait."""
    assert x_host.dtype == np.float32 and y_host.dtype == np.float32
    assert x_host.flags["C_CONTIGUOUS"] and y_host.flags["C_CONTIGUOUS"]
    if x_host.size != m * w.cols or y_host.size != m * w.rows:
        raise ShapeError("host projection geometry")
    d.check(d._L.fq_project_host(d.handle, w.handle, C.c_void_p(x_host.ctypes.data), m, C.c_void_p(y_host.ctypes.data)))


def project_many_host(d: Device, ws: Sequence[Matrix], x_host: np.ndarray, m: int, ys: Sequence[np.ndarray]) -> None:
    n = len(ws)
    wa = (C.c_void_p * n)(*[w.handle.value for w in ws])
    ya = (C.c_void_p * n)(*[y.ctypes.data for y in ys])
    for w, y in zip(ws, ys):
        if y.size != m * w.rows or y.dtype != np.float32:
            raise ShapeError("host projection geometry")
    d.check(d._L.fq_project_many_host(d.handle, wa, n, C.c_void_p(x_host.ctypes.data), m, ya))
