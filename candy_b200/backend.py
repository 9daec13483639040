"""Host-side mirror of candy's device / storage interface for the quantized linear.

The reference's plug-in boundary is ``candy.BackendDevice[T]`` (device.go:49-82) and
``candy.BackendStorage[T]`` (backend.go:4-238).  This module carries the slice of those
interfaces the quantized linear needs -- ``StorageFromSlice``, ``Alloc``/``Zeros``,
``Synchronize``, ``Data``, ``Clone``, ``MatMul`` -- under the same names (snake-cased) over
the C ABI, plus the two things the reference lacks: a storage type for block-quantized
weights (``QStorage``) and ``QLinear``, the quantized twin of ``nn.Linear`` (nn/linear.go:
58-112).  Error messages follow the reference's ``"<op>: <reason>"`` wrapping style.
Everything computes on the GPU through ``libcandyq``; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import abi
from .abi import (ACT_F16, ACT_F32, ACT_Q8_1, ORDER_GGML_SPLIT, ORDER_GO_INTERLEAVED, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, CandyqError)

__all__ = ["CudaDevice", "CudaStorage", "QStorage", "QLinear", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "ORDER_GO_INTERLEAVED",
           "ORDER_GGML_SPLIT", "ACT_F32", "ACT_Q8_1", "ACT_F16", "CandyqError"]


class CudaDevice:
    """candy.BackendDevice for one GPU (device.go:49-82): owns a libcandyq context."""

    def __init__(self, ordinal: int = 0):
        self._lib = abi.lib()
        ctx = C.c_void_p()
        st = self._lib.cq_ctx_create(ordinal, C.byref(ctx))
        if st != abi.OK:
            raise CandyqError(st, f"cuda device {ordinal}: failed to create context")
        self._ctx = ctx
        self.ordinal = ordinal

    # -- BackendDevice ---------------------------------------------------------------
    def location(self) -> str:  # device.go:51 (GpuLocation)
        return "gpu"

    def is_same(self, other: "CudaDevice") -> bool:  # device.go:54
        return isinstance(other, CudaDevice) and other.ordinal == self.ordinal

    def storage_from_slice(self, data) -> "CudaStorage":  # device.go:57
        a = np.ascontiguousarray(data, dtype=np.float32)
        st = self.alloc(a.size)
        self._check(self._lib.cq_memcpy_h2d(self._ctx, st.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes), "storage from slice")
        return st

    def alloc(self, numel: int) -> "CudaStorage":  # device.go:69
        return CudaStorage(self, self.malloc(4 * int(numel)), int(numel))

    def zeros(self, numel: int) -> "CudaStorage":  # device.go:72
        st = self.alloc(numel)
        self._check(self._lib.cq_memset(self._ctx, st.ptr, 0, 4 * int(numel)), "zeros")
        return st

    def synchronize(self) -> None:  # device.go:80-81
        self._check(self._lib.cq_synchronize(self._ctx), "synchronize")

    # -- raw helpers -----------------------------------------------------------------
    def malloc(self, nbytes: int) -> C.c_void_p:
        p = C.c_void_p()
        self._check(self._lib.cq_malloc(self._ctx, nbytes, C.byref(p)), "alloc")
        return p

    def free(self, ptr) -> None:
        if self._ctx:
            self._lib.cq_free(self._ctx, ptr)

    def set_stream(self, cuda_stream: int) -> None:
        self._check(self._lib.cq_ctx_set_stream(self._ctx, C.c_void_p(cuda_stream)), "set stream")

    def set_option(self, key: str, value: int) -> None:
        self._check(self._lib.cq_ctx_set_option(self._ctx, key.encode(), int(value)), "set option")

    def upload_bytes(self, data: np.ndarray) -> "RawBuffer":
        a = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        buf = RawBuffer(self, a.nbytes)
        self._check(self._lib.cq_memcpy_h2d(self._ctx, buf.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes), "upload")
        return buf

    def _check(self, status: int, where: str) -> None:
        abi.check(self._ctx, status, where)

    @property
    def ctx(self):
        return self._ctx

    def close(self) -> None:
        if self._ctx:
            self._lib.cq_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RawBuffer:
    """Untyped device bytes (quantized blocks, Q8_1 activations)."""

    def __init__(self, device: CudaDevice, nbytes: int):
        self.device_ = device
        self.nbytes = int(nbytes)
        self.ptr = device.malloc(max(self.nbytes, 1))

    def data(self) -> np.ndarray:
        out = np.empty(self.nbytes, dtype=np.uint8)
        d = self.device_
        d._check(d._lib.cq_memcpy_d2h(d.ctx, out.ctypes.data_as(C.c_void_p), self.ptr, self.nbytes), "data")
        return out

    def __del__(self):
        try:
            self.device_.free(self.ptr)
        except Exception:
            pass


class CudaStorage:
    """candy.BackendStorage[float32] on the GPU (backend.go:4-238), the part the path uses."""

    def __init__(self, device: CudaDevice, ptr, numel: int):
        self._dev = device
        self.ptr = ptr
        self.numel = numel

    def device(self) -> CudaDevice:  # backend.go:12
        return self._dev

    def dtype(self) -> str:  # backend.go:15
        return "f32"

    def data(self) -> np.ndarray:  # backend.go:9 -- a host copy
        out = np.empty(self.numel, dtype=np.float32)
        d = self._dev
        d._check(d._lib.cq_memcpy_d2h(d.ctx, out.ctypes.data_as(C.c_void_p), self.ptr, out.nbytes), "data")
        return out

    def clone(self) -> "CudaStorage":  # backend.go:6
        d = self._dev
        out = d.alloc(self.numel)
        d._check(d._lib.cq_memcpy_d2d(d.ctx, out.ptr, self.ptr, 4 * self.numel), "clone")
        return out

    def matmul(self, rhs: "QStorage", b: int, m: int, n: int, k: int, actmode: int = ACT_F32) -> "CudaStorage":
        """BackendStorage.MatMul (backend.go:77-78) with a block-quantized right-hand side
        viewed as W^T [k, n], the case nn.Linear.Forward produces (nn/linear.go:65-84).
        Returns a newly allocated [b*m, n] storage, like CpuStorage.MatMul (tensor/internal/
        cpu/storage.go:881)."""
        if not isinstance(rhs, QStorage):
            raise TypeError("matmul: right-hand side must be a QStorage")
        if b < 1 or m < 1:
            raise ValueError(f"matmul: bad batch/rows {b}x{m}")
        if k != rhs.k or n != rhs.n:
            raise ValueError(f"matmul: inner dims mismatch: {k} vs {rhs.k}" if k != rhs.k else f"matmul: n mismatch: {n} vs {rhs.n}")
        if self.numel < b * m * k:
            raise ValueError("matmul: lhs storage smaller than b*m*k")
        d = self._dev
        rows = b * m
        out = d.alloc(rows * n)
        d._check(d._lib.cq_qmatmul(d.ctx, rhs.qtype, rhs.order, actmode, self.ptr, rows, k, k, rhs.buf.ptr, n, out.ptr, n),
                 "matmul")
        return out

    def __del__(self):
        try:
            self._dev.free(self.ptr)
        except Exception:
            pass


class QStorage:
    """Block-quantized weight W[n, k] resident on the GPU: n*k/32 blocks, row-major.

    The reference has only the block structs and per-block dequantizers for these formats
    (tensor/internal/cpu/kernels/quantized.go:8-11, :34-37, :85-93, :131-136); this is the
    storage type that carries them behind the device API."""

    def __init__(self, device: CudaDevice, qtype: int, order: int, n: int, k: int, buf: RawBuffer):
        if qtype not in abi.BLOCK_BYTES and qtype not in abi.K_BLOCK_BYTES:
            raise ValueError(f"qstorage: unknown block format {qtype}")
        per = 256 if qtype in abi.K_BLOCK_BYTES else 32  # values per block
        if k <= 0 or k % per != 0:
            raise ValueError(f"qstorage: k must be a positive multiple of {per}, got {k}")
        if buf.nbytes != n * (k // per) * (abi.K_BLOCK_BYTES.get(qtype) or abi.BLOCK_BYTES[qtype]):
            raise ValueError("qstorage: byte count does not match the block count")
        self._dev, self.qtype, self.order, self.n, self.k, self.buf = device, qtype, order, n, k, buf

    @classmethod
    def from_blocks(cls, device: CudaDevice, qtype: int, order: int, n: int, k: int, blocks: np.ndarray) -> "QStorage":
        return cls(device, qtype, order, n, k, device.upload_bytes(blocks))

    @classmethod
    def quantize(cls, device: CudaDevice, qtype: int, order: int, w: np.ndarray) -> "QStorage":
        """f32 W[n,k] on the host -> blocks, quantized on the GPU with the arithmetic of the
        reference's weight quantizers (tensor/internal/metal/kernels/quantized.metal:4149-4214,
        :4091-4147)."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        if k % 32 != 0:
            raise ValueError(f"qstorage: k must be a positive multiple of 32, got {k}")
        src = device.storage_from_slice(w)
        buf = RawBuffer(device, n * (k // 32) * abi.BLOCK_BYTES[qtype])
        device._check(device._lib.cq_quantize_rows(device.ctx, qtype, order, src.ptr, n, k, buf.ptr), "quantize")
        return cls(device, qtype, order, n, k, buf)

    def device(self) -> CudaDevice:
        return self._dev

    def data(self) -> np.ndarray:
        return self.buf.data()

    def dequantize(self) -> CudaStorage:
        d = self._dev
        out = d.alloc(self.n * self.k)
        per = 256 if self.qtype in abi.K_BLOCK_BYTES else 32
        d._check(d._lib.cq_dequantize(d.ctx, self.qtype, self.order, self.buf.ptr, self.n * (self.k // per), out.ptr), "dequantize")
        return out


class QLinear:
    """y = x W^T (+ b) with block-quantized W [out, in]: nn.Linear.Forward (nn/linear.go:58-112)
    for a contiguous input, which is flattened to [prod(batch dims), in] and multiplied in
    one call (nn/linear.go:72-92)."""

    def __init__(self, w: QStorage, b: Optional[np.ndarray] = None, actmode: int = ACT_F32):
        self.w, self.actmode = w, actmode
        self.b = None if b is None else np.ascontiguousarray(b, dtype=np.float32)
        if self.b is not None and self.b.shape != (w.n,):
            raise ValueError("linear: bias shape must be [out]")
        self._b_dev = None if self.b is None else w.device().storage_from_slice(self.b)  # the bias lives on the device

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, dtype=np.float32)
        if x.ndim < 2:
            raise ValueError(f"linear: input rank must be >= 2, got {x.ndim}")
        if x.shape[-1] != self.w.k:
            raise ValueError(f"linear: failed to matmul: matmul forward: inner dims mismatch: {x.shape[-1]} vs {self.w.k}")
        bs: Sequence[int] = x.shape[:-1]
        rows = int(np.prod(bs))
        dev = self.w.device()
        xs = dev.storage_from_slice(np.ascontiguousarray(x).reshape(rows, self.w.k))
        if self._b_dev is None:
            ys = xs.matmul(self.w, 1, rows, self.w.n, self.w.k, self.actmode)
        else:  # BroadcastAdd (nn/linear.go:105-110) on the device, in the matmul's epilogue where its kernel has one
            ys = dev.alloc(rows * self.w.n)
            dev._check(dev._lib.cq_qlinear(dev.ctx, self.w.qtype, self.w.order, self.actmode, xs.ptr, rows, self.w.k, self.w.k,
                                           self.w.buf.ptr, self.w.n, self._b_dev.ptr, ys.ptr, self.w.n), "linear")
        return ys.data().reshape(*bs, self.w.n)
