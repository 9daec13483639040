"""Weight files for the quantized linear: a GGUF tensor reader (F32 / F16 / Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q8_0 / Q2_K .. Q6_K) and NPZ.

GGUF is the container llama.cpp-family tools write; its Q4_0 / Q8_0 tensors are exactly the block
streams this library consumes (18 / 34 bytes per 32 values, f16 scale first), with the Q4_0 nibbles
in the "split" element order (low nibbles = values 0..15, high nibbles = values 16..31), the order
the reference's CUDA and Metal kernels read (quantized.cu:862-866) -- so a tensor is uploaded as it
is, with `ORDER_GGML_SPLIT`; nothing is repacked.  NPZ / NPY is the checkpoint format candy itself
reads and writes for f32 tensors (tensor/npy.go:310-583); NumPy reads it, and
`quantize_linear` turns such a matrix into blocks on the device.

The reader is a from-scratch parser of the published GGUF layout (versions 2 and 3, little
endian): header (magic "GGUF", version, tensor count, metadata count), typed metadata key/values,
tensor infos (name, dims innermost first, ggml type, offset), then the data section aligned to
`general.alignment` (default 32).  Only the tensor types named above are decoded; others are
listed with their raw bytes.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Tuple

import numpy as np

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0 = 0, 1, 2, 3, 6, 7, 8
GGML_Q2_K, GGML_Q3_K, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 10, 11, 12, 13, 14
_BLOCK = {GGML_Q4_0: (32, 18), GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24), GGML_Q8_0: (32, 34),
          GGML_Q2_K: (256, 84), GGML_Q3_K: (256, 110), GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_Q6_K: (256, 210)}  # values, bytes per block
_ELEM = {GGML_F32: 4, GGML_F16: 2}

# metadata value types of the GGUF specification
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GGUFError(ValueError):
    pass


@dataclass
class GGUFTensor:
    name: str
    shape: Tuple[int, ...]      # outermost first (NumPy order): a linear's weight is (n, k)
    ggml_type: int
    data: np.ndarray            # uint8 view of the tensor's bytes inside the (memory-mapped) file

    @property
    def is_quantized(self) -> bool:
        return self.ggml_type in _BLOCK

    def to_float32(self) -> np.ndarray:
        """F32 / F16 tensors as float32 arrays of `shape`."""
        if self.ggml_type == GGML_F32:
            return self.data.view("<f4").reshape(self.shape)
        if self.ggml_type == GGML_F16:
            return self.data.view("<f2").astype(np.float32).reshape(self.shape)
        raise GGUFError(f"{self.name}: type {self.ggml_type} is a block format; upload it with load_linear")


class _Reader:
    def __init__(self, buf: np.ndarray):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > self.buf.size:
            raise GGUFError("truncated file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > self.buf.size:
            raise GGUFError("truncated string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            etype, count = self.take("<I"), self.take("<Q")
            if etype in _SCALARS:  # bulk-skip numeric arrays (token tables can hold 10^5 entries)
                fmt = _SCALARS[etype]
                size = struct.calcsize(fmt)
                if self.pos + size * count > self.buf.size:
                    raise GGUFError("truncated array")
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt[1:]).newbyteorder("<"), count=count, offset=self.pos)
                self.pos += size * count
                return arr
            return [self.value(etype) for _ in range(count)]
        raise GGUFError(f"unknown metadata type {vtype}")


def read_gguf(path) -> Tuple[Dict[str, object], Dict[str, GGUFTensor]]:
    """Parses a GGUF file; returns (metadata, tensors by name).  Tensor bytes are views of a memory map."""
    buf = np.memmap(Path(path), dtype=np.uint8, mode="r")
    r = _Reader(buf)
    if buf.size < 24 or bytes(buf[:4]) != b"GGUF":
        raise GGUFError("not a GGUF file")
    r.pos = 4
    version = r.take("<I")
    if version not in (2, 3):
        raise GGUFError(f"unsupported GGUF version {version}")
    n_tensors, n_kv = r.take("<Q"), r.take("<Q")
    meta: Dict[str, object] = {}
    for _ in range(n_kv):
        key = r.string()
        meta[key] = r.value(r.take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = r.string()
        nd = r.take("<I")
        if nd < 1 or nd > 4:
            raise GGUFError(f"{name}: {nd} dimensions")
        dims = [r.take("<Q") for _ in range(nd)]  # innermost first
        infos.append((name, dims, r.take("<I"), r.take("<Q")))
    align = int(meta.get("general.alignment", 32))
    base = (r.pos + align - 1) // align * align
    tensors: Dict[str, GGUFTensor] = {}
    for name, dims, gtype, off in infos:
        count = int(np.prod(dims, dtype=np.int64))
        if gtype in _BLOCK:
            per, bb = _BLOCK[gtype]
            if dims[0] % per:
                raise GGUFError(f"{name}: innermost dimension {dims[0]} is not a multiple of {per}")
            nbytes = count // per * bb
        elif gtype in _ELEM:
            nbytes = count * _ELEM[gtype]
        else:
            nbytes = None  # a type this reader does not decode: keep what is known
        start = base + off
        if nbytes is None:
            data = buf[start:start]
        else:
            if start + nbytes > buf.size:
                raise GGUFError(f"{name}: data past the end of the file")
            data = buf[start:start + nbytes]
        tensors[name] = GGUFTensor(name, tuple(int(d) for d in reversed(dims)), int(gtype), data)
    return meta, tensors


def load_linear(dev, t: GGUFTensor):
    """A 2-D block-format tensor [n, k] (Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q8_0 / Q2_K .. Q6_K) as a device QStorage in the GGML order, bytes unchanged."""
    from .backend import QStorage, ORDER_GGML_SPLIT
    if len(t.shape) != 2 or not t.is_quantized:
        raise GGUFError(f"{t.name}: expected a 2-D block-quantized tensor, got type {t.ggml_type} shape {t.shape}")
    n, k = t.shape
    qtype = t.ggml_type  # the library's qtype ids are the GGML ids
    return QStorage.from_blocks(dev, qtype, ORDER_GGML_SPLIT, n, k, np.ascontiguousarray(t.data))


def load_npz(path) -> Dict[str, np.ndarray]:
    """The f32 tensors of an NPZ / NPY checkpoint (candy's own format), by name."""
    path = Path(path)
    if path.suffix == ".npy":
        return {path.stem: np.asarray(np.load(path), dtype=np.float32)}
    with np.load(path) as z:
        return {k: np.asarray(z[k], dtype=np.float32) for k in z.files}


def quantize_linear(dev, w: np.ndarray, qtype: int, order: int = 0):
    """An f32 [n, k] matrix (e.g. from an NPZ checkpoint) quantized on the device into a QStorage."""
    from .backend import QStorage
    return QStorage.quantize(dev, qtype, order, np.ascontiguousarray(w, dtype=np.float32))
