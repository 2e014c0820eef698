"""Reader for GGUF container files: the load-side counterpart of the packed-block entry points.

The reference loads weights from safetensors through a memory map and hands out zero-copy views
(``getMmapView``, workspace/safetensors/src/safetensors.nim:256-274; header parsing :192-254); it has no GGUF
reader.  This module does the same job for the container the block formats of this library ship in: it maps the
file, parses the header, the metadata key/value table and the tensor table of the public GGUF layout (versions
2 and 3, little endian), and returns each quantized tensor as a zero-copy ``uint8`` view ``[rows, bytes_per_row]``
of canonical blocks -- exactly what ``QuantLinear`` / ``ttq_weight_create`` take.  Pure Python + numpy: no GPU is
needed to open a file and nothing here computes on weights.

Layout (all integers little endian):
  magic "GGUF" | version u32 | tensor_count u64 | kv_count u64
  kv_count x ( key: string | value_type u32 | value )        string = length u64 + bytes (UTF-8)
  tensor_count x ( name: string | n_dims u32 | dims u64 x n_dims | ggml_type u32 | offset u64 )
  padding to ``general.alignment`` (default 32) | tensor data, each tensor at data_start + offset
``dims[0]`` is the innermost (contiguous) dimension: a linear weight [out, in] is stored with dims = (in, out).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np
import torch

from ._lib import FMT_Q4_K, FMT_Q6_K, FMT_Q8_0

# ggml tensor types this reader knows the size of: type id -> (name, elements per block, bytes per block)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 8: ("Q8_0", 32, 34), 12: ("Q4_K", 256, 144), 14: ("Q6_K", 256, 210),
    24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8), 30: ("BF16", 1, 2),
}
# ggml type id -> library format of the block-quantized types QuantLinear accepts
TTQ_FORMATS = {8: FMT_Q8_0, 12: FMT_Q4_K, 14: FMT_Q6_K}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GGUFError(ValueError):
    """Malformed or unsupported file (the reference raises ValueError-style exceptions for bad safetensors
    headers the same way, safetensors.nim:180-190,213-216)."""


@dataclass
class TensorInfo:
    name: str
    shape: tuple          # outermost first: (rows, ..., innermost)
    ggml_type: int
    offset: int           # relative to the data section
    nbytes: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0]


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("file ends inside the header")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGUFError("string runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int, depth: int = 0):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            if depth > 4:
                raise GGUFError("arrays nested too deeply")
            itype, count = self.take("<I"), self.take("<Q")
            if itype in _SCALARS:  # bulk path for numeric arrays (token tables run to 10^5 entries)
                fmt = _SCALARS[itype]
                size = struct.calcsize(fmt)
                if self.pos + size * count > len(self.buf):
                    raise GGUFError("array runs past the end of the file")
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=count, offset=self.pos)
                self.pos += size * count
                return arr
            return [self.value(itype, depth + 1) for _ in range(count)]
        raise GGUFError(f"unknown metadata value type {vtype}")


class GGUFFile:
    """A memory-mapped GGUF file.  ``metadata``: dict of the key/value table; ``tensors``: dict name -> TensorInfo.
    Views returned by ``raw`` / ``blocks`` alias the map: keep the object alive while they are in use (the same
    rule as the reference's MemFile views, safetensors.nim:100-108) or upload them first."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        try:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as exc:  # empty file
            self._f.close()
            raise GGUFError(f"{path}: cannot map ({exc})") from exc
        self._view = memoryview(self._map)
        cur = _Cursor(self._view)
        if len(self._view) < 24 or bytes(self._view[:4]) != b"GGUF":
            raise GGUFError(f"{path}: not a GGUF file (bad magic)")
        cur.pos = 4
        self.version = cur.take("<I")
        if self.version not in (2, 3):
            raise GGUFError(f"{path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = cur.take("<Q"), cur.take("<Q")
        if n_tensors > (1 << 24) or n_kv > (1 << 24):
            raise GGUFError(f"{path}: implausible table sizes ({n_tensors} tensors, {n_kv} keys)")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = cur.string()
            self.metadata[key] = cur.value(cur.take("<I"))
        self.alignment = int(self.metadata.get("general.alignment", 32))
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            raise GGUFError(f"{path}: alignment {self.alignment} is not a power of two")
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = cur.string()
            n_dims = cur.take("<I")
            if n_dims > 8:
                raise GGUFError(f"{path}: tensor {name!r} has {n_dims} dimensions")
            dims = [cur.take("<Q") for _ in range(n_dims)]
            gtype, offset = cur.take("<I"), cur.take("<Q")
            if gtype not in GGML_TYPES:
                raise GGUFError(f"{path}: tensor {name!r} has ggml type {gtype}, which this reader cannot size")
            _, per_block, block_bytes = GGML_TYPES[gtype]
            inner = dims[0] if dims else 1
            if inner % per_block:
                raise GGUFError(f"{path}: tensor {name!r}: innermost dimension {inner} is not a multiple of {per_block}")
            count = int(np.prod(dims, dtype=np.int64)) if dims else 1
            if offset % self.alignment:
                raise GGUFError(f"{path}: tensor {name!r}: offset {offset} is not aligned to {self.alignment}")
            self.tensors[name] = TensorInfo(name, tuple(reversed(dims)), gtype, offset, count // per_block * block_bytes)
        self.data_start = (cur.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if self.data_start + t.offset + t.nbytes > len(self._view):
                raise GGUFError(f"{path}: tensor {t.name!r} runs past the end of the file")

    # ---- views -------------------------------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only 1-D uint8 view of the map."""
        t = self._info(name)
        return np.frombuffer(self._view, dtype=np.uint8, count=t.nbytes, offset=self.data_start + t.offset)

    def blocks(self, name: str) -> torch.Tensor:
        """Canonical blocks of a 2-D block-quantized tensor as uint8 ``[out_features, bytes_per_row]`` (zero copy)."""
        t = self._info(name)
        if t.ggml_type not in TTQ_FORMATS:
            raise GGUFError(f"tensor {name!r} is {t.type_name}, not one of the block formats Q8_0 / Q4_K / Q6_K")
        if len(t.shape) != 2:
            raise GGUFError(f"tensor {name!r} has shape {t.shape}; a linear weight is 2-D")
        rows = t.shape[0]
        arr = self.raw(name).reshape(rows, t.nbytes // rows)
        with _quiet_readonly():
            return torch.from_numpy(arr)

    def array(self, name: str) -> np.ndarray:
        """Unquantized tensors (F32 / F16 / BF16-as-uint16 / integers) as a numpy view in their stored shape."""
        t = self._info(name)
        dt = {0: np.float32, 1: np.float16, 24: np.int8, 25: np.int16, 26: np.int32, 27: np.int64, 28: np.float64, 30: np.uint16}.get(t.ggml_type)
        if dt is None:
            raise GGUFError(f"tensor {name!r} is {t.type_name}: use blocks()")
        return self.raw(name).view(dt).reshape(t.shape)

    def linear(self, ctx, name: str, bias: Optional[torch.Tensor] = None, shard=None):
        """``QuantLinear`` over a block-quantized 2-D tensor (uploads and repacks; the map can be closed afterwards)."""
        from .layers import QuantLinear

        t = self._info(name)
        blocks = self.blocks(name)  # raises for anything but a 2-D Q8_0 / Q4_K / Q6_K tensor
        return QuantLinear(ctx, TTQ_FORMATS[t.ggml_type], blocks, t.shape[1], bias=bias, shard=shard)

    # ---- housekeeping --------------------------------------------------------------------------------------
    def _info(self, name: str) -> TensorInfo:
        try:
            return self.tensors[name]
        except KeyError:
            raise GGUFError(f"{self.path}: no tensor named {name!r}") from None

    def close(self) -> None:
        """Unmap.  Fails with BufferError while numpy / torch views of the map are still alive."""
        view, self._view = self._view, None
        if view is not None:
            view.release()
            self._map.close()
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        try:
            self.close()
        except BufferError:
            pass  # views handed out are still referenced; the map goes away with them
        return False


class _quiet_readonly:
    """torch.from_numpy warns that a read-only array is not writable; the views are only ever read."""

    def __enter__(self):
        import warnings

        self._cm = warnings.catch_warnings()
        self._cm.__enter__()
        warnings.simplefilter("ignore")

    def __exit__(self, *exc):
        return self._cm.__exit__(*exc)
