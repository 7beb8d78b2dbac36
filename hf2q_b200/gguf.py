"""GGUF v3 container: a writer with the layout hf2q's ``GgufWriter`` emits
(src/backends/gguf/writer.rs:142-361, types.rs:17-118) and the reader side the inference path
needs -- tensor table + RAW block bytes handed to the device unchanged, the contract of
``GgufFile::load_tensor`` as hf2q uses it (src/inference/models/qwen35/weight_loader.rs:147-159,
src/serve/forward_mlx.rs:9356-9386).

Layout: "GGUF" | version u32 = 3 | tensor_count u64 | kv_count u64 | kv pairs | tensor infos
(name, n_dims u32, dims u64[] innermost first, ggml_type u32, offset u64 relative to the data
region) | pad to 32 | tensor payloads, each padded to 32 bytes.  Everything little-endian.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

GGUF_MAGIC = b"GGUF"
GGUF_VERSION = 3
ALIGNMENT = 32

# metadata value types (types.rs:33-45)
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
               T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}

# bytes per block / elements per block for the tensor types this path handles (ggml_type.rs:60-127)
BLOCK = {0: (1, 4), 1: (1, 2), 2: (32, 18), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210), 30: (1, 2)}


def _pad(n: int) -> int:
    return (-n) % ALIGNMENT


def tensor_nbytes(ggml_type: int, dims_inner_first) -> int:
    elems, size = BLOCK[ggml_type]
    n = 1
    for d in dims_inner_first:
        n *= int(d)
    if dims_inner_first[0] % elems:
        raise ValueError(f"innermost dim {dims_inner_first[0]} is not a multiple of the {elems}-element block")
    return n // elems * size


def _gguf_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _encode_value(vtype: int, value) -> bytes:
    if vtype == T_STRING:
        return _gguf_string(value)
    if vtype == T_ARRAY:
        etype, items = value
        out = struct.pack("<IQ", etype, len(items))
        for it in items:
            out += _encode_value(etype, it)
        return out
    return struct.pack(_SCALAR_FMT[vtype], value)


class GgufWriter:
    """Collects metadata and tensors, then writes the file in one pass (offsets are known up front,
    so no seek-back is needed; the bytes on disk are the same as the reference writer's)."""

    def __init__(self):
        self._kv: list[tuple[str, int, object]] = []
        self._tensors: list[tuple[str, tuple[int, ...], int, bytes]] = []

    def add_kv(self, key: str, vtype: int, value) -> None:
        self._kv.append((key, vtype, value))

    def add_tensor(self, name: str, shape_outer_first, ggml_type: int, payload) -> None:
        """shape is given outer-first ([rows, cols] / [experts, rows, cols]); GGUF stores it inner-first."""
        dims = tuple(int(d) for d in reversed(tuple(shape_outer_first)))
        data = bytes(memoryview(np.ascontiguousarray(payload)).cast("B"))
        want = tensor_nbytes(ggml_type, dims)
        if len(data) != want:
            raise ValueError(f"{name}: payload is {len(data)} bytes, type {ggml_type} with dims {dims} needs {want}")
        self._tensors.append((name, dims, ggml_type, data))

    def write(self, path) -> None:
        head = GGUF_MAGIC + struct.pack("<IQQ", GGUF_VERSION, len(self._tensors), len(self._kv))
        for key, vtype, value in self._kv:
            head += _gguf_string(key) + struct.pack("<I", vtype) + _encode_value(vtype, value)
        off = 0
        for name, dims, t, data in self._tensors:
            head += _gguf_string(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
            head += struct.pack("<IQ", t, off)
            off += len(data) + _pad(len(data))
        with open(path, "wb") as f:
            f.write(head)
            f.write(b"\0" * _pad(len(head)))
            for _, _, _, data in self._tensors:
                f.write(data)
                f.write(b"\0" * _pad(len(data)))


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple[int, ...]      # outer-first, as the reference's reader reports it (rows = shape[0])
    ggml_type: int
    offset: int                 # absolute file offset of the payload
    nbytes: int


class GgufFile:
    """Memory-mapped reader: metadata, tensor table, raw payload views."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata: dict[str, object] = {}
        self.tensors: dict[str, TensorInfo] = {}
        self._parse()

    def close(self) -> None:
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- parsing ---------------------------------------------------------------------------------
    def _u(self, fmt: str, pos: int):
        size = struct.calcsize(fmt)
        if pos + size > len(self._mm):
            raise ValueError("truncated GGUF file")
        return struct.unpack_from(fmt, self._mm, pos), pos + size

    def _string(self, pos: int):
        (n,), pos = self._u("<Q", pos)
        if pos + n > len(self._mm):
            raise ValueError("truncated GGUF string")
        return self._mm[pos:pos + n].decode("utf-8"), pos + n

    def _value(self, vtype: int, pos: int):
        if vtype == T_STRING:
            return self._string(pos)
        if vtype == T_ARRAY:
            (etype, count), pos = self._u("<IQ", pos)
            items = []
            for _ in range(count):
                v, pos = self._value(etype, pos)
                items.append(v)
            return items, pos
        if vtype not in _SCALAR_FMT:
            raise ValueError(f"unknown GGUF metadata type {vtype}")
        (v,), pos = self._u(_SCALAR_FMT[vtype], pos)
        return v, pos

    def _parse(self) -> None:
        if self._mm[:4] != GGUF_MAGIC:
            raise ValueError("not a GGUF file (bad magic)")
        (version, n_tensors, n_kv), pos = self._u("<IQQ", 4)
        if version != GGUF_VERSION:
            raise ValueError(f"unsupported GGUF version {version}")
        for _ in range(n_kv):
            key, pos = self._string(pos)
            (vtype,), pos = self._u("<I", pos)
            self.metadata[key], pos = self._value(vtype, pos)
        raw = []
        for _ in range(n_tensors):
            name, pos = self._string(pos)
            (nd,), pos = self._u("<I", pos)
            dims, pos = self._u(f"<{nd}Q", pos)
            (t, off), pos = self._u("<IQ", pos)
            raw.append((name, dims, t, off))
        align = int(self.metadata.get("general.alignment", ALIGNMENT))
        data_start = pos + ((-pos) % align)
        for name, dims, t, off in raw:
            if t not in BLOCK:
                raise ValueError(f"{name}: ggml type {t} is not handled by this reader")
            nbytes = tensor_nbytes(t, dims)
            if data_start + off + nbytes > len(self._mm):
                raise ValueError(f"{name}: payload runs past the end of the file")
            self.tensors[name] = TensorInfo(name, tuple(reversed(dims)), t, data_start + off, nbytes)

    # -- access ----------------------------------------------------------------------------------
    def tensor_info(self, name: str) -> TensorInfo:
        return self.tensors[name]

    def load_tensor(self, name: str) -> np.ndarray:
        """The tensor's payload exactly as stored: a read-only uint8 view into the mapping."""
        ti = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=ti.nbytes, offset=ti.offset)

    def load_quant_weight(self, ctx, name: str):
        """load_gguf_qweight (forward_mlx.rs:9356-9386): raw blocks -> device, bytes unchanged;
        rows = shape[0], cols = shape[1] (stacked experts: rows = experts * shape[1], cols = shape[2])."""
        from . import ops
        ti = self.tensors[name]
        if len(ti.shape) == 2:
            rows, cols = ti.shape
        elif len(ti.shape) == 3:
            rows, cols = ti.shape[0] * ti.shape[1], ti.shape[2]
        else:
            raise ValueError(f"{name}: expected a 2-D or stacked 3-D tensor, got shape {ti.shape}")
        return ops.load_quant_weight(ctx, self.load_tensor(name), ti.ggml_type, rows, cols)
