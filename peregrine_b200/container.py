"""Checkpoint container -> quantised weight, the load path in front of the GPU residency calls.

Mirrors the reference's host-side types for this step:

* ``SafeTensors``  — reader for ``*.safetensors`` files of a model directory (8-byte little-endian
  header length, JSON header with dtype / shape / data_offsets per tensor, raw payload).
* ``QtInfo.detect`` / ``detect_group_size`` — the container format of a weight ``[O, I]`` is inferred
  from byte counts, not declared (crates/peregrine-core/src/qt.rs:64-166): a U8 payload ``name`` plus
  an F32 sibling ``name.qs``; per-row int8, packed int4, packed int2, or grouped int4 whose group size
  is probed from the number of scales.
* ``QtWeight.load`` / ``raw`` / ``dequant`` — crates/peregrine-model/src/weight.rs:91-145.

Formats outside the expert-FFN int4 path (int3-g64, affine int2-g64) are detected as the reference
detects them but are not loadable here.
"""
from __future__ import annotations

import enum
import json
import os
import struct
from dataclasses import dataclass

import numpy as np


class ContainerError(ValueError):
    """A weight that cannot be loaded; the message follows the reference's ``Error::Format`` texts."""


_DTYPES = {"U8": np.uint8, "I8": np.int8, "F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


class SafeTensors:
    """All tensors of the ``*.safetensors`` files in a directory (or of one file), memory-mapped."""

    def __init__(self, path: str):
        files = [path] if os.path.isfile(path) else sorted(
            os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
        if not files:
            raise ContainerError(f"no .safetensors file under '{path}'")
        self._index = {}
        self._maps = []
        for f in files:
            with open(f, "rb") as fh:
                (hlen,) = struct.unpack("<Q", fh.read(8))
                header = json.loads(fh.read(hlen))
            mm = np.memmap(f, dtype=np.uint8, mode="r", offset=8 + hlen)
            self._maps.append(mm)
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                lo, hi = meta["data_offsets"]
                self._index[name] = (len(self._maps) - 1, meta["dtype"], tuple(meta["shape"]), lo, hi)

    def has(self, name: str) -> bool:
        return name in self._index

    def names(self):
        return list(self._index)

    def nbytes(self, name: str):
        e = self._index.get(name)
        return None if e is None else e[4] - e[3]

    def numel(self, name: str):
        e = self._index.get(name)
        return None if e is None else int(np.prod(e[2], dtype=np.int64)) if e[2] else 1

    def read_raw(self, name: str) -> np.ndarray:
        m, _, _, lo, hi = self._index[name]
        return np.array(self._maps[m][lo:hi], dtype=np.uint8)

    def read_f32(self, name: str) -> np.ndarray:
        m, dtype, _, lo, hi = self._index[name]
        raw = np.array(self._maps[m][lo:hi], dtype=np.uint8)
        if dtype not in ("F32", "F16"):
            raise ContainerError(f"tensor '{name}' is {dtype}, not a float tensor")
        return raw.view(_DTYPES[dtype]).astype(np.float32)


def write_safetensors(path: str, tensors: dict) -> None:
    """Writes ``{name: ndarray}`` as one safetensors file (uint8 arrays as U8, float32 as F32)."""
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        dt = {np.dtype(np.uint8): "U8", np.dtype(np.float32): "F32", np.dtype(np.int8): "I8",
              np.dtype(np.int32): "I32"}[arr.dtype]
        b = arr.tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(h)))
        fh.write(h)
        for b in blobs:
            fh.write(b)


class QtFmt(enum.IntEnum):
    """crates/peregrine-core/src/qt.rs:13-48 (discriminants as in the container's C ``fmt`` field)."""
    F32 = 0
    Int8 = 1
    Int4 = 2
    Int2 = 3
    Int4Grouped = 4
    Int3G64 = 5
    Unknown = 6
    Int2G64 = 7


def detect_group_size(o: int, i: int, ns: int) -> int:
    """Group size of a grouped-int4 weight from its scale count: candidates finest first, the first
    whose ``O * ceil(I / gs)`` equals ``ns``; 0 = per-row (crates/peregrine-core/src/qt.rs:64-85)."""
    if o <= 0 or ns <= o or i <= 0:
        return 0
    for gs in (16, 32, 48, 64, 96, 128, 192, 256):
        if gs > i:
            break
        if ns == o * ((i + gs - 1) // gs):
            return gs
    return 0


@dataclass(frozen=True)
class QtInfo:
    fmt: QtFmt
    o: int
    i: int
    gs: int
    scale_count: int

    @staticmethod
    def detect(st: SafeTensors, name: str, o: int, i: int) -> "QtInfo":
        """crates/peregrine-core/src/qt.rs:87-166, same precedence of the size tests."""
        nb = st.nbytes(name)
        if nb is None or not st.has(name + ".qs"):
            return QtInfo(QtFmt.F32, o, i, 0, 0)
        ns = st.numel(name + ".qs") or 0
        g64 = (i + 63) // 64
        if g64 >= 2 and nb == o * g64 * 16 and ns == o * g64 * 2:
            fmt = QtFmt.Int2G64
        elif nb == o * i:
            fmt = QtFmt.Int8
        elif nb == o * ((i + 1) // 2):
            fmt = QtFmt.Int4
        elif nb == o * ((i + 3) // 4):
            fmt = QtFmt.Int2
        elif nb == o * g64 * 24 and ns == o * g64:
            fmt = QtFmt.Int3G64
        else:
            return QtInfo(QtFmt.Unknown, o, i, 0, 0)
        gs = 0
        if fmt == QtFmt.Int4:
            gs = detect_group_size(o, i, ns)
            if gs > 0:
                fmt = QtFmt.Int4Grouped
        if fmt == QtFmt.Int4Grouped:
            count = o * ((i + gs - 1) // gs)
        elif fmt == QtFmt.Int3G64:
            count = o * g64
        elif fmt == QtFmt.Int2G64:
            count = o * g64 * 2
        else:
            count = o
        if fmt in (QtFmt.Int3G64, QtFmt.Int2G64):
            gs = 64
        return QtInfo(fmt, o, i, gs, count)


@dataclass
class QtWeight:
    """One quantised matrix ``[O, I]``: packed bytes + scales (crates/peregrine-model/src/weight.rs:55-75)."""
    fmt: QtFmt
    o: int
    i: int
    q: np.ndarray       # uint8
    scale: np.ndarray   # float32: O per-row, or O * ceil(I / gs) at scale[o * ng + g]
    gs: int = 0

    @staticmethod
    def load(st: SafeTensors, name: str, o: int, i: int) -> "QtWeight":
        info = QtInfo.detect(st, name, o, i)
        if info.fmt == QtFmt.Unknown:
            raise ContainerError(f"weight '{name}': {st.nbytes(name) or 0} bytes match no quantized container for "
                                 f"[{o},{i}] (truncated tensor, or the shape disagrees with the checkpoint)")
        if info.fmt == QtFmt.F32:
            raise ContainerError(f"weight '{name}': no `.qs` scale sibling (runtime-f32 weights are not supported on "
                                 "the quantized expert path)")
        if info.fmt in (QtFmt.Int3G64, QtFmt.Int2G64):
            raise ContainerError(f"weight '{name}': {info.fmt.name} is outside the int4 expert path of this backend")
        q = st.read_raw(name)
        scale = st.read_f32(name + ".qs")
        if scale.size != info.scale_count:
            raise ContainerError(f"weight '{name}': {scale.size} scales, expected {info.scale_count}")
        return QtWeight(info.fmt, o, i, q, np.ascontiguousarray(scale, np.float32), info.gs)

    def raw(self):
        """``(packed bytes, scales)`` as handed to the uploader (weight.rs:126-131)."""
        return self.q, self.scale

    def dequant(self) -> np.ndarray:
        """fp32 ``[O, I]`` = integer value x its scale, the matrix the reference uploads for experts
        it cannot keep packed (weight.rs ``dequant``)."""
        o, i = self.o, self.i
        if self.fmt == QtFmt.Int8:
            v = self.q.view(np.int8).reshape(o, i).astype(np.float32)
            return v * self.scale[:, None]
        if self.fmt in (QtFmt.Int4, QtFmt.Int4Grouped):
            rb = (i + 1) // 2
            b = self.q.reshape(o, rb)
            v = np.empty((o, rb * 2), np.float32)
            v[:, 0::2] = (b & 15).astype(np.float32) - 8.0
            v[:, 1::2] = (b >> 4).astype(np.float32) - 8.0
            v = v[:, :i]
            if self.fmt == QtFmt.Int4:
                return v * self.scale[:, None]
            ng = (i + self.gs - 1) // self.gs
            sc = np.repeat(self.scale.reshape(o, ng), self.gs, axis=1)[:, :i]
            return v * sc
        if self.fmt == QtFmt.Int2:
            rb = (i + 3) // 4
            b = self.q.reshape(o, rb)
            v = np.empty((o, rb * 4), np.float32)
            for j in range(4):
                v[:, j::4] = ((b >> (2 * j)) & 3).astype(np.float32) - 2.0
            return v[:, :i] * self.scale[:, None]
        raise ContainerError(f"no dequantisation for {self.fmt.name}")


def expert_names(layer: int, e: int):
    """Tensor names of one routed expert in the checkpoint (crates/peregrine-model/src/gpu.rs:1370-1374)."""
    p = f"model.layers.{layer}.mlp.experts.{e}."
    return p + "gate_proj.weight", p + "up_proj.weight", p + "down_proj.weight"


def shared_names(layer: int):
    p = f"model.layers.{layer}.mlp.shared_experts."
    return p + "gate_proj.weight", p + "up_proj.weight", p + "down_proj.weight"
