"""Reads grouped-affine (gaf) weights out of a safetensors file and uploads them.

The on-disk contract is the one talu's converter writes
(core/src/converter/grouped_affine.zig:565-593): per quantized matrix three
tensors `<base>.weight` (dtype string `U32`, shape [N, K/vpw]), `<base>.scales`
and `<base>.biases` (`BF16` or `F16`, shape [N, K/G]).  Bits and group size are
not stored per tensor; they are inferred from the shapes the way talu's loader
does it (inferGaffineParams, core/src/models/load/transforms.zig:75-155), with
the model-level `quantization {bits, group_size}` of config.json, when given, as
the expected value.

safetensors layout: 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets: [begin, end]}, "__metadata__": {...}}, then
the tensor bytes.  The file is memory-mapped; the arrays handed to the upload
are views into the map (they may be unaligned: the library copies them as
bytes).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterator, Optional, Tuple

import numpy as np

MAX_SUPPORTED_GAFFINE_GROUPS = 1024  # core/src/models/op_types.zig:333
_VALID_GROUPS = (32, 64, 128)


class GafFormatError(ValueError):
    pass


@dataclass
class GafTensor:
    """One quantized matrix as it sits in the file (views into the memory map)."""
    name: str              # base name, without ".weight"
    packed: np.ndarray     # uint32 [N, K/vpw]
    scales: np.ndarray     # uint16 [N, K/G] (bit patterns)
    biases: np.ndarray     # uint16 [N, K/G]
    bits: int
    group: int
    scales_dtype: int      # 0 = f16, 1 = bf16 (the tags of gaffine_u4_matvec.zig:13-14)

    @property
    def N(self) -> int:
        return int(self.packed.shape[0])

    @property
    def K(self) -> int:
        return int(self.packed.shape[1]) * (32 // self.bits)


def infer_bits_and_group(in_packed: int, n_groups: int, expected_dim: Optional[int] = None,
                         expected_bits: Optional[int] = None) -> Tuple[int, int]:
    """inferGaffineParams' rule (transforms.zig:119-139): a width is plausible when it gives a group size of
    32, 64 or 128; when both are, the expected unpacked dimension (or, here, the configured bit width)
    decides, else 4-bit wins only if it is the only plausible one."""
    if n_groups <= 0:
        raise GafFormatError("no groups")
    g4, g8 = (in_packed * 8) // n_groups, (in_packed * 4) // n_groups
    v4, v8 = g4 in _VALID_GROUPS, g8 in _VALID_GROUPS
    if v4 and v8:
        if expected_dim is not None:
            is4 = in_packed * 8 == expected_dim
        elif expected_bits is not None:
            is4 = expected_bits == 4
        else:
            is4 = False  # the reference compares against the expected dimension; without one it falls to 8-bit
    else:
        is4 = v4
    if not is4 and not v8:
        raise GafFormatError(f"no valid group size for packed width {in_packed} and {n_groups} groups")
    return (4, g4) if is4 else (8, g8)


class SafetensorsGaf:
    """Memory-mapped safetensors file with grouped-affine tensors."""

    def __init__(self, path, config: Optional[dict] = None):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise GafFormatError("file shorter than the header length field")
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if 8 + hlen > len(self._mm):
            raise GafFormatError("header length exceeds the file")
        try:
            self.header: Dict[str, dict] = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except Exception as e:  # noqa: BLE001
            raise GafFormatError(f"bad header: {e}") from e
        self._data0 = 8 + hlen
        self.metadata = self.header.pop("__metadata__", {}) or {}
        q = (config or {}).get("quantization") or {}
        self.config_bits = q.get("bits")
        self.config_group = q.get("group_size")

    def close(self) -> None:
        if getattr(self, "_mm", None) is not None:
            try:
                self._mm.close()
            except BufferError:
                pass  # views are still alive; the map goes with them
            self._mm = None
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- raw access --
    def _bytes(self, name: str) -> Tuple[memoryview, dict]:
        info = self.header.get(name)
        if info is None:
            raise KeyError(name)
        b, e = info["data_offsets"]
        if not (0 <= b <= e <= len(self._mm) - self._data0):
            raise GafFormatError(f"{name}: data offsets out of range")
        return memoryview(self._mm)[self._data0 + b:self._data0 + e], info

    def gaf_bases(self) -> Iterator[str]:
        """Base names that have a U32 `.weight` with `.scales` and `.biases` beside it."""
        for name, info in self.header.items():
            if name.endswith(".weight") and info.get("dtype") == "U32":
                base = name[: -len(".weight")]
                if base + ".scales" in self.header and base + ".biases" in self.header:
                    yield base

    def tensor(self, base: str, expected_dim: Optional[int] = None) -> GafTensor:
        wb, wi = self._bytes(base + ".weight")
        sb, si = self._bytes(base + ".scales")
        bb, bi = self._bytes(base + ".biases")
        if wi.get("dtype") != "U32" or len(wi.get("shape", [])) != 2:
            raise GafFormatError(f"{base}.weight is not a 2-D U32 tensor")
        N, in_packed = (int(v) for v in wi["shape"])
        if N == 0 or len(wb) != N * in_packed * 4:
            raise GafFormatError(f"{base}.weight: byte size does not match its shape")
        sdt = si.get("dtype")
        if sdt not in ("BF16", "F16") or bi.get("dtype") != sdt:
            raise GafFormatError(f"{base}: scales / biases must both be BF16 or both F16")
        if len(sb) % (N * 2) != 0 or len(bb) != len(sb):
            raise GafFormatError(f"{base}: scales / biases sizes do not match {N} rows")
        n_groups = len(sb) // (N * 2)
        bits, group = infer_bits_and_group(in_packed, n_groups, expected_dim, self.config_bits)
        K = in_packed * (32 // bits)
        if K // group > MAX_SUPPORTED_GAFFINE_GROUPS:
            raise GafFormatError(f"{base}: {K // group} groups (max {MAX_SUPPORTED_GAFFINE_GROUPS})")  # error.TooManyGroups
        packed = np.frombuffer(wb, dtype=np.uint8).view(np.uint32).reshape(N, in_packed) if (
            (self._data0 + wi["data_offsets"][0]) % 4 == 0) else np.frombuffer(bytes(wb), dtype=np.uint32).reshape(N, in_packed)
        scales = _u16_view(sb, self._data0 + si["data_offsets"][0]).reshape(N, n_groups)
        biases = _u16_view(bb, self._data0 + bi["data_offsets"][0]).reshape(N, n_groups)
        return GafTensor(base, packed, scales, biases, bits, group, 1 if sdt == "BF16" else 0)

    def upload(self, ctx, base: str, shard_kind: int = 0, tp_rank: int = 0, tp_size: int = 1,
               expected_dim: Optional[int] = None):
        """`base` as a device weight (this rank's shard under tensor parallelism)."""
        from . import gaf
        t = self.tensor(base, expected_dim)
        return gaf.Weight.from_host(ctx, t.packed, t.scales, t.biases, t.group, t.bits, sdtype=t.scales_dtype,
                                    shard=shard_kind, tp_rank=tp_rank, tp_size=tp_size)


def _u16_view(buf: memoryview, file_offset: int) -> np.ndarray:
    if file_offset % 2 == 0:
        return np.frombuffer(buf, dtype=np.uint8).view(np.uint16)
    return np.frombuffer(bytes(buf), dtype=np.uint16)  # odd offset in the map: copy


def write_safetensors(path, tensors: Dict[str, Tuple[str, np.ndarray]], metadata: Optional[dict] = None) -> None:
    """Minimal writer ({name: (dtype string, array)}), the counterpart of
    core/src/io/safetensors/writer.zig:132-151; used to build fixtures and to round-trip quantized weights."""
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": [int(v) for v in arr.shape], "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)  # keep the data section 8-byte aligned, as the usual writers do
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
