"""Tensor-parallel layout of the gaf linears of a decoder layer (host logic only).

The reference is single-device; this is the sharding the C ABI's
tgaf_weight_upload applies (include/talu_gaf.h): column-parallel weights
(qkv, gate, up) keep a contiguous block of output rows, row-parallel weights
(o, down) keep a contiguous block of input columns cut on group boundaries and
produce partial sums that one allreduce per layer half adds up.
"""
from __future__ import annotations

from dataclasses import dataclass

SHARD_NONE, SHARD_COL, SHARD_ROW = 0, 1, 2


@dataclass(frozen=True)
class ShardSlice:
    n0: int
    n1: int
    k0: int
    k1: int

    @property
    def n(self) -> int:
        return self.n1 - self.n0

    @property
    def k(self) -> int:
        return self.k1 - self.k0


def shard_slice(N: int, K: int, group: int, bits: int, kind: int, rank: int, size: int) -> ShardSlice:
    """Rows [n0, n1) and columns [k0, k1) of the full weight that `rank` keeps."""
    if size < 1 or not (0 <= rank < size):
        raise ValueError(f"bad rank {rank} of {size}")
    vpw = 32 // bits
    if K % group or K % vpw or group % vpw:
        raise ValueError("bad shape")
    if kind == SHARD_NONE or size == 1:
        return ShardSlice(0, N, 0, K)
    if kind == SHARD_COL:
        if N % size:
            raise ValueError(f"N={N} not divisible by {size} ranks")
        n = N // size
        return ShardSlice(rank * n, (rank + 1) * n, 0, K)
    if kind == SHARD_ROW:
        if K % (size * group):
            raise ValueError(f"K={K} not divisible by ranks*group = {size}*{group}")
        k = K // size
        return ShardSlice(0, N, rank * k, (rank + 1) * k)
    raise ValueError(f"bad shard kind {kind}")


def slice_arrays(packed, scales, biases, group: int, bits: int, sl: ShardSlice):
    """The canonical-layout arrays of one shard (what the library keeps on `rank`'s device)."""
    vpw = 32 // bits
    return (packed[sl.n0:sl.n1, sl.k0 // vpw: sl.k1 // vpw],
            scales[sl.n0:sl.n1, sl.k0 // group: sl.k1 // group],
            biases[sl.n0:sl.n1, sl.k0 // group: sl.k1 // group])


# Llama-3-70B-shaped decoder-layer linears: name -> (N, K, shard kind)
LLAMA3_70B_LINEARS = {
    "qkv": (10240, 8192, SHARD_COL),
    "o": (8192, 8192, SHARD_ROW),
    "gate_up": (2 * 28672, 8192, SHARD_COL),   # gate and up stacked along N (one fused launch)
    "down": (8192, 28672, SHARD_ROW),
}
