"""The unit partition of a launch list, restated in Python (talu_b200/csrc/gaf_gemv.cu: range_begin, unit_owner,
range_index, plan_gemv, gemv_list_ctas and the rotation in gemv_list_create) and checked for the properties the kernel
relies on: every unit of every operation belongs to exactly one CTA, a row group is cut into no more pieces than the
scratch has slots for, and over a whole list no CTA carries more than one unit above any other."""
import random

import pytest

ROWS, CHUNK_BYTES = 128, 256


def range_begin(cta, units, ctas):
    q, rem = divmod(units, ctas)
    return cta * q + min(cta, rem)


def unit_owner(u, units, ctas):
    q, rem = divmod(units, ctas)
    cut = rem * (q + 1)
    return u // (q + 1) if u < cut else rem + (u - cut) // q


def plan(N, row_bytes, ctas_wanted):
    rgs = -(-N // ROWS)
    chunks = -(-row_bytes // CHUNK_BYTES)
    units = rgs * chunks
    ctas = max(1, min(ctas_wanted, units))
    q = units // ctas
    return dict(rgs=rgs, chunks=chunks, units=units, ctas=ctas, max_slots=-(-chunks // q) + 1)


def list_partition(shapes, M, sms=148):
    """-> (grid, per operation: plan, rot)"""
    plans = [plan(N, K // 2, sms) for (N, K) in shapes]          # gaf4: K / 2 packed bytes per row
    grid = max(p["ctas"] for p in plans) if M <= 4 else min(p["ctas"] for p in plans)
    out, rot = [], 0
    for p in plans:
        out.append((p, rot))
        rot = (rot + grid - p["units"] % grid) % grid
    return grid, out


LLAMA8B_FFN = [(28672, 4096), (4096, 14336)] * 12
LLAMA70B = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]


def shard(shapes, world):
    out = []
    for i, (N, K) in enumerate(shapes):
        out.append((N // world, K) if i % 2 == 0 else (N, K // world))   # column-parallel, row-parallel in turn
    return out


CASES = [("8B FFN stack", LLAMA8B_FFN, 1), ("8B FFN stack", LLAMA8B_FFN, 4), ("8B FFN stack, eight rows", LLAMA8B_FFN, 8)]
CASES += [(f"70B shards of {w} ranks", shard(LLAMA70B, w) * 8, 1) for w in (1, 2, 4, 8)]
CASES += [("K = N = 4096", [(4096, 4096)] * 48, 1), ("small and large", [(8192, 8192), (256, 1024), (1024, 2048), (8192, 1024), (20480, 4608)], 3)]


@pytest.mark.parametrize("label,shapes,M", CASES, ids=[c[0] for c in CASES])
def test_every_unit_once_slots_bounded_totals_balanced(label, shapes, M):
    grid, ops = list_partition(shapes, M)
    totals = [0] * grid
    for p, rot in ops:
        units, chunks = p["units"], p["chunks"]
        seen = 0
        for b in range(grid):
            v = (b + rot) % grid
            lo, hi = range_begin(v, units, grid), range_begin(v + 1, units, grid)
            assert lo <= hi <= units
            totals[b] += hi - lo
            seen += hi - lo
            if hi > lo:
                assert unit_owner(lo, units, grid) == v and unit_owner(hi - 1, units, grid) == v
        assert seen == units                                  # contiguous ranges of distinct indices: every unit once
        for rg in range(p["rgs"]):
            first, last = unit_owner(rg * chunks, units, grid), unit_owner(rg * chunks + chunks - 1, units, grid)
            assert last - first + 1 <= p["max_slots"], (label, rg)
    if M <= 4:
        assert max(totals) - min(totals) <= 1, (label, max(totals), min(totals))


def test_without_rotation_the_same_ctas_carry_every_remainder():
    """What the rotation is for: with rot = 0 throughout, CTAs 0..7 of the 8B stack have 20 units per layer (13 of the
    1792 of gate|up, 7 of the 896 of down) against a mean of 18.2 and 18 on most CTAs: 24 units more than the lightest
    CTA over 12 layers, a tenth of the launch."""
    grid, ops = list_partition(LLAMA8B_FFN, 1)
    totals = [0] * grid
    for p, _ in ops:
        for b in range(grid):
            totals[b] += range_begin(b + 1, p["units"], grid) - range_begin(b, p["units"], grid)
    assert max(totals) == 20 * 12 and min(totals) == 18 * 12


def test_random_lists():
    rnd = random.Random(5)
    for _ in range(200):
        shapes = [(rnd.choice([128, 384, 1000, 4096, 8192, 20480]), rnd.choice([512, 1024, 4096, 4608, 14336])) for _ in range(rnd.randint(1, 9))]
        M = rnd.choice([1, 2, 3, 4])
        grid, ops = list_partition(shapes, M, sms=rnd.choice([148, 132, 64]))
        totals = [0] * grid
        for p, rot in ops:
            covered = set()
            for b in range(grid):
                v = (b + rot) % grid
                lo, hi = range_begin(v, p["units"], grid), range_begin(v + 1, p["units"], grid)
                totals[b] += hi - lo
                covered.update(range(lo, hi))
            assert len(covered) == p["units"]
        assert max(totals) - min(totals) <= 1
