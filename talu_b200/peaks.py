"""Roofline denominators: the copy bandwidth and bf16 GEMM throughput measured on the GPU pool,
read from MEASURED_PEAKS.json beside the package's parent directory when present."""
from __future__ import annotations

import json
from pathlib import Path

_FILE = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"

# an earlier measurement on B200, used only when the file is absent
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = (1590.0, 1400.0)


def _load():
    try:
        return json.loads(_FILE.read_text())
    except Exception:
        return None


def measured_peak_hbm():
    """(GB/s, "measured" | "fallback")"""
    j = _load()
    try:
        return float(j["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_peak_tflops():
    """(burst TFLOP/s, sustained TFLOP/s, "measured" | "fallback")"""
    j = _load()
    try:
        return float(j["bf16_tflops"]), float(j["bf16_tflops_sustained"]), "measured"
    except Exception:
        return (*FALLBACK_BF16_TFLOPS, "fallback")
