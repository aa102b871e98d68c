"""Measured roofline denominators for this GPU pool.

``MEASURED_PEAKS.json`` at the repository root (written by the benchmark driver) holds a
STREAM-style copy bandwidth and cuBLAS bf16 throughput measured on the pool's B200s. When the
file is absent the stated fallback (an earlier measurement on the same pool) is used.
"""
from __future__ import annotations

import json
from pathlib import Path

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_peaks() -> dict:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            d["source"] = "measured"
            return d
        except Exception:
            pass
    return dict(FALLBACK)
