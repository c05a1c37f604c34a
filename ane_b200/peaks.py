"""Roofline denominators: the HBM copy bandwidth measured on the target machines (a file
MEASURED_PEAKS.json at the repository root, key "hbm_gbs"), else an earlier measurement."""
from __future__ import annotations

import json
import os

FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hbm_peak_gbs():
    """(GB/s, "measured" | "fallback")"""
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"
