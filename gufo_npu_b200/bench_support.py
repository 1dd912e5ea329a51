"""Small helpers shared by bench.py and the multi-GPU bench arm."""
from __future__ import annotations

import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def measured_hbm_peak():
    """(GB/s, "measured" | "fallback"): the copy bandwidth measured on this pool's B200s where
    the file with it is present, else an earlier measurement of the same pool."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"
