"""The roofline denominators: measured on this pool if the driver wrote them, else the stated fallback."""
from __future__ import annotations

import json
import os
from typing import Tuple

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load() -> Tuple[dict, str]:
    """(peaks, "measured" or "fallback")."""
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path, "r", encoding="utf-8") as handle:
                raw = json.load(handle)
            peaks = dict(FALLBACK)
            for key in FALLBACK:
                if isinstance(raw.get(key), (int, float)) and raw[key] > 0:
                    peaks[key] = float(raw[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK), "fallback"


def hbm_gbs() -> float:
    return load()[0]["hbm_gbs"]
