"""Pieces shared by the benchmark launcher (bench.py) and the sharded benchmark entry: the metric
name, the measured-peak lookup and the read-only nvidia-smi clock sampler."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
METRIC = "K tokens scored+attended/sec (decode step, one layer)"
UNIT = "Ktok/s"
FALLBACK_HBM_GBS = 6650.0


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi sampling in a child process during the timed region (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return res
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            self.out.close()
            rows = [r.split(",") for r in Path(self.path).read_text().strip().splitlines() if r.strip()]
            os.unlink(self.path)
            sm = [float(r[1]) for r in rows if len(r) >= 9]
            if sm:
                res["sm_mhz"] = statistics.median(sm)
                res["sm_max_mhz"] = float(rows[0][2])
                res["power_w_max"] = max(float(r[3]) for r in rows if len(r) >= 9)
                res["samples"] = len(sm)
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for j, n in enumerate(names):
                    if any("Active" == r[5 + j].strip() for r in rows if len(r) >= 9):
                        res["reasons"].append(n)
        except Exception:
            pass
        return res



def hbm_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


