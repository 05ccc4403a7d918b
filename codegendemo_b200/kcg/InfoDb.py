"""Kernel database: best tuning config per (M, N, K, dtype, IS_ATRANS).

The reference leaves this as a stub (Runtime/python/kcg/InfoDb.py:9-16, "cache system not done yet"
in its README): every run re-tunes. Here the top-K json files the autotuner writes
(``PerfTester.jsonfyBestPerfs``, KCGTask.py:207-211 in the reference) can be merged into one json
file, and ``lookup`` returns the fastest known config of a shape so that an operator call picks a
tuned cubin without tuning again.
"""
import json
import os
from typing import Dict, Optional

from codegendemo_b200.kcg.Utils import ConfigKeywords as kw


def default_db_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "TuningCombs", "best_b200.json")


class KernelDb:
    def __init__(self, path: Optional[str] = None):
        self.path = path or os.environ.get("KCG_KERNEL_DB", default_db_path())
        self.entries: Dict[str, Dict] = {}
        if os.path.exists(self.path):
            with open(self.path) as f:
                for e in json.load(f).get("results", []):
                    self.entries[self.key_of(e["config"])] = e

    @staticmethod
    def key(M: int, N: int, K: int, dtype: int, atrans: int) -> str:
        return f"{int(M)}x{int(N)}x{int(K)}:dt{int(dtype)}:at{1 if atrans else 0}"

    @staticmethod
    def key_of(config: Dict) -> str:
        return KernelDb.key(config[kw.KEY_M], config[kw.KEY_N], config[kw.KEY_K], config[kw.KEY_DTYPE_A],
                            config[kw.KEY_IS_A_TRANSPOSE])

    def lookup(self, M: int, N: int, K: int, dtype: int, atrans: int = 0) -> Optional[Dict]:
        """The stored result record ({'config', 'kcgMs', 'tflops', ...}) of the shape, or None."""
        return self.entries.get(self.key(M, N, K, dtype, atrans))

    def update(self, results) -> int:
        """Merges result records (dicts as KernelTestResult.jsonfy produces); keeps the fastest
        correct one per shape. Returns how many entries changed."""
        changed = 0
        for r in results:
            if not r.get("correct", False) or r.get("kcgMs", 0) <= 0:
                continue
            k = self.key_of(r["config"])
            old = self.entries.get(k)
            if old is None or r["kcgMs"] < old["kcgMs"]:
                self.entries[k] = r
                changed += 1
        return changed

    def update_from_perf_json(self, perf_json_path: str) -> int:
        with open(perf_json_path) as f:
            return self.update(json.load(f).get("results", []))

    def save(self, path: Optional[str] = None) -> str:
        path = path or self.path
        os.makedirs(os.path.dirname(path), exist_ok=True)
        tmp = path + ".part"
        with open(tmp, "w") as f:
            json.dump({"results": [self.entries[k] for k in sorted(self.entries)]}, f, indent=1)
        os.replace(tmp, path)
        return path
