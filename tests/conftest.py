import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "llm-pruning_b200")
for p in (ROOT, PKG_DIR, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ---- strict-form error numbers --------------------------------------------------------------
# The tolerance is stated as max|err| <= 2e-2 * rms(whole expected output).  Where a test
# asserts a refined form instead (RMS over the non-zero entries, per-row RMS, a wider bound on
# an intermediate), it also records the strict-form number here; the numbers are printed in
# the terminal summary and written to a JSON file (the path in DPK_PARITY_REPORT, else pytest's
# cache directory) so that the distance from the stated bound is on record.

STRICT = {}


def record_strict(label: str, value: float, asserted: str = "") -> None:
    key = label
    n = 1
    while key in STRICT:
        n += 1
        key = f"{label}#{n}"
    STRICT[key] = {"max_abs_over_global_rms": float(value), "asserted": asserted}


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    if not STRICT:
        return
    import json

    tr = terminalreporter
    tr.section("strict-form error, max|err| / rms(whole expected output), where a refined form is asserted")
    worst = sorted(STRICT.items(), key=lambda kv: -kv[1]["max_abs_over_global_rms"])
    for key, rec in worst[:40]:
        tr.write_line(f"{rec['max_abs_over_global_rms']:9.4g}  {key}  [{rec['asserted']}]")
    path = os.environ.get("DPK_PARITY_REPORT")
    if not path:
        cache = os.path.join(ROOT, ".pytest_cache")
        if os.path.isdir(cache):
            path = os.path.join(cache, "parity_strict_metrics.json")
    if path:
        try:
            with open(path, "w") as f:
                json.dump(STRICT, f, indent=1, sort_keys=True)
        except OSError:
            pass
