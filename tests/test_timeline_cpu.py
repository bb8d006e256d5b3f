"""CPU test of the timeline tool's reduction (catccos_b200/timeline.py): per-CTA stamps and accumulated waits in,
[min, median, max] in microseconds out.  The slot numbers are those of catccos_b200/csrc/trace.cuh."""
import re
from pathlib import Path

import numpy as np

from catccos_b200 import timeline

ROOT = Path(__file__).resolve().parents[1]


def test_slot_numbers_match_the_device_header():
    text = (ROOT / "catccos_b200" / "csrc" / "trace.cuh").read_text()
    slots = {name: int(val) for name, val in re.findall(r"(kTr\w+)\s*=\s*(\d+)", text)}
    assert int(re.search(r"kTraceSlots\s*=\s*(\d+)", text).group(1)) >= 75
    assert slots["kTrCtaStart"] == 0 and slots["kTrCtaEnd"] == 72
    assert slots["kTrQuantKernelStart"] == 73 and slots["kTrQuantKernelEnd"] == 74
    assert slots["kTrTileStart"] == timeline.TILE_START and slots["kTrTileEnd"] == timeline.TILE_END
    assert slots["kTrPushFirst"] == timeline.PUSH_FIRST and slots["kTrPushLast"] == timeline.PUSH_LAST
    by_col = {col: name for name, col in timeline.WAITS}
    for name in ("kTrProdFlagWaitNs", "kTrProdEmptyWaitNs", "kTrMmaFullWaitNs", "kTrMmaAccWaitNs", "kTrEpiWaitNs",
                 "kTrQuantPublishNs"):
        assert slots[name] in by_col, name
    assert slots["kTrSfGateWaitNs"] == timeline.SF_GATE and slots["kTrSfEmptyWaitNs"] == timeline.SF_EMPTY
    assert slots["kTrPushFlagWaitNs"] == timeline.PUSH_FLAGWAIT and slots["kTrPushFenceNs"] == timeline.PUSH_FENCE


def test_summarise_reduces_over_ctas():
    ctas = 6
    tr = np.zeros((ctas, 80), dtype=np.uint64)
    base = 1_000_000
    tr[:, 0] = base + np.arange(ctas) * 1000          # CTA start: 0, 1, ... 5 us
    tr[:, 72] = base + 50_000 + np.arange(ctas) * 2000  # CTA end: 50, 52, ... 60 us
    tr[:, 4] = np.array([0, 3000, 3000, 5000, 0, 9000])  # flag waits in ns; zero = this CTA never waited
    tr[:3, timeline.TILE_START] = base + 2000
    tr[:3, timeline.TILE_END] = base + 2000 + np.array([20_000, 22_000, 30_000])
    tr[0, 73], tr[0, 74] = 0xFFFFFFFFFFFFFFFF, 0       # quantise-kernel stamps untouched
    out = timeline.summarise(tr)
    assert out["ctas"] == ctas
    assert out["CTA start"] == [0.0, 2.5, 5.0]
    assert out["CTA end"] == [50.0, 55.0, 60.0]
    assert out["TMA producer waiting for ready flags (total per CTA)"] == [3.0, 4.0, 9.0]
    assert out["tile 0: duration"] == [20.0, 22.0, 30.0]
    assert "quantise kernel: first CTA starts / last CTA ends" not in out
    assert out["first MMA"] is None  # nobody wrote the slot
    tr[0, 73], tr[0, 74] = base - 10_000, base + 4000
    out = timeline.summarise(tr)
    assert out["quantise kernel: first CTA starts / last CTA ends"] == [-10.0, 4.0]
