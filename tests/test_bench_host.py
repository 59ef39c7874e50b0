"""Host-side logic of bench.py that needs no GPU: the byte counts behind the roofline, the peaks file, and the
reference arm (the CPU oracle timed on the host cores) with its one JSON line."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_algorithmic_bytes_of_a_block():
    one = bench.layer_bytes(1)
    # gate/up: 6 routed experts (codes + scales) and 2 shared BF16 experts; down likewise; the router's 258 rows
    assert one["gate_up"] == 56_623_104 + 67_108_864
    assert one["down"] == 28_311_552 + 33_554_432
    assert one["router"] == 258 * 4096 * 2
    assert one["total"] == 187_711_536
    eight = bench.layer_bytes(8)
    assert eight["gate_up"] * 8 == one["gate_up"] and eight["down"] * 8 == one["down"] and eight["router"] == one["router"]
    # what a rank keeps resident: every expert's slice, the shared experts' slices, the router
    assert bench.resident_bytes_per_layer(1) * 40 < 180e9 and bench.resident_bytes_per_layer(8) * 40 < 25e9


def test_peaks_come_from_the_measured_file_when_it_is_there():
    peaks, kind = bench.load_peaks()
    assert kind in ("measured", "fallback") and peaks["hbm_gbs"] > 1000
    if (ROOT / "MEASURED_PEAKS.json").exists():
        assert kind == "measured"


def _reference_arm(rank: int):
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2")
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                           "--warmup", "1", "--layers", "2"], env=env, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_line_on_rank_zero_and_nothing_elsewhere():
    other = _reference_arm(1)
    assert other.returncode == 0 and other.stdout.strip() == ""
    first = _reference_arm(0)
    assert first.returncode == 0, first.stderr[-2000:]
    lines = [line for line in first.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert line["value"] > 0 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
