"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one
line and exit code 2, the reference arm reports that it is unavailable and exits 0, and the
measured peaks are found wherever the file keeps them."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    proc = run_bench("--gpus", "2")
    assert proc.returncode == 2
    assert len([l for l in proc.stdout.splitlines() if l.strip()]) == 1 and "one GPU" in proc.stdout


def test_reference_arm_says_it_is_unavailable():
    proc = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_measured_peaks_are_found_at_any_depth(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setattr(bench, "HERE", str(tmp_path))
    assert bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"gpu": "B200", "peaks": {"hbm_gbs": 6700.5, "bf16_tflops": 1601.0, "bf16_tflops_sustained": 1405.0}}))
    pk = bench.peaks()
    assert pk["source"] == "measured" and pk["hbm_gbs"] == 6700.5 and pk["bf16_tflops"] == 1601.0
    (tmp_path / "MEASURED_PEAKS.json").write_text("{not json")
    assert bench.peaks()["source"] == "fallback"
