"""What ``bench.py`` owes its caller where no GPU is needed: more than one GPU is refused with exit code 2,
the reference arm says why it is unavailable, and the roofline denominators come from the measured peaks."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=900)


def test_more_than_one_gpu_is_refused_with_exit_code_2():
    r = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_the_reference_arm_says_that_it_is_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks() == (bench.FALLBACK_HBM_GBS, bench.FALLBACK_BF16_TFLOPS, "fallback", None)
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6000.5, "bf16_tflops": 1500, "bf16_tflops_sustained": 1300}))
    assert bench.peaks() == (6000.5, 1500.0, "measured", 1300)
    (tmp_path / "MEASURED_PEAKS.json").write_text("{broken")
    assert bench.peaks()[2] == "fallback"
