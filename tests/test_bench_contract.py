"""What bench.py promises without a GPU: more than one GPU is refused with exit code 2, the reference arm
says why it is unavailable, and the roofline denominators come from the peaks file when it can be read."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT)


def test_more_than_one_gpu_is_refused():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert "one GPU" in p.stdout and len(p.stdout.strip().splitlines()) == 1


def test_the_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_peaks_come_from_the_file_or_fall_back(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks() == (bench.FALLBACK_PEAKS, "fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6700, "bf16_tflops": 1600, "bf16_tflops_sustained": 1400}))
    pk, src = bench.peaks()
    assert src == "measured" and pk == {"hbm_gbs": 6700.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0}
    for broken in ("{", json.dumps({"hbm_gbs": None, "bf16_tflops": 1}), json.dumps({"hbm_gbs": 1})):
        (tmp_path / "MEASURED_PEAKS.json").write_text(broken)
        assert bench.peaks() == (bench.FALLBACK_PEAKS, "fallback")
