"""bench.py's command-line contract and host-side helpers (no GPU): the defaults the driver relies on,
the peak denominators, and that the reference arm leaves every rank but 0 without work."""
import importlib.util
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_defaults(monkeypatch):
    bench = load_bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert args.gpus == 1 and args.steps >= 20 and args.warmup >= 3 and args.impl == "ours"
    assert not args.no_gather and not args.no_c5            # C5 and the gather timings are on by default
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "20", "--warmup", "5", "--impl", "reference"])
    args = bench.parse_args()
    assert (args.gpus, args.steps, args.warmup, args.impl) == (8, 20, 5, "reference")


def test_peak_denominators(tmp_path, monkeypatch):
    bench = load_bench()
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    assert bench.measured_peaks() == (bench.FALLBACK_BF16_TFLOPS, bench.FALLBACK_BF16_SUSTAINED_TFLOPS, "fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"bf16_tflops": 1663.5, "bf16_tflops_sustained": 1396.0}))
    assert bench.measured_peaks() == (1663.5, 1396.0, "measured")
    assert bench.PARITY_TOL == 5e-3 and bench.PARITY_ROWS >= 16


def test_reference_arm_is_silent_on_other_ranks():
    """Under torchrun the reference arm runs on rank 0 alone; the others exit 0 without output or work."""
    env = dict(os.environ, RANK="3", WORLD_SIZE="8", LOCAL_RANK="3")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "8"], env=env,
                          capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0 and proc.stdout.strip() == ""
