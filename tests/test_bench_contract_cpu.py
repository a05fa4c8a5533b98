"""bench.py without a GPU: the reference arm's line, and the reporter that prints the result line exactly
once, also when an extra measurement after the headline never comes back."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(code):
    return subprocess.run([sys.executable, "-c", f"import sys; sys.path.insert(0, {str(ROOT)!r}); import bench\n" + code],
                          capture_output=True, text=True, timeout=120)


def test_reference_arm_prints_its_unavailable_line_and_exits_zero():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and rec["unavailable"]


def test_result_line_is_printed_once_with_the_extras_that_finished():
    p = _run("r = bench.Reporter(0); r.out = {'value': 1.0}\n"
             "w = r.guard(30, 'alt'); r.out['alt'] = {'value': 2.0}; w.cancel(); r.emit(); r.emit()")
    assert p.returncode == 0
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1 and json.loads(lines[0]) == {"value": 1.0, "alt": {"value": 2.0}}


def test_an_extra_measurement_that_never_returns_ends_the_run_with_the_headline_line():
    p = _run("import time\nr = bench.Reporter(0); r.out = {'value': 1.0}\nr.guard(0.3, 'alt'); time.sleep(60); print('late')")
    assert p.returncode == 0 and "late" not in p.stdout
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["value"] == 1.0 and "error" in rec["alt"]


def test_other_ranks_leave_without_printing():
    p = _run("import time\nr = bench.Reporter(3); r.out = {'value': 1.0}\nr.guard(0.3, 'alt'); time.sleep(60)")
    assert p.returncode == 0 and p.stdout.strip() == ""
