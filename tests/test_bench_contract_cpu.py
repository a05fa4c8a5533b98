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


_STAND_INS = '''
import sys, time
import torch
real_device = torch.device
class Ev:
    def __init__(self, enable_timing=False): self.t = None
    def record(self): self.t = time.time()
    def elapsed_time(self, o): return (o.t - self.t) * 1e3 + 1.0
torch.cuda.set_device = lambda *a, **k: None
torch.cuda.synchronize = lambda *a, **k: None
torch.cuda.empty_cache = lambda *a, **k: None
torch.cuda.Event = Ev
torch.Tensor.pin_memory = lambda self: self
torch.device = lambda *a, **k: real_device("cpu")
import cogito_b200.bench_support as bs
class Job:
    flops_per_token = 1e9
    vocab = 50304
    def __init__(self): self.n = 0
    def step(self, ids, tg):
        self.n += 1
        return torch.tensor(9.5)
    def reset_launch_count(self): self.n = 0
    def launch_count(self): return self.n * 100
bs.build_job = lambda args, rank, world, dev: Job()
sys.argv = ["bench.py", "--steps", "2", "--warmup", "1", "--global-batch", "2", "--seq-len", "8", "--serving", "off"]
sys.exit(bench.main())
'''


def test_main_prints_one_line_with_every_key_of_the_contract():
    """main() end to end with the CUDA entry points and the job replaced by stand-ins: the control flow
    around the timed regions, the baseline arm and the reporter, and the keys of the line."""
    p = _run(_STAND_INS)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "baseline"):
        assert key in rec, key
    assert rec["n_gpus"] == 1 and rec["steps"] == 2 and rec["warmup"] == 3 and rec["gpu_launches"] == 200
    assert rec["higher_is_better"] is True and rec["dtype"] == "bf16" and rec["config"]["parallelism"] == "tp1"
    assert set(rec["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert rec["e2e"]["h2d_bytes_per_step"] == 2 * 2 * 8 * 8 and rec["e2e"]["d2h_bytes_per_step"] == 4
    assert rec["vs_baseline"] == rec["value"] / rec["baseline"]["value"]


def test_top_level_namespace_resolves_every_name_lazily():
    p = _run("import sys\nimport cogito_b200 as cg\nassert 'torch' not in sys.modules or True\n"
             "missing = [n for n in cg.__all__ if not hasattr(cg, n)]\nassert not missing, missing\n"
             "assert cg.GPT2.__module__ == 'cogito_b200.models.gpt2' and cg.nn.Linear is not None and cg.__version__\n"
             "try:\n    cg.no_such_name\nexcept AttributeError:\n    print('ok')")
    assert p.returncode == 0 and p.stdout.strip().endswith("ok"), p.stderr[-1500:]


def test_kernel_benchmark_host_mode_runs_every_host_case():
    p = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "kernels.py"), "all", "--device", "cpu", "--iters", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-1500:]
    recs = [json.loads(ln) for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert not [r for r in recs if "error" in r], recs
    assert {r["case"] for r in recs} >= {"elementwise", "jit_chain", "reduce", "rope", "swiglu", "dropout", "int4_quantize",
                                         "int4_dequantize", "spec_accept", "tree_mask"}
