"""Memory-safety check of the host runtime: the C++ sources are compiled with AddressSanitizer and
UndefinedBehaviorSanitizer (``python -m cogito_b200.build --sanitize``) and C programs that walk
through the subsystems run against that copy with leak detection on.  The reference has no
sanitizer build at all (no flags in its CMakeLists.txt); its latent out-of-bounds writes in the
pool's free lists and opcode-name table are the kind of defect this run is there to catch."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def asan_lib():
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    probe = subprocess.run([cc, "-fsanitize=address,undefined", "-x", "c", "-", "-o", os.devnull],
                           input="int main(void){return 0;}", text=True, capture_output=True)
    if probe.returncode != 0:
        pytest.skip("the toolchain has no sanitizer runtime")
    sys.path.insert(0, str(ROOT))
    from cogito_b200.build import build_capi_sanitized
    return cc, build_capi_sanitized()


def _run(cc, lib, src, tmp_path, *args):
    exe = tmp_path / (Path(src).stem + "_asan")
    subprocess.check_call([cc, "-std=c11", "-g", "-Wall", "-Werror", "-fsanitize=address,undefined", "-I", str(ROOT / "include"),
                           str(src), str(lib), f"-Wl,-rpath,{lib.parent}", "-lm", "-o", str(exe)])
    env = dict(os.environ, COGITO_FORCE_HOST="1", ASAN_OPTIONS="detect_leaks=1:abort_on_error=0:halt_on_error=1",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    return subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True, env=env, cwd=tmp_path, timeout=600)


def test_subsystem_walk_is_clean_under_asan_and_ubsan(asan_lib, tmp_path):
    cc, lib = asan_lib
    r = _run(cc, lib, ROOT / "tests" / "capi_stress.c", tmp_path, tmp_path / "stress.cog")
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-6000:]
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr and "LeakSanitizer" not in r.stderr, r.stderr[-6000:]


@pytest.mark.parametrize("example", ["xor.c", "mnist.c"])
def test_examples_are_clean_under_asan_and_ubsan(asan_lib, tmp_path, example):
    cc, lib = asan_lib
    r = _run(cc, lib, ROOT / "examples" / example, tmp_path)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-6000:]
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr and "LeakSanitizer" not in r.stderr, r.stderr[-6000:]
