"""The ctypes mirrors of the kernel library's argument structs have the layout the C header gives them:
a C program prints size and field offsets of every struct, and they are compared with ctypes'."""
import ctypes
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _pairs():
    from cogito_b200.ops import _lib, attention
    from cogito_b200.parallel import data_parallel, tp_ops
    from cogito_b200.serve import kv_cache
    return [("cgk_gemm_args", _lib.GemmArgs), ("cgk_flash_args", attention.FlashArgs), ("cgk_ag_args", tp_ops.AgArgs),
            ("cgk_rs_args", tp_ops.RsArgs), ("cgk_dp_bucket_args", data_parallel.DpBucketArgs),
            ("cgk_dp_finish_args", data_parallel.DpFinishArgs), ("cgk_kv_args", kv_cache.KvArgs)]


@pytest.mark.skipif(shutil.which("gcc") is None and shutil.which("cc") is None, reason="needs a C compiler")
def test_argument_structs_match_the_header(tmp_path):
    pairs = _pairs()
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "cogito_kernels.h"', 'int main(void) {']
    for cname, cls in pairs:
        lines.append(f'  printf("{cname} . %zu\\n", sizeof({cname}));')
        for field in cls._fields_:
            lines.append(f'  printf("{cname} {field[0]} %zu\\n", offsetof({cname}, {field[0]}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    cc = shutil.which("gcc") or shutil.which("cc")
    subprocess.run([cc, "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True, capture_output=True, text=True)
    got = {}
    for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines():
        s, f, v = ln.split()
        got[(s, f)] = int(v)
    for cname, cls in pairs:
        assert got[(cname, ".")] == ctypes.sizeof(cls), cname
        for field in cls._fields_:
            assert got[(cname, field[0])] == getattr(cls, field[0]).offset, (cname, field[0])


@pytest.mark.skipif(shutil.which("gcc") is None and shutil.which("cc") is None, reason="needs a C compiler")
def test_host_library_mirrors_used_by_the_tests_match_the_public_headers(tmp_path):
    """The ctypes mirrors in tests/capi_defs.py (shared by the CPU and the B200 test files) against include/cogito.h:
    every mirrored field sits at the header's offset; a mirror may stop before the end of a struct the library allocates."""
    import sys
    sys.path.insert(0, str(ROOT / "tests"))
    import capi_defs as d
    pairs = [("cg_flash_attn_config", d.FlashConfig, True), ("cg_flash_attn_params", d.FlashParams, True),
             ("cg_memory_stats", d.MemoryStats, True), ("cg_schedule_step", d.ScheduleStep, True),
             ("cg_transformer_config", d.TransformerConfig, True), ("cg_mixed_precision", d.MixedPrecision, False),
             ("cg_speculative_decoder", d.SpecDecoder, False), ("cg_3d_parallel", d.Parallel3D, False)]
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "cogito.h"', 'int main(void) {']
    for cname, cls, _ in pairs:
        lines.append(f'  printf("{cname} . %zu\\n", sizeof({cname}));')
        for field in cls._fields_:
            lines.append(f'  printf("{cname} {field[0]} %zu\\n", offsetof({cname}, {field[0]}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "host_layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "host_layout"
    cc = shutil.which("gcc") or shutil.which("cc")
    subprocess.run([cc, "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True, capture_output=True, text=True)
    got = {}
    for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines():
        s, f, v = ln.split()
        got[(s, f)] = int(v)
    for cname, cls, whole in pairs:
        assert ctypes.sizeof(cls) == got[(cname, ".")] if whole else ctypes.sizeof(cls) <= got[(cname, ".")], cname
        for field in cls._fields_:
            assert got[(cname, field[0])] == getattr(cls, field[0]).offset, (cname, field[0])
