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
