"""In-tree build of the two native libraries.

* ``cogito_b200/lib/libcogito_kernels.so`` — every ``csrc/kernels/*.cu`` and
  ``csrc/comm/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``).
* ``cogito_b200/lib/libcogito.so`` — the host C++17 runtime exporting the
  ``cg_*`` C ABI (``csrc/capi/*.cpp``), compiled by g++.

Objects are cached under ``build/`` and rebuilt when a source or any header is
newer.  ``python -m cogito_b200.build`` builds both; ``--kernels`` / ``--capi``
build one; ``--debug-bounds`` builds the index-checking copy of the kernel library.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LIB_DIR = ROOT / "cogito_b200" / "lib"
BUILD_DIR = ROOT / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]
# the file that holds the host runtime's hot loops: full vectorisation, sqrt without errno
CXX_FILE_FLAGS = {"host_simd.cpp": ["-O3", "-fno-math-errno"]}


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _compile_one(cmd: list[str], log: Path) -> tuple[int, str]:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(proc.stdout + proc.stderr)
    return proc.returncode, proc.stdout + proc.stderr


def _build(sources: list[Path], headers: list[Path], out: Path, compiler: list[str],
           link: list[str], tag: str, verbose: bool, file_flags: dict | None = None) -> bool:
    """Compile `sources` to objects (in parallel) and link `out`. Returns True if relinked.
    file_flags: extra flags by source file name (appended, so a later -O wins)."""
    obj_dir = BUILD_DIR / tag
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    hdr_time = _newest(headers)
    jobs = []
    objs = []
    for src in sources:
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_time):
            continue
        jobs.append((src, obj))
    failed = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {
                ex.submit(_compile_one, compiler + (file_flags or {}).get(src.name, []) + ["-c", str(src), "-o", str(obj)],
                          obj_dir / (src.stem + ".log")): src
                for src, obj in jobs
            }
            for fut in cf.as_completed(futs):
                rc, text = fut.result()
                src = futs[fut]
                if rc != 0:
                    failed.append((src, text))
                elif verbose:
                    print(f"[build] {src.name} ok")
    if failed:
        for src, text in failed:
            sys.stderr.write(f"---- {src} ----\n{text}\n")
        raise RuntimeError(f"compilation failed for: {', '.join(s.name for s, _ in failed)}")
    if out.exists() and not jobs and out.stat().st_mtime >= _newest(objs):
        return False
    cmd = link + [str(o) for o in objs] + ["-o", str(out)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"link failed for {out.name}")
    return True


def build_kernels(verbose: bool = False, debug_bounds: bool = False) -> Path:
    """debug_bounds: the same sources with -DCGK_DEBUG_BOUNDS as ``libcogito_kernels_dbg.so``: indices
    that come from data or from tile edges are checked, the first violation per source file is
    recorded (never a trap) and the access redirected inside the array.  ``COGITO_KERNELS_DEBUG=1``
    makes the package load that library, and ``ops._lib.assert_device_ok`` (which the GPU tests
    call after every test) then fails on a recorded violation."""
    srcs = sorted((ROOT / "csrc" / "kernels").glob("*.cu")) + sorted((ROOT / "csrc" / "comm").glob("*.cu"))
    hdrs = (list((ROOT / "csrc").rglob("*.cuh")) + list((ROOT / "csrc").rglob("*.h")) + list((ROOT / "csrc").rglob("*.inc"))
            + list((ROOT / "include").glob("*.h")))
    out = LIB_DIR / ("libcogito_kernels_dbg.so" if debug_bounds else "libcogito_kernels.so")
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-DCGK_DEBUG_BOUNDS"] if debug_bounds else [])
    _build(srcs, hdrs, out, [nvcc] + flags + ["-I", str(ROOT / "include")],
           [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
            "-cudart", "shared"],
           "kernels_dbg" if debug_bounds else "kernels", verbose)
    return out


def build_capi(verbose: bool = False) -> Path:
    srcs = sorted((ROOT / "csrc" / "capi").glob("*.cpp"))
    hdrs = list((ROOT / "include").glob("*.h")) + list((ROOT / "csrc" / "capi").glob("*.h*"))
    out = LIB_DIR / "libcogito.so"
    if not srcs:
        return out
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    _build(srcs, hdrs, out, [cxx] + CXX_FLAGS + ["-I", str(ROOT / "include")],
           # a toolchain that links libstdc++ statically must not export (or be interposed on)
           # its copy inside a process that already holds another libstdc++
           [cxx, "-shared", "-fPIC", "-Wl,--exclude-libs,ALL", "-Wl,-Bsymbolic", "-lpthread", "-ldl"], "capi", verbose,
           file_flags=CXX_FILE_FLAGS)
    return out


def build_capi_sanitized(verbose: bool = False) -> Path:
    """The host runtime compiled with AddressSanitizer + UndefinedBehaviorSanitizer, as
    ``build/libcogito_asan.so`` (not shipped; the memory-safety tests link C programs against it)."""
    srcs = sorted((ROOT / "csrc" / "capi").glob("*.cpp"))
    hdrs = list((ROOT / "include").glob("*.h")) + list((ROOT / "csrc" / "capi").glob("*.h*"))
    out = BUILD_DIR / "libcogito_asan.so"
    # the first compiler whose installation carries the sanitizer runtime
    cxx = None
    for cand in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++"):
        if not cand:
            continue
        probe = subprocess.run([cand, "-print-file-name=libasan.so"], capture_output=True, text=True)
        if probe.returncode == 0 and Path(probe.stdout.strip()).is_absolute() and Path(probe.stdout.strip()).exists():
            cxx = cand
            break
    if cxx is None:
        raise RuntimeError("no C++ compiler with an AddressSanitizer runtime found")
    san = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g"]
    flags = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1"] + san
    _build(srcs, hdrs, out, [cxx] + flags + ["-I", str(ROOT / "include")],
           [cxx, "-shared", "-fPIC"] + san + ["-lpthread", "-ldl"], "capi_asan", verbose)
    return out


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_capi(verbose)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--kernels", action="store_true")
    ap.add_argument("--capi", action="store_true")
    ap.add_argument("--sanitize", action="store_true", help="only build the ASan + UBSan copy of the host runtime")
    ap.add_argument("--debug-bounds", action="store_true",
                    help="only build libcogito_kernels_dbg.so: every kernel with index checks that record the first violation")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args()
    if args.sanitize:
        print(build_capi_sanitized(args.verbose))
        return
    if args.debug_bounds:
        print(build_kernels(args.verbose, debug_bounds=True))
        return
    if args.kernels or not args.capi:
        print(build_kernels(args.verbose))
    if args.capi or not args.kernels:
        print(build_capi(args.verbose))


if __name__ == "__main__":
    main()
