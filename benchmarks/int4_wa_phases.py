"""Where a step of the weights-as-A INT4 GEMM spends its cycles.

    python benchmarks/int4_wa_phases.py

Builds csrc/kernels/int4_gemm_wa.cu with -DCGK_WA_TIMING (thread 0 of CTA 0 sums the clock cycles between
the marked points of a step) into a temporary library and prints cycles per 128-k step for three shapes.
Needs nvcc and a B200.
"""
import ctypes, os, subprocess, sys, tempfile, torch
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from cogito_b200.quant.int4 import quantize_int4
from ctypes import c_void_p, c_int, c_longlong
tmp = tempfile.mkdtemp()
so = os.path.join(tmp, "libwa_timing.so")
subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
                       "-DCGK_WA_TIMING", f"-I{ROOT}/include", f"-I{ROOT}/csrc/kernels", f"{ROOT}/csrc/kernels/int4_gemm_wa.cu", f"{ROOT}/csrc/kernels/host_common.cu", "-o", so])
L = ctypes.CDLL(so)
L.cgk_int4_wa_tiles_bytes.restype = c_longlong
L.cgk_int4_wa_tile_weights.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
L.cgk_int4_wa_gemm.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
L.cgk_int4_wa_times.argtypes = [ctypes.POINTER(c_longlong)]
dev = "cuda"
lab = ["wait a_empty", "barrier", "convert+st issue", "x chunk+ldw", "ldx+st wait", "fences+arrive", "-", "-"]
for (M, K, N, splits) in [(16, 4096, 32000, 1), (80, 4096, 4096, 1), (16, 4096, 4096, 4)]:
    w = torch.randn(K, N, device=dev) * 0.02
    packed, scales = quantize_int4(w, 128)
    tiles = torch.empty(L.cgk_int4_wa_tiles_bytes(K, N), dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert L.cgk_int4_wa_tile_weights(packed.data_ptr(), scales.data_ptr(), K, N, 128, tiles.data_ptr(), st) == 0
    x = torch.randn(M, K, device=dev).bfloat16()
    acc = torch.zeros(M * N, dtype=torch.float32, device=dev)
    cnt = torch.zeros(4096, dtype=torch.int32, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    buf = (c_longlong * 8)()
    for it in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = L.cgk_int4_wa_gemm(x.data_ptr(), K, tiles.data_ptr(), acc.data_ptr(), cnt.data_ptr(), out.data_ptr(), N, None, M, N, K, splits, st)
        b.record(); torch.cuda.synchronize()
        assert rc == 0
    L.cgk_int4_wa_times(buf)
    steps = K // 128 // splits
    print(f"--- M{M} K{K} N{N} splits{splits}: event {a.elapsed_time(b)*1e3:.1f} us, {steps} steps; thread 0 of CTA 0, cycles per step")
    print("   " + ", ".join(f"{lab[i]} {buf[i]/steps:.0f}" for i in range(8)) + f"  | total {sum(buf)/steps:.0f}")
