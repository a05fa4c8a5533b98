"""Checkpoint format against the reference's own writer, and round trips of every tensor type.

The reference's ``src/core/serialization.c`` is compiled unchanged (with ``<stdint.h>`` supplied on
the command line, the one header it forgets) into a tiny program that saves two tensors; the file
it writes must load byte for byte through ``cg_load_model`` of this library and through
``cogito_b200.io.checkpoint``.  Skipped where the reference sources are not present.
"""
import os
import shutil
import subprocess
from ctypes import POINTER, byref, c_char_p, c_int

import numpy as np
import pytest
import torch

from capi_defs import L, T, TensorP, borrowed
from cogito_b200.io import checkpoint as ckpt

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("COGITO_REFERENCE_DIR", os.path.join(os.path.dirname(REPO), "reference"))

WRITER_MAIN = r"""
#include "cg_serialization.h"
#include <string.h>
/* the reference's loader, in the same file, wants the tensor constructor; the writer does not use it */
cg_tensor* cg_tensor_new(int* shape, int ndim, bool requires_grad) { (void)shape; (void)ndim; (void)requires_grad; return 0; }
int main(int argc, char** argv) {
  static float wdata[12], bdata[3];
  for (int i = 0; i < 12; ++i) wdata[i] = 0.25f * (float)i - 1.0f;
  bdata[0] = 3.5f; bdata[1] = -7.0f; bdata[2] = 1e-3f;
  cg_tensor w, b;
  memset(&w, 0, sizeof(w)); memset(&b, 0, sizeof(b));
  w.data = wdata; w.ndim = 2; w.shape[0] = 3; w.shape[1] = 4; w.size = 12;
  b.data = bdata; b.ndim = 1; b.shape[0] = 3; b.size = 3;
  cg_tensor* ts[2] = {&w, &b};
  const char* names[2] = {"encoder.layer0.weight", "encoder.layer0.bias"};
  cg_save_model(argv[1], ts, names, 2);
  return 0;
}
"""


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE, "src", "core", "serialization.c")) or shutil.which("gcc") is None,
                    reason="reference sources or gcc not available")
def test_file_written_by_the_reference_writer_loads_here(tmp_path):
    main_c = tmp_path / "writer_main.c"
    main_c.write_text(WRITER_MAIN)
    exe = tmp_path / "ref_writer"
    subprocess.run(["gcc", "-std=gnu11", "-O1", "-include", "stdint.h", "-include", "stdbool.h", "-I", os.path.join(REFERENCE, "include"),
                    os.path.join(REFERENCE, "src", "core", "serialization.c"), str(main_c), "-o", str(exe)], check=True,
                   capture_output=True)
    path = tmp_path / "ref.cog"
    subprocess.run([str(exe), str(path)], check=True)
    raw = path.read_bytes()
    assert raw[:4] == bytes([0x31, 0x47, 0x4F, 0x43]) and len(raw) == 24 + 2 * 120 + 48 + 12
    want_w = (0.25 * np.arange(12, dtype=np.float32) - 1.0).reshape(3, 4)
    want_b = np.array([3.5, -7.0, 1e-3], np.float32)
    # Python reader
    got = ckpt.load_tensors(str(path))
    assert list(got) == ["encoder.layer0.weight", "encoder.layer0.bias"]
    assert np.array_equal(got["encoder.layer0.weight"].numpy(), want_w) and np.array_equal(got["encoder.layer0.bias"].numpy(), want_b)
    # C reader of this library
    lib = L()
    ts, ns, n = POINTER(TensorP)(), POINTER(c_char_p)(), c_int()
    lib.cg_load_model(str(path).encode(), byref(ts), byref(ns), byref(n))
    assert n.value == 2 and ns[0] == b"encoder.layer0.weight" and ns[1] == b"encoder.layer0.bias"
    assert np.array_equal(borrowed(ts[0]), want_w) and np.array_equal(borrowed(ts[1]), want_b)
    # and the other way round: the payload bytes this library writes for the same tensors are the same
    mine = tmp_path / "mine.cog"
    tw, tb = T(want_w), T(want_b)                      # keep the wrappers alive across the call
    lib.cg_save_model(str(mine).encode(), (TensorP * 2)(tw._ptr, tb._ptr),
                      (c_char_p * 2)(b"encoder.layer0.weight", b"encoder.layer0.bias"), 2)
    mraw = mine.read_bytes()
    assert mraw[24 + 240:] == raw[24 + 240:] and mraw[:12] == raw[:12]
    assert mraw[24:24 + 240] == raw[24:24 + 240]          # directory entries are memset-zero padded in both


def test_zero_dim_zero_size_and_integer_tensors_round_trip(tmp_path):
    p = str(tmp_path / "t.cog")
    big = torch.tensor([2 ** 40 + 1, -3], dtype=torch.int64)
    src = {"scalar": torch.tensor(3.0), "empty": torch.zeros(0, 5), "count": big, "steps": torch.tensor(7, dtype=torch.int64),
           "mask": torch.tensor([True, False, True]), "bytes": torch.arange(6, dtype=torch.uint8).view(2, 3),
           "h": torch.tensor([0.5, -2.0, 65504.0], dtype=torch.float16), "d": torch.tensor([1e-300], dtype=torch.float64),
           "i32": torch.tensor([[1, -2]], dtype=torch.int32), "w16": torch.randn(3, 2).bfloat16()}
    ckpt.save_tensors(p, src)
    back = ckpt.load_tensors(p)
    for k, v in src.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape and torch.equal(back[k], v), k
    assert not hasattr(back["bytes"], "logical_shape")
    with pytest.raises(TypeError):
        ckpt.save_tensors(p, {"c": torch.zeros(2, dtype=torch.complex64)})
    # a module with an integer buffer (BatchNorm's num_batches_tracked) saves and loads
    bn = torch.nn.BatchNorm1d(4)
    bn(torch.randn(8, 4))
    ckpt.save_model(p, bn)
    bn2 = torch.nn.BatchNorm1d(4)
    ckpt.load_model(p, bn2)
    assert int(bn2.num_batches_tracked) == 1 and torch.equal(bn2.running_mean, bn.running_mean)


def test_c_loader_reads_python_written_int4_and_integer_entries(tmp_path):
    from cogito_b200.quant.int4 import dequantize_int4, quantize_int4
    torch.manual_seed(0)
    w = torch.randn(16, 32)
    packed, scales = quantize_int4(w, group=128)
    p = str(tmp_path / "q.cog")
    ckpt.save_tensors(p, {"norm": torch.ones(4), "proj": packed, "proj.scales": scales, "step": torch.tensor([9], dtype=torch.int64),
                          "half": torch.tensor([0.5, -3.0], dtype=torch.float16)}, int4_shapes={"proj": (16, 32)})
    lib = L()
    ts, ns, n = POINTER(TensorP)(), POINTER(c_char_p)(), c_int()
    lib.cg_load_model(p.encode(), byref(ts), byref(ns), byref(n))
    assert n.value == 5 and [ns[i] for i in range(5)] == [b"norm", b"proj", b"proj.scales", b"step", b"half"]
    want = dequantize_int4(packed, scales, 16 * 32, 128).view(16, 32).numpy()
    assert borrowed(ts[1]).shape == (16, 32) and np.allclose(borrowed(ts[1]), want, atol=0, rtol=0)
    assert borrowed(ts[3]).tolist() == [9.0] and borrowed(ts[4]).tolist() == [0.5, -3.0] and borrowed(ts[0]).sum() == 4
