"""The cg_cuda_* device layer of the C API in host mode (no GPU): the same calls and the same
checks as on a B200, computed by the host implementations, as the reference's tests/test_cuda.c
runs against its simulation build."""
import os

import pytest

import capi_device_cases as c1
import capi_device_cases2 as c2


@pytest.fixture(scope="module")
def lib():
    lib = c1.D()
    lib.cg_cuda_shutdown()
    os.environ["COGITO_FORCE_HOST"] = "1"            # read by cg_cuda_init: host mode even where a GPU is present
    try:
        c1.case_bringup(lib, expect_device=False)
    finally:
        del os.environ["COGITO_FORCE_HOST"]
    yield lib
    lib.cg_cuda_shutdown()


@pytest.fixture(autouse=True)
def _fresh_error_state(lib):
    lib.cg_last_error()          # reading clears it: an error left by an earlier test of the same process is not this test's
    yield


def test_memory_round_trip(lib):
    c1.case_memory(lib)


def test_elementwise_and_errors(lib):
    c1.case_elementwise(lib, expect_device=False)


def test_reductions(lib):
    c1.case_reductions(lib)


def test_matmul_bmm_transpose(lib):
    c2.case_matmul(lib, expect_device=False)


def test_activations_and_gradients(lib):
    c2.case_activations(lib)


def test_softmax_any_axis(lib):
    c2.case_softmax(lib)


def test_layernorm_rmsnorm(lib):
    c2.case_norms(lib)


def test_attention_gqa_window_paged_backward(lib):
    c2.case_attention(lib, expect_device=False)


def test_rope_and_tile_helpers(lib):
    c2.case_rope(lib)


def test_python_binding_of_the_device_layer(lib):
    import numpy as np
    from capi_defs import cg
    a = cg.Tensor.from_numpy(np.arange(6, dtype=np.float32).reshape(2, 3))
    b = cg.Tensor.from_numpy(np.ones((3, 4), dtype=np.float32))
    da, db = a.cuda(), b.cuda()
    assert not cg.device_mode() and not da.is_cuda               # host mode in this test
    out = da.device_matmul(db).cpu()
    np.testing.assert_allclose(out.numpy(), a.numpy() @ b.numpy())


def test_shutdown_and_reinit(lib):
    lib.cg_cuda_shutdown()
    assert not lib.cg_cuda_is_available()
    assert lib.cg_cuda_init() and lib.cg_cuda_is_available()
