"""The cg_cuda_* device layer of the C API on a B200: libcogito.so opens the kernel library at run
time, device tensors hold device memory and every operation launches sm_100a kernels (the
tcgen05 GEMM for matmul / bmm, the flash kernels for attention).  Same cases as the host-mode
test, compared against numpy."""
import os

import pytest

import capi_device_cases as c1
import capi_device_cases2 as c2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = c1.D()
    lib.cg_cuda_shutdown()
    os.environ.pop("COGITO_FORCE_HOST", None)
    c1.case_bringup(lib, expect_device=True)           # fails loudly when the kernel library did not load
    yield lib
    lib.cg_cuda_shutdown()


@pytest.fixture(autouse=True)
def _fresh_error_state(lib):
    lib.cg_last_error()          # reading clears it: an error left by an earlier test of the same process is not this test's
    yield


def test_memory_round_trip(lib):
    c1.case_memory(lib)


def test_elementwise_and_errors(lib):
    c1.case_elementwise(lib, expect_device=True)


def test_reductions(lib):
    c1.case_reductions(lib)


def test_matmul_bmm_transpose(lib):
    c2.case_matmul(lib, expect_device=True)


def test_activations_and_gradients(lib):
    c2.case_activations(lib)


def test_softmax_any_axis(lib):
    c2.case_softmax(lib)


def test_layernorm_rmsnorm(lib):
    c2.case_norms(lib)


def test_attention_gqa_window_paged_backward(lib):
    c2.case_attention(lib, expect_device=True)


def test_rope_and_tile_helpers(lib):
    c2.case_rope(lib)
