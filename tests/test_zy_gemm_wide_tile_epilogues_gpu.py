"""GEMM epilogues on the widest tile (128 x 256), where outputs leave as bulk tensor stores from the
epilogue's staging tiles and one input may arrive by bulk loads: shapes large enough for the launcher to
pick that tile, with ragged row and column counts, strided outputs and both bias types, against the fp32
restatement of the same formula."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def relerr(x, ref):
    x, ref = x.float(), ref.float()
    return ((x - ref).abs().max() / (ref.abs().max() + 1e-6)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    from cogito_b200.ops import _lib
    yield
    _lib.assert_device_ok()


def _operands(M, N, K, seed=0):
    torch.manual_seed(seed)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    return a, b


@pytest.mark.parametrize("M,N", [(4096, 1024), (4000, 1000), (4104, 1016)])
@pytest.mark.parametrize("bias_dtype", [torch.bfloat16, torch.float32])
def test_bias_activation_pre_activation_and_residual(M, N, bias_dtype):
    from cogito_b200.ops.gemm import gemm, gemm_reference
    K = 256
    a, b = _operands(M, N, K)
    bias = torch.randn(N, device=DEV).to(bias_dtype)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    aux = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, act="gelu", residual=res, aux_out=aux)
    ref, raux = gemm_reference(a, b, bias=bias, act="gelu", residual=res, want_aux=True, out_dtype=torch.float32)
    assert relerr(out, ref) < 1e-2 and relerr(aux, raux) < 1e-2
    # bias alone and bias + residual (the residual then comes through the staging tile)
    assert relerr(gemm(a, b, bias=bias), gemm_reference(a, b, bias=bias, out_dtype=torch.float32)) < 1e-2
    assert relerr(gemm(a, b, bias=bias, residual=res),
                  gemm_reference(a, b, bias=bias, residual=res, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("M,N", [(4096, 1024), (4000, 1000)])
@pytest.mark.parametrize("act", ["gelu", "silu", "relu"])
def test_activation_derivative_operand(M, N, act):
    from cogito_b200.ops.gemm import gemm, gemm_reference
    a, b = _operands(M, N, 256, seed=1)
    auxin = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    assert relerr(gemm(a, b, aux_in=auxin, dact=act),
                  gemm_reference(a, b, aux_in=auxin, dact=act, out_dtype=torch.float32)) < 1e-2
    assert relerr(gemm(a, b, aux_in=auxin, dact=act, residual=res),
                  gemm_reference(a, b, aux_in=auxin, dact=act, residual=res, out_dtype=torch.float32)) < 1e-2


def test_strided_output_keeps_its_neighbours():
    """The output is a column slice of a wider matrix: the stores are clipped at the slice's last column."""
    from cogito_b200.ops.gemm import gemm, gemm_reference
    M, N, K = 4096, 1000, 256
    a, b = _operands(M, N, K, seed=2)
    wide = torch.full((M, N + 72), 7.0, device=DEV, dtype=torch.bfloat16)
    out = wide[:, :N]
    gemm(a, b, out=out)
    assert relerr(out, gemm_reference(a, b, out_dtype=torch.float32)) < 1e-2
    assert torch.all(wide[:, N:] == 7.0)


def test_b_operand_with_the_reduction_dimension_outermost():
    """dX = dY W with W stored [out, in]: the B operand is read with its N dimension contiguous."""
    from cogito_b200.ops.gemm import gemm, gemm_reference
    torch.manual_seed(3)
    M, K, N = 4096, 256, 1024
    dy = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(K, N, device=DEV, dtype=torch.bfloat16) * 0.1
    auxin = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    assert relerr(gemm(dy, w, b_mn=True, aux_in=auxin, dact="gelu"),
                  gemm_reference(dy, w, b_mn=True, aux_in=auxin, dact="gelu", out_dtype=torch.float32)) < 1e-2
