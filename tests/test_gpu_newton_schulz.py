"""The tensor-core matrix product behind Newton-Schulz (``pylo_b200_gemm_tn_3xtf32``) and the iteration built on it.

The reference runs ``orthogonalize_via_newton_schulz`` (CELO2_naive.py:59-73) as fp32 ``torch.matmul``.  The kernel
here evaluates the same products from TF32 high / low parts of the operands; the checks are against fp64:

* the product itself, on exact-tile, ragged, batched and strided cases with the scaled addition, must be as
  accurate as an fp32 product (error measured against sum_k |a| |b|);
* the whole iteration must end as close to its fp64 evaluation as the fp32 ``torch.matmul`` chain does;
* the CELO2 classes with ``ns_precision="3xtf32"`` must stay inside the usual parity bounds against the oracle.
"""

import pytest
import torch

import cases
import cuda_util as CU

pytestmark = pytest.mark.gpu

COEFFS = (3.4445, -4.7750, 2.0315)


def _gemm(A, B, D=None, alpha=1.0, beta=0.0):
    from pylo_b200.optim._common import _gemm_tn

    C = torch.full((A.shape[0], A.shape[1], B.shape[1]), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _gemm_tn(A, B, C, D, alpha, beta, status, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    return C


# (batch, M, N, K): one exact tile; several tiles; ragged edges in every dimension; a K tail; a batch of small ones
GEMM_SHAPES = [(1, 128, 256, 32), (1, 256, 512, 128), (1, 100, 260, 36), (2, 300, 200, 1000), (3, 64, 64, 68),
               (1, 768, 768, 3072), (5, 132, 4, 8)]


@pytest.mark.parametrize("shape", GEMM_SHAPES)
@pytest.mark.parametrize("with_d", [False, True])
def test_product_is_fp32_faithful(shape, with_d):
    nb, M, N, K = shape
    gen = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    A = torch.randn(nb, M, K, device="cuda", generator=gen) * 3.0
    B = torch.rand(nb, N, K, device="cuda", generator=gen) - 0.5
    D = torch.randn(nb, M, N, device="cuda", generator=gen) if with_d else None
    alpha, beta = (-4.775, 2.0315) if with_d else (1.0, 0.0)
    got = _gemm(A, B, D, alpha, beta).double()
    exact = alpha * (A.double() @ B.double().transpose(1, 2)) + (beta * D.double() if with_d else 0.0)
    mag = abs(alpha) * (A.abs().double() @ B.abs().double().transpose(1, 2)) + (abs(beta) * D.abs().double() if with_d else 0.0)
    err = float(((got - exact).abs() / mag).max())
    ref32 = alpha * (A @ B.transpose(1, 2)) + (beta * D if with_d else 0.0)
    err32 = float(((ref32.double() - exact).abs() / mag).max())
    CU.log_parity(f"gemm{shape}{'+D' if with_d else ''}", err=err, torch_fp32=err32)
    assert torch.isfinite(got).all()
    assert err < 1e-6 and err < 8 * max(err32, 6e-8), (err, err32)


def test_product_takes_strided_views():
    """Row pitches and batch strides larger than the matrices (views into bigger buffers)."""
    gen = torch.Generator(device="cuda").manual_seed(3)
    bufA = torch.randn(2, 160, 80, device="cuda", generator=gen)
    bufB = torch.randn(2, 300, 80, device="cuda", generator=gen)
    A, B = bufA[:, :132, :64], bufB[:, :260, :64]
    got = _gemm(A, B).double()
    exact = A.double() @ B.double().transpose(1, 2)
    assert float((got - exact).abs().max()) < 1e-4


def test_product_rejects_what_it_cannot_take():
    from pylo_b200 import _lib as L
    from pylo_b200.optim._common import _gemm_tn

    s = torch.cuda.current_stream().cuda_stream
    A = torch.zeros(1, 8, 6, device="cuda")   # K = 6 is not a multiple of 4
    C = torch.zeros(1, 8, 8, device="cuda")
    with pytest.raises(L.PyloLibError):
        _gemm_tn(A, A, C, None, 1.0, 0.0, None, s)
    A = torch.zeros(1, 8, 8, device="cuda")
    with pytest.raises(L.PyloLibError):
        _gemm_tn(A, A, C, C, 1.0, 1.0, None, s)   # D must not be C


@pytest.mark.parametrize("shape", [(768, 2304), (1024, 1024), (300, 200), (3, 128, 96), (2304, 768), (4096, 4096)])
def test_iteration_is_as_accurate_as_fp32_matmul(shape):
    from pylo_b200.optim._common import newton_schulz, newton_schulz_tc

    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(shape, device="cuda", generator=gen)
    if len(shape) == 2 and shape[0] == shape[1]:
        x = x * torch.exp(-7 + torch.randn(shape[0], 1, device="cuda", generator=gen))  # badly conditioned rows
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    exact = newton_schulz(x.double(), COEFFS)
    e32 = float((newton_schulz(x, COEFFS).double() - exact).norm() / exact.norm())
    etc = float((newton_schulz_tc(x, COEFFS, status=status).double() - exact).norm() / exact.norm())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    CU.log_parity(f"newton_schulz{shape}", tensor_cores=etc, torch_fp32=e32)
    assert etc < max(4 * e32, 2e-5), (etc, e32)


@pytest.mark.parametrize("family", ["celo2", "elo_celo2"])
def test_classes_with_tensor_core_newton_schulz_match_oracle(family):
    from test_gpu_config_sizes import HP, _assert_bounds, _run_both

    case = dict(shapes=[(256, 384), (384,), (128, 64), (3, 64, 96)], init_seed=3, init_scale=0.02, grad_seed=4, grad_scale=1e-3)
    hp = dict(HP[family], ns_precision="3xtf32")
    got, want, init, opt, _ = _run_both(family, case, 3, [1, 3], hp=hp)
    assert opt.extra_launches > 0, "no matrix took the tensor-core Newton-Schulz"
    _assert_bounds(f"ns_classes[{family}]", got, want, init)


@pytest.mark.parametrize("r,k,nb", [(256, 64, 1), (300, 1000, 2), (1000, 36, 1), (4096, 256, 1), (132, 8, 3)])
def test_symmetric_product_equals_the_full_one(r, k, nb):
    """x x^T computed on the tiles on and above the diagonal and mirrored must equal the product computed in full,
    bit for bit above the diagonal and as its exact mirror image below."""
    from pylo_b200.optim._common import _gemm_tn

    gen = torch.Generator(device="cuda").manual_seed(r + k)
    x = torch.randn(nb, r, k, device="cuda", generator=gen)
    d = torch.randn(nb, r, r, device="cuda", generator=gen)
    d = d + d.transpose(1, 2)
    s = torch.cuda.current_stream().cuda_stream
    full = torch.empty(nb, r, r, device="cuda")
    half = torch.full((nb, r, r), float("nan"), device="cuda")
    _gemm_tn(x, x, full, d, 2.0, -0.5, None, s)
    _gemm_tn(x, x, half, d, 2.0, -0.5, None, s, symmetric=True)
    torch.cuda.synchronize()
    assert torch.isfinite(half).all()
    assert torch.equal(torch.triu(half), torch.triu(full))
    assert torch.equal(half, half.transpose(1, 2))


def test_transpose_kernel():
    from pylo_b200.optim._common import _transpose

    gen = torch.Generator(device="cuda").manual_seed(9)
    for shape in [(1, 32, 32), (3, 100, 260), (2, 768, 2304), (1, 5, 4100)]:
        x = torch.randn(shape, device="cuda", generator=gen)
        out = torch.full((shape[0], shape[2], shape[1]), float("nan"), device="cuda")
        _transpose(x, out, torch.cuda.current_stream().cuda_stream)
        assert torch.equal(out, x.transpose(1, 2))
