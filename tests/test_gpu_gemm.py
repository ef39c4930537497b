"""tcgen05 GEMM engine and fp32 SIMT GEMM against a plain PyTorch fp32 matmul of the same operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm()).item()


SHAPES = [(128, 128, 64), (128, 256, 64), (512, 512, 512), (384, 1152, 320), (200, 136, 96), (1000, 264, 72),
          (2048, 2304, 1152)]


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_bf16_gemm_all_operand_orders(M, N, K, a_mn, b_mn):
    from pom_b200 import _abi, ops

    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(N, K, device="cuda").bfloat16()
    ref = A.float() @ B.float().t()
    out = ops.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, a_mn=a_mn, b_mn=b_mn,
                   out_dtype=torch.float32)
    assert _abi.read_status("cuda") == 0
    assert _rel(out, ref) < 1e-5          # fp32 accumulation of exact bf16 products
    out16 = ops.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, a_mn=a_mn, b_mn=b_mn)
    assert _rel(out16, ref) < 4e-3        # one bf16 rounding of the result


@pytest.mark.parametrize("split_k", [0, 1, 3, 8])
def test_bf16_gemm_split_k_accumulates(split_k):
    from pom_b200 import ops

    torch.manual_seed(1)
    M, N, K = 1152, 520, 4096
    A = torch.randn(K, M, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    base = torch.randn(M, N, device="cuda")
    out = base.clone()
    ops.gemm(A, B, a_mn=True, b_mn=True, out=out, accumulate=True, split_k=split_k)
    ref = base + A.float().t() @ B.float()
    assert _rel(out, ref) < 1e-5


def test_bf16_gemm_rejects_misaligned_leading_dimension():
    from pom_b200 import ops
    from pom_b200._abi import PomError

    A = torch.randn(64, 100, device="cuda").bfloat16()[:, :99]
    B = torch.randn(64, 100, device="cuda").bfloat16()[:, :99]
    with pytest.raises((PomError, ValueError)):
        ops.gemm(A, B)


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,K", [(64, 64, 16), (130, 67, 45), (512, 96, 300)])
def test_fp32_gemm(M, N, K, a_mn, b_mn):
    from pom_b200 import ops

    torch.manual_seed(2)
    A = torch.randn(M, K, device="cuda")
    B = torch.randn(N, K, device="cuda")
    out = ops.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, a_mn=a_mn, b_mn=b_mn)
    assert _rel(out, A.double() @ B.double().t()) < 1e-6


def test_bf16_gemm_gelu_and_residual_epilogue():
    """The feed-forward epilogue options: exact GELU, then a bf16 residual add."""
    from pom_b200 import ops

    torch.manual_seed(3)
    M, N, K = 520, 392, 264
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    R = torch.randn(M, N, device="cuda").bfloat16()
    acc = A.float() @ B.float().t()
    got = ops.gemm(A, B, act="gelu")
    assert _rel(got, torch.nn.functional.gelu(acc)) < 4e-3
    got = ops.gemm(A, B, residual=R)
    assert _rel(got, acc + R.float()) < 4e-3
    got = ops.gemm(A, B, act="gelu", residual=R)
    assert _rel(got, torch.nn.functional.gelu(acc) + R.float()) < 4e-3
