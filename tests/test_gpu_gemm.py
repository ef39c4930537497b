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


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("nb,M,N,K", [(3, 200, 136, 96), (4, 16, 264, 304), (2, 304, 16, 16), (5, 128, 128, 32)])
def test_bf16_gemm_strided_batches(nb, M, N, K, a_mn, b_mn):
    """One launch for all batches, each with its own A and B (any operand order), against per-batch fp32 products;
    includes inner and outer dimensions far below a tile (zero-filled by TMA)."""
    from pom_b200 import _abi, ops

    torch.manual_seed(2)
    A = torch.randn(nb, M, K, device="cuda").bfloat16()
    B = torch.randn(nb, N, K, device="cuda").bfloat16()
    ref = torch.matmul(A.float(), B.float().transpose(1, 2))
    a = A.transpose(1, 2).contiguous() if a_mn else A
    b = B.transpose(1, 2).contiguous() if b_mn else B
    out = ops.gemm_batched(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert _abi.read_status("cuda") == 0
    assert _rel(out, ref) < 1e-5
    out16 = ops.gemm_batched(a, b, a_mn=a_mn, b_mn=b_mn)
    assert _rel(out16, ref) < 4e-3
    shared = ops.gemm_batched(a, b[0], a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)  # one B for all batches
    assert _rel(shared, torch.matmul(A.float(), B[0].float().t())) < 1e-5


def test_bf16_gemm_batches_as_column_blocks_of_wider_matrices():
    """Heads that sit side by side inside (rows, heads * hd) matrices, passed as strided views: per-head products
    written into / accumulated onto column blocks of a wider output."""
    from pom_b200 import ops

    torch.manual_seed(3)
    rows, heads, hd, D = 24, 4, 40, 72
    H = torch.randn(rows, heads * hd, device="cuda").bfloat16()
    W = torch.randn(D, heads * hd, device="cuda").bfloat16()
    Mb = torch.empty(rows, heads, D, device="cuda", dtype=torch.bfloat16)
    ops.gemm_batched(H.view(rows, heads, hd).transpose(0, 1), W.view(D, heads, hd).transpose(0, 1),
                     out=Mb.transpose(0, 1))
    ref = torch.einsum("bhj,dhj->bhd", H.float().view(rows, heads, hd), W.float().view(D, heads, hd))
    assert _rel(Mb, ref) < 4e-3
    # accumulate onto column blocks: acc[d, h*hd + j] += sum_b G[b, h, d] * H[b, h*hd + j]
    G = torch.randn(rows, heads, D, device="cuda").bfloat16()
    acc = torch.ones(D, heads * hd, device="cuda")
    ops.gemm_batched(G.transpose(0, 1), H.view(rows, heads, hd).transpose(0, 1), a_mn=True, b_mn=True,
                     out=acc.view(D, heads, hd).transpose(0, 1), accumulate=True)
    ref2 = 1.0 + torch.einsum("bhd,bhj->dhj", G.float(), H.float().view(rows, heads, hd)).reshape(D, heads * hd)
    assert _rel(acc, ref2) < 1e-5
