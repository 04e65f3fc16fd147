"""tcgen05 GEMM vs a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.ops import functional as F
from geeps_b200.ops import _lib as L


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    Bm = b.float().t() if b_mn else b.float()
    return A @ Bm.t()


def _mk(rows, k, mn, dev, pad=0):
    shape = (k, rows + pad) if mn else (rows, k + pad)
    t = (torch.randn(shape, device=dev) * 0.5).to(torch.bfloat16)
    return t[:, :rows] if mn else t[:, :k]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 1024), (200, 136, 328), (64, 1000, 4096), (384, 96, 72)])
def test_gemm_tc_matches_fp32(M, N, K, a_mn, b_mn):
    dev = torch.device("cuda:0")
    torch.manual_seed(M * 7 + N * 3 + K)
    a = _mk(M, K, a_mn, dev, pad=8)
    b = _mk(N, K, b_mn, dev, pad=16)
    out = torch.empty((M, N), dtype=torch.float32, device=dev)
    st = L.new_status(dev)
    F.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, status=st, impl="tc")
    torch.cuda.synchronize()
    assert L.read_status(st)["code"] == 0, L.read_status(st)
    ref = _ref(a, b, a_mn, b_mn)
    assert torch.allclose(out, ref, atol=1e-2, rtol=1e-2), (out - ref).abs().max().item()


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tc_block_n_and_epilogue(bn):
    dev = torch.device("cuda:0")
    torch.manual_seed(bn)
    M, N, K = 300, 520, 448
    a = (torch.randn(M, K, device=dev) * 0.3).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * 0.3).to(torch.bfloat16)
    bias = torch.randn(N, device=dev)
    wide = torch.zeros((M, N + 24), dtype=torch.bfloat16, device=dev)
    out = wide[:, 8:8 + N]  # column slice of a wider matrix: exercises ldc and unaligned stores
    st = L.new_status(dev)
    F.gemm(a, b, out, bias=bias, relu=True, alpha=0.5, block_n=bn, status=st, impl="tc")
    torch.cuda.synchronize()
    assert L.read_status(st)["code"] == 0
    ref = torch.relu(0.5 * (a.float() @ b.float().t()) + bias)
    assert torch.allclose(out.float(), ref, atol=6e-2, rtol=2e-2)
    assert wide[:, :8].abs().max().item() == 0 and wide[:, 8 + N:].abs().max().item() == 0


def test_gemm_tc_beta_and_bias_m():
    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    M, N, K = 160, 264, 200
    a = (torch.randn(M, K, device=dev) * 0.3).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * 0.3).to(torch.bfloat16)
    bias = torch.randn(M, device=dev)
    c0 = torch.randn(M, N, device=dev)
    out = c0.clone()
    F.gemm(a, b, out, bias=bias, bias_mode=2, beta=0.75, impl="tc")
    ref = a.float() @ b.float().t() + 0.75 * c0 + bias[:, None]
    torch.cuda.synchronize()
    assert torch.allclose(out, ref, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("split", [0, 4])
def test_gemm_tc_split_k(split):
    dev = torch.device("cuda:0")
    torch.manual_seed(11)
    M, N, K = 96, 368, 8192  # weight-gradient shape: tiny output, very long K
    a = (torch.randn(K, M, device=dev) * 0.1).to(torch.bfloat16)   # stored [K, M]
    b = (torch.randn(K, N, device=dev) * 0.1).to(torch.bfloat16)   # stored [K, N]
    out = torch.full((M, N), 3.0, device=dev)
    F.gemm(a, b, out, a_mn=True, b_mn=True, beta=0.0, split_k=split, impl="tc")
    torch.cuda.synchronize()
    ref = a.float().t() @ b.float()
    assert torch.allclose(out, ref, atol=3e-2, rtol=1e-2)


def test_gemm_simt_matches_tc():
    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    M, N, K = 130, 77, 90
    a = (torch.randn(M, K, device=dev) * 0.3).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * 0.3).to(torch.bfloat16)
    out = torch.empty((M, N), dtype=torch.float32, device=dev)
    F.gemm(a, b, out, impl="auto")  # K=90 is not a multiple of 8: takes the SIMT path
    torch.cuda.synchronize()
    assert torch.allclose(out, a.float() @ b.float().t(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K,bn,fp32", [(512, 64, 256, 64, False), (512, 256, 256, 256, False),
                                           (1000, 384, 520, 0, False), (4096, 1000, 1024, 0, True)])
def test_gemm_cta_pair_matches_fp32(M, N, K, bn, fp32):
    """CTA-pair kernel (tcgen05 cta_group::2, 256-row tiles): bias + ReLU epilogue, ragged M / N / K edges."""
    dev = torch.device("cuda:0")
    torch.manual_seed(M + N + K)
    a = _mk(M, K, False, dev, pad=8)
    b = _mk(N, K, False, dev, pad=16)
    bias = torch.randn(N, device=dev)
    out = torch.full((M, N + 8), 7.0, dtype=torch.float32 if fp32 else torch.bfloat16, device=dev)[:, :N]
    st = L.new_status(dev)
    F.gemm(a, b, out, bias=bias, relu=True, block_n=bn, status=st, impl="pair")
    torch.cuda.synchronize()
    assert L.read_status(st)["code"] == 0, L.read_status(st)
    ref = torch.relu(_ref(a, b, False, False) + bias)
    assert ((out.float() - ref).norm() / ref.norm()).item() < (1e-5 if fp32 else 5e-3)


def test_gemm_auto_dispatch_uses_pairs_for_large_products():
    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    M, N, K = 20000, 512, 192
    a, b = _mk(M, K, False, dev), _mk(N, K, False, dev)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    F.gemm(a, b, out)
    ref = _ref(a, b, False, False)
    assert ((out.float() - ref).norm() / ref.norm()).item() < 5e-3
