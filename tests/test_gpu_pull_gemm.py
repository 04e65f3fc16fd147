"""Fused pull + GEMM kernel on one GPU: the shards' weight rows are separate allocations (on one GPU a
"peer" pointer is just another local pointer), checked against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.ops import functional as F
from geeps_b200.ops import _lib as L

BF = torch.bfloat16


@pytest.mark.parametrize("M,N,K,shards,bn", [(256, 4096, 1024, 4, 0), (100, 1000, 512, 3, 32), (256, 520, 256, 8, 64),
                                             (32, 21841, 1024, 8, 0)])
def test_pull_gemm_matches_reference(M, N, K, shards, bn):
    dev = torch.device("cuda:0")
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device=dev) * 0.3).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    bias = torch.randn(N, device=dev)
    per = (N + shards - 1) // shards
    n_start = [min(s * per, N) for s in range(shards)]
    parts = [w[n_start[s]:(n_start[s + 1] if s + 1 < shards else N)].clone() for s in range(shards)]
    ready = torch.full((shards,), 5, dtype=torch.int32, device=dev)
    w_local = torch.zeros_like(w)
    n_pad = (N + 7) // 8 * 8
    out = torch.zeros(M, n_pad, dtype=torch.float32, device=dev)[:, :N]
    st = L.new_status(dev)
    F.pull_gemm(x, [t.data_ptr() if t.numel() else 0 for t in parts], n_start, out, ldw=K, bias=bias, relu=True,
                ready_ptrs=[ready.data_ptr() + 4 * s for s in range(shards)], needed_stamp=5, w_local=w_local, status=st,
                block_n=bn)
    torch.cuda.synchronize()
    assert L.read_status(st)["code"] == 0, L.read_status(st)
    ref = torch.relu(x.float() @ w.float().t() + bias)
    assert torch.allclose(out, ref, atol=2e-2, rtol=1e-2), (out - ref).abs().max().item()
    assert torch.equal(w_local, w)          # the pulled rows also landed in the local cache


def test_pull_gemm_wait_times_out_cleanly():
    dev = torch.device("cuda:0")
    x = torch.zeros(64, 128, dtype=BF, device=dev)
    w = torch.zeros(64, 128, dtype=BF, device=dev)
    ready = torch.zeros(1, dtype=torch.int32, device=dev)     # never reaches the stamp
    out = torch.zeros(64, 64, dtype=torch.float32, device=dev)
    st = L.new_status(dev)
    F.pull_gemm(x, [w.data_ptr()], [0], out, ldw=128, ready_ptrs=[ready.data_ptr()], needed_stamp=3, status=st,
                wait_budget_ns=100_000_000)
    torch.cuda.synchronize()
    s = L.read_status(st)
    assert s["name"] == "timeout" and s["kernel"] == 22
    assert float(torch.ones(3, device=dev).sum()) == 3.0      # context still usable
