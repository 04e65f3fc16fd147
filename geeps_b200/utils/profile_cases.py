"""Small, self-terminating workloads for `ncu` captures: python -m geeps_b200.utils.profile_cases <case>

Each case allocates well under 1 GB (but more than the 126 MB L2 where DRAM figures matter), warms up
once and launches the kernel of interest three times.
  gemm        conv3-forward-shaped bf16 GEMM (M=43264, N=384, K=2304), tcgen05 kernel
  gemm_dgrad  conv3 data-gradient shape (small K, MN-major B, output-heavy)
  gemm_fc6    fully-connected forward at batch 256 (M=256, N=4096, K=9216): weight-streaming bound
  gemm_pair   8192^3 on the CTA-pair kernel (tcgen05 cta_group::2)
  maxpool     3x3 stride-2 max pooling forward + backward on a conv1-sized activation (256 x 55 x 55 x 96)
  push_apply  fused reduce + momentum-SGD apply + publish over a 256 MB table (1 rank)
  lrn         LRN forward + backward on a conv1-sized activation
  lrn_pool    LRN fused with the 3x3 stride-2 max pooling after it, forward + backward (256 x 55 x 55 x 96)
  pull_gemm   fused pull + GEMM on an fc6-shaped layer (4 local shards)
  conv_fwd / conv_dgrad / conv_wgrad   implicit-GEMM convolution, conv3 shape (256 x 13 x 13, 256 -> 384, 3x3)
  conv1_fwd   AlexNet conv1 after space-to-depth (256 x 57 x 57 x 64 (48 + 16 zero) -> 96, 3x3, no padding);
              routed to the halo-tile kernel, like conv2_fwd / conv2_dgrad (GEEPS_HALO_CONV=0: the box kernel)
  conv2_fwd / conv2_dgrad   one group of AlexNet conv2 (256 x 27 x 27, 48 of 96 -> 128 of 256 channels, 5x5)
  conv1_wgrad / conv2_wgrad   the weight gradients of the same two layers (filter-row kernel, conv_wgrad_halo.cu)
"""
from __future__ import annotations

import ctypes as C
import sys

import torch

from ..ops import _lib as L
from ..ops import functional as F

BF = torch.bfloat16


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    dev = torch.device("cuda")
    if case in ("gemm", "gemm_dgrad"):
        M, N, K, b_mn = (43264, 384, 2304, False) if case == "gemm" else (43264, 2304, 384, True)
        a = (torch.randn(M, K, device=dev) * 0.1).to(BF)
        b = (torch.randn((K, N) if b_mn else (N, K), device=dev) * 0.1).to(BF)
        out = torch.empty(M, N, dtype=BF, device=dev)
        for _ in range(4):
            F.gemm(a, b, out, b_mn=b_mn)
    elif case == "gemm_fc6":
        M, N, K = 256, 4096, 9216
        a = (torch.randn(M, K, device=dev) * 0.1).to(BF)
        b = (torch.randn(N, K, device=dev) * 0.1).to(BF)
        bias = torch.zeros(N, device=dev)
        out = torch.empty(M, N, dtype=BF, device=dev)
        for _ in range(4):
            F.gemm(a, b, out, bias=bias, relu=True)
    elif case == "gemm_pair":
        M = N = K = 8192
        a = (torch.randn(M, K, device=dev) * 0.1).to(BF)
        b = (torch.randn(N, K, device=dev) * 0.1).to(BF)
        out = torch.empty(M, N, dtype=BF, device=dev)
        for _ in range(3):
            F.gemm(a, b, out)
    elif case == "maxpool":
        B, H, Cc = 256, 55, 96
        x = torch.randn(B, H, H, Cc, device=dev).to(BF)
        g = F.pool_geom(x.shape, 3, 2, 0, Cc, Cc)
        y = torch.empty(B, g.OH, g.OW, Cc, dtype=BF, device=dev)
        arg = torch.empty(B, g.OH, g.OW, Cc, dtype=torch.uint8, device=dev)
        dx = torch.empty_like(x)
        for _ in range(3):
            F.maxpool_forward(x, y, arg, g)
            F.maxpool_backward(y, arg, dx, g)
    elif case == "push_apply":
        rows = 512 * 1024          # 256 MB table
        upd = torch.randn(rows, 128, device=dev) * 0.01
        master = torch.zeros(rows, 128, device=dev)
        mom = torch.zeros(rows, 128, device=dev)
        cache = torch.zeros(rows, 128, device=dev)
        cache16 = torch.zeros(rows, 128, dtype=BF, device=dev)
        flags = torch.zeros(64, dtype=torch.int32, device=dev)
        p = L.PushApplyParams()
        p.upd[0], p.cache[0], p.cache16[0] = upd.data_ptr(), cache.data_ptr(), cache16.data_ptr()
        p.data_age[0] = flags.data_ptr() + 32
        p.master, p.momentum = master.data_ptr(), mom.data_ptr()
        p.push_ready, p.global_clock, p.cta_counter = None, flags.data_ptr() + 64, flags.data_ptr() + 68
        p.status = None
        p.n_owned, p.row_start, p.row_stride, p.total_rows = rows, 0, 1, rows
        p.wait_budget_ns, p.n_ranks, p.rank, p.mode, p.publish = 10 ** 9, 1, 0, 1, 1
        p.lr, p.momentum_coef, p.weight_decay, p.grad_scale = 0.01, 0.9, 5e-4, 1.0
        for i in range(4):
            p.clock_stamp = i + 1
            L.check(L.lib().geeps_ps_push_apply(C.byref(p), 0, L.stream_ptr()), "push_apply")
    elif case == "lrn":
        P, Cc = 256 * 55 * 55, 96
        x = torch.randn(P, Cc, device=dev).to(BF)
        y = torch.empty_like(x); dx = torch.empty_like(x)
        scale = torch.empty(P, Cc, dtype=BF, device=dev)
        for _ in range(4):
            F.lrn_forward(x, y, scale)
            F.lrn_backward(x, y, scale, y, dx)
    elif case == "lrn_pool":
        B, H, Cc = 256, 55, 96
        x = torch.relu(torch.randn(B, H, H, Cc, device=dev)).to(BF)
        g = F.pool_geom(x.shape, 3, 2, 0, Cc, Cc)
        pooled = torch.empty(B, g.OH, g.OW, Cc, dtype=BF, device=dev)
        arg = torch.empty(B, g.OH, g.OW, Cc, dtype=torch.uint8, device=dev)
        dp = torch.randn_like(pooled)
        dx = torch.empty_like(x)
        cs = torch.zeros(Cc, device=dev)
        for _ in range(3):
            F.lrn_maxpool_forward(x, pooled, arg, g)
            F.lrn_maxpool_backward(x, dp, arg, dx, g, relu_mask=True, colsum=cs)
    elif case == "pull_gemm":
        M, N, K, shards = 256, 4096, 9216, 4
        x = (torch.randn(M, K, device=dev) * 0.3).to(BF)
        parts = [(torch.randn(N // shards, K, device=dev) * 0.1).to(BF) for _ in range(shards)]
        out = torch.zeros(M, N, dtype=torch.float32, device=dev)
        for _ in range(4):
            F.pull_gemm(x, [t.data_ptr() for t in parts], [s * (N // shards) for s in range(shards)], out, ldw=K)
    elif case in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
        B, H, cin, cout, k, pad = 256, 13, 256, 384, 3, 1
        x = (torch.randn(B, H, H, cin, device=dev) * 0.5).to(BF)
        y = (torch.randn(B, H, H, cout, device=dev) * 0.5).to(BF)
        w = (torch.randn(cout, k * k * cin, device=dev) * 0.02).to(BF)
        dw = torch.empty(cout, k * k * cin, device=dev)
        for _ in range(4):
            if case == "conv_fwd":
                F.conv_tc(F.CONV_FWD, x, y, w, k, pad, relu=True)
            elif case == "conv_dgrad":
                F.conv_tc(F.CONV_DGRAD, x, y, w, k, pad)
            else:
                F.conv_tc(F.CONV_WGRAD, x, y, dw, k, pad)
    elif case in ("conv1_fwd", "conv2_fwd", "conv2_dgrad", "conv1_wgrad", "conv2_wgrad"):
        if case.startswith("conv1"):
            B, H, ct, cg, ot, og, k, pad = 256, 57, 64, 64, 96, 96, 3, 0
        else:
            B, H, ct, cg, ot, og, k, pad = 256, 27, 96, 48, 256, 128, 5, 2
        OH = H + 2 * pad - k + 1
        x = (torch.randn(B, H, H, ct, device=dev) * 0.5).to(BF)[..., :cg]
        y = (torch.randn(B, OH, OH, ot, device=dev) * 0.5).to(BF)[..., :og]
        w = (torch.randn(og, k * k * cg, device=dev) * 0.02).to(BF)
        if case.endswith("wgrad"):
            dw = torch.empty(og, k * k * cg, device=dev)
            for _ in range(4):
                F.conv_tc(F.CONV_WGRAD, x, y, dw, k, pad)
        else:
            for _ in range(4):
                F.conv_tc(F.CONV_DGRAD if case == "conv2_dgrad" else F.CONV_FWD, x, y, w, k, pad)
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    print("done", case)


if __name__ == "__main__":
    main()
