"""Kernel micro-benchmarks: python -m geeps_b200.utils.microbench [gemm|conv|lrn_pool|rows|input|all]

Every number is a CUDA-event time on the launching stream after warm-up, with a buffer larger than
L2 written between timed launches.  GEMM lines also give cuBLAS (torch.matmul) on the same shape and
the fraction of the measured bf16 peak (MEASURED_PEAKS.json if present, else 1590 TFLOP/s)."""
from __future__ import annotations

import json
import os
import sys

import torch

from ..ops import functional as F

BF = torch.bfloat16


def _peaks():
    path = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def timeit(fn, iters=10, flush=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)          # 256 MB write: evicts L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(shapes=None):
    dev = torch.device("cuda")
    peak, _, src = _peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    shapes = shapes or [
        ("square 8192", 8192, 8192, 8192, False, False, False),
        ("square 4096", 4096, 4096, 4096, False, False, False),
        ("conv1 fwd", 774400, 96, 488, False, False, False),
        ("conv2 fwd (1 group)", 186624, 128, 1200, False, False, False),
        ("conv3 fwd", 43264, 384, 2304, False, False, False),
        ("conv3 dgrad", 43264, 2304, 384, False, True, False),
        ("conv3 wgrad", 384, 2304, 43264, True, True, True),
        ("conv2 dgrad (1 group)", 186624, 1200, 128, False, True, False),
        ("fc6 fwd", 256, 4096, 9216, False, False, False),
        ("fc6 dgrad", 256, 9216, 4096, False, True, False),
        ("fc6 wgrad", 4096, 9216, 256, True, True, True),
    ]
    rows = []
    for name, M, N, K, a_mn, b_mn, f32 in shapes:
        a = (torch.randn((K, M) if a_mn else (M, K), device=dev) * 0.1).to(BF)
        b = (torch.randn((K, N) if b_mn else (N, K), device=dev) * 0.1).to(BF)
        out = torch.empty(M, N, dtype=torch.float32 if f32 else BF, device=dev)
        t = timeit(lambda: F.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, split_k=0 if f32 else 1), flush=flush)
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        t_ref = timeit(lambda: torch.matmul(A, Bm), flush=flush)
        tf = 2.0 * M * N * K / t / 1e9
        rows.append({"shape": name, "M": M, "N": N, "K": K, "ms": round(t, 4), "tflops": round(tf, 1),
                     "frac_of_peak": round(tf / peak, 3), "peak_source": src, "cublas_ms": round(t_ref, 4),
                     "cublas_tflops": round(2.0 * M * N * K / t_ref / 1e9, 1)})
        if M <= 256 and not f32:
            # batch-sized M: a few wide tiles leave most SMs idle, so the k range is split over the SMs, the partial
            # sums are reduce-added in fp32 and a finishing pass converts (bias + ReLU of the layer included)
            ws = torch.empty(M, N, dtype=torch.float32, device=dev)
            bias = torch.zeros(N, device=dev)
            t2 = timeit(lambda: (F.gemm(a, b, ws, a_mn=a_mn, b_mn=b_mn, bias=bias, split_k=0),
                                 F.f32_to_bf16_2d(ws, out, relu=True)), flush=flush)
            rows[-1]["split_k_plus_finish_ms"] = round(t2, 4)
        print(json.dumps(rows[-1]), flush=True)
        del a, b, out
    return rows


def bench_rows():
    dev = torch.device("cuda")
    _, hbm, src = _peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    n = 1 << 20   # 512 MB of rows
    cache = torch.randn(n, 128, device=dev)
    buf = torch.empty(n, 128, device=dev)
    idx = torch.stack([torch.arange(n, device=dev), torch.randperm(n, device=dev)], 1).contiguous()
    for name, fn, nbytes in (("row_gather", lambda: F.row_gather(buf, cache, idx), 2 * n * 512),
                             ("row_scatter_add", lambda: F.row_scatter_add(cache, buf, idx), 3 * n * 512)):
        t = timeit(fn, flush=flush)
        gbs = nbytes / t / 1e6
        print(json.dumps({"kernel": name, "rows": n, "ms": round(t, 4), "gb_s": round(gbs, 1),
                          "frac_of_hbm": round(gbs / hbm, 3), "peak_source": src}), flush=True)


def bench_lrn_pool():
    """LRN + max pooling of AlexNet (after conv1: 55x55x96, after conv2: 27x27x256; batch 256): the fused kernels
    against the separate LRN and pooling kernels, with the bytes each formulation has to move."""
    dev = torch.device("cuda")
    _, hbm, src = _peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    for name, H, Cc in (("lrn+pool after conv1", 55, 96), ("lrn+pool after conv2", 27, 256)):
        B = 256
        x = torch.relu(torch.randn(B, H, H, Cc, device=dev)).to(BF)
        g = F.pool_geom(x.shape, 3, 2, 0, Cc, Cc)
        pooled = torch.empty(B, g.OH, g.OW, Cc, dtype=BF, device=dev)
        arg = torch.empty(B, g.OH, g.OW, Cc, dtype=torch.uint8, device=dev)
        dp = torch.randn_like(pooled)
        dx = torch.empty_like(x)
        cs = torch.zeros(Cc, device=dev)
        y, scale, dy = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        x2, y2, s2, dy2, dx2 = (t.view(-1, Cc) for t in (x, y, scale, dy, dx))
        nx, npool = x.numel() * 2, pooled.numel() * 2
        cases = [
            ("fused forward", lambda: F.lrn_maxpool_forward(x, pooled, arg, g), nx + npool + npool // 2),
            ("fused backward", lambda: F.lrn_maxpool_backward(x, dp, arg, dx, g, relu_mask=True, colsum=cs),
             2 * nx + npool + npool // 2),
            ("separate forward", lambda: (F.lrn_forward(x2, y2, s2), F.maxpool_forward(y, pooled, arg, g)),
             4 * nx + npool + npool // 2),
            ("separate backward", lambda: (F.maxpool_backward(dp, arg, dy, g),
                                           F.lrn_backward(x2, y2, s2, dy2, dx2, relu_mask=True, colsum=cs)),
             6 * nx + npool + npool // 2),
        ]
        for what, fn, nbytes in cases:
            t = timeit(fn, flush=flush)
            gbs = nbytes / t / 1e6
            print(json.dumps({"kernel": f"{name}: {what}", "ms": round(t, 4), "algorithmic_mb": round(nbytes / 1e6, 1),
                              "gb_s": round(gbs, 1), "frac_of_hbm": round(gbs / hbm, 3), "peak_source": src}), flush=True)


def bench_conv():
    """Stride-1 convolutions of AlexNet (batch 256) and Inception (batch 128): the box kernel (one activation load
    per filter tap) against the halo-tile kernel (one load per channel chunk), forward and data gradient."""
    dev = torch.device("cuda")
    peak, _, src = _peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    shapes = [
        # name, B, H, cg, og, k, pad, groups sharing the tensors
        ("alexnet conv1 (space-to-depth, pixel padded to 64 channels)", 256, 57, 64, 96, 3, 0, 1),
        ("alexnet conv2 (one of 2 groups)", 256, 27, 48, 128, 5, 2, 2),
        ("inception 3x3 56x56 64->192", 128, 56, 64, 192, 3, 1, 1),
        ("inception 3x3 28x28 128->192", 128, 28, 128, 192, 3, 1, 1),
        ("inception 5x5 28x28 32->96", 128, 28, 32, 96, 5, 2, 1),
        ("inception 3x3 14x14 112->224", 128, 14, 112, 224, 3, 1, 1),
    ]
    for name, B, H, cg, og, k, pad, groups in shapes:
        OH = H + 2 * pad - k + 1
        xf = torch.randn(B, H, H, cg * groups, device=dev).to(BF)
        yf = torch.empty(B, OH, OH, og * groups, device=dev, dtype=BF)
        x, y = xf[..., :cg], yf[..., :og]
        kd = k * k * cg
        w = (torch.randn(og, kd, device=dev) / kd ** 0.5).to(BF)
        bias = torch.zeros(og, device=dev)
        flops = 2.0 * B * OH * OH * og * kd
        for mode, mname in ((F.CONV_FWD, "fwd"), (F.CONV_DGRAD, "dgrad")):
            kw = dict(bias=bias, relu=True) if mode == F.CONV_FWD else {}
            t_box = timeit(lambda: F.conv_tc(mode, x, y, w, k, pad, split_k=-1, **kw), flush=flush)
            t_halo = timeit(lambda: F.conv_halo(mode, x, y, w, k, pad, **kw), flush=flush)
            print(json.dumps({"kernel": f"{name} {mname}", "box_ms": round(t_box, 4), "halo_ms": round(t_halo, 4),
                              "halo_tflops": round(flops / t_halo / 1e9, 1),
                              "halo_frac_of_peak": round(flops / t_halo / 1e9 / peak, 3), "peak_source": src,
                              "routed_to_halo": bool(F.conv_halo_applicable(F.conv_tc_params(mode, x, y, w, k, pad)))}),
                  flush=True)
        dw = torch.empty(og, (kd + 7) // 8 * 8, device=dev)
        t_box = timeit(lambda: F.conv_tc(F.CONV_WGRAD, x, y, dw, k, pad, split_k=-1), flush=flush)
        t_halo = timeit(lambda: F.conv_wgrad_halo(x, y, dw, k, pad), flush=flush)
        print(json.dumps({"kernel": f"{name} wgrad", "box_ms": round(t_box, 4), "halo_ms": round(t_halo, 4),
                          "halo_tflops": round(flops / t_halo / 1e9, 1),
                          "halo_frac_of_peak": round(flops / t_halo / 1e9 / peak, 3), "peak_source": src}), flush=True)


def bench_input():
    """The input layer of AlexNet at batch 256 (3 x 227 x 227 -> space-to-depth 57 x 57 x 64 bf16) from fp32, bf16 and
    uint8 batches; the uint8 form also from 256 x 256 source images with a random crop and mirror per image."""
    from ..ops.layers import Input
    dev = torch.device("cuda")
    _, hbm, src = _peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    B, H = 256, 227
    for name, dtype, Hin in (("fp32 batch", torch.float32, H), ("bf16 batch", BF, H), ("uint8 batch", torch.uint8, H),
                             ("uint8 256x256 source, random crop + mirror", torch.uint8, 256)):
        inp = Input(s2d=4, s2d_k=11, cpad=64, mean=(104.0, 117.0, 123.0), scale=1.0 / 58.0)
        out_shape = inp.setup((B, 3, H, H), dev)
        if dtype == torch.uint8:
            x = torch.randint(0, 256, (B, 3, Hin, Hin), device=dev, dtype=torch.uint8)
            if Hin > H:
                inp.randomize((Hin, Hin))
        else:
            x = torch.randn(B, 3, H, H, device=dev).to(dtype)
        t = timeit(lambda: inp.forward(x), flush=flush)
        nbytes = B * 3 * H * H * x.element_size() + 2 * out_shape[0] * out_shape[1] * out_shape[2] * out_shape[3]
        gbs = nbytes / t / 1e6
        print(json.dumps({"kernel": f"input layer, {name}", "ms": round(t, 4), "algorithmic_mb": round(nbytes / 1e6, 1),
                          "gb_s": round(gbs, 1), "frac_of_hbm": round(gbs / hbm, 3), "peak_source": src}), flush=True)


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("conv", "all"):
        bench_conv()
    if what in ("lrn_pool", "all"):
        bench_lrn_pool()
    if what in ("gemm", "all"):
        bench_gemm()
    if what in ("rows", "all"):
        bench_rows()
    if what in ("input", "all"):
        bench_input()


if __name__ == "__main__":
    main()
