"""Row ops and training-op kernels vs plain PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu

from geeps_b200.ops import functional as F
from geeps_b200.ops import _lib as L

DEV = "cuda:0"
BF = torch.bfloat16


def test_row_gather_scatter_add():
    torch.manual_seed(0)
    cache = torch.randn(1000, 128, device=DEV)
    n = 333
    id1 = torch.randperm(1000, device=DEV)[:n]
    index = torch.stack([torch.arange(n, device=DEV), id1], dim=1).contiguous()
    buf = torch.full((n, 128), -7.0, device=DEV)
    st = L.new_status(DEV)
    limit = (n - 1) * 128 + 37  # last row only partly inside the value limit
    F.row_gather(buf, cache, index, num_vals_limit=limit, status=st)
    ref = cache[id1].clone()
    ref.view(-1)[limit:] = -7.0
    assert torch.equal(buf, ref)
    # scatter-add back twice the gathered rows
    oplog = torch.zeros_like(cache)
    F.row_scatter_add(oplog, buf, index, status=st)
    F.row_scatter_add(oplog, buf, index, status=st)
    ref2 = torch.zeros_like(cache)
    ref2[id1] = 2 * buf
    assert torch.allclose(oplog, ref2)
    dst = torch.zeros_like(cache)
    F.row_scatter(dst, buf, index, status=st)
    ref3 = torch.zeros_like(cache)
    ref3[id1] = buf
    assert torch.equal(dst, ref3)
    assert L.read_status(st)["code"] == 0


def test_row_op_bounds_are_reported_not_faulted():
    cache = torch.zeros(10, 128, device=DEV)
    buf = torch.ones(4, 128, device=DEV)
    index = torch.tensor([[0, 1], [1, 99], [2, 3], [3, -5]], device=DEV, dtype=torch.int64)
    st = L.new_status(DEV)
    F.row_scatter_add(cache, buf, index, status=st)
    torch.cuda.synchronize()
    s = L.read_status(st)
    assert s["name"] == "bounds"
    assert cache[1].sum().item() == 128 and cache[3].sum().item() == 128 and cache.sum().item() == 256


def test_axpy_and_convert():
    x = torch.randn(100003, device=DEV)
    y = torch.randn(100003, device=DEV)
    ref = y + 0.25 * x
    F.axpy(y, x, 0.25)
    assert torch.allclose(y, ref)
    h = torch.empty(100003, dtype=BF, device=DEV)
    F.f32_to_bf16(x, h)
    assert torch.equal(h, x.to(BF))


@pytest.mark.parametrize("cfg", [
    dict(B=3, H=13, W=13, C=16, groups=1, Cout=24, k=3, s=1, p=1),
    dict(B=2, H=27, W=27, C=32, groups=2, Cout=48, k=5, s=1, p=2),
    dict(B=2, H=35, W=35, C=3, groups=1, Cout=16, k=11, s=4, p=0),
    dict(B=2, H=16, W=16, C=24, groups=1, Cout=40, k=3, s=2, p=0),
])
def test_conv_via_im2col_gemm(cfg):
    torch.manual_seed(1)
    B, H, W, Cc, G, Cout, k, s, p = (cfg[n] for n in ("B", "H", "W", "C", "groups", "Cout", "k", "s", "p"))
    x = torch.randn(B, Cc, H, W, device=DEV)
    w = torch.randn(Cout, Cc // G, k, k, device=DEV) * 0.1
    xh = F.nchw_to_nhwc_bf16(x)
    assert torch.equal(xh, x.permute(0, 2, 3, 1).to(BF))
    Cg, Og = Cc // G, Cout // G
    kd = k * k * Cg
    ld = (kd + 7) // 8 * 8
    g0 = F.conv_geom(xh.shape, 0, Cg, k, k, s, p, ld)
    OH, OW = g0.OH, g0.OW
    y = torch.empty(B * OH * OW, Cout, dtype=BF, device=DEV)
    ref = TF.conv2d(xh.float().permute(0, 3, 1, 2), w.to(BF).float(), stride=s, padding=p, groups=G)
    dy = torch.randn_like(ref)
    dyh = dy.permute(0, 2, 3, 1).reshape(-1, Cout).to(BF).contiguous()
    dx = torch.empty_like(xh)
    dw = torch.empty(Cout, ld, device=DEV)
    for gi in range(G):
        g = F.conv_geom(xh.shape, gi * Cg, Cg, k, k, s, p, ld)
        col = torch.empty(B * OH * OW, ld, dtype=BF, device=DEV)
        F.im2col(xh, col, g)
        wg = torch.zeros(Og, ld, dtype=BF, device=DEV)
        wg[:, :kd] = w[gi * Og:(gi + 1) * Og].permute(0, 2, 3, 1).reshape(Og, kd).to(BF)
        F.gemm(col, wg, y[:, gi * Og:(gi + 1) * Og])
        # data gradient: dcol = dy_g @ W_g ; weight gradient: dW_g = dy_g^T @ col
        dcol = torch.empty_like(col)
        F.gemm(dyh[:, gi * Og:(gi + 1) * Og], wg, dcol, b_mn=True)
        F.col2im(dcol, dx, g)
        F.gemm(dyh[:, gi * Og:(gi + 1) * Og], col, dw[gi * Og:(gi + 1) * Og], a_mn=True, b_mn=True, split_k=0)
    torch.cuda.synchronize()
    got = y.view(B, OH, OW, Cout).permute(0, 3, 1, 2).float()
    assert torch.allclose(got, ref, atol=5e-2, rtol=2e-2)
    xr = xh.float().permute(0, 3, 1, 2).requires_grad_(True)
    wr = w.to(BF).float().requires_grad_(True)
    TF.conv2d(xr, wr, stride=s, padding=p, groups=G).backward(dyh.float().view(B, OH, OW, Cout).permute(0, 3, 1, 2))
    assert torch.allclose(dx.float().permute(0, 3, 1, 2), xr.grad, atol=8e-2, rtol=3e-2)
    dw_ref = wr.grad.permute(0, 2, 3, 1).reshape(Cout, kd)
    assert torch.allclose(dw[:, :kd], dw_ref, atol=1e-1, rtol=2e-2), (dw[:, :kd] - dw_ref).abs().max()


@pytest.mark.parametrize("relu", [False, True])
def test_batchnorm_forward_backward(relu):
    torch.manual_seed(2)
    P, Cc = 3000, 48
    x = (torch.randn(P, Cc, device=DEV) * 2 + 1).to(BF)
    gamma = torch.rand(Cc, device=DEV) + 0.5
    beta = torch.randn(Cc, device=DEV) * 0.1
    y = torch.empty_like(x)
    sums = torch.empty(2 * Cc, device=DEV)
    mr = torch.empty(2 * Cc, device=DEV)
    rm, rv = torch.zeros(Cc, device=DEV), torch.ones(Cc, device=DEV)
    F.bn_forward(x, y, gamma, beta, sums, mr, rm, rv, eps=1e-5, momentum=0.1, relu=relu)
    xr = x.float().requires_grad_(True)
    gr, br = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    yr = TF.batch_norm(xr, None, None, gr, br, training=True, eps=1e-5)
    if relu:
        yr = torch.relu(yr)
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    dy = torch.randn(P, Cc, device=DEV).to(BF)
    dx = torch.empty_like(x)
    dg, db = torch.empty(Cc, device=DEV), torch.empty(Cc, device=DEV)
    F.bn_backward(x, dy, y, dx, mr, gamma, sums, dg, db, relu=relu)
    # reference masks with its own fp32 y; use the kernel's bf16 y mask for an exact match
    yr2 = TF.batch_norm(xr, None, None, gr, br, training=True, eps=1e-5)
    if relu:
        yr2 = yr2 * (y.float() > 0)
    yr2.backward(dy.float())
    assert torch.allclose(dx.float(), xr.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(dg, gr.grad, atol=0.5, rtol=2e-2)
    assert torch.allclose(db, br.grad, atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("relu", [False, True])
def test_batchnorm_layer_alternating_and_repeated_passes(relu):
    """The BatchNorm layer's training-loop form (two launches per direction, each zeroing the other direction's
    scratch) over forward / backward / forward / forward / backward: every result matches torch."""
    from geeps_b200.ops import layers as GL
    torch.manual_seed(4)
    P, Cc = 2048, 64
    bn = GL.BatchNorm("bn", relu=relu)
    bn.setup((P, Cc), torch.device(DEV))
    gamma = torch.rand(Cc, device=DEV) + 0.5
    beta = torch.randn(Cc, device=DEV) * 0.1
    bn.p32 = {"gamma": gamma, "beta": beta}
    bn.g32 = {"gamma": torch.empty(Cc, device=DEV), "beta": torch.empty(Cc, device=DEV)}

    def check(x, dy):
        xr = x.float().requires_grad_(True)
        gr, br = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
        yr = TF.batch_norm(xr, None, None, gr, br, training=True, eps=bn.eps)
        y = bn.forward(x)
        assert torch.allclose(y.float(), torch.relu(yr) if relu else yr, atol=3e-2, rtol=2e-2)
        if dy is None:
            return
        dx = bn.backward(dy)
        (yr * (y.float() > 0) if relu else yr).backward(dy.float())
        assert torch.allclose(dx.float(), xr.grad, atol=3e-2, rtol=3e-2)
        assert torch.allclose(bn.g32["gamma"], gr.grad, atol=0.5, rtol=2e-2)
        assert torch.allclose(bn.g32["beta"], br.grad, atol=0.5, rtol=2e-2)

    mk = lambda: (torch.randn(P, Cc, device=DEV) * 2 + 1).to(BF)
    check(mk(), torch.randn(P, Cc, device=DEV).to(BF))
    check(mk(), None)                      # forward only ...
    check(mk(), None)                      # ... twice in a row: the scratch was not zeroed by a backward pass
    check(mk(), torch.randn(P, Cc, device=DEV).to(BF))
    check(mk(), torch.randn(P, Cc, device=DEV).to(BF))
    torch.cuda.synchronize()


def test_lrn_forward_backward():
    torch.manual_seed(3)
    P, Cc = 500, 96
    x = (torch.randn(P, Cc, device=DEV) * 3).to(BF)
    y = torch.empty_like(x)
    scale = torch.empty(P, Cc, dtype=BF, device=DEV)      # receives 1 / scale in bf16
    F.lrn_forward(x, y, scale, size=5, alpha=1e-2, beta=0.75, k=1.0)
    xr = x.float().requires_grad_(True)
    yr = TF.local_response_norm(xr.view(P, Cc, 1, 1), 5, alpha=1e-2, beta=0.75, k=1.0).view(P, Cc)
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    dy = torch.randn(P, Cc, device=DEV).to(BF)
    dx = torch.empty_like(x)
    F.lrn_backward(x, y, scale, dy, dx, size=5, alpha=1e-2, beta=0.75)
    yr.backward(dy.float())
    assert torch.allclose(dx.float(), xr.grad, atol=3e-2, rtol=3e-2)
    # with the producer's ReLU backward folded in: no gradient where the input is not positive
    dxm = torch.empty_like(x)
    F.lrn_backward(x, y, scale, dy, dxm, size=5, alpha=1e-2, beta=0.75, relu_mask=True)
    assert torch.equal(dxm, torch.where(x > 0, dx, torch.zeros_like(dx)))
    # ... and the per-channel sums of that gradient (the producer's bias gradient) from the same pass
    cs = torch.full((Cc,), 5.0, device=DEV)
    dxs = torch.empty_like(x)
    F.lrn_backward(x, y, scale, dy, dxs, size=5, alpha=1e-2, beta=0.75, relu_mask=True, colsum=cs)
    assert torch.equal(dxs, dxm)
    assert torch.allclose(cs, dxm.float().sum(0), atol=1e-2, rtol=1e-4)


def test_relu_backward_with_column_sums_in_one_pass():
    torch.manual_seed(12)
    P, Cc = 3000, 384
    wide_dy = torch.randn(P, Cc + 16, device=DEV).to(BF)
    dy = wide_dy[:, 8:8 + Cc]                                # a channel slice of a wider tensor
    y = torch.relu(torch.randn(P, Cc, device=DEV)).to(BF)
    dx = torch.empty(P, Cc, dtype=BF, device=DEV)
    cs = torch.full((Cc,), 3.0, device=DEV)
    F.relu_backward_colsum(dy, y, dx, cs)
    ref = torch.where(y > 0, dy, torch.zeros_like(dy))
    assert torch.equal(dx, ref)
    assert torch.allclose(cs, ref.float().sum(0), atol=1e-2, rtol=1e-4)


@pytest.mark.parametrize("H,Cc,k,s,p,size", [(13, 96, 3, 2, 0, 5), (27, 256, 3, 2, 0, 5), (16, 24, 3, 2, 0, 3),
                                              (9, 40, 3, 1, 1, 5), (8, 8, 2, 2, 0, 7)])
def test_fused_lrn_maxpool_matches_fp32_reference_and_the_unfused_kernels(H, Cc, k, s, p, size):
    """maxpool(LRN(x)) in one kernel per direction against torch in fp32 (LRN + max_pool2d + autograd) and against
    this library's separate LRN and pooling kernels; with the ReLU mask and the per-channel sums of dx."""
    torch.manual_seed(11)
    B = 3
    alpha, beta, kk = 1e-2, 0.75, 1.0
    x = torch.relu(torch.randn(B, H, H, Cc, device=DEV) * 3).to(BF)        # a ReLU output, as in the network
    g = F.pool_geom(x.shape, k, s, p, Cc, Cc)
    assert F.lrn_maxpool_supported(g, size)
    pooled = torch.empty(B, g.OH, g.OW, Cc, dtype=BF, device=DEV)
    arg = torch.empty(B, g.OH, g.OW, Cc, dtype=torch.uint8, device=DEV)
    F.lrn_maxpool_forward(x, pooled, arg, g, size, alpha, beta, kk)
    # unfused kernels of this library
    y = torch.empty_like(x)
    scale = torch.empty_like(x)
    F.lrn_forward(x.view(-1, Cc), y.view(-1, Cc), scale.view(-1, Cc), size, alpha, beta, kk)
    pooled_u = torch.empty_like(pooled)
    arg_u = torch.empty_like(arg)
    F.maxpool_forward(y, pooled_u, arg_u, g)
    # same values up to the last bf16 digit (the fused kernel evaluates the power as a polynomial), same window choice
    # except where two candidates are that close
    assert torch.allclose(pooled.float(), pooled_u.float(), atol=1e-2, rtol=1e-2)
    assert (arg != arg_u).float().mean().item() < 2e-2
    # fp32 reference
    xr = x.float().permute(0, 3, 1, 2).requires_grad_(True)
    yr = TF.max_pool2d(TF.local_response_norm(xr, size, alpha=alpha, beta=beta, k=kk), k, s, p, ceil_mode=True)
    assert yr.shape[2] == g.OH
    assert torch.allclose(pooled.float().permute(0, 3, 1, 2), yr, atol=3e-2, rtol=2e-2)
    dp = torch.randn_like(pooled)
    yr.backward(dp.float().permute(0, 3, 1, 2))
    ref = xr.grad.permute(0, 2, 3, 1)
    dx = torch.empty_like(x)
    cs = torch.full((Cc,), 7.0, device=DEV)
    F.lrn_maxpool_backward(x, dp, arg, dx, g, size, alpha, beta, kk, relu_mask=True, colsum=cs)
    ref_masked = torch.where(x > 0, ref, torch.zeros_like(ref))
    bad = ((dx.float() - ref_masked).abs() > 3e-2 + 3e-2 * ref_masked.abs()).float().mean().item()
    assert bad < 5e-3, bad       # the window maximum is taken on bf16-rounded values: rare near-ties pick another element
    # the sums are taken before dx is rounded to bf16
    assert torch.allclose(cs, dx.float().sum((0, 1, 2)), atol=8e-2, rtol=5e-3)
    # unfused backward of this library (pool backward, then LRN backward with the mask)
    dy_u = torch.empty_like(x)
    F.maxpool_backward(dp, arg, dy_u, g)
    dx_u = torch.empty_like(x)
    F.lrn_backward(x.view(-1, Cc), y.view(-1, Cc), scale.view(-1, Cc), dy_u.view(-1, Cc), dx_u.view(-1, Cc), size, alpha,
                   beta, relu_mask=True)
    assert torch.allclose(dx.float(), dx_u.float(), atol=4e-2, rtol=4e-2)
    # without the mask and the sums
    dx2 = torch.empty_like(x)
    F.lrn_maxpool_backward(x, dp, arg, dx2, g, size, alpha, beta, kk)
    assert torch.equal(torch.where(x > 0, dx2, torch.zeros_like(dx2)), dx)


@pytest.mark.parametrize("k,s,p,H", [(3, 2, 0, 13), (3, 2, 0, 16), (3, 1, 1, 9), (2, 2, 0, 8)])
def test_maxpool_avgpool(k, s, p, H):
    torch.manual_seed(4)
    B, Cc = 2, 24
    x = torch.randn(B, H, H, Cc, device=DEV).to(BF)
    g = F.pool_geom(x.shape, k, s, p, Cc, Cc + 8)
    wide = torch.zeros(B, g.OH, g.OW, Cc + 8, dtype=BF, device=DEV)
    y = wide[..., :Cc]
    arg = torch.empty(B, g.OH, g.OW, Cc, dtype=torch.uint8, device=DEV)
    F.maxpool_forward(x, y, arg, g)
    xr = x.float().permute(0, 3, 1, 2).requires_grad_(True)
    yr = TF.max_pool2d(xr, k, s, p, ceil_mode=True)
    assert yr.shape[2] == g.OH
    assert torch.equal(y.float().permute(0, 3, 1, 2), yr)
    dyw = torch.zeros_like(wide)
    dyw[..., :Cc] = torch.randn(B, g.OH, g.OW, Cc, device=DEV).to(BF)
    dx = torch.empty_like(x)
    F.maxpool_backward(dyw, arg, dx, g)
    yr.backward(dyw[..., :Cc].float().permute(0, 3, 1, 2))
    assert torch.allclose(dx.float().permute(0, 3, 1, 2), xr.grad, atol=2e-2, rtol=2e-2)
    # average pooling (floor mode shapes for the reference)
    ga = F.pool_geom(x.shape, k, s, p, Cc, Cc, ceil_mode=False)
    ya = torch.empty(B, ga.OH, ga.OW, Cc, dtype=BF, device=DEV)
    F.avgpool_forward(x, ya, ga)
    xa = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)  # NCHW-contiguous reference
    yar = TF.avg_pool2d(xa, k, s, p, ceil_mode=False, count_include_pad=True)
    assert torch.allclose(ya.float().permute(0, 3, 1, 2), yar, atol=2e-2, rtol=2e-2)
    dya = torch.randn_like(ya)
    dxa = torch.empty_like(x)
    F.avgpool_backward(dya, dxa, ga)
    yar.backward(dya.float().permute(0, 3, 1, 2).contiguous())
    assert torch.allclose(dxa.float().permute(0, 3, 1, 2), xa.grad, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("Cc", [10, 1000, 21841])
def test_softmax_cross_entropy(Cc):
    torch.manual_seed(5)
    B = 32
    logits = torch.randn(B, Cc, device=DEV) * 3
    labels = torch.randint(0, Cc, (B,), device=DEV)
    loss = torch.empty(1, device=DEV)
    ldd = (Cc + 7) // 8 * 8
    dl = torch.zeros(B, ldd, dtype=BF, device=DEV)
    F.softmax_ce(logits, labels, loss, dl[:, :Cc], loss_scale=1.0 / B, grad_scale=1.0 / B)
    lr = logits.clone().requires_grad_(True)
    ref = TF.cross_entropy(lr, labels)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-3 * max(1, abs(ref.item()))
    assert torch.allclose(dl[:, :Cc].float(), lr.grad, atol=2e-3, rtol=2e-2)


def test_colsum_relu_backward_dropout():
    torch.manual_seed(6)
    x = torch.randn(777, 64, device=DEV).to(BF)
    out = torch.empty(64, device=DEV)
    F.colsum(x, out, scale=0.5)
    assert torch.allclose(out, 0.5 * x.float().sum(0), atol=5e-2, rtol=1e-2)
    x2 = torch.randn(32, 1001, device=DEV).to(BF)
    out2 = torch.empty(1001, device=DEV)
    F.colsum(x2, out2)
    assert torch.allclose(out2, x2.float().sum(0), atol=5e-2, rtol=1e-2)
    y = torch.randn(1000, 8, device=DEV).to(BF)
    dy = torch.randn(1000, 8, device=DEV).to(BF)
    dx = torch.empty_like(dy)
    F.relu_backward(dy, y, dx)
    assert torch.equal(dx, torch.where(y.float() > 0, dy, torch.zeros_like(dy)))
    big = torch.ones(1 << 20, dtype=BF, device=DEV)
    o1, o2 = torch.empty_like(big), torch.empty_like(big)
    F.dropout(big, o1, 0.5, seed=42)
    F.dropout(big, o2, 0.5, seed=42)
    assert torch.equal(o1, o2)
    keep = (o1 > 0).float().mean().item()
    assert abs(keep - 0.5) < 0.01 and o1.max().item() == 2.0


@pytest.mark.parametrize("relu,fp32_out", [(True, False), (False, False), (False, True)])
def test_linear_with_the_k_range_split_over_the_sms_matches_fp32(relu, fp32_out, monkeypatch):
    """Batch-sized M: split-K GEMM into an fp32 workspace plus the converting pass, forward and data gradient,
    against torch in fp32 on the bf16-rounded operands."""
    from geeps_b200.ops import layers as GL
    monkeypatch.setattr(GL, "SPLIT_K_LINEAR", True)
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(11)
    B, K, N = 64, 1024, 264
    lin = GL.Linear("fc", N, relu=relu, fp32_out=fp32_out)
    lin.setup((B, K), dev)
    w = (torch.randn(N, K, device=dev, generator=gen) * 0.05).to(BF)
    bias = torch.randn(N, device=dev, generator=gen)
    lin.p16, lin.p32 = {"weight": w}, {"bias": bias}
    lin.g32 = {"weight": torch.zeros(N, K, device=dev), "bias": torch.zeros(N, device=dev)}
    x = torch.randn(B, K, device=dev, generator=gen).to(BF)
    y = lin.forward(x)
    ref = x.float() @ w.float().t() + bias
    if relu:
        ref = torch.relu(ref)
    assert y.dtype == (torch.float32 if fp32_out else BF)
    assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    dy = torch.randn(B, N, device=dev, generator=gen).to(torch.float32 if fp32_out else BF)
    dyb = dy.to(BF)
    dx = lin.backward(dyb)
    mask = (ref > 0).float() if relu else torch.ones_like(ref)
    dx_ref = (dyb.float() * mask) @ w.float()
    assert ((dx.float() - dx_ref).norm() / dx_ref.norm()).item() < 1e-2
    torch.cuda.synchronize()
