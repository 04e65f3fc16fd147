"""Implicit-GEMM convolution (tcgen05 + 4-D TMA, stride 1) against torch's fp32 convolution."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CASES = [
    # B, H, W, C_total, c_off, cg, O_total, o_off, og, k, pad
    (8, 13, 13, 64, 0, 64, 96, 0, 96, 3, 1),            # one channel chunk, one N tile
    (4, 27, 27, 96, 48, 48, 256, 128, 128, 5, 2),       # a 48-channel group slice (zero-filled to 64), 5x5
    (16, 13, 13, 192, 0, 192, 384, 0, 384, 3, 1),       # three chunks, two N tiles
    (5, 10, 12, 16, 0, 16, 40, 0, 40, 3, 0),            # no padding: output smaller than input
    (3, 9, 9, 32, 0, 32, 64, 0, 64, 1, 0),              # 1x1
    (2, 32, 32, 96, 0, 96, 32, 0, 32, 3, 1),            # wide image: boxes split the width
]


@pytest.mark.parametrize("case", CASES)
def test_conv_tc_forward_dgrad_wgrad_match_torch(case):
    from geeps_b200.ops import functional as F
    B, H, W, Ct, c_off, cg, Ot, o_off, og, k, pad = case
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(hash(case) % 1000)
    OH, OW = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    kd = k * k * cg
    ld = (kd + 7) // 8 * 8
    x_full = torch.randn(B, H, W, Ct, device=dev, generator=gen).to(BF)
    w = torch.zeros(og, ld, device=dev, dtype=BF)
    w[:, :kd] = (torch.randn(og, kd, device=dev, generator=gen) / kd ** 0.5).to(BF)
    bias = torch.randn(og, device=dev, generator=gen)
    dy_full = torch.randn(B, OH, OW, Ot, device=dev, generator=gen).to(BF)
    x = x_full[..., c_off:c_off + cg]
    dy = dy_full[..., o_off:o_off + og]
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    # fp32 reference on the bf16-rounded operands
    xr = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wr = w[:, :kd].float().view(og, k, k, cg).permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    yr = torch.nn.functional.conv2d(xr, wr, bias, padding=pad)
    yr.backward(dy.float().permute(0, 3, 1, 2))
    y_ref = torch.relu(yr.detach()).permute(0, 2, 3, 1)
    dx_ref = xr.grad.permute(0, 2, 3, 1)
    dw_ref = wr.grad.permute(0, 2, 3, 1).reshape(og, kd)

    y_full = torch.full((B, OH, OW, Ot), 7.0, device=dev, dtype=BF)
    y = y_full[..., o_off:o_off + og]
    assert F.conv_tc_supported(F.conv_tc_params(F.CONV_FWD, x, y, w, k, pad))
    F.conv_tc(F.CONV_FWD, x, y, w, k, pad, bias=bias, relu=True, status=status)
    assert _rel(y, y_ref) < 1e-2
    if Ot != og:      # channels outside the slice are untouched
        rest = torch.cat([y_full[..., :o_off], y_full[..., o_off + og:]], dim=-1)
        assert bool((rest == 7.0).all())

    dx_full = torch.full((B, H, W, Ct), 3.0, device=dev, dtype=BF)
    dx = dx_full[..., c_off:c_off + cg]
    F.conv_tc(F.CONV_DGRAD, dx, dy, w, k, pad, status=status)
    assert _rel(dx, dx_ref) < 1e-2
    if Ct != cg:
        rest = torch.cat([dx_full[..., :c_off], dx_full[..., c_off + cg:]], dim=-1)
        assert bool((rest == 3.0).all())

    for split in (0, 1):
        dw = torch.full((og, ld), 5.0, device=dev)
        F.conv_tc(F.CONV_WGRAD, x, dy, dw, k, pad, split_k=split, status=status)
        assert _rel(dw[:, :kd], dw_ref) < 1e-2, split
        assert bool((dw[:, kd:] == 0).all())
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0


STRIDED = [
    # B, H, W, cg, og, k, pad, stride
    (4, 28, 28, 64, 96, 3, 1, 2),        # Inception down-sampling branch
    (2, 64, 64, 8, 64, 7, 3, 2),         # first layer of the 22K net (3 channels padded to 8), scaled down
    (3, 17, 17, 32, 32, 3, 0, 2),        # no padding, odd size
    (2, 23, 23, 16, 48, 5, 2, 3),        # stride 3
]


@pytest.mark.parametrize("case", STRIDED)
def test_strided_conv_forward_and_gradients_match_torch(case):
    """Strided layers: the activation boxes are loaded with a TMA element stride, the data gradient runs per parity
    class of the input; no patch matrix."""
    from geeps_b200.ops import functional as F
    B, H, W, cg, og, k, pad, st = case
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(5)
    OH, OW = (H + 2 * pad - k) // st + 1, (W + 2 * pad - k) // st + 1
    kd = k * k * cg
    ld = (kd + 7) // 8 * 8
    x = torch.randn(B, H, W, cg, device=dev, generator=gen).to(BF)
    w = torch.zeros(og, ld, device=dev, dtype=BF)
    w[:, :kd] = (torch.randn(og, kd, device=dev, generator=gen) / kd ** 0.5).to(BF)
    bias = torch.randn(og, device=dev, generator=gen)
    dy = torch.randn(B, OH, OW, og, device=dev, generator=gen).to(BF)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    xr = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wr = w[:, :kd].float().view(og, k, k, cg).permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    yr = torch.nn.functional.conv2d(xr, wr, bias, stride=st, padding=pad)
    yr.backward(dy.float().permute(0, 3, 1, 2))
    y = torch.empty(B, OH, OW, og, device=dev, dtype=BF)
    assert F.conv_tc_supported(F.conv_tc_params(F.CONV_FWD, x, y, w, k, pad, stride=st))
    assert F.conv_tc_supported(F.conv_tc_params(F.CONV_DGRAD, x, y, w, k, pad, stride=st))
    assert not F.conv_tc_supported(F.conv_tc_params(F.CONV_DGRAD, x, y, w[:, :cg], 1, 0, stride=st))
    F.conv_tc(F.CONV_FWD, x, y, w, k, pad, bias=bias, relu=True, status=status, stride=st)
    assert _rel(y, torch.relu(yr.detach()).permute(0, 2, 3, 1)) < 1e-2
    dw_ref = wr.grad.permute(0, 2, 3, 1).reshape(og, kd)
    for split in (0, 1):
        dw = torch.full((og, ld), 5.0, device=dev)
        F.conv_tc(F.CONV_WGRAD, x, dy, dw, k, pad, split_k=split, status=status, stride=st)
        assert _rel(dw[:, :kd], dw_ref) < 1e-2, split
    dx = torch.full((B, H, W, cg), 3.0, device=dev, dtype=BF)
    F.conv_tc(F.CONV_DGRAD, dx, dy, w, k, pad, status=status, stride=st)
    assert _rel(dx, xr.grad.permute(0, 2, 3, 1)) < 1e-2
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0


HALO_CASES = CASES + [
    (3, 57, 57, 48, 0, 48, 96, 0, 96, 3, 0),            # AlexNet conv1 after space-to-depth: 96 channels leave in 32-wide slabs
    (3, 28, 28, 192, 0, 192, 96, 0, 96, 3, 1),          # three chunks, rows split 4 + 4 per tile, last tile short
    (2, 14, 14, 96, 32, 32, 64, 0, 48, 5, 2),           # 5x5 on a small map, channel slices on both sides
    (2, 56, 56, 64, 0, 64, 192, 0, 192, 3, 1),          # two rows per block, two N tiles
]


@pytest.mark.parametrize("case", HALO_CASES)
def test_conv_halo_forward_dgrad_match_torch(case):
    """The halo-tile kernel called directly on every shape it accepts (conv_tc() picks it only where it pays)."""
    from geeps_b200.ops import functional as F
    B, H, W, Ct, c_off, cg, Ot, o_off, og, k, pad = case
    if k * k < 4:
        pytest.skip("single-tap filters have no halo")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(hash(case) % 1000)
    OH, OW = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    kd = k * k * cg
    ld = (kd + 7) // 8 * 8
    x_full = torch.randn(B, H, W, Ct, device=dev, generator=gen).to(BF)
    w = torch.zeros(og, ld, device=dev, dtype=BF)
    w[:, :kd] = (torch.randn(og, kd, device=dev, generator=gen) / kd ** 0.5).to(BF)
    bias = torch.randn(og, device=dev, generator=gen)
    dy_full = torch.randn(B, OH, OW, Ot, device=dev, generator=gen).to(BF)
    x = x_full[..., c_off:c_off + cg]
    dy = dy_full[..., o_off:o_off + og]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    xr = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wr = w[:, :kd].float().view(og, k, k, cg).permute(0, 3, 1, 2).contiguous()
    yr = torch.nn.functional.conv2d(xr, wr, bias, padding=pad)
    yr.backward(dy.float().permute(0, 3, 1, 2))
    y_ref = torch.relu(yr.detach()).permute(0, 2, 3, 1)
    dx_ref = xr.grad.permute(0, 2, 3, 1)

    y_full = torch.full((B, OH, OW, Ot), 7.0, device=dev, dtype=BF)
    y = y_full[..., o_off:o_off + og]
    F.conv_halo(F.CONV_FWD, x, y, w, k, pad, bias=bias, relu=True, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    assert _rel(y, y_ref) < 1e-2
    if Ot != og:
        rest = torch.cat([y_full[..., :o_off], y_full[..., o_off + og:]], dim=-1)
        assert bool((rest == 7.0).all())
    dx_full = torch.full((B, H, W, Ct), 3.0, device=dev, dtype=BF)
    dx = dx_full[..., c_off:c_off + cg]
    F.conv_halo(F.CONV_DGRAD, dx, dy, w, k, pad, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    assert _rel(dx, dx_ref) < 1e-2
    if Ct != cg:
        rest = torch.cat([dx_full[..., :c_off], dx_full[..., c_off + cg:]], dim=-1)
        assert bool((rest == 3.0).all())


@pytest.mark.parametrize("case", [c for c in HALO_CASES if c[9] > 1 and c[9] <= 8])
def test_conv_wgrad_halo_matches_torch(case):
    """The filter-row weight-gradient kernel (one activation tile serves the taps of a row through overlapping
    N panels) called directly on every shape it accepts."""
    from geeps_b200.ops import functional as F
    B, H, W, Ct, c_off, cg, Ot, o_off, og, k, pad = case
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(hash(case) % 1000)
    OH, OW = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    kd = k * k * cg
    ld = (kd + 7) // 8 * 8
    x = torch.randn(B, H, W, Ct, device=dev, generator=gen).to(BF)[..., c_off:c_off + cg]
    dy = torch.randn(B, OH, OW, Ot, device=dev, generator=gen).to(BF)[..., o_off:o_off + og]
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    xr = x.float().permute(0, 3, 1, 2).contiguous()
    wr = torch.zeros(og, cg, k, k, device=dev, requires_grad=True)
    torch.nn.functional.conv2d(xr, wr, None, padding=pad).backward(dy.float().permute(0, 3, 1, 2))
    dw_ref = wr.grad.permute(0, 2, 3, 1).reshape(og, kd)
    dw = torch.full((og, ld), 5.0, device=dev)
    F.conv_wgrad_halo(x, dy, dw, k, pad, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    assert _rel(dw[:, :kd], dw_ref) < 1e-2
    assert bool((dw[:, kd:] == 0).all())


@pytest.mark.parametrize("cpad", [None, 64])
def test_space_to_depth_conv_matches_strided_torch_conv(cpad):
    """Input(s2d) + Conv2d(s2d): an 11x11 stride-4 convolution run as a 3-tap stride-1 implicit GEMM; with cpad the
    48-channel space-to-depth pixel is zero-padded to one 128-byte line."""
    from geeps_b200.ops.layers import Conv2d, Input
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(3)
    B, C, H, k, S, cout = 4, 3, 67, 11, 4, 32
    x = torch.randn(B, C, H, H, device=dev, generator=gen)
    inp = Input(s2d=S, s2d_k=k, cpad=cpad)
    conv = Conv2d("c1", cout, k, stride=S, relu=True, need_dx=False, s2d=S, cin_valid=C if cpad else None)
    shape = conv.setup(inp.setup((B, C, H, H), dev), dev)
    OH = (H - k) // S + 1
    assert shape == (B, OH, OH, cout)
    spec = conv.param_specs()[0]
    assert spec.num_valid() == cout * k * k * C
    w32 = spec.initial(torch.Generator().manual_seed(1)).to(dev) * 5
    bias = torch.randn(cout, device=dev, generator=gen)
    conv.p32, conv.p16 = {"weight": w32, "bias": bias}, {"weight": w32.to(BF)}
    conv.g32 = {"weight": torch.full_like(w32, 9.0), "bias": torch.zeros(cout, device=dev)}
    y = conv.forward(inp.forward(x)).view(B, OH, OH, cout)

    # the same weights as a [cout, C, k, k] filter: column (a*T + b)*48 + (dy*S + dx)*C + c -> tap (a*S+dy, b*S+dx)
    T, Cs, Cp = conv.k, S * S * C, conv.in_shape[-1]
    assert Cp == (cpad or Cs)
    wt = w32.to(BF).float()[:, :T * T * Cp].view(cout, T, T, Cp)[..., :Cs].reshape(cout, T, T, S, S, C)   # [o, a, b, dy, dx, c]
    wfull = wt.permute(0, 5, 1, 3, 2, 4).reshape(cout, C, T * S, T * S)[:, :, :k, :k].contiguous().requires_grad_(True)
    xr = x.to(BF).float()
    yr = torch.nn.functional.conv2d(xr, wfull, bias, stride=S)
    assert _rel(y, torch.relu(yr).permute(0, 2, 3, 1)) < 1e-2

    dy = torch.randn(B, OH, OH, cout, device=dev, generator=gen).to(BF)
    conv.backward(dy.view(-1, cout))
    mask = (yr > 0).float()
    yr.backward(dy.float().permute(0, 3, 1, 2) * mask)
    gfull = conv.g32["weight"][:, :T * T * Cp].view(cout, T, T, Cp)
    assert float(gfull[..., Cs:].abs().max()) == 0 if Cp > Cs else True      # padding channels receive no gradient
    gw = gfull[..., :Cs].reshape(cout, T, T, S, S, C).permute(0, 5, 1, 3, 2, 4).reshape(cout, C, T * S, T * S)
    assert _rel(gw[:, :, :k, :k], wfull.grad) < 1e-2
    # taps past the 11 x 11 filter receive no gradient, so they stay zero under SGD
    assert float(gw[:, :, k:, :].abs().max()) == 0 and float(gw[:, :, :, k:].abs().max()) == 0


@pytest.mark.parametrize("layout", ["s2d64", "s2d48", "nhwc8", "s2d2"])
@pytest.mark.parametrize("mode", ["centre", "random"])
def test_uint8_data_transformer_matches_torch(layout, mode):
    """Input on uint8 source images: crop, mirror, mean subtraction and scale on the device give exactly what the
    same arithmetic in torch followed by the fp32 input path gives (both round the same fp32 value to bf16)."""
    from geeps_b200.ops.layers import Input
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(11)
    B, C, Hin, Win, H, W = 5, 3, 80, 90, 67, 71
    mean, scale = (104.0, 117.0, 123.5), 1.0 / 57.0
    kw = {"s2d64": dict(s2d=4, s2d_k=11, cpad=64), "s2d48": dict(s2d=4, s2d_k=11), "nhwc8": dict(cpad=8),
          "s2d2": dict(s2d=2, s2d_k=7, cpad=16)}[layout]
    inp, ref = Input(mean=mean, scale=scale, **kw), Input(**kw)
    shape = inp.setup((B, C, H, W), dev)
    assert ref.setup((B, C, H, W), dev) == shape
    x = torch.randint(0, 256, (B, C, Hin, Win), device=dev, generator=gen, dtype=torch.uint8)
    if mode == "random":
        inp.randomize((Hin, Win), mirror=True, generator=gen)
        aug = inp.aug.cpu()
        assert int(aug[:, 2].max()) == 1 and int(aug[:, 2].min()) == 0      # both orientations are in the batch
    else:
        aug = torch.tensor([[(Hin - H) // 2, (Win - W) // 2, 0]] * B)
    y = inp.forward(x).clone()
    m = torch.tensor(mean, device=dev).view(1, C, 1, 1)
    rows = []
    for b in range(B):
        ho, wo, mir = (int(v) for v in aug[b])
        win = x[b:b + 1, :, ho:ho + H, wo:wo + W].float()
        rows.append(win.flip(-1) if mir else win)
    xr = (torch.cat(rows) - m) * scale
    yr = ref.forward(xr.contiguous())
    assert y.shape == yr.shape == shape
    assert torch.equal(y, yr)
    if mode == "random":
        inp.set_augmentation(None)          # back to the centre crop, through the same buffer
        y2 = inp.forward(x)
        xc = (x[:, :, (Hin - H) // 2:(Hin - H) // 2 + H, (Win - W) // 2:(Win - W) // 2 + W].float() - m) * scale
        assert torch.equal(y2, ref.forward(xc.contiguous()))
