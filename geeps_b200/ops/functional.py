"""Functional wrappers: one Python function per native kernel, on torch tensors.

Activations are NHWC bf16 (2-D views [pixels, channels] with a channel pitch), parameters
and statistics fp32.  Nothing here falls back to a torch implementation: without the
native library or without a GPU these functions raise.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from ._lib import ConvGeom, ConvTcParams, GemmParams, PoolGeom, check, launch, lib, ptr, stream_ptr

bf16 = torch.bfloat16


def _ld(t: torch.Tensor) -> int:
    """Row pitch (elements) of a 2-D tensor whose last dim is contiguous."""
    assert t.dim() == 2 and (t.stride(1) == 1 or t.shape[1] == 1), "need a row-major 2-D view"
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: torch.Tensor | None = None, bias_mode: int = 1, relu: bool = False, alpha: float = 1.0,
         beta: float = 0.0, split_k: int = 1, block_n: int = 0, status: torch.Tensor | None = None,
         impl: str = "auto") -> torch.Tensor:
    """out[M,N] = alpha * A[M,K] @ B[N,K]^T + beta*out + bias  (bf16 operands, fp32 accumulate).

    a_mn / b_mn: the operand is stored transposed ([K, M] / [K, N] row-major).
    out is bf16 or fp32 and may be a column slice of a wider matrix.
    impl: "auto" (tcgen05 when the layout allows, else SIMT), "tc", "pair" (CTA pairs, 256-row tiles) or "simt".
    """
    L.require_cuda()
    assert a.dtype == bf16 and b.dtype == bf16 and out.dtype in (bf16, torch.float32)
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    assert (a.shape == (K, M)) if a_mn else (a.shape == (M, K)), (a.shape, M, K, a_mn)
    assert (b.shape == (K, N)) if b_mn else (b.shape == (N, K)), (b.shape, N, K, b_mn)
    p = GemmParams()
    p.A, p.B, p.C, p.bias = a.data_ptr(), b.data_ptr(), out.data_ptr(), (bias.data_ptr() if bias is not None else None)
    p.M, p.N, p.K = M, N, K
    p.lda, p.ldb, p.ldc = _ld(a), _ld(b), _ld(out)
    p.alpha, p.beta = alpha, beta
    p.a_mn_major, p.b_mn_major = int(a_mn), int(b_mn)
    p.out_fp32 = int(out.dtype == torch.float32)
    p.bias_mode = bias_mode if bias is not None else 0
    p.relu = int(relu)
    p.split_k = split_k
    p.block_n = block_n
    p.status = status.data_ptr() if status is not None else None
    if bias is not None:
        assert bias.dtype == torch.float32
    if impl == "pair":
        launch(lib().geeps_gemm_bf16_pair, "gemm_bf16(tcgen05 pair)", C.byref(p), stream_ptr())
        return out
    use_tc = impl == "tc" or (impl == "auto" and lib().geeps_gemm_tc_supported(C.byref(p)))
    if use_tc:
        launch(lib().geeps_gemm_bf16, "gemm_bf16(tcgen05)", C.byref(p), stream_ptr())
    else:
        if split_k != 1:
            p.split_k = 1
        launch(lib().geeps_gemm_bf16_simt, "gemm_bf16(simt)", C.byref(p), stream_ptr())
    return out


CONV_FWD, CONV_DGRAD, CONV_WGRAD = 0, 1, 2


def conv_tc_params(mode: int, x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, k: int, pad: int, *,
                   bias: torch.Tensor | None = None, relu: bool = False, split_k: int = 0,
                   status: torch.Tensor | None = None, stride: int = 1) -> ConvTcParams:
    """Arguments of the implicit-GEMM convolution (stride 1 .. 8; the data gradient of a strided layer needs a
    filter at least as wide as the stride).  x: [B, H, W, cg] and y: [B, OH, OW, og] are NHWC
    bf16 tensors or channel slices of wider ones (last-dim stride 1, dense pixels); w: [og, ldw] with column
    (kh * k + kw) * cg + ci, bf16 for forward / data gradient, fp32 (the gradient) for the weight gradient."""
    B, H, W, cg = x.shape
    _, OH, OW, og = y.shape
    assert x.stride(3) == 1 and y.stride(3) == 1 and w.stride(1) == 1
    xp, yp = x.stride(2), y.stride(2)
    assert x.stride(1) == W * xp and x.stride(0) == H * W * xp, "x pixels must be dense"
    assert y.stride(1) == OW * yp and y.stride(0) == OH * OW * yp, "y pixels must be dense"
    p = ConvTcParams()
    p.x, p.y, p.w = x.data_ptr(), y.data_ptr(), w.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    p.status = status.data_ptr() if status is not None else None
    p.x_pitch, p.y_pitch, p.ldw = xp, yp, w.stride(0)
    p.B, p.H, p.W, p.cg, p.OH, p.OW, p.og = B, H, W, cg, OH, OW, og
    p.KH, p.KW, p.pad, p.relu, p.mode, p.split_k = k, k, pad, int(relu), mode, split_k
    p.stride = stride
    return p


def conv_tc_supported(p: ConvTcParams) -> bool:
    return bool(lib().geeps_conv_tc_supported(C.byref(p)))


def conv_tc(mode: int, x, y, w, k: int, pad: int, **kw) -> None:
    """Convolution without a patch matrix (tcgen05 + 4-D TMA): forward writes y, CONV_DGRAD writes x (y holds dY),
    CONV_WGRAD writes w (fp32, y holds dY).  stride=s: forward and weight gradient load the activation boxes with
    TMA element stride s; the data gradient runs s * s stride-1 problems, one per parity class of x."""
    L.require_cuda()
    assert x.dtype == bf16 and y.dtype == bf16
    assert w.dtype == (torch.float32 if mode == CONV_WGRAD else bf16)
    p = conv_tc_params(mode, x, y, w, k, pad, **kw)
    launch(lib().geeps_conv_tc, "conv_tc", C.byref(p), stream_ptr())


def conv_halo_applicable(p: ConvTcParams) -> bool:
    """Does conv_tc() route this call to the halo-tile kernel (activations fetched once per channel chunk)?"""
    return bool(lib().geeps_conv_halo_applicable(C.byref(p)))


def conv_halo(mode: int, x, y, w, k: int, pad: int, **kw) -> None:
    """The halo-tile kernel called directly (forward / data gradient), whatever conv_tc() would have chosen."""
    L.require_cuda()
    assert mode in (CONV_FWD, CONV_DGRAD) and x.dtype == bf16 and y.dtype == bf16 and w.dtype == bf16
    p = conv_tc_params(mode, x, y, w, k, pad, **kw)
    launch(lib().geeps_conv_halo, "conv_halo", C.byref(p), stream_ptr())


def conv_wgrad_halo(x, dy, dw, k: int, pad: int, **kw) -> None:
    """The filter-row weight-gradient kernel called directly (dw fp32 [og, ldw], overwritten)."""
    L.require_cuda()
    assert x.dtype == bf16 and dy.dtype == bf16 and dw.dtype == torch.float32
    p = conv_tc_params(CONV_WGRAD, x, dy, dw, k, pad, **kw)
    launch(lib().geeps_conv_wgrad_halo, "conv_wgrad_halo", C.byref(p), stream_ptr())


def nchw_to_nhwc_bf16(x: torch.Tensor, cpad: int | None = None) -> torch.Tensor:
    L.require_cuda()
    B, Cc, H, W = x.shape
    cpad = cpad or Cc
    assert x.dtype in (torch.float32, bf16) and x.is_contiguous()
    y = torch.empty((B, H, W, cpad), dtype=bf16, device=x.device)
    launch(lib().geeps_nchw_to_nhwc_bf16, "nchw_to_nhwc", ptr(x), int(x.dtype == bf16), ptr(y), B, Cc, H, W, cpad,
           stream_ptr())
    return y


def nchw_to_s2d_bf16(x: torch.Tensor, y: torch.Tensor, S: int) -> torch.Tensor:
    """NCHW (fp32 or bf16) -> space-to-depth NHWC bf16: y[b, hs, ws, (dy*S + dx)*C + c] = x[b, c, hs*S + dy, ws*S + dx]."""
    L.require_cuda()
    B, Cc, H, W = x.shape
    _, Hs, Ws, cpad = y.shape
    assert x.dtype in (torch.float32, bf16) and y.dtype == bf16 and x.is_contiguous() and y.is_contiguous()
    launch(lib().geeps_nchw_to_s2d_bf16, "nchw_to_s2d", ptr(x), int(x.dtype == bf16), ptr(y), B, Cc, H, W, S, Hs, Ws,
           cpad, stream_ptr())
    return y


def u8_transform(x: torch.Tensor, y: torch.Tensor, crop, S: int = 0, aug: torch.Tensor | None = None,
                 mean=(0.0, 0.0, 0.0, 0.0), scale: float = 1.0) -> torch.Tensor:
    """Data transformer on the device: uint8 NCHW source images -> bf16 activations of the crop = (H, W) window, as
    NHWC (S <= 1, y [B, H, W, cpad]) or space-to-depth (y [B, Hs, Ws, cpad]); value = (pixel - mean[c]) * scale.
    aug: None (centre crop, no mirror) or int32 [B, 3] on the device: h_off, w_off, mirror per image."""
    L.require_cuda()
    B, Cc, Hin, Win = x.shape
    H, W = crop
    _, Hs, Ws, cpad = y.shape
    assert x.dtype == torch.uint8 and y.dtype == bf16 and x.is_contiguous() and y.is_contiguous()
    assert aug is None or (aug.dtype == torch.int32 and aug.is_contiguous() and aug.numel() == 3 * B and aug.is_cuda)
    p = L.U8Transform()
    p.x, p.y, p.aug = x.data_ptr(), y.data_ptr(), (aug.data_ptr() if aug is not None else None)
    p.B, p.C, p.Hin, p.Win, p.H, p.W, p.S, p.Hs, p.Ws, p.Cpad = B, Cc, Hin, Win, H, W, S, Hs, Ws, cpad
    m = list(mean) + [0.0] * 4
    for c in range(4):
        p.mean[c] = float(m[c])
    p.scale = float(scale)
    launch(lib().geeps_u8_transform_bf16, "u8_transform", C.byref(p), stream_ptr())
    return y


def col_mask(g: torch.Tensor, mask: torch.Tensor) -> None:
    """Zero the columns of the fp32 matrix g whose mask byte is 0."""
    assert g.dtype == torch.float32 and mask.dtype == torch.uint8 and g.stride(1) == 1
    launch(lib().geeps_col_mask_f32, "col_mask", ptr(g), ptr(mask), C.c_longlong(g.shape[0]), int(mask.numel()),
           C.c_longlong(g.stride(0)), stream_ptr())


def conv_geom(x_shape, c0: int, cg: int, kh: int, kw: int, stride: int, pad: int, ldcol: int) -> ConvGeom:
    B, H, W, Cc = x_shape
    g = ConvGeom()
    g.B, g.H, g.W, g.C, g.c0, g.Cg = B, H, W, Cc, c0, cg
    g.KH, g.KW, g.stride, g.pad = kh, kw, stride, pad
    g.OH = (H + 2 * pad - kh) // stride + 1
    g.OW = (W + 2 * pad - kw) // stride + 1
    g.ldcol = ldcol
    return g


def im2col(x: torch.Tensor, col: torch.Tensor, g: ConvGeom) -> None:
    launch(lib().geeps_im2col, "im2col", ptr(x), ptr(col), C.byref(g), stream_ptr())


def col2im(dcol: torch.Tensor, dx: torch.Tensor, g: ConvGeom, accumulate: bool = False) -> None:
    launch(lib().geeps_col2im, "col2im", ptr(dcol), ptr(dx), C.byref(g), int(accumulate), stream_ptr())


def bn_forward(x2d, y2d, gamma, beta, sums, mean_rstd, running_mean, running_var, eps=1e-5, momentum=0.1,
               relu=False) -> None:
    P, Cc = x2d.shape
    launch(lib().geeps_bn_forward, "bn_forward", ptr(x2d), ptr(y2d), ptr(gamma), ptr(beta), ptr(sums), ptr(mean_rstd),
                                 ptr(running_mean), ptr(running_var), C.c_longlong(P), Cc,
                                 C.c_longlong(_ld(x2d)), C.c_longlong(_ld(y2d)), C.c_float(eps),
                                 C.c_float(momentum), int(relu), stream_ptr())


def bn_backward(x2d, dy2d, y2d, dx2d, mean_rstd, gamma, sums, dgamma, dbeta, relu=False, grad_scale=1.0) -> None:
    P, Cc = x2d.shape
    launch(lib().geeps_bn_backward, "bn_backward", ptr(x2d), ptr(dy2d), ptr(y2d), ptr(dx2d), ptr(mean_rstd), ptr(gamma), ptr(sums),
                                  ptr(dgamma), ptr(dbeta), C.c_longlong(P), Cc, C.c_longlong(_ld(x2d)),
                                  C.c_longlong(_ld(dy2d)), C.c_longlong(_ld(dx2d)), int(relu),
                                  C.c_float(grad_scale), stream_ptr())


def bn_forward_fused(x2d, y2d, gamma, beta, sums, mean_rstd, running_mean, running_var, zero_after=None, barrier=None,
                     eps=1e-5, momentum=0.1, relu=False) -> None:
    """BatchNorm forward in two launches, or one with `barrier` (4 int32, zero at first use, private to the layer and
    direction): `sums` (2 C floats) must be zero on entry, `zero_after` is zeroed for the layer's next reduction (its
    backward scratch)."""
    P, Cc = x2d.shape
    launch(lib().geeps_bn_forward_fused, "bn_forward_fused", ptr(x2d), ptr(y2d), ptr(gamma), ptr(beta), ptr(sums),
           ptr(mean_rstd), ptr(running_mean), ptr(running_var), ptr(zero_after) if zero_after is not None else None,
           ptr(barrier) if barrier is not None else None, C.c_longlong(P), Cc, C.c_longlong(_ld(x2d)), C.c_longlong(_ld(y2d)), C.c_float(eps), C.c_float(momentum),
           int(relu), stream_ptr())


def bn_backward_fused(x2d, dy2d, y2d, dx2d, mean_rstd, gamma, sums, dgamma, dbeta, zero_after=None, barrier=None,
                      relu=False, grad_scale=1.0) -> None:
    """BatchNorm backward in two launches (one with `barrier`): `sums` must be zero on entry, `zero_after` (the forward
    scratch) is zeroed."""
    P, Cc = x2d.shape
    launch(lib().geeps_bn_backward_fused, "bn_backward_fused", ptr(x2d), ptr(dy2d), ptr(y2d), ptr(dx2d), ptr(mean_rstd),
           ptr(gamma), ptr(sums), ptr(dgamma), ptr(dbeta), ptr(zero_after) if zero_after is not None else None,
           ptr(barrier) if barrier is not None else None, C.c_longlong(P), Cc, C.c_longlong(_ld(x2d)), C.c_longlong(_ld(dy2d)), C.c_longlong(_ld(dx2d)), int(relu),
           C.c_float(grad_scale), stream_ptr())


def colsum(x2d, out, scale=1.0, zero_first=True) -> None:
    P, Cc = x2d.shape
    launch(lib().geeps_colsum, "colsum", ptr(x2d), ptr(out), C.c_longlong(P), Cc, C.c_longlong(_ld(x2d)), C.c_float(scale),
                             int(zero_first), stream_ptr())


def relu_backward(dy, y, dx) -> None:
    assert dy.is_contiguous() and y.is_contiguous() and dx.is_contiguous()
    launch(lib().geeps_relu_backward, "relu_backward", ptr(dy), ptr(y), ptr(dx), C.c_longlong(dy.numel()), stream_ptr())


def relu_backward_2d(dy2d, y2d, dx2d) -> None:
    P, Cc = dy2d.shape
    launch(lib().geeps_relu_backward_2d, "relu_backward_2d", ptr(dy2d), ptr(y2d), ptr(dx2d), C.c_longlong(P), Cc, C.c_longlong(_ld(dy2d)),
                                       C.c_longlong(_ld(y2d)), C.c_longlong(_ld(dx2d)), stream_ptr())


def relu_backward_colsum(dy2d, y2d, dx2d, colsum_out) -> None:
    """dx = dy where y > 0 else 0, and colsum_out[c] = sum of dx over the rows, in one pass."""
    P, Cc = dy2d.shape
    assert colsum_out.dtype == torch.float32 and colsum_out.numel() == Cc and colsum_out.is_contiguous()
    launch(lib().geeps_relu_backward_colsum, "relu_backward_colsum", ptr(dy2d), ptr(y2d), ptr(dx2d), ptr(colsum_out),
           C.c_longlong(P), Cc, C.c_longlong(_ld(dy2d)), C.c_longlong(_ld(y2d)), C.c_longlong(_ld(dx2d)), stream_ptr())


def stream_order(src_stream, dst_stream, event) -> None:
    """Everything enqueued on dst_stream from now on waits for what src_stream holds now (`event`: a handle from
    new_event()).  Recorded like a launch, so forks and joins of network branches replay and capture with the step."""
    L.record_call(lib().geeps_stream_order, "stream_order", C.c_void_p(src_stream.cuda_stream),
                  C.c_void_p(dst_stream.cuda_stream), C.c_void_p(event))


def new_event() -> int:
    lib().geeps_event_new.restype = C.c_void_p
    return int(lib().geeps_event_new())


def add_2d(dst2d, src2d) -> None:
    P, Cc = dst2d.shape
    launch(lib().geeps_add_bf16_2d, "add_bf16_2d", ptr(dst2d), ptr(src2d), C.c_longlong(P), Cc, C.c_longlong(_ld(dst2d)),
                                  C.c_longlong(_ld(src2d)), stream_ptr())


def f32_to_bf16_2d(src2d, dst2d, relu: bool = False) -> None:
    """dst (bf16) = src (fp32), optionally through ReLU; both may be column slices of wider matrices."""
    P, Cc = src2d.shape
    assert src2d.dtype == torch.float32 and dst2d.dtype == bf16 and dst2d.shape == src2d.shape
    launch(lib().geeps_f32_to_bf16_2d, "f32_to_bf16_2d", ptr(src2d), ptr(dst2d), C.c_longlong(P), Cc,
           C.c_longlong(_ld(src2d)), C.c_longlong(_ld(dst2d)), int(relu), stream_ptr())


def dropout(x, y, p: float, seed: int, step_ref: int | None = None) -> None:
    """step_ref: address of a device int added to the seed when the kernel runs (the launch arguments then do not
    change from step to step)."""
    assert x.is_contiguous() and y.is_contiguous()
    if step_ref:
        launch(lib().geeps_dropout_ref, "dropout_ref", ptr(x), ptr(y), C.c_longlong(x.numel()), C.c_float(p),
               C.c_ulonglong(seed), C.c_void_p(step_ref), stream_ptr())
        return
    launch(lib().geeps_dropout, "dropout", ptr(x), ptr(y), C.c_longlong(x.numel()), C.c_float(p), C.c_ulonglong(seed),
                              stream_ptr())


def lrn_forward(x2d, y2d, scale, size=5, alpha=1e-4, beta=0.75, k=1.0) -> None:
    """scale: bf16 [P, C] buffer that receives 1 / (k + alpha/size * window sum of x^2) for lrn_backward."""
    assert scale.dtype == bf16
    P, Cc = x2d.shape
    assert x2d.is_contiguous() and y2d.is_contiguous()
    launch(lib().geeps_lrn_forward, "lrn_forward", ptr(x2d), ptr(y2d), ptr(scale), C.c_longlong(P), Cc, size, C.c_float(alpha),
                                  C.c_float(beta), C.c_float(k), stream_ptr())


def lrn_backward(x2d, y2d, scale, dy2d, dx2d, size=5, alpha=1e-4, beta=0.75, relu_mask=False, colsum=None) -> None:
    """relu_mask: x2d is a ReLU output whose backward is folded in (dx = 0 where x <= 0).
    colsum: optional fp32 [C] tensor that receives the per-channel sums of dx (the bias gradient of the layer
    that produced x2d)."""
    assert scale.dtype == bf16
    assert colsum is None or (colsum.dtype == torch.float32 and colsum.numel() == x2d.shape[1])
    P, Cc = x2d.shape
    launch(lib().geeps_lrn_backward, "lrn_backward", ptr(x2d), ptr(y2d), ptr(scale), ptr(dy2d), ptr(dx2d), C.c_longlong(P), Cc, size,
           C.c_float(alpha), C.c_float(beta), int(relu_mask), ptr(colsum) if colsum is not None else None, stream_ptr())


def copy_f32(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst[:] = src for contiguous fp32 tensors of the same size (device-to-device, on the current stream)."""
    assert dst.dtype == torch.float32 and src.dtype == torch.float32 and dst.numel() == src.numel()
    assert dst.is_contiguous() and src.is_contiguous()
    launch(lib().geeps_copy_f32, "copy_f32", ptr(dst), ptr(src), C.c_longlong(dst.numel()), stream_ptr())


def pool_geom(x_shape, k: int, stride: int, pad: int, ldx: int, ldy: int, ceil_mode: bool = True) -> PoolGeom:
    B, H, W, Cc = x_shape
    g = PoolGeom()
    g.B, g.H, g.W, g.C, g.K, g.stride, g.pad = B, H, W, Cc, k, stride, pad

    def osz(n):
        num = n + 2 * pad - k
        o = (-(-num // stride) if ceil_mode else num // stride) + 1
        if pad > 0 and (o - 1) * stride >= n + pad:
            o -= 1
        return o

    g.OH, g.OW = osz(H), osz(W)
    g.ldx, g.ldy = ldx, ldy
    return g


def maxpool_forward(x, y, argmax, g: PoolGeom) -> None:
    launch(lib().geeps_maxpool_forward, "maxpool_forward", ptr(x), ptr(y), ptr(argmax), C.byref(g), stream_ptr())


def maxpool_backward(dy, argmax, dx, g: PoolGeom, accumulate=False) -> None:
    launch(lib().geeps_maxpool_backward, "maxpool_backward", ptr(dy), ptr(argmax), ptr(dx), C.byref(g), int(accumulate), stream_ptr())


def lrn_maxpool_supported(g: PoolGeom, size: int) -> bool:
    return bool(lib().geeps_lrn_maxpool_supported(C.byref(g), int(size)))


def lrn_maxpool_forward(x, p, argmax, g: PoolGeom, size=5, alpha=1e-4, beta=0.75, k=1.0) -> None:
    """p = maxpool(LRN(x)) in one kernel; argmax receives the window codes (the only thing the backward needs
    besides x)."""
    assert x.is_contiguous() and x.dtype == bf16
    launch(lib().geeps_lrn_maxpool_forward, "lrn_maxpool_forward", ptr(x), ptr(p), ptr(argmax), C.byref(g), int(size),
           C.c_float(alpha), C.c_float(beta), C.c_float(k), stream_ptr())


def lrn_maxpool_backward(x, dp, argmax, dx, g: PoolGeom, size=5, alpha=1e-4, beta=0.75, k=1.0, relu_mask=False,
                         colsum=None) -> None:
    """dx = gradient w.r.t. x of maxpool(LRN(x)) given dp; relu_mask zeroes it where x <= 0; colsum (fp32 [C])
    receives the per-channel sums of dx."""
    assert x.is_contiguous() and dx.is_contiguous()
    assert colsum is None or (colsum.dtype == torch.float32 and colsum.numel() == g.C)
    launch(lib().geeps_lrn_maxpool_backward, "lrn_maxpool_backward", ptr(x), ptr(dp), ptr(argmax), ptr(dx), C.byref(g),
           int(size), C.c_float(alpha), C.c_float(beta), C.c_float(k), int(relu_mask),
           ptr(colsum) if colsum is not None else None, stream_ptr())


def avgpool_forward(x, y, g: PoolGeom) -> None:
    launch(lib().geeps_avgpool_forward, "avgpool_forward", ptr(x), ptr(y), C.byref(g), stream_ptr())


def avgpool_backward(dy, dx, g: PoolGeom, accumulate=False) -> None:
    launch(lib().geeps_avgpool_backward, "avgpool_backward", ptr(dy), ptr(dx), C.byref(g), int(accumulate), stream_ptr())


def softmax_ce(logits, labels, loss_sum, dlogits, per_sample=None, loss_scale=1.0, grad_scale=1.0, zero_loss=True,
               status=None) -> None:
    B, Cc = logits.shape
    assert logits.dtype == torch.float32 and labels.dtype == torch.int64
    launch(lib().geeps_softmax_ce, "softmax_ce", ptr(logits), ptr(labels), ptr(loss_sum), ptr(per_sample), ptr(dlogits), B, Cc,
                                 C.c_longlong(_ld(logits)), C.c_longlong(_ld(dlogits) if dlogits is not None else 0),
                                 C.c_float(loss_scale), C.c_float(grad_scale), int(zero_loss), ptr(status),
                                 stream_ptr())


def f32_to_bf16(src, dst) -> None:
    launch(lib().geeps_f32_to_bf16, "f32_to_bf16", ptr(src), ptr(dst), C.c_longlong(src.numel()), stream_ptr())


def axpy(y, x, alpha: float) -> None:
    launch(lib().geeps_axpy, "axpy", ptr(y), ptr(x), C.c_float(alpha), C.c_longlong(y.numel()), stream_ptr())


def _row_op(fn, name, dst, src, index, dst_off, src_off, num_vals_limit, status):
    n = index.shape[0]
    lim = num_vals_limit if num_vals_limit is not None else (1 << 62)
    launch(fn, name, ptr(dst), ptr(src), ptr(index), C.c_longlong(n), C.c_longlong(dst_off), C.c_longlong(src_off),
           C.c_longlong(lim), C.c_longlong(dst.shape[0]), C.c_longlong(src.shape[0]), ptr(status), stream_ptr())


def row_gather(dst, src, index, dst_off=0, src_off=0, num_vals_limit=None, status=None) -> None:
    """dst[id0 + dst_off] = src[id1 + src_off] for each (id0, id1) in index (int64 [n,2])."""
    _row_op(lib().geeps_row_gather, "row_gather", dst, src, index, dst_off, src_off, num_vals_limit, status)


def row_scatter(dst, src, index, dst_off=0, src_off=0, num_vals_limit=None, status=None) -> None:
    """dst[id1 + dst_off] = src[id0 + src_off]."""
    _row_op(lib().geeps_row_scatter, "row_scatter", dst, src, index, dst_off, src_off, num_vals_limit, status)


def row_scatter_add(dst, src, index, dst_off=0, src_off=0, num_vals_limit=None, status=None) -> None:
    """dst[id1 + dst_off] += src[id0 + src_off]."""
    _row_op(lib().geeps_row_scatter_add, "row_scatter_add", dst, src, index, dst_off, src_off, num_vals_limit, status)


def pull_gemm(x, w_shard_ptrs, n_start, out, *, ldw, bias=None, relu=False, ready_ptrs=None, needed_stamp=0,
              w_local=None, status=None, wait_budget_ns=2_000_000_000, block_n=0) -> torch.Tensor:
    """out[M,N] = x[M,K] @ W[N,K]^T (+bias, ReLU) where W's rows are pulled from the shards while the
    GEMM runs.  w_shard_ptrs[s]: device address (local or peer) of shard s's bf16 rows
    [n_start[s], n_start[s+1]); ready_ptrs[s]: address of the int flag that must reach needed_stamp."""
    L.require_cuda()
    M, K = x.shape
    N = out.shape[1]
    p = L.PullGemmParams()
    p.X, p.Y, p.bias = x.data_ptr(), out.data_ptr(), (bias.data_ptr() if bias is not None else None)
    for s, a in enumerate(w_shard_ptrs):
        p.w_shard[s] = a
        p.ready[s] = ready_ptrs[s] if ready_ptrs is not None else None
    for s, v in enumerate(n_start):
        p.n_start[s] = v
    p.n_start[len(w_shard_ptrs)] = N
    p.w_local = w_local.data_ptr() if w_local is not None else None
    p.status = status.data_ptr() if status is not None else None
    p.M, p.N, p.K = M, N, K
    p.ldx, p.ldw, p.ldy = _ld(x), ldw, _ld(out)
    p.wait_budget_ns = wait_budget_ns
    p.n_shards, p.needed_stamp, p.relu = len(w_shard_ptrs), needed_stamp, int(relu)
    p.out_fp32 = int(out.dtype == torch.float32)
    p.block_n = block_n
    launch(lib().geeps_pull_gemm_bf16, "pull_gemm_bf16", C.byref(p), stream_ptr())
    return out
