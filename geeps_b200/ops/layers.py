"""Caffe-style layers with explicit forward / backward on the native kernels.

Activations are NHWC bf16 tensors with static shapes; every buffer is allocated once at
setup and reused each step.  Parameters are NOT owned by the layers: the parameter-server
module binds, per step, fp32 views of the rows it Read (`p32`), bf16 compute copies (`p16`) and
fp32 views of the PreUpdate buffers the gradients are written into (`g32`).

The reference's layer code lived in its (absent) Caffe application; layer definitions here
follow Caffe's AlexNet / Inception-BN usage: conv with groups, LRN across channels, ceil-mode
max pooling, BatchNorm + scale, inner product, softmax loss.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from . import functional as F

BF = torch.bfloat16
# stride-1 convolutions as implicit GEMM (GEEPS_IMPLICIT_CONV=0 keeps the im2col + GEMM + col2im formulation)
IMPLICIT_CONV = os.environ.get("GEEPS_IMPLICIT_CONV", "1") != "0"
# fully-connected layers at batch <= 256 split their k range over the SMs (GEEPS_SPLIT_K_LINEAR=0: one wide tile row)
SPLIT_K_LINEAR = os.environ.get("GEEPS_SPLIT_K_LINEAR", "0") != "0"


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclass
class ParamSpec:
    name: str
    shape: tuple          # stored shape (may include K padding)
    init: str             # "gaussian:<std>", "msra:<fan_in>", "const:<v>"
    valid_cols: int = 0   # for 2-D weights: columns [valid_cols, shape[1]) are padding and stay zero
    decay: bool = True
    col_mask: object = None   # optional bool tensor [shape[1]]: columns that are real parameters (others stay zero)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def initial(self, gen: torch.Generator) -> torch.Tensor:
        kind, _, arg = self.init.partition(":")
        if kind == "const":
            return torch.full(self.shape, float(arg))
        std = float(arg) if kind == "gaussian" else math.sqrt(2.0 / float(arg))
        t = torch.randn(self.shape, generator=gen) * std
        if self.valid_cols and len(self.shape) == 2:
            t[:, self.valid_cols:] = 0
        if self.col_mask is not None:
            t[:, ~self.col_mask] = 0
        return t

    def num_valid(self) -> int:
        """Number of real parameters (padding and masked columns excluded)."""
        if len(self.shape) != 2:
            return self.numel
        if self.col_mask is not None:
            return self.shape[0] * int(self.col_mask.sum())
        return self.shape[0] * (self.valid_cols or self.shape[1])


class Layer:
    name = "layer"

    def __init__(self):
        self.p32, self.p16, self.g32 = {}, {}, {}
        self.training = True

    def param_specs(self) -> list:
        return []

    def setup(self, in_shape, device):
        raise NotImplementedError

    def forward(self, x):
        raise NotImplementedError

    def backward(self, dy):
        raise NotImplementedError

    # ---- hooks for activations managed by the parameter server's memory plan ----
    def out_numel(self) -> int:
        n = 1
        for s_ in self.out_shape:
            n *= s_
        return n

    def set_output(self, flat: "torch.Tensor") -> None:
        """Use `flat` (bf16, >= out_numel elements) as this layer's output buffer from now on."""
        self.y = flat[:self.out_numel()].view(-1, self.out_shape[-1])

    def set_input(self, x: "torch.Tensor") -> None:
        """The input this layer saved in forward now lives in `x` (it was evicted and fetched back)."""
        if hasattr(self, "x"):
            self.x = x.view(self.x.shape) if x.numel() == self.x.numel() else x


class Input(Layer):
    """NCHW batch -> NHWC bf16 (optionally zero-padding the channel count).  The batch is fp32 or bf16 (values as
    they are), or uint8 source images that this layer crops, mirrors, mean-subtracts and scales on the device."""

    def __init__(self, cpad: int | None = None, s2d: int = 0, s2d_k: int = 0, mean=(0.0, 0.0, 0.0), scale: float = 1.0):
        """s2d = S > 0: emit the space-to-depth layout [B, Hs, Ws, S*S*C] that turns the following k x k
        stride-S convolution (k = s2d_k, no padding) into a stride-1 convolution with ceil(k/S) taps.  cpad widens
        the pixel with zero channels (48 -> 64 makes every pixel one aligned 128-byte line, which the TMA loads of
        the convolution reward: 0.26 -> 0.14 ms on the box kernel at batch 256).
        mean, scale: for uint8 batches, value = (pixel - mean[channel]) * scale (Caffe's mean_value / scale)."""
        super().__init__()
        self.cpad, self.s2d, self.s2d_k = cpad, s2d, s2d_k
        self.mean, self.scale = tuple(mean), float(scale)
        self.aug = None            # int32 [B, 3] on the device: h_off, w_off, mirror of every image (uint8 batches)
        self._src_hw = None        # source image size of the last uint8 batch that went through forward
        self._centre = True        # aug holds the centre crop (no set_augmentation call in force)

    def setup(self, in_shape, device):
        B, C, H, W = in_shape
        self.in_shape, self.device = tuple(in_shape), device
        if self.s2d:
            S, k = self.s2d, self.s2d_k
            taps = -(-k // S)
            Hs, Ws = (H - k) // S + taps, (W - k) // S + taps
            self.out_shape = (B, Hs, Ws, self.cpad or _pad8(S * S * C))
            self.y = torch.empty(self.out_shape, dtype=BF, device=device)
        else:
            self.out_shape = (B, H, W, self.cpad or C)
        return self.out_shape

    def set_transform(self, mean, scale: float) -> None:
        """Mean per channel and scale applied to uint8 batches (takes effect on steps not yet recorded or captured)."""
        self.mean, self.scale = tuple(mean), float(scale)

    def _centre_crop(self) -> None:
        B, _, H, W = self.in_shape
        centre = torch.tensor([(self._src_hw[0] - H) // 2, (self._src_hw[1] - W) // 2, 0], dtype=torch.int32)
        self.aug.copy_(centre.to(self.device).expand(B, 3))

    def set_augmentation(self, aug: "torch.Tensor | None") -> None:
        """Crop offsets and mirror flags of the next uint8 batch: int [B, 3] (h_off, w_off, mirror), host or device.
        The values land in a buffer this layer owns (the one every uint8 step reads, recorded and captured steps
        included).  None goes back to the centre crop without mirroring."""
        B = self.in_shape[0]
        self._centre = aug is None
        if aug is None:
            if self.aug is not None and self._src_hw is not None:
                self._centre_crop()
            return
        if self.aug is None:
            self.aug = torch.zeros(B, 3, dtype=torch.int32, device=self.device)
        self.aug.copy_(aug.to(torch.int32).reshape(B, 3), non_blocking=True)

    def randomize(self, src_hw, mirror: bool = True, generator=None) -> None:
        """Random crop window (and mirror flag) per image for source images of size src_hw, drawn on the device."""
        B, _, H, W = self.in_shape
        Hin, Win = src_hw
        dev = self.device
        a = torch.stack([torch.randint(0, Hin - H + 1, (B,), device=dev, generator=generator),
                         torch.randint(0, Win - W + 1, (B,), device=dev, generator=generator),
                         torch.randint(0, 2 if mirror else 1, (B,), device=dev, generator=generator)], dim=1)
        self.set_augmentation(a)

    def forward(self, x):
        if x.dtype == BF and tuple(x.shape) == tuple(self.out_shape) and x.is_contiguous():
            return x           # already in this layer's output layout (HostFeeder(layout=...) converts while it copies)
        if x.dtype == torch.uint8:
            B, C, H, W = self.in_shape
            src_hw = (int(x.shape[2]), int(x.shape[3]))
            if self.aug is None:
                self.aug = torch.zeros(B, 3, dtype=torch.int32, device=self.device)
            if self._centre and src_hw != self._src_hw:
                self._src_hw = src_hw
                self._centre_crop()
            self._src_hw = src_hw
            y = self.y if self.s2d else torch.empty(self.out_shape, dtype=BF, device=x.device)
            return F.u8_transform(x, y, (H, W), self.s2d, self.aug, self.mean, self.scale)
        if self.s2d:
            return F.nchw_to_s2d_bf16(x, self.y, self.s2d)
        return F.nchw_to_nhwc_bf16(x, self.cpad)

    def backward(self, dy):
        return None


class Conv2d(Layer):
    def __init__(self, name, cout, k, stride=1, pad=0, groups=1, relu=False, bias=True, std=0.01, bias_value=0.0,
                 need_dx=True, cin_valid=None, s2d=0):
        """s2d = S: the input arrives in space-to-depth layout (Input(s2d=S, s2d_k=k)); the k x k stride-S
        convolution runs as a ceil(k/S)-tap stride-1 convolution whose weight columns for taps past k stay zero.
        cin_valid: the image's own channel count when the space-to-depth pixel is zero-padded past S*S*channels."""
        super().__init__()
        self.s2d, self.orig_k = s2d, k
        self.dy_is_masked = False       # set by Net when the consumer of the output applies this layer's ReLU mask
        self.bias_grad_src = None       # set by Net: the consumer's backward already summed dy per channel into this
        if s2d:
            assert stride == s2d and pad == 0 and groups == 1
            k, stride = -(-k // s2d), 1
        self.name, self.cout, self.k, self.stride, self.pad, self.groups = name, cout, k, stride, pad, groups
        self.relu, self.has_bias, self.std, self.bias_value, self.need_dx = relu, bias, std, bias_value, need_dx
        self.cin_valid = cin_valid

    def setup(self, in_shape, device):
        B, H, W, C = in_shape
        self.in_shape = in_shape
        self.device = device
        G = self.groups
        self.cg, self.og = C // G, self.cout // G
        self.kd = self.k * self.k * self.cg
        self.ld = _pad8(self.kd)
        self.geoms = [F.conv_geom(in_shape, g * self.cg, self.cg, self.k, self.k, self.stride, self.pad, self.ld)
                      for g in range(G)]
        self.OH, self.OW = self.geoms[0].OH, self.geoms[0].OW
        self.M = B * self.OH * self.OW
        self.col_mask = self.col_mask_dev = None
        if self.s2d:
            # column (a*T + b)*Cs + (dy*S + dx)*C0 + c is filter tap (a*S + dy, b*S + dx) of input channel c
            S, T = self.s2d, self.k
            c0 = self.cin_valid or C // (S * S)
            col = torch.arange(self.ld)
            tap, j = col // C, col % C
            kh = (tap // T) * S + (j // c0) // S
            kw = (tap % T) * S + (j // c0) % S
            self.col_mask = (col < self.kd) & (j < S * S * c0) & (kh < self.orig_k) & (kw < self.orig_k)
            self.col_mask_dev = self.col_mask.to(torch.uint8).to(device)
        self.pointwise = self.k == 1 and self.stride == 1 and self.pad == 0 and G == 1 and C % 8 == 0
        # stride-1 layers run as an implicit GEMM (no patch matrix); the final say comes from the kernel's own
        # alignment check on the first forward, when the output binding is known
        self.implicit = (IMPLICIT_CONV and not self.pointwise and 1 <= self.stride <= 8 and self.cg % 8 == 0
                         and self.og % 8 == 0 and C % 8 == 0)
        if self.stride > 1 and self.cg < 32:
            # every tap is a k-step of 64 channels: with 8 channels (the 7 x 7 stride-2 first layer of the 22K net)
            # 49 mostly-zero k-steps lose to 7 dense ones over a patch matrix (6.8 against 5.8 ms per step)
            self.implicit = False
        # a strided layer's forward and weight gradient load the activation boxes with a TMA element stride; its data
        # gradient runs one parity class of dX at a time (stride^2 stride-1 problems with sub-filters), unless the
        # filter is narrower than the stride (then some classes have no taps): GEMM + col2im for those
        self.implicit_dgrad = self.implicit and (self.stride == 1 or self.k >= self.stride)
        self.cols = self.dcol = None
        if not self.pointwise and not self.implicit:
            self._alloc_patch_buffers()
        elif self.implicit and not self.implicit_dgrad and self.need_dx:
            self.dcol = torch.empty(self.M, self.ld, dtype=BF, device=device)
        self.y = None
        self.dx = torch.empty(in_shape, dtype=BF, device=device) if self.need_dx else None
        self.out_shape = (B, self.OH, self.OW, self.cout)
        self.device = device
        return self.out_shape

    def _alloc_patch_buffers(self):
        self.cols = [torch.empty(self.M, self.ld, dtype=BF, device=self.device) for _ in range(self.groups)]
        self.dcol = torch.empty(self.M, self.ld, dtype=BF, device=self.device) if self.need_dx else None

    def _x4(self, x, g):
        B, H, W, C = self.in_shape
        return x.view(B, H, W, C)[..., g * self.cg:(g + 1) * self.cg]

    def _y4(self, y2d, g):
        B = self.in_shape[0]
        return y2d.unflatten(0, (B, self.OH, self.OW))[..., g * self.og:(g + 1) * self.og]

    def param_specs(self):
        fan_in = int(self.col_mask.sum()) if self.col_mask is not None else self.kd
        specs = [ParamSpec("weight", (self.cout, self.ld), f"gaussian:{self.std}" if self.std > 0 else f"msra:{fan_in}",
                           valid_cols=self.kd, col_mask=self.col_mask)]
        if self.has_bias:
            specs.append(ParamSpec("bias", (self.cout,), f"const:{self.bias_value}", decay=False))
        return specs

    def bind_output(self, y2d):
        """Write the output into a channel slice of a wider (concat) tensor."""
        self.y = y2d

    def forward(self, x):
        self.x = x
        if self.y is None:
            self.y = torch.empty(self.M, self.cout, dtype=BF, device=self.device)
        w16 = self.p16["weight"]
        bias = self.p32.get("bias")
        if self.implicit and self.cols is None and not getattr(self, "_implicit_checked", False):
            self._implicit_checked = True
            ok = all(F.conv_tc_supported(F.conv_tc_params(F.CONV_FWD, self._x4(x, g), self._y4(self.y, g),
                                                          w16[g * self.og:(g + 1) * self.og], self.k, self.pad,
                                                          stride=self.stride))
                     for g in range(self.groups))
            if not ok:
                self.implicit = False
                self._alloc_patch_buffers()
        for g in range(self.groups):
            if self.implicit:
                F.conv_tc(F.CONV_FWD, self._x4(x, g), self._y4(self.y, g), w16[g * self.og:(g + 1) * self.og],
                          self.k, self.pad, bias=None if bias is None else bias[g * self.og:(g + 1) * self.og],
                          relu=self.relu, stride=self.stride)
                continue
            if self.pointwise:
                a = x.view(self.M, -1)
            else:
                F.im2col(x, self.cols[g], self.geoms[g])
                a = self.cols[g]
            F.gemm(a, w16[g * self.og:(g + 1) * self.og], self.y[:, g * self.og:(g + 1) * self.og],
                   bias=None if bias is None else bias[g * self.og:(g + 1) * self.og], relu=self.relu)
        return self.y

    def backward(self, dy):
        # dy: [M, cout] bf16 (possibly a slice view of a wider tensor)
        if dy.dim() != 2:
            dy = dy.view(self.M, self.cout)
        bias_done = False
        if self.relu and not self.dy_is_masked:
            if self.has_bias and self.bias_grad_src is None and self.cout % 8 == 0 and self.cout <= 8192:
                dy = self._relu_mask(dy, colsum=self.g32["bias"])     # mask and bias gradient in one pass
                bias_done = True
            else:
                dy = self._relu_mask(dy)
        gw = self.g32["weight"]
        if self.has_bias and not bias_done:
            if self.bias_grad_src is not None:
                F.copy_f32(self.g32["bias"], self.bias_grad_src)
            else:
                F.colsum(dy, self.g32["bias"])
        w16 = self.p16["weight"]
        for g in range(self.groups):
            if self.implicit:
                xg, dy4 = self._x4(self.x, g), self._y4(dy, g)
                F.conv_tc(F.CONV_WGRAD, xg, dy4, gw[g * self.og:(g + 1) * self.og], self.k, self.pad,
                          stride=self.stride)
                if self.need_dx and self.implicit_dgrad:
                    F.conv_tc(F.CONV_DGRAD, self._x4(self.dx, g), dy4, w16[g * self.og:(g + 1) * self.og],
                              self.k, self.pad, stride=self.stride)
                elif self.need_dx:
                    F.gemm(dy[:, g * self.og:(g + 1) * self.og], w16[g * self.og:(g + 1) * self.og], self.dcol, b_mn=True)
                    F.col2im(self.dcol, self.dx, self.geoms[g])
                continue
            dyg = dy[:, g * self.og:(g + 1) * self.og]
            a = self.x.view(self.M, -1) if self.pointwise else self.cols[g]
            # dW_g[og, ld] = dy_g^T @ col_g      (both operands stored K-outermost)
            F.gemm(dyg, a, gw[g * self.og:(g + 1) * self.og], a_mn=True, b_mn=True, split_k=0)
            if self.need_dx:
                wg = w16[g * self.og:(g + 1) * self.og]
                if self.pointwise:
                    F.gemm(dyg, wg, self.dx.view(self.M, -1), b_mn=True)
                else:
                    F.gemm(dyg, wg, self.dcol, b_mn=True)
                    F.col2im(self.dcol, self.dx, self.geoms[g])
        if self.col_mask_dev is not None:
            F.col_mask(gw, self.col_mask_dev)
        return self.dx

    def _relu_mask(self, dy, colsum=None):
        if not hasattr(self, "_dy_masked"):
            self._dy_masked = torch.empty(self.M, self.cout, dtype=BF, device=self.device)
        if colsum is not None:
            F.relu_backward_colsum(dy, self.y, self._dy_masked, colsum)
        else:
            F.relu_backward_2d(dy, self.y, self._dy_masked)
        return self._dy_masked


class Linear(Layer):
    def __init__(self, name, out_features, relu=False, std=0.01, bias_value=0.0, need_dx=True, fp32_out=False):
        super().__init__()
        self.name, self.out, self.relu, self.std, self.bias_value = name, out_features, relu, std, bias_value
        self.need_dx, self.fp32_out = need_dx, fp32_out

    def setup(self, in_shape, device):
        self.in_shape = in_shape
        B = in_shape[0]
        self.B = B
        self.k_in = 1
        for s in in_shape[1:]:
            self.k_in *= s
        self.ld = _pad8(self.k_in)
        assert self.ld == self.k_in, "Linear input width must be a multiple of 8"
        self.out_ld = _pad8(self.out)
        ybuf = torch.zeros(B, self.out_ld, dtype=torch.float32 if self.fp32_out else BF, device=device)
        self.y = ybuf[:, :self.out]
        self.dx = torch.empty(B, self.k_in, dtype=BF, device=device) if self.need_dx else None
        self.device = device
        self.out_shape = (B, self.out)
        return self.out_shape

    def param_specs(self):
        return [ParamSpec("weight", (self.out, self.ld), f"gaussian:{self.std}", valid_cols=self.k_in),
                ParamSpec("bias", (self.out,), f"const:{self.bias_value}", decay=False)]

    def forward(self, x):
        self.x = x.reshape(self.B, self.k_in)
        pull = getattr(self, "pull", None)
        if pull:
            # uncached table: the weight rows are read from the owning shards while the GEMM runs; p16["weight"]
            # receives the local bf16 copy that the backward pass uses
            shards, n_start = pull
            F.pull_gemm(self.x, shards, n_start, self.y, ldw=self.ld, bias=self.p32["bias"], relu=self.relu,
                        w_local=self.p16["weight"])
        elif self._split_k():
            # batch-sized M: two or four wide output tiles would leave most SMs idle while the weights stream, so the
            # k range is split over the SMs (partial sums reduce-added in fp32) and a finishing pass converts
            if self.fp32_out:
                F.gemm(self.x, self.p16["weight"], self.y, bias=self.p32["bias"], split_k=0)
            else:
                ws = self._workspace(self.out_ld)[:, :self.out]
                F.gemm(self.x, self.p16["weight"], ws, bias=self.p32["bias"], split_k=0)
                F.f32_to_bf16_2d(ws, self.y, relu=self.relu)
        else:
            F.gemm(self.x, self.p16["weight"], self.y, bias=self.p32["bias"], relu=self.relu)
        return self.y

    def _split_k(self) -> bool:
        return SPLIT_K_LINEAR and self.B <= 256 and self.out % 8 == 0

    def _workspace(self, width):
        """fp32 [B, width] scratch shared by the forward and the data gradient of this layer."""
        w = max(self.out_ld, self.k_in)
        if getattr(self, "_ws", None) is None:
            self._ws = torch.empty(self.B, w, dtype=torch.float32, device=self.device)
        return self._ws.view(-1)[:self.B * width].view(self.B, width)

    def backward(self, dy):
        if self.relu:
            if not hasattr(self, "_dym"):
                self._dym = torch.empty(self.B, self.out_ld, dtype=BF, device=self.device)[:, :self.out]
            if self.out % 8 == 0 and self.out <= 8192:
                F.relu_backward_colsum(dy, self.y, self._dym, self.g32["bias"])
            else:
                F.relu_backward_2d(dy, self.y, self._dym)
                F.colsum(self._dym, self.g32["bias"])
            dy = self._dym
        else:
            F.colsum(dy, self.g32["bias"])
        # dW[out, in] = dy^T @ x ; dx[B, in] = dy @ W
        F.gemm(dy, self.x, self.g32["weight"], a_mn=True, b_mn=True, split_k=0)
        if self.need_dx:
            if self._split_k():
                ws = self._workspace(self.k_in)
                F.gemm(dy, self.p16["weight"], ws, b_mn=True, split_k=0)
                F.f32_to_bf16_2d(ws, self.dx)
            else:
                F.gemm(dy, self.p16["weight"], self.dx, b_mn=True)
            return self.dx.view(self.in_shape)
        return None


class BatchNorm(Layer):
    def __init__(self, name, relu=False, eps=1e-5, momentum=0.1):
        super().__init__()
        self.name, self.relu, self.eps, self.momentum = name, relu, eps, momentum

    def setup(self, in_shape, device):
        self.in_shape = in_shape
        self.C = in_shape[-1]
        self.P = 1
        for s in in_shape[:-1]:
            self.P *= s
        # reduction scratch of the two directions: each kernel pair leaves the other direction's scratch zeroed, so a
        # training loop (forward, backward, forward, ...) needs no memset in front of a reduction
        self.sums = torch.zeros(2 * self.C, device=device)
        self.sums_b = torch.zeros(2 * self.C, device=device)
        self._clean_f = self._clean_b = True
        self.bar = torch.zeros(8, dtype=torch.int32, device=device)      # grid-barrier words: forward [0:4], backward [4:8]
        self.mean_rstd = torch.empty(2 * self.C, device=device)
        self.running_mean = torch.zeros(self.C, device=device)
        self.running_var = torch.ones(self.C, device=device)
        self.y = torch.empty(self.P, self.C, dtype=BF, device=device)
        self.dx = torch.empty(self.P, self.C, dtype=BF, device=device)
        self.out_shape = in_shape
        return in_shape

    def param_specs(self):
        return [ParamSpec("gamma", (self.C,), "const:1.0", decay=False),
                ParamSpec("beta", (self.C,), "const:0.0", decay=False)]

    def bind_output(self, y2d):
        self.y = y2d

    def forward(self, x):
        self.x = x if x.dim() == 2 else x.view(self.P, self.C)
        if not self._clean_f:       # two forward passes in a row (no backward in between zeroed the scratch)
            F.bn_forward(self.x, self.y, self.p32["gamma"], self.p32["beta"], self.sums, self.mean_rstd,
                         self.running_mean, self.running_var, eps=self.eps, momentum=self.momentum, relu=self.relu)
            return self.y
        F.bn_forward_fused(self.x, self.y, self.p32["gamma"], self.p32["beta"], self.sums, self.mean_rstd,
                           self.running_mean, self.running_var, zero_after=self.sums_b, barrier=self.bar[0:4],
                           eps=self.eps,
                           momentum=self.momentum, relu=self.relu)
        self._clean_f, self._clean_b = False, True
        return self.y

    def backward(self, dy):
        if dy.dim() != 2:
            dy = dy.view(self.P, self.C)
        if not self._clean_b:
            F.bn_backward(self.x, dy, self.y, self.dx, self.mean_rstd, self.p32["gamma"], self.sums_b, self.g32["gamma"],
                          self.g32["beta"], relu=self.relu)
            return self.dx
        F.bn_backward_fused(self.x, dy, self.y, self.dx, self.mean_rstd, self.p32["gamma"], self.sums_b,
                            self.g32["gamma"], self.g32["beta"], zero_after=self.sums, barrier=self.bar[4:8],
                            relu=self.relu)
        self._clean_b, self._clean_f = False, True
        return self.dx


class LRN(Layer):
    def __init__(self, size=5, alpha=1e-4, beta=0.75, k=1.0):
        super().__init__()
        self.size, self.alpha, self.beta, self.k = size, alpha, beta, k
        self.mask_relu_input = False    # set by Net when the producer's ReLU backward is folded into this layer's
        self.bias_grad = None           # set by Net: fp32 [C] that receives the producer's bias gradient (sum of dx)

    def setup(self, in_shape, device):
        self.C = in_shape[-1]
        self.P = 1
        for s in in_shape[:-1]:
            self.P *= s
        self.y = torch.empty(self.P, self.C, dtype=BF, device=device)
        self.scale = torch.empty(self.P, self.C, dtype=BF, device=device)    # 1 / scale, kept for backward
        self.dx = torch.empty(self.P, self.C, dtype=BF, device=device)
        self.out_shape = in_shape
        return in_shape

    def forward(self, x):
        self.x = x.reshape(self.P, self.C)
        F.lrn_forward(self.x, self.y, self.scale, self.size, self.alpha, self.beta, self.k)
        return self.y

    def backward(self, dy):
        F.lrn_backward(self.x, self.y, self.scale, dy.reshape(self.P, self.C), self.dx, self.size, self.alpha, self.beta,
                       relu_mask=self.mask_relu_input, colsum=self.bias_grad)
        return self.dx


class LRNMaxPool(Layer):
    """LRN across channels followed by max pooling as one fused kernel per direction (the normalised tensor and
    its gradient never reach global memory; the backward recomputes the normalisation from the input).  Built by
    Net.setup from an adjacent (LRN, max Pool) pair; `lrn` and `pool` keep the pair's definition."""

    def __init__(self, lrn: "LRN", pool: "Pool"):
        super().__init__()
        self.lrn, self.pool = lrn, pool
        self.size, self.alpha, self.beta, self.k = lrn.size, lrn.alpha, lrn.beta, lrn.k
        self.mask_relu_input = False
        self.bias_grad = None

    @staticmethod
    def fusable(lrn, pool, in_shape) -> bool:
        if not (isinstance(lrn, LRN) and isinstance(pool, Pool) and pool.kind == "max" and pool.k > 0):
            return False
        if os.environ.get("GEEPS_FUSE_LRN_POOL", "1") == "0" or not torch.cuda.is_available():
            return False
        C = in_shape[-1]
        g = F.pool_geom(in_shape, pool.k, pool.stride, pool.pad, C, C, pool.ceil_mode)
        return F.lrn_maxpool_supported(g, lrn.size)

    def setup(self, in_shape, device):
        B, H, W, C = in_shape
        self.in_shape, self.C = in_shape, C
        p = self.pool
        self.g = F.pool_geom(in_shape, p.k, p.stride, p.pad, C, C, p.ceil_mode)
        self.out_shape = (B, self.g.OH, self.g.OW, C)
        self.y = None
        self.argmax = torch.empty(self.out_shape, dtype=torch.uint8, device=device)
        self.dx = torch.empty(in_shape, dtype=BF, device=device)
        self.device = device
        return self.out_shape

    def bind_output(self, y2d, ldy):
        self.y = y2d
        self.g.ldy = ldy

    def set_output(self, flat):
        self.y = flat[:self.out_numel()].view(self.out_shape)
        self.g.ldy = self.out_shape[-1]

    def forward(self, x):
        if self.y is None:
            self.y = torch.empty(self.out_shape, dtype=BF, device=self.device)
        self.x = x.reshape(self.in_shape)
        F.lrn_maxpool_forward(self.x, self.y, self.argmax, self.g, self.size, self.alpha, self.beta, self.k)
        return self.y

    def backward(self, dy):
        F.lrn_maxpool_backward(self.x, dy, self.argmax, self.dx, self.g, self.size, self.alpha, self.beta, self.k,
                               relu_mask=self.mask_relu_input, colsum=self.bias_grad)
        return self.dx


class Pool(Layer):
    def __init__(self, kind, k, stride, pad=0, ceil_mode=True):
        super().__init__()
        self.kind, self.k, self.stride, self.pad, self.ceil_mode = kind, k, stride, pad, ceil_mode

    def setup(self, in_shape, device):
        B, H, W, C = in_shape
        self.in_shape = in_shape
        k = H if self.k == 0 else self.k      # k = 0: global pooling
        self.g = F.pool_geom(in_shape, k, self.stride, self.pad, C, C, self.ceil_mode)
        self.out_shape = (B, self.g.OH, self.g.OW, C)
        self.y = None
        self.argmax = torch.empty(self.out_shape, dtype=torch.uint8, device=device) if self.kind == "max" else None
        self.dx = torch.empty(in_shape, dtype=BF, device=device)
        self.device = device
        return self.out_shape

    def bind_output(self, y2d, ldy):
        self.y = y2d
        self.g.ldy = ldy

    def set_output(self, flat):
        self.y = flat[:self.out_numel()].view(self.out_shape)
        self.g.ldy = self.out_shape[-1]

    def forward(self, x):
        if self.y is None:
            self.y = torch.empty(self.out_shape, dtype=BF, device=self.device)
        self.g.ldx = x.stride(-2) if x.dim() >= 2 else self.g.C
        if self.kind == "max":
            F.maxpool_forward(x, self.y, self.argmax, self.g)
        else:
            F.avgpool_forward(x, self.y, self.g)
        return self.y

    def backward(self, dy):
        ldx = self.g.ldx
        self.g.ldx = self.g.C       # dx is a dense tensor of the input shape
        if self.kind == "max":
            F.maxpool_backward(dy, self.argmax, self.dx, self.g)
        else:
            F.avgpool_backward(dy, self.dx, self.g)
        self.g.ldx = ldx
        return self.dx


class Dropout(Layer):
    def __init__(self, p=0.5, seed=1234):
        super().__init__()
        self.p, self.seed, self.step = p, seed, 0
        self.step_ref = None      # address of a device-resident step counter (set by the trainer in graph mode)

    def setup(self, in_shape, device):
        self.y = torch.empty(in_shape, dtype=BF, device=device)
        self.dx = torch.empty(in_shape, dtype=BF, device=device)
        self.out_shape = in_shape
        return in_shape

    def forward(self, x):
        self.step += 1
        if not self.training:
            return x
        if self.step_ref:
            F.dropout(x.contiguous(), self.y, self.p, self.seed, self.step_ref)
        else:
            F.dropout(x.contiguous(), self.y, self.p, self.seed + self.step)
        return self.y

    def backward(self, dy):
        if not self.training:
            return dy
        if self.step_ref:
            F.dropout(dy.contiguous(), self.dx, self.p, self.seed, self.step_ref)
        else:
            F.dropout(dy.contiguous(), self.dx, self.p, self.seed + self.step)
        return self.dx


class SoftmaxLoss(Layer):
    """Mean softmax cross-entropy over the batch; backward seeds dlogits = (softmax - onehot) / B."""

    def setup(self, in_shape, device):
        B, C = in_shape
        self.B, self.C = B, C
        self.loss = torch.zeros(1, device=device)
        self.dlogits = torch.zeros(B, _pad8(C), dtype=BF, device=device)[:, :C]
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.out_shape = (1,)
        return self.out_shape

    def forward(self, logits, labels):
        F.softmax_ce(logits, labels, self.loss, self.dlogits, loss_scale=1.0 / self.B, grad_scale=1.0 / self.B,
                     status=self.status)
        return self.loss

    def backward(self, dy=None):
        return self.dlogits
