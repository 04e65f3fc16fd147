"""A plain-PyTorch twin of a geeps_b200 Net, built layer by layer from the Net's own definition.

Two uses: the library-ops baseline of every model (torch eager: cuDNN convolutions, cuBLAS GEMMs, torch
LRN / BatchNorm / pooling, torch.optim.SGD), and loss-parity checks - the twin takes the very initial
values the parameter server was bootstrapped with (`PSModule(keep_init=True).initial_params`), so both
frameworks start from the same weights.

Activations of the twin are NCHW like any torch model, except that the flatten in front of a Linear layer
orders the features (h, w, c) as the NHWC framework does, so fully-connected weights map one to one.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..models.net import Concat
from ..ops import layers as GL


class _FlattenNHWC(nn.Module):
    def forward(self, x):
        return x.permute(0, 2, 3, 1).flatten(1) if x.dim() == 4 else x


class _ConcatT(nn.Module):
    def __init__(self, branches):
        super().__init__()
        self.branches = nn.ModuleList(branches)

    def forward(self, x):
        return torch.cat([b(x) for b in self.branches], 1)


def _conv_weight_from_rows(layer: GL.Conv2d, w: torch.Tensor, cin_true: int) -> torch.Tensor:
    """[cout, ld] rows of the framework (column = (kh * KW + kw) * cg + ci, or the space-to-depth order of the
    first AlexNet convolution) -> torch's [cout, cin / groups, KH, KW]."""
    cout = w.shape[0]
    if layer.s2d:
        S, T, k = layer.s2d, layer.k, layer.orig_k
        C = layer.in_shape[-1]            # padded space-to-depth channels
        c0 = cin_true
        out = torch.zeros(cout, c0, k, k, dtype=w.dtype)
        for a in range(T):
            for b in range(T):
                for dy in range(S):
                    for dx in range(S):
                        kh, kw = a * S + dy, b * S + dx
                        if kh >= k or kw >= k:
                            continue
                        col = (a * T + b) * C + (dy * S + dx) * c0
                        out[:, :, kh, kw] = w[:, col:col + c0]
        return out
    k, cg = layer.k, layer.cg
    w4 = w[:, :layer.kd].reshape(cout, k, k, cg).permute(0, 3, 1, 2)
    return w4[:, :cin_true].contiguous()


class TorchMirror(nn.Module):
    def __init__(self, net, in_shape):
        """`net` must have been set up (PSModule does that) for `in_shape` = (B, C, H, W)."""
        super().__init__()
        self.loaders = []            # (param name in the framework, fn(tensor) -> None)
        mods = []
        c_true = in_shape[1]         # channels that really exist (the framework may pad them)
        for l in net.layers:
            m, c_true = self._convert(l, c_true)
            mods.extend(m)
        self.body = nn.Sequential(*mods)

    def _convert(self, l, c_true):
        if isinstance(l, Concat):
            branches, widths = [], []
            for br in l.branches:
                mods, c = [], c_true
                for sub in br:
                    m, c = self._convert(sub, c)
                    mods.extend(m)
                branches.append(nn.Sequential(*mods))
                widths.append(c)
            return [_ConcatT(branches)], sum(widths)
        if isinstance(l, GL.Conv2d):
            k = l.orig_k if l.s2d else l.k
            stride = l.s2d if l.s2d else l.stride
            conv = nn.Conv2d(c_true, l.cout, k, stride, l.pad, groups=l.groups, bias=l.has_bias)
            cin_g = c_true // l.groups
            self.loaders.append((f"{l.name}.weight",
                                 lambda t, conv=conv, l=l, cin_g=cin_g: conv.weight.data.copy_(_conv_weight_from_rows(l, t, cin_g))))
            if l.has_bias:
                self.loaders.append((f"{l.name}.bias", lambda t, conv=conv: conv.bias.data.copy_(t)))
            return [conv] + ([nn.ReLU()] if l.relu else []), l.cout
        if isinstance(l, GL.BatchNorm):
            bn = nn.BatchNorm2d(l.C, eps=l.eps, momentum=l.momentum)
            self.loaders.append((f"{l.name}.gamma", lambda t, bn=bn: bn.weight.data.copy_(t)))
            self.loaders.append((f"{l.name}.beta", lambda t, bn=bn: bn.bias.data.copy_(t)))
            return [bn] + ([nn.ReLU()] if l.relu else []), c_true
        if isinstance(l, GL.LRNMaxPool):
            return [nn.LocalResponseNorm(l.size, l.alpha, l.beta, l.k),
                    nn.MaxPool2d(l.pool.k, l.pool.stride, l.pool.pad, ceil_mode=l.pool.ceil_mode)], c_true
        if isinstance(l, GL.LRN):
            return [nn.LocalResponseNorm(l.size, l.alpha, l.beta, l.k)], c_true
        if isinstance(l, GL.Pool):
            if l.kind == "max":
                return [nn.MaxPool2d(l.k, l.stride, l.pad, ceil_mode=l.ceil_mode)], c_true
            if l.k == 0:
                return [nn.AdaptiveAvgPool2d(1)], c_true
            return [nn.AvgPool2d(l.k, l.stride, l.pad, ceil_mode=l.ceil_mode, count_include_pad=True)], c_true
        if isinstance(l, GL.Linear):
            lin = nn.Linear(l.k_in, l.out)
            self.loaders.append((f"{l.name}.weight", lambda t, lin=lin, l=l: lin.weight.data.copy_(t[:, :l.k_in])))
            self.loaders.append((f"{l.name}.bias", lambda t, lin=lin: lin.bias.data.copy_(t)))
            return [_FlattenNHWC(), lin] + ([nn.ReLU()] if l.relu else []), l.out
        if isinstance(l, GL.Dropout):
            return [nn.Dropout(l.p)], c_true
        raise TypeError(f"no torch twin for layer {type(l).__name__}")

    def load_initial(self, initial_params: dict) -> None:
        for name, fn in self.loaders:
            fn(initial_params[name].float())

    def forward(self, x):
        return self.body(x)


def train_mirror(mirror: nn.Module, x: torch.Tensor, y: torch.Tensor, steps: int, lr: float, momentum: float,
                 weight_decay: float = 0.0, bf16: bool = True) -> list:
    """`steps` momentum-SGD steps on the fixed batch (x NCHW, y labels); returns the loss before each step."""
    opt = torch.optim.SGD(mirror.parameters(), lr=lr, momentum=momentum, weight_decay=weight_decay)
    losses = []
    for _ in range(steps):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf16):
            loss = nn.functional.cross_entropy(mirror(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(loss.detach())
    return [float(v) for v in losses]
