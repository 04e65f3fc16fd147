"""AlexNet as trained by Caffe (bvlc_alexnet): 5 conv (groups 2 in conv2/4/5) + LRN + 3 FC,
~61 M parameters, 3x227x227 input, 1000 classes."""
from __future__ import annotations

from ..ops.layers import LRN, Conv2d, Dropout, Input, Linear, Pool
from .net import Net


def alexnet(num_classes: int = 1000, dropout: float = 0.5) -> Net:
    layers = [
        # the input layer emits a space-to-depth(4) layout [B, 57, 57, 48 + 16 zero channels]: the 11 x 11 stride-4
        # convolution becomes a 3 x 3 stride-1 implicit GEMM (taps past 11 and the padding channels are zero
        # columns), so no patch matrix is built and every pixel is one aligned 128-byte line
        Conv2d("conv1", 96, 11, stride=4, relu=True, std=0.01, need_dx=False, s2d=4, cin_valid=3),
        LRN(5, 1e-4, 0.75, 1.0),
        Pool("max", 3, 2),
        Conv2d("conv2", 256, 5, pad=2, groups=2, relu=True, std=0.01, bias_value=0.1),
        LRN(5, 1e-4, 0.75, 1.0),
        Pool("max", 3, 2),
        Conv2d("conv3", 384, 3, pad=1, relu=True, std=0.01),
        Conv2d("conv4", 384, 3, pad=1, groups=2, relu=True, std=0.01, bias_value=0.1),
        Conv2d("conv5", 256, 3, pad=1, groups=2, relu=True, std=0.01, bias_value=0.1),
        Pool("max", 3, 2),
        Linear("fc6", 4096, relu=True, std=0.005, bias_value=0.1),
        Dropout(dropout, seed=61),
        Linear("fc7", 4096, relu=True, std=0.005, bias_value=0.1),
        Dropout(dropout, seed=71),
        Linear("fc8", num_classes, std=0.01, fp32_out=True),
    ]
    return Net("alexnet", Input(s2d=4, s2d_k=11, cpad=64), layers)
