"""Inception-BN family: the small 32x32 variant (CIFAR-shaped) and the ImageNet-22K-shaped
GoogLeNet-BN with a 1024 x 21841 classifier."""
from __future__ import annotations

from ..ops.layers import BatchNorm, Conv2d, Input, Linear, Pool
from .net import Concat, Net


def _conv_bn(name, cout, k, stride=1, pad=0, need_dx=True):
    return [Conv2d(name, cout, k, stride=stride, pad=pad, bias=False, std=0.0, need_dx=need_dx),
            BatchNorm(name + "_bn", relu=True)]


def _module(name, c1, c3):
    return Concat(name, [_conv_bn(name + "_1x1", c1, 1), _conv_bn(name + "_3x3", c3, 3, pad=1)])


def _downsample(name, c3):
    return Concat(name, [_conv_bn(name + "_3x3", c3, 3, stride=2, pad=1), [Pool("max", 3, 2, pad=1, ceil_mode=False)]])


def inception_bn_small(num_classes: int = 10) -> Net:
    """conv3x3-96; modules (32|32), (32|48); downsample (80|pool); modules (112|48), (96|64),
    (80|80), (48|96); downsample (96|pool); modules (176|160) x2; global avgpool; FC."""
    layers = _conv_bn("conv1", 96, 3, pad=1, need_dx=False)
    layers += [_module("in3a", 32, 32), _module("in3b", 32, 48), _downsample("in3c", 80)]
    layers += [_module("in4a", 112, 48), _module("in4b", 96, 64), _module("in4c", 80, 80), _module("in4d", 48, 96),
               _downsample("in4e", 96)]
    layers += [_module("in5a", 176, 160), _module("in5b", 176, 160)]
    layers += [Pool("avg", 0, 1, ceil_mode=False), Linear("fc", num_classes, std=0.01, fp32_out=True)]
    return Net("inception_bn_small", Input(cpad=8), layers)


def _inception(name, c1, c3r, c3, cd3r, cd3, pool, cproj):
    """GoogLeNet-BN module: 1x1 | 1x1-3x3 | 1x1-3x3-3x3 | pool-1x1."""
    branches = []
    if c1:
        branches.append(_conv_bn(name + "_1x1", c1, 1))
    branches.append(_conv_bn(name + "_3x3r", c3r, 1) + _conv_bn(name + "_3x3", c3, 3, pad=1))
    branches.append(_conv_bn(name + "_d3r", cd3r, 1) + _conv_bn(name + "_d3a", cd3, 3, pad=1)
                    + _conv_bn(name + "_d3b", cd3, 3, pad=1))
    branches.append([Pool(pool, 3, 1, pad=1, ceil_mode=False)] + _conv_bn(name + "_proj", cproj, 1))
    return Concat(name, branches)


def _inception_down(name, c3r, c3, cd3r, cd3):
    """Stride-2 module: 1x1-3x3/2 | 1x1-3x3-3x3/2 | maxpool/2."""
    return Concat(name, [
        _conv_bn(name + "_3x3r", c3r, 1) + _conv_bn(name + "_3x3", c3, 3, stride=2, pad=1),
        _conv_bn(name + "_d3r", cd3r, 1) + _conv_bn(name + "_d3a", cd3, 3, pad=1)
        + _conv_bn(name + "_d3b", cd3, 3, stride=2, pad=1),
        [Pool("max", 3, 2, pad=1, ceil_mode=False)],
    ])


def inception_bn_22k(num_classes: int = 21841) -> Net:
    """GoogLeNet-BN trunk (224x224 input, 1024-wide final feature) + a 1024 x 21841 classifier."""
    layers = _conv_bn("conv1", 64, 7, stride=2, pad=3, need_dx=False) + [Pool("max", 3, 2, ceil_mode=True)]
    layers += _conv_bn("conv2r", 64, 1) + _conv_bn("conv2", 192, 3, pad=1) + [Pool("max", 3, 2, ceil_mode=True)]
    layers += [
        _inception("in3a", 64, 64, 64, 64, 96, "avg", 32),
        _inception("in3b", 64, 64, 96, 64, 96, "avg", 64),
        _inception_down("in3c", 128, 160, 64, 96),
        _inception("in4a", 224, 64, 96, 96, 128, "avg", 128),
        _inception("in4b", 192, 96, 128, 96, 128, "avg", 128),
        _inception("in4c", 160, 128, 160, 128, 160, "avg", 128),
        _inception("in4d", 96, 128, 192, 160, 192, "avg", 128),
        _inception_down("in4e", 128, 192, 192, 256),
        _inception("in5a", 352, 192, 320, 160, 224, "avg", 128),
        _inception("in5b", 352, 192, 320, 192, 224, "max", 128),
        Pool("avg", 0, 1, ceil_mode=False),
        Linear("fc", num_classes, std=0.01, fp32_out=True),
    ]
    return Net("inception_bn_22k", Input(cpad=8), layers)
