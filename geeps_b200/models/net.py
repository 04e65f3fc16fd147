"""Network containers: a sequential net of layers and an Inception-style concat module."""
from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.layers import BF, LRN, BatchNorm, Conv2d, Layer, LRNMaxPool, Pool, SoftmaxLoss


class Concat(Layer):
    """Parallel branches whose outputs are concatenated along channels.  The last layer of each
    branch writes straight into its channel slice of the joint output (no copy); in backward
    each branch reads its slice of the joint gradient and the branch input-gradients are summed."""

    def __init__(self, name, branches):
        super().__init__()
        self.name = name
        self.branches = branches       # list of lists of layers

    def sublayers(self):
        for br in self.branches:
            for l in br:
                yield l

    def setup(self, in_shape, device):
        self.in_shape = in_shape
        outs = []
        for br in self.branches:
            s = in_shape
            for l in br:
                s = l.setup(s, device)
            outs.append(s)
        B, OH, OW = outs[0][0], outs[0][1], outs[0][2]
        assert all(o[:3] == (B, OH, OW) for o in outs), outs
        self.widths = [o[3] for o in outs]
        ctot = sum(self.widths)
        self.P = B * OH * OW
        self.y = torch.empty(self.P, ctot, dtype=BF, device=device)
        off = 0
        for br, w in zip(self.branches, self.widths):
            last = br[-1]
            view = self.y[:, off:off + w]
            if isinstance(last, Pool):
                last.bind_output(view, ctot)
            else:
                last.bind_output(view)
            off += w
        self.out_shape = (B, OH, OW, ctot)
        self.dx = None
        return self.out_shape

    def out_numel(self):
        return self.P * sum(self.widths)

    def set_output(self, flat):
        ctot = sum(self.widths)
        self.y = flat[:self.P * ctot].view(self.P, ctot)
        off = 0
        for br, w in zip(self.branches, self.widths):
            last, view = br[-1], self.y[:, off:off + w]
            if isinstance(last, Pool):
                last.bind_output(view, ctot)
            else:
                last.bind_output(view)
            off += w

    def set_input(self, x):
        for br in self.branches:
            br[0].set_input(x)

    def forward(self, x):
        x4 = x if x.dim() == 4 else x.view(self.in_shape)
        for br in self.branches:
            h = x4
            for l in br:
                h = l.forward(h)
        return self.y

    def backward(self, dy):
        if dy.dim() != 2:
            dy = dy.view(self.P, -1)
        off = 0
        total = None
        for br, w in zip(self.branches, self.widths):
            g = dy[:, off:off + w]
            for l in reversed(br):
                g = l.backward(g)
            g2 = g.view(-1, self.in_shape[-1])
            if total is None:
                total = g2
            else:
                F.add_2d(total, g2)
            off += w
        return total


class Net:
    """input layer -> layers -> linear logits -> softmax loss."""

    def __init__(self, name, input_layer, layers, loss=None):
        self.name = name
        self.input_layer = input_layer
        self.layers = layers
        self.loss_layer = loss or SoftmaxLoss()

    def all_layers(self):
        for l in self.layers:
            if isinstance(l, Concat):
                yield from l.sublayers()
            else:
                yield l

    def param_layers(self):
        return [l for l in self.all_layers() if l.param_specs()]

    def setup(self, in_shape, device):
        s = self.input_layer.setup(in_shape, device)
        # an LRN directly followed by a max pooling becomes one fused layer (GEEPS_FUSE_LRN_POOL=0 keeps the pair)
        fused, i = [], 0
        while i < len(self.layers):
            l = self.layers[i]
            nxt = self.layers[i + 1] if i + 1 < len(self.layers) else None
            if isinstance(l, LRN) and isinstance(nxt, Pool) and LRNMaxPool.fusable(l, nxt, s):
                l = LRNMaxPool(l, nxt)
                i += 1
            s = l.setup(s, device)
            fused.append(l)
            i += 1
        self.layers = fused
        self.loss_layer.setup(s, device)
        self.device = device
        # conv + ReLU followed by LRN: the LRN backward already reads the ReLU output, so it applies the ReLU
        # mask to the gradient it hands down and the convolution skips its own masking pass
        for a, b in zip(self.layers, self.layers[1:]):
            if isinstance(a, Conv2d) and a.relu and isinstance(b, (LRN, LRNMaxPool)):
                a.dy_is_masked, b.mask_relu_input = True, True
                if a.has_bias and b.C % 8 == 0 and b.size in (3, 5, 7):
                    # the same pass also sums the masked gradient per channel: the convolution's bias gradient
                    b.bias_grad = torch.zeros(b.C, device=device)
                    a.bias_grad_src = b.bias_grad
        return s

    def num_params(self, valid_only=True):
        n = 0
        for l in self.param_layers():
            for sp in l.param_specs():
                n += sp.num_valid() if valid_only else sp.numel
        return n

    def train(self, mode=True):
        for l in self.all_layers():
            l.training = mode
