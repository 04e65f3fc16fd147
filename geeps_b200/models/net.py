"""Network containers: a sequential net of layers and an Inception-style concat module."""
from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.layers import BF, LRN, BatchNorm, Conv2d, Layer, LRNMaxPool, Pool, SoftmaxLoss


_side_streams = {}


def side_streams(device, n: int) -> list:
    """n CUDA streams of `device` shared by all Concat modules (branch i of every module runs on stream i)."""
    pool = _side_streams.setdefault(str(device), [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device=device))
    return pool[:n]


class Concat(Layer):
    """Parallel branches whose outputs are concatenated along channels.  The last layer of each
    branch writes straight into its channel slice of the joint output (no copy); in backward
    each branch reads its slice of the joint gradient and the branch input-gradients are summed.

    The branches are independent, and at the image sizes where these modules sit a single kernel rarely fills
    the GPU: with concurrent=True (default on a GPU; GEEPS_CONCAT_STREAMS=0 turns it off) branch i > 0 runs on a
    side stream, forked from and joined back into the caller's stream, so the branches overlap - also inside a
    captured step graph, where the fork / join become graph edges."""

    def __init__(self, name, branches, concurrent=None):
        super().__init__()
        self.name = name
        self.branches = branches       # list of lists of layers
        import os
        self.concurrent = (os.environ.get("GEEPS_CONCAT_STREAMS", "1") != "0") if concurrent is None else concurrent
        self._events = None

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

    def _run_branches(self, fn):
        """fn(i, branch) for every branch; branches 1.. on side streams between a fork and a join when concurrent."""
        n = len(self.branches)
        if not (self.concurrent and n > 1 and self.y.is_cuda):
            for i, br in enumerate(self.branches):
                fn(i, br)
            return
        main = torch.cuda.current_stream(self.y.device)
        sides = side_streams(self.y.device, n - 1)
        if self._events is None:
            self._events = [F.new_event() for _ in range(2 * (n - 1))]
        for i in range(1, n):
            F.stream_order(main, sides[i - 1], self._events[i - 1])                 # fork
        fn(0, self.branches[0])
        for i in range(1, n):
            with torch.cuda.stream(sides[i - 1]):
                fn(i, self.branches[i])
            F.stream_order(sides[i - 1], main, self._events[n - 1 + i - 1])         # join

    def forward(self, x):
        x4 = x if x.dim() == 4 else x.view(self.in_shape)

        def run(i, br):
            h = x4
            for l in br:
                h = l.forward(h)
        self._run_branches(run)
        return self.y

    def backward(self, dy):
        if dy.dim() != 2:
            dy = dy.view(self.P, -1)
        offs, off = [], 0
        for w in self.widths:
            offs.append(off)
            off += w
        grads = [None] * len(self.branches)

        def run(i, br):
            g = dy[:, offs[i]:offs[i] + self.widths[i]]
            for l in reversed(br):
                g = l.backward(g)
            grads[i] = g.view(-1, self.in_shape[-1])
        self._run_branches(run)
        total = grads[0]
        for g2 in grads[1:]:
            F.add_2d(total, g2)
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
