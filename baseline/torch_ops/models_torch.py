#!/usr/bin/env python
"""Baseline (c) for every model of the framework: the same network built from library ops (torch eager:
cuDNN convolutions, cuBLAS GEMMs, torch BatchNorm / LRN / pooling / cross-entropy, torch.optim.SGD with momentum,
bf16 autocast, channels_last) - the stand-in for the reference's cuDNN/cuBLAS Caffe application, which is not in
its tree.  The torch network is derived layer by layer from the framework's own model definition
(geeps_b200/utils/torch_mirror.py), so both sides train the same architecture.

  python baseline/torch_ops/models_torch.py --model alexnet|inception_bn_small|inception_bn_22k [--batch N]

Prints one JSON line with images/s (CUDA events, inputs resident on the device)."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch
import torch.nn as nn

CONFIGS = {"alexnet": ((3, 227, 227), 1000, 256), "inception_bn_small": ((3, 32, 32), 10, 100),
           "inception_bn_22k": ((3, 224, 224), 21841, 32)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="alexnet", choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=0)
    a = ap.parse_args()
    from geeps_b200.models.alexnet import alexnet
    from geeps_b200.models.inception_bn import inception_bn_22k, inception_bn_small
    from geeps_b200.utils.torch_mirror import TorchMirror
    image, classes, batch = CONFIGS[a.model]
    batch = a.batch or batch
    dev = torch.device("cuda:0")
    torch.backends.cudnn.benchmark = True
    net = {"alexnet": alexnet, "inception_bn_small": inception_bn_small, "inception_bn_22k": inception_bn_22k}[a.model]()
    net.setup((batch,) + image, dev)            # shapes only; the framework's kernels are not used here
    m = TorchMirror(net, (batch,) + image).to(dev).to(memory_format=torch.channels_last)
    del net
    torch.cuda.empty_cache()
    opt = torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9, weight_decay=5e-4)
    x = torch.randn((batch,) + image, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, classes, (batch,), device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(m(x).float(), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    print(json.dumps({"baseline": "torch_eager_cudnn_cublas", "model": a.model, "batch": batch, "ms_per_step": ms,
                      "images_per_s": batch / ms * 1e3, "dtype": "bf16 autocast, channels_last",
                      "optimizer": "torch SGD momentum 0.9, lr 0.01, weight decay 5e-4"}))


if __name__ == "__main__":
    main()
