#!/usr/bin/env python
"""Baseline (c): the same AlexNet training step with library ops (torch eager: cuDNN convolutions,
cuBLAS GEMMs, torch LRN / pooling / dropout / cross-entropy, torch.optim.SGD with momentum) on one
GPU - the stand-in for the reference's cuDNN/cuBLAS Caffe application, which is not in its tree.
Same config as bench.py: batch 256, 3x227x227 synthetic input, bf16 autocast, channels_last.
Prints one JSON line with images/s (CUDA events)."""
import argparse
import json

import torch
import torch.nn as nn


def alexnet(classes=1000):
    return nn.Sequential(
        nn.Conv2d(3, 96, 11, 4), nn.ReLU(inplace=True), nn.LocalResponseNorm(5, 1e-4, 0.75, 1.0),
        nn.MaxPool2d(3, 2, ceil_mode=True),
        nn.Conv2d(96, 256, 5, padding=2, groups=2), nn.ReLU(inplace=True), nn.LocalResponseNorm(5, 1e-4, 0.75, 1.0),
        nn.MaxPool2d(3, 2, ceil_mode=True),
        nn.Conv2d(256, 384, 3, padding=1), nn.ReLU(inplace=True),
        nn.Conv2d(384, 384, 3, padding=1, groups=2), nn.ReLU(inplace=True),
        nn.Conv2d(384, 256, 3, padding=1, groups=2), nn.ReLU(inplace=True),
        nn.MaxPool2d(3, 2, ceil_mode=True), nn.Flatten(),
        nn.Linear(9216, 4096), nn.ReLU(inplace=True), nn.Dropout(0.5),
        nn.Linear(4096, 4096), nn.ReLU(inplace=True), nn.Dropout(0.5),
        nn.Linear(4096, classes))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.backends.cudnn.benchmark = True
    m = alexnet().to(dev).to(memory_format=torch.channels_last)
    opt = torch.optim.SGD(m.parameters(), lr=0.01, momentum=0.9, weight_decay=5e-4)
    x = torch.randn(a.batch, 3, 227, 227, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(m(x), y)
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
    print(json.dumps({"baseline": "torch_eager_cudnn_cublas", "model": "alexnet", "batch": a.batch, "ms_per_step": ms,
                      "images_per_s": a.batch / ms * 1e3, "dtype": "bf16 autocast", "optimizer": "torch SGD momentum"}))


if __name__ == "__main__":
    main()
