"""Command-line trainer: python -m geeps_b200.train --model alexnet --max-iter 1000 ...
(one process per GPU; for N GPUs: python -m torch.distributed.run --nnodes=1 --nproc-per-node N
 --master-addr 127.0.0.1 -m geeps_b200.train ...)

The counterpart of the reference's Caffe application and its launch scripts (README.md:31-69 of the reference;
the application itself is an empty submodule there): builds a model, drives it through the parameter server
(`PSModule`), feeds it from pinned host memory, follows a Caffe learning-rate policy, prints the loss, writes table
snapshots and resumes from them.

Data: `--data synthetic` (random uint8 images and labels, generated once) or a directory holding `images.npy`
(uint8 [N, 3, H, W], H and W at least the network's input size; read through a memory map) and `labels.npy`
(integers [N]).  Every rank walks its own slice of a per-epoch permutation; the input layer crops (randomly, with
mirroring, unless --no-augment), subtracts --mean and multiplies by --scale on the device.
"""
from __future__ import annotations

import argparse
import os

MODELS = {"alexnet": ((3, 227, 227), 1000, 256), "inception_bn_small": ((3, 32, 32), 10, 128),
          "inception_bn_22k": ((3, 224, 224), 21841, 32)}


class ArraySource:
    """Batches from host arrays: rank r of `world` takes every world-th index of a permutation that all ranks draw
    from the same seed, one permutation per epoch.  next() fills pinned staging tensors (two sets, used in turn, so
    the copy of one batch to the device can still run while the next is gathered)."""

    def __init__(self, images, labels, batch: int, rank: int = 0, world: int = 1, seed: int = 0, pin: bool = True,
                 sets: int = 2):
        import numpy as np
        import torch
        if len(images) != len(labels) or len(images) < batch * world:
            raise ValueError(f"{len(images)} images, {len(labels)} labels: need at least batch x world = {batch * world}")
        self.np, self.images, self.labels = np, images, labels
        self.batch, self.rank, self.world, self.seed = batch, rank, world, seed
        self.epoch, self.pos, self.order = -1, 0, None
        shape = (batch,) + tuple(images.shape[1:])
        mk = (lambda t: t.pin_memory()) if pin else (lambda t: t)
        self.x = [mk(torch.empty(shape, dtype=torch.uint8)) for _ in range(sets)]
        self.y = [mk(torch.empty((batch,), dtype=torch.int64)) for _ in range(sets)]
        self.turn = 0

    def _new_epoch(self):
        self.epoch += 1
        perm = self.np.random.default_rng(self.seed + self.epoch).permutation(len(self.images))
        usable = len(perm) // (self.batch * self.world) * (self.batch * self.world)     # every rank the same count
        self.order, self.pos = perm[:usable][self.rank::self.world], 0

    def _take(self):
        if self.order is None or self.pos + self.batch > len(self.order):
            self._new_epoch()
        idx = self.order[self.pos:self.pos + self.batch]
        self.pos += self.batch
        return idx

    def skip(self, batches: int) -> None:
        """Pass over `batches` batches without reading them (a resumed run continues where the data walk stood)."""
        for _ in range(batches):
            self._take()

    def next(self, into: int | None = None):
        """The next batch in staging set `into` (default: the sets in turn)."""
        import torch
        idx = self.np.sort(self._take())          # ascending: friendlier to a memory map
        s = self.turn if into is None else into
        self.turn = (s + 1) % len(self.x)
        self.x[s].copy_(torch.from_numpy(self.np.ascontiguousarray(self.images[idx])))
        self.y[s].copy_(torch.from_numpy(self.np.asarray(self.labels[idx], dtype=self.np.int64)))
        return self.x[s], self.y[s]


def synthetic_arrays(n: int, image, classes: int, src_hw, seed: int = 0):
    import numpy as np
    rng = np.random.default_rng(seed)
    return (rng.integers(0, 256, size=(n, image[0]) + tuple(src_hw), dtype=np.uint8),
            rng.integers(0, classes, size=(n,), dtype=np.int64))


def device_batches(source, feeder, stream):
    """(images, labels) on the device, each batch's copy started one step ahead on the feeder's copy stream.  Batch k
    goes through staging set and device slot k mod depth; before a staging set is filled again the host waits until
    the copy that last read it is done (that copy waits for the step two before it, so the host stays at most a few
    steps ahead of the device)."""
    def submit():
        s = feeder.put_i % feeder.depth
        feeder.wait_copied(s)
        feeder.submit(*source.next(into=s))
    submit()
    held = None
    while True:
        if held is not None:
            feeder.release(held, stream)      # the step that used the previous slot has been enqueued
        x, y, held = feeder.next(stream)
        submit()
        yield x, y


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="alexnet", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=0, help="per GPU (0: the model's default)")
    ap.add_argument("--max-iter", type=int, default=1000)
    ap.add_argument("--data", default="synthetic", help="'synthetic' or a directory with images.npy and labels.npy")
    ap.add_argument("--synthetic-images", type=int, default=2048)
    ap.add_argument("--source-size", type=int, default=0, help="synthetic data: source image size (0: input size + 29)")
    ap.add_argument("--mean", type=float, nargs=3, default=(104.0, 117.0, 123.0))
    ap.add_argument("--scale", type=float, default=1.0 / 58.0)
    ap.add_argument("--no-augment", action="store_true", help="centre crop, no mirroring")
    ap.add_argument("--base-lr", type=float, default=0.01)
    ap.add_argument("--lr-policy", default="step", choices=["fixed", "step", "multistep", "exp", "inv", "poly", "sigmoid"])
    ap.add_argument("--gamma", type=float, default=0.1)
    ap.add_argument("--stepsize", type=int, default=100000)
    ap.add_argument("--stepvalue", type=int, action="append", default=[])
    ap.add_argument("--power", type=float, default=1.0)
    ap.add_argument("--lr-hold", type=int, default=200)
    ap.add_argument("--momentum", type=float, default=0.9)
    ap.add_argument("--weight-decay", type=float, default=5e-4)
    ap.add_argument("--slack", type=int, default=0)
    ap.add_argument("--display", type=int, default=20)
    ap.add_argument("--snapshot", type=int, default=0)
    ap.add_argument("--snapshot-dir", default=None)
    ap.add_argument("--resume", action="store_true", help="continue from the latest snapshot in --snapshot-dir")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--seed", type=int, default=1)
    args = ap.parse_args(argv)

    import numpy as np
    import torch

    from .models.alexnet import alexnet
    from .models.inception_bn import inception_bn_22k, inception_bn_small
    from .parallel.ps_module import PSModule
    from .utils.affinity import bind_to_gpu_cores
    from .utils.config import DEVICE_CUDA, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK, GeePsConfig
    from .utils.feeder import HostFeeder
    from .utils.solver import LrPolicy, Solver

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    bind_to_gpu_cores(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", world)))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # no torch.distributed process group: the parameter server's own control plane (TCP, host_list / port_list)
    # connects the ranks, and its peer-memory fabric carries the data

    image, classes, default_batch = MODELS[args.model]
    B = args.batch or default_batch
    net = {"alexnet": alexnet, "inception_bn_small": inception_bn_small, "inception_bn_22k": inception_bn_22k}[args.model]()
    if args.data == "synthetic":
        src = args.source_size or image[1] + 29
        images, labels = synthetic_arrays(max(args.synthetic_images, B * world), image, classes, (src, src), args.seed)
    else:
        images = np.load(os.path.join(args.data, "images.npy"), mmap_mode="r")
        labels = np.load(os.path.join(args.data, "labels.npy"))
    if images.dtype != np.uint8 or images.ndim != 4 or images.shape[1] != image[0] or \
            images.shape[2] < image[1] or images.shape[3] < image[2]:
        raise SystemExit(f"images: need uint8 [N, {image[0]}, >= {image[1]}, >= {image[2]}], got {images.dtype} {images.shape}")
    src_hw = (int(images.shape[2]), int(images.shape[3]))

    base_port = 10000 + (int(os.environ.get("MASTER_PORT", "29500")) % 500) * 40
    cfg = GeePsConfig(host_list=["127.0.0.1"] * world, port_list=[base_port + 10 * r for r in range(world)],
                      device=DEVICE_CUDA, cuda_device=local_rank, transport=TRANSPORT_NVLINK,
                      table_mode=TABLE_SGD_MOMENTUM, learning_rate=args.base_lr, momentum=args.momentum,
                      weight_decay=args.weight_decay, grad_scale=1.0 / world, bf16_compute_cache=1)
    resume = args.snapshot_dir if args.resume else None
    if args.resume and not (args.snapshot_dir and os.path.exists(os.path.join(args.snapshot_dir, "LATEST"))):
        raise SystemExit("--resume needs a --snapshot-dir that holds a snapshot")
    stream = torch.cuda.Stream(device=dev, priority=-1)
    with torch.cuda.stream(stream):
        mod = PSModule(net, (B,) + image, cfg, rank=rank, world=world, device=dev, slack=args.slack, seed=args.seed,
                       bf16_weights_only=True, use_graph=not args.no_graph, resume_from=resume)
        inp = mod.net.input_layer
        inp.set_transform(args.mean, args.scale)
        policy = LrPolicy(args.lr_policy, args.base_lr, args.gamma, args.stepsize, args.stepvalue, args.power, args.max_iter)
        solver = Solver(mod, policy, momentum=args.momentum, weight_decay=args.weight_decay, display=args.display,
                        snapshot=args.snapshot, snapshot_dir=args.snapshot_dir, lr_hold=args.lr_hold, rank=rank)
        feeder_depth = 2
        source = ArraySource(images, labels, B, rank, world, seed=args.seed, sets=feeder_depth)
        source.skip(solver.iter)       # a resumed run goes on with the batches that follow the ones already consumed
        feeder = HostFeeder((B, image[0]) + src_hw, (B,), dev, depth=feeder_depth, x_dtype=torch.uint8)
        augment = None
        if not args.no_augment:
            aug_gen = torch.Generator(device=dev).manual_seed(args.seed * 7919 + rank)
            augment = lambda it: inp.randomize(src_hw, mirror=True, generator=aug_gen)
        if rank == 0:
            print(f"{args.model}: batch {B} x {world} GPUs, {len(images)} images {src_hw[0]}x{src_hw[1]}, "
                  f"iterations {solver.iter} -> {args.max_iter}, lr policy {args.lr_policy}", flush=True)
        solver.run(device_batches(source, feeder, stream), args.max_iter, before_step=augment)
        torch.cuda.synchronize(dev)
        mod.close()


if __name__ == "__main__":
    main()
