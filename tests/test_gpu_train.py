"""End-to-end training steps through the parameter server on one GPU: the layer stack against a
PyTorch fp32 reference of the same network, and loss going down on a fixed batch."""
import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu

from geeps_b200.models.alexnet import alexnet
from geeps_b200.models.inception_bn import inception_bn_small
from geeps_b200.ops.layers import Conv2d, Linear, Pool, LRN, Input
from geeps_b200.models.net import Net
from geeps_b200.parallel.ps_module import PSModule
from geeps_b200.utils.config import (DEVICE_CUDA, TABLE_ADDITIVE, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK, TRANSPORT_TCP,
                                     GeePsConfig)

_port = [26000]


def cfg(transport, **kw):
    _port[0] += 20
    base = dict(device=DEVICE_CUDA, cuda_device=0, transport=transport, table_mode=TABLE_SGD_MOMENTUM,
                tcp_base_port=_port[0], bf16_compute_cache=1, learning_rate=0.01, momentum=0.9)
    base.update(kw)
    return GeePsConfig(**base)


def tiny_net():
    layers = [Conv2d("c1", 16, 3, pad=1, relu=True, std=0.1, need_dx=False), LRN(5, 1e-2, 0.75, 1.0), Pool("max", 3, 2),
              Conv2d("c2", 32, 3, pad=1, groups=2, relu=True, std=0.1), Pool("max", 3, 2),
              Linear("f1", 64, relu=True, std=0.05), Linear("f2", 10, std=0.05, fp32_out=True)]
    return Net("tiny", Input(cpad=8), layers)


@pytest.mark.parametrize("transport", [TRANSPORT_NVLINK, TRANSPORT_TCP])
def test_tiny_net_gradients_match_torch(transport):
    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    B = 16
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(transport, learning_rate=1.0, momentum=0.0), device=dev,
                       keep_init=True)
        x = torch.randn(B, 3, 16, 16, device=dev)
        y = torch.randint(0, 10, (B,), device=dev)
        loss = mod.step(x, y).item()                     # clock 1: update = -lr * grad with lr 1, momentum 0
        mod.step(x, y, capture=True)                     # clock 2 reads p1 = p0 - grad(p0)
        torch.cuda.synchronize()
        before = {k: v.to(dev) for k, v in mod.initial_params.items()}
        after = mod.captured
        grads = {k: (before[k] - after[k]) for k in before}
        # ---- the same network in plain PyTorch fp32 on the bf16-rounded parameters ----
        p = {k: v.to(torch.bfloat16).float().requires_grad_(True) for k, v in before.items()}
        xb = torch.zeros(B, 8, 16, 16, device=dev)
        xb[:, :3] = x.to(torch.bfloat16).float()

        def conv_w(w, cin, k):
            return w[:, :k * k * cin].view(w.shape[0], k, k, cin).permute(0, 3, 1, 2)

        def q(t):   # activations are stored as bf16 between layers (differentiable rounding)
            return t.to(torch.bfloat16).float()

        h = q(torch.relu(TF.conv2d(xb, conv_w(p["c1.weight"], 8, 3), p["c1.bias"], padding=1)))
        h = q(TF.local_response_norm(h, 5, alpha=1e-2, beta=0.75, k=1.0))
        h = TF.max_pool2d(h, 3, 2, ceil_mode=True)
        h = q(torch.relu(TF.conv2d(h, conv_w(p["c2.weight"], 8, 3), p["c2.bias"], padding=1, groups=2)))
        h = TF.max_pool2d(h, 3, 2, ceil_mode=True)
        h = h.permute(0, 2, 3, 1).reshape(B, -1)          # NHWC flatten order
        h = q(torch.relu(h @ p["f1.weight"].t() + p["f1.bias"]))
        logits = h @ p["f2.weight"][:, :64].t() + p["f2.bias"]
        ref_loss = TF.cross_entropy(logits, y)
        ref_loss.backward()
        assert abs(loss - ref_loss.item()) < 3e-2 * max(1.0, abs(ref_loss.item())), (loss, ref_loss.item())
        for k in ("f2.weight", "f1.weight", "c2.weight", "c1.weight", "f2.bias", "c1.bias"):
            g_ref = p[k].grad
            g = grads[k]
            # Frobenius-relative error: a ReLU unit whose pre-activation sits within bf16 rounding of zero
            # may flip between the two computations and move single entries by one sample's contribution
            err = ((g - g_ref).norm() / (g_ref.norm() + 1e-12)).item()
            assert err < 8e-2, (k, err)
        mod.close()


def test_inception_small_loss_decreases():
    torch.manual_seed(1)
    dev = torch.device("cuda:0")
    B = 100
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(inception_bn_small(), (B, 3, 32, 32), cfg(TRANSPORT_NVLINK, learning_rate=0.01), device=dev)
        x = torch.randn(B, 3, 32, 32, device=dev)
        y = torch.randint(0, 10, (B,), device=dev)
        losses = [mod.step(x, y).item() for _ in range(12)]
        assert all(l == l for l in losses), losses
        # decreasing; around the momentum plateau (steps 8-10 move by ~1e-3) reduction-order noise of the split-K
        # partial sums, which are added in arrival order, may flip the sign of a step
        assert losses[-1] < losses[0] - 0.05 and all(b < a + 5e-3 for a, b in zip(losses, losses[1:])), losses
        mod.close()


def test_alexnet_step_runs_and_learns():
    torch.manual_seed(2)
    dev = torch.device("cuda:0")
    B = 16
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        net = alexnet(dropout=0.0)
        mod = PSModule(net, (B, 3, 227, 227), cfg(TRANSPORT_NVLINK, learning_rate=0.01), device=dev)
        x = torch.randn(B, 3, 227, 227, device=dev)
        y = torch.randint(0, 1000, (B,), device=dev)
        losses = [mod.step(x, y).item() for _ in range(8)]
        assert all(l == l for l in losses), losses
        assert abs(losses[0] - 6.9) < 0.3, losses       # ln(1000) at random init
        assert losses[-1] < losses[0], losses
        assert mod.ps.last_error() == 0
        mod.close()


@pytest.mark.parametrize("frac", [None, 0.55, 0.25])
def test_managed_activations_match_unmanaged(frac):
    """Activations routed through LocalAccess (and swapped to pinned host memory under a budget of 55 % of the working set) give the
    same losses as ordinary buffers."""
    torch.manual_seed(4)
    dev = torch.device("cuda:0")
    B = 64
    losses = {}
    for managed in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            mod = PSModule(inception_bn_small(), (B, 3, 32, 32), cfg(TRANSPORT_NVLINK, learning_rate=0.01), device=dev,
                           seed=9, manage_activations=managed, cache_fraction=frac if managed else None)
            gen = torch.Generator(device=dev).manual_seed(5)
            x = torch.randn(B, 3, 32, 32, device=dev, generator=gen)
            y = torch.randint(0, 10, (B,), device=dev, generator=gen)
            losses[managed] = [mod.step(x, y).item() for _ in range(5)]
            if managed:
                st = mod.ps.get_stats()["client"]
                assert len(mod.managed) > 0
                if frac is not None:
                    assert st["cpu_local_rows"] > 0 and st["swap_h2d_bytes"] > 0
            assert mod.ps.last_error() == 0
            mod.close()
    assert losses[True] == pytest.approx(losses[False], rel=2e-3), losses


def test_tape_replay_matches_python_path():
    """Replaying the recorded native calls of a step gives the same losses as running the layer code, keeps
    counting launches, and still advances the dropout seeds."""
    from geeps_b200.ops import _lib as L
    dev = torch.device("cuda:0")
    B = 64
    losses, launches = {}, {}
    for tape in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            mod = PSModule(inception_bn_small(), (B, 3, 32, 32), cfg(TRANSPORT_NVLINK, learning_rate=0.01), device=dev,
                           seed=9, use_tape=tape)
            gen = torch.Generator(device=dev).manual_seed(5)
            x = torch.randn(B, 3, 32, 32, device=dev, generator=gen)
            y = torch.randint(0, 10, (B,), device=dev, generator=gen)
            n0 = L.launch_count()
            losses[tape] = [mod.step(x, y).item() for _ in range(10)]
            launches[tape] = L.launch_count() - n0
            assert (len(mod._tapes) == 2) == tape
            assert mod.ps.last_error() == 0
            mod.close()
    assert losses[True] == pytest.approx(losses[False], rel=2e-3), losses
    assert launches[True] == launches[False]


@pytest.mark.parametrize("slack", [0, 1])
def test_graph_replay_matches_python_path(slack):
    """One CUDA graph per (buffers, ring phase) replayed with a single launch gives the same losses as running the
    layer code: the runtime's clock lives in a device word, the host bookkeeping advances per replay, errors still
    surface, and the launch counter keeps counting the kernels inside the graph."""
    from geeps_b200.ops import _lib as L
    dev = torch.device("cuda:0")
    B = 64
    losses, launches = {}, {}
    for graph in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            mod = PSModule(inception_bn_small(), (B, 3, 32, 32), cfg(TRANSPORT_NVLINK, learning_rate=0.01), device=dev,
                           seed=9, slack=slack, use_graph=graph)
            gen = torch.Generator(device=dev).manual_seed(5)
            x = torch.randn(B, 3, 32, 32, device=dev, generator=gen)
            y = torch.randint(0, 10, (B,), device=dev, generator=gen)
            n0 = L.launch_count()
            losses[graph] = [mod.step(x, y).item() for _ in range(16)]
            launches[graph] = L.launch_count() - n0
            stats = mod.ps.get_stats()
            assert (len(mod._graphs) == 2) == graph, len(mod._graphs)
            assert (stats["client"]["nr_replayed_clocks"] > 0) == graph
            assert stats["client"]["nr_clock"] == 17          # bootstrap + 16 steps, replayed or not
            assert mod.ps.last_error() == 0
            mod.close()
    assert losses[True] == pytest.approx(losses[False], rel=2e-3), losses
    assert launches[True] == launches[False]


def test_graph_replay_alexnet_with_dropout_trains():
    """AlexNet in graph mode: dropout masks follow the device-resident step counter (they change every step and
    are the same in a step's forward and backward), and the loss on a fixed batch goes down."""
    from geeps_b200.models.alexnet import alexnet
    dev = torch.device("cuda:0")
    B = 16
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(alexnet(), (B, 3, 227, 227), cfg(TRANSPORT_NVLINK, learning_rate=0.01, bf16_compute_cache=1),
                       device=dev, seed=2, use_graph=True, bf16_weights_only=True)
        gen = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(B, 3, 227, 227, device=dev, generator=gen)
        y = torch.randint(0, 1000, (B,), device=dev, generator=gen)
        drop = next(l for l in mod.net.all_layers() if type(l).__name__ == "Dropout")
        losses, masks = [], []
        for i in range(30):
            losses.append(mod.step(x, y).item())
            masks.append((drop.y != 0).float().mean().item())
        assert len(mod._graphs) == 2
        assert mod.ps.last_error() == 0
        assert all(0.3 < m < 0.7 for m in masks), masks
        zs = [(drop.y == 0).clone()]
        mod.step(x, y)
        zs.append((drop.y == 0).clone())
        assert not torch.equal(zs[0], zs[1])                  # a new mask every step, also under replay
        assert sum(losses[-5:]) / 5 < sum(losses[:5]) / 5, losses
        mod.close()


def test_uint8_batches_with_augmentation_train_like_float_batches_under_graph_replay():
    """8-bit source images, cropped / mirrored / normalised by the input layer with a new augmentation every step: the
    captured step reads the augmentation from the layer's buffer, so replayed steps follow it and the losses equal
    those of a module fed the same crops as float batches through the layer code."""
    dev = torch.device("cuda:0")
    B, Hin, Win, H, W, steps = 32, 20, 22, 16, 16, 12
    mean, scale = (120.0, 128.0, 131.0), 1.0 / 64.0
    gen = torch.Generator(device=dev).manual_seed(7)
    x8 = torch.randint(0, 256, (B, 3, Hin, Win), device=dev, generator=gen, dtype=torch.uint8)
    y = torch.randint(0, 10, (B,), device=dev, generator=gen)
    augs = [torch.stack([torch.randint(0, Hin - H + 1, (B,), generator=gen, device=dev),
                         torch.randint(0, Win - W + 1, (B,), generator=gen, device=dev),
                         torch.randint(0, 2, (B,), generator=gen, device=dev)], dim=1) for _ in range(steps)]
    m = torch.tensor(mean, device=dev).view(1, 3, 1, 1)

    def as_float(aug):
        rows = []
        for b in range(B):
            ho, wo, mir = (int(v) for v in aug[b])
            win = x8[b:b + 1, :, ho:ho + H, wo:wo + W].float()
            rows.append(win.flip(-1) if mir else win)
        return ((torch.cat(rows) - m) * scale).contiguous()

    losses = {}
    for u8 in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            mod = PSModule(tiny_net(), (B, 3, H, W), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=3,
                           use_graph=u8)
            inp = mod.net.input_layer
            inp.set_transform(mean, scale)
            out = []
            for aug in augs:
                if u8:
                    inp.set_augmentation(aug)
                    out.append(mod.step(x8, y).item())
                else:
                    out.append(mod.step(as_float(aug), y).item())
            if u8:
                assert len(mod._graphs) >= 1 and mod.ps.get_stats()["client"]["nr_replayed_clocks"] > 0
            assert mod.ps.last_error() == 0
            losses[u8] = out
            mod.close()
    assert losses[True] == pytest.approx(losses[False], rel=2e-3), losses
    assert len(set(round(v, 5) for v in losses[True])) > steps // 2          # the batches did differ from step to step


@pytest.mark.parametrize("graph", [False, True])
def test_hyper_parameter_changes_take_effect_at_the_next_step(graph):
    """set_hyper_params between steps on the NVLINK path: with learning rate and momentum at zero the shard's step
    leaves the parameters where they are (the loss on a fixed batch stops moving), and training picks up again when
    they come back.  Under graph replay the captured steps are dropped at every change and captured again."""
    dev = torch.device("cuda:0")
    B = 32
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=3,
                       use_graph=graph)
        gen = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn(B, 3, 16, 16, device=dev, generator=gen)
        y = torch.randint(0, 10, (B,), device=dev, generator=gen)
        assert mod.ps.hyper_params() == pytest.approx((0.05, 0.9, 0.0))
        losses = []
        for i in range(24):
            if i == 8:
                mod.set_hyper_params(learning_rate=0.0, momentum=0.0)
                assert not mod._graphs and not mod._tapes
            if i == 14:
                mod.set_hyper_params(learning_rate=0.05, momentum=0.9)
            losses.append(mod.step(x, y).item())
        assert mod.ps.last_error() == 0
        if graph:
            assert len(mod._graphs) >= 1 and mod.ps.get_stats()["client"]["nr_replayed_clocks"] > 0
        mod.close()
    # (the loss is a sum of per-sample terms added in no fixed order: equal up to rounding)
    assert abs(losses[8] - losses[7]) > 2e-5, losses                # the update of step 7 still moved the parameters
    assert all(abs(v - losses[8]) <= 1e-5 * abs(losses[8]) for v in losses[9:15]), losses    # steps 8 .. 13 did not
    assert abs(losses[15] - losses[14]) > 2e-5 and losses[-1] < losses[0], losses


def test_snapshot_and_resume_on_the_nvlink_path(tmp_path):
    """Table snapshot of a training run on the GPU transport (master rows, momentum, clocks read from the device
    arena) and a new module resumed from it: the resumed run continues with the losses of the original one."""
    dev = torch.device("cuda:0")
    B = 32
    gen = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(B, 3, 16, 16, device=dev, generator=gen)
    y = torch.randint(0, 10, (B,), device=dev, generator=gen)
    snap = str(tmp_path / "snap")
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=3)
        first = [mod.step(x, y).item() for _ in range(6)]
        mod.save_snapshot(snap)
        clock = mod.ps.clock_value
        cont = [mod.step(x, y).item() for _ in range(4)]
        assert mod.ps.last_error() == 0
        mod.close()
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=99,
                       resume_from=snap)
        assert mod.ps.clock_value == clock and mod.steps == 6
        resumed = [mod.step(x, y).item() for _ in range(4)]
        assert mod.ps.last_error() == 0
        mod.close()
    assert resumed == pytest.approx(cont, rel=2e-3), (first, cont, resumed)
    assert abs(resumed[0] - first[0]) > 1e-3          # not a fresh start


@pytest.mark.parametrize("mode", ["pull_fc", "uncached"])
def test_uncached_tables_train_like_published_ones(mode):
    """Tables the shards do not publish: (pull_fc) the fully-connected layers pull their weight rows from the shards
    inside the forward GEMM, (uncached) a convolution's table is fetched from the shards by every Read.  Both give
    the losses of the ordinary publish path, bit for bit in the first case (same bf16 rows, same GEMM order)."""
    dev = torch.device("cuda:0")
    B = 64
    losses, stats = {}, {}
    for on in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            kw = {}
            if on:
                kw = dict(pull_fc=True) if mode == "pull_fc" else dict(uncached=("c2",))
            mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=3,
                           use_graph=True, **kw)
            gen = torch.Generator(device=dev).manual_seed(5)
            x = torch.randn(B, 3, 16, 16, device=dev, generator=gen)
            y = torch.randint(0, 10, (B,), device=dev, generator=gen)
            losses[on] = [mod.step(x, y).item() for _ in range(12)]
            torch.cuda.synchronize()
            assert mod.ps.last_error() == 0
            stats[on] = mod.ps.get_stats()["client"]
            plan = mod.ps.plan()
            pulled = [t for t in plan["tables"] if t["pull"]]
            assert (len(pulled) > 0) == on
            if on:
                assert plan["uncached_param_rows"] == sum(t["num_rows"] for t in pulled)
            mod.close()
    assert stats[True]["rows_pulled"] > 0 and stats[False]["rows_pulled"] == 0
    if mode == "pull_fc":
        assert stats[True]["nr_read_pull"] > 0
    assert losses[True] == pytest.approx(losses[False], rel=1e-3), losses
    assert losses[True][-1] < losses[True][0]


def test_bf16_only_weight_publish_trains_identically():
    """Weights published to the bf16 caches only: same losses (the layers never read fp32 weights), biases still
    refreshed in fp32, fp32 weight views left at their initial values."""
    dev = torch.device("cuda:0")
    B = 64
    losses, mods = {}, {}
    for only16 in (False, True):
        with torch.cuda.stream(torch.cuda.Stream(device=dev)):
            mod = PSModule(tiny_net(), (B, 3, 16, 16), cfg(TRANSPORT_NVLINK, learning_rate=0.05), device=dev, seed=3,
                           keep_init=True, bf16_weights_only=only16)
            gen = torch.Generator(device=dev).manual_seed(5)
            x = torch.randn(B, 3, 16, 16, device=dev, generator=gen)
            y = torch.randint(0, 10, (B,), device=dev, generator=gen)
            losses[only16] = [mod.step(x, y).item() for _ in range(6)]
            torch.cuda.synchronize()
            p = {k: v.clone() for k, v in mod.params_fp32().items()}
            init = mod.initial_params
            wname = next(k for k in p if k.endswith(".weight"))
            bname = next(k for k in p if k.endswith(".bias"))
            assert not torch.equal(p[bname].cpu(), init[bname].cpu())          # biases move in fp32 either way
            assert torch.equal(p[wname].cpu(), init[wname].cpu()) == only16    # fp32 weights only when published
            assert mod.ps.last_error() == 0
            mod.close()
    assert losses[True] == pytest.approx(losses[False], rel=1e-3), losses
