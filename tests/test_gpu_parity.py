"""Loss parity with the library-ops baseline: the same network, the same initial weights and the same fixed batch
trained for the same number of momentum-SGD steps here (parameter server + sm_100a kernels, bf16 compute, fp32
master rows) and in plain PyTorch (cuDNN / cuBLAS, bf16 autocast).  The final loss here must not be worse."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.models.alexnet import alexnet
from geeps_b200.models.inception_bn import inception_bn_small
from geeps_b200.parallel.ps_module import PSModule
from geeps_b200.utils.config import DEVICE_CUDA, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK, GeePsConfig
from geeps_b200.utils.torch_mirror import TorchMirror, train_mirror

_port = [31000]


def _both(make_net, in_shape, classes, steps, lr):
    dev = torch.device("cuda:0")
    _port[0] += 20
    cfg = GeePsConfig(device=DEVICE_CUDA, cuda_device=0, transport=TRANSPORT_NVLINK, table_mode=TABLE_SGD_MOMENTUM,
                      tcp_base_port=_port[0], bf16_compute_cache=1, learning_rate=lr, momentum=0.9, weight_decay=0.0)
    gen = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn(in_shape, device=dev, generator=gen)
    y = torch.randint(0, classes, (in_shape[0],), device=dev, generator=gen)
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        mod = PSModule(make_net(), in_shape, cfg, device=dev, seed=4, keep_init=True, use_graph=True,
                       bf16_weights_only=True)
        ours = [mod.step(x, y).item() for _ in range(steps)]
        assert mod.ps.last_error() == 0
        torch.cuda.synchronize()
        mirror = TorchMirror(mod.net, in_shape).to(dev)
        mirror.load_initial(mod.initial_params)
        mod.close()
    mirror = mirror.to(memory_format=torch.channels_last)
    theirs = train_mirror(mirror, x.contiguous(memory_format=torch.channels_last), y, steps, lr, 0.9)
    return ours, theirs


def test_alexnet_loss_parity_with_torch():
    ours, theirs = _both(lambda: alexnet(dropout=0.0), (256, 3, 227, 227), 1000, 40, 0.01)
    print("alexnet ours  ", [round(v, 4) for v in ours[::5]], "\nalexnet torch ", [round(v, 4) for v in theirs[::5]])
    assert abs(ours[0] - theirs[0]) < 0.02, (ours[0], theirs[0])          # same weights, same batch, same forward
    assert theirs[-1] < theirs[0]
    assert ours[-1] <= theirs[-1] + 0.03, (ours[-1], theirs[-1])


def test_inception_bn_small_loss_parity_with_torch():
    ours, theirs = _both(inception_bn_small, (100, 3, 32, 32), 10, 40, 0.01)
    print("inception ours  ", [round(v, 4) for v in ours[::5]], "\ninception torch ", [round(v, 4) for v in theirs[::5]])
    assert abs(ours[0] - theirs[0]) < 0.05, (ours[0], theirs[0])
    assert theirs[-1] < theirs[0] - 0.2
    assert ours[-1] <= theirs[-1] + 0.05, (ours[-1], theirs[-1])
