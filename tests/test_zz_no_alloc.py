"""Allocation-free BatchNorm forward (geeps_bn_forward_noalloc).

Some users of the library cannot hand a kernel scratch memory: code that runs inside the parameter
server's fully planned GPU budget has no allocator once the clocks are running, and a host program
that links the library without a device allocator of its own does not want cudaMalloc (which
synchronises the whole device) inside its step loop.  For them the entry point takes its reduction
scratch from a fixed array inside the library.  This test calls it through the exported C symbol
and checks it against the ordinary entry point, twice in a row, because the built-in array keeps
the previous call's contents and must be cleared by the call itself.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from geeps_b200 import _native
    lib = C.CDLL(str(_native.build()))          # exported C symbols, no Python wrapper in between
    return lib.geeps_bn_forward_noalloc, lib.geeps_bn_forward, lib.geeps_bn_noalloc_max_channels


def _call_noalloc(fn, x, y, gamma, beta, mean_rstd, relu, stream):
    P, Cc = x.shape
    return fn(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(gamma.data_ptr()),
              C.c_void_p(beta.data_ptr()), C.c_void_p(mean_rstd.data_ptr()), C.c_void_p(0), C.c_void_p(0),
              C.c_longlong(P), C.c_int(Cc), C.c_longlong(x.stride(0)), C.c_longlong(y.stride(0)),
              C.c_float(1e-5), C.c_float(0.1), C.c_int(int(relu)), C.c_void_p(stream))


def _call_plain(fn, x, y, gamma, beta, sums, mean_rstd, relu, stream):
    P, Cc = x.shape
    return fn(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(gamma.data_ptr()),
              C.c_void_p(beta.data_ptr()), C.c_void_p(sums.data_ptr()), C.c_void_p(mean_rstd.data_ptr()),
              C.c_void_p(0), C.c_void_p(0), C.c_longlong(P), C.c_int(Cc), C.c_longlong(x.stride(0)),
              C.c_longlong(y.stride(0)), C.c_float(1e-5), C.c_float(0.1), C.c_int(int(relu)), C.c_void_p(stream))


def test_bn_forward_noalloc_matches_plain_entry_point_twice():
    noalloc, plain, max_channels = _sym()
    dev = torch.device("cuda:0")
    torch.manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream or 1   # 0x1 = CUDA's legacy default stream
    # two calls in a row with different widths: the second one reuses (part of) the array the first one
    # filled, so stale sums would show up as wrong statistics
    for call, (P, Cc, relu) in enumerate([(4000, 96, True), (2500, 48, False)]):
        x = (torch.randn(P, Cc, device=dev) * (call + 1.5) + call).to(torch.bfloat16)
        gamma = torch.rand(Cc, device=dev) + 0.5
        beta = torch.randn(Cc, device=dev) * 0.1
        y0, y1 = torch.empty_like(x), torch.empty_like(x)
        mr0, mr1 = torch.empty(2 * Cc, device=dev), torch.empty(2 * Cc, device=dev)
        sums = torch.empty(2 * Cc, device=dev)
        torch.cuda.synchronize()
        assert _call_plain(plain, x, y0, gamma, beta, sums, mr0, relu, stream) == 0
        assert _call_noalloc(noalloc, x, y1, gamma, beta, mr1, relu, stream) == 0
        torch.cuda.synchronize()
        assert torch.allclose(mr1, mr0, atol=1e-4, rtol=1e-4), (call, (mr1 - mr0).abs().max().item())
        assert torch.allclose(y1.float(), y0.float(), atol=3e-2, rtol=2e-2), call
        ref = torch.nn.functional.batch_norm(x.float(), None, None, gamma, beta, training=True, eps=1e-5)
        if relu:
            ref = torch.relu(ref)
        assert torch.allclose(y1.float(), ref, atol=3e-2, rtol=2e-2), call


def test_bn_forward_noalloc_rejects_too_many_channels():
    noalloc, _, max_channels = _sym()
    dev = torch.device("cuda:0")
    Cc = max_channels() + 8
    x = torch.zeros(16, Cc, dtype=torch.bfloat16, device=dev)
    y = torch.empty_like(x)
    g = torch.ones(Cc, device=dev)
    b = torch.zeros(Cc, device=dev)
    mr = torch.zeros(2 * Cc, device=dev)
    rc = _call_noalloc(noalloc, x, y, g, b, mr, False, torch.cuda.current_stream().cuda_stream or 1)
    assert rc == -2                          # GEEPS_ERR_NOALLOC_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
    assert mr.abs().sum().item() == 0
