"""Geometry of the halo-tile convolution kernels over a sweep of layer shapes (host arithmetic only, no GPU): every
plan the kernels would accept keeps its tiles inside shared memory, tensor memory and the MMA's shape limits."""
import ctypes as C
import itertools

import pytest

from geeps_b200.ops import _lib as L

SMEM_LIMIT = 227 * 1024


def _params(mode, B, H, W, cg, og, k, pad, stride=1):
    p = L.ConvTcParams()
    # the planners only look at shapes, pitches and alignment: any 16-byte aligned non-null addresses will do
    p.x, p.y, p.w = 0x10000, 0x20000, 0x30000
    p.bias, p.status = None, None
    OH, OW = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    p.x_pitch, p.y_pitch = cg, og
    p.ldw = (k * k * cg + 7) // 8 * 8
    p.B, p.H, p.W, p.cg, p.OH, p.OW, p.og = B, H, W, cg, OH, OW, og
    p.KH, p.KW, p.pad, p.relu, p.mode, p.split_k, p.stride = k, k, pad, 0, mode, 0, stride
    return p, OH, OW


SHAPES = [(B, H, cg, og, k, pad)
          for B, H, (cg, og), (k, pad) in itertools.product(
              (1, 8, 32, 256), (7, 13, 14, 27, 28, 55, 56, 57, 64, 112),
              ((8, 16), (16, 40), (32, 96), (48, 128), (64, 192), (96, 96), (192, 384), (256, 256)),
              ((2, 0), (3, 0), (3, 1), (5, 2), (7, 3)))
          if H + 2 * pad >= k]


@pytest.mark.parametrize("mode", [0, 1])
def test_forward_and_data_gradient_plans_respect_the_hardware_limits(mode):
    lib = L.lib()
    seen = routed = 0
    for B, H, cg, og, k, pad in SHAPES:
        p, OH, OW = _params(mode, B, H, H, cg, og, k, pad)
        info = L.HaloPlanInfo()
        if not lib.geeps_conv_halo_plan(C.byref(p), C.byref(info)):
            assert info.ok == 0
            continue
        seen += 1
        routed += info.routed
        GW, GH = (OW, OH) if mode == 0 else (H, H)
        nch = og if mode == 0 else cg
        assert info.PW >= GW + k - 1 and info.PW <= 128
        assert info.positions == info.R * info.PW and info.positions % 8 == 0 and 0 < info.positions <= 128
        assert info.ncols2 % 16 == 0 and 2 * info.positions <= info.ncols2 <= 256
        assert info.ncols1 % 16 == 0 and info.positions <= info.ncols1 <= 128
        assert 2 * info.R * info.row_tiles >= GH                     # the tiles cover every output row
        assert 2 * info.R * (info.row_tiles - 1) < GH                # and no tile is entirely outside the image
        assert info.m_tiles == (nch + 127) // 128
        # a tap-shifted MMA of ncols2 rows stays inside one activation stage
        rows_read = (k - 1) * info.PW + (k - 1) + info.ncols2
        assert rows_read * 128 <= info.x_stage_bytes
        assert ((2 * info.R + k - 1) * info.PW) * 128 <= info.x_stage_bytes
        assert info.x_stage_bytes % 1024 == 0
        assert info.stages_w >= 3 and info.stages_x == 2
        assert info.smem_bytes <= SMEM_LIMIT
        assert info.tmem_cols == 512
        assert 0.0 < info.util <= 1.0
    assert seen > 100 and routed > 0


def test_strided_calls_are_not_given_to_the_halo_kernels():
    lib = L.lib()
    for mode in (0, 1, 2):
        p, _, _ = _params(mode, 32, 28, 28, 64, 96, 3, 1, stride=2)
        info = L.HaloPlanInfo()
        fn = lib.geeps_conv_wgrad_halo_plan if mode == 2 else lib.geeps_conv_halo_plan
        assert fn(C.byref(p), C.byref(info)) == 0 and info.ok == 0


def test_weight_gradient_plans_respect_the_hardware_limits():
    lib = L.lib()
    seen = routed = 0
    for B, H, cg, og, k, pad in SHAPES:
        p, OH, OW = _params(2, B, H, H, cg, og, k, pad)
        p.ldw = (k * k * cg + 3) // 4 * 4
        info = L.HaloPlanInfo()
        if not lib.geeps_conv_wgrad_halo_plan(C.byref(p), C.byref(info)):
            continue
        seen += 1
        routed += info.routed
        assert info.PW >= OW + k - 1 and info.PW <= 128
        assert info.positions == info.R * info.PW and info.positions % 16 == 0 and 0 < info.positions <= 128
        assert 1 <= info.TY <= k and info.TY * k * 64 <= 512 and info.passes == -(-k // info.TY)
        assert info.tmem_cols >= info.TY * k * 64 and info.tmem_cols <= 512
        assert info.n_blocks == B * info.row_tiles and info.R * info.row_tiles >= OH
        per = -(-info.n_blocks // info.split)
        assert 1 <= info.split <= info.n_blocks and per * (info.split - 1) < info.n_blocks    # no empty slice
        rows_read = (info.TY - 1) * info.PW + (k - 1) + info.positions
        assert rows_read * 128 <= info.x_stage_bytes
        assert info.stages_x >= 2 and info.smem_bytes <= SMEM_LIMIT
    assert seen > 100 and routed > 0
