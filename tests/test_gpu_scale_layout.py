"""The interleaved (32 x 4 x 4) scale-tile order, selected by clef_set_scale_layout, for every NVFP4 entry point:
packed codes are unchanged, and the scale bytes are the activation-side bytes rearranged exactly as
src/swizzle.rs:66-68 (restated by the oracle's swizzle_tiled, which the CPU tests pin) arranges a row-major matrix."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef
from oracle import binding as orc
from gpu_util import dev_bf16, unswizzle
from util import normal_bf16, to_bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _reset():
    clef.set_kernel_choice(0)
    clef.set_scale_layout(clef.SF_ACTIVATION)
    yield
    clef.set_kernel_choice(0)
    clef.set_scale_layout(clef.SF_ACTIVATION)


def both_layouts(run):
    clef.set_scale_layout(clef.SF_ACTIVATION)
    p0, s0 = run()
    clef.set_scale_layout(clef.SF_INTERLEAVED)
    p1, s1 = run()
    torch.cuda.synchronize()
    return p0.cpu().numpy(), s0.cpu().numpy(), p1.cpu().numpy(), s1.cpu().numpy()


def check(p0, s0, p1, s1, rows, cols, tile_m):
    blk_mn = orc.blk_mn_for_tile_m(tile_m)
    rows_padded = (rows + blk_mn - 1) // blk_mn * blk_mn
    blocks = cols // 16
    assert np.array_equal(p0, p1), "the packed codes must not depend on the scale layout"
    row_major = unswizzle(s0.reshape(-1), rows_padded, blocks, blk_mn)
    want = orc.swizzle_tiled(row_major, rows_padded, blocks, tile_m, conflict_free=False)
    assert np.array_equal(s1.reshape(-1), want), "interleaved scale bytes differ from swizzle.rs's arrangement"
    assert not np.array_equal(s0, s1) or rows_padded <= 32


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tile_m", [128, 192])
@pytest.mark.parametrize("rows,cols", [(7, 2048), (778, 2048), (300, 4096), (129, 512), (65, 1088)])
def test_rms_norm_and_plain_quantiser(rows, cols, tile_m, choice):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(rows + cols + tile_m)
    x = dev_bf16(normal_bf16(rng, (rows, cols), outlier_channels=3))
    w = torch.from_numpy((rng.standard_normal(cols) * 0.1).astype(np.float32)).cuda()
    check(*both_layouts(lambda: dev.rms_norm_quantise_nvfp4_dev(x, w, rows, cols, 1e-6, 64.0, tile_m)), rows, cols, tile_m)
    check(*both_layouts(lambda: dev.quantise_nvfp4_dev(x, rows, cols, 3.0, tile_m)), rows, cols, tile_m)
    b = dev_bf16(normal_bf16(rng, (rows, cols)))
    check(*both_layouts(lambda: dev.add_rms_norm_quantise_nvfp4_dev(x, b, w, rows, cols, 1e-6, 64.0, tile_m)[1:]), rows, cols, tile_m)


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tile_m", [128, 192])
@pytest.mark.parametrize("rows,cols", [(5, 6144), (778, 1024), (130, 576)])
def test_swiglu_and_sigmoid_mul(rows, cols, tile_m, choice):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(rows * cols + tile_m)
    g = dev_bf16(to_bf16_bits((rng.standard_normal((rows, cols)) * 2).astype(np.float32)))
    u = dev_bf16(normal_bf16(rng, (rows, cols)))
    check(*both_layouts(lambda: dev.swiglu_quantise_nvfp4_dev(g, u, rows, cols, 48.0, tile_m)), rows, cols, tile_m)
    check(*both_layouts(lambda: dev.sigmoid_mul_quantise_nvfp4_dev(u, g, rows, cols, 48.0, tile_m)), rows, cols, tile_m)


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tile_m", [128, 192])
@pytest.mark.parametrize("tokens,vh", [(7, 16), (300, 16), (129, 32)])
def test_gated_norm(tokens, vh, tile_m, choice):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(tokens * vh + tile_m)
    o = dev_bf16(normal_bf16(rng, (tokens * vh, 128)))
    z = dev_bf16(normal_bf16(rng, (tokens * vh, 128)))
    w = torch.from_numpy((1.0 + rng.standard_normal(128) * 0.1).astype(np.float32)).cuda()
    p0, s0, p1, s1 = both_layouts(lambda: dev.rms_norm_gated_quantise_nvfp4_dev(o, z, w, tokens * vh, 128, vh, 1e-6, 96.0, tile_m))
    check(p0, s0, p1, s1, tokens, vh * 128, tile_m)


def test_layout_argument_is_checked():
    assert clef.load().clef_set_scale_layout(2) == -1
    assert clef.load().clef_set_scale_layout(clef.SF_INTERLEAVED) == 0
