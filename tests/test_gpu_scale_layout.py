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
@pytest.mark.parametrize("f32", [False, True], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(7, 2048), (778, 2048), (300, 4096), (129, 512), (65, 1088)])
def test_rms_norm_and_plain_quantiser(rows, cols, tile_m, choice, f32):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(rows + cols + tile_m)
    as_dev = (lambda bits: dev_bf16(bits).float()) if f32 else dev_bf16
    x = as_dev(normal_bf16(rng, (rows, cols), outlier_channels=3))
    w = torch.from_numpy((rng.standard_normal(cols) * 0.1).astype(np.float32)).cuda()
    check(*both_layouts(lambda: dev.rms_norm_quantise_nvfp4_dev(x, w, rows, cols, 1e-6, 64.0, tile_m)), rows, cols, tile_m)
    check(*both_layouts(lambda: dev.quantise_nvfp4_dev(x, rows, cols, 3.0, tile_m)), rows, cols, tile_m)
    b = as_dev(normal_bf16(rng, (rows, cols)))
    check(*both_layouts(lambda: dev.add_rms_norm_quantise_nvfp4_dev(x, b, w, rows, cols, 1e-6, 64.0, tile_m)[1:]), rows, cols, tile_m)


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tile_m", [128, 192])
@pytest.mark.parametrize("f32", [False, True], ids=["bf16", "f32"])
@pytest.mark.parametrize("rows,cols", [(5, 6144), (778, 1024), (130, 576)])
def test_swiglu_and_sigmoid_mul(rows, cols, tile_m, choice, f32):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(rows * cols + tile_m)
    as_dev = (lambda bits: dev_bf16(bits).float()) if f32 else dev_bf16
    g = as_dev(to_bf16_bits((rng.standard_normal((rows, cols)) * 2).astype(np.float32)))
    u = as_dev(normal_bf16(rng, (rows, cols)))
    check(*both_layouts(lambda: dev.swiglu_quantise_nvfp4_dev(g, u, rows, cols, 48.0, tile_m)), rows, cols, tile_m)
    check(*both_layouts(lambda: dev.sigmoid_mul_quantise_nvfp4_dev(u, g, rows, cols, 48.0, tile_m)), rows, cols, tile_m)


@pytest.mark.parametrize("choice", [0, 1], ids=["tuned", "general"])
@pytest.mark.parametrize("tile_m", [128, 192])
@pytest.mark.parametrize("f32", [False, True], ids=["bf16", "f32"])
@pytest.mark.parametrize("tokens,vh", [(7, 16), (300, 16), (129, 32)])
def test_gated_norm(tokens, vh, tile_m, choice, f32):
    clef.set_kernel_choice(choice)
    dev = clef.Device(0)
    rng = np.random.default_rng(tokens * vh + tile_m)
    as_dev = (lambda bits: dev_bf16(bits).float()) if f32 else dev_bf16
    o = as_dev(normal_bf16(rng, (tokens * vh, 128)))
    z = as_dev(normal_bf16(rng, (tokens * vh, 128)))
    w = torch.from_numpy((1.0 + rng.standard_normal(128) * 0.1).astype(np.float32)).cuda()
    p0, s0, p1, s1 = both_layouts(lambda: dev.rms_norm_gated_quantise_nvfp4_dev(o, z, w, tokens * vh, 128, vh, 1e-6, 96.0, tile_m))
    check(p0, s0, p1, s1, tokens, vh * 128, tile_m)


def test_layout_argument_is_checked():
    assert clef.load().clef_set_scale_layout(2) == -1
    assert clef.load().clef_set_scale_layout(clef.SF_INTERLEAVED) == 0


def test_two_streams_use_different_orders_at_the_same_time():
    """The `_ex` entry points take the tile order per call: two streams quantise with different orders, interleaved
    call by call, while the process default stays untouched; every result equals the one the process-wide switch
    gives for that order. Covers the six `_ex` entry points."""
    import ctypes

    from gpu_util import Guarded, call, ptr

    lib = clef.load()
    rows, cols, inter, vh = 300, 2048, 1024, 16
    rp = (rows + 127) // 128 * 128
    rng = np.random.default_rng(91)
    x, b = dev_bf16(normal_bf16(rng, (rows, cols), outlier_channels=3)), dev_bf16(normal_bf16(rng, (rows, cols)))
    g, u = dev_bf16(normal_bf16(rng, (rows, inter))), dev_bf16(normal_bf16(rng, (rows, inter)))
    o, z = dev_bf16(normal_bf16(rng, (rows * vh, 128))), dev_bf16(normal_bf16(rng, (rows * vh, 128)))
    w = torch.from_numpy((rng.standard_normal(cols) * 0.1).astype(np.float32)).cuda()
    wg = torch.from_numpy((1.0 + rng.standard_normal(128) * 0.1).astype(np.float32)).cuda()
    torch.cuda.synchronize()

    def run_all(stream_handle, layout, ex):
        """The six quantising calls on one stream; returns the guarded (packed, scales) pairs."""
        sfx = "_ex" if ex else ""
        tail = [layout] if ex else []
        outs = []

        def buffers(c):
            pair = (Guarded(rp * c // 2), Guarded(rp * c // 16))
            outs.append(pair)
            return pair[0].ptr, pair[1].ptr

        s = ctypes.c_void_p(stream_handle)
        pk, sc = buffers(cols)
        assert call("clef_quantise_nvfp4" + sfx, s, ptr(x), pk, sc, rows, cols, 3.0, 128, 512, 0, *tail) == 0
        pk, sc = buffers(cols)
        assert call("clef_rms_norm_quantise_nvfp4" + sfx, s, ptr(x), ptr(w), pk, sc, rows, cols, 1e-6, 64.0, 128, 512, 0, *tail) == 0
        pk, sc = buffers(vh * 128)
        assert call("clef_rms_norm_gated_quantise_nvfp4" + sfx, s, ptr(o), ptr(z), ptr(wg), pk, sc, rp * vh, 128, 1e-6, 96.0, 128, 512,
                    vh, rows * vh, 0, *tail) == 0
        pk, sc = buffers(inter)
        assert call("clef_swiglu_quantise_nvfp4" + sfx, s, ptr(g), ptr(u), pk, sc, rows, inter, 48.0, 128, 512, 0, *tail) == 0
        pk, sc = buffers(inter)
        assert call("clef_sigmoid_mul_quantise_nvfp4" + sfx, s, ptr(u), ptr(g), pk, sc, rows, inter, 48.0, 128, 512, 0, *tail) == 0
        pk, sc = buffers(cols)
        total = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
        assert call("clef_add_rms_norm_quantise_nvfp4" + sfx, s, ptr(total), ptr(x), ptr(b), ptr(w), pk, sc, rows, cols, 1e-6, 64.0,
                    128, 512, 0, *tail) == 0
        return outs, total

    # what each order gives through the process-wide switch
    want = {}
    for layout in (clef.SF_ACTIVATION, clef.SF_INTERLEAVED):
        clef.set_scale_layout(layout)
        outs, _ = run_all(torch.cuda.current_stream().cuda_stream, layout, ex=False)
        torch.cuda.synchronize()
        want[layout] = [(p.bytes(), s.bytes()) for p, s in outs]
    clef.set_scale_layout(clef.SF_ACTIVATION)
    assert not np.array_equal(want[0][0][1], want[1][0][1])

    s_a, s_b = torch.cuda.Stream(), torch.cuda.Stream()
    got = {0: [], 1: []}
    keep = []
    for _ in range(3):   # both streams stay busy while the other one launches
        for layout, st in ((clef.SF_INTERLEAVED, s_b), (clef.SF_ACTIVATION, s_a)):
            outs, total = run_all(st.cuda_stream, layout, ex=True)
            got[layout] = outs
            keep.append((outs, total))
    torch.cuda.synchronize()
    for layout in (0, 1):
        for (p, s), (wp, ws) in zip(got[layout], want[layout]):
            p.check_guards("packed")
            s.check_guards("scales")
            assert np.array_equal(p.bytes(), wp) and np.array_equal(s.bytes(), ws)
    # the process default was not touched by the per-call orders
    pk, sc = Guarded(rp * cols // 2), Guarded(rp * cols // 16)
    assert call("clef_quantise_nvfp4", ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ptr(x), pk.ptr, sc.ptr, rows, cols,
                3.0, 128, 512, 0) == 0
    torch.cuda.synchronize()
    assert np.array_equal(sc.bytes(), want[0][0][1])
    assert lib.clef_quantise_nvfp4_ex(None, ptr(x), pk.ptr, sc.ptr, rows, cols, 3.0, 48, 192, 0, clef.SF_INTERLEAVED) == -1
