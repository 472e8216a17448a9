"""Tuned kernels against the shape-general kernels of the same entry points on seeded random row counts, both storage
types: every output byte (pad rows included) must be equal. The general kernels are compared with the reference's own
kernels and the CPU oracle elsewhere; this file covers the row counts, ragged last tiles and grid tails in between."""
import numpy as np
import pytest
import torch

import aiis_clef_b200 as clef

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _restore_choice():
    clef.set_kernel_choice(0)
    yield
    clef.set_kernel_choice(0)
    torch.cuda.empty_cache()


def both(fn):
    """The entry point's outputs on the tuned (0) and on the shape-general (1) kernels."""
    got = []
    for choice in (0, 1):
        clef.set_kernel_choice(choice)
        out = fn()
        torch.cuda.synchronize()
        got.append([t for t in (out if isinstance(out, (tuple, list)) else (out,)) if t is not None])
    clef.set_kernel_choice(0)
    return got


def assert_same(name, rows, got):
    tuned, general = got
    assert len(tuned) == len(general)
    for i, (a, b) in enumerate(zip(tuned, general)):
        assert a.dtype == b.dtype and a.shape == b.shape
        same = torch.equal(a.view(torch.uint8), b.view(torch.uint8))
        assert same, f"{name}, {rows} rows, output {i}: tuned and general kernels differ"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
@pytest.mark.parametrize("seed", range(6))
def test_random_row_counts_tuned_equals_general(seed, dtype):
    dev = clef.Device(0)
    rng = np.random.default_rng(1000 + seed)
    gen = torch.Generator(device="cuda").manual_seed(2000 + seed)
    rows = int(rng.integers(1, 2600))
    hidden = int(rng.choice([2048, 4096]))
    inter = int(rng.choice([1536, 2048, 6144]))
    heads, kv_heads, vh = int(rng.choice([3, 8, 16])), int(rng.choice([1, 2, 4])), int(rng.choice([8, 16, 32]))
    gs = float(rng.choice([1.0, 48.0, 215.0, 1.0 / 12.5]))

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=gen) * scale).to(dtype)

    x = rnd(rows, hidden, scale=1.5)
    x[:, int(rng.integers(0, hidden))] *= 30.0
    x[rows // 2] = 0.0
    res = rnd(rows, hidden)
    w = torch.randn(hidden, device="cuda", generator=gen) * 0.2
    gate, up = rnd(rows, inter, scale=3.0), rnd(rows, inter, scale=2.0)
    gate[:, 5] *= 20.0                                    # beyond the short silu's range
    assert_same("rms_norm", rows, both(lambda: dev.rms_norm_dev(x, w, rows, hidden, 1e-6)))
    assert_same("quantise_nvfp4", rows, both(lambda: dev.quantise_nvfp4_dev(x, rows, hidden, gs, 128)))
    assert_same("rms_norm_quantise_nvfp4", rows, both(lambda: dev.rms_norm_quantise_nvfp4_dev(x, w, rows, hidden, 1e-6, gs, 128)))
    assert_same("add_rms_norm_quantise_nvfp4", rows,
                both(lambda: dev.add_rms_norm_quantise_nvfp4_dev(x, res, w, rows, hidden, 1e-6, gs, 128)))
    assert_same("swiglu_quantise_nvfp4", rows, both(lambda: dev.swiglu_quantise_nvfp4_dev(gate, up, rows, inter, gs, 128)))
    assert_same("sigmoid_mul_quantise_nvfp4", rows,
                both(lambda: dev.sigmoid_mul_quantise_nvfp4_dev(up[:, :1536].contiguous(), gate[:, :1536].contiguous(), rows, 1536, gs, 128)))
    assert_same("quantise_fp8", rows, both(lambda: dev.quantise_fp8_dev(gate, rows, inter)))
    assert_same("swiglu_quantise_fp8", rows, both(lambda: dev.swiglu_quantise_fp8_dev(gate, up, rows, inter)))
    fp8 = both(lambda: dev.rms_norm_fp8_bf16_dev(x, w, rows, hidden, 1e-6))
    assert_same("rms_norm_fp8_bf16", rows, [t[:2] for t in fp8])   # codes and scales; the twin's NaN pattern is not compared
    # 128-wide heads: the gated norm and its two quantisers
    hr = rows * vh
    o, z = rnd(hr, 128, scale=1.5), rnd(hr, 128, scale=3.0)
    wg = 1.0 + torch.randn(128, device="cuda", generator=gen) * 0.1
    assert_same("rms_norm_gated", rows, both(lambda: dev.rms_norm_gated_dev(o, z, wg, hr, 128, 1e-6)))
    assert_same("rms_norm_gated_quantise_nvfp4", rows,
                both(lambda: dev.rms_norm_gated_quantise_nvfp4_dev(o, z, wg, hr, 128, vh, 1e-6, gs, 128)))
    assert_same("rms_norm_gated_quantise_fp8", rows, both(lambda: dev.rms_norm_gated_quantise_fp8_dev(o, z, wg, hr, 128, vh, 1e-6)))
    # RoPE and the per-head norm + RoPE through a shuffled position map
    pos = torch.from_numpy(rng.permutation(rows).astype(np.int32)).cuda()
    cos, sin = dev.rope_tables_dev(torch.arange(rows, dtype=torch.int32, device="cuda"), rows, 64, 1e6)
    q, k = rnd(rows, heads, 128), rnd(rows, kv_heads, 128)
    wh = torch.randn(128, device="cuda", generator=gen) * 0.1
    assert_same("rope", rows, both(lambda: dev.rope_apply_dev(q, cos, sin, rows, heads, 128, 64, pos_map=pos)))
    assert_same("rope_qk", rows, both(lambda: dev.rope_qk_dev(q.clone(), k.clone(), cos, sin, rows, heads, kv_heads, 128, 64, pos_map=pos)))
    assert_same("qk_norm_rope 128", rows,
                both(lambda: dev.qk_norm_rope_dev(q.view(rows * heads, 128), wh, cos, sin, rows * heads, heads, 128, 64, 1e-6, pos_map=pos)))
    qg = rnd(rows * heads, 256)
    assert_same("qk_norm_rope 128 + gate", rows,
                both(lambda: dev.qk_norm_rope_dev(qg, wh, cos, sin, rows * heads, heads, 128, 64, 1e-6, pos_map=pos, with_gate=True)))
    q256 = rnd(rows * heads, 512)
    wh256 = torch.randn(256, device="cuda", generator=gen) * 0.1
    assert_same("qk_norm_rope 256 + gate", rows,
                both(lambda: dev.qk_norm_rope_dev(q256, wh256, cos, sin, rows * heads, heads, 256, 64, 1e-6, pos_map=pos, with_gate=True)))
    # the causal convolution in front of the GDN scan, two sequences
    channels = int(rng.choice([512, 8192]))
    mixed = rnd(rows, channels)
    wc = torch.randn(channels, 4, device="cuda", generator=gen) * 0.5
    starts = torch.zeros(rows, dtype=torch.int32, device="cuda")
    starts[rows // 3:] = rows // 3
    assert_same("causal_conv_silu", rows, both(lambda: dev.causal_conv_silu_dev(mixed, wc, rows, channels, 4, seq_start=starts)))
