"""Device-side comparison of the NVFP4 codec with the reference's encoder header
(kernels/nvfp4_quant.h compiled into oracle/_ref/ref_probe.cubin): every f32 bit pattern."""
import numpy as np
import pytest
import torch

from oracle import binding as orc
from oracle import ref_gpu
from gpu_util import unswizzle

pytestmark = pytest.mark.gpu


def _fmt(res):
    return ", ".join(f"{r['mismatches']}/{r['checked']} bad (first {[hex(b) for b in r['first_bad'][:6]]})" for r in res)


def test_e2m1_all_patterns():
    """Hardware-converter path on its domain (both nibbles) and the literal encoder everywhere."""
    res = ref_gpu.probe_e2m1(0, 1 << 32)
    assert res[2]["checked"] == 1 << 32
    assert res[0]["checked"] == res[1]["checked"] and res[0]["checked"] > (1 << 31)
    assert all(r["mismatches"] == 0 for r in res), _fmt(res)


def test_e4m3_encoder_all_patterns():
    """The encoders (the block-scale one, the FP8 quantisers' element one in its general, short and hardware-converter
    forms) against the reference's to_e4m3."""
    res = ref_gpu.probe_e4m3(0, 1 << 32)
    assert res[0]["checked"] == 1 << 32 and res[1]["checked"] == 1 << 32
    assert res[2]["checked"] == 0x43E80000            # every pattern of [+0, 464)
    assert res[3]["checked"] == 0x43E80000            # the hardware-converter form with its flagged bytes, the same patterns
    assert all(r["mismatches"] == 0 for r in res), _fmt(res)


@pytest.mark.parametrize("global_scale", [1.0, 64.0, 215.0, 1.0 / 12.5, 2688.0, 1e-3])
def test_e4m3_decoder_and_inverse_scale(global_scale):
    res = ref_gpu.probe_e4m3_decode(global_scale)
    assert res[0]["checked"] == 256 and res[1]["checked"] == 256
    assert all(r["mismatches"] == 0 for r in res), _fmt(res)


def _adversarial_blocks(rng):
    """Blocks that hit exact ties, sign corner cases, denormals, huge and non-finite values."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    blocks = []
    for amax in [6.0, 3.0, 1.0, 448.0, 0.001, 12.0]:
        base = np.zeros(16, np.float32)
        base[0] = amax                                    # scale maps amax to 6
        vals = ties * np.float32(amax / 6.0)
        for shift in (0, 1, -1):
            b = base.copy()
            v = vals.view(np.uint32).astype(np.int64) + shift
            b[1:8] = v.astype(np.uint32).view(np.float32)
            b[8:15] = -b[1:8]
            b[15] = -0.0
            blocks.append(b)
    blocks.append(np.zeros(16, np.float32))
    blocks.append(np.full(16, -0.0, np.float32))
    blocks.append(np.full(16, 1e-45, np.float32))                      # denormals only
    blocks.append(np.array([1e-40, -1e-40, 3e-39, 1.0] + [0] * 12, np.float32))
    blocks.append(np.array([np.nan, 1.0, -2.0, 3.0] + [0.5] * 12, np.float32))
    blocks.append(np.array([np.inf, 1.0, -2.0, 3.0] + [0.5] * 12, np.float32))
    blocks.append(np.array([-np.inf, np.nan, -2.0, 3.0] + [0.5] * 12, np.float32))
    blocks.append(np.array([3e38, -3e38, 1e30, 1e20] + [1.0] * 12, np.float32))
    blocks.append(np.array([1e12, -5e11, 1e9, 7e7] + [1.0] * 12, np.float32))
    blocks.append(np.full(16, np.nan, np.float32))
    rnd = rng.standard_normal((4096, 16)).astype(np.float32) * np.float32(10.0) ** rng.integers(-6, 6, (4096, 1)).astype(np.float32)
    out = np.concatenate([np.stack(blocks), rnd])
    return out[: out.shape[0] // 4 * 4]


@pytest.mark.parametrize("use_pairs", [False, True], ids=["scalar", "packed-pairs"])
@pytest.mark.parametrize("global_scale", [1.0, 64.0, 215.0, 1.0 / 12.5, 2688.0, 1e-6, 1e6, 0.0, -3.0, 3e38])
def test_block_quantiser_on_adversarial_blocks(global_scale, use_pairs):
    rng = np.random.default_rng(11)
    blocks = _adversarial_blocks(rng)
    vals = torch.from_numpy(blocks).cuda()
    res, ws, wp, gs, gp = ref_gpu.probe_blocks(vals, global_scale, use_pairs)
    assert res[0]["checked"] == blocks.shape[0]
    assert all(r["mismatches"] == 0 for r in res), f"global {global_scale}: " + _fmt(res)
    # the CPU oracle agrees with the reference header on the same blocks, non-finite ones included
    rows = blocks.shape[0] // 4
    want_p, want_s = orc.quantise_nvfp4(blocks.reshape(rows, 64), rows, 64, global_scale)
    rows_padded = (rows + 127) // 128 * 128
    cpu_scales = unswizzle(want_s, rows_padded, 4)[:rows].reshape(-1)
    assert np.array_equal(ws.cpu().numpy(), cpu_scales), "CPU oracle scale bytes differ from the reference header's"
    assert np.array_equal(wp.cpu().numpy(), want_p[: rows * 32]), "CPU oracle codes differ from the reference header's"


@pytest.mark.parametrize("use_pairs", [False, True], ids=["scalar", "packed-pairs"])
def test_block_quantiser_on_random_blocks_large(use_pairs):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((1 << 20, 16)).astype(np.float32)
    x[:, 3] *= 20.0
    res, *_ = ref_gpu.probe_blocks(torch.from_numpy(x).cuda(), 448.0 * 6.0 / 100.0, use_pairs)
    assert all(r["mismatches"] == 0 for r in res), _fmt(res)


def test_short_silu_forms_on_every_bf16_value():
    """The tuned SwiGLU / gated-norm kernels replace g / (1 + __expf(-g)) and __fdividef(g, 1 + __expf(-g)) by
    short sequences for |g| <= 44; both must equal the reference expressions for every bf16 g in that range."""
    res = ref_gpu.probe_silu_bf16()
    assert res[0]["checked"] == res[1]["checked"] and res[0]["checked"] > 30000
    assert all(r["mismatches"] == 0 for r in res), _fmt(res)


def test_short_silu_on_f32_accumulators():
    """The causal convolution applies silu to f32 accumulators: its short form (one Newton step on the approximate
    reciprocal, exact-remainder correction, the sign of g copied) must equal g / (1 + __expf(-g)) bit for bit on
    every f32 pattern with |g| <= 44, in its packed and in its scalar spelling. The gated norm's approximate-quotient
    form (third result) must equal __fdividef(g, 1 + __expf(-g)) on the same patterns: the tuned f32 gated kernel
    relies on it."""
    res = [{"checked": 0, "mismatches": 0, "first_bad": []} for _ in range(3)]
    for base in (0x00000000, 0x80000000):          # |g| <= 44 lies in the first 0x42300001 patterns of each sign
        part = ref_gpu.probe_silu_f32(base, 0x42300001)
        for r, q in zip(res, part):
            r["checked"] += q["checked"]
            r["mismatches"] += q["mismatches"]
            r["first_bad"] += q["first_bad"]
    assert res[0]["checked"] == res[1]["checked"] == res[2]["checked"] == 2 * 0x42300001
    assert res[0]["mismatches"] == 0 and res[1]["mismatches"] == 0 and res[2]["mismatches"] == 0, _fmt(res)


def test_short_division_by_six():
    res = ref_gpu.probe_div_six()
    assert res[0]["checked"] > 1_000_000_000
    assert res[0]["mismatches"] == 0, _fmt(res)
