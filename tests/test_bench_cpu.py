"""CPU-side checks of bench.py: the algorithmic byte counts it divides by, the recorded DRAM traffic of the dominant
kernel, and the reference arm's line (the CPU restatement timed on the host cores, no GPU involved)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, os.fspath(ROOT))

import bench  # noqa: E402


def test_algorithmic_bytes_per_row():
    b = bench.BYTES_PER_ROW
    assert b["rms_norm_quantise_nvfp4"] == 5248 and b["swiglu_quantise_nvfp4"] == 28032 and b["rope_qk"] == 9476
    assert b["embed_gather"] == 8196 and b["rms_norm_gated_quantise_nvfp4"] == 9344 and b["embed_rms_norm_quantise_nvfp4"] == 9348
    assert sum(b[k] for k in bench.FULL_KERNELS) == 60296
    assert set(bench.STEP_KERNELS) == {"rms_norm_quantise_nvfp4", "swiglu_quantise_nvfp4", "rope_qk"}
    # f32 activations: 4-byte activations, the same quantised outputs
    f = bench.F32_BYTES_PER_ROW
    assert f["rms_norm_quantise_nvfp4"] == 4 * 2048 + 1024 + 128 and f["swiglu_quantise_nvfp4"] == 8 * 6144 + 3072 + 384
    assert f["rope_qk"] == 2 * 18 * 128 * 4 + 4 + 256 and set(f) <= set(b)
    for name in f:   # an f32 entry never moves fewer bytes than its bf16 form, and at most twice as many
        assert b[name] <= f[name] <= 2 * b[name]


def test_recorded_traffic_of_the_dominant_kernel():
    total, note = bench.dominant_traffic()
    assert total is not None, note
    algorithmic = bench.BYTES_PER_ROW[bench.DOMINANT] * bench.ROWS
    assert 0.85 * algorithmic < total < 1.1 * algorithmic     # reads equal the inputs; part of the output stays in L2
    assert "capture" in note


def test_reference_arm_line():
    out = subprocess.run([sys.executable, os.fspath(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": bench.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("configs[1]")


def test_shard_checksums_address_the_same_bytes_as_a_shard_of_its_own():
    """bench.py compares every rank's shard with the same row range of a single-GPU run through checksums of slices:
    the slice arithmetic (packed rows, 128-row scale atoms, RoPE and gather rows) must pick, out of the whole pass's
    buffers, exactly the bytes a shard holds in buffers of its own."""
    import types

    import torch

    import aiis_clef_b200 as clef

    h = types.SimpleNamespace(torch=torch)
    rows, world = 1000, 3
    padded = (rows + 127) // 128 * 128
    gen = torch.Generator().manual_seed(3)

    def rnd(n):
        return torch.randint(0, 256, (n,), generator=gen, dtype=torch.uint8)

    H, I = bench.HIDDEN, bench.INTER
    whole = {"pkh": rnd(padded * H // 2), "sch": rnd(padded * H // 16), "pki": rnd(padded * I // 2), "sci": rnd(padded * I // 16),
             "pkg": rnd(padded * H // 2), "scg": rnd(padded * H // 16),
             "qo": torch.randn(rows, bench.Q_HEADS, bench.HEAD_DIM, generator=gen).to(torch.bfloat16),
             "ko": torch.randn(rows, bench.KV_HEADS, bench.HEAD_DIM, generator=gen).to(torch.bfloat16),
             "h": torch.randn(rows, H, generator=gen).to(torch.bfloat16)}
    covered = 0
    for r in range(world):
        first, n = clef.shard_rows(rows, 128, world, r)
        rp = (n + 127) // 128 * 128
        own = {}
        for pk, sc, cols in (("pkh", "sch", H), ("pki", "sci", I), ("pkg", "scg", H)):
            own[pk] = whole[pk][first * cols // 2:(first + rp) * cols // 2].clone()
            own[sc] = whole[sc][first * cols // 16:(first + rp) * cols // 16].clone()
        for name in ("qo", "ko", "h"):
            own[name] = whole[name][first:first + n].clone()
        assert bench.shard_checksums(h, own, first, n, first) == bench.shard_checksums(h, whole, first, n, 0)
        covered += n
    assert covered == rows
    # a single flipped byte changes a checksum
    before = bench.shard_checksums(h, whole, 0, rows, 0)
    whole["sci"][12345] ^= 1
    assert bench.shard_checksums(h, whole, 0, rows, 0) != before
