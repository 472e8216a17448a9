"""Generates tests/golden/fused_path_b200.npz: seeded inputs of every entry point together with the
outputs of the REFERENCE's own kernels (oracle/_ref cubins, built from the reference tree for
sm_100a) run on a B200, and the CPU oracle's outputs for the kernels it reproduces exactly.

Run on a machine with a B200 and oracle/_ref present:

    python tests/golden/make_fixtures.py [output.npz]

The tests load the file and never need the reference tree: tests/test_golden.py checks the CPU oracle
against it (CPU) and the CUDA path against it (GPU). f32 results of the reference kernels are stored
rounded to bf16 (nearest even), which is what the bf16 entry points are compared with.
"""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, os.fspath(ROOT))
sys.path.insert(0, os.fspath(ROOT / "tests"))


def bf16(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def main(out_path):
    import torch

    from oracle import binding as orc
    from oracle import ref_gpu

    assert torch.cuda.is_available() and ref_gpu.available(), "needs a GPU and oracle/_ref"
    rng = np.random.default_rng(20261125)
    f = {}

    def dev_f32(bits):
        return torch.from_numpy(orc.bf16_to_f32(bits)).cuda()

    def host(t):
        return t.detach().cpu().numpy()

    # config 1 in miniature: embedding gather -> RMSNorm -> NVFP4, 24 rows of hidden 2048
    rows, hidden, vocab = 12, 2048, 16
    table = bf16(rng.standard_normal((vocab, hidden)) * 0.02)
    ids = rng.integers(0, vocab, rows).astype(np.int32)
    w = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    h = table[ids]
    gs_norm = float(np.float32(448.0 * 6.0 / 40.0))
    normed = ref_gpu.rms_norm(dev_f32(h), torch.from_numpy(w).cuda(), rows, hidden, 1e-6)
    p, s = ref_gpu.quantise_nvfp4(normed, rows, hidden, gs_norm)
    f.update(embed_table=table, embed_ids=ids, norm_w=w, norm_gs=np.float32(gs_norm),
             norm_bf16=bf16(host(normed)), norm_packed=host(p), norm_scales=host(s))
    cp, cs = orc.rms_norm_quantise_nvfp4(h, w, rows, hidden, 1e-6, gs_norm)
    assert np.array_equal(cp, host(p)) and np.array_equal(cs, host(s)), "CPU oracle and reference kernels disagree"

    # activations with outlier channels (config 1's second variant), plain quantiser
    x = rng.standard_normal((rows, hidden)).astype(np.float32)
    x[:, rng.choice(hidden, 8, replace=False)] *= 20.0
    xb = bf16(x)
    gs_q = float(np.float32(448.0 * 6.0) / np.abs(orc.bf16_to_f32(xb)).max())
    p, s = ref_gpu.quantise_nvfp4(dev_f32(xb), rows, hidden, gs_q)
    f.update(quant_x=xb, quant_gs=np.float32(gs_q), quant_packed=host(p), quant_scales=host(s))

    # SwiGLU + NVFP4 (approximate exp on the GPU: only the reference kernel is the authority)
    rows_s, inter = 3, 6144
    gate, up = bf16(rng.standard_normal((rows_s, inter))), bf16(rng.standard_normal((rows_s, inter)))
    gs_s = 48.0
    p, s = ref_gpu.swiglu_quantise_nvfp4(dev_f32(gate), dev_f32(up), rows_s, inter, gs_s)
    act = ref_gpu.swiglu(dev_f32(gate), dev_f32(up), rows_s * inter)
    f.update(swiglu_gate=gate, swiglu_up=up, swiglu_gs=np.float32(gs_s), swiglu_packed=host(p), swiglu_scales=host(s),
             swiglu_bf16=bf16(host(act)))

    # gated RMSNorm + NVFP4, 5 tokens x 16 heads x 128
    tokens, vh, cols = 3, 16, 128
    xg, zg = bf16(rng.standard_normal((tokens * vh, cols))), bf16(rng.standard_normal((tokens * vh, cols)))
    wg = (1.0 + rng.standard_normal(cols) * 0.1).astype(np.float32)
    gs_g = 96.0
    p, s = ref_gpu.rms_norm_gated_quantise_nvfp4(dev_f32(xg), dev_f32(zg), torch.from_numpy(wg).cuda(), tokens * vh, cols,
                                                 vh, 1e-6, gs_g)
    gated = ref_gpu.rms_norm_gated(dev_f32(xg), dev_f32(zg), torch.from_numpy(wg).cuda(), tokens * vh, cols, 1e-6)
    f.update(gated_x=xg, gated_z=zg, gated_w=wg, gated_gs=np.float32(gs_g), gated_packed=host(p), gated_scales=host(s),
             gated_bf16=bf16(host(gated)))

    # partial RoPE with a scattered position map, 16 q heads and 2 kv heads x 128, rotary 64, theta 1e7
    rows_r, rot, table_rows = 6, 64, 48
    q, k = bf16(rng.standard_normal((rows_r, 16, 128))), bf16(rng.standard_normal((rows_r, 2, 128)))
    pos = rng.integers(0, table_rows, rows_r).astype(np.int32)
    cos, sin = ref_gpu.rope_tables(torch.arange(table_rows, dtype=torch.int32, device="cuda"), table_rows, rot, 1e7)
    dpos = torch.from_numpy(pos).cuda()
    rq = ref_gpu.rope(dev_f32(q), cos, sin, rows_r, 16, 128, rot, None, None, dpos)
    rk = ref_gpu.rope(dev_f32(k), cos, sin, rows_r, 2, 128, rot, None, None, dpos)
    f.update(rope_q=q, rope_k=k, rope_pos=pos, rope_cos=host(cos), rope_sin=host(sin), rope_q_bf16=bf16(host(rq)),
             rope_k_bf16=bf16(host(rk)))
    cq, _ = orc.rope(orc.bf16_to_f32(q), host(cos), host(sin), rows_r, 16, 128, rot, pos_map=pos)
    assert np.array_equal(cq.view(np.uint32), host(rq).view(np.uint32)), "CPU oracle and reference rope kernel disagree"

    torch.cuda.synchronize()
    np.savez_compressed(out_path, **f)
    print(f"wrote {out_path}: {os.path.getsize(out_path)} bytes, {len(f)} arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.fspath(Path(__file__).with_name("fused_path_b200.npz")))
