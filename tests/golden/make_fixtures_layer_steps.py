"""Generates tests/golden/layer_steps_b200.npz: seeded inputs of the entry points either side of the fused
quantisers (KV-cache write, sigmoid_mul, residual add) and of the FP8 quantisers, together with the outputs of
the REFERENCE's own kernels and kernel chains (oracle/_ref cubins built from the reference tree for sm_100a) run
on a B200.

Run on a machine with a B200 and oracle/_ref present:

    python tests/golden/make_fixtures_layer_steps.py [output.npz]

tests/test_golden.py checks the CPU oracle against the file (CPU) and the CUDA path against it (GPU); neither
needs the reference tree.
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
    rng = np.random.default_rng(20261126)
    f = {}

    def dev_f32(bits):
        return torch.from_numpy(orc.bf16_to_f32(bits)).cuda()

    def host(t):
        return t.detach().cpu().numpy()

    def u16(t):
        return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)

    def i32(a):
        return torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()

    # key-side RoPE + KV-cache write: 6 tokens, 2 kv heads x 128, rotary 64, scattered into a 9-row cache
    tokens, heads, hd, rot, table_rows, cache_rows = 6, 2, 128, 64, 40, 9
    k, v = bf16(rng.standard_normal((tokens, heads, hd))), bf16(rng.standard_normal((tokens, heads, hd)))
    pos = rng.integers(0, table_rows, tokens).astype(np.int32)
    cmap = rng.permutation(cache_rows)[:tokens].astype(np.int32)
    cos, sin = ref_gpu.rope_tables(torch.arange(table_rows, dtype=torch.int32, device="cuda"), table_rows, rot, 1e7)
    k_rot = ref_gpu.rope(dev_f32(k), cos, sin, tokens, heads, hd, rot, None, None, i32(pos))
    stride = heads * hd
    cache_k = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    cache_v = torch.full((cache_rows * stride,), -1.0, dtype=torch.bfloat16, device="cuda")
    ref_gpu.to_bf16_scatter(k_rot.reshape(-1), cache_k, tokens * stride, i32(cmap), stride)
    ref_gpu.to_bf16_scatter(dev_f32(v).reshape(-1), cache_v, tokens * stride, i32(cmap), stride)
    f.update(kv_k=k, kv_v=v, kv_pos=pos, kv_map=cmap, kv_cos=host(cos), kv_sin=host(sin), kv_cache_k=u16(cache_k),
             kv_cache_v=u16(cache_v))

    # sigmoid_mul (+ NVFP4): 3 rows x 2048
    rows, cols = 3, 2048
    x, g = bf16(rng.standard_normal((rows, cols))), bf16(rng.standard_normal((rows, cols)) * 3)
    act = ref_gpu.sigmoid_mul(dev_f32(x), dev_f32(g), rows * cols)
    p, s = ref_gpu.quantise_nvfp4(act, rows, cols, 64.0)
    f.update(sig_x=x, sig_gate=g, sig_bf16=bf16(host(act)), sig_packed=host(p), sig_scales=host(s))

    # residual add (+ RMSNorm + NVFP4 on the stored bf16 sum): 4 rows x 2048
    rows = 4
    a, b = bf16(rng.standard_normal((rows, cols))), bf16(rng.standard_normal((rows, cols)) * 0.5)
    w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
    total = ref_gpu.add(dev_f32(a), dev_f32(b), rows * cols).to(torch.bfloat16)
    normed = ref_gpu.rms_norm(total.float(), torch.from_numpy(w).cuda(), rows, cols, 1e-6)
    p, s = ref_gpu.quantise_nvfp4(normed, rows, cols, 64.0)
    f.update(add_a=a, add_b=b, add_w=w, add_sum=u16(total), add_packed=host(p), add_scales=host(s))

    # FP8: plain (3 x 2048, one outlier column), RMSNorm with bf16 twin (2 x 4096), SwiGLU (2 x 6144), gated norm (1 token x 32 x 128)
    x8 = rng.standard_normal((3, 2048)).astype(np.float32)
    x8[:, 77] *= 25.0
    x8 = bf16(x8)
    q, qs = ref_gpu.quantise_fp8(dev_f32(x8), 3, 2048)
    f.update(fp8_x=x8, fp8_codes=host(q), fp8_scales=u16(qs))
    xr = bf16(rng.standard_normal((2, 4096)))
    wr = (rng.standard_normal(4096) * 0.3).astype(np.float32)
    q, qs, bfo = ref_gpu.rms_norm_fp8_bf16(dev_f32(xr), torch.from_numpy(wr).cuda(), 2, 4096, 1e-6)
    f.update(fp8n_x=xr, fp8n_w=wr, fp8n_codes=host(q), fp8n_scales=u16(qs), fp8n_bf16=u16(bfo))
    gs, us = bf16(rng.standard_normal((2, 6144)) * 2), bf16(rng.standard_normal((2, 6144)))
    q, qs = ref_gpu.swiglu_quantise_fp8(dev_f32(gs), dev_f32(us), 2, 6144)
    f.update(fp8s_gate=gs, fp8s_up=us, fp8s_codes=host(q), fp8s_scales=u16(qs))
    xg, zg = bf16(rng.standard_normal((32, 128))), bf16(rng.standard_normal((32, 128)))
    wg = (1.0 + rng.standard_normal(128) * 0.1).astype(np.float32)
    q, qs = ref_gpu.rms_norm_gated_quantise_fp8(dev_f32(xg), dev_f32(zg), torch.from_numpy(wg).cuda(), 32, 128, 32, 1e-6)
    f.update(fp8g_x=xg, fp8g_z=zg, fp8g_w=wg, fp8g_codes=host(q), fp8g_scales=u16(qs))

    torch.cuda.synchronize()
    # the CPU oracle must agree where its arithmetic has no approximate intrinsic
    cq, cs = orc.quantise_fp8(x8, 3, 2048)
    assert np.array_equal(cq, f["fp8_codes"]) and np.array_equal(cs, f["fp8_scales"]), "CPU oracle and quantise_fp8_kernel disagree"
    _, csum = orc.add(a, b)
    assert np.array_equal(csum.reshape(-1), f["add_sum"].reshape(-1)), "CPU oracle and add_kernel disagree"
    np.savez_compressed(out_path, **f)
    print(f"wrote {out_path}: {os.path.getsize(out_path)} bytes, {len(f)} arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.fspath(Path(__file__).with_name("layer_steps_b200.npz")))
