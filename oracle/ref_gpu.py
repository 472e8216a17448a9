"""Launch the REFERENCE's own CUDA kernels (oracle/_ref/*.cubin) on torch tensors.

TEST INFRASTRUCTURE. The cubins are compiled by oracle/Makefile from the reference's unmodified
kernels/elementwise.cu, kernels/quantise.cu, kernels/head.cu and kernels/attention_mma.cu (for its
bf16 conversion kernels) for sm_100a; this module only loads them with the
CUDA driver API (cuda-python) and launches them with the grid/block shapes the reference's
launch layer uses (aiis-clef src/cuda/mod.rs, cited per function). The reference kernels take
f32 activations; bf16 test inputs are widened exactly before the call.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent / "_ref"
_modules: dict[str, object] = {}
_functions: dict[tuple[str, str], object] = {}


def available() -> bool:
    return all((_DIR / f"{n}.cubin").exists() for n in ("elementwise", "quantise", "ref_probe", "head", "to_bf16", "gdn_prep"))


def _cu():
    from cuda.bindings import driver as cu

    return cu


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


def function(module: str, name: str):
    key = (module, name)
    if key not in _functions:
        cu = _cu()
        torch.cuda.init()
        torch.zeros(1, device="cuda")   # makes torch's primary context current on this thread
        if module not in _modules:
            data = (_DIR / f"{module}.cubin").read_bytes()
            _modules[module] = _check(cu.cuModuleLoadData(data))
        _functions[key] = _check(cu.cuModuleGetFunction(_modules[module], name.encode()))
    return _functions[key]


def launch(module: str, name: str, grid, block, args, smem: int = 0):
    cu = _cu()
    vals, types = [], []
    for a in args:
        if a is None:
            vals.append(0)
            types.append(ctypes.c_void_p)
        elif isinstance(a, torch.Tensor):
            vals.append(a.data_ptr())
            types.append(ctypes.c_void_p)
        elif isinstance(a, tuple):
            vals.append(a[0])
            types.append(a[1])
        elif isinstance(a, bool):
            raise TypeError("pass ints, not bools")
        elif isinstance(a, int):
            vals.append(a)
            types.append(ctypes.c_int)
        elif isinstance(a, float):
            vals.append(a)
            types.append(ctypes.c_float)
        else:
            raise TypeError(type(a))
    gx, gy, gz = (list(grid) + [1, 1])[:3]
    bx, by, bz = (list(block) + [1, 1])[:3]
    stream = torch.cuda.current_stream().cuda_stream
    res = cu.cuLaunchKernel(function(module, name), gx, gy, gz, bx, by, bz, smem, stream,
                            (tuple(vals), tuple(types)), 0)
    if int(res[0]) != 0:
        raise RuntimeError(f"cuLaunchKernel({name}) -> {res[0]}")


def _row_blocks(rows: int, cols: int) -> int:
    # src/cuda/mod.rs:5435-5439
    tpr = min(256, max(32, -(-cols // 256) * 32))
    rpb = 256 // tpr
    return -(-rows // rpb)


def _round_up(v, n):
    return -(-v // n) * n


# ---- the steps either side of the fused quantisers -----------------------------------------------
def sigmoid_mul(x, gate, total):
    """src/cuda/mod.rs:2838-2856."""
    out = torch.empty(total, dtype=torch.float32, device=x.device)
    launch("elementwise", "sigmoid_mul_kernel", ((total + 1023) // 1024,), (256,), [out, x, gate, total])
    return out


def add(a, b, total):
    """src/cuda/mod.rs:1686-1704 (kernels/head.cu add_kernel)."""
    out = torch.empty(total, dtype=torch.float32, device=a.device)
    launch("head", "add_kernel", ((total + 1023) // 1024,), (256,), [out, a, b, total])
    return out


def to_bf16(x, out, n, off_tokens=None, off_stride=0):
    """src/cuda/mod.rs:3201-3227, the arm without a position map (kernels/attention_mma.cu to_bf16_kernel).
    x f32; out a bf16 tensor written in place. The reference sizes its grid from n / 8 (its n is always a
    multiple of 8); here the grid is sized from ceil(n / 8) so the kernel's scalar tail branch has a thread."""
    blocks = max(1, (((n + 7) // 8) + 255) // 256)
    launch("to_bf16", "to_bf16_kernel", (blocks,), (256,), [x, out, (n, ctypes.c_longlong), off_tokens, int(off_stride)])
    return out


def to_bf16_scatter(x, out, n, pos_map, stride):
    """src/cuda/mod.rs:3201-3227, the arm with KvCache::pos_map (to_bf16_scatter_kernel)."""
    blocks = max(1, ((n // 8) + 255) // 256)
    launch("to_bf16", "to_bf16_scatter_kernel", (blocks,), (256,), [x, out, (n, ctypes.c_longlong), pos_map, int(stride)])
    return out


# ---- elementwise kernels in front of the GDN scan ------------------------------------------------
def causal_conv_silu(x, w, rows, channels, k, seq_start=None, history=None, slot_map=None):
    """src/cuda/mod.rs:2784-2812."""
    out = torch.empty(rows * channels, dtype=torch.float32, device=x.device)
    launch("elementwise", "causal_conv_silu_kernel", ((channels + 127) // 128, min(rows, 65535), -(-rows // 65535)), (128,),
           [x, w, out, rows, channels, k, seq_start, history, slot_map])
    return out.view(rows, channels)


def conv_hist_save(src, hist, saves, n_saves, rows, k, channels):
    """src/cuda/mod.rs:2814-2836 (hist is written in place)."""
    launch("elementwise", "conv_hist_save_kernel", (n_saves,), (128,), [src, hist, saves, n_saves, rows, k, channels])
    return hist


def gdn_gates(a, b, a_log, dt_bias, tokens, heads):
    """src/cuda/mod.rs:2858-2882."""
    decay = torch.empty(tokens * heads, dtype=torch.float32, device=a.device)
    beta = torch.empty(tokens * heads, dtype=torch.float32, device=a.device)
    launch("elementwise", "gdn_gates_kernel", ((tokens * heads + 255) // 256,), (256,), [a, b, a_log, dt_bias, decay, beta, tokens, heads])
    return decay.view(tokens, heads), beta.view(tokens, heads)


def gdn_prep(mixed, seq_len, kh, kd, heads, conv_dim):
    """src/cuda/mod.rs:3606-3647: gdn_prep_kernel of kernels/gdn_chunk.cu, one block per token, zeroed operand buffers."""
    nchunks = (seq_len + 63) // 64
    nbytes = heads * nchunks * 2 * 64 * 128
    dev = mixed.device
    out = {"v": torch.empty(seq_len * heads * kd, dtype=torch.float32, device=dev),
           "kn": torch.zeros(seq_len * heads * kd, dtype=torch.float32, device=dev)}
    for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
        out[name] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    import numpy as np

    q_scale = float(np.float32(1.0) / np.sqrt(np.float32(kd)))
    launch("gdn_prep", "gdn_prep_kernel", (seq_len,), (256,),
           [mixed, out["v"], out["q_hi"], out["q_lo"], out["k_hi"], out["k_lo"], out["kn"], seq_len, heads, kh, kd, nchunks,
            conv_dim, q_scale])
    return out


def split_q_gate(qg, tokens, heads, head_dim):
    """src/cuda/mod.rs:2884-2906."""
    total = tokens * heads * head_dim
    q = torch.empty(total, dtype=torch.float32, device=qg.device)
    gate = torch.empty(total, dtype=torch.float32, device=qg.device)
    launch("elementwise", "split_q_gate_kernel", ((total + 255) // 256,), (256,), [qg, q, gate, tokens, heads, head_dim])
    return q.view(tokens, heads, head_dim), gate.view(tokens, heads, head_dim)


def split_qkv(mixed, tokens, kh, kd, vh, vd):
    """src/cuda/mod.rs:2930-2958."""
    total = tokens * (2 * kh * kd + vh * vd)
    q = torch.empty(tokens * kh * kd, dtype=torch.float32, device=mixed.device)
    k = torch.empty(tokens * kh * kd, dtype=torch.float32, device=mixed.device)
    v = torch.empty(tokens * vh * vd, dtype=torch.float32, device=mixed.device)
    launch("elementwise", "split_qkv_kernel", ((total + 255) // 256,), (256,), [mixed, q, k, v, tokens, kh, kd, vh, vd])
    return q.view(tokens, kh * kd), k.view(tokens, kh * kd), v.view(tokens, vh * vd)


def repeat_interleave(src, tokens, kh, ratio, dim):
    """src/cuda/mod.rs:2959-2982."""
    total = tokens * kh * ratio * dim
    out = torch.empty(total, dtype=torch.float32, device=src.device)
    launch("elementwise", "repeat_interleave_kernel", ((total + 255) // 256,), (256,), [src, out, tokens, kh, ratio, dim])
    return out.view(tokens, kh * ratio, dim)


# ---- FP8 quantisers (quantise.cu) ----------------------------------------------------------------
def quantise_fp8(x, rows, cols):
    """src/cuda/mod.rs:2246-2266. Meaningful for cols > 1792 only (one row per CTA): for narrower rows the
    reference kernel reads row blockIdx.x for every row of the block."""
    assert cols > 1792
    out = torch.empty(rows * cols, dtype=torch.uint8, device=x.device)
    scales = torch.empty(rows, dtype=torch.int16, device=x.device)
    launch("quantise", "quantise_fp8_kernel", (_row_blocks(rows, cols),), (256,), [x, out, scales, rows, cols])
    return out.view(rows, cols), scales


def swiglu_quantise_fp8(gate, up, rows, cols):
    """src/cuda/mod.rs:2402-2427."""
    assert cols <= 768 * 16
    out = torch.empty(rows * cols, dtype=torch.uint8, device=gate.device)
    scales = torch.empty(rows, dtype=torch.int16, device=gate.device)
    launch("quantise", "swiglu_quantise_fp8_kernel", (rows,), (768,), [gate, up, out, scales, rows, cols])
    return out.view(rows, cols), scales


def rms_norm_fp8_bf16(x, weight, rows, cols, eps):
    """src/cuda/mod.rs:2330-2358 (cols 4096 only)."""
    assert cols == 4096
    q = torch.empty(rows * cols, dtype=torch.uint8, device=x.device)
    qs = torch.empty(rows, dtype=torch.int16, device=x.device)
    bf = torch.empty(rows * cols, dtype=torch.bfloat16, device=x.device)
    launch("quantise", "rms_norm_fp8_bf16_kernel", (rows,), (256,), [x, weight, q, qs, bf, rows, cols, float(eps)])
    return q.view(rows, cols), qs, bf.view(rows, cols)


def rms_norm_gated_quantise_fp8(x, gate, weight, rows, cols, vh, eps):
    """src/cuda/mod.rs:2304-2328 (cols 128, vh <= 32)."""
    assert cols == 128 and vh <= 32
    tokens = rows // vh
    out = torch.zeros(rows * cols, dtype=torch.uint8, device=x.device)
    scales = torch.empty(tokens, dtype=torch.int16, device=x.device)
    # The reference launches 1,024 threads: warp w of block t takes head row t * vh + w, so with vh < 32 the
    # surplus warps would also quantise rows of token t + 1 with token t's scale, racing with block t + 1.
    # One warp per head row is launched here, which is the reference launch itself at vh = 32.
    launch("quantise", "rms_norm_gated_quantise_fp8_kernel", (tokens,), (32 * vh,),
           [x, gate, weight, out, scales, rows, cols, float(eps), vh, rows])
    return out.view(rows, cols), scales


# ---- elementwise.cu ------------------------------------------------------------------------------
def rms_norm(x, weight, rows, cols, eps):
    """src/cuda/mod.rs:2718-2739."""
    out = torch.empty(rows * cols, dtype=torch.float32, device=x.device)
    launch("elementwise", "rms_norm_kernel", (_row_blocks(rows, cols),), (256,), [x, weight, out, rows, cols, float(eps)])
    return out.view(rows, cols)


def rms_norm_gated(x, gate, weight, rows, cols, eps):
    """src/cuda/mod.rs:2741-2763."""
    out = torch.empty(rows * cols, dtype=torch.float32, device=x.device)
    launch("elementwise", "rms_norm_gated_kernel", (_row_blocks(rows, cols),), (256,),
           [x, gate, weight, out, rows, cols, float(eps)])
    return out.view(rows, cols)


def swiglu(gate, up, total):
    """src/cuda/mod.rs:2765-2782."""
    out = torch.empty(total, dtype=torch.float32, device=gate.device)
    launch("elementwise", "swiglu_kernel", ((total + 1023) // 1024,), (256,), [gate, up, out, total])
    return out


def embed_gather(table, ids, tokens, hidden):
    """src/cuda/mod.rs:2908-2928."""
    out = torch.empty(tokens * hidden, dtype=torch.float32, device=table.device)
    launch("elementwise", "embed_gather_kernel", ((tokens * hidden + 255) // 256,), (256,),
           [table, ids, out, tokens, hidden])
    return out.view(tokens, hidden)


def rope_tables(positions, rows, rotary_dim, theta):
    """src/cuda/mod.rs:2983-3005."""
    cos = torch.empty(rows * rotary_dim, dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    launch("elementwise", "rope_tables_kernel", ((rows * rotary_dim + 255) // 256,), (256,),
           [positions, cos, sin, rows, rotary_dim, float(theta)])
    return cos.view(rows, rotary_dim), sin.view(rows, rotary_dim)


def rope(x, cos, sin, rows, heads, head_dim, rotary_dim, seq_start=None, pos_base=None, pos_map=None):
    """src/cuda/mod.rs:3045-3074."""
    out = torch.empty(rows * heads * head_dim, dtype=torch.float32, device=x.device)
    total = rows * heads * (head_dim // 2)
    launch("elementwise", "rope_kernel", ((total + 255) // 256,), (256,),
           [out, x, cos, sin, rows, heads, head_dim, rotary_dim, seq_start, pos_base, pos_map])
    return out.view(rows, heads, head_dim)


def qk_norm_rope(x, weight, cos, sin, rows, heads, head_dim, rotary_dim, eps, seq_start=None, pos_base=None,
                 pos_map=None, with_gate=False):
    """src/cuda/mod.rs:3008-3043 (head_dim 256 only)."""
    assert head_dim == 256
    out = torch.empty(rows * head_dim, dtype=torch.float32, device=x.device)
    gate = torch.empty(rows * head_dim, dtype=torch.float32, device=x.device) if with_gate else None
    launch("elementwise", "qk_norm_rope_kernel", ((rows + 7) // 8,), (256,),
           [x, weight, cos, sin, out, gate, rows, heads, head_dim, rotary_dim, float(eps), seq_start, pos_base,
            pos_map])
    return out.view(rows, head_dim), (gate.view(rows, head_dim) if with_gate else None)


# ---- quantise.cu -----------------------------------------------------------------------------------
def _zeroed_outputs(rows_padded, cols, device, slack_rows=0):
    # The reference allocates both outputs zeroed (src/cuda/mod.rs:2186-2187). `slack_rows` covers
    # the rows its folded (grid.y, grid.z) launch touches beyond rows_padded above 65535 rows.
    packed = torch.zeros((rows_padded + slack_rows) * (cols // 2), dtype=torch.uint8, device=device)
    scales = torch.zeros((rows_padded + slack_rows) * (cols // 16), dtype=torch.uint8, device=device)
    return packed, scales


def quantise_nvfp4(x, rows, cols, global_scale, blk_mn=128, chunk=512):
    """src/cuda/mod.rs:2169-2207."""
    rows_padded = _round_up(rows, blk_mn)
    gy, gz = min(rows_padded, 65535), -(-rows_padded // 65535)
    slack = _round_up(gy * gz, blk_mn) - rows_padded
    packed, scales = _zeroed_outputs(rows_padded, cols, x.device, slack)
    blocks = cols // 16
    launch("quantise", "quantise_nvfp4_kernel", ((blocks + 63) // 64, gy, gz), (64,),
           [x, packed, scales, rows, cols, float(global_scale), blk_mn, chunk])
    return packed[: rows_padded * (cols // 2)], scales[: rows_padded * (cols // 16)]


def rms_norm_quantise_nvfp4(x, weight, rows, cols, eps, global_scale, blk_mn=128, chunk=512):
    """src/cuda/mod.rs:2133-2167 (cols 4096 only)."""
    assert cols == 4096
    rows_padded = _round_up(rows, blk_mn)
    packed, scales = _zeroed_outputs(rows_padded, cols, x.device)
    launch("quantise", "rms_norm_quantise_nvfp4_kernel", (rows_padded,), (256,),
           [x, weight, packed, scales, rows, cols, float(eps), float(global_scale), blk_mn, chunk])
    return packed, scales


def rms_norm_gated_quantise_nvfp4(x, gate, weight, rows, cols, vh, eps, global_scale, blk_mn=128, chunk=512):
    """src/cuda/mod.rs:2269-2302 (cols 128 only); `rows` = live head rows."""
    assert cols == 128
    tokens = rows // vh
    tokens_padded = _round_up(tokens, blk_mn)
    rows_padded = tokens_padded * vh
    packed = torch.zeros(rows_padded * (cols // 2), dtype=torch.uint8, device=x.device)
    scales = torch.zeros(tokens_padded * (vh * cols // 16), dtype=torch.uint8, device=x.device)
    launch("quantise", "rms_norm_gated_quantise_nvfp4_kernel", ((rows_padded + 7) // 8,), (256,),
           [x, gate, weight, packed, scales, rows_padded, cols, float(eps), float(global_scale), blk_mn, chunk, vh,
            rows])
    return packed, scales


def swiglu_quantise_nvfp4(gate, up, rows, cols, global_scale, blk_mn=128, chunk=512):
    """src/cuda/mod.rs:2359-2400."""
    assert cols <= 768 * 16
    rows_padded = _round_up(rows, blk_mn)
    gy, gz = min(rows_padded, 65535), -(-rows_padded // 65535)
    slack = _round_up(gy * gz, blk_mn) - rows_padded
    packed, scales = _zeroed_outputs(rows_padded, cols, gate.device, slack)
    per_row = cols // 16
    threads = max(32, min(768, per_row))
    launch("quantise", "swiglu_quantise_nvfp4_kernel", (-(-per_row // threads), gy, gz), (threads,),
           [gate, up, packed, scales, rows, cols, float(global_scale), blk_mn, chunk])
    return packed[: rows_padded * (cols // 2)], scales[: rows_padded * (cols // 16)]


# ---- ref_probe.cubin -----------------------------------------------------------------------------------
def _result_buffer(n):
    # struct ProbeResult { u64 checked; u64 mismatches; u32 first_bad[16]; } = 80 bytes
    return torch.zeros(n * 80, dtype=torch.uint8, device="cuda")


def _read_results(buf, n):
    import numpy as np

    raw = buf.cpu().numpy()
    out = []
    for i in range(n):
        rec = raw[i * 80:(i + 1) * 80]
        checked, mism = np.frombuffer(rec[:16].tobytes(), np.uint64)
        bad = np.frombuffer(rec[16:].tobytes(), np.uint32)[: min(int(mism), 16)]
        out.append({"checked": int(checked), "mismatches": int(mism), "first_bad": [int(b) for b in bad]})
    return out


def probe_e2m1(base: int, count: int):
    buf = _result_buffer(3)
    launch("ref_probe", "probe_e2m1", (148 * 8,), (256,),
           [(base, ctypes.c_ulonglong), (count, ctypes.c_ulonglong), buf])
    torch.cuda.synchronize()
    return _read_results(buf, 3)


def probe_e4m3(base: int, count: int):
    """[scale encoder e4m3_encode_finite (+inf literal), element encoder e4m3_encode_any, short element encoder
    e4m3_mag_fast on 0 <= v < 464, hardware-converter form e4m3x4_hw with its flagged bytes on the same patterns]
    against to_e4m3."""
    buf = _result_buffer(4)
    launch("ref_probe", "probe_e4m3", (148 * 8,), (256,),
           [(base, ctypes.c_ulonglong), (count, ctypes.c_ulonglong), buf])
    torch.cuda.synchronize()
    return _read_results(buf, 4)


def probe_e4m3_decode(global_scale: float):
    buf = _result_buffer(2)
    launch("ref_probe", "probe_e4m3_decode", (1,), (256,), [float(global_scale), buf])
    torch.cuda.synchronize()
    return _read_results(buf, 2)


def probe_silu_bf16():
    buf = _result_buffer(2)
    launch("ref_probe", "probe_silu_bf16", (256,), (256,), [buf])
    torch.cuda.synchronize()
    return _read_results(buf, 2)


def probe_silu_f32(base: int, count: int):
    """[packed, scalar] short silu of f32 accumulators against the literal expression, and [2] the approximate-quotient
    form of the gated norm against __fdividef(g, 1 + __expf(-g))."""
    buf = _result_buffer(3)
    launch("ref_probe", "probe_silu_f32", (148 * 8,), (256,), [(base, ctypes.c_ulonglong), (count, ctypes.c_ulonglong), buf])
    torch.cuda.synchronize()
    return _read_results(buf, 3)


def probe_sigmoid_mul_bf16():
    buf = _result_buffer(2)
    launch("ref_probe", "probe_sigmoid_mul_bf16", (256,), (256,), [buf])
    torch.cuda.synchronize()
    return _read_results(buf, 2)


def probe_div_six():
    buf = _result_buffer(1)
    launch("ref_probe", "probe_div_six", (148 * 8,), (256,), [buf])
    torch.cuda.synchronize()
    return _read_results(buf, 1)


def probe_blocks(values, global_scale: float, use_pairs: bool = False):
    """values: CUDA f32 tensor of n_blocks*16. Returns (results, want_scale, want_packed, got_scale, got_packed).
    use_pairs selects the tuned kernels' packed-pair quantiser (with its literal fallback)."""
    n = values.numel() // 16
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    wp = torch.empty(n * 8, dtype=torch.uint8, device="cuda")
    gs = torch.empty_like(ws)
    gp = torch.empty_like(wp)
    buf = _result_buffer(2)
    launch("ref_probe", "probe_blocks", (min(148 * 8, (n + 255) // 256),), (256,),
           [values, (n, ctypes.c_ulonglong), float(global_scale), ws, wp, gs, gp, buf, int(use_pairs)])
    torch.cuda.synchronize()
    return _read_results(buf, 2), ws, wp, gs, gp


def probe_epilogue(accg, accu, a_rows: int, rows_padded: int, cols: int, gscale_g: float, gscale_u: float, out_global: float,
                   mode: int, blk_mn: int = 128, interleaved: bool = False):
    """The GEMM-epilogue quantiser of aiis_clef_b200/csrc/nvfp4_epilogue.cuh (mode 0: a thread holds a block; 1: the
    mma.sync fragment layout) or the reference header's arithmetic in that fragment layout (mode 2) on f32
    "accumulators" [rows_padded, cols]; returns (packed, scales) in clef_swiglu_quantise_nvfp4's layout."""
    assert rows_padded % blk_mn == 0 and rows_padded % 16 == 0 and cols % 64 == 0
    packed = torch.zeros(rows_padded * (cols // 2), dtype=torch.uint8, device=accg.device)
    scales = torch.zeros(rows_padded * (cols // 16), dtype=torch.uint8, device=accg.device)
    chunk = 4 * blk_mn
    launch("ref_probe", "probe_epilogue", (148 * 4,), (256,),
           [accg, accu, a_rows, rows_padded, cols, float(gscale_g), float(gscale_u), float(out_global), blk_mn,
            -chunk if interleaved else chunk, packed, scales, mode])
    return packed, scales
