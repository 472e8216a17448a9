"""numpy/ctypes binding of the CPU oracle (oracle/libclef_oracle.so, built from clef_oracle.cpp).

TEST INFRASTRUCTURE: imported only by tests/, by __graft_entry__.smoke() and by the CPU-baseline
legs of bench.py. Activations are passed as bf16 bit patterns (uint16 arrays) or float32 arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
LIB_PATH = _DIR / "libclef_oracle.so"

# FMA contraction of the reference build, fixed by comparison with the reference cubin on the GPU
# (see clef_oracle.cpp: fma_mode / rope_fma).
SUMSQ_FMA = 1
ROPE_FMA = 1 + 3 * 2   # lo_mode + 3 * hi_mode (rope_head in clef_oracle.cpp): fma(lo,c,-(hi*s)) and fma(lo,s,hi*c)

_lib = None
_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float
_sz = ctypes.c_size_t


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            subprocess.run(["make", "-C", os.fspath(_DIR), "oracle"], check=True, capture_output=True)
        lib = ctypes.CDLL(os.fspath(LIB_PATH))
        lib.oracle_to_e2m1.restype = ctypes.c_uint8
        lib.oracle_to_e2m1.argtypes = [_f]
        lib.oracle_to_e4m3.restype = ctypes.c_uint8
        lib.oracle_to_e4m3.argtypes = [_f]
        lib.oracle_from_e4m3.restype = _f
        lib.oracle_from_e4m3.argtypes = [ctypes.c_uint8]
        lib.oracle_e4m3_one.restype = _f
        lib.oracle_e4m3_one.argtypes = [ctypes.c_uint8]
        lib.oracle_max_threads.restype = _i
        lib.oracle_blk_mn_for_tile_m.restype = _i
        lib.oracle_blk_mn_for_tile_m.argtypes = [_i]
        lib.oracle_swizzled_index_of.restype = _sz
        lib.oracle_swizzled_index_of.argtypes = [_sz, _sz, _sz, _i, _i]
        lib.oracle_swizzled_len_tiled.restype = _sz
        lib.oracle_swizzled_len_tiled.argtypes = [_sz, _sz, _i]
        _lib = lib
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _c(a, dtype=None):
    a = np.ascontiguousarray(a) if dtype is None else np.ascontiguousarray(a, dtype=dtype)
    return a


def max_threads() -> int:
    return load().oracle_max_threads()


# ---- dtype helpers ---------------------------------------------------------------------------------
def bf16_bits(t) -> np.ndarray:
    """uint16 bit patterns of a torch bfloat16 CPU tensor."""
    import torch

    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_torch_bf16(bits: np.ndarray):
    import torch

    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    load().oracle_f32_to_bf16(_p(x), _sz(x.size), _p(out))
    return out


def _dtype_code(a: np.ndarray) -> int:
    if a.dtype == np.uint16:
        return 0
    if a.dtype == np.float32:
        return 1
    raise TypeError(f"activations must be uint16 (bf16 bits) or float32, got {a.dtype}")


# ---- scalar codecs ------------------------------------------------------------------------------------
def to_e2m1(v: float) -> int:
    return load().oracle_to_e2m1(v)


def to_e4m3(v: float) -> int:
    return load().oracle_to_e4m3(v)


def from_e4m3(b: int) -> float:
    return load().oracle_from_e4m3(b)


def e4m3_one(b: int) -> float:
    return load().oracle_e4m3_one(b)


def to_e2m1_many(v: np.ndarray) -> np.ndarray:
    v = _c(v, np.float32)
    out = np.empty(v.shape, np.uint8)
    load().oracle_to_e2m1_many(_p(v), _sz(v.size), _p(out))
    return out


def to_e4m3_many(v: np.ndarray) -> np.ndarray:
    v = _c(v, np.float32)
    out = np.empty(v.shape, np.uint8)
    load().oracle_to_e4m3_many(_p(v), _sz(v.size), _p(out))
    return out


E4M3_TABLE = None


def e4m3_table() -> np.ndarray:
    """from_e4m3 of all 256 bytes (unsigned decode: bit 7 ignored)."""
    global E4M3_TABLE
    if E4M3_TABLE is None:
        E4M3_TABLE = np.array([from_e4m3(b) for b in range(256)], np.float32)
    return E4M3_TABLE


# ---- layouts ------------------------------------------------------------------------------------------
def blk_mn_for_tile_m(tile_m: int) -> int:
    return load().oracle_blk_mn_for_tile_m(tile_m)


def swizzled_index_of(row, block, blocks, tile_m, conflict_free) -> int:
    return load().oracle_swizzled_index_of(row, block, blocks, tile_m, int(conflict_free))


def swizzled_len_tiled(rows, cols, tile_m) -> int:
    return load().oracle_swizzled_len_tiled(rows, cols, tile_m)


def swizzle_tiled(scales: np.ndarray, rows, cols, tile_m=128, conflict_free=False) -> np.ndarray:
    scales = _c(scales, np.uint8)
    out = np.empty(swizzled_len_tiled(rows, cols, tile_m), np.uint8)
    load().oracle_swizzle_tiled(_p(scales), _sz(rows), _sz(cols), tile_m, int(conflict_free), _p(out))
    return out


def unswizzle_tiled(sw: np.ndarray, rows, cols, tile_m=128, conflict_free=False) -> np.ndarray:
    sw = _c(sw, np.uint8)
    assert sw.size == swizzled_len_tiled(rows, cols, tile_m)
    out = np.empty(rows * cols, np.uint8)
    load().oracle_unswizzle_tiled(_p(sw), _sz(rows), _sz(cols), tile_m, int(conflict_free), _p(out))
    return out


def dequantise(packed: np.ndarray, scales_f32: np.ndarray, global_scale: float, cols: int, rows: int) -> np.ndarray:
    packed = _c(packed, np.uint8)
    scales_f32 = _c(scales_f32, np.float32)
    out = np.empty(rows * cols, np.float32)
    load().oracle_dequantise(_p(packed), _p(scales_f32), _f(global_scale), _sz(cols), _sz(rows), _p(out))
    return out


# ---- model routines (tolerance references) ---------------------------------------------------------------
def model_rms_norm(x, w, eps):
    x, w = _c(x, np.float32), _c(w, np.float32)
    out = np.empty_like(x)
    load().oracle_model_rms_norm(_p(x), _p(w), _sz(x.size), _f(eps), _p(out))
    return out


def model_rms_norm_gated(x, g, w, eps):
    x, g, w = _c(x, np.float32), _c(g, np.float32), _c(w, np.float32)
    out = np.empty_like(x)
    load().oracle_model_rms_norm_gated(_p(x), _p(g), _p(w), _sz(x.size), _f(eps), _p(out))
    return out


def rope_tables(positions, rotary_dim, theta):
    positions = _c(positions, np.int32)
    cos = np.empty((positions.size, rotary_dim), np.float32)
    sin = np.empty_like(cos)
    load().oracle_rope_tables(_p(positions), positions.size, rotary_dim, _f(theta), _p(cos), _p(sin))
    return cos, sin


def model_apply_rope(vec, cos_row, sin_row):
    vec = _c(vec, np.float32).copy()
    cos_row, sin_row = _c(cos_row, np.float32), _c(sin_row, np.float32)
    load().oracle_model_apply_rope(_p(vec), _p(cos_row), _p(sin_row), cos_row.size)
    return vec


# ---- kernel restatements -------------------------------------------------------------------------------------
def embed_gather(table, ids, tokens, hidden, nthreads=0):
    table, ids = _c(table), _c(ids, np.int32)
    out = np.empty((tokens, hidden), table.dtype)
    load().oracle_embed_gather(_p(table), _p(ids), _p(out), tokens, hidden, _dtype_code(table), nthreads)
    return out


def rms_norm(x, w, rows, cols, eps, fma_mode=None, nthreads=0):
    """Returns (f32 result, result narrowed to the activation dtype)."""
    x = _c(x)
    w = None if w is None else _c(w, np.float32)
    f32 = np.empty((rows, cols), np.float32)
    out = np.empty((rows, cols), x.dtype)
    load().oracle_rms_norm(_p(x), _p(w), rows, cols, _f(eps), _dtype_code(x),
                           SUMSQ_FMA if fma_mode is None else fma_mode, _p(f32), _p(out), nthreads)
    return f32, out


def rms_norm_gated(x, g, w, rows, cols, eps, fma_mode=None, nthreads=0):
    x = _c(x)
    g = None if g is None else _c(g)
    w = None if w is None else _c(w, np.float32)
    f32 = np.empty((rows, cols), np.float32)
    out = np.empty((rows, cols), x.dtype)
    load().oracle_rms_norm_gated(_p(x), _p(g), _p(w), rows, cols, _f(eps), _dtype_code(x),
                                 SUMSQ_FMA if fma_mode is None else fma_mode, _p(f32), _p(out), nthreads)
    return f32, out


def swiglu(gate, up, nthreads=0):
    gate, up = _c(gate), _c(up)
    f32 = np.empty(gate.shape, np.float32)
    out = np.empty(gate.shape, gate.dtype)
    load().oracle_swiglu(_p(gate), _p(up), _sz(gate.size), _dtype_code(gate), _p(f32), _p(out), nthreads)
    return f32, out


def rope(x, cos, sin, rows, heads, head_dim, rotary_dim, seq_start=None, pos_base=None, pos_map=None,
         rope_fma=None, nthreads=0):
    x = _c(x)
    cos, sin = _c(cos, np.float32), _c(sin, np.float32)
    seq_start = None if seq_start is None else _c(seq_start, np.int32)
    pos_base = None if pos_base is None else _c(pos_base, np.int32)
    pos_map = None if pos_map is None else _c(pos_map, np.int32)
    f32 = np.empty((rows, heads, head_dim), np.float32)
    out = np.empty((rows, heads, head_dim), x.dtype)
    load().oracle_rope(_p(out), _p(f32), _p(x), _p(cos), _p(sin), rows, heads, head_dim, rotary_dim, _p(seq_start),
                       _p(pos_base), _p(pos_map), _dtype_code(x), ROPE_FMA if rope_fma is None else rope_fma, nthreads)
    return f32, out


def qk_norm_rope(x, w, cos, sin, rows, heads, head_dim, rotary_dim, eps, seq_start=None, pos_base=None, pos_map=None,
                 with_gate=False, fma_mode=None, rope_fma=None, nthreads=0):
    x = _c(x)
    w, cos, sin = _c(w, np.float32), _c(cos, np.float32), _c(sin, np.float32)
    seq_start = None if seq_start is None else _c(seq_start, np.int32)
    pos_base = None if pos_base is None else _c(pos_base, np.int32)
    pos_map = None if pos_map is None else _c(pos_map, np.int32)
    f32 = np.empty((rows, head_dim), np.float32)
    out = np.empty((rows, head_dim), x.dtype)
    gate = np.empty((rows, head_dim), x.dtype) if with_gate else None
    load().oracle_qk_norm_rope(_p(x), _p(w), _p(cos), _p(sin), _p(out), _p(f32), _p(gate), rows, heads, head_dim,
                               rotary_dim, _f(eps), _p(seq_start), _p(pos_base), _p(pos_map), _dtype_code(x),
                               SUMSQ_FMA if fma_mode is None else fma_mode,
                               ROPE_FMA if rope_fma is None else rope_fma, nthreads)
    return f32, out, gate


def _quant_out(rows, cols, blk_mn):
    rows_padded = (rows + blk_mn - 1) // blk_mn * blk_mn
    return rows_padded, np.empty(rows_padded * (cols // 2), np.uint8), np.empty(rows_padded * (cols // 16), np.uint8)


def quantise_nvfp4(x, rows, cols, global_scale, blk_mn=128, chunk=512, nthreads=0):
    x = _c(x)
    _, packed, scales = _quant_out(rows, cols, blk_mn)
    load().oracle_quantise_nvfp4(_p(x), _p(packed), _p(scales), rows, cols, _f(global_scale), blk_mn, chunk,
                                 _dtype_code(x), nthreads)
    return packed, scales


def rms_norm_quantise_nvfp4(x, w, rows, cols, eps, global_scale, blk_mn=128, chunk=512, fma_mode=None, nthreads=0):
    x, w = _c(x), _c(w, np.float32)
    _, packed, scales = _quant_out(rows, cols, blk_mn)
    load().oracle_rms_norm_quantise_nvfp4(_p(x), _p(w), _p(packed), _p(scales), rows, cols, _f(eps), _f(global_scale),
                                          blk_mn, chunk, _dtype_code(x), SUMSQ_FMA if fma_mode is None else fma_mode,
                                          nthreads)
    return packed, scales


def rms_norm_gated_quantise_nvfp4(x, g, w, rows_live, cols, vh, eps, global_scale, blk_mn=128, chunk=512,
                                  fma_mode=None, want_pre=False, nthreads=0):
    """rows_live = tokens * vh live head rows; outputs are sized for tokens rounded up to blk_mn."""
    x, g, w = _c(x), _c(g), _c(w, np.float32)
    tokens = rows_live // vh
    tokens_padded = (tokens + blk_mn - 1) // blk_mn * blk_mn
    rows = tokens_padded * vh
    packed = np.empty(rows * (cols // 2), np.uint8)
    scales = np.empty(tokens_padded * (vh * cols // 16), np.uint8)
    pre = np.empty((rows_live, cols), np.float32) if want_pre else None
    load().oracle_rms_norm_gated_quantise_nvfp4(_p(x), _p(g), _p(w), _p(packed), _p(scales), rows, cols, _f(eps),
                                                _f(global_scale), blk_mn, chunk, vh, rows_live, _dtype_code(x),
                                                SUMSQ_FMA if fma_mode is None else fma_mode, _p(pre), nthreads)
    return (packed, scales, pre) if want_pre else (packed, scales)


def swiglu_quantise_nvfp4(gate, up, rows, cols, global_scale, blk_mn=128, chunk=512, want_pre=False, nthreads=0):
    gate, up = _c(gate), _c(up)
    _, packed, scales = _quant_out(rows, cols, blk_mn)
    pre = np.empty((rows, cols), np.float32) if want_pre else None
    load().oracle_swiglu_quantise_nvfp4(_p(gate), _p(up), _p(packed), _p(scales), rows, cols, _f(global_scale),
                                        blk_mn, chunk, _dtype_code(gate), _p(pre), nthreads)
    return (packed, scales, pre) if want_pre else (packed, scales)


# ---- the steps either side of the fused quantisers -----------------------------------------------------

def to_bf16_rows(x, out_bits, pos_map=None, off_tokens=None, stride=0):
    """In place on `out_bits` (uint16 cache): kernels/attention_mma.cu:118-171."""
    x = _c(x)
    pos_map = None if pos_map is None else _c(pos_map, np.int32)
    off = None if off_tokens is None else _c(np.asarray([off_tokens]), np.int32)
    load().oracle_to_bf16_rows(_p(x), _p(out_bits), _sz(x.size), _p(pos_map), _p(off), int(stride), _dtype_code(x))
    return out_bits


def sigmoid_mul(x, gate, nthreads=0):
    x, gate = _c(x), _c(gate)
    f32 = np.empty(x.shape, np.float32)
    out = np.empty(x.shape, x.dtype)
    load().oracle_sigmoid_mul(_p(x), _p(gate), _sz(x.size), _dtype_code(x), _p(f32), _p(out), nthreads)
    return f32, out


def sigmoid_mul_quantise_nvfp4(x, gate, rows, cols, global_scale, blk_mn=128, chunk=512, want_pre=False, nthreads=0):
    x, gate = _c(x), _c(gate)
    _, packed, scales = _quant_out(rows, cols, blk_mn)
    pre = np.empty((rows, cols), np.float32) if want_pre else None
    load().oracle_sigmoid_mul_quantise_nvfp4(_p(x), _p(gate), _p(packed), _p(scales), rows, cols, _f(global_scale),
                                             blk_mn, chunk, _dtype_code(x), _p(pre), nthreads)
    return (packed, scales, pre) if want_pre else (packed, scales)


def add(a, b):
    a, b = _c(a), _c(b)
    f32 = np.empty(a.shape, np.float32)
    out = np.empty(a.shape, a.dtype)
    load().oracle_add(_p(a), _p(b), _sz(a.size), _dtype_code(a), _p(f32), _p(out))
    return f32, out


# ---- FP8 (E4M3) activation quantisers --------------------------------------------------------------------

def _fp8_rows(mode, a, b, w, rows, cols, eps, want_bf16, fma_mode, nthreads):
    a = _c(a)
    b = None if b is None else _c(b)
    w = None if w is None else _c(w, np.float32)
    out = np.empty((rows, cols), np.uint8)
    scales = np.empty(rows, np.uint16)
    bf = np.empty((rows, cols), np.uint16) if want_bf16 else None
    load().oracle_fp8_rows(mode, _p(a), _p(b), _p(w), _p(out), _p(scales), _p(bf), rows, cols, _f(eps), _dtype_code(a),
                           SUMSQ_FMA if fma_mode is None else fma_mode, nthreads)
    return (out, scales, bf) if want_bf16 else (out, scales)


def quantise_fp8(x, rows, cols, nthreads=0):
    return _fp8_rows(0, x, None, None, rows, cols, 0.0, False, None, nthreads)


def swiglu_quantise_fp8(gate, up, rows, cols, nthreads=0):
    return _fp8_rows(1, gate, up, None, rows, cols, 0.0, False, None, nthreads)


def rms_norm_fp8_bf16(x, w, rows, cols, eps, fma_mode=None, nthreads=0):
    return _fp8_rows(2, x, None, w, rows, cols, eps, True, fma_mode, nthreads)


def rms_norm_gated_quantise_fp8(x, g, w, rows, cols, vh, eps, rows_live=None, fma_mode=None, nthreads=0):
    x, g, w = _c(x), _c(g), _c(w, np.float32)
    out = np.zeros((rows, cols), np.uint8)
    scales = np.empty(rows // vh, np.uint16)
    load().oracle_rms_norm_gated_quantise_fp8(_p(x), _p(g), _p(w), _p(out), _p(scales), rows, cols, _f(eps), vh,
                                              rows if rows_live is None else rows_live, _dtype_code(x),
                                              SUMSQ_FMA if fma_mode is None else fma_mode, nthreads)
    return out, scales


# ---- elementwise kernels in front of the GDN scan ------------------------------------------------------------

def causal_conv_silu(x, w, rows, channels, k, seq_start=None, history=None, slot_map=None, nthreads=0):
    """(f32 result, result in x's dtype, f32 pre-activation sums)."""
    x, w = _c(x), _c(w, np.float32)
    seq_start = None if seq_start is None else _c(seq_start, np.int32)
    slot_map = None if slot_map is None else _c(slot_map, np.int32)
    history = None if history is None else _c(history)
    f32 = np.empty((rows, channels), np.float32)
    acc = np.empty((rows, channels), np.float32)
    out = np.empty((rows, channels), x.dtype)
    load().oracle_causal_conv_silu(_p(x), _p(w), _p(f32), _p(out), rows, channels, k, _p(seq_start), _p(history),
                                   _p(slot_map), _dtype_code(x), _p(acc), nthreads)
    return f32, out, acc


def gdn_gates(a, b, a_log, dt_bias, tokens, heads):
    a, b = _c(a), _c(b)
    decay, beta = np.empty((tokens, heads), np.float32), np.empty((tokens, heads), np.float32)
    load().oracle_gdn_gates(_p(a), _p(b), _p(_c(a_log, np.float32)), _p(_c(dt_bias, np.float32)), _p(decay), _p(beta),
                            tokens, heads, _dtype_code(a))
    return decay, beta


def gdn_prep(mixed, seq_len, kh, kd, heads, conv_dim):
    """kernels/gdn_chunk.cu:1176-1239 restated on the CPU -> dict(v, q_hi, q_lo, k_hi, k_lo (uint16 bf16 words), kn)."""
    mixed = _c(mixed)
    nchunks = (seq_len + 63) // 64
    words = heads * nchunks * 2 * 64 * 64
    out = {"v": np.empty((seq_len, heads * kd), np.float32), "kn": np.empty((seq_len, heads, kd), np.float32)}
    for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
        out[name] = np.zeros(words, np.uint16)
    q_scale = np.float32(1.0) / np.sqrt(np.float32(kd))
    load().oracle_gdn_prep(_p(mixed), _p(out["v"]), _p(out["q_hi"]), _p(out["q_lo"]), _p(out["k_hi"]), _p(out["k_lo"]),
                           _p(out["kn"]), seq_len, heads, kh, kd, conv_dim, ctypes.c_float(float(q_scale)), _dtype_code(mixed))
    return out
