"""ctypes binding of libclef_fused.so (the C-ABI declared in include/clef_fused.h).

`Device` mirrors, name for name, the launchers of the reference's `impl Device`
(aiis-clef src/cuda/mod.rs:2133-2400, 2718-3074): each `*_dev` method takes device buffers
(torch CUDA tensors stand in for the reference's `Buffer`), allocates the outputs the reference
launcher allocates, issues one asynchronous launch on the current torch stream and returns the
outputs; a shape the entry point declines returns None (the reference's `Ok(None)`).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

CLEF_BF16 = 0
CLEF_F32 = 1

CLEF_OK = 0
CLEF_DECLINED = 1

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libclef_fused.so"

# (name, restype, argtypes) of every symbol include/clef_fused.h declares.
_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_SZ = ctypes.c_size_t
SYMBOLS = {
    "clef_last_error": (ctypes.c_char_p, []),
    "clef_version": (_I, []),
    "clef_sf_atom_for_tile_m": (_I, [_I, ctypes.POINTER(_I), ctypes.POINTER(_I)]),
    "clef_nvfp4_sizes": (_I, [_I, _I, _I, ctypes.POINTER(_I), ctypes.POINTER(_SZ), ctypes.POINTER(_SZ)]),
    "clef_embed_gather": (_I, [_P, _P, _P, _P, _I, _I, _I]),
    "clef_rms_norm": (_I, [_P, _P, _P, _P, _I, _I, _F, _I]),
    "clef_rms_norm_gated": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I]),
    "clef_swiglu": (_I, [_P, _P, _P, _P, _SZ, _I]),
    "clef_rope": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _I]),
    "clef_qk_norm_rope": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P, _P, _P, _I]),
    "clef_rope_tables": (_I, [_P, _P, _P, _P, _I, _I, _F]),
    "clef_quantise_nvfp4": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _I, _I]),
    "clef_rms_norm_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I]),
    "clef_rms_norm_gated_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I, _I, _I]),
    "clef_swiglu_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I]),
    "clef_to_bf16": (_I, [_P, _P, _P, _SZ, _P, _I, _I]),
    "clef_to_bf16_scatter": (_I, [_P, _P, _P, _SZ, _P, _I, _I]),
    "clef_rope_kv_write": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I]),
    "clef_rope_qk": (_I, [_P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I]),
    "clef_rope_qkv_write": (_I, [_P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _I]),
    "clef_qk_norm_rope_kv_write": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P, _P, _P, _P, _P, _I]),
    "clef_sigmoid_mul": (_I, [_P, _P, _P, _P, _SZ, _I]),
    "clef_sigmoid_mul_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I]),
    "clef_copy_bytes": (_I, [_P, _P, _SZ, _P, _SZ, _SZ]),
    "clef_add": (_I, [_P, _P, _P, _P, _SZ, _I]),
    "clef_add_rms_norm_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I]),
    "clef_embed_rms_norm_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I]),
    "clef_embed_rms_norm_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I, _I]),
    "clef_quantise_fp8": (_I, [_P, _P, _P, _P, _I, _I, _I]),
    "clef_swiglu_quantise_fp8": (_I, [_P, _P, _P, _P, _P, _I, _I, _I]),
    "clef_rms_norm_fp8_bf16": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _I]),
    "clef_rms_norm_gated_quantise_fp8": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I]),
    "clef_causal_conv_silu": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I]),
    "clef_conv_hist_save": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I]),
    "clef_gdn_gates": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I]),
    "clef_gdn_prep": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I]),
    "clef_gdn_conv_prep": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _F, _I]),
    "clef_split_q_gate": (_I, [_P, _P, _P, _P, _I, _I, _I, _I]),
    "clef_split_qkv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "clef_repeat_interleave": (_I, [_P, _P, _P, _I, _I, _I, _I, _I]),
    "clef_set_scale_layout": (_I, [_I]),
    "clef_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _I]),
    "clef_rms_norm_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I, _I]),
    "clef_rms_norm_gated_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I, _I, _I, _I]),
    "clef_swiglu_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _I]),
    "clef_sigmoid_mul_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _I]),
    "clef_add_rms_norm_quantise_nvfp4_ex": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I, _I, _I]),
    "clef_set_kernel_choice": (None, [_I]),
}


class ClefError(RuntimeError):
    """A C-ABI call returned a negative status, or the library could not be loaded."""


_lib = None


def load() -> ctypes.CDLL:
    """Load libclef_fused.so (built in-tree by aiis_clef_b200.build) and type its symbols."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ClefError(
            f"{LIB_PATH} is missing: build it with `python -m aiis_clef_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)   # AttributeError if the header and the library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().clef_last_error().decode()


def _check(status: int, what: str):
    if status < 0:
        raise ClefError(f"{what} failed ({status}): {last_error()}")
    return status


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return CLEF_BF16
    if t.dtype == torch.float32:
        return CLEF_F32
    raise ClefError(f"activations must be bfloat16 or float32, got {t.dtype}")


def _dev_tensor(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ClefError(f"{what} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ClefError(f"{what} must be contiguous")
    return t


def sf_atom_for_tile_m(tile_m: int) -> tuple[int, int]:
    """(blk_mn, chunk) for a GEMM M-tile (aiis-clef src/swizzle.rs:16-30)."""
    blk, chunk = _I(0), _I(0)
    _check(load().clef_sf_atom_for_tile_m(tile_m, ctypes.byref(blk), ctypes.byref(chunk)), "clef_sf_atom_for_tile_m")
    return blk.value, chunk.value


def nvfp4_sizes(rows: int, cols: int, blk_mn: int) -> tuple[int, int, int]:
    """(rows_padded, packed_bytes, scale_bytes) (aiis-clef src/cuda/mod.rs:2183-2187)."""
    rp, pb, sb = _I(0), _SZ(0), _SZ(0)
    _check(load().clef_nvfp4_sizes(rows, cols, blk_mn, ctypes.byref(rp), ctypes.byref(pb), ctypes.byref(sb)),
           "clef_nvfp4_sizes")
    return rp.value, pb.value, sb.value


def nvfp4_m_tile_for(m: int) -> int:
    """GEMM M-tile the reference picks for m rows (src/cuda/mod.rs:1164-1181 without env overrides)."""
    return 128


def set_kernel_choice(choice: int) -> None:
    """0: tuned kernel when the shape has one (default); 1: always the shape-general kernel."""
    load().clef_set_kernel_choice(int(choice))


SF_ACTIVATION, SF_INTERLEAVED = 0, 1


def set_scale_layout(layout: int) -> None:
    """Row order inside a scale tile for every NVFP4 entry point: SF_ACTIVATION (the reference's activation side,
    default) or SF_INTERLEAVED (the 32 x 4 x 4 order of src/swizzle.rs:66-68, read directly by block-scaled GEMMs)."""
    _check(load().clef_set_scale_layout(int(layout)), "clef_set_scale_layout")


class Device:
    """Mirror of the hot-path launchers of the reference's `Device` (src/cuda/mod.rs).

    Outputs are allocated here with torch (uninitialised: the kernels write every byte, padding
    included); all launches go to the current torch stream of `device`.
    """

    def __init__(self, device: int | str | torch.device = 0):
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.lib = load()
        if not torch.cuda.is_available():
            raise ClefError("no CUDA device: the fused kernels run on a B200 only")

    # -- helpers ------------------------------------------------------------------------------
    def _empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _quant_outputs(self, rows: int, cols: int, tile_m: int):
        blk_mn, chunk = sf_atom_for_tile_m(tile_m)
        rows_padded, packed_bytes, scale_bytes = nvfp4_sizes(rows, cols, blk_mn)
        packed = self._empty((rows_padded, cols // 2), torch.uint8)
        scales = self._empty((scale_bytes,), torch.uint8)
        return blk_mn, chunk, rows_padded, packed, scales

    # -- src/cuda/mod.rs:2908-2928 ------------------------------------------------------------
    def embed_gather_dev(self, table, ids, tokens: int, hidden: int):
        _dev_tensor(table, "table"), _dev_tensor(ids, "ids")
        out = self._empty((tokens, hidden), table.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_embed_gather(_stream(), _ptr(table), _ptr(ids), _ptr(out), tokens, hidden,
                                              _dtype_code(table)), "clef_embed_gather")
        return out

    # -- src/cuda/mod.rs:2718-2739 ------------------------------------------------------------
    def rms_norm_dev(self, x, weight, rows: int, cols: int, eps: float):
        _dev_tensor(x, "x")
        out = self._empty((rows, cols), x.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rms_norm(_stream(), _ptr(x), _ptr(weight), _ptr(out), rows, cols, eps,
                                          _dtype_code(x)), "clef_rms_norm")
        return out

    # -- src/cuda/mod.rs:2741-2763 ------------------------------------------------------------
    def rms_norm_gated_dev(self, x, gate, weight, rows: int, cols: int, eps: float):
        _dev_tensor(x, "x")
        out = self._empty((rows, cols), x.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rms_norm_gated(_stream(), _ptr(x), _ptr(gate), _ptr(weight), _ptr(out), rows, cols,
                                                eps, _dtype_code(x)), "clef_rms_norm_gated")
        return out

    # -- src/cuda/mod.rs:2765-2782 ------------------------------------------------------------
    def swiglu_dev(self, gate, up, total: int):
        _dev_tensor(gate, "gate"), _dev_tensor(up, "up")
        out = self._empty((total,), gate.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_swiglu(_stream(), _ptr(gate), _ptr(up), _ptr(out), total, _dtype_code(gate)),
                   "clef_swiglu")
        return out

    # -- src/cuda/mod.rs:2983-3005 ------------------------------------------------------------
    def rope_tables_dev(self, positions, rows: int, rotary_dim: int, theta: float):
        _dev_tensor(positions, "positions")
        cos = self._empty((rows, rotary_dim), torch.float32)
        sin = self._empty((rows, rotary_dim), torch.float32)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rope_tables(_stream(), _ptr(positions), _ptr(cos), _ptr(sin), rows, rotary_dim,
                                             theta), "clef_rope_tables")
        return cos, sin

    # -- src/cuda/mod.rs:3045-3074 ------------------------------------------------------------
    def rope_apply_dev(self, x, cos, sin, rows: int, heads: int, head_dim: int, rotary_dim: int,
                       seq_start=None, pos_base=None, pos_map=None):
        _dev_tensor(x, "x")
        out = self._empty((rows, heads, head_dim), x.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rope(_stream(), _ptr(out), _ptr(x), _ptr(cos), _ptr(sin), rows, heads, head_dim,
                                      rotary_dim, _ptr(seq_start), _ptr(pos_base), _ptr(pos_map), _dtype_code(x)),
                   "clef_rope")
        return out

    # -- src/cuda/mod.rs:3008-3043 ------------------------------------------------------------
    def qk_norm_rope_dev(self, x, weight, cos, sin, rows: int, heads: int, head_dim: int, rotary_dim: int,
                         eps: float, seq_start=None, pos_base=None, pos_map=None, with_gate: bool = False):
        _dev_tensor(x, "x")
        out = self._empty((rows, head_dim), x.dtype)
        gate = self._empty((rows, head_dim), x.dtype) if with_gate else None
        with torch.cuda.device(self.device):
            _check(self.lib.clef_qk_norm_rope(_stream(), _ptr(x), _ptr(weight), _ptr(cos), _ptr(sin), _ptr(out),
                                              _ptr(gate), rows, heads, head_dim, rotary_dim, eps, _ptr(seq_start),
                                              _ptr(pos_base), _ptr(pos_map), _dtype_code(x)), "clef_qk_norm_rope")
        return out, gate

    # -- src/cuda/mod.rs:2169-2207 ------------------------------------------------------------
    def quantise_nvfp4_dev(self, x, rows: int, cols: int, global_scale: float, tile_m: int):
        _dev_tensor(x, "x")
        blk_mn, chunk, _, packed, scales = self._quant_outputs(rows, cols, tile_m)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_quantise_nvfp4(_stream(), _ptr(x), _ptr(packed), _ptr(scales), rows, cols,
                                                global_scale, blk_mn, chunk, _dtype_code(x)), "clef_quantise_nvfp4")
        return packed, scales

    # -- src/cuda/mod.rs:2133-2167 ------------------------------------------------------------
    def rms_norm_quantise_nvfp4_dev(self, x, weight, rows: int, cols: int, eps: float, global_scale: float,
                                    tile_m: int):
        _dev_tensor(x, "x")
        if cols % 64 != 0:
            return None   # declined: the caller runs rms_norm_dev + quantise_nvfp4_dev
        blk_mn, chunk, _, packed, scales = self._quant_outputs(rows, cols, tile_m)
        with torch.cuda.device(self.device):
            st = _check(self.lib.clef_rms_norm_quantise_nvfp4(_stream(), _ptr(x), _ptr(weight), _ptr(packed),
                                                              _ptr(scales), rows, cols, eps, global_scale, blk_mn,
                                                              chunk, _dtype_code(x)), "clef_rms_norm_quantise_nvfp4")
        return None if st == CLEF_DECLINED else (packed, scales)

    # -- src/cuda/mod.rs:2269-2302 ------------------------------------------------------------
    def rms_norm_gated_quantise_nvfp4_dev(self, x, gate, weight, rows: int, cols: int, vh: int, eps: float,
                                          global_scale: float, tile_m: int):
        """`rows` counts live head rows (tokens * vh), as in the reference launcher."""
        _dev_tensor(x, "x"), _dev_tensor(gate, "gate")
        flat_cols = vh * cols
        tokens = rows // vh
        blk_mn, chunk, tokens_padded, _, scales = self._quant_outputs(tokens, flat_cols, tile_m)
        rows_padded = tokens_padded * vh
        packed = self._empty((rows_padded, cols // 2), torch.uint8)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rms_norm_gated_quantise_nvfp4(_stream(), _ptr(x), _ptr(gate), _ptr(weight),
                                                               _ptr(packed), _ptr(scales), rows_padded, cols, eps,
                                                               global_scale, blk_mn, chunk, vh, rows,
                                                               _dtype_code(x)),
                   "clef_rms_norm_gated_quantise_nvfp4")
        return packed, scales

    # -- src/cuda/mod.rs:2359-2400 ------------------------------------------------------------
    def swiglu_quantise_nvfp4_dev(self, gate, up, rows: int, cols: int, global_scale: float, tile_m: int):
        _dev_tensor(gate, "gate"), _dev_tensor(up, "up")
        if cols % 64 != 0:
            return None
        blk_mn, chunk, _, packed, scales = self._quant_outputs(rows, cols, tile_m)
        with torch.cuda.device(self.device):
            st = _check(self.lib.clef_swiglu_quantise_nvfp4(_stream(), _ptr(gate), _ptr(up), _ptr(packed),
                                                            _ptr(scales), rows, cols, global_scale, blk_mn, chunk,
                                                            _dtype_code(gate)), "clef_swiglu_quantise_nvfp4")
        return None if st == CLEF_DECLINED else (packed, scales)

    # ==== the steps either side of the fused quantisers ==========================================

    # -- src/cuda/mod.rs:1462-1465, 3201-3227 (to_bf16_kernel) ---------------------------------
    def to_bf16_dev(self, x, total: int, out=None, off_tokens=None, off_stride: int = 0):
        """bf16 copy of `x`; with `out` (a cache) and `off_tokens` it is written at *off_tokens * off_stride."""
        _dev_tensor(x, "x")
        if out is None:
            out = self._empty((total,), torch.bfloat16)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_to_bf16(_stream(), _ptr(out), _ptr(x), total, _ptr(off_tokens), off_stride,
                                         _dtype_code(x)), "clef_to_bf16")
        return out

    # -- src/cuda/mod.rs:3201-3227 (to_bf16_scatter_kernel) ------------------------------------
    def to_bf16_scatter_dev(self, out, x, total: int, pos_map, stride: int):
        _dev_tensor(x, "x"), _dev_tensor(out, "out")
        with torch.cuda.device(self.device):
            _check(self.lib.clef_to_bf16_scatter(_stream(), _ptr(out), _ptr(x), total, _ptr(pos_map), stride,
                                                 _dtype_code(x)), "clef_to_bf16_scatter")
        return out

    def rope_kv_write_dev(self, cache_k, cache_v, k, v, cos, sin, tokens: int, kv_heads: int, head_dim: int,
                          rotary_dim: int, seq_start=None, pos_base=None, pos_map=None, cache_map=None,
                          cache_len=None):
        """rope_apply_dev on k, then k and v into the bf16 caches (in place), one launch."""
        _dev_tensor(k, "k"), _dev_tensor(v, "v"), _dev_tensor(cache_k, "cache_k"), _dev_tensor(cache_v, "cache_v")
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rope_kv_write(_stream(), _ptr(cache_k), _ptr(cache_v), _ptr(k), _ptr(v), _ptr(cos),
                                               _ptr(sin), tokens, kv_heads, head_dim, rotary_dim, _ptr(seq_start),
                                               _ptr(pos_base), _ptr(pos_map), _ptr(cache_map), _ptr(cache_len),
                                               _dtype_code(k)), "clef_rope_kv_write")

    def rope_qk_dev(self, q, k, cos, sin, rows: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                    seq_start=None, pos_base=None, pos_map=None):
        """rope_apply_dev on q and on k in one launch; returns (q_out, k_out)."""
        _dev_tensor(q, "q"), _dev_tensor(k, "k")
        q_out, k_out = self._empty((rows, q_heads, head_dim), q.dtype), self._empty((rows, kv_heads, head_dim), k.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rope_qk(_stream(), _ptr(q_out), _ptr(q), q_heads, _ptr(k_out), _ptr(k), kv_heads, _ptr(cos),
                                         _ptr(sin), rows, head_dim, rotary_dim, _ptr(seq_start), _ptr(pos_base), _ptr(pos_map),
                                         _dtype_code(q)), "clef_rope_qk")
        return q_out, k_out

    def rope_qkv_write_dev(self, q, cache_k, cache_v, k, v, cos, sin, tokens: int, q_heads: int, kv_heads: int,
                           head_dim: int, rotary_dim: int, seq_start=None, pos_base=None, pos_map=None, cache_map=None,
                           cache_len=None):
        """rope_apply_dev on q (returned) and rope_kv_write_dev on k, v (caches written in place), one launch."""
        _dev_tensor(q, "q"), _dev_tensor(k, "k"), _dev_tensor(v, "v")
        q_out = self._empty((tokens, q_heads, head_dim), q.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rope_qkv_write(_stream(), _ptr(q_out), _ptr(q), q_heads, _ptr(cache_k), _ptr(cache_v), _ptr(k),
                                                _ptr(v), kv_heads, _ptr(cos), _ptr(sin), tokens, head_dim, rotary_dim,
                                                _ptr(seq_start), _ptr(pos_base), _ptr(pos_map), _ptr(cache_map),
                                                _ptr(cache_len), _dtype_code(q)), "clef_rope_qkv_write")
        return q_out

    def qk_norm_rope_kv_write_dev(self, cache_k, cache_v, k_raw, v, weight, cos, sin, tokens: int, kv_heads: int,
                                  head_dim: int, rotary_dim: int, eps: float, seq_start=None, pos_base=None,
                                  pos_map=None, cache_map=None, cache_len=None):
        """qk_norm_rope_dev on k_raw, then k and v into the bf16 caches (in place)."""
        _dev_tensor(k_raw, "k_raw"), _dev_tensor(v, "v"), _dev_tensor(cache_k, "cache_k"), _dev_tensor(cache_v, "cache_v")
        with torch.cuda.device(self.device):
            _check(self.lib.clef_qk_norm_rope_kv_write(_stream(), _ptr(cache_k), _ptr(cache_v), _ptr(k_raw), _ptr(v),
                                                       _ptr(weight), _ptr(cos), _ptr(sin), tokens, kv_heads, head_dim,
                                                       rotary_dim, eps, _ptr(seq_start), _ptr(pos_base), _ptr(pos_map),
                                                       _ptr(cache_map), _ptr(cache_len), _dtype_code(k_raw)),
                   "clef_qk_norm_rope_kv_write")

    # -- src/cuda/mod.rs:2838-2856 ------------------------------------------------------------
    def sigmoid_mul_dev(self, x, gate, total: int):
        _dev_tensor(x, "x"), _dev_tensor(gate, "gate")
        out = self._empty((total,), x.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_sigmoid_mul(_stream(), _ptr(out), _ptr(x), _ptr(gate), total, _dtype_code(x)),
                   "clef_sigmoid_mul")
        return out

    def sigmoid_mul_quantise_nvfp4_dev(self, x, gate, rows: int, cols: int, global_scale: float, tile_m: int):
        """sigmoid_mul_dev followed by quantise_nvfp4_dev, one launch."""
        _dev_tensor(x, "x"), _dev_tensor(gate, "gate")
        blk_mn, chunk, _, packed, scales = self._quant_outputs(rows, cols, tile_m)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_sigmoid_mul_quantise_nvfp4(_stream(), _ptr(x), _ptr(gate), _ptr(packed), _ptr(scales),
                                                            rows, cols, global_scale, blk_mn, chunk, _dtype_code(x)),
                   "clef_sigmoid_mul_quantise_nvfp4")
        return packed, scales

    # -- src/cuda/mod.rs:1686-1704 ------------------------------------------------------------
    def add_dev(self, a, b, total: int, out=None):
        _dev_tensor(a, "a"), _dev_tensor(b, "b")
        if out is None:
            out = self._empty((total,), a.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_add(_stream(), _ptr(out), _ptr(a), _ptr(b), total, _dtype_code(a)), "clef_add")
        return out

    # -- src/cuda/mod.rs:4642-4720 (copy_into, copy_bytes_at, copy_bytes) ------------------------------------
    def copy_bytes_dev(self, dst, dst_offset: int, src, src_offset: int, nbytes: int):
        _dev_tensor(dst, "dst"), _dev_tensor(src, "src")
        with torch.cuda.device(self.device):
            _check(self.lib.clef_copy_bytes(_stream(), _ptr(dst), dst_offset, _ptr(src), src_offset, nbytes), "clef_copy_bytes")

    def add_rms_norm_quantise_nvfp4_dev(self, a, b, weight, rows: int, cols: int, eps: float, global_scale: float,
                                        tile_m: int, sum_out=None):
        """add_dev followed by rms_norm_quantise_nvfp4_dev on the stored sum, one pass; returns (sum, packed, scales)."""
        _dev_tensor(a, "a"), _dev_tensor(b, "b")
        if sum_out is None:
            sum_out = self._empty((rows, cols), a.dtype)
        blk_mn, chunk, _, packed, scales = self._quant_outputs(rows, cols, tile_m)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_add_rms_norm_quantise_nvfp4(_stream(), _ptr(sum_out), _ptr(a), _ptr(b), _ptr(weight),
                                                             _ptr(packed), _ptr(scales), rows, cols, eps, global_scale,
                                                             blk_mn, chunk, _dtype_code(a)),
                   "clef_add_rms_norm_quantise_nvfp4")
        return sum_out, packed, scales

    def embed_rms_norm_quantise_nvfp4_dev(self, table, ids, weight, tokens: int, hidden: int, eps: float, global_scale: float,
                                          tile_m: int, h_out=None):
        """embed_gather_dev followed by rms_norm_quantise_nvfp4_dev on the gathered rows, one pass; returns
        (h, packed, scales)."""
        _dev_tensor(table, "table"), _dev_tensor(ids, "ids")
        if h_out is None:
            h_out = self._empty((tokens, hidden), table.dtype)
        blk_mn, chunk, _, packed, scales = self._quant_outputs(tokens, hidden, tile_m)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_embed_rms_norm_quantise_nvfp4(_stream(), _ptr(table), _ptr(ids), _ptr(h_out), _ptr(weight),
                                                               _ptr(packed), _ptr(scales), tokens, hidden, eps, global_scale,
                                                               blk_mn, chunk, _dtype_code(table)),
                   "clef_embed_rms_norm_quantise_nvfp4")
        return h_out, packed, scales

    # ==== FP8 (E4M3) activation quantisers ======================================================

    # -- src/cuda/mod.rs:2246-2266 ------------------------------------------------------------
    def quantise_fp8_dev(self, x, rows: int, cols: int):
        _dev_tensor(x, "x")
        out, scales = self._empty((rows, cols), torch.uint8), self._empty((rows,), torch.int16)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_quantise_fp8(_stream(), _ptr(x), _ptr(out), _ptr(scales), rows, cols, _dtype_code(x)),
                   "clef_quantise_fp8")
        return out, scales

    # -- src/cuda/mod.rs:2402-2427 ------------------------------------------------------------
    def swiglu_quantise_fp8_dev(self, gate, up, rows: int, cols: int):
        _dev_tensor(gate, "gate"), _dev_tensor(up, "up")
        out, scales = self._empty((rows, cols), torch.uint8), self._empty((rows,), torch.int16)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_swiglu_quantise_fp8(_stream(), _ptr(gate), _ptr(up), _ptr(out), _ptr(scales), rows, cols,
                                                     _dtype_code(gate)), "clef_swiglu_quantise_fp8")
        return out, scales

    # -- src/cuda/mod.rs:2330-2358 ------------------------------------------------------------
    def rms_norm_fp8_bf16_dev(self, x, weight, rows: int, cols: int, eps: float):
        """(codes, row scales, bf16 copy) of the normalised rows."""
        _dev_tensor(x, "x")
        q, qs = self._empty((rows, cols), torch.uint8), self._empty((rows,), torch.int16)
        bf = self._empty((rows, cols), torch.bfloat16)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rms_norm_fp8_bf16(_stream(), _ptr(x), _ptr(weight), _ptr(q), _ptr(qs), _ptr(bf), rows, cols,
                                                   eps, _dtype_code(x)), "clef_rms_norm_fp8_bf16")
        return q, qs, bf

    # -- src/cuda/mod.rs:2304-2328 ------------------------------------------------------------
    def rms_norm_gated_quantise_fp8_dev(self, x, gate, weight, rows: int, cols: int, vh: int, eps: float):
        _dev_tensor(x, "x"), _dev_tensor(gate, "gate")
        out, scales = self._empty((rows, cols), torch.uint8), self._empty((rows // vh,), torch.int16)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_rms_norm_gated_quantise_fp8(_stream(), _ptr(x), _ptr(gate), _ptr(weight), _ptr(out),
                                                             _ptr(scales), rows, cols, eps, vh, rows, _dtype_code(x)),
                   "clef_rms_norm_gated_quantise_fp8")
        return out, scales

    # ==== elementwise kernels in front of the GDN scan ==========================================

    # -- src/cuda/mod.rs:2784-2812 ------------------------------------------------------------
    def causal_conv_silu_dev(self, x, w, rows: int, channels: int, k: int, seq_start=None, history=None, slot_map=None):
        _dev_tensor(x, "x")
        out = self._empty((rows, channels), x.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_causal_conv_silu(_stream(), _ptr(out), _ptr(x), _ptr(w), rows, channels, k, _ptr(seq_start),
                                                  _ptr(history), _ptr(slot_map), _dtype_code(x)), "clef_causal_conv_silu")
        return out

    # -- src/cuda/mod.rs:2814-2836 ------------------------------------------------------------
    def conv_hist_save_dev(self, src, hist, saves, n_saves: int, rows: int, k: int, channels: int):
        _dev_tensor(src, "src"), _dev_tensor(hist, "hist")
        with torch.cuda.device(self.device):
            _check(self.lib.clef_conv_hist_save(_stream(), _ptr(hist), _ptr(src), _ptr(saves), n_saves, rows, k, channels,
                                                _dtype_code(src)), "clef_conv_hist_save")

    # -- src/cuda/mod.rs:3606-3647 ------------------------------------------------------------
    def gdn_prep_dev(self, mixed, seq_len: int, kh: int, kd: int, heads: int, conv_dim: int):
        """-> dict(v, q_hi, q_lo, k_hi, k_lo, kn): the chunked scan's operands of the convolved rows; q_scale is
        1 / sqrt(kd) as in the reference launcher."""
        _dev_tensor(mixed, "mixed")
        nchunks = (seq_len + 63) // 64
        nbytes = heads * nchunks * 2 * 64 * 128
        out = {"v": self._empty((seq_len, heads * kd), torch.float32), "kn": self._empty((seq_len, heads, kd), torch.float32)}
        for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
            out[name] = self._empty((nbytes,), torch.uint8)
        q_scale = float(_np.float32(1.0) / _np.sqrt(_np.float32(kd)))
        with torch.cuda.device(self.device):
            _check(self.lib.clef_gdn_prep(_stream(), _ptr(mixed), _ptr(out["v"]), _ptr(out["q_hi"]), _ptr(out["q_lo"]),
                                          _ptr(out["k_hi"]), _ptr(out["k_lo"]), _ptr(out["kn"]), seq_len, heads, kh, kd, conv_dim,
                                          q_scale, _dtype_code(mixed)), "clef_gdn_prep")
        return out

    # -- src/cuda/mod.rs:3649-3707 ------------------------------------------------------------
    def gdn_conv_prep_dev(self, x, w, seq_len: int, kh: int, kd: int, heads: int, conv_dim: int, k: int, seq_start=None,
                          history=None, slot_map=None):
        """Causal convolution + silu + gdn_prep in one launch -> dict(v, q_hi, q_lo, k_hi, k_lo, kn)."""
        _dev_tensor(x, "x")
        nchunks = (seq_len + 63) // 64
        nbytes = heads * nchunks * 2 * 64 * 128
        out = {"v": self._empty((seq_len, heads * kd), torch.float32), "kn": self._empty((seq_len, heads, kd), torch.float32)}
        for name in ("q_hi", "q_lo", "k_hi", "k_lo"):
            out[name] = self._empty((nbytes,), torch.uint8)
        q_scale = float(_np.float32(1.0) / _np.sqrt(_np.float32(kd)))
        with torch.cuda.device(self.device):
            status = _check(self.lib.clef_gdn_conv_prep(_stream(), _ptr(x), _ptr(w), _ptr(out["v"]), _ptr(out["q_hi"]),
                                                        _ptr(out["q_lo"]), _ptr(out["k_hi"]), _ptr(out["k_lo"]), _ptr(out["kn"]),
                                                        seq_len, conv_dim, k, _ptr(seq_start), _ptr(history), _ptr(slot_map),
                                                        heads, kh, kd, q_scale, _dtype_code(x)), "clef_gdn_conv_prep")
        if status == CLEF_DECLINED:   # a tap count other than 4, heads / kh other than 1, 2, 4, or the general kernel choice: the two calls
            mixed = self.causal_conv_silu_dev(x, w, seq_len, conv_dim, k, seq_start, history, slot_map)
            return self.gdn_prep_dev(mixed, seq_len, kh, kd, heads, conv_dim)
        return out

    # -- src/cuda/mod.rs:2858-2882 ------------------------------------------------------------
    def gdn_gates_dev(self, a, b, a_log, dt_bias, tokens: int, heads: int):
        _dev_tensor(a, "a"), _dev_tensor(b, "b")
        decay, beta = self._empty((tokens, heads), torch.float32), self._empty((tokens, heads), torch.float32)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_gdn_gates(_stream(), _ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias), _ptr(decay), _ptr(beta),
                                           tokens, heads, _dtype_code(a)), "clef_gdn_gates")
        return decay, beta

    # -- src/cuda/mod.rs:2884-2906 ------------------------------------------------------------
    def split_q_gate_dev(self, qg, tokens: int, heads: int, head_dim: int):
        _dev_tensor(qg, "qg")
        q, gate = self._empty((tokens, heads, head_dim), qg.dtype), self._empty((tokens, heads, head_dim), qg.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_split_q_gate(_stream(), _ptr(qg), _ptr(q), _ptr(gate), tokens, heads, head_dim,
                                              _dtype_code(qg)), "clef_split_q_gate")
        return q, gate

    # -- src/cuda/mod.rs:2930-2958 ------------------------------------------------------------
    def split_qkv_dev(self, mixed, tokens: int, kh: int, kd: int, vh: int, vd: int):
        _dev_tensor(mixed, "mixed")
        q, k = self._empty((tokens, kh * kd), mixed.dtype), self._empty((tokens, kh * kd), mixed.dtype)
        v = self._empty((tokens, vh * vd), mixed.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_split_qkv(_stream(), _ptr(mixed), _ptr(q), _ptr(k), _ptr(v), tokens, kh, kd, vh, vd,
                                           _dtype_code(mixed)), "clef_split_qkv")
        return q, k, v

    # -- src/cuda/mod.rs:2959-2982 ------------------------------------------------------------
    def repeat_interleave_dev(self, src, tokens: int, kh: int, ratio: int, dim: int):
        _dev_tensor(src, "src")
        out = self._empty((tokens, kh * ratio, dim), src.dtype)
        with torch.cuda.device(self.device):
            _check(self.lib.clef_repeat_interleave(_stream(), _ptr(src), _ptr(out), tokens, kh, ratio, dim,
                                                   _dtype_code(src)), "clef_repeat_interleave")
        return out


# =================================================================================================
# Host-side companions (include/clef_host.h): device handle + host-slice launchers, per-token maps.
# =================================================================================================
import numpy as _np  # noqa: E402


class _ChunkSpec(ctypes.Structure):
    _fields_ = [("ids", ctypes.POINTER(ctypes.c_uint32)), ("ids_len", _SZ), ("pos", _SZ), ("slot", _SZ), ("rows", _SZ)]


class _PassMaps(ctypes.Structure):
    _fields_ = [("ids", _P), ("seq_start", _P), ("seq_end", _P), ("cpos", _P), ("cbase", _P), ("slot_map", _P),
                ("rope_pos", _P), ("chunk_start", _P), ("state_slot", _P), ("hist_save", _P), ("rows_real", _P),
                ("offs", _P), ("cache_len", ctypes.c_int32), ("total", _SZ)]


HOST_SYMBOLS = {
    "clef_device_open": (_I, [_I, ctypes.POINTER(_P)]),
    "clef_device_close": (_I, [_P]),
    "clef_device_ordinal": (_I, [_P]),
    "clef_device_stream": (_P, [_P]),
    "clef_device_synchronize": (_I, [_P]),
    "clef_device_set_pipelined": (_I, [_P, _I]),
    "clef_device_alloc": (_I, [_P, _SZ, ctypes.POINTER(_P)]),
    "clef_device_free": (_I, [_P, _P]),
    "clef_device_upload": (_I, [_P, _P, _P, _SZ]),
    "clef_device_download": (_I, [_P, _P, _P, _SZ]),
    "clef_host_alloc_pinned": (_I, [_SZ, ctypes.POINTER(_P)]),
    "clef_host_free_pinned": (_I, [_P]),
    "clef_host_embed_gather": (_I, [_P, _P, _P, _P, _I, _I, _I]),
    "clef_host_quantise_fp8": (_I, [_P, _P, _P, _P, _I, _I, _I]),
    "clef_host_quantise_nvfp4": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _I]),
    "clef_host_rms_norm_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _I]),
    "clef_host_swiglu_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I]),
    "clef_host_rms_norm_gated_quantise_nvfp4": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _F, _I, _I]),
    "clef_host_rope": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I]),
    "clef_host_rms_norm": (_I, [_P, _P, _P, _P, _I, _I, _F, _I]),
    "clef_host_rms_norm_gated": (_I, [_P, _P, _P, _P, _P, _I, _I, _F, _I]),
    "clef_host_swiglu": (_I, [_P, _P, _P, _P, _SZ, _I]),
    "clef_host_causal_conv_silu": (_I, [_P, _P, _P, _P, _I, _I, _I, _I]),
    "clef_host_rope_tables": (_I, [_P, _P, _P, _P, _I, _I, _F]),
    "clef_pass_maps_build": (_I, [ctypes.POINTER(_ChunkSpec), _SZ, _SZ, _I, _SZ, _SZ, ctypes.POINTER(_PassMaps)]),
    "clef_pass_geometries": (_I, [_SZ, _SZ, ctypes.POINTER(_SZ), _SZ]),
    "clef_rungs_decompose": (_I, [_SZ, _SZ, _SZ, ctypes.POINTER(_SZ), ctypes.POINTER(_SZ), _SZ]),
    "clef_shard_rows": (_I, [_I, _I, _I, _I, ctypes.POINTER(_I), ctypes.POINTER(_I)]),
}

_host_typed = False


def load_host() -> ctypes.CDLL:
    """The same shared library with the symbols of include/clef_host.h typed."""
    global _host_typed
    lib = load()
    if not _host_typed:
        for name, (restype, argtypes) in HOST_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _host_typed = True
    return lib


def pass_geometries(slots: int = 1, max_chunk: int = 8192) -> list[int]:
    """Row totals a pass may have (aiis-clef src/gpu.rs:779-795)."""
    lib = load_host()
    buf = (_SZ * 4096)()
    n = lib.clef_pass_geometries(slots, max_chunk, buf, 4096)
    return [int(buf[i]) for i in range(n)]


def rungs_decompose(tokens: int, slots: int = 1, max_chunk: int = 8192) -> list[tuple[int, int]]:
    """Rungs::decompose (src/gpu.rs:762-775): (base, rows) chunks, largest rung first."""
    lib = load_host()
    cap = tokens // 64 + 2
    bases, rows = (_SZ * cap)(), (_SZ * cap)()
    n = lib.clef_rungs_decompose(tokens, slots, max_chunk, bases, rows, cap)
    return [(int(bases[i]), int(rows[i])) for i in range(n)]


def shard_rows(rows: int, blk_mn: int, n_shards: int, shard: int) -> tuple[int, int]:
    """(first_row, n_rows) of a shard: contiguous, aligned to the scale atom."""
    first, n = _I(0), _I(0)
    _check(load_host().clef_shard_rows(rows, blk_mn, n_shards, shard, ctypes.byref(first), ctypes.byref(n)),
           "clef_shard_rows")
    return first.value, n.value


def pass_maps(chunks, capacity: int, check_geometry: bool = False, slots: int = 1, max_chunk: int = 8192) -> dict:
    """Per-token maps of one pass (src/gpu.rs:948-1013).

    chunks: iterable of (ids: uint32 array, pos, slot, rows). Returns a dict of numpy arrays
    (ids, seq_start, seq_end, cpos, cbase, slot_map, rope_pos per row; chunk_start, state_slot per
    64-row granule; hist_save [n, 2]; rows_real, offs per chunk) plus cache_len and total.
    """
    lib = load_host()
    chunks = list(chunks)
    n = len(chunks)
    specs = (_ChunkSpec * max(n, 1))()
    keep = []
    total = 0
    for i, (ids, pos, slot, rows) in enumerate(chunks):
        arr = _np.ascontiguousarray(ids, dtype=_np.uint32)
        keep.append(arr)
        specs[i] = _ChunkSpec(arr.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), arr.size, pos, slot, rows)
        total += int(rows)
    gran = max(total // 64, 1)
    out = {
        "ids": _np.zeros(total, _np.uint32), "seq_start": _np.zeros(total, _np.int32),
        "seq_end": _np.zeros(total, _np.int32), "cpos": _np.zeros(total, _np.int32),
        "cbase": _np.zeros(total, _np.int32), "slot_map": _np.zeros(total, _np.int32),
        "rope_pos": _np.zeros(total, _np.int32), "chunk_start": _np.zeros(gran, _np.int32),
        "state_slot": _np.zeros(gran, _np.int32), "hist_save": _np.zeros((max(n, 1), 2), _np.uint32),
        "rows_real": _np.zeros(max(n, 1), _np.uint64), "offs": _np.zeros(max(n, 1), _np.uint64),
    }
    m = _PassMaps(*[out[k].ctypes.data_as(_P) for k in ("ids", "seq_start", "seq_end", "cpos", "cbase", "slot_map",
                                                        "rope_pos", "chunk_start", "state_slot", "hist_save",
                                                        "rows_real", "offs")], 0, 0)
    _check(lib.clef_pass_maps_build(specs, n, capacity, int(check_geometry), slots, max_chunk, ctypes.byref(m)),
           "clef_pass_maps_build")
    out["chunk_start"] = out["chunk_start"][: total // 64]
    out["state_slot"] = out["state_slot"][: total // 64]
    out["hist_save"] = out["hist_save"][:n]
    out["rows_real"] = out["rows_real"][:n].astype(_np.int64)
    out["offs"] = out["offs"][:n].astype(_np.int64)
    out["cache_len"] = int(m.cache_len)
    out["total"] = int(m.total)
    return out


class HostDevice:
    """Device handle with the host-slice launchers (include/clef_host.h): numpy arrays or pinned torch
    CPU tensors in, the same out. Mirrors the reference's host-slice wrappers
    (aiis-clef src/cuda/mod.rs:853-1075), which upload, launch and download in one call."""

    def __init__(self, ordinal: int = 0):
        self.lib = load_host()
        handle = _P()
        _check(self.lib.clef_device_open(ordinal, ctypes.byref(handle)), "clef_device_open")
        self.handle = handle
        self.ordinal = ordinal

    def close(self):
        if self.handle:
            self.lib.clef_device_close(self.handle)
            self.handle = None

    def set_pipelined(self, on: bool):
        """Pipelined mode: the calls below return once enqueued; `synchronize()` completes them. Every buffer passed
        to a call (weights included) must stay alive and unchanged until then."""
        _check(self.lib.clef_device_set_pipelined(self.handle, int(bool(on))), "clef_device_set_pipelined")

    def synchronize(self):
        _check(self.lib.clef_device_synchronize(self.handle), "clef_device_synchronize")

    # stream-ordered device memory of the handle (raw device addresses; clef_device_alloc / _upload / _download / _free)
    def alloc(self, nbytes: int) -> int:
        out = _P()
        _check(self.lib.clef_device_alloc(self.handle, ctypes.c_size_t(nbytes), ctypes.byref(out)), "clef_device_alloc")
        return out.value

    def free(self, address: int):
        _check(self.lib.clef_device_free(self.handle, ctypes.c_void_p(address)), "clef_device_free")

    def upload(self, address: int, src, nbytes: int):
        """Enqueue a host-to-device copy (returns at once: `src` must stay alive until the handle is synchronised)."""
        _check(self.lib.clef_device_upload(self.handle, ctypes.c_void_p(address), self._hp(src), ctypes.c_size_t(nbytes)),
               "clef_device_upload")

    def download(self, dst, address: int, nbytes: int):
        _check(self.lib.clef_device_download(self.handle, self._hp(dst), ctypes.c_void_p(address), ctypes.c_size_t(nbytes)),
               "clef_device_download")

    def embed_gather_from(self, table_address: int, ids, out, tokens: int, hidden: int, dtype_code: int = CLEF_BF16):
        """clef_host_embed_gather with the table given as a raw device address (one obtained from `alloc`)."""
        _check(self.lib.clef_host_embed_gather(self.handle, ctypes.c_void_p(table_address), self._hp(ids), self._hp(out), tokens,
                                               hidden, dtype_code), "clef_host_embed_gather")

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _hp(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            assert not a.is_cuda and a.is_contiguous()
            return ctypes.c_void_p(a.data_ptr())
        assert a.flags["C_CONTIGUOUS"]
        return ctypes.c_void_p(a.ctypes.data)

    @staticmethod
    def _code(a):
        dt = a.dtype
        if dt in (torch.bfloat16, _np.uint16):
            return CLEF_BF16
        if dt in (torch.float32, _np.float32):
            return CLEF_F32
        raise ClefError(f"activations must be bf16 (uint16 bits / torch.bfloat16) or float32, got {dt}")

    def embed_gather(self, table_dev: torch.Tensor, ids, out, tokens: int, hidden: int):
        _check(self.lib.clef_host_embed_gather(self.handle, _ptr(table_dev), self._hp(ids), self._hp(out), tokens,
                                               hidden, _dtype_code(table_dev)), "clef_host_embed_gather")

    def quantise_fp8(self, x, out, scales, rows, cols):
        _check(self.lib.clef_host_quantise_fp8(self.handle, self._hp(x), self._hp(out), self._hp(scales), rows, cols,
                                               self._code(x)), "clef_host_quantise_fp8")

    def quantise_nvfp4(self, x, packed, scales, rows, cols, global_scale, tile_m=128):
        _check(self.lib.clef_host_quantise_nvfp4(self.handle, self._hp(x), self._hp(packed), self._hp(scales), rows,
                                                 cols, global_scale, tile_m, self._code(x)), "clef_host_quantise_nvfp4")

    def rms_norm_quantise_nvfp4(self, x, weight, packed, scales, rows, cols, eps, global_scale, tile_m=128):
        _check(self.lib.clef_host_rms_norm_quantise_nvfp4(self.handle, self._hp(x), self._hp(weight), self._hp(packed),
                                                          self._hp(scales), rows, cols, eps, global_scale, tile_m,
                                                          self._code(x)), "clef_host_rms_norm_quantise_nvfp4")

    def swiglu_quantise_nvfp4(self, gate, up, packed, scales, rows, cols, global_scale, tile_m=128):
        _check(self.lib.clef_host_swiglu_quantise_nvfp4(self.handle, self._hp(gate), self._hp(up), self._hp(packed),
                                                        self._hp(scales), rows, cols, global_scale, tile_m,
                                                        self._code(gate)), "clef_host_swiglu_quantise_nvfp4")

    def rms_norm_gated_quantise_nvfp4(self, x, gate, weight, packed, scales, rows, cols, vh, eps, global_scale,
                                      tile_m=128):
        _check(self.lib.clef_host_rms_norm_gated_quantise_nvfp4(self.handle, self._hp(x), self._hp(gate),
                                                                self._hp(weight), self._hp(packed), self._hp(scales),
                                                                rows, cols, vh, eps, global_scale, tile_m,
                                                                self._code(x)),
               "clef_host_rms_norm_gated_quantise_nvfp4")

    # -- the reference's plain host-slice wrappers, src/cuda/mod.rs:853-973 ------------------------------------
    def rms_norm(self, x, weight, out, rows, cols, eps):
        _check(self.lib.clef_host_rms_norm(self.handle, self._hp(x), self._hp(weight), self._hp(out), rows, cols, eps,
                                           self._code(x)), "clef_host_rms_norm")

    def rms_norm_gated(self, x, gate, weight, out, rows, cols, eps):
        _check(self.lib.clef_host_rms_norm_gated(self.handle, self._hp(x), self._hp(gate), self._hp(weight), self._hp(out), rows,
                                                 cols, eps, self._code(x)), "clef_host_rms_norm_gated")

    def swiglu(self, gate, up, out, total):
        _check(self.lib.clef_host_swiglu(self.handle, self._hp(gate), self._hp(up), self._hp(out), total, self._code(gate)),
               "clef_host_swiglu")

    def causal_conv_silu(self, x, w, out, rows, channels, k):
        _check(self.lib.clef_host_causal_conv_silu(self.handle, self._hp(x), self._hp(w), self._hp(out), rows, channels, k,
                                                   self._code(x)), "clef_host_causal_conv_silu")

    def rope_tables(self, positions, cos_out, sin_out, count, rotary_dim, theta):
        _check(self.lib.clef_host_rope_tables(self.handle, self._hp(positions), self._hp(cos_out), self._hp(sin_out), count,
                                              rotary_dim, theta), "clef_host_rope_tables")

    def rope(self, out, x, cos, sin, table_rows, rows, heads, head_dim, rotary_dim, pos_map=None):
        _check(self.lib.clef_host_rope(self.handle, self._hp(out), self._hp(x), self._hp(cos), self._hp(sin),
                                       table_rows, rows, heads, head_dim, rotary_dim, self._hp(pos_map),
                                       self._code(x)), "clef_host_rope")
