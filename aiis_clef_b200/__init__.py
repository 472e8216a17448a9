"""B200 (sm_100a) implementation of aiis-clef's fused per-layer elementwise hot path.

The product is the C-ABI shared library built from csrc/ (see include/clef_fused.h); this package
holds its build step and a ctypes binding whose `Device` class mirrors the reference launchers.
"""
from .lib import (CLEF_BF16, CLEF_F32, ClefError, Device, HostDevice, load, load_host, nvfp4_m_tile_for,  # noqa: F401
                  nvfp4_sizes, pass_geometries, pass_maps, rungs_decompose, shard_rows,
                  set_kernel_choice, set_scale_layout, sf_atom_for_tile_m, SF_ACTIVATION, SF_INTERLEAVED)
