"""Build libclef_fused.so in-tree with nvcc for sm_100a (`python -m aiis_clef_b200.build`).

The role of the reference's build.rs for this path: one arch (sm_100a), -O3 -lineinfo, ptxas -v
captured so register/spill regressions are visible, a failure if a -D macro is "redefined" by a
source (build.rs:233-240). The reference's SASS check is not carried over (nothing is disassembled).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libclef_fused.so"
SOURCES = ["clef_fused_abi.cu", "clef_layer_abi.cu", "clef_fp8_abi.cu", "clef_gdn_prep_abi.cu", "clef_host.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or put it on PATH")
    return cand


def needs_build() -> bool:
    if not OUT.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*")) + list((PKG.parent / "include").glob("*.h")))
    return newest > OUT.stat().st_mtime


def build_library(force: bool = False, defines: list[str] | None = None, verbose: bool = False) -> Path:
    if not force and not needs_build() and not defines:
        return OUT
    cmd = [find_nvcc(), *ARCH_FLAGS, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
           "-Xptxas", "-v", "-o", os.fspath(OUT)]
    cmd += [f"-D{d}" for d in (defines or [])]
    cmd += [os.fspath(CSRC / s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    (PKG / "build").mkdir(exist_ok=True)
    (PKG / "build" / "ptxas.log").write_text(" ".join(cmd) + "\n" + log)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{log}")
    if "redefined" in log:
        bad = "\n".join(line for line in log.splitlines() if "redefined" in line)
        raise RuntimeError(f"a -D flag was ignored because a source redefines it:\n{bad}")
    spills = [line for line in log.splitlines() if "spill" in line and "0 bytes spill stores, 0 bytes spill loads" not in line]
    if spills:
        print("warning: register spills:\n" + "\n".join(spills), file=sys.stderr)
    if verbose:
        print(log)
    return OUT


if __name__ == "__main__":
    path = build_library(force=True, verbose="-v" in sys.argv)
    print(f"built {path}")
