#!/usr/bin/env python
"""Benchmark of the fused per-layer elementwise hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun, one rank per GPU)
    python bench.py --impl reference ...                     (the reference arithmetic on the host cores)
    python bench.py --profile-case KERNEL[,KERNEL...]        (three launches of the named entry points, for ncu)

A step is one pass of the hot path over one 8,192-row chunk (hidden 2048, bf16 activations, fp32
math): RMSNorm+NVFP4, SwiGLU(2x6144)+NVFP4, partial RoPE on 16 q and 2 kv heads x 128 (rotary 64,
theta 1e7, cpos = 0..8191). Inputs are seeded synthetic tensors already resident in HBM; buffer
sets rotate so no step can be served from L2. Rank 0 prints ONE JSON line: rows/s over all ranks
(`value`: K graph replays per batch, the median of five batches, device-timed, max over ranks), the
end-to-end figure through the host-slice C-ABI with host<->device copies inside the timed region
(`e2e`), the HBM roofline of the dominant kernel (`roofline`), the CPU restatement timed on the host
cores (`cpu_baseline`), clocks, per-kernel figures (each kernel rotating over at least three L2
sizes of its own buffers), the 130,712-row pass sharded by row range over the ranks as one CUDA graph
(strong scaling, with a check that the shards' bytes equal a single-GPU run's), and on one GPU the
benchmark definition's other configurations (the gated chain in four chunks, the 130,712-row pass as
rung-sized passes, the rung sweep with four coalesced requests). Every rank works on its own chunk
in the headline (weak scaling); the path has no collective.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, os.fspath(ROOT))

METRIC = "fused_layer_rows_per_s"
UNIT = "rows/s"
ROWS = 8192
HIDDEN, INTER = 2048, 6144
Q_HEADS, KV_HEADS, HEAD_DIM, ROTARY, THETA = 16, 2, 128, 64, 1e7
VH = 16                      # GDN value heads (x 128) of the gated RMSNorm, reported under "kernels"
CONV_DIM, CONV_K = 8192, 4   # GDN convolution: 2 x 16 x 128 (q, k) + 32 x 128 (v) channels, 4 taps
VOCAB = 32768
EPS = 1e-6
GS_NORM, GS_SWIGLU, GS_GATED = 64.0, 48.0, 96.0     # per-projection input_global_scale stand-ins
NSETS = 4                    # rotating buffer sets of the step (each far larger than L2)
FULL_ROWS = 130712
BATCHES = 5                  # timed batches per figure; the median is reported
ROTATE_BYTES = 400e6         # a kernel timed alone rotates over at least this much of its own buffers (3 x the 126 MB L2)

# Algorithmic bytes per row (inputs read once + outputs written once; shared vectors excluded).
BYTES_PER_ROW = {
    "rms_norm_quantise_nvfp4": 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,                       # 5,248
    "swiglu_quantise_nvfp4": 2 * 2 * INTER + INTER // 2 + INTER // 16,                        # 28,032
    "rope_q": 2 * Q_HEADS * HEAD_DIM * 2 + 4 + 2 * (ROTARY // 2) * 4,                         # 8,452
    "rope_k": 2 * KV_HEADS * HEAD_DIM * 2 + 4 + 2 * (ROTARY // 2) * 4,                        # 1,284
    "rope_qk": 2 * (Q_HEADS + KV_HEADS) * HEAD_DIM * 2 + 4 + 2 * (ROTARY // 2) * 4,           # 9,476 (q and k, one launch)
    "embed_gather": 4 + 2 * HIDDEN + 2 * HIDDEN,                                              # 8,196
    "rms_norm_gated_quantise_nvfp4": 2 * 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,             # 9,344
    # the first layer's gather and norm + quantiser in one pass (writes h too)
    "embed_rms_norm_quantise_nvfp4": 4 + 2 * HIDDEN + 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,   # 9,348
    # the unfused entry points (what the engine runs when a fusion is switched off), bf16 in and out
    "quantise_nvfp4": 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,                                # 5,248
    "rms_norm": 2 * HIDDEN + 2 * HIDDEN,                                                      # 8,192
    "swiglu": 3 * 2 * INTER,                                                                  # 36,864
    "rms_norm_gated": 3 * 2 * HIDDEN,                                                         # 12,288
    "qk_norm_rope_q": 2 * Q_HEADS * HEAD_DIM * 2 + 4 + 2 * (ROTARY // 2) * 4,                 # 8,452
    # the head shape the reference's fused kernel serves: 16 heads x 256 with the gate half split off ([q | gate] in)
    "qk_norm_rope_q_hd256_gate": 2 * Q_HEADS * 512 * 2 + 4 + 2 * (ROTARY // 2) * 4,           # 33,028
    # the steps either side of the fused quantisers (attention width = Q_HEADS * HEAD_DIM = HIDDEN here)
    "rope_kv_write": 4 * KV_HEADS * HEAD_DIM * 2 + 8 + 2 * (ROTARY // 2) * 4,                 # 2,312 (k, v in; both caches out)
    "qk_norm_rope_kv_write": 4 * KV_HEADS * HEAD_DIM * 2 + 8 + 2 * (ROTARY // 2) * 4,         # 2,312
    "sigmoid_mul_quantise_nvfp4": 2 * 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,                # 9,344
    "sigmoid_mul": 3 * 2 * HIDDEN,                                                            # 12,288
    "add": 3 * 2 * HIDDEN,                                                                    # 12,288
    "add_rms_norm_quantise_nvfp4": 3 * 2 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,               # 13,440
    # FP8 (E4M3) quantisers: one code byte per value, one 2-byte scale per row
    "quantise_fp8": 2 * HIDDEN + HIDDEN + 2,                                                  # 6,146
    "rms_norm_fp8_bf16": 2 * HIDDEN + HIDDEN + 2 + 2 * HIDDEN,                                # 10,242 (codes + bf16 twin)
    "swiglu_quantise_fp8": 2 * 2 * INTER + INTER + 2,                                         # 30,722
    "rms_norm_gated_quantise_fp8": 2 * 2 * HIDDEN + HIDDEN + 2,                               # 10,242
    # in front of the GDN scan: causal convolution (4 taps) + silu over the 8,192 mixed q/k/v channels
    "causal_conv_silu": 2 * 2 * CONV_DIM + 4,                                                 # 32,772
    # the scan's operands from the convolved row (16 q/k heads, 32 v heads of 128): bf16 row in; q and k as bf16
    # hi + lo pairs for 32 expanded heads, normalised k and v as f32 out
    "gdn_prep": 2 * CONV_DIM + 4 * 32 * 128 * 2 + 2 * 32 * 128 * 4,                           # 81,920
    # the two above in one launch (the convolved row never goes through memory): mixed row in, the scan's operands out
    "gdn_conv_prep": 2 * CONV_DIM + 4 * 32 * 128 * 2 + 2 * 32 * 128 * 4 + 4,                  # 81,924
}
# The same entry points on f32 activations (the reference engine's own residual-stream type: the bit-exact drop-in),
# reported under "other_configurations": 4-byte activations in and out, the quantised outputs unchanged.
F32_BYTES_PER_ROW = {
    "rms_norm_quantise_nvfp4": 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "swiglu_quantise_nvfp4": 2 * 4 * INTER + INTER // 2 + INTER // 16,
    "rope_qk": 2 * (Q_HEADS + KV_HEADS) * HEAD_DIM * 4 + 4 + 2 * (ROTARY // 2) * 4,
    "rms_norm_gated_quantise_nvfp4": 2 * 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "embed_rms_norm_quantise_nvfp4": 4 + 4 * HIDDEN + 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "quantise_nvfp4": 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "rms_norm": 2 * 4 * HIDDEN,
    "rms_norm_gated": 3 * 4 * HIDDEN,
    "qk_norm_rope_q_hd256_gate": 2 * Q_HEADS * 512 * 4 + 4 + 2 * (ROTARY // 2) * 4,
    "sigmoid_mul_quantise_nvfp4": 2 * 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "add_rms_norm_quantise_nvfp4": 3 * 4 * HIDDEN + HIDDEN // 2 + HIDDEN // 16,
    "quantise_fp8": 4 * HIDDEN + HIDDEN + 2,
    "rms_norm_fp8_bf16": 4 * HIDDEN + HIDDEN + 2 + 2 * HIDDEN,
    "swiglu_quantise_fp8": 2 * 4 * INTER + INTER + 2,
    "rms_norm_gated_quantise_fp8": 2 * 4 * HIDDEN + HIDDEN + 2,
}
# The step, in the order a layer runs its kernels: the partial RoPE of the q and the k heads (attention block; they
# share their positions and go out as one launch, clef_rope_qk), RMSNorm+NVFP4 (the MLP block's input norm) and
# SwiGLU+NVFP4. rope_q / rope_k alone are reported under "kernels". The order matters by up to 3 us per step: the
# first kernel of a graph replay starts cold (no overlap with its predecessor), which costs the RoPE kernel least.
STEP_KERNELS = ["rope_qk", "rms_norm_quantise_nvfp4", "swiglu_quantise_nvfp4"]
FULL_KERNELS = ["embed_gather", "rms_norm_quantise_nvfp4", "swiglu_quantise_nvfp4", "rope_qk",
                "rms_norm_gated_quantise_nvfp4"]     # the full fused chain over 130,712 rows
DOMINANT = "swiglu_quantise_nvfp4"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel at 8,192 rows: read from a small
# text file under profiles/ that also records a hash of the kernel sources it was measured on.
TRAFFIC_FILE = ROOT / "profiles" / "swiglu_quantise_nvfp4_8192rows_dram_traffic.txt"
KERNEL_SOURCES = ["kernels_hot.cuh", "nvfp4_codec.cuh", "common.cuh", "f32x2.cuh", "silu_forms.cuh"]


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def kernel_sources_hash() -> str:
    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        h.update((ROOT / "aiis_clef_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def dominant_traffic():
    """(bytes per launch or None, note). The file holds `key: value` lines written from an ncu capture."""
    if not TRAFFIC_FILE.exists():
        return None, "no ncu capture recorded"
    fields = {}
    for line in TRAFFIC_FILE.read_text().splitlines():
        if ":" in line and not line.lstrip().startswith("#"):
            k, v = line.split(":", 1)
            fields[k.strip()] = v.strip()
    try:
        total = int(fields["dram_bytes_read"]) + int(fields["dram_bytes_write"])
    except (KeyError, ValueError):
        return None, "capture file unreadable"
    same = fields.get("kernel_sources_sha256_16") == kernel_sources_hash()
    note = f"ncu capture of {fields.get('captured', '?')}" + ("" if same else "; the kernel sources have changed since that capture")
    return total, note


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [v for v in sm if v > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference kernels on the host cores
# ---------------------------------------------------------------------------------------------------------
def host_inputs(rows: int, seed: int):
    """Seeded synthetic inputs of the step as bf16 bit patterns (numpy)."""
    rng = np.random.default_rng(seed)

    def bf16(a):
        u = np.ascontiguousarray(a, np.float32).view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    x = rng.standard_normal((rows, HIDDEN), dtype=np.float32)
    x[:, rng.choice(HIDDEN, 8, replace=False)] *= 20.0
    return {
        "x": bf16(x), "w": (rng.standard_normal(HIDDEN) * 0.1).astype(np.float32),
        "gate": bf16(rng.standard_normal((rows, INTER), dtype=np.float32)),
        "up": bf16(rng.standard_normal((rows, INTER), dtype=np.float32)),
        "q": bf16(rng.standard_normal((rows, Q_HEADS, HEAD_DIM), dtype=np.float32)),
        "k": bf16(rng.standard_normal((rows, KV_HEADS, HEAD_DIM), dtype=np.float32)),
        "cpos": np.arange(rows, dtype=np.int32),
    }


def cpu_step(orc, inp, cos, sin, rows, threads):
    orc.rms_norm_quantise_nvfp4(inp["x"], inp["w"], rows, HIDDEN, EPS, GS_NORM, nthreads=threads)
    orc.swiglu_quantise_nvfp4(inp["gate"], inp["up"], rows, INTER, GS_SWIGLU, nthreads=threads)
    orc.rope(inp["q"], cos, sin, rows, Q_HEADS, HEAD_DIM, ROTARY, pos_map=inp["cpos"], nthreads=threads)
    orc.rope(inp["k"], cos, sin, rows, KV_HEADS, HEAD_DIM, ROTARY, pos_map=inp["cpos"], nthreads=threads)


def time_cpu(steps: int, warmup: int, budget_s: float = 25.0):
    """rows/s of the CPU restatement (oracle port) with every host thread, on the same 8,192-row step."""
    from oracle import binding as orc

    # every host core this process may use (torchrun exports OMP_NUM_THREADS=1; the oracle takes the count explicitly)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    inp = host_inputs(ROWS, 1234)
    cos, sin = orc.rope_tables(np.arange(ROWS, dtype=np.int32), ROTARY, THETA)
    for _ in range(max(1, min(warmup, 2))):
        cpu_step(orc, inp, cos, sin, ROWS, threads)
    times = []
    t_begin = time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        cpu_step(orc, inp, cos, sin, ROWS, threads)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    per_step = float(np.mean(times))
    return {"value": ROWS / per_step, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{len(times)} step(s) of the full {ROWS}-row chunk (same shapes as the GPU step), "
                      f"C++/OpenMP restatement of the reference kernels, all {threads} host threads"}, per_step, len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu, per_step, done = time_cpu(args.steps, args.warmup, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": min(args.warmup, 2), "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(), "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's host toolchain (Rust) is absent and its kernels are GPU code; this arm times the "
                "CPU restatement of the reference kernels' arithmetic (oracle port) on the host cores",
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {
        "workload": "configs[1]: one 8,192-row chunk per GPU, hidden 2048 bf16: RMSNorm+NVFP4; SwiGLU 2x6144 "
                    "+NVFP4; partial RoPE 16 q / 2 kv heads x 128, rotary 64, theta 1e7, cpos = 0..8191",
        "rows_per_gpu": ROWS, "hidden": HIDDEN, "intermediate": INTER, "activation_storage": "bf16",
        "l2": f"inputs larger than L2: {NSETS} rotating buffer sets of about 0.37 GB each; a kernel timed alone rotates over "
              f"at least {ROTATE_BYTES / 1e6:.0f} MB of its own buffers",
        "launch": "one CUDA graph replay per step (3 kernels in layer order: RoPE q + k, RMSNorm+NVFP4, SwiGLU+NVFP4)",
        "parallelism": "row-range replicas, no collective",
        "timing": f"median of {BATCHES} batches of `steps` replays, CUDA events, max over ranks",
    }


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
class Recorder(dict):
    """A buffer set that remembers which of its tensors a launcher touched."""

    def __init__(self, base):
        super().__init__(base)
        self.used = []

    def __getitem__(self, key):
        if key not in self.used:
            self.used.append(key)
        return super().__getitem__(key)


class Harness:
    """Device buffers, C-ABI launch closures and graph-replayed timing shared by the sections of the GPU arm."""

    def __init__(self, args):
        import ctypes

        import torch
        import torch.distributed as dist

        import aiis_clef_b200 as clef

        self.torch, self.dist, self.clef, self.ctypes = torch, dist, clef, ctypes
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus > 1 and self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={self.world})")
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.lib = clef.load()
        self.dev = clef.Device(self.local_rank)
        self.gen = torch.Generator(device="cuda")
        self.gen.manual_seed(1000 + self.rank)
        self.launches = 0

    # -- small helpers ----------------------------------------------------------------------------------
    def p(self, t):
        return None if t is None else self.ctypes.c_void_p(t.data_ptr())

    def stream(self):
        return self.ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def ok(self, status):
        if status != 0:
            raise RuntimeError(f"C-ABI call failed ({status}): {self.clef.lib.last_error()}")

    def randn_bf16(self, *shape, gen=None):
        t = self.torch
        return t.randn(*shape, device="cuda", generator=gen or self.gen, dtype=t.float32).to(t.bfloat16)

    def u8(self, n):
        return self.torch.empty(n, dtype=self.torch.uint8, device="cuda")

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values: list[float]) -> list[float]:
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(values, device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.cpu().tolist()

    # -- timing -----------------------------------------------------------------------------------------
    def capture(self, launches):
        """One CUDA graph holding `launches` (closures that return a C-ABI status) in order."""
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for fn in launches:
                self.ok(fn())
        return g

    def time_graphs(self, graphs, replays: int, batches: int = BATCHES, sync_ranks: bool = False):
        """Milliseconds per batch of `replays` replays (graphs taken round-robin), one entry per batch."""
        torch = self.torch
        for g in graphs[: max(1, min(len(graphs), 3))]:
            g.replay()
        torch.cuda.synchronize()
        out = []
        for _ in range(batches):
            if sync_ranks:
                self.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(replays):
                graphs[i % len(graphs)].replay()
            e.record()
            if sync_ranks:
                self.barrier()
            else:
                torch.cuda.synchronize()
            out.append(s.elapsed_time(e))
        return out


def make_f32_set(h: Harness, proto: dict):
    """The tensors the F32_BYTES_PER_ROW entry points touch, as f32 activations (the values of `proto` widened)."""
    torch = h.torch
    acts = ("x", "gate", "up", "q", "k", "o", "z", "res", "qg256")
    outs = ("q_out", "k_out", "h", "g_out", "sum", "q256", "gate256")
    d = dict(proto)
    for key in acts:
        d[key] = proto[key].float()
    for key in outs:
        d[key] = torch.empty(proto[key].shape, dtype=torch.float32, device="cuda")
    return d


def make_step_set(h: Harness):
    """One buffer set holding every tensor the timed entry points use at 8,192 rows."""
    torch = h.torch
    rows_padded, pk_h, sc_h = h.clef.nvfp4_sizes(ROWS, HIDDEN, 128)
    _, pk_i, sc_i = h.clef.nvfp4_sizes(ROWS, INTER, 128)
    x = h.randn_bf16(ROWS, HIDDEN)
    x[:, torch.randperm(HIDDEN, device="cuda", generator=h.gen)[:8]] *= 20.0
    bf = torch.bfloat16
    return {
        "x": x, "gate": h.randn_bf16(ROWS, INTER), "up": h.randn_bf16(ROWS, INTER),
        "q": h.randn_bf16(ROWS, Q_HEADS, HEAD_DIM), "k": h.randn_bf16(ROWS, KV_HEADS, HEAD_DIM),
        "o": h.randn_bf16(ROWS * VH, HEAD_DIM), "z": h.randn_bf16(ROWS * VH, HEAD_DIM),
        "ids": torch.randint(0, VOCAB, (ROWS,), device="cuda", generator=h.gen, dtype=torch.int32),
        "pk_h": h.u8(pk_h), "sc_h": h.u8(sc_h), "pk_i": h.u8(pk_i), "sc_i": h.u8(sc_i), "pk_g": h.u8(pk_h), "sc_g": h.u8(sc_h),
        "q_out": torch.empty(ROWS, Q_HEADS, HEAD_DIM, dtype=bf, device="cuda"),
        "k_out": torch.empty(ROWS, KV_HEADS, HEAD_DIM, dtype=bf, device="cuda"),
        "h": torch.empty(ROWS, HIDDEN, dtype=bf, device="cuda"),
        "act_i": torch.empty(ROWS, INTER, dtype=bf, device="cuda"),
        "g_out": torch.empty(ROWS * VH, HEAD_DIM, dtype=bf, device="cuda"),
        "v": h.randn_bf16(ROWS, KV_HEADS, HEAD_DIM), "res": h.randn_bf16(ROWS, HIDDEN),
        "cache_k": torch.empty(ROWS, KV_HEADS, HEAD_DIM, dtype=bf, device="cuda"),
        "cache_v": torch.empty(ROWS, KV_HEADS, HEAD_DIM, dtype=bf, device="cuda"),
        "sum": torch.empty(ROWS, HIDDEN, dtype=bf, device="cuda"),
        "q8_h": h.u8(ROWS * HIDDEN), "q8_i": h.u8(ROWS * INTER),
        "s8": torch.empty(ROWS, dtype=torch.int16, device="cuda"),
        "mixed": h.randn_bf16(ROWS, CONV_DIM), "conv_out": torch.empty(ROWS, CONV_DIM, dtype=bf, device="cuda"),
        "qg256": h.randn_bf16(ROWS, Q_HEADS, 512), "q256": torch.empty(ROWS, Q_HEADS, 256, dtype=bf, device="cuda"),
        "gate256": torch.empty(ROWS, Q_HEADS, 256, dtype=bf, device="cuda"),
        "gdn_ops": h.u8(4 * 32 * ((ROWS + 63) // 64) * 2 * 64 * 128),     # the scan's four operand tensors, back to back
        "gdn_kn": torch.empty(ROWS, 32 * 128, dtype=torch.float32, device="cuda"),
        "gdn_v": torch.empty(ROWS, 32 * 128, dtype=torch.float32, device="cuda"),
    }


def make_launchers(h: Harness, shared: dict, code: int = 0):
    """name -> closure(buffer set) -> C-ABI status, at 8,192 rows; `code` is the activations' dtype (0 bf16, 1 f32)."""
    lib, p, stream = h.lib, h.p, h.stream
    rows_padded = (ROWS + 127) // 128 * 128
    w_norm, w_gated, cos, sin, cpos = (shared[k] for k in ("w_norm", "w_gated", "cos", "sin", "cpos"))
    table = shared["table_f32"] if code else shared["table"]
    w_conv, seq_start, cache_map, w_head, w_head256 = (shared[k] for k in ("w_conv", "seq_start", "cache_map", "w_head", "w_head256"))
    op_bytes = 32 * ((ROWS + 63) // 64) * 2 * 64 * 128

    def ops(d, i):
        return h.ctypes.c_void_p(d["gdn_ops"].data_ptr() + i * op_bytes)

    def gdn_conv_prep(d):
        """The convolution and the scan's operands in one launch."""
        return lib.clef_gdn_conv_prep(stream(), p(d["mixed"]), p(w_conv), p(d["gdn_v"]), ops(d, 0), ops(d, 1), ops(d, 2), ops(d, 3),
                                      p(d["gdn_kn"]), ROWS, CONV_DIM, CONV_K, p(seq_start), None, None, 32, 16, 128, 128 ** -0.5, code)

    return {
        "rms_norm_quantise_nvfp4": lambda d: lib.clef_rms_norm_quantise_nvfp4(
            stream(), p(d["x"]), p(w_norm), p(d["pk_h"]), p(d["sc_h"]), ROWS, HIDDEN, EPS, GS_NORM, 128, 512, code),
        "swiglu_quantise_nvfp4": lambda d: lib.clef_swiglu_quantise_nvfp4(
            stream(), p(d["gate"]), p(d["up"]), p(d["pk_i"]), p(d["sc_i"]), ROWS, INTER, GS_SWIGLU, 128, 512, code),
        "rope_q": lambda d: lib.clef_rope(stream(), p(d["q_out"]), p(d["q"]), p(cos), p(sin), ROWS, Q_HEADS, HEAD_DIM,
                                          ROTARY, None, None, p(cpos), code),
        "rope_qk": lambda d: lib.clef_rope_qk(stream(), p(d["q_out"]), p(d["q"]), Q_HEADS, p(d["k_out"]), p(d["k"]), KV_HEADS,
                                              p(cos), p(sin), ROWS, HEAD_DIM, ROTARY, None, None, p(cpos), code),
        "rope_k": lambda d: lib.clef_rope(stream(), p(d["k_out"]), p(d["k"]), p(cos), p(sin), ROWS, KV_HEADS, HEAD_DIM,
                                          ROTARY, None, None, p(cpos), code),
        "embed_gather": lambda d: lib.clef_embed_gather(stream(), p(table), p(d["ids"]), p(d["h"]), ROWS, HIDDEN, code),
        "embed_rms_norm_quantise_nvfp4": lambda d: lib.clef_embed_rms_norm_quantise_nvfp4(
            stream(), p(table), p(d["ids"]), p(d["h"]), p(w_norm), p(d["pk_g"]), p(d["sc_g"]), ROWS, HIDDEN, EPS, GS_NORM, 128, 512, code),
        "rms_norm_gated_quantise_nvfp4": lambda d: lib.clef_rms_norm_gated_quantise_nvfp4(
            stream(), p(d["o"]), p(d["z"]), p(w_gated), p(d["pk_g"]), p(d["sc_g"]), rows_padded * VH, HEAD_DIM, EPS,
            GS_GATED, 128, 512, VH, ROWS * VH, code),
        "quantise_nvfp4": lambda d: lib.clef_quantise_nvfp4(stream(), p(d["x"]), p(d["pk_g"]), p(d["sc_g"]), ROWS, HIDDEN,
                                                            GS_NORM, 128, 512, code),
        "rms_norm": lambda d: lib.clef_rms_norm(stream(), p(d["x"]), p(w_norm), p(d["h"]), ROWS, HIDDEN, EPS, code),
        "swiglu": lambda d: lib.clef_swiglu(stream(), p(d["gate"]), p(d["up"]), p(d["act_i"]), ROWS * INTER, code),
        "rms_norm_gated": lambda d: lib.clef_rms_norm_gated(stream(), p(d["o"]), p(d["z"]), p(w_gated), p(d["g_out"]),
                                                            ROWS * VH, HEAD_DIM, EPS, code),
        "qk_norm_rope_q": lambda d: lib.clef_qk_norm_rope(stream(), p(d["q"]), p(w_head), p(cos), p(sin), p(d["h"]),
                                                          None, ROWS * Q_HEADS, Q_HEADS, HEAD_DIM, ROTARY, EPS, None,
                                                          None, p(cpos), code),
        "qk_norm_rope_q_hd256_gate": lambda d: lib.clef_qk_norm_rope(
            stream(), p(d["qg256"]), p(w_head256), p(cos), p(sin), p(d["q256"]), p(d["gate256"]), ROWS * Q_HEADS, Q_HEADS, 256,
            ROTARY, EPS, None, None, p(cpos), code),
        "rope_kv_write": lambda d: lib.clef_rope_kv_write(
            stream(), p(d["cache_k"]), p(d["cache_v"]), p(d["k"]), p(d["v"]), p(cos), p(sin), ROWS, KV_HEADS, HEAD_DIM,
            ROTARY, None, None, p(cpos), p(cache_map), None, code),
        "qk_norm_rope_kv_write": lambda d: lib.clef_qk_norm_rope_kv_write(
            stream(), p(d["cache_k"]), p(d["cache_v"]), p(d["k"]), p(d["v"]), p(w_head), p(cos), p(sin), ROWS, KV_HEADS,
            HEAD_DIM, ROTARY, EPS, None, None, p(cpos), p(cache_map), None, code),
        # attention output (q-shaped) gated by a same-shaped gate, as the operand of o_proj
        "sigmoid_mul_quantise_nvfp4": lambda d: lib.clef_sigmoid_mul_quantise_nvfp4(
            stream(), p(d["q"]), p(d["res"]), p(d["pk_g"]), p(d["sc_g"]), ROWS, HIDDEN, GS_NORM, 128, 512, code),
        "sigmoid_mul": lambda d: lib.clef_sigmoid_mul(stream(), p(d["sum"]), p(d["q"]), p(d["res"]), ROWS * HIDDEN, code),
        "add": lambda d: lib.clef_add(stream(), p(d["sum"]), p(d["x"]), p(d["res"]), ROWS * HIDDEN, code),
        "add_rms_norm_quantise_nvfp4": lambda d: lib.clef_add_rms_norm_quantise_nvfp4(
            stream(), p(d["sum"]), p(d["x"]), p(d["res"]), p(w_norm), p(d["pk_g"]), p(d["sc_g"]), ROWS, HIDDEN, EPS,
            GS_NORM, 128, 512, code),
        "quantise_fp8": lambda d: lib.clef_quantise_fp8(stream(), p(d["x"]), p(d["q8_h"]), p(d["s8"]), ROWS, HIDDEN, code),
        "rms_norm_fp8_bf16": lambda d: lib.clef_rms_norm_fp8_bf16(stream(), p(d["x"]), p(w_norm), p(d["q8_h"]), p(d["s8"]),
                                                                  p(d["sum"]), ROWS, HIDDEN, EPS, code),
        "swiglu_quantise_fp8": lambda d: lib.clef_swiglu_quantise_fp8(stream(), p(d["gate"]), p(d["up"]), p(d["q8_i"]),
                                                                      p(d["s8"]), ROWS, INTER, code),
        "rms_norm_gated_quantise_fp8": lambda d: lib.clef_rms_norm_gated_quantise_fp8(
            stream(), p(d["o"]), p(d["z"]), p(w_gated), p(d["q8_h"]), p(d["s8"]), ROWS * VH, HEAD_DIM, EPS, VH, ROWS * VH, code),
        "gdn_prep": lambda d: lib.clef_gdn_prep(stream(), p(d["mixed"]), p(d["gdn_v"]), ops(d, 0), ops(d, 1), ops(d, 2),
                                                ops(d, 3), p(d["gdn_kn"]), ROWS, 32, 16, 128, CONV_DIM, 128 ** -0.5, code),
        "causal_conv_silu": lambda d: lib.clef_causal_conv_silu(stream(), p(d["conv_out"]), p(d["mixed"]), p(w_conv), ROWS,
                                                                CONV_DIM, CONV_K, p(seq_start), None, None, code),
        "gdn_conv_prep": gdn_conv_prep,
    }


def make_shared(h: Harness):
    torch = h.torch
    cpos = torch.arange(ROWS, dtype=torch.int32, device="cuda")
    cos, sin = h.dev.rope_tables_dev(cpos, ROWS, ROTARY, THETA)
    return {
        "w_norm": (torch.randn(HIDDEN, device="cuda", generator=h.gen) * 0.1).contiguous(),
        "w_gated": (1.0 + torch.randn(HEAD_DIM, device="cuda", generator=h.gen) * 0.1).contiguous(),
        "cpos": cpos, "cos": cos, "sin": sin,
        "table": h.randn_bf16(VOCAB, HIDDEN) * 0.02,
        "w_conv": (torch.randn(CONV_DIM, CONV_K, device="cuda", generator=h.gen) * 0.5).contiguous(),
        "seq_start": torch.zeros(ROWS, dtype=torch.int32, device="cuda"),
        "cache_map": torch.randperm(ROWS, device="cuda", generator=h.gen).to(torch.int32),   # the engine's cpos: a slot per token
        "w_head": (torch.randn(HEAD_DIM, device="cuda", generator=h.gen) * 0.1).contiguous(),
        "w_head256": (torch.randn(256, device="cuda", generator=h.gen) * 0.1).contiguous(),
    }


def time_each_kernel(h: Harness, launchers, proto, steps: int, bytes_per_row=None):
    """ms per launch of every entry point alone: a graph of launches that rotates over `sets` private copies of the
    tensors the entry point touches (at least ROTATE_BYTES of them, so neither reads nor writes are served by L2)."""
    torch = h.torch
    out, sets_used = {}, {}
    bytes_per_row = bytes_per_row or BYTES_PER_ROW
    for name, fn in launchers.items():
        if name not in bytes_per_row:
            continue
        rec = Recorder(proto)
        h.ok(fn(rec))
        torch.cuda.synchronize()
        per_set = bytes_per_row[name] * ROWS
        nsets = int(min(160, max(4, math.ceil(ROTATE_BYTES / per_set))))
        sets = [proto]
        for i in range(1, nsets):
            d = dict(proto)
            for key in rec.used:
                t = proto[key]
                if key == "ids":      # other token ids per set, so that the gathered table rows differ from launch to launch
                    d[key] = torch.randint(0, VOCAB, t.shape, device="cuda", generator=h.gen, dtype=torch.int32)
                else:
                    d[key] = t.roll(i * 131, 0) if t.dim() > 1 else torch.empty_like(t)
            sets.append(d)
        per_graph = nsets * max(1, -(-12 // nsets))
        graph = h.capture([(lambda d=sets[i % nsets]: fn(d)) for i in range(per_graph)])
        replays = max(2, -(-max(steps, 24) // per_graph))
        ms = h.time_graphs([graph], replays)
        out[name] = float(np.median(ms)) / (replays * per_graph)
        sets_used[name] = nsets
        del graph, sets
    return out, sets_used


def run_gpu_arm(args):
    h = Harness(args)
    torch, clef, lib, p = h.torch, h.clef, h.lib, h.p
    shared = make_shared(h)
    launchers = make_launchers(h, shared)
    sets = [make_step_set(h) for _ in range(NSETS)]

    def step(d):
        for name in STEP_KERNELS:
            h.ok(launchers[name](d))

    # One CUDA graph per buffer set: the reference replays one graph per pass geometry.
    for d in sets:
        step(d)
    torch.cuda.synchronize()
    graphs = []
    for d in sets:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step(d)
        graphs.append(g)

    sampler = ClockSampler(h.local_rank) if h.rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.5)          # let nvidia-smi come up: the timed region is only tens of milliseconds long
    for i in range(args.warmup):
        graphs[i % NSETS].replay()
    batch_ms = h.time_graphs(graphs, args.steps, BATCHES, sync_ranks=True)
    batch_ms = h.max_over_ranks(batch_ms)
    elapsed_ms = float(np.median(batch_ms))

    kernel_ms, kernel_sets = time_each_kernel(h, launchers, sets[0], args.steps)
    clocks = sampler.stop() if sampler else None

    e2e = end_to_end(h, args, sets[0], shared)
    full = full_pass(h, shared)
    extras = other_configurations(h, shared, launchers, sets) if h.world == 1 else None

    names = list(launchers)
    flat = [e2e["ms_total"]] + [kernel_ms[k] for k in names] + [full["chain_ms"]] + [full["kernel_ms"][k] for k in FULL_KERNELS] \
        + [full["alt_chain_ms"]]
    flat = h.max_over_ranks(flat)
    e2e_ms = flat[0]
    kernel_ms = dict(zip(names, flat[1:1 + len(names)]))
    rest = flat[1 + len(names):]
    full["chain_ms"], full["alt_chain_ms"] = rest[0], rest[-1]
    full["kernel_ms"] = dict(zip(FULL_KERNELS, rest[1:1 + len(FULL_KERNELS)]))

    if h.rank == 0:
        peak, peak_kind = measured_peak_gbs()
        ms_per_step = elapsed_ms / args.steps
        value = h.world * ROWS * args.steps / (elapsed_ms * 1e-3)
        kernels = {}
        for name, ms in kernel_ms.items():
            gbs = BYTES_PER_ROW[name] * ROWS / (ms * 1e-3) / 1e9
            kernels[name] = {"us": round(ms * 1e3, 2), "rows_per_s": ROWS / (ms * 1e-3), "GBs": round(gbs, 1),
                             "frac_of_measured_peak": round(gbs / peak, 4), "frac_of_8TBs": round(gbs / 8000.0, 4),
                             "bytes_per_row": BYTES_PER_ROW[name], "sets": kernel_sets[name],
                             "l2_defeated": bool(kernel_sets[name] * BYTES_PER_ROW[name] * ROWS >= 3 * 126e6)}
        dom = kernels[DOMINANT]
        traffic, traffic_note = dominant_traffic()
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": h.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(),
            "batches_ms_per_step": {"median": ms_per_step, "min": min(batch_ms) / args.steps, "max": max(batch_ms) / args.steps,
                                    "n": len(batch_ms)},
            "roofline": {"bound": "hbm", "kernel": DOMINANT, "achieved": dom["GBs"], "peak": peak, "unit": "GB/s",
                         "frac": round(dom["GBs"] / peak, 4), "peak_kind": f"of {peak_kind}",
                         "traffic": traffic, "traffic_source": traffic_note,
                         "algorithmic_bytes_per_launch": BYTES_PER_ROW[DOMINANT] * ROWS},
            "e2e": {"value": h.world * ROWS * e2e["steps"] / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": e2e["h2d"],
                    "d2h_bytes_per_step": e2e["d2h"], "steps": e2e["steps"], "outputs_equal_device_path": e2e["equal"],
                    "outputs_compared": e2e["compared"],
                    "api": "clef_host_* (host-slice C-ABI, pinned host buffers, two-stream row tiles, pipelined mode: "
                           "one clef_device_synchronize per step)"},
            "gpu_launches": len(STEP_KERNELS) * args.steps * BATCHES,
            "gpu_launches_note": f"{len(STEP_KERNELS)} kernels x {args.steps} steps x {BATCHES} timed batches",
            "clocks": clocks,
            "kernels": kernels,
            "step_GBs": round(sum(BYTES_PER_ROW[k] for k in STEP_KERNELS) * ROWS / (ms_per_step * 1e-3) / 1e9, 1),
            "step_frac_of_measured_peak": round(sum(BYTES_PER_ROW[k] for k in STEP_KERNELS) * ROWS / (ms_per_step * 1e-3) / 1e9 / peak, 4),
            "full_pass_130712_rows": summarise_full(full, h.world, peak),
        }
        if extras is not None:
            line["other_configurations"] = summarise_extras(extras, peak)
        if h.world == 1:
            cpu, _, _ = time_cpu(3, 1, budget_s=20.0)
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if h.world > 1:
        h.dist.barrier()
        h.dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------
# end to end: host buffers in, host buffers out, through the host-slice C-ABI
# ---------------------------------------------------------------------------------------------------------
def end_to_end(h: Harness, args, d0, shared):
    torch, clef = h.torch, h.clef
    _, pk_h, sc_h = clef.nvfp4_sizes(ROWS, HIDDEN, 128)
    _, pk_i, sc_i = clef.nvfp4_sizes(ROWS, INTER, 128)
    hd = clef.HostDevice(h.local_rank)
    host = {k: d0[k].cpu().pin_memory() for k in ("x", "gate", "up", "q", "k")}
    host["cpos"] = shared["cpos"].cpu().pin_memory()
    host_w = shared["w_norm"].cpu().numpy()
    host_cos, host_sin = shared["cos"].cpu().pin_memory(), shared["sin"].cpu().pin_memory()
    out = {
        "pk_h": torch.empty(pk_h, dtype=torch.uint8).pin_memory(), "sc_h": torch.empty(sc_h, dtype=torch.uint8).pin_memory(),
        "pk_i": torch.empty(pk_i, dtype=torch.uint8).pin_memory(), "sc_i": torch.empty(sc_i, dtype=torch.uint8).pin_memory(),
        "q": torch.empty_like(host["q"]).pin_memory(), "k": torch.empty_like(host["k"]).pin_memory(),
    }

    def e2e_step():
        hd.rms_norm_quantise_nvfp4(host["x"], host_w, out["pk_h"], out["sc_h"], ROWS, HIDDEN, EPS, GS_NORM)
        hd.swiglu_quantise_nvfp4(host["gate"], host["up"], out["pk_i"], out["sc_i"], ROWS, INTER, GS_SWIGLU)
        hd.rope(out["q"], host["q"], host_cos, host_sin, ROWS, ROWS, Q_HEADS, HEAD_DIM, ROTARY, host["cpos"])
        hd.rope(out["k"], host["k"], host_cos, host_sin, ROWS, ROWS, KV_HEADS, HEAD_DIM, ROTARY, host["cpos"])
        hd.synchronize()     # every output of the step is in host memory from here on

    # Pipelined host-slice mode: the four calls of a step are enqueued back to back (uploads of one call run under
    # the downloads of the previous one) and the step ends with one synchronisation.
    hd.set_pipelined(True)
    h2d = sum(host[k].numel() * host[k].element_size() for k in ("x", "gate", "up", "q", "k")) + 2 * host["cpos"].numel() * 4 \
        + host_w.nbytes + 2 * 2 * host_cos.numel() * 4
    d2h = sum(t.numel() * t.element_size() for t in out.values())
    steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    h.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    # every output of the end-to-end step is the device path's output
    pairs = [("pk_h", "pk_h"), ("sc_h", "sc_h"), ("pk_i", "pk_i"), ("sc_i", "sc_i"), ("q", "q_out"), ("k", "k_out")]
    equal = all(bool(torch.equal(out[a], d0[b].cpu())) for a, b in pairs)
    hd.close()
    return {"ms_total": seconds * 1e3, "steps": steps, "h2d": int(h2d), "d2h": int(d2h), "equal": equal, "compared": len(pairs)}


# ---------------------------------------------------------------------------------------------------------
# the 130,712-row pass, row-range sharded over the ranks (strong scaling)
# ---------------------------------------------------------------------------------------------------------
def checksum(torch, t):
    """Two 64-bit wrap-around sums over the bytes of a tensor (length a multiple of 8): plain and position-weighted."""
    w = t.reshape(-1).view(torch.uint8).view(torch.int64)
    idx = torch.arange(1, w.numel() + 1, device=w.device, dtype=torch.int64)
    return [int(w.sum().item()), int((w * (2 * idx + 1)).sum().item())]


def full_pass_inputs(h: Harness, first: int, n: int):
    """This rank's row range of the identically seeded 130,712-row inputs (every rank draws the same full tensors)."""
    torch = h.torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(424242)

    def rows_of(*shape):
        full = h.randn_bf16(FULL_ROWS, *shape, gen=gen)
        part = full[first:first + n].contiguous()
        del full
        return part

    x = rows_of(HIDDEN)
    gate, up = rows_of(INTER), rows_of(INTER)
    q, k = rows_of(Q_HEADS, HEAD_DIM), rows_of(KV_HEADS, HEAD_DIM)
    o, z = rows_of(VH, HEAD_DIM), rows_of(VH, HEAD_DIM)
    ids = torch.randint(0, VOCAB, (FULL_ROWS,), device="cuda", generator=gen, dtype=torch.int32)[first:first + n].contiguous()
    return {"x": x, "gate": gate, "up": up, "q": q, "k": k, "o": o.view(n * VH, HEAD_DIM), "z": z.view(n * VH, HEAD_DIM), "ids": ids}


def full_pass_outputs(h: Harness, n: int):
    torch, clef = h.torch, h.clef
    _, pk_h, sc_h = clef.nvfp4_sizes(n, HIDDEN, 128)
    _, pk_i, sc_i = clef.nvfp4_sizes(n, INTER, 128)
    bf = torch.bfloat16
    return {"pkh": h.u8(pk_h), "sch": h.u8(sc_h), "pki": h.u8(pk_i), "sci": h.u8(sc_i), "pkg": h.u8(pk_h), "scg": h.u8(sc_h),
            "pke": h.u8(pk_h), "sce": h.u8(sc_h),
            "qo": torch.empty(n, Q_HEADS, HEAD_DIM, dtype=bf, device="cuda"), "ko": torch.empty(n, KV_HEADS, HEAD_DIM, dtype=bf, device="cuda"),
            "h": torch.empty(n, HIDDEN, dtype=bf, device="cuda")}


def full_pass_calls(h: Harness, shared, tables, inp, out, n: int, first: int):
    lib, p, stream = h.lib, h.p, h.stream
    rp = (n + 127) // 128 * 128
    cos, sin, positions = tables
    cpos = positions[first:first + n]
    w_norm, table = shared["w_norm"], shared["table"]
    w_gated = shared["w_gated"]
    return {
        "embed_gather": lambda: lib.clef_embed_gather(stream(), p(table), p(inp["ids"]), p(out["h"]), n, HIDDEN, 0),
        "rms_norm_quantise_nvfp4": lambda: lib.clef_rms_norm_quantise_nvfp4(stream(), p(inp["x"]), p(w_norm), p(out["pkh"]), p(out["sch"]), n,
                                                                             HIDDEN, EPS, GS_NORM, 128, 512, 0),
        "swiglu_quantise_nvfp4": lambda: lib.clef_swiglu_quantise_nvfp4(stream(), p(inp["gate"]), p(inp["up"]), p(out["pki"]), p(out["sci"]), n,
                                                                         INTER, GS_SWIGLU, 128, 512, 0),
        "rope_qk": lambda: lib.clef_rope_qk(stream(), p(out["qo"]), p(inp["q"]), Q_HEADS, p(out["ko"]), p(inp["k"]), KV_HEADS, p(cos), p(sin), n,
                                            HEAD_DIM, ROTARY, None, None, p(cpos), 0),
        "rms_norm_gated_quantise_nvfp4": lambda: lib.clef_rms_norm_gated_quantise_nvfp4(
            stream(), p(inp["o"]), p(inp["z"]), p(w_gated), p(out["pkg"]), p(out["scg"]), rp * VH, HEAD_DIM, EPS, GS_GATED, 128, 512, VH,
            n * VH, 0),
        # alternative head of the chain: gather + norm + quantiser of the gathered rows in one pass (its own outputs)
        "embed_rms_norm_quantise_nvfp4": lambda: lib.clef_embed_rms_norm_quantise_nvfp4(
            stream(), p(table), p(inp["ids"]), p(out["h"]), p(w_norm), p(out["pke"]), p(out["sce"]), n, HIDDEN, EPS, GS_NORM, 128, 512, 0),
    }


def shard_checksums(h: Harness, out, first_row: int, n: int, base_row: int):
    """Checksums of the rows [first_row, first_row + n) of a pass whose buffers start at row `base_row` (both multiples
    of the 128-row scale atom, except the ragged end): packed and scale slices are contiguous per atom-aligned range."""
    torch = h.torch
    lo = first_row - base_row
    rp = (n + 127) // 128 * 128
    sums = []
    for pk, sc, cols in (("pkh", "sch", HIDDEN), ("pki", "sci", INTER), ("pkg", "scg", HIDDEN)):
        sums += checksum(torch, out[pk][lo * cols // 2:(lo + rp) * cols // 2])
        sums += checksum(torch, out[sc][lo * cols // 16:(lo + rp) * cols // 16])
    for name in ("qo", "ko", "h"):
        sums += checksum(torch, out[name][lo:lo + n])
    return sums


def full_pass(h: Harness, shared):
    """The five fused kernels over this rank's row range of the 130,712-row pass as ONE CUDA graph (programmatic
    dependent launch between its kernels), replayed over rotating buffer sets; plus each kernel alone, and the
    comparison of every shard's bytes with a single-GPU run of the same seeded inputs."""
    torch, clef = h.torch, h.clef
    first, n = clef.shard_rows(FULL_ROWS, 128, h.world, h.rank)
    positions = torch.arange(FULL_ROWS, dtype=torch.int32, device="cuda")
    cos, sin = h.dev.rope_tables_dev(positions, FULL_ROWS, ROTARY, THETA)   # one request of 130,712 tokens at slot 0
    tables = (cos, sin, positions)
    # the replicated operands of the pass (norm weights, embedding table) are the same on every rank
    wgen = torch.Generator(device="cuda")
    wgen.manual_seed(515151)
    shared = dict(shared)
    shared["w_norm"] = (torch.randn(HIDDEN, device="cuda", generator=wgen) * 0.1).contiguous()
    shared["w_gated"] = (1.0 + torch.randn(HEAD_DIM, device="cuda", generator=wgen) * 0.1).contiguous()
    shared["table"] = h.randn_bf16(VOCAB, HIDDEN, gen=wgen) * 0.02
    inp = full_pass_inputs(h, first, n)
    per_set = sum(BYTES_PER_ROW[k] for k in FULL_KERNELS) * n
    nsets = int(max(1, min(4, math.ceil(2e9 / per_set))))      # 1 set of 7.9 GB on one GPU, 3 sets of 1 GB each on eight
    in_sets = [inp] + [{k: (v.roll(7 * i, 0) if v.dtype != torch.int32 else v.clone()) for k, v in inp.items()} for i in range(1, nsets)]
    out_sets = [full_pass_outputs(h, n) for _ in range(nsets)]
    calls = [full_pass_calls(h, shared, tables, in_sets[i], out_sets[i], n, first) for i in range(nsets)]
    for c in calls:
        for name in FULL_KERNELS:
            h.ok(c[name]())
    torch.cuda.synchronize()
    sums = shard_checksums(h, out_sets[0], first, n, first)     # before anything overwrites set 0's outputs

    chain = [h.capture([c[name] for name in FULL_KERNELS]) for c in calls]
    replays = max(20, 4 * nsets)
    chain_ms = float(np.median(h.time_graphs(chain, replays, BATCHES, sync_ranks=True))) / replays
    alt_names = ["embed_rms_norm_quantise_nvfp4"] + [k for k in FULL_KERNELS if k not in ("embed_gather", "rms_norm_quantise_nvfp4")]
    alt = [h.capture([c[name] for name in alt_names]) for c in calls]
    alt_chain_ms = float(np.median(h.time_graphs(alt, replays, BATCHES, sync_ranks=True))) / replays
    kernel_ms = {}
    for name in FULL_KERNELS:
        per = max(1, min(6, int(ROTATE_BYTES // max(1, BYTES_PER_ROW[name] * n)) + 1))
        g = [h.capture([c[name]]) for c in calls]
        reps = max(10, 2 * per * nsets)
        kernel_ms[name] = float(np.median(h.time_graphs(g, reps))) / reps
        del g
    del chain, alt

    # every shard's bytes against a single-GPU run of the same inputs (rank 0 runs the whole pass once more)
    equal = None
    if h.world > 1:
        mine = torch.tensor(sums, device="cuda", dtype=torch.int64)
        gathered = [torch.empty_like(mine) for _ in range(h.world)]
        h.dist.all_gather(gathered, mine)
        if h.rank == 0:
            del in_sets, out_sets, calls
            torch.cuda.empty_cache()
            whole_in = full_pass_inputs(h, 0, FULL_ROWS)
            whole_out = full_pass_outputs(h, FULL_ROWS)
            whole = full_pass_calls(h, shared, tables, whole_in, whole_out, FULL_ROWS, 0)
            for name in FULL_KERNELS:
                h.ok(whole[name]())
            torch.cuda.synchronize()
            equal = True
            for r in range(h.world):
                f, m = clef.shard_rows(FULL_ROWS, 128, h.world, r)
                equal = equal and (shard_checksums(h, whole_out, f, m, 0) == gathered[r].cpu().tolist())
            del whole_in, whole_out
    return {"chain_ms": chain_ms, "alt_chain_ms": alt_chain_ms, "kernel_ms": kernel_ms, "rows_this_rank": n, "sets": nsets,
            "replays": replays, "shards_equal_single_gpu": equal}


def summarise_full(full, world, peak):
    chain_ms = full["chain_ms"]
    total_bytes = sum(BYTES_PER_ROW[k] for k in FULL_KERNELS) * FULL_ROWS
    alt_bytes = total_bytes - (BYTES_PER_ROW["embed_gather"] + BYTES_PER_ROW["rms_norm_quantise_nvfp4"] -
                               BYTES_PER_ROW["embed_rms_norm_quantise_nvfp4"]) * FULL_ROWS
    per_kernel = {k: {"ms": round(v, 4), "GBs_per_gpu": round(BYTES_PER_ROW[k] * FULL_ROWS / world / (v * 1e-3) / 1e9, 1)}
                  for k, v in full["kernel_ms"].items()}
    return {"n_gpus": world, "scaling": "strong (row-range shards aligned to the 128-row scale atom, max over ranks)",
            "chain_ms": round(chain_ms, 4), "chain": "the five kernels of a rank's shard as one CUDA graph, timed as a whole "
            f"({full['replays']} replays per batch over {full['sets']} rotating buffer set(s), median of {BATCHES} batches)",
            "rows_per_s": FULL_ROWS / (chain_ms * 1e-3),
            "GBs_aggregate": round(total_bytes / (chain_ms * 1e-3) / 1e9, 1),
            "frac_of_measured_peak_per_gpu": round(total_bytes / (chain_ms * 1e-3) / 1e9 / world / peak, 4),
            "sum_of_kernels_timed_alone_ms": round(sum(full["kernel_ms"].values()), 4),
            "kernels_timed_alone": per_kernel,
            "chain_with_fused_embed_norm_ms": round(full["alt_chain_ms"], 4),
            "chain_with_fused_embed_norm_GBs_aggregate": round(alt_bytes / (full["alt_chain_ms"] * 1e-3) / 1e9, 1),
            "shards_equal_single_gpu": full["shards_equal_single_gpu"],
            "l2": "every rank's chain touches far more than L2 per replay (60,296 B per row) and rotates over buffer sets"}


# ---------------------------------------------------------------------------------------------------------
# the benchmark definition's other configurations (one GPU)
# ---------------------------------------------------------------------------------------------------------
def other_configurations(h: Harness, shared, launchers, sets):
    torch, clef, lib, p, stream = h.torch, h.clef, h.lib, h.p, h.stream
    out = {}
    # -- the gated chain: 32,768 tokens in four 8,192-token chunks (one graph replay per chunk), two requests rotating
    gated_sets = [dict(sets[i % NSETS]) for i in range(8)]
    for i in range(NSETS, 8):
        for key in ("o", "z", "pk_g", "sc_g"):
            gated_sets[i][key] = sets[i % NSETS][key].roll(17 * i, 0) if key in ("o", "z") else torch.empty_like(sets[0][key])
    graphs = [h.capture([lambda d=d: launchers["rms_norm_gated_quantise_nvfp4"](d)]) for d in gated_sets]
    ms = float(np.median(h.time_graphs(graphs, 40))) / 40
    out["gated_chain_4x8192"] = {"ms_per_chunk": ms, "bytes_per_chunk": BYTES_PER_ROW["rms_norm_gated_quantise_nvfp4"] * ROWS}
    del graphs, gated_sets

    # -- the 130,712-row pass the way the reference cuts it: rung-sized passes, one graph per pass
    cuts = clef.rungs_decompose(FULL_ROWS)
    padded = cuts[-1][0] + cuts[-1][1]
    positions = torch.arange(padded, dtype=torch.int32, device="cuda")
    cos, sin = h.dev.rope_tables_dev(positions, padded, ROTARY, THETA)
    inp = full_pass_inputs(h, 0, FULL_ROWS)
    pad = padded - FULL_ROWS
    if pad:   # the last pass is padded to its rung (64-row granule), as the engine pads it
        inp = {k: torch.cat([v, v[:pad * (VH if k in ("o", "z") else 1)]]) for k, v in inp.items()}
    passes = []
    for base, rows in cuts:
        sl = {k: v[base * (VH if k in ("o", "z") else 1):(base + rows) * (VH if k in ("o", "z") else 1)] for k, v in inp.items()}
        # output slices of a pass: rows are multiples of 64; scale tiles are 128-row atoms, so each pass owns buffers of its own
        o = full_pass_outputs(h, rows)
        calls = full_pass_calls(h, shared, (cos, sin, positions), sl, o, rows, base)
        passes.append((h.capture([calls[name] for name in FULL_KERNELS]), o))
    graphs = [g for g, _ in passes]
    ms = float(np.median(h.time_graphs(graphs, len(graphs) * 3))) / 3
    out["full_pass_as_rung_passes"] = {"ms": ms, "passes": len(cuts), "rungs": sorted({r for _, r in cuts}, reverse=True), "rows": padded}
    del passes, graphs, inp

    # -- rung sweep: four coalesced requests per pass, per-token maps uploaded before every replay
    rng = np.random.default_rng(0xED)
    table_rows = 16384
    positions = torch.arange(table_rows, dtype=torch.int32, device="cuda")
    cos, sin = h.dev.rope_tables_dev(positions, table_rows, ROTARY, THETA)
    sweep = {}
    pool_rows = NSETS * ROWS
    for rung in (64, 128, 256, 512, 1024, 2048, 4096, 8192):
        gran = rung // 64
        nreq = min(4, gran)
        cuts_g = np.sort(rng.choice(np.arange(1, gran), nreq - 1, replace=False)) if nreq > 1 else np.zeros(0, np.int64)
        sizes = np.diff(np.concatenate([[0], cuts_g, [gran]])) * 64
        chunks = []
        for slot, s in enumerate(sizes):       # a request that already holds `start` tokens in its cache slot continues by s rows
            start = int(rng.integers(0, (8192 - int(s)) // 64 + 1)) * 64
            chunks.append((rng.integers(0, VOCAB, start + int(s)).astype(np.uint32), start, slot, int(s)))
        maps = clef.pass_maps(chunks, 8192)
        # the pass's seven per-token maps travel as one pinned block, as the engine uploads them before a replay
        names7 = ("ids", "seq_start", "seq_end", "cpos", "cbase", "slot_map", "rope_pos")
        host_maps = torch.from_numpy(np.stack([maps[k].astype(np.int32) for k in names7])).pin_memory()
        dev_maps = torch.empty(7, rung, dtype=torch.int32, device="cuda")
        dev_pos = dev_maps[6]
        rp = (rung + 127) // 128 * 128
        slices = min(pool_rows // rp, 256)
        launches = []
        for i in range(slices):
            d = sets[(i * rp // ROWS) % NSETS]
            r0 = (i * rp) % ROWS
            if r0 + rp > ROWS:
                continue
            view = {k: d[k][r0:r0 + rung] for k in ("x", "gate", "up", "q", "k")}
            o = {"pk_h": d["pk_h"][r0 * HIDDEN // 2:], "sc_h": d["sc_h"][r0 * HIDDEN // 16:], "pk_i": d["pk_i"][r0 * INTER // 2:],
                 "sc_i": d["sc_i"][r0 * INTER // 16:], "q_out": d["q_out"][r0:], "k_out": d["k_out"][r0:]}
            launches.append(lambda v=view, o=o: lib.clef_rope_qk(
                stream(), p(o["q_out"]), p(v["q"]), Q_HEADS, p(o["k_out"]), p(v["k"]), KV_HEADS, p(cos), p(sin), rung, HEAD_DIM, ROTARY,
                None, None, p(dev_pos), 0))
            launches.append(lambda v=view, o=o: lib.clef_rms_norm_quantise_nvfp4(
                stream(), p(v["x"]), p(shared["w_norm"]), p(o["pk_h"]), p(o["sc_h"]), rung, HIDDEN, EPS, GS_NORM, 128, 512, 0))
            launches.append(lambda v=view, o=o: lib.clef_swiglu_quantise_nvfp4(
                stream(), p(v["gate"]), p(v["up"]), p(o["pk_i"]), p(o["sc_i"]), rung, INTER, GS_SWIGLU, 128, 512, 0))
        per_pass = [h.capture(launches[3 * i:3 * i + 3]) for i in range(len(launches) // 3)]
        dev_maps.copy_(host_maps, non_blocking=True)
        for g in per_pass[:3]:
            g.replay()
        torch.cuda.synchronize()
        times = []
        n_pass = max(len(per_pass), 24)
        for _ in range(BATCHES):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(n_pass):
                dev_maps.copy_(host_maps, non_blocking=True)    # the pass's maps go up before its graph is replayed
                per_pass[i % len(per_pass)].replay()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) / n_pass)
        sweep[rung] = {"us_per_pass": float(np.median(times)) * 1e3, "requests": nreq, "slices": len(per_pass)}
        del per_pass, launches
    out["rung_sweep"] = sweep

    # -- f32 activations (the reference engine's residual-stream type): the same entry points, each alone as above
    shared32 = dict(shared)
    shared32["table_f32"] = shared["table"].float()
    proto32 = make_f32_set(h, sets[0])
    ms32, sets32 = time_each_kernel(h, make_launchers(h, shared32, code=1), proto32, 24, F32_BYTES_PER_ROW)
    out["f32_activations"] = {"ms": ms32, "sets": sets32}
    # the step itself on f32 activations: the three kernels in layer order, one graph per rotating buffer set
    launch32 = make_launchers(h, shared32, code=1)
    sets_f32 = [proto32] + [make_f32_set(h, sets[i]) for i in (1, 2)]
    graphs = [h.capture([lambda d=d, n=n: launch32[n](d) for n in STEP_KERNELS]) for d in sets_f32]
    out["f32_step_ms"] = float(np.median(h.time_graphs(graphs, 60))) / 60
    del graphs, sets_f32, proto32, shared32
    return out


def summarise_extras(extras, peak):
    step_bytes = sum(BYTES_PER_ROW[k] for k in STEP_KERNELS)
    g = extras["gated_chain_4x8192"]
    gbs = g["bytes_per_chunk"] / (g["ms_per_chunk"] * 1e-3) / 1e9
    r = extras["full_pass_as_rung_passes"]
    total = sum(BYTES_PER_ROW[k] for k in FULL_KERNELS) * r["rows"]
    sweep = {}
    for rung, v in extras["rung_sweep"].items():
        gb = step_bytes * rung / (v["us_per_pass"] * 1e-6) / 1e9
        sweep[str(rung)] = {"us_per_pass": round(v["us_per_pass"], 2), "rows_per_s": rung / (v["us_per_pass"] * 1e-6), "GBs": round(gb, 1),
                            "frac_of_measured_peak": round(gb / peak, 4), "requests": v["requests"]}
    f32 = {}
    for name, ms in extras["f32_activations"]["ms"].items():
        gb = F32_BYTES_PER_ROW[name] * ROWS / (ms * 1e-3) / 1e9
        f32[name] = {"us": round(ms * 1e3, 2), "GBs": round(gb, 1), "frac_of_measured_peak": round(gb / peak, 4),
                     "bytes_per_row": F32_BYTES_PER_ROW[name], "sets": extras["f32_activations"]["sets"][name]}
    f32_step_bytes = sum(F32_BYTES_PER_ROW[k] for k in STEP_KERNELS) * ROWS
    f32_step_gbs = f32_step_bytes / (extras["f32_step_ms"] * 1e-3) / 1e9
    return {
        "f32_activation_kernels_8192_rows": f32,
        "f32_activation_step_8192_rows": {
            "us_per_step": round(extras["f32_step_ms"] * 1e3, 2), "rows_per_s": ROWS / (extras["f32_step_ms"] * 1e-3),
            "GBs": round(f32_step_gbs, 1), "frac_of_measured_peak": round(f32_step_gbs / peak, 4), "bytes_per_step": f32_step_bytes,
            "note": "the headline step's three launches on f32 activations (the reference engine's own type), one graph per "
                    "rotating buffer set, median of 5 batches of 60 replays"},
        "gated_chain_32768_rows_in_four_chunks": {
            "us_per_8192_row_chunk": round(g["ms_per_chunk"] * 1e3, 2), "ms_per_32768_rows": round(4 * g["ms_per_chunk"], 4),
            "rows_per_s": ROWS / (g["ms_per_chunk"] * 1e-3), "GBs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4)},
        "full_pass_130712_rows_as_rung_passes": {
            "ms": round(r["ms"], 4), "passes": r["passes"], "rungs": r["rungs"], "rows_incl_padding": r["rows"],
            "rows_per_s": FULL_ROWS / (r["ms"] * 1e-3), "GBs": round(total / (r["ms"] * 1e-3) / 1e9, 1),
            "frac_of_measured_peak": round(total / (r["ms"] * 1e-3) / 1e9 / peak, 4),
            "note": "one CUDA graph of the five kernels per pass (src/gpu.rs:762-775 cuts the request into rungs)"},
        "rung_sweep_step_with_four_coalesced_requests": sweep,
    }


# ---------------------------------------------------------------------------------------------------------
# --profile-case: a small, self-ending run for ncu
# ---------------------------------------------------------------------------------------------------------
def run_profile_case(args):
    """Launch each named entry point three times at 8,192 rows on fresh buffers and exit: the case ncu captures are
    taken on, one kernel per ncu call (`-k regex:<kernel> -s 1 -c 1`; see profiles/)."""
    h = Harness(args)
    shared = make_shared(h)
    launchers = make_launchers(h, shared)
    names = [n for n in args.profile_case.split(",") if n]
    unknown = [n for n in names if n not in launchers]
    if unknown:
        raise SystemExit(f"unknown entry point(s) {unknown}; known: {sorted(launchers)}")
    for _ in range(3):
        d = make_step_set(h)          # fresh inputs: nothing of them is in L2 when the kernel starts
        for n in names:
            h.ok(launchers[n](d))
        h.torch.cuda.synchronize()
    print(json.dumps({"profile_case": "ok", "rows": ROWS, "entry_points": names, "launches_each": 3}))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--profile-case", default="",
                    help="comma-separated entry points: launch each three times at 8,192 rows and exit (for ncu)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
