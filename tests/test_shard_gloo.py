"""The multi-GPU path on CPU: two gloo ranks shard one pass by row range (clef_shard_rows), each
runs its slice, and the concatenation of the shard outputs equals the single-rank result byte for
byte. The per-rank compute is the CPU oracle here (no GPU in this test); what is under test is the
host logic the GPU ranks use: the split, the slice offsets of every operand and the tiled scale
layout staying contiguous per shard."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
ROWS, COLS = 1000, 512


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((ROWS, COLS)).astype(np.float32)
    w = (rng.standard_normal(COLS) * 0.1).astype(np.float32)
    return x, w


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, os.fspath(ROOT))
    sys.path.insert(0, os.fspath(ROOT / "tests"))
    import aiis_clef_b200 as clef
    from oracle import binding as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, w = _inputs()
    first, count = clef.shard_rows(ROWS, 128, world, rank)
    packed, scales = orc.rms_norm_quantise_nvfp4(x[first:first + count], w, count, COLS, 1e-6, 64.0, nthreads=1)
    # every rank reports its padded row count; rank 0 gathers the byte counts like the bench gathers timings
    sizes = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([packed.size, scales.size], dtype=torch.int64))
    np.save(os.path.join(out_dir, f"packed{rank}.npy"), packed)
    np.save(os.path.join(out_dir, f"scales{rank}.npy"), scales)
    dist.barrier()
    if rank == 0:
        np.save(os.path.join(out_dir, "sizes.npy"), torch.stack(sizes).numpy())
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_reproduce_the_single_rank_bytes(tmp_path):
    sys.path.insert(0, os.fspath(ROOT))
    from oracle import binding as orc

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), os.fspath(tmp_path)), nprocs=world, join=True)
    x, w = _inputs()
    want_p, want_s = orc.rms_norm_quantise_nvfp4(x, w, ROWS, COLS, 1e-6, 64.0)
    got_p = np.concatenate([np.load(tmp_path / f"packed{r}.npy") for r in range(world)])
    got_s = np.concatenate([np.load(tmp_path / f"scales{r}.npy") for r in range(world)])
    assert np.array_equal(got_p, want_p)
    assert np.array_equal(got_s, want_s)
    sizes = np.load(tmp_path / "sizes.npy")
    assert sizes[:, 0].sum() == want_p.size and sizes[:, 1].sum() == want_s.size
