"""The multi-rank path on CPU (gloo, world_size 2): the row partition, the gather used for
checking, the max-over-ranks timing reduction, and the rank behaviour of the reference arm.
The kernels themselves are not involved (no GPU here); the per-shard arithmetic is the CPU
oracle's, which is what a sharded GPU run is compared with."""
import json
import os
import subprocess
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from oracle import g4_oracle
    lib = g4_oracle.load("port")
    total, cols = 24, 4096
    lo, hi = bench.shard_bounds(total, world, rank)
    y = lib.fill_bf16(1, 3.0, total * cols).reshape(total, cols)
    res = lib.fill_bf16(2, 3.0, total * cols).reshape(total, cols)
    w = lib.fill_bf16(3, 1.5, cols)
    h, n = lib.add_rmsnorm(y[lo:hi], res[lo:hi], w, 1e-5, 0.22)
    codes, scale, amax = lib.quant_fp8(n)
    # gather for checking only: no collective belongs to the data path
    parts = [torch.empty(hi - lo, cols, dtype=torch.int32) for _ in range(world)]  # gloo has no int16
    dist.all_gather(parts, torch.from_numpy(h.astype(np.int32)))
    amaxes = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(amaxes, torch.tensor([float(amax)]))
    ms = bench.max_over_ranks(10.0 + rank, None)
    if rank == 0:
        h_all = torch.cat(parts).numpy().astype(np.uint16)
        h_ref, n_ref = lib.add_rmsnorm(y, res, w, 1e-5, 0.22)
        _, _, amax_ref = lib.quant_fp8(n_ref)
        with open(os.path.join(out_dir, "result.json"), "w") as f:
            json.dump({"h_equal": bool((h_all == h_ref).all()),
                       "amax_max": max(a.item() for a in amaxes), "amax_ref": float(amax_ref),
                       "ms": ms, "bounds": [lo, hi]}, f)
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharding_over_two_gloo_ranks(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = json.load(open(tmp_path / "result.json"))
    assert r["h_equal"]                      # bf16 outputs do not depend on the partition
    assert r["amax_max"] == r["amax_ref"]    # the batch amax is the max of the shard amaxes
    assert r["ms"] == 11.0                   # timing = max over ranks
    assert r["bounds"] == [0, 12]


def test_shard_bounds_cover_all_rows_once():
    sys.path.insert(0, ROOT)
    import bench
    for world in (1, 2, 4, 8):
        spans = [bench.shard_bounds(65536, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 65536
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert len({hi - lo for lo, hi in spans}) == 1


def test_reference_arm_only_rank0_prints():
    env = dict(os.environ, G4_BENCH_CPU_ROWS="8", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1")
    out1 = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                           "--gpus", "2", "--steps", "1", "--warmup", "0"],
                          env=dict(env, RANK="1", LOCAL_RANK="1"), capture_output=True, text=True, timeout=600)
    assert out1.returncode == 0 and out1.stdout.strip() == ""
    out0 = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                           "--gpus", "2", "--steps", "1", "--warmup", "0"],
                          env=dict(env, RANK="0", LOCAL_RANK="0"), capture_output=True, text=True, timeout=600)
    assert out0.returncode == 0
    line = json.loads(out0.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["e2e"]["h2d_bytes_per_step"] == 0
