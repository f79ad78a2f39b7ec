"""CPU tests of host-side logic: synthetic inputs, schedule, frame sharding across ranks (gloo, world 2)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synthetic_frames_are_reproducible_and_in_range(pkg):
    S = pkg.synth
    a, b = S.single_frame(), S.single_frame()
    np.testing.assert_array_equal(a, b)
    assert a.shape == (20000, 4) and a.dtype == np.float32
    xmin, ymin, zmin, xmax, ymax, zmax = S.POINT_RANGE
    assert (a[:, 0] >= xmin).all() and (a[:, 0] < xmax).all() and (a[:, 1] >= ymin).all() and (a[:, 1] < ymax).all()
    assert (a[:, 2] >= zmin).all() and (a[:, 2] < zmax).all() and (a[:, 3] >= 0).all() and (a[:, 3] < 1).all()
    f0, f1 = S.sweep_frame(0, 5000), S.sweep_frame(1, 5000)
    assert f0.shape == (5000, 4) and not np.array_equal(f0, f1)
    # first outputs of the documented generator for seed 1 (splitmix64 reference values)
    assert [int(v) for v in S.Stream(1).bits(2)] == [0x910A2DEC89025CC1, 0xBEEB8DA1658EEC67]


def test_active_voxels_are_unique_and_in_grid(pkg):
    c = pkg.synth.active_voxels()
    assert c.shape == (16000, 4) and (c[:, 0] == 0).all()
    Z, Y, X = pkg.synth.GRID_ZYX
    key = (c[:, 1].astype(np.int64) * Y + c[:, 2]) * X + c[:, 3]
    assert np.unique(key).size == 16000
    assert (c[:, 1] < Z).all() and (c[:, 2] < Y).all() and (c[:, 3] < X).all() and (c >= 0).all()


def test_schedule_matches_the_reference_wiring(pkg):
    L = pkg.schedule.LAYERS
    assert len(L) == 14
    assert [l.subm for l in L] == [True, True, False, True, True, False, True, True, True, False, True, True, True, False]
    assert [(l.cin, l.cout) for l in L] == [(4, 16), (16, 16), (16, 32), (32, 32), (32, 32), (32, 64)] + [(64, 64)] * 8
    assert L[9].padding == (0, 1, 1) and L[13].ksize == (3, 1, 1) and L[13].stride == (2, 1, 1)
    for a, b in zip(L, L[1:]):
        assert a.out_shape == b.in_shape and a.cout == b.cin
    for l in L:
        if not l.subm:
            want = tuple((l.in_shape[j] + 2 * l.padding[j] - l.ksize[j]) // l.stride[j] + 1 for j in range(3))
            assert l.out_shape == want
    assert L[-1].out_shape == (2, 200, 176)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package

    pkg = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # each rank owns its own frames (weak scaling): disjoint seeds, no exchange on the data path
    first = pkg.sharding.first_frame(rank, frames_per_rank=3)
    seeds = [pkg.sharding.frame_seed(first + i) for i in range(3)]
    # the only collective: max over ranks of the device time, then frames/s of the whole job
    t = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
    value = pkg.sharding.job_throughput(t, frames_per_rank=3, steps=2, world=world,
                                        all_reduce_max=lambda x: dist.all_reduce(x, op=dist.ReduceOp.MAX))
    gathered = [None] * world
    dist.all_gather_object(gathered, seeds)
    q.put((rank, value, gathered))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_frames_and_reduce_time_over_gloo():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    out = [q.get(timeout=120) for _ in ps]
    [p.join(timeout=60) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    for rank, value, gathered in out:
        # 2 ranks x 3 frames x 2 steps over the slower rank's 15 ms
        assert value == pytest.approx(12 / 0.015)
        flat = [s for seeds in gathered for s in seeds]
        assert len(set(flat)) == 6


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the metric of the main arm, the CPU
    baseline that produced it and an end-to-end object that repeats the value with no device copies."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "single",
                          "--frames", "4", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "impl"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "frames/s" and line["value"] > 0
    assert line["vs_baseline"] is None and line["higher_is_better"] is True and line["data"] == "synthetic"
    assert line["config"]["workload"] == "single"
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == dict(value=line["value"], unit=line["unit"], h2d_bytes_per_step=0, d2h_bytes_per_step=0)
