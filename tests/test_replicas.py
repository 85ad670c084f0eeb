"""The N > 1 path on CPU: two gloo ranks run minml_b200.replicas (work assignment, barrier, max-over-ranks timing), and
bench.py's reference arm under torchrun prints exactly one line, from rank 0."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    from minml_b200.replicas import Replicas
    import bench
    r = Replicas("gloo")
    r.barrier()
    # each rank pretends to have taken a different time for the same number of positions
    local_seconds = 0.5 + 0.25 * rank
    value, slowest = r.throughput(1024 * 10, local_seconds)
    maxima = r.max_over_ranks([float(rank), 10.0 - rank])
    cfg = bench.CONFIGS["c1"]
    _, packed = bench.synthetic.bernoulli_planes((4, cfg["height"], cfg["width"], cfg["planes"]), r.input_seed(bench.SEED))
    per_rank = r.gather_floats(10.0 + rank)
    r.barrier()
    with open(os.path.join(out_dir, "rank%d.json" % rank), "w") as f:
        json.dump({"value": value, "slowest": slowest, "maxima": maxima, "seed": r.input_seed(bench.SEED), "checksum": int(packed.astype(np.int64).sum()),
                   "global_units": r.global_units(1024), "per_rank": per_rank}, f)
    r.close()


def test_two_gloo_ranks(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = [json.load(open(tmp_path / ("rank%d.json" % r))) for r in range(world)]
    for g in got:  # every rank sees the same whole-job figure: all positions over the slowest rank's time
        assert g["slowest"] == 0.75
        assert abs(g["value"] - 2 * 10240 / 0.75) < 1e-6
        assert g["maxima"] == [1.0, 10.0]
        assert g["global_units"] == 2048
        assert g["per_rank"] == [10.0, 11.0]  # every rank's own figure, in rank order, on every rank
    assert got[0]["seed"] != got[1]["seed"] and got[0]["checksum"] != got[1]["checksum"]  # each rank draws its own positions


def test_reference_arm_under_torchrun_prints_one_line():
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--config", "c1", "--steps", "1", "--warmup", "0"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["n_gpus"] == 2 and rec["value"] > 0
    assert rec["cpu_baseline"]["kind"] in ("reference", "port") and rec["e2e"]["h2d_bytes_per_step"] == 0
    assert rec["steps"] == 1 and rec["warmup"] == 0  # the arm honours the command line


def test_reference_arm_does_not_map_the_cuda_library():
    """The CPU arm times minml's CPU backend and nothing else: the process must never load libminml_b200.so (nor torch)."""
    code = ("import sys; sys.argv = ['bench.py', '--impl', 'reference', '--config', 'c0', '--steps', '1', '--warmup', '0']; "
            "import runpy; runpy.run_path(%r, run_name='__main__'); "
            "maps = open('/proc/self/maps').read(); "
            "assert 'libminml_b200' not in maps, 'the CUDA library was mapped'; assert 'torch' not in sys.modules; print('CLEAN')"
            % os.path.join(ROOT, "bench.py"))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and "CLEAN" in out.stdout, out.stdout[-500:] + out.stderr[-2000:]
