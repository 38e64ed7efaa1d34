"""The multi-rank plumbing of bench.py on CPU: two gloo ranks, the job time is the maximum over ranks and the
aggregate throughput is (ranks x steps) / that time; the reference arm runs on rank 0 only."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, %r)
    import bench
    world, rank, local, dist = bench.dist_setup(2)
    assert world == 2 and dist is not None
    ms = 10.0 + 5.0 * rank            # rank 1 is the slower replica
    ms_all = bench.reduce_max_time(ms, dist)
    value = world * 64 / (ms_all / 1e3)
    dist.barrier()
    print(json.dumps({"rank": rank, "ms_all": ms_all, "value": value}))
    dist.destroy_process_group()
""") % ROOT


def test_two_gloo_ranks_take_the_slowest_time(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29000 + os.getpid() % 2000
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    for o in outs:
        assert abs(o["ms_all"] - 15.0) < 1e-9
        assert abs(o["value"] - 2 * 64 / 0.015) < 1e-6


def test_reference_arm_non_zero_ranks_exit_quietly():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29499")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                       env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip() == ""
