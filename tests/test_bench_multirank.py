"""bench.py's N > 1 logic on CPU: two gloo ranks agree on the slowest rank's time and on the
whole-job rate (replica per GPU, weak scaling); the reference arm runs on rank 0 only."""
import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_gloo_ranks_take_the_max_and_scale_tokens(tmp_path):
    port = _free_port()
    out = str(tmp_path / "r")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), out], env=env))
    for p in procs:
        assert p.wait(timeout=120) == 0
    res = [json.load(open(out + ".%d" % r)) for r in range(2)]
    for r in res:
        assert abs(r["dev_max"] - 550.0) < 1e-9 and abs(r["wall_max"] - 0.66) < 1e-9   # rank 1 is the slowest
        assert abs(r["value"] - 2 * 3 * 200 / 0.550) < 1e-6                              # both ranks' tokens
        assert abs(r["e2e"] - 2 * 3 * 200 / 0.66) < 1e-6


def test_single_process_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_max_over_ranks([1.5, 2.5], None, "cpu") == [1.5, 2.5]
    v, e = bench.whole_job_rates(1, 3, 200, 600.0, 0.75)
    assert abs(v - 1000.0) < 1e-9 and abs(e - 800.0) < 1e-9


def test_reference_arm_runs_on_rank_zero_only():
    """Under torchrun the reference arm prints on rank 0; the other ranks exit 0 without work."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and p.stdout.strip() == ""
