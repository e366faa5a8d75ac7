"""Expert-parallel MoE block, host side: the exchange plan, the lockstep emulation of N ranks and a
real two-rank gloo run, all with the CPU oracle as the compute back end.  The output must equal the
single-device block's bits for every N."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import ep_helpers as eh

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ep(pkg):
    from ornith_rs_b200 import ep as mod
    return mod


@pytest.mark.parametrize("N", [1, 2, 4, 8])
def test_plan_delivers_every_pair_to_its_expert_owner(ep, N):
    rng = np.random.default_rng(N)
    R, k, E = 5, 8, 64
    all_inds = np.stack([np.stack([rng.choice(E, k, replace=False) for _ in range(R)]) for _ in range(N)])
    plans = [ep.make_plan(all_inds, r, E) for r in range(N)]
    per = E // N
    # rows carry (rank, row) tags; the "expert" returns (tag, global expert id)
    xs = [np.array([[s, i] for i in range(R)]) for s in range(N)]
    sends = [np.split(xs[s][plans[s].send_rows], np.cumsum(plans[s].send_counts)[:-1]) for s in range(N)]
    backs = [[None] * N for _ in range(N)]
    for d in range(N):
        recv = np.concatenate([sends[s][d] for s in range(N)])
        assert [len(sends[s][d]) for s in range(N)] == plans[d].recv_counts
        assert len(np.unique(recv, axis=0)) == len(recv)            # a row crosses to an owner once
        assert (plans[d].rhs < per).all()
        y = np.concatenate([recv[plans[d].lhs], (plans[d].rhs + d * per)[:, None]], axis=1)
        for s, part in enumerate(np.split(y, np.cumsum(plans[d].pair_counts)[:-1])):
            backs[s][d] = part
    for s in range(N):
        assert [len(b) for b in backs[s]] == plans[s].back_counts
        home = np.concatenate(backs[s])[plans[s].home_index].reshape(R, k, 3)
        for i in range(R):
            for j in range(k):
                assert tuple(home[i, j]) == (s, i, all_inds[s, i, j])


def test_plan_rejects_bad_input(ep):
    with pytest.raises(ValueError):
        ep.make_plan(np.zeros((3, 1, 2), np.int64), 0, 64)       # 64 experts over 3 ranks
    with pytest.raises(ValueError):
        ep.make_plan(np.full((2, 1, 2), 64), 0, 64)               # index out of range


@pytest.mark.parametrize("N", [1, 2, 4])
def test_lockstep_ranks_equal_the_single_device_block(ep, N):
    seed, R, H, E, I, k = 3, 3, 256, 16, 256, 4
    ws = eh.layer_weights(seed, H, E, I)
    xs = [eh.rows_of(seed, r, R, H) for r in range(N)]
    blocks = [ep.EpMoeBlock(eh.OracleOps(eh.rank_weights(ws, r, N), k, 1), eh.FixedComm(r, N), E) for r in range(N)]
    outs = eh.run_lockstep(blocks, [torch.from_numpy(x.view(np.int16).copy()) for x in xs], lambda t: t.numpy())
    for got, want in zip(outs, eh.expected(ws, xs, k)):
        assert np.array_equal(got.numpy().view(np.uint16), want)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_gloo_ranks_equal_the_single_device_block(tmp_path):
    seed, R, H, E, I, k = 5, 3, 256, 16, 256, 4
    port, out = _free_port(), str(tmp_path / "y")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), "oracle", out] +
                                      [str(v) for v in (seed, R, H, E, I, k)], env=env))
    for p in procs:
        assert p.wait(timeout=300) == 0
    ws = eh.layer_weights(seed, H, E, I)
    xs = [eh.rows_of(seed, r, R, H) for r in range(2)]
    for r, want in enumerate(eh.expected(ws, xs, k)):
        assert np.array_equal(np.load("%s.%d.npy" % (out, r)), want)
