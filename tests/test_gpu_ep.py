"""Expert-parallel MoE block on the GPU: a world of one against the single-device block and the
oracle, N ranks' blocks in lockstep on one device (sharded experts, the N > 1 data path), and two
ranks on two GPUs over NCCL where the box has them.  Bit-exact in every case."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import ep_helpers as eh

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
SHAPE = dict(H=2048, E=32, I=512, k=8)


@pytest.fixture(scope="module")
def ep(pkg):
    from ornith_rs_b200 import ep as mod
    return mod


def cuda_ops(pkg, ctx, ep, ws, k):
    L = {n: pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K) for n, w in ws.items()}
    return ep.CudaOps(ctx, L, k, 1), L


def dev_rows(ops, x):
    return torch.from_numpy(x.view(np.int16).copy()).to(ops.device)


def test_world_of_one_equals_the_single_device_block(pkg, ctx, ep):
    H, E, I, k = (SHAPE[n] for n in "HEIk")
    ws = eh.layer_weights(11, H, E, I)
    ops, L = cuda_ops(pkg, ctx, ep, ws, k)
    x = eh.rows_of(11, 0, 4, H)
    y = ep.EpMoeBlock(ops, ep.SelfComm(), E).forward(dev_rows(ops, x))
    ctx.sync()
    got = y.cpu().numpy().view(np.uint16)
    out, inds = ctx.empty((4, H), np.uint16), ctx.empty((4, k), np.uint32)
    order = ["gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate"]
    ctx.check(ctx._lib.orn_moe_block(ctx.h, *[L[n].h for n in order], ctx.upload(x).ptr, 4, k, 1, out.ptr, inds.ptr),
              "moe_block")
    assert np.array_equal(got, out.numpy())
    assert np.array_equal(got, eh.expected(ws, [x], k)[0])
    for l in L.values():
        l.free()


@pytest.mark.parametrize("N", [2, 4])
def test_lockstep_ranks_on_one_device_equal_the_single_device_block(pkg, ctx, ep, N):
    H, E, I, k = (SHAPE[n] for n in "HEIk")
    R = 6                                             # more rows than one mat-vec group of 4
    ws = eh.layer_weights(12, H, E, I)
    xs = [eh.rows_of(12, r, R, H) for r in range(N)]
    made = [cuda_ops(pkg, ctx, ep, eh.rank_weights(ws, r, N), k) for r in range(N)]
    blocks = [ep.EpMoeBlock(ops, eh.FixedComm(r, N), E) for r, (ops, _) in enumerate(made)]
    with made[0][0].run():
        outs = eh.run_lockstep(blocks, [dev_rows(made[0][0], x) for x in xs], lambda t: t.cpu().numpy())
        outs = [o.cpu().numpy().view(np.uint16) for o in outs]
    for got, want in zip(outs, eh.expected(ws, xs, k)):
        assert np.array_equal(got, want)
    for _, L in made:
        for n, l in L.items():
            l.free()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_over_nccl_equal_the_single_device_block(tmp_path):
    H, E, I, k = (SHAPE[n] for n in "HEIk")
    seed, R = 13, 6
    port, out = _free_port(), str(tmp_path / "y")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), "cuda", out] +
                                      [str(v) for v in (seed, R, H, E, I, k)], env=env))
    for p in procs:
        assert p.wait(timeout=600) == 0
    ws = eh.layer_weights(seed, H, E, I)
    xs = [eh.rows_of(seed, r, R, H) for r in range(2)]
    for r, want in enumerate(eh.expected(ws, xs, k)):
        assert np.array_equal(np.load("%s.%d.npy" % (out, r)), want)


# ---- the library's own block (csrc/ep.cu): plan on the device, NCCL inside the library -------------
def test_library_block_world_of_one_equals_the_oracle(pkg, ctx, ep):
    """BASELINE config 5's decode width on one rank: 128 rows (64 sequences x width 2), 256 experts
    top-8, through orn_ep_moe_block: every expert's records streamed once for all its rows by the
    grouped mat-vec, each row with the one-row arithmetic, so rows and routing indices equal the
    oracle's single-device block bit for bit."""
    H, E, I, k, R = 2048, 256, 512, 8, 128
    ws = eh.layer_weights(21, H, E, I)
    L = {n: pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K) for n, w in ws.items()}
    x = eh.rows_of(21, 0, R, H)
    group = ep.LibEp(ctx, exact=True)
    inds = ctx.empty((R, k), np.uint32)
    l0 = ctx.launches()
    y = group.moe_block(L, ctx.upload(x), R, k, 1, inds=inds)
    ctx.sync()
    assert ctx.launches() - l0 <= 20     # a fixed number of launches, whatever the row count
    import orn_oracle as orc
    import helpers as hp
    want, want_inds = orc.moe_block(ws, x, R, k, 1)
    assert np.array_equal(inds.numpy(), want_inds)
    assert np.array_equal(y.numpy(), want)
    # the default: routed experts on the tensor cores.  Routing stays bit-exact; rows agree to rounding
    # (raw-field weights are of one sign, so the bound is the reference's own for its bfloat16 tile,
    # 1/256 of the largest output, tests/q4k.rs:444-450, plus one bfloat16 step of the stored value)
    fast = ep.LibEp(ctx)
    inds2 = ctx.empty((R, k), np.uint32)
    y2 = fast.moe_block(L, ctx.upload(x), R, k, 1, inds=inds2)
    ctx.sync()
    assert np.array_equal(inds2.numpy(), want_inds)
    g, w = hp.bf16_to_f32(y2.numpy()).astype(np.float64), hp.bf16_to_f32(want).astype(np.float64)
    assert np.all(np.abs(g - w) <= np.abs(w).max() / 256.0 + np.abs(w) * 2.0 ** -7)
    fast.close()
    # a second call on other rows reuses the scratch; ragged row counts work too
    x2 = eh.rows_of(22, 0, 37, H)
    y2 = group.moe_block(L, ctx.upload(x2), 37, k, 1)
    ctx.sync()
    assert np.array_equal(y2.numpy(), orc.moe_block(ws, x2, 37, k, 1)[0])
    # more routes than one pass of the route kernel takes (1024): 1600 routes, sorted in two passes
    x3 = eh.rows_of(23, 0, 200, H)
    y3 = group.moe_block(L, ctx.upload(x3), 200, k, 1)
    ctx.sync()
    assert np.array_equal(y3.numpy(), orc.moe_block(ws, x3, 200, k, 1)[0])
    group.close()
    for l in L.values():
        l.free()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_library_block_two_gpus_equal_the_single_device_block(tmp_path):
    H, E, I, k = (SHAPE[n] for n in "HEIk")
    seed, R = 14, 10
    port, out = _free_port(), str(tmp_path / "y")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), "lib-exact", out] +
                                      [str(v) for v in (seed, R, H, E, I, k)], env=env))
    for p in procs:
        assert p.wait(timeout=600) == 0
    ws = eh.layer_weights(seed, H, E, I)
    xs = [eh.rows_of(seed, r, R, H) for r in range(2)]
    for r, want in enumerate(eh.expected(ws, xs, k)):
        assert np.array_equal(np.load("%s.%d.npy" % (out, r)), want)


@pytest.mark.parametrize("exchange", ["peer memory", "nccl"])
def test_batched_mtp_decode_over_two_gpus_equals_the_single_sequence_engine(tmp_path, exchange):
    """Whole-model batched decode with the experts of every layer (and of the MTP head) split over two
    ranks: each rank's sequences, stepped through prompt windows and MTP depth-1 cycles with the
    expert-parallel block, reproduce the single-sequence engine bit for bit (the worker compares
    drafts, targets and hidden rows and exits non-zero on any difference).  Once with the library's own
    exchange kernels over peer memory (the worker asserts that the windows were mapped), once with the
    NCCL collectives they replace."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port, out = _free_port(), str(tmp_path / "ok")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", ORN_EP_NCCL="1" if exchange == "nccl" else "0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py"), "batch", out, "31"], env=env))
    for p in procs:
        assert p.wait(timeout=600) == 0
    for r in range(2):
        assert int(np.load("%s.%d.npy" % (out, r))[0]) == 1
