"""Test scaffolding of the expert-parallel MoE block: seeded layer weights, expert shards, a
compute back end on the CPU oracle (the checker), and a driver that runs several ranks' blocks in
lockstep inside one process."""
import numpy as np
import torch

import helpers as hp
import orn_oracle as orc

NAMES = ["gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate"]


def layer_weights(seed, H, E, I):
    """One MoE layer in BASELINE config 2's formats: bf16 router, Q4_K gate/up, Q6_K down,
    shared expert of the same shapes, 8-bit affine shared-expert gate."""
    rng = np.random.default_rng(seed)
    return {
        "gate": hp.make_weights(rng, orc.BF16, 1, E, H),
        "sw_gate": hp.raw_q4k(rng, E, I, H), "sw_up": hp.raw_q4k(rng, E, I, H),
        "sw_down": hp.raw_q6k(rng, E, H, I),
        "sh_gate": hp.raw_q4k(rng, 1, I, H), "sh_up": hp.raw_q4k(rng, 1, I, H),
        "sh_down": hp.raw_q6k(rng, 1, H, I), "sh_egate": hp.make_weights(rng, orc.A8, 1, 1, H),
    }


def rows_of(seed, rank, R, H):
    rng = np.random.default_rng(seed * 1000 + rank)
    return hp.f32_to_bf16(rng.standard_normal((R, H)).astype(np.float32))


def shard(W, rank, world):
    """Experts [rank*E/N, (rank+1)*E/N) of an expert-stacked oracle weight."""
    per = W.E // world

    def cut(a):
        if a is None:
            return None
        flat = a.reshape(-1)
        step = flat.size // W.E
        return flat[rank * per * step:(rank + 1) * per * step].copy()
    return orc.Weights(W.kind, per, W.O, W.K, cut(W.w), cut(W.s), cut(W.b))


def rank_weights(ws, rank, world):
    return {n: (shard(w, rank, world) if n.startswith("sw_") else w) for n, w in ws.items()}


def _u16(t):
    return np.ascontiguousarray(t.numpy()).view(np.uint16)


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy())


class OracleOps:
    """The block's compute steps on the CPU oracle, on torch CPU tensors (bf16 bits as int16)."""

    def __init__(self, ws, top_k, norm_topk):
        self.w, self.k, self.norm = ws, top_k, int(bool(norm_topk))
        self.E, self.H = ws["gate"].O, ws["gate"].K

    def router(self, x):
        R = x.shape[0]
        probs = orc.softmax_precise(orc.gemv(self.w["gate"], _u16(x), R), R, self.E)
        inds, scores = orc.router_topk(probs, R, self.E, self.k)
        return torch.from_numpy(inds.astype(np.int32)), _t(scores)

    def shared(self, x):
        R = x.shape[0]
        xs = _u16(x)
        act = orc.swiglu(orc.gemv(self.w["sh_gate"], xs, R), orc.gemv(self.w["sh_up"], xs, R))
        return _t(orc.gemv(self.w["sh_down"], act, R)), _t(orc.gemv(self.w["sh_egate"], xs, R))

    def experts(self, x, lhs, rhs):
        P = len(lhs)
        if P == 0:
            return torch.zeros((0, self.H), dtype=torch.int16)
        xs = _u16(x)
        lhs, rhs = np.asarray(lhs, np.uint32), np.asarray(rhs, np.uint32)
        g = orc.gather_gemv(self.w["sw_gate"], xs, lhs, rhs)
        u = orc.gather_gemv(self.w["sw_up"], xs, lhs, rhs)
        act = orc.swiglu(g, u).reshape(P, -1)
        return _t(orc.gather_gemv(self.w["sw_down"], act, np.arange(P, dtype=np.uint32), rhs))

    def combine(self, scores, y, gs, sy):
        R = scores.shape[0]
        return _t(orc.moe_combine(_u16(scores), _u16(y), _u16(gs), _u16(sy), R, self.k, self.H, self.norm))

    def stage_indices(self, arrays):
        return {n: np.asarray(a) for n, a in arrays.items()}

    def index_rows(self, x, idx):
        return x.index_select(0, torch.from_numpy(np.asarray(idx, np.int64)))

    def to_host(self, t):
        return t.numpy()

    def run(self):
        import contextlib
        return contextlib.nullcontext()


class FixedComm:
    """Rank and world size only: the lockstep driver moves the buffers itself."""

    def __init__(self, rank, world):
        self.rank, self.world = rank, world


def _chunks(t, counts):
    return list(torch.split(t, [int(c) for c in counts], dim=0))


def run_lockstep(blocks, xs, to_host):
    """All ranks' blocks phase by phase; the exchanges are slices and concatenations."""
    N = len(blocks)
    inds = [b.route(x) for b, x in zip(blocks, xs)]
    all_inds = np.stack([np.asarray(to_host(i)) for i in inds])
    plans = [b.plan(all_inds) for b in blocks]
    sends = [_chunks(b.dispatch_buffer(), p.send_counts) for b, p in zip(blocks, plans)]
    for d in range(N):
        assert [int(sends[s][d].shape[0]) for s in range(N)] == [int(c) for c in plans[d].recv_counts]
    ys = [_chunks(blocks[d].compute(torch.cat([sends[s][d] for s in range(N)])), plans[d].pair_counts)
          for d in range(N)]
    for s in range(N):
        assert [int(ys[d][s].shape[0]) for d in range(N)] == [int(c) for c in plans[s].back_counts]
    return [blocks[s].finish(torch.cat([ys[d][s] for d in range(N)])) for s in range(N)]


def expected(ws, xs, top_k, norm_topk=1):
    """The single-device block of the oracle on every rank's rows."""
    return [orc.moe_block(ws, x, x.shape[0], top_k, norm_topk)[0] for x in xs]
