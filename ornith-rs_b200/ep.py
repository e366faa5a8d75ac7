"""Expert-parallel form of the sparse MoE block (sparse_moe_block, src/ops/moe.rs:662-741).

The 256 experts of a layer are split evenly over the ranks of one node (rank r holds experts
[r*E/N, (r+1)*E/N)); router, shared expert and the token rows stay data-parallel at the rank that
owns the sequence ("home").  One block is

    home    router logits -> softmax -> top-k (same ops as the single-GPU block)
    all     all-gather of the routing indices: every rank can derive the whole exchange plan
    home    dispatch: each needed row of x goes ONCE to every rank that holds one of its experts
    owner   gate/up mat-vec + SwiGLU + down mat-vec per routed (row, slot) pair, one-row arithmetic
    owner   return: the bf16 down outputs go back to the row's home
    home    combine in ascending slot order + shared expert (moe_combine, src/ops/moe.rs:548-596)

Every routed pair is computed with the one-row arithmetic of `gather_qmv` (kquant.rs:741-770) and
the combine runs at home in the reference's order, so the block's output bits do not depend on
the number of ranks.

Compute goes through the C ABI on raw device pointers; torch supplies the device buffers, the
stream object and the collectives (`torch.distributed`, NCCL over NVLink).  All device work of a
block, collectives included, is ordered on the context's stream; the one host read per block is
the routing table the plan is made from.  The context must outlive every torch tensor that was
used on its stream (torch records an event on that stream when it frees such a buffer).
"""
import ctypes as C

import numpy as np


# --------------------------------------------------------------------------- plan (host, numpy)
class Plan:
    """What one rank sends, computes and receives for one block.

    send_rows    rows of the local x to send, grouped by destination rank (ascending row inside)
    send_counts  [N] rows per destination
    recv_counts  [N] rows that arrive per source rank
    lhs, rhs     per routed pair computed here: index into the received rows, LOCAL expert id
    pair_counts  [N] pairs computed here per source rank (= rows returned to that rank)
    back_counts  [N] pairs this rank gets back per owner rank
    home_index   [R*k] position in the returned buffer of pair (row, slot), row-major
    """

    __slots__ = ("send_rows", "send_counts", "recv_counts", "lhs", "rhs", "pair_counts", "back_counts",
                 "home_index")


def _pairs(inds_src, dest, experts_per_rank):
    """Pairs (row, slot) of one source rank whose expert lives on `dest`, in (row, slot) order,
    and the distinct rows among them (ascending)."""
    owner = inds_src // experts_per_rank
    rows, slots = np.nonzero(owner == dest)          # row-major: ascending row, then slot
    uniq = np.unique(rows)
    return rows, slots, uniq


def make_plan(all_inds, rank, n_experts):
    """all_inds: integer array [N, R, k] of every rank's routing indices (global expert ids)."""
    all_inds = np.asarray(all_inds).astype(np.int64)
    N, R, k = all_inds.shape
    if n_experts % N:
        raise ValueError("experts (%d) do not split evenly over %d ranks" % (n_experts, N))
    if all_inds.size and (all_inds.min() < 0 or all_inds.max() >= n_experts):
        raise ValueError("routing index out of range")
    per = n_experts // N
    p = Plan()
    # what this rank sends (as home) and gets back
    send_rows, send_counts, back_counts = [], [], []
    home_index = np.empty(R * k, np.int64)
    off = 0
    for d in range(N):
        rows, slots, uniq = _pairs(all_inds[rank], d, per)
        send_rows.append(uniq)
        send_counts.append(len(uniq))
        back_counts.append(len(rows))
        home_index[rows * k + slots] = off + np.arange(len(rows))
        off += len(rows)
    p.send_rows = np.concatenate(send_rows).astype(np.int64) if N else np.zeros(0, np.int64)
    p.send_counts, p.back_counts, p.home_index = send_counts, back_counts, home_index
    # what this rank receives and computes (as owner)
    lhs, rhs, recv_counts, pair_counts = [], [], [], []
    base = 0
    for s in range(N):
        rows, slots, uniq = _pairs(all_inds[s], rank, per)
        recv_counts.append(len(uniq))
        pair_counts.append(len(rows))
        lhs.append(base + np.searchsorted(uniq, rows))
        rhs.append(all_inds[s][rows, slots] - rank * per)
        base += len(uniq)
    p.lhs = np.concatenate(lhs).astype(np.uint32)
    p.rhs = np.concatenate(rhs).astype(np.uint32)
    p.recv_counts, p.pair_counts = recv_counts, pair_counts
    return p


# --------------------------------------------------------------------------- compute back ends
class CudaOps:
    """The block's compute steps on the CUDA library, on torch device tensors (bf16 bits as int16).

    weights: dict with `gate` (router [E, H]), `sh_gate`, `sh_up`, `sh_down`, `sh_egate` (whole) and
    `sw_gate`, `sw_up`, `sw_down` (this rank's experts [E/N, ...]) as `Linear` objects.
    """

    def __init__(self, ctx, weights, top_k, norm_topk):
        import torch
        self.torch = torch
        self.ctx, self.w, self.k, self.norm = ctx, weights, top_k, int(bool(norm_topk))
        self.lib = ctx._lib
        sp = C.c_void_p()
        ctx.check(self.lib.orn_ctx_stream(ctx.h, C.byref(sp)), "orn_ctx_stream")
        self.device = torch.device("cuda", ctx.device)
        self.stream = torch.cuda.ExternalStream(sp.value, device=self.device)
        self.H = weights["gate"].K
        self.E = weights["gate"].O
        self._iota = {}

    # -- helpers
    def empty(self, shape, dtype=None):
        return self.torch.empty(shape, dtype=dtype or self.torch.int16, device=self.device)

    def _gemv(self, lin, x, rows):
        """y[rows, O] = x W^T for a replicated matrix.  Up to 4 rows go through `orn_gemv`; more rows
        go through ONE gather launch with every row on "expert" 0 (the same one-row dot, so the same
        bits) instead of a launch per group of 4."""
        if rows > 4:
            if rows not in self._iota:
                self._iota[rows] = (self.torch.arange(rows, dtype=self.torch.int32, device=self.device),
                                    self.torch.zeros(rows, dtype=self.torch.int32, device=self.device))
            ident, zeros = self._iota[rows]
            return self._gather(lin, x, ident, zeros, rows)
        y = self.empty((rows, lin.O))
        if rows:
            self.ctx.check(self.lib.orn_gemv(self.ctx.h, lin.h, x.data_ptr(), rows, y.data_ptr(), 0), "orn_gemv")
        return y

    def _gather(self, lin, x, lhs, rhs, rows):
        y = self.empty((rows, lin.O))
        if rows:
            self.ctx.check(self.lib.orn_gather_gemv(self.ctx.h, lin.h, x.data_ptr(), lhs.data_ptr(),
                                                    rhs.data_ptr(), rows, y.data_ptr()), "orn_gather_gemv")
        return y

    def _swiglu(self, g, u):
        out = self.empty(tuple(g.shape))
        if g.numel():
            self.ctx.check(self.lib.orn_swiglu(self.ctx.h, g.data_ptr(), u.data_ptr(), g.numel(), out.data_ptr()),
                           "orn_swiglu")
        return out

    # -- the block's steps
    def router(self, x):
        R = x.shape[0]
        logits = self._gemv(self.w["gate"], x, R)
        probs = self.empty((R, self.E))
        self.ctx.check(self.lib.orn_softmax_precise(self.ctx.h, logits.data_ptr(), R, self.E, probs.data_ptr()),
                       "orn_softmax_precise")
        inds = self.empty((R, self.k), self.torch.int32)
        scores = self.empty((R, self.k))
        self.ctx.check(self.lib.orn_router_topk(self.ctx.h, probs.data_ptr(), R, self.E, self.k, inds.data_ptr(),
                                                scores.data_ptr()), "orn_router_topk")
        return inds, scores

    def shared(self, x):
        R = x.shape[0]
        act = self._swiglu(self._gemv(self.w["sh_gate"], x, R), self._gemv(self.w["sh_up"], x, R))
        return self._gemv(self.w["sh_down"], act, R), self._gemv(self.w["sh_egate"], x, R)

    def experts(self, x, lhs, rhs):
        """x [U, H] received rows; pair p = expert rhs[p] applied to x[lhs[p]] -> [P, H]."""
        P = int(lhs.shape[0])
        lhs_d = self.torch.from_numpy(lhs.astype(np.int32)).to(self.device, non_blocking=False)
        rhs_d = self.torch.from_numpy(rhs.astype(np.int32)).to(self.device, non_blocking=False)
        ident = self.torch.arange(P, dtype=self.torch.int32, device=self.device)
        g = self._gather(self.w["sw_gate"], x, lhs_d, rhs_d, P)
        u = self._gather(self.w["sw_up"], x, lhs_d, rhs_d, P)
        act = self._swiglu(g, u)
        return self._gather(self.w["sw_down"], act, ident, rhs_d, P)

    def combine(self, scores, y, gs, sy):
        R = scores.shape[0]
        out = self.empty((R, self.H))
        self.ctx.check(self.lib.orn_moe_combine(self.ctx.h, scores.data_ptr(), y.data_ptr(), gs.data_ptr(),
                                                sy.data_ptr(), R, self.k, self.H, self.norm, out.data_ptr()),
                       "orn_moe_combine")
        return out

    def index_rows(self, x, idx):
        return x.index_select(0, self.torch.from_numpy(np.asarray(idx, np.int64)).to(self.device))

    def to_host(self, t):
        return t.cpu().numpy()   # waits for the context's stream

    def run(self):
        """Context manager: torch work issued inside is ordered on the context's stream."""
        return self.torch.cuda.stream(self.stream)


# --------------------------------------------------------------------------- exchange
class DistComm:
    """The block's three collectives on a torch.distributed group (NCCL on GPUs)."""

    def __init__(self, dist, group=None):
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def all_gather(self, t):
        import torch
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out.reshape((self.world,) + tuple(t.shape))

    def all_to_all_rows(self, t, send_counts, recv_counts):
        import torch
        out = torch.empty((int(sum(recv_counts)),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        # rows travel as bytes: every back end moves uint8
        self.dist.all_to_all_single(out.view(torch.uint8), t.contiguous().view(torch.uint8),
                                    output_split_sizes=list(map(int, recv_counts)),
                                    input_split_sizes=list(map(int, send_counts)), group=self.group)
        return out


class SelfComm:
    """World of one rank: the exchanges are identities."""

    rank, world = 0, 1

    def all_gather(self, t):
        return t.reshape((1,) + tuple(t.shape))

    def all_to_all_rows(self, t, send_counts, recv_counts):
        return t


# --------------------------------------------------------------------------- the block
class EpMoeBlock:
    """forward(x [R, H]) -> [R, H]; R must be the same on every rank of the group."""

    def __init__(self, ops, comm, n_experts):
        self.ops, self.comm, self.E = ops, comm, n_experts
        if n_experts % comm.world:
            raise ValueError("experts (%d) do not split evenly over %d ranks" % (n_experts, comm.world))

    # The block in phases; `forward` runs them back to back.  They are separate so that a test can
    # drive several ranks' blocks in lockstep inside one process.
    def route(self, x):
        self.x = x
        self.inds, self.scores = self.ops.router(x)
        return self.inds

    def plan(self, all_inds_host):
        self.p = make_plan(all_inds_host, self.comm.rank, self.E)
        return self.p

    def dispatch_buffer(self):
        return self.ops.index_rows(self.x, self.p.send_rows)

    def compute(self, received):
        # pairs of one expert run next to each other (their weight reads meet in L2); the outputs go
        # back into the plan's return order
        order = np.argsort(self.p.rhs, kind="stable")
        inverse = np.empty_like(order)
        inverse[order] = np.arange(len(order))
        y = self.ops.experts(received, self.p.lhs[order], self.p.rhs[order])
        return self.ops.index_rows(y, inverse)

    def finish(self, returned):
        y = self.ops.index_rows(returned, self.p.home_index)
        sy, gs = self.ops.shared(self.x)
        return self.ops.combine(self.scores, y, gs, sy)

    def forward(self, x):
        with self.ops.run():
            inds = self.route(x)
            all_inds = self.ops.to_host(self.comm.all_gather(inds))
            p = self.plan(all_inds)
            recv = self.comm.all_to_all_rows(self.dispatch_buffer(), p.send_counts, p.recv_counts)
            y = self.compute(recv)
            back = self.comm.all_to_all_rows(y, p.pair_counts, p.back_counts)
            return self.finish(back)


def shard_experts(ctx, lin, rank, world):
    """This rank's slice [rank*E/N, (rank+1)*E/N) of an expert-stacked `Linear` as a new `Linear`
    (the artifact tensors are expert-major, so a shard is a contiguous range of each)."""
    from . import Linear
    if lin.E % world:
        raise ValueError("experts (%d) do not split evenly over %d ranks" % (lin.E, world))
    per = lin.E // world
    parts = []
    for a in lin.export():
        step = a.size // lin.E
        parts.append(a[rank * per * step:(rank + 1) * per * step] if a.size else None)
    return Linear.from_numpy(ctx, lin.kind, parts[0], parts[1], parts[2], E=per, O=lin.O, K=lin.K)
