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


def make_plan(all_inds, rank, n_experts):
    """all_inds: integer array [N, R, k] of every rank's routing indices (global expert ids).
    Pairs are ordered by (row, slot) inside every (source, owner) group, rows ascending inside
    every (source, destination) group."""
    all_inds = np.asarray(all_inds).astype(np.int64)
    N, R, k = all_inds.shape
    if n_experts % N:
        raise ValueError("experts (%d) do not split evenly over %d ranks" % (n_experts, N))
    if all_inds.size and (all_inds.min() < 0 or all_inds.max() >= n_experts):
        raise ValueError("routing index out of range")
    per = n_experts // N
    owner = all_inds // per                                       # [N, R, k]
    p = Plan()
    # home side: this rank's pairs grouped by owner; a row goes once to every owner it needs
    mine = owner[rank].reshape(-1)                                # row-major (row, slot)
    by_owner = np.argsort(mine, kind="stable")
    p.home_index = np.empty(R * k, np.int64)
    p.home_index[by_owner] = np.arange(R * k)
    p.back_counts = np.bincount(mine, minlength=N).tolist()
    need = np.zeros((N, R), bool)
    need[mine, np.repeat(np.arange(R), k)] = True
    p.send_rows = np.nonzero(need)[1].astype(np.int64)            # owner-major, rows ascending
    p.send_counts = need.sum(1).tolist()
    # owner side: the pairs of every source whose expert lives here, source-major
    here = owner == rank
    src, row, slot = np.nonzero(here)
    p.pair_counts = np.bincount(src, minlength=N).tolist()
    arrive = here.any(2)                                          # [N, R]: rows that arrive, in buffer order
    p.recv_counts = arrive.sum(1).tolist()
    position = np.cumsum(arrive.reshape(-1)) - 1
    p.lhs = position[src * R + row].astype(np.uint32)
    p.rhs = (all_inds[src, row, slot] - rank * per).astype(np.uint32)
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
            ident, zeros = self._iota_pair(rows)
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

    def stage_indices(self, arrays):
        """All index vectors of one block in one host-to-device copy (int32 views of one buffer)."""
        sizes = [len(a) for a in arrays.values()]
        packed = np.concatenate([np.asarray(a).astype(np.int32) for a in arrays.values()]) if sum(sizes) else \
            np.zeros(0, np.int32)
        dev = self.torch.from_numpy(packed).to(self.device)
        return dict(zip(arrays.keys(), self.torch.split(dev, sizes)))

    def _iota_pair(self, rows):
        if rows not in self._iota:
            self._iota[rows] = (self.torch.arange(rows, dtype=self.torch.int32, device=self.device),
                                self.torch.zeros(rows, dtype=self.torch.int32, device=self.device))
        return self._iota[rows]

    def experts(self, x, lhs, rhs):
        """x [U, H] received rows; pair p = expert rhs[p] applied to x[lhs[p]] -> [P, H]."""
        P = int(lhs.shape[0])
        g = self._gather(self.w["sw_gate"], x, lhs, rhs, P)
        u = self._gather(self.w["sw_up"], x, lhs, rhs, P)
        act = self._swiglu(g, u)
        return self._gather(self.w["sw_down"], act, self._iota_pair(P)[0], rhs, P)

    def combine(self, scores, y, gs, sy):
        R = scores.shape[0]
        out = self.empty((R, self.H))
        self.ctx.check(self.lib.orn_moe_combine(self.ctx.h, scores.data_ptr(), y.data_ptr(), gs.data_ptr(),
                                                sy.data_ptr(), R, self.k, self.H, self.norm, out.data_ptr()),
                       "orn_moe_combine")
        return out

    def index_rows(self, x, idx):
        return x.index_select(0, idx)

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
        self.p = p = make_plan(all_inds_host, self.comm.rank, self.E)
        # pairs of one expert run next to each other (their weight reads meet in L2); `inverse`
        # puts the outputs back into the plan's return order
        order = np.argsort(p.rhs, kind="stable")
        inverse = np.empty_like(order)
        inverse[order] = np.arange(len(order))
        self.ix = self.ops.stage_indices({"send_rows": p.send_rows, "lhs": p.lhs[order], "rhs": p.rhs[order],
                                          "inverse": inverse, "home_index": p.home_index})
        return p

    def dispatch_buffer(self):
        return self.ops.index_rows(self.x, self.ix["send_rows"])

    def compute(self, received):
        y = self.ops.experts(received, self.ix["lhs"], self.ix["rhs"])
        return self.ops.index_rows(y, self.ix["inverse"])

    def finish(self, returned):
        y = self.ops.index_rows(returned, self.ix["home_index"])
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


# --------------------------------------------------------------------------- the library's block
class LibEp:
    """orn_ep: the expert-parallel block inside the library (csrc/ep.cu).  The plan is derived on
    the device from the gathered routing table, the two exchanges per layer are the library's own
    kernels over peer memory (`peer_windows` tells; NCCL collectives otherwise), enqueued on the
    context's stream, the expert owner runs the grouped product: no torch in the data path and no
    host read inside the block.  exact=True runs the routed experts through the
    row-invariant grouped mat-vec (bit-identical to the single-GPU block) instead of the grouped
    tensor-core product (identical routing, rows equal to rounding).  `uid` is the 128-byte id rank 0 got from
    `LibEp.unique_id(lib)` and the caller carried to the other ranks; a world of one needs none."""

    ORDER = ("gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate")

    def __init__(self, ctx, rank=0, world=1, uid=None, exact=False):
        self.ctx, self.rank, self.world = ctx, rank, world
        h = C.c_void_p()
        buf = None
        if world > 1:
            if uid is None or len(uid) != 128:
                raise ValueError("LibEp: world > 1 needs the 128-byte unique id made by rank 0")
            buf = (C.c_uint8 * 128).from_buffer_copy(bytes(uid))
        ctx.check(ctx._lib.orn_ep_init(ctx.h, buf, rank, world, 1 if exact else 0, C.byref(h)), "orn_ep_init")
        self.h = h
        self.peer_windows = bool(ctx._lib.orn_ep_peer_windows(h))

    @staticmethod
    def unique_id(lib):
        buf = (C.c_uint8 * 128)()
        rc = lib.orn_ep_unique_id(buf)
        if rc != 0:
            raise RuntimeError("orn_ep_unique_id failed with status %d (is libnccl.so.2 loadable?)" % rc)
        return bytes(buf)

    def moe_block(self, lins, x, R, top_k, norm_topk=1, out=None, inds=None):
        """lins: the eight Linear handles by name (sw_* hold this rank's experts); x: device rows
        [R, H]; returns the device buffer of the output rows."""
        H = lins["gate"].K
        if out is None:
            out = self.ctx.empty((R, H), np.uint16)
        xp = x.ptr if hasattr(x, "ptr") else x
        ip = None if inds is None else (inds.ptr if hasattr(inds, "ptr") else inds)
        self.ctx.check(self.ctx._lib.orn_ep_moe_block(self.h, *[lins[n].h for n in self.ORDER], xp, R, top_k,
                                                      int(bool(norm_topk)), out.ptr, ip), "orn_ep_moe_block")
        return out

    def close(self):
        if self.h:
            self.ctx._lib.orn_ep_destroy(self.h)
            self.h = None
