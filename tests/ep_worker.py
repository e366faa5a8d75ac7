"""One rank of the expert-parallel MoE block under torch.distributed.
Usage: python ep_worker.py <oracle|cuda|lib|lib-exact> <out_prefix> <seed> <R> <H> <E> <I> <k>
       python ep_worker.py batch <out_prefix> <seed>
(oracle: the Python exchange over the CPU oracle and gloo; cuda: the Python exchange over the C-ABI
ops and NCCL; lib: the library's own block, orn_ep_moe_block, NCCL id carried by gloo)
RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT (and LOCAL_RANK for cuda) come from the env.  The rank
builds the layer from the seed, keeps its expert shard, runs the block on its own rows and writes
the output rows to <out_prefix>.<rank>.npy."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import conftest  # noqa: E402,F401  (puts the repo root and the oracle on sys.path)
import ep_helpers as eh  # noqa: E402


def batch_main(out, seed):
    """Batched MTP decode with the experts split over the ranks (row-invariant arithmetic): every rank
    steps its own two sequences through prompt windows and MTP depth-1 cycles with the group's block in
    every layer, and compares drafts, targets and hidden rows with the single-sequence engine run on
    the same rank with the whole model.  Exit code 0 = every bit equal."""
    import helpers as hp
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = int(os.environ.get("LOCAL_RANK", rank))
    pkg = conftest.load_package()
    from ornith_rs_b200 import ep
    dist.init_process_group("gloo", rank=rank, world_size=world)   # carries the NCCL id only
    ctx = pkg.Context(dev)
    box = [ep.LibEp.unique_id(ctx._lib) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    group = ep.LibEp(ctx, rank, world, box[0], exact=True)
    # the exchanges run over peer memory unless the environment asks for NCCL
    assert group.peer_windows == (os.environ.get("ORN_EP_NCCL") != "1"), "exchange windows were not mapped"
    cfg = hp.tiny_config(pkg.Config)
    gm = hp.upload_model(pkg, ctx, cfg, hp.tiny_model_weights(cfg, seed=seed))
    rng = np.random.default_rng(100 + rank)
    B, NP, CYC = 2, 5, 5
    prompts = rng.integers(0, cfg.vocab, (B, NP)).astype(np.uint32)
    accept = rng.integers(0, 2, (CYC, B)).astype(np.int32)      # the acceptance pattern both sides follow
    # single-sequence engine, whole model on this rank
    want = []
    cache = gm.make_cache()
    for b in range(B):
        cache.reset()
        gm.forward(cache, prompts[b][:NP - 1])
        h = gm.forward(cache, prompts[b][NP - 1:])
        primary = int(gm.head_greedy(h, 1)[0])
        hrow = ctx.upload(h.numpy()[0:1].copy())
        ctx.check(ctx._lib.orn_cache_set_mtp_offset(cache.h, 0), "mtp offset")
        log = []
        for cyc in range(CYC):
            off = ctx._lib.orn_cache_mtp_offset(cache.h)
            draft = gm.mtp_forward(cache, hrow, [primary])
            vh = gm.forward(cache, np.array([primary, draft], np.uint32), capture=True)
            tg = gm.head_greedy(vh, 2)
            k = int(accept[cyc, b])
            cache.rewind(k + 1)
            ctx.check(ctx._lib.orn_cache_set_mtp_offset(cache.h, off + 1), "mtp offset")
            if k:
                gm.mtp_forward(cache, vh, [draft], kv_only=True)
            hrow = ctx.upload(vh.numpy()[k:k + 1].copy())
            log.append((draft, [int(t) for t in tg], vh.numpy().copy()))
            primary = int(tg[k])
        want.append(log)
    cache.free()
    # batched engine over the group
    bt = pkg.Batch(gm, B, t_max=2, cap=64, exact=True)
    for a in range(0, NP - 1, 2):
        bt.forward(prompts[:, a:a + 2], ep=group, want_targets=False)
        bt.commit(np.full(B, 2, np.int32))
    tg, _ = bt.forward(prompts[:, NP - 1:], ep=group)
    bt.commit(np.ones(B, np.int32))
    primary = tg[:, 0].copy()
    ok = True
    for cyc in range(CYC):
        drafts = bt.mtp_draft(primary, ep=group)
        tg, hid = bt.forward(np.stack([primary, drafts], 1), ep=group, want_hidden=True)
        hid = hid.numpy().reshape(B, 2, cfg.hidden)
        bt.commit(accept[cyc] + 1)
        for b in range(B):
            d, t, vh = want[b][cyc]
            ok = ok and int(drafts[b]) == d and [int(v) for v in tg[b]] == t and np.array_equal(hid[b], vh)
            primary[b] = tg[b, accept[cyc, b]]
    np.save("%s.%d.npy" % (out, rank), np.array([1 if ok else 0]))
    dist.barrier()
    bt.free()
    group.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 3)


def main():
    backend, out = sys.argv[1], sys.argv[2]
    if backend == "batch":
        return batch_main(out, int(sys.argv[3]))
    seed, R, H, E, I, k = (int(a) for a in sys.argv[3:9])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    pkg = conftest.load_package()
    from ornith_rs_b200 import ep
    ws = eh.rank_weights(eh.layer_weights(seed, H, E, I), rank, world)
    x = eh.rows_of(seed, rank, R, H)
    if backend in ("lib", "lib-exact"):
        dev = int(os.environ.get("LOCAL_RANK", rank))
        dist.init_process_group("gloo", rank=rank, world_size=world)   # carries the NCCL id only
        ctx = pkg.Context(dev)
        box = [ep.LibEp.unique_id(ctx._lib) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        group = ep.LibEp(ctx, rank, world, box[0], exact=backend == "lib-exact")
        L = {n: pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K) for n, w in ws.items()}
        y = group.moe_block(L, ctx.upload(x), R, k, 1)
        ctx.sync()
        np.save("%s.%d.npy" % (out, rank), y.numpy())
        dist.barrier()
        group.close()
        dist.destroy_process_group()
        return
    if backend == "oracle":
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ops = eh.OracleOps(ws, k, 1)
        xt = torch.from_numpy(x.view(np.int16).copy())
    else:
        dev = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", dev))
        ctx = pkg.Context(dev)
        L = {n: pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K) for n, w in ws.items()}
        ops = ep.CudaOps(ctx, L, k, 1)
        xt = torch.from_numpy(x.view(np.int16).copy()).to(ops.device)
    block = ep.EpMoeBlock(ops, ep.DistComm(dist), E)
    y = block.forward(xt)
    if backend != "oracle":
        ctx.sync()
    np.save("%s.%d.npy" % (out, rank), y.cpu().numpy().view(np.uint16))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
