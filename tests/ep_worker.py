"""One rank of the expert-parallel MoE block under torch.distributed.
Usage: python ep_worker.py <oracle|cuda|lib|lib-exact> <out_prefix> <seed> <R> <H> <E> <I> <k>
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


def main():
    backend, out = sys.argv[1], sys.argv[2]
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
