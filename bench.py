"""Benchmark: MTP depth-1 greedy speculative decode of a random-init
Qwen3.5-MoE 35B-A3B (k-quant mix) at batch 1, on N GPUs of one node.

  python bench.py --gpus 1 --steps 5 --warmup 3
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
  python bench.py --impl reference      (the CPU restatement on the host cores)

One "step" is one 200-token generation from a 51-token prompt (BASELINE config
4: drafts forced to the target with probability p so that acceptance is
controlled).  `value` is generated tokens / device time of the decode loop
(CUDA events on the library's stream, weights and caches resident in HBM).
`e2e` is generated tokens / host wall-clock of the whole public call
`orn_generate_step_mtp` (prompt upload, prefill, every per-cycle device->host
read of targets and drafts included).  At N > 1 every rank decodes its own
sequence on a replica ("weak" scaling); there is no data-path collective.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "MTP-depth-1 decode tok/s (35B-A3B k-quant, batch 1)"
PROMPT_LEN, GEN_TOKENS, FORCE_P, SEED = 51, 200, 0.5, 20240611


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the kernel above, from the ncu
# capture summarised in profiles/
NCU_TRAFFIC_BYTES = 28.60e6  # profiles/fused_kernels_ncu_profile_step_4layer.md: 27.06 MB read + 1.54 MB written


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def load_pkg():
    import __graft_entry__ as ge
    return ge.load_package()


def step_bytes(cfg, T):
    """Algorithmic bytes one trunk forward of T rows must move (weights at their
    format size: Q4_K 144 B and Q6_K 210 B per 256 weights, affine-8 8.5 bit,
    bf16 2 B; gated-delta state read once and written once per row)."""
    H, V = cfg.hidden, cfg.vocab
    a8 = lambda o, k: o * k * 1.0625
    q4 = lambda o, k: o * k * 0.5625
    q6 = lambda o, k: o * k * 0.8203125
    D = 2 * cfg.gdn_k_heads * 128 + cfg.gdn_v_heads * 128
    VD, QD, KVD = cfg.gdn_v_heads * 128, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    n_lin = sum(1 for i in range(cfg.n_layers) if (i + 1) % cfg.full_attn_interval)
    n_att = cfg.n_layers - n_lin
    gdn = a8(D, H) + a8(VD, H) + a8(H, VD) + 2 * cfg.gdn_v_heads * H * 2 + D * 4 * 2
    state = cfg.gdn_v_heads * 128 * 128 * 4 * (1 + T)
    att = a8(2 * QD, H) + 2 * a8(KVD, H) + a8(H, QD)
    expert = 2 * q4(cfg.expert_inter, H) + q6(H, cfg.expert_inter)
    k, E = cfg.top_k, cfg.n_experts
    distinct = E * (1.0 - (1.0 - k / E) ** T)  # expected distinct routed experts for T rows
    moe = a8(E, H) + distinct * expert + 2 * q4(cfg.shared_inter, H) + q6(H, cfg.shared_inter) + a8(1, H)
    head = a8(V, H)
    return n_lin * (gdn + state) + n_att * att + cfg.n_layers * moe + head


def draft_bytes(cfg, head_rows):
    H = cfg.hidden
    QD, KVD = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    bf = lambda o, k: o * k * 2.0
    expert = 3 * bf(cfg.expert_inter, H)
    return (bf(H, 2 * H) + bf(2 * QD, H) + 2 * bf(KVD, H) + bf(H, QD) + bf(cfg.n_experts, H)
            + (cfg.top_k + 1) * expert + head_rows * H * 1.0625)


def cpu_arm(pkg, ctx, max_seconds=15.0):
    """The reference's scalar CPU path (the C restatement under oracle/) timed on
    this host.  Sample: one 3:1 period of the stack (4 of 40 layers, real layer
    sizes) plus the MTP head and the full lm_head, MTP depth-1 cycles with the
    same forced-draft rule; the per-cycle layer time is scaled by 10 to the 40
    layers."""
    threads = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(threads)  # torchrun sets it to 1 for its workers
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orn_oracle as orc
    orc.lib().orc_set_threads(threads)
    threads = orc.lib().orc_get_threads()

    cfg4 = pkg.qwen35_config(max_ctx=128, n_layers=4)
    gm = pkg.TextModel(ctx, cfg4)
    gm.init_random(SEED)
    gm.make_cache().free()  # resolves the weight table
    om = orc.export_gpu_model(gm)
    gm.free()
    rng = np.random.default_rng(SEED)
    ids = rng.integers(0, cfg4.vocab, 2).astype(np.uint32)
    cache = om.new_cache()
    om.forward(cache, ids[:1])  # warm
    t_layers, t_head, n = 0.0, 0.0, 0
    t_start = time.perf_counter()
    while n < 3 or time.perf_counter() - t_start < max_seconds:
        t0 = time.perf_counter()
        h = om.forward(cache, ids)                      # a 2-row verify window through 4 layers
        t1 = time.perf_counter()
        om.head_greedy(h, 2)                            # lm_head + greedy for both rows
        t2 = time.perf_counter()
        t_layers += t1 - t0
        t_head += t2 - t1
        n += 1
        if n % 40 == 0:  # stay inside the sample model's 128-token context
            om.free_cache(cache)
            cache = om.new_cache()
    om.free_cache(cache)
    om.free()
    verify_s = 10.0 * t_layers / n + t_head / n
    # draft level: MTP head is one attention layer with bf16 weights + lm_head row: bounded by head time / 2
    draft_s = t_head / n / 2 + (t_layers / n) / 4
    tok_per_cycle = 1.0 + FORCE_P
    value = tok_per_cycle / (verify_s + draft_s)
    return {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": "%d verify windows (T=2) through 4 of 40 layers + full lm_head on the C oracle with "
                      "OpenMP over rows; layer time x10, draft level estimated from the same parts; "
                      "%.1f s of CPU work" % (n, time.perf_counter() - t_start)}


FMT_BYTES = {0: 144.0 / 256, 1: 210.0 / 256, 2: 1.0625, 3: 2.0}  # Q4_K, Q6_K, affine-8 g64, bf16 bytes per weight


def kernel_roofline(pkg, ctx, model, cfg, iters=20):
    """The dominant kernel of the timed region: the persistent norm + dequant
    mat-vec kernel (k_norm_gemv) at verify width 2 on a gated-delta layer's four
    input projections (qkv [8192,2048], z [4096,2048] affine-8; a, b [32,2048]
    bf16), launched through orn_add_norm_gemv exactly as the decode step does.
    The launches cycle through the 30 layers' matrices (0.8 GB > L2) so that
    every launch reads its weights from HBM.  achieved = algorithmic bytes of
    one launch / average launch time (CUDA events on the launching stream)."""
    M = 2
    layers = [i for i in range(cfg.n_layers) if (i + 1) % cfg.full_attn_interval]
    sets = []
    for i in layers:
        p = "layers.%d.linear_attn." % i
        sets.append([model.get_linear(p + n) for n in ("in_proj_qkv", "in_proj_z", "in_proj_a.weight", "in_proj_b.weight")])
    rng = np.random.default_rng(1)
    to_bf = lambda v: (v.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    a = ctx.upload(to_bf(rng.standard_normal((M, cfg.hidden))))
    b = ctx.upload(to_bf(rng.standard_normal((M, cfg.hidden))))
    w = ctx.upload(to_bf(1.0 + 0.05 * rng.standard_normal(cfg.hidden)))
    outs = [ctx.empty((M, L.O), np.uint16) for L in sets[0]]
    import ctypes as C
    out_arr = (C.c_void_p * 4)(*[o.ptr for o in outs])
    lin_arrs = [(C.c_void_p * 4)(*[L.h for L in ls]) for ls in sets]
    lib = ctx._lib

    def launch(la):
        ctx.check(lib.orn_add_norm_gemv(ctx.h, a.ptr, b.ptr, w.ptr, M, cfg.hidden, 1e-6, la, out_arr, 4, None, None),
                  "orn_add_norm_gemv")

    for la in lin_arrs:  # warm-up
        launch(la)
    ctx.timer_start()
    n = 0
    for _ in range(iters):
        for la in lin_arrs:
            launch(la)
            n += 1
    ms = ctx.timer_stop()
    per = ms / n
    alg = sum(L.O * L.K * FMT_BYTES[L.kind] for L in sets[0])      # weights at their format size
    alg += 2 * M * cfg.hidden * 2 + cfg.hidden * 2                  # two addends and the norm weight
    alg += sum(M * L.O * 2 for L in sets[0])                        # bf16 outputs
    peak, which = peaks()
    ach = alg / (per * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": "k_norm_gemv<M=2> add+rms_norm + in_proj_{qkv,z,a,b} [12352x2048]",
            "achieved": ach, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": ach / peak,
            "traffic": NCU_TRAFFIC_BYTES, "launch_us": per * 1e3, "algorithmic_bytes": alg, "launches_timed": n}


def reduce_max_over_ranks(values, dist, device):
    """Element-wise maximum of `values` over all ranks (the slowest rank times the job).
    `dist` is torch.distributed after init_process_group, or None for one process."""
    if dist is None:
        return list(values)
    import torch
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_rates(world, steps, gen_tokens, dev_ms, wall_s):
    """Replica per GPU (weak scaling): every rank generates steps x gen_tokens tokens; the job's
    rate is all ranks' tokens over the slowest rank's time.  Returns (device-timed, end-to-end)."""
    total_tokens = world * steps * gen_tokens
    return total_tokens / (dev_ms * 1e-3), total_tokens / wall_s


def ours(args):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_pkg()
    ctx = pkg.Context(local)
    cfg = pkg.qwen35_config(max_ctx=512)
    model = pkg.TextModel(ctx, cfg)
    model.init_random(SEED)
    cache = model.make_cache()
    rng = np.random.default_rng(SEED + rank)
    prompt = rng.integers(0, cfg.vocab, PROMPT_LEN).astype(np.uint32)
    # the non-speculative stream: the target the forced drafts come from, and the parity check
    ar = pkg.generate_step(model, cache, prompt, GEN_TOKENS)
    ar_prof = model.prof()

    def one():
        cache.reset()
        t0 = time.perf_counter()
        toks, st = pkg.generate_step_mtp(model, cache, prompt, 1, GEN_TOKENS, force=(ar, FORCE_P, SEED))
        wall = time.perf_counter() - t0
        return toks, st, model.prof(), wall

    for _ in range(args.warmup):
        toks, st, _, _ = one()
        assert toks == ar, "speculative output differs from the autoregressive output"

    def barrier():
        ctx.sync()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    dev_ms, walls, launches, cycles, accepted, prefill_ms = 0.0, 0.0, 0, 0, 0, 0.0
    for _ in range(args.steps):
        toks, st, prof, wall = one()
        dev_ms += prof.total_ms
        prefill_ms += prof.prefill_ms
        walls += wall
        launches += prof.kernel_launches
        cycles += st.cycles
        accepted += st.accepted
    barrier()
    clocks = sampler.stop()
    assert toks == ar

    dev_ms, walls = reduce_max_over_ranks([dev_ms, walls], dist, "cuda")
    value, e2e = whole_job_rates(world, args.steps, GEN_TOKENS, dev_ms, walls)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    roof = kernel_roofline(pkg, ctx, model, cfg)
    peak, which = peaks()
    vb, db = step_bytes(cfg, 2), draft_bytes(cfg, cfg.vocab)
    cyc_s = dev_ms * 1e-3 / max(cycles, 1)
    step_roof = {"bytes_per_cycle": vb + db, "verify_bytes": vb, "draft_bytes": db,
                 "cycle_ms": cyc_s * 1e3, "achieved_gbs": (vb + db) / cyc_s / 1e9,
                 "frac": (vb + db) / cyc_s / 1e9 / peak, "peak_source": which,
                 "ar_ms_per_token": ar_prof.total_ms / GEN_TOKENS,
                 "ar_frac": step_bytes(cfg, 1) / (ar_prof.total_ms * 1e-3 / GEN_TOKENS) / 1e9 / peak}
    cache.free()
    model.free()
    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate",
        "data": "synthetic (random-init weights, random prompt ids)",
        "config": {"workload": "BASELINE config 4: 40-layer 35B-A3B, Q4_K/Q6_K experts + affine-8 dense + bf16 MTP head, "
                               "51-token prompt, 200 greedy tokens, MTP depth 1, forced-draft p=%.2f; value = decode loop "
                               "(200 tokens) on the device, e2e = the whole call on the host clock including the "
                               "prompt upload, the 51-token prefill and the per-cycle readback" % FORCE_P,
                   "l2_policy": "weights read per step (2.7 GB) exceed L2 (126 MB)", "parallelism": "replica per GPU"},
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": PROMPT_LEN * 4,
                "d2h_bytes_per_step": int(16 * cycles / args.steps) + 4},
        "gpu_launches": launches, "clocks": clocks, "roofline": roof, "step_roofline": step_roof,
        "acceptance": accepted / max(cycles, 1), "tokens_per_cycle": args.steps * GEN_TOKENS / max(cycles, 1),
        "mtp_equals_autoregressive": True, "prefill_ms_per_step": prefill_ms / args.steps,
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_arm(pkg, ctx)
    emit(line)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


def ep_layer(args):
    """Second workload (`--workload ep-layer`): one MoE decode layer in expert-parallel form at
    BASELINE config 5's decode width (64 sequences x verify width 2 = 128 rows in all, split evenly
    over the ranks; experts 256/N per rank; dispatch and return all-to-all over NCCL).  The total
    work is fixed, so scaling is strong.  `checksum` is a sum over every output element of every
    rank: it must be the same number at every N (the block's bits do not depend on N)."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_pkg()
    from ornith_rs_b200 import ep
    ctx = pkg.Context(local)
    H, E, I, k, ROWS = 2048, 256, 512, 8, 128
    assert ROWS % world == 0 and E % world == 0
    R = ROWS // world
    kinds = {"gate": (pkg.A8, 1, E, H), "sw_gate": (pkg.Q4K, E, I, H), "sw_up": (pkg.Q4K, E, I, H),
             "sw_down": (pkg.Q6K, E, H, I), "sh_gate": (pkg.Q4K, 1, I, H), "sh_up": (pkg.Q4K, 1, I, H),
             "sh_down": (pkg.Q6K, 1, H, I), "sh_egate": (pkg.A8, 1, 1, H)}
    L = {}
    for i, (name, (kind, e, o, kk)) in enumerate(kinds.items()):
        full = pkg.Linear.random(ctx, kind, e, o, kk, SEED + i)     # the same tensor on every rank
        if name.startswith("sw_") and world > 1:
            L[name] = ep.shard_experts(ctx, full, rank, world)
            full.free()
        else:
            L[name] = full
    ops = ep.CudaOps(ctx, L, k, 1)
    comm = ep.DistComm(dist) if dist is not None else ep.SelfComm()
    block = ep.EpMoeBlock(ops, comm, E)
    rng = np.random.default_rng(SEED)
    x_all = (rng.standard_normal((ROWS, H)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    x_host = torch.from_numpy(x_all[rank * R:(rank + 1) * R].view(np.int16).copy()).pin_memory()

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    x_dev = x_host.to(ops.device)
    for _ in range(args.warmup):
        y = block.forward(x_dev)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    l0 = ctx.launches()
    ctx.timer_start()
    for _ in range(args.steps):
        y = block.forward(x_dev)
    dev_ms = ctx.timer_stop()
    launches = ctx.launches() - l0
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        with ops.run():   # upload, block and readback all on the context's stream
            y_host = block.forward(x_host.to(ops.device, non_blocking=True)).cpu()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    check = torch.tensor([int(y_host.to(torch.int64).bitwise_and(0xffff).sum())], dtype=torch.int64, device=ops.device)
    if dist is not None:
        dist.all_reduce(check)
    dev_ms, wall = reduce_max_over_ranks([dev_ms, wall], dist, "cuda")
    if rank == 0:
        rows = ROWS * args.steps
        emit({
            "metric": "ep_moe_layer_rows_per_s", "value": rows / (dev_ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate",
            "data": "synthetic (random-init weights, N(0,1) rows)",
            "config": {"workload": "one expert-parallel MoE decode layer: 128 rows (BASELINE config 5: 64 sequences x "
                                   "width 2), hidden 2048, 256 experts top-8 (Q4_K gate/up, Q6_K down) split %d per rank, "
                                   "shared expert + router replicated; all-gather of routing, dispatch and return "
                                   "all-to-all (NCCL)" % (E // world),
                       "l2_policy": "routed weights read per step (about 1 GB over all ranks) exceed L2",
                       "parallelism": "ep%d" % world},
            "e2e": {"value": rows / wall, "unit": "rows/s", "h2d_bytes_per_step": R * H * 2,
                    "d2h_bytes_per_step": R * H * 2 + R * k * 4},
            "gpu_launches": launches, "clocks": clocks, "checksum": int(check.item()),
        })
    # the context (and its stream) stays open until the process ends: torch buffers that were used
    # on that stream are still alive here, and freeing them after the stream is gone is an error
    ctx.sync()
    if dist is not None:
        dist.destroy_process_group()


def reference(args):
    """The reference's own CPU statement of the path (its Metal path cannot run
    on Linux): the C restatement under oracle/, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pkg = load_pkg()
    try:
        ctx = pkg.Context(0)
    except Exception as e:  # the weights of the sample are generated on the GPU
        emit({"impl": "reference", "unavailable": "no CUDA device to generate the sample weights: %s" % e})
        return
    cb = cpu_arm(pkg, ctx, max_seconds=max(10.0, 8.0 * args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": GEN_TOKENS / cb["value"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": "BASELINE config 4 (bounded sample, see cpu_baseline.sample)"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)
    ctx.close()


_RESULT_FD = None


def emit(line):
    """The one JSON line, on the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # Libraries write banners to stdout (NCCL prints its version there): from here on file
    # descriptor 1 is stderr, and only `emit` writes to the original stdout.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--gen-tokens", type=int, default=200, help="tokens per generation (profiling runs use fewer)")
    ap.add_argument("--prompt-len", type=int, default=51)
    ap.add_argument("--workload", default="decode", choices=["decode", "ep-layer"],
                    help="decode: the MTP depth-1 decode loop (the headline); ep-layer: one expert-parallel MoE layer")
    args = ap.parse_args()
    global GEN_TOKENS, PROMPT_LEN
    GEN_TOKENS, PROMPT_LEN = args.gen_tokens, args.prompt_len
    if args.impl == "reference":
        reference(args)
    elif args.workload == "ep-layer":
        ep_layer(args)
    else:
        ours(args)


if __name__ == "__main__":
    main()
