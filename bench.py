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
LONG_PROMPT = 6621  # the reference's long-prompt measurement (its perplexity text, 6621 tokens, chunks of 2048)


# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised under
# profiles/ (4-layer full-width model: the kernels and their matrices are those of the 40-layer run)
NCU_TRAFFIC_BYTES = {
    "k_norm_gemv M=2 kind=2 8192x2048": 28.61e6,   # add + norm + in_proj: 27.03 MB read + 1.58 MB written
    "k_moe_up M=2 kind=0 512x2048": 19.80e6,       # 16 distinct experts: 18.88 MB read + 0.92 MB written
    "k_moe_down M=2 kind=1 2048x512": 15.79e6,     # 15.06 MB read + 0.73 MB written
}


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


def step_bytes(cfg, T, with_state=True):
    """Algorithmic bytes one trunk forward of T rows must move (weights at their
    format size: Q4_K 144 B and Q6_K 210 B per 256 weights, affine-8 8.5 bit,
    bf16 2 B; gated-delta state read once and written once per row).  with_state=False: the
    weight bytes alone, the quantity the reference's tools/step_bytes.py reports (2.6664 GB per
    token for this mix, tests/golden/step_bytes_golden.json)."""
    H, V = cfg.hidden, cfg.vocab
    a8 = lambda o, k: o * k * 1.0625
    q4 = lambda o, k: o * k * 0.5625
    q6 = lambda o, k: o * k * 0.8203125
    D = 2 * cfg.gdn_k_heads * 128 + cfg.gdn_v_heads * 128
    VD, QD, KVD = cfg.gdn_v_heads * 128, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    n_lin = sum(1 for i in range(cfg.n_layers) if (i + 1) % cfg.full_attn_interval)
    n_att = cfg.n_layers - n_lin
    gdn = a8(D, H) + a8(VD, H) + a8(H, VD) + 2 * cfg.gdn_v_heads * H * 2 + D * 4 * 2
    state = cfg.gdn_v_heads * 128 * 128 * 4 * (1 + T) if with_state else 0
    att = a8(2 * QD, H) + 2 * a8(KVD, H) + a8(H, QD)
    expert = 2 * q4(cfg.expert_inter, H) + q6(H, cfg.expert_inter)
    k, E = cfg.top_k, cfg.n_experts
    distinct = E * (1.0 - (1.0 - k / E) ** T)  # expected distinct routed experts for T rows
    moe = a8(E, H) + distinct * expert + 2 * q4(cfg.shared_inter, H) + q6(H, cfg.shared_inter) + a8(1, H)
    head = a8(V, H)
    return n_lin * (gdn + state) + n_att * att + cfg.n_layers * moe + head


def batch_step_bytes(cfg, B, T, ctx_len, world):
    """Algorithmic bytes ONE GPU moves for one batched MTP cycle of B local sequences (draft pass of
    one row, verify pass of T rows each) at ctx_len cached positions: every dense weight once; this rank's E / world experts of
    every layer once (B * T * top_k routes of the whole job touch every expert); per sequence the
    KV cache of every attention layer once and the gated-delta state once in, T times out."""
    one = step_bytes(cfg, 1, with_state=False)
    H, k, E = cfg.hidden, cfg.top_k, cfg.n_experts
    expert = 2 * cfg.expert_inter * H * 0.5625 + H * cfg.expert_inter * 0.8203125
    dense = one - cfg.n_layers * E * (1.0 - (1.0 - k / E)) * expert       # step_bytes' routed term at T = 1
    n_lin = sum(1 for i in range(cfg.n_layers) if (i + 1) % cfg.full_attn_interval)
    n_att = cfg.n_layers - n_lin
    kv = n_att * 2 * cfg.n_kv_heads * cfg.head_dim * 2 * ctx_len
    state = n_lin * cfg.gdn_v_heads * 128 * 128 * 4 * (1 + T)
    # the draft pass: the bf16 MTP layer (join, attention, router, this rank's experts, shared expert),
    # the lm_head a second time, the head's own KV cache once per sequence
    QD, KVD = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    bf = lambda o, kk: o * kk * 2.0
    mtp = (bf(H, 2 * H) + bf(2 * QD, H) + 2 * bf(KVD, H) + bf(H, QD) + bf(E, H) + ((E // world) + 1) * 3 * bf(cfg.expert_inter, H)
           + cfg.vocab * H * 1.0625 + B * 2 * cfg.n_kv_heads * cfg.head_dim * 2 * ctx_len)
    return dense + cfg.n_layers * (E // world) * expert + B * (kv + state) + mtp


def ep_decode(pkg, ctx, dist, rank, world, model, cfg, steps=8, warmup=3, total_seqs=64, ctx_len=4096, T=2):
    """BASELINE config 5: batched decode of the whole model, 64 sequences in all at 4096 cached
    positions each, every sequence stepping a verify window of 2 rows (MTP depth 1) per pass over
    the weights; sequences split evenly over the ranks (data parallel), the routed experts of every
    layer split E / N per rank (expert parallel) through the library's own block.  Every rank runs
    this.  A step = one MTP depth-1 cycle of every sequence: the MTP head's draft pass (B rows: its
    attention layer over its own cache, its MoE block, lm_head, argmax; drafts back on the host), the
    verify pass (B * 2 rows through the trunk, lm_head, greedy targets back on the host), per-sequence
    acceptance and commit with the Committed re-encode.  Acceptance is the benchmark's forced pattern
    (keep 2 with p, else 1) whatever the head drafted: random weights accept nothing by themselves,
    and traffic and arithmetic do not depend on the outcome.  tokens/s counts kept tokens."""
    from ornith_rs_b200 import ep
    if total_seqs % world or cfg.n_experts % world:
        return None
    B = total_seqs // world
    group = None
    if world > 1:
        box = [ep.LibEp.unique_id(ctx._lib) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        group = ep.LibEp(ctx, rank, world, box[0])
    bt = pkg.Batch(model, B, t_max=T, cap=ctx_len + T * (steps + warmup) + 8)
    bt.fill_random(ctx_len, seed=SEED + rank)
    rng = np.random.default_rng(SEED + 50 + rank)
    ids = [rng.integers(0, cfg.vocab, (B, T)).astype(np.uint32) for _ in range(steps + warmup)]
    keeps = [(1 + (rng.random(B) < FORCE_P)).astype(np.int32) for _ in range(steps + warmup)]

    primary = ids[0][:, 0].copy()

    def step(i):
        # one MTP depth-1 cycle per sequence: draft, verify window [primary, draft], acceptance, commit
        drafts = bt.mtp_draft(primary, ep=group)
        tg, _ = bt.forward(np.stack([primary, drafts], 1), ep=group)
        bt.commit(keeps[i])
        primary[:] = tg[np.arange(B), keeps[i] - 1]
        return tg

    for i in range(warmup):
        step(i)
    ctx.sync()
    if dist is not None:
        dist.barrier()
    l0 = ctx.launches()
    t0 = time.perf_counter()
    ctx.timer_start()
    tokens = 0
    for i in range(warmup, warmup + steps):
        tg = step(i)
        tokens += int(keeps[i].sum())
    ms = ctx.timer_stop()
    wall = time.perf_counter() - t0
    launches = ctx.launches() - l0
    check = int(tg.astype(np.int64).sum())
    if dist is not None:
        import torch
        mx = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
        sm = torch.tensor([float(tokens), float(check)], dtype=torch.float64, device="cuda")
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, wall, tokens, check = float(mx[0]), float(mx[1]), int(sm[0]), int(sm[1])
    bt.free()
    if group is not None:
        group.close()
    peak, which = peaks()
    per_gpu = batch_step_bytes(cfg, B, T, ctx_len, world)
    step_ms = ms / steps
    return {"sequences": total_seqs, "sequences_per_rank": B, "rows_per_step": total_seqs * T, "context": ctx_len,
            "experts_per_rank": cfg.n_experts // world, "layers": cfg.n_layers, "steps": steps, "ms_per_step": step_ms,
            "tokens_per_s": tokens / (ms * 1e-3), "e2e_tokens_per_s": tokens / wall,
            "tokens_per_step": tokens / steps, "bytes_per_gpu_per_step": per_gpu,
            "frac": per_gpu / (step_ms * 1e-3) / 1e9 / peak, "peak_source": which,
            "launches_per_step": int(launches // steps), "h2d_bytes_per_step": B * 4 + B * T * 4 + B * 4,
            "d2h_bytes_per_step": B * 4 + B * T * 4, "targets_checksum": check,
            "scope": "MTP depth-1 cycle: draft pass + verify pass (trunk, lm_head, greedy) + per-sequence commit and re-encode",
            "parallelism": "dp%d over sequences x ep%d over experts" % (world, world),
            "exchange": "none (one rank)" if group is None else
                        ("the library's kernels over peer memory" if group.peer_windows else "NCCL collectives")}


def draft_bytes(cfg, head_rows):
    H = cfg.hidden
    QD, KVD = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    bf = lambda o, k: o * k * 2.0
    expert = 3 * bf(cfg.expert_inter, H)
    return (bf(H, 2 * H) + bf(2 * QD, H) + 2 * bf(KVD, H) + bf(H, QD) + bf(cfg.n_experts, H)
            + (cfg.top_k + 1) * expert + head_rows * H * 1.0625)


def sample_weights_cpu(cfg, seed):
    """Seeded weights of a full-width model in the benchmark's mix, made on the host with numpy
    (name -> oracle Weights / bf16 tensor).  Raw fields are drawn so that the dequantised weights
    are zero-mean with a standard deviation near 0.02, like the GPU-side random-init: the sample
    only has to move the same bytes through the same arithmetic as the real layers."""
    import orn_oracle as orc
    rng = np.random.default_rng(seed)
    bfv = lambda v: np.uint16(np.float32(v).view(np.uint32) >> 16)
    to_bf = lambda a: (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)

    def a8(E, O, K):
        q = rng.integers(0, 256, (E * O, K), dtype=np.uint8)
        g = E * O * (K // 64)
        return orc.Weights(orc.A8, E, O, K, q, np.full(g, bfv(0.07 / 255), np.uint16), np.full(g, bfv(-0.035), np.uint16))

    def q4(E, O, K):
        n = E * O * (K // 256)
        qs = rng.integers(0, 256, (n, 128), dtype=np.uint8)
        sc = rng.integers(4, 9, (n, 8), dtype=np.uint8)           # 6-bit scales 4..8
        mn = np.rint(7.5 * sc).astype(np.uint8)                   # mins that centre the 0..15 codes
        scales = np.zeros((n, 12), np.uint8)
        for j in range(4):
            scales[:, j] = sc[:, j] & 63
            scales[:, j + 4] = mn[:, j] & 63
        for j in range(4, 8):
            scales[:, j + 4] = (sc[:, j] & 0xF) | ((mn[:, j] & 0xF) << 4)
            scales[:, j - 4] |= (sc[:, j] >> 4) << 6
            scales[:, j] |= (mn[:, j] >> 4) << 6
        dm = np.full((n, 2), np.float16(7.2e-4)).view(np.uint16)
        return orc.Weights(orc.Q4K, E, O, K, qs, scales, dm)

    def q6(E, O, K):
        n = E * O * (K // 256)
        w = rng.integers(0, 256, (n, 192), dtype=np.uint8)
        sc = rng.integers(20, 41, (n, 16)).astype(np.int8).view(np.uint8)
        d = np.full(n, np.float16(3.6e-5)).view(np.uint16)
        return orc.Weights(orc.Q6K, E, O, K, w, sc, d)

    def bf(E, O, K):
        # random sign, magnitudes spread over [2^-7, 2^-5): bfloat16 bit patterns straight from the generator
        r = rng.integers(0, 1024, (E * O, K), dtype=np.uint16)
        return orc.Weights(orc.BF16, E, O, K, ((r >> 9) << 15) | (np.uint16(0x3C00) + (r & 511)))

    H, V = cfg.hidden, cfg.vocab
    D = 2 * cfg.gdn_k_heads * 128 + cfg.gdn_v_heads * 128
    VD, QD, KVD = cfg.gdn_v_heads * 128, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    W = {}
    ten = lambda name, n, mean, std: W.__setitem__(name, to_bf(mean + std * rng.standard_normal(n).astype(np.float32)))

    def moe(p, dense):
        f4, f6, f8 = (bf, bf, bf) if dense else (q4, q6, a8)
        W[p + "gate"] = f8(1, cfg.n_experts, H)
        W[p + "switch_mlp.gate_proj"] = f4(cfg.n_experts, cfg.expert_inter, H)
        W[p + "switch_mlp.up_proj"] = f4(cfg.n_experts, cfg.expert_inter, H)
        W[p + "switch_mlp.down_proj"] = f6(cfg.n_experts, H, cfg.expert_inter)
        W[p + "shared_expert.gate_proj"] = f4(1, cfg.shared_inter, H)
        W[p + "shared_expert.up_proj"] = f4(1, cfg.shared_inter, H)
        W[p + "shared_expert.down_proj"] = f6(1, H, cfg.shared_inter)
        W[p + "shared_expert_gate"] = f8(1, 1, H)

    W["embed_tokens"] = a8(1, V, H)
    W["lm_head"] = a8(1, V, H)
    ten("norm.weight", H, 1.0, 0.05)
    for i in range(cfg.n_layers):
        lp = "layers.%d." % i
        ten(lp + "input_layernorm.weight", H, 1.0, 0.05)
        ten(lp + "post_attention_layernorm.weight", H, 1.0, 0.05)
        if (i + 1) % cfg.full_attn_interval != 0:
            a = lp + "linear_attn."
            W[a + "in_proj_qkv"], W[a + "in_proj_z"], W[a + "out_proj"] = a8(1, D, H), a8(1, VD, H), a8(1, H, VD)
            W[a + "in_proj_a.weight"], W[a + "in_proj_b.weight"] = bf(1, cfg.gdn_v_heads, H), bf(1, cfg.gdn_v_heads, H)
            ten(a + "conv1d.weight", D * cfg.gdn_conv_kernel, 0.0, 0.2)
            ten(a + "dt_bias", cfg.gdn_v_heads, 0.0, 0.3)
            ten(a + "A_log", cfg.gdn_v_heads, 0.0, 0.3)
            ten(a + "norm.weight", 128, 1.0, 0.05)
        else:
            a = lp + "self_attn."
            W[a + "q_proj"], W[a + "k_proj"] = a8(1, 2 * QD, H), a8(1, KVD, H)
            W[a + "v_proj"], W[a + "o_proj"] = a8(1, KVD, H), a8(1, H, QD)
            ten(a + "q_norm.weight", cfg.head_dim, 1.0, 0.05)
            ten(a + "k_norm.weight", cfg.head_dim, 1.0, 0.05)
        moe(lp + "mlp.", False)
    lp = "mtp.layers.0."
    ten("mtp.pre_fc_norm_embedding.weight", H, 1.0, 0.05)
    ten("mtp.pre_fc_norm_hidden.weight", H, 1.0, 0.05)
    W["mtp.fc.weight"] = bf(1, H, 2 * H)
    ten("mtp.norm.weight", H, 1.0, 0.05)
    ten(lp + "input_layernorm.weight", H, 1.0, 0.05)
    ten(lp + "post_attention_layernorm.weight", H, 1.0, 0.05)
    W[lp + "self_attn.q_proj.weight"], W[lp + "self_attn.k_proj.weight"] = bf(1, 2 * QD, H), bf(1, KVD, H)
    W[lp + "self_attn.v_proj.weight"], W[lp + "self_attn.o_proj.weight"] = bf(1, KVD, H), bf(1, H, QD)
    ten(lp + "self_attn.q_norm.weight", cfg.head_dim, 1.0, 0.05)
    ten(lp + "self_attn.k_norm.weight", cfg.head_dim, 1.0, 0.05)
    moe(lp + "mlp.", True)
    return W


class _Cfg:
    """The benchmark model's dimensions as a plain object (the CPU arm builds no CUDA context)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def qwen35_dims(n_layers, max_ctx):
    return _Cfg(hidden=2048, n_layers=n_layers, full_attn_interval=4, n_heads=16, n_kv_heads=2, head_dim=256,
                rope_dims=64, rope_theta=1e7, gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128, gdn_conv_kernel=4,
                n_experts=256, top_k=8, expert_inter=512, shared_inter=512, norm_topk_prob=1, vocab=248320,
                rms_eps=1e-6, max_ctx=max_ctx)


def cpu_arm(max_seconds=15.0):
    """The reference's scalar CPU path (the C restatement under oracle/) timed on this host's
    cores; no GPU and no product library involved.  Sample: a 4-layer full-width model (one 3:1
    period of the stack, real layer sizes, full vocabulary, MTP head), weights made on the host.
    Measured: (a) whole MTP depth-1 cycles of that model with the benchmark's forced-draft rule
    (draft level, 2-row verify window through 4 layers, lm_head + greedy for both rows, accept and
    rewind); (b) the 2-row window through its 4 layers alone.  The 40-layer cycle is (a) + 9 x (b):
    the only extrapolation is the layer count."""
    threads = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(threads)  # torchrun sets it to 1 for its workers
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orn_oracle as orc
    orc.lib().orc_set_threads(threads)
    threads = orc.lib().orc_get_threads()
    cfg4 = qwen35_dims(4, 160)
    t_make = time.perf_counter()
    om = orc.Model(cfg4, sample_weights_cpu(cfg4, SEED))
    t_make = time.perf_counter() - t_make
    rng = np.random.default_rng(SEED)
    prompt = rng.integers(0, cfg4.vocab, 4).astype(np.uint32)

    def measure(budget_s, gen):
        """-> (seconds per cycle of the 4-layer model, tokens per cycle, seconds per 2-row 4-layer window)"""
        ar = om.generate(prompt, gen)
        t0 = time.perf_counter()
        toks, st = om.generate_mtp(prompt, 1, gen, policy=1, force=(ar, FORCE_P, SEED))
        t_gen = time.perf_counter() - t0
        assert toks == ar
        # the prompt's prefill and first step are inside t_gen; take them out with a zero-token run
        t0 = time.perf_counter()
        om.generate(prompt, 1)
        t_pre = time.perf_counter() - t0
        cyc = max(st.cycles, 1)
        cache = om.new_cache()
        om.forward(cache, prompt[:2])
        n, t_lay = 0, 0.0
        while n < 2 or t_lay < budget_s * 0.25:
            if n % 60 == 59:  # stay inside the sample model's context
                om.free_cache(cache)
                cache = om.new_cache()
            t0 = time.perf_counter()
            om.forward(cache, prompt[:2])
            t_lay += time.perf_counter() - t0
            n += 1
        om.free_cache(cache)
        return max(t_gen - t_pre, 1e-9) / cyc, gen / cyc, t_lay / n

    t_start = time.perf_counter()
    c4, tpc, l4 = measure(max_seconds, 24)
    value = tpc / (c4 + 9.0 * l4)
    t_multi = time.perf_counter() - t_start
    # the single-thread figure of the same sample (shorter: a scalar core is ~cores x slower)
    orc.lib().orc_set_threads(1)
    t1 = time.perf_counter()
    c4s, tpcs, l4s = measure(max_seconds * 0.3, 3)
    single = tpcs / (c4s + 9.0 * l4s)
    t_single = time.perf_counter() - t1
    orc.lib().orc_set_threads(threads)
    om.free()
    return {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "single_thread_value": single,
            "sample": "C oracle, OpenMP over rows: MTP depth-1 cycles (draft level + 2-row verify + lm_head + accept) of a "
                      "4-layer full-width model timed whole (%.3f s per cycle, %.2f tokens per cycle), plus the 2-row "
                      "window through its 4 layers (%.3f s); 40-layer cycle = cycle + 9 x window: extrapolated from 4 "
                      "of 40 layers; %.1f s of CPU work at %d threads, %.1f s at 1 thread; weights made on the host in "
                      "%.1f s" % (c4, tpc, l4, t_multi, threads, t_single, t_make)}


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
            "traffic": NCU_TRAFFIC_BYTES["k_norm_gemv M=2 kind=2 8192x2048"], "launch_us": per * 1e3, "algorithmic_bytes": alg, "launches_timed": n}


def label_bytes(cfg, label):
    """Algorithmic bytes of one launch with this per-kernel label (kernel, rows M, first job's
    format and shape), or None for bookkeeping kernels.  Expert kernels: expected distinct experts
    of M rows x their format size; the add + norm + mat-vec launches: all jobs of that launch."""
    H, E, k, I = cfg.hidden, cfg.n_experts, cfg.top_k, cfg.expert_inter
    parts = label.split()
    if len(parts) != 4 or not parts[1].startswith("M="):
        return None
    kern, M, kind, shape = parts[0], int(parts[1][2:]), int(parts[2][5:]), parts[3]
    O, K = (int(v) for v in shape.split("x"))
    fb = FMT_BYTES[kind]
    distinct = E * (1.0 - (1.0 - k / E) ** M)
    act = lambda rows, n: rows * n * 2
    if kern == "k_moe_up":
        return distinct * 2 * O * K * fb + act(M, K) + act(M * k, O) + M * E * 2
    if kern == "k_moe_down":
        return (distinct + 1) * O * K * fb + act(M * k + M, K) + act(M, O)
    if kern == "k_norm_gemv":
        VD, QD, KVD = cfg.gdn_v_heads * 128, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        D = 2 * cfg.gdn_k_heads * 128 + VD
        rows = O
        extra = 0.0
        if (O, K) == (D, H):                     # in_proj qkv + z (+ the two bf16 gate rows)
            rows += VD
            extra = 2 * cfg.gdn_v_heads * K * 2.0
        elif (O, K) == (2 * QD, H):              # q + k + v
            rows += 2 * KVD
        elif (O, K) == (E, H):                   # router + shared gate/up (Q4_K or bf16) + shared-expert gate row
            sh = 2 * cfg.shared_inter * K * (FMT_BYTES[0] if kind == 2 else 2.0)
            extra = sh + K * fb
        return rows * K * fb + extra + act(2 * M, K) + act(M, rows)
    return None


def kernel_table(pkg, ctx, model, cache, prompt, ar, cfg, cycle_ms):
    """Per-kernel device times of one whole generation, live (CUDA events on the launching stream
    after every launch, eager launches): for every kernel label its launches, average time, share
    of the decode loop, algorithmic bytes and the fraction of the measured HBM peak it reaches.
    Eager event-to-event times include the gap between launches, so fractions read low."""
    peak, _ = peaks()
    cache.reset()
    ctx.ktime_begin()
    toks, st = pkg.generate_step_mtp(model, cache, prompt, 1, GEN_TOKENS, force=(ar, FORCE_P, SEED))
    table = ctx.ktime_end()
    assert toks == ar
    table = {l: v for l, v in table.items() if " M=4 " not in l and " M=3 " not in l}  # prompt windows are not the decode loop
    rows, total = [], sum(ms for _, ms in table.values())
    for label, (n, ms) in table.items():
        b = label_bytes(cfg, label)
        us = 1e3 * ms / n
        rows.append({"kernel": label, "launches": n, "launch_us": us, "share": ms / total,
                     "bytes": b, "frac": None if b is None else b / (us * 1e-6) / 1e9 / peak})
    rows.sort(key=lambda r: -r["share"])
    return rows


def long_prefill(pkg, ctx, model, cache, cfg):
    """BASELINE config 5's single-sequence prefill: 6621 seeded random ids through orn_prefill in
    the reference's chunks of 2048 rows (generate.rs:25), every projection a wide tensor-core product.
    Device time by CUDA events on the library's stream; wall time includes the upload of the ids."""
    ids = np.random.default_rng(SEED + 1).integers(0, cfg.vocab, LONG_PROMPT).astype(np.uint32)
    cache.reset()
    model.prefill(cache, ids[:600])  # warm-up: scratch allocation, first launches
    def timed(step):
        cache.reset()
        model.prefill(cache, ids[:min(LONG_PROMPT, step + 100)], prefill_step=step)  # scratch of this chunk width
        best_dev, best_wall = None, None
        for _ in range(2):
            cache.reset()
            ctx.sync()
            t0 = time.perf_counter()
            ctx.timer_start()
            model.prefill(cache, ids, prefill_step=step)
            dev = ctx.timer_stop()
            wall = (time.perf_counter() - t0) * 1e3
            best_dev = dev if best_dev is None else min(best_dev, dev)
            best_wall = wall if best_wall is None else min(best_wall, wall)
        return best_dev, best_wall

    best_dev, best_wall = timed(2048)
    one_dev, _ = timed(8192)
    return {"tokens": LONG_PROMPT, "chunk": 2048, "ms": best_dev, "wall_ms": best_wall,
            "tokens_per_s": LONG_PROMPT / (best_dev * 1e-3),
            "ms_one_chunk": one_dev,   # prefill_step 8192: the whole prompt as one chunk (more rows per expert per product)
            "reference_published_s": 4.22, "reference_hardware": "Apple M4 Max (the reference's own figure, other hardware)"}


EP_ROWS = 128  # BASELINE config 5's decode width: 64 sequences x verify width 2


def ep_moe_layer(pkg, ctx, dist, rank, world, exact=False, steps=30, warmup=5):
    """BASELINE config 5's per-layer exchange, run by every rank of the job: one expert-parallel
    MoE decode layer through the library's own block (orn_ep_moe_block): 128 rows in all, split
    evenly over the ranks; 256 experts top-8 (Q4_K gate/up, Q6_K down) split 256 / N per rank;
    router, shared expert and its gate replicated.  The total work is fixed (strong scaling).
    `checksum` sums every output element's bits over all ranks: the same number at every N, because
    every product is the row-invariant mat-vec and the combine runs at the row's home."""
    from ornith_rs_b200 import ep
    H, E, I, k = 2048, 256, 512, 8
    if EP_ROWS % world or E % world:
        return None
    Rr = EP_ROWS // world
    kinds = {"gate": (pkg.A8, 1, E, H), "sw_gate": (pkg.Q4K, E, I, H), "sw_up": (pkg.Q4K, E, I, H),
             "sw_down": (pkg.Q6K, E, H, I), "sh_gate": (pkg.Q4K, 1, I, H), "sh_up": (pkg.Q4K, 1, I, H),
             "sh_down": (pkg.Q6K, 1, H, I), "sh_egate": (pkg.A8, 1, 1, H)}
    L = {}
    for i, (name, (kind, e, o, kk)) in enumerate(kinds.items()):
        full = pkg.Linear.random(ctx, kind, e, o, kk, SEED + 100 + i)     # the same tensor on every rank
        if name.startswith("sw_") and world > 1:
            L[name] = ep.shard_experts(ctx, full, rank, world)
            full.free()
        else:
            L[name] = full
    uid = None
    if world > 1:
        box = [ep.LibEp.unique_id(ctx._lib) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]
    group = ep.LibEp(ctx, rank, world, uid, exact=exact)
    rng = np.random.default_rng(SEED + 7)
    x_all = (rng.standard_normal((EP_ROWS, H)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    x = ctx.upload(x_all[rank * Rr:(rank + 1) * Rr])
    out = ctx.empty((Rr, H), np.uint16)
    for _ in range(warmup):
        group.moe_block(L, x, Rr, k, 1, out=out)
    ctx.sync()
    if dist is not None:
        dist.barrier()
    l0 = ctx.launches()
    ctx.timer_start()
    for _ in range(steps):
        group.moe_block(L, x, Rr, k, 1, out=out)
    ms = ctx.timer_stop() / steps
    launches = (ctx.launches() - l0) // steps
    check = int(out.numpy().astype(np.int64).sum())
    if dist is not None:
        import torch
        t = torch.tensor([ms, float(check)], dtype=torch.float64, device="cuda")
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, check = float(mx[0]), int(t[1])
    group.close()
    for l in L.values():
        l.free()
    peak, which = peaks()
    expert = 2 * I * H * 0.5625 + H * I * 0.8203125
    per_gpu = (E // world) * expert + expert + E * H * 1.0625 + H * 1.0625 + 3 * Rr * H * 2
    return {"rows": EP_ROWS, "rows_per_rank": Rr, "experts_per_rank": E // world, "ms_per_layer": ms,
            "rows_per_s": EP_ROWS / (ms * 1e-3), "bytes_per_gpu": per_gpu, "frac": per_gpu / (ms * 1e-3) / 1e9 / peak,
            "peak_source": which, "launches_per_layer": int(launches), "checksum": check,
            "routed_experts": "grouped row-invariant mat-vec (bits of the single-GPU block)" if exact
                              else "grouped tensor-core product (tcgen05), routing and combine row-invariant",
            "collectives": "none (one rank)" if world == 1 else
                           "rows and routing indices stored into every rank's window, expert outputs stored into their home "
                           "rank's window (the library's kernels over peer memory, flags with bounded waits)" if group.peer_windows else
                           "all-gather of routing indices and rows, all-to-all of fixed return blocks (NCCL, library stream)"}


def oracle_check(pkg, ctx):
    """The decode loop's integers against the CPU oracle on a 4-layer full-width model (the
    oracle is the checker here): emitted ids and accepted count at the benchmark's p."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orn_oracle as orc
    cfg4 = pkg.qwen35_config(max_ctx=96, n_layers=4)
    gm = pkg.TextModel(ctx, cfg4)
    gm.init_random(SEED)
    gm.make_cache().free()
    om = orc.export_gpu_model(gm)
    prompt = np.random.default_rng(SEED).integers(0, cfg4.vocab, 6).astype(np.uint32)
    n = 16
    ar = om.generate(prompt, n)
    ref, rst = om.generate_mtp(prompt, 1, n, policy=1, force=(ar, FORCE_P, SEED))
    c = gm.make_cache()
    got, gst = pkg.generate_step_mtp(gm, c, prompt, 1, n, force=(ar, FORCE_P, SEED))
    ok = got == ref == ar and (gst.cycles, gst.drafted, gst.accepted) == (rst.cycles, rst.drafted, rst.accepted)
    c.free()
    gm.free()
    om.free()
    assert ok, "decode loop differs from the CPU oracle on the 4-layer full-width sample"
    return {"model": "4 full-width layers + MTP head + full vocabulary", "tokens": n, "p": FORCE_P,
            "cycles": gst.cycles, "accepted": gst.accepted, "oracle_accepted": rst.accepted, "equal": True}


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
    cfg = pkg.qwen35_config(max_ctx=max(LONG_PROMPT + 64, PROMPT_LEN + GEN_TOKENS + 64), n_layers=args.n_layers)
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
    launch_index = ctx.launches()   # kernels launched before the timed region (where a profiler's capture window starts)
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
    epl = ep_moe_layer(pkg, ctx, dist, rank, world)   # every rank takes part
    if epl is not None:
        epl["row_invariant_variant"] = ep_moe_layer(pkg, ctx, dist, rank, world, exact=True)
    epd = ep_decode(pkg, ctx, dist, rank, world, model, cfg) if cfg.n_layers == 40 or args.ep_decode else None
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, which = peaks()
    iso = kernel_roofline(pkg, ctx, model, cfg)
    kt = kernel_table(pkg, ctx, model, cache, prompt, ar, cfg, dev_ms / max(cycles, 1))
    # the roofline object names the kernel with the largest share of the decode loop
    top = next(r for r in kt if r["bytes"] is not None)
    roof = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["frac"] * peak, "peak": peak, "peak_source": which,
            "unit": "GB/s", "frac": top["frac"], "traffic": NCU_TRAFFIC_BYTES.get(top["kernel"]),
            "launch_us": top["launch_us"], "algorithmic_bytes": top["bytes"], "launches_timed": top["launches"],
            "share_of_decode_loop": top["share"],
            "timing": "CUDA events on the launching stream after every launch of one whole generation (eager)"}
    lp = long_prefill(pkg, ctx, model, cache, cfg) if cfg.n_layers == 40 or args.long_prefill else None
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
        "gpu_launches": launches, "launches_before_timed_region": int(launch_index), "clocks": clocks, "roofline": roof, "step_roofline": step_roof,
        "kernels": kt[:12], "isolated_in_proj_launch": iso, "prefill_6621": lp, "ep_moe_layer": epl, "ep_decode": epd,
        "acceptance": accepted / max(cycles, 1), "tokens_per_cycle": args.steps * GEN_TOKENS / max(cycles, 1),
        "mtp_equals_autoregressive": True, "prefill_ms_per_step": prefill_ms / args.steps,
    }
    if world == 1 and not args.no_cpu:
        line["oracle_check"] = oracle_check(pkg, ctx)
        line["cpu_baseline"] = cpu_arm()
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
    """The reference's own CPU statement of the path (its Metal path cannot run on Linux): the C
    restatement under oracle/, all host threads.  Builds no CUDA context and loads no product
    library: the sample's weights are made on the host."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_arm(max_seconds=max(10.0, 6.0 * args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": GEN_TOKENS / cb["value"] * 1e3, "ms_per_step_is": "extrapolated from the bounded sample",
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": "BASELINE config 4 (bounded sample, see cpu_baseline.sample)"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


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
    ap.add_argument("--n-layers", type=int, default=40, help="fewer layers at the full layer sizes (profiling runs)")
    ap.add_argument("--long-prefill", action="store_true", help="run the 6621-token prefill leg at any layer count")
    ap.add_argument("--ep-decode", action="store_true", help="run the batched expert-parallel decode leg at any layer count")
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
