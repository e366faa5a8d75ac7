"""Generates the golden fixtures from the reference's own numpy tools.

Run where the reference tree is mounted:
    python tests/golden/make_golden.py /path/to/ornith-rs
It imports tools/q4k.py and tools/aq.py from that tree (the only importable
pieces of the reference's arithmetic) and writes small .npz files next to this
script.  The tests read only the .npz files.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "tools"))
    import aq
    import q4k

    rng = np.random.default_rng(20240607)

    # 1. Q4_K field packing: 8 scales + 8 mins <-> 12 bytes
    sc = rng.integers(0, 64, (64, 8)).astype(np.uint8)
    mn = rng.integers(0, 64, (64, 8)).astype(np.uint8)
    packed = q4k.put_scale_min_k4(sc, mn)
    for j in range(8):
        d, m = q4k.get_scale_min_k4(j, packed)
        assert np.array_equal(d, sc[:, j]) and np.array_equal(m, mn[:, j])

    # 2. Q4_K quantise + dequantise of real-looking weights, and of raw random blocks
    w = (rng.standard_t(4, (24, 256)) * 0.015).astype(np.float32)
    blocks_q = q4k.quantize(w)
    deq_q = q4k.dequantize(blocks_q)
    blocks_r = rng.integers(0, 256, (24, q4k.BLOCK_BYTES)).astype(np.uint8)
    # keep d and dmin finite, positive halves
    dm = (np.abs(rng.standard_normal((24, 2))) * 1e-3).astype(np.float16)
    blocks_r[:, 0:4] = dm.view(np.uint8).reshape(24, 4)
    deq_r = q4k.dequantize(blocks_r)
    qs_q, scales_q, dm_q = q4k.split(blocks_q, 24, 1)
    qs_r, scales_r, dm_r = q4k.split(blocks_r, 24, 1)
    np.savez_compressed(
        os.path.join(HERE, "q4k_golden.npz"),
        sc=sc, mn=mn, packed=packed, w=w,
        blocks_q=blocks_q, deq_q=deq_q, qs_q=qs_q, scales_q=scales_q, dm_q=dm_q.view(np.uint16),
        blocks_r=blocks_r, deq_r=deq_r, qs_r=qs_r, scales_r=scales_r, dm_r=dm_r.view(np.uint16))

    # 2b. Q6_K artifact layout: raw 210-byte ggml blocks (ql 128, qh 64, scales 16, d 2) cut into the three
    # tensors an artifact stores by the reference's own split (tools/q4k.py:75-96): ql|qh together, the
    # int8 sub-block scales, one float16 d per block
    rng6 = np.random.default_rng(20240608)   # a stream of its own: the other fixtures keep their values
    blocks6 = rng6.integers(0, 256, (24 * 2, 210)).astype(np.uint8)
    d6 = (np.abs(rng6.standard_normal(24 * 2)) * 1e-3).astype(np.float16)
    blocks6[:, 208:210] = d6.view(np.uint8).reshape(-1, 2)
    qs6, scales6, dm6 = q4k.split(blocks6, 24, 2, kind="q6_K")
    np.savez_compressed(os.path.join(HERE, "q6k_golden.npz"), blocks=blocks6, qs=qs6, scales=scales6,
                        dm=dm6.view(np.uint16))

    # 2c. the FR-Spec id file as the reference's own tool writes it (tools/merge_frspec.py write_ids: the
    # module needs a tokenizer at import, so only its two file functions and its constants are taken)
    import ast
    import tempfile as _tf
    tree = ast.parse(open(os.path.join(ref_root, "tools", "merge_frspec.py")).read())
    keep = [n for n in tree.body
            if isinstance(n, ast.Import)
            or (isinstance(n, ast.FunctionDef) and n.name in ("read_ids", "write_ids"))
            or (isinstance(n, ast.Assign) and any(getattr(t, "id", "") == "VOCAB" for t in n.targets))]
    ns = {}
    exec(compile(ast.Module(keep, []), "merge_frspec_subset", "exec"), ns)
    rngf = np.random.default_rng(20240609)
    ids_in = rngf.integers(0, 248320, 300).astype(np.uint32)
    ids_in[10:20] = ids_in[0:10]                     # duplicates, unsorted: the tool sorts and dedupes
    with _tf.TemporaryDirectory() as td:
        n_written = ns["write_ids"](os.path.join(td, "ids.bin"), ids_in.tolist())
        raw = open(os.path.join(td, "ids.bin"), "rb").read()
        assert ns["read_ids"](os.path.join(td, "ids.bin")) == sorted(set(int(i) for i in ids_in))
    np.savez_compressed(os.path.join(HERE, "frspec_ids_golden.npz"), ids_in=ids_in, file_bytes=np.frombuffer(raw, np.uint8),
                        n=np.int64(n_written))

    # 3. affine 8-bit group-64 quantise + pack
    wa = (rng.standard_normal((16, 256)) * 0.02).astype(np.float32)
    q, s, b = aq.quantize(wa, group_size=64, bits=8)
    words = aq.pack(q, 8, 256 // 4)
    deq = (s[:, None] * q.astype(np.float32) + b[:, None]).reshape(16, 256)
    np.savez_compressed(os.path.join(HERE, "a8_golden.npz"), w=wa, q=q.reshape(16, 256), scales=s.reshape(16, 4),
                        biases=b.reshape(16, 4), words=words, deq=deq)

    # 3b. affine 4-bit group-32 quantise + pack (the artifact's default mode)
    q4, s4, b4 = aq.quantize(wa, group_size=32, bits=4)
    words4 = aq.pack(q4, 4, 256 // 8)
    deq4 = (s4[:, None] * q4.astype(np.float32) + b4[:, None]).reshape(16, 256)
    np.savez_compressed(os.path.join(HERE, "a4_golden.npz"), w=wa, q=q4.reshape(16, 256), scales=s4.reshape(16, 8),
                        biases=b4.reshape(16, 8), words=words4, deq=deq4)

    # 4. bfloat16 rounding as the tool states it (ties to even)
    xs = rng.standard_normal(4096).astype(np.float32) * np.float32(10.0) ** rng.integers(-6, 6, 4096)
    np.savez_compressed(os.path.join(HERE, "bf16_golden.npz"), x=xs.astype(np.float32), r=aq.bf16(xs))
    # 5. weight bytes one decode step reads, by the reference's own accounting tool run on
    # header-only artifacts (tools/step_bytes.py reads shapes and dtypes, never the data)
    import json
    import re
    import subprocess
    import tempfile
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
    import helpers as hp

    class Dims:
        hidden, n_layers, full_attn_interval, n_heads, n_kv_heads, head_dim = 2048, 40, 4, 16, 2, 256
        gdn_k_heads, gdn_v_heads, gdn_head_dim, gdn_conv_kernel = 16, 32, 128, 4
        n_experts, top_k, expert_inter, shared_inter, vocab = 256, 8, 512, 512, 248320

    out = {}
    for mix in ("benchmark", "published"):
        with tempfile.TemporaryDirectory() as tmp:
            art = os.path.join(tmp, "art-" + mix)
            os.makedirs(art)
            inv = hp.artifact_inventory(Dims, mix)
            header, off = {}, 0
            size = {"BF16": 2, "F16": 2, "U32": 4, "U8": 1, "I8": 1}
            for name, (dt, shape) in inv.items():
                n = int(np.prod(shape)) * size[dt]
                header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + n]}
                off += n
            hj = json.dumps(header).encode()
            with open(os.path.join(art, "model.safetensors"), "wb") as f:
                f.write(len(hj).to_bytes(8, "little") + hj)
            json.dump({"weight_map": {n: "model.safetensors" for n in inv}}, open(os.path.join(art, "model.safetensors.index.json"), "w"))
            json.dump({"text_config": {"num_experts": Dims.n_experts, "num_experts_per_tok": Dims.top_k, "vocab_size": Dims.vocab},
                       "quantization": {"group_size": 32, "bits": 4, "mode": "affine"}}, open(os.path.join(art, "config.json"), "w"))
            txt = subprocess.run([sys.executable, os.path.join(ref_root, "tools", "step_bytes.py"), art], capture_output=True,
                                 text=True, check=True).stdout
        groups = {m.group(1).strip(): float(m.group(2)) for m in re.finditer(r"^\s{4}(.+?)\s+([0-9.]+) GB", txt, flags=re.M)}
        out[mix] = {"total_gb": groups.pop("TOTAL"), "groups_gb": groups}
    json.dump(out, open(os.path.join(HERE, "step_bytes_golden.json"), "w"), indent=1)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference>")
    main(sys.argv[1])
