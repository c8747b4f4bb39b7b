"""Writes the committed fixtures of this folder.  Run from the repository root: python tests/golden/make_golden.py

reference_kats.json — the only exact known-answer tests the reference holds for this path, restated as data:
  * rearrange::Scheme::new and distribute_unit (operators/src/rearrange/args.rs:248-303);
  * all_reduce over 4 in-process ranks, u32 [rank; 8] -> [6; 8] (operators/src/all_reduce/common_cpu.rs:152-177);
  * broadcast from root 1 over 4 ranks -> [1; 8] (operators/src/broadcast/common_cpu/mod.rs:77-102).
twin_vectors.npz — seeded small inputs with the outputs of the NumPy twin (oracle/oracle_np.py), so that a change
  in either restatement shows up as a diff against a committed file.  The reference itself cannot run here
  (Rust crate, no toolchain), so these are NOT reference outputs; the file says so in its `note` entry.
"""
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    twin = _load("oracle_np", os.path.join(ROOT, "oracle", "oracle_np.py"))
    synth = _load("synth", os.path.join(ROOT, "operators-rs_b200", "synth.py"))
    big = [33554432 * 2, 16777216 * 2, 524288 * 2, 128 * 2, 1 * 2]
    kats = {
        "rearrange_scheme": [
            {"dt_nbytes": 2, "shape": [4, 3, 2, 1, 2, 3, 4], "dst_strides": [288, 96, 48, 48, 24, 8, 2],
             "src_strides": [576, 192, 96, 48, 8, 16, 2],
             "expect": {"ndim": 3, "unit": 8, "count": 144, "idx_strides": [6, 3, 1], "dst_strides": [48, 24, 8],
                        "src_strides": [96, 8, 16], "shape": [24, 2, 3]}},
            {"dt_nbytes": 2, "shape": [32, 2, 32, 456, 128], "dst_strides": big, "src_strides": big,
             "expect": {"scheme": [116736, 2048, 1, 1048576, 1048576],
                        "distributed_1024": [1024, 116736 // 1024 * 2048, 116736 // 1024, 1, 1048576, 1024, 1048576, 1024]}},
        ],
        "all_reduce": {"ranks": 4, "dtype": "u32", "len": 8, "input": "rank", "expect": 6},
        "broadcast": {"ranks": 4, "dtype": "u32", "len": 8, "root": 1, "input": "rank", "expect": 1},
    }
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(kats, f, indent=1)

    out = {"note": np.array("outputs of oracle/oracle_np.py (NumPy twin of the restated common_cpu), not of the reference crate")}
    x = synth.normal(0xB2000010, (3, 64), 1.0).astype(np.float16)
    w = synth.uniform(0xB2000011, (64,), 0.5, 1.5).astype(np.float16)
    out.update(rms_x=x, rms_w=w, rms_y=twin.rms_norm(x, w, 1e-5))
    t = synth.normal(0xB2000020, (5, 2, 16), 1.0).astype(np.float16)
    pos = np.array([0, 1, 7, 63, 4095], dtype=np.uint32)
    out.update(rope_t=t, rope_pos=pos, rope_out=twin.rope(t, pos, 1e4))
    s = synth.normal(0xB2000012, (2, 5, 9), 2.0).astype(np.float16)
    out.update(sm_in=s, sm_causal=twin.fused_softmax(s, True), sm_none=twin.fused_softmax(s, False))
    g = synth.normal(0xB2000030, (4, 24), 1.0).astype(np.float16)
    u = synth.normal(0xB2000031, (4, 24), 1.0).astype(np.float16)
    out.update(sw_gate=g, sw_up=u, sw_out=twin.swiglu(g, u))
    q = synth.normal(100, (4, 3, 8), 1.0).astype(np.float16)
    k = synth.normal(101, (2, 6, 8), 1.0).astype(np.float16)
    v = synth.normal(102, (2, 6, 8), 1.0).astype(np.float16)
    out.update(att_q=q, att_k=k, att_v=v, att_o=twin.attention(q, k, v, True))
    lg = synth.normal(0xB2000050, (500,), 3.0).astype(np.float16)
    lg[[7, 300]] = lg.max()  # a tie for the maximum
    out.update(rs_logits=lg, rs_argmax=np.array(twin.argmax(lg), dtype=np.uint32),
               rs_sample=np.array([twin.random_sample(lg, 0.8, 0.9, 50, sd) for sd in (0.0, 0.25, 0.5, 0.9)], dtype=np.uint32),
               rs_seeds=np.array([0.0, 0.25, 0.5, 0.9], dtype=np.float32))
    parts = [synth.normal(200 + r, (33,), 1.0).astype(np.float16) for r in range(8)]
    out.update(ar_in=np.stack(parts), ar_out=twin.all_reduce(parts)[0])
    np.savez_compressed(os.path.join(HERE, "twin_vectors.npz"), **out)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    sys.exit(main())
