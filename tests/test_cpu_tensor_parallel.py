"""Tensor-parallel host logic on CPU: the column/row sharding of the layer and the exchange pattern, run as two
real processes over the gloo backend.  Arithmetic comes from the CPU oracle (there is no CPU path in the product);
what is under test is `layer.shard_weights` and the rank-0-folds-the-residual scheme the GPU driver uses.
"""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as graft

CFG = dict(d=64, nh=8, nkvh=4, dh=16, ffn=96, theta=1e4, eps=1e-5)
T = 24


def _weights(synth):
    d, nh, nkvh, dh, ffn = CFG["d"], CFG["nh"], CFG["nkvh"], CFG["dh"], CFG["ffn"]
    f16 = np.float16
    return {"w_norm1": synth.uniform(1, (d,), 0.5, 1.5).astype(f16), "w_norm2": synth.uniform(2, (d,), 0.5, 1.5).astype(f16),
            "w_qkv": synth.normal(3, (d, (nh + 2 * nkvh) * dh), 0.1).astype(f16), "w_o": synth.normal(4, (nh * dh, d), 0.1).astype(f16),
            "w_gu": synth.normal(5, (d, 2 * ffn), 0.1).astype(f16), "w_down": synth.normal(6, (ffn, d), 0.1).astype(f16)}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    graft.load_package()
    orc = graft.load_oracle()
    orc.set_num_threads(1)
    synth = importlib.import_module(graft.PKG_NAME + ".synth")
    layer = importlib.import_module(graft.PKG_NAME + ".layer")
    cfg = layer.LayerConfig(**CFG)
    w = layer.shard_weights(_weights(synth), rank, world, cfg)
    x = synth.normal(7, (T, CFG["d"]), 1.0).astype(np.float16)
    pos = np.arange(T, dtype=np.uint32)
    dh, nq, nkv, f = CFG["dh"], CFG["nh"] // world, CFG["nkvh"] // world, CFG["ffn"] // world

    def reduce(part):  # f16 partials summed across ranks (gloo sums in the tensor dtype, like the crate's CPU all_reduce)
        t = torch.from_numpy(part)
        dist.all_reduce(t)
        return t.numpy()

    h = orc.rms_norm(np.empty_like(x), x, w["w_norm1"], CFG["eps"])
    qkv = orc.mat_mul(np.zeros((T, (nq + 2 * nkv) * dh), np.float16), 0.0, h, w["w_qkv"], 1.0)
    heads = qkv.reshape(T, nq + 2 * nkv, dh)
    orc.rope(heads[:, : nq + nkv], pos, CFG["theta"])
    att = np.zeros((T, nq * dh), np.float16)
    orc.attention(heads[:, :nq].transpose(1, 0, 2), heads[:, nq:nq + nkv].transpose(1, 0, 2), heads[:, nq + nkv:].transpose(1, 0, 2),
                  att.reshape(T, nq, dh).transpose(1, 0, 2), True)
    part = x.copy() if rank == 0 else np.zeros_like(x)
    orc.mat_mul(part, 1.0 if rank == 0 else 0.0, att, w["w_o"], 1.0)
    x1 = reduce(part)
    h = orc.rms_norm(np.empty_like(x), x1, w["w_norm2"], CFG["eps"])
    gu = orc.mat_mul(np.zeros((T, 2 * f), np.float16), 0.0, h, w["w_gu"], 1.0)
    orc.swiglu(gu[:, :f], gu[:, f:])
    part = x1.copy() if rank == 0 else np.zeros_like(x)
    orc.mat_mul(part, 1.0 if rank == 0 else 0.0, gu[:, :f], w["w_down"], 1.0)
    out = reduce(part)
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_process_tensor_parallel_layer(tmp_path, orc, synth, world):
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outs = [np.load(tmp_path / f"out{r}.npy") for r in range(world)]
    np.testing.assert_array_equal(outs[0], outs[1])  # every rank ends with the same stream
    x = synth.normal(7, (T, CFG["d"]), 1.0).astype(np.float16)
    pos = np.arange(T, dtype=np.uint32)
    full = orc.decoder_layer(x, pos, [_weights(synth)], CFG)
    # splitting a sum over ranks changes f16 rounding points only: one or two f16 ulps at |x| ~ 2
    assert float(np.abs(outs[0].astype(np.float32) - full.astype(np.float32)).max()) <= 8e-3
    # the oracle's own emulation of the ranks (tree-ordered f16 all_reduce) against the real processes
    layer = importlib.import_module(graft.PKG_NAME + ".layer")
    cfg = layer.LayerConfig(**CFG)
    emu = orc.decoder_layer(x, pos, [layer.shard_weights(_weights(synth), r, world, cfg) for r in range(world)], CFG)
    np.testing.assert_array_equal(emu.view(np.uint16), outs[0].view(np.uint16))


def test_shard_weights_partition(synth):
    layer = importlib.import_module(graft.PKG_NAME + ".layer")
    cfg = layer.LayerConfig(**CFG)
    w = _weights(synth)
    for tp in (1, 2, 4):
        shards = [layer.shard_weights(w, r, tp, cfg) for r in range(tp)]
        dh, nq, nkv, f = cfg.dh, cfg.nh // tp, cfg.nkvh // tp, cfg.ffn // tp
        # columns: every q / k / v head and every gate / up column lands on exactly one rank, GQA groups stay together
        q = np.concatenate([s["w_qkv"][:, : nq * dh] for s in shards], 1)
        k = np.concatenate([s["w_qkv"][:, nq * dh:(nq + nkv) * dh] for s in shards], 1)
        v = np.concatenate([s["w_qkv"][:, (nq + nkv) * dh:] for s in shards], 1)
        np.testing.assert_array_equal(np.concatenate([q, k, v], 1), w["w_qkv"])
        gate = np.concatenate([s["w_gu"][:, :f] for s in shards], 1)
        up = np.concatenate([s["w_gu"][:, f:] for s in shards], 1)
        np.testing.assert_array_equal(np.concatenate([gate, up], 1), w["w_gu"])
        # rows
        np.testing.assert_array_equal(np.concatenate([s["w_o"] for s in shards], 0), w["w_o"])
        np.testing.assert_array_equal(np.concatenate([s["w_down"] for s in shards], 0), w["w_down"])
    with pytest.raises(AssertionError):
        layer.shard_weights(w, 0, 3, cfg)
