"""Multi-GPU parity: all_reduce (NCCL and the NVLink peer-to-peer kernels) and the tensor-parallel layer, one process
per GPU.  Skipped with fewer than 2 GPUs.  The oracle sums f16 partials in the crate's pairwise tree
(operators/src/all_reduce/common_cpu.rs:66-145); the GPU paths accumulate in f32 and round once, so agreement is to f16
rounding: max-abs <= 1e-2 (the benchmark's budget) for partials ~N(0,1)/sqrt(p) whose sum is ~N(0,1); the peer-to-peer
kernels are additionally checked bit for bit against their own specification (f32 sum in rank order, one rounding).
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

pytestmark = pytest.mark.gpu
CFG = dict(d=1024, nh=16, nkvh=8, dh=64, ffn=2048, theta=5e5, eps=1e-5)
T_LAYER = 192


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _weights(synth):
    d, nh, nkvh, dh, ffn = CFG["d"], CFG["nh"], CFG["nkvh"], CFG["dh"], CFG["ffn"]
    f16 = np.float16
    return {"w_norm1": synth.uniform(1, (d,), 0.5, 1.5).astype(f16), "w_norm2": synth.uniform(2, (d,), 0.5, 1.5).astype(f16),
            "w_qkv": synth.normal(3, (d, (nh + 2 * nkvh) * dh), 0.02).astype(f16), "w_o": synth.normal(4, (nh * dh, d), 0.02).astype(f16),
            "w_gu": synth.normal(5, (d, 2 * ffn), 0.02).astype(f16), "w_down": synth.normal(6, (ffn, d), 0.02).astype(f16)}


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    pkg = graft.load_package()
    synth = importlib.import_module(graft.PKG_NAME + ".synth")
    layer_mod = importlib.import_module(graft.PKG_NAME + ".layer")
    ids = [pkg.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    comm = pkg.Comm(rank, rank, world, ids[0])
    assert comm.rank() == rank and comm.group_size() == world
    handles = [None] * world
    dist.all_gather_object(handles, comm.p2p_export(4096 * 4096 * 2))
    comm.p2p_attach(handles)
    op = pkg.AllReduce(comm)
    results = {}
    for T in (1, 64, 4096):
        part = (synth.normal(0xB2000040 + 16 * T + rank, (T, 4096), 1.0) / np.sqrt(world)).astype(np.float16)
        for name, algo in (("nccl", pkg.ALL_REDUCE_NCCL), ("one_shot", pkg.ALL_REDUCE_P2P_ONE_SHOT), ("two_shot", pkg.ALL_REDUCE_P2P_TWO_SHOT)):
            op.set_algo(algo)
            for rep in range(2):  # twice: the second call reuses the other half of the double-buffered staging
                buf = torch.from_numpy(part).to(dev)
                op.launch(pkg.AllReduceArgs.of(buf, buf))
                torch.cuda.synchronize()
            results[f"ar_{T}_{name}"] = buf.cpu().numpy()
        # out of place, auto algorithm
        op.set_algo(pkg.ALL_REDUCE_AUTO)
        src = torch.from_numpy(part).to(dev)
        dst = torch.zeros_like(src)
        op.launch(pkg.AllReduceArgs.of(dst, src))
        torch.cuda.synchronize()
        results[f"ar_{T}_auto"] = dst.cpu().numpy()
        assert torch.equal(src.cpu(), torch.from_numpy(part))
        # dst <- dst + sum(src) with src in the zero-copy region: the residual (same on every rank) enters the sum first
        resid = synth.normal(0xB2000099 + T, (T, 4096), 1.0).astype(np.float16)
        direct = comm.p2p_direct(torch.float16)[: T * 4096].view(T, 4096)
        for rep in range(2):
            direct.copy_(torch.from_numpy(part).to(dev))
            acc = torch.from_numpy(resid).to(dev)
            op.launch_add(pkg.AllReduceArgs.of(acc, direct))
            torch.cuda.synchronize()
        results[f"ar_{T}_add"] = acc.cpu().numpy()
        # and with a staged (ordinary) source buffer
        acc = torch.from_numpy(resid).to(dev)
        op.launch_add(pkg.AllReduceArgs.of(acc, torch.from_numpy(part).to(dev)))
        torch.cuda.synchronize()
        results[f"ar_{T}_add_staged"] = acc.cpu().numpy()
    assert comm.p2p_status() == 0
    # replayed launches: the peer-to-peer kernels keep their launch counter on the device, so a CUDA graph holding three
    # one-shot all_reduces can be replayed (every rank replays the same sequence)
    op.set_algo(pkg.ALL_REDUCE_P2P_ONE_SHOT)
    gsrc = torch.from_numpy((synth.normal(0xB20000AA + rank, (64, 4096), 1.0) / np.sqrt(world)).astype(np.float16)).to(dev)
    gdst = [torch.zeros_like(gsrc) for _ in range(3)]
    op.launch(pkg.AllReduceArgs.of(gdst[0], gsrc))  # warm-up outside the capture
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream(dev)
    cg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(cg, stream=side):
        for i in range(3):
            op.launch(pkg.AllReduceArgs.of(gdst[i], gsrc))
    for rep in range(3):
        for t_ in gdst:
            t_.zero_()
        cg.replay()
        torch.cuda.synchronize()
    results["ar_graph_replay"] = torch.stack(gdst).cpu().numpy()
    assert comm.p2p_status() == 0
    op.set_algo(pkg.ALL_REDUCE_AUTO)
    # broadcast from the last rank (bytes), in place on the root and out of place elsewhere
    bc = pkg.Broadcast(comm)
    payload = torch.full((1000,), rank + 1, dtype=torch.int32, device=dev)
    recv = torch.zeros_like(payload)
    bc.launch(pkg.BroadcastArgs.of(recv, payload, world - 1))
    torch.cuda.synchronize()
    results["broadcast"] = recv.cpu().numpy()
    # tensor-parallel layer
    cfg = layer_mod.LayerConfig(**CFG)
    w = {k: torch.from_numpy(v).to(dev) for k, v in layer_mod.shard_weights(_weights(synth), rank, world, cfg).items()}
    # mat_mul + all_reduce as one kernel against mat_mul followed by the one-shot kernel: same f16 partials, same f32 sum in
    # rank order -> the same bits.  Twice (staging parity), with and without the residual folded in on rank 0.
    mm = pkg.MatMul(rank)
    a_part = torch.from_numpy(synth.normal(900 + rank, (320, 256), 1.0).astype(np.float16)).to(dev)
    w_part = torch.from_numpy(synth.normal(950 + rank, (256, 1024), 0.05).astype(np.float16)).to(dev)
    resid = torch.from_numpy(synth.normal(999, (320, 1024), 1.0).astype(np.float16)).to(dev)
    op.set_algo(pkg.ALL_REDUCE_P2P_ONE_SHOT)
    for rep in range(2):
        beta = 1.0 if (rank == 0 and rep == 1) else 0.0
        c_ref = resid.clone()
        mm.launch(pkg.MatMulArgs.of(c_ref, beta, a_part, w_part, 1.0))
        op.launch(pkg.AllReduceArgs.of(c_ref, c_ref))
        c_fused = resid.clone()
        mm.launch_all_reduce(comm, pkg.MatMulArgs.of(c_fused, beta, a_part, w_part, 1.0))
        torch.cuda.synchronize()
        assert mm.status() == 0 and comm.p2p_status() == 0
        assert torch.equal(c_ref, c_fused), f"fused mat_mul+all_reduce differs (rep {rep})"
    results["fused_gemm_ar"] = c_fused.cpu().numpy()
    layer_mod.DecoderLayer.DIRECT_MIN_BYTES = 1 << 16  # let the small test layer take the zero-copy exchange
    layer_mod.DecoderLayer.PIPELINE_MIN_ROWS = 64      # ... and the two-chunk pipelined tail (rows 0-127 and 128-191)
    for name, algo, fused, direct, pipe in (("nccl", pkg.ALL_REDUCE_NCCL, False, False, 1), ("p2p", pkg.ALL_REDUCE_P2P_ONE_SHOT, False, False, 1),
                                            ("fused", pkg.ALL_REDUCE_AUTO, True, False, 1), ("direct", pkg.ALL_REDUCE_AUTO, False, True, 1),
                                            ("pipelined", pkg.ALL_REDUCE_AUTO, False, True, 2)):
        lay = layer_mod.DecoderLayer(cfg, w, T_LAYER, dev, comm=comm, tp=world, rank=rank, all_reduce_algo=algo, fused_all_reduce=fused,
                                     direct=direct, pipeline=pipe)
        x = torch.from_numpy(synth.normal(7, (T_LAYER, CFG["d"]), 1.0).astype(np.float16)).to(dev)
        pos = torch.arange(T_LAYER, dtype=torch.int32, device=dev).view(torch.uint32)
        out = lay.forward(x, pos)
        torch.cuda.synchronize()
        results[f"layer_{name}"] = out.cpu().numpy()
    assert comm.p2p_status() == 0
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    del op, lay
    comm.destroy()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_reduce_and_tp_layer(tmp_path, orc, synth, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    for T in (1, 64, 4096):
        parts = [(synth.normal(0xB2000040 + 16 * T + r, (T, 4096), 1.0) / np.sqrt(world)).astype(np.float16) for r in range(world)]
        ref = orc.all_reduce([p.copy() for p in parts])[0]
        acc = np.zeros((T, 4096), np.float32)
        for p_ in parts:  # what the peer-to-peer kernels do: f32 accumulation in rank order, one rounding to f16
            acc = (acc + p_.astype(np.float32)).astype(np.float32)
        for name in ("nccl", "one_shot", "two_shot", "auto"):
            outs = [res[r][f"ar_{T}_{name}"] for r in range(world)]
            for o in outs[1:]:
                np.testing.assert_array_equal(o.view(np.uint16), outs[0].view(np.uint16))  # every rank holds the same bits
            # the oracle rounds to f16 after each of its log2(p) tree levels (up to 2e-3 per level at |x| in [4,8)); the GPU
            # paths round once: the benchmark's max-abs 1e-2 budget covers three levels at p = 8
            assert float(np.abs(outs[0].astype(np.float32) - ref.astype(np.float32)).max()) <= 1e-2, (T, name)
            if name in ("one_shot", "two_shot"):
                np.testing.assert_array_equal(outs[0].view(np.uint16), acc.astype(np.float16).view(np.uint16))
        resid = synth.normal(0xB2000099 + T, (T, 4096), 1.0).astype(np.float16)
        acc = resid.astype(np.float32)
        for p_ in parts:  # the residual first, then the ranks in order, one rounding
            acc = (acc + p_.astype(np.float32)).astype(np.float32)
        for name in ("add", "add_staged"):
            outs = [res[r][f"ar_{T}_{name}"] for r in range(world)]
            for o in outs:
                np.testing.assert_array_equal(o.view(np.uint16), acc.astype(np.float16).view(np.uint16))
    gparts = [(synth.normal(0xB20000AA + r, (64, 4096), 1.0) / np.sqrt(world)).astype(np.float16) for r in range(world)]
    gacc = np.zeros((64, 4096), np.float32)
    for p_ in gparts:
        gacc = (gacc + p_.astype(np.float32)).astype(np.float32)
    for r in range(world):
        for i in range(3):
            np.testing.assert_array_equal(res[r]["ar_graph_replay"][i].view(np.uint16), gacc.astype(np.float16).view(np.uint16))
    for r in range(world):
        assert (res[r]["broadcast"] == world).all()
    layer = importlib.import_module(graft.PKG_NAME + ".layer")
    cfg = layer.LayerConfig(**CFG)
    x = synth.normal(7, (T_LAYER, CFG["d"]), 1.0).astype(np.float16)
    emu = orc.decoder_layer(x, np.arange(T_LAYER, dtype=np.uint32), [layer.shard_weights(_weights(synth), r, world, cfg) for r in range(world)], CFG)
    for name in ("nccl", "p2p", "fused", "direct", "pipelined"):
        outs = [res[r][f"layer_{name}"] for r in range(world)]
        for o in outs[1:]:
            np.testing.assert_array_equal(o.view(np.uint16), outs[0].view(np.uint16))
        assert float(np.abs(outs[0].astype(np.float32) - emu.astype(np.float32)).max()) <= 1e-2, name
