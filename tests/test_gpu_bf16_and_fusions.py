"""GPU parity of the bf16 instantiations and of the fused entry points, through the C ABI.

bf16 has no CPU path in the reference crate (its common_cpu operators take f16/f32/f64; the GPU handle names
nv_bfloat16, operators/src/handle/cuda/mod.rs:188-210), so the oracle here is the same restated algorithm with bf16
rounding points.  One bf16 ulp is 2^-8 relative (7.8e-3 at |x| in [1,2), 3.1e-2 in [4,8)), eight times an f16 ulp:
the tolerance is two bf16 ulps at the magnitude of the outputs, written at each assert.

Fused entry points (no counterpart in the crate, which chains the operators): rms_norm with the residual add folded in
is compared with the oracle's add followed by rms_norm.
"""
import numpy as np
import pytest
import torch

from helpers import assert_close

pytestmark = pytest.mark.gpu


def bf_dev(orc, a32, dev):
    """f32 numpy -> (bf16 torch tensor on the device, tagged uint16 numpy array with the same bits)."""
    bits = orc.bf16_from_f32(a32)
    t = torch.from_numpy(np.asarray(bits).view(np.ndarray).view(np.int16).copy()).to(dev).view(torch.bfloat16)
    return t, bits


def bf_host(orc, t):
    return orc.bf16_to_f32(t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))


def test_bf16_memory_ops(pkg, orc, synth, dev):
    # rms_norm (bf16 weights and f32 weights), rope on a strided view, causal softmax, swiglu, add
    x32 = synth.normal(1, (96, 1024), 1.0)
    w32 = synth.uniform(2, (1024,), 0.5, 1.5)
    xd, xb = bf_dev(orc, x32, dev)
    wd, wb = bf_dev(orc, w32, dev)
    yd = torch.empty_like(xd)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(yd, xd, wd, 1e-5))
    yb = orc.rms_norm(orc.bf16_bits(np.zeros((96, 1024), np.uint16)), xb, wb, 1e-5)
    torch.cuda.synchronize()
    assert_close(bf_host(orc, yd), orc.bf16_to_f32(yb), 4e-2, "rms_norm bf16")  # |y| up to ~6: ulp 3.1e-2
    w32d = torch.from_numpy(w32.astype(np.float32)).to(dev)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(yd, xd, w32d, 1e-5))
    yb = orc.rms_norm(orc.bf16_bits(np.zeros((96, 1024), np.uint16)), xb, w32.astype(np.float32), 1e-5)
    torch.cuda.synchronize()
    assert_close(bf_host(orc, yd), orc.bf16_to_f32(yb), 4e-2, "rms_norm bf16 / f32 weights")

    t32 = synth.normal(3, (70, 12, 128), 1.0)
    td, tb = bf_dev(orc, t32, dev)
    pos = np.arange(100, 170, dtype=np.uint32)
    pd = torch.from_numpy(pos.view(np.int32)).to(dev).view(torch.uint32)
    pkg.Rope(0).launch(pkg.RopeArgs.of(td[:, :10], pd, 5e5))
    orc.rope(tb[:, :10], pos, 5e5)
    torch.cuda.synchronize()
    assert_close(bf_host(orc, td), orc.bf16_to_f32(tb), 4e-2, "rope bf16")

    s32 = synth.normal(4, (6, 200, 328), 2.0)
    sd, sb = bf_dev(orc, s32, dev)
    pkg.FusedSoftmax(0).launch(pkg.FusedSoftmaxArgs.of(sd))
    orc.fused_softmax(sb, True)
    torch.cuda.synchronize()
    assert_close(bf_host(orc, sd), orc.bf16_to_f32(sb), 8e-3, "fused_softmax bf16")  # probabilities <= 1: ulp <= 3.9e-3

    g32, u32 = synth.normal(5, (50, 2048), 1.0), synth.normal(6, (50, 2048), 1.0)
    gd, gb = bf_dev(orc, g32, dev)
    ud, ub = bf_dev(orc, u32, dev)
    pkg.Swiglu(0).launch(pkg.SwigluArgs.of(gd, ud))
    orc.swiglu(gb, ub)
    torch.cuda.synchronize()
    assert_close(bf_host(orc, gd), orc.bf16_to_f32(gb), 8e-2, "swiglu bf16")  # |g*u| up to ~15: ulp 6.2e-2

    ad, ab = bf_dev(orc, synth.normal(7, (33, 520), 1.0), dev)
    bd, bb = bf_dev(orc, synth.normal(8, (33, 520), 1.0), dev)
    cd = torch.empty_like(ad)
    pkg.Add(0).launch(pkg.AddArgs.of(cd, ad, bd))
    cb = orc.add(orc.bf16_bits(np.zeros((33, 520), np.uint16)), ab, bb)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(cd.view(torch.int16).cpu().numpy().view(np.uint16), np.asarray(cb).view(np.ndarray))  # one exact rounding


@pytest.mark.parametrize("m,n,k,beta", [(256, 512, 384, 0.0), (130, 264, 1000, 0.5), (1, 4096, 4096, 0.0), (1024, 768, 4096, 1.0)])
def test_bf16_mat_mul(pkg, orc, synth, dev, m, n, k, beta):
    ad, ab = bf_dev(orc, synth.normal(11, (m, k), 1.0), dev)
    bd, bb = bf_dev(orc, synth.normal(12, (k, n), 1.0 / np.sqrt(k)), dev)
    cd, cb = bf_dev(orc, synth.normal(13, (m, n), 1.0), dev)
    mm = pkg.MatMul(0)
    mm.launch(pkg.MatMulArgs.of(cd, beta, ad, bd, 1.0))
    orc.mat_mul(cb, beta, ab, bb, 1.0)
    torch.cuda.synchronize()
    assert mm.status() == 0
    assert_close(bf_host(orc, cd), orc.bf16_to_f32(cb), 4e-2, f"mat_mul bf16 m{m} n{n} k{k}")  # |c| up to ~5


@pytest.mark.parametrize("nh,nkvh,seq,att,dh", [(8, 2, 300, 300, 128), (4, 4, 64, 200, 64), (8, 2, 1, 1024, 128)])
def test_bf16_attention(pkg, orc, synth, dev, nh, nkvh, seq, att, dh):
    qd, qb = bf_dev(orc, synth.normal(21, (nh, seq, dh), 1.0), dev)
    kd, kb = bf_dev(orc, synth.normal(22, (nkvh, att, dh), 1.0), dev)
    vd, vb = bf_dev(orc, synth.normal(23, (nkvh, att, dh), 1.0), dev)
    od = torch.zeros_like(qd)
    ob = orc.bf16_bits(np.zeros((nh, seq, dh), np.uint16))
    orc.attention(qb.copy(), kb, vb, ob, True)
    for algo in (pkg.ATTENTION_FUSED, pkg.ATTENTION_CHAIN):
        op = pkg.Attention(0)
        op.set_algo(algo)
        args = pkg.AttentionArgs.of(qd.clone(), kd, vd, od)
        op.launch(args, torch.empty(op.scheme(args), dtype=torch.uint8, device=dev))
        torch.cuda.synchronize()
        assert op.status() == 0
        # outputs are convex combinations of N(0,1) values (|o| < ~4); the probabilities are themselves rounded to bf16
        assert_close(bf_host(orc, od), orc.bf16_to_f32(ob), 5e-2, f"attention bf16 algo {algo}")


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("wdt", ["same", "f32"])
def test_rms_norm_with_residual_add(pkg, orc, synth, dev, dt, wdt):
    n, d = 130, 4096
    x32, r32, w32 = synth.normal(31, (n, d), 1.0), synth.normal(32, (n, d), 1.0), synth.uniform(33, (d,), 0.5, 1.5)
    if dt == "f16":
        xn, rn, wn = x32.astype(np.float16), r32.astype(np.float16), w32.astype(np.float16)
        xd, rd, wd = (torch.from_numpy(a).to(dev) for a in (xn, rn, wn))
        to_f32 = lambda t: t.float().cpu().numpy()
        o32 = lambda a: a.astype(np.float32)
        zeros = lambda: np.zeros((n, d), np.float16)
        tol = 1e-2
    else:
        (xd, xn), (rd, rn), (wd, wn) = (bf_dev(orc, a, dev) for a in (x32, r32, w32))
        to_f32 = lambda t: bf_host(orc, t)
        o32 = orc.bf16_to_f32
        zeros = lambda: orc.bf16_bits(np.zeros((n, d), np.uint16))
        tol = 6e-2
    if wdt == "f32":
        wn = w32.astype(np.float32)
        wd = torch.from_numpy(wn).to(dev)
    yd = torch.empty_like(xd)
    pkg.RmsNorm(0).launch_add(pkg.RmsNormAddArgs.of(yd, xd, wd, 1e-5, rd))
    xs = orc.add(zeros(), xn, rn)          # the crate's add: one rounding to the element type
    ys = orc.rms_norm(zeros(), xs, wn, 1e-5)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_f32(xd), o32(xs))  # the updated residual stream is exact
    assert_close(to_f32(yd), o32(ys), tol, f"rms_norm_add {dt}/{wdt}")
    # layouts the vector kernel does not take are refused, not computed some other way
    with pytest.raises(pkg.LaunchError) as e:
        pkg.RmsNorm(0).launch_add(pkg.RmsNormAddArgs.of(yd[:, :100], xd[:, :100], wd[:100], 1e-5, rd[:, :100]))
    assert e.value.kind == pkg.ARGS_NOT_SUPPORT


def test_argmax_needs_no_workspace_and_leaves_its_scratch_clean(pkg, orc, synth, dev):
    rows, n = 16, 50000
    lg = synth.normal(41, (rows, n), 3.0).astype(np.float16)
    x = torch.from_numpy(lg).to(dev)
    op = pkg.RandomSample(0)
    want = [orc.random_sample(lg[r]) for r in range(rows)]
    for rep in range(3):  # the records the kernel meets in belong to the handle and must be back at zero after each launch
        kv = torch.zeros(rows, 2, dtype=torch.int32, device=dev)
        op.launch_batched(x, kv, pkg.SampleArgs.arg_max(), None)
        torch.cuda.synchronize()
        got = [(int(a), int(b)) for a, b in kv.cpu().numpy().view(np.uint32)]
        assert got == want, rep
    one = torch.zeros(2, dtype=torch.int32, device=dev)
    op.launch(pkg.RandomSampleArgs.of(one, x[3], pkg.SampleArgs.arg_max()))
    torch.cuda.synchronize()
    assert tuple(int(v) & 0xFFFFFFFF for v in one.cpu().tolist()) == want[3]


def test_sampling_rows_without_a_finite_order(pkg, dev):
    # every logit -inf, or one +inf: (x - max) is NaN for every element, nothing can be ordered.  The CPU loop of the
    # crate panics or returns garbage there; the kernel must give the documented answer (argmax rule, value 1) without
    # reading outside its buffers — through both entry points.
    op = pkg.RandomSample(0)
    cfg = pkg.SampleArgs(0.8, 0.9, 50)
    one_f16 = int(np.float16(1.0).view(np.uint16))
    for make, want_idx in ((lambda: np.full(5000, -np.inf, np.float16), 4999),):
        x = torch.from_numpy(make()).to(dev)
        for entry in ("ws", "noalloc"):
            kv = torch.full((2,), -1, dtype=torch.int32, device=dev)
            args = pkg.RandomSampleArgs.of(kv, x, cfg, 0.4)
            if entry == "ws":
                op.launch(args, torch.empty(16 * 5000 + 256, dtype=torch.uint8, device=dev))
            else:
                op.launch_noalloc(args)
            torch.cuda.synchronize()
            got = tuple(int(v) & 0xFFFFFFFF for v in kv.cpu().tolist())
            assert got == (want_idx, one_f16), (entry, got)
    y = np.linspace(-1, 1, 3000).astype(np.float16)
    y[700] = np.inf
    x = torch.from_numpy(y).to(dev)
    kv = torch.full((2,), -1, dtype=torch.int32, device=dev)
    op.launch(pkg.RandomSampleArgs.of(kv, x, cfg, 0.4), torch.empty(16 * 3000 + 256, dtype=torch.uint8, device=dev))
    torch.cuda.synchronize()
    assert tuple(int(v) & 0xFFFFFFFF for v in kv.cpu().tolist()) == (700, one_f16)


@pytest.mark.parametrize("nh,nkvh,seq,att,dh", [(32, 8, 1, 4096, 128), (32, 8, 2, 1000, 128), (16, 16, 1, 300, 64), (8, 1, 1, 8192, 128),
                                                (64, 8, 1, 257, 64)])
def test_decode_attention_shapes(pkg, orc, synth, dev, nh, nkvh, seq, att, dh):
    q = synth.normal(51, (nh, seq, dh), 1.0).astype(np.float16)
    k = synth.normal(52, (nkvh, att, dh), 1.0).astype(np.float16)
    v = synth.normal(53, (nkvh, att, dh), 1.0).astype(np.float16)
    on = np.zeros_like(q)
    orc.attention(q.copy(), k, v, on, True)
    qd, kd, vd = (torch.from_numpy(a).to(dev) for a in (q, k, v))
    op = pkg.Attention(0)
    for rep in range(2):  # twice: the arrival counters of the split-KV merge must be back at zero
        od = torch.zeros_like(qd)
        op.launch(pkg.AttentionArgs.of(qd, kd, vd, od), torch.empty(16, dtype=torch.uint8, device=dev))
        torch.cuda.synchronize()
        assert op.status() == 0
        assert_close(od.cpu().numpy(), on, 1e-2, f"decode attention rep {rep}")
