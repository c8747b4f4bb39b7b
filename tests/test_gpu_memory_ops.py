"""GPU parity of the memory-bound operators against the CPU oracle, through the C ABI.

Shapes: benchmark config 1 (the CPU-runnable chain), the shapes of the reference's own tests
(operators/src/<op>/cuda/mod.rs test_compute), ragged/strided/edge cases, and a full-size slice of the
Llama-3-8B-shaped layer.  Tolerance: max-abs 1e-2 on f16 outputs vs the f16 oracle (the benchmark's budget), plus the
reference's own outlier rule vs an f64 oracle run.  rearrange is bit-exact.
"""
import numpy as np
import pytest
import torch

from helpers import assert_close, assert_reference_rule

pytestmark = pytest.mark.gpu


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def u32(t):
    return t.view(torch.uint32)


# ------------------------------------------------------------------------------------------ rms_norm
@pytest.mark.parametrize("n,d,wdt", [(64, 2048, np.float16), (4, 256, np.float32), (4, 512, np.float16), (4, 1024, np.float32),
                                      (4, 2048, np.float16), (4, 4096, np.float32), (4, 8192, np.float16),
                                      (3, 40, np.float16), (5, 1000, np.float32), (1, 8, np.float16), (7, 16384, np.float16)])
def test_rms_norm(pkg, orc, synth, dev, n, d, wdt):
    x = synth.normal(0xB2000010, (n, d), 1.0).astype(np.float16)
    w = synth.uniform(0xB2000011, (d,), 0.5, 1.5).astype(wdt)
    y = torch.empty(n, d, dtype=torch.float16, device=dev)
    xd, wd = to_dev(x, dev), to_dev(w, dev)
    op = pkg.RmsNorm(0)
    assert op.scheme(pkg.RmsNormArgs.of(y, xd, wd, 1e-5)) == 0
    op.launch(pkg.RmsNormArgs.of(y, xd, wd, 1e-5))
    ref = orc.rms_norm(np.empty_like(x), x, w, 1e-5)
    assert_close(y.cpu().numpy(), ref, 1e-2, "rms_norm")
    ref64 = orc.rms_norm(np.empty((n, d), np.float64), x.astype(np.float64), w.astype(np.float64), 1e-5)
    assert_reference_rule(y.cpu().numpy(), ref64, 1e-3, "rms_norm")


def test_rms_norm_strided_rows_and_f32(pkg, orc, synth, dev):
    # x is a column slice of a wider matrix (row stride != d), y likewise; and an all-f32 call
    big = synth.normal(1, (9, 3 * 512), 1.0).astype(np.float16)
    w = synth.uniform(2, (512,), 0.5, 1.5).astype(np.float16)
    bd = to_dev(big, dev)
    out = torch.zeros(9, 2 * 512, dtype=torch.float16, device=dev)
    xs, ys = bd[:, 512:1024], out[:, 512:]
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(ys, xs, to_dev(w, dev), 1e-6))
    ref = orc.rms_norm(np.empty((9, 512), np.float16), big[:, 512:1024], w, 1e-6)
    assert_close(ys.cpu().numpy(), ref, 1e-2, "rms_norm strided")
    assert float(out[:, :512].abs().max()) == 0.0  # nothing written outside the slice
    # element stride 2 on x (generic kernel)
    xe = bd[:, ::3][:, :512]
    y2 = torch.empty(9, 512, dtype=torch.float16, device=dev)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(y2, xe, to_dev(w, dev), 1e-6))
    ref2 = orc.rms_norm(np.empty((9, 512), np.float16), big[:, ::3][:, :512], w, 1e-6)
    assert_close(y2.cpu().numpy(), ref2, 1e-2, "rms_norm element stride")
    x32 = synth.normal(3, (6, 300), 1.0)
    w32 = synth.uniform(4, (300,), 0.5, 1.5)
    y32 = torch.empty(6, 300, dtype=torch.float32, device=dev)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(y32, to_dev(x32, dev), to_dev(w32, dev), 1e-5))
    ref32 = orc.rms_norm(np.empty_like(x32), x32, w32, 1e-5)
    np.testing.assert_allclose(y32.cpu().numpy(), ref32, rtol=2e-6, atol=1e-6)


def test_rms_norm_full_size_rows(pkg, orc, synth, dev):
    # config 3 size on the GPU (4096 x 4096); the oracle checks a sample of rows (rows are independent)
    n, d = 4096, 4096
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(n, d, generator=g, device=dev, dtype=torch.float32).half()
    w = (torch.rand(d, generator=g, device=dev) + 0.5).half()
    y = torch.empty_like(x)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(y, x, w, 1e-5))
    rows = [0, 1, 777, 2048, 4095]
    xs = x[rows].cpu().numpy()
    ref = orc.rms_norm(np.empty_like(xs), xs, w.cpu().numpy(), 1e-5)
    assert_close(y[rows].cpu().numpy(), ref, 1e-2, "rms_norm 4096x4096")


# ------------------------------------------------------------------------------------------ rope
@pytest.mark.parametrize("nt,nh,dh,theta,pdt", [(64, 32, 64, 1e4, np.uint32), (7, 32, 64, 1e4, np.uint64), (5, 3, 128, 5e5, np.uint32),
                                                (3, 2, 6, 1e4, np.uint32), (2, 1, 1024, 1e4, np.uint32)])
def test_rope(pkg, orc, synth, dev, nt, nh, dh, theta, pdt):
    t = synth.normal(0xB2000020, (nt, nh, dh), 1.0).astype(np.float16)
    pos = np.array([0, 1, 2, 3, 7, 8, 1][:nt] if nt == 7 else np.arange(nt), dtype=pdt)
    td = to_dev(t, dev)
    pd_ = to_dev(pos.view(np.int32 if pdt == np.uint32 else np.int64), dev).view(torch.uint32 if pdt == np.uint32 else torch.uint64)
    pkg.Rope(0).launch(pkg.RopeArgs.of(td, pd_, theta))
    ref = orc.rope(t.copy(), pos, theta)
    assert_close(td.cpu().numpy(), ref, 1e-2, "rope")
    ref64 = orc.rope(t.astype(np.float64), pos, theta)
    assert_reference_rule(td.cpu().numpy(), ref64, 0.0 if dh <= 128 else 1e-3, "rope")


def test_rope_large_positions_and_qkv_view(pkg, orc, synth, dev):
    # rope over the q and k heads of a fused [nt, 48*128] QKV buffer (strided view), positions up to 4095, theta 5e5
    nt, nh_total, nh, dh = 16, 48, 40, 128
    qkv = synth.normal(5, (nt, nh_total * dh), 1.0).astype(np.float16)
    pos = np.array([4095 - 37 * i for i in range(nt)], dtype=np.uint32)
    qd = to_dev(qkv, dev)
    view = qd.view(nt, nh_total, dh)[:, :nh, :]
    pkg.Rope(0).launch(pkg.RopeArgs.of(view, u32(to_dev(pos.view(np.int32), dev)), 5e5))
    ref = qkv.copy().reshape(nt, nh_total, dh)
    orc.rope(ref[:, :nh, :], pos, 5e5)
    assert_close(qd.cpu().numpy().reshape(nt, nh_total, dh), ref, 1e-2, "rope qkv view")
    np.testing.assert_array_equal(qd.cpu().numpy().reshape(nt, nh_total, dh)[:, nh:], qkv.reshape(nt, nh_total, dh)[:, nh:])


# ------------------------------------------------------------------------------------------ fused_softmax
@pytest.mark.parametrize("nh,seq,att", [(32, 64, 64), (32, 1, 511), (32, 1, 2048), (32, 7, 511), (32, 7, 2048), (2, 5, 7), (3, 16, 4096),
                                        (1, 3, 8200), (2, 33, 1000), (4, 128, 1024)])
@pytest.mark.parametrize("causal", [True, False])
def test_fused_softmax(pkg, orc, synth, dev, nh, seq, att, causal):
    if causal and att < seq:
        pytest.skip("causal needs att >= seq")
    x = synth.normal(0xB2000012, (nh, seq, att), 2.0).astype(np.float16)
    xd = to_dev(x, dev)
    pkg.FusedSoftmax(0).launch(pkg.FusedSoftmaxArgs.of(xd, pkg.MASK_CAUSAL if causal else pkg.MASK_NONE))
    ref = orc.fused_softmax(x.copy(), causal)
    got = xd.cpu().numpy()
    assert_close(got, ref, 1e-2, "fused_softmax")
    assert_reference_rule(got, orc.fused_softmax(x.astype(np.float64), causal), 0.0, "fused_softmax")
    if causal:  # masked tail is exactly +0
        k = seq - 1 if att == seq else 0
        lim = att - seq + k + 1
        assert (got[:, k, lim:].view(np.uint16) == 0).all()


def test_fused_softmax_strided(pkg, orc, synth, dev):
    # rows padded (row stride > att): generic and vector paths both take byte strides from the layout
    x = synth.normal(9, (4, 6, 96), 2.0).astype(np.float16)
    xd = to_dev(x, dev)
    view = xd[:, :, :64]
    pkg.FusedSoftmax(0).launch(pkg.FusedSoftmaxArgs.of(view))
    ref = x.copy()
    orc.fused_softmax(ref[:, :, :64], True)
    assert_close(xd.cpu().numpy(), ref, 1e-2, "fused_softmax padded rows")
    v2 = xd[:, :, 1:62:2]  # element stride 2, odd start -> generic kernel
    x2 = xd.cpu().numpy().copy()
    pkg.FusedSoftmax(0).launch(pkg.FusedSoftmaxArgs.of(v2, pkg.MASK_NONE))
    orc.fused_softmax(x2[:, :, 1:62:2], False)
    assert_close(xd.cpu().numpy(), x2, 1e-2, "fused_softmax element stride")


# ------------------------------------------------------------------------------------------ swiglu
@pytest.mark.parametrize("n,d", [(5632 // 8, 2048), (3, 40), (1, 8), (17, 14336)])
def test_swiglu(pkg, orc, synth, dev, n, d):
    gate = synth.normal(0xB2000030, (n, d), 1.0).astype(np.float16)
    up = synth.normal(0xB2000031, (n, d), 1.0).astype(np.float16)
    gd, ud = to_dev(gate, dev), to_dev(up, dev)
    pkg.Swiglu(0).launch(pkg.SwigluArgs.of(gd, ud))
    ref = orc.swiglu(gate.copy(), up)
    assert_close(gd.cpu().numpy(), ref, 1e-2, "swiglu")
    # the reference's own rule (abs 9.77e-4 vs an f64 run) on the reference's input distribution, U[0,1)
    # (operators/src/swiglu/cuda/mod.rs:195-240): |out| < 1 keeps one f16 ulp below the absolute threshold
    g01 = synth.uniform01(0xB2000032, (n, d)).astype(np.float16)
    u01 = synth.uniform01(0xB2000033, (n, d)).astype(np.float16)
    g01d = to_dev(g01, dev)
    pkg.Swiglu(0).launch(pkg.SwigluArgs.of(g01d, to_dev(u01, dev)))
    assert_reference_rule(g01d.cpu().numpy(), orc.swiglu(g01.astype(np.float64), u01.astype(np.float64)), 0.0, "swiglu")


def test_swiglu_halves_of_one_buffer(pkg, orc, synth, dev):
    # gate and up are the two column halves of one [n, 2*ffn] GEMM output, as in the layer
    n, ffn = 33, 1792
    gu = synth.normal(11, (n, 2 * ffn), 1.0).astype(np.float16)
    gud = to_dev(gu, dev)
    pkg.Swiglu(0).launch(pkg.SwigluArgs.of(gud[:, :ffn], gud[:, ffn:]))
    ref = gu.copy()
    orc.swiglu(ref[:, :ffn], ref[:, ffn:])
    assert_close(gud.cpu().numpy(), ref, 1e-2, "swiglu halves")


# ------------------------------------------------------------------------------------------ rearrange (bit-exact)
def test_rearrange_transpose_u32(pkg, orc, dev):
    # the reference's test: u32 [32,7,128] -> transposed (operators/src/rearrange/cuda/mod.rs:271-324)
    rng = np.random.default_rng(0)
    src = rng.integers(0, 2 ** 31, size=(32, 7, 128), dtype=np.int32)
    sd = to_dev(src, dev)
    dst = torch.zeros(7, 32, 128, dtype=torch.int32, device=dev)
    pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst.permute(1, 0, 2), sd))
    np.testing.assert_array_equal(dst.cpu().numpy(), src.transpose(1, 0, 2))


@pytest.mark.parametrize("case", ["kv_cache", "q_token_major", "broadcast", "bytes_odd", "negative_like", "scalar", "five_d"])
def test_rearrange_cases(pkg, orc, dev, case):
    rng = np.random.default_rng(1)
    if case == "kv_cache":  # config 2: k [8,2048,128] into cache [8,4096,128] at pos 2048
        src = rng.integers(-30000, 30000, size=(8, 512, 128), dtype=np.int16)
        cache = rng.integers(-30000, 30000, size=(8, 1024, 128), dtype=np.int16)
        cd, sd = to_dev(cache, dev).view(torch.float16), to_dev(src, dev).view(torch.float16)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(cd[:, 512:, :], sd))
        exp = cache.copy()
        orc.rearrange(exp[:, 512:, :], src)
        np.testing.assert_array_equal(cd.view(torch.int16).cpu().numpy(), exp)
    elif case == "q_token_major":  # [seq, nh, dh] viewed head-major -> contiguous [nh, seq, dh]
        src = rng.integers(-30000, 30000, size=(37, 12, 64), dtype=np.int16)
        sd = to_dev(src, dev)
        dst = torch.zeros(12, 37, 64, dtype=torch.int16, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst, sd.permute(1, 0, 2)))
        np.testing.assert_array_equal(dst.cpu().numpy(), src.transpose(1, 0, 2))
    elif case == "broadcast":  # src stride 0
        src = rng.integers(0, 255, size=(1, 40), dtype=np.uint8)
        sd = to_dev(src, dev)
        dst = torch.zeros(9, 40, dtype=torch.uint8, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst, sd.expand(9, 40)))
        np.testing.assert_array_equal(dst.cpu().numpy(), np.broadcast_to(src, (9, 40)))
    elif case == "bytes_odd":  # odd sizes and offsets: 1-byte accesses
        src = rng.integers(0, 255, size=(5, 13), dtype=np.uint8)
        sd = to_dev(src, dev)
        dst = torch.zeros(5, 29, dtype=torch.uint8, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst[:, 3:16], sd))
        exp = np.zeros((5, 29), np.uint8)
        exp[:, 3:16] = src
        np.testing.assert_array_equal(dst.cpu().numpy(), exp)
    elif case == "negative_like":  # column gather with a big stride on src, element-sized units
        src = rng.integers(-9, 9, size=(64, 48), dtype=np.int32)
        sd = to_dev(src, dev)
        dst = torch.zeros(48, 64, dtype=torch.int32, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst, sd.t()))
        np.testing.assert_array_equal(dst.cpu().numpy(), src.T)
    elif case == "scalar":  # rank 0 and all-ones shapes collapse to a single unit
        sd = to_dev(np.array([[[42]]], dtype=np.int64), dev)
        dst = torch.zeros(1, 1, 1, dtype=torch.int64, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst, sd))
        assert int(dst.item()) == 42
    else:  # 5-d permutation
        src = rng.integers(-30000, 30000, size=(3, 4, 5, 6, 8), dtype=np.int16)
        sd = to_dev(src, dev)
        dst = torch.zeros(5, 3, 6, 4, 8, dtype=torch.int16, device=dev)
        pkg.Rearrange(0).launch(pkg.RearrangeArgs.of(dst, sd.permute(2, 0, 3, 1, 4)))
        np.testing.assert_array_equal(dst.cpu().numpy(), src.transpose(2, 0, 3, 1, 4))


def test_rearrange_full_size_kv_cache(pkg, dev):
    # config 2 at full size: k,v [8,2048,128] f16 into [8,4096,128] caches at pos 0 and 2048; round trip is exact
    g = torch.Generator(device=dev).manual_seed(3)
    k = torch.randn(8, 2048, 128, generator=g, device=dev).half()
    cache = torch.zeros(8, 4096, 128, dtype=torch.float16, device=dev)
    op = pkg.Rearrange(0)
    for pos in (0, 2048):
        op.launch(pkg.RearrangeArgs.of(cache[:, pos:pos + 2048, :], k))
    assert torch.equal(cache[:, :2048], k) and torch.equal(cache[:, 2048:], k)
    back = torch.empty_like(k)
    op.launch(pkg.RearrangeArgs.of(back, cache[:, 2048:, :]))
    assert torch.equal(back, k)
