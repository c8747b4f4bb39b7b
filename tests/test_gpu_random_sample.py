"""GPU parity of random_sample against the CPU oracle, through the C ABI: BIT-EXACT (index and value bits).

Shapes: the reference's test (n = 32000 f32, argmax and t=0.9/p=0.9/k=200/seed=0.75;
operators/src/random_sample/cuda/mod.rs:256-368) and benchmark config 5 (64 x 128256 f16 ~N(0,3), argmax and
t=0.8/p=0.9/k=50 with one seeded uniform draw per row).  Edge cases: ties (last index wins), -0/+0, NaN
rows, tiny rows, k >= n, top_p = 1, seeds at the ends of [0,1).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def run_one(pkg, dev, logits, cfg, seed):
    kv = torch.zeros(2, dtype=torch.int32, device=dev)
    pkg.RandomSample(0).launch(pkg.RandomSampleArgs.of(kv, to_dev(logits, dev), cfg, seed))
    return tuple(int(v) & 0xFFFFFFFF for v in kv.cpu().tolist())


def run_batched(pkg, dev, logits, cfg, seeds):
    rows = logits.shape[0]
    kv = torch.zeros(rows, 2, dtype=torch.int32, device=dev)
    sd = to_dev(np.asarray(seeds, dtype=np.float32), dev) if seeds is not None else None
    pkg.RandomSample(0).launch_batched(to_dev(logits, dev), kv, cfg, sd)
    out = kv.cpu().numpy().view(np.uint32)
    return [(int(a), int(b)) for a, b in out]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_reference_case(pkg, orc, synth, dev, dtype):
    lg = synth.uniform01(0xB2000050, (32000,)).astype(dtype)
    assert run_one(pkg, dev, lg, pkg.SampleArgs.arg_max(), 0.0) == orc.random_sample(lg)
    cfg = pkg.SampleArgs(0.9, 0.9, 200)
    assert run_one(pkg, dev, lg, cfg, 0.75) == orc.random_sample(lg, 0.9, 0.9, 200, 0.75)


def test_argmax_ties_zero_signs_and_nan(pkg, orc, dev):
    cfg = pkg.SampleArgs.arg_max()
    x = np.zeros(5000, np.float16)
    x[[17, 4000, 4999]] = 3.5  # equal maxima: the last index wins
    assert run_one(pkg, dev, x, cfg, 0.0) == orc.random_sample(x) == (4999, int(np.float16(3.5).view(np.uint16)))
    z = np.full(100, -1.0, np.float32)
    z[3], z[50] = 0.0, -0.0  # +0 and -0 compare equal: the later one wins and its own bits are reported
    assert run_one(pkg, dev, z, cfg, 0.0) == orc.random_sample(z) == (50, 0x80000000)
    for nan_at in ([10], [10, 700], [999]):  # a NaN is taken, then replaced by whatever follows it
        y = np.linspace(-1, 1, 1000).astype(np.float32)
        y[nan_at] = np.nan
        y[5] = 100.0
        assert run_one(pkg, dev, y, cfg, 0.0) == orc.random_sample(y)
    assert run_one(pkg, dev, np.array([2.0], np.float16), cfg, 0.0) == orc.random_sample(np.array([2.0], np.float16))
    # top_k == 1 is argmax whatever the temperature (operators/src/random_sample/args.rs:81-83)
    w = np.array([0.5, 3.0, -1.0, 3.0], np.float32)
    assert run_one(pkg, dev, w, pkg.SampleArgs(0.7, 0.9, 1), 0.3) == orc.random_sample(w, 0.7, 0.9, 1, 0.3) == (3, 0x40400000)


@pytest.mark.parametrize("n,t,p,k", [(1, 1.0, 1.0, 5), (7, 0.5, 0.9, 3), (100, 2.0, 1.0, 2 ** 64 - 1), (1000, 1.0, 0.5, 1000), (4097, 0.3, 0.99, 64),
                                     (33000, 5.0, 0.9, 50), (128256, 0.8, 0.9, 50), (128256, 100.0, 1.0, 2 ** 64 - 1)])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_sampling_bit_exact(pkg, orc, synth, dev, n, t, p, k, dtype):
    lg = synth.normal(0xB2000051 + n, (n,), 3.0).astype(dtype)
    cfg = pkg.SampleArgs(t, p, k)
    for seed in (0.0, 0.123, 0.5, 0.75, 0.9999999):
        seed = float(np.float32(seed))
        assert run_one(pkg, dev, lg, cfg, seed) == orc.random_sample(lg, t, p, k, seed), (n, t, p, k, seed)


def test_sampling_many_equal_logits(pkg, orc, dev):
    # all-equal and few-distinct rows: every term is 1, sums cross many binades and hit exact ties
    for n in (10, 3000, 70000):
        x = np.full(n, 0.25, np.float16)
        cfg = pkg.SampleArgs(1.0, 1.0, 2 ** 64 - 1)
        for seed in (0.0, 0.3, 0.77):
            assert run_one(pkg, dev, x, cfg, seed) == orc.random_sample(x, 1.0, 1.0, 2 ** 64 - 1, seed)
    y = np.tile(np.array([1.0, 0.5, 0.0, -0.5], np.float16), 5000)
    cfg = pkg.SampleArgs(0.5, 0.95, 12000)
    for seed in (0.1, 0.6, 0.95):
        assert run_one(pkg, dev, y, cfg, seed) == orc.random_sample(y, 0.5, 0.95, 12000, seed)


def test_config5_batched(pkg, orc, synth, dev):
    # benchmark config 5: 64 rows x 128256 f16 ~N(0,3); argmax, then t=0.8 / top_p=0.9 / top_k=50 with a seeded draw per row
    rows, n = 64, 128256
    lg = synth.normal(0xB2000050, (rows, n), 3.0).astype(np.float16)
    seeds = synth.uniform01(0xB2000051, (rows,))
    got = run_batched(pkg, dev, lg, pkg.SampleArgs.arg_max(), None)
    assert got == [orc.random_sample(lg[r]) for r in range(rows)]
    got = run_batched(pkg, dev, lg, pkg.SampleArgs(0.8, 0.9, 50), seeds)
    assert got == [orc.random_sample(lg[r], 0.8, 0.9, 50, float(seeds[r])) for r in range(rows)]


def test_errors(pkg, dev):
    kv = torch.zeros(2, dtype=torch.int32, device=dev)
    lg = torch.zeros(16, dtype=torch.float16, device=dev)
    op = pkg.RandomSample(0)
    bad = pkg.RandomSampleArgs(pkg.TensorLayout(pkg.U32, (), ()), kv, lg, lg, pkg.TensorLayout.new_contiguous(pkg.U32, (16,)), None,
                               pkg.SampleArgs.arg_max(), 0.0)
    with pytest.raises(pkg.LaunchError) as e:
        op.launch(bad)
    assert e.value.kind == pkg.TYPE_NOT_SUPPORT and "KVpair" in e.value.info
    strided = pkg.RandomSampleArgs(pkg.TensorLayout(pkg.KVPAIR, (), ()), kv, pkg.TensorLayout(pkg.F16, (8,), (4,)), lg,
                                   pkg.TensorLayout.new_contiguous(pkg.U32, (8,)), None, pkg.SampleArgs.arg_max(), 0.0)
    with pytest.raises(pkg.LaunchError) as e:
        op.launch(strided)
    assert e.value.kind == pkg.STRIDES_NOT_SUPPORT
    with pytest.raises(pkg.SampleArgsError):
        pkg.SampleArgs(-1.0, 0.5, 3)
    with pytest.raises(pkg.SampleArgsError):
        pkg.SampleArgs(1.0, 0.0, 3)
    assert pkg.SampleArgs(1.0, 7.0, 3).c.top_p == 1.0
