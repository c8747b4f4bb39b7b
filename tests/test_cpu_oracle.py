"""CPU-only tests: the oracle against the reference's known-answer tests and the committed fixtures, the
host-side logic of the library (planning, argument constructors), and the C ABI surface.

No compute call is made on the product library here: without a GPU it must refuse, loudly.
"""
import ctypes
import json
import os
import re

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = os.path.join(HERE, "golden")


@pytest.fixture(scope="module")
def kats():
    with open(os.path.join(GOLD, "reference_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def vec():
    return np.load(os.path.join(GOLD, "twin_vectors.npz"))


def one_f16_ulp(got, ref):
    """got and ref (f16 arrays) differ by at most one f16 unit in the last place, element-wise."""
    a, b = got.astype(np.float32), ref.astype(np.float32)
    ulp = np.maximum(np.spacing(np.abs(ref).astype(np.float16)).astype(np.float32), np.float32(6e-8))
    return bool((np.abs(a - b) <= ulp).all())


# ------------------------------------------------------------------ reference known-answer tests
def test_rearrange_scheme_kats_oracle_and_product(kats, orc, pkg):
    for case in kats["rearrange_scheme"]:
        got = orc.rearrange_scheme(case["dt_nbytes"], case["shape"], case["dst_strides"], case["src_strides"])
        lay = lambda st: pkg.TensorLayout(pkg.F16, case["shape"], st)
        mine = pkg.Rearrange.plan(pkg.RearrangeArgs(lay(case["dst_strides"]), None, lay(case["src_strides"]), None))
        assert got == mine, "oracle and product planners disagree"
        exp = case["expect"]
        if "scheme" in exp:
            assert got == exp["scheme"]
            # distribute_unit to 1024-byte pieces (rearrange/args.rs:157-195) restated on the scheme vector
            unit, nd = got[0], (len(got) - 2) // 3
            extra = unit // 1024
            dist = [1024] + [v * extra for v in got[1:2 + nd]] + [1] + got[2 + nd:2 + 2 * nd] + [1024] + got[2 + 2 * nd:] + [1024]
            assert dist == exp["distributed_1024"]
        else:
            nd = (len(got) - 2) // 3
            assert nd == exp["ndim"] and got[0] == exp["unit"] and got[1] == exp["count"]
            assert got[2:2 + nd] == exp["idx_strides"]
            assert got[2 + nd:2 + 2 * nd] == exp["dst_strides"] and got[2 + 2 * nd:] == exp["src_strides"]
            assert [got[1 + i] // got[2 + i] for i in range(nd)] == exp["shape"]


def test_all_reduce_and_broadcast_kats(kats, orc):
    k = kats["all_reduce"]
    bufs = [np.full(k["len"], r, dtype=np.uint32) for r in range(k["ranks"])]
    orc.all_reduce(bufs)
    for b in bufs:
        assert (b == k["expect"]).all()
    k = kats["broadcast"]
    bufs = [np.full(k["len"], r, dtype=np.uint32) for r in range(k["ranks"])]
    orc.broadcast(bufs, k["root"])
    for b in bufs:
        assert (b == k["expect"]).all()


# ------------------------------------------------------------------ oracle.cc against the committed fixtures
def test_oracle_matches_fixtures(orc, vec):
    y = orc.rms_norm(np.empty_like(vec["rms_x"]), vec["rms_x"], vec["rms_w"], 1e-5)
    np.testing.assert_array_equal(y.view(np.uint16), vec["rms_y"].view(np.uint16))  # no transcendental: exact
    assert one_f16_ulp(orc.rope(vec["rope_t"].copy(), vec["rope_pos"], 1e4), vec["rope_out"])
    assert one_f16_ulp(orc.fused_softmax(vec["sm_in"].copy(), True), vec["sm_causal"])
    assert one_f16_ulp(orc.fused_softmax(vec["sm_in"].copy(), False), vec["sm_none"])
    assert (orc.fused_softmax(vec["sm_in"].copy(), True)[:, 0, 5:] == 0).all()
    assert one_f16_ulp(orc.swiglu(vec["sw_gate"].copy(), vec["sw_up"]), vec["sw_out"])
    q = vec["att_q"].copy()
    o = orc.attention(q, vec["att_k"], vec["att_v"], np.zeros_like(q), True)
    assert float(np.abs(o.astype(np.float32) - vec["att_o"].astype(np.float32)).max()) <= 2e-3
    np.testing.assert_array_equal(q, o)  # head-major q is overwritten with the result, as in the crate
    assert orc.random_sample(vec["rs_logits"]) == tuple(int(v) for v in vec["rs_argmax"])
    lg = vec["rs_logits"]
    ties = np.flatnonzero(lg == lg.max())
    assert len(ties) >= 3 and int(vec["rs_argmax"][0]) == ties[-1]  # the LAST of the equal maxima
    for sd, exp in zip(vec["rs_seeds"], vec["rs_sample"]):
        assert orc.random_sample(vec["rs_logits"], 0.8, 0.9, 50, float(sd)) == tuple(int(v) for v in exp)
    bufs = [vec["ar_in"][r].copy() for r in range(8)]
    orc.all_reduce(bufs)
    for b in bufs:
        np.testing.assert_array_equal(b.view(np.uint16), vec["ar_out"].view(np.uint16))


def test_oracle_strides_and_dtypes(orc, synth):
    # byte strides are honoured: a transposed / sliced view gives the same numbers as its contiguous copy
    x = synth.normal(1, (6, 40), 1.0).astype(np.float16)
    w = synth.uniform(2, (40,), 0.5, 1.5).astype(np.float32)
    big = np.zeros((6, 80), np.float16)
    big[:, ::2] = x
    y1 = orc.rms_norm(np.empty_like(x), x, w, 1e-5)
    y2 = orc.rms_norm(np.empty_like(x), big[:, ::2], w, 1e-5)
    np.testing.assert_array_equal(y1, y2)
    a = synth.normal(3, (33, 70), 1.0).astype(np.float16)
    b = synth.normal(4, (70, 50), 0.1).astype(np.float16)
    c1 = orc.mat_mul(np.zeros((33, 50), np.float16), 0.0, a, b, 1.0)
    c2 = orc.mat_mul(np.zeros((50, 33), np.float16).T, 0.0, np.ascontiguousarray(a.T).T, np.ascontiguousarray(b.T).T, 1.0)
    np.testing.assert_array_equal(c1, c2)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert float(np.abs(c1.astype(np.float64) - ref).max()) < 4e-3
    c64 = orc.mat_mul(np.ones((33, 50)), 0.5, a.astype(np.float64), b.astype(np.float64), 2.0)
    np.testing.assert_allclose(c64, 0.5 + 2.0 * ref, rtol=1e-12)
    # mat_mul error kinds (operators/src/mat_mul/args.rs:73-120)
    with pytest.raises(orc.OracleError) as e:
        orc.mat_mul(np.zeros((3, 4), np.float16), 0.0, np.zeros((3, 5), np.float16), np.zeros((6, 4), np.float16), 1.0)
    assert e.value.kind == 6
    with pytest.raises(orc.OracleError) as e:
        orc.mat_mul(np.zeros((3, 8), np.float16)[:, ::2], 0.0, np.zeros((6, 5), np.float16)[::2], np.zeros((5, 4), np.float16), 1.0)
    assert e.value.kind == 7


def test_oracle_rearrange_and_cache(orc):
    rng = np.random.default_rng(0)
    src = rng.integers(0, 1 << 30, size=(32, 7, 128), dtype=np.int32)
    dst = np.zeros((7, 32, 128), np.int32)
    orc.rearrange(dst.transpose(1, 0, 2), src)
    np.testing.assert_array_equal(dst, src.transpose(1, 0, 2))
    with pytest.raises(orc.OracleError) as e:  # a zero dst stride would reduce
        orc.rearrange(np.broadcast_to(np.zeros((1, 4), np.int32), (3, 4)), np.zeros((3, 4), np.int32))
    assert e.value.kind == 5
    # attention_kv_cached: cache rows [pos, pos+seq) are overwritten byte for byte, the rest untouched
    q = rng.standard_normal((4, 3, 8)).astype(np.float16)
    k = rng.standard_normal((2, 3, 8)).astype(np.float16)
    v = rng.standard_normal((2, 3, 8)).astype(np.float16)
    kc = rng.standard_normal((2, 10, 8)).astype(np.float16)
    vc = rng.standard_normal((2, 10, 8)).astype(np.float16)
    kc0 = kc.copy()
    o = orc.attention_kv_cached(q.copy(), k, v, np.zeros_like(q), kc, vc, 5, True)
    np.testing.assert_array_equal(kc[:, 5:8], k)
    np.testing.assert_array_equal(vc[:, 5:8], v)
    np.testing.assert_array_equal(kc[:, :5], kc0[:, :5])
    o2 = orc.attention(q.copy(), kc[:, :8], vc[:, :8], np.zeros_like(q), True)
    np.testing.assert_array_equal(o, o2)
    with pytest.raises(orc.OracleError) as e:
        orc.attention_kv_cached(q.copy(), k, v, np.zeros_like(q), kc, vc, 8, True)
    assert e.value.kind == 6  # "Out of cache buffer"


def test_oracle_sampling_properties(orc, synth):
    lg = synth.normal(5, (2000,), 3.0).astype(np.float32)
    order = np.lexsort((np.arange(2000), -lg))
    # seed 0 always picks the largest logit; the reported value is the cumulative mass there (1.0)
    idx, bits = orc.random_sample(lg, 0.7, 0.9, 40, 0.0)
    assert idx == order[0] and np.array([bits], np.uint32).view(np.float32)[0] == 1.0
    picks = [orc.random_sample(lg, 0.7, 0.9, 40, s)[0] for s in np.linspace(0, 0.999, 50, dtype=np.float32)]
    ranks = [int(np.where(order == p)[0][0]) for p in picks]
    assert ranks == sorted(ranks) and max(ranks) < 40  # monotone in the draw, never beyond top_k


# ------------------------------------------------------------------ host-side logic of the product
def test_sample_args_and_build_helpers(pkg):
    assert pkg.SampleArgs.arg_max().is_argmax() and pkg.SampleArgs(0.5, 0.5, 1).is_argmax()
    assert not pkg.SampleArgs(0.5, 0.5, 2).is_argmax()
    with pytest.raises(pkg.SampleArgsError):
        pkg.SampleArgs(1.0, 0.5, 0)
    np.testing.assert_array_equal(pkg.RandomSample.build_indices(5), np.arange(5, dtype=np.uint32))
    pos = pkg.Rope.build_pos(pkg.U32, 7, [(0, 4), (7, 2), (1, 5)])  # truncated at nt like the crate's zip
    np.testing.assert_array_equal(pos, [0, 1, 2, 3, 7, 8, 1])
    pos64 = pkg.Rope.build_pos(pkg.U64, 3, [(10, 3)])
    assert pos64.dtype == np.uint64 and list(pos64) == [10, 11, 12]


def test_rearrange_plan_errors(pkg):
    lay = pkg.TensorLayout
    with pytest.raises(pkg.SchemeError) as e:
        pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (2, 3), (6, 2)), None, lay(pkg.F32, (2, 3), (12, 4)), None))
    assert e.value.kind == pkg.TYPE_MISMATCH
    with pytest.raises(pkg.SchemeError) as e:
        pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (2, 3), (6, 2)), None, lay(pkg.F16, (6,), (2,)), None))
    assert e.value.kind == pkg.RANK_MISMATCH
    with pytest.raises(pkg.SchemeError) as e:
        pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (2, 3), (6, 2)), None, lay(pkg.F16, (2, 4), (8, 2)), None))
    assert e.value.kind == pkg.SHAPE_MISMATCH
    with pytest.raises(pkg.SchemeError) as e:
        pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (2, 3), (0, 2)), None, lay(pkg.F16, (2, 3), (6, 2)), None))
    assert e.value.kind == pkg.SHAPE_NOT_SUPPORT and "Reducing" in e.value.info
    with pytest.raises(pkg.SchemeError) as e:
        pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (pkg.DYN_SIZE, 3), (6, 2)), None, lay(pkg.F16, (pkg.DYN_SIZE, 3), (6, 2)), None))
    assert e.value.kind == pkg.DYNAMIC_NOT_SUPPORT
    # contiguous tensors collapse to one unit; a broadcast source keeps stride 0
    assert pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.F16, (4, 5), (10, 2)), None, lay(pkg.F16, (4, 5), (10, 2)), None)) == [40, 1]
    assert pkg.Rearrange.plan(pkg.RearrangeArgs(lay(pkg.U8, (9, 40), (40, 1)), None, lay(pkg.U8, (9, 40), (0, 1)), None)) == [40, 9, 1, 40, 0]


def test_layout_helpers(pkg):
    t = pkg.TensorLayout.new_contiguous(pkg.F16, (2, 3, 4))
    assert t.strides == (24, 8, 2) and t.ndim == 3
    a = np.zeros((5, 6), np.float32)[:, ::2]
    assert pkg.TensorLayout.of(a).strides == (24, 8) and pkg.TensorLayout.of(a).dt == pkg.F32
    assert pkg.dtype_nbytes(pkg.KVPAIR) == 8 == pkg.lib().ops_dtype_nbytes(pkg.KVPAIR)


# ------------------------------------------------------------------ the C ABI surface
def test_library_exports_every_declared_symbol(pkg):
    with open(os.path.join(ROOT, "include", "ops_b200.h")) as f:
        header = f.read()
    declared = set(re.findall(r"\b(ops_[a-z0-9_]+)\s*\(", header))
    assert len(declared) > 55
    L = ctypes.CDLL(pkg.LIB_PATH)
    missing = [name for name in sorted(declared) if not hasattr(L, name)]
    assert not missing, f"declared in include/ops_b200.h but not exported: {missing}"
    assert set(pkg.EXPORTS) <= declared


def test_no_cpu_fallback(pkg):
    """Without a CUDA device the library refuses to create operators; it never computes on the host."""
    if pkg.device_count() > 0:
        pytest.skip("a CUDA device is present")
    for cls in (pkg.RmsNorm, pkg.Rope, pkg.FusedSoftmax, pkg.Swiglu, pkg.Rearrange, pkg.MatMul, pkg.Attention,
                pkg.AttentionKvCached, pkg.RandomSample):
        with pytest.raises(pkg.SchemeError) as e:
            cls(0)
        assert e.value.kind == pkg.EXECUTION_FAILED and "no CPU path" in e.value.info
    with pytest.raises(pkg.SchemeError):
        pkg.Comm(0, 0, 1)


def test_product_does_not_reach_the_oracle():
    """Nothing under the package may import, load or run anything under oracle/."""
    pkg_dir = os.path.join(ROOT, "operators-rs_b200")
    for base, _, files in os.walk(pkg_dir):
        if os.path.basename(base) == "build":
            continue
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".cc")):
                with open(os.path.join(base, fn)) as f:
                    text = f.read()
                hit = re.search(r"liboracle|oracle\.py|oracle_np|oracle_cpu|import\s+oracle|from\s+oracle|oracle/|load_oracle", text)
                assert hit is None, f"{fn} reaches for the oracle: {hit.group(0)}"
