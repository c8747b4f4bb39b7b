"""Argument validation through the C ABI: every operator answers the reference's error kind for the reference's
checks (`Args::meta`, `Args::layout`, `Scheme::new`; SchemeErrorKind of operators/src/common/error.rs:2-12), accepts
dynamic values in scheme() and refuses them in launch().  Needs a device only because handles cannot be created
without one; no kernel is launched by the failing calls.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def L(pkg, dt, shape, strides=None):
    return pkg.TensorLayout.new_contiguous(dt, shape) if strides is None else pkg.TensorLayout(dt, shape, strides)


def expect(pkg, kind, fn):
    with pytest.raises(pkg.SchemeError) as e:
        fn()
    assert e.value.kind == kind, (e.value.kind, e.value.info)
    return e.value


def test_rms_norm_checks(pkg, dev):
    op, F16, F32 = pkg.RmsNorm(0), pkg.F16, pkg.F32
    ok = lambda **kw: pkg.RmsNormArgs(kw.get("y", L(pkg, F16, (4, 64))), 1, kw.get("x", L(pkg, F16, (4, 64))), 1, kw.get("w", L(pkg, F16, (64,))), 1, 1e-5)
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.scheme(ok(y=L(pkg, F16, (4, 64, 1)))))      # rms_norm/args.rs:33-41
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.scheme(ok(w=L(pkg, F16, (1, 64)))))
    expect(pkg, pkg.TYPE_MISMATCH, lambda: op.scheme(ok(y=L(pkg, F32, (4, 64)))))             # :44
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(ok(x=L(pkg, F16, (5, 64)))))            # :46
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(ok(w=L(pkg, F16, (32,)))))              # :47
    # dynamic dims merge with static ones in scheme() (common/maybe_dyn.rs:80-94) and are refused by launch()
    dyn = ok(x=L(pkg, F16, (pkg.DYN_SIZE, 64), (pkg.DYN_STRIDE, 2)))
    assert op.scheme(dyn) == 0
    expect(pkg, pkg.DYNAMIC_NOT_SUPPORT, lambda: op.launch(dyn))
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: op.launch(ok(y=L(pkg, pkg.F64, (4, 64)), x=L(pkg, pkg.F64, (4, 64)), w=L(pkg, pkg.F64, (64,)))))


def test_rope_checks(pkg, dev):
    op, F16 = pkg.Rope(0), pkg.F16
    sc = L(pkg, F16, (0, 64))

    def args(t=None, p=None, sin=None, cos=None):
        return pkg.RopeArgs(t or L(pkg, F16, (7, 4, 64)), 1, p or L(pkg, pkg.U32, (7,)), 1, sin or sc, None, cos or sc, None, 1e4)

    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.scheme(args(t=L(pkg, F16, (7, 256)))))         # rope/args.rs:38-49
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.scheme(args(sin=L(pkg, F16, (64,)))))
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: op.scheme(args(t=L(pkg, pkg.U32, (7, 4, 64)))))  # :53-58 tokens must be floats
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: op.scheme(args(p=L(pkg, pkg.I32, (7,)))))         # :60-64 positions unsigned
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(args(p=L(pkg, pkg.U32, (8,)))))           # :69
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(args(cos=L(pkg, F16, (0, 32)))))          # :70
    expect(pkg, pkg.STRIDES_NOT_SUPPORT, lambda: op.launch(args(t=L(pkg, F16, (7, 4, 64), (1024, 256, 4)))))  # rope/common_cpu/mod.rs:98-100


def test_softmax_swiglu_checks(pkg, dev):
    sm, sw, F16 = pkg.FusedSoftmax(0), pkg.Swiglu(0), pkg.F16
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: sm.scheme(pkg.FusedSoftmaxArgs(pkg.MASK_CAUSAL, L(pkg, F16, (8, 8)), 1)))  # fuesd_softmax/args.rs:33-35
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: sm.launch(pkg.FusedSoftmaxArgs(pkg.MASK_CAUSAL, L(pkg, pkg.F64, (2, 8, 8)), 1)))
    expect(pkg, pkg.DYNAMIC_NOT_SUPPORT, lambda: sm.launch(pkg.FusedSoftmaxArgs(pkg.MASK_NONE, L(pkg, F16, (2, pkg.DYN_SIZE, 8), (128, 16, 2)), 1)))
    g = lambda **kw: pkg.SwigluArgs(kw.get("g", L(pkg, F16, (4, 64))), 1, kw.get("u", L(pkg, F16, (4, 64))), 1)
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: sw.scheme(g(u=L(pkg, F16, (256,)))))              # swiglu/args.rs:38-43
    expect(pkg, pkg.TYPE_MISMATCH, lambda: sw.scheme(g(u=L(pkg, pkg.F32, (4, 64)))))            # :46
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: sw.scheme(g(u=L(pkg, F16, (4, 65)))))               # :48


def test_mat_mul_checks(pkg, dev):
    op, F16 = pkg.MatMul(0), pkg.F16

    def mm(c, a, b):
        return pkg.MatMulArgs(c, 1, 0.0, a, 1, b, 1, 1.0)

    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.launch(mm(L(pkg, F16, (4, 8)), L(pkg, F16, (4, 6)), L(pkg, F16, (7, 8)))))      # mat_mul/args.rs:76-78
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.launch(mm(L(pkg, F16, (3, 4, 8)), L(pkg, F16, (2, 4, 6)), L(pkg, F16, (3, 6, 8)))))  # :81-83 batch
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.launch(mm(L(pkg, F16, (8,)), L(pkg, F16, (4, 6)), L(pkg, F16, (6, 8)))))      # :147-149
    expect(pkg, pkg.SHAPE_NOT_SUPPORT, lambda: op.launch(mm(L(pkg, F16, (2, 2, 4, 8)), L(pkg, F16, (2, 2, 4, 6)), L(pkg, F16, (2, 2, 6, 8)))))  # :163
    expect(pkg, pkg.STRIDES_NOT_SUPPORT, lambda: op.launch(mm(L(pkg, F16, (4, 8), (32, 4)), L(pkg, F16, (4, 6)), L(pkg, F16, (6, 8)))))  # :96, :185
    expect(pkg, pkg.DYNAMIC_NOT_SUPPORT, lambda: op.launch(mm(L(pkg, F16, (pkg.DYN_SIZE, 8), (16, 2)), L(pkg, F16, (4, 6)), L(pkg, F16, (6, 8)))))
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: op.launch(mm(L(pkg, pkg.U32, (4, 8)), L(pkg, pkg.U32, (4, 6)), L(pkg, pkg.U32, (6, 8)))))  # common_cpu/mod.rs:104


def test_attention_checks(pkg, dev):
    op, F16 = pkg.Attention(0), pkg.F16

    def at(q=None, k=None, v=None, o=None):
        return pkg.AttentionArgs(q or L(pkg, F16, (8, 4, 64)), 1, k or L(pkg, F16, (2, 16, 64)), 1, v or L(pkg, F16, (2, 16, 64)), 1,
                                 o or L(pkg, F16, (8, 4, 64)), 1, pkg.MASK_CAUSAL)

    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: op.scheme(at(q=L(pkg, F16, (8, 256)))))            # attention/args.rs:69-80
    expect(pkg, pkg.TYPE_MISMATCH, lambda: op.scheme(at(v=L(pkg, pkg.F32, (2, 16, 64)))))       # :83
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(at(o=L(pkg, F16, (4, 4, 64)))))           # :84 nh
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(at(v=L(pkg, F16, (2, 17, 64)))))          # :87 att
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.scheme(at(k=L(pkg, F16, (2, 16, 32)))))          # :88 dh
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: op.launch(at(k=L(pkg, F16, (3, 16, 64)), v=L(pkg, F16, (3, 16, 64)))))  # nh % nkvh
    # scheme() with every dim known reports the crate's q copy + score matrix (attention/operator.rs:96-104); with a dynamic dim, 0
    assert op.scheme(at()) == (8 * 4 * 64 + 8 * 4 * 16) * 2
    assert op.scheme(at(), max_workspace_size=8 * 4 * 64 * 2) == 8 * 4 * 64 * 2  # greedy prefix that fits (common/workspace.rs:78-89)
    assert op.scheme(at(q=L(pkg, F16, (8, pkg.DYN_SIZE, 64), (pkg.DYN_STRIDE,) * 3), o=L(pkg, F16, (8, pkg.DYN_SIZE, 64), (pkg.DYN_STRIDE,) * 3))) == 0


def test_random_sample_and_all_reduce_checks(pkg, dev):
    rs = pkg.RandomSample(0)
    kv, lg = torch.zeros(2, dtype=torch.int32, device=dev), torch.zeros(16, dtype=torch.float16, device=dev)
    mk = lambda **kw: pkg.RandomSampleArgs(kw.get("kv", pkg.TensorLayout(pkg.KVPAIR, (), ())), kv, kw.get("lg", L(pkg, pkg.F16, (16,))), lg,
                                           kw.get("ix", L(pkg, pkg.U32, (16,))), None, pkg.SampleArgs.arg_max(), 0.0)
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: rs.scheme(mk(lg=L(pkg, pkg.F64, (16,)))))          # random_sample/args.rs:105-107 element too large
    expect(pkg, pkg.TYPE_NOT_SUPPORT, lambda: rs.scheme(mk(ix=L(pkg, pkg.U64, (16,)))))          # :108-110
    expect(pkg, pkg.RANK_NOT_SUPPORT, lambda: rs.scheme(mk(lg=L(pkg, pkg.F16, (4, 4)))))         # :111-113
    assert rs.scheme(mk(), max_workspace_size=10) == 0 and rs.scheme(mk()) == 256                # both modes fit / nothing fits (cuda/mod.rs:58-81)
    comm = pkg.Comm(0, 0, 1)
    ar = pkg.AllReduce(comm)
    x = torch.zeros(4, 8, dtype=torch.float16, device=dev)
    expect(pkg, pkg.TYPE_MISMATCH, lambda: ar.launch(pkg.AllReduceArgs(L(pkg, pkg.F16, (4, 8)), x, L(pkg, pkg.F32, (4, 8)), x)))   # all_reduce/args.rs:38
    expect(pkg, pkg.STRIDES_NOT_SUPPORT, lambda: ar.launch(pkg.AllReduceArgs(L(pkg, pkg.F16, (4, 8), (32, 2)), x, L(pkg, pkg.F16, (4, 8)), x)))  # :46-52
    expect(pkg, pkg.SHAPE_MISMATCH, lambda: ar.launch(pkg.AllReduceArgs(L(pkg, pkg.F16, (4, 8)), x, L(pkg, pkg.F16, (31,)), x)))  # :70-72
    # a single rank behaves like NonAllReduce: copy unless in place (operators/src/lib.rs:199-224)
    src = torch.arange(32, dtype=torch.float16, device=dev).view(4, 8)
    dst = torch.zeros_like(src)
    ar.launch(pkg.AllReduceArgs.of(dst, src))
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    del ar
    comm.destroy()
