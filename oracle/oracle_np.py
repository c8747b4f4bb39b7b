"""NumPy twin of oracle.cc — a second, independent restatement of the reference's `common_cpu` operators.

TEST INFRASTRUCTURE ONLY.  It exists to cross-check the C++ restatement (two people copying the same
Rust by hand rarely make the same mistake) and to generate the small golden fixtures under
tests/golden/.  Pure-Python loops, so small cases only.  Arithmetic is done with np.float32 scalars so
that every intermediate rounds like Rust's f32; transcendental functions come from Python's `math`
(libm, in double) rounded to f32, which can differ from libm's expf/powf/sincosf in the last bit —
comparisons against oracle.cc therefore allow one f16 ulp where such a function is involved and are
exact elsewhere.
"""
import math

import numpy as np

f32 = np.float32
f16 = np.float16


def rms_norm(x, w, eps):
    """rms_norm/common_cpu/mod.rs:128-137, :195-208 (f16 data: f32 math, one rounding)."""
    n, d = x.shape
    y = np.empty_like(x)
    for i in range(n):
        s = f32(0)
        for j in range(d):
            v = f32(x[i, j])
            s = f32(s + f32(v * v))
        k = f32(f32(1) / f32(np.sqrt(f32(f32(s / f32(d)) + f32(eps)))))
        for j in range(d):
            y[i, j] = x.dtype.type(f32(f32(k * f32(w[j])) * f32(x[i, j])))
    return y


def rope(t, pos, theta):
    """rope/common_cpu/mod.rs:193-202, :164-171, :212-240."""
    nt, nh, dh = t.shape
    h = dh // 2
    out = t.copy()
    for i in range(nt):
        for k in range(h):
            denom = f32(math.pow(float(f32(theta)), float(f32(f32(k) / f32(h)))))
            ang = f32(f32(pos[i]) / denom)
            s, c = f32(math.sin(float(ang))), f32(math.cos(float(ang)))
            for j in range(nh):
                a, b = f32(t[i, j, 2 * k]), f32(t[i, j, 2 * k + 1])
                out[i, j, 2 * k] = t.dtype.type(f32(f32(a * c) - f32(b * s)))
                out[i, j, 2 * k + 1] = t.dtype.type(f32(f32(a * s) + f32(b * c)))
    return out


def fused_softmax(att, causal=True):
    """fuesd_softmax/common_cpu/mod.rs:99-145 (f16: exp stored rounded, sum unrounded, second rounding)."""
    nh, seq, al = att.shape
    out = att.copy()
    for j in range(nh):
        for k in range(seq):
            lim = al - seq + k + 1 if causal else al
            row = out[j, k]
            m = f32(max(float(v) for v in row[:lim]))
            s = f32(0)
            for p in range(lim):
                e = f32(math.exp(float(f32(f32(row[p]) - m))))
                row[p] = att.dtype.type(e)
                s = f32(s + e)
            r = f32(f32(1) / s)
            for p in range(lim):
                row[p] = att.dtype.type(f32(f32(row[p]) * r))
            row[lim:] = 0
    return out


def swiglu(gate, up):
    """swiglu/common_cpu/mod.rs:109-137."""
    out = gate.copy()
    n, d = gate.shape
    for i in range(n):
        for j in range(d):
            a, b = f32(gate[i, j]), f32(up[i, j])
            sig = f32(f32(1) / f32(f32(1) + f32(math.exp(float(-a)))))
            out[i, j] = gate.dtype.type(f32(f32(a * sig) * b))
    return out


def rearrange_scheme(esize, shape, dst_strides, src_strides):
    """rearrange/args.rs:34-153 -> [unit, idx_strides..., 1, dst_strides..., src_strides...]."""
    dims = [[l, d, s] for l, d, s in zip(shape, dst_strides, src_strides) if l != 1]
    for l, d, s in dims:
        if d == 0:
            raise ValueError("Reducing is not allowed for rearrangement.")
    dims.sort(key=lambda t: (-abs(t[1]), -abs(t[2]), t[0]))
    unit = esize
    while dims and dims[-1][1] == unit and dims[-1][2] == unit:
        unit *= dims.pop()[0]
    for i in range(len(dims) - 1, 0, -1):
        f, b = dims[i - 1], dims[i]
        if b[1] * b[0] == f[1] and b[2] * b[0] == f[2]:
            dims[i - 1] = [b[0] * f[0], b[1], b[2]]
            dims[i] = [1, 0, 0]
    dims = [d for d in dims if d[0] != 1]
    nd = len(dims)
    idx = [d[0] for d in dims] + [1]
    for i in range(nd - 1, -1, -1):
        idx[i] *= idx[i + 1]
    return [unit] + idx + [d[1] for d in dims] + [d[2] for d in dims]


def mat_mul(c, beta, a, b, alpha):
    """mat_mul/common_cpu/mod.rs:60-105 for f16: alpha/beta rounded to f16, f32 accumulation, one rounding."""
    al, be = f32(f16(alpha)), f32(f16(beta))
    acc = np.matmul(a.astype(np.float32), b.astype(np.float32))
    keep = be * c.astype(np.float32) if beta != 0 else np.zeros_like(acc)
    return (keep + al * acc).astype(c.dtype)


def attention(q, k, v, causal=True):
    """attention/operator.rs:199-275 with q [nh,seq,dh], k,v [nkvh,att,dh]; returns o [nh,seq,dh]."""
    nh, seq, dh = q.shape
    nkvh, att, _ = k.shape
    g = nh // nkvh
    alpha = f32(f32(1) / f32(np.sqrt(f32(dh))))
    qx = q.reshape(nkvh, g * seq, dh)
    scores = mat_mul(np.zeros((nkvh, g * seq, att), q.dtype), 0.0, qx, np.swapaxes(k, 1, 2), float(alpha))
    probs = fused_softmax(scores.reshape(nh, seq, att), causal)
    o = mat_mul(np.zeros_like(qx), 0.0, probs.reshape(nkvh, g * seq, att), v, 1.0)
    return o.reshape(nh, seq, dh)


def argmax(x):
    """random_sample/common_cpu/mod.rs:102-109: the last of equal maxima; unordered compares count as Equal."""
    best = 0
    for i in range(1, len(x)):
        if not (float(x[best]) > float(x[i])):
            best = i
    return best, int(np.array(x[best]).view(np.uint16 if x.dtype == np.float16 else np.uint32))


def random_sample(x, t, top_p, top_k, seed):
    """random_sample/common_cpu/mod.rs:111-144."""
    n = len(x)
    order = sorted(range(n), key=lambda i: (-float(x[i]), i))
    vals = [f32(x[i]) for i in order]
    mx = vals[0]
    c = [f32(1)]
    for i in range(1, n):
        c.append(f32(c[-1] + f32(math.exp(float(f32(f32(vals[i] - mx) / f32(t)))))))
    pk = c[min(top_k, n) - 1]
    pp = f32(c[-1] * f32(min(top_p, 1.0)))
    lim = f32(f32(seed) * min(pk, pp))
    j = next(i for i in range(n) if c[i] >= lim)
    val = np.array(c[j]).astype(x.dtype)
    return order[j], int(val.view(np.uint16 if x.dtype == np.float16 else np.uint32))


def all_reduce(bufs):
    """all_reduce/common_cpu.rs:66-104 + broadcast: pairwise tree towards the last rank, each add rounded in the dtype."""
    p = len(bufs)
    bufs = [b.copy() for b in bufs]
    stride = 1
    while stride < p:
        for r in range(2 * stride - 1, p, 2 * stride):
            if bufs[r].dtype == np.float16:
                bufs[r] = (bufs[r].astype(np.float32) + bufs[r - stride].astype(np.float32)).astype(np.float16)
            else:
                bufs[r] = bufs[r] + bufs[r - stride]
        stride *= 2
    return [bufs[p - 1].copy() for _ in range(p)]
