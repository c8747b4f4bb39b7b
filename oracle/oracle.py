"""ctypes binding of the CPU oracle (liboracle.so, built from oracle.cc by the Makefile beside it).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's CPU-baseline legs.
The product package never imports this module.

All functions take NumPy arrays (any strides; byte strides are read from the array) and work in
place where the reference operator does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

# dtype codes of include/ops_b200.h
DT = {np.dtype(np.float16): 1, np.dtype(np.float32): 3, np.dtype(np.float64): 4, np.dtype(np.uint8): 5,
      np.dtype(np.uint16): 6, np.dtype(np.uint32): 7, np.dtype(np.uint64): 8, np.dtype(np.int8): 9,
      np.dtype(np.int16): 10, np.dtype(np.int32): 11, np.dtype(np.int64): 12}

_lib = None


class Bf16Array(np.ndarray):
    """bf16 values held as their uint16 bit patterns (NumPy has no bf16 type).  Slices, reshapes and transposes keep
    the tag, which is what tells the functions below to run the bf16 instantiation of the oracle."""


def bf16_from_f32(a):
    """Round f32 values to bf16 (nearest, ties to even) -> tagged uint16 array."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16).view(Bf16Array)


def bf16_bits(a):
    """Tag an array of uint16 bit patterns as bf16."""
    return np.asarray(a, dtype=np.uint16).view(Bf16Array)


def bf16_to_f32(a):
    return (np.asarray(a).view(np.ndarray).astype(np.uint32) << 16).view(np.float32)


def _dt(a):
    if isinstance(a, Bf16Array):
        return 2
    return DT[a.dtype]


def _zeros(shape, like):
    z = np.zeros(shape, like.dtype)
    return z.view(Bf16Array) if isinstance(like, Bf16Array) else z


def _empty_like(a):
    return _zeros(a.shape, a)


def build():
    """Compile liboracle.so with the Makefile (g++)."""
    subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_dtype_nbytes.restype = ctypes.c_size_t
    return _lib


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))


class OracleError(RuntimeError):
    def __init__(self, kind):
        super().__init__(f"oracle error kind {kind}")
        self.kind = kind


def _chk(rc):
    if rc != 0:
        raise OracleError(rc)


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _sz(v):
    return ctypes.c_size_t(int(v))


def _isz(v):
    return ctypes.c_ssize_t(int(v))


def _arr_sz(vals):
    return (ctypes.c_size_t * len(vals))(*[int(v) for v in vals])


def _arr_isz(vals):
    return (ctypes.c_ssize_t * len(vals))(*[int(v) for v in vals])


def rms_norm(y, x, w, eps):
    n, d = x.shape
    _chk(lib().orc_rms_norm(_dt(x), _dt(w), _sz(n), _sz(d), _p(y), _isz(y.strides[0]), _isz(y.strides[1]),
                            _p(x), _isz(x.strides[0]), _isz(x.strides[1]), _p(w), _isz(w.strides[0]),
                            ctypes.c_float(eps)))
    return y


def rope(t, pos, theta):
    nt, nh, dh = t.shape
    assert t.strides[2] == t.itemsize
    _chk(lib().orc_rope(_dt(t), _dt(pos), _sz(nt), _sz(nh), _sz(dh), _p(t), _isz(t.strides[0]),
                        _isz(t.strides[1]), _p(pos), _isz(pos.strides[0]), ctypes.c_float(theta)))
    return t


def fused_softmax(att, causal=True):
    nh, seq, al = att.shape
    _chk(lib().orc_fused_softmax(_dt(att), _sz(nh), _sz(seq), _sz(al), _p(att), _isz(att.strides[0]),
                                 _isz(att.strides[1]), _isz(att.strides[2]), ctypes.c_int(1 if causal else 0)))
    return att


def swiglu(gate, up):
    n, d = gate.shape
    _chk(lib().orc_swiglu(_dt(gate), _sz(n), _sz(d), _p(gate), _isz(gate.strides[0]), _isz(gate.strides[1]),
                          _p(up), _isz(up.strides[0]), _isz(up.strides[1])))
    return gate


def rearrange_scheme(esize, shape, dst_strides, src_strides, src_shape=None):
    """Returns the reference's Scheme vector [unit, idx..., 1, dst..., src...] as a list."""
    nd = len(shape)
    out = (ctypes.c_ssize_t * (2 + 3 * nd + 3))()
    out_len = ctypes.c_size_t(0)
    _chk(lib().orc_rearrange_scheme(_sz(esize), _sz(nd), _arr_sz(shape), _arr_sz(src_shape or shape),
                                    _arr_isz(dst_strides), _arr_isz(src_strides), out, ctypes.byref(out_len)))
    return list(out[: out_len.value])


def rearrange(dst, src):
    assert dst.dtype == src.dtype
    _chk(lib().orc_rearrange(_sz(dst.itemsize), _sz(dst.ndim), _arr_sz(dst.shape), _arr_sz(src.shape), _p(dst),
                             _arr_isz(dst.strides), _p(src), _arr_isz(src.strides)))
    return dst


def mat_mul(c, beta, a, b, alpha):
    _chk(lib().orc_mat_mul(_dt(c), _sz(c.ndim), _arr_sz(c.shape), _arr_isz(c.strides), _p(c), ctypes.c_float(beta),
                           _sz(a.ndim), _arr_sz(a.shape), _arr_isz(a.strides), _p(a),
                           _sz(b.ndim), _arr_sz(b.shape), _arr_isz(b.strides), _p(b), ctypes.c_float(alpha)))
    return c


def attention(q, k, v, o, causal=True):
    nh, seq, dh = q.shape
    nkvh, att, _ = k.shape
    _chk(lib().orc_attention(_dt(q), _sz(nh), _sz(nkvh), _sz(seq), _sz(att), _sz(dh), _p(q), _arr_isz(q.strides),
                             _p(k), _arr_isz(k.strides), _p(v), _arr_isz(v.strides), _p(o), _arr_isz(o.strides),
                             ctypes.c_int(1 if causal else 0)))
    return o


def attention_kv_cached(q, k, v, o, k_cache, v_cache, pos, causal=True):
    nh, seq, dh = q.shape
    nkvh = k.shape[0]
    _chk(lib().orc_attention_kv_cached(_dt(q), _sz(nh), _sz(nkvh), _sz(seq), _sz(dh), _sz(k_cache.shape[1]),
                                       _sz(v_cache.shape[1]), _sz(pos), _p(q), _arr_isz(q.strides), _p(k),
                                       _arr_isz(k.strides), _p(v), _arr_isz(v.strides), _p(o), _arr_isz(o.strides),
                                       _p(k_cache), _arr_isz(k_cache.strides), _p(v_cache),
                                       ctypes.c_int(1 if causal else 0)))
    return o


def random_sample(logits, temperature=0.0, top_p=1.0, top_k=2 ** 64 - 1, seed=0.0):
    """Returns (idx, val_bits) of the KVPair the reference would write."""
    assert logits.ndim == 1 and logits.strides[0] == logits.itemsize
    out = (ctypes.c_uint32 * 2)()
    _chk(lib().orc_random_sample(_dt(logits), _sz(logits.shape[0]), _p(logits), ctypes.c_float(temperature),
                                 ctypes.c_float(min(top_p, 1.0)), _sz(top_k), ctypes.c_float(seed), out))
    return int(out[0]), int(out[1])


def all_reduce(bufs):
    """Sum over the list of per-rank arrays, in place in every array (tree order of the reference)."""
    p = len(bufs)
    ptrs = (ctypes.c_void_p * p)(*[b.ctypes.data for b in bufs])
    _chk(lib().orc_all_reduce(_dt(bufs[0]), _sz(p), _sz(bufs[0].size), ptrs))
    return bufs


def broadcast(bufs, root):
    p = len(bufs)
    ptrs = (ctypes.c_void_p * p)(*[b.ctypes.data for b in bufs])
    _chk(lib().orc_broadcast(_sz(p), _sz(bufs[0].nbytes), _sz(root), ptrs))
    return bufs


def add(c, a, b):
    _chk(lib().orc_add(_dt(c), _sz(c.ndim), _arr_sz(c.shape), _p(c), _arr_isz(c.strides), _p(a), _arr_isz(a.strides), _p(b),
                       _arr_isz(b.strides)))
    return c


def add_rows(dst, src, idx):
    batch, m, n = dst.shape
    _chk(lib().orc_add_rows(_dt(dst), _dt(idx), _sz(batch), _sz(m), _sz(n), _sz(src.shape[0]), _p(dst), _isz(dst.strides[0]),
                            _isz(dst.strides[1]), _isz(dst.strides[2]), _p(src), _isz(src.strides[0]), _isz(src.strides[1]), _p(idx),
                            _isz(idx.strides[0]), _isz(idx.strides[1])))
    return dst


def decoder_layer(x, pos, shards, cfg):
    """The decoder-layer chain on the oracle operators (what a caller of the reference's common_cpu operators computes).

    x [T, d] f16, pos [T] u32, shards = list of per-rank weight dicts (one entry = no tensor parallelism),
    cfg = dict(d, nh, nkvh, dh, ffn, theta, eps).  Tensor-parallel ranks are emulated one after the other;
    partial sums meet in all_reduce (f16 tree order of all_reduce/common_cpu.rs).  Rank 0 folds the residual with beta = 1.
    Returns the layer output [T, d].
    """
    tp = len(shards)
    T, d = x.shape
    dh, nq, nkv, f = cfg["dh"], cfg["nh"] // tp, cfg["nkvh"] // tp, cfg["ffn"] // tp
    xs = [x.copy() for _ in range(tp)]

    def project(r, a, w_):
        if r == 0:
            out = xs[r]
            mat_mul(out, 1.0, a, w_, 1.0)
        else:
            out = _zeros((T, d), x)
            mat_mul(out, 0.0, a, w_, 1.0)
        return out

    parts = []
    for r, w in enumerate(shards):
        h = rms_norm(_empty_like(x), xs[r], w["w_norm1"], cfg["eps"])
        qkv = mat_mul(_zeros((T, (nq + 2 * nkv) * dh), x), 0.0, h, w["w_qkv"], 1.0)
        heads = qkv.reshape(T, nq + 2 * nkv, dh)
        rope(heads[:, : nq + nkv], pos, cfg["theta"])
        att_out = _zeros((T, nq * dh), x)
        attention(heads[:, :nq].transpose(1, 0, 2), heads[:, nq:nq + nkv].transpose(1, 0, 2), heads[:, nq + nkv:].transpose(1, 0, 2),
                  att_out.reshape(T, nq, dh).transpose(1, 0, 2), True)
        parts.append(project(r, att_out, w["w_o"]))
    if tp > 1:
        all_reduce(parts)
    xs = parts
    parts = []
    for r, w in enumerate(shards):
        h = rms_norm(_empty_like(x), xs[r], w["w_norm2"], cfg["eps"])
        gu = mat_mul(_zeros((T, 2 * f), x), 0.0, h, w["w_gu"], 1.0)
        swiglu(gu[:, :f], gu[:, f:])
        parts.append(project(r, gu[:, :f], w["w_down"]))
    if tp > 1:
        all_reduce(parts)
    return parts[0]
