"""operators-rs_b200 — host-side mirror of the operators-rs per-operator interface over the C ABI.

The reference crate exposes every operator as `Operator::{new, scheme, launch}` taking an `Args`
struct of `TensorLayout`s + base pointers (operators/src/lib.rs:105-144).  This module keeps those
names and meanings for Python callers (tests, bench, the layer driver) and forwards every call to
`libops_b200.so` through ctypes — the same entry points a Rust shim binds (include/ops_b200.h).

There is no CPU path here: the compute lives in the CUDA library, and importing this package
without the built library raises.  PyTorch is used only as the owner of device memory and streams
(the `QueueAlloc` of the crate): tensors provide base pointers, `torch.cuda.current_stream()` the
queue, `torch.empty` the workspace fallback.
"""
import ctypes
import os

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libops_b200.so")

# ---- error kinds (operators/src/common/error.rs:2-12, :21-25) ----
OK = 0
TYPE_NOT_SUPPORT, TYPE_MISMATCH, RANK_NOT_SUPPORT, RANK_MISMATCH, SHAPE_NOT_SUPPORT = 1, 2, 3, 4, 5
SHAPE_MISMATCH, STRIDES_NOT_SUPPORT, ARGS_NOT_SUPPORT, DYNAMIC_NOT_SUPPORT = 6, 7, 8, 9
EXECUTION_FAILED, WORKSPACE_TOO_SMALL = 100, 101
KIND_NAMES = {1: "TypeNotSupport", 2: "TypeMismatch", 3: "RankNotSupport", 4: "RankMismatch", 5: "ShapeNotSupport",
              6: "ShapeMismatch", 7: "StridesNotSupport", 8: "ArgsNotSupport", 9: "DynamicNotSupport",
              100: "ExecutionFailed", 101: "WorkspaceTooSmall"}

# ---- element types ----
F16, BF16, F32, F64, U8, U16, U32, U64, I8, I16, I32, I64, KVPAIR = range(1, 14)
DYN_SIZE = (1 << 64) - 1          # usize::MAX
DYN_STRIDE = (1 << 63) - 1        # isize::MAX
DYN_F32 = float("inf")
MASK_NONE, MASK_CAUSAL = 0, 1
REDUCE_SUM, REDUCE_PROD, REDUCE_MIN, REDUCE_MAX, REDUCE_MEAN = range(5)
ATTENTION_CHAIN, ATTENTION_FUSED, ATTENTION_FUSED_ONE_TILE = 0, 1, 2
ATTENTION_MAX_RUNS, ATTENTION_RUN_RECORD_BYTES = 4, 528  # OPS_ATTENTION_MAX_RUNS, OPS_ATTENTION_RUN_RECORD_BYTES
ALL_REDUCE_AUTO, ALL_REDUCE_NCCL, ALL_REDUCE_P2P_ONE_SHOT, ALL_REDUCE_P2P_TWO_SHOT = range(4)
COMM_ID_BYTES, COMM_P2P_HANDLE_BYTES = 128, 128


class SchemeError(RuntimeError):
    """SchemeError { kind, info } (operators/src/common/error.rs:14-18)."""

    def __init__(self, kind, info):
        super().__init__(f"{KIND_NAMES.get(kind, kind)}: {info}")
        self.kind, self.info = kind, info


class LaunchError(SchemeError):
    """LaunchError { kind: Scheme(kind) | ExecutionFailed, info } (operators/src/common/error.rs:27-31)."""


class _Layout(ctypes.Structure):
    _fields_ = [("dt", ctypes.c_uint32), ("ndim", ctypes.c_uint32),
                ("shape", ctypes.POINTER(ctypes.c_size_t)), ("strides", ctypes.POINTER(ctypes.c_ssize_t))]


class TensorLayout:
    """dtype + shape + BYTE strides (operators/src/common/tensor.rs:17-61)."""

    def __init__(self, dt, shape, strides):
        assert len(shape) == len(strides)
        self.dt, self.shape, self.strides = int(dt), tuple(int(s) for s in shape), tuple(int(s) for s in strides)
        n = len(self.shape)
        self._shape = (ctypes.c_size_t * max(n, 1))(*self.shape)
        self._strides = (ctypes.c_ssize_t * max(n, 1))(*self.strides)
        self.c = _Layout(self.dt, n, self._shape, self._strides)

    @classmethod
    def new_contiguous(cls, dt, shape):
        strides, mul = [], dtype_nbytes(dt)
        for d in reversed(shape):
            strides.append(mul)
            mul *= d
        return cls(dt, shape, strides[::-1])

    @classmethod
    def of(cls, tensor):
        """Layout of a torch tensor (or numpy array)."""
        if hasattr(tensor, "element_size"):
            es = tensor.element_size()
            return cls(_torch_dt(tensor.dtype), tuple(tensor.shape), tuple(s * es for s in tensor.stride()))
        return cls(_numpy_dt(tensor.dtype), tensor.shape, tensor.strides)

    @property
    def ndim(self):
        return len(self.shape)

    def __repr__(self):
        return f"TensorLayout(dt={self.dt}, shape={self.shape}, strides={self.strides})"


def _torch_dt(dtype):
    import torch
    return {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.float64: F64, torch.uint8: U8,
            torch.int8: I8, torch.int16: I16, torch.int32: I32, torch.int64: I64, torch.uint16: U16,
            torch.uint32: U32, torch.uint64: U64}[dtype]


def _numpy_dt(dtype):
    import numpy as np
    return {np.dtype(np.float16): F16, np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.uint8): U8,
            np.dtype(np.uint16): U16, np.dtype(np.uint32): U32, np.dtype(np.uint64): U64, np.dtype(np.int8): I8,
            np.dtype(np.int16): I16, np.dtype(np.int32): I32, np.dtype(np.int64): I64}[np.dtype(dtype)]


def ptr(t):
    """Base pointer of a torch tensor (None -> null = dynamic)."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


# ---------------------------------------------------------------------------------------------------
# library loading
# ---------------------------------------------------------------------------------------------------
_lib = None


def lib():
    """The C-ABI library.  Raises if it is not built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(the operators have no CPU or PyTorch fallback)")
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def build(force=False):
    return _build.build(force=force)


def _declare(L):
    L.ops_last_error.restype = ctypes.c_char_p
    L.ops_last_workspace_need.restype = ctypes.c_size_t
    L.ops_dtype_nbytes.restype = ctypes.c_size_t
    L.ops_dtype_nbytes.argtypes = [ctypes.c_uint32]
    L.ops_build_info.restype = ctypes.c_char_p
    L.ops_random_sample_batched_workspace.restype = ctypes.c_size_t
    L.ops_random_sample_batched_workspace.argtypes = [ctypes.c_uint32, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p]
    for name in EXPORTS:
        getattr(L, name)  # fail early on a stale library


_NBYTES = {F16: 2, BF16: 2, F32: 4, F64: 8, U8: 1, U16: 2, U32: 4, U64: 8, I8: 1, I16: 2, I32: 4, I64: 8, KVPAIR: 8}


def dtype_nbytes(dt):
    return _NBYTES[dt]


def device_count():
    return lib().ops_device_count()


def last_error():
    return lib().ops_last_error().decode(errors="replace")


def _check(rc, launching):
    if rc == OK:
        return
    cls = LaunchError if launching else SchemeError
    raise cls(rc, last_error())


# ---------------------------------------------------------------------------------------------------
# Args structs (field order = include/ops_b200.h)
# ---------------------------------------------------------------------------------------------------
def _vp(v):
    return ctypes.c_void_p(ptr(v))


class _ArgsBase:
    """Keeps the TensorLayouts — and the tensors whose base pointers were taken — alive next to the ctypes struct
    that points into them (a tensor that dies before launch would hand its memory back to the allocator)."""
    c = None
    _alive = ()

    def byref(self):
        return ctypes.byref(self.c)


def _struct(name, fields):
    return type(name, (ctypes.Structure,), {"_fields_": fields})


_RmsNormArgs = _struct("_RmsNormArgs", [("y_layout", _Layout), ("y_base", ctypes.c_void_p), ("x_layout", _Layout),
                                        ("x_base", ctypes.c_void_p), ("w_layout", _Layout), ("w_base", ctypes.c_void_p),
                                        ("epsilon", ctypes.c_float)])
_RopeArgs = _struct("_RopeArgs", [("t_layout", _Layout), ("t_base", ctypes.c_void_p), ("p_layout", _Layout),
                                  ("p_base", ctypes.c_void_p), ("sin_layout", _Layout), ("sin_base", ctypes.c_void_p),
                                  ("cos_layout", _Layout), ("cos_base", ctypes.c_void_p), ("theta", ctypes.c_float)])
_SoftmaxArgs = _struct("_SoftmaxArgs", [("att_mask", ctypes.c_uint8), ("att_layout", _Layout), ("att_base", ctypes.c_void_p)])
_SwigluArgs = _struct("_SwigluArgs", [("gate_layout", _Layout), ("gate_base", ctypes.c_void_p), ("up_layout", _Layout),
                                      ("up_base", ctypes.c_void_p)])
_RearrangeArgs = _struct("_RearrangeArgs", [("dst_layout", _Layout), ("dst_base", ctypes.c_void_p), ("src_layout", _Layout),
                                            ("src_base", ctypes.c_void_p)])
_MatMulArgs = _struct("_MatMulArgs", [("c_layout", _Layout), ("c_base", ctypes.c_void_p), ("beta", ctypes.c_float),
                                      ("a_layout", _Layout), ("a_base", ctypes.c_void_p), ("b_layout", _Layout),
                                      ("b_base", ctypes.c_void_p), ("alpha", ctypes.c_float)])
_AttentionArgs = _struct("_AttentionArgs", [("q_layout", _Layout), ("q_base", ctypes.c_void_p), ("k_layout", _Layout),
                                            ("k_base", ctypes.c_void_p), ("v_layout", _Layout), ("v_base", ctypes.c_void_p),
                                            ("o_layout", _Layout), ("o_base", ctypes.c_void_p), ("mask", ctypes.c_uint8)])
_AttnCachedArgs = _struct("_AttnCachedArgs", [("q_layout", _Layout), ("q_base", ctypes.c_void_p), ("k_layout", _Layout),
                                              ("k_base", ctypes.c_void_p), ("v_layout", _Layout), ("v_base", ctypes.c_void_p),
                                              ("o_layout", _Layout), ("o_base", ctypes.c_void_p),
                                              ("k_cache_layout", _Layout), ("k_cache_base", ctypes.c_void_p),
                                              ("v_cache_layout", _Layout), ("v_cache_base", ctypes.c_void_p),
                                              ("mask", ctypes.c_uint8), ("pos", ctypes.c_size_t)])
_SampleArgs = _struct("_SampleArgs", [("temperature", ctypes.c_float), ("top_p", ctypes.c_float), ("top_k", ctypes.c_size_t)])
_RandomSampleArgs = _struct("_RandomSampleArgs", [("kv_pair", _Layout), ("kv_pair_base", ctypes.c_void_p), ("logits", _Layout),
                                                  ("logits_base", ctypes.c_void_p), ("indices", _Layout),
                                                  ("indices_base", ctypes.c_void_p), ("config", _SampleArgs),
                                                  ("seed", ctypes.c_float)])
_AllReduceArgs = _struct("_AllReduceArgs", [("pair", _RearrangeArgs), ("op", ctypes.c_uint8)])
_BroadcastArgs = _struct("_BroadcastArgs", [("pair", _RearrangeArgs), ("root", ctypes.c_size_t)])
_RmsNormAddArgs = _struct("_RmsNormAddArgs", [("norm", _RmsNormArgs), ("r_layout", _Layout), ("r_base", ctypes.c_void_p)])
_AddArgs = _struct("_AddArgs", [("c_layout", _Layout), ("c_base", ctypes.c_void_p), ("a_layout", _Layout), ("a_base", ctypes.c_void_p),
                                ("b_layout", _Layout), ("b_base", ctypes.c_void_p)])
_AddRowsArgs = _struct("_AddRowsArgs", [("dst_layout", _Layout), ("dst_base", ctypes.c_void_p), ("src_layout", _Layout),
                                        ("src_base", ctypes.c_void_p), ("idx_layout", _Layout), ("idx_base", ctypes.c_void_p)])


def _lay(x):
    return x if isinstance(x, TensorLayout) else TensorLayout.of(x)


class RmsNormArgs(_ArgsBase):
    """rms_norm::Args (operators/src/rms_norm/args.rs:7-15)."""

    def __init__(self, y_layout, y_base, x_layout, x_base, w_layout, w_base, epsilon):
        self._alive = (y_base, x_base, w_base,)
        self.keep = (_lay(y_layout), _lay(x_layout), _lay(w_layout))
        self.c = _RmsNormArgs(self.keep[0].c, _vp(y_base), self.keep[1].c, _vp(x_base), self.keep[2].c, _vp(w_base), epsilon)

    @classmethod
    def of(cls, y, x, w, epsilon):
        return cls(y, y, x, x, w, w, epsilon)


class RmsNormAddArgs(_ArgsBase):
    """Arguments of the extension ops_rms_norm_add_launch: x <- x + r in place, then y <- rms_norm(x)."""

    def __init__(self, y, x, w, epsilon, r):
        self.norm = RmsNormArgs.of(y, x, w, epsilon)
        self._alive = (r,)
        self.keep = (_lay(r),)
        self.c = _RmsNormAddArgs(self.norm.c, self.keep[0].c, _vp(r))

    @classmethod
    def of(cls, y, x, w, epsilon, r):
        return cls(y, x, w, epsilon, r)


class RopeArgs(_ArgsBase):
    """rope::Args (operators/src/rope/args.rs:8-18)."""

    def __init__(self, t_layout, t_base, p_layout, p_base, sin_layout, sin_base, cos_layout, cos_base, theta):
        self._alive = (t_base, p_base, sin_base, cos_base,)
        self.keep = (_lay(t_layout), _lay(p_layout), _lay(sin_layout), _lay(cos_layout))
        self.c = _RopeArgs(self.keep[0].c, _vp(t_base), self.keep[1].c, _vp(p_base), self.keep[2].c, _vp(sin_base),
                           self.keep[3].c, _vp(cos_base), theta)

    @classmethod
    def of(cls, t, pos, theta):
        dh = t.shape[2]
        dt = TensorLayout.of(t).dt
        empty = TensorLayout.new_contiguous(dt, (0, dh))  # the CPU path's empty sin/cos table (rope/common_cpu/mod.rs:12-25)
        return cls(t, t, pos, pos, empty, None, empty, None, theta)


class FusedSoftmaxArgs(_ArgsBase):
    """fuesd_softmax::Args (operators/src/fuesd_softmax/args.rs:5-9)."""

    def __init__(self, att_mask, att_layout, att_base):
        self._alive = (att_base,)
        self.keep = (_lay(att_layout),)
        self.c = _SoftmaxArgs(att_mask, self.keep[0].c, _vp(att_base))

    @classmethod
    def of(cls, att, mask=MASK_CAUSAL):
        return cls(mask, att, att)


class SwigluArgs(_ArgsBase):
    """swiglu::Args (operators/src/swiglu/args.rs:7-12)."""

    def __init__(self, gate_layout, gate_base, up_layout, up_base):
        self._alive = (gate_base, up_base,)
        self.keep = (_lay(gate_layout), _lay(up_layout))
        self.c = _SwigluArgs(self.keep[0].c, _vp(gate_base), self.keep[1].c, _vp(up_base))

    @classmethod
    def of(cls, gate, up):
        return cls(gate, gate, up, up)


class RearrangeArgs(_ArgsBase):
    """rearrange::Args (operators/src/rearrange/args.rs:11-17)."""

    def __init__(self, dst_layout, dst_base, src_layout, src_base):
        self._alive = (dst_base, src_base,)
        self.keep = (_lay(dst_layout), _lay(src_layout))
        self.c = _RearrangeArgs(self.keep[0].c, _vp(dst_base), self.keep[1].c, _vp(src_base))

    @classmethod
    def of(cls, dst, src):
        return cls(dst, dst, src, src)


class MatMulArgs(_ArgsBase):
    """mat_mul::Args (operators/src/mat_mul/args.rs:11-20): C = beta*C + alpha*A*B."""

    def __init__(self, c_layout, c_base, beta, a_layout, a_base, b_layout, b_base, alpha):
        self._alive = (c_base, a_base, b_base,)
        self.keep = (_lay(c_layout), _lay(a_layout), _lay(b_layout))
        self.c = _MatMulArgs(self.keep[0].c, _vp(c_base), beta, self.keep[1].c, _vp(a_base), self.keep[2].c, _vp(b_base), alpha)

    @classmethod
    def of(cls, c, beta, a, b, alpha):
        return cls(c, c, beta, a, a, b, b, alpha)


class AttentionArgs(_ArgsBase):
    """attention::Args (operators/src/attention/args.rs:10-24)."""

    def __init__(self, q_layout, q_base, k_layout, k_base, v_layout, v_base, o_layout, o_base, mask):
        self._alive = (q_base, k_base, v_base, o_base,)
        self.keep = (_lay(q_layout), _lay(k_layout), _lay(v_layout), _lay(o_layout))
        self.c = _AttentionArgs(self.keep[0].c, _vp(q_base), self.keep[1].c, _vp(k_base), self.keep[2].c, _vp(v_base),
                                self.keep[3].c, _vp(o_base), mask)

    @classmethod
    def of(cls, q, k, v, o, mask=MASK_CAUSAL):
        return cls(q, q, k, k, v, v, o, o, mask)


class AttentionKvCachedArgs(_ArgsBase):
    """attention_kv_cached::Args (operators/src/attention_kv_cached/args.rs:8-30)."""

    def __init__(self, q_layout, q_base, k_layout, k_base, v_layout, v_base, o_layout, o_base, k_cache_layout,
                 k_cache_base, v_cache_layout, v_cache_base, mask, pos):
        self._alive = (q_base, k_base, v_base, o_base, k_cache_base, v_cache_base,)
        self.keep = tuple(_lay(x) for x in (q_layout, k_layout, v_layout, o_layout, k_cache_layout, v_cache_layout))
        k = self.keep
        self.c = _AttnCachedArgs(k[0].c, _vp(q_base), k[1].c, _vp(k_base), k[2].c, _vp(v_base), k[3].c, _vp(o_base),
                                 k[4].c, _vp(k_cache_base), k[5].c, _vp(v_cache_base), mask, pos)

    @classmethod
    def of(cls, q, k, v, o, k_cache, v_cache, pos, mask=MASK_CAUSAL):
        return cls(q, q, k, k, v, v, o, o, k_cache, k_cache, v_cache, v_cache, mask, pos)


class SampleArgsError(ValueError):
    """SampleArgsError::{NegativeTemperature, NonPositiveTop} (operators/src/random_sample/args.rs:27-31)."""


class SampleArgs:
    """random_sample::SampleArgs (operators/src/random_sample/args.rs:20-84)."""

    def __init__(self, temperature, top_p, top_k):
        c = _SampleArgs()
        rc = lib().ops_sample_args_new(ctypes.c_float(temperature), ctypes.c_float(top_p), ctypes.c_size_t(top_k), ctypes.byref(c))
        if rc == 1:
            raise SampleArgsError("NegativeTemperature")
        if rc == 2:
            raise SampleArgsError("NonPositiveTop")
        self.c = c

    @classmethod
    def arg_max(cls):
        return cls(0.0, 1.0, DYN_SIZE)

    def is_argmax(self):
        return self.c.temperature == 0.0 or self.c.top_k == 1


class RandomSampleArgs(_ArgsBase):
    """random_sample::Args (operators/src/random_sample/args.rs:9-18)."""

    def __init__(self, kv_pair, kv_pair_base, logits, logits_base, indices, indices_base, config, seed):
        self._alive = (kv_pair_base, logits_base, indices_base,)
        self.keep = (_lay(kv_pair), _lay(logits), _lay(indices), config)
        self.c = _RandomSampleArgs(self.keep[0].c, _vp(kv_pair_base), self.keep[1].c, _vp(logits_base), self.keep[2].c,
                                   _vp(indices_base), config.c, seed)

    @classmethod
    def of(cls, kv_out, logits, config, seed=0.0):
        n = logits.shape[0]
        return cls(TensorLayout(KVPAIR, (), ()), kv_out, logits, logits, TensorLayout.new_contiguous(U32, (n,)), None, config, seed)


class AllReduceArgs(_ArgsBase):
    """all_reduce::Args { pair: rearrange::Args, op: ReduceOp } (operators/src/all_reduce/args.rs:9-12)."""

    def __init__(self, dst_layout, dst_base, src_layout, src_base, op=REDUCE_SUM):
        self._alive = (dst_base, src_base,)
        self.keep = (_lay(dst_layout), _lay(src_layout))
        self.c = _AllReduceArgs(_RearrangeArgs(self.keep[0].c, _vp(dst_base), self.keep[1].c, _vp(src_base)), op)

    @classmethod
    def of(cls, dst, src, op=REDUCE_SUM):
        return cls(dst, dst, src, src, op)


class BroadcastArgs(_ArgsBase):
    """broadcast::Args { pair: rearrange::Args, root } (operators/src/broadcast/args.rs:7-10)."""

    def __init__(self, dst_layout, dst_base, src_layout, src_base, root):
        self.keep = (_lay(dst_layout), _lay(src_layout))
        self._alive = (dst_base, src_base,)
        self.c = _BroadcastArgs(_RearrangeArgs(self.keep[0].c, _vp(dst_base), self.keep[1].c, _vp(src_base)), root)

    @classmethod
    def of(cls, dst, src, root):
        return cls(dst, dst, src, src, root)


class AddArgs(_ArgsBase):
    """add::Args (operators/src/add/args.rs:12-20): c = a + b."""

    def __init__(self, c_layout, c_base, a_layout, a_base, b_layout, b_base):
        self.keep = (_lay(c_layout), _lay(a_layout), _lay(b_layout))
        self._alive = (c_base, a_base, b_base,)
        self.c = _AddArgs(self.keep[0].c, _vp(c_base), self.keep[1].c, _vp(a_base), self.keep[2].c, _vp(b_base))

    @classmethod
    def of(cls, c, a, b):
        return cls(c, c, a, a, b, b)


class AddRowsArgs(_ArgsBase):
    """add_rows::Args (operators/src/add_rows/args.rs:10-17): dst[b, m, :] += src[idx[b, m], :]."""

    def __init__(self, dst_layout, dst_base, src_layout, src_base, idx_layout, idx_base):
        self.keep = (_lay(dst_layout), _lay(src_layout), _lay(idx_layout))
        self._alive = (dst_base, src_base, idx_base,)
        self.c = _AddRowsArgs(self.keep[0].c, _vp(dst_base), self.keep[1].c, _vp(src_base), self.keep[2].c, _vp(idx_base))

    @classmethod
    def of(cls, dst, src, idx):
        return cls(dst, dst, src, src, idx, idx)


# ---------------------------------------------------------------------------------------------------
# operators
# ---------------------------------------------------------------------------------------------------
def current_stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


class TorchQueueAlloc:
    """QueueAlloc of the crate (operators/src/lib.rs:95-102) on top of torch's caching allocator."""

    def __init__(self, device=None, stream=None):
        self.device, self.stream = device, stream

    def queue(self):
        return self.stream if self.stream is not None else current_stream()

    def alloc(self, size):
        import torch
        return torch.empty(max(int(size), 1), dtype=torch.uint8, device=self.device if self.device is not None else "cuda")


class Operator:
    """Operator::{new, scheme, launch} (operators/src/lib.rs:105-144) bound to ops_<NAME>_*."""
    NAME = None

    def __init__(self, node=0):
        L = lib()
        self._h = ctypes.c_void_p()
        self._destroy = getattr(L, f"ops_{self.NAME}_destroy")
        self._destroy.argtypes = [ctypes.c_void_p]
        self._destroy.restype = None
        self._scheme = getattr(L, f"ops_{self.NAME}_scheme")
        self._launch = getattr(L, f"ops_{self.NAME}_launch")
        self._create(L, node)

    def _create(self, L, node):
        self.device = int(node)
        _check(getattr(L, f"ops_{self.NAME}_create")(ctypes.c_int(self.device), ctypes.byref(self._h)), False)

    @classmethod
    def new(cls, node=0):
        return cls(node)

    def scheme(self, args, max_workspace_size=DYN_SIZE):
        out = ctypes.c_size_t(0)
        _check(self._scheme(self._h, args.byref(), ctypes.c_size_t(max_workspace_size), ctypes.byref(out)), False)
        return out.value

    def launch(self, args, workspace=None, queue_alloc=None):
        """Enqueue on queue_alloc.queue().  A short workspace is topped up from queue_alloc and the
        call repeated, as Workspace::new does in the crate (operators/src/common/workspace.rs:12-21)."""
        qa = queue_alloc or TorchQueueAlloc()
        stream = ctypes.c_void_p(qa.queue())
        self._last_args = args  # the enqueued kernels read these buffers: keep them until the next launch
        ws_ptr, ws_len = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        rc = self._launch(self._h, args.byref(), ctypes.c_void_p(ws_ptr), ctypes.c_size_t(ws_len), stream)
        if rc == WORKSPACE_TOO_SMALL:
            need = lib().ops_last_workspace_need()
            own = qa.alloc(need)
            rc = self._launch(self._h, args.byref(), ctypes.c_void_p(own.data_ptr()), ctypes.c_size_t(need), stream)
            self._last_ws = own  # stream-ordered reuse by torch's allocator keeps this safe once dropped
        _check(rc, True)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and h.value:
            try:
                self._destroy(h)
            except Exception:
                pass


class RmsNorm(Operator):
    NAME = "rms_norm"

    def launch_add(self, args, queue_alloc=None):
        """ops_rms_norm_add_launch: the residual add in front of the norm folded into it (one pass over every row)."""
        qa = queue_alloc or TorchQueueAlloc()
        self._last_args = args
        _check(lib().ops_rms_norm_add_launch(self._h, args.byref(), ctypes.c_void_p(qa.queue())), True)


class Rope(Operator):
    NAME = "rope"

    @staticmethod
    def build_pos(dt, nt, seqs):
        """Rope::build_pos (operators/src/rope/mod.rs:17-21): seqs = [(pos, len), ...] -> host numpy array."""
        import numpy as np
        out = np.zeros(nt, dtype=np.uint32 if dt == U32 else np.uint64)
        pos = (ctypes.c_size_t * max(len(seqs), 1))(*[p for p, _ in seqs])
        ln = (ctypes.c_size_t * max(len(seqs), 1))(*[l for _, l in seqs])
        _check(lib().ops_rope_build_pos(ctypes.c_uint32(dt), ctypes.c_size_t(nt), pos, ln, ctypes.c_size_t(len(seqs)),
                                        ctypes.c_void_p(out.ctypes.data)), False)
        return out


class FusedSoftmax(Operator):
    NAME = "fused_softmax"


class Swiglu(Operator):
    NAME = "swiglu"


class Rearrange(Operator):
    NAME = "rearrange"

    @staticmethod
    def plan(args):
        """rearrange::Scheme::new as host arithmetic -> the crate's scheme vector."""
        nd = args.keep[0].ndim
        out = (ctypes.c_ssize_t * (2 + 3 * nd + 3))()
        ndim = ctypes.c_size_t(0)
        _check(lib().ops_rearrange_plan(args.byref(), out, ctypes.c_size_t(len(out)), ctypes.byref(ndim)), False)
        return list(out[: 2 + 3 * ndim.value])


class MatMul(Operator):
    NAME = "mat_mul"

    def launch_all_reduce(self, comm, args, queue_alloc=None):
        """ops_mat_mul_all_reduce_launch: C = beta*C + alpha*A*B summed over the ranks of `comm`, one kernel."""
        qa = queue_alloc or TorchQueueAlloc()
        self._last_args = args
        _check(lib().ops_mat_mul_all_reduce_launch(self._h, comm._h, args.byref(), ctypes.c_void_p(qa.queue())), True)

    def status(self):
        return lib().ops_mat_mul_status(self._h)

    def status_reset(self):
        _check(lib().ops_mat_mul_status_reset(self._h), False)


class Attention(Operator):
    NAME = "attention"

    def set_algo(self, algo):
        _check(lib().ops_attention_set_algo(self._h, ctypes.c_int(algo)), False)

    def status(self):
        return lib().ops_attention_status(self._h)

    def status_reset(self):
        _check(lib().ops_attention_status_reset(self._h), False)


class AttentionKvCached(Operator):
    NAME = "attention_kv_cached"

    def set_algo(self, algo):
        _check(lib().ops_attention_kv_cached_set_algo(self._h, ctypes.c_int(algo)), False)


class RandomSample(Operator):
    NAME = "random_sample"

    @staticmethod
    def build_indices(n):
        import numpy as np
        out = np.zeros(n, dtype=np.uint32)
        _check(lib().ops_random_sample_build_indices(ctypes.c_size_t(n), ctypes.c_void_p(out.ctypes.data)), False)
        return out

    @staticmethod
    def noalloc_max_logits():
        f = lib().ops_random_sample_noalloc_max_logits
        f.restype = ctypes.c_size_t
        return f()

    def launch_noalloc(self, args, queue_alloc=None):
        """ops_random_sample_launch_noalloc: same result as launch(), no workspace and no allocation anywhere —
        for callers that cannot allocate where they sample.  Rows longer than noalloc_max_logits() are refused;
        overlapping calls on one device share the built-in scratch array and must be serialised by the caller."""
        qa = queue_alloc or TorchQueueAlloc()
        self._last_args = args
        _check(lib().ops_random_sample_launch_noalloc(self._h, args.byref(), ctypes.c_void_p(qa.queue())), True)

    def launch_batched(self, logits, kv_out, config, seeds=None, workspace=None, queue_alloc=None):
        """Extension: all rows of logits [rows, n] in one launch; kv_out [rows, 2] int32/uint32 view."""
        qa = queue_alloc or TorchQueueAlloc(device=logits.device)
        rows, n = logits.shape
        dt = _torch_dt(logits.dtype)
        need = lib().ops_random_sample_batched_workspace(ctypes.c_uint32(dt), ctypes.c_size_t(rows), ctypes.c_size_t(n), ctypes.byref(config.c))
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = qa.alloc(need)
        self._last_ws = workspace
        rc = lib().ops_random_sample_launch_batched(
            self._h, ctypes.c_uint32(dt), ctypes.c_size_t(rows), ctypes.c_size_t(n), ctypes.c_void_p(logits.data_ptr()),
            ctypes.c_ssize_t(logits.stride(0) * logits.element_size()), ctypes.c_void_p(kv_out.data_ptr()), ctypes.byref(config.c),
            ctypes.c_void_p(seeds.data_ptr() if seeds is not None else None), ctypes.c_void_p(workspace.data_ptr()),
            ctypes.c_size_t(workspace.numel() * workspace.element_size()), ctypes.c_void_p(qa.queue()))
        _check(rc, True)


class Comm:
    """The topology node of a communication operator (TopoNode: rank, group_size; operators/src/lib.rs:62-66),
    counterpart of NcclNode (operators/src/handle/cuda/nccl.rs:6-33)."""

    def __init__(self, device, rank, group_size, unique_id=None):
        self._h = ctypes.c_void_p()
        idbuf = (ctypes.c_uint8 * COMM_ID_BYTES)(*unique_id) if unique_id is not None else None
        _check(lib().ops_comm_init_rank(ctypes.c_int(device), ctypes.c_int(rank), ctypes.c_int(group_size), idbuf, ctypes.byref(self._h)), False)
        self.device = device

    @classmethod
    def loopback(cls, device, group_size, staging_bytes):
        """ops_comm_create_loopback: every peer is this rank's own buffer; for exercising the bounded waits on one GPU."""
        self = cls.__new__(cls)
        self._h = ctypes.c_void_p()
        self.device = device
        _check(lib().ops_comm_create_loopback(ctypes.c_int(device), ctypes.c_int(group_size), ctypes.c_size_t(staging_bytes), ctypes.byref(self._h)), False)
        return self

    @staticmethod
    def unique_id():
        buf = (ctypes.c_uint8 * COMM_ID_BYTES)()
        _check(lib().ops_comm_unique_id(buf), False)
        return bytes(buf)

    def rank(self):
        return lib().ops_comm_rank(self._h)

    def group_size(self):
        return lib().ops_comm_group_size(self._h)

    def p2p_export(self, staging_bytes):
        buf = (ctypes.c_uint8 * COMM_P2P_HANDLE_BYTES)()
        _check(lib().ops_comm_p2p_export(self._h, ctypes.c_size_t(staging_bytes), buf), False)
        return bytes(buf)

    def p2p_attach(self, all_handles):
        blob = b"".join(all_handles)
        buf = (ctypes.c_uint8 * len(blob))(*blob)
        _check(lib().ops_comm_p2p_attach(self._h, buf), False)

    def p2p_status(self):
        return lib().ops_comm_p2p_status(self._h)

    def p2p_reset(self):
        """ops_comm_p2p_reset: start over after a time-out (every rank, streams idle, after a host-side barrier)."""
        _check(lib().ops_comm_p2p_reset(self._h), False)

    def p2p_direct(self, dtype=None):
        """The zero-copy input region of this rank as a torch tensor (uint8, or `dtype`) that aliases it: a kernel that
        writes its partial there lets all_reduce read it in place (ops_comm_p2p_direct)."""
        import torch
        ptr, size = ctypes.c_void_p(), ctypes.c_size_t()
        _check(lib().ops_comm_p2p_direct(self._h, ctypes.byref(ptr), ctypes.byref(size)), False)

        class _Region:  # the CUDA array interface is how torch is told about memory it did not allocate
            __cuda_array_interface__ = {"shape": (size.value,), "typestr": "|u1", "data": (ptr.value, False), "version": 2}

        t = torch.as_tensor(_Region(), device=torch.device("cuda", self.device))
        self._direct_owner = t
        return t if dtype is None else t.view(dtype)

    def nvls_attach(self, multicast_ptr, local_tensor):
        """ops_comm_nvls_attach: `local_tensor` (uint8, this rank's part of a buffer bound to an NVLink multicast object whose
        multicast address is `multicast_ptr`) becomes [zero-copy input region | reserved] of the in-switch all_reduce.
        Returns the input region as a tensor view (first half)."""
        n = local_tensor.numel() * local_tensor.element_size()
        _check(lib().ops_comm_nvls_attach(self._h, ctypes.c_void_p(int(multicast_ptr)), ctypes.c_void_p(local_tensor.data_ptr()), ctypes.c_size_t(n)), False)
        self._nvls_owner = local_tensor
        return local_tensor.view(-1)[: n // 2] if local_tensor.dtype.itemsize == 1 else local_tensor.view(-1).view(__import__("torch").uint8)[: n // 2]

    def nvls_detach(self):
        _check(lib().ops_comm_nvls_attach(self._h, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_size_t(0)), False)
        self._nvls_owner = None

    def destroy(self):
        h, self._h = self._h, None
        if h and h.value:
            lib().ops_comm_destroy(h)


class AllReduce(Operator):
    NAME = "all_reduce"

    def _create(self, L, node):
        self.comm = node
        self.device = node.device
        _check(L.ops_all_reduce_create(node._h, ctypes.byref(self._h)), False)

    def set_algo(self, algo):
        _check(lib().ops_all_reduce_set_algo(self._h, ctypes.c_int(algo)), False)

    def launch_add(self, args, queue_alloc=None):
        """ops_all_reduce_add_launch: dst <- dst + sum over ranks of src, one kernel (dst replicated, dst is not src)."""
        qa = queue_alloc or TorchQueueAlloc()
        self._last_args = args
        _check(lib().ops_all_reduce_add_launch(self._h, args.byref(), ctypes.c_void_p(qa.queue())), True)


class Broadcast(Operator):
    NAME = "broadcast"

    def _create(self, L, node):
        self.comm = node
        self.device = node.device
        _check(L.ops_broadcast_create(node._h, ctypes.byref(self._h)), False)


class Add(Operator):
    NAME = "add"


class AddRows(Operator):
    NAME = "add_rows"

    def status(self):
        return lib().ops_add_rows_status(self._h)


EXPORTS = [
    "ops_last_error", "ops_last_workspace_need", "ops_dtype_nbytes", "ops_device_count", "ops_build_info",
    *[f"ops_{op}_{fn}" for op in ("rms_norm", "rope", "fused_softmax", "swiglu", "rearrange", "mat_mul", "attention",
                                  "attention_kv_cached", "random_sample", "all_reduce", "broadcast", "add", "add_rows")
      for fn in ("create", "scheme", "launch", "destroy")],
    "ops_rope_build_pos", "ops_rearrange_plan", "ops_mat_mul_status", "ops_mat_mul_status_reset", "ops_attention_set_algo", "ops_attention_status",
    "ops_attention_status_reset",
    "ops_attention_kv_cached_set_algo", "ops_sample_args_new", "ops_random_sample_build_indices",
    "ops_random_sample_batched_workspace", "ops_random_sample_launch_batched",
    "ops_random_sample_noalloc_max_logits", "ops_random_sample_launch_noalloc", "ops_comm_unique_id",
    "ops_comm_init_rank", "ops_comm_rank", "ops_comm_group_size", "ops_comm_destroy", "ops_comm_p2p_export",
    "ops_comm_p2p_attach", "ops_comm_p2p_status", "ops_comm_p2p_reset", "ops_comm_p2p_direct", "ops_comm_nvls_attach", "ops_all_reduce_add_launch",
    "ops_rms_norm_add_launch", "ops_comm_create_loopback", "ops_all_reduce_set_algo", "ops_add_rows_status", "ops_mat_mul_all_reduce_launch",
]
