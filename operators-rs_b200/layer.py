"""The decoder-layer operator chain, as a caller of the per-operator API.

The reference crate ships operators only; the chain below is what a downstream runtime does with
them for one Llama-shaped layer (BASELINE config 3) and its tensor-parallel form (config 4):

    rms_norm -> mat_mul(QKV) -> rope(q,k heads) -> attention -> mat_mul(O, beta=1 residual)
             -> [all_reduce] -> rms_norm -> mat_mul(gate|up) -> swiglu -> mat_mul(down, beta=1) -> [all_reduce]

Every step is one `Operator.launch` through the C ABI on torch-owned device buffers.  Tensor
parallelism follows the usual split: QKV and gate|up by columns (whole heads per rank, the GQA group
kept together), O and down by rows, f16 sum all_reduce of the [T, d] partials.  Rank 0 folds the
residual into its partial with beta = 1; the other ranks write their partial to a scratch buffer
(beta = 0) that becomes their residual stream after the all_reduce — no extra copy, no `add` operator.
"""
from dataclasses import dataclass

from . import (ALL_REDUCE_AUTO, MASK_CAUSAL, AllReduce, AllReduceArgs, Attention, AttentionArgs, FusedSoftmax, MatMul,
               MatMulArgs, Rearrange, RmsNorm, RmsNormArgs, Rope, RopeArgs, Swiglu, SwigluArgs)


@dataclass
class LayerConfig:
    d: int = 4096
    nh: int = 32
    nkvh: int = 8
    dh: int = 128
    ffn: int = 14336
    theta: float = 5e5
    eps: float = 1e-5

    def flops(self, tokens, tp=1):
        """Algorithmic flops of one layer pass on ONE rank: the four GEMMs + causal-useful attention."""
        d, ffn = self.d, self.ffn // tp
        qkv = (self.nh + 2 * self.nkvh) * self.dh // tp
        gemm = 2 * tokens * (d * qkv + (self.nh * self.dh // tp) * d + d * 2 * ffn + ffn * d)
        att = 4 * (self.nh // tp) * self.dh * (tokens * (tokens + 1) // 2)
        return gemm, att


def shard_weights(w, rank, tp, cfg):
    """Column/row split of the full weights for `rank` of `tp` (works on numpy arrays and torch tensors).

    w: dict with w_norm1 [d], w_qkv [d, (nh+2*nkvh)*dh] (q heads | k heads | v heads), w_o [nh*dh, d],
       w_norm2 [d], w_gu [d, 2*ffn] (gate | up), w_down [ffn, d].
    """
    if tp == 1:
        return dict(w)
    assert cfg.nh % tp == 0 and cfg.nkvh % tp == 0 and cfg.ffn % tp == 0, "heads and ffn must divide by tp"
    cat = _cat(w["w_qkv"])
    dh, nq, nkv, f = cfg.dh, cfg.nh // tp, cfg.nkvh // tp, cfg.ffn // tp
    q0, k0, v0 = 0, cfg.nh * dh, (cfg.nh + cfg.nkvh) * dh
    qkv = cat([w["w_qkv"][:, q0 + rank * nq * dh: q0 + (rank + 1) * nq * dh],
               w["w_qkv"][:, k0 + rank * nkv * dh: k0 + (rank + 1) * nkv * dh],
               w["w_qkv"][:, v0 + rank * nkv * dh: v0 + (rank + 1) * nkv * dh]], 1)
    gu = cat([w["w_gu"][:, rank * f:(rank + 1) * f], w["w_gu"][:, cfg.ffn + rank * f: cfg.ffn + (rank + 1) * f]], 1)
    return {"w_norm1": w["w_norm1"], "w_norm2": w["w_norm2"], "w_qkv": qkv, "w_gu": gu,
            "w_o": _contig(w["w_o"][rank * nq * dh:(rank + 1) * nq * dh]), "w_down": _contig(w["w_down"][rank * f:(rank + 1) * f])}


def _cat(x):
    if hasattr(x, "element_size"):
        import torch
        return lambda parts, dim: torch.cat(parts, dim).contiguous()
    import numpy as np
    return lambda parts, dim: np.ascontiguousarray(np.concatenate(parts, dim))


def _contig(x):
    if hasattr(x, "element_size"):
        return x.contiguous()
    import numpy as np
    return np.ascontiguousarray(x)


class DecoderLayer:
    """One (possibly tensor-parallel) decoder layer on one GPU.  `weights` are this rank's shards on the device."""

    STEPS = ("rms_norm_1", "mat_mul_qkv", "rope", "attention", "mat_mul_o", "all_reduce_1", "rms_norm_2", "mat_mul_gate_up",
             "swiglu", "mat_mul_down", "all_reduce_2")

    def __init__(self, cfg, weights, max_tokens, device, comm=None, tp=1, rank=0, all_reduce_algo=ALL_REDUCE_AUTO, overlap_chunks=1, fused_all_reduce=False):
        import torch
        self.overlap_chunks = max(1, int(overlap_chunks))
        self.fused_all_reduce = bool(fused_all_reduce) and tp > 1  # row-parallel GEMM and its all_reduce as one kernel
        self.comm = comm
        self.comm_stream = torch.cuda.Stream(device) if (tp > 1 and self.overlap_chunks > 1) else None
        self.cfg, self.w, self.device, self.tp, self.rank = cfg, weights, device, tp, rank
        idx = device.index if device.index is not None else 0
        self.rms_norm, self.rope, self.swiglu = RmsNorm(idx), Rope(idx), Swiglu(idx)
        self.mat_mul, self.attention = MatMul(idx), Attention(idx)
        self.all_reduce = None
        if tp > 1:
            self.all_reduce = AllReduce(comm)
            self.all_reduce.set_algo(all_reduce_algo)
        self.nq, self.nkv, self.f = cfg.nh // tp, cfg.nkvh // tp, cfg.ffn // tp
        T, f16 = max_tokens, torch.float16
        self.h = torch.empty(T, cfg.d, dtype=f16, device=device)
        self.qkv = torch.empty(T, (self.nq + 2 * self.nkv) * cfg.dh, dtype=f16, device=device)
        self.att_out = torch.empty(T, self.nq * cfg.dh, dtype=f16, device=device)
        self.gu = torch.empty(T, 2 * self.f, dtype=f16, device=device)
        self.scratch = torch.empty(T, cfg.d, dtype=f16, device=device) if (tp > 1 and rank != 0) else None
        ws_bytes = self.nq * T * (cfg.dh + T) * 2
        self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        self.max_tokens = T

    def forward(self, x, pos, on_step=None):
        """x [T, d] f16 on the device (the residual stream; updated in place on rank 0 / single GPU), pos [T] u32.
        Returns the tensor holding the layer output.  `on_step(name)` is called after each launch (timing hooks)."""
        cfg, T = self.cfg, x.shape[0]
        assert T <= self.max_tokens
        mark = on_step or (lambda name: None)
        h, qkv, att_out, gu = self.h[:T], self.qkv[:T], self.att_out[:T], self.gu[:T]
        self.rms_norm.launch(RmsNormArgs.of(h, x, self.w["w_norm1"], cfg.eps))
        mark("rms_norm_1")
        self.mat_mul.launch(MatMulArgs.of(qkv, 0.0, h, self.w["w_qkv"], 1.0))
        mark("mat_mul_qkv")
        heads = qkv.view(T, self.nq + 2 * self.nkv, cfg.dh)
        self.rope.launch(RopeArgs.of(heads[:, : self.nq + self.nkv], pos, cfg.theta))
        mark("rope")
        q = heads[:, : self.nq].permute(1, 0, 2)
        k = heads[:, self.nq: self.nq + self.nkv].permute(1, 0, 2)
        v = heads[:, self.nq + self.nkv:].permute(1, 0, 2)
        o = att_out.view(T, self.nq, cfg.dh).permute(1, 0, 2)
        self.attention.launch(AttentionArgs.of(q, k, v, o, MASK_CAUSAL), self.ws)
        mark("attention")
        x = self._project_and_reduce(x, att_out, self.w["w_o"], "mat_mul_o", "all_reduce_1", mark)
        self.rms_norm.launch(RmsNormArgs.of(h, x, self.w["w_norm2"], cfg.eps))
        mark("rms_norm_2")
        self.mat_mul.launch(MatMulArgs.of(gu, 0.0, h, self.w["w_gu"], 1.0))
        mark("mat_mul_gate_up")
        self.swiglu.launch(SwigluArgs.of(gu[:, : self.f], gu[:, self.f:]))
        mark("swiglu")
        x = self._project_and_reduce(x, gu[:, : self.f], self.w["w_down"], "mat_mul_down", "all_reduce_2", mark)
        return x

    def _project_and_reduce(self, x, a, w, mm_name, ar_name, mark):
        """Row-parallel projection + all_reduce.  With overlap_chunks > 1 the token dimension is cut into chunks: the
        all_reduce of chunk c runs on a second stream while the tensor cores work on chunk c+1."""
        import torch
        T = x.shape[0]
        first = self.tp == 1 or self.rank == 0
        # rank 0 (and the single-GPU case) folds the residual in: x <- x + a w.  The other ranks never read the
        # residual: their partial goes to scratch, which holds the stream from here on.
        out, beta = (x, 1.0) if first else (self.scratch[:T], 0.0)
        chunks = self.overlap_chunks if (self.tp > 1 and T >= 256 * self.overlap_chunks) else 1
        if self.fused_all_reduce:
            self.mat_mul.launch_all_reduce(self.comm, MatMulArgs.of(out, beta, a, w, 1.0))
            mark(mm_name)
            mark(ar_name)
            return out
        if chunks == 1:
            self.mat_mul.launch(MatMulArgs.of(out, beta, a, w, 1.0))
            mark(mm_name)
            if self.tp > 1:
                self.all_reduce.launch(AllReduceArgs.of(out, out))
                mark(ar_name)
            return out
        main = torch.cuda.current_stream()
        step = (T + chunks - 1) // chunks
        step = (step + 127) // 128 * 128
        for lo in range(0, T, step):
            hi = min(T, lo + step)
            self.mat_mul.launch(MatMulArgs.of(out[lo:hi], beta, a[lo:hi], w, 1.0))
            ready = main.record_event()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.all_reduce.launch(AllReduceArgs.of(out[lo:hi], out[lo:hi]))
        mark(mm_name)
        main.wait_stream(self.comm_stream)
        mark(ar_name)
        return out
