"""The decoder-layer operator chain, as a caller of the per-operator API.

The reference crate ships operators only; the chain below is what a downstream runtime does with
them for one Llama-shaped layer (benchmark config 3) and its tensor-parallel form (config 4):

    rms_norm -> mat_mul(QKV) -> rope(q,k heads) -> attention -> mat_mul(O, beta=1 residual)
             -> [all_reduce] -> rms_norm -> mat_mul(gate|up) -> swiglu -> mat_mul(down, beta=1) -> [all_reduce]

Every step is one `Operator.launch` through the C ABI on torch-owned device buffers.  Tensor
parallelism follows the usual split: QKV and gate|up by columns (whole heads per rank, the GQA group
kept together), O and down by rows, f16 sum all_reduce of the [T, d] partials — see DecoderLayer for
how the partials and the residual meet.
"""
from dataclasses import dataclass

from . import (ALL_REDUCE_AUTO, ATTENTION_MAX_RUNS, ATTENTION_RUN_RECORD_BYTES, MASK_CAUSAL, AllReduce, AllReduceArgs, Attention, AttentionArgs, FusedSoftmax, MatMul,
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


class _Lane:
    """What one stream of the pipelined tail needs for itself: a stream and operator handles whose scratch must not be
    shared between streams (the K-split partials of mat_mul)."""

    def __init__(self, idx, device, own_stream):
        import torch
        self.rms_norm, self.swiglu, self.mat_mul = RmsNorm(idx), Swiglu(idx), MatMul(idx)
        self.stream = torch.cuda.Stream(device) if own_stream else None


class DecoderLayer:
    """One (possibly tensor-parallel) decoder layer on one GPU.  `weights` are this rank's shards on the device.

    Tensor-parallel exchange, in order of preference:
      * direct (default once peer-to-peer staging is attached, messages of 1 MiB or more): the row-parallel projection
        writes its partial straight into the communicator's zero-copy region and ONE kernel adds the partials of all
        ranks onto the residual stream (ops_all_reduce_add_launch) — no copy-in, no residual read in the GEMM;
      * otherwise rank 0 folds the residual into its partial with beta = 1 and an in-place all_reduce follows.
    With `pipeline` > 1 the rows are cut into that many chunks after attention (everything behind attention is row-wise
    independent).  Each chunk runs the rest of the chain on its own stream; the exchanges of all chunks go, in a fixed
    order, through ONE communication stream, so that at any time at most one exchange kernel waits for its peers (two
    that wait at once could starve each other of SMs in opposite orders on different ranks) while the projections of the
    other chunk keep the tensor cores busy.  (Measured on 2 and 8 B200s it is slower than running in order — two
    persistent GEMMs and the exchange kernel contend for the same SMs — so the default is `pipeline` = 1.)
    With `direct_region` (the first half of an attached NVLink multicast buffer, Comm.nvls_attach) the partials are written
    there instead and the reduce-scatter half of the exchange is done inside the switch.
    """

    STEPS = ("rms_norm_1", "mat_mul_qkv", "rope", "attention", "mat_mul_o", "all_reduce_1", "rms_norm_2", "mat_mul_gate_up",
             "swiglu", "mat_mul_down", "all_reduce_2")
    DIRECT_MIN_BYTES = 1 << 20
    PIPELINE_MIN_ROWS = 256  # rows per chunk below which cutting the tail does not pay

    def __init__(self, cfg, weights, max_tokens, device, comm=None, tp=1, rank=0, all_reduce_algo=ALL_REDUCE_AUTO, overlap_chunks=1,
                 fused_all_reduce=False, direct=True, pipeline=1, direct_region=None):
        import torch
        self.overlap_chunks = max(1, int(overlap_chunks))
        self.fused_all_reduce = bool(fused_all_reduce) and tp > 1  # row-parallel GEMM and its all_reduce as one kernel
        self.comm = comm
        self.cfg, self.w, self.device, self.tp, self.rank = cfg, weights, device, tp, rank
        idx = device.index if device.index is not None else 0
        self.rope, self.attention = Rope(idx), Attention(idx)
        self.all_reduce = None
        self.direct_buf = None
        if tp > 1:
            self.all_reduce = AllReduce(comm)
            self.all_reduce.set_algo(all_reduce_algo)
            if direct_region is not None:
                # the zero-copy input region of an attached NVLink multicast buffer (Comm.nvls_attach): the exchange is then
                # reduced inside the switch
                self.direct_buf = direct_region
            else:
                try:
                    self.direct_buf = comm.p2p_direct(torch.float16)
                except Exception:
                    self.direct_buf = None  # no staging attached: NCCL only
        self.direct = bool(direct) and tp > 1 and not self.fused_all_reduce and self.overlap_chunks == 1 and self.direct_buf is not None
        self.pipeline = max(1, int(pipeline)) if self.direct else 1
        self.comm_stream = torch.cuda.Stream(device) if (tp > 1 and (self.overlap_chunks > 1 or self.pipeline > 1)) else None
        self.lanes = [_Lane(idx, device, self.pipeline > 1) for _ in range(self.pipeline)]
        self.rms_norm, self.swiglu, self.mat_mul = self.lanes[0].rms_norm, self.lanes[0].swiglu, self.lanes[0].mat_mul
        self.nq, self.nkv, self.f = cfg.nh // tp, cfg.nkvh // tp, cfg.ffn // tp
        T, f16 = max_tokens, torch.float16
        self.h = torch.empty(T, cfg.d, dtype=f16, device=device)
        self.qkv = torch.empty(T, (self.nq + 2 * self.nkv) * cfg.dh, dtype=f16, device=device)
        self.att_out = torch.empty(T, self.nq * cfg.dh, dtype=f16, device=device)
        self.gu = torch.empty(T, 2 * self.f, dtype=f16, device=device)
        self.scratch = torch.empty(T, cfg.d, dtype=f16, device=device) if (tp > 1 and rank != 0) else None
        # The fused attention kernels need no workspace on a whole layer; a tensor-parallel shard has few heads, and with
        # room for the partial results the kernel cuts the key blocks of every tile pair into runs so that all SMs work
        ws_bytes = 16 if tp == 1 else self.nq * T * ATTENTION_MAX_RUNS * ATTENTION_RUN_RECORD_BYTES
        self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        self.max_tokens = T

    def forward(self, x, pos, on_step=None):
        """x [T, d] f16 on the device (the residual stream; updated in place on rank 0 / single GPU / in direct mode),
        pos [T] u32.  Returns the tensor holding the layer output.  `on_step(name)` is called after each launch (timing
        hooks; with it the tail runs unpipelined so that the hooks see one operator at a time)."""
        import torch
        cfg, T = self.cfg, x.shape[0]
        assert T <= self.max_tokens
        mark = on_step or (lambda name: None)
        h, qkv, att_out = self.h[:T], self.qkv[:T], self.att_out[:T]
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
        if self.pipeline > 1 and on_step is None and T >= self.PIPELINE_MIN_ROWS * self.pipeline and self._use_direct(T // self.pipeline):
            main = torch.cuda.current_stream()
            ready = main.record_event()
            step = (T + self.pipeline - 1) // self.pipeline
            step = (step + 127) // 128 * 128
            spans = [(lo, min(T, lo + step)) for lo in range(0, T, step)]
            for lane in self.lanes[: len(spans)]:
                lane.stream.wait_event(ready)
            # the launches are issued stage by stage, chunk after chunk, so that the exchanges enter the communication
            # stream in the order in which their inputs become ready
            for lane, (lo, hi) in zip(self.lanes, spans):
                with torch.cuda.stream(lane.stream):
                    self._stage_o(lane, x, lo, hi, mark)
            for lane, (lo, hi) in zip(self.lanes, spans):
                with torch.cuda.stream(lane.stream):
                    self._stage_mlp(lane, x[lo:hi], lo, hi, mark)
            for lane in self.lanes[: len(spans)]:
                main.wait_stream(lane.stream)
            return x
        lane = self.lanes[0]
        xr = self._stage_o(lane, x, 0, T, mark)
        return self._stage_mlp(lane, xr, 0, T, mark)

    def _use_direct(self, rows):
        return self.direct and rows * self.cfg.d * 2 >= self.DIRECT_MIN_BYTES

    def _stage_o(self, lane, x, lo, hi, mark):
        """O projection of rows [lo, hi) and its exchange; returns the tensor that holds those rows of the stream."""
        return self._project_and_reduce(lane, x[lo:hi], self.att_out[lo:hi], self.w["w_o"], "mat_mul_o", "all_reduce_1", mark, lo, hi)

    def _stage_mlp(self, lane, xr, lo, hi, mark):
        """rms_norm, gate|up, swiglu, down projection and its exchange for rows [lo, hi) held in `xr`."""
        cfg = self.cfg
        h, gu = self.h[lo:hi], self.gu[lo:hi]
        lane.rms_norm.launch(RmsNormArgs.of(h, xr, self.w["w_norm2"], cfg.eps))
        mark("rms_norm_2")
        lane.mat_mul.launch(MatMulArgs.of(gu, 0.0, h, self.w["w_gu"], 1.0))
        mark("mat_mul_gate_up")
        lane.swiglu.launch(SwigluArgs.of(gu[:, : self.f], gu[:, self.f:]))
        mark("swiglu")
        return self._project_and_reduce(lane, xr, gu[:, : self.f], self.w["w_down"], "mat_mul_down", "all_reduce_2", mark, lo, hi)

    def _project_and_reduce(self, lane, x, a, w, mm_name, ar_name, mark, lo, hi):
        """Row-parallel projection + exchange for the rows held in `x`.  With overlap_chunks > 1 the token dimension is cut
        into chunks: the all_reduce of chunk c runs on a second stream while the tensor cores work on chunk c+1."""
        import torch
        T = x.shape[0]
        if self.tp > 1 and self._use_direct(T):
            part = self.direct_buf[lo * self.cfg.d: hi * self.cfg.d].view(T, self.cfg.d)
            lane.mat_mul.launch(MatMulArgs.of(part, 0.0, a, w, 1.0))
            mark(mm_name)
            if lane.stream is not None and torch.cuda.current_stream() == lane.stream:
                # pipelined: the exchange runs on the communication stream, this chunk's stream waits for it
                ready = lane.stream.record_event()
                self.comm_stream.wait_event(ready)
                with torch.cuda.stream(self.comm_stream):
                    self.all_reduce.launch_add(AllReduceArgs.of(x, part))
                    done = self.comm_stream.record_event()
                lane.stream.wait_event(done)
            else:
                self.all_reduce.launch_add(AllReduceArgs.of(x, part))
            mark(ar_name)
            return x
        first = self.tp == 1 or self.rank == 0
        # rank 0 (and the single-GPU case) folds the residual in: x <- x + a w.  The other ranks never read the
        # residual: their partial goes to scratch, which holds the stream from here on.
        out, beta = (x, 1.0) if first else (self.scratch[lo:hi], 0.0)
        chunks = self.overlap_chunks if (self.tp > 1 and T >= 256 * self.overlap_chunks) else 1
        if self.fused_all_reduce:
            lane.mat_mul.launch_all_reduce(self.comm, MatMulArgs.of(out, beta, a, w, 1.0))
            mark(mm_name)
            mark(ar_name)
            return out
        if chunks == 1:
            lane.mat_mul.launch(MatMulArgs.of(out, beta, a, w, 1.0))
            mark(mm_name)
            if self.tp > 1:
                self.all_reduce.launch(AllReduceArgs.of(out, out))
                mark(ar_name)
            return out
        main = torch.cuda.current_stream()
        step = (T + chunks - 1) // chunks
        step = (step + 127) // 128 * 128
        for c0 in range(0, T, step):
            c1 = min(T, c0 + step)
            lane.mat_mul.launch(MatMulArgs.of(out[c0:c1], beta, a[c0:c1], w, 1.0))
            ready = main.record_event()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.all_reduce.launch(AllReduceArgs.of(out[c0:c1], out[c0:c1]))
        mark(mm_name)
        main.wait_stream(self.comm_stream)
        mark(ar_name)
        return out
