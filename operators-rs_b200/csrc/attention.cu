// attention.cu — o = softmax_mask(q k^T / sqrt(dh)) v with grouped-query heads, and the KV-cached form.
//
// Replaces attention::Operator (operators/src/attention/operator.rs:36-277, checks
// operators/src/attention/args.rs:60-90) and attention_kv_cached::Operator
// (operators/src/attention_kv_cached/operator.rs:76-183, checks attention_kv_cached/args.rs:72-115).
//
// Algorithm 1 (OPS_ATTENTION_FUSED, the default) runs one kernel whenever the layouts allow it (f16, dh 64 or 128,
// 16-byte aligned rows): the split-KV decode kernel of attention_decode.cu for at most 8 query rows per kv head over
// 256 keys or more, else the tensor-core flash attention of attention_fused.cu; it falls back to algorithm 0 otherwise.
// Algorithm 0 (OPS_ATTENTION_CHAIN) is the crate's own composition, step for step, on this library's
// kernels: [copy q to a contiguous buffer unless its (nh, seq) dims merge] -> att = alpha q k^T
// (batched over kv heads, the q rows of one group stacked) -> causal softmax in place -> q = att v ->
// copy to o.  The f16 score matrix lives in the caller's workspace, as in the crate.
#include "common.h"
#include "internal.h"

using namespace ops;

struct ops_attention {
  ops::OpBase base;
  ops_mat_mul *mat_mul;
  int algo;
  int *status_dev;      // written by the fused kernel when a bounded wait runs out
  bool attr_set[3];
  float *decode_scratch;          // split-KV partials of the decode kernel (owned by the handle; one stream at a time)
  unsigned int *decode_tickets;   // arrival counters, left at zero by every launch
};

namespace ops {

struct AttnMeta {
  uint32_t dt;
  usz nh, nkvh, seq, att, dh;
};

static int attn_meta(const ops_attention_args *a, AttnMeta *m) {
  if (a->q_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "q.ndim = %u, 3 expected", a->q_layout.ndim);
  if (a->k_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "k.ndim = %u, 3 expected", a->k_layout.ndim);
  if (a->v_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "v.ndim = %u, 3 expected", a->v_layout.ndim);
  if (a->o_layout.ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "o.ndim = %u, 3 expected", a->o_layout.ndim);
  m->dt = a->q_layout.dt;
  if (a->k_layout.dt != m->dt || a->v_layout.dt != m->dt || a->o_layout.dt != m->dt) return fail(OPS_TYPE_MISMATCH, "q, k, v, o element types differ");
  const usz nh[2] = {a->q_layout.shape[0], a->o_layout.shape[0]};
  const usz nkvh[2] = {a->k_layout.shape[0], a->v_layout.shape[0]};
  const usz seq[2] = {a->q_layout.shape[1], a->o_layout.shape[1]};
  const usz att[2] = {a->k_layout.shape[1], a->v_layout.shape[1]};
  const usz dh[4] = {a->q_layout.shape[2], a->k_layout.shape[2], a->v_layout.shape[2], a->o_layout.shape[2]};
  if (!merge_dims(nh, 2, &m->nh)) return fail(OPS_SHAPE_MISMATCH, "nh of q and o differ");
  if (!merge_dims(nkvh, 2, &m->nkvh)) return fail(OPS_SHAPE_MISMATCH, "nkvh of k and v differ");
  if (!merge_dims(seq, 2, &m->seq)) return fail(OPS_SHAPE_MISMATCH, "seq of q and o differ");
  if (!merge_dims(att, 2, &m->att)) return fail(OPS_SHAPE_MISMATCH, "att of k and v differ");
  if (!merge_dims(dh, 4, &m->dh)) return fail(OPS_SHAPE_MISMATCH, "dh of q, k, v, o differ");
  return OPS_OK;
}

// WorkspaceCollector::cauculate (operators/src/common/workspace.rs:78-89)
static usz greedy_workspace(const usz *parts, int n, usz max_ws) {
  usz ans = 0;
  for (int i = 0; i < n; ++i) {
    if (ans + parts[i] <= max_ws) ans += parts[i];
    else return ans;
  }
  return ans;
}

static ops_layout make_layout(uint32_t dt, const usz *shape, const isz *strides) { return ops_layout{dt, 3, shape, strides}; }

static int attention_chain(const ops_attention *op, const ops_attention_args *a, const AttnMeta &m, void *ws, usz ws_len, cudaStream_t s) {
  const usz ele = dt_size(m.dt);
  const isz *sq = a->q_layout.strides, *sk = a->k_layout.strides;
  const usz group = m.nh / m.nkvh;
  const bool merged = sq[0] == (isz)m.seq * sq[1];  // (nh, seq) fold into one dim (merge_be(0, 2))
  const usz q_size = merged ? 0 : m.nh * m.seq * m.dh * ele;
  const usz att_size = m.nh * m.seq * m.att * ele;
  if (ws_len < q_size + att_size || (!ws && q_size + att_size)) return need_workspace(q_size + att_size);
  char *q_buf = (char *)ws, *att_buf = (char *)ws + q_size;

  const usz shp_q[3] = {m.nh, m.seq, m.dh};
  const isz cont_q[3] = {(isz)(m.seq * m.dh * ele), (isz)(m.dh * ele), (isz)ele};
  const usz shp_x[3] = {m.nkvh, group * m.seq, m.dh};
  isz str_x[3];
  isz str_qv[3];  // strides of the [nh, seq, dh] view of whatever buffer holds q from here on
  void *q_base;
  if (!merged) {
    ops_rearrange_args r{make_layout(m.dt, shp_q, cont_q), q_buf, a->q_layout, a->q_base};
    OPS_TRY(rearrange_enqueue(op->base, &r, s));
    q_base = q_buf;
    str_x[0] = (isz)(group * m.seq * m.dh * ele);
    str_x[1] = (isz)(m.dh * ele);
    str_x[2] = (isz)ele;
    for (int i = 0; i < 3; ++i) str_qv[i] = cont_q[i];
  } else {
    q_base = a->q_base;
    str_x[0] = (isz)(group * m.seq) * sq[1];
    str_x[1] = sq[1];
    str_x[2] = sq[2];
    for (int i = 0; i < 3; ++i) str_qv[i] = sq[i];
  }
  const usz shp_kt[3] = {m.nkvh, m.dh, m.att};
  const isz str_kt[3] = {sk[0], sk[2], sk[1]};
  const usz shp_am[3] = {m.nkvh, group * m.seq, m.att};
  const isz str_am[3] = {(isz)(group * m.seq * m.att * ele), (isz)(m.att * ele), (isz)ele};
  const usz shp_as[3] = {m.nh, m.seq, m.att};
  const isz str_as[3] = {(isz)(m.seq * m.att * ele), (isz)(m.att * ele), (isz)ele};

  // att = q . k^T / sqrt(dh)
  ops_mat_mul_args mm1{make_layout(m.dt, shp_am, str_am), att_buf, 0.f, make_layout(m.dt, shp_x, str_x), q_base,
                       make_layout(m.dt, shp_kt, str_kt), a->k_base, 1.f / sqrtf((float)m.dh)};
  OPS_TRY(mat_mul_enqueue(op->mat_mul, &mm1, s));
  // att = softmax(att)
  ops_fused_softmax_args sm{a->mask, make_layout(m.dt, shp_as, str_as), att_buf};
  OPS_TRY(fused_softmax_enqueue(op->base, &sm, s));
  // q = att . v
  ops_mat_mul_args mm2{make_layout(m.dt, shp_x, str_x), q_base, 0.f, make_layout(m.dt, shp_am, str_am), att_buf, a->v_layout, a->v_base, 1.f};
  OPS_TRY(mat_mul_enqueue(op->mat_mul, &mm2, s));
  // o = rearrange(q)
  if (q_base != a->o_base) {
    ops_rearrange_args r{a->o_layout, a->o_base, make_layout(m.dt, shp_q, str_qv), q_base};
    OPS_TRY(rearrange_enqueue(op->base, &r, s));
  }
  return OPS_OK;
}

int attention_enqueue(const ops_attention *op, const ops_attention_args *a, void *ws, usz ws_len, cudaStream_t s) {
  AttnMeta m;
  OPS_TRY(attn_meta(a, &m));
  const isz *sq = a->q_layout.strides, *sk = a->k_layout.strides;
  if (dyn(m.nh) || dyn(m.seq) || dyn(m.dh) || dyn(m.nkvh) || dyn(m.att) || dyn(sq[0]) || dyn(sq[1]) || dyn(sq[2]) || dyn(sk[0]) ||
      dyn(sk[1]) || dyn(sk[2]))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "attention: every shape and the q, k strides must be static at launch");
  if (m.dt != OPS_DT_F16 && m.dt != OPS_DT_BF16 && m.dt != OPS_DT_F32) return fail(OPS_TYPE_NOT_SUPPORT, "attention: f16, bf16 or f32 expected");
  if (m.nkvh == 0 || m.nh % m.nkvh != 0) return fail(OPS_SHAPE_MISMATCH, "attention: nh must be a multiple of nkvh");
  if (a->mask == OPS_MASK_CAUSAL && m.att < m.seq) return fail(OPS_SHAPE_NOT_SUPPORT, "attention: causal mask needs att >= seq");
  if (m.nh == 0 || m.seq == 0 || m.dh == 0 || m.att == 0) return OPS_OK;
  const bool fused = op->algo == OPS_ATTENTION_FUSED || op->algo == OPS_ATTENTION_FUSED_ONE_TILE;
  if (fused && a->q_base && a->k_base && a->v_base && a->o_base && op->decode_scratch &&
      attention_decode_supported(a, m.nh, m.nkvh, m.seq, m.att, m.dh))
    return attention_decode_enqueue(op->base, a, m.nh, m.nkvh, m.seq, m.att, m.dh, op->decode_scratch, op->decode_tickets, s);
  if (fused && a->q_base && a->k_base && a->v_base && a->o_base && attention_fused_supported(a, m.nh, m.nkvh, m.seq, m.att, m.dh)) {
    ops_attention *mop = const_cast<ops_attention *>(op);
    return attention_fused_enqueue(op->base, a, m.nh, m.nkvh, m.seq, m.att, m.dh, op->status_dev, mop->attr_set, ws, ws_len, s,
                                   op->algo == OPS_ATTENTION_FUSED_ONE_TILE);
  }
  return attention_chain(op, a, m, ws, ws_len, s);
}

}  // namespace ops

OPS_API int ops_attention_create(int device, ops_attention **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  ops_attention *h = new ops_attention();
  h->mat_mul = nullptr;
  h->algo = OPS_ATTENTION_FUSED;
  h->status_dev = nullptr;
  h->attr_set[0] = h->attr_set[1] = h->attr_set[2] = false;
  h->decode_scratch = nullptr;
  h->decode_tickets = nullptr;
  int rc = init_base(&h->base, device);
  if (rc == OPS_OK) rc = ops_mat_mul_create(device, &h->mat_mul);
  if (rc == OPS_OK) {
    cudaSetDevice(device);
    if (cudaMalloc(&h->status_dev, sizeof(int)) != cudaSuccess || cudaMemset(h->status_dev, 0, sizeof(int)) != cudaSuccess)
      rc = fail(OPS_EXECUTION_FAILED, "attention: cannot allocate the status word");
    else if (cudaMalloc(&h->decode_scratch, attention_decode_scratch_bytes()) != cudaSuccess ||
             cudaMalloc(&h->decode_tickets, attention_decode_ticket_bytes()) != cudaSuccess ||
             cudaMemset(h->decode_tickets, 0, attention_decode_ticket_bytes()) != cudaSuccess)
      rc = fail(OPS_EXECUTION_FAILED, "attention: cannot allocate the decode scratch");
  }
  if (rc != OPS_OK) {
    if (h->mat_mul) ops_mat_mul_destroy(h->mat_mul);
    if (h->status_dev) cudaFree(h->status_dev);
    if (h->decode_scratch) cudaFree(h->decode_scratch);
    if (h->decode_tickets) cudaFree(h->decode_tickets);
    delete h;
    return rc;
  }
  *out = h;
  return OPS_OK;
}

OPS_API void ops_attention_destroy(ops_attention *op) {
  if (!op) return;
  if (op->mat_mul) ops_mat_mul_destroy(op->mat_mul);
  if (op->status_dev) cudaFree(op->status_dev);
  if (op->decode_scratch) cudaFree(op->decode_scratch);
  if (op->decode_tickets) cudaFree(op->decode_tickets);
  delete op;
}

OPS_API int ops_attention_set_algo(ops_attention *op, int algo) {
  if (algo != OPS_ATTENTION_CHAIN && algo != OPS_ATTENTION_FUSED && algo != OPS_ATTENTION_FUSED_ONE_TILE) return fail(OPS_ARGS_NOT_SUPPORT, "attention: unknown algorithm %d", algo);
  op->algo = algo;
  return OPS_OK;
}

// 0, or which bounded wait ran out: 11/12 producer, 21-26 issuer, 31-33 softmax of the fused kernel, 1-4 of the
// tensor-core mat_mul used by the chain.  Synchronises the device.
OPS_API int ops_attention_status(const ops_attention *op) {
  int v = -1;
  cudaSetDevice(op->base.device);
  if (cudaMemcpy(&v, op->status_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v == 0) v = ops_mat_mul_status(op->mat_mul);
  return v;
}

// Counterpart of ops_mat_mul_status_reset for the attention kernels: status word, the split-KV arrival counters and the
// handle's own mat_mul.
OPS_API int ops_attention_status_reset(ops_attention *op) {
  if (!op) return fail(OPS_ARGS_NOT_SUPPORT, "null handle");
  cudaSetDevice(op->base.device);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(op->status_dev, 0, sizeof(int));
  if (e == cudaSuccess && op->decode_tickets) e = cudaMemset(op->decode_tickets, 0, attention_decode_ticket_bytes());
  if (e != cudaSuccess) return fail(OPS_EXECUTION_FAILED, "attention status reset: %s", cudaGetErrorString(e));
  return ops_mat_mul_status_reset(op->mat_mul);
}

// attention::Operator::scheme (operators/src/attention/operator.rs:45-134): with static nh, seq, att,
// dh the need is q_size + att_size (sub-operators need nothing), cut greedily to max_ws.
OPS_API int ops_attention_scheme(ops_attention *op, const ops_attention_args *args, size_t max_ws, size_t *ws_out) {
  (void)op;
  AttnMeta m;
  OPS_TRY(attn_meta(args, &m));
  if (ws_out) {
    *ws_out = 0;
    if (!dyn(m.nh) && !dyn(m.seq) && !dyn(m.att) && !dyn(m.dh)) {
      const usz ele = dt_size(m.dt);
      const usz parts[3] = {m.nh * m.seq * m.dh * ele, m.nh * m.seq * m.att * ele, 0};
      *ws_out = greedy_workspace(parts, 3, max_ws);
    }
  }
  return OPS_OK;
}

OPS_API int ops_attention_launch(const ops_attention *op, const ops_attention_args *args, void *ws, size_t ws_len, void *stream) {
  return attention_enqueue(op, args, ws, ws_len, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------
// attention_kv_cached
// ------------------------------------------------------------------------------------------------
struct ops_attention_kv_cached {
  ops_attention *attention;
};

namespace ops {

struct CachedMeta {
  uint32_t dt;
  usz nh, nkvh, dh, seq;
};

static int cached_meta(const ops_attention_kv_cached_args *a, CachedMeta *m) {
  const ops_layout *ls[6] = {&a->q_layout, &a->k_layout, &a->v_layout, &a->o_layout, &a->k_cache_layout, &a->v_cache_layout};
  static const char *names[6] = {"q", "k", "v", "o", "k_cache", "v_cache"};
  for (int i = 0; i < 6; ++i)
    if (ls[i]->ndim != 3) return fail(OPS_RANK_NOT_SUPPORT, "%s.ndim = %u, 3 expected", names[i], ls[i]->ndim);
  m->dt = a->q_layout.dt;
  for (int i = 1; i < 6; ++i)
    if (ls[i]->dt != m->dt) return fail(OPS_TYPE_MISMATCH, "element types of q, k, v, o and the caches differ");
  const usz nh[2] = {a->q_layout.shape[0], a->o_layout.shape[0]};
  const usz nkvh[4] = {a->k_layout.shape[0], a->v_layout.shape[0], a->k_cache_layout.shape[0], a->v_cache_layout.shape[0]};
  const usz dh[6] = {a->q_layout.shape[2], a->k_layout.shape[2], a->v_layout.shape[2], a->o_layout.shape[2], a->k_cache_layout.shape[2], a->v_cache_layout.shape[2]};
  const usz seq[4] = {a->q_layout.shape[1], a->k_layout.shape[1], a->v_layout.shape[1], a->o_layout.shape[1]};
  if (!merge_dims(nh, 2, &m->nh)) return fail(OPS_SHAPE_MISMATCH, "nh of q and o differ");
  if (!merge_dims(nkvh, 4, &m->nkvh)) return fail(OPS_SHAPE_MISMATCH, "nkvh of k, v and the caches differ");
  if (!merge_dims(dh, 6, &m->dh)) return fail(OPS_SHAPE_MISMATCH, "dh of q, k, v, o and the caches differ");
  if (!merge_dims(seq, 4, &m->seq)) return fail(OPS_SHAPE_MISMATCH, "seq of q, k, v, o differ");
  return OPS_OK;
}

}  // namespace ops

OPS_API int ops_attention_kv_cached_create(int device, ops_attention_kv_cached **out) {
  if (!out) return fail(OPS_ARGS_NOT_SUPPORT, "null out pointer");
  ops_attention_kv_cached *h = new ops_attention_kv_cached();
  int rc = ops_attention_create(device, &h->attention);
  if (rc != OPS_OK) {
    delete h;
    return rc;
  }
  *out = h;
  return OPS_OK;
}

OPS_API void ops_attention_kv_cached_destroy(ops_attention_kv_cached *op) {
  if (!op) return;
  ops_attention_destroy(op->attention);
  delete op;
}

OPS_API int ops_attention_kv_cached_set_algo(ops_attention_kv_cached *op, int algo) { return ops_attention_set_algo(op->attention, algo); }

// attention_kv_cached::Operator::scheme (operators/src/attention_kv_cached/operator.rs:36-74): the
// attention need at att = pos + seq when both are static.
OPS_API int ops_attention_kv_cached_scheme(ops_attention_kv_cached *op, const ops_attention_kv_cached_args *a, size_t max_ws, size_t *ws_out) {
  (void)op;
  CachedMeta m;
  OPS_TRY(cached_meta(a, &m));
  if (ws_out) {
    *ws_out = 0;
    if (!dyn(m.nh) && !dyn(m.seq) && !dyn(m.dh) && !dyn(a->pos)) {
      const usz ele = dt_size(m.dt), att = a->pos + m.seq;
      const usz parts[3] = {m.nh * m.seq * m.dh * ele, m.nh * m.seq * att * ele, 0};
      *ws_out = greedy_workspace(parts, 3, max_ws);
    }
  }
  return OPS_OK;
}

OPS_API int ops_attention_kv_cached_launch(const ops_attention_kv_cached *op, const ops_attention_kv_cached_args *a, void *ws, size_t ws_len, void *stream) {
  CachedMeta m;
  OPS_TRY(cached_meta(a, &m));
  const usz buf_k = a->k_cache_layout.shape[1], buf_v = a->v_cache_layout.shape[1];
  // as in the crate, the v cache is addressed with the K cache's strides (operator.rs:110-115, :156)
  const isz *skc = a->k_cache_layout.strides;
  if (dyn(a->pos) || dyn(m.seq) || dyn(buf_k) || dyn(buf_v) || dyn(m.nkvh) || dyn(m.dh) || dyn(skc[0]) || dyn(skc[1]) || dyn(skc[2]))
    return fail(OPS_DYNAMIC_NOT_SUPPORT, "attention_kv_cached: pos, shapes and cache strides must be static at launch");
  const usz att = a->pos + m.seq;
  if (buf_k < att || buf_v < att) return fail(OPS_SHAPE_MISMATCH, "Out of cache buffer");
  cudaStream_t s = (cudaStream_t)stream;
  const ops_attention *at = op->attention;
  const usz shp_cat[3] = {m.nkvh, m.seq, m.dh};
  const isz off = (isz)a->pos * skc[1];
  if (m.seq && m.nkvh && m.dh) {
    if (!a->k_cache_base || !a->v_cache_base) return fail(OPS_DYNAMIC_NOT_SUPPORT, "attention_kv_cached: null cache pointer at launch");
    ops_rearrange_args rk{ops_layout{m.dt, 3, shp_cat, skc}, (char *)a->k_cache_base + off, a->k_layout, a->k_base};
    OPS_TRY(rearrange_enqueue(at->base, &rk, s));
    ops_rearrange_args rv{ops_layout{m.dt, 3, shp_cat, skc}, (char *)a->v_cache_base + off, a->v_layout, a->v_base};
    OPS_TRY(rearrange_enqueue(at->base, &rv, s));
  }
  const usz shp_kv[3] = {m.nkvh, att, m.dh};
  ops_attention_args aa{a->q_layout, a->q_base, ops_layout{m.dt, 3, shp_kv, skc}, a->k_cache_base, ops_layout{m.dt, 3, shp_kv, skc},
                        a->v_cache_base, a->o_layout, a->o_base, a->mask};
  return attention_enqueue(at, &aa, ws, ws_len, s);
}
