/*
 * ops_b200.h — flat C ABI of the B200 (sm_100a) operator library.
 *
 * Every entry point mirrors one item of the operators-rs crate's per-operator interface
 * (`trait Operator { new; scheme; launch }`, operators/src/lib.rs:105-144) so that a Rust
 * `impl Operator` can bind it one to one:
 *
 *     Operator::new(node)                   -> ops_<op>_create(device|topo, &handle)
 *     Operator::scheme(args, max_workspace) -> ops_<op>_scheme(handle, &args, max_ws, &ws_out)
 *     Operator::launch(args, workspace, qa) -> ops_<op>_launch(handle, &args, ws, ws_len, stream)
 *     Drop                                  -> ops_<op>_destroy(handle)
 *
 * Conventions
 *   - All tensor base pointers are DEVICE pointers; `stream` is a `cudaStream_t` passed as `void*`.
 *     `launch` only enqueues on that stream (same contract as the crate's GPU backends).
 *   - Layouts carry BYTE strides (operators/src/common/tensor.rs:10-47).
 *   - "Dynamic" values (operators/src/common/maybe_dyn.rs:6-37): shape == SIZE_MAX,
 *     stride == PTRDIFF_MAX, float == +inf, pointer == NULL.  `scheme` accepts them,
 *     `launch` answers OPS_DYNAMIC_NOT_SUPPORT.
 *   - Return value: 0 on success, else the error kind below; a human readable message for the
 *     calling thread is available from ops_last_error().  Nothing throws, nothing aborts.
 *   - Workspace: `scheme` reports the bytes `launch` wants (never more than `max_ws`, 0 if unknown,
 *     operators/src/lib.rs:116-131).  `launch` with a shorter workspace answers
 *     OPS_WORKSPACE_TOO_SMALL and ops_last_workspace_need() tells the size; the caller's allocator
 *     (the crate's `Workspace::new` fallback, operators/src/common/workspace.rs:12-21) provides it
 *     and calls again.  The library itself never allocates device memory in `launch`.
 *   - There is no CPU path: without a CUDA device `create` fails with OPS_EXECUTION_FAILED.
 */
#ifndef OPS_B200_H
#define OPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error kinds: SchemeErrorKind order of operators/src/common/error.rs:2-12, then
 *      LaunchErrorKind::ExecutionFailed (:21-25) ---- */
enum {
  OPS_OK = 0,
  OPS_TYPE_NOT_SUPPORT = 1,
  OPS_TYPE_MISMATCH = 2,
  OPS_RANK_NOT_SUPPORT = 3,
  OPS_RANK_MISMATCH = 4,
  OPS_SHAPE_NOT_SUPPORT = 5,
  OPS_SHAPE_MISMATCH = 6,
  OPS_STRIDES_NOT_SUPPORT = 7,
  OPS_ARGS_NOT_SUPPORT = 8,
  OPS_DYNAMIC_NOT_SUPPORT = 9,
  OPS_EXECUTION_FAILED = 100,
  OPS_WORKSPACE_TOO_SMALL = 101 /* not an error of the crate: the shim allocates and retries */
};

/* ---- element types (the subset of digit-layout's types the path uses) ---- */
enum {
  OPS_DT_F16 = 1,
  OPS_DT_BF16 = 2,
  OPS_DT_F32 = 3,
  OPS_DT_F64 = 4,
  OPS_DT_U8 = 5,
  OPS_DT_U16 = 6,
  OPS_DT_U32 = 7,
  OPS_DT_U64 = 8,
  OPS_DT_I8 = 9,
  OPS_DT_I16 = 10,
  OPS_DT_I32 = 11,
  OPS_DT_I64 = 12,
  OPS_DT_KVPAIR = 13 /* KVPair::LAYOUT = u32 x 2, operators/src/random_sample/kv_pair.rs:8-17 */
};

#define OPS_DYN_SIZE ((size_t)-1)          /* usize::MAX */
#define OPS_DYN_STRIDE ((ptrdiff_t)(((size_t)-1) >> 1)) /* isize::MAX */

/* TensorLayout (operators/src/common/tensor.rs:10-98): dtype, rank, shape, byte strides. */
typedef struct {
  uint32_t dt;
  uint32_t ndim;
  const size_t *shape;
  const ptrdiff_t *strides;
} ops_layout;

/* AttnMask (operators/src/fuesd_softmax/args.rs:11-16) */
enum { OPS_MASK_NONE = 0, OPS_MASK_CAUSAL = 1 };
/* ReduceOp (operators/src/all_reduce/mod.rs:14-22) */
enum { OPS_REDUCE_SUM = 0, OPS_REDUCE_PROD = 1, OPS_REDUCE_MIN = 2, OPS_REDUCE_MAX = 3, OPS_REDUCE_MEAN = 4 };

const char *ops_last_error(void);          /* message of the calling thread's last failure */
size_t ops_last_workspace_need(void);      /* bytes wanted by the calling thread's last OPS_WORKSPACE_TOO_SMALL */
size_t ops_dtype_nbytes(uint32_t dt);      /* digit_layout::DigitLayout::nbytes */
int ops_device_count(void);                /* 0 when there is no usable CUDA device */
const char *ops_build_info(void);          /* "sm_100a ..." */

/* ---------------------------------------------------------------------------------------------
 * rms_norm — rms_norm::Args (operators/src/rms_norm/args.rs:7-15); replaces
 * rms_norm::common_cpu::Operator (operators/src/rms_norm/common_cpu/mod.rs:10-93).
 * y[i,j] = x[i,j] * w[j] / sqrt(mean_j(x[i,:]^2) + epsilon); y,x f16, bf16 or f32, w of the same type or f32.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_rms_norm ops_rms_norm;
typedef struct {
  ops_layout y_layout; void *y_base;
  ops_layout x_layout; const void *x_base;
  ops_layout w_layout; const void *w_base;
  float epsilon;
} ops_rms_norm_args;
int ops_rms_norm_create(int device, ops_rms_norm **out);
int ops_rms_norm_scheme(ops_rms_norm *op, const ops_rms_norm_args *args, size_t max_ws, size_t *ws_out);
int ops_rms_norm_launch(const ops_rms_norm *op, const ops_rms_norm_args *args, void *ws, size_t ws_len, void *stream);
void ops_rms_norm_destroy(ops_rms_norm *op);
/* Extension with no counterpart in the crate, which chains add (operators/src/add/common_cpu/mod.rs:29-75) and rms_norm as
 * two operators: x <- x + r in place (rounded to the element type as add rounds), then y <- rms_norm(x), in one pass over
 * every row.  f16 or bf16 rows with unit inner stride, 16-byte aligned, d a multiple of 8 up to 32768; other layouts are
 * answered with OPS_ARGS_NOT_SUPPORT (chain ops_add_launch and ops_rms_norm_launch then). */
typedef struct {
  ops_rms_norm_args norm;               /* y, x (read and written), w, epsilon */
  ops_layout r_layout; const void *r_base; /* what is added to x first: same shape and type as x */
} ops_rms_norm_add_args;
int ops_rms_norm_add_launch(const ops_rms_norm *op, const ops_rms_norm_add_args *args, void *stream);

/* ---------------------------------------------------------------------------------------------
 * rope — rope::Args (operators/src/rope/args.rs:8-18); replaces rope::common_cpu::Operator
 * (operators/src/rope/common_cpu/mod.rs:10-130).  In place on t [nt, nh, dh], adjacent pairs
 * (2k, 2k+1), angle = pos / theta^(k/(dh/2)).  sin/cos layouts are validated and otherwise unused,
 * exactly as on the crate's CPU path.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_rope ops_rope;
typedef struct {
  ops_layout t_layout; void *t_base;
  ops_layout p_layout; const void *p_base;
  ops_layout sin_layout; const void *sin_base;
  ops_layout cos_layout; const void *cos_base;
  float theta;
} ops_rope_args;
int ops_rope_create(int device, ops_rope **out);
int ops_rope_scheme(ops_rope *op, const ops_rope_args *args, size_t max_ws, size_t *ws_out);
int ops_rope_launch(const ops_rope *op, const ops_rope_args *args, void *ws, size_t ws_len, void *stream);
void ops_rope_destroy(ops_rope *op);
/* Rope::build_pos (operators/src/rope/mod.rs:17-21, fill_pos :44-58): writes, for every (pos,len)
 * sequence in order, pos..pos+len into a HOST buffer of `nt` u32 or u64; the caller uploads it. */
int ops_rope_build_pos(uint32_t dt, size_t nt, const size_t *seq_pos, const size_t *seq_len, size_t nseq, void *host_out);

/* ---------------------------------------------------------------------------------------------
 * fused_softmax — fuesd_softmax::Args (operators/src/fuesd_softmax/args.rs:5-16); replaces
 * fuesd_softmax::common_cpu::Operator (operators/src/fuesd_softmax/common_cpu/mod.rs:9-82).
 * In place over the last dim of att [nh, seq, att]; causal row k keeps att - seq + k + 1 entries.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_fused_softmax ops_fused_softmax;
typedef struct {
  uint8_t att_mask;
  ops_layout att_layout; void *att_base;
} ops_fused_softmax_args;
int ops_fused_softmax_create(int device, ops_fused_softmax **out);
int ops_fused_softmax_scheme(ops_fused_softmax *op, const ops_fused_softmax_args *args, size_t max_ws, size_t *ws_out);
int ops_fused_softmax_launch(const ops_fused_softmax *op, const ops_fused_softmax_args *args, void *ws, size_t ws_len, void *stream);
void ops_fused_softmax_destroy(ops_fused_softmax *op);

/* ---------------------------------------------------------------------------------------------
 * swiglu — swiglu::Args (operators/src/swiglu/args.rs:7-12); replaces
 * swiglu::common_cpu::Operator (operators/src/swiglu/common_cpu/mod.rs:9-81).
 * gate <- gate * sigmoid(gate) * up, in place on gate.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_swiglu ops_swiglu;
typedef struct {
  ops_layout gate_layout; void *gate_base;
  ops_layout up_layout; const void *up_base;
} ops_swiglu_args;
int ops_swiglu_create(int device, ops_swiglu **out);
int ops_swiglu_scheme(ops_swiglu *op, const ops_swiglu_args *args, size_t max_ws, size_t *ws_out);
int ops_swiglu_launch(const ops_swiglu *op, const ops_swiglu_args *args, void *ws, size_t ws_len, void *stream);
void ops_swiglu_destroy(ops_swiglu *op);

/* ---------------------------------------------------------------------------------------------
 * rearrange — rearrange::Args (operators/src/rearrange/args.rs:11-17); replaces
 * rearrange::common_cpu::Operator (operators/src/rearrange/common_cpu/mod.rs:8-59).
 * Byte-exact strided copy of any rank and dtype; src stride 0 broadcasts.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_rearrange ops_rearrange;
typedef struct {
  ops_layout dst_layout; void *dst_base;
  ops_layout src_layout; const void *src_base;
} ops_rearrange_args;
int ops_rearrange_create(int device, ops_rearrange **out);
int ops_rearrange_scheme(ops_rearrange *op, const ops_rearrange_args *args, size_t max_ws, size_t *ws_out);
int ops_rearrange_launch(const ops_rearrange *op, const ops_rearrange_args *args, void *ws, size_t ws_len, void *stream);
void ops_rearrange_destroy(ops_rearrange *op);
/* rearrange::Scheme::new (operators/src/rearrange/args.rs:34-153) as host arithmetic: writes
 * [unit, idx_strides(count first)…, 1, dst_strides…, src_strides…] (2 + 3*ndim words) to `out`
 * (capacity `cap` words) and the merged rank to *ndim_out.  No device needed. */
int ops_rearrange_plan(const ops_rearrange_args *args, ptrdiff_t *out, size_t cap, size_t *ndim_out);

/* ---------------------------------------------------------------------------------------------
 * mat_mul — mat_mul::Args (operators/src/mat_mul/args.rs:11-20); replaces
 * mat_mul::common_cpu::Operator (operators/src/mat_mul/common_cpu/mod.rs:9-107).
 * C <- beta*C + alpha*A*B, rank 2 or 3 (one batch dim, batch 1 broadcasts), every matrix with a
 * unit stride in one of its two dims.  f16 and bf16 run on tcgen05 tensor cores with f32 accumulation.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_mat_mul ops_mat_mul;
typedef struct {
  ops_layout c_layout; void *c_base;
  float beta;
  ops_layout a_layout; const void *a_base;
  ops_layout b_layout; const void *b_base;
  float alpha;
} ops_mat_mul_args;
int ops_mat_mul_create(int device, ops_mat_mul **out);
int ops_mat_mul_scheme(ops_mat_mul *op, const ops_mat_mul_args *args, size_t max_ws, size_t *ws_out);
int ops_mat_mul_launch(const ops_mat_mul *op, const ops_mat_mul_args *args, void *ws, size_t ws_len, void *stream);
void ops_mat_mul_destroy(ops_mat_mul *op);
/* 0, or which bounded wait inside the tensor-core kernel ran out (1 producer, 2/3 issuer, 4 epilogue).
 * Synchronises the device: for tests and post-mortems.  No counterpart in the crate. */
int ops_mat_mul_status(const ops_mat_mul *op);
/* The first failure sticks, and the output of a launch that set the status is undefined.  _status_reset clears the word
 * and the handle's internal arrival counters (synchronises the device).  No counterpart in the crate. */
int ops_mat_mul_status_reset(ops_mat_mul *op);

/* ---------------------------------------------------------------------------------------------
 * attention — attention::Args (operators/src/attention/args.rs:10-24); replaces
 * attention::Operator<Cpu, …> (operators/src/attention/operator.rs:9-277).
 * o = softmax_mask(q k^T / sqrt(dh)) v with grouped-query heads; q [nh,seq,dh], k,v [nkvh,att,dh].
 * As in the crate, q may be overwritten when its (nh, seq) dims are mergeable.
 * `algo`: 0 = the crate's own chain (rearrange, mat_mul, fused_softmax, mat_mul, rearrange) with
 * the score matrix in workspace, every intermediate rounded to f16 where the crate rounds it;
 * 1 = one fused flash-attention kernel (no score matrix, no workspace, q left untouched); for dh = 128 a CTA owns two
 *     128-row q tiles whose softmax and tensor-core work interleave; 2 = the same with one q tile per CTA (the kernel
 *     dh = 64 always takes), kept selectable for comparison.
 * The fused kernel uses the workspace for one thing only: with few heads (heads x ceil(seq / 256) below ~0.9 x the SM
 * count, e.g. a tensor-parallel shard) and a 16-byte aligned workspace of at least
 * nh * seq * OPS_ATTENTION_MAX_RUNS * OPS_ATTENTION_RUN_RECORD_BYTES bytes, the key blocks of every tile pair are cut into
 * up to OPS_ATTENTION_MAX_RUNS runs computed by different CTAs and merged by a second kernel.  Without it (or with a
 * smaller one) every CTA walks its whole key range; the result differs only in the last bit of the 16-bit output.
 * ------------------------------------------------------------------------------------------- */
#define OPS_ATTENTION_MAX_RUNS 4
#define OPS_ATTENTION_RUN_RECORD_BYTES 528 /* 128 f32 of unnormalised output + reference point + row sum, 16-byte aligned */
typedef struct ops_attention ops_attention;
typedef struct {
  ops_layout q_layout; void *q_base;
  ops_layout k_layout; const void *k_base;
  ops_layout v_layout; const void *v_base;
  ops_layout o_layout; void *o_base;
  uint8_t mask;
} ops_attention_args;
enum { OPS_ATTENTION_CHAIN = 0, OPS_ATTENTION_FUSED = 1, OPS_ATTENTION_FUSED_ONE_TILE = 2 };
int ops_attention_create(int device, ops_attention **out);
int ops_attention_set_algo(ops_attention *op, int algo); /* default OPS_ATTENTION_FUSED (falls back to the chain when a layout rules it out) */
int ops_attention_status(const ops_attention *op);      /* 0, or the code of a bounded wait that ran out; synchronises; no counterpart in the crate */
int ops_attention_status_reset(ops_attention *op);      /* clears it (and the handle's arrival counters); outputs of the failed launch are undefined */
int ops_attention_scheme(ops_attention *op, const ops_attention_args *args, size_t max_ws, size_t *ws_out);
int ops_attention_launch(const ops_attention *op, const ops_attention_args *args, void *ws, size_t ws_len, void *stream);
void ops_attention_destroy(ops_attention *op);

/* ---------------------------------------------------------------------------------------------
 * attention_kv_cached — attention_kv_cached::Args (operators/src/attention_kv_cached/args.rs:8-30);
 * replaces attention_kv_cached::Operator (operators/src/attention_kv_cached/operator.rs:76-183).
 * Copies k,v into the caches at [pos, pos+seq) and attends over cache rows [0, pos+seq).
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_attention_kv_cached ops_attention_kv_cached;
typedef struct {
  ops_layout q_layout; void *q_base;
  ops_layout k_layout; const void *k_base;
  ops_layout v_layout; const void *v_base;
  ops_layout o_layout; void *o_base;
  ops_layout k_cache_layout; void *k_cache_base;
  ops_layout v_cache_layout; void *v_cache_base;
  uint8_t mask;
  size_t pos;
} ops_attention_kv_cached_args;
int ops_attention_kv_cached_create(int device, ops_attention_kv_cached **out);
int ops_attention_kv_cached_set_algo(ops_attention_kv_cached *op, int algo);
int ops_attention_kv_cached_scheme(ops_attention_kv_cached *op, const ops_attention_kv_cached_args *args, size_t max_ws, size_t *ws_out);
int ops_attention_kv_cached_launch(const ops_attention_kv_cached *op, const ops_attention_kv_cached_args *args, void *ws, size_t ws_len, void *stream);
void ops_attention_kv_cached_destroy(ops_attention_kv_cached *op);

/* ---------------------------------------------------------------------------------------------
 * random_sample — random_sample::Args, SampleArgs (operators/src/random_sample/args.rs:9-84);
 * replaces random_sample::common_cpu::Operator (operators/src/random_sample/common_cpu/mod.rs:11-144).
 * One row of logits (f16, bf16 or f32, contiguous) -> one KVPair {u32 idx, u32 val-bits}.
 * argmax when temperature == 0 or top_k == 1 (last index among equal maxima, val = the logit);
 * otherwise seeded sampling where `seed` is the caller's uniform draw in [0,1) and val = the
 * cumulative mass at the chosen entry converted to the logit type.
 * `indices` is accepted for signature parity and never read (as on the crate's CPU path).
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_random_sample ops_random_sample;
typedef struct {
  float temperature;
  float top_p;
  size_t top_k;
} ops_sample_args;
typedef struct {
  ops_layout kv_pair; void *kv_pair_base;
  ops_layout logits; const void *logits_base;
  ops_layout indices; const void *indices_base;
  ops_sample_args config;
  float seed;
} ops_random_sample_args;
/* SampleArgs::new (operators/src/random_sample/args.rs:66-78): 0 ok (top_p clamped to <= 1),
 * 1 NegativeTemperature, 2 NonPositiveTop. */
int ops_sample_args_new(float temperature, float top_p, size_t top_k, ops_sample_args *out);
int ops_random_sample_create(int device, ops_random_sample **out);
int ops_random_sample_scheme(ops_random_sample *op, const ops_random_sample_args *args, size_t max_ws, size_t *ws_out);
int ops_random_sample_launch(const ops_random_sample *op, const ops_random_sample_args *args, void *ws, size_t ws_len, void *stream);
void ops_random_sample_destroy(ops_random_sample *op);
/* RandomSample::build_indices (operators/src/random_sample/mod.rs:16-19): 0..n as u32 on the HOST. */
int ops_random_sample_build_indices(size_t n, uint32_t *host_out);
/* Extension with no counterpart in the crate (its API samples one row per launch): `rows` rows of
 * `n` logits, row stride `row_stride` bytes, one seed per row (device array of f32), `rows` KVPairs
 * out; one kernel launch for all rows.  Workspace as reported by the _batched_workspace call. */
size_t ops_random_sample_batched_workspace(uint32_t dt, size_t rows, size_t n, const ops_sample_args *config);
int ops_random_sample_launch_batched(const ops_random_sample *op, uint32_t dt, size_t rows, size_t n,
                                     const void *logits_base, ptrdiff_t row_stride, void *kv_pairs_base,
                                     const ops_sample_args *config, const float *seeds_dev,
                                     void *ws, size_t ws_len, void *stream);

/* No counterpart in the reference.  ops_random_sample_launch for callers that cannot allocate device memory where
 * they sample (a decode loop with the allocator locked down, a plugin that is given a stream but no allocator, a
 * process with a fixed memory budget): it takes no workspace.  The scratch is a fixed 2 MiB array inside the
 * library's device image, enough for one row of up to ops_random_sample_noalloc_max_logits() = 131072 logits; longer
 * rows are refused with OPS_SHAPE_NOT_SUPPORT.  Nothing is allocated or freed, here or in any routine it calls.
 * The array's device address is looked up when a random_sample handle is created on the device (if that failed, by
 * the first call, which should then come before any stream capture).
 * All calls on a device share the array: calls that overlap on the GPU race, so keep them on one stream or order
 * them yourself.  Results are identical to ops_random_sample_launch. */
size_t ops_random_sample_noalloc_max_logits(void);
int ops_random_sample_launch_noalloc(const ops_random_sample *op, const ops_random_sample_args *args, void *stream);

/* ---------------------------------------------------------------------------------------------
 * all_reduce — all_reduce::Args {pair: rearrange::Args, op} (operators/src/all_reduce/args.rs:9-12);
 * replaces all_reduce::common_cpu::Operator over InprocNode (operators/src/all_reduce/common_cpu.rs:15-104)
 * and the NCCL operator (operators/src/all_reduce/nccl.rs:12-62).  The topology node
 * (TopoNode: rank, group_size; operators/src/lib.rs:62-66) is an ops_comm: one per process/GPU.
 * ------------------------------------------------------------------------------------------- */
typedef struct ops_comm ops_comm;
#define OPS_COMM_ID_BYTES 128
/* rank 0 makes the id, the caller ships the 128 bytes to every rank (any transport), each rank
 * calls _init_rank with its own device current.  group_size 1 needs no id (NULL). */
int ops_comm_unique_id(uint8_t id_out[OPS_COMM_ID_BYTES]);
int ops_comm_init_rank(int device, int rank, int group_size, const uint8_t id[OPS_COMM_ID_BYTES], ops_comm **out);
int ops_comm_rank(const ops_comm *c);
int ops_comm_group_size(const ops_comm *c);
void ops_comm_destroy(ops_comm *c);
/* Peer-to-peer (NVLink) path: each rank allocates a symmetric staging buffer inside the library,
 * exports one handle of OPS_COMM_P2P_HANDLE_BYTES bytes, the caller all-gathers the handles
 * (group_size * OPS_COMM_P2P_HANDLE_BYTES bytes, rank order) and hands them back.  After _p2p_attach
 * the all_reduce operator may use the one-shot / two-shot kernels; before it, NCCL only.
 * `staging_bytes` is the largest message the peer-to-peer kernels will be given; the library holds
 * five regions of that size (double-buffered input and output staging, and the zero-copy input region).
 * The launch counter that tells the ranks' launches apart lives on the device and is advanced by the
 * kernels, so a launch recorded in a CUDA graph stays correct when the graph is replayed, provided
 * every rank replays the same sequence. */
#define OPS_COMM_P2P_HANDLE_BYTES 128
int ops_comm_p2p_export(ops_comm *c, size_t staging_bytes, uint8_t handle_out[OPS_COMM_P2P_HANDLE_BYTES]);
int ops_comm_p2p_attach(ops_comm *c, const uint8_t *all_handles /* group_size * OPS_COMM_P2P_HANDLE_BYTES */);
/* Status word of the P2P kernels on this rank: 0 ok, else a bounded wait ran out (read after the
 * stream is synchronised); the first failure sticks.  The output of a launch that set it is undefined. */
int ops_comm_p2p_status(ops_comm *c);
/* Start over after a time-out: once every rank's streams are idle and the ranks have met at a
 * host-side barrier, each rank calls this; status word, launch counter and all flags return to zero. */
int ops_comm_p2p_reset(ops_comm *c);
/* The zero-copy input region of this rank (staging_bytes long).  A kernel that writes its partial
 * there — the same offset on every rank — lets ops_all_reduce_launch / ops_all_reduce_add_launch read
 * it in place when given that pointer as src: no copy-in.  No counterpart in the crate. */
int ops_comm_p2p_direct(ops_comm *c, void **ptr_out, size_t *bytes_out);
/* In-switch reduction (NVLS).  `local` is this rank's address of a buffer of `bytes` bytes that the caller has bound to an
 * NVLink multicast object together with the same-sized buffers of every rank, `multicast` its multicast address (how the
 * object is made is the caller's business: the CUDA driver's cuMulticast* calls, or a library that wraps them).  The
 * first half of the buffer then serves as a zero-copy input region like the one above: an all_reduce (or all_reduce_add)
 * whose src lies there has its reduce-scatter half done inside the NVSwitch (multimem.ld_reduce); the second half is
 * reserved.  Needs ops_comm_p2p_attach first (the ranks synchronise through its flags).  Nulls detach.
 * No counterpart in the crate. */
int ops_comm_nvls_attach(ops_comm *c, void *multicast, void *local, size_t bytes);
/* Test aid with no counterpart in the crate: a communicator of `group_size` ranks that all map this rank's own staging
 * buffer.  Its peers never run, so a peer-to-peer all_reduce on it ends through its bounded waits (about one second)
 * with a non-zero ops_comm_p2p_status and an intact context: the time-out path can be exercised on one GPU. */
int ops_comm_create_loopback(int device, int group_size, size_t staging_bytes, ops_comm **out);

typedef struct ops_all_reduce ops_all_reduce;
typedef struct {
  ops_rearrange_args pair;
  uint8_t op;
} ops_all_reduce_args;
enum { OPS_ALL_REDUCE_AUTO = 0, OPS_ALL_REDUCE_NCCL = 1, OPS_ALL_REDUCE_P2P_ONE_SHOT = 2, OPS_ALL_REDUCE_P2P_TWO_SHOT = 3 };
int ops_all_reduce_create(ops_comm *node, ops_all_reduce **out);
int ops_all_reduce_set_algo(ops_all_reduce *op, int algo);
int ops_all_reduce_scheme(ops_all_reduce *op, const ops_all_reduce_args *args, size_t max_ws, size_t *ws_out);
int ops_all_reduce_launch(const ops_all_reduce *op, const ops_all_reduce_args *args, void *ws, size_t ws_len, void *stream);
void ops_all_reduce_destroy(ops_all_reduce *op);
/* Extension with no counterpart in the crate, which chains all_reduce and add (operators/src/add/common_cpu/mod.rs:29-75):
 * dst <- dst + sum over ranks of src in one kernel.  dst must hold the same values on every rank (a replicated residual
 * stream) and differ from src; f16/bf16/f32, peer-to-peer staging attached, >= 2 ranks; OPS_ARGS_NOT_SUPPORT otherwise
 * (chain ops_all_reduce_launch and ops_add_launch then).  The old dst enters the f32 sum first, then the ranks in order. */
int ops_all_reduce_add_launch(const ops_all_reduce *op, const ops_all_reduce_args *args, void *stream);

/* No counterpart in the crate (it chains mat_mul and all_reduce as two operators): C <- beta*C + alpha*A*B followed by
 * the f16 sum all_reduce of C over the group of `node`, as ONE kernel — finished tiles cross NVLink while the tensor
 * cores work on the remaining ones.  Needs ops_comm_p2p_attach with a staging region of at least m*n*2 bytes, f16
 * operands the tensor-core path accepts and a single dense row-major C.  beta applies to this rank's partial (fold the
 * residual in on exactly one rank).  Every rank of the group must call it with the same shapes. */
int ops_mat_mul_all_reduce_launch(const ops_mat_mul *op, ops_comm *node, const ops_mat_mul_args *args, void *stream);

/* =============================================================================================
 * Operators on either side of the decoder layer (the crate's operators a caller chains around it).
 * ============================================================================================= */

/* add — add::Args (operators/src/add/args.rs:12-20); replaces add::common_cpu::Operator
 * (operators/src/add/common_cpu/mod.rs:10-75).  c = a + b over N-d strided tensors of equal shape. */
typedef struct ops_add ops_add;
typedef struct {
  ops_layout c_layout; void *c_base;
  ops_layout a_layout; const void *a_base;
  ops_layout b_layout; const void *b_base;
} ops_add_args;
int ops_add_create(int device, ops_add **out);
int ops_add_scheme(ops_add *op, const ops_add_args *args, size_t max_ws, size_t *ws_out);
int ops_add_launch(const ops_add *op, const ops_add_args *args, void *ws, size_t ws_len, void *stream);
void ops_add_destroy(ops_add *op);

/* add_rows — add_rows::Args (operators/src/add_rows/args.rs:10-17); replaces add_rows::common_cpu::Operator
 * (operators/src/add_rows/common_cpu/mod.rs:12-148).  dst[b, m, :] += src[idx[b, m], :]; dst [batch, m, n],
 * src [k, n], idx [batch, m] u32 or u64.  An index >= k (an assert in the crate) leaves the row untouched and
 * sets the status word read by ops_add_rows_status (synchronises; no counterpart in the crate). */
typedef struct ops_add_rows ops_add_rows;
typedef struct {
  ops_layout dst_layout; void *dst_base;
  ops_layout src_layout; const void *src_base;
  ops_layout idx_layout; const void *idx_base;
} ops_add_rows_args;
int ops_add_rows_create(int device, ops_add_rows **out);
int ops_add_rows_scheme(ops_add_rows *op, const ops_add_rows_args *args, size_t max_ws, size_t *ws_out);
int ops_add_rows_launch(const ops_add_rows *op, const ops_add_rows_args *args, void *ws, size_t ws_len, void *stream);
int ops_add_rows_status(const ops_add_rows *op);
void ops_add_rows_destroy(ops_add_rows *op);

/* broadcast — broadcast::Args {pair: rearrange::Args, root} (operators/src/broadcast/args.rs:7-10); replaces
 * broadcast::common_cpu::Operator (operators/src/broadcast/common_cpu/mod.rs:12-69) and the NCCL operator
 * (operators/src/broadcast/nccl/mod.rs:36-60).  Every rank's dst receives root's src (bytes). */
typedef struct ops_broadcast ops_broadcast;
typedef struct {
  ops_rearrange_args pair;
  size_t root;
} ops_broadcast_args;
int ops_broadcast_create(ops_comm *node, ops_broadcast **out);
int ops_broadcast_scheme(ops_broadcast *op, const ops_broadcast_args *args, size_t max_ws, size_t *ws_out);
int ops_broadcast_launch(const ops_broadcast *op, const ops_broadcast_args *args, void *ws, size_t ws_len, void *stream);
void ops_broadcast_destroy(ops_broadcast *op);

#ifdef __cplusplus
}
#endif
#endif /* OPS_B200_H */
