// internal.h — entry points the composite operators (attention, attention_kv_cached) call on the
// primitive ones, bypassing the C ABI but running exactly the same code.
#pragma once
#include "common.h"

struct ops_mat_mul;

namespace ops {

int rearrange_enqueue(const OpBase &base, const ops_rearrange_args *args, cudaStream_t s);
int fused_softmax_enqueue(const OpBase &base, const ops_fused_softmax_args *args, cudaStream_t s);
int mat_mul_enqueue(const ops_mat_mul *op, const ops_mat_mul_args *args, cudaStream_t s);
bool attention_fused_supported(const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh);
int attention_fused_enqueue(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh, int *status,
                            bool *attr_set, void *ws, usz ws_len, cudaStream_t s, bool single_tile);

bool attention_decode_supported(const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh);
usz attention_decode_scratch_bytes();
usz attention_decode_ticket_bytes();
int attention_decode_enqueue(const OpBase &base, const ops_attention_args *a, usz nh, usz nkvh, usz seq, usz att, usz dh, float *scratch,
                             unsigned int *tickets, cudaStream_t s);

}  // namespace ops
