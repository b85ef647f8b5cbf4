/*
 * Graph sampling entry points of the WholeGraph C ABI
 * (reference: cpp/include/wholegraph/wholegraph_op.h:31-95).
 *
 * Declared and exported so that a binding built against the reference's headers links and loads;
 * this library does not build the sampling path: every function here logs an error and returns
 * WHOLEGRAPH_NOT_IMPLEMENTED without touching its arguments.
 */
#pragma once

#include <stdint.h>

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Neighbour sampling without replacement on a CSR graph held in WholeGraph tensors (row offsets,
 * column ids), at most `fanout` neighbours per centre node.  Offsets per centre go to
 * `sample_offsets`; sampled neighbours, their centre's position and the edge ids go to caller
 * memory contexts through env->output_fns. */
wholegraph_error_code_t wholegraph_csr_unweighted_sample_without_replacement(
  wholegraph_tensor_t row_offsets, wholegraph_tensor_t column_ids, wholegraph_tensor_t centres, int fanout,
  wholegraph_tensor_t sample_offsets, void* neighbours_context, void* centre_position_context,
  void* edge_id_context, unsigned long long seed, wholegraph_env_func_t* env, void* stream);

/* The same with one weight per edge (`edge_weights`, laid out like `column_ids`). */
wholegraph_error_code_t wholegraph_csr_weighted_sample_without_replacement(
  wholegraph_tensor_t row_offsets, wholegraph_tensor_t column_ids, wholegraph_tensor_t edge_weights,
  wholegraph_tensor_t centres, int fanout, wholegraph_tensor_t sample_offsets, void* neighbours_context,
  void* centre_position_context, void* edge_id_context, unsigned long long seed, wholegraph_env_func_t* env,
  void* stream);

/* Host-side restatements of the sampler's random streams (positive integers; negated
 * exponential variates), used by the reference's tests: `out` is a 1-D host tensor. */
wholegraph_error_code_t generate_random_positive_int_cpu(int64_t seed, int64_t subsequence, wholegraph_tensor_t out);
wholegraph_error_code_t generate_exponential_distribution_negative_float_cpu(int64_t seed, int64_t subsequence,
                                                                             wholegraph_tensor_t out);

#ifdef __cplusplus
}
#endif
