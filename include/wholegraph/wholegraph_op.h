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

/* Neighbour sampling without replacement on a CSR graph held in WholeGraph tensors; outputs go to
 * caller memory contexts through env->output_fns. */
wholegraph_error_code_t wholegraph_csr_unweighted_sample_without_replacement(
  wholegraph_tensor_t wg_csr_row_ptr_tensor,
  wholegraph_tensor_t wg_csr_col_ptr_tensor,
  wholegraph_tensor_t center_nodes_tensor,
  int max_sample_count,
  wholegraph_tensor_t output_sample_offset_tensor,
  void* output_dest_memory_context,
  void* output_center_localid_memory_context,
  void* output_edge_gid_memory_context,
  unsigned long long random_seed,
  wholegraph_env_func_t* p_env_fns,
  void* stream);

/* The same with per-edge weights. */
wholegraph_error_code_t wholegraph_csr_weighted_sample_without_replacement(
  wholegraph_tensor_t wg_csr_row_ptr_tensor,
  wholegraph_tensor_t wg_csr_col_ptr_tensor,
  wholegraph_tensor_t wg_csr_weight_ptr_tensor,
  wholegraph_tensor_t center_nodes_tensor,
  int max_sample_count,
  wholegraph_tensor_t output_sample_offset_tensor,
  void* output_dest_memory_context,
  void* output_center_localid_memory_context,
  void* output_edge_gid_memory_context,
  unsigned long long random_seed,
  wholegraph_env_func_t* p_env_fns,
  void* stream);

/* Host-side restatements of the sampler's random streams, used by the reference's tests. */
wholegraph_error_code_t generate_random_positive_int_cpu(int64_t random_seed,
                                                          int64_t subsequence,
                                                          wholegraph_tensor_t output);
wholegraph_error_code_t generate_exponential_distribution_negative_float_cpu(
  int64_t random_seed, int64_t subsequence, wholegraph_tensor_t output);

#ifdef __cplusplus
}
#endif
