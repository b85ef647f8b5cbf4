/*
 * Graph utility entry points of the WholeGraph C ABI
 * (reference: cpp/include/wholegraph/graph_op.h:27-48).
 *
 * Same declarations, argument checks and return codes.  One stated difference in
 * graph_append_unique: the reference appends the new neighbours in the order its hash table
 * happens to hold them; here they are appended in ascending id order, so results are reproducible.
 */
#pragma once

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Node list of a sampled hop: the target nodes in their order, then every distinct neighbour that is
 * not a target (ascending).  The list is allocated through env->output_fns for
 * output_unique_node_memory_context once its length is known; the optional int32 mapping tensor
 * receives, per neighbour, its position in the list.  Ids are int32 or int64 (same type for both
 * inputs), tensors 1-D and dense.  Synchronises the stream; outputs are complete on return. */
wholegraph_error_code_t graph_append_unique(
  wholegraph_tensor_t target_nodes_tensor,
  wholegraph_tensor_t neighbor_nodes_tensor,
  void* output_unique_node_memory_context,
  wholegraph_tensor_t output_neighbor_raw_to_unique_mapping_tensor,
  wholegraph_env_func_t* p_env_fns,
  void* stream);

/* CSR graph (int32 row pointers and columns) with edge (r, r) put first in every row r:
 * output_row_ptr[r] = row_ptr[r] + r.  The outputs must hold rows + 1 and edges + rows entries.
 * Asynchronous on the stream. */
wholegraph_error_code_t csr_add_self_loop(wholegraph_tensor_t csr_row_ptr_tensor,
                                           wholegraph_tensor_t csr_col_ptr_tensor,
                                           wholegraph_tensor_t output_csr_row_ptr_tensor,
                                           wholegraph_tensor_t output_csr_col_ptr_tensor,
                                           void* stream);

#ifdef __cplusplus
}
#endif
