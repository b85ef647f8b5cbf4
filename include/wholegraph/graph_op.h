/*
 * Graph utility entry points of the WholeGraph C ABI
 * (reference: cpp/include/wholegraph/graph_op.h:27-48).
 *
 * Declared and exported so that a binding built against the reference's headers links and loads;
 * not built here: both functions log an error and return WHOLEGRAPH_NOT_IMPLEMENTED.
 */
#pragma once

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Distinct node ids of target nodes followed by neighbour nodes, and the neighbours' positions in
 * that list. */
wholegraph_error_code_t graph_append_unique(
  wholegraph_tensor_t target_nodes_tensor,
  wholegraph_tensor_t neighbor_nodes_tensor,
  void* output_unique_node_memory_context,
  wholegraph_tensor_t output_neighbor_raw_to_unique_mapping_tensor,
  wholegraph_env_func_t* p_env_fns,
  void* stream);

/* CSR graph with one self loop added per row. */
wholegraph_error_code_t csr_add_self_loop(wholegraph_tensor_t csr_row_ptr_tensor,
                                           wholegraph_tensor_t csr_col_ptr_tensor,
                                           wholegraph_tensor_t output_csr_row_ptr_tensor,
                                           wholegraph_tensor_t output_csr_col_ptr_tensor,
                                           void* stream);

#ifdef __cplusplus
}
#endif
