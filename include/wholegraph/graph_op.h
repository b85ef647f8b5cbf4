/*
 * Graph utility entry points of the WholeGraph C ABI
 * (reference: cpp/include/wholegraph/graph_op.h:27-48).
 *
 * Same functions, argument order, checks and return codes.  One stated difference in
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
 * not a target (ascending).  The list is allocated through env->output_fns for `unique_nodes_context`
 * once its length is known; the optional int32 tensor `neighbour_positions` receives, per neighbour,
 * its position in the list.  Ids are int32 or int64 (same type for both inputs), tensors 1-D and
 * dense.  Synchronises the stream; outputs are complete on return. */
wholegraph_error_code_t graph_append_unique(wholegraph_tensor_t targets, wholegraph_tensor_t neighbours,
                                            void* unique_nodes_context, wholegraph_tensor_t neighbour_positions,
                                            wholegraph_env_func_t* env, void* stream);

/* CSR graph (int32 row offsets and column ids) with edge (r, r) put first in every row r:
 * looped_row_offsets[r] = row_offsets[r] + r.  The outputs must hold rows + 1 and edges + rows
 * entries.  Asynchronous on the stream. */
wholegraph_error_code_t csr_add_self_loop(wholegraph_tensor_t row_offsets, wholegraph_tensor_t column_ids,
                                          wholegraph_tensor_t looped_row_offsets,
                                          wholegraph_tensor_t looped_column_ids, void* stream);

#ifdef __cplusplus
}
#endif
