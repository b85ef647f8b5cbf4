/*
 * wholegraph-b200: row gather / scatter.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/wholegraph_tensor_op.h:25-68.
 */
#pragma once

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * output[i, :] = cast(table[indices[i], :]) for every i with indices[i] >= 0; rows whose
 * index is negative are left untouched. Replaces wholegraph_gather
 * (cpp/src/wholegraph_tensor_ops/gather_op.cpp:12-106).
 *   wholegraph_tensor : 1-D or 2-D table; a handle tensor of any memory type, or a pointer tensor.
 *   indices_tensor    : 1-D int32 / int64, device memory, not a handle tensor.
 *   output_tensor     : same dimensionality as the table, sizes[0] == indices.size, device memory.
 *   stream            : cudaStream_t.
 *   gather_sms        : -1, or a CTA-count hint for the copy kernel.
 * Table and output dtypes must both be floating point or both be integer.
 */
wholegraph_error_code_t wholegraph_gather(wholegraph_tensor_t wholegraph_tensor,
                                            wholegraph_tensor_t indices_tensor,
                                            wholegraph_tensor_t output_tensor,
                                            wholegraph_env_func_t* p_env_fns,
                                            void* stream,
                                            int gather_sms = -1);

/*
 * table[indices[i], :] = cast(input[i, :]) for every i with indices[i] >= 0. Duplicate
 * indices race; one of the writers wins per row segment. Replaces wholegraph_scatter
 * (cpp/src/wholegraph_tensor_ops/scatter_op.cpp:12-98).
 */
wholegraph_error_code_t wholegraph_scatter(wholegraph_tensor_t input_tensor,
                                             wholegraph_tensor_t indices_tensor,
                                             wholegraph_tensor_t wholegraph_tensor,
                                             wholegraph_env_func_t* p_env_fns,
                                             void* stream,
                                             int scatter_sms = -1);

/*
 * Allocator-callback self test (wholegraph_tensor_op.h:60-68): copies `input_tensor` to
 * `output_fixed_tensor` through a temporary buffer and fills three outputs of
 * `output_variable_entry_count` rows allocated through `output_fns`.
 */
wholegraph_error_code_t wholegraph_env_test_op(wholegraph_tensor_t input_tensor,
                                                 wholegraph_tensor_t output_fixed_tensor,
                                                 void* output_variable_device_tensor_handle,
                                                 void* output_variable_pinned_tensor_handle,
                                                 void* output_variable_host_tensor_handle,
                                                 int64_t output_variable_entry_count,
                                                 wholegraph_env_func_t* p_env_fns,
                                                 void* stream);

#ifdef __cplusplus
}
#endif
