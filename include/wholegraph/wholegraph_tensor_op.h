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
 *   table      : 1-D or 2-D; a handle tensor of any memory type, or a pointer tensor.
 *   indices    : 1-D int32 / int64, device memory, not a handle tensor.
 *   output     : same dimensionality as the table, sizes[0] == indices.size, device memory.
 *   env        : allocator callbacks for scratch memory.
 *   stream     : cudaStream_t.
 *   gather_sms : -1, or a CTA-count hint for the copy kernel.
 * Table and output dtypes must both be floating point or both be integer.
 */
wholegraph_error_code_t wholegraph_gather(wholegraph_tensor_t table, wholegraph_tensor_t indices,
                                          wholegraph_tensor_t output, wholegraph_env_func_t* env, void* stream,
                                          int gather_sms = -1);

/*
 * table[indices[i], :] = cast(input[i, :]) for every i with indices[i] >= 0. Duplicate
 * indices race; one of the writers wins per row segment. Replaces wholegraph_scatter
 * (cpp/src/wholegraph_tensor_ops/scatter_op.cpp:12-98).
 */
wholegraph_error_code_t wholegraph_scatter(wholegraph_tensor_t input, wholegraph_tensor_t indices,
                                           wholegraph_tensor_t table, wholegraph_env_func_t* env, void* stream,
                                           int scatter_sms = -1);

/*
 * Allocator-callback self test (wholegraph_tensor_op.h:60-68): copies `input` to `fixed_output`
 * through a temporary buffer and fills three outputs of `rows` rows allocated through
 * env->output_fns for the three given contexts (device, pinned host, pageable host memory).
 */
wholegraph_error_code_t wholegraph_env_test_op(wholegraph_tensor_t input, wholegraph_tensor_t fixed_output,
                                               void* device_output_context, void* pinned_output_context,
                                               void* host_output_context, int64_t rows,
                                               wholegraph_env_func_t* env, void* stream);

#ifdef __cplusplus
}
#endif
