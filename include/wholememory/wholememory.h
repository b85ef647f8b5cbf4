/*
 * wholememory_* spelling of the wholegraph C API.
 *
 * The interface of this library descends from a project that named everything wholememory_*;
 * the reference renamed it to wholegraph_* (rename policy: cpp/docs/DEVELOPER_GUIDE.md:21-23) but
 * still carries callers written against the old names: its optional torch extension
 * (python/wholegraph-torch/src/wholegraph_torch/torch_cpp_ext/torch_utils.cpp:11-181,
 * torch_env_func_ptrs.cpp:13-38) and the Python shim
 * python/pylibwholegraph/src/pylibwholegraph/binding/wholememory_binding.py:17-29.
 *
 * Types and enumerators are aliases of the wholegraph ones (same layout, same values).  The
 * functions are real exported symbols of libwholegraph.so: every wholegraph_* function has a
 * wholememory_* twin at the same address, so a binary built against the old names links and runs
 * unchanged.  This header declares the ones on the gather / scatter / optimizer path and the
 * tensor helpers the torch extension calls; for the rest, include the wholegraph header and call
 * the wholegraph name.
 */
#pragma once

#include <wholegraph/embedding.h>
#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/tensor_description.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>
#include <wholegraph/wholegraph_tensor_op.h>

/* ---- types ---- */
typedef wholegraph_access_type_t wholememory_access_type_t;
typedef wholegraph_array_description_t wholememory_array_description_t;
typedef wholegraph_comm_t wholememory_comm_t;
typedef wholegraph_create_memory_context_func_t wholememory_create_memory_context_func_t;
typedef wholegraph_destroy_memory_context_func_t wholememory_destroy_memory_context_func_t;
typedef wholegraph_distributed_backend_t wholememory_distributed_backend_t;
typedef wholegraph_dtype_t wholememory_dtype_t;
typedef wholegraph_embedding_cache_policy_t wholememory_embedding_cache_policy_t;
typedef wholegraph_embedding_optimizer_t wholememory_embedding_optimizer_t;
typedef wholegraph_embedding_t wholememory_embedding_t;
typedef wholegraph_env_func_t wholememory_env_func_t;
typedef wholegraph_error_code_t wholememory_error_code_t;
typedef wholegraph_free_func_t wholememory_free_func_t;
typedef wholegraph_gref_t wholememory_gref_t;
typedef wholegraph_handle_t wholememory_handle_t;
typedef wholegraph_malloc_func_t wholememory_malloc_func_t;
typedef wholegraph_matrix_description_t wholememory_matrix_description_t;
typedef wholegraph_memory_allocation_type_t wholememory_memory_allocation_type_t;
typedef wholegraph_memory_location_t wholememory_memory_location_t;
typedef wholegraph_memory_type_t wholememory_memory_type_t;
typedef wholegraph_optimizer_type_t wholememory_optimizer_type_t;
typedef wholegraph_output_memory_func_t wholememory_output_memory_func_t;
typedef wholegraph_temp_memory_func_t wholememory_temp_memory_func_t;
typedef wholegraph_tensor_description_t wholememory_tensor_description_t;
typedef wholegraph_tensor_t wholememory_tensor_t;
typedef wholegraph_unique_id_t wholememory_unique_id_t;

/* ---- enumerators and constants ---- */
#define WHOLEMEMORY_AT_NONE WHOLEGRAPH_AT_NONE
#define WHOLEMEMORY_AT_READONLY WHOLEGRAPH_AT_READONLY
#define WHOLEMEMORY_AT_READWRITE WHOLEGRAPH_AT_READWRITE
#define WHOLEMEMORY_COMMUNICATION_ERROR WHOLEGRAPH_COMMUNICATION_ERROR
#define WHOLEMEMORY_CUDA_ERROR WHOLEGRAPH_CUDA_ERROR
#define WHOLEMEMORY_DB_NCCL WHOLEGRAPH_DB_NCCL
#define WHOLEMEMORY_DB_NONE WHOLEGRAPH_DB_NONE
#define WHOLEMEMORY_DT_BF16 WHOLEGRAPH_DT_BF16
#define WHOLEMEMORY_DT_COUNT WHOLEGRAPH_DT_COUNT
#define WHOLEMEMORY_DT_DOUBLE WHOLEGRAPH_DT_DOUBLE
#define WHOLEMEMORY_DT_FLOAT WHOLEGRAPH_DT_FLOAT
#define WHOLEMEMORY_DT_HALF WHOLEGRAPH_DT_HALF
#define WHOLEMEMORY_DT_INT WHOLEGRAPH_DT_INT
#define WHOLEMEMORY_DT_INT16 WHOLEGRAPH_DT_INT16
#define WHOLEMEMORY_DT_INT64 WHOLEGRAPH_DT_INT64
#define WHOLEMEMORY_DT_INT8 WHOLEGRAPH_DT_INT8
#define WHOLEMEMORY_DT_UNKNOWN WHOLEGRAPH_DT_UNKNOWN
#define WHOLEMEMORY_INVALID_INPUT WHOLEGRAPH_INVALID_INPUT
#define WHOLEMEMORY_INVALID_VALUE WHOLEGRAPH_INVALID_VALUE
#define WHOLEMEMORY_LOGIC_ERROR WHOLEGRAPH_LOGIC_ERROR
#define WHOLEMEMORY_MAX_TENSOR_DIM WHOLEGRAPH_MAX_TENSOR_DIM
#define WHOLEMEMORY_MA_DEVICE WHOLEGRAPH_MA_DEVICE
#define WHOLEMEMORY_MA_HOST WHOLEGRAPH_MA_HOST
#define WHOLEMEMORY_MA_NONE WHOLEGRAPH_MA_NONE
#define WHOLEMEMORY_MA_PINNED WHOLEGRAPH_MA_PINNED
#define WHOLEMEMORY_ML_DEVICE WHOLEGRAPH_ML_DEVICE
#define WHOLEMEMORY_ML_HOST WHOLEGRAPH_ML_HOST
#define WHOLEMEMORY_ML_NONE WHOLEGRAPH_ML_NONE
#define WHOLEMEMORY_MT_CHUNKED WHOLEGRAPH_MT_CHUNKED
#define WHOLEMEMORY_MT_CONTINUOUS WHOLEGRAPH_MT_CONTINUOUS
#define WHOLEMEMORY_MT_DISTRIBUTED WHOLEGRAPH_MT_DISTRIBUTED
#define WHOLEMEMORY_MT_NONE WHOLEGRAPH_MT_NONE
#define WHOLEMEMORY_NOT_IMPLEMENTED WHOLEGRAPH_NOT_IMPLEMENTED
#define WHOLEMEMORY_NOT_SUPPORTED WHOLEGRAPH_NOT_SUPPORTED
#define WHOLEMEMORY_OPT_ADAGRAD WHOLEGRAPH_OPT_ADAGRAD
#define WHOLEMEMORY_OPT_LAZY_ADAM WHOLEGRAPH_OPT_LAZY_ADAM
#define WHOLEMEMORY_OPT_NONE WHOLEGRAPH_OPT_NONE
#define WHOLEMEMORY_OPT_RMSPROP WHOLEGRAPH_OPT_RMSPROP
#define WHOLEMEMORY_OPT_SGD WHOLEGRAPH_OPT_SGD
#define WHOLEMEMORY_OUT_OF_MEMORY WHOLEGRAPH_OUT_OF_MEMORY
#define WHOLEMEMORY_SPILT_NO_COLOR WHOLEGRAPH_SPILT_NO_COLOR
#define WHOLEMEMORY_SUCCESS WHOLEGRAPH_SUCCESS
#define WHOLEMEMORY_SYSTEM_ERROR WHOLEGRAPH_SYSTEM_ERROR
#define WHOLEMEMORY_UNIQUE_ID_BYTES WHOLEGRAPH_UNIQUE_ID_BYTES
#define WHOLEMEMORY_UNKNOW_ERROR WHOLEGRAPH_UNKNOW_ERROR
#define WHOLEMEMORY_RETURN_ON_FAIL(X) WHOLEGRAPH_RETURN_ON_FAIL(X)

#ifdef __cplusplus
extern "C" {
#endif

/* ---- the hot path (same arguments and return codes as the wholegraph functions) ---- */
wholememory_error_code_t wholememory_gather(wholememory_tensor_t wholememory_tensor,
                                            wholememory_tensor_t indices_tensor,
                                            wholememory_tensor_t output_tensor,
                                            wholememory_env_func_t* p_env_fns,
                                            void* stream,
                                            int gather_sms);
wholememory_error_code_t wholememory_scatter(wholememory_tensor_t input_tensor,
                                             wholememory_tensor_t indices_tensor,
                                             wholememory_tensor_t wholememory_tensor,
                                             wholememory_env_func_t* p_env_fns,
                                             void* stream,
                                             int scatter_sms);
wholememory_error_code_t wholememory_embedding_gather(wholememory_embedding_t wholememory_embedding,
                                                      wholememory_tensor_t indices,
                                                      wholememory_tensor_t output,
                                                      bool adjust_cache,
                                                      wholememory_env_func_t* p_env_fns,
                                                      int64_t stream_int);
wholememory_error_code_t wholememory_embedding_gather_gradient_apply(wholememory_embedding_t wholememory_embedding,
                                                                     wholememory_tensor_t indices,
                                                                     wholememory_tensor_t grads,
                                                                     bool adjust_cache,
                                                                     float lr,
                                                                     wholememory_env_func_t* p_env_fns,
                                                                     int64_t stream_int);

/* ---- memory handles: continuous, chunked and distributed ---- */
wholememory_error_code_t wholememory_malloc(wholememory_handle_t* wholememory_handle_ptr,
                                            size_t total_size,
                                            wholememory_comm_t comm,
                                            wholememory_memory_type_t memory_type,
                                            wholememory_memory_location_t memory_location,
                                            size_t data_granularity,
                                            size_t* rank_entry_partition);
wholememory_error_code_t wholememory_free(wholememory_handle_t wholememory_handle);
wholememory_error_code_t wholememory_create_tensor(wholememory_tensor_t* wholememory_tensor,
                                                   wholememory_tensor_description_t* tensor_description,
                                                   wholememory_comm_t comm,
                                                   wholememory_memory_type_t memory_type,
                                                   wholememory_memory_location_t memory_location,
                                                   size_t* tensor_entry_partition);

/* ---- tensor helpers ---- */
void wholememory_initialize_tensor_desc(wholememory_tensor_description_t* p_tensor_description);
wholememory_error_code_t wholememory_make_tensor_from_pointer(wholememory_tensor_t* wholememory_tensor,
                                                              void* storage_ptr,
                                                              wholememory_tensor_description_t* tensor_description);
wholememory_error_code_t wholememory_destroy_tensor(wholememory_tensor_t wholememory_tensor);
wholememory_tensor_description_t* wholememory_tensor_get_tensor_description(wholememory_tensor_t wholememory_tensor);
bool wholememory_unsqueeze_tensor(wholememory_tensor_description_t* p_tensor_description, int dim);
bool wholememory_squeeze_tensor(wholememory_tensor_description_t* p_tensor_description, int dim);
size_t wholememory_dtype_get_element_size(wholememory_dtype_t dtype);

#ifdef __cplusplus
}
#endif
