/*
 * wholegraph-b200: caller-supplied allocator callbacks.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/env_func_ptrs.h:17-62.
 * Every temporary an op needs is requested through `temporary_fns`:
 *   create_memory_context -> malloc(desc, DEVICE|HOST|PINNED) -> free -> destroy_memory_context.
 * One context owns at most one buffer.
 */
#pragma once

#include <cuda_runtime_api.h>
#include <wholegraph/tensor_description.h>

#ifdef __cplusplus
extern "C" {
#endif

enum wholegraph_memory_allocation_type_t {
  WHOLEGRAPH_MA_NONE = 0,
  WHOLEGRAPH_MA_DEVICE,
  WHOLEGRAPH_MA_HOST,
  WHOLEGRAPH_MA_PINNED,
};

typedef void (*wholegraph_create_memory_context_func_t)(void** memory_context,
                                                         void* global_context);

typedef void (*wholegraph_destroy_memory_context_func_t)(void* memory_context,
                                                          void* global_context);

typedef void* (*wholegraph_malloc_func_t)(
  wholegraph_tensor_description_t* desc,
  wholegraph_memory_allocation_type_t memory_allocation_type,
  void* memory_context,
  void* global_context);

typedef void (*wholegraph_free_func_t)(void* memory_context, void* global_context);

struct wholegraph_temp_memory_func_t {
  wholegraph_create_memory_context_func_t create_memory_context_fn;
  wholegraph_destroy_memory_context_func_t destroy_memory_context_fn;
  wholegraph_malloc_func_t malloc_fn;
  wholegraph_free_func_t free_fn;
  void* global_context;
};

struct wholegraph_output_memory_func_t {
  wholegraph_malloc_func_t malloc_fn;
  wholegraph_free_func_t free_fn;
  void* global_context;
};

struct wholegraph_env_func_t {
  wholegraph_temp_memory_func_t temporary_fns; /* scratch buffers of one op call */
  wholegraph_output_memory_func_t output_fns;  /* variable-size op outputs */
};

/* Cached cudaDeviceProp of a device (env_func_ptrs.h:64). */
cudaDeviceProp* get_device_prop(int dev_id);

#ifdef __cplusplus
}
#endif
