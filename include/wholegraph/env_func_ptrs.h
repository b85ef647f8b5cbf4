/*
 * wholegraph-b200: caller-supplied allocator callbacks.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/env_func_ptrs.h:17-62 (same type and member
 * names, same layouts).  How the library uses them:
 *
 *   scratch   env->temporary_fns: create_memory_context_fn(&ctx, global) once per buffer, then
 *             malloc_fn(&description, where, ctx, global) exactly once for that context, later
 *             free_fn(ctx, global) and destroy_memory_context_fn(ctx, global).  One context owns
 *             at most one buffer; `where` says device, pageable host or pinned host memory.
 *   outputs   env->output_fns: for results whose size only the op knows, malloc_fn is called with
 *             the context pointer the caller passed to the op; the buffer belongs to the caller.
 *
 * The library's own allocators (wholegraph_b200.h) are instances of these tables.
 */
#pragma once

#include <cuda_runtime_api.h>
#include <wholegraph/tensor_description.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Where a requested buffer must live. */
enum wholegraph_memory_allocation_type_t {
  WHOLEGRAPH_MA_NONE = 0,
  WHOLEGRAPH_MA_DEVICE,  /* 1: device memory */
  WHOLEGRAPH_MA_HOST,    /* 2: pageable host memory */
  WHOLEGRAPH_MA_PINNED,  /* 3: page-locked host memory */
};

/* ctx_out receives a new context; user is the table's global_context. */
typedef void (*wholegraph_create_memory_context_func_t)(void** ctx_out, void* user);
typedef void (*wholegraph_destroy_memory_context_func_t)(void* ctx, void* user);
/* Returns the buffer for a tensor of the given description (element count x element size bytes). */
typedef void* (*wholegraph_malloc_func_t)(wholegraph_tensor_description_t* what,
                                           wholegraph_memory_allocation_type_t where, void* ctx, void* user);
typedef void (*wholegraph_free_func_t)(void* ctx, void* user);

/* Scratch buffers of one op call. */
struct wholegraph_temp_memory_func_t {
  wholegraph_create_memory_context_func_t create_memory_context_fn;
  wholegraph_destroy_memory_context_func_t destroy_memory_context_fn;
  wholegraph_malloc_func_t malloc_fn;
  wholegraph_free_func_t free_fn;
  void* global_context;
};

/* Variable-size op outputs. */
struct wholegraph_output_memory_func_t {
  wholegraph_malloc_func_t malloc_fn;
  wholegraph_free_func_t free_fn;
  void* global_context;
};

struct wholegraph_env_func_t {
  wholegraph_temp_memory_func_t temporary_fns;
  wholegraph_output_memory_func_t output_fns;
};

/* Properties of device `dev_id` (the current device when negative), queried once and cached
 * (reference: env_func_ptrs.h:64). */
cudaDeviceProp* get_device_prop(int dev_id);

#ifdef __cplusplus
}
#endif
