/*
 * wholegraph-b200: entry points that exist only in this library (no counterpart in the
 * reference's public headers).  They cover what the reference keeps in internal C++ symbols
 * (wholegraph::get_default_env_func / get_cached_env_func, cpp/src/wholegraph/env_func_ptrs.hpp)
 * so that C and ctypes callers can reach them, plus run-time introspection for benchmarks.
 */
#pragma once

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Allocator callbacks backed by cudaMalloc / cudaMallocHost / malloc; every free waits for the device. */
wholegraph_env_func_t* wholegraph_b200_get_default_env_func();

/*
 * Allocator callbacks with a size-class free list: a buffer released by one op is handed to
 * the next one without touching the CUDA allocator.  Work that reuses a buffer must be ordered
 * on the stream(s) the ops were given.
 */
wholegraph_env_func_t* wholegraph_b200_get_cached_env_func();

/* Return every block of the caching allocator to CUDA (synchronizes the device first). */
void wholegraph_b200_drop_cached_env_func_memory();

/*
 * cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream) for callers that hold raw
 * pointers (a shard of a handle, a ctypes buffer) but no CUDA runtime binding of their own.
 */
wholegraph_error_code_t wholegraph_b200_memcpy_async(void* dst, const void* src, size_t bytes,
                                                       void* stream);

/* Number of kernels this library has launched in this process since load. */
unsigned long long wholegraph_b200_kernel_launch_count();

/* Library identification string, e.g. "wholegraph-b200 sm_100a". */
const char* wholegraph_b200_version();

#ifdef __cplusplus
}
#endif
