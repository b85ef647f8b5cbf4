// Temporary-memory RAII over the caller's allocator callbacks, and the two allocators this
// library ships for callers that have none (plain and caching).
// Role of the reference's cpp/src/wholegraph_tensor_ops/temp_memory_handle.hpp:12-82 and
// cpp/src/wholegraph/env_func_ptrs.cpp.
#pragma once

#include <cstddef>
#include <cstdint>

#include <wholegraph/env_func_ptrs.h>

namespace wgb {

// One scratch buffer obtained through env->temporary_fns; released in the destructor.
class temp_buffer {
 public:
  explicit temp_buffer(wholegraph_env_func_t* env);
  ~temp_buffer();
  temp_buffer(const temp_buffer&)            = delete;
  temp_buffer& operator=(const temp_buffer&) = delete;

  void* device(size_t count, wholegraph_dtype_t dt) { return get(count, dt, WHOLEGRAPH_MA_DEVICE); }
  void* host(size_t count, wholegraph_dtype_t dt) { return get(count, dt, WHOLEGRAPH_MA_HOST); }
  void* pinned(size_t count, wholegraph_dtype_t dt) { return get(count, dt, WHOLEGRAPH_MA_PINNED); }
  void* device_bytes(size_t bytes) { return device((bytes + 7) / 8, WHOLEGRAPH_DT_INT64); }
  void* pinned_bytes(size_t bytes) { return pinned((bytes + 7) / 8, WHOLEGRAPH_DT_INT64); }
  void* pointer() const { return ptr_; }
  void release();

 private:
  void* get(size_t count, wholegraph_dtype_t dt, wholegraph_memory_allocation_type_t where);
  wholegraph_env_func_t* env_;
  void* ctx_ = nullptr;
  void* ptr_ = nullptr;
};

}  // namespace wgb
