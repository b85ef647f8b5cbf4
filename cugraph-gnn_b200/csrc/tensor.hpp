// Tensor object behind wholegraph_tensor_t: a descriptor over a handle or a raw pointer.
// The struct is POD and malloc'd, like the reference's (cpp/src/wholegraph/wholegraph_tensor.cpp:27-36).
#pragma once

#include <wholegraph/wholegraph_tensor.h>

struct wholegraph_tensor_ {
  union {
    wholegraph_handle_t handle;
    void* storage_ptr;
  };
  wholegraph_tensor_description_t desc;
  wholegraph_tensor_t root;
  bool is_wholegraph;
  bool own_handle;
};
