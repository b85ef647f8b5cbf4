// graph_append_unique / csr_add_self_loop: the two node-list utilities between neighbour sampling
// and the embedding gather of a mini-batch.
//
// Reference behaviour: cpp/src/graph_ops/append_unique.cpp:9-78 and csr_add_self_loop.cpp:9-91
// (argument checks and return codes), append_unique_func.cuh:263-341 (outputs: target_count +
// unique neighbour count nodes through the output allocator, optional int32 mapping).
#include <wholegraph/graph_op.h>

#include "common.hpp"
#include "env.hpp"
#include "kernels/graph_ops.hpp"

extern "C" {

wholegraph_error_code_t graph_append_unique(wholegraph_tensor_t target_nodes_tensor,
                                            wholegraph_tensor_t neighbor_nodes_tensor,
                                            void* output_unique_node_memory_context,
                                            wholegraph_tensor_t output_neighbor_raw_to_unique_mapping_tensor,
                                            wholegraph_env_func_t* p_env_fns,
                                            void* stream_ptr)
{
  if (target_nodes_tensor == nullptr || neighbor_nodes_tensor == nullptr || p_env_fns == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  auto* td = wholegraph_tensor_get_tensor_description(target_nodes_tensor);
  auto* nd = wholegraph_tensor_get_tensor_description(neighbor_nodes_tensor);
  if (td->dim != 1) {
    WGB_ERROR("target_nodes_tensor should be 1D tensor.");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (nd->dim != 1) {
    WGB_ERROR("neighbor_nodes_tensor should be 1D tensor.");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  int* mapping = nullptr;
  if (output_neighbor_raw_to_unique_mapping_tensor != nullptr) {
    auto* md = wholegraph_tensor_get_tensor_description(output_neighbor_raw_to_unique_mapping_tensor);
    if (md->dim != 1 && md->dim != 0) {
      WGB_ERROR("output_neighbor_raw_to_unique_mapping_tensor should be 1D tensor or None.");
      return WHOLEGRAPH_INVALID_INPUT;
    }
    if (md->dim == 1) {
      if (md->dtype != WHOLEGRAPH_DT_INT) {
        WGB_ERROR("output_neighbor_raw_to_unique_mapping_tensor should be int tensor or None.");
        return WHOLEGRAPH_INVALID_INPUT;
      }
      if (md->sizes[0] < nd->sizes[0] || md->strides[0] != 1) {
        WGB_ERROR("output_neighbor_raw_to_unique_mapping_tensor must hold one dense entry per neighbour.");
        return WHOLEGRAPH_INVALID_INPUT;
      }
      mapping = static_cast<int*>(wholegraph_tensor_get_data_pointer(output_neighbor_raw_to_unique_mapping_tensor));
    }
  }
  if (td->dtype != nd->dtype) {
    WGB_ERROR("target_nodes_dtype should be the same with neighbor_nodes_dtype");
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  if (td->dtype != WHOLEGRAPH_DT_INT && td->dtype != WHOLEGRAPH_DT_INT64) {
    WGB_ERROR("node ids must be int32 or int64");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (td->strides[0] != 1 || nd->strides[0] != 1) {
    WGB_ERROR("node id tensors must be dense");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  WGB_API_BEGIN
  auto stream           = static_cast<cudaStream_t>(stream_ptr);
  const bool ids_are_64 = td->dtype == WHOLEGRAPH_DT_INT64;
  const int64_t t_count = td->sizes[0], n_count = nd->sizes[0];
  const void* targets   = wholegraph_tensor_get_data_pointer(target_nodes_tensor);
  const void* neighbors = wholegraph_tensor_get_data_pointer(neighbor_nodes_tensor);
  wgb::temp_buffer ws(p_env_fns), count_buf(p_env_fns);
  void* workspace = ws.device_bytes(wgb::append_unique_workspace_bytes(t_count, n_count, ids_are_64));
  int* new_count  = static_cast<int*>(count_buf.pinned(1, WHOLEGRAPH_DT_INT));
  wgb::append_unique_group(targets, t_count, neighbors, n_count, ids_are_64, workspace, new_count, stream);
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));  // the output's size is needed to allocate it
  // The list of unique nodes is allocated by the caller's output allocator once its length is known.
  wholegraph_tensor_description_t od;
  wholegraph_initialize_tensor_desc(&od);
  od.dim        = 1;
  od.dtype      = td->dtype;
  od.sizes[0]   = t_count + *new_count;
  od.strides[0] = 1;
  void* unique  = p_env_fns->output_fns.malloc_fn(&od, WHOLEGRAPH_MA_DEVICE, output_unique_node_memory_context,
                                                 p_env_fns->output_fns.global_context);
  if (unique == nullptr && od.sizes[0] > 0) {
    WGB_ERROR("the output allocator returned no memory for %ld unique nodes", (long)od.sizes[0]);
    return WHOLEGRAPH_OUT_OF_MEMORY;
  }
  wgb::append_unique_write(targets, t_count, n_count, ids_are_64, workspace, unique, mapping, stream);
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));  // as the reference: outputs are complete on return
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("graph_append_unique")
}

wholegraph_error_code_t csr_add_self_loop(wholegraph_tensor_t csr_row_ptr_tensor,
                                          wholegraph_tensor_t csr_col_ptr_tensor,
                                          wholegraph_tensor_t output_csr_row_ptr_tensor,
                                          wholegraph_tensor_t output_csr_col_ptr_tensor,
                                          void* stream_ptr)
{
  wholegraph_tensor_t all[4]  = {csr_row_ptr_tensor, csr_col_ptr_tensor, output_csr_row_ptr_tensor,
                                 output_csr_col_ptr_tensor};
  const char* const names[4] = {"Input csr_row_ptr_tensor", "Input csr_col_ptr_tensor",
                                "Output output_csr_row_ptr_tensor", "Output output_csr_col_ptr_tensor"};
  for (int i = 0; i < 4; i++) {
    if (all[i] == nullptr) return WHOLEGRAPH_INVALID_INPUT;
    auto* d = wholegraph_tensor_get_tensor_description(all[i]);
    if (d->dim != 1) {
      WGB_ERROR("%s should be 1D tensor.", names[i]);
      return WHOLEGRAPH_INVALID_INPUT;
    }
    if (d->dtype != WHOLEGRAPH_DT_INT) {
      WGB_ERROR("%s should be int tensor.", names[i]);
      return WHOLEGRAPH_INVALID_INPUT;
    }
    if (d->strides[0] != 1) {
      WGB_ERROR("%s should be dense.", names[i]);
      return WHOLEGRAPH_INVALID_INPUT;
    }
  }
  auto* rd = wholegraph_tensor_get_tensor_description(csr_row_ptr_tensor);
  auto* cd = wholegraph_tensor_get_tensor_description(csr_col_ptr_tensor);
  auto* ord = wholegraph_tensor_get_tensor_description(output_csr_row_ptr_tensor);
  auto* ocd = wholegraph_tensor_get_tensor_description(output_csr_col_ptr_tensor);
  if (rd->sizes[0] < 1 || ord->sizes[0] < rd->sizes[0] || ocd->sizes[0] < cd->sizes[0] + rd->sizes[0] - 1) {
    WGB_ERROR("output CSR tensors are too small for %ld rows and %ld edges", (long)(rd->sizes[0] - 1),
              (long)cd->sizes[0]);
    return WHOLEGRAPH_INVALID_INPUT;
  }
  WGB_API_BEGIN
  auto stream        = static_cast<cudaStream_t>(stream_ptr);
  const int64_t rows = rd->sizes[0] - 1;
  const int* row_ptr = static_cast<const int*>(wholegraph_tensor_get_data_pointer(csr_row_ptr_tensor));
  int* out_row_ptr   = static_cast<int*>(wholegraph_tensor_get_data_pointer(output_csr_row_ptr_tensor));
  if (rows == 0) {
    WGB_CUDA_CHECK(cudaMemcpyAsync(out_row_ptr, row_ptr, sizeof(int), cudaMemcpyDeviceToDevice, stream));
    return WHOLEGRAPH_SUCCESS;
  }
  wgb::csr_add_self_loops(row_ptr, static_cast<const int*>(wholegraph_tensor_get_data_pointer(csr_col_ptr_tensor)),
                          rows, out_row_ptr,
                          static_cast<int*>(wholegraph_tensor_get_data_pointer(output_csr_col_ptr_tensor)), stream);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("csr_add_self_loop")
}

}  // extern "C"
