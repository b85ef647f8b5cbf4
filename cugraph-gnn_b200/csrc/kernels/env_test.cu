// wholegraph_env_test_op: allocator-callback self test.
// Behaviour follows the reference's cpp/src/wholegraph_tensor_ops/wholegraph_test_op.cu:12-160:
// row i of every output is input + T(float(i)), computed in a temporary buffer obtained from
// the caller's callbacks and copied to the fixed output and to three outputs allocated through
// output_fns (device, pinned, host).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <wholegraph/wholegraph_tensor_op.h>

#include "../common.hpp"
#include "../env.hpp"
#include "row_copy.hpp"

namespace {

template <typename T>
__global__ void env_test_kernel(const T* input, T* out, int64_t dim, int64_t stride)
{
  const int64_t row = blockIdx.x;
  const float f     = static_cast<float>(row);
  for (int64_t c = threadIdx.x; c < dim; c += blockDim.x)
    out[row * stride + c] = static_cast<T>(static_cast<float>(static_cast<T>(f)) + static_cast<float>(input[c]));
}
template <typename T>
__global__ void env_test_kernel_native(const T* input, T* out, int64_t dim, int64_t stride)
{
  const int64_t row = blockIdx.x;
  for (int64_t c = threadIdx.x; c < dim; c += blockDim.x)
    out[row * stride + c] = static_cast<T>(static_cast<float>(row)) + input[c];
}

template <typename T>
void run_native(const void* in, void* out, int64_t dim, int64_t rows, int64_t stride, cudaStream_t s)
{
  env_test_kernel_native<T><<<static_cast<unsigned>(rows), 256, 0, s>>>(static_cast<const T*>(in),
                                                                        static_cast<T*>(out), dim, stride);
}
template <typename T>
void run_via_float(const void* in, void* out, int64_t dim, int64_t rows, int64_t stride, cudaStream_t s)
{
  env_test_kernel<T><<<static_cast<unsigned>(rows), 256, 0, s>>>(static_cast<const T*>(in),
                                                                 static_cast<T*>(out), dim, stride);
}

}  // namespace

extern "C" wholegraph_error_code_t wholegraph_env_test_op(wholegraph_tensor_t input_tensor,
                                                            wholegraph_tensor_t output_fixed_tensor,
                                                            void* out_device_handle,
                                                            void* out_pinned_handle,
                                                            void* out_host_handle,
                                                            int64_t entry_count,
                                                            wholegraph_env_func_t* env,
                                                            void* stream_ptr)
{
  if (input_tensor == nullptr || output_fixed_tensor == nullptr || env == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = static_cast<cudaStream_t>(stream_ptr);
  auto* id    = wholegraph_tensor_get_tensor_description(input_tensor);
  auto* od    = wholegraph_tensor_get_tensor_description(output_fixed_tensor);
  WGB_EXPECTS(id->dim == 1 && od->dim == 2 && od->sizes[0] == entry_count && od->sizes[1] == id->sizes[0] &&
                id->dtype == od->dtype,
              "env test op: shapes or dtypes do not match");
  const int64_t dim = id->sizes[0];
  const size_t es   = wholegraph_dtype_get_element_size(id->dtype);
  if (entry_count == 0 || dim == 0) return WHOLEGRAPH_SUCCESS;
  wgb::temp_buffer tmp(env);
  void* t        = tmp.device(static_cast<size_t>(entry_count * dim), id->dtype);
  const void* in = wholegraph_tensor_get_data_pointer(input_tensor);
  switch (id->dtype) {
    case WHOLEGRAPH_DT_FLOAT: run_native<float>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_DOUBLE: run_native<double>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_HALF: run_via_float<__half>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_BF16: run_via_float<__nv_bfloat16>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_INT: run_native<int32_t>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_INT64: run_native<int64_t>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_INT16: run_native<int16_t>(in, t, dim, entry_count, dim, stream); break;
    case WHOLEGRAPH_DT_INT8: run_native<int8_t>(in, t, dim, entry_count, dim, stream); break;
    default: return WHOLEGRAPH_INVALID_INPUT;
  }
  wgb::count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
  const size_t row_bytes = static_cast<size_t>(dim) * es;
  WGB_CUDA_CHECK(cudaMemcpy2DAsync(wholegraph_tensor_get_data_pointer(output_fixed_tensor),
                                   static_cast<size_t>(od->strides[0]) * es, t, row_bytes, row_bytes,
                                   static_cast<size_t>(entry_count), cudaMemcpyDeviceToDevice, stream));
  wholegraph_tensor_description_t vd = *od;
  vd.strides[0]                       = dim;
  vd.storage_offset                   = 0;
  auto variable_output = [&](void* handle, wholegraph_memory_allocation_type_t where) {
    if (handle == nullptr) return;
    void* p = env->output_fns.malloc_fn(&vd, where, handle, env->output_fns.global_context);
    if (p == nullptr) throw std::bad_alloc();
    WGB_CUDA_CHECK(cudaMemcpyAsync(p, t, row_bytes * entry_count, cudaMemcpyDefault, stream));
  };
  variable_output(out_device_handle, WHOLEGRAPH_MA_DEVICE);
  variable_output(out_pinned_handle, WHOLEGRAPH_MA_PINNED);
  variable_output(out_host_handle, WHOLEGRAPH_MA_HOST);
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));  // host outputs are read right after the call
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_env_test_op")
}
