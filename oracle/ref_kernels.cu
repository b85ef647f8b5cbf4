// The reference's OWN device code, compiled from its sources where they lie, as a GPU-side
// cross-check for the CPU oracle and for this repository's kernels.  TEST INFRASTRUCTURE ONLY:
// built into oracle/_ref/libwg_ref_kernels.so by `make -C oracle ref` when the reference checkout
// is present; nothing from the reference is copied into this repository.
//
// Included from the reference (paths relative to its cpp/src):
//   wholegraph_tensor_ops/functions/gather_scatter_func.cuh   gather_temp_func / scatter_temp_func
//   wholegraph_tensor_ops/functions/embedding_optimizer_func.cu  the four optimizer step kernels
//   wholegraph_tensor_ops/functions/exchange_embeddings_nccl_func.cu  dedup_indice_and_gradients
//   wholegraph_tensor_ops/thrust_allocator.cpp                 the allocator that function uses
// The wrappers below only pick template arguments and launch.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "wholegraph_tensor_ops/functions/gather_scatter_func.cuh"
#include "wholegraph_tensor_ops/functions/embedding_optimizer_func.cu"
#include "wholegraph_tensor_ops/functions/exchange_embeddings_nccl_func.cu"
#include "wholegraph_tensor_ops/thrust_allocator.cpp"

using namespace wholegraph_tensor_ops;

namespace {

wholegraph_matrix_description_t mat(int64_t rows, int64_t dim, int64_t stride, int64_t off, int dt)
{
  wholegraph_matrix_description_t d;
  d.sizes[0] = rows, d.sizes[1] = dim, d.stride = stride, d.storage_offset = off;
  d.dtype = static_cast<wholegraph_dtype_t>(dt);
  return d;
}

template <typename E, typename O>
int gather_idx(int idx64, wholegraph_gref_t g, wholegraph_matrix_description_t ed, void* idx, int64_t n,
               void* out, wholegraph_matrix_description_t od, cudaStream_t s)
{
  if (idx64)
    gather_temp_func<E, int64_t, O>(g, ed, idx, n, false, nullptr, out, od, s, -1);
  else
    gather_temp_func<E, int, O>(g, ed, idx, n, false, nullptr, out, od, s, -1);
  return 0;
}
template <typename I, typename E>
int scatter_idx(int idx64, const void* in, wholegraph_matrix_description_t id, void* idx, int64_t n,
                wholegraph_gref_t g, wholegraph_matrix_description_t ed, cudaStream_t s)
{
  if (idx64)
    scatter_temp_func<I, int64_t, E>(in, id, idx, n, g, ed, s, -1);
  else
    scatter_temp_func<I, int, E>(in, id, idx, n, g, ed, s, -1);
  return 0;
}

}  // namespace

// dtype codes are wholegraph_dtype_t: 1 fp32, 2 fp16, 4 bf16.
#define WGREF_PAIRS(X)                                                                       \
  X(1, 1, float, float) X(1, 2, float, __half) X(1, 4, float, __nv_bfloat16)                 \
  X(2, 1, __half, float) X(2, 2, __half, __half) X(2, 4, __half, __nv_bfloat16)              \
  X(4, 1, __nv_bfloat16, float) X(4, 2, __nv_bfloat16, __half) X(4, 4, __nv_bfloat16, __nv_bfloat16)

extern "C" int wgref_gather(void* table, int tab_dt, int64_t rows, int64_t dim, int64_t tab_stride,
                            int64_t tab_off, void* idx, int idx64, int64_t n, void* out, int out_dt,
                            int64_t out_stride, int64_t out_off, void* stream)
{
  try {
    wholegraph_gref_t g{table};
    auto ed = mat(rows, dim, tab_stride, tab_off, tab_dt);
    auto od = mat(n, dim, out_stride, out_off, out_dt);
    auto s  = static_cast<cudaStream_t>(stream);
#define X(A, B, TA, TB) \
  if (tab_dt == A && out_dt == B) return gather_idx<TA, TB>(idx64, g, ed, idx, n, out, od, s);
    WGREF_PAIRS(X)
#undef X
    return -2;
  } catch (...) {
    return -1;
  }
}

extern "C" int wgref_scatter(const void* in, int in_dt, int64_t dim, int64_t in_stride, int64_t in_off,
                             void* idx, int idx64, int64_t n, void* table, int tab_dt, int64_t rows,
                             int64_t tab_stride, int64_t tab_off, void* stream)
{
  try {
    wholegraph_gref_t g{table};
    auto id = mat(n, dim, in_stride, in_off, in_dt);
    auto ed = mat(rows, dim, tab_stride, tab_off, tab_dt);
    auto s  = static_cast<cudaStream_t>(stream);
#define X(A, B, TA, TB) \
  if (in_dt == A && tab_dt == B) return scatter_idx<TA, TB>(idx64, in, id, idx, n, g, ed, s);
    WGREF_PAIRS(X)
#undef X
    return -2;
  } catch (...) {
    return -1;
  }
}

// One optimizer step on already-deduplicated int64 ids with fp32 gradients [n, grad_stride]:
// opt codes are wholegraph_optimizer_type_t (1 SGD, 2 Lazy Adam, 3 RMSProp, 4 AdaGrad).
template <typename E>
static int optimizer_step(int opt, const int64_t* ids, const float* grads, int64_t n, E* w, float* state,
                          float* beta12t, int64_t local_start, int dim, int grad_stride, int w_stride,
                          float lr, float wd, float eps, float b1, float b2, float alpha, int adam_w,
                          cudaStream_t s)
{
  int threads = (dim + 3) / 4;
  threads     = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  if (n == 0) return 0;
  switch (opt) {
    case 1:
      sgd_optimizer_step_kernel<int64_t, E, false><<<n, threads, 0, s>>>(
        ids, grads, w, nullptr, nullptr, local_start, dim, grad_stride, w_stride, 0, wd, lr);
      break;
    case 2:
      if (adam_w)
        lazy_adam_optimizer_step_kernel<int64_t, E, false, true><<<n, threads, 0, s>>>(
          ids, grads, w, nullptr, nullptr, state, nullptr, nullptr, beta12t, local_start, dim, grad_stride,
          w_stride, 0, wd, eps, b1, b2, lr);
      else
        lazy_adam_optimizer_step_kernel<int64_t, E, false, false><<<n, threads, 0, s>>>(
          ids, grads, w, nullptr, nullptr, state, nullptr, nullptr, beta12t, local_start, dim, grad_stride,
          w_stride, 0, wd, eps, b1, b2, lr);
      break;
    case 3:
      rms_prop_optimizer_step_kernel<int64_t, E, false><<<n, threads, 0, s>>>(
        ids, grads, w, nullptr, nullptr, state, nullptr, nullptr, local_start, dim, grad_stride, w_stride, 0,
        wd, eps, alpha, lr);
      break;
    case 4:
      ada_grad_optimizer_step_kernel<int64_t, E, false><<<n, threads, 0, s>>>(
        ids, grads, w, nullptr, nullptr, state, nullptr, nullptr, local_start, dim, grad_stride, w_stride, 0,
        wd, eps, lr);
      break;
    default: return -2;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int wgref_optimizer_step(int opt, const int64_t* ids, const float* grads, int64_t n, void* w,
                                    int w_dt, float* state, float* beta12t, int64_t local_start, int dim,
                                    int grad_stride, int w_stride, float lr, float wd, float eps, float b1,
                                    float b2, float alpha, int adam_w, void* stream)
{
  auto s = static_cast<cudaStream_t>(stream);
  if (w_dt == 1)
    return optimizer_step<float>(opt, ids, grads, n, static_cast<float*>(w), state, beta12t, local_start, dim,
                                 grad_stride, w_stride, lr, wd, eps, b1, b2, alpha, adam_w, s);
  if (w_dt == 2)
    return optimizer_step<__half>(opt, ids, grads, n, static_cast<__half*>(w), state, beta12t, local_start, dim,
                                  grad_stride, w_stride, lr, wd, eps, b1, b2, alpha, adam_w, s);
  if (w_dt == 4)
    return optimizer_step<__nv_bfloat16>(opt, ids, grads, n, static_cast<__nv_bfloat16*>(w), state, beta12t,
                                         local_start, dim, grad_stride, w_stride, lr, wd, eps, b1, b2, alpha,
                                         adam_w, s);
  return -2;
}

// The reference's duplicate-gradient reduction (sort by id, unique, one block per distinct id adding
// its rows one after the other): int64 ids, fp32 gradients [n, stride].  dedup_grads must hold
// n * stride floats (the reference strides its output like its input).  `env` is a
// wholegraph_env_func_t* whose temporary allocator serves the scratch.  Returns the number of
// distinct ids; the call synchronises the stream (thrust::unique_by_key returns to the host).
extern "C" long wgref_dedup_gradients(const int64_t* ids, int64_t n, const float* grads, int64_t dim,
                                      int64_t stride, int64_t* dedup_ids, float* dedup_grads, void* env,
                                      void* stream)
{
  wholegraph_array_description_t id;
  id.size = n, id.storage_offset = 0, id.dtype = WHOLEGRAPH_DT_INT64;
  auto gd = mat(n, dim, stride, 0, WHOLEGRAPH_DT_FLOAT);
  return dedup_indice_and_gradients(ids, id, grads, gd, dedup_ids, dedup_grads,
                                    static_cast<wholegraph_env_func_t*>(env), static_cast<cudaStream_t>(stream));
}

// The reference's launch wrappers (compiled above but never called here) name two tensor
// accessors of its runtime; give the loader something to bind them to.
extern "C" void* wholegraph_tensor_get_data_pointer(wholegraph_tensor_t) { abort(); }
extern "C" wholegraph_tensor_description_t* wholegraph_tensor_get_tensor_description(wholegraph_tensor_t)
{
  abort();
}
// Likewise for the row exchange that shares a file with the reduction: never called here.
extern "C" wholegraph_error_code_t wholegraph_communicator_get_size(int*, wholegraph_comm_t) { abort(); }
void wholegraph_comm_::alltoallv(const void*, void*, const size_t*, const size_t*, const size_t*, const size_t*,
                                 wholegraph_dtype_t, cudaStream_t) const
{
  ::abort();
}
