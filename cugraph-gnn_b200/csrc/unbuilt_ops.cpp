// Entry points of the reference ABI that lie outside the embedding path (graph sampling and the
// host restatements of its random streams; cpp/include/wholegraph/wholegraph_op.h).  They are
// exported so that bindings built against the reference's headers resolve every symbol, and they
// refuse loudly: nothing is computed, on any device or on the host.
#include <wholegraph/wholegraph_op.h>

#include "common.hpp"

namespace {
wholegraph_error_code_t refuse(const char* name)
{
  WGB_ERROR("%s is not built in this library (only the embedding gather / scatter / optimizer path is)", name);
  return WHOLEGRAPH_NOT_IMPLEMENTED;
}
}  // namespace

extern "C" {

wholegraph_error_code_t wholegraph_csr_unweighted_sample_without_replacement(
  wholegraph_tensor_t, wholegraph_tensor_t, wholegraph_tensor_t, int, wholegraph_tensor_t, void*, void*, void*,
  unsigned long long, wholegraph_env_func_t*, void*)
{
  return refuse("wholegraph_csr_unweighted_sample_without_replacement");
}

wholegraph_error_code_t wholegraph_csr_weighted_sample_without_replacement(
  wholegraph_tensor_t, wholegraph_tensor_t, wholegraph_tensor_t, wholegraph_tensor_t, int, wholegraph_tensor_t, void*,
  void*, void*, unsigned long long, wholegraph_env_func_t*, void*)
{
  return refuse("wholegraph_csr_weighted_sample_without_replacement");
}

wholegraph_error_code_t generate_random_positive_int_cpu(int64_t, int64_t, wholegraph_tensor_t)
{
  return refuse("generate_random_positive_int_cpu");
}

wholegraph_error_code_t generate_exponential_distribution_negative_float_cpu(int64_t, int64_t, wholegraph_tensor_t)
{
  return refuse("generate_exponential_distribution_negative_float_cpu");
}

}  // extern "C"
