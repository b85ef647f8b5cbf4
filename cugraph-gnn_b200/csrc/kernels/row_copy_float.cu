// Row copy kernels that cast between floating point types (fp32, fp16, fp64, bf16).
#include "row_copy.cuh"

namespace wgb {

namespace {

template <typename From, typename To, int EPV, bool CHUNKED>
row_copy_kernel_fn pick()
{
  if constexpr (sizeof(From) * EPV <= 16 && sizeof(To) * EPV <= 16) {
    return row_copy_kernel<sizeof(From) * EPV, sizeof(To) * EPV, vector_cast<From, To, EPV>, CHUNKED>;
  } else {
    return nullptr;
  }
}

template <typename From, typename To>
row_copy_kernel_fn by_width(int epv, bool chunked)
{
#define WGB_CASE(N)  \
  case N: return chunked ? pick<From, To, N, true>() : pick<From, To, N, false>();
  switch (epv) {
    WGB_CASE(1)
    WGB_CASE(2)
    WGB_CASE(4)
    WGB_CASE(8)
    default: return nullptr;
  }
#undef WGB_CASE
}

template <typename From>
row_copy_kernel_fn by_target(wholegraph_dtype_t to, int epv, bool chunked)
{
  switch (to) {
    case WHOLEGRAPH_DT_FLOAT: return by_width<From, float>(epv, chunked);
    case WHOLEGRAPH_DT_HALF: return by_width<From, __half>(epv, chunked);
    case WHOLEGRAPH_DT_DOUBLE: return by_width<From, double>(epv, chunked);
    case WHOLEGRAPH_DT_BF16: return by_width<From, __nv_bfloat16>(epv, chunked);
    default: return nullptr;
  }
}

}  // namespace

row_copy_kernel_fn float_cast_kernel(wholegraph_dtype_t from, wholegraph_dtype_t to, int epv,
                                     bool chunked)
{
  switch (from) {
    case WHOLEGRAPH_DT_FLOAT: return by_target<float>(to, epv, chunked);
    case WHOLEGRAPH_DT_HALF: return by_target<__half>(to, epv, chunked);
    case WHOLEGRAPH_DT_DOUBLE: return by_target<double>(to, epv, chunked);
    case WHOLEGRAPH_DT_BF16: return by_target<__nv_bfloat16>(to, epv, chunked);
    default: return nullptr;
  }
}

}  // namespace wgb
