// Row copy kernels that cast between integer types (int8, int16, int32, int64).
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
    WGB_CASE(16)
    default: return nullptr;
  }
#undef WGB_CASE
}

template <typename From>
row_copy_kernel_fn by_target(wholegraph_dtype_t to, int epv, bool chunked)
{
  switch (to) {
    case WHOLEGRAPH_DT_INT: return by_width<From, int32_t>(epv, chunked);
    case WHOLEGRAPH_DT_INT64: return by_width<From, int64_t>(epv, chunked);
    case WHOLEGRAPH_DT_INT16: return by_width<From, int16_t>(epv, chunked);
    case WHOLEGRAPH_DT_INT8: return by_width<From, int8_t>(epv, chunked);
    default: return nullptr;
  }
}

}  // namespace

row_copy_kernel_fn int_cast_kernel(wholegraph_dtype_t from, wholegraph_dtype_t to, int epv,
                                     bool chunked)
{
  switch (from) {
    case WHOLEGRAPH_DT_INT: return by_target<int32_t>(to, epv, chunked);
    case WHOLEGRAPH_DT_INT64: return by_target<int64_t>(to, epv, chunked);
    case WHOLEGRAPH_DT_INT16: return by_target<int16_t>(to, epv, chunked);
    case WHOLEGRAPH_DT_INT8: return by_target<int8_t>(to, epv, chunked);
    default: return nullptr;
  }
}

}  // namespace wgb
