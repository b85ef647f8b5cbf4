// Same-dtype row copies (raw byte vectors) and the host-side launcher of all row copy kernels.
#include "row_copy.cuh"

#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "../common.hpp"

namespace wgb {

row_copy_kernel_fn same_type_kernel(int vector_bytes, bool chunked)
{
#define WGB_CASE(N)                                                             \
  case N:                                                                       \
    return chunked ? row_copy_kernel<N, N, raw_copy<N>, true>                   \
                   : row_copy_kernel<N, N, raw_copy<N>, false>;
  switch (vector_bytes) {
    WGB_CASE(1)
    WGB_CASE(2)
    WGB_CASE(4)
    WGB_CASE(8)
    WGB_CASE(16)
    default: return nullptr;
  }
#undef WGB_CASE
}

static std::atomic<unsigned long long> g_launches{0};
unsigned long long kernel_launch_count() { return g_launches.load(); }
void count_kernel_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n)); }

int row_copy_vector_elements(const row_copy_args& a)
{
  const int64_t es_src = static_cast<int64_t>(wholegraph_dtype_get_element_size(a.src_dt));
  const int64_t es_dst = static_cast<int64_t>(wholegraph_dtype_get_element_size(a.dst_dt));
  int epv              = static_cast<int>(16 / std::max(es_src, es_dst));
  // First-element addresses in units of elements.  Chunked tables are allocations of their
  // own (256-byte aligned), so only the storage offset matters on that side.
  auto first_elt = [](const void* p, int64_t es, int64_t off, bool chunked_side) -> int64_t {
    int64_t addr = chunked_side ? 0 : reinterpret_cast<intptr_t>(p);
    return addr / es + off;
  };
  // A side addressed row by row (chunked table or explicit addresses) contributes only its
  // offset and stride: its rows are allocations or lines aligned to their stride.
  const bool src_chunked = (a.chunks.ranks > 0 && a.src_select == ROW_BY_INDEX) || a.src_select == ROW_BY_ADDRESS;
  const bool dst_chunked = (a.chunks.ranks > 0 && a.dst_select == ROW_BY_INDEX) || a.dst_select == ROW_BY_ADDRESS;
  const int64_t s0       = first_elt(a.src, es_src, a.src_offset, src_chunked);
  const int64_t d0       = first_elt(a.dst, es_dst, a.dst_offset, dst_chunked);
  for (; epv > 1; epv /= 2) {
    if (a.dim % epv == 0 && a.src_stride % epv == 0 && a.dst_stride % epv == 0 && s0 % epv == 0 &&
        d0 % epv == 0)
      break;
  }
  return epv;
}

void launch_row_copy(const row_copy_args& a, cudaStream_t stream)
{
  const bool src_f = wholegraph_dtype_is_floating_number(a.src_dt);
  const bool dst_f = wholegraph_dtype_is_floating_number(a.dst_dt);
  const bool src_i = wholegraph_dtype_is_integer_number(a.src_dt);
  const bool dst_i = wholegraph_dtype_is_integer_number(a.dst_dt);
  WGB_EXPECTS((src_f && dst_f) || (src_i && dst_i),
              "row copy between dtype %d and dtype %d is not supported", (int)a.src_dt,
              (int)a.dst_dt);
  if (a.count == 0 || a.dim == 0) return;
  if (a.src_select == ROW_BY_ADDRESS || a.dst_select == ROW_BY_ADDRESS) {
    // Rows named by address: same kernel, with "row number" = address, stride 1 byte and the
    // storage offset as base.  Alignment comes from the stated stride and offset.
    WGB_EXPECTS(a.indices != nullptr && a.indices_are_64 && a.chunks.ranks == 0 &&
                  !(a.src_select == ROW_BY_ADDRESS && a.dst_select == ROW_BY_ADDRESS),
                "bad by-address row copy");
  }
  const bool need_index = a.src_select == ROW_BY_INDEX || a.dst_select == ROW_BY_INDEX ||
                          a.src_select == ROW_BY_ADDRESS || a.dst_select == ROW_BY_ADDRESS;
  const bool need_pos   = a.src_select == ROW_BY_POSITION || a.dst_select == ROW_BY_POSITION;
  WGB_EXPECTS(!need_index || a.indices != nullptr, "row copy by index without indices");
  WGB_EXPECTS(!need_pos || a.positions != nullptr, "row copy by position without positions");
  const bool chunked = a.chunks.ranks > 0;
  WGB_EXPECTS(!chunked || (need_index && a.chunks.ranks <= kMaxChunkedRanks), "bad chunk table");

  const int64_t es_src = static_cast<int64_t>(wholegraph_dtype_get_element_size(a.src_dt));
  const int64_t es_dst = static_cast<int64_t>(wholegraph_dtype_get_element_size(a.dst_dt));
  const int epv        = row_copy_vector_elements(a);

  row_copy_kernel_fn fn = nullptr;
  if (a.src_dt == a.dst_dt)
    fn = same_type_kernel(static_cast<int>(es_src) * epv, chunked);
  else if (src_f)
    fn = float_cast_kernel(a.src_dt, a.dst_dt, epv, chunked);
  else
    fn = int_cast_kernel(a.src_dt, a.dst_dt, epv, chunked);
  WGB_EXPECTS(fn != nullptr, "no row copy kernel for dtypes %d -> %d at %d elements per vector",
              (int)a.src_dt, (int)a.dst_dt, epv);

  row_copy_params p;
  p.src              = static_cast<const char*>(a.src) + a.src_offset * es_src;
  p.dst              = static_cast<char*>(a.dst) + a.dst_offset * es_dst;
  p.src_stride_bytes = a.src_stride * es_src;
  p.dst_stride_bytes = a.dst_stride * es_dst;
  p.indices          = a.indices;
  p.positions        = a.positions;
  p.count            = a.count;
  p.vectors_per_row  = static_cast<int>((a.dim + epv - 1) / epv);
  int lpr            = 1;
  while (lpr < 32 && lpr < p.vectors_per_row) lpr *= 2;
  p.lanes_per_row      = lpr;
  p.src_select         = a.src_select;
  p.dst_select         = a.dst_select;
  if (a.src_select == ROW_BY_ADDRESS) {
    p.src              = reinterpret_cast<const char*>(a.src_offset * es_src);
    p.src_stride_bytes = 1;
    p.src_select       = ROW_BY_INDEX;
  }
  if (a.dst_select == ROW_BY_ADDRESS) {
    p.dst              = reinterpret_cast<char*>(a.dst_offset * es_dst);
    p.dst_stride_bytes = 1;
    p.dst_select       = ROW_BY_INDEX;
  }
  p.indices_are_64     = a.indices_are_64 ? 1 : 0;
  p.chunks             = a.chunks;
  p.segments           = a.segments;
  WGB_EXPECTS(a.segments.n == 0 || a.segments.total() == a.count, "segment list does not add up to count");
  p.chunk_offset_bytes = 0;
  if (chunked)
    p.chunk_offset_bytes = a.src_select == ROW_BY_INDEX ? a.src_offset * es_src : a.dst_offset * es_dst;

  // One warp tile per warp unless that exceeds a few waves of the machine; then grid-stride.
  static int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  const int ctas_per_sm = 2048 / kRowCopyThreads;
  const int64_t tiles   = (a.count + kRowCopyTile - 1) / kRowCopyTile;
  int64_t ctas          = (tiles + kRowCopyWarps - 1) / kRowCopyWarps;
  const int64_t cap     = static_cast<int64_t>(sm_count) * ctas_per_sm * 32;
  if (ctas > cap) ctas = cap;
  if (a.sm_hint > 0) ctas = std::min<int64_t>(ctas, static_cast<int64_t>(a.sm_hint) * ctas_per_sm);
  if (ctas < 1) ctas = 1;

  fn<<<static_cast<unsigned>(ctas), kRowCopyThreads, 0, stream>>>(p);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
