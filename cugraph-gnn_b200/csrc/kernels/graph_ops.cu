// append-unique by one radix sort and two scans, and the self-loop CSR rewrite.
//
// append-unique: positions 0..T-1 name the targets, T..T+N-1 the neighbours.  A stable sort of
// (id, position) puts equal ids side by side with the lowest position first, so a run of equal ids
// starts with a target if any target has that id.  Runs that start with a neighbour are the new
// nodes; an exclusive sum over those run heads numbers them in ascending id order, and an inclusive
// max-scan carries every element the index of its run's head.
#include "graph_ops.hpp"

#include <algorithm>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "../common.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads = 256;

template <typename K>
__global__ void pairs_kernel(const K* targets, int64_t t_count, const K* neighbors, int64_t n_count, K* keys,
                             int32_t* positions)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= t_count + n_count) return;
  keys[i]      = i < t_count ? targets[i] : neighbors[i - t_count];
  positions[i] = static_cast<int32_t>(i);
}

// head_index[i] = i at the first element of a run of equal ids, else 0 (a max-scan then gives every
// element its run's head); is_new[i] = 1 at heads whose first element is a neighbour.
template <typename K>
__global__ void heads_kernel(const K* keys, const int32_t* positions, int64_t m, int32_t t_count, int32_t* head_index,
                             int32_t* is_new)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const bool head = i == 0 || keys[i] != keys[i - 1];
  head_index[i]   = head ? static_cast<int32_t>(i) : 0;
  is_new[i]       = head && positions[i] >= t_count ? 1 : 0;
}

__global__ void count_kernel(const int32_t* is_new, const int32_t* new_rank, int64_t m, int* new_count)
{
  if (threadIdx.x == 0 && blockIdx.x == 0) *new_count = m > 0 ? new_rank[m - 1] + is_new[m - 1] : 0;
}

template <typename K>
__global__ void write_kernel(const K* keys, const int32_t* positions, const int32_t* head_index, const int32_t* is_new,
                             const int32_t* new_rank, int64_t m, int32_t t_count, K* unique_nodes, int* mapping)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const int32_t h      = head_index[i];  // after the max-scan: head of this element's run
  const int32_t first  = positions[h];
  const int32_t unique = first < t_count ? first : t_count + new_rank[h];
  if (h == i && is_new[i]) unique_nodes[unique] = keys[i];
  const int32_t pos = positions[i];
  if (mapping != nullptr && pos >= t_count) mapping[pos - t_count] = unique;
}

struct max_op {
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t b) const { return a > b ? a : b; }
};

struct layout {
  size_t keys_in, keys_out, pos_in, pos_out, head_index, is_new, new_rank, cub, cub_bytes, total;
};

template <typename K>
layout layout_for(int64_t m)
{
  layout l{};
  auto align       = [](size_t x) { return (x + 255) / 256 * 256; };
  const size_t cnt = static_cast<size_t>(std::max<int64_t>(m, 1));
  size_t off       = 0;
  l.keys_in = off, off += align(cnt * sizeof(K));
  l.keys_out = off, off += align(cnt * sizeof(K));
  l.pos_in = off, off += align(cnt * 4);
  l.pos_out = off, off += align(cnt * 4);
  l.head_index = off, off += align(cnt * 4);
  l.is_new = off, off += align(cnt * 4);
  l.new_rank = off, off += align(cnt * 4);
  size_t a = 0, b = 0, c = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, static_cast<const K*>(nullptr), static_cast<K*>(nullptr),
                                  static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                  static_cast<int>(cnt));
  cub::DeviceScan::ExclusiveSum(nullptr, b, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                static_cast<int>(cnt));
  cub::DeviceScan::InclusiveScan(nullptr, c, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                 max_op{}, static_cast<int>(cnt));
  l.cub_bytes = std::max(a, std::max(b, c));
  l.cub = off, off += align(l.cub_bytes);
  l.total = off;
  return l;
}

unsigned blocks_for(int64_t n) { return static_cast<unsigned>((n + kThreads - 1) / kThreads); }

template <typename K>
void group_typed(const void* targets, int64_t t_count, const void* neighbors, int64_t n_count, void* workspace,
                 int* new_count, cudaStream_t stream)
{
  const int64_t m = t_count + n_count;
  const layout l  = layout_for<K>(m);
  char* ws        = static_cast<char*>(workspace);
  auto* keys_in   = reinterpret_cast<K*>(ws + l.keys_in);
  auto* keys_out  = reinterpret_cast<K*>(ws + l.keys_out);
  auto* pos_in    = reinterpret_cast<int32_t*>(ws + l.pos_in);
  auto* pos_out   = reinterpret_cast<int32_t*>(ws + l.pos_out);
  auto* head      = reinterpret_cast<int32_t*>(ws + l.head_index);
  auto* is_new    = reinterpret_cast<int32_t*>(ws + l.is_new);
  auto* new_rank  = reinterpret_cast<int32_t*>(ws + l.new_rank);
  if (m > 0) {
    pairs_kernel<K><<<blocks_for(m), kThreads, 0, stream>>>(static_cast<const K*>(targets), t_count,
                                                           static_cast<const K*>(neighbors), n_count, keys_in, pos_in);
    size_t bytes = l.cub_bytes;
    WGB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(ws + l.cub, bytes, keys_in, keys_out, pos_in, pos_out,
                                                   static_cast<int>(m), 0, static_cast<int>(sizeof(K) * 8), stream));
    heads_kernel<K><<<blocks_for(m), kThreads, 0, stream>>>(keys_out, pos_out, m, static_cast<int32_t>(t_count), head,
                                                           is_new);
    bytes = l.cub_bytes;
    WGB_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(ws + l.cub, bytes, is_new, new_rank, static_cast<int>(m), stream));
    bytes = l.cub_bytes;
    WGB_CUDA_CHECK(cub::DeviceScan::InclusiveScan(ws + l.cub, bytes, head, head, max_op{}, static_cast<int>(m), stream));
  }
  count_kernel<<<1, 32, 0, stream>>>(is_new, new_rank, m, new_count);
  count_kernel_launch(6);
  WGB_LAUNCH_CHECK(stream);
}

template <typename K>
void write_typed(const void* targets, int64_t t_count, int64_t n_count, void* workspace, void* unique_nodes,
                 int* mapping, cudaStream_t stream)
{
  const int64_t m = t_count + n_count;
  const layout l  = layout_for<K>(m);
  char* ws        = static_cast<char*>(workspace);
  if (t_count > 0)
    WGB_CUDA_CHECK(cudaMemcpyAsync(unique_nodes, targets, static_cast<size_t>(t_count) * sizeof(K),
                                   cudaMemcpyDeviceToDevice, stream));
  if (m == 0) return;
  write_kernel<K><<<blocks_for(m), kThreads, 0, stream>>>(
    reinterpret_cast<const K*>(ws + l.keys_out), reinterpret_cast<const int32_t*>(ws + l.pos_out),
    reinterpret_cast<const int32_t*>(ws + l.head_index), reinterpret_cast<const int32_t*>(ws + l.is_new),
    reinterpret_cast<const int32_t*>(ws + l.new_rank), m, static_cast<int32_t>(t_count),
    static_cast<K*>(unique_nodes), mapping);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

// One warp per row.
__global__ void __launch_bounds__(kThreads) self_loop_kernel(const int* row_ptr, const int* col, int64_t rows,
                                                             int* out_row_ptr, int* out_col)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r = warp_global; r < rows; r += warp_stride) {
    const int begin = row_ptr[r], end = row_ptr[r + 1];
    const int out   = begin + static_cast<int>(r);
    if (lane == 0) {
      out_row_ptr[r] = out;
      out_col[out]   = static_cast<int>(r);
      if (r == rows - 1) out_row_ptr[rows] = end + static_cast<int>(rows);
    }
    for (int k = begin + lane; k < end; k += 32) out_col[k + r + 1] = col[k];
  }
}

}  // namespace

size_t append_unique_workspace_bytes(int64_t target_count, int64_t neighbor_count, bool ids_are_64)
{
  const int64_t m = target_count + neighbor_count;
  return ids_are_64 ? layout_for<int64_t>(m).total : layout_for<int32_t>(m).total;
}

void append_unique_group(const void* targets, int64_t target_count, const void* neighbors, int64_t neighbor_count,
                         bool ids_are_64, void* workspace, int* new_count, cudaStream_t stream)
{
  WGB_EXPECTS(target_count + neighbor_count < (int64_t(1) << 31), "node lists of %ld entries are too long",
              (long)(target_count + neighbor_count));
  if (ids_are_64)
    group_typed<int64_t>(targets, target_count, neighbors, neighbor_count, workspace, new_count, stream);
  else
    group_typed<int32_t>(targets, target_count, neighbors, neighbor_count, workspace, new_count, stream);
}

void append_unique_write(const void* targets, int64_t target_count, int64_t neighbor_count, bool ids_are_64,
                         void* workspace, void* unique_nodes, int* mapping, cudaStream_t stream)
{
  if (ids_are_64)
    write_typed<int64_t>(targets, target_count, neighbor_count, workspace, unique_nodes, mapping, stream);
  else
    write_typed<int32_t>(targets, target_count, neighbor_count, workspace, unique_nodes, mapping, stream);
}

void csr_add_self_loops(const int* row_ptr, const int* col, int64_t rows, int* out_row_ptr, int* out_col,
                        cudaStream_t stream)
{
  if (rows <= 0) return;
  const int64_t ctas = std::min<int64_t>((rows + 7) / 8, 148 * 16);
  self_loop_kernel<<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(row_ptr, col, rows, out_row_ptr, out_col);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
