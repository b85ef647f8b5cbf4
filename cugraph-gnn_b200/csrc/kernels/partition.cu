// Stable partition of a request list by owning rank ("bucketed sort-by-owner").
//
// Replaces the reference's owner histogram (cpp/src/wholegraph_tensor_ops/functions/
// bucket_ids_func.cu:21-129) and its full-width radix sort of (id, position) pairs
// (exchange_ids_nccl_func.cu:32-104): shards are contiguous row ranges, so grouping ids by
// owner while keeping arrival order inside a group yields the same exchange as sorting by id,
// in three small kernels and 2 passes over the ids instead of a 64-bit radix sort.
//
//   1. partition_count_kernel   per-CTA owner histogram
//   2. partition_scan_kernel    exclusive scan of the owner-major histogram -> CTA bases, totals
//   3. partition_scatter_kernel stable placement of (id, position) into owner buckets
#include "partition.hpp"

#include <algorithm>
#include <mutex>

#include "../common.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads      = 256;
constexpr int kWarps        = kThreads / 32;
constexpr int kItems        = 8;                  // ids per thread
constexpr int kTile         = kThreads * kItems;  // ids per CTA
constexpr int kSlots        = kItems * kWarps;    // (item, warp) pairs, in list order
constexpr int kScanThreads  = 1024;

struct owner_table {
  int world;
  int64_t per_rank_estimate;
  int64_t first_row[kMaxPartitionRanks + 1];
};

// Owner of `id`: the last rank whose first row is <= id.  Returns `world` for ids that no
// rank owns (negative or past the end); those are dropped.
__device__ __forceinline__ int owner_of(int64_t id, const int64_t* first_row, int world,
                                        int64_t per_rank_estimate)
{
  if (id < 0 || id >= first_row[world]) return world;
  int r = static_cast<int>(id / per_rank_estimate);
  if (r > world - 1) r = world - 1;
  while (r > 0 && first_row[r] > id) r--;
  while (r + 1 < world && first_row[r + 1] <= id) r++;
  return r;
}

__device__ __forceinline__ int64_t load_id(const void* ids, int is64, int64_t i)
{
  return is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
              : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
}

__global__ void __launch_bounds__(kThreads)
  partition_count_kernel(const void* ids, int is64, int64_t n, owner_table t, int* cta_hist,
                         int num_ctas)
{
  __shared__ int64_t s_first[kMaxPartitionRanks + 1];
  __shared__ int s_hist[kMaxPartitionRanks + 1];
  for (int i = threadIdx.x; i <= t.world; i += kThreads) {
    s_first[i] = t.first_row[i];
    s_hist[i]  = 0;
  }
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  const int lane     = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < kItems; j++) {
    const int64_t i = base + j * kThreads + threadIdx.x;
    int owner       = t.world;
    if (i < n) owner = owner_of(load_id(ids, is64, i), s_first, t.world, t.per_rank_estimate);
    const unsigned peers = __match_any_sync(0xffffffffu, owner);
    if (owner < t.world && lane == __ffs(peers) - 1) atomicAdd(&s_hist[owner], __popc(peers));
  }
  __syncthreads();
  for (int o = threadIdx.x; o < t.world; o += kThreads)
    cta_hist[static_cast<int64_t>(o) * num_ctas + blockIdx.x] = s_hist[o];
}

// In-place exclusive scan of `hist` (owner-major, `total` = world * num_ctas entries) by one CTA.
__global__ void __launch_bounds__(kScanThreads) partition_scan_kernel(int* hist, int64_t total)
{
  __shared__ int64_t s_warp[kScanThreads / 32];
  const int64_t chunk = (total + kScanThreads - 1) / kScanThreads;
  const int64_t lo    = min(total, chunk * static_cast<int64_t>(threadIdx.x));
  const int64_t hi    = min(total, lo + chunk);
  int64_t sum         = 0;
  for (int64_t i = lo; i < hi; i++) sum += hist[i];
  // block-wide exclusive scan of the per-thread sums
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t incl   = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int64_t v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int64_t w = s_warp[lane];
    int64_t x = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int64_t v = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += v;
    }
    s_warp[lane] = x - w;  // exclusive
  }
  __syncthreads();
  int64_t run = s_warp[warp] + incl - sum;
  for (int64_t i = lo; i < hi; i++) {
    int v   = hist[i];
    hist[i] = static_cast<int>(run);
    run += v;
  }
}

__global__ void __launch_bounds__(kThreads)
  partition_scatter_kernel(const void* ids, int is64, int64_t n, owner_table t,
                           const int* cta_base, int num_ctas, int64_t* sorted_ids,
                           int64_t* positions)
{
  __shared__ int64_t s_first[kMaxPartitionRanks + 1];
  __shared__ int s_slot[kSlots][kMaxPartitionRanks];
  for (int i = threadIdx.x; i <= t.world; i += kThreads) s_first[i] = t.first_row[i];
  for (int i = threadIdx.x; i < kSlots * kMaxPartitionRanks; i += kThreads)
    (&s_slot[0][0])[i] = 0;
  __syncthreads();

  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t id[kItems];
  int owner[kItems];
  int rank_in_warp[kItems];
#pragma unroll
  for (int j = 0; j < kItems; j++) {
    const int64_t i = base + j * kThreads + threadIdx.x;
    owner[j]        = t.world;
    id[j]           = -1;
    if (i < n) {
      id[j]    = load_id(ids, is64, i);
      owner[j] = owner_of(id[j], s_first, t.world, t.per_rank_estimate);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, owner[j]);
    rank_in_warp[j]      = __popc(peers & ((1u << lane) - 1u));
    if (owner[j] < t.world && rank_in_warp[j] == 0) s_slot[j * kWarps + warp][owner[j]] = __popc(peers);
  }
  __syncthreads();
  // Per owner: running offset over the (item, warp) slots, which is list order inside the tile.
  for (int o = threadIdx.x; o < t.world; o += kThreads) {
    int run = cta_base[static_cast<int64_t>(o) * num_ctas + blockIdx.x];
    for (int s = 0; s < kSlots; s++) {
      const int c  = s_slot[s][o];
      s_slot[s][o] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kItems; j++) {
    if (owner[j] < t.world) {
      const int64_t dst = s_slot[j * kWarps + warp][owner[j]] + rank_in_warp[j];
      sorted_ids[dst]   = id[j];
      positions[dst]    = base + j * kThreads + threadIdx.x;
    }
  }
}

// counts / starts from the scanned histogram and the raw histogram of the LAST CTA column.
__global__ void partition_totals_kernel(const int* scanned, const int* last_column_raw, int world,
                                        int num_ctas, int64_t* counts, int64_t* starts)
{
  const int o = threadIdx.x;
  if (o >= world) return;
  const int64_t begin = scanned[static_cast<int64_t>(o) * num_ctas];
  int64_t end;
  if (o + 1 < world) {
    end = scanned[static_cast<int64_t>(o + 1) * num_ctas];
  } else {
    end = static_cast<int64_t>(scanned[static_cast<int64_t>(world) * num_ctas - 1]) + last_column_raw[0];
  }
  counts[o] = end - begin;
  starts[o] = begin;
}

// Save the raw count of the very last histogram entry before the scan overwrites it.
__global__ void partition_save_last_kernel(const int* hist, int64_t total, int* out)
{
  out[0] = hist[total - 1];
}

}  // namespace

// Built-in scratch of the allocation-free entry point.  It lives in every GPU context that loads
// this library, from load until exit.  In host code this name is only a handle for the runtime
// (cudaGetSymbolAddress); it is not an address a kernel could be given.
constexpr size_t kBuiltinScratchBytes = 66048;  // 64.5 KiB: 4,194,304 ids at 8 ranks
static __device__ __align__(256) unsigned char g_builtin_partition_scratch[kBuiltinScratchBytes];

// Device address of the built-in scratch on the current device, looked up once per device.
static void* builtin_scratch_of_current_device()
{
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* address[kMaxDevices] = {};
  int dev = -1;
  WGB_CUDA_CHECK(cudaGetDevice(&dev));
  WGB_EXPECTS(dev >= 0 && dev < kMaxDevices, "device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (address[dev] == nullptr) {
    void* p = nullptr;
    WGB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_builtin_partition_scratch));
    address[dev] = p;
  }
  return address[dev];
}

size_t partition_builtin_scratch_bytes() { return kBuiltinScratchBytes; }

void partition_by_owner_builtin_scratch(const void* ids, bool ids_are_64, int64_t n,
                                        const int64_t* first_row, int world, int64_t* sorted_ids,
                                        int64_t* positions, int64_t* counts, int64_t* starts,
                                        cudaStream_t stream)
{
  WGB_EXPECTS(world >= 1 && world <= kMaxPartitionRanks, "world size %d exceeds %d", world,
              kMaxPartitionRanks);
  check_owner_table(first_row, world);
  const size_t need = partition_workspace_bytes(n, world);
  if (need > kBuiltinScratchBytes) {
    throw invalid_input(WHOLEGRAPH_INVALID_VALUE,
                        format_string("%ld ids over %d ranks need %zu bytes of scratch, the built-in "
                                      "scratch holds %zu; use the entry point that takes a workspace",
                                      (long)n, world, need, kBuiltinScratchBytes));
  }
  // Every scratch word the kernels read is written earlier in the same call, so nothing has to
  // be cleared between calls.
  partition_by_owner(ids, ids_are_64, n, first_row, world, builtin_scratch_of_current_device(),
                     sorted_ids, positions, counts, starts, stream);
}

void check_owner_table(const int64_t* first_row, int world)
{
  // The kernels walk the table from an estimate towards the owner; a table that does not start
  // at row 0 or is out of order would send that walk outside it.
  bool ok = first_row[0] == 0;
  for (int r = 0; ok && r < world; r++) ok = first_row[r] <= first_row[r + 1];
  if (!ok)
    throw invalid_input(WHOLEGRAPH_INVALID_VALUE,
                        "first_row must start at 0 and must not decrease from one rank to the next");
}

size_t partition_workspace_bytes(int64_t n, int world)
{
  const int64_t ctas = std::max<int64_t>(1, (n + kTile - 1) / kTile);
  return static_cast<size_t>(ctas * world + 4) * sizeof(int);
}

void partition_by_owner(const void* ids, bool ids_are_64, int64_t n, const int64_t* first_row,
                        int world, void* workspace, int64_t* sorted_ids, int64_t* positions,
                        int64_t* counts, int64_t* starts, cudaStream_t stream)
{
  WGB_EXPECTS(world >= 1 && world <= kMaxPartitionRanks, "world size %d exceeds %d", world,
              kMaxPartitionRanks);
  WGB_EXPECTS(n < (int64_t(1) << 31), "request list of %ld ids is too long", (long)n);
  check_owner_table(first_row, world);
  if (n == 0) {
    WGB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int64_t) * world, stream));
    WGB_CUDA_CHECK(cudaMemsetAsync(starts, 0, sizeof(int64_t) * world, stream));
    return;
  }
  owner_table t;
  t.world = world;
  for (int r = 0; r <= world; r++) t.first_row[r] = first_row[r];
  t.per_rank_estimate = std::max<int64_t>(1, (first_row[world] + world - 1) / world);

  const int ctas      = static_cast<int>((n + kTile - 1) / kTile);
  int* hist           = static_cast<int*>(workspace);
  const int64_t total = static_cast<int64_t>(ctas) * world;
  int* last_raw       = hist + total;

  partition_count_kernel<<<ctas, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, t, hist, ctas);
  partition_save_last_kernel<<<1, 1, 0, stream>>>(hist, total, last_raw);
  partition_scan_kernel<<<1, kScanThreads, 0, stream>>>(hist, total);
  partition_totals_kernel<<<1, kMaxPartitionRanks, 0, stream>>>(hist, last_raw, world, ctas, counts,
                                                               starts);
  partition_scatter_kernel<<<ctas, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, t, hist, ctas,
                                                          sorted_ids, positions);
  count_kernel_launch(5);
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
