// De-duplication of a gather's request list before it goes on the wire.
//
// Two implementations with the same outputs up to the order of the distinct ids inside an
// owner's group (which nothing downstream depends on: every list position finds its id through
// `inverse`).  Lists of up to 2^27 ids go through a hash table (four short kernels, below); longer
// ones, or callers that ask for ascending ids, through a sort:
//
// A skewed request list (a GNN mini-batch hits hub nodes again and again) sends the same id to
// the same owner many times; the owner of a hot row then serves - and its NVLink egress
// carries - several times the average.  Sorting the ids once gives both the grouping by owner
// (shards are contiguous row ranges) and the runs of equal ids, so only distinct ids travel and
// every row comes back once; the requester expands the rows with one more local gather.
//
//   1. keys_kernel      valid id -> 32-bit key, everything else -> sentinel; value = list position
//   2. cub radix sort   (key, position) pairs over the bits a row id can use
//   3. cub scan         running count of run heads -> slot of every sorted element
//   4. emit_kernel      unique_ids[slot] = key at run heads; inverse[position] = slot
//   5. bounds_kernel    per-owner group boundaries by binary search in the distinct ids
#include "unique_ids.hpp"

#include <algorithm>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <thrust/iterator/counting_iterator.h>
#include <thrust/iterator/transform_iterator.h>

#include "../common.hpp"
#include "partition.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads = 256;

__global__ void keys_kernel(const void* ids, int is64, int64_t n, int64_t total_rows, uint32_t* keys,
                            int32_t* positions)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t id = is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
                          : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
  keys[i]      = (id >= 0 && id < total_rows) ? static_cast<uint32_t>(id) : static_cast<uint32_t>(total_rows);
  positions[i] = static_cast<int32_t>(i);
}

struct head_flag {
  const uint32_t* keys;
  uint32_t sentinel;
  __device__ __forceinline__ int operator()(int j) const
  {
    const uint32_t k = keys[j];
    return (k != sentinel && (j == 0 || keys[j - 1] != k)) ? 1 : 0;
  }
};

__global__ void emit_kernel(const uint32_t* keys, const int32_t* positions, const int32_t* run_index,
                            int64_t n, uint32_t sentinel, int64_t* unique_ids, int64_t* inverse)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const uint32_t k = keys[j];
  if (k == sentinel) {
    inverse[positions[j]] = -1;
    return;
  }
  const int slot        = run_index[j] - 1;
  inverse[positions[j]] = slot;
  if (j == 0 || keys[j - 1] != k) unique_ids[slot] = k;
}

struct bounds_args {
  int world;
  int64_t first_row[kMaxPartitionRanks + 1];
};

// starts[r] = first slot whose id is >= first_row[r]; counts[r] = starts[r + 1] - starts[r].
__global__ void bounds_kernel(const int64_t* unique_ids, const int32_t* run_index, int64_t n, bounds_args a,
                              int64_t* counts, int64_t* starts)
{
  __shared__ int64_t s_start[kMaxPartitionRanks + 1];
  const int64_t distinct = run_index[n - 1];
  const int r            = threadIdx.x;
  if (r <= a.world) {
    int64_t lo = 0, hi = distinct;
    const int64_t target = a.first_row[r];
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (unique_ids[mid] < target)
        lo = mid + 1;
      else
        hi = mid;
    }
    s_start[r] = lo;
  }
  __syncthreads();
  if (r < a.world) {
    starts[r] = s_start[r];
    counts[r] = s_start[r + 1] - s_start[r];
  }
}

int key_bits(int64_t total_rows)
{
  int bits = 1;
  while (bits < 32 && (int64_t(1) << bits) <= total_rows) bits++;
  return bits;
}

struct layout {
  size_t keys_in, keys_out, pos_in, pos_out, run_index, cub, total, cub_bytes;
};

layout layout_for(int64_t n, int64_t total_rows)
{
  layout l{};
  auto align       = [](size_t x) { return (x + 255) / 256 * 256; };
  const size_t cnt = static_cast<size_t>(std::max<int64_t>(n, 1));
  size_t off       = 0;
  l.keys_in = off, off += align(cnt * 4);
  l.keys_out = off, off += align(cnt * 4);
  l.pos_in = off, off += align(cnt * 4);
  l.pos_out = off, off += align(cnt * 4);
  l.run_index = off, off += align(cnt * 4);
  size_t sort_bytes = 0, scan_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, static_cast<const uint32_t*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), static_cast<int>(cnt), 0, key_bits(total_rows));
  auto flags = thrust::make_transform_iterator(thrust::counting_iterator<int>(0), head_flag{nullptr, 0});
  cub::DeviceScan::InclusiveSum(nullptr, scan_bytes, flags, static_cast<int32_t*>(nullptr), static_cast<int>(cnt));
  l.cub_bytes = std::max(sort_bytes, scan_bytes);
  l.cub = off, off += align(l.cub_bytes);
  l.total = off;
  return l;
}

// ---- hash-table variant ------------------------------------------------------------------------
//   1. insert_kernel  every valid id claims (or finds) its entry of an open-addressing table of
//                     at least 2 n entries; the claimer counts as one distinct id of its owner
//   2. starts_kernel  exclusive scan of the per-owner counts
//   3. place_kernel   claimers take the next slot of their owner's group and leave it in the entry
//   4. inverse_kernel every list position reads its slot from its entry
// A table entry is {id + 1, slot}; 0 marks an empty entry.  An id that is already in the table is
// recognised with a plain load, so a hot id costs one compare-and-swap, not one per occurrence.
struct owner_bounds {
  int world;
  int64_t first_row[kMaxPartitionRanks + 1];
};

__device__ __forceinline__ int owner_of_row(int64_t id, const int64_t* first_row, int world)
{
  int lo = 0, hi = world - 1;  // last rank whose first row is <= id
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (first_row[mid] <= id) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ uint32_t mix(uint32_t x)
{
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

constexpr uint32_t kNoEntry    = 0xffffffffu;
constexpr uint32_t kClaimedBit = 0x80000000u;

constexpr int kHashItems = 8;                      // ids per thread
constexpr int kHashTile  = kThreads * kHashItems;  // ids per CTA

// Per-owner counts go through shared memory first: a CTA adds its 2048 ids' worth to the global
// counters with one atomic per owner (one atomic per warp and owner on the same few global
// addresses cost 0.3 ms for 4,194,304 ids).
__global__ void __launch_bounds__(kThreads)
  insert_kernel(const void* ids, int is64, int64_t n, owner_bounds b, uint2* table, uint32_t table_mask,
                uint32_t* entry_of, unsigned long long* owner_count)
{
  __shared__ int64_t s_first[kMaxPartitionRanks + 1];
  __shared__ int s_count[kMaxPartitionRanks];
  for (int i = threadIdx.x; i <= b.world; i += kThreads) s_first[i] = b.first_row[i];
  for (int i = threadIdx.x; i < b.world; i += kThreads) s_count[i] = 0;
  __syncthreads();
  const int lane     = threadIdx.x & 31;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kHashTile;
#pragma unroll
  for (int j = 0; j < kHashItems; j++) {
    const int64_t i = base + j * kThreads + threadIdx.x;
    int owner       = b.world;  // b.world: nothing to count
    if (i < n) {
      const int64_t id = is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
                              : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
      uint32_t where   = kNoEntry;
      if (id >= 0 && id < s_first[b.world]) {
        const uint32_t key = static_cast<uint32_t>(id) + 1u;
        uint32_t s         = mix(key) & table_mask;
        bool claimed       = false;
        bool found         = false;
        while (!found) {
          uint32_t seen = __ldcg(&table[s].x);
          if (seen == 0u) {
            seen    = atomicCAS(&table[s].x, 0u, key);
            claimed = seen == 0u;
          }
          found = claimed || seen == key;
          if (!found) s = (s + 1u) & table_mask;
        }
        where = s | (claimed ? kClaimedBit : 0u);
        if (claimed) owner = owner_of_row(id, s_first, b.world);
      }
      entry_of[i] = where;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, owner);
    if (owner < b.world && lane == __ffs(peers) - 1) atomicAdd(&s_count[owner], __popc(peers));
  }
  __syncthreads();
  for (int o = threadIdx.x; o < b.world; o += kThreads)
    if (s_count[o] != 0) atomicAdd(owner_count + o, static_cast<unsigned long long>(s_count[o]));
}

__global__ void starts_kernel(unsigned long long* owner_count, int world, int64_t* counts, int64_t* starts)
{
  if (threadIdx.x != 0) return;
  int64_t run = 0;
  for (int r = 0; r < world; r++) {
    const int64_t c = static_cast<int64_t>(owner_count[r]);
    counts[r]       = c;
    starts[r]       = run;
    owner_count[r]  = static_cast<unsigned long long>(run);  // becomes the group's fill cursor
    run += c;
  }
}

// Claimers take slots of their owner's group: positions inside the CTA first (shared memory),
// then one reservation per owner and CTA on the global cursors.
__global__ void __launch_bounds__(kThreads)
  place_kernel(const void* ids, int is64, int64_t n, owner_bounds b, uint2* table, const uint32_t* entry_of,
               unsigned long long* cursor, int64_t* unique_ids)
{
  __shared__ int64_t s_first[kMaxPartitionRanks + 1];
  __shared__ int s_count[kMaxPartitionRanks];
  __shared__ unsigned long long s_base[kMaxPartitionRanks];
  for (int i = threadIdx.x; i <= b.world; i += kThreads) s_first[i] = b.first_row[i];
  for (int i = threadIdx.x; i < b.world; i += kThreads) s_count[i] = 0;
  __syncthreads();
  const int lane     = threadIdx.x & 31;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kHashTile;
  int64_t id[kHashItems];
  uint32_t where[kHashItems];
  int owner[kHashItems], local[kHashItems];
#pragma unroll
  for (int j = 0; j < kHashItems; j++) {
    const int64_t i = base + j * kThreads + threadIdx.x;
    owner[j]        = b.world;
    where[j]        = kNoEntry;
    id[j]           = -1;
    local[j]        = 0;
    if (i < n) {
      where[j] = entry_of[i];
      if (where[j] != kNoEntry && (where[j] & kClaimedBit) != 0u) {
        id[j]    = is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
                        : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
        owner[j] = owner_of_row(id[j], s_first, b.world);
      }
    }
    const unsigned peers = __match_any_sync(0xffffffffu, owner[j]);
    const int leader     = __ffs(peers) - 1;
    int first            = 0;
    if (owner[j] < b.world && lane == leader) first = atomicAdd(&s_count[owner[j]], __popc(peers));
    first    = __shfl_sync(0xffffffffu, first, leader);
    local[j] = first + __popc(peers & ((1u << lane) - 1u));
  }
  __syncthreads();
  for (int o = threadIdx.x; o < b.world; o += kThreads)
    s_base[o] = s_count[o] != 0 ? atomicAdd(cursor + o, static_cast<unsigned long long>(s_count[o])) : 0ull;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kHashItems; j++) {
    if (owner[j] < b.world) {
      const int64_t slot = static_cast<int64_t>(s_base[owner[j]]) + local[j];
      unique_ids[slot]   = id[j];
      table[where[j] & ~kClaimedBit].y = static_cast<uint32_t>(slot);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
  inverse_kernel(int64_t n, const uint2* table, const uint32_t* entry_of, int64_t* inverse)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t where = entry_of[i];
  inverse[i] = where == kNoEntry ? -1 : static_cast<int64_t>(__ldcg(&table[where & ~kClaimedBit].y));
}

struct hashed_layout {
  size_t table, entry_of, owner_count, total;
  uint32_t entries;
};

hashed_layout hashed_layout_for(int64_t n)
{
  hashed_layout l{};
  auto align       = [](size_t x) { return (x + 255) / 256 * 256; };
  uint32_t entries = 1024;
  while (static_cast<int64_t>(entries) < 2 * n) entries <<= 1;
  l.entries  = entries;
  size_t off = 0;
  l.table = off, off += align(static_cast<size_t>(entries) * sizeof(uint2));
  l.owner_count = off, off += align(sizeof(unsigned long long) * (kMaxPartitionRanks + 1));
  l.entry_of = off, off += align(static_cast<size_t>(std::max<int64_t>(n, 1)) * 4);
  l.total = off;
  return l;
}

constexpr int64_t kHashedLimit = int64_t(1) << 27;

}  // namespace

bool unique_supported(int64_t n, int64_t total_rows)
{
  return n < (int64_t(1) << 31) && total_rows < (int64_t(1) << 32) - 1;
}

size_t unique_workspace_bytes(int64_t n, int64_t total_rows)
{
  // room for either variant
  return std::max(layout_for(n, total_rows).total, n <= kHashedLimit ? hashed_layout_for(n).total : size_t(0));
}

void unique_by_owner(const void* ids, bool ids_are_64, int64_t n, const int64_t* first_row, int world,
                     void* workspace, int64_t* unique_ids, int64_t* inverse, int64_t* counts,
                     int64_t* starts, cudaStream_t stream, bool ascending)
{
  WGB_EXPECTS(world >= 1 && world <= kMaxPartitionRanks, "world size %d exceeds %d", world, kMaxPartitionRanks);
  const int64_t total_rows = first_row[world];
  WGB_EXPECTS(unique_supported(n, total_rows), "request list or table too large for 32-bit sort keys");
  if (n == 0) {
    WGB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int64_t) * world, stream));
    WGB_CUDA_CHECK(cudaMemsetAsync(starts, 0, sizeof(int64_t) * world, stream));
    return;
  }
  if (!ascending && n <= kHashedLimit) {
    const hashed_layout l = hashed_layout_for(n);
    char* ws              = static_cast<char*>(workspace);
    auto* table           = reinterpret_cast<uint2*>(ws + l.table);
    auto* entry_of        = reinterpret_cast<uint32_t*>(ws + l.entry_of);
    auto* owner_count     = reinterpret_cast<unsigned long long*>(ws + l.owner_count);
    // table and counters are adjacent: one clear
    WGB_CUDA_CHECK(cudaMemsetAsync(ws + l.table, 0, l.entry_of - l.table, stream));
    owner_bounds b;
    b.world = world;
    for (int r = 0; r <= world; r++) b.first_row[r] = first_row[r];
    const unsigned blocks = static_cast<unsigned>((n + kThreads - 1) / kThreads);
    const unsigned tiles  = static_cast<unsigned>((n + kHashTile - 1) / kHashTile);
    insert_kernel<<<tiles, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, b, table, l.entries - 1, entry_of,
                                                  owner_count);
    starts_kernel<<<1, 32, 0, stream>>>(owner_count, world, counts, starts);
    place_kernel<<<tiles, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, b, table, entry_of, owner_count,
                                                 unique_ids);
    inverse_kernel<<<blocks, kThreads, 0, stream>>>(n, table, entry_of, inverse);
    count_kernel_launch(4);
    WGB_LAUNCH_CHECK(stream);
    return;
  }
  const layout l        = layout_for(n, total_rows);
  char* ws              = static_cast<char*>(workspace);
  auto* keys_in         = reinterpret_cast<uint32_t*>(ws + l.keys_in);
  auto* keys_out        = reinterpret_cast<uint32_t*>(ws + l.keys_out);
  auto* pos_in          = reinterpret_cast<int32_t*>(ws + l.pos_in);
  auto* pos_out         = reinterpret_cast<int32_t*>(ws + l.pos_out);
  auto* run_index       = reinterpret_cast<int32_t*>(ws + l.run_index);
  const unsigned blocks = static_cast<unsigned>((n + kThreads - 1) / kThreads);
  const uint32_t sentinel = static_cast<uint32_t>(total_rows);

  keys_kernel<<<blocks, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, total_rows, keys_in, pos_in);
  size_t bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(ws + l.cub, bytes, keys_in, keys_out, pos_in, pos_out,
                                                 static_cast<int>(n), 0, key_bits(total_rows), stream));
  auto flags = thrust::make_transform_iterator(thrust::counting_iterator<int>(0), head_flag{keys_out, sentinel});
  bytes      = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceScan::InclusiveSum(ws + l.cub, bytes, flags, run_index, static_cast<int>(n), stream));
  emit_kernel<<<blocks, kThreads, 0, stream>>>(keys_out, pos_out, run_index, n, sentinel, unique_ids, inverse);
  bounds_args a;
  a.world = world;
  for (int r = 0; r <= world; r++) a.first_row[r] = first_row[r];
  bounds_kernel<<<1, kMaxPartitionRanks + 1 + 31, 0, stream>>>(unique_ids, run_index, n, a, counts, starts);
  count_kernel_launch(5);
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
