// Set-associative embedding cache for sm_100a: lookup, LFU update, write-back.
//
// Own design behind the reference's geometry and tag format (see cache.hpp).  Where the reference
// keeps approximate scaled counters for cached lines and runs a library warp top-k
// (embedding_cache_func.cuh:152-373), this version keeps exact int64 access counters for every
// row in memory and selects the 32 most-accessed rows of a set with an in-warp bitonic top-32
// merge; rows that stay cached never move, so their modified bits and contents are untouched.
#include "cache.hpp"

#include <algorithm>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_run_length_encode.cuh>
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include "../common.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int64_t load_id(const void* ids, int is64, int64_t i)
{
  return is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
              : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
}

// Four lanes per id, eight ids per warp: each lane of a group loads 16 bytes (8 tags) of the id's
// 64-byte tag set and compares them; the group's answer is combined with two shuffles.  (One warp
// per id, one tag per lane, spent 108 us on 1,048,576 ids whose tag sets sat in L2.)
constexpr int kLookupLanes = 4;
constexpr int kLookupIds   = 32 / kLookupLanes;

__global__ void __launch_bounds__(kThreads) lookup_kernel(const void* ids, int is64, int64_t n, cache_view c,
                                                          int mark_modified, int64_t* row_address, int64_t* miss_ids)
{
  const int lane            = threadIdx.x & 31;
  const int sub             = lane & (kLookupLanes - 1);  // which quarter of the tag set
  const int slot            = lane / kLookupLanes;        // which of the warp's ids
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t base = warp_global * kLookupIds; base < n; base += warp_stride * kLookupIds) {
    const int64_t i     = base + slot;
    const bool live     = i < n;
    const int64_t id    = live ? load_id(ids, is64, i) : -1;
    const int64_t local = live ? id - c.first_row : -1;
    const bool in_range = live && local >= 0 && local < c.rows;
    int64_t set         = 0;
    int hit             = -1;
    if (in_range) {
      set                = local / c.coverage;
      const uint32_t row = static_cast<uint32_t>(local - set * c.coverage);
      const uint4 v      = *reinterpret_cast<const uint4*>(c.tags + set * kCacheSetSize + sub * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const uint32_t tag = (w[k >> 1] >> ((k & 1) * 16)) & 0xffffu;
        if ((tag & kTagValid) != 0 && (tag & kTagRowMask) == row) hit = sub * 8 + k;
      }
    }
    hit = max(hit, __shfl_xor_sync(0xffffffffu, hit, 1));
    hit = max(hit, __shfl_xor_sync(0xffffffffu, hit, 2));
    if (sub != 0 || !live) continue;
    if (miss_ids != nullptr) miss_ids[i] = (in_range && hit >= 0) ? -1 : id;  // negative ids stay skipped
    if (!in_range || (hit < 0 && c.raw_rows == nullptr)) {
      row_address[i] = -1;
    } else if (hit >= 0) {
      // equal ids in other groups may store the same value at the same time
      if (mark_modified) c.tags[set * kCacheSetSize + hit] |= kTagModified;
      row_address[i] = reinterpret_cast<int64_t>(c.lines + (set * kCacheSetSize + hit) * c.line_bytes);
    } else {
      row_address[i] = reinterpret_cast<int64_t>(c.raw_rows + local * c.line_bytes);
    }
  }
}

// ---- update -------------------------------------------------------------------------------------
__global__ void local_keys_kernel(const void* ids, int is64, int64_t n, int64_t first_row, int64_t rows,
                                  uint32_t* keys)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t local = load_id(ids, is64, i) - first_row;
  keys[i] = (local >= 0 && local < rows) ? static_cast<uint32_t>(local) : static_cast<uint32_t>(rows);
}

// First distinct id of every touched set (distinct ids are ascending, so a set's ids are adjacent).
struct set_head {
  const uint32_t* distinct;
  const int* distinct_count;
  uint32_t sentinel;
  int coverage;
  __device__ __forceinline__ bool operator()(int j) const
  {
    if (j >= *distinct_count) return false;
    const uint32_t r = distinct[j];
    if (r == sentinel) return false;
    return j == 0 || distinct[j - 1] / coverage != r / coverage;
  }
};

struct entry {
  long long key;  // count * 2 + (1 if currently cached); -1 = empty
  int row;        // row number inside the set, -1 = empty
  int slot;       // line the row occupies now, -1 if not cached
};

__device__ __forceinline__ bool before(const entry& a, const entry& b)
{
  // descending by key; ties by ascending row so that the order is total and deterministic
  return a.key > b.key || (a.key == b.key && a.row < b.row);
}

__device__ __forceinline__ entry shfl_entry(const entry& e, int src)
{
  entry o;
  o.key  = __shfl_sync(0xffffffffu, e.key, src);
  o.row  = __shfl_sync(0xffffffffu, e.row, src);
  o.slot = __shfl_sync(0xffffffffu, e.slot, src);
  return o;
}

// Bitonic network over the 32 lanes; `k_start` = 2 sorts arbitrary input, `k_start` = 32 merges a
// bitonic sequence.  Result: lane 0 holds the entry that comes first.
__device__ __forceinline__ void bitonic(entry& e, int lane, int k_start)
{
  for (int k = k_start; k <= 32; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      const entry o        = shfl_entry(e, lane ^ j);
      const bool ascending = (lane & k) == 0 || k == 32;  // final pass sorts the whole warp one way
      const bool lower     = (lane & j) == 0;
      const bool take_o    = (lower == ascending) ? before(o, e) : before(e, o);
      if (take_o) e = o;
    }
  }
}

__device__ __forceinline__ void copy_line(char* dst, const char* src, int64_t bytes, int lane)
{
  for (int64_t b = lane * 16; b < bytes; b += 32 * 16)
    *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(src + b);
}

// One warp per touched set.
__global__ void __launch_bounds__(kThreads)
  update_sets_kernel(cache_view c, const uint32_t* distinct, const int* counts, const int* distinct_count,
                     const int* set_first, const int* set_count)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int touched         = *set_count;
  int total_distinct        = *distinct_count;
  if (total_distinct > 0 && distinct[total_distinct - 1] == static_cast<uint32_t>(c.rows)) total_distinct--;

  for (int64_t t = warp_global; t < touched; t += warp_stride) {
    const int first     = set_first[t];
    const int64_t set   = distinct[first] / c.coverage;
    const int64_t row0  = set * c.coverage;  // first row (local numbering) of the set
    // ids of this set: [first, last)
    int last = first;
    {
      // the next touched set starts where this one ends; set_first is ascending
      last = (t + 1 < touched) ? set_first[t + 1] : total_distinct;
    }
    uint16_t* tags      = c.tags + set * kCacheSetSize;
    uint16_t* lfu       = c.lfu + set * kCacheSetSize;
    const uint16_t tag  = tags[lane];
    const int my_row    = (tag & kTagValid) ? (tag & kTagRowMask) : -1;
    const bool modified = (tag & kTagModified) != 0;

    // 1. exact counters
    for (int j = first + lane; j < last; j += 32) c.access_count[distinct[j]] += counts[j];
    __syncwarp();

    // 2. top 32 of (cached rows) U (accessed rows) by counter
    entry top;
    top.row  = my_row;
    top.slot = my_row >= 0 ? lane : -1;
    top.key  = my_row >= 0 ? c.access_count[row0 + my_row] * 2 + 1 : -1;
    bitonic(top, lane, 2);
    for (int base = first; base < last; base += 32) {
      const int j = base + lane;
      entry cand{-1, -1, -1};
      const int r = j < last ? static_cast<int>(distinct[j] - row0) : -2;
      // already cached?  compare against the 32 line rows (all lanes take part in every shuffle)
      bool cached = false;
      for (int l = 0; l < 32; l++) cached |= (__shfl_sync(0xffffffffu, my_row, l) == r);
      if (r >= 0 && !cached) {
        cand.row = r;
        cand.key = c.access_count[distinct[j]] * 2;
      }
      bitonic(cand, lane, 2);
      // top (descending) and reversed cand form a bitonic sequence whose element-wise "first"
      // halves are the 32 best of the 64
      const entry rev = shfl_entry(cand, 31 - lane);
      if (before(rev, top)) top = rev;
      bitonic(top, lane, 32);
    }

    // 3. slots: rows that stay keep theirs, new rows take freed ones in order
    const unsigned keep   = __reduce_or_sync(0xffffffffu, top.slot >= 0 ? (1u << top.slot) : 0u);
    const unsigned freed  = ~keep;
    const bool is_new     = top.row >= 0 && top.slot < 0;
    const unsigned new_m  = __ballot_sync(0xffffffffu, is_new);
    const int new_rank    = __popc(new_m & ((1u << lane) - 1u));
    const int target      = is_new ? static_cast<int>(__fns(freed, 0, new_rank + 1)) : -1;

    // 4. move data: evicted modified lines go back to the table, new rows are loaded
    const bool evicted = my_row >= 0 && ((keep >> lane) & 1u) == 0;
    if (c.raw_rows == nullptr) {
      // The table has no address here (and the cache is read-only: no line is modified): list
      // the rows to load with their lines and let the caller move them.
      int base = 0;
      if (lane == 0 && new_m != 0) base = atomicAdd(c.load_count, __popc(new_m));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (is_new) {
        c.load_rows[base + new_rank]  = c.first_row + row0 + top.row;
        c.load_lines[base + new_rank] = set * kCacheSetSize + target;
      }
    } else {
      for (int l = 0; l < 32; l++) {
        const int ev_row = __shfl_sync(0xffffffffu, (evicted && modified) ? my_row : -1, l);
        if (ev_row >= 0)
          copy_line(c.raw_rows + (row0 + ev_row) * c.line_bytes, c.lines + (set * kCacheSetSize + l) * c.line_bytes,
                    c.line_bytes, lane);
      }
    }
    __syncwarp();
    if (c.raw_rows != nullptr) {
      for (int l = 0; l < 32; l++) {
        const int nrow  = __shfl_sync(0xffffffffu, is_new ? top.row : -1, l);
        const int nslot = __shfl_sync(0xffffffffu, target, l);
        if (nrow >= 0)
          copy_line(c.lines + (set * kCacheSetSize + nslot) * c.line_bytes, c.raw_rows + (row0 + nrow) * c.line_bytes,
                    c.line_bytes, lane);
      }
    }

    // 5. new tags and scaled LFU words: lane = line
    int new_row   = evicted ? -1 : my_row;
    bool new_mod  = evicted ? false : modified;
    for (int l = 0; l < 32; l++) {
      const int nrow  = __shfl_sync(0xffffffffu, is_new ? top.row : -1, l);
      const int nslot = __shfl_sync(0xffffffffu, target, l);
      if (nrow >= 0 && nslot == lane) {
        new_row = nrow;
        new_mod = false;
      }
    }
    const long long cnt = new_row >= 0 ? c.access_count[row0 + new_row] : 0;
    int scale           = cnt > 0 ? 64 - __clzll(cnt) : 0;
    scale               = max(scale, 14) - 14;
    const int max_scale = __reduce_max_sync(0xffffffffu, scale);
    uint16_t word       = static_cast<uint16_t>((cnt >> max_scale) & kTagRowMask);
    word |= static_cast<uint16_t>(((max_scale >> lane) & 1) << 14);
    tags[lane] = new_row >= 0 ? static_cast<uint16_t>(kTagValid | (new_mod ? kTagModified : 0) | new_row) : 0;
    lfu[lane]  = word;
  }
}

__global__ void __launch_bounds__(kThreads) writeback_kernel(cache_view c, int drop)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t sets        = c.rows / c.coverage;
  for (int64_t set = warp_global; set < sets; set += warp_stride) {
    uint16_t* tags     = c.tags + set * kCacheSetSize;
    const uint16_t tag = tags[lane];
    const bool dirty   = (tag & kTagValid) && (tag & kTagModified);
    for (int l = 0; l < 32; l++) {
      const int row = __shfl_sync(0xffffffffu, dirty ? (tag & kTagRowMask) : -1, l);
      if (row >= 0)
        copy_line(c.raw_rows + (set * c.coverage + row) * c.line_bytes,
                  c.lines + (set * kCacheSetSize + l) * c.line_bytes, c.line_bytes, lane);
    }
    tags[lane] = drop ? 0 : static_cast<uint16_t>(tag & ~kTagModified);
  }
}

int key_bits(int64_t rows)
{
  int bits = 1;
  while (bits < 32 && (int64_t(1) << bits) <= rows) bits++;
  return bits;
}

struct layout {
  size_t keys, sorted, distinct, counts, num, set_first, cub, total, cub_bytes;
};

layout layout_for(int64_t n)
{
  layout l{};
  auto align       = [](size_t x) { return (x + 255) / 256 * 256; };
  const size_t cnt = static_cast<size_t>(std::max<int64_t>(n, 1));
  size_t off       = 0;
  l.keys = off, off += align(cnt * 4);
  l.sorted = off, off += align(cnt * 4);
  l.distinct = off, off += align(cnt * 4);
  l.counts = off, off += align(cnt * 4);
  l.num = off, off += 256;  // [0] distinct ids, [1] touched sets
  l.set_first = off, off += align(cnt * 4);
  size_t a = 0, b = 0, d = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, a, static_cast<const uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                 static_cast<int>(cnt), 0, 32);
  cub::DeviceRunLengthEncode::Encode(nullptr, b, static_cast<const uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                     static_cast<int*>(nullptr), static_cast<int*>(nullptr), static_cast<int>(cnt));
  cub::DeviceSelect::If(nullptr, d, thrust::counting_iterator<int>(0), static_cast<int*>(nullptr),
                        static_cast<int*>(nullptr), static_cast<int>(cnt), set_head{nullptr, nullptr, 0, 1});
  l.cub_bytes = std::max(a, std::max(b, d));
  l.cub = off, off += align(l.cub_bytes);
  l.total = off;
  return l;
}

int grid_for(int64_t warps)
{
  static int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  const int64_t ctas = (warps + 7) / 8;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(ctas, static_cast<int64_t>(sm_count) * 8 * 4)));
}

void check_view(const cache_view& c)
{
  WGB_EXPECTS(c.coverage >= kCacheSetSize && c.coverage <= kCacheMaxCoverage, "cache set coverage %d", c.coverage);
  WGB_EXPECTS(c.rows % c.coverage == 0, "cached rows are not a multiple of the set coverage");
  WGB_EXPECTS(c.line_bytes % 16 == 0, "cache lines must be multiples of 16 bytes");
  WGB_EXPECTS(c.rows < (int64_t(1) << 32) - 1, "cached range too large");
  WGB_EXPECTS(reinterpret_cast<uintptr_t>(c.tags) % 16 == 0, "cache tags must be 16-byte aligned");
}

}  // namespace

void cache_lookup(const void* ids, bool ids_are_64, int64_t n, const cache_view& c, bool mark_modified,
                  int64_t* row_address, cudaStream_t stream, int64_t* miss_ids)
{
  if (n == 0) return;
  check_view(c);
  WGB_EXPECTS(c.raw_rows != nullptr || miss_ids != nullptr, "a cache without table addresses needs a miss list");
  lookup_kernel<<<grid_for((n + kLookupIds - 1) / kLookupIds), kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, c, mark_modified ? 1 : 0,
                                                      row_address, miss_ids);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

size_t cache_update_workspace_bytes(int64_t n) { return layout_for(n).total; }

void cache_update(const void* ids, bool ids_are_64, int64_t n, const cache_view& c, void* workspace,
                  cudaStream_t stream)
{
  if (n == 0) return;
  check_view(c);
  WGB_EXPECTS(n < (int64_t(1) << 31), "access batch of %ld ids is too long", (long)n);
  WGB_EXPECTS(c.raw_rows != nullptr || (c.load_rows != nullptr && c.load_lines != nullptr && c.load_count != nullptr),
              "a cache without table addresses needs load lists");
  const layout l  = layout_for(n);
  char* ws        = static_cast<char*>(workspace);
  auto* keys      = reinterpret_cast<uint32_t*>(ws + l.keys);
  auto* sorted    = reinterpret_cast<uint32_t*>(ws + l.sorted);
  auto* distinct  = reinterpret_cast<uint32_t*>(ws + l.distinct);
  auto* counts    = reinterpret_cast<int*>(ws + l.counts);
  auto* num       = reinterpret_cast<int*>(ws + l.num);
  auto* set_first = reinterpret_cast<int*>(ws + l.set_first);
  const unsigned blocks = static_cast<unsigned>((n + kThreads - 1) / kThreads);
  local_keys_kernel<<<blocks, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, n, c.first_row, c.rows, keys);
  size_t bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceRadixSort::SortKeys(ws + l.cub, bytes, keys, sorted, static_cast<int>(n), 0,
                                                key_bits(c.rows), stream));
  bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceRunLengthEncode::Encode(ws + l.cub, bytes, sorted, distinct, counts, num,
                                                    static_cast<int>(n), stream));
  bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceSelect::If(ws + l.cub, bytes, thrust::counting_iterator<int>(0), set_first, num + 1,
                                       static_cast<int>(n),
                                       set_head{distinct, num, static_cast<uint32_t>(c.rows), c.coverage}, stream));
  update_sets_kernel<<<grid_for(std::min<int64_t>(n, c.rows / c.coverage)), kThreads, 0, stream>>>(
    c, distinct, counts, num, set_first, num + 1);
  count_kernel_launch(5);
  WGB_LAUNCH_CHECK(stream);
}

void cache_writeback(const cache_view& c, bool drop, cudaStream_t stream)
{
  if (c.rows == 0) return;
  check_view(c);
  writeback_kernel<<<grid_for(c.rows / c.coverage), kThreads, 0, stream>>>(c, drop ? 1 : 0);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
