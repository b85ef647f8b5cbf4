// Host interface of the set-associative embedding cache kernels (lookup, LFU update,
// write-back / drop).  Geometry and tag format are those of the reference
// (cpp/src/wholegraph/embedding_cache.hpp:64-74, cpp/src/wholegraph_tensor_ops/functions/
// embedding_cache_func.cuh:132-141): sets of 32 lines, a set covers `coverage` consecutive rows,
// a tag is valid (bit 14) | modified (bit 15) | 14-bit row number inside the set, and the LFU
// word is a 14-bit count scaled by a per-set shift whose bits are spread over bit 14 of the 32
// lines.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace wgb {

constexpr int kCacheSetSize     = 32;
constexpr int kCacheMaxCoverage = 1 << 14;
constexpr uint16_t kTagValid    = 1u << 14;
constexpr uint16_t kTagModified = 1u << 15;
constexpr uint16_t kTagRowMask  = (1u << 14) - 1;

// The cache lines that cover rows [first_row, first_row + rows) of a table, and the table rows
// themselves.  For a rank's own part the pointers are local; for a CONTINUOUS cache they may be
// the mapped global arrays with first_row = 0.
struct cache_view {
  uint16_t* tags        = nullptr;  // [sets, 32]
  uint16_t* lfu         = nullptr;  // [sets, 32]
  char* lines           = nullptr;  // [sets * 32] cache lines of line_bytes each
  int64_t* access_count = nullptr;  // [rows] exact access counters
  char* raw_rows        = nullptr;  // row first_row of the cached table
  int64_t first_row     = 0;
  int64_t rows          = 0;        // multiple of coverage
  int coverage          = 32;
  int64_t line_bytes    = 0;        // = table row stride in bytes (multiple of 16)
  // A read-only cache whose table this rank cannot address (raw_rows == nullptr; the table lives
  // on a larger communicator): an update then only decides which rows get which lines and
  // appends them to these lists, and the caller moves the rows (a gather from the table, a
  // scatter into the lines).  Entries beyond *load_count are left as they were (callers fill the
  // lists with -1, which both copies skip, so the count never has to reach the host).
  int64_t* load_rows    = nullptr;  // out: global row id of every line to load
  int64_t* load_lines   = nullptr;  // out: index of that line in `lines`
  int* load_count       = nullptr;  // in/out: entries used
};

// row_address[i] = address of the current copy of row ids[i]: its cache line on a hit, the table
// row otherwise, -1 for ids outside [first_row, first_row + rows).  With mark_modified, hit lines
// get their modified bit set (the caller is about to write the row).
// With `miss_ids` (n int64, for caches whose table rows have no address here): on a hit
// miss_ids[i] = -1 and row_address[i] is the line; on a miss row_address[i] = -1 and miss_ids[i] is
// the id itself, so that a gather of `miss_ids` from the table fills exactly the rows the cache
// left out (role of the reference's try_gather_cached_func, gather_cached_func.cu:251-467).
void cache_lookup(const void* ids, bool ids_are_64, int64_t n, const cache_view& c, bool mark_modified,
                  int64_t* row_address, cudaStream_t stream, int64_t* miss_ids = nullptr);

size_t cache_update_workspace_bytes(int64_t n);

// LFU update with the ids of one access batch (duplicates allowed, foreign ids ignored): exact
// per-row counters are incremented, and in every touched set the 32 rows with the highest
// counters become / stay cached.  Lines that stay keep their slot and modified bit; evicted
// modified lines are written back to the table first; new lines are loaded from the table.
void cache_update(const void* ids, bool ids_are_64, int64_t n, const cache_view& c, void* workspace,
                  cudaStream_t stream);

// Write every modified line back to the table and clear the modified bits; with `drop` also
// invalidate every line.
void cache_writeback(const cache_view& c, bool drop, cudaStream_t stream);

}  // namespace wgb
