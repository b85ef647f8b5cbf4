// Host interface of the row copy kernels (gather, scatter and reorder share one kernel).
// Replaces the launchers of the reference's
// cpp/src/wholegraph_tensor_ops/functions/gather_scatter_func.cuh:367-650.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

#include <wholegraph/tensor_description.h>

namespace wgb {

// How the row number on one side of the copy is chosen for list position i.
enum row_select_t : int {
  ROW_SEQUENTIAL = 0,  // row i
  ROW_BY_INDEX   = 1,  // row indices[i]          (the table side)
  ROW_BY_POSITION = 2, // row positions[i]        (reorder through a permutation)
  ROW_BY_ADDRESS  = 3, // indices[i] is the int64 byte address of the row itself (negative: skip);
                       // the side's pointer is ignored, its offset is added, its stride only
                       // states the rows' alignment
};

// A table whose rows live behind one base pointer per rank (CHUNKED memory).  When
// `ranks` > 0 the BY_INDEX side resolves row r to base[owner] + (r - first_row[owner]) * stride.
constexpr int kMaxChunkedRanks = 16;
struct chunked_table {
  int ranks = 0;
  const void* base[kMaxChunkedRanks];
  int64_t first_row[kMaxChunkedRanks + 1];
};

// A list made of up to kMaxListSegments disjoint pieces of the index / position / sequential-row
// arrays: logical position l of the copy maps to array position begin[s] + (l - prefix[s]) for the
// segment s with prefix[s] <= l < prefix[s + 1].  n = 0 means one piece starting at 0.
constexpr int kMaxListSegments = 64;
struct list_segments {
  int n = 0;
  int64_t begin[kMaxListSegments];
  int64_t prefix[kMaxListSegments + 1];
  void add(int64_t first, int64_t count)
  {
    if (count <= 0) return;
    if (n == 0) prefix[0] = 0;
    begin[n]      = first;
    prefix[n + 1] = prefix[n] + count;
    n++;
  }
  int64_t total() const { return n == 0 ? 0 : prefix[n]; }
};

struct row_copy_args {
  // source rows
  const void* src          = nullptr;  // element 0 of the storage (before src_offset)
  wholegraph_dtype_t src_dt = WHOLEGRAPH_DT_UNKNOWN;
  int64_t src_stride       = 0;  // elements between rows
  int64_t src_offset       = 0;  // elements before row 0
  row_select_t src_select  = ROW_SEQUENTIAL;
  // destination rows
  void* dst                = nullptr;
  wholegraph_dtype_t dst_dt = WHOLEGRAPH_DT_UNKNOWN;
  int64_t dst_stride       = 0;
  int64_t dst_offset       = 0;
  row_select_t dst_select  = ROW_SEQUENTIAL;
  // the list
  int64_t count            = 0;        // list length
  int64_t dim              = 0;        // elements per row
  const void* indices      = nullptr;  // int32 / int64 row ids; a negative id skips position i
  bool indices_are_64      = true;
  const int64_t* positions = nullptr;  // for ROW_BY_POSITION
  chunked_table chunks;                // optional, BY_INDEX side only
  list_segments segments;              // optional; when n > 0, `count` must equal segments.total()
  int sm_hint              = -1;       // -1, or roughly how many SMs to occupy
};

// Enqueue the copy on `stream`.  Throws logic_error for dtype pairs that mix floating point
// and integer types (reference: gather_func.cu:63-70).
void launch_row_copy(const row_copy_args& a, cudaStream_t stream);

// Largest power-of-two element count <= 16 bytes / max element size that divides dim, both
// strides and both first-element addresses (reference rule: gather_scatter_func.cuh:204-240).
int row_copy_vector_elements(const row_copy_args& a);

unsigned long long kernel_launch_count();
void count_kernel_launch(int n = 1);

}  // namespace wgb
