// Host interface of the two graph utilities that sit between neighbour sampling and the
// embedding gather of a mini-batch (reference: cpp/src/graph_ops/append_unique_func.cuh,
// csr_add_self_loop_func.cuh).
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace wgb {

// ---- append unique ----------------------------------------------------------------------------
// Node list of a sampled hop: the targets, in their order, followed by the distinct neighbours that
// are not targets.  Where the reference appends the new neighbours in hash-table order (which
// depends on which thread wins a slot), this version appends them in ascending id order, so the
// result is reproducible; every property the reference guarantees holds (targets first and
// unchanged, every other neighbour exactly once, mapping[j] = position of neighbours[j] in the
// list).  A neighbour that equals several targets maps to the first of them.
//
// Step 1 sorts (id, position) pairs of targets and neighbours together and counts the new
// neighbours; the count comes back through `new_count` (pinned host memory, valid once `stream`
// has been synchronised).  Step 2 writes the outputs: unique_nodes[target_count + new_count] and,
// when not null, mapping[neighbor_count] (int32).
size_t append_unique_workspace_bytes(int64_t target_count, int64_t neighbor_count, bool ids_are_64);
void append_unique_group(const void* targets, int64_t target_count, const void* neighbors, int64_t neighbor_count,
                         bool ids_are_64, void* workspace, int* new_count, cudaStream_t stream);
void append_unique_write(const void* targets, int64_t target_count, int64_t neighbor_count, bool ids_are_64,
                         void* workspace, void* unique_nodes, int* mapping, cudaStream_t stream);

// ---- self loops ---------------------------------------------------------------------------------
// CSR of `rows` rows -> CSR with edge (r, r) put first in every row r: out_row_ptr[r] = row_ptr[r] + r,
// out_col[out_row_ptr[r]] = r, then the row's columns (reference: csr_add_self_loop_func.cuh:13-32).
void csr_add_self_loops(const int* row_ptr, const int* col, int64_t rows, int* out_row_ptr, int* out_col,
                        cudaStream_t stream);

}  // namespace wgb
