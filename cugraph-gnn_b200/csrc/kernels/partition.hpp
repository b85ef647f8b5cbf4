// Host interface of the stable partition-by-owner kernels.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace wgb {

constexpr int kMaxPartitionRanks = 64;

// Throws invalid_input(WHOLEGRAPH_INVALID_VALUE) unless first_row[0] == 0 and
// first_row[r] <= first_row[r + 1] for every rank (HOST array of world + 1 entries).
void check_owner_table(const int64_t* first_row, int world);

// Bytes of device scratch partition_by_owner needs for a list of n ids.
size_t partition_workspace_bytes(int64_t n, int world);

// Group the ids of a request list by owning rank, keeping list order inside each group.
//   ids          : n row ids (int32 or int64), device memory
//   first_row    : HOST array of world + 1 first rows per rank (first_row[world] = table rows)
//   sorted_ids   : out, n int64; group of rank r occupies [starts[r], starts[r] + counts[r])
//   positions    : out, n int64; list position each sorted id came from
//   counts/starts: out, world int64 each, DEVICE memory
// Ids that are negative or >= first_row[world] belong to no group and are not written; the
// groups are packed at the front of the output arrays.  n must be below 2^31.
void partition_by_owner(const void* ids, bool ids_are_64, int64_t n, const int64_t* first_row,
                        int world, void* workspace, int64_t* sorted_ids, int64_t* positions,
                        int64_t* counts, int64_t* starts, cudaStream_t stream);

// Same result as partition_by_owner, with the scratch taken from a fixed array inside the
// library instead of from the caller.  Throws invalid_input(WHOLEGRAPH_INVALID_VALUE) when
// partition_workspace_bytes(n, world) exceeds partition_builtin_scratch_bytes().  The first call
// on a device looks the array's address up; calls that overlap on one GPU race on the array.
size_t partition_builtin_scratch_bytes();
void partition_by_owner_builtin_scratch(const void* ids, bool ids_are_64, int64_t n,
                                        const int64_t* first_row, int world, int64_t* sorted_ids,
                                        int64_t* positions, int64_t* counts, int64_t* starts,
                                        cudaStream_t stream);

}  // namespace wgb
