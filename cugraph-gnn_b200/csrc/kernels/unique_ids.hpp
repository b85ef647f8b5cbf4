// Host interface of the request de-duplication used by the distributed gather.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace wgb {

// True when unique_by_owner can handle a table of `total_rows` rows (32-bit sort keys).
bool unique_supported(int64_t n, int64_t total_rows);

size_t unique_workspace_bytes(int64_t n, int64_t total_rows);

// Distinct valid ids of a request list, grouped by owner (shards are contiguous row ranges), and
// for every list position the slot of its id in that list.  With `ascending` the distinct ids are
// sorted (one radix sort); without it their order inside an owner's group is whatever a hash
// table's insertion races give (four short kernels, several times cheaper), which is enough for a
// gather: only `inverse` ties list positions to slots.
//   unique_ids : out, n int64 (device); first sum(counts) entries valid
//   inverse    : out, n int64 (device); slot in unique_ids, or -1 for ids that are negative or
//                >= first_row[world]
//   counts / starts : out, world int64 each (device): distinct ids owned by each rank and where
//                their group starts
// first_row is a HOST array of world + 1 entries.  Replaces, for gathers, the reference's sort of
// the full request list (exchange_ids_nccl_func.cu:32-104), which keeps duplicates on the wire.
void unique_by_owner(const void* ids, bool ids_are_64, int64_t n, const int64_t* first_row, int world,
                     void* workspace, int64_t* unique_ids, int64_t* inverse, int64_t* counts,
                     int64_t* starts, cudaStream_t stream, bool ascending = true);

}  // namespace wgb
