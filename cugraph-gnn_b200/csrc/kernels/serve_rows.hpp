// Host interface of the owner-side kernel of a distributed gather whose request counts never
// reach the host.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace wgb {

constexpr int kMaxServeRanks = 64;

// Region of one rank in the peer-mapped exchange arena, as seen from this process.  The rank
// fills `header` and `ids` with its own request; the owners fill `rows`.
//   header : 2 * world int64: counts[o] = distinct ids the rank asks of owner o, starts[o] = where
//            that group begins in `ids` (and in `rows`)
//   ids    : the rank's distinct ids, grouped by owner
//   rows   : row j of the region answers ids[j]
struct serve_region {
  const int64_t* header;
  const int64_t* ids;
  char* rows;
};

struct serve_rows_args {
  int world = 1, me = 0;
  serve_region region[kMaxServeRanks];  // by rank
  int64_t capacity      = 0;            // ids a region can hold; larger counts are refused
  const void* shard     = nullptr;      // row `first_local_row` of the table (storage offset applied)
  int64_t first_local_row = 0, local_rows = 0;
  int64_t shard_stride_bytes = 0;       // bytes between rows of the shard
  int64_t row_bytes     = 0;            // bytes per row moved (and between rows of `rows`)
  int64_t rows_upper_bound = 0;         // no more than this many rows are asked of this rank in total
  bool bulk             = false;        // stage tiles of rows in shared memory with bulk asynchronous copies and send each
                                        // tile with one bulk store (rows and strides must be multiples of 16 bytes, rows of
                                        // 128 bytes to 16 KiB; other shapes take the register kernel whatever this says)
  int* status           = nullptr;      // device word: set non-zero when a header or an id is out of range
};

// Every rank's requests to this rank, answered in one kernel: for each requester q (its
// neighbours first, itself last) read counts[me] and starts[me] from q's header, then copy row
// ids[starts + j] of the local shard to rows[starts + j] of q's region - a peer load of the id, a
// local load of the row, a peer store of the row.  Nothing here depends on the host knowing the
// counts.  Ids outside the local shard (in the bulk form: the tile of up to 32 slots holding one)
// and headers that do not fit the region are skipped and reported through `status`: 1 header,
// 2 id, 3 a bulk copy that did not complete within the wait limit.  Enqueued on `stream`.
void launch_serve_rows(const serve_rows_args& a, cudaStream_t stream);

}  // namespace wgb
