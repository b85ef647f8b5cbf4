// Memory handles: a sharded allocation over a communicator.
// Role of the reference's cpp/src/wholegraph/memory_handle.cpp (partition rule :1241-1262,
// CONTINUOUS/DEVICE mapping :928-988, accessors :1557-1660).
#pragma once

#include <cstddef>
#include <vector>

#include <wholegraph/wholegraph.h>

#include "comm.hpp"

struct wholegraph_handle_ {
  int id                               = -1;
  wholegraph_comm_* comm               = nullptr;
  wholegraph_memory_type_t type        = WHOLEGRAPH_MT_NONE;
  wholegraph_memory_location_t location = WHOLEGRAPH_ML_NONE;
  size_t total_size                    = 0;
  size_t granularity                   = 0;
  std::vector<size_t> part_sizes;    // world_size byte sizes (logical shards)
  std::vector<size_t> part_offsets;  // world_size + 1 byte offsets

  void* global_base = nullptr;       // CONTINUOUS: first byte of the single mapped range
  void* local_ptr   = nullptr;       // first byte of this rank's logical shard
  std::vector<void*> rank_ptrs;      // CHUNKED: first byte of every rank's shard (device pointers)
  void** dev_rank_ptrs = nullptr;    // CHUNKED: the same table in device memory

  struct backing;                    // allocation-specific state
  backing* impl = nullptr;
};

namespace wgb {

// Default split: ceil(units / world) units per rank, trailing ranks short or empty.
void plan_partition(size_t total_size, size_t granularity, int world, const size_t* rank_units,
                    std::vector<size_t>* sizes, std::vector<size_t>* offsets);

wholegraph_handle_* create_handle(size_t total_size, wholegraph_comm_* comm,
                                  wholegraph_memory_type_t type,
                                  wholegraph_memory_location_t location, size_t granularity,
                                  size_t* rank_entry_partition);
void destroy_handle(wholegraph_handle_* h);

}  // namespace wgb
