// Shared pieces of the distributed ops: the id exchange plan.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <string>
#include <utility>
#include <vector>

#include <wholegraph/tensor_description.h>

#include "comm.hpp"
#include "common.hpp"
#include "env.hpp"
#include "handle.hpp"

namespace wgb {

// Result of routing one rank's request list to the owners of the rows
// (role of the reference's bucket_and_exchange_ids_func,
// cpp/src/wholegraph_tensor_ops/functions/exchange_ids_nccl_func.cu:146-215).
struct exchange_plan {
  explicit exchange_plan(wholegraph_env_func_t* env);

  // Partition `ids` by owner, exchange the per-rank counts (one host synchronisation of
  // `stream`) and then the ids themselves (asynchronous on `stream`).
  // With `dedup`, only the distinct valid ids are routed (ascending inside each owner's group):
  // sorted_ids then holds them, `inverse[i]` is the slot of list position i in sorted_ids (-1 for
  // ids nobody owns) and `positions` is not filled.
  void build(const void* ids, bool ids_are_64, int64_t n, const std::vector<int64_t>& first_row,
             wholegraph_comm_* comm, cudaStream_t stream, bool dedup = false);

  // Same exchange for a list that is already grouped by owner: `grouped_ids` holds the ids to
  // route and `group_counts_dev` the device layout [counts | starts | scratch], `world` entries
  // each, that describes its groups.  sorted_ids aliases grouped_ids; positions stays null.
  void build_grouped(int64_t* grouped_ids, int64_t* group_counts_dev, wholegraph_comm_* comm,
                     cudaStream_t stream);

  int world = 1, me = 0;
  int64_t count = 0;  // length of the request list
  // Host copies, in rows.  send_* describe this rank's requests grouped by owner (positions in
  // sorted_ids / positions); recv_* describe the requests other ranks sent here (in recv_ids).
  std::vector<int64_t> send_counts, send_displs, recv_counts, recv_displs;
  int64_t total_send = 0, total_recv = 0;
  // rows[q * world + r]: rows rank q routes to rank r, known to every rank.  Groups sit in owner
  // order, so rank q's group for owner r starts at group_start(q, r) in q's own numbering, and
  // the rows rank q sends to owner r arrive at arrival_start(q, r) in r's receive numbering.
  std::vector<int64_t> rows;
  int64_t group_start(int q, int r) const;
  int64_t arrival_start(int q, int r) const;
  int64_t max_total_send() const;
  int64_t max_total_recv() const;
  // Chunks of a pipelined exchange of rows of `row_bytes` bytes under this plan (see
  // exchange_chunk_count); the same number on every rank.
  int chunk_count(size_t row_bytes, int wanted, int forced) const;
  int64_t* sorted_ids = nullptr;  // device, global row ids grouped by owner
  int64_t* positions  = nullptr;  // device, list position of each sorted id
  int64_t* recv_ids   = nullptr;  // device, global row ids this rank must serve
  int64_t* inverse    = nullptr;  // device, dedup only: slot in sorted_ids of every list position

 private:
  void exchange_counts_and_ids(int64_t* cdev, wholegraph_comm_* comm, cudaStream_t stream);
  temp_buffer workspace, sorted_ids_buf, positions_buf, recv_ids_buf, counts_dev, counts_pin, matrix_dev;
};

// Row exchange of a distributed op, cut into chunks so that packing chunk k + 1, moving chunk k
// over NVLink and unpacking chunk k - 1 overlap.  Rows for peer p occupy
// [out_displs[p], out_displs[p] + out_counts[p]) of `out_buf` and arrive at
// [in_displs[p], in_displs[p] + in_counts[p]) of `in_buf`; chunk k of a segment of c rows is rows
// [c * k / K, c * (k + 1) / K).  `pack(segments)` must enqueue on `stream` whatever fills the
// outgoing rows named by `segments` (array positions in out_buf's row numbering);
// `unpack(segments)` consumes the incoming rows named by `segments`.  Every chunk is ONE NCCL
// group over all peers on the communicator's exchange stream.  On return `stream` is ordered
// after the last unpack.  The self segment (p == rank) is never touched.  K must be the same on
// every rank (each chunk is a matched set of sends and receives): take it from
// exchange_plan::chunk_count.
struct list_segments;
void pipelined_exchange(wholegraph_comm_* comm, const std::vector<int64_t>& out_counts,
                        const std::vector<int64_t>& out_displs, const std::vector<int64_t>& in_counts,
                        const std::vector<int64_t>& in_displs, char* out_buf, char* in_buf,
                        size_t row_bytes, cudaStream_t stream,
                        const std::function<void(const list_segments&)>& pack,
                        const std::function<void(const list_segments&)>& unpack, int K);

// Number of chunks K for pipelined_exchange, from data every rank holds identically: the
// world x world count matrix (matrix[q * world + r] = rows rank q routes to rank r).  `forced` > 0
// (WG_EXCHANGE_CHUNKS) wins, then `wanted` > 0 (callers whose pack and unpack do little pass 1:
// with nothing to overlap one large exchange is fastest, measured at 8 GPUs 2.21 ms with K = 1
// against 2.29 ms with K = 4); otherwise 4 when the busiest rank moves 16 MB or more, else 1.
int exchange_chunk_count(const int64_t* matrix, int world, size_t row_bytes, int wanted, int forced);

struct cache_view;
// Gather rows of a DISTRIBUTED table (descriptor `tab` over handle `h`) into `out`.  With
// `cache` (this rank's part of a set-associative cache in front of its shard) owners serve each
// row from its cache line when it has one, after an optional LFU update with the ids they
// received (`adjust_cache`); duplicates are then routed as they are, because the update counts
// them.
void gather_distributed(wholegraph_handle_* h, const wholegraph_matrix_description_t& tab, const void* ids,
                        bool ids_are_64, int64_t n, void* out, const wholegraph_matrix_description_t& od,
                        wholegraph_env_func_t* env, cudaStream_t stream, int sms,
                        const cache_view* cache = nullptr, bool adjust_cache = false);

// Peer-mapped exchange arena of a communicator with at least `bytes_per_rank` per rank.
// Collective: every rank must pass the same size.  Returns false (on every rank alike) when peer
// mapping is not available or WG_PEER_EXCHANGE=0; the caller then exchanges through NCCL.
bool ensure_peer_arena(wholegraph_comm_* comm, size_t bytes_per_rank, cudaStream_t stream);
// Region of `rank` as mapped into this process.
char* peer_arena_region(wholegraph_comm_* comm, int rank);

// WG_TIMING=1: distributed ops record CUDA events at their phase boundaries and print the phase
// durations when they return (this synchronises the stream; diagnosis only).
struct phase_timer {
  bool on;
  cudaStream_t stream;
  std::vector<std::pair<const char*, cudaEvent_t>> marks;
  explicit phase_timer(cudaStream_t s) : stream(s)
  {
    const char* e = getenv("WG_TIMING");
    on            = e != nullptr && e[0] == '1';
  }
  void mark(const char* name)
  {
    if (!on) return;
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, stream);
    marks.push_back({name, e});
  }
  ~phase_timer()
  {
    if (!on || marks.empty()) return;
    cudaStreamSynchronize(stream);
    std::string line;
    for (size_t i = 1; i < marks.size(); i++) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, marks[i - 1].second, marks[i].second);
      line += format_string(" %s=%.3f", marks[i].first, ms);
    }
    float total = 0.f;
    cudaEventElapsedTime(&total, marks.front().second, marks.back().second);
    fprintf(stderr, "[wholegraph timing]%s total=%.3f ms\n", line.c_str(), total);
    for (auto& m : marks) cudaEventDestroy(m.second);
  }
};

// First row of every rank's shard (world + 1 entries) for rows of `entry_bytes` bytes.
std::vector<int64_t> entry_offsets_of(wholegraph_handle_* h, size_t entry_bytes);

}  // namespace wgb
