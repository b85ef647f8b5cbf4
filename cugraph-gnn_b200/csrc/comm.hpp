// Communicator: one NCCL communicator per wholegraph_comm_ (none when world_size == 1),
// plus the small host-side collectives the handle and embedding code need.
// Role of the reference's cpp/src/wholegraph/communicator.cpp:255-810 and nccl_comms.cpp.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include <wholegraph/wholegraph.h>

struct wholegraph_handle_;

namespace wgb {

// Switches of the distributed ops, read from the environment when a communicator is created
// (and again by reload_tuning).  Every rank of a communicator must hold the same values, because
// they select which collectives an op issues; creation checks that.
struct exchange_tuning {
  int peer_exchange   = 1;  // WG_PEER_EXCHANGE=0: rows travel by NCCL instead of peer stores
  int gather_dedup    = 1;  // WG_GATHER_DEDUP=0: duplicates are routed as they are
  int gradient_presum = 1;  // WG_GRADIENT_PRESUM=0: every gradient row goes to its owner
  int peer_gradient   = 0;  // WG_PEER_GRADIENT=1: gradient sums are stored into the owner's arena
  int exchange_chunks = 0;  // WG_EXCHANGE_CHUNKS=k: chunks of a pipelined NCCL exchange (0: automatic)
  int sync_free       = 1;  // WG_SYNC_FREE=0: distributed gathers exchange their counts through the host
  int serve_bulk      = 1;  // WG_SERVE_BULK=0: the owner-side kernel of a distributed gather moves rows through
                            // registers with 16-byte peer stores instead of bulk asynchronous copies through
                            // shared memory (one store per tile of 32 rows)
  int single_rank_exchange = 0;  // WG_SINGLE_RANK_EXCHANGE=1: a one-rank communicator runs the exchange code of the
                                 // distributed ops (with itself as its only peer) instead of the direct kernels,
                                 // so that this code can be tested on one GPU
};
exchange_tuning tuning_from_environment();

}  // namespace wgb

struct wholegraph_comm_ {
  int world_rank = 0;
  int world_size = 1;
  int dev_id     = 0;
  void* nccl     = nullptr;  // ncclComm_t; null for a single-rank communicator
  wholegraph_distributed_backend_t backend = WHOLEGRAPH_DB_NCCL;
  std::mutex mu;
  std::set<wholegraph_handle_*> handles;  // freed when the communicator is destroyed
  int next_handle_id = 0;
  uint64_t tag       = 0;  // identical on all ranks; names the side-band unix sockets
  wgb::exchange_tuning tuning;
  // Read the tuning variables again and check that all ranks agree (collective, blocking).
  void reload_tuning();

  // Staging for host-side collectives (1 MiB per rank).
  cudaStream_t side_stream = nullptr;
  void* dev_stage          = nullptr;
  void* pin_stage          = nullptr;
  size_t stage_bytes       = 0;

  // Second stream on which the row exchange of a distributed op runs while the caller's
  // stream keeps gathering, and the events that fence the two.
  cudaStream_t xchg_stream = nullptr;
  std::vector<cudaEvent_t> events;
  cudaEvent_t event(size_t i);  // i-th pooled event (created on demand, timing disabled)

  // Peer-mapped exchange arena: a CONTINUOUS/DEVICE allocation with one region of arena_bytes
  // per rank, mapped on every rank, into which owners write the rows a rank asked for (and
  // senders their gradient sums) with plain stores over NVLink.  Created on first use and grown
  // collectively; null when peer mapping is not available (then every exchange goes through NCCL).
  wholegraph_handle_* arena = nullptr;
  size_t arena_bytes        = 0;
  bool arena_unavailable    = false;
  cudaEvent_t arena_idle    = nullptr;  // this rank's last read of its own region
  int* barrier_word         = nullptr;  // device word of stream_barrier
  int* status_word          = nullptr;  // device word a kernel sets when it refuses peer-provided sizes or ids
  int* status_host          = nullptr;  // pinned copy of status_word, refreshed after every call that uses it

  // Host-to-host board in POSIX shared memory (ranks of one node only): every rank posts a few
  // numbers per collective call and reads everybody's, without touching a CUDA stream, so that
  // an op can agree on sizes while the GPUs are still busy with earlier work.  Null when the
  // ranks cannot share memory; callers then fall back to a stream-synchronising exchange.
  struct host_board;
  host_board* board = nullptr;
  static constexpr int kBoardValues = 6;
  // Post `mine` (kBoardValues numbers) and return every rank's numbers, rank-major, in `all`
  // (world_size * kBoardValues).  Collective: every rank calls it the same number of times, in
  // the same order.  Blocks the host until all ranks have posted (60 s limit, then comm_error).
  void board_exchange(const int64_t* mine, int64_t* all);

  // ---- host collectives (blocking; caller memory is pageable host memory) ----
  void host_allgather(const void* send, void* recv, size_t bytes_per_rank);
  void host_alltoall(const void* send, void* recv, size_t bytes_per_pair);
  void barrier();
  // True when every rank passed the same bytes.
  bool all_same(const void* value, size_t bytes);

  // ---- device collectives, asynchronous on `stream` ----
  // Byte alltoallv: send_counts / recv_counts / displacements in units of `unit_bytes`.
  void alltoallv(const void* send, const int64_t* send_counts, const int64_t* send_displs,
                 void* recv, const int64_t* recv_counts, const int64_t* recv_displs,
                 size_t unit_bytes, cudaStream_t stream);
  // Any number of sends and receives of raw bytes in ONE NCCL group, so that all peers move
  // data at the same time (empty transfers are skipped; transfers to this rank are not allowed).
  struct transfer {
    void* ptr;
    size_t bytes;
    int peer;
  };
  void exchange(const std::vector<transfer>& sends, const std::vector<transfer>& recvs,
                cudaStream_t stream);
  // One send and one receive of raw bytes in a single NCCL group (either may be empty).
  void sendrecv(const void* send, size_t send_bytes, int to, void* recv, size_t recv_bytes,
                int from, cudaStream_t stream);
  // Fixed-size alltoall of device buffers.
  void alltoall(const void* send, void* recv, size_t bytes_per_pair, cudaStream_t stream);
  // Fixed-size allgather of device buffers.
  void allgather(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream);
  // Barrier in stream order: work enqueued on `stream` after it starts only when every rank's
  // work enqueued before it has finished (no host synchronisation).
  void stream_barrier(cudaStream_t stream);
  // Poll the communicator for an asynchronous error; throws comm_error.
  void check_async_error();
};

namespace wgb {

void nccl_get_unique_id(wholegraph_unique_id_t* id);
wholegraph_comm_* create_comm(const wholegraph_unique_id_t& id, int rank, int size);
wholegraph_comm_* split_comm(wholegraph_comm_* comm, int color, int key);
void destroy_comm(wholegraph_comm_* comm);
void destroy_all_comms();

}  // namespace wgb
