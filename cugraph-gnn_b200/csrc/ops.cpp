// wholegraph_gather / wholegraph_scatter: argument checks, mapped (direct pointer) path and
// the distributed path.
//
// Reference behaviour: cpp/src/wholegraph_tensor_ops/gather_op.cpp:12-106, scatter_op.cpp:12-98,
// gather_op_impl_nccl.cu:23-171, scatter_op_impl_nccl.cu:23-170.  The distributed gather here
// routes distinct ids only; one allgather gives every rank the whole count matrix and one host
// synchronisation (NCCL needs host counts) replaces the reference's three.  Rows then travel
// either by plain stores of the owner's gather kernel into the requester's region of a
// peer-mapped arena, or, where that is not available, through NCCL in pipelined chunks on a
// second stream.
#include "ops.hpp"

#include <algorithm>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

#include <wholegraph/wholegraph_b200.h>
#include <wholegraph/wholegraph_tensor_op.h>

#include "common.hpp"
#include "env.hpp"
#include "handle.hpp"
#include "kernels/cache.hpp"
#include "kernels/partition.hpp"
#include "kernels/row_copy.hpp"
#include "kernels/serve_rows.hpp"
#include "kernels/unique_ids.hpp"
#include "tensor.hpp"

namespace wgb {

// ---- exchange plan -------------------------------------------------------------------------

exchange_plan::exchange_plan(wholegraph_env_func_t* env)
  : workspace(env), sorted_ids_buf(env), positions_buf(env), recv_ids_buf(env), counts_dev(env),
    counts_pin(env), matrix_dev(env)
{
}

void exchange_plan::build(const void* ids, bool ids_are_64, int64_t n,
                          const std::vector<int64_t>& first_row, wholegraph_comm_* comm,
                          cudaStream_t stream, bool dedup)
{
  world = comm->world_size;
  me    = comm->world_rank;
  count = n;
  send_counts.assign(world, 0);
  send_displs.assign(world, 0);
  recv_counts.assign(world, 0);
  recv_displs.assign(world, 0);

  sorted_ids = static_cast<int64_t*>(sorted_ids_buf.device(n, WHOLEGRAPH_DT_INT64));
  positions  = static_cast<int64_t*>(positions_buf.device(n, WHOLEGRAPH_DT_INT64));
  // Device layout: [send counts | send starts | recv counts], world entries each.
  int64_t* cdev = static_cast<int64_t*>(counts_dev.device(3 * world, WHOLEGRAPH_DT_INT64));
  if (dedup) {
    void* ws = workspace.device_bytes(unique_workspace_bytes(n, first_row[world]));
    inverse  = positions;  // same storage, other meaning
    unique_by_owner(ids, ids_are_64, n, first_row.data(), world, ws, sorted_ids, inverse, cdev, cdev + world,
                    stream);
    positions = nullptr;
  } else {
    void* ws = workspace.device_bytes(partition_workspace_bytes(n, world));
    partition_by_owner(ids, ids_are_64, n, first_row.data(), world, ws, sorted_ids, positions, cdev,
                       cdev + world, stream);
  }
  exchange_counts_and_ids(cdev, comm, stream);
}

void exchange_plan::build_grouped(int64_t* grouped_ids, int64_t* group_counts_dev, wholegraph_comm_* comm,
                                  cudaStream_t stream)
{
  world = comm->world_size;
  me    = comm->world_rank;
  send_counts.assign(world, 0);
  send_displs.assign(world, 0);
  recv_counts.assign(world, 0);
  recv_displs.assign(world, 0);
  sorted_ids = grouped_ids;
  positions  = nullptr;
  exchange_counts_and_ids(group_counts_dev, comm, stream);
  count = total_send;
}

void exchange_plan::exchange_counts_and_ids(int64_t* cdev, wholegraph_comm_* comm, cudaStream_t stream)
{
  // Every rank learns every rank's per-owner counts (world * world numbers) in one allgather.
  int64_t* mdev = static_cast<int64_t*>(matrix_dev.device(static_cast<size_t>(world) * world, WHOLEGRAPH_DT_INT64));
  int64_t* mpin = static_cast<int64_t*>(counts_pin.pinned(static_cast<size_t>(world) * world, WHOLEGRAPH_DT_INT64));
  comm->allgather(cdev, mdev, sizeof(int64_t) * world, stream);
  WGB_CUDA_CHECK(cudaMemcpyAsync(mpin, mdev, sizeof(int64_t) * world * world, cudaMemcpyDeviceToHost, stream));
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));  // the one host sync of a distributed op
  comm->check_async_error();
  rows.assign(mpin, mpin + static_cast<size_t>(world) * world);
  total_send = total_recv = 0;
  for (int r = 0; r < world; r++) {
    send_counts[r] = rows[static_cast<size_t>(me) * world + r];
    send_displs[r] = total_send;
    recv_counts[r] = rows[static_cast<size_t>(r) * world + me];
    recv_displs[r] = total_recv;
    total_send += send_counts[r];
    total_recv += recv_counts[r];
  }
  recv_ids = static_cast<int64_t*>(recv_ids_buf.device(total_recv, WHOLEGRAPH_DT_INT64));
  comm->alltoallv(sorted_ids, send_counts.data(), send_displs.data(), recv_ids, recv_counts.data(),
                  recv_displs.data(), sizeof(int64_t), stream);
}

int64_t exchange_plan::group_start(int q, int r) const
{
  int64_t s = 0;
  for (int k = 0; k < r; k++) s += rows[static_cast<size_t>(q) * world + k];
  return s;
}

int64_t exchange_plan::arrival_start(int q, int r) const
{
  int64_t s = 0;
  for (int k = 0; k < q; k++) s += rows[static_cast<size_t>(k) * world + r];
  return s;
}

int64_t exchange_plan::max_total_send() const
{
  int64_t best = 0;
  for (int q = 0; q < world; q++) best = std::max(best, group_start(q, world));
  return best;
}

int64_t exchange_plan::max_total_recv() const
{
  int64_t best = 0;
  for (int r = 0; r < world; r++) best = std::max(best, arrival_start(world, r));
  return best;
}

bool ensure_peer_arena(wholegraph_comm_* comm, size_t bytes_per_rank, cudaStream_t stream)
{
  if ((comm->world_size == 1 && !comm->tuning.single_rank_exchange) || comm->arena_unavailable ||
      !comm->tuning.peer_exchange)
    return false;
  if (comm->arena_idle == nullptr)
    WGB_CUDA_CHECK(cudaEventCreateWithFlags(&comm->arena_idle, cudaEventDisableTiming));
  if (comm->arena != nullptr && comm->arena_bytes >= bytes_per_rank) return true;
  // (Re)create, with head room.  Every rank takes this branch together: the size is the same
  // everywhere and so is the current arena.  No peer touches the old regions any more: each
  // rank has passed the stream barrier that ended the last exchange through them.
  constexpr size_t kUnit = size_t(64) << 20;
  const size_t want      = (std::max(bytes_per_rank + bytes_per_rank / 4, size_t(256) << 20) + kUnit - 1) / kUnit * kUnit;
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
  int ok = 1;
  try {
    if (comm->arena != nullptr) {
      destroy_handle(comm->arena);
      comm->arena = nullptr, comm->arena_bytes = 0;
    }
    comm->arena = create_handle(want * comm->world_size, comm, WHOLEGRAPH_MT_CONTINUOUS, WHOLEGRAPH_ML_DEVICE, want,
                                nullptr);
    comm->arena_bytes = want;
  } catch (const std::exception& ex) {
    WGB_WARN("no peer-mapped exchange arena (%s): distributed ops keep to NCCL", ex.what());
    ok = 0;
  }
  std::vector<int> all(comm->world_size, 0);
  comm->host_allgather(&ok, all.data(), sizeof(int));
  for (int v : all) ok &= v;
  if (!ok) {
    if (comm->arena != nullptr) {
      try {
        destroy_handle(comm->arena);
      } catch (...) {
      }
    }
    comm->arena = nullptr, comm->arena_bytes = 0, comm->arena_unavailable = true;
    return false;
  }
  return true;
}

char* peer_arena_region(wholegraph_comm_* comm, int rank)
{
  return static_cast<char*>(comm->arena->global_base) + comm->arena->part_offsets[rank];
}

int exchange_chunk_count(const int64_t* matrix, int world, size_t row_bytes, int wanted, int forced)
{
  if (forced > 0) return std::min(forced, 16);
  if (wanted > 0) return std::min(wanted, 16);
  // The busiest rank decides for everybody: rows leaving or reaching one rank, its own left out.
  int64_t busiest = 0;
  for (int q = 0; q < world; q++) {
    int64_t out = 0, in = 0;
    for (int r = 0; r < world; r++) {
      if (r == q) continue;
      out += matrix[static_cast<size_t>(q) * world + r];
      in += matrix[static_cast<size_t>(r) * world + q];
    }
    busiest = std::max(busiest, std::max(out, in));
  }
  return static_cast<size_t>(busiest) * row_bytes < (size_t(16) << 20) ? 1 : 4;
}

int exchange_plan::chunk_count(size_t row_bytes, int wanted, int forced) const
{
  return exchange_chunk_count(rows.data(), world, row_bytes, wanted, forced);
}

void pipelined_exchange(wholegraph_comm_* comm, const std::vector<int64_t>& out_counts,
                        const std::vector<int64_t>& out_displs, const std::vector<int64_t>& in_counts,
                        const std::vector<int64_t>& in_displs, char* out_buf, char* in_buf,
                        size_t row_bytes, cudaStream_t stream,
                        const std::function<void(const list_segments&)>& pack,
                        const std::function<void(const list_segments&)>& unpack, int K)
{
  const int W = comm->world_size, me = comm->world_rank;
  WGB_EXPECTS(K >= 1 && K <= 16, "an exchange runs in 1 to 16 chunks, not %d", K);
  cudaStream_t xs = comm->xchg_stream;
  auto cut        = [K](int64_t c, int k, int64_t* b, int64_t* n) {
    *b = c * k / K;
    *n = c * (k + 1) / K - *b;
  };
  auto segments_of = [&](const std::vector<int64_t>& counts, const std::vector<int64_t>& displs, int k) {
    list_segments seg;
    for (int step = 1; step < W; step++) {
      const int p = (me + step) % W;
      int64_t b, n;
      cut(counts[p], k, &b, &n);
      seg.add(displs[p] + b, n);
    }
    return seg;
  };
  for (int k = 0; k < K; k++) {
    const list_segments out_seg = segments_of(out_counts, out_displs, k);
    if (out_seg.n > 0) pack(out_seg);
    WGB_CUDA_CHECK(cudaEventRecord(comm->event(2 * k), stream));
    WGB_CUDA_CHECK(cudaStreamWaitEvent(xs, comm->event(2 * k), 0));
    std::vector<wholegraph_comm_::transfer> sends, recvs;
    for (int step = 1; step < W; step++) {
      const int to = (me + step) % W, from = (me - step + W) % W;
      int64_t b, n;
      cut(out_counts[to], k, &b, &n);
      sends.push_back({out_buf + (out_displs[to] + b) * row_bytes, static_cast<size_t>(n) * row_bytes, to});
      cut(in_counts[from], k, &b, &n);
      recvs.push_back({in_buf + (in_displs[from] + b) * row_bytes, static_cast<size_t>(n) * row_bytes, from});
    }
    comm->exchange(sends, recvs, xs);
    WGB_CUDA_CHECK(cudaEventRecord(comm->event(2 * k + 1), xs));
    if (k > 0) {  // overlaps with the exchange just enqueued
      WGB_CUDA_CHECK(cudaStreamWaitEvent(stream, comm->event(2 * (k - 1) + 1), 0));
      const list_segments in_seg = segments_of(in_counts, in_displs, k - 1);
      if (in_seg.n > 0) unpack(in_seg);
    }
  }
  WGB_CUDA_CHECK(cudaStreamWaitEvent(stream, comm->event(2 * (K - 1) + 1), 0));
  const list_segments in_seg = segments_of(in_counts, in_displs, K - 1);
  if (in_seg.n > 0) unpack(in_seg);
}

std::vector<int64_t> entry_offsets_of(wholegraph_handle_* h, size_t entry_bytes)
{
  std::vector<int64_t> first(h->part_offsets.size());
  for (size_t i = 0; i < first.size(); i++) {
    WGB_EXPECTS(h->part_offsets[i] % entry_bytes == 0,
                "shard offset %zu of rank %zu is not a multiple of the row size %zu",
                h->part_offsets[i], i, entry_bytes);
    first[i] = static_cast<int64_t>(h->part_offsets[i] / entry_bytes);
  }
  return first;
}

namespace {

struct matrix_view {
  void* ptr;  // element 0 of the storage (offset not applied)
  wholegraph_matrix_description_t d;
};

// 1-D tensors are [N, 1] matrices (reference: gather_op.cpp:33-38, :53-58).
bool as_matrix(wholegraph_tensor_t t, wholegraph_matrix_description_t* m)
{
  wholegraph_tensor_description_t d = *wholegraph_tensor_get_tensor_description(t);
  if (d.dim != 1 && d.dim != 2) return false;
  if (d.dim == 1 && !wholegraph_unsqueeze_tensor(&d, 1)) return false;
  return wholegraph_convert_tensor_desc_to_matrix(m, &d);
}

void fill_chunks(chunked_table* c, wholegraph_handle_* h, size_t entry_bytes)
{
  int W = h->comm->world_size;
  WGB_EXPECTS(W <= kMaxChunkedRanks, "CHUNKED memory supports up to %d ranks", kMaxChunkedRanks);
  auto first = entry_offsets_of(h, entry_bytes);
  c->ranks   = W;
  for (int r = 0; r < W; r++) {
    c->base[r]      = h->rank_ptrs[r];
    c->first_row[r] = first[r];
  }
  c->first_row[W] = first[W];
}

// A pointer such that row `first_local_row` of the global numbering lands on local_ptr
// (reference: gather_op_impl_nccl.cu:111-115).
const void* fake_global_base(wholegraph_handle_* h)
{
  return static_cast<const char*>(h->local_ptr) - h->part_offsets[h->comm->world_rank];
}

struct table_side {
  const void* base = nullptr;
  chunked_table chunks;
};

}  // namespace

// ---- distributed gather without host-side counts --------------------------------------------
namespace {

// Layout of a rank's region of the exchange arena during such a gather.
constexpr size_t kRegionHeaderBytes = 2 * sizeof(int64_t) * kMaxServeRanks;  // counts | starts
size_t region_ids_offset() { return kRegionHeaderBytes; }
size_t region_rows_offset(int64_t capacity) { return kRegionHeaderBytes + (static_cast<size_t>(capacity) * 8 + 255) / 256 * 256; }
size_t region_bytes(int64_t capacity, size_t row_bytes)
{
  return region_rows_offset(capacity) + static_cast<size_t>(capacity) * row_bytes;
}

}  // namespace

// Distinct ids only, and nothing about them ever reaches the host: every rank leaves its distinct
// ids (grouped by owner) and the W group sizes in its own region of the peer-mapped arena; after a
// barrier in stream order every owner reads, for each requester, "how many ids do you ask of me
// and where do they start" from that requester's region and stores the rows into the same
// region (one kernel: peer loads of ids, local loads of rows, peer stores); after a second barrier
// the requester expands the rows into its output, casting to the output dtype there.  The hosts
// agree on the region size through the communicator's shared-memory board (request lengths are
// host data), which synchronises hosts with hosts but no host with a GPU.  Returns false when
// this path does not apply (no board, no arena, tuning), before anything was enqueued and on
// every rank alike.
static bool gather_distributed_sync_free(wholegraph_handle_* h, const wholegraph_matrix_description_t& tab,
                                         const std::vector<int64_t>& first_row, const void* ids, bool ids_are_64,
                                         int64_t n, void* out, const wholegraph_matrix_description_t& od,
                                         wholegraph_env_func_t* env, cudaStream_t stream, int sms)
{
  auto* comm          = h->comm;
  const int W         = comm->world_size;
  const int me        = comm->world_rank;
  const size_t es_tab = wholegraph_dtype_get_element_size(tab.dtype);
  const size_t es_out = wholegraph_dtype_get_element_size(od.dtype);
  const int64_t dim   = tab.sizes[1];
  // Rows travel as they are stored; where that would put more bytes on the wire than casting at
  // the owner (a narrower output dtype), the other path is taken.
  if (!comm->tuning.sync_free || !comm->tuning.peer_exchange || (comm->board == nullptr && W > 1) ||
      comm->arena_unavailable || W > kMaxServeRanks || es_tab > es_out)
    return false;
  const size_t row_b = static_cast<size_t>(dim) * es_tab;

  // Hosts agree on the largest request and check that they are in the same call.
  int64_t mine[wholegraph_comm_::kBoardValues] = {n, static_cast<int64_t>(row_b), static_cast<int64_t>(h->id),
                                                  static_cast<int64_t>(tab.dtype) * 16 + static_cast<int64_t>(od.dtype),
                                                  unique_supported(n, first_row[W]) ? 1 : 0, 0x67617468 /* "gath" */};
  std::vector<int64_t> all(static_cast<size_t>(W) * wholegraph_comm_::kBoardValues);
  comm->board_exchange(mine, all.data());
  int64_t capacity = 1;
  bool supported   = true;
  for (int r = 0; r < W; r++) {
    const int64_t* v = all.data() + static_cast<size_t>(r) * wholegraph_comm_::kBoardValues;
    WGB_EXPECTS(v[1] == mine[1] && v[2] == mine[2] && v[3] == mine[3] && v[5] == mine[5],
                "rank %d is in another collective call than rank %d (distributed gather)", r, me);
    capacity  = std::max(capacity, v[0]);
    supported = supported && v[4] != 0;
  }
  if (!supported) return false;
  if (!ensure_peer_arena(comm, region_bytes(capacity, row_b), stream)) return false;
  // The arena is usually larger than asked for: every rank derives the same capacity from its size.
  {
    int64_t most = (static_cast<int64_t>(comm->arena_bytes) - static_cast<int64_t>(kRegionHeaderBytes) - 256) /
                   static_cast<int64_t>(row_b + 8);
    most = std::min<int64_t>(most, (int64_t(1) << 31) - 2);
    while (most > capacity && region_bytes(most, row_b) > comm->arena_bytes) most--;
    capacity = std::max(capacity, most);
  }
  if (comm->status_word == nullptr) {
    WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&comm->status_word), 256));
    WGB_CUDA_CHECK(cudaMemset(comm->status_word, 0, 256));
    WGB_CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&comm->status_host), 64));
    *comm->status_host = 0;
  }
  // An earlier call's kernel may have refused a header or an id: the word is copied to the host
  // after every call and looked at, without waiting, at the next one.
  if (*comm->status_host != 0) {
    const int code     = *comm->status_host;
    *comm->status_host = 0;
    WGB_CUDA_CHECK(cudaMemsetAsync(comm->status_word, 0, sizeof(int), stream));
    throw comm_error(format_string("an earlier distributed gather %s",
                                   code == 1   ? "refused a request header that did not fit its region"
                                   : code == 2 ? "refused ids outside the shard they were sent to"
                                               : "gave up waiting for its own bulk copies"));
  }

  phase_timer timer(stream);
  timer.mark("start");
  char* my_region     = peer_arena_region(comm, me);
  int64_t* my_header  = reinterpret_cast<int64_t*>(my_region);
  int64_t* my_ids     = reinterpret_cast<int64_t*>(my_region + region_ids_offset());
  char* my_rows       = my_region + region_rows_offset(capacity);
  temp_buffer workspace(env), inverse_buf(env);
  int64_t* inverse = static_cast<int64_t*>(inverse_buf.device(std::max<int64_t>(n, 1), WHOLEGRAPH_DT_INT64));
  void* ws         = workspace.device_bytes(unique_workspace_bytes(n, first_row[W]));
  unique_by_owner(ids, ids_are_64, n, first_row.data(), W, ws, my_ids, inverse, my_header, my_header + W, stream,
                  /*ascending=*/false);
  timer.mark("unique");
  comm->stream_barrier(stream);  // every rank's header and ids are in place
  timer.mark("barrier");

  serve_rows_args s;
  s.world = W, s.me = me;
  for (int r = 0; r < W; r++) {
    char* region       = peer_arena_region(comm, r);
    s.region[r].header = reinterpret_cast<const int64_t*>(region);
    s.region[r].ids    = reinterpret_cast<const int64_t*>(region + region_ids_offset());
    s.region[r].rows   = region + region_rows_offset(capacity);
  }
  s.capacity           = capacity;
  s.first_local_row    = first_row[me];
  s.local_rows         = first_row[me + 1] - first_row[me];
  s.shard              = static_cast<const char*>(h->local_ptr) + tab.storage_offset * es_tab;
  s.shard_stride_bytes = tab.stride * static_cast<int64_t>(es_tab);
  s.row_bytes          = static_cast<int64_t>(row_b);
  s.status             = comm->status_word;
  s.bulk               = comm->tuning.serve_bulk != 0;
  int64_t bound        = 0;  // a requester asks one owner for at most as many rows as its list is long
  for (int r = 0; r < W; r++)
    bound += std::min(all[static_cast<size_t>(r) * wholegraph_comm_::kBoardValues], s.local_rows);
  s.rows_upper_bound = bound;
  launch_serve_rows(s, stream);
  timer.mark("serve");
  comm->stream_barrier(stream);  // every owner's rows have landed
  timer.mark("barrier");

  if (n > 0) {
    row_copy_args expand;  // rows[inverse[i]] -> output row i, cast here; ids nobody owns leave their row untouched
    expand.src = my_rows, expand.src_dt = tab.dtype, expand.src_stride = dim, expand.src_select = ROW_BY_INDEX;
    expand.dst = out, expand.dst_dt = od.dtype, expand.dst_stride = od.stride, expand.dst_offset = od.storage_offset;
    expand.dst_select = ROW_SEQUENTIAL, expand.dim = dim, expand.sm_hint = sms;
    expand.indices = inverse, expand.indices_are_64 = true, expand.count = n;
    launch_row_copy(expand, stream);
  }
  WGB_CUDA_CHECK(cudaMemcpyAsync(comm->status_host, comm->status_word, sizeof(int), cudaMemcpyDeviceToHost, stream));
  if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaEventRecord(comm->arena_idle, stream));
  timer.mark("expand");
  return true;
}

// ---- distributed gather ----------------------------------------------------------------------
void gather_distributed(wholegraph_handle_* h, const wholegraph_matrix_description_t& tab,
                        const void* ids, bool ids_are_64, int64_t n, void* out,
                        const wholegraph_matrix_description_t& od, wholegraph_env_func_t* env,
                        cudaStream_t stream, int sms, const cache_view* cache, bool adjust_cache)
{
  WGB_EXPECTS(tab.storage_offset >= 0 && tab.storage_offset + tab.sizes[1] <= tab.stride,
              "distributed gather needs storage_offset + dim <= stride");
  auto* comm           = h->comm;
  const int W          = comm->world_size;
  const int me         = comm->world_rank;
  const size_t es_tab  = wholegraph_dtype_get_element_size(tab.dtype);
  const size_t es_out  = wholegraph_dtype_get_element_size(od.dtype);
  const int64_t dim    = tab.sizes[1];
  const size_t row_b   = static_cast<size_t>(dim) * es_out;
  auto first_row       = entry_offsets_of(h, es_tab * static_cast<size_t>(tab.stride));
  const void* fake_tab = fake_global_base(h);

  row_copy_args g;  // local shard -> rows, by index
  g.src = fake_tab, g.src_dt = tab.dtype, g.src_stride = tab.stride, g.src_offset = tab.storage_offset;
  g.src_select = ROW_BY_INDEX;
  g.dst_dt = od.dtype, g.dim = dim, g.indices_are_64 = true, g.sm_hint = sms;

  temp_buffer cache_ws(env), address_buf(env);
  if (W == 1 && !(comm->tuning.single_rank_exchange && cache == nullptr)) {
    g.dst = out, g.dst_stride = od.stride, g.dst_offset = od.storage_offset;
    g.indices = ids, g.indices_are_64 = ids_are_64, g.count = n;
    if (cache != nullptr) {
      if (adjust_cache)
        cache_update(ids, ids_are_64, n, *cache, cache_ws.device_bytes(cache_update_workspace_bytes(n)), stream);
      auto* addr = static_cast<int64_t*>(address_buf.device(n, WHOLEGRAPH_DT_INT64));
      cache_lookup(ids, ids_are_64, n, *cache, false, addr, stream);
      g.src_select = ROW_BY_ADDRESS, g.indices = addr, g.indices_are_64 = true;
    }
    launch_row_copy(g, stream);
    return;
  }

  // A call on another stream may still be reading this rank's arena region.
  if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaStreamWaitEvent(stream, comm->arena_idle, 0));
  if (cache == nullptr && comm->tuning.gather_dedup &&
      gather_distributed_sync_free(h, tab, first_row, ids, ids_are_64, n, out, od, env, stream, sms))
    return;
  phase_timer timer(stream);
  timer.mark("start");
  exchange_plan plan(env);
  // WG_GATHER_DEDUP=0 routes every request, duplicates included, as the reference does.
  const bool dedup = cache == nullptr && comm->tuning.gather_dedup && unique_supported(n, first_row[W]);
  plan.build(ids, ids_are_64, n, first_row, comm, stream, dedup);
  timer.mark(dedup ? "unique+counts+ids" : "partition+counts+ids");

  if (dedup) {
    // Distinct ids only: owners serve each row once into `rows` (own rows are gathered into
    // their slots locally), then one local gather expands them into the output.
    // Where the arena is available the owners write the rows straight into the requester's
    // region over NVLink (gather, cast and transfer in one kernel per requester); otherwise they
    // pack them and NCCL moves them.
    const bool peer = ensure_peer_arena(comm, static_cast<size_t>(plan.max_total_send()) * row_b, stream);
    temp_buffer serve_buf(env), rows_buf(env);
    char* rows = peer ? peer_arena_region(comm, me)
                      : static_cast<char*>(rows_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));
    row_copy_args from_shard = g;  // local shard -> dense rows, by index, cast at the owner
    from_shard.dst_stride = dim, from_shard.dst_offset = 0, from_shard.dst_select = ROW_SEQUENTIAL;
    if (plan.send_counts[me] > 0) {
      row_copy_args a = from_shard;
      a.dst = rows, a.indices = plan.sorted_ids;
      a.segments.add(plan.send_displs[me], plan.send_counts[me]);
      a.count = a.segments.total();
      launch_row_copy(a, stream);
    }
    timer.mark("own_rows");
    if (peer) {
      // No requester still reads its region from an earlier call: it joined this call's counts
      // exchange, which this stream has passed, only after that read.
      for (int step = 1; step < W; step++) {
        const int q = (me + step) % W;
        if (plan.recv_counts[q] == 0) continue;
        row_copy_args a = from_shard;
        a.dst     = peer_arena_region(comm, q) + plan.group_start(q, me) * row_b;
        a.indices = plan.recv_ids + plan.recv_displs[q];
        a.count   = plan.recv_counts[q];
        launch_row_copy(a, stream);
      }
      comm->stream_barrier(stream);  // every owner's rows have landed
    } else {
      char* serve = static_cast<char*>(serve_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));
      pipelined_exchange(
        comm, plan.recv_counts, plan.recv_displs, plan.send_counts, plan.send_displs, serve, rows, row_b, stream,
        [&](const list_segments& seg) {
          row_copy_args a = from_shard;
          a.dst = serve, a.indices = plan.recv_ids;
          a.segments = seg, a.count = seg.total();
          launch_row_copy(a, stream);
        },
        [](const list_segments&) {}, plan.chunk_count(row_b, 1, comm->tuning.exchange_chunks));
    }
    timer.mark("exchange");
    row_copy_args expand;  // rows[inverse[i]] -> output row i; ids nobody owns leave their row untouched
    expand.src = rows, expand.src_dt = od.dtype, expand.src_stride = dim, expand.src_select = ROW_BY_INDEX;
    expand.dst = out, expand.dst_dt = od.dtype, expand.dst_stride = od.stride, expand.dst_offset = od.storage_offset;
    expand.dst_select = ROW_SEQUENTIAL, expand.dim = dim, expand.sm_hint = sms;
    expand.indices = plan.inverse, expand.indices_are_64 = true, expand.count = n;
    launch_row_copy(expand, stream);
    if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaEventRecord(comm->arena_idle, stream));
    timer.mark("expand");
    return;
  }

  temp_buffer serve_buf(env), recv_buf(env);
  char* serve = static_cast<char*>(serve_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));
  char* recv  = static_cast<char*>(recv_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));

  // With a cache, every id this rank serves (its own requests included: they are part of
  // recv_ids) is resolved to the address of the row's current copy first.
  const int64_t* serve_index = plan.recv_ids;
  if (cache != nullptr && plan.total_recv > 0) {
    if (adjust_cache)
      cache_update(plan.recv_ids, true, plan.total_recv, *cache,
                   cache_ws.device_bytes(cache_update_workspace_bytes(plan.total_recv)), stream);
    auto* addr = static_cast<int64_t*>(address_buf.device(plan.total_recv, WHOLEGRAPH_DT_INT64));
    cache_lookup(plan.recv_ids, true, plan.total_recv, *cache, false, addr, stream);
    serve_index  = addr;
    g.src_select = ROW_BY_ADDRESS;
  }

  // Step 0: rows this rank owns go straight from the shard to their final output rows.
  {
    row_copy_args a = g;
    a.dst = out, a.dst_stride = od.stride, a.dst_offset = od.storage_offset;
    a.dst_select = ROW_BY_POSITION;
    a.indices    = cache != nullptr ? serve_index + plan.recv_displs[me] : plan.sorted_ids + plan.send_displs[me];
    a.positions  = plan.positions + plan.send_displs[me];
    a.count      = plan.send_counts[me];
    launch_row_copy(a, stream);
  }
  timer.mark("own_rows");
  row_copy_args reorder;  // received rows -> output rows, by position
  reorder.src = recv, reorder.src_dt = od.dtype, reorder.src_stride = dim, reorder.src_select = ROW_SEQUENTIAL;
  reorder.dst = out, reorder.dst_dt = od.dtype, reorder.dst_stride = od.stride;
  reorder.dst_offset = od.storage_offset, reorder.dst_select = ROW_BY_POSITION;
  reorder.dim = dim, reorder.sm_hint = sms, reorder.positions = plan.positions;

  row_copy_args serve_rows = g;  // rows other ranks asked for -> serve buffer, in their order
  serve_rows.dst = serve, serve_rows.dst_stride = dim, serve_rows.dst_offset = 0;
  serve_rows.dst_select = ROW_SEQUENTIAL, serve_rows.indices = serve_index;

  pipelined_exchange(
    comm, plan.recv_counts, plan.recv_displs, plan.send_counts, plan.send_displs, serve, recv, row_b, stream,
    [&](const list_segments& seg) {
      row_copy_args a = serve_rows;
      a.segments = seg, a.count = seg.total();
      launch_row_copy(a, stream);
    },
    [&](const list_segments& seg) {
      row_copy_args r = reorder;
      r.segments = seg, r.count = seg.total();
      launch_row_copy(r, stream);
    },
    plan.chunk_count(row_b, 0, comm->tuning.exchange_chunks));
  timer.mark("exchange+reorder");
}

namespace {

// ---- distributed scatter ---------------------------------------------------------------------
void scatter_distributed(const void* in, const wholegraph_matrix_description_t& id_,
                         const void* ids, bool ids_are_64, int64_t n, wholegraph_handle_* h,
                         const wholegraph_matrix_description_t& tab, wholegraph_env_func_t* env,
                         cudaStream_t stream, int sms)
{
  WGB_EXPECTS(tab.storage_offset >= 0 && tab.storage_offset + tab.sizes[1] <= tab.stride,
              "distributed scatter needs storage_offset + dim <= stride");
  auto* comm          = h->comm;
  const int W         = comm->world_size;
  const int me        = comm->world_rank;
  const size_t es_tab = wholegraph_dtype_get_element_size(tab.dtype);
  const size_t es_in  = wholegraph_dtype_get_element_size(id_.dtype);
  const int64_t dim   = tab.sizes[1];
  const size_t row_b  = static_cast<size_t>(dim) * es_in;  // rows travel in the input dtype
  auto first_row      = entry_offsets_of(h, es_tab * static_cast<size_t>(tab.stride));
  void* fake_tab      = const_cast<void*>(fake_global_base(h));

  row_copy_args put;  // rows -> local shard, by index (cast to the table dtype happens here)
  put.src_dt = id_.dtype, put.dst = fake_tab, put.dst_dt = tab.dtype, put.dst_stride = tab.stride;
  put.dst_offset = tab.storage_offset, put.dst_select = ROW_BY_INDEX;
  put.dim = dim, put.indices_are_64 = true, put.sm_hint = sms;

  if (W == 1 && !comm->tuning.single_rank_exchange) {
    put.src = in, put.src_stride = id_.stride, put.src_offset = id_.storage_offset;
    put.indices = ids, put.indices_are_64 = ids_are_64, put.count = n;
    launch_row_copy(put, stream);
    WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
    return;
  }

  exchange_plan plan(env);
  plan.build(ids, ids_are_64, n, first_row, comm, stream);
  temp_buffer send_buf(env), recv_buf(env);
  char* send = static_cast<char*>(send_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));
  char* recv = static_cast<char*>(recv_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));

  {  // step 0: this rank's own rows
    row_copy_args a = put;
    a.src = in, a.src_stride = id_.stride, a.src_offset = id_.storage_offset;
    a.src_select = ROW_BY_POSITION;
    a.indices    = plan.sorted_ids + plan.send_displs[me];
    a.positions  = plan.positions + plan.send_displs[me];
    a.count      = plan.send_counts[me];
    launch_row_copy(a, stream);
  }
  row_copy_args pack;  // input rows, in send order
  pack.src = in, pack.src_dt = id_.dtype, pack.src_stride = id_.stride;
  pack.src_offset = id_.storage_offset, pack.src_select = ROW_BY_POSITION;
  pack.dst = send, pack.dst_dt = id_.dtype, pack.dst_stride = dim;
  pack.dim = dim, pack.sm_hint = sms, pack.positions = plan.positions;
  row_copy_args store = put;  // received rows -> local shard
  store.src = recv, store.src_stride = dim, store.src_offset = 0, store.src_select = ROW_SEQUENTIAL;
  store.indices = plan.recv_ids;
  pipelined_exchange(
    comm, plan.send_counts, plan.send_displs, plan.recv_counts, plan.recv_displs, send, recv, row_b, stream,
    [&](const list_segments& seg) {
      row_copy_args a = pack;
      a.segments = seg, a.count = seg.total();
      launch_row_copy(a, stream);
    },
    [&](const list_segments& seg) {
      row_copy_args a = store;
      a.segments = seg, a.count = seg.total();
      launch_row_copy(a, stream);
    },
    plan.chunk_count(row_b, 0, comm->tuning.exchange_chunks));
  // The reference returns with the local shard updated (scatter_op_impl_nccl.cu:157).
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
}

}  // namespace
}  // namespace wgb

using namespace wgb;

extern "C" {

wholegraph_error_code_t wholegraph_gather(wholegraph_tensor_t table,
                                            wholegraph_tensor_t indices_tensor,
                                            wholegraph_tensor_t output_tensor,
                                            wholegraph_env_func_t* p_env_fns,
                                            void* stream_ptr,
                                            int gather_sms)
{
  if (table == nullptr || indices_tensor == nullptr || output_tensor == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = static_cast<cudaStream_t>(stream_ptr);
  wholegraph_matrix_description_t tab, od;
  const int table_dim = wholegraph_tensor_get_tensor_description(table)->dim;
  if (table_dim != 1 && table_dim != 2) {
    WGB_ERROR("wholegraph_gather: the table must be 1-D or 2-D");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (!as_matrix(table, &tab)) return WHOLEGRAPH_LOGIC_ERROR;
  auto* idx_td = wholegraph_tensor_get_tensor_description(indices_tensor);
  if (idx_td->dim != 1) {
    WGB_ERROR("wholegraph_gather: indices must be 1-D");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (wholegraph_tensor_get_tensor_description(output_tensor)->dim != table_dim) {
    WGB_ERROR("wholegraph_gather: output must have as many dimensions as the table");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  wholegraph_array_description_t idx;
  if (!wholegraph_convert_tensor_desc_to_array(&idx, idx_td)) return WHOLEGRAPH_INVALID_INPUT;
  if (!as_matrix(output_tensor, &od)) return WHOLEGRAPH_INVALID_INPUT;
  void* ids = wholegraph_tensor_get_data_pointer(indices_tensor);  // offset applied
  void* out = wholegraph_tensor_get_data_pointer(output_tensor);
  if (out != nullptr)
    out = static_cast<char*>(out) - od.storage_offset * wholegraph_dtype_get_element_size(od.dtype);
  // Anything that is not int32 is read as int64 (reference: gather_func.cu:82-86).
  const bool ids_are_64 = idx.dtype != WHOLEGRAPH_DT_INT;
  const bool f_ok = wholegraph_dtype_is_floating_number(tab.dtype) &&
                    wholegraph_dtype_is_floating_number(od.dtype);
  const bool i_ok = wholegraph_dtype_is_integer_number(tab.dtype) &&
                    wholegraph_dtype_is_integer_number(od.dtype);
  if (!f_ok && !i_ok) {
    WGB_ERROR("wholegraph_gather: table dtype %d and output dtype %d do not mix", (int)tab.dtype,
              (int)od.dtype);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  if (od.sizes[0] != idx.size) {
    WGB_ERROR("wholegraph_gather: output has %ld rows for %ld indices", (long)od.sizes[0],
              (long)idx.size);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  if (od.sizes[1] != tab.sizes[1]) {
    WGB_ERROR("wholegraph_gather: output rows have %ld elements, table rows %ld", (long)od.sizes[1],
              (long)tab.sizes[1]);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(table);
  // A distributed gather is a collective: a rank with nothing to ask for still serves the others.
  const bool collective = h != nullptr && h->type == WHOLEGRAPH_MT_DISTRIBUTED && h->comm->world_size > 1;
  if ((idx.size == 0 && !collective) || tab.sizes[1] == 0) return WHOLEGRAPH_SUCCESS;
  if (idx.size > 0 && (ids == nullptr || out == nullptr)) return WHOLEGRAPH_INVALID_INPUT;

  if (h != nullptr && h->type == WHOLEGRAPH_MT_DISTRIBUTED) {
    gather_distributed(h, tab, ids, ids_are_64, idx.size, out, od, p_env_fns, stream, gather_sms);
    return WHOLEGRAPH_SUCCESS;
  }
  row_copy_args a;
  a.src_dt = tab.dtype, a.src_stride = tab.stride, a.src_offset = tab.storage_offset;
  a.src_select = ROW_BY_INDEX;
  a.dst = out, a.dst_dt = od.dtype, a.dst_stride = od.stride, a.dst_offset = od.storage_offset;
  a.count = idx.size, a.dim = tab.sizes[1], a.indices = ids, a.indices_are_64 = ids_are_64;
  a.sm_hint = gather_sms;
  if (h != nullptr && h->type == WHOLEGRAPH_MT_CHUNKED) {
    fill_chunks(&a.chunks, h,
                wholegraph_dtype_get_element_size(tab.dtype) *
                  static_cast<size_t>(table->root->desc.dim == 2 ? table->root->desc.strides[0] : 1));
  } else {
    wholegraph_gref_t gref;
    WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_global_reference(table, &gref));
    a.src = gref.pointer;
  }
  launch_row_copy(a, stream);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_gather")
}

wholegraph_error_code_t wholegraph_b200_gather_from_handle(wholegraph_handle_t handle,
                                                             const wholegraph_matrix_description_t* table_desc,
                                                             const void* indices,
                                                             const wholegraph_array_description_t* indices_desc,
                                                             void* output,
                                                             const wholegraph_matrix_description_t* output_desc,
                                                             wholegraph_env_func_t* p_env_fns,
                                                             void* stream_ptr,
                                                             int gather_sms)
{
  if (handle == nullptr || table_desc == nullptr || indices_desc == nullptr || output_desc == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = static_cast<cudaStream_t>(stream_ptr);
  const wholegraph_matrix_description_t& tab = *table_desc;
  const wholegraph_matrix_description_t& od  = *output_desc;
  const bool f_ok = wholegraph_dtype_is_floating_number(tab.dtype) && wholegraph_dtype_is_floating_number(od.dtype);
  const bool i_ok = wholegraph_dtype_is_integer_number(tab.dtype) && wholegraph_dtype_is_integer_number(od.dtype);
  if (!f_ok && !i_ok) return WHOLEGRAPH_LOGIC_ERROR;
  if (od.sizes[0] != indices_desc->size || od.sizes[1] != tab.sizes[1]) return WHOLEGRAPH_LOGIC_ERROR;
  if (indices_desc->dtype != WHOLEGRAPH_DT_INT && indices_desc->dtype != WHOLEGRAPH_DT_INT64) return WHOLEGRAPH_INVALID_INPUT;
  const bool ids_are_64 = indices_desc->dtype == WHOLEGRAPH_DT_INT64;
  const int64_t n       = indices_desc->size;
  const bool collective = handle->type == WHOLEGRAPH_MT_DISTRIBUTED && handle->comm->world_size > 1;
  if ((n == 0 && !collective) || tab.sizes[1] == 0) return WHOLEGRAPH_SUCCESS;
  if (n > 0 && (indices == nullptr || output == nullptr)) return WHOLEGRAPH_INVALID_INPUT;
  const void* ids = indices == nullptr ? nullptr
                                       : static_cast<const char*>(indices) +
                                           indices_desc->storage_offset * (ids_are_64 ? 8 : 4);
  const size_t row_bytes = wholegraph_dtype_get_element_size(tab.dtype) * static_cast<size_t>(tab.stride);
  if (handle->type == WHOLEGRAPH_MT_DISTRIBUTED) {
    gather_distributed(handle, tab, ids, ids_are_64, n, output, od, p_env_fns, stream, gather_sms);
    return WHOLEGRAPH_SUCCESS;
  }
  row_copy_args a;
  a.src_dt = tab.dtype, a.src_stride = tab.stride, a.src_offset = tab.storage_offset;
  a.src_select = ROW_BY_INDEX;
  a.dst = output, a.dst_dt = od.dtype, a.dst_stride = od.stride, a.dst_offset = od.storage_offset;
  a.count = n, a.dim = tab.sizes[1], a.indices = ids, a.indices_are_64 = ids_are_64, a.sm_hint = gather_sms;
  if (handle->type == WHOLEGRAPH_MT_CHUNKED)
    fill_chunks(&a.chunks, handle, row_bytes);
  else
    a.src = handle->global_base;
  WGB_EXPECTS(handle->type == WHOLEGRAPH_MT_CHUNKED || a.src != nullptr, "the handle has no mapped range");
  launch_row_copy(a, stream);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_b200_gather_from_handle")
}

wholegraph_error_code_t wholegraph_scatter(wholegraph_tensor_t input_tensor,
                                             wholegraph_tensor_t indices_tensor,
                                             wholegraph_tensor_t table,
                                             wholegraph_env_func_t* p_env_fns,
                                             void* stream_ptr,
                                             int scatter_sms)
{
  if (table == nullptr || indices_tensor == nullptr || input_tensor == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = static_cast<cudaStream_t>(stream_ptr);
  wholegraph_matrix_description_t tab, id_;
  const int table_dim = wholegraph_tensor_get_tensor_description(table)->dim;
  if (table_dim != 1 && table_dim != 2) {
    WGB_ERROR("wholegraph_scatter: the table must be 1-D or 2-D");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (!as_matrix(table, &tab)) return WHOLEGRAPH_LOGIC_ERROR;
  auto* idx_td = wholegraph_tensor_get_tensor_description(indices_tensor);
  if (idx_td->dim != 1) {
    WGB_ERROR("wholegraph_scatter: indices must be 1-D");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (wholegraph_tensor_get_tensor_description(input_tensor)->dim != table_dim) {
    WGB_ERROR("wholegraph_scatter: input must have as many dimensions as the table");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  wholegraph_array_description_t idx;
  if (!wholegraph_convert_tensor_desc_to_array(&idx, idx_td)) return WHOLEGRAPH_INVALID_INPUT;
  if (!as_matrix(input_tensor, &id_)) return WHOLEGRAPH_INVALID_INPUT;
  void* ids      = wholegraph_tensor_get_data_pointer(indices_tensor);
  const void* in = wholegraph_tensor_get_data_pointer(input_tensor);
  if (in != nullptr)
    in = static_cast<const char*>(in) -
         id_.storage_offset * wholegraph_dtype_get_element_size(id_.dtype);
  const bool ids_are_64 = idx.dtype != WHOLEGRAPH_DT_INT;
  const bool f_ok = wholegraph_dtype_is_floating_number(tab.dtype) &&
                    wholegraph_dtype_is_floating_number(id_.dtype);
  const bool i_ok = wholegraph_dtype_is_integer_number(tab.dtype) &&
                    wholegraph_dtype_is_integer_number(id_.dtype);
  if (!f_ok && !i_ok) {
    WGB_ERROR("wholegraph_scatter: table dtype %d and input dtype %d do not mix", (int)tab.dtype,
              (int)id_.dtype);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  if (id_.sizes[0] != idx.size) {
    WGB_ERROR("wholegraph_scatter: input has %ld rows for %ld indices", (long)id_.sizes[0],
              (long)idx.size);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  if (id_.sizes[1] != tab.sizes[1]) {
    WGB_ERROR("wholegraph_scatter: input rows have %ld elements, table rows %ld",
              (long)id_.sizes[1], (long)tab.sizes[1]);
    return WHOLEGRAPH_LOGIC_ERROR;
  }
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(table);
  // A distributed scatter is a collective: a rank with nothing to store still receives rows.
  const bool collective = h != nullptr && h->type == WHOLEGRAPH_MT_DISTRIBUTED && h->comm->world_size > 1;
  if ((idx.size == 0 && !collective) || tab.sizes[1] == 0) return WHOLEGRAPH_SUCCESS;
  if (idx.size > 0 && (ids == nullptr || in == nullptr)) return WHOLEGRAPH_INVALID_INPUT;

  if (h != nullptr && h->type == WHOLEGRAPH_MT_DISTRIBUTED) {
    scatter_distributed(in, id_, ids, ids_are_64, idx.size, h, tab, p_env_fns, stream, scatter_sms);
    return WHOLEGRAPH_SUCCESS;
  }
  row_copy_args a;
  a.src = in, a.src_dt = id_.dtype, a.src_stride = id_.stride, a.src_offset = id_.storage_offset;
  a.dst_dt = tab.dtype, a.dst_stride = tab.stride, a.dst_offset = tab.storage_offset;
  a.dst_select = ROW_BY_INDEX;
  a.count = idx.size, a.dim = tab.sizes[1], a.indices = ids, a.indices_are_64 = ids_are_64;
  a.sm_hint = scatter_sms;
  if (h != nullptr && h->type == WHOLEGRAPH_MT_CHUNKED) {
    fill_chunks(&a.chunks, h,
                wholegraph_dtype_get_element_size(tab.dtype) *
                  static_cast<size_t>(table->root->desc.dim == 2 ? table->root->desc.strides[0] : 1));
  } else {
    wholegraph_gref_t gref;
    WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_global_reference(table, &gref));
    a.dst = gref.pointer;
  }
  launch_row_copy(a, stream);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_scatter")
}

}  // extern "C"
