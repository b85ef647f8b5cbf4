// C entry points for library lifetime, communicators and memory handles.
// Behaviour follows the reference's cpp/src/wholegraph/wholegraph.cpp and initialize.cpp:24-60;
// no exception leaves this file.
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>

#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_b200.h>

#include "comm.hpp"
#include "common.hpp"
#include "handle.hpp"
#include "kernels/partition.hpp"
#include "kernels/row_copy.hpp"
#include "kernels/unique_ids.hpp"
#include "ops.hpp"

static bool g_inited = false;

extern "C" {

wholegraph_error_code_t wholegraph_init(unsigned int flags, LogLevel log_level)
{
  if (flags != 0) return WHOLEGRAPH_INVALID_INPUT;
  if (g_inited) return WHOLEGRAPH_SUCCESS;
  wgb::log_level() = log_level;
  g_inited         = true;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_finalize()
{
  WGB_API_BEGIN
  wgb::destroy_all_comms();
  g_inited = false;
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_finalize")
}

wholegraph_error_code_t wholegraph_create_unique_id(wholegraph_unique_id_t* unique_id)
{
  if (unique_id == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  wgb::nccl_get_unique_id(unique_id);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_create_unique_id")
}

wholegraph_error_code_t wholegraph_create_communicator(wholegraph_comm_t* comm,
                                                         wholegraph_unique_id_t unique_id,
                                                         int rank,
                                                         int size)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  *comm = wgb::create_comm(unique_id, rank, size);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_create_communicator")
}

wholegraph_error_code_t wholegraph_split_communicator(wholegraph_comm_t* new_comm,
                                                        wholegraph_comm_t comm,
                                                        int color,
                                                        int key)
{
  if (new_comm == nullptr || comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  *new_comm = wgb::split_comm(comm, color, key);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_split_communicator")
}

wholegraph_error_code_t wholegraph_destroy_communicator(wholegraph_comm_t comm)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  wgb::destroy_comm(comm);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_destroy_communicator")
}

wholegraph_error_code_t wholegraph_communicator_support_type_location(
  wholegraph_comm_t comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (memory_location != WHOLEGRAPH_ML_DEVICE && memory_location != WHOLEGRAPH_ML_HOST)
    return WHOLEGRAPH_NOT_SUPPORTED;
  switch (memory_type) {
    case WHOLEGRAPH_MT_CONTINUOUS:
    case WHOLEGRAPH_MT_DISTRIBUTED: return WHOLEGRAPH_SUCCESS;
    case WHOLEGRAPH_MT_CHUNKED:
      return memory_location == WHOLEGRAPH_ML_DEVICE ? WHOLEGRAPH_SUCCESS : WHOLEGRAPH_NOT_SUPPORTED;
    default: return WHOLEGRAPH_NOT_SUPPORTED;
  }
}

wholegraph_error_code_t wholegraph_communicator_get_rank(int* rank, wholegraph_comm_t comm)
{
  if (rank == nullptr || comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *rank = comm->world_rank;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_communicator_get_size(int* size, wholegraph_comm_t comm)
{
  if (size == nullptr || comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *size = comm->world_size;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_communicator_get_local_size(int* local_size,
                                                                 wholegraph_comm_t comm)
{
  // One node: every rank of the communicator is local.
  if (local_size == nullptr || comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *local_size = comm->world_size;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_communicator_get_clique_info(clique_info_t* clique_info,
                                                                  wholegraph_comm_t comm)
{
  if (clique_info == nullptr || comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  // No multi-node NVLink domain is modelled: report "not in a clique".
  memset(clique_info, 0, sizeof(*clique_info));
  clique_info->clique_id = -1;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_communicator_set_distributed_backend(
  wholegraph_comm_t comm, wholegraph_distributed_backend_t distributed_backend)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (distributed_backend != WHOLEGRAPH_DB_NCCL) return WHOLEGRAPH_NOT_SUPPORTED;
  comm->backend = distributed_backend;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_distributed_backend_t wholegraph_communicator_get_distributed_backend(
  wholegraph_comm_t comm)
{
  return comm == nullptr ? WHOLEGRAPH_DB_NONE : comm->backend;
}

wholegraph_error_code_t wholegraph_communicator_barrier(wholegraph_comm_t comm)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  comm->barrier();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_communicator_barrier")
}

bool wholegraph_is_intranode_communicator(wholegraph_comm_t comm) { return comm != nullptr; }
bool wholegraph_is_intra_mnnvl_communicator(wholegraph_comm_t) { return false; }

wholegraph_error_code_t wholegraph_malloc(wholegraph_handle_t* handle_ptr,
                                            size_t total_size,
                                            wholegraph_comm_t comm,
                                            wholegraph_memory_type_t memory_type,
                                            wholegraph_memory_location_t memory_location,
                                            size_t data_granularity,
                                            size_t* rank_entry_partition)
{
  if (handle_ptr == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *handle_ptr = nullptr;
  WGB_API_BEGIN
  *handle_ptr = wgb::create_handle(total_size, comm, memory_type, memory_location, data_granularity,
                                   rank_entry_partition);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_malloc")
}

wholegraph_error_code_t wholegraph_free(wholegraph_handle_t h)
{
  if (h == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  wgb::destroy_handle(h);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_free")
}

wholegraph_error_code_t wholegraph_get_communicator(wholegraph_comm_t* comm, wholegraph_handle_t h)
{
  if (comm == nullptr || h == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *comm = h->comm;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_memory_type_t wholegraph_get_memory_type(wholegraph_handle_t h)
{
  return h == nullptr ? WHOLEGRAPH_MT_NONE : h->type;
}
wholegraph_memory_location_t wholegraph_get_memory_location(wholegraph_handle_t h)
{
  return h == nullptr ? WHOLEGRAPH_ML_NONE : h->location;
}
wholegraph_distributed_backend_t wholegraph_get_distributed_backend(wholegraph_handle_t h)
{
  return (h == nullptr || h->comm == nullptr) ? WHOLEGRAPH_DB_NONE : h->comm->backend;
}
size_t wholegraph_get_total_size(wholegraph_handle_t h) { return h == nullptr ? 0 : h->total_size; }
size_t wholegraph_get_data_granularity(wholegraph_handle_t h)
{
  return h == nullptr ? 0 : h->granularity;
}

wholegraph_error_code_t wholegraph_get_local_memory(void** local_ptr,
                                                      size_t* local_size,
                                                      size_t* local_offset,
                                                      wholegraph_handle_t h)
{
  if (h == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  int me = h->comm->world_rank;
  if (local_ptr != nullptr) *local_ptr = h->local_ptr;
  if (local_size != nullptr) *local_size = h->part_sizes[me];
  if (local_offset != nullptr) *local_offset = h->part_offsets[me];
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_local_size(size_t* local_size, wholegraph_handle_t h)
{
  if (h == nullptr || local_size == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *local_size = h->part_sizes[h->comm->world_rank];
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_local_offset(size_t* local_offset, wholegraph_handle_t h)
{
  if (h == nullptr || local_offset == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *local_offset = h->part_offsets[h->comm->world_rank];
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_rank_memory(void** rank_memory_ptr,
                                                     size_t* rank_memory_size,
                                                     size_t* rank_memory_offset,
                                                     int rank,
                                                     wholegraph_handle_t h)
{
  if (h == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (rank < 0 || rank >= h->comm->world_size) return WHOLEGRAPH_INVALID_INPUT;
  void* p = nullptr;
  if (h->type == WHOLEGRAPH_MT_CONTINUOUS)
    p = static_cast<char*>(h->global_base) + h->part_offsets[rank];
  else if (h->type == WHOLEGRAPH_MT_CHUNKED)
    p = h->rank_ptrs[rank];
  else if (rank == h->comm->world_rank)
    p = h->local_ptr;
  if (rank_memory_ptr != nullptr) *rank_memory_ptr = p;
  if (rank_memory_size != nullptr) *rank_memory_size = h->part_sizes[rank];
  if (rank_memory_offset != nullptr) *rank_memory_offset = h->part_offsets[rank];
  return p == nullptr ? WHOLEGRAPH_INVALID_INPUT : WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_equal_entry_partition_plan(size_t* entry_per_rank,
                                                                size_t total_entry_count,
                                                                int world_size)
{
  if (entry_per_rank == nullptr || world_size <= 0) return WHOLEGRAPH_INVALID_INPUT;
  *entry_per_rank = (total_entry_count + world_size - 1) / world_size;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_global_pointer(void** global_ptr, wholegraph_handle_t h)
{
  if (h == nullptr || global_ptr == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *global_ptr = h->type == WHOLEGRAPH_MT_CONTINUOUS ? h->global_base : nullptr;
  return *global_ptr == nullptr ? WHOLEGRAPH_INVALID_INPUT : WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_global_reference(wholegraph_gref_t* gref,
                                                          wholegraph_handle_t h)
{
  if (h == nullptr || gref == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  gref->pointer = h->type == WHOLEGRAPH_MT_CONTINUOUS ? h->global_base : nullptr;
  return gref->pointer == nullptr ? WHOLEGRAPH_INVALID_INPUT : WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_rank_partition_sizes(size_t* rank_mem_sizes,
                                                              wholegraph_handle_t h)
{
  if (h == nullptr || rank_mem_sizes == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  for (size_t i = 0; i < h->part_sizes.size(); i++) rank_mem_sizes[i] = h->part_sizes[i];
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_get_rank_partition_offsets(size_t* rank_mem_offsets,
                                                                wholegraph_handle_t h)
{
  if (h == nullptr || rank_mem_offsets == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  for (size_t i = 0; i < h->part_offsets.size(); i++) rank_mem_offsets[i] = h->part_offsets[i];
  return WHOLEGRAPH_SUCCESS;
}

int fork_get_device_count()
{
  int fds[2];
  if (pipe(fds) != 0) return -1;
  pid_t pid = fork();
  if (pid < 0) {
    close(fds[0]);
    close(fds[1]);
    return -1;
  }
  if (pid == 0) {
    close(fds[0]);
    int n = -1;
    if (cudaGetDeviceCount(&n) != cudaSuccess) n = -1;
    ssize_t w = write(fds[1], &n, sizeof(n));
    (void)w;
    close(fds[1]);
    _exit(0);
  }
  close(fds[1]);
  int n     = -1;
  ssize_t r = read(fds[0], &n, sizeof(n));
  close(fds[0]);
  int status = 0;
  waitpid(pid, &status, 0);
  return r == static_cast<ssize_t>(sizeof(n)) ? n : -1;
}

wholegraph_error_code_t wholegraph_b200_memcpy_async(void* dst, const void* src, size_t bytes,
                                                       void* stream)
{
  if (bytes == 0) return WHOLEGRAPH_SUCCESS;
  if (dst == nullptr || src == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  WGB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_b200_memcpy_async")
}

size_t wholegraph_b200_partition_workspace_bytes(int64_t n, int world)
{
  return wgb::partition_workspace_bytes(n, world);
}

wholegraph_error_code_t wholegraph_b200_partition_by_owner(const void* ids,
                                                             int ids_are_64,
                                                             int64_t n,
                                                             const int64_t* first_row,
                                                             int world,
                                                             void* workspace,
                                                             size_t workspace_bytes,
                                                             int64_t* sorted_ids,
                                                             int64_t* positions,
                                                             int64_t* counts,
                                                             int64_t* starts,
                                                             void* stream)
{
  if (n < 0 || first_row == nullptr || counts == nullptr || starts == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  if (n > 0 && (ids == nullptr || workspace == nullptr || sorted_ids == nullptr || positions == nullptr))
    return WHOLEGRAPH_INVALID_INPUT;
  if (world < 1 || world > wgb::kMaxPartitionRanks) return WHOLEGRAPH_INVALID_VALUE;
  if (workspace_bytes < wgb::partition_workspace_bytes(n, world)) return WHOLEGRAPH_INVALID_VALUE;
  WGB_API_BEGIN
  wgb::partition_by_owner(ids, ids_are_64 != 0, n, first_row, world, workspace, sorted_ids, positions,
                          counts, starts, static_cast<cudaStream_t>(stream));
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_b200_partition_by_owner")
}

wholegraph_error_code_t wholegraph_b200_partition_by_owner_no_alloc(const void* ids,
                                                                      int ids_are_64,
                                                                      int64_t n,
                                                                      const int64_t* first_row,
                                                                      int world,
                                                                      int64_t* sorted_ids,
                                                                      int64_t* positions,
                                                                      int64_t* counts,
                                                                      int64_t* starts,
                                                                      void* stream)
{
  if (n < 0 || first_row == nullptr || counts == nullptr || starts == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  if (n > 0 && (ids == nullptr || sorted_ids == nullptr || positions == nullptr))
    return WHOLEGRAPH_INVALID_INPUT;
  if (world < 1 || world > wgb::kMaxPartitionRanks) return WHOLEGRAPH_INVALID_VALUE;
  WGB_API_BEGIN
  wgb::partition_by_owner_builtin_scratch(ids, ids_are_64 != 0, n, first_row, world, sorted_ids,
                                          positions, counts, starts,
                                          static_cast<cudaStream_t>(stream));
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_b200_partition_by_owner_no_alloc")
}

size_t wholegraph_b200_unique_workspace_bytes(int64_t n, int64_t total_rows)
{
  return wgb::unique_workspace_bytes(n, total_rows);
}

static wholegraph_error_code_t unique_by_owner_entry(bool ascending, const char* where, const void* ids,
                                                          int ids_are_64,
                                                          int64_t n,
                                                          const int64_t* first_row,
                                                          int world,
                                                          void* workspace,
                                                          size_t workspace_bytes,
                                                          int64_t* unique_ids,
                                                          int64_t* inverse,
                                                          int64_t* counts,
                                                          int64_t* starts,
                                                          void* stream)
{
  if (n < 0 || first_row == nullptr || counts == nullptr || starts == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  if (n > 0 && (ids == nullptr || workspace == nullptr || unique_ids == nullptr || inverse == nullptr))
    return WHOLEGRAPH_INVALID_INPUT;
  if (world < 1 || world > wgb::kMaxPartitionRanks) return WHOLEGRAPH_INVALID_VALUE;
  WGB_API_BEGIN
  wgb::check_owner_table(first_row, world);
  if (!wgb::unique_supported(n, first_row[world])) return WHOLEGRAPH_INVALID_VALUE;
  if (workspace_bytes < wgb::unique_workspace_bytes(n, first_row[world])) return WHOLEGRAPH_INVALID_VALUE;
  wgb::unique_by_owner(ids, ids_are_64 != 0, n, first_row, world, workspace, unique_ids, inverse, counts,
                       starts, static_cast<cudaStream_t>(stream), ascending);
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END(where)
}

wholegraph_error_code_t wholegraph_b200_unique_by_owner(const void* ids,
                                                          int ids_are_64,
                                                          int64_t n,
                                                          const int64_t* first_row,
                                                          int world,
                                                          void* workspace,
                                                          size_t workspace_bytes,
                                                          int64_t* unique_ids,
                                                          int64_t* inverse,
                                                          int64_t* counts,
                                                          int64_t* starts,
                                                          void* stream)
{
  return unique_by_owner_entry(true, "wholegraph_b200_unique_by_owner", ids, ids_are_64, n, first_row, world, workspace,
                               workspace_bytes, unique_ids, inverse, counts, starts, stream);
}

wholegraph_error_code_t wholegraph_b200_unique_by_owner_any_order(const void* ids,
                                                                    int ids_are_64,
                                                                    int64_t n,
                                                                    const int64_t* first_row,
                                                                    int world,
                                                                    void* workspace,
                                                                    size_t workspace_bytes,
                                                                    int64_t* unique_ids,
                                                                    int64_t* inverse,
                                                                    int64_t* counts,
                                                                    int64_t* starts,
                                                                    void* stream)
{
  return unique_by_owner_entry(false, "wholegraph_b200_unique_by_owner_any_order", ids, ids_are_64, n, first_row, world,
                               workspace, workspace_bytes, unique_ids, inverse, counts, starts, stream);
}

int wholegraph_b200_exchange_chunk_count(const int64_t* matrix, int world, size_t row_bytes, int wanted,
                                         int forced)
{
  if (matrix == nullptr || world < 1) return 1;
  return wgb::exchange_chunk_count(matrix, world, row_bytes, wanted, forced);
}

wholegraph_error_code_t wholegraph_b200_reload_tuning(wholegraph_comm_t comm)
{
  if (comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  comm->reload_tuning();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_b200_reload_tuning")
}

unsigned long long wholegraph_b200_kernel_launch_count() { return wgb::kernel_launch_count(); }

const char* wholegraph_b200_version() { return "wholegraph-b200 0.1 sm_100a"; }

}  // extern "C"
