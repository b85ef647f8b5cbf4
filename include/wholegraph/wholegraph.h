/*
 * wholegraph-b200: library lifetime, communicators and memory handles.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/wholegraph.h: error codes
 * :21-33, memory type / location :50-64, communicator calls :88-231, handle calls
 * :239-402, file I/O :415-437. Declarations, default arguments, struct layouts
 * and enum values are identical so that the reference's nanobind module and C++
 * callers link against this library unchanged.
 */
#pragma once

#include <stdio.h>
#include <unistd.h>

#include <wholegraph/global_reference.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes; values are part of the ABI (wholegraph.h:21-33). */
enum wholegraph_error_code_t {
  WHOLEGRAPH_SUCCESS = 0,
  WHOLEGRAPH_UNKNOW_ERROR,        /* 1 */
  WHOLEGRAPH_NOT_IMPLEMENTED,     /* 2 */
  WHOLEGRAPH_LOGIC_ERROR,         /* 3 */
  WHOLEGRAPH_CUDA_ERROR,          /* 4 */
  WHOLEGRAPH_COMMUNICATION_ERROR, /* 5 */
  WHOLEGRAPH_INVALID_INPUT,       /* 6: e.g. a null pointer */
  WHOLEGRAPH_INVALID_VALUE,       /* 7 */
  WHOLEGRAPH_OUT_OF_MEMORY,       /* 8 */
  WHOLEGRAPH_NOT_SUPPORTED,       /* 9 */
  WHOLEGRAPH_SYSTEM_ERROR,        /* 10 */
};

#define WHOLEGRAPH_RETURN_ON_FAIL(X)                                                  \
  do {                                                                                \
    auto err = X;                                                                     \
    if (err != WHOLEGRAPH_SUCCESS) {                                                  \
      const char* error_str = #X;                                                     \
      fprintf(stderr, "File %s line %d %s failed.\n", __FILE__, __LINE__, error_str); \
      return err;                                                                     \
    }                                                                                 \
  } while (0)

/*
 * How the shards of an allocation are addressed (wholegraph.h:50-54).
 * CONTINUOUS: all ranks' shards mapped into one virtual range on every rank;
 *             kernels dereference peers' memory directly (NVLink P2P).
 * DISTRIBUTED: a rank sees only its own shard; remote rows travel by alltoallv.
 * CHUNKED (extension of this library, value 3; the reference stops at 2): peers'
 *             shards are reachable through one base pointer per rank instead of a
 *             single range.
 */
enum wholegraph_memory_type_t {
  WHOLEGRAPH_MT_NONE = 0,
  WHOLEGRAPH_MT_CONTINUOUS,
  WHOLEGRAPH_MT_DISTRIBUTED,
  WHOLEGRAPH_MT_CHUNKED,
};

enum wholegraph_memory_location_t {
  WHOLEGRAPH_ML_NONE = 0,
  WHOLEGRAPH_ML_DEVICE,
  WHOLEGRAPH_ML_HOST,
};

enum wholegraph_distributed_backend_t {
  WHOLEGRAPH_DB_NONE = 0,
  WHOLEGRAPH_DB_NCCL,
};

enum LogLevel {
  LEVEL_FATAL = 0,
  LEVEL_ERROR,
  LEVEL_WARN,
  LEVEL_INFO,
  LEVEL_DEBUG,
  LEVEL_TRACE
};

#define WHOLEGRAPH_SPILT_NO_COLOR -1

/* Start / stop the library. `flags` must be 0. */
wholegraph_error_code_t wholegraph_init(unsigned int flags, LogLevel log_level = LEVEL_INFO);
wholegraph_error_code_t wholegraph_finalize();

typedef struct wholegraph_comm_* wholegraph_comm_t;

/* Multi-node NVLink domain description; a single NVSwitch node is one clique. */
struct clique_info_t {
  int is_in_clique;
  int clique_first_rank;
  int clique_rank;
  int clique_rank_num;
  int clique_id;
  int clique_num;
};

#define WHOLEGRAPH_UNIQUE_ID_BYTES (128)
/* Rendezvous token; holds an ncclUniqueId. */
struct wholegraph_unique_id_t {
  char internal[WHOLEGRAPH_UNIQUE_ID_BYTES];
};

wholegraph_error_code_t wholegraph_create_unique_id(wholegraph_unique_id_t* unique_id);

/* Collective over all `size` ranks: every rank passes the same id. */
wholegraph_error_code_t wholegraph_create_communicator(wholegraph_comm_t* comm,
                                                         wholegraph_unique_id_t unique_id,
                                                         int rank,
                                                         int size);

/*
 * Collective: ranks with equal non-negative `color` form a new communicator ordered by
 * (`key`, old rank); color WHOLEGRAPH_SPILT_NO_COLOR yields *new_comm = NULL.
 */
wholegraph_error_code_t wholegraph_split_communicator(wholegraph_comm_t* new_comm,
                                                        wholegraph_comm_t comm,
                                                        int color,
                                                        int key);

/* Collective. Also frees every handle still allocated on the communicator. */
wholegraph_error_code_t wholegraph_destroy_communicator(wholegraph_comm_t comm);

/* WHOLEGRAPH_SUCCESS if the (type, location) pair can be allocated, else NOT_SUPPORTED. */
wholegraph_error_code_t wholegraph_communicator_support_type_location(
  wholegraph_comm_t comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location);

wholegraph_error_code_t wholegraph_communicator_get_rank(int* rank, wholegraph_comm_t comm);
wholegraph_error_code_t wholegraph_communicator_get_size(int* size, wholegraph_comm_t comm);
wholegraph_error_code_t wholegraph_communicator_get_local_size(int* local_size,
                                                                 wholegraph_comm_t comm);
wholegraph_error_code_t wholegraph_communicator_get_clique_info(clique_info_t* clique_info,
                                                                  wholegraph_comm_t comm);

wholegraph_error_code_t wholegraph_communicator_set_distributed_backend(
  wholegraph_comm_t comm, wholegraph_distributed_backend_t distributed_backend);
wholegraph_distributed_backend_t wholegraph_communicator_get_distributed_backend(
  wholegraph_comm_t comm);

wholegraph_error_code_t wholegraph_communicator_barrier(wholegraph_comm_t comm);

typedef struct wholegraph_handle_* wholegraph_handle_t;

/*
 * Collective allocation of `total_size` bytes sharded over the communicator in
 * units of `data_granularity` bytes (a unit never straddles two ranks).
 * `rank_entry_partition` (world_size unit counts, all > 0, summing to
 * total_size / data_granularity) overrides the default ceil(units / world_size)
 * contiguous split.
 */
wholegraph_error_code_t wholegraph_malloc(wholegraph_handle_t* wholegraph_handle_ptr,
                                            size_t total_size,
                                            wholegraph_comm_t comm,
                                            wholegraph_memory_type_t memory_type,
                                            wholegraph_memory_location_t memory_location,
                                            size_t data_granularity,
                                            size_t* rank_entry_partition = nullptr);

/* Collective. */
wholegraph_error_code_t wholegraph_free(wholegraph_handle_t wholegraph_handle);

wholegraph_error_code_t wholegraph_get_communicator(wholegraph_comm_t* comm,
                                                      wholegraph_handle_t wholegraph_handle);
wholegraph_memory_type_t wholegraph_get_memory_type(wholegraph_handle_t wholegraph_handle);
wholegraph_memory_location_t wholegraph_get_memory_location(
  wholegraph_handle_t wholegraph_handle);
wholegraph_distributed_backend_t wholegraph_get_distributed_backend(
  wholegraph_handle_t wholegraph_handle);
size_t wholegraph_get_total_size(wholegraph_handle_t wholegraph_handle);
size_t wholegraph_get_data_granularity(wholegraph_handle_t wholegraph_handle);

/* This rank's shard: pointer, byte size and byte offset inside the allocation. */
wholegraph_error_code_t wholegraph_get_local_memory(void** local_ptr,
                                                      size_t* local_size,
                                                      size_t* local_offset,
                                                      wholegraph_handle_t wholegraph_handle);
wholegraph_error_code_t wholegraph_get_local_size(size_t* local_size,
                                                    wholegraph_handle_t wholegraph_handle);
wholegraph_error_code_t wholegraph_get_local_offset(size_t* local_offset,
                                                      wholegraph_handle_t wholegraph_handle);

/* Another rank's shard; the pointer is valid only for mapped (CONTINUOUS / CHUNKED) types. */
wholegraph_error_code_t wholegraph_get_rank_memory(void** rank_memory_ptr,
                                                     size_t* rank_memory_size,
                                                     size_t* rank_memory_offset,
                                                     int rank,
                                                     wholegraph_handle_t wholegraph_handle);

/* Default split: ceil(total_entry_count / world_size) entries per rank. */
wholegraph_error_code_t wholegraph_equal_entry_partition_plan(size_t* entry_per_rank,
                                                                size_t total_entry_count,
                                                                int world_size);

/* CONTINUOUS only. */
wholegraph_error_code_t wholegraph_get_global_pointer(void** global_ptr,
                                                        wholegraph_handle_t wholegraph_handle);
wholegraph_error_code_t wholegraph_get_global_reference(wholegraph_gref_t* wholegraph_gref,
                                                          wholegraph_handle_t wholegraph_handle);

/* world_size byte sizes / world_size + 1 byte offsets. */
wholegraph_error_code_t wholegraph_get_rank_partition_sizes(
  size_t* rank_mem_sizes, wholegraph_handle_t wholegraph_handle);
wholegraph_error_code_t wholegraph_get_rank_partition_offsets(
  size_t* rank_mem_offsets, wholegraph_handle_t wholegraph_handle);

/* Device count probed in a forked child so the caller creates no CUDA context; -1 on error. */
int fork_get_device_count();

/*
 * Collective: fill the allocation from the logical concatenation of binary files holding
 * `file_entry_size`-byte records, placed `memory_entry_size` bytes apart from `memory_offset`.
 */
wholegraph_error_code_t wholegraph_load_from_file(wholegraph_handle_t wholegraph_handle,
                                                    size_t memory_offset,
                                                    size_t memory_entry_size,
                                                    size_t file_entry_size,
                                                    const char** file_names,
                                                    int file_count,
                                                    int round_robin_size);

/* Collective: every rank writes its shard's records to its own file. */
wholegraph_error_code_t wholegraph_store_to_file(wholegraph_handle_t wholegraph_handle,
                                                   size_t memory_offset,
                                                   size_t memory_entry_stride,
                                                   size_t file_entry_size,
                                                   const char* local_file_name);

bool wholegraph_is_intranode_communicator(wholegraph_comm_t comm);
bool wholegraph_is_intra_mnnvl_communicator(wholegraph_comm_t comm);

#ifdef __cplusplus
}
#endif
