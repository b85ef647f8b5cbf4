/*
 * wholegraph-b200: tensors = a descriptor over a memory handle or a plain pointer.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/wholegraph_tensor.h:20-183.
 */
#pragma once

#include <wholegraph/tensor_description.h>
#include <wholegraph/wholegraph.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct wholegraph_tensor_* wholegraph_tensor_t;

/*
 * Collective. Allocate a sharded 1-D or 2-D tensor (unit inner stride, zero offset);
 * rows are the sharding unit. `tensor_entry_partition` = optional rows per rank.
 */
wholegraph_error_code_t wholegraph_create_tensor(
  wholegraph_tensor_t* wholegraph_tensor,
  wholegraph_tensor_description_t* tensor_description,
  wholegraph_comm_t comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location,
  size_t* tensor_entry_partition = nullptr);

/* Frees the handle too when the tensor owns it (collective in that case). */
wholegraph_error_code_t wholegraph_destroy_tensor(wholegraph_tensor_t wholegraph_tensor);

/* Non-owning view of caller memory; `storage_ptr` is element 0 BEFORE storage_offset. */
wholegraph_error_code_t wholegraph_make_tensor_from_pointer(
  wholegraph_tensor_t* wholegraph_tensor,
  void* storage_ptr,
  wholegraph_tensor_description_t* tensor_description);

/* Non-owning view of an existing handle. */
wholegraph_error_code_t wholegraph_make_tensor_from_handle(
  wholegraph_tensor_t* wholegraph_tensor,
  wholegraph_handle_t wholegraph_handle,
  wholegraph_tensor_description_t* tensor_description);

bool wholegraph_tensor_has_handle(wholegraph_tensor_t wholegraph_tensor);
wholegraph_handle_t wholegraph_tensor_get_memory_handle(wholegraph_tensor_t wholegraph_tensor);
wholegraph_tensor_description_t* wholegraph_tensor_get_tensor_description(
  wholegraph_tensor_t wholegraph_tensor);
wholegraph_error_code_t wholegraph_tensor_get_global_reference(
  wholegraph_tensor_t wholegraph_tensor, wholegraph_gref_t* wholegraph_gref);

/*
 * View of this rank's rows as a pointer tensor (caller destroys it). Needs a handle;
 * 1-D: zero offset; 2-D: storage_offset + sizes[1] <= strides[0].
 */
wholegraph_error_code_t wholegraph_tensor_map_local_tensor(
  wholegraph_tensor_t wholegraph_tensor, wholegraph_tensor_t* local_tensor);

/* Address of the first element; NULL for a handle that has no single range. */
void* wholegraph_tensor_get_data_pointer(wholegraph_tensor_t wholegraph_tensor);

/* world_size + 1 first-row offsets / world_size row counts of the root tensor's shards. */
wholegraph_error_code_t wholegraph_tensor_get_entry_offsets(
  size_t* entry_offsets, wholegraph_tensor_t wholegraph_tensor);
wholegraph_error_code_t wholegraph_tensor_get_entry_partition_sizes(
  size_t* entry_partition, wholegraph_tensor_t wholegraph_tensor);
wholegraph_error_code_t wholegraph_tensor_get_local_entry_count(
  size_t* local_entry_count, wholegraph_tensor_t wholegraph_tensor);
wholegraph_error_code_t wholegraph_tensor_get_local_entry_start(
  size_t* local_entry_start, wholegraph_tensor_t wholegraph_tensor);

/* Half-open [starts, ends) per dimension; -1 = from the beginning / to the end. */
wholegraph_error_code_t wholegraph_tensor_get_subtensor(
  wholegraph_tensor_t wholegraph_tensor,
  int64_t* starts,
  int64_t* ends,
  wholegraph_tensor_t* sub_wholegraph_tensor);

/* The tensor this one was sliced from (itself when it is no slice). */
wholegraph_tensor_t wholegraph_tensor_get_root(wholegraph_tensor_t wholegraph_tensor);

#define WG_TENSOR_COUNT_DEBUG
/* Live tensor objects, for leak checks. */
int64_t get_wholegraph_tensor_count();

#ifdef __cplusplus
}
#endif
