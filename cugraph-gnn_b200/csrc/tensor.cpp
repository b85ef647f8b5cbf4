// Tensor C API. Behaviour follows the reference's cpp/src/wholegraph/wholegraph_tensor.cpp
// (create :39-96, views :112-207, local mapping :224-261, entry queries :283-395,
// sub-tensors :397-452).
#include "tensor.hpp"

#include <atomic>
#include <algorithm>
#include <cstdlib>

#include "common.hpp"
#include "handle.hpp"

static std::atomic<int64_t> g_tensor_count{0};

static wholegraph_tensor_* new_tensor()
{
  auto* t = static_cast<wholegraph_tensor_*>(calloc(1, sizeof(wholegraph_tensor_)));
  if (t != nullptr) g_tensor_count.fetch_add(1);
  return t;
}

static bool desc_ok_for_view(const wholegraph_tensor_description_t* d)
{
  return d != nullptr && d->dim >= 0 && d->dim <= WHOLEGRAPH_MAX_TENSOR_DIM &&
         d->dtype > WHOLEGRAPH_DT_UNKNOWN && d->dtype < WHOLEGRAPH_DT_COUNT;
}

// Bytes per sharding unit of the root tensor (one row, or one element for 1-D).
static size_t root_entry_bytes(wholegraph_tensor_t t)
{
  const auto& rd = t->root->desc;
  size_t es      = wholegraph_dtype_get_element_size(t->desc.dtype);
  return es * (rd.dim == 2 ? static_cast<size_t>(rd.strides[0]) : 1);
}

extern "C" {

int64_t get_wholegraph_tensor_count() { return g_tensor_count.load(); }

wholegraph_error_code_t wholegraph_create_tensor(wholegraph_tensor_t* out,
                                                   wholegraph_tensor_description_t* d,
                                                   wholegraph_comm_t comm,
                                                   wholegraph_memory_type_t memory_type,
                                                   wholegraph_memory_location_t memory_location,
                                                   size_t* tensor_entry_partition)
{
  if (out == nullptr || d == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (d->dim != 1 && d->dim != 2) return WHOLEGRAPH_INVALID_INPUT;
  if (d->storage_offset != 0 || d->strides[d->dim - 1] != 1) return WHOLEGRAPH_INVALID_INPUT;
  if (d->dtype <= WHOLEGRAPH_DT_UNKNOWN || d->dtype >= WHOLEGRAPH_DT_COUNT)
    return WHOLEGRAPH_INVALID_INPUT;
  size_t es          = wholegraph_dtype_get_element_size(d->dtype);
  size_t total_bytes = static_cast<size_t>(wholegraph_get_memory_element_count_from_tensor(d)) * es;
  size_t granularity = es * static_cast<size_t>(d->strides[0]);
  wholegraph_handle_t h = nullptr;
  auto rc = wholegraph_malloc(&h, total_bytes, comm, memory_type, memory_location, granularity,
                              tensor_entry_partition);
  if (rc != WHOLEGRAPH_SUCCESS) return rc;
  auto* t = new_tensor();
  if (t == nullptr) {
    wholegraph_free(h);
    return WHOLEGRAPH_OUT_OF_MEMORY;
  }
  t->handle        = h;
  t->desc          = *d;
  t->root          = t;
  t->is_wholegraph = true;
  t->own_handle    = true;
  *out             = t;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_destroy_tensor(wholegraph_tensor_t t)
{
  if (t == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (t->own_handle) {
    if (t->is_wholegraph) {
      WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_free(t->handle));
    } else {
      free(t->storage_ptr);
    }
  }
  g_tensor_count.fetch_add(-1);
  free(t);
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_make_tensor_from_pointer(wholegraph_tensor_t* out,
                                                              void* storage_ptr,
                                                              wholegraph_tensor_description_t* d)
{
  if (out == nullptr || !desc_ok_for_view(d)) return WHOLEGRAPH_INVALID_INPUT;
  if (d->dim > 0 && d->strides[d->dim - 1] != 1) return WHOLEGRAPH_INVALID_INPUT;
  auto* t = new_tensor();
  if (t == nullptr) return WHOLEGRAPH_OUT_OF_MEMORY;
  t->storage_ptr   = storage_ptr;
  t->desc          = *d;
  t->root          = t;
  t->is_wholegraph = false;
  t->own_handle    = false;
  *out             = t;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_make_tensor_from_handle(wholegraph_tensor_t* out,
                                                             wholegraph_handle_t handle,
                                                             wholegraph_tensor_description_t* d)
{
  if (out == nullptr || handle == nullptr || !desc_ok_for_view(d)) return WHOLEGRAPH_INVALID_INPUT;
  if (d->dim != 1 && d->dim != 2) return WHOLEGRAPH_INVALID_INPUT;
  if (d->strides[d->dim - 1] != 1) return WHOLEGRAPH_INVALID_INPUT;
  auto* t = new_tensor();
  if (t == nullptr) return WHOLEGRAPH_OUT_OF_MEMORY;
  t->handle        = handle;
  t->desc          = *d;
  t->root          = t;
  t->is_wholegraph = true;
  t->own_handle    = false;
  *out             = t;
  return WHOLEGRAPH_SUCCESS;
}

bool wholegraph_tensor_has_handle(wholegraph_tensor_t t) { return t != nullptr && t->is_wholegraph; }

wholegraph_handle_t wholegraph_tensor_get_memory_handle(wholegraph_tensor_t t)
{
  return (t != nullptr && t->is_wholegraph) ? t->handle : nullptr;
}

wholegraph_tensor_description_t* wholegraph_tensor_get_tensor_description(wholegraph_tensor_t t)
{
  return &t->desc;
}

wholegraph_error_code_t wholegraph_tensor_get_global_reference(wholegraph_tensor_t t,
                                                                 wholegraph_gref_t* gref)
{
  if (t == nullptr || gref == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (t->is_wholegraph) return wholegraph_get_global_reference(gref, t->handle);
  *gref = wholegraph_create_continuous_global_reference(t->storage_ptr);
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_tensor_map_local_tensor(wholegraph_tensor_t t,
                                                             wholegraph_tensor_t* local_tensor)
{
  if (t == nullptr || local_tensor == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!t->is_wholegraph) return WHOLEGRAPH_INVALID_VALUE;
  const auto& d = t->desc;
  if (d.dim != 1 && d.dim != 2) return WHOLEGRAPH_INVALID_VALUE;
  if (d.dim == 1 && d.storage_offset != 0) return WHOLEGRAPH_INVALID_VALUE;
  if (d.dim == 2 && d.storage_offset + d.sizes[1] > d.strides[0]) return WHOLEGRAPH_INVALID_VALUE;
  void* local_ptr   = nullptr;
  size_t local_size = 0, local_offset = 0;
  WHOLEGRAPH_RETURN_ON_FAIL(
    wholegraph_get_local_memory(&local_ptr, &local_size, &local_offset, t->handle));
  size_t es   = wholegraph_dtype_get_element_size(d.dtype);
  size_t gran = d.dim == 1 ? es : es * static_cast<size_t>(d.strides[0]);
  // The view may stop short of the allocation's tail (never of its head).
  size_t view_bytes = static_cast<size_t>(d.sizes[0]) * gran;
  size_t avail      = view_bytes > local_offset ? view_bytes - local_offset : 0;
  local_size        = std::min(local_size, avail);
  if (local_size % gran != 0) return WHOLEGRAPH_LOGIC_ERROR;
  wholegraph_tensor_description_t ld = d;
  ld.sizes[0]                         = static_cast<int64_t>(local_size / gran);
  return wholegraph_make_tensor_from_pointer(local_tensor, local_ptr, &ld);
}

void* wholegraph_tensor_get_data_pointer(wholegraph_tensor_t t)
{
  if (t == nullptr) return nullptr;
  char* p = nullptr;
  if (t->is_wholegraph) {
    if (wholegraph_get_memory_type(t->handle) != WHOLEGRAPH_MT_CONTINUOUS) return nullptr;
    if (wholegraph_get_global_pointer(reinterpret_cast<void**>(&p), t->handle) != WHOLEGRAPH_SUCCESS)
      return nullptr;
  } else {
    p = static_cast<char*>(t->storage_ptr);
  }
  return p + wholegraph_dtype_get_element_size(t->desc.dtype) * t->desc.storage_offset;
}

wholegraph_error_code_t wholegraph_tensor_get_entry_offsets(size_t* entry_offsets,
                                                              wholegraph_tensor_t t)
{
  if (entry_offsets == nullptr || t == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!t->is_wholegraph) {
    entry_offsets[0] = 0;
    entry_offsets[1] = static_cast<size_t>(t->root->desc.sizes[0]);
    return WHOLEGRAPH_SUCCESS;
  }
  size_t eb = root_entry_bytes(t);
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_get_rank_partition_offsets(entry_offsets, t->handle));
  int W = t->handle->comm->world_size;
  for (int i = 0; i <= W; i++) {
    if (entry_offsets[i] % eb != 0) return WHOLEGRAPH_LOGIC_ERROR;
    entry_offsets[i] /= eb;
  }
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_tensor_get_entry_partition_sizes(size_t* entry_partition,
                                                                      wholegraph_tensor_t t)
{
  if (entry_partition == nullptr || t == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!t->is_wholegraph) {
    entry_partition[0] = static_cast<size_t>(t->root->desc.sizes[0]);
    return WHOLEGRAPH_SUCCESS;
  }
  size_t eb = root_entry_bytes(t);
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_get_rank_partition_sizes(entry_partition, t->handle));
  int W = t->handle->comm->world_size;
  for (int i = 0; i < W; i++) {
    if (entry_partition[i] % eb != 0) return WHOLEGRAPH_LOGIC_ERROR;
    entry_partition[i] /= eb;
  }
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_tensor_get_local_entry_count(size_t* local_entry_count,
                                                                  wholegraph_tensor_t t)
{
  if (local_entry_count == nullptr || t == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!t->is_wholegraph) {
    *local_entry_count = static_cast<size_t>(t->root->desc.sizes[0]);
    return WHOLEGRAPH_SUCCESS;
  }
  size_t bytes = 0;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_get_local_size(&bytes, t->handle));
  size_t eb = root_entry_bytes(t);
  if (bytes % eb != 0) return WHOLEGRAPH_LOGIC_ERROR;
  *local_entry_count = bytes / eb;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_tensor_get_local_entry_start(size_t* local_entry_start,
                                                                  wholegraph_tensor_t t)
{
  if (local_entry_start == nullptr || t == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!t->is_wholegraph) {
    *local_entry_start = 0;
    return WHOLEGRAPH_SUCCESS;
  }
  size_t bytes = 0;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_get_local_offset(&bytes, t->handle));
  size_t eb = root_entry_bytes(t);
  if (bytes % eb != 0) return WHOLEGRAPH_LOGIC_ERROR;
  *local_entry_start = bytes / eb;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_tensor_get_subtensor(wholegraph_tensor_t t,
                                                          int64_t* starts,
                                                          int64_t* ends,
                                                          wholegraph_tensor_t* sub)
{
  if (t == nullptr || starts == nullptr || ends == nullptr || sub == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  if (t->desc.dim > 2) return WHOLEGRAPH_NOT_IMPLEMENTED;
  int dim            = t->desc.dim;
  int64_t new_offset = t->desc.storage_offset;
  int64_t new_size[2] = {0, 0};
  for (int i = 0; i < dim; i++) {
    int64_t s = starts[i] == -1 ? 0 : starts[i];
    int64_t e = ends[i] == -1 ? t->desc.sizes[i] : ends[i];
    if (e <= s || s >= t->desc.sizes[i] || e <= 0) return WHOLEGRAPH_INVALID_INPUT;
    new_offset += t->desc.strides[i] * s;
    new_size[i] = e - s;
  }
  auto* st = new_tensor();
  if (st == nullptr) return WHOLEGRAPH_OUT_OF_MEMORY;
  *st                     = *t;  // same storage and root
  st->own_handle          = false;
  st->desc.storage_offset = new_offset;
  for (int i = 0; i < dim; i++) st->desc.sizes[i] = new_size[i];
  *sub = st;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_tensor_t wholegraph_tensor_get_root(wholegraph_tensor_t t) { return t->root; }

}  // extern "C"
