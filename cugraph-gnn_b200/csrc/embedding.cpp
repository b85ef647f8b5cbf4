// Embedding objects: padded table + user view, optimizer and its state tensors, forward
// gather and the backward gather_gradient_apply step.
//
// Reference behaviour: cpp/src/wholegraph/embedding.cpp (allocate :77-134, gradient apply
// :136-314, state creation :316-420, C API :886-1110) and embedding_optimizer.cpp (parameter
// names and defaults :159-180, :286-297, :385-400; state names and initial values :179-211).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <wholegraph/embedding.h>
#include <wholegraph/wholegraph_b200.h>
#include <wholegraph/wholegraph_tensor_op.h>

#include "common.hpp"
#include "env.hpp"
#include "handle.hpp"
#include "kernels/cache.hpp"
#include "kernels/row_copy.hpp"
#include "kernels/sparse_optimizer.hpp"
#include "ops.hpp"
#include "tensor.hpp"

struct wholegraph_embedding_cache_policy_ {
  wholegraph_comm_t cache_comm;
  wholegraph_memory_type_t memory_type;
  wholegraph_memory_location_t memory_location;
  wholegraph_access_type_t access_type;
  float cache_ratio;
};

struct wholegraph_embedding_optimizer_ {
  wholegraph_optimizer_type_t type = WHOLEGRAPH_OPT_NONE;
  const char* name                 = "";
  std::map<std::string, float*> setters;
  std::vector<const char*> state_names;  // NULL-terminated
  float weight_decay = 0.f, epsilon = 1e-8f, beta1 = 0.9f, beta2 = 0.999f, adam_w = 0.f, alpha = 0.99f;
};

// A set-associative cache in front of an embedding table (reference: embedding_cache.hpp:64-74,
// embedding_cache.cpp:78-150): per set 32 tags, 32 LFU words and 32 lines, sharded like the rows
// they cover, plus this rank's exact access counters.
struct embedding_cache {
  int coverage               = 32;
  // A cache on another (smaller) communicator than its table: the ranks of that communicator
  // cache the WHOLE table between them, read-only; rank r of it holds the sets of table rows
  // [r * local_rows, (r + 1) * local_rows).
  bool node_level            = false;
  int64_t local_rows         = 0;
  wholegraph_tensor_t tags   = nullptr;  // int16 [sets, 32]
  wholegraph_tensor_t lfu    = nullptr;  // int16 [sets, 32]
  wholegraph_tensor_t lines  = nullptr;  // table dtype [sets * 32, padded dim]
  int64_t* access_count      = nullptr;  // device, one counter per local row
  ~embedding_cache()
  {
    if (tags) wholegraph_destroy_tensor(tags);
    if (lfu) wholegraph_destroy_tensor(lfu);
    if (lines) wholegraph_destroy_tensor(lines);
    if (access_count) cudaFree(access_count);
  }
};

struct wholegraph_embedding_ {
  wholegraph_comm_t comm            = nullptr;
  wholegraph_dtype_t dtype          = WHOLEGRAPH_DT_UNKNOWN;
  wholegraph_tensor_t allocated     = nullptr;  // [rows, padded dim], owns the handle
  wholegraph_tensor_t user          = nullptr;  // [rows, dim] view
  wholegraph_embedding_cache_policy_t cache_policy = nullptr;
  std::unique_ptr<embedding_cache> cache;
  int gather_sms                    = -1;
  int round_robin_size              = 0;
  int64_t dim = 0, padded_dim = 0;
  // optimizer
  wholegraph_embedding_optimizer_t optimizer = nullptr;
  wholegraph_embedding_t state_embedding     = nullptr;  // fp32 [rows, states * padded dim]
  std::map<std::string, wholegraph_tensor_t> state_views;
  wholegraph_tensor_t beta12t_padded = nullptr, beta12t_view = nullptr;
};

namespace {

using namespace wgb;

// Turn a failed call into the exception that carries its code to the C boundary.
void wgb_check(wholegraph_error_code_t rc, const char* what)
{
  if (rc != WHOLEGRAPH_SUCCESS) throw invalid_input(rc, format_string("%s failed with code %d", what, (int)rc));
}

// Row stride padded to 16 bytes (reference: embedding.cpp:32-39).
int64_t padded_dim_of(int64_t dim, size_t element_size)
{
  const int64_t align = static_cast<int64_t>(16 / element_size);
  return (dim + align - 1) / align * align;
}

struct local_rows_view {
  void* ptr;
  int64_t rows, start;
};
local_rows_view local_view_of(wholegraph_tensor_t t)
{
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(t);
  WGB_EXPECTS(h != nullptr, "tensor has no memory handle");
  const auto& d   = t->root->desc;
  const size_t eb = wholegraph_dtype_get_element_size(d.dtype) * (d.dim == 2 ? d.strides[0] : 1);
  const int me    = h->comm->world_rank;
  return {h->local_ptr, static_cast<int64_t>(h->part_sizes[me] / eb),
          static_cast<int64_t>(h->part_offsets[me] / eb)};
}

// Rows of one cache set for a cache ratio: round(32 / ratio), at most 16384 (the 14-bit row
// field of a tag).  Reference: embedding_cache.cpp:47-60.
int coverage_of(float cache_ratio)
{
  const long c = std::lround(static_cast<double>(kCacheSetSize) / cache_ratio);
  return static_cast<int>(std::min<long>(std::max<long>(c, kCacheSetSize), kCacheMaxCoverage));
}

// This rank's part of the cache and of the table behind it.
cache_view local_cache_of(const wholegraph_embedding_* e)
{
  cache_view v;
  if (e == nullptr || !e->cache) return v;
  if (e->cache->node_level) {
    // this rank's sets of a cache over the whole table; the table rows have no address here
    v.tags         = static_cast<uint16_t*>(local_view_of(e->cache->tags).ptr);
    v.lfu          = static_cast<uint16_t*>(local_view_of(e->cache->lfu).ptr);
    v.lines        = static_cast<char*>(local_view_of(e->cache->lines).ptr);
    v.access_count = e->cache->access_count;
    v.raw_rows     = nullptr;
    v.first_row    = e->cache->local_rows * e->cache_policy->cache_comm->world_rank;
    v.rows         = e->cache->local_rows;
    v.coverage     = e->cache->coverage;
    v.line_bytes   = e->padded_dim * static_cast<int64_t>(wholegraph_dtype_get_element_size(e->dtype));
    return v;
  }
  auto wl        = local_view_of(e->allocated);
  v.tags         = static_cast<uint16_t*>(local_view_of(e->cache->tags).ptr);
  v.lfu          = static_cast<uint16_t*>(local_view_of(e->cache->lfu).ptr);
  v.lines        = static_cast<char*>(local_view_of(e->cache->lines).ptr);
  v.access_count = e->cache->access_count;
  v.raw_rows     = static_cast<char*>(wl.ptr);
  v.first_row    = wl.start;
  v.rows         = wl.rows;
  v.coverage     = e->cache->coverage;
  v.line_bytes   = e->padded_dim * static_cast<int64_t>(wholegraph_dtype_get_element_size(e->dtype));
  return v;
}

// True when every rank can read every cache line and every table row through its own mapping,
// so that a gather needs no exchange of rows.
bool cache_is_mapped(const wholegraph_embedding_* e)
{
  auto mapped = [](wholegraph_tensor_t t) {
    wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(t);
    return h->type == WHOLEGRAPH_MT_CONTINUOUS && h->global_base != nullptr;
  };
  return mapped(e->allocated) && mapped(e->cache->tags) && mapped(e->cache->lfu) && mapped(e->cache->lines);
}

// The whole cache and table seen through the CONTINUOUS mappings (lookup only).
cache_view global_cache_of(const wholegraph_embedding_* e)
{
  cache_view v   = local_cache_of(e);
  auto base      = [](wholegraph_tensor_t t) { return wholegraph_tensor_get_memory_handle(t)->global_base; };
  v.tags         = static_cast<uint16_t*>(base(e->cache->tags));
  v.lfu          = static_cast<uint16_t*>(base(e->cache->lfu));
  v.lines        = static_cast<char*>(base(e->cache->lines));
  v.access_count = nullptr;
  v.raw_rows     = static_cast<char*>(base(e->allocated));
  v.first_row    = 0;
  v.rows         = e->allocated->desc.sizes[0];
  return v;
}

// Cache arrays of a cache on its own communicator (reference: local_cached_global_readonly_embedding,
// embedding.cpp:761-884, and the cache tensors of embedding_cache.cpp:78-150 created on the cache
// communicator): sets over all rows of the table, split evenly over the cache communicator's ranks.
wholegraph_error_code_t create_node_level_cache(wholegraph_embedding_* e)
{
  auto* policy = e->cache_policy;
  std::unique_ptr<embedding_cache> c(new embedding_cache());
  c->coverage    = coverage_of(policy->cache_ratio);
  c->node_level  = true;
  auto* cc       = policy->cache_comm;
  const int CW   = cc->world_size;
  const int64_t table_rows = e->allocated->desc.sizes[0];
  const int64_t sets_total = (table_rows + c->coverage - 1) / c->coverage;
  const int64_t per_rank   = (sets_total + CW - 1) / CW;
  c->local_rows            = per_rank * c->coverage;
  std::vector<size_t> sets_of(CW, static_cast<size_t>(per_rank)), lines_of(CW, static_cast<size_t>(per_rank) * kCacheSetSize);
  wholegraph_tensor_description_t d;
  wholegraph_initialize_tensor_desc(&d);
  d.dim = 2, d.dtype = WHOLEGRAPH_DT_INT16;
  d.sizes[0] = per_rank * CW, d.sizes[1] = kCacheSetSize, d.strides[0] = kCacheSetSize, d.strides[1] = 1;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->tags, &d, cc, WHOLEGRAPH_MT_CONTINUOUS, policy->memory_location,
                                                       sets_of.data()));
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->lfu, &d, cc, WHOLEGRAPH_MT_CONTINUOUS, policy->memory_location,
                                                       sets_of.data()));
  d.dtype    = e->dtype;
  d.sizes[0] = per_rank * CW * kCacheSetSize, d.sizes[1] = e->padded_dim, d.strides[0] = e->padded_dim;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->lines, &d, cc, WHOLEGRAPH_MT_CONTINUOUS, policy->memory_location,
                                                       lines_of.data()));
  WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&c->access_count), c->local_rows * sizeof(int64_t)));
  WGB_CUDA_CHECK(cudaMemset(c->access_count, 0, c->local_rows * sizeof(int64_t)));
  WGB_CUDA_CHECK(cudaMemset(local_view_of(c->tags).ptr, 0, per_rank * kCacheSetSize * sizeof(uint16_t)));
  WGB_CUDA_CHECK(cudaMemset(local_view_of(c->lfu).ptr, 0, per_rank * kCacheSetSize * sizeof(uint16_t)));
  WGB_CUDA_CHECK(cudaDeviceSynchronize());
  cc->barrier();
  e->cache = std::move(c);
  return WHOLEGRAPH_SUCCESS;
}

// Cache arrays for a table whose shards are whole sets.
wholegraph_error_code_t create_cache(wholegraph_embedding_* e)
{
  auto* policy = e->cache_policy;
  if (policy->cache_comm != e->comm) return create_node_level_cache(e);
  std::unique_ptr<embedding_cache> c(new embedding_cache());
  c->coverage = coverage_of(policy->cache_ratio);
  const int W = e->comm->world_size;
  std::vector<size_t> rows_of(W), sets_of(W), lines_of(W);
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_entry_partition_sizes(rows_of.data(), e->allocated));
  int64_t sets = 0;
  for (int r = 0; r < W; r++) {
    if (rows_of[r] == 0 || rows_of[r] % c->coverage != 0) {
      WGB_ERROR("with a cache every rank must hold a positive multiple of %d rows, rank %d holds %zu",
                c->coverage, r, rows_of[r]);
      return WHOLEGRAPH_INVALID_VALUE;
    }
    sets_of[r]  = rows_of[r] / c->coverage;
    lines_of[r] = sets_of[r] * kCacheSetSize;
    sets += static_cast<int64_t>(sets_of[r]);
  }
  wholegraph_tensor_description_t d;
  wholegraph_initialize_tensor_desc(&d);
  d.dim = 2, d.dtype = WHOLEGRAPH_DT_INT16;
  d.sizes[0] = sets, d.sizes[1] = kCacheSetSize, d.strides[0] = kCacheSetSize, d.strides[1] = 1;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->tags, &d, policy->cache_comm, policy->memory_type,
                                                       policy->memory_location, sets_of.data()));
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->lfu, &d, policy->cache_comm, policy->memory_type,
                                                       policy->memory_location, sets_of.data()));
  d.dtype    = e->dtype;
  d.sizes[0] = sets * kCacheSetSize, d.sizes[1] = e->padded_dim, d.strides[0] = e->padded_dim;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&c->lines, &d, policy->cache_comm, policy->memory_type,
                                                       policy->memory_location, lines_of.data()));
  const int me       = e->comm->world_rank;
  const size_t local = rows_of[me];
  WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&c->access_count), local * sizeof(int64_t)));
  WGB_CUDA_CHECK(cudaMemset(c->access_count, 0, local * sizeof(int64_t)));
  // Empty cache: no valid tag, zero counts.
  WGB_CUDA_CHECK(cudaMemset(local_view_of(c->tags).ptr, 0, sets_of[me] * kCacheSetSize * sizeof(uint16_t)));
  WGB_CUDA_CHECK(cudaMemset(local_view_of(c->lfu).ptr, 0, sets_of[me] * kCacheSetSize * sizeof(uint16_t)));
  WGB_CUDA_CHECK(cudaDeviceSynchronize());
  e->comm->barrier();
  e->cache = std::move(c);
  return WHOLEGRAPH_SUCCESS;
}

// Gather through a read-only cache that lives on a smaller communicator than its table (every
// node caching the whole table for itself).  Reference: local_cached_global_readonly_embedding::gather,
// embedding.cpp:772-884, with update_cache_different_comm (embedding_cache_func.cu:511-622) and
// try_gather_cached_func (gather_cached_func.cu:366-467).
//   adjust_cache: the ids go to the cache ranks that hold their sets; there the LFU update only
//   decides which rows get which lines; the rows are then gathered from the table (a collective of
//   the table's communicator when the table is DISTRIBUTED) and scattered into the lines.
//   lookup: hits are copied from the lines (every cache rank maps all of them), misses are left to
//   one gather from the table over the list of missed ids.
void node_level_cached_gather(wholegraph_embedding_* e, wholegraph_tensor_t indices, wholegraph_tensor_t output,
                              const void* ids, bool ids_are_64, int64_t n, void* out,
                              const wholegraph_matrix_description_t& od, const wholegraph_matrix_description_t& tab,
                              bool adjust_cache, wholegraph_env_func_t* env, cudaStream_t stream)
{
  auto* cc      = e->cache_policy->cache_comm;
  const int CW  = cc->world_size;
  const size_t es = wholegraph_dtype_get_element_size(e->dtype);
  cache_view mine = local_cache_of(e);
  auto table_gather = [&](void* id_ptr, wholegraph_dtype_t id_dt, int64_t count, wholegraph_tensor_t dst) {
    // collective on the table's communicator when the table is DISTRIBUTED: always called
    wholegraph_tensor_description_t idd;
    wholegraph_initialize_tensor_desc(&idd);
    idd.dim = 1, idd.dtype = id_dt, idd.sizes[0] = count, idd.strides[0] = 1;
    wholegraph_tensor_t idt = nullptr;
    wgb_check(wholegraph_make_tensor_from_pointer(&idt, id_ptr, &idd), "make_tensor_from_pointer");
    auto rc = wholegraph_gather(e->user, idt, dst, env, stream, e->gather_sms);
    wholegraph_destroy_tensor(idt);
    wgb_check(rc, "wholegraph_gather");
  };
  if (adjust_cache) {
    std::vector<int64_t> first_row(CW + 1);
    for (int r = 0; r <= CW; r++) first_row[r] = e->cache->local_rows * r;
    exchange_plan plan(env);
    plan.build(ids, ids_are_64, n, first_row, cc, stream);
    const int64_t m = std::max<int64_t>(plan.total_recv, 1);
    temp_buffer ws(env), rows_buf(env), lines_buf(env), count_buf(env), fetched(env);
    auto* load_rows  = static_cast<int64_t*>(rows_buf.device(m, WHOLEGRAPH_DT_INT64));
    auto* load_lines = static_cast<int64_t*>(lines_buf.device(m, WHOLEGRAPH_DT_INT64));
    auto* load_count = static_cast<int*>(count_buf.device(64, WHOLEGRAPH_DT_INT));
    WGB_CUDA_CHECK(cudaMemsetAsync(load_rows, 0xff, sizeof(int64_t) * m, stream));   // -1: skipped by both copies
    WGB_CUDA_CHECK(cudaMemsetAsync(load_lines, 0xff, sizeof(int64_t) * m, stream));
    WGB_CUDA_CHECK(cudaMemsetAsync(load_count, 0, sizeof(int), stream));
    if (plan.total_recv > 0) {
      cache_view decide  = mine;
      decide.load_rows   = load_rows;
      decide.load_lines  = load_lines;
      decide.load_count  = load_count;
      cache_update(plan.recv_ids, true, plan.total_recv, decide,
                   ws.device_bytes(cache_update_workspace_bytes(plan.total_recv)), stream);
    }
    // rows to load: table -> dense buffer -> lines (entries left at -1 move nothing)
    char* rows = static_cast<char*>(fetched.device_bytes(static_cast<size_t>(m) * e->padded_dim * es));
    wholegraph_tensor_description_t rd;
    wholegraph_initialize_tensor_desc(&rd);
    rd.dim = 2, rd.dtype = e->dtype, rd.sizes[0] = m, rd.sizes[1] = e->dim, rd.strides[0] = e->padded_dim, rd.strides[1] = 1;
    wholegraph_tensor_t rt = nullptr;
    wgb_check(wholegraph_make_tensor_from_pointer(&rt, rows, &rd), "make_tensor_from_pointer");
    table_gather(load_rows, WHOLEGRAPH_DT_INT64, m, rt);
    wholegraph_destroy_tensor(rt);
    row_copy_args put;
    put.src = rows, put.src_dt = e->dtype, put.src_stride = e->padded_dim, put.src_select = ROW_SEQUENTIAL;
    put.dst = mine.lines, put.dst_dt = e->dtype, put.dst_stride = e->padded_dim, put.dst_select = ROW_BY_INDEX;
    put.dim = e->dim, put.count = m, put.indices = load_lines, put.indices_are_64 = true;
    launch_row_copy(put, stream);
    // the other ranks of the cache communicator read these lines next
    WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
    cc->barrier();
  }
  // lookup in all sets of the cache communicator (tags and lines are mapped on each of its ranks)
  cache_view all = mine;
  auto base      = [](wholegraph_tensor_t t) { return wholegraph_tensor_get_memory_handle(t)->global_base; };
  all.tags       = static_cast<uint16_t*>(base(e->cache->tags));
  all.lfu        = static_cast<uint16_t*>(base(e->cache->lfu));
  all.lines      = static_cast<char*>(base(e->cache->lines));
  all.access_count = nullptr;
  all.first_row  = 0;
  all.rows       = e->cache->local_rows * CW;
  temp_buffer address_buf(env), miss_buf(env);
  const int64_t cap = std::max<int64_t>(n, 1);
  auto* addr = static_cast<int64_t*>(address_buf.device(cap, WHOLEGRAPH_DT_INT64));
  auto* miss = static_cast<int64_t*>(miss_buf.device(cap, WHOLEGRAPH_DT_INT64));
  if (n > 0) {
    cache_lookup(ids, ids_are_64, n, all, false, addr, stream, miss);
    row_copy_args g;
    g.src_dt = tab.dtype, g.src_stride = tab.stride, g.src_offset = 0;
    g.src_select = ROW_BY_ADDRESS, g.indices = addr, g.indices_are_64 = true;
    g.dst = out, g.dst_dt = od.dtype, g.dst_stride = od.stride, g.dst_offset = od.storage_offset;
    g.dim = e->dim, g.count = n, g.sm_hint = e->gather_sms;
    launch_row_copy(g, stream);
  }
  (void)indices;
  table_gather(miss, WHOLEGRAPH_DT_INT64, n, output);  // rows the cache left out
}

// Forward gather through the cache.
void cached_gather(wholegraph_embedding_* e, wholegraph_tensor_t indices, wholegraph_tensor_t output,
                   bool adjust_cache, wholegraph_env_func_t* env, cudaStream_t stream)
{
  auto* id = wholegraph_tensor_get_tensor_description(indices);
  WGB_EXPECTS(id->dim == 1 && id->strides[0] == 1, "indices must be a dense 1-D tensor");
  WGB_EXPECTS(id->dtype == WHOLEGRAPH_DT_INT || id->dtype == WHOLEGRAPH_DT_INT64,
              "indices must be int32 or int64");
  wholegraph_matrix_description_t od, tab;
  WGB_EXPECTS(wholegraph_convert_tensor_desc_to_matrix(&od, wholegraph_tensor_get_tensor_description(output)),
              "output must be a 2-D tensor");
  WGB_EXPECTS(wholegraph_convert_tensor_desc_to_matrix(&tab, wholegraph_tensor_get_tensor_description(e->user)),
              "bad embedding tensor");
  WGB_EXPECTS(od.sizes[0] == id->sizes[0], "%ld output rows for %ld indices", (long)od.sizes[0],
              (long)id->sizes[0]);
  WGB_EXPECTS(od.sizes[1] == e->dim, "output rows have %ld elements, the embedding %ld", (long)od.sizes[1],
              (long)e->dim);
  const int64_t n       = id->sizes[0];
  const bool ids_are_64 = id->dtype == WHOLEGRAPH_DT_INT64;
  const void* ids       = wholegraph_tensor_get_data_pointer(indices);
  void* out             = wholegraph_tensor_get_data_pointer(output);
  WGB_EXPECTS(n == 0 || (ids != nullptr && out != nullptr), "indices and output must be device buffers");
  // The copy launchers add the storage offset themselves: hand them the start of the storage.
  if (out != nullptr) out = static_cast<char*>(out) - od.storage_offset * wholegraph_dtype_get_element_size(od.dtype);
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(e->allocated);
  auto* comm            = e->comm;
  const cache_view mine = local_cache_of(e);
  if (e->cache->node_level) {
    node_level_cached_gather(e, indices, output, ids, ids_are_64, n, out, od, tab, adjust_cache, env, stream);
    return;
  }
  if (comm->world_size == 1 || !cache_is_mapped(e)) {
    // Owners look their cache up for the ids routed to them and serve the rows.
    gather_distributed(h, tab, ids, ids_are_64, n, out, od, env, stream, e->gather_sms, &mine, adjust_cache);
    return;
  }
  // Cache and table are mapped everywhere: only the LFU update needs the ids at their owners.
  if (adjust_cache) {
    auto first_row = entry_offsets_of(h, wholegraph_dtype_get_element_size(e->dtype) * e->padded_dim);
    exchange_plan plan(env);
    plan.build(ids, ids_are_64, n, first_row, comm, stream);
    temp_buffer ws(env);
    if (plan.total_recv > 0)
      cache_update(plan.recv_ids, true, plan.total_recv, mine,
                   ws.device_bytes(cache_update_workspace_bytes(plan.total_recv)), stream);
    // Peers read these lines next.
    WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
    comm->barrier();
  }
  if (n == 0) return;
  temp_buffer address_buf(env);
  auto* addr = static_cast<int64_t*>(address_buf.device(n, WHOLEGRAPH_DT_INT64));
  cache_lookup(ids, ids_are_64, n, global_cache_of(e), false, addr, stream);
  row_copy_args g;
  g.src_dt = tab.dtype, g.src_stride = tab.stride, g.src_offset = tab.storage_offset;
  g.src_select = ROW_BY_ADDRESS, g.indices = addr, g.indices_are_64 = true;
  g.dst = out, g.dst_dt = od.dtype, g.dst_stride = od.stride, g.dst_offset = od.storage_offset;
  g.dim = e->dim, g.count = n, g.sm_hint = e->gather_sms;
  launch_row_copy(g, stream);
}

void destroy_states(wholegraph_embedding_* e)
{
  for (auto& kv : e->state_views) wholegraph_destroy_tensor(kv.second);
  e->state_views.clear();
  if (e->beta12t_view) wholegraph_destroy_tensor(e->beta12t_view);
  if (e->beta12t_padded) wholegraph_destroy_tensor(e->beta12t_padded);
  e->beta12t_view = e->beta12t_padded = nullptr;
  if (e->state_embedding) wholegraph_destroy_embedding(e->state_embedding);
  e->state_embedding = nullptr;
}

wholegraph_error_code_t create_states(wholegraph_embedding_* e)
{
  auto* opt = e->optimizer;
  std::vector<std::string> per_element;
  if (opt->type == WHOLEGRAPH_OPT_LAZY_ADAM) per_element = {"m", "v"};
  if (opt->type == WHOLEGRAPH_OPT_ADAGRAD) per_element = {"state_sum"};
  if (opt->type == WHOLEGRAPH_OPT_RMSPROP) per_element = {"v"};
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(e->allocated);
  const int W           = e->comm->world_size;
  std::vector<size_t> partition(W);
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_entry_partition_sizes(partition.data(), e->allocated));
  const int64_t rows = e->allocated->desc.sizes[0];
  if (!per_element.empty()) {
    // Every per-element state is padded like the table row (in table elements), so that state
    // k of a row starts k * padded_dim floats into the state row.
    wholegraph_tensor_description_t sd;
    wholegraph_initialize_tensor_desc(&sd);
    sd.dim        = 2;
    sd.dtype      = WHOLEGRAPH_DT_FLOAT;
    sd.sizes[0]   = rows;
    sd.sizes[1]   = static_cast<int64_t>(per_element.size()) * e->padded_dim;
    sd.strides[0] = sd.sizes[1];
    sd.strides[1] = 1;
    WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_embedding(&e->state_embedding, &sd, e->comm, h->type,
                                                            h->location, e->cache_policy, partition.data()));
    wholegraph_tensor_t st = wholegraph_embedding_get_embedding_tensor(e->state_embedding);
    for (size_t k = 0; k < per_element.size(); k++) {
      int64_t starts[2] = {0, static_cast<int64_t>(k) * e->padded_dim};
      int64_t ends[2]   = {e->user->desc.sizes[0], starts[1] + e->dim};
      wholegraph_tensor_t view = nullptr;
      WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_subtensor(st, starts, ends, &view));
      e->state_views[per_element[k]] = view;
    }
    auto lv = local_view_of(e->state_embedding->allocated);
    WGB_CUDA_CHECK(cudaMemset(lv.ptr, 0, static_cast<size_t>(lv.rows) * e->state_embedding->padded_dim * 4));
  }
  if (opt->type == WHOLEGRAPH_OPT_LAZY_ADAM) {
    wholegraph_tensor_description_t bd;
    wholegraph_initialize_tensor_desc(&bd);
    bd.dim        = 2;
    bd.dtype      = WHOLEGRAPH_DT_FLOAT;
    bd.sizes[0]   = rows;
    bd.sizes[1]   = 2;
    bd.strides[0] = 2;
    bd.strides[1] = 1;
    WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&e->beta12t_padded, &bd, e->comm,
                                                         WHOLEGRAPH_MT_DISTRIBUTED, WHOLEGRAPH_ML_DEVICE,
                                                         partition.data()));
    int64_t starts[2] = {0, 0};
    int64_t ends[2]   = {e->user->desc.sizes[0], 2};
    WHOLEGRAPH_RETURN_ON_FAIL(
      wholegraph_tensor_get_subtensor(e->beta12t_padded, starts, ends, &e->beta12t_view));
    auto lv = local_view_of(e->beta12t_padded);
    fill_float(static_cast<float*>(lv.ptr), 1.0f, lv.rows * 2, nullptr);
  }
  WGB_CUDA_CHECK(cudaDeviceSynchronize());
  e->comm->barrier();
  return WHOLEGRAPH_SUCCESS;
}

// Gradient apply over several ranks with nothing sized on the host: every rank adds up its own
// duplicates (as in the default path) but leaves the sums in ITS OWN region of the peer-mapped
// arena, together with its distinct ids and the number of them it has for every owner; after a
// barrier in stream order every owner merges what the senders hold for it (merged_apply: bitmaps
// over its rows instead of a sort) and reads the sums rows straight from the senders' regions
// while it updates its rows - transfer and update are one kernel.  The order of additions is that
// of the default path: per rank in arrival order, then the per-rank sums in rank order.  Returns
// false, on every rank alike and before anything was enqueued, when the path does not apply.
bool gradient_apply_sync_free(wholegraph_embedding_* e, const sparse_apply_args& shard, const void* ids, bool ids_are_64,
                              int64_t n, const float* g, int64_t g_stride, const std::vector<int64_t>& first_row,
                              wholegraph_env_func_t* env, cudaStream_t stream)
{
  auto* comm   = e->comm;
  const int W  = comm->world_size;
  const int me = comm->world_rank;
  if (!comm->tuning.sync_free || !comm->tuning.gradient_presum || !comm->tuning.peer_exchange ||
      (comm->board == nullptr && W > 1) || comm->arena_unavailable || W > kMaxMergeRanks ||
      shard.weight_cache.tags != nullptr || shard.state_cache.tags != nullptr)
    return false;
  int64_t widest = 0;  // rows of the largest shard: the merge bitmaps must stay small
  for (int r = 0; r < W; r++) widest = std::max(widest, first_row[r + 1] - first_row[r]);
  if (widest >= (int64_t(1) << 31) || static_cast<int64_t>(W) * ((widest + 31) / 32) > (int64_t(1) << 27)) return false;
  const size_t row_b = static_cast<size_t>(e->dim) * sizeof(float);

  int64_t mine[wholegraph_comm_::kBoardValues] = {n, e->dim, static_cast<int64_t>(shard.hyper.type),
                                                  reduce_duplicates_supported(n, first_row[W], W) ? 1 : 0,
                                                  static_cast<int64_t>(wholegraph_tensor_get_memory_handle(e->allocated)->id),
                                                  0x67726164 /* "grad" */};
  std::vector<int64_t> all(static_cast<size_t>(W) * wholegraph_comm_::kBoardValues);
  comm->board_exchange(mine, all.data());
  int64_t capacity = 1, total_n = 0;
  bool supported   = true;
  for (int r = 0; r < W; r++) {
    const int64_t* v = all.data() + static_cast<size_t>(r) * wholegraph_comm_::kBoardValues;
    WGB_EXPECTS(v[1] == mine[1] && v[2] == mine[2] && v[4] == mine[4] && v[5] == mine[5],
                "rank %d is in another collective call than rank %d (gradient apply)", r, me);
    capacity  = std::max(capacity, v[0]);
    total_n += v[0];
    supported = supported && v[3] != 0;
  }
  if (!supported) return false;
  auto ids_offset  = []() { return size_t(2) * sizeof(int64_t) * kMaxMergeRanks; };
  auto sums_offset = [&](int64_t cap) { return ids_offset() + (static_cast<size_t>(cap) * 8 + 255) / 256 * 256; };
  auto region_size = [&](int64_t cap) { return sums_offset(cap) + static_cast<size_t>(cap) * row_b; };
  if (!ensure_peer_arena(comm, region_size(capacity), stream)) return false;
  {  // every rank derives the same capacity from the arena's size
    int64_t most = (static_cast<int64_t>(comm->arena_bytes) - static_cast<int64_t>(ids_offset()) - 256) /
                   static_cast<int64_t>(row_b + 8);
    most = std::min<int64_t>(most, (int64_t(1) << 31) - 2);
    while (most > capacity && region_size(most) > comm->arena_bytes) most--;
    capacity = std::max(capacity, most);
  }
  if (comm->status_word == nullptr) {
    WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&comm->status_word), 256));
    WGB_CUDA_CHECK(cudaMemset(comm->status_word, 0, 256));
    WGB_CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&comm->status_host), 64));
    *comm->status_host = 0;
  }
  if (*comm->status_host != 0) {
    *comm->status_host = 0;
    WGB_CUDA_CHECK(cudaMemsetAsync(comm->status_word, 0, sizeof(int), stream));
    throw comm_error("an earlier distributed op refused ids or sizes a peer had left for this rank");
  }

  phase_timer timer(stream);
  timer.mark("start");
  char* region     = peer_arena_region(comm, me);
  int64_t* header  = reinterpret_cast<int64_t*>(region);
  int64_t* uids    = reinterpret_cast<int64_t*>(region + ids_offset());
  float* sums      = reinterpret_cast<float*>(region + sums_offset(capacity));
  temp_buffer presum_ws(env), merge_ws(env);
  if (n > 0) {
    void* pws = presum_ws.device_bytes(reduce_duplicates_workspace_bytes(n, first_row[W], e->dim));
    reduce_duplicates_group(ids, ids_are_64, n, e->dim, first_row.data(), W, pws, uids, header, header + W, stream);
    timer.mark("group");
    // the sums of the k-th distinct id go to row k: one destination, whatever its owner
    const int64_t everything = n;
    float* dest              = sums;
    reduce_duplicates_sum(n, first_row[W], g, g_stride, e->dim, 1, &everything, &dest, pws, stream);
    timer.mark("presum");
  } else {
    WGB_CUDA_CHECK(cudaMemsetAsync(header, 0, sizeof(int64_t) * 2 * W, stream));
  }
  comm->stream_barrier(stream);  // every sender's header, ids and sums are in place
  timer.mark("barrier");

  merged_apply_args m;
  m.world = W, m.me = me;
  for (int r = 0; r < W; r++) {
    char* rr           = peer_arena_region(comm, r);
    m.sender[r].header = reinterpret_cast<const int64_t*>(rr);
    m.sender[r].ids    = reinterpret_cast<const int64_t*>(rr + ids_offset());
    m.sender[r].sums   = reinterpret_cast<const float*>(rr + sums_offset(capacity));
  }
  m.capacity            = capacity;
  m.entries_upper_bound = std::min<int64_t>(total_n, static_cast<int64_t>(W) * shard.local_rows);
  m.status              = comm->status_word;
  m.shard               = shard;
  merged_apply(m, merge_ws.device_bytes(merged_apply_workspace_bytes(W, shard.local_rows, m.entries_upper_bound)), stream);
  timer.mark("merge+apply");
  comm->stream_barrier(stream);  // nobody reads a sender's region any more
  WGB_CUDA_CHECK(cudaMemcpyAsync(comm->status_host, comm->status_word, sizeof(int), cudaMemcpyDeviceToHost, stream));
  if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaEventRecord(comm->arena_idle, stream));
  timer.mark("barrier");
  return true;
}

// Backward step on already-mapped ids.
void gradient_apply(wholegraph_embedding_* e, wholegraph_tensor_t indices, wholegraph_tensor_t grads,
                    bool adjust_cache, float lr, wholegraph_env_func_t* env, cudaStream_t stream)
{
  WGB_EXPECTS(e->optimizer != nullptr, "the embedding has no optimizer");
  auto* id = wholegraph_tensor_get_tensor_description(indices);
  auto* gd = wholegraph_tensor_get_tensor_description(grads);
  WGB_EXPECTS(id->dim == 1 && id->strides[0] == 1, "indices must be a dense 1-D tensor");
  WGB_EXPECTS(gd->dim == 2 && gd->strides[1] == 1 && gd->dtype == WHOLEGRAPH_DT_FLOAT,
              "gradients must be a 2-D fp32 tensor");
  WGB_EXPECTS(gd->sizes[0] == id->sizes[0], "%ld gradient rows for %ld indices", (long)gd->sizes[0],
              (long)id->sizes[0]);
  WGB_EXPECTS(gd->sizes[1] == e->dim, "gradient rows have %ld elements, the embedding %ld",
              (long)gd->sizes[1], (long)e->dim);
  const int64_t n       = id->sizes[0];
  const bool ids_are_64 = id->dtype != WHOLEGRAPH_DT_INT;
  const void* ids       = wholegraph_tensor_get_data_pointer(indices);
  const float* g        = static_cast<const float*>(wholegraph_tensor_get_data_pointer(grads));
  auto* comm            = e->comm;
  const int W           = comm->world_size;
  const int me          = comm->world_rank;

  auto wl = local_view_of(e->allocated);
  sparse_apply_args a;
  a.dim           = e->dim;
  a.local_start   = wl.start;
  a.local_rows    = wl.rows;
  a.weights       = wl.ptr;
  a.weight_dtype  = e->dtype;
  a.weight_stride = e->padded_dim;
  if (e->state_embedding != nullptr) {
    auto sl        = local_view_of(e->state_embedding->allocated);
    a.state        = static_cast<float*>(sl.ptr);
    a.state_stride = e->state_embedding->padded_dim;
    a.v_offset     = e->padded_dim;
  }
  if (e->beta12t_padded != nullptr) a.beta12t = static_cast<float*>(local_view_of(e->beta12t_padded).ptr);
  auto* o              = e->optimizer;
  a.hyper.type         = o->type;
  a.hyper.lr           = lr;
  a.hyper.weight_decay = o->weight_decay;
  a.hyper.epsilon      = o->epsilon;
  a.hyper.beta1        = o->beta1;
  a.hyper.beta2        = o->beta2;
  a.hyper.alpha        = o->alpha;
  a.hyper.adam_w       = o->adam_w > 0.5f;

  // With caches the update reads and writes a row's current copy: its line (marked modified)
  // when it has one.  An LFU update with the ids this rank owns may come first.
  a.weight_cache = local_cache_of(e);
  a.state_cache  = local_cache_of(e->state_embedding);
  temp_buffer cache_ws(env);
  auto adjust = [&](const void* owned_ids, bool are_64, int64_t count) {
    if (!adjust_cache || count == 0) return;
    for (const cache_view* c : {&a.weight_cache, &a.state_cache}) {
      if (c->tags == nullptr) continue;
      cache_update(owned_ids, are_64, count, *c, cache_ws.device_bytes(cache_update_workspace_bytes(count)),
                   stream);
    }
  };

  temp_buffer ws(env);
  if (W == 1 && !(comm->tuning.single_rank_exchange && a.weight_cache.tags == nullptr && a.state_cache.tags == nullptr)) {
    if (n == 0) return;
    a.ids = ids, a.ids_are_64 = ids_are_64, a.count = n;
    a.grads = g, a.grad_stride = gd->strides[0];
    adjust(ids, ids_are_64, n);
    sparse_apply(a, ws.device_bytes(sparse_apply_workspace_bytes(n, wl.rows, e->dim)), stream);
    return;
  }

  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(e->allocated);
  auto first_row        = entry_offsets_of(h, wholegraph_dtype_get_element_size(e->dtype) * e->padded_dim);
  const size_t row_b    = static_cast<size_t>(e->dim) * sizeof(float);
  exchange_plan plan(env);
  temp_buffer send_buf(env), recv_buf(env), uid_buf(env), counts_buf(env), presum_ws(env);
  // A call on another stream may still be reading this rank's arena region.
  if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaStreamWaitEvent(stream, comm->arena_idle, 0));
  if (gradient_apply_sync_free(e, a, ids, ids_are_64, n, g, gd->strides[0], first_row, env, stream)) return;
  char* recv = nullptr;
  phase_timer timer(stream);
  timer.mark("start");

  // WG_GRADIENT_PRESUM=0 routes every gradient row, as the reference does.  By default each rank
  // first adds up its own duplicates, so that an id crosses the wire at most once per rank and a
  // hot row does not flood its owner; the owner then adds the per-rank sums in rank order.
  const bool presum = comm->tuning.gradient_presum && reduce_duplicates_supported(n, first_row[W], W);
  if (presum) {
    int64_t* cdev = static_cast<int64_t*>(counts_buf.device(3 * W, WHOLEGRAPH_DT_INT64));
    int64_t* uids = static_cast<int64_t*>(uid_buf.device(std::max<int64_t>(n, 1), WHOLEGRAPH_DT_INT64));
    void* pws     = n > 0 ? presum_ws.device_bytes(reduce_duplicates_workspace_bytes(n, first_row[W], e->dim)) : nullptr;
    if (n > 0) {
      reduce_duplicates_group(ids, ids_are_64, n, e->dim, first_row.data(), W, pws, uids, cdev, cdev + W, stream);
    } else {
      WGB_CUDA_CHECK(cudaMemsetAsync(cdev, 0, sizeof(int64_t) * 2 * W, stream));
    }
    timer.mark("group");
    plan.build_grouped(uids, cdev, comm, stream);
    timer.mark("counts+ids");
    // The sums go into a dense buffer that NCCL moves, or - with WG_PEER_GRADIENT=1 and the
    // peer-mapped arena - straight into their owner's region (summation and transfer in one
    // kernel).  At 8 GPUs the fused kernel's remote stores ran no faster than the NCCL exchange
    // (2.74 against 2.63 ms per step), so it is not the default.
    const bool peer = comm->tuning.peer_gradient &&
                      ensure_peer_arena(comm, static_cast<size_t>(plan.max_total_recv()) * row_b, stream);
    std::vector<float*> dest(W);
    char* sums = nullptr;
    if (peer) {
      recv = peer_arena_region(comm, me);
      for (int r = 0; r < W; r++)
        dest[r] = reinterpret_cast<float*>(peer_arena_region(comm, r) + plan.arrival_start(me, r) * row_b);
    } else {
      sums = static_cast<char*>(send_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));
      recv = static_cast<char*>(recv_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));
      for (int r = 0; r < W; r++) dest[r] = reinterpret_cast<float*>(sums + plan.send_displs[r] * row_b);
      // own rows go straight into their slot of the receive buffer
      dest[me] = reinterpret_cast<float*>(recv + plan.recv_displs[me] * row_b);
    }
    if (n > 0)
      reduce_duplicates_sum(n, first_row[W], g, gd->strides[0], e->dim, W, plan.send_counts.data(), dest.data(), pws,
                            stream);
    timer.mark("presum");
    if (peer) {
      comm->stream_barrier(stream);  // every sender's sums have landed
    } else {
      auto nothing = [](const list_segments&) {};  // rows are already where the exchange reads them
      pipelined_exchange(comm, plan.send_counts, plan.send_displs, plan.recv_counts, plan.recv_displs, sums, recv,
                         row_b, stream, nothing, nothing, plan.chunk_count(row_b, 1, comm->tuning.exchange_chunks));
    }
  } else {
    // Every gradient row goes to the owner of its id: the pipeline of a distributed scatter, with
    // fp32 rows on the wire.
    plan.build(ids, ids_are_64, n, first_row, comm, stream);
    char* send = static_cast<char*>(send_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));
    recv       = static_cast<char*>(recv_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));
    row_copy_args pack;
    pack.src = g, pack.src_dt = WHOLEGRAPH_DT_FLOAT, pack.src_stride = gd->strides[0];
    pack.src_select = ROW_BY_POSITION;
    pack.dst_dt = WHOLEGRAPH_DT_FLOAT, pack.dst_stride = e->dim, pack.dim = e->dim;
    {  // own rows go straight into their slot of the receive buffer
      row_copy_args s0 = pack;
      s0.dst           = recv + plan.recv_displs[me] * row_b;
      s0.positions     = plan.positions + plan.send_displs[me];
      s0.count         = plan.send_counts[me];
      launch_row_copy(s0, stream);
    }
    pack.dst = send, pack.positions = plan.positions;
    pipelined_exchange(
      comm, plan.send_counts, plan.send_displs, plan.recv_counts, plan.recv_displs, send, recv, row_b, stream,
      [&](const list_segments& seg) {
        row_copy_args ps = pack;
        ps.segments = seg, ps.count = seg.total();
        launch_row_copy(ps, stream);
      },
      [](const list_segments&) {},  // the update below needs every row: nothing to do per chunk
      plan.chunk_count(row_b, 0, comm->tuning.exchange_chunks));
  }
  timer.mark("exchange");
  if (plan.total_recv == 0) {
    if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaEventRecord(comm->arena_idle, stream));
    return;
  }
  a.ids = plan.recv_ids, a.ids_are_64 = true, a.count = plan.total_recv;
  a.grads = reinterpret_cast<const float*>(recv), a.grad_stride = e->dim;
  adjust(plan.recv_ids, true, plan.total_recv);
  sparse_apply(a, ws.device_bytes(sparse_apply_workspace_bytes(plan.total_recv, wl.rows, e->dim)), stream);
  if (comm->arena_idle != nullptr) WGB_CUDA_CHECK(cudaEventRecord(comm->arena_idle, stream));
  timer.mark("apply");
}

// Run `fn(mapped indices)`, remapping the ids first when the embedding is sharded round-robin.
template <typename F>
wholegraph_error_code_t with_mapped_indices(wholegraph_embedding_* e, wholegraph_tensor_t indices,
                                             wholegraph_env_func_t* env, cudaStream_t stream, F fn)
{
  if (e->round_robin_size == 0) return fn(indices);
  auto* d = wholegraph_tensor_get_tensor_description(indices);
  temp_buffer mapped(env);
  void* out = mapped.device(static_cast<size_t>(d->sizes[0]), d->dtype);
  size_t entry_start = 0;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_tensor_get_local_entry_start(&entry_start, e->allocated));
  round_robin_remap(wholegraph_tensor_get_data_pointer(indices), out, d->dtype != WHOLEGRAPH_DT_INT,
                    d->sizes[0], e->comm->world_size, static_cast<int64_t>(entry_start),
                    e->round_robin_size, stream);
  wholegraph_tensor_description_t md = *d;
  md.storage_offset                   = 0;
  wholegraph_tensor_t mt              = nullptr;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_make_tensor_from_pointer(&mt, out, &md));
  auto rc = fn(mt);
  wholegraph_destroy_tensor(mt);
  return rc;
}

}  // namespace

extern "C" {

wholegraph_error_code_t wholegraph_create_embedding_optimizer(
  wholegraph_embedding_optimizer_t* optimizer, wholegraph_optimizer_type_t optimizer_type)
{
  if (optimizer == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  std::unique_ptr<wholegraph_embedding_optimizer_> o(new wholegraph_embedding_optimizer_());
  o->type = optimizer_type;
  o->setters["weight_decay"] = &o->weight_decay;
  switch (optimizer_type) {
    case WHOLEGRAPH_OPT_SGD:
      o->name        = "SGD";
      o->state_names = {nullptr};
      break;
    case WHOLEGRAPH_OPT_LAZY_ADAM:
      o->name               = "LazyAdam";
      o->setters["epsilon"] = &o->epsilon;
      o->setters["beta1"]   = &o->beta1;
      o->setters["beta2"]   = &o->beta2;
      o->setters["adam_w"]  = &o->adam_w;
      o->state_names        = {"m", "v", "beta12t", nullptr};
      break;
    case WHOLEGRAPH_OPT_ADAGRAD:
      o->name               = "AdaGrad";
      o->setters["epsilon"] = &o->epsilon;
      o->state_names        = {"state_sum", nullptr};
      break;
    case WHOLEGRAPH_OPT_RMSPROP:
      o->name               = "RMSProp";
      o->setters["epsilon"] = &o->epsilon;
      o->setters["alpha"]   = &o->alpha;
      o->state_names        = {"v", nullptr};
      break;
    default: return WHOLEGRAPH_NOT_IMPLEMENTED;
  }
  *optimizer = o.release();
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_optimizer_set_parameter(
  wholegraph_embedding_optimizer_t optimizer, const char* parameter_name, void* value)
{
  if (optimizer == nullptr || parameter_name == nullptr || value == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  auto it = optimizer->setters.find(parameter_name);
  if (it == optimizer->setters.end()) {
    WGB_ERROR("parameter name %s is not valid for optimizer %s", parameter_name, optimizer->name);
    return WHOLEGRAPH_INVALID_INPUT;
  }
  *it->second = *static_cast<const float*>(value);
  return WHOLEGRAPH_SUCCESS;
}

void wholegraph_destroy_embedding_optimizer(wholegraph_embedding_optimizer_t optimizer)
{
  delete optimizer;
}

wholegraph_error_code_t wholegraph_create_embedding_cache_policy(
  wholegraph_embedding_cache_policy_t* cache_policy,
  wholegraph_comm_t cache_level_comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location,
  wholegraph_access_type_t access_type,
  float cache_ratio)
{
  if (cache_policy == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (cache_ratio > 1.0f || cache_ratio < 1.0f / 512) {
    WGB_ERROR("cache_ratio should be in [1/512, 1]");
    return WHOLEGRAPH_INVALID_VALUE;
  }
  *cache_policy = new wholegraph_embedding_cache_policy_{cache_level_comm, memory_type, memory_location,
                                                         access_type, cache_ratio};
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_destroy_embedding_cache_policy(
  wholegraph_embedding_cache_policy_t cache_policy)
{
  delete cache_policy;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_create_embedding(
  wholegraph_embedding_t* wholegraph_embedding,
  wholegraph_tensor_description_t* embedding_description,
  wholegraph_comm_t comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location,
  wholegraph_embedding_cache_policy_t cache_policy,
  size_t* embedding_entry_partition,
  int user_defined_sms,
  int round_robin_size)
{
  if (wholegraph_embedding == nullptr || embedding_description == nullptr || comm == nullptr)
    return WHOLEGRAPH_INVALID_INPUT;
  wholegraph_matrix_description_t md;
  if (!wholegraph_convert_tensor_desc_to_matrix(&md, embedding_description)) {
    WGB_ERROR("wholegraph_create_embedding: the description must be a 2-D matrix");
    return WHOLEGRAPH_INVALID_INPUT;
  }
  if (cache_policy != nullptr && cache_policy->cache_comm == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (cache_policy != nullptr && cache_policy->cache_comm != comm) {
    // A cache on its own, smaller communicator: every such group of ranks caches the whole table
    // for itself, read-only (reference rules: embedding.cpp:972-987).
    if (cache_policy->cache_comm->world_size > comm->world_size) {
      WGB_ERROR("the cache communicator must not be larger than the embedding's");
      return WHOLEGRAPH_INVALID_INPUT;
    }
    if (cache_policy->memory_type != WHOLEGRAPH_MT_CONTINUOUS) {
      WGB_ERROR("For local cached global readonly embedding, cache_memory_type should be continuous.");
      return WHOLEGRAPH_INVALID_INPUT;
    }
    if (cache_policy->access_type != WHOLEGRAPH_AT_READONLY) {
      WGB_ERROR("Only ReadOnly access type supported for local cached global readonly embedding.");
      return WHOLEGRAPH_INVALID_INPUT;
    }
  }
  if (cache_policy != nullptr && cache_policy->memory_location != WHOLEGRAPH_ML_DEVICE) {
    WGB_ERROR("a cache must be in device memory");
    return WHOLEGRAPH_NOT_IMPLEMENTED;
  }
  WGB_API_BEGIN
  if (embedding_entry_partition != nullptr && round_robin_size != 0) {
    WGB_WARN("Parameter 'round_robin_size' is ignored.");
    round_robin_size = 0;
  }
  std::unique_ptr<wholegraph_embedding_> e(new wholegraph_embedding_());
  e->comm             = comm;
  e->dtype            = md.dtype;
  e->round_robin_size = round_robin_size;
  e->cache_policy     = cache_policy;
  e->gather_sms       = (user_defined_sms >= 1 && user_defined_sms <= 1568) ? user_defined_sms : -1;
  if (user_defined_sms != -1 && e->gather_sms == -1)
    WGB_WARN("user_defined_sms=%d is outside 1..1568 and is ignored", user_defined_sms);
  int64_t rows = md.sizes[0];
  if (round_robin_size != 0) {
    // Every rank stores the same number of rows (reference: embedding.cpp:459-476).
    const int W       = comm->world_size;
    int64_t extra     = rows % (static_cast<int64_t>(W) * round_robin_size);
    if (extra > round_robin_size) extra = round_robin_size;
    const int64_t per = rows / (static_cast<int64_t>(W) * round_robin_size) * round_robin_size + extra;
    rows              = per * W;
  }
  if (cache_policy != nullptr && embedding_entry_partition == nullptr) {
    // Shards of whole cache sets (reference: embedding.cpp:77-98 pads the same way).
    const int64_t unit = static_cast<int64_t>(comm->world_size) * coverage_of(cache_policy->cache_ratio);
    rows               = (rows + unit - 1) / unit * unit;
  }
  e->dim        = md.sizes[1];
  e->padded_dim = padded_dim_of(e->dim, wholegraph_dtype_get_element_size(md.dtype));
  wholegraph_tensor_description_t pd;
  wholegraph_initialize_tensor_desc(&pd);
  pd.dim        = 2;
  pd.dtype      = md.dtype;
  pd.sizes[0]   = rows;
  pd.sizes[1]   = e->padded_dim;
  pd.strides[0] = e->padded_dim;
  pd.strides[1] = 1;
  WHOLEGRAPH_RETURN_ON_FAIL(wholegraph_create_tensor(&e->allocated, &pd, comm, memory_type, memory_location,
                                                       embedding_entry_partition));
  int64_t starts[2] = {0, 0};
  int64_t ends[2]   = {rows, e->dim};
  auto rc           = wholegraph_tensor_get_subtensor(e->allocated, starts, ends, &e->user);
  if (rc == WHOLEGRAPH_SUCCESS && cache_policy != nullptr) rc = create_cache(e.get());
  if (rc != WHOLEGRAPH_SUCCESS) {
    if (e->user) wholegraph_destroy_tensor(e->user);
    wholegraph_destroy_tensor(e->allocated);
    return rc;
  }
  *wholegraph_embedding = e.release();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_create_embedding")
}

wholegraph_error_code_t wholegraph_destroy_embedding(wholegraph_embedding_t e)
{
  if (e == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  destroy_states(e);
  e->cache.reset();
  if (e->user) wholegraph_destroy_tensor(e->user);
  if (e->allocated) wholegraph_destroy_tensor(e->allocated);
  delete e;
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_destroy_embedding")
}

wholegraph_tensor_t wholegraph_embedding_get_embedding_tensor(wholegraph_embedding_t e)
{
  return e == nullptr ? nullptr : e->user;
}

wholegraph_error_code_t wholegraph_embedding_set_optimizer(wholegraph_embedding_t e,
                                                             wholegraph_embedding_optimizer_t optimizer)
{
  if (e == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (e->optimizer != nullptr) {
    WGB_ERROR("optimizer can only be set once.");
    return WHOLEGRAPH_NOT_SUPPORTED;
  }
  if (optimizer == nullptr) return WHOLEGRAPH_SUCCESS;
  if (e->cache && e->cache->node_level) {
    WGB_ERROR("an embedding behind a read-only cache cannot be trained");
    return WHOLEGRAPH_NOT_SUPPORTED;
  }
  if (e->dtype != WHOLEGRAPH_DT_FLOAT && e->dtype != WHOLEGRAPH_DT_HALF && e->dtype != WHOLEGRAPH_DT_BF16) {
    WGB_ERROR("Only float, half and bf16 embeddings support training.");
    return WHOLEGRAPH_NOT_IMPLEMENTED;
  }
  WGB_API_BEGIN
  e->optimizer = optimizer;
  auto rc      = create_states(e);
  if (rc != WHOLEGRAPH_SUCCESS) {
    destroy_states(e);
    e->optimizer = nullptr;
  }
  return rc;
  WGB_API_END("wholegraph_embedding_set_optimizer")
}

wholegraph_error_code_t wholegraph_embedding_gather(wholegraph_embedding_t e,
                                                      wholegraph_tensor_t indices,
                                                      wholegraph_tensor_t output,
                                                      bool adjust_cache,
                                                      wholegraph_env_func_t* p_env_fns,
                                                      int64_t stream_int)
{
  if (e == nullptr || indices == nullptr || output == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = reinterpret_cast<cudaStream_t>(stream_int);
  return with_mapped_indices(e, indices, p_env_fns, stream, [&](wholegraph_tensor_t ids) {
    if (e->cache) {
      cached_gather(e, ids, output, adjust_cache, p_env_fns, stream);
      return WHOLEGRAPH_SUCCESS;
    }
    return wholegraph_gather(e->user, ids, output, p_env_fns, stream, e->gather_sms);
  });
  WGB_API_END("wholegraph_embedding_gather")
}

wholegraph_error_code_t wholegraph_embedding_gather_gradient_apply(wholegraph_embedding_t e,
                                                                     wholegraph_tensor_t indices,
                                                                     wholegraph_tensor_t grads,
                                                                     bool adjust_cache,
                                                                     float lr,
                                                                     wholegraph_env_func_t* p_env_fns,
                                                                     int64_t stream_int)
{
  if (e == nullptr || indices == nullptr || grads == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = reinterpret_cast<cudaStream_t>(stream_int);
  return with_mapped_indices(e, indices, p_env_fns, stream, [&](wholegraph_tensor_t ids) {
    gradient_apply(e, ids, grads, adjust_cache, lr, p_env_fns, stream);
    return WHOLEGRAPH_SUCCESS;
  });
  WGB_API_END("wholegraph_embedding_gather_gradient_apply")
}

const char* const* wholegraph_embedding_get_optimizer_state_names(wholegraph_embedding_t e)
{
  if (e == nullptr || e->optimizer == nullptr) return nullptr;
  return e->optimizer->state_names.data();
}

wholegraph_tensor_t wholegraph_embedding_get_optimizer_state(wholegraph_embedding_t e, const char* name)
{
  if (e == nullptr || name == nullptr || e->optimizer == nullptr) return nullptr;
  if (strcmp(name, "beta12t") == 0) return e->beta12t_view;
  auto it = e->state_views.find(name);
  return it == e->state_views.end() ? nullptr : it->second;
}

wholegraph_error_code_t wholegraph_b200_embedding_get_cache_tensors(wholegraph_embedding_t e,
                                                                      wholegraph_tensor_t* tags,
                                                                      wholegraph_tensor_t* lfu,
                                                                      wholegraph_tensor_t* lines,
                                                                      int* set_coverage)
{
  if (e == nullptr || !e->cache) return WHOLEGRAPH_INVALID_INPUT;
  if (tags) *tags = e->cache->tags;
  if (lfu) *lfu = e->cache->lfu;
  if (lines) *lines = e->cache->lines;
  if (set_coverage) *set_coverage = e->cache->coverage;
  return WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_b200_embedding_get_cache_counters(wholegraph_embedding_t e,
                                                                       int64_t** counters,
                                                                       int64_t* local_rows)
{
  if (e == nullptr || !e->cache || counters == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  *counters = e->cache->access_count;
  if (local_rows != nullptr) *local_rows = local_cache_of(e).rows;
  return WHOLEGRAPH_SUCCESS;
}

}  // extern "C"

namespace {
// Modified lines of the embedding and of its optimizer state go back to their tables; every rank
// waits until all have finished, so that the tables can be read or saved right after.
wholegraph_error_code_t flush_cache(wholegraph_embedding_t e, bool drop, int64_t stream_int)
{
  if (e == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (!e->cache) return WHOLEGRAPH_SUCCESS;  // nothing to write back
  WGB_API_BEGIN
  auto stream = reinterpret_cast<cudaStream_t>(stream_int);
  cache_writeback(local_cache_of(e), drop, stream);
  if (e->state_embedding != nullptr && e->state_embedding->cache)
    cache_writeback(local_cache_of(e->state_embedding), drop, stream);
  WGB_CUDA_CHECK(cudaStreamSynchronize(stream));
  e->comm->barrier();
  return WHOLEGRAPH_SUCCESS;
  WGB_API_END("wholegraph_embedding_writeback_cache")
}
}  // namespace

extern "C" {

wholegraph_error_code_t wholegraph_embedding_writeback_cache(wholegraph_embedding_t e, int64_t stream_int)
{
  return flush_cache(e, false, stream_int);
}

wholegraph_error_code_t wholegraph_embedding_drop_all_cache(wholegraph_embedding_t e, int64_t stream_int)
{
  return flush_cache(e, true, stream_int);
}

}  // extern "C"
