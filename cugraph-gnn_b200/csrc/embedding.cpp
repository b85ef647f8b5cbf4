// Embedding objects: padded table + user view, optimizer and its state tensors, forward
// gather and the backward gather_gradient_apply step.
//
// Reference behaviour: cpp/src/wholegraph/embedding.cpp (allocate :77-134, gradient apply
// :136-314, state creation :316-420, C API :886-1110) and embedding_optimizer.cpp (parameter
// names and defaults :159-180, :286-297, :385-400; state names and initial values :179-211).
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <wholegraph/embedding.h>
#include <wholegraph/wholegraph_tensor_op.h>

#include "common.hpp"
#include "env.hpp"
#include "handle.hpp"
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

struct wholegraph_embedding_ {
  wholegraph_comm_t comm            = nullptr;
  wholegraph_dtype_t dtype          = WHOLEGRAPH_DT_UNKNOWN;
  wholegraph_tensor_t allocated     = nullptr;  // [rows, padded dim], owns the handle
  wholegraph_tensor_t user          = nullptr;  // [rows, dim] view
  wholegraph_embedding_cache_policy_t cache_policy = nullptr;
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
                                                            h->location, nullptr, partition.data()));
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

// Backward step on already-mapped ids.
void gradient_apply(wholegraph_embedding_* e, wholegraph_tensor_t indices, wholegraph_tensor_t grads,
                    float lr, wholegraph_env_func_t* env, cudaStream_t stream)
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

  temp_buffer ws(env);
  if (W == 1) {
    if (n == 0) return;
    a.ids = ids, a.ids_are_64 = ids_are_64, a.count = n;
    a.grads = g, a.grad_stride = gd->strides[0];
    sparse_apply(a, ws.device_bytes(sparse_apply_workspace_bytes(n, wl.rows, e->dim)), stream);
    return;
  }

  // Route every gradient row to the owner of its id: same W-step pipeline as a distributed
  // scatter, with fp32 rows on the wire.
  wholegraph_handle_* h = wholegraph_tensor_get_memory_handle(e->allocated);
  auto first_row        = entry_offsets_of(h, wholegraph_dtype_get_element_size(e->dtype) * e->padded_dim);
  exchange_plan plan(env);
  plan.build(ids, ids_are_64, n, first_row, comm, stream);
  const size_t row_b = static_cast<size_t>(e->dim) * sizeof(float);
  temp_buffer send_buf(env), recv_buf(env);
  char* send = static_cast<char*>(send_buf.device_bytes(std::max<size_t>(1, plan.total_send * row_b)));
  char* recv = static_cast<char*>(recv_buf.device_bytes(std::max<size_t>(1, plan.total_recv * row_b)));
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
    [](const list_segments&) {});  // the update below needs every row: nothing to do per chunk
  if (plan.total_recv == 0) return;
  a.ids = plan.recv_ids, a.ids_are_64 = true, a.count = plan.total_recv;
  a.grads = reinterpret_cast<const float*>(recv), a.grad_stride = e->dim;
  sparse_apply(a, ws.device_bytes(sparse_apply_workspace_bytes(plan.total_recv, wl.rows, e->dim)), stream);
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
  if (cache_policy != nullptr) {
    WGB_ERROR("cached embeddings are not available in this build");
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
  if (rc != WHOLEGRAPH_SUCCESS) {
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
  (void)adjust_cache;
  if (e == nullptr || indices == nullptr || output == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = reinterpret_cast<cudaStream_t>(stream_int);
  return with_mapped_indices(e, indices, p_env_fns, stream, [&](wholegraph_tensor_t ids) {
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
  (void)adjust_cache;
  if (e == nullptr || indices == nullptr || grads == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  WGB_API_BEGIN
  auto stream = reinterpret_cast<cudaStream_t>(stream_int);
  return with_mapped_indices(e, indices, p_env_fns, stream, [&](wholegraph_tensor_t ids) {
    gradient_apply(e, ids, grads, lr, p_env_fns, stream);
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

wholegraph_error_code_t wholegraph_embedding_writeback_cache(wholegraph_embedding_t e, int64_t)
{
  // Without a cache there is nothing to write back.
  return e == nullptr ? WHOLEGRAPH_INVALID_INPUT : WHOLEGRAPH_SUCCESS;
}

wholegraph_error_code_t wholegraph_embedding_drop_all_cache(wholegraph_embedding_t e, int64_t)
{
  return e == nullptr ? WHOLEGRAPH_INVALID_INPUT : WHOLEGRAPH_SUCCESS;
}

}  // extern "C"
