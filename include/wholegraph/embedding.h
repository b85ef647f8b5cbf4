/*
 * wholegraph-b200: embedding tables with optional cache and sparse optimizer.
 *
 * ABI mirror of the reference's cpp/include/wholegraph/embedding.h:20-233.
 */
#pragma once

#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/wholegraph_tensor.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct wholegraph_embedding_cache_policy_* wholegraph_embedding_cache_policy_t;
typedef struct wholegraph_embedding_optimizer_* wholegraph_embedding_optimizer_t;
typedef struct wholegraph_embedding_* wholegraph_embedding_t;

enum wholegraph_access_type_t {
  WHOLEGRAPH_AT_NONE = 0,
  WHOLEGRAPH_AT_READONLY,
  WHOLEGRAPH_AT_READWRITE,
};

enum wholegraph_optimizer_type_t {
  WHOLEGRAPH_OPT_NONE = 0,
  WHOLEGRAPH_OPT_SGD,
  WHOLEGRAPH_OPT_LAZY_ADAM,
  WHOLEGRAPH_OPT_RMSPROP,
  WHOLEGRAPH_OPT_ADAGRAD,
};

wholegraph_error_code_t wholegraph_create_embedding_optimizer(
  wholegraph_embedding_optimizer_t* optimizer, wholegraph_optimizer_type_t optimizer_type);

/*
 * Set one float hyper-parameter by name (`value` points to a float). Names and defaults
 * (cpp/src/wholegraph/embedding_optimizer.cpp:159-180, :286-297, :385-400):
 *   SGD       weight_decay=0
 *   LazyAdam  weight_decay=0 epsilon=1e-8 beta1=0.9 beta2=0.999 adam_w=0 (>0.5: decoupled decay)
 *   AdaGrad   weight_decay=0 epsilon=1e-8
 *   RMSProp   weight_decay=0 epsilon=1e-8 alpha=0.99
 * An unknown name returns WHOLEGRAPH_INVALID_INPUT.
 */
wholegraph_error_code_t wholegraph_optimizer_set_parameter(
  wholegraph_embedding_optimizer_t optimizer, const char* parameter_name, void* value);

void wholegraph_destroy_embedding_optimizer(wholegraph_embedding_optimizer_t optimizer);

/*
 * Describe a set-associative row cache kept at `cache_level_comm`; `cache_ratio` in
 * [1/512, 1] is the cached fraction of the table.
 */
wholegraph_error_code_t wholegraph_create_embedding_cache_policy(
  wholegraph_embedding_cache_policy_t* cache_policy,
  wholegraph_comm_t cache_level_comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location,
  wholegraph_access_type_t access_type,
  float cache_ratio);

wholegraph_error_code_t wholegraph_destroy_embedding_cache_policy(
  wholegraph_embedding_cache_policy_t cache_policy);

/*
 * Collective. Create a [rows, dim] table (only sizes and dtype of the description are
 * used); the row stride is padded to 16 bytes and the user-visible tensor is a sub-view.
 * `user_defined_sms` in 1..1568 is passed on as the CTA hint of gather / scatter.
 */
wholegraph_error_code_t wholegraph_create_embedding(
  wholegraph_embedding_t* wholegraph_embedding,
  wholegraph_tensor_description_t* embedding_tensor_description,
  wholegraph_comm_t comm,
  wholegraph_memory_type_t memory_type,
  wholegraph_memory_location_t memory_location,
  wholegraph_embedding_cache_policy_t cache_policy,
  size_t* embedding_entry_partition = nullptr,
  int user_defined_sms              = -1,
  int round_robin_size              = 0);

wholegraph_error_code_t wholegraph_destroy_embedding(
  wholegraph_embedding_t wholegraph_embedding);

wholegraph_tensor_t wholegraph_embedding_get_embedding_tensor(
  wholegraph_embedding_t wholegraph_embedding);

/* Collective; allocates and initialises the optimizer states. Allowed once per embedding. */
wholegraph_error_code_t wholegraph_embedding_set_optimizer(
  wholegraph_embedding_t wholegraph_embedding, wholegraph_embedding_optimizer_t optimizer);

/* Forward lookup; `stream_int` is a cudaStream_t passed as an integer. */
wholegraph_error_code_t wholegraph_embedding_gather(wholegraph_embedding_t wholegraph_embedding,
                                                      wholegraph_tensor_t indices,
                                                      wholegraph_tensor_t output,
                                                      bool adjust_cache,
                                                      wholegraph_env_func_t* p_env_fns,
                                                      int64_t stream_int);

/*
 * Collective backward step: route the fp32 gradient rows `grads` [n, dim] of `indices` [n]
 * to the owners of the rows, sum the gradients of equal indices and apply the attached
 * optimizer with learning rate `lr` to weights and states. Replaces
 * embedding_base::gather_gradient_apply (cpp/src/wholegraph/embedding.cpp:136-314).
 */
wholegraph_error_code_t wholegraph_embedding_gather_gradient_apply(
  wholegraph_embedding_t wholegraph_embedding,
  wholegraph_tensor_t indices,
  wholegraph_tensor_t grads,
  bool adjust_cache,
  float lr,
  wholegraph_env_func_t* p_env_fns,
  int64_t stream_int);

/* NULL-terminated list owned by the optimizer: {"m","v","beta12t"}, {"state_sum"}, {"v"} or {}. */
const char* const* wholegraph_embedding_get_optimizer_state_names(
  wholegraph_embedding_t wholegraph_embedding);

/* State tensor by name, NULL if there is none. */
wholegraph_tensor_t wholegraph_embedding_get_optimizer_state(
  wholegraph_embedding_t wholegraph_embedding, const char* name);

wholegraph_error_code_t wholegraph_embedding_writeback_cache(
  wholegraph_embedding_t wholegraph_embedding, int64_t stream_int);

wholegraph_error_code_t wholegraph_embedding_drop_all_cache(
  wholegraph_embedding_t wholegraph_embedding, int64_t stream_int);

#ifdef __cplusplus
}
#endif
