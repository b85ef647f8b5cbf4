#include "env.hpp"

#include <algorithm>

#include <wholegraph/wholegraph_b200.h>

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

#include "common.hpp"
#include <wholegraph/wholegraph_b200.h>

namespace wgb {

temp_buffer::temp_buffer(wholegraph_env_func_t* env) : env_(env)
{
  WGB_EXPECTS(env != nullptr && env->temporary_fns.create_memory_context_fn != nullptr &&
                env->temporary_fns.malloc_fn != nullptr,
              "environment functions are missing");
  env_->temporary_fns.create_memory_context_fn(&ctx_, env_->temporary_fns.global_context);
}

void* temp_buffer::get(size_t count, wholegraph_dtype_t dt,
                       wholegraph_memory_allocation_type_t where)
{
  release();
  wholegraph_tensor_description_t d;
  wholegraph_initialize_tensor_desc(&d);
  d.dim      = 1;
  d.dtype    = dt;
  d.sizes[0] = static_cast<int64_t>(count > 0 ? count : 1);
  ptr_       = env_->temporary_fns.malloc_fn(&d, where, ctx_, env_->temporary_fns.global_context);
  if (ptr_ == nullptr) throw std::bad_alloc();
  return ptr_;
}

void temp_buffer::release()
{
  if (ptr_ != nullptr && env_->temporary_fns.free_fn != nullptr) {
    env_->temporary_fns.free_fn(ctx_, env_->temporary_fns.global_context);
  }
  ptr_ = nullptr;
}

temp_buffer::~temp_buffer()
{
  release();
  if (env_->temporary_fns.destroy_memory_context_fn != nullptr)
    env_->temporary_fns.destroy_memory_context_fn(ctx_, env_->temporary_fns.global_context);
}

namespace {

// ---- plain allocator: every request is a cudaMalloc / malloc / cudaMallocHost -----------
struct plain_ctx {
  void* ptr                                 = nullptr;
  wholegraph_memory_allocation_type_t where = WHOLEGRAPH_MA_NONE;
};

void raw_free(void* p, wholegraph_memory_allocation_type_t where)
{
  if (p == nullptr) return;
  if (where == WHOLEGRAPH_MA_DEVICE)
    cudaFree(p);
  else if (where == WHOLEGRAPH_MA_PINNED)
    cudaFreeHost(p);
  else
    free(p);
}

void* raw_alloc(size_t bytes, wholegraph_memory_allocation_type_t where)
{
  void* p = nullptr;
  if (bytes == 0) bytes = 1;
  if (where == WHOLEGRAPH_MA_DEVICE) {
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
  } else if (where == WHOLEGRAPH_MA_PINNED) {
    if (cudaMallocHost(&p, bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
  } else {
    p = malloc(bytes);
  }
  return p;
}

void plain_create(void** ctx, void*) { *ctx = new plain_ctx(); }
void plain_free(void* ctx, void*)
{
  auto* c = static_cast<plain_ctx*>(ctx);
  // A buffer may still be in use by work queued on a stream: wait before releasing it.
  if (c->ptr != nullptr && c->where != WHOLEGRAPH_MA_HOST) cudaDeviceSynchronize();
  raw_free(c->ptr, c->where);
  c->ptr = nullptr;
}
void plain_destroy(void* ctx, void* g)
{
  plain_free(ctx, g);
  delete static_cast<plain_ctx*>(ctx);
}
void* plain_malloc(wholegraph_tensor_description_t* d, wholegraph_memory_allocation_type_t where,
                   void* ctx, void* g)
{
  auto* c = static_cast<plain_ctx*>(ctx);
  plain_free(ctx, g);
  size_t bytes = static_cast<size_t>(wholegraph_get_memory_size_from_tensor(d));
  c->ptr       = raw_alloc(bytes, where);
  c->where     = where;
  return c->ptr;
}

// ---- caching allocator: freed blocks are kept per (kind, device, power-of-two size) and reused.
// Reuse is safe without a synchronize because a block goes back to the pool only when the op
// that used it has finished enqueueing, and every consumer of the pool enqueues on the stream
// it was given; callers that mix streams must order them themselves.  Device blocks are only
// handed back on the device they were allocated on.
struct cache_pool {
  std::mutex mu;
  std::multimap<std::pair<int, size_t>, void*> free_blocks;
  std::vector<std::pair<void*, int>> all_blocks;
  ~cache_pool() { drop(); }
  void drop()
  {
    std::lock_guard<std::mutex> lk(mu);
    for (auto& b : all_blocks) raw_free(b.first, static_cast<wholegraph_memory_allocation_type_t>(b.second));
    all_blocks.clear();
    free_blocks.clear();
  }
};
struct cached_ctx {
  void* ptr   = nullptr;
  int where   = 0;  // pool key: allocation kind and, for device memory, the device ordinal
  size_t size = 0;
};

int pool_kind(wholegraph_memory_allocation_type_t where)
{
  int dev = 0;
  if (where == WHOLEGRAPH_MA_DEVICE) cudaGetDevice(&dev);
  return static_cast<int>(where) * 1024 + dev;
}

size_t size_class(size_t bytes)
{
  size_t s = 512;
  while (s < bytes) s <<= 1;
  return s;
}

void cached_create(void** ctx, void*) { *ctx = new cached_ctx(); }
void cached_free(void* ctx, void* g)
{
  auto* c    = static_cast<cached_ctx*>(ctx);
  auto* pool = static_cast<cache_pool*>(g);
  if (c->ptr == nullptr) return;
  std::lock_guard<std::mutex> lk(pool->mu);
  pool->free_blocks.insert({{c->where, c->size}, c->ptr});
  c->ptr = nullptr;
}
void cached_destroy(void* ctx, void* g)
{
  cached_free(ctx, g);
  delete static_cast<cached_ctx*>(ctx);
}
void* cached_malloc(wholegraph_tensor_description_t* d, wholegraph_memory_allocation_type_t where,
                    void* ctx, void* g)
{
  auto* c    = static_cast<cached_ctx*>(ctx);
  auto* pool = static_cast<cache_pool*>(g);
  cached_free(ctx, g);
  size_t cls = size_class(static_cast<size_t>(wholegraph_get_memory_size_from_tensor(d)));
  {
    std::lock_guard<std::mutex> lk(pool->mu);
    auto it = pool->free_blocks.find({pool_kind(where), cls});
    if (it != pool->free_blocks.end()) {
      c->ptr = it->second;
      pool->free_blocks.erase(it);
    }
  }
  if (c->ptr == nullptr) {
    c->ptr = raw_alloc(cls, where);
    if (c->ptr == nullptr) return nullptr;
    std::lock_guard<std::mutex> lk(pool->mu);
    pool->all_blocks.push_back({c->ptr, static_cast<int>(where)});
  }
  c->where = pool_kind(where);
  c->size  = cls;
  return c->ptr;
}

cache_pool& the_pool()
{
  static cache_pool* p = new cache_pool();  // leaked on purpose: outlives CUDA teardown order
  return *p;
}

// Output memory: the "memory context" is a caller-owned wholegraph_b200_output_slot_t that
// receives the pointer and the description of what was allocated.
void* output_malloc(wholegraph_tensor_description_t* d, wholegraph_memory_allocation_type_t where,
                    void* ctx, void*)
{
  const size_t bytes = static_cast<size_t>(wholegraph_get_memory_size_from_tensor(d));
  void* p            = raw_alloc(std::max<size_t>(bytes, 16), where);
  if (ctx != nullptr) {
    auto* slot        = static_cast<wholegraph_b200_output_slot_t*>(ctx);
    slot->pointer     = p;
    slot->description = *d;
  }
  return p;
}
void output_free(void* ctx, void*)
{
  (void)ctx;  // the caller owns output buffers and releases them itself
}

}  // namespace
}  // namespace wgb

extern "C" {

wholegraph_env_func_t* wholegraph_b200_get_default_env_func()
{
  static wholegraph_env_func_t env = {
    {wgb::plain_create, wgb::plain_destroy, wgb::plain_malloc, wgb::plain_free, nullptr},
    {wgb::output_malloc, wgb::output_free, nullptr}};
  return &env;
}

wholegraph_env_func_t* wholegraph_b200_get_cached_env_func()
{
  static wholegraph_env_func_t env = {
    {wgb::cached_create, wgb::cached_destroy, wgb::cached_malloc, wgb::cached_free, &wgb::the_pool()},
    {wgb::output_malloc, wgb::output_free, nullptr}};
  return &env;
}

wholegraph_error_code_t wholegraph_b200_release_output(wholegraph_b200_output_slot_t* slot)
{
  if (slot == nullptr) return WHOLEGRAPH_INVALID_INPUT;
  if (slot->pointer != nullptr) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, slot->pointer) != cudaSuccess) {
      (void)cudaGetLastError();
      return WHOLEGRAPH_CUDA_ERROR;
    }
    cudaError_t e = cudaSuccess;
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged)
      e = cudaFree(slot->pointer);
    else if (attr.type == cudaMemoryTypeHost)
      e = cudaFreeHost(slot->pointer);
    else
      free(slot->pointer);  // pageable host memory of WHOLEGRAPH_MA_HOST
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return WHOLEGRAPH_CUDA_ERROR;
    }
  }
  slot->pointer = nullptr;
  return WHOLEGRAPH_SUCCESS;
}

void wholegraph_b200_drop_cached_env_func_memory()
{
  cudaDeviceSynchronize();
  wgb::the_pool().drop();
}

cudaDeviceProp* get_device_prop(int dev_id)
{
  static std::mutex mu;
  static std::map<int, cudaDeviceProp> props;
  std::lock_guard<std::mutex> lk(mu);
  if (dev_id < 0 && cudaGetDevice(&dev_id) != cudaSuccess) return nullptr;
  auto it = props.find(dev_id);
  if (it == props.end()) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev_id) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    it = props.emplace(dev_id, p).first;
  }
  return &it->second;
}

}  // extern "C"
