/*
 * wholegraph-b200: entry points that exist only in this library (no counterpart in the
 * reference's public headers).  They cover what the reference keeps in internal C++ symbols
 * (wholegraph::get_default_env_func / get_cached_env_func, cpp/src/wholegraph/env_func_ptrs.hpp)
 * so that C and ctypes callers can reach them, plus run-time introspection for benchmarks.
 */
#pragma once

#include <stdint.h>

#include <wholegraph/embedding.h>
#include <wholegraph/env_func_ptrs.h>
#include <wholegraph/tensor_description.h>
#include <wholegraph/wholegraph.h>
#include <wholegraph/wholegraph_tensor.h>

/*
 * Duplicate-gradient reduction of wholegraph_embedding_gather_gradient_apply: gradients of equal
 * ids are added one after the other in arrival order, as in the reference, as long as an id
 * occurs at most this many times in one call.  Longer runs are cut into blocks of this many
 * rows; each block is summed in order and the block sums are added in block order.
 */
#define WHOLEGRAPH_B200_DEDUP_BLOCK 256

#ifdef __cplusplus
extern "C" {
#endif

/* Allocator callbacks backed by cudaMalloc / cudaMallocHost / malloc; every free waits for the device. */
wholegraph_env_func_t* wholegraph_b200_get_default_env_func();

/*
 * Allocator callbacks with a size-class free list: a buffer released by one op is handed to
 * the next one without touching the CUDA allocator and without an event in between.  The
 * contract: ops that draw from it are ordered on the streams they are given (one stream, or
 * streams the caller orders itself); an op on stream B that starts while an op on stream A still
 * runs may be handed A's buffer.  Device buffers are pooled per device and only handed back on the
 * device that allocated them (the current device of the calling thread at the time of the call).
 */
wholegraph_env_func_t* wholegraph_b200_get_cached_env_func();

/* Return every block of the caching allocator to CUDA (synchronizes the device first). */
void wholegraph_b200_drop_cached_env_func_memory();

/*
 * cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream) for callers that hold raw
 * pointers (a shard of a handle, a ctypes buffer) but no CUDA runtime binding of their own.
 */
wholegraph_error_code_t wholegraph_b200_memcpy_async(void* dst, const void* src, size_t bytes,
                                                       void* stream);

/*
 * Stable partition of a request list by owning rank, the first step of every DISTRIBUTED op
 * (role of the reference's internal bucket_and_exchange_ids_func,
 * cpp/src/wholegraph_tensor_ops/functions/exchange_ids_nccl_func.cu:146-215, which has no C entry
 * point of its own).
 *   ids            n row ids, int32 (ids_are_64 = 0) or int64, device memory
 *   first_row      HOST array of world + 1 first rows per rank; first_row[world] = table rows
 *   workspace      device scratch of at least wholegraph_b200_partition_workspace_bytes(n, world)
 *   sorted_ids     out, n int64 (device): ids grouped by owner, list order kept inside a group
 *   positions      out, n int64 (device): list position each sorted id came from
 *   counts, starts out, world int64 each (device): size and first slot of every group
 * Ids that are negative or >= first_row[world] belong to no group and are dropped; the groups
 * are packed at the front of the outputs.  n < 2^31, world <= 64.  Asynchronous on `stream`.
 */
size_t wholegraph_b200_partition_workspace_bytes(int64_t n, int world);
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
                                                             void* stream);

/*
 * wholegraph_b200_partition_by_owner without any allocation, by this call or asked of the
 * caller.  It has no counterpart in the reference.
 *
 * Who needs it: callers that must not reach the CUDA allocator while they run - a serving
 * loop whose device memory is already handed out in full to its own pool, or a step that
 * cannot afford the device-wide stall a cudaMalloc / cudaFree brings - and that therefore have
 * no workspace to pass either.  The caller still owns ids and all four outputs; only the
 * scratch moves into the library: a fixed 66,048-byte (64.5 KiB) array in device memory, held
 * by every GPU that loads the library until the process exits.
 *
 * Limit: wholegraph_b200_partition_workspace_bytes(n, world) must not exceed 66,048, i.e.
 * ceil(n / 2048) * world <= 16,508 (4,194,304 ids at 8 ranks, 33 million ids at 1 rank).
 * Larger requests return WHOLEGRAPH_INVALID_VALUE and launch nothing.
 *
 * The first call on a device looks up the array's device address (a one-time set-up inside
 * the CUDA runtime); make that call before starting any stream capture.  All calls on a GPU
 * share the one array, which keeps whatever the previous call left in it: nothing needs
 * clearing, because each call writes every word before reading it, but two calls that overlap
 * on the GPU (different streams, no ordering) race on it and corrupt each other's result.
 * Outputs, argument meaning and asynchrony are those of wholegraph_b200_partition_by_owner.
 */
wholegraph_error_code_t wholegraph_b200_partition_by_owner_no_alloc(const void* ids,
                                                                      int ids_are_64,
                                                                      int64_t n,
                                                                      const int64_t* first_row,
                                                                      int world,
                                                                      int64_t* sorted_ids,
                                                                      int64_t* positions,
                                                                      int64_t* counts,
                                                                      int64_t* starts,
                                                                      void* stream);

/*
 * De-duplication of a gather's request list, the first step of a DISTRIBUTED gather here (the
 * reference sorts the whole list and keeps duplicates on the wire,
 * cpp/src/wholegraph_tensor_ops/functions/exchange_ids_nccl_func.cu:32-104; no C entry point of its
 * own there).
 *   ids            n row ids, int32 (ids_are_64 = 0) or int64, device memory
 *   first_row      HOST array of world + 1 first rows per rank; first_row[0] = 0, not decreasing
 *   workspace      device scratch of at least wholegraph_b200_unique_workspace_bytes(n, first_row[world])
 *   unique_ids     out, n int64 (device): the distinct valid ids, ascending, hence grouped by owner;
 *                  the first sum(counts) entries are written
 *   inverse        out, n int64 (device): slot in unique_ids of every list position, -1 for ids
 *                  that are negative or >= first_row[world]
 *   counts, starts out, world int64 each (device): distinct ids owned by each rank, first slot of its group
 * n < 2^31 and first_row[world] < 2^32 - 1 (32-bit sort keys), world <= 64; otherwise
 * WHOLEGRAPH_INVALID_VALUE.  Asynchronous on `stream`.
 */
size_t wholegraph_b200_unique_workspace_bytes(int64_t n, int64_t total_rows);
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
                                                          void* stream);

/*
 * The same de-duplication without the promise of ascending ids: the distinct ids of an owner's group come
 * in whatever order a hash table's insertion races give (it may differ from call to call); counts, starts
 * and the meaning of `inverse` are unchanged.  Several times cheaper than the sorted form and what the
 * distributed gather uses, since only `inverse` ties list positions to slots.  Lists longer than 2^27 ids
 * fall back to the sorted form.
 */
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
                                                                    void* stream);

/*
 * Number of chunks a pipelined NCCL row exchange runs in (no counterpart in the reference, whose
 * exchange is one alltoallv, exchange_embeddings_nccl_func.cu:23-64).  Every chunk is a matched set
 * of sends and receives, so all ranks must arrive at the same number: it is a function of the
 * world x world count matrix only (matrix[q * world + r] = rows rank q routes to rank r, HOST
 * memory), which every rank holds after the counts exchange.  forced > 0 wins, then wanted > 0
 * (both capped at 16); otherwise 4 when the busiest rank sends or receives 16 MiB or more, else 1.
 */
int wholegraph_b200_exchange_chunk_count(const int64_t* matrix, int world, size_t row_bytes, int wanted,
                                         int forced);

/*
 * Read the WG_* tuning variables of the distributed ops again (WG_PEER_EXCHANGE, WG_GATHER_DEDUP,
 * WG_GRADIENT_PRESUM, WG_PEER_GRADIENT, WG_EXCHANGE_CHUNKS, WG_SYNC_FREE, WG_SERVE_BULK).  They are read when a
 * communicator is created; a process that changes them afterwards calls this on every rank
 * (collective, blocking).  WHOLEGRAPH_LOGIC_ERROR when the ranks do not agree, the check the
 * reference applies to the parameters of its collective calls
 * (cpp/src/wholegraph/communicator.hpp:220-249).
 */
wholegraph_error_code_t wholegraph_b200_reload_tuning(wholegraph_comm_t comm);

/*
 * wholegraph_gather on a memory handle and raw device pointers instead of tensors: the form in which the
 * reference's NCCL-mode neighbour sampling calls the distributed gather on the CSR row-pointer and column
 * handles of a graph (wholegraph_gather_nccl, cpp/src/wholegraph_tensor_ops/gather_op_impl.h:24-32, called
 * from cpp/src/wholegraph_ops/unweighted_sample_without_replacement_nccl_func.cuh:236 and :364; an internal
 * C++ symbol there).  Works on CONTINUOUS, CHUNKED and DISTRIBUTED handles.
 *   table_desc    rows x columns view of the handle's memory (stride and storage offset in elements)
 *   indices       int32 / int64 row ids, device memory; indices_desc->storage_offset elements are skipped
 *   output        first element of the output storage; output_desc gives rows (= number of indices),
 *                 columns (= the table's), row stride and storage offset
 * Same checks, casts and skipped negative ids as wholegraph_gather.  Collective for a DISTRIBUTED handle.
 */
wholegraph_error_code_t wholegraph_b200_gather_from_handle(wholegraph_handle_t handle,
                                                             const wholegraph_matrix_description_t* table_desc,
                                                             const void* indices,
                                                             const wholegraph_array_description_t* indices_desc,
                                                             void* output,
                                                             const wholegraph_matrix_description_t* output_desc,
                                                             wholegraph_env_func_t* p_env_fns,
                                                             void* stream,
                                                             int gather_sms);

/* The arrays of a cached embedding, for inspection and tests (no counterpart in the reference's
 * C API; its cache object keeps them private, cpp/src/wholegraph/embedding_cache.hpp:64-74):
 * tags and LFU words as int16 [sets, 32] tensors, the cache lines as a [sets * 32, padded dim]
 * tensor of the table's dtype, and the number of consecutive table rows one set covers.  A tag is
 * valid (bit 14) | modified (bit 15) | row number inside the set (bits 0-13).  The tensors belong
 * to the embedding.  WHOLEGRAPH_INVALID_INPUT for an embedding without a cache. */
wholegraph_error_code_t wholegraph_b200_embedding_get_cache_tensors(wholegraph_embedding_t embedding,
                                                                      wholegraph_tensor_t* tags,
                                                                      wholegraph_tensor_t* lfu,
                                                                      wholegraph_tensor_t* lines,
                                                                      int* set_coverage);

/* This rank's exact access counters of a cached embedding: one int64 per local row (device memory owned by
 * the embedding), in local row order.  The replacement rule ranks the rows of a set by these counters; the
 * reference keeps approximate scaled counters for cached lines instead and exact ones only for the rest
 * (cpp/src/wholegraph_tensor_ops/functions/embedding_cache_func.cuh:132-141), and exposes neither.  For
 * inspection and tests.  WHOLEGRAPH_INVALID_INPUT for an embedding without a cache. */
wholegraph_error_code_t wholegraph_b200_embedding_get_cache_counters(wholegraph_embedding_t embedding,
                                                                       int64_t** counters,
                                                                       int64_t* local_rows);

/* Memory context for the output allocator of the two built-in env functions above: an op that
 * produces an output of a size only it knows (graph_append_unique) calls
 * env->output_fns.malloc_fn with the caller's context pointer, and these allocators fill the slot
 * with the device pointer and the description (dtype, length) of what they allocated.  The caller
 * owns the buffer and releases it with wholegraph_b200_release_output.  Callers with their own allocator pass whatever
 * context their own malloc_fn expects, as with the reference. */
typedef struct wholegraph_b200_output_slot_t {
  void* pointer;
  wholegraph_tensor_description_t description;
} wholegraph_b200_output_slot_t;

/* Release the buffer of a slot filled by the built-in output allocator (cudaFree, cudaFreeHost or free,
 * by where it was allocated) and clear the slot.  Other kinds of context must not be passed. */
wholegraph_error_code_t wholegraph_b200_release_output(wholegraph_b200_output_slot_t* slot);

/* Number of kernels this library has launched in this process since load. */
unsigned long long wholegraph_b200_kernel_launch_count();

/* Library identification string, e.g. "wholegraph-b200 sm_100a". */
const char* wholegraph_b200_version();

#ifdef __cplusplus
}
#endif
