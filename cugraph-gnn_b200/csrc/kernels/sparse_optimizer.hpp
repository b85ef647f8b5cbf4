// Host interface of the sparse optimizer: duplicate-gradient reduction fused with the update.
// Replaces the reference's dedup_indice_and_gradients
// (cpp/src/wholegraph_tensor_ops/functions/exchange_embeddings_nccl_func.cu:98-200) followed by
// the per-row optimizer kernels (embedding_optimizer_func.cu:168-1022).
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include <wholegraph/embedding.h>
#include <wholegraph/wholegraph_b200.h>
#include <wholegraph/tensor_description.h>

#include "cache.hpp"

namespace wgb {

struct optimizer_hyper {
  wholegraph_optimizer_type_t type = WHOLEGRAPH_OPT_NONE;
  float lr           = 0.f;
  float weight_decay = 0.f;
  float epsilon      = 1e-8f;
  float beta1        = 0.9f;
  float beta2        = 0.999f;
  float alpha        = 0.99f;
  bool adam_w        = false;
};

struct sparse_apply_args {
  // Gradient list as it arrived at the owner: ids[k] is a GLOBAL row id, its fp32 gradient row
  // starts at grads + k * grad_stride.  Ids outside [local_start, local_start + local_rows) are
  // ignored.
  const void* ids      = nullptr;  // int32 or int64
  bool ids_are_64      = true;
  int64_t count        = 0;
  const float* grads   = nullptr;
  int64_t grad_stride  = 0;
  int64_t dim          = 0;
  // This rank's shard.
  int64_t local_start  = 0;
  int64_t local_rows   = 0;
  void* weights        = nullptr;  // row r at weights + r * weight_stride elements
  wholegraph_dtype_t weight_dtype = WHOLEGRAPH_DT_FLOAT;  // fp32 / fp16 / bf16
  int64_t weight_stride = 0;
  float* state         = nullptr;  // per-element fp32 state rows (m | v, state_sum, or v)
  int64_t state_stride = 0;
  int64_t v_offset     = 0;        // Lazy Adam: v lives v_offset elements after m in a state row
  float* beta12t       = nullptr;  // Lazy Adam: [local_rows, 2] running beta1^t, beta2^t per row
  // Optional caches in front of the weight rows and the state rows (tags == nullptr: none).  A row
  // that is cached is updated in its cache line, which is marked modified; the table row is left
  // alone until the line is written back (reference: optimizer_get_ptr_from_cache,
  // embedding_optimizer_func.cu:140-164).
  cache_view weight_cache;
  cache_view state_cache;
  optimizer_hyper hyper;
};

// Device scratch needed for a list of `count` gradient rows.
size_t sparse_apply_workspace_bytes(int64_t count, int64_t local_rows, int64_t dim);

// Enqueue: group equal ids (stable radix sort of local row ids), add each group's gradient rows
// one after the other in arrival order in fp32, and apply the optimizer to the row - without
// materialising the summed gradients.  A group of more than WHOLEGRAPH_B200_DEDUP_BLOCK rows is
// cut into blocks of that many rows (in arrival order); each block is summed in order, and the
// block sums are then added in block order.  That is the one place where the order of additions
// differs from the reference's single chain; it keeps a hot row from serialising the step.  Every product, sum, quotient and square root is
// a separately rounded fp32 operation, in the order of the reference kernels.
void sparse_apply(const sparse_apply_args& a, void* workspace, cudaStream_t stream);

// Sender-side half of a two-level reduction: group the gradient rows of one rank by id and write
// one fp32 row of sums per distinct id.  Distinct ids ascend, so the rows of every owner are one
// contiguous range of them.  The order of additions inside a group is that of sparse_apply
// (arrival order; groups longer than WHOLEGRAPH_B200_DEDUP_BLOCK rows block by block).
//
// Step 1, reduce_duplicates_group: sort and group.
//   unique_ids   [count]  distinct ids that some rank owns (0 <= id < first_row[world]), ascending
//   owner_counts / owner_starts  device arrays of `world` entries: distinct ids per owner and
//                                where they start in unique_ids
//   first_row is a HOST array of world + 1 entries.
// Step 2, reduce_duplicates_sum, once the caller knows owner_counts on the host: the sums of the
// k-th distinct id of owner r are written to owner_out[r] + k * dim floats - local memory or a
// peer's, so that summation and transfer are one kernel.  Same workspace, count, table rows
// (= first_row[world]) and dim as in step 1, nothing else in between on that workspace.
size_t reduce_duplicates_workspace_bytes(int64_t count, int64_t table_rows, int64_t dim);
bool reduce_duplicates_supported(int64_t count, int64_t table_rows, int world);
void reduce_duplicates_group(const void* ids, bool ids_are_64, int64_t count, int64_t dim, const int64_t* first_row,
                             int world, void* workspace, int64_t* unique_ids, int64_t* owner_counts,
                             int64_t* owner_starts, cudaStream_t stream);
void reduce_duplicates_sum(int64_t count, int64_t table_rows, const float* grads, int64_t grad_stride, int64_t dim,
                           int world, const int64_t* owner_counts, float* const* owner_out, void* workspace,
                           cudaStream_t stream);

// Owner-side half of the two-level reduction when the per-rank sums stay where their senders
// computed them: every sender's region (mapped here: peer memory over NVLink, or local) holds a
// header, its distinct ids grouped by owner and one row of sums per id, and this rank merges and
// applies them without any count ever reaching the host and without a sort:
//   1. mark       every id sent here sets bit (row) in its sender's bitmap over this shard's rows
//   2. rank       exclusive prefix of the bitmaps' popcounts: a row's position in a sender's list
//                 is then two loads away (ids ascend inside a sender's group)
//   3. heads      the rows some sender touched, compacted
//   4. apply      one warp per such row: the senders that hold it, in rank order; their sums rows
//                 are read straight from the senders' regions while weights and state are read
//                 locally; sums added in rank order, then the same update as sparse_apply
// Results are those of sparse_apply on the concatenation of the senders' lists in rank order.
constexpr int kMaxMergeRanks = 32;
struct sender_region {
  const int64_t* header = nullptr;  // 2 * world int64: counts per owner | group starts
  const int64_t* ids    = nullptr;  // distinct ids, grouped by owner, ascending inside a group
  const float* sums     = nullptr;  // row k: the sums for ids[k], `dim` floats
};
struct merged_apply_args {
  int world = 1, me = 0;
  sender_region sender[kMaxMergeRanks];  // by rank
  int64_t capacity            = 0;       // ids a region can hold; headers claiming more are refused
  int64_t entries_upper_bound = 0;       // no more than this many ids are sent here in total
  int* status                 = nullptr; // device word, set non-zero on a refused header or id
  // the shard and the optimizer, as in sparse_apply_args (ids / grads / caches unused)
  sparse_apply_args shard;
};
size_t merged_apply_workspace_bytes(int world, int64_t local_rows, int64_t entries_upper_bound);
void merged_apply(const merged_apply_args& a, void* workspace, cudaStream_t stream);

// Fill `count` floats with `value` (state initialisation).
void fill_float(float* data, float value, int64_t count, cudaStream_t stream);

// Round-robin id remap, literal restatement of the reference's storage_idx2wg_emb_idx_kernel
// (cpp/src/wholegraph_tensor_ops/functions/map_indices_func.cu:16-34):
//   out[i] = entry_start + round_robin_size * ((ids[i] / round_robin_size) / world) + ids[i] % round_robin_size
void round_robin_remap(const void* ids, void* out, bool ids_are_64, int64_t count, int world,
                       int64_t entry_start, int round_robin_size, cudaStream_t stream);

}  // namespace wgb
