// Sparse SGD / Lazy Adam / AdaGrad / RMSProp apply fused with duplicate-gradient reduction.
//
//   1. keys_kernel        local row id (or a sentinel) and list position per gradient row
//   2. cub radix sort     (key, position) pairs, only the bits a local row id can use; stable, so
//                         equal ids keep their arrival order
//   3. cub select         first element of every run of equal keys, in order (run r ends where
//                         run r + 1 starts)
//   4. apply_kernel       a CTA stages the metadata of 256 runs, then one warp per distinct row
//                         requests the first gradient row, weights and state together, adds
//                         further duplicates in arrival order (fp32, 16-byte loads), updates
//                         and writes back; runs longer than 256 rows are registered only
//   5. sum_blocks_kernel  long runs: one warp per (block of 256 rows, column group), handed out by
//                         a device-side counter to a grid that just fills the GPU
//   6. apply_long_kernel  long runs: block sums added in order, then the same update
//
// The summed gradients never go to memory (the reference writes them to a [unique, dim] fp32
// buffer and reads them back).  Arithmetic follows the reference kernels
// (embedding_optimizer_func.cu:203-214 SGD, :386-421 Lazy Adam, :655-671 AdaGrad, :865-881
// RMSProp) with every operation rounded separately (no fused multiply-add), which is also what
// the reference's CPU test optimizer computes.
#include "sparse_optimizer.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>
#include <thrust/iterator/transform_iterator.h>

#include "../common.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads    = 256;
constexpr int kMaxOwnerRanks = 64;
constexpr int kDedupBlock = WHOLEGRAPH_B200_DEDUP_BLOCK;  // rows per block of a long duplicate run

__global__ void keys_kernel(const void* ids, int is64, int64_t n, int64_t local_start,
                            int64_t local_rows, uint32_t* keys, int32_t* positions)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t id = is64 ? __ldg(static_cast<const int64_t*>(ids) + i)
                          : static_cast<int64_t>(__ldg(static_cast<const int*>(ids) + i));
  const int64_t r  = id - local_start;
  keys[i]         = (r >= 0 && r < local_rows) ? static_cast<uint32_t>(r) : static_cast<uint32_t>(local_rows);
  positions[i]    = static_cast<int32_t>(i);
}

// True for the first element of every run of equal keys (sorted order).
struct is_run_head {
  const uint32_t* keys;
  __device__ __forceinline__ bool operator()(int i) const { return i == 0 || keys[i] != keys[i - 1]; }
};

template <typename T>
__device__ __forceinline__ float load_weight(const T* p)
{
  return static_cast<float>(*p);
}
template <typename T>
__device__ __forceinline__ void store_weight(T* p, float v)
{
  *p = static_cast<T>(v);  // fp16 / bf16: round to nearest even
}

// VEC consecutive elements as fp32, with one vector access when VEC = 4.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[VEC])
{
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    union {
      uint2 raw;
      T e[4];
    } u;
    u.raw = *reinterpret_cast<const uint2*>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) out[i] = static_cast<float>(u.e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; i++) out[i] = load_weight(p + i);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&in)[VEC])
{
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    union {
      uint2 raw;
      T e[4];
    } u;
#pragma unroll
    for (int i = 0; i < 4; i++) u.e[i] = static_cast<T>(in[i]);
    *reinterpret_cast<uint2*>(p) = u.raw;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; i++) store_weight(p + i, in[i]);
  }
}

struct apply_params {
  const uint32_t* keys;       // sorted local row ids
  const int32_t* positions;   // list position of each sorted element
  const int32_t* heads;       // first sorted element of every run, ascending
  const int32_t* head_count;  // number of runs (the run of foreign ids, if any, included)
  uint32_t sentinel;          // key of ids outside this rank's shard
  int64_t n;
  const float* grads;
  int64_t grad_stride;
  int dim;
  void* weights;
  int64_t weight_stride;
  float* state;
  int64_t state_stride;
  int64_t v_offset;
  float* beta12t;
  optimizer_hyper h;
  // Runs longer than kDedupBlock rows are summed in blocks (see sum_blocks_kernel).
  int32_t* long_first;    // per long run: index of its first sorted element
  int32_t* long_len;      // per long run: number of elements
  int32_t* long_slot;     // per long run: first partial-sum slot
  float2* long_beta;      // per long run: the row's stepped beta1^t, beta2^t (Lazy Adam)
  int32_t* long_run;      // per long run: its number among all runs (reduce-only mode)
  // Reduce-only mode: runs [owner_first_run[o], owner_first_run[o + 1]) belong to owner o and the
  // sums of run k go to owner_out[o] + (k - owner_first_run[o]) * dim floats (local or peer memory).
  int owners;
  int32_t owner_first_run[kMaxOwnerRanks + 1];
  float* owner_out[kMaxOwnerRanks];
  // Long runs and their slots are handed out by ONE 64-bit counter (long runs in the high word,
  // slots in the low word), so that a run registered later also has the higher first slot: long_slot
  // ascends and the run of a slot is found by bisection.
  unsigned long long* long_pack;
  int32_t* long_count;    // number of long runs (high word of long_pack)
  int32_t* slot_count;    // number of partial-sum slots handed out (low word of long_pack)
  int32_t* unit_cursor;   // next (slot, column group) unit (sum_blocks_kernel)
  float* partial;         // [slots, dim] block sums
  cache_view weight_cache;
  cache_view state_cache;
};

// Where row `row` of this rank's shard lives right now: its cache line (marked modified) when
// it is cached, `table_row` otherwise.  Warp-wide: lane l inspects line l of the row's set.
__device__ __forceinline__ char* current_copy(const cache_view& c, uint32_t row, int lane, char* table_row)
{
  if (c.tags == nullptr) return table_row;
  const int64_t set  = row / c.coverage;
  const uint16_t r   = static_cast<uint16_t>(row - set * c.coverage);
  uint16_t* tag_ptr  = c.tags + set * kCacheSetSize + lane;
  const uint16_t tag = *tag_ptr;
  const bool hit     = (tag & kTagValid) != 0 && (tag & kTagRowMask) == r;
  const unsigned m   = __ballot_sync(0xffffffffu, hit);
  if (m == 0) return table_row;
  const int line = __ffs(m) - 1;
  if (lane == line) *tag_ptr = tag | kTagModified;
  return c.lines + (set * kCacheSetSize + line) * c.line_bytes;
}

// One element of the update.  g is the summed gradient; w, s0, s1 are read-modify-write.
template <int OPT>
__device__ __forceinline__ void update_element(const optimizer_hyper& h, float g, float& w, float& s0,
                                               float& s1, float beta1t, float beta2t)
{
  if (OPT == WHOLEGRAPH_OPT_SGD) {
    g = __fadd_rn(g, __fmul_rn(h.weight_decay, w));
    w = __fsub_rn(w, __fmul_rn(h.lr, g));
  } else if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) {
    if (h.adam_w) {
      w = __fsub_rn(w, __fmul_rn(__fmul_rn(h.lr, h.weight_decay), w));
    } else {
      g = __fadd_rn(g, __fmul_rn(h.weight_decay, w));
    }
    float m = s0, v = s1;
    m = __fadd_rn(__fmul_rn(h.beta1, m), __fmul_rn(__fsub_rn(1.f, h.beta1), g));
    v = __fadd_rn(__fmul_rn(h.beta2, v), __fmul_rn(__fmul_rn(__fsub_rn(1.f, h.beta2), g), g));
    const float mhat = __fdiv_rn(m, __fsub_rn(1.f, beta1t));
    const float vhat = __fdiv_rn(v, __fsub_rn(1.f, beta2t));
    w  = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, mhat), __fadd_rn(__fsqrt_rn(vhat), h.epsilon)));
    s0 = m;
    s1 = v;
  } else if (OPT == WHOLEGRAPH_OPT_ADAGRAD) {
    g  = __fadd_rn(g, __fmul_rn(h.weight_decay, w));
    s0 = __fadd_rn(s0, __fmul_rn(g, g));
    w  = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, g), __fadd_rn(__fsqrt_rn(s0), h.epsilon)));
  } else {  // RMSProp
    g  = __fadd_rn(g, __fmul_rn(h.weight_decay, w));
    s0 = __fadd_rn(__fmul_rn(h.alpha, s0), __fmul_rn(__fmul_rn(__fsub_rn(1.f, h.alpha), g), g));
    w  = __fsub_rn(w, __fdiv_rn(__fmul_rn(h.lr, g), __fadd_rn(__fsqrt_rn(s0), h.epsilon)));
  }
}

// VEC gradient elements through the read-only path; nothing is read when `on` is false.
template <int VEC>
__device__ __forceinline__ void load_grad(const float* g, bool on, float (&out)[VEC])
{
  if (!on) return;
  if constexpr (VEC == 4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(g));
    out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
  } else {
    out[0] = __ldg(g);
  }
}

// Reduce-only mode: where the sums of run `run` go.
__device__ __forceinline__ float* reduce_destination(const apply_params& p, int64_t run)
{
  int o = 0;
  while (o + 1 < p.owners && run >= p.owner_first_run[o + 1]) o++;
  return p.owner_out[o] + (run - p.owner_first_run[o]) * p.dim;
}

// Weights and state of columns [c, c + VEC) of one row, held in registers between the loads
// (issued together with the first gradient loads) and the update.
template <int OPT, typename W, int VEC>
struct row_columns {
  float w[VEC], s0[VEC], s1[VEC];
  __device__ __forceinline__ void load(const apply_params& p, const W* w_row, const float* s_row, int c, bool on)
  {
    if (!on || OPT == WHOLEGRAPH_OPT_NONE) return;
    load_vec<W, VEC>(w_row + c, w);
    if (OPT != WHOLEGRAPH_OPT_SGD) load_vec<float, VEC>(s_row + c, s0);
    if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) load_vec<float, VEC>(s_row + p.v_offset + c, s1);
  }
  __device__ __forceinline__ void update_and_store(const apply_params& p, W* w_row, float* s_row, int c, bool on,
                                                   const float (&g)[VEC], float beta1t, float beta2t)
  {
    if (!on) return;
    if constexpr (OPT == WHOLEGRAPH_OPT_NONE) {  // reduce only: the row of sums is the output
      store_vec<W, VEC>(w_row + c, g);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; e++) update_element<OPT>(p.h, g[e], w[e], s0[e], s1[e], beta1t, beta2t);
      if (OPT != WHOLEGRAPH_OPT_SGD) store_vec<float, VEC>(s_row + c, s0);
      if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) store_vec<float, VEC>(s_row + p.v_offset + c, s1);
      store_vec<W, VEC>(w_row + c, w);
    }
  }
};

constexpr int kTileRuns    = kThreads;  // runs whose metadata one CTA stages at a time, one per thread (64-run tiles measured slower: 1.26 against 1.18 ms per C5 step)
constexpr int kApplyFlight = 4;         // duplicate rows a lane requests (for two column groups) before adding
// CTAs per SM of the two update kernels.  With 4 rows in flight they fit 80 registers without
// spills, which buys a third CTA per SM (24 warps instead of 16); measured on the 2,097,152-row
// Zipf(1.1) Lazy Adam step this beats 8 rows in flight at two CTAs (0.91 against 0.97 ms), the
// update being bound by instruction issue and latency together, not by duplicate rows in flight.
constexpr int kApplyCtas = 3;

// Distinct rows with at most kDedupBlock duplicates: summed and applied here.  Longer runs are
// only registered, with one partial-sum slot per block of kDedupBlock rows.
//
// A CTA takes kTileRuns consecutive runs.  Its first kTileRuns threads stage, in parallel and with
// coalesced loads, everything a run's update depends on: where the run starts and ends, its row,
// the list position of its first gradient row and (Lazy Adam) the row's stepped beta powers.
// Its warps then take runs from the tile one by one; with the metadata in shared memory a warp
// can request the first gradient row, the weights and the state of up to two column groups in
// one go, so that a run costs one memory round trip plus one per kApplyFlight further duplicates
// (their list positions come 32 at a time from one coalesced load, handed out by shuffles).
// VEC = 4: dim, strides and base pointers allow 16-byte accesses; VEC = 1 otherwise.
template <int OPT, typename W, int VEC>
__global__ void __launch_bounds__(kThreads, kApplyCtas) apply_kernel(const apply_params p)
{
  __shared__ int32_t s_first[kTileRuns + 1];
  __shared__ uint32_t s_row[kTileRuns];
  __shared__ int32_t s_pos0[kTileRuns];  // -1: nothing to do here (foreign ids, long run)
  __shared__ float s_beta[OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? kTileRuns : 1][2];
  __shared__ int s_next;
  const int lane = threadIdx.x & 31;
  const int t    = threadIdx.x;
  const int runs = *p.head_count;
  W* weights     = static_cast<W*>(p.weights);
  constexpr unsigned kFull = 0xffffffffu;

  for (int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kTileRuns; tile0 < runs;
       tile0 += static_cast<int64_t>(gridDim.x) * kTileRuns) {
    __syncthreads();  // the previous tile has been consumed
    const bool stager = t < kTileRuns;
    const int64_t run = tile0 + t;
    int32_t first     = static_cast<int32_t>(p.n);
    uint32_t row      = p.sentinel;
    int32_t pos0      = -1;
    if (stager && run < runs) {
      first = p.heads[run];
      row   = p.keys[first];
      pos0  = p.positions[first];
    }
    if (stager) s_first[t] = first;
    if (t == 0) {
      s_first[kTileRuns] = tile0 + kTileRuns < runs ? p.heads[tile0 + kTileRuns] : static_cast<int32_t>(p.n);
      s_next             = 0;
    }
    __syncthreads();
    if (row == p.sentinel) pos0 = -1;  // ids this rank does not own sort last
    if (pos0 >= 0) {
      const int len = s_first[t + 1] - first;  // heads ascend: a run ends where the next one starts
      float beta1t = 0.f, beta2t = 0.f;
      if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) {
        // per-row running beta1^t, beta2^t: multiplied on every touch of the row
        float2* b = reinterpret_cast<float2*>(p.beta12t) + row;
        float2 v  = *b;
        v.x = beta1t = __fmul_rn(v.x, p.h.beta1);
        v.y = beta2t = __fmul_rn(v.y, p.h.beta2);
        *b           = v;
      }
      if (len > kDedupBlock) {
        const int blocks = (len + kDedupBlock - 1) / kDedupBlock;
        const unsigned long long old =
          atomicAdd(p.long_pack, (1ull << 32) | static_cast<unsigned long long>(blocks));
        const int li     = static_cast<int>(old >> 32);
        const int slot   = static_cast<int>(old & 0xffffffffull);
        p.long_first[li] = first;
        p.long_len[li]   = len;
        p.long_slot[li]  = slot;
        p.long_beta[li]  = make_float2(beta1t, beta2t);
        p.long_run[li]   = static_cast<int32_t>(run);
        pos0 = -1;
      } else if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) {
        s_beta[t][0] = beta1t, s_beta[t][1] = beta2t;
      }
    }
    if (stager) {
      s_row[t]  = row;
      s_pos0[t] = pos0;
    }
    __syncthreads();

    const int in_tile = static_cast<int>(runs - tile0 < kTileRuns ? runs - tile0 : kTileRuns);
    auto next_run = [&]() -> int {
      int r = 0;
      if (lane == 0) r = atomicAdd(&s_next, 1);
      return __shfl_sync(kFull, r, 0);
    };
    for (int r = next_run(); r < in_tile; r = next_run()) {
      const int first_pos = s_pos0[r];
      if (first_pos < 0) continue;
      const int64_t begin = s_first[r], end = s_first[r + 1];
      const uint32_t urow = s_row[r];
      const float beta1t  = OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? s_beta[r][0] : 0.f;
      const float beta2t  = OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? s_beta[r][1] : 0.f;
      // reduce only: the sums go to the run's row at its owner, which stands in for the table row
      W* w_row = OPT == WHOLEGRAPH_OPT_NONE ? reinterpret_cast<W*>(reduce_destination(p, tile0 + r))
                                            : weights + static_cast<int64_t>(urow) * p.weight_stride;
      float* s_rw  = p.state != nullptr ? p.state + static_cast<int64_t>(urow) * p.state_stride : nullptr;
      w_row        = reinterpret_cast<W*>(current_copy(p.weight_cache, urow, lane, reinterpret_cast<char*>(w_row)));
      if (s_rw != nullptr)
        s_rw = reinterpret_cast<float*>(current_copy(p.state_cache, urow, lane, reinterpret_cast<char*>(s_rw)));
      const float* g_first = p.grads + static_cast<int64_t>(first_pos) * p.grad_stride;

      for (int cb = 0; cb < p.dim; cb += 64 * VEC) {  // two column groups per pass, warp-uniform trip count
        const int c0 = cb + lane * VEC, c1 = c0 + 32 * VEC;
        const bool on0 = c0 < p.dim, on1 = c1 < p.dim;
        float acc0[VEC] = {}, acc1[VEC] = {};
        row_columns<OPT, W, VEC> x0, x1;
        load_grad<VEC>(g_first + c0, on0, acc0);
        load_grad<VEC>(g_first + c1, on1, acc1);
        x0.load(p, w_row, s_rw, c0, on0);
        x1.load(p, w_row, s_rw, c1, on1);
        // further duplicates, in arrival order
        for (int64_t base = begin; end - begin > 1 && base < end; base += 32) {
          const int chunk = static_cast<int>(end - base < 32 ? end - base : 32);
          const int mine  = lane < chunk ? p.positions[base + lane] : 0;
          for (int j = base == begin ? 1 : 0; j < chunk; j += kApplyFlight) {
            float v0[kApplyFlight][VEC], v1[kApplyFlight][VEC];
#pragma unroll
            for (int u = 0; u < kApplyFlight; u++) {
              const int pos   = __shfl_sync(kFull, mine, (j + u) & 31);
              const bool live = j + u < chunk;
              const float* g  = p.grads + static_cast<int64_t>(pos) * p.grad_stride;
              load_grad<VEC>(g + c0, live && on0, v0[u]);
              load_grad<VEC>(g + c1, live && on1, v1[u]);
            }
#pragma unroll
            for (int u = 0; u < kApplyFlight; u++) {
              if (j + u < chunk) {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                  acc0[e] = __fadd_rn(acc0[e], v0[u][e]);
                  acc1[e] = __fadd_rn(acc1[e], v1[u][e]);
                }
              }
            }
          }
        }
        x0.update_and_store(p, w_row, s_rw, c0, on0, acc0, beta1t, beta2t);
        x1.update_and_store(p, w_row, s_rw, c1, on1, acc1, beta1t, beta2t);
      }
    }
  }
}

constexpr int kBlockFlight = 8;  // gradient rows in flight per lane while a block is summed

// One warp per (partial-sum slot, group of 32 * VEC columns): block b of a long run, rows
// [b * kDedupBlock, (b + 1) * kDedupBlock) of the run, added in order.  List positions are read 32
// at a time, one coalesced load ahead of their use.  The units are handed out by a device-side
// counter to a grid that just fills the GPU (their number is only known on the device, and a
// fixed split leaves most SMs idle while the last wave runs).  The long run a slot belongs to is
// found by bisection over the runs' first slots, which ascend.
template <int VEC>
__global__ void __launch_bounds__(kThreads, 3) sum_blocks_kernel(const apply_params p)
{
  constexpr unsigned kFull = 0xffffffffu;
  const int lane           = threadIdx.x & 31;
  const int groups         = (p.dim + 32 * VEC - 1) / (32 * VEC);
  const int long_runs      = *p.long_count;
  const int64_t units      = static_cast<int64_t>(*p.slot_count) * groups;
  auto next_unit = [&]() -> int64_t {
    int u = 0;
    if (lane == 0) u = atomicAdd(p.unit_cursor, 1);
    return __shfl_sync(kFull, u, 0);
  };
  for (int64_t unit = next_unit(); unit < units; unit = next_unit()) {
    const int s   = static_cast<int>(unit / groups);
    const int c   = static_cast<int>(unit - static_cast<int64_t>(s) * groups) * 32 * VEC + lane * VEC;
    const bool on = c < p.dim;
    int lo = 0, hi = long_runs - 1;  // last long run whose first slot is <= s
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.long_slot[mid] <= s) lo = mid;
      else hi = mid - 1;
    }
    const int li        = lo;
    const int64_t begin = p.long_first[li];
    const int64_t end   = begin + p.long_len[li];
    const int64_t first = begin + static_cast<int64_t>(s - p.long_slot[li]) * kDedupBlock;
    const int64_t last  = first + kDedupBlock < end ? first + kDedupBlock : end;
    float acc[VEC]      = {};
    int next_pos        = first + lane < last ? p.positions[first + lane] : 0;
    for (int64_t base = first; base < last; base += 32) {
      const int chunk = static_cast<int>(last - base < 32 ? last - base : 32);
      const int mine  = next_pos;
      if (base + 32 < last) next_pos = base + 32 + lane < last ? p.positions[base + 32 + lane] : 0;
      for (int j = 0; j < chunk; j += kBlockFlight) {
        float v[kBlockFlight][VEC];
#pragma unroll
        for (int u = 0; u < kBlockFlight; u++) {
          const int pos = __shfl_sync(kFull, mine, (j + u) & 31);
          load_grad<VEC>(p.grads + static_cast<int64_t>(pos) * p.grad_stride + c, on && j + u < chunk, v[u]);
        }
#pragma unroll
        for (int u = 0; u < kBlockFlight; u++) {
          if (j + u < chunk) {
            if (base == first && j + u == 0) {  // the first row starts the sum
#pragma unroll
              for (int e = 0; e < VEC; e++) acc[e] = v[u][e];
            } else {
#pragma unroll
              for (int e = 0; e < VEC; e++) acc[e] = __fadd_rn(acc[e], v[u][e]);
            }
          }
        }
      }
    }
    if (on) {
      float* out = p.partial + static_cast<int64_t>(s) * p.dim + c;
#pragma unroll
      for (int e = 0; e < VEC; e++) out[e] = acc[e];
    }
  }
}

constexpr int kPartialFlight = 32;  // block sums in flight per lane while a long run is finished

// One warp per (long run, group of 32 columns): adds the run's block sums in block order and
// applies the optimizer to its columns.  The additions of a column are one chain in block order,
// so what a warp can do about latency is keep many block sums in flight: one float per lane
// (a warp reads 128 contiguous bytes of every block sum) and kPartialFlight loads issued before the
// first addition, which also gives a long run eight warps per 256 columns instead of two.
template <int OPT, typename W>
__global__ void __launch_bounds__(kThreads, 2) apply_long_kernel(const apply_params p)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int groups          = (p.dim + 31) / 32;
  const int64_t units       = static_cast<int64_t>(*p.long_count) * groups;
  W* weights                = static_cast<W*>(p.weights);
  for (int64_t unit = warp_global; unit < units; unit += warp_stride) {
    const int64_t li   = unit / groups;
    const int c        = static_cast<int>(unit - li * groups) * 32 + lane;
    const bool on      = c < p.dim;
    const uint32_t row = p.keys[p.long_first[li]];
    const int blocks   = (p.long_len[li] + kDedupBlock - 1) / kDedupBlock;
    const float* part  = p.partial + static_cast<int64_t>(p.long_slot[li]) * p.dim + c;
    const float2 beta  = p.long_beta[li];
    W* w_row = OPT == WHOLEGRAPH_OPT_NONE ? reinterpret_cast<W*>(reduce_destination(p, p.long_run[li]))
                                          : weights + static_cast<int64_t>(row) * p.weight_stride;
    float* s_row = p.state != nullptr ? p.state + static_cast<int64_t>(row) * p.state_stride : nullptr;
    w_row        = reinterpret_cast<W*>(current_copy(p.weight_cache, row, lane, reinterpret_cast<char*>(w_row)));
    if (s_row != nullptr)
      s_row = reinterpret_cast<float*>(current_copy(p.state_cache, row, lane, reinterpret_cast<char*>(s_row)));
    row_columns<OPT, W, 1> x;
    x.load(p, w_row, s_row, c, on);
    float acc[1] = {0.f};
    if (on) {
      acc[0] = part[0];
      for (int b = 1; b < blocks; b += kPartialFlight) {
        float v[kPartialFlight];
#pragma unroll
        for (int u = 0; u < kPartialFlight; u++)
          if (b + u < blocks) v[u] = part[static_cast<int64_t>(b + u) * p.dim];
#pragma unroll
        for (int u = 0; u < kPartialFlight; u++)
          if (b + u < blocks) acc[0] = __fadd_rn(acc[0], v[u]);
      }
    }
    x.update_and_store(p, w_row, s_row, c, on, acc, beta.x, beta.y);
  }
}

__global__ void fill_kernel(float* data, float value, int64_t n)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) data[i] = value;
}

template <typename I>
__global__ void round_robin_kernel(const I* ids, I* out, int64_t n, int world, int64_t entry_start, int rr)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const I id    = ids[i];
  const I block = id / rr;
  out[i]        = static_cast<I>(entry_start + static_cast<int64_t>(rr) * (block / world) + id % rr);
}

struct workspace_layout {
  size_t keys_in, keys_out, pos_in, pos_out, heads, counters, cub, total;
  size_t long_first, long_len, long_slot, long_beta, long_run, partial;
  size_t cub_bytes, select_bytes;
};

int key_bits(int64_t local_rows)
{
  int bits = 1;
  while (bits < 32 && (int64_t(1) << bits) <= local_rows) bits++;  // the sentinel is local_rows itself
  return bits;
}

workspace_layout layout_for(int64_t n, int64_t local_rows, int64_t dim)
{
  workspace_layout l{};
  auto align = [](size_t x) { return (x + 255) / 256 * 256; };
  const size_t cnt = static_cast<size_t>(std::max<int64_t>(n, 1));
  size_t off       = 0;
  l.keys_in        = off, off += align(cnt * 4);
  l.keys_out       = off, off += align(cnt * 4);
  l.pos_in         = off, off += align(cnt * 4);
  l.pos_out        = off, off += align(cnt * 4);
  l.heads          = off, off += align(cnt * 4);
  l.counters       = off, off += 256;  // head count, long-run and slot counter, work cursors
  // At most n / block runs are long, and they need at most n / block + (their number) slots.
  const size_t max_long  = cnt / kDedupBlock + 1;
  const size_t max_slots = 2 * max_long;
  l.long_first = off, off += align(max_long * 4);
  l.long_len   = off, off += align(max_long * 4);
  l.long_slot  = off, off += align(max_long * 4);
  l.long_beta  = off, off += align(max_long * 8);
  l.long_run   = off, off += align(max_long * 4);
  l.partial    = off, off += align(max_slots * static_cast<size_t>(std::max<int64_t>(dim, 1)) * 4);
  l.cub_bytes      = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, l.cub_bytes, static_cast<const uint32_t*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), static_cast<int>(cnt), 0,
                                  key_bits(local_rows));
  l.select_bytes = 0;
  cub::DeviceSelect::If(nullptr, l.select_bytes, thrust::counting_iterator<int>(0), static_cast<int32_t*>(nullptr),
                        static_cast<int32_t*>(nullptr), static_cast<int>(cnt), is_run_head{nullptr});
  l.cub_bytes = std::max(l.cub_bytes, l.select_bytes);
  l.cub   = off, off += align(l.cub_bytes);
  l.total = off;
  return l;
}

int sm_count()
{
  static int n = [] {
    int dev = 0, count = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    return count;
  }();
  return n;
}

template <int OPT, typename W>
void launch_apply(const apply_params& p, bool vec4, int ctas, cudaStream_t stream)
{
  // The number of long runs and of their blocks is only known on the device: the block sums
  // take a grid that just fills the GPU and draw their work from a counter; the few long runs
  // themselves take a fixed modest grid.
  const int sms       = sm_count();
  const int long_ctas = sms * 4;
  if (vec4) {
    apply_kernel<OPT, W, 4><<<ctas, kThreads, 0, stream>>>(p);
    sum_blocks_kernel<4><<<sms * 3, kThreads, 0, stream>>>(p);
  } else {
    apply_kernel<OPT, W, 1><<<ctas, kThreads, 0, stream>>>(p);
    sum_blocks_kernel<1><<<sms * 3, kThreads, 0, stream>>>(p);
  }
  apply_long_kernel<OPT, W><<<long_ctas, kThreads, 0, stream>>>(p);
}

template <typename W>
void launch_apply_opt(const apply_params& p, bool vec4, int ctas, cudaStream_t stream)
{
  switch (p.h.type) {
    case WHOLEGRAPH_OPT_NONE:
      if constexpr (sizeof(W) == 4) launch_apply<WHOLEGRAPH_OPT_NONE, W>(p, vec4, ctas, stream);
      break;
    case WHOLEGRAPH_OPT_SGD: launch_apply<WHOLEGRAPH_OPT_SGD, W>(p, vec4, ctas, stream); break;
    case WHOLEGRAPH_OPT_LAZY_ADAM: launch_apply<WHOLEGRAPH_OPT_LAZY_ADAM, W>(p, vec4, ctas, stream); break;
    case WHOLEGRAPH_OPT_ADAGRAD: launch_apply<WHOLEGRAPH_OPT_ADAGRAD, W>(p, vec4, ctas, stream); break;
    case WHOLEGRAPH_OPT_RMSPROP: launch_apply<WHOLEGRAPH_OPT_RMSPROP, W>(p, vec4, ctas, stream); break;
    default: WGB_EXPECTS(false, "unknown optimizer type %d", (int)p.h.type);
  }
}

}  // namespace

size_t sparse_apply_workspace_bytes(int64_t count, int64_t local_rows, int64_t dim)
{
  return layout_for(count, local_rows, dim).total;
}

void fill_float(float* data, float value, int64_t count, cudaStream_t stream)
{
  if (count <= 0) return;
  fill_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream>>>(data, value, count);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

void round_robin_remap(const void* ids, void* out, bool ids_are_64, int64_t count, int world,
                       int64_t entry_start, int round_robin_size, cudaStream_t stream)
{
  if (count <= 0) return;
  const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
  if (ids_are_64)
    round_robin_kernel<int64_t><<<blocks, 256, 0, stream>>>(static_cast<const int64_t*>(ids),
                                                            static_cast<int64_t*>(out), count, world,
                                                            entry_start, round_robin_size);
  else
    round_robin_kernel<int><<<blocks, 256, 0, stream>>>(static_cast<const int*>(ids), static_cast<int*>(out),
                                                        count, world, entry_start, round_robin_size);
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

namespace {

// The grouping fields of `p` and its long-run scratch pointers inside a workspace.
void bind_workspace(int64_t count, int64_t key_rows, const workspace_layout& l, char* ws, apply_params* p)
{
  auto* counters = reinterpret_cast<int32_t*>(ws + l.counters);
  p->keys        = reinterpret_cast<uint32_t*>(ws + l.keys_out);
  p->positions   = reinterpret_cast<int32_t*>(ws + l.pos_out);
  p->heads       = reinterpret_cast<int32_t*>(ws + l.heads);
  p->head_count = counters, p->n = count;
  p->sentinel   = static_cast<uint32_t>(key_rows);
  // counters: [0] run heads, [2..3] the 64-bit long-run / slot counter (slots in the low word),
  // [4] block-sum cursor
  p->long_pack   = reinterpret_cast<unsigned long long*>(counters + 2);
  p->slot_count  = counters + 2, p->long_count = counters + 3;
  p->unit_cursor = counters + 4;
  p->long_first = reinterpret_cast<int32_t*>(ws + l.long_first);
  p->long_len   = reinterpret_cast<int32_t*>(ws + l.long_len);
  p->long_slot  = reinterpret_cast<int32_t*>(ws + l.long_slot);
  p->long_beta  = reinterpret_cast<float2*>(ws + l.long_beta);
  p->long_run   = reinterpret_cast<int32_t*>(ws + l.long_run);
  p->partial    = reinterpret_cast<float*>(ws + l.partial);
  p->owners     = 0;
}

// Steps 1-3 of every pass: keys, stable sort, ordered run heads.
void group_rows(const void* ids, bool ids_are_64, int64_t count, int64_t key_start, int64_t key_rows,
                const workspace_layout& l, char* ws, cudaStream_t stream, apply_params* p)
{
  auto* keys_in         = reinterpret_cast<uint32_t*>(ws + l.keys_in);
  auto* keys_out        = reinterpret_cast<uint32_t*>(ws + l.keys_out);
  auto* pos_in          = reinterpret_cast<int32_t*>(ws + l.pos_in);
  auto* pos_out         = reinterpret_cast<int32_t*>(ws + l.pos_out);
  auto* heads           = reinterpret_cast<int32_t*>(ws + l.heads);
  auto* counters        = reinterpret_cast<int32_t*>(ws + l.counters);
  const unsigned blocks = static_cast<unsigned>((count + kThreads - 1) / kThreads);
  keys_kernel<<<blocks, kThreads, 0, stream>>>(ids, ids_are_64 ? 1 : 0, count, key_start, key_rows, keys_in, pos_in);
  size_t cub_bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(ws + l.cub, cub_bytes, keys_in, keys_out, pos_in, pos_out,
                                                 static_cast<int>(count), 0, key_bits(key_rows), stream));
  WGB_CUDA_CHECK(cudaMemsetAsync(counters, 0, 8 * sizeof(int32_t), stream));
  size_t select_bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceSelect::If(ws + l.cub, select_bytes, thrust::counting_iterator<int>(0), heads, counters,
                                       static_cast<int>(count), is_run_head{keys_out}, stream));
  bind_workspace(count, key_rows, l, ws, p);
}

int apply_grid(int64_t count)
{
  // One CTA per tile of kTileRuns distinct rows (the hardware hands a new CTA to an SM as soon
  // as one finishes, so tiles of uneven weight balance themselves), grid-stride beyond a few
  // waves.  The number of rows is only known on the device, so the grid covers the case that
  // every gradient row has its own id; CTAs without a tile leave at once.
  const int64_t tiles = (count + kTileRuns - 1) / kTileRuns;
  return static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(sm_count()) * kApplyCtas * 8));
}

struct owner_table {
  int world;
  int64_t first_row[kMaxOwnerRanks + 1];
};

// Runs are ascending by id, so every owner's runs are one contiguous range: thread r finds where
// owner r's range starts (first run whose id is >= first_row[r]) by bisection over the heads.
__global__ void owner_ranges_kernel(const uint32_t* keys, const int32_t* heads, const int32_t* head_count,
                                    const owner_table t, int64_t* counts, int64_t* starts)
{
  __shared__ int64_t s_start[kMaxOwnerRanks + 1];
  const int r = threadIdx.x;
  if (r <= t.world) {
    int lo = 0, hi = *head_count;  // the run of rejected ids (key = table rows), if any, stays right of every range
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (static_cast<int64_t>(keys[heads[mid]]) < t.first_row[r]) lo = mid + 1;
      else hi = mid;
    }
    s_start[r] = lo;
  }
  __syncthreads();
  if (r < t.world) {
    starts[r] = s_start[r];
    counts[r] = s_start[r + 1] - s_start[r];
  }
}

// Id of every run (ascending); the run of rejected ids is left out.
__global__ void run_ids_kernel(const uint32_t* keys, const int32_t* heads, const int32_t* head_count,
                               uint32_t sentinel, int64_t* unique_ids)
{
  const int64_t run = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (run >= *head_count) return;
  const uint32_t key = keys[heads[run]];
  if (key != sentinel) unique_ids[run] = key;
}

}  // namespace

size_t reduce_duplicates_workspace_bytes(int64_t count, int64_t table_rows, int64_t dim)
{
  return layout_for(count, table_rows, dim).total;
}

bool reduce_duplicates_supported(int64_t count, int64_t table_rows, int world)
{
  return count < (int64_t(1) << 31) && table_rows < (int64_t(1) << 32) - 1 && world <= kMaxOwnerRanks;
}

void reduce_duplicates_group(const void* ids, bool ids_are_64, int64_t count, int64_t dim, const int64_t* first_row,
                             int world, void* workspace, int64_t* unique_ids, int64_t* owner_counts,
                             int64_t* owner_starts, cudaStream_t stream)
{
  WGB_EXPECTS(count > 0 && dim > 0, "nothing to reduce");
  WGB_EXPECTS(reduce_duplicates_supported(count, first_row[world], world), "gradient list too large to pre-reduce");
  const int64_t table_rows = first_row[world];
  const workspace_layout l = layout_for(count, table_rows, dim);
  apply_params p{};
  group_rows(ids, ids_are_64, count, 0, table_rows, l, static_cast<char*>(workspace), stream, &p);
  owner_table t;
  t.world = world;
  for (int r = 0; r <= world; r++) t.first_row[r] = first_row[r];
  owner_ranges_kernel<<<1, kMaxOwnerRanks + 1, 0, stream>>>(p.keys, p.heads, p.head_count, t, owner_counts,
                                                            owner_starts);
  run_ids_kernel<<<static_cast<unsigned>((count + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
    p.keys, p.heads, p.head_count, p.sentinel, unique_ids);
  count_kernel_launch(6);
  WGB_LAUNCH_CHECK(stream);
}

void reduce_duplicates_sum(int64_t count, int64_t table_rows, const float* grads, int64_t grad_stride, int64_t dim,
                           int world, const int64_t* owner_counts, float* const* owner_out, void* workspace,
                           cudaStream_t stream)
{
  const workspace_layout l = layout_for(count, table_rows, dim);
  apply_params p{};
  bind_workspace(count, table_rows, l, static_cast<char*>(workspace), &p);
  p.grads = grads, p.grad_stride = grad_stride, p.dim = static_cast<int>(dim);
  p.weights = nullptr, p.weight_stride = dim;
  p.state = nullptr, p.beta12t = nullptr;
  p.h.type = WHOLEGRAPH_OPT_NONE;
  p.owners = world;
  bool vec4 = dim % 4 == 0 && grad_stride % 4 == 0 && reinterpret_cast<uintptr_t>(grads) % 16 == 0;
  int64_t first = 0;
  for (int r = 0; r < world; r++) {
    p.owner_first_run[r] = static_cast<int32_t>(first);
    p.owner_out[r]       = owner_out[r];
    first += owner_counts[r];
    vec4 = vec4 && reinterpret_cast<uintptr_t>(owner_out[r]) % 16 == 0;
  }
  p.owner_first_run[world] = static_cast<int32_t>(first);
  launch_apply_opt<float>(p, vec4, apply_grid(count), stream);
  count_kernel_launch(3);
  WGB_LAUNCH_CHECK(stream);
}

// ---- merged apply: per-rank sums read from their senders' regions --------------------------------
namespace {

struct merge_params {
  int world, me;
  int64_t capacity;
  int64_t local_start, local_rows;
  int words;                 // 32-bit bitmap words per sender
  uint32_t* bitmap;          // [world][words]
  int32_t* rank;             // [world * words + 1] exclusive prefix of popcounts
  int32_t* heads;            // rows some sender touched
  int32_t* head_count;
  int* status;
  int dim;
  void* weights;
  int64_t weight_stride;
  float* state;
  int64_t state_stride, v_offset;
  float* beta12t;
  optimizer_hyper h;
  sender_region sender[kMaxMergeRanks];
};

// Group of this rank in sender q's lists: counts[me] ids starting at starts[me]; refused (and
// treated as empty) when it does not fit the region.
__device__ __forceinline__ void read_group(const merge_params& p, int q, int64_t* count, int64_t* start)
{
  const int64_t* h = p.sender[q].header;
  int64_t c        = __ldcg(h + p.me);
  const int64_t s  = __ldcg(h + p.world + p.me);
  if (c < 0 || s < 0 || s + c > p.capacity) {
    atomicExch(p.status, 1);
    c = 0;
  }
  *count = c, *start = s;
}

__global__ void __launch_bounds__(kThreads) merge_mark_kernel(const merge_params p)
{
  __shared__ int64_t s_prefix[kMaxMergeRanks + 1];
  __shared__ int64_t s_start[kMaxMergeRanks];
  if (threadIdx.x < p.world) {
    int64_t c, s;
    read_group(p, threadIdx.x, &c, &s);
    s_start[threadIdx.x]      = s;
    s_prefix[threadIdx.x + 1] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_prefix[0] = 0;
    for (int q = 0; q < p.world; q++) s_prefix[q + 1] += s_prefix[q];
  }
  __syncthreads();
  const int64_t total = s_prefix[p.world];
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int q = 0;
    while (q + 1 < p.world && i >= s_prefix[q + 1]) q++;
    const int64_t id  = __ldcg(p.sender[q].ids + s_start[q] + (i - s_prefix[q]));
    const int64_t row = id - p.local_start;
    if (row < 0 || row >= p.local_rows) {
      atomicExch(p.status, 2);
      continue;
    }
    atomicOr(p.bitmap + static_cast<int64_t>(q) * p.words + (row >> 5), 1u << (row & 31));
  }
}

struct popcount_of {
  const uint32_t* words;
  __device__ __forceinline__ int operator()(int i) const { return __popc(words[i]); }
};

// Rows with a bit in any sender's bitmap, ascending inside a warp's 32 words.
__global__ void __launch_bounds__(kThreads) merge_heads_kernel(const merge_params p)
{
  const int lane = threadIdx.x & 31;
  for (int64_t w0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) & ~int64_t(31); w0 < p.words;
       w0 += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t w = w0 + lane;
    uint32_t any    = 0;
    if (w < p.words)
      for (int q = 0; q < p.world; q++) any |= p.bitmap[static_cast<int64_t>(q) * p.words + w];
    const int mine = __popc(any);
    int incl       = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) continue;
    int base = 0;
    if (lane == 31) base = atomicAdd(p.head_count, total);
    base    = __shfl_sync(0xffffffffu, base, 31);
    int out = base + incl - mine;
    while (any != 0u) {
      const int bit  = __ffs(any) - 1;
      p.heads[out++] = static_cast<int32_t>(w * 32 + bit);
      any &= any - 1u;
    }
  }
}

// Senders' rows in flight per lane (for two column groups) and CTAs per SM, measured on the
// 2,097,152-row Lazy Adam step: with one rank (sums in local memory) 3 rows in flight at 3 CTAs
// per SM (80 registers, no spill) take 1.09 ms against 1.25 ms for 4 rows at 2 CTAs; with eight
// ranks (most sums read over NVLink, hot rows held by every sender) it is the other way round,
// 1.59 against 1.65 ms - fewer round trips per row beat more warps.
struct merge_shape_local {
  static constexpr int kFlight = 3, kCtas = 3;
};
struct merge_shape_peers {
  static constexpr int kFlight = 4, kCtas = 2;
};

// One warp per touched row.  As in apply_kernel, a CTA first stages what a row's update depends
// on for kThreads rows at once, one row per thread with coalesced and independent loads: the row
// number, for every sender whether it holds the row and at which position of its list (bitmap word
// and rank word), and the row's stepped beta powers.  A warp then finds everything in shared memory
// and requests weights, state and every sender's sums row in one go.
template <int OPT, typename W, int VEC, typename SHAPE>
__global__ void __launch_bounds__(kThreads, SHAPE::kCtas) merge_apply_kernel(const merge_params p)
{
  extern __shared__ int32_t s_pos[];  // [world][kThreads]: position in sender q's group, -1 = not held
  __shared__ int64_t s_start[kMaxMergeRanks];
  __shared__ int32_t s_row[kThreads];
  __shared__ float s_beta[OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? kThreads : 1][2];
  __shared__ int s_next;
  if (threadIdx.x < p.world) {
    int64_t c, s;
    read_group(p, threadIdx.x, &c, &s);
    s_start[threadIdx.x] = s;
  }
  constexpr unsigned kFull = 0xffffffffu;
  const int lane           = threadIdx.x & 31;
  const int t              = threadIdx.x;
  const int heads          = *p.head_count;
  W* weights               = static_cast<W*>(p.weights);
  apply_params ap{};  // the fields row_columns reads
  ap.v_offset = p.v_offset, ap.h = p.h;
  auto next_row = [&]() -> int {
    int r = 0;
    if (lane == 0) r = atomicAdd(&s_next, 1);
    return __shfl_sync(kFull, r, 0);
  };
  for (int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kThreads; tile0 < heads;
       tile0 += static_cast<int64_t>(gridDim.x) * kThreads) {
    __syncthreads();  // the previous tile has been consumed (and s_start is in place)
    const int64_t hd = tile0 + t;
    int row          = -1;
    if (hd < heads) {
      row = p.heads[hd];
      for (int q = 0; q < p.world; q++) {
        const int64_t wi    = static_cast<int64_t>(q) * p.words + (row >> 5);
        const uint32_t word = p.bitmap[wi];
        int pos             = -1;
        if ((word >> (row & 31)) & 1u)
          pos = p.rank[wi] - p.rank[static_cast<int64_t>(q) * p.words] + __popc(word & ((1u << (row & 31)) - 1u));
        s_pos[q * kThreads + t] = pos;
      }
      if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) {
        // per-row running beta1^t, beta2^t: multiplied on every touch of the row
        float2* b = reinterpret_cast<float2*>(p.beta12t) + row;
        float2 v  = *b;
        v.x       = __fmul_rn(v.x, p.h.beta1);
        v.y       = __fmul_rn(v.y, p.h.beta2);
        *b        = v;
        s_beta[t][0] = v.x, s_beta[t][1] = v.y;
      }
    }
    s_row[t] = row;
    if (t == 0) s_next = 0;
    __syncthreads();
    const int in_tile = static_cast<int>(heads - tile0 < kThreads ? heads - tile0 : kThreads);
    for (int r = next_row(); r < in_tile; r = next_row()) {
      const int urow   = s_row[r];
      const float* src = nullptr;
      if (lane < p.world) {
        const int pos = s_pos[lane * kThreads + r];
        if (pos >= 0) src = p.sender[lane].sums + (s_start[lane] + pos) * p.dim;
      }
      const unsigned senders = __ballot_sync(kFull, src != nullptr);
      const float beta1t     = OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? s_beta[r][0] : 0.f;
      const float beta2t     = OPT == WHOLEGRAPH_OPT_LAZY_ADAM ? s_beta[r][1] : 0.f;
      W* w_row     = weights + static_cast<int64_t>(urow) * p.weight_stride;
      float* s_rw  = p.state != nullptr ? p.state + static_cast<int64_t>(urow) * p.state_stride : nullptr;
      for (int cb = 0; cb < p.dim; cb += 64 * VEC) {
        const int c0 = cb + lane * VEC, c1 = c0 + 32 * VEC;
        const bool on0 = c0 < p.dim, on1 = c1 < p.dim;
        float acc0[VEC] = {}, acc1[VEC] = {};
        row_columns<OPT, W, VEC> x0, x1;
        x0.load(ap, w_row, s_rw, c0, on0);
        x1.load(ap, w_row, s_rw, c1, on1);
        unsigned left = senders;
        bool first    = true;
        while (left != 0u) {
          float v0[SHAPE::kFlight][VEC], v1[SHAPE::kFlight][VEC];
          bool live[SHAPE::kFlight];
#pragma unroll
          for (int u = 0; u < SHAPE::kFlight; u++) {
            live[u]     = left != 0u;
            const int q = live[u] ? __ffs(left) - 1 : 0;
            if (live[u]) left &= left - 1u;
            const float* g = reinterpret_cast<const float*>(
              __shfl_sync(kFull, reinterpret_cast<unsigned long long>(src), q));
            load_grad<VEC>(g + c0, live[u] && on0, v0[u]);
            load_grad<VEC>(g + c1, live[u] && on1, v1[u]);
          }
#pragma unroll
          for (int u = 0; u < SHAPE::kFlight; u++) {
            if (live[u]) {
#pragma unroll
              for (int e = 0; e < VEC; e++) {
                acc0[e] = first ? v0[u][e] : __fadd_rn(acc0[e], v0[u][e]);
                acc1[e] = first ? v1[u][e] : __fadd_rn(acc1[e], v1[u][e]);
              }
              first = false;
            }
          }
        }
        x0.update_and_store(ap, w_row, s_rw, c0, on0, acc0, beta1t, beta2t);
        x1.update_and_store(ap, w_row, s_rw, c1, on1, acc1, beta1t, beta2t);
      }
    }
  }
}

struct merge_layout {
  size_t bitmap, rank, heads, counters, cub, total, cub_bytes;
  int words;
};

merge_layout merge_layout_for(int world, int64_t local_rows, int64_t entries_upper_bound)
{
  merge_layout l{};
  auto align = [](size_t x) { return (x + 255) / 256 * 256; };
  l.words    = static_cast<int>((local_rows + 31) / 32);
  size_t off = 0;
  const size_t all_words = static_cast<size_t>(world) * static_cast<size_t>(std::max(l.words, 1));
  l.bitmap = off, off += align(all_words * 4);
  l.counters = off, off += 256;
  l.rank = off, off += align((all_words + 1) * 4);
  l.heads = off, off += align(static_cast<size_t>(std::max<int64_t>(1, std::min(local_rows, entries_upper_bound))) * 4);
  l.cub_bytes = 0;
  auto counts = thrust::make_transform_iterator(thrust::counting_iterator<int>(0), popcount_of{nullptr});
  cub::DeviceScan::ExclusiveSum(nullptr, l.cub_bytes, counts, static_cast<int32_t*>(nullptr),
                                static_cast<int>(all_words + 1));
  l.cub = off, off += align(l.cub_bytes);
  l.total = off;
  return l;
}

template <int OPT, typename W>
void launch_merge_apply(const merge_params& p, bool vec4, cudaStream_t stream)
{
  // One CTA per tile of kThreads touched rows up to a few waves, then grid-stride; their number is
  // device data, CTAs without a tile leave at once.
  const bool peers   = p.world > 1;
  const int ctas     = sm_count() * (peers ? merge_shape_peers::kCtas : merge_shape_local::kCtas) * 8;
  const size_t smem  = static_cast<size_t>(p.world) * kThreads * sizeof(int32_t);
  if (vec4 && peers)
    merge_apply_kernel<OPT, W, 4, merge_shape_peers><<<ctas, kThreads, smem, stream>>>(p);
  else if (vec4)
    merge_apply_kernel<OPT, W, 4, merge_shape_local><<<ctas, kThreads, smem, stream>>>(p);
  else if (peers)
    merge_apply_kernel<OPT, W, 1, merge_shape_peers><<<ctas, kThreads, smem, stream>>>(p);
  else
    merge_apply_kernel<OPT, W, 1, merge_shape_local><<<ctas, kThreads, smem, stream>>>(p);
}

template <typename W>
void launch_merge_apply_opt(const merge_params& p, bool vec4, cudaStream_t stream)
{
  switch (p.h.type) {
    case WHOLEGRAPH_OPT_SGD: launch_merge_apply<WHOLEGRAPH_OPT_SGD, W>(p, vec4, stream); break;
    case WHOLEGRAPH_OPT_LAZY_ADAM: launch_merge_apply<WHOLEGRAPH_OPT_LAZY_ADAM, W>(p, vec4, stream); break;
    case WHOLEGRAPH_OPT_ADAGRAD: launch_merge_apply<WHOLEGRAPH_OPT_ADAGRAD, W>(p, vec4, stream); break;
    case WHOLEGRAPH_OPT_RMSPROP: launch_merge_apply<WHOLEGRAPH_OPT_RMSPROP, W>(p, vec4, stream); break;
    default: WGB_EXPECTS(false, "unknown optimizer type %d", (int)p.h.type);
  }
}

}  // namespace

size_t merged_apply_workspace_bytes(int world, int64_t local_rows, int64_t entries_upper_bound)
{
  return merge_layout_for(world, local_rows, entries_upper_bound).total;
}

void merged_apply(const merged_apply_args& a, void* workspace, cudaStream_t stream)
{
  const sparse_apply_args& sh = a.shard;
  WGB_EXPECTS(a.world >= 1 && a.world <= kMaxMergeRanks, "world size %d exceeds %d", a.world, kMaxMergeRanks);
  WGB_EXPECTS(a.status != nullptr, "merged apply needs a status word");
  WGB_EXPECTS(sh.local_rows < (int64_t(1) << 31) && static_cast<int64_t>(a.world) * ((sh.local_rows + 31) / 32) < (int64_t(1) << 31) - 2,
              "shard too large for the merge bitmaps");
  WGB_EXPECTS(sh.weight_cache.tags == nullptr && sh.state_cache.tags == nullptr, "merged apply does not go through caches");
  WGB_EXPECTS(sh.hyper.type == WHOLEGRAPH_OPT_SGD || sh.state != nullptr, "optimizer state is missing");
  WGB_EXPECTS(sh.hyper.type != WHOLEGRAPH_OPT_LAZY_ADAM || sh.beta12t != nullptr, "beta12t is missing");
  if (sh.local_rows == 0 || sh.dim == 0 || a.entries_upper_bound <= 0) return;
  const merge_layout l = merge_layout_for(a.world, sh.local_rows, a.entries_upper_bound);
  char* ws             = static_cast<char*>(workspace);
  merge_params p{};
  p.world = a.world, p.me = a.me, p.capacity = a.capacity;
  p.local_start = sh.local_start, p.local_rows = sh.local_rows;
  p.words      = l.words;
  p.bitmap     = reinterpret_cast<uint32_t*>(ws + l.bitmap);
  p.rank       = reinterpret_cast<int32_t*>(ws + l.rank);
  p.heads      = reinterpret_cast<int32_t*>(ws + l.heads);
  p.head_count = reinterpret_cast<int32_t*>(ws + l.counters);
  p.status     = a.status;
  p.dim = static_cast<int>(sh.dim), p.weights = sh.weights, p.weight_stride = sh.weight_stride;
  p.state = sh.state, p.state_stride = sh.state_stride, p.v_offset = sh.v_offset, p.beta12t = sh.beta12t;
  p.h = sh.hyper;
  for (int q = 0; q < a.world; q++) p.sender[q] = a.sender[q];
  // bitmaps and the head counter sit next to each other: one clear
  WGB_CUDA_CHECK(cudaMemsetAsync(ws + l.bitmap, 0, l.rank - l.bitmap, stream));
  const int64_t mark_ctas = std::min<int64_t>((a.entries_upper_bound + kThreads - 1) / kThreads, sm_count() * 16);
  merge_mark_kernel<<<static_cast<unsigned>(std::max<int64_t>(1, mark_ctas)), kThreads, 0, stream>>>(p);
  const size_t all_words = static_cast<size_t>(a.world) * static_cast<size_t>(l.words);
  auto counts = thrust::make_transform_iterator(thrust::counting_iterator<int>(0), popcount_of{p.bitmap});
  size_t cub_bytes = l.cub_bytes;
  // one entry past the bitmaps (the zeroed counter word) closes the last sender's prefix
  WGB_CUDA_CHECK(cub::DeviceScan::ExclusiveSum(ws + l.cub, cub_bytes, counts, p.rank, static_cast<int>(all_words + 1), stream));
  const int64_t head_ctas = std::min<int64_t>((l.words + kThreads - 1) / kThreads, sm_count() * 16);
  merge_heads_kernel<<<static_cast<unsigned>(std::max<int64_t>(1, head_ctas)), kThreads, 0, stream>>>(p);
  const size_t w_es = wholegraph_dtype_get_element_size(sh.weight_dtype);
  bool vec4 = sh.dim % 4 == 0 && sh.weight_stride % 4 == 0 && reinterpret_cast<uintptr_t>(sh.weights) % (4 * w_es) == 0 &&
              (sh.state == nullptr || (sh.state_stride % 4 == 0 && sh.v_offset % 4 == 0 &&
                                       reinterpret_cast<uintptr_t>(sh.state) % 16 == 0));
  for (int q = 0; q < a.world; q++) vec4 = vec4 && reinterpret_cast<uintptr_t>(a.sender[q].sums) % 16 == 0;
  if (sh.weight_dtype == WHOLEGRAPH_DT_FLOAT)
    launch_merge_apply_opt<float>(p, vec4, stream);
  else if (sh.weight_dtype == WHOLEGRAPH_DT_HALF)
    launch_merge_apply_opt<__half>(p, vec4, stream);
  else
    launch_merge_apply_opt<__nv_bfloat16>(p, vec4, stream);
  count_kernel_launch(4);
  WGB_LAUNCH_CHECK(stream);
}

void sparse_apply(const sparse_apply_args& a, void* workspace, cudaStream_t stream)
{
  if (a.count == 0 || a.dim == 0) return;
  WGB_EXPECTS(a.count < (int64_t(1) << 31), "gradient list of %ld rows is too long", (long)a.count);
  WGB_EXPECTS(a.local_rows < (int64_t(1) << 32) - 1, "shard of %ld rows is too large", (long)a.local_rows);
  WGB_EXPECTS(a.weight_dtype == WHOLEGRAPH_DT_FLOAT || a.weight_dtype == WHOLEGRAPH_DT_HALF ||
                a.weight_dtype == WHOLEGRAPH_DT_BF16,
              "only float, half and bf16 tables can be trained");
  WGB_EXPECTS(a.hyper.type == WHOLEGRAPH_OPT_SGD || a.hyper.type == WHOLEGRAPH_OPT_LAZY_ADAM ||
                a.hyper.type == WHOLEGRAPH_OPT_ADAGRAD || a.hyper.type == WHOLEGRAPH_OPT_RMSPROP,
              "unknown optimizer type %d", (int)a.hyper.type);
  WGB_EXPECTS(a.hyper.type == WHOLEGRAPH_OPT_SGD || a.state != nullptr, "optimizer state is missing");
  WGB_EXPECTS(a.hyper.type != WHOLEGRAPH_OPT_LAZY_ADAM || a.beta12t != nullptr, "beta12t is missing");
  const workspace_layout l = layout_for(a.count, a.local_rows, a.dim);
  apply_params p{};
  group_rows(a.ids, a.ids_are_64, a.count, a.local_start, a.local_rows, l, static_cast<char*>(workspace), stream, &p);
  p.grads = a.grads, p.grad_stride = a.grad_stride, p.dim = static_cast<int>(a.dim);
  p.weights = a.weights, p.weight_stride = a.weight_stride;
  p.state = a.state, p.state_stride = a.state_stride, p.v_offset = a.v_offset, p.beta12t = a.beta12t;
  p.h = a.hyper;
  p.weight_cache = a.weight_cache, p.state_cache = a.state_cache;
  const size_t w_es = wholegraph_dtype_get_element_size(a.weight_dtype);
  const bool vec4   = a.dim % 4 == 0 && a.grad_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(a.grads) % 16 == 0 && a.weight_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(a.weights) % (4 * w_es) == 0 &&
                    (a.state == nullptr || (a.state_stride % 4 == 0 && a.v_offset % 4 == 0 &&
                                            reinterpret_cast<uintptr_t>(a.state) % 16 == 0));
  const int ctas = apply_grid(a.count);
  if (a.weight_dtype == WHOLEGRAPH_DT_FLOAT)
    launch_apply_opt<float>(p, vec4, ctas, stream);
  else if (a.weight_dtype == WHOLEGRAPH_DT_HALF)
    launch_apply_opt<__half>(p, vec4, ctas, stream);
  else
    launch_apply_opt<__nv_bfloat16>(p, vec4, ctas, stream);
  count_kernel_launch(6);
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
