// Sparse SGD / Lazy Adam / AdaGrad / RMSProp apply fused with duplicate-gradient reduction.
//
//   1. keys_kernel        local row id (or a sentinel) and list position per gradient row
//   2. cub radix sort     (key, position) pairs, only the bits a local row id can use; stable, so
//                         equal ids keep their arrival order
//   3. cub select         first element of every run of equal keys, in order (run r ends where
//                         run r + 1 starts)
//   4. apply_kernel       one warp per distinct row: walks its run, adds the gradient rows in
//                         arrival order (fp32, 16-byte loads, 4 rows in flight), then reads
//                         weights and state once, updates them and writes them back
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
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include "../common.hpp"
#include "row_copy.hpp"

namespace wgb {

namespace {

constexpr int kThreads    = 256;
constexpr int kDedupBlock = WHOLEGRAPH_B200_DEDUP_BLOCK;  // rows per block of a long duplicate run
constexpr int kRowsInFlight = 8;  // gradient rows a lane requests before it starts adding

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
  int32_t* long_count;    // number of long runs
  int32_t* slot_count;    // number of partial-sum slots handed out
  int32_t* slot_run;      // per slot: long run it belongs to
  int32_t* slot_block;    // per slot: block number inside the run
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

// Sum of the gradient rows of sorted elements [first, last) for columns [c, c + VEC), added one
// after the other in that order; kRowsInFlight rows are requested before the first is added.
template <int VEC>
__device__ __forceinline__ void sum_rows(const apply_params& p, int64_t first, int64_t last, int c,
                                         float (&acc)[VEC])
{
  {
    const float* g0 = p.grads + static_cast<int64_t>(p.positions[first]) * p.grad_stride + c;
    if constexpr (VEC == 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(g0));
      acc[0] = v.x, acc[1] = v.y, acc[2] = v.z, acc[3] = v.w;
    } else {
      acc[0] = __ldg(g0);
    }
  }
  for (int64_t k = first + 1; k < last; k += kRowsInFlight) {
    float v[kRowsInFlight][VEC];
    bool on[kRowsInFlight];
#pragma unroll
    for (int u = 0; u < kRowsInFlight; u++) {
      on[u] = k + u < last;
      if (on[u]) {
        const float* g = p.grads + static_cast<int64_t>(p.positions[k + u]) * p.grad_stride + c;
        if constexpr (VEC == 4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(g));
          v[u][0] = t.x, v[u][1] = t.y, v[u][2] = t.z, v[u][3] = t.w;
        } else {
          v[u][0] = __ldg(g);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kRowsInFlight; u++) {
      if (on[u]) {
#pragma unroll
        for (int e = 0; e < VEC; e++) acc[e] = __fadd_rn(acc[e], v[u][e]);
      }
    }
  }
}

// Read-modify-write of weights and state for columns [c, c + VEC) of one row.
template <int OPT, typename W, int VEC>
__device__ __forceinline__ void update_columns(const apply_params& p, W* w_row, float* s_row, int c,
                                               const float (&acc)[VEC], float beta1t, float beta2t)
{
  float w[VEC], s0[VEC], s1[VEC];
  load_vec<W, VEC>(w_row + c, w);
  if (OPT != WHOLEGRAPH_OPT_SGD) load_vec<float, VEC>(s_row + c, s0);
  if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) load_vec<float, VEC>(s_row + p.v_offset + c, s1);
#pragma unroll
  for (int e = 0; e < VEC; e++) update_element<OPT>(p.h, acc[e], w[e], s0[e], s1[e], beta1t, beta2t);
  if (OPT != WHOLEGRAPH_OPT_SGD) store_vec<float, VEC>(s_row + c, s0);
  if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) store_vec<float, VEC>(s_row + p.v_offset + c, s1);
  store_vec<W, VEC>(w_row + c, w);
}

// Per-row running beta1^t, beta2^t of Lazy Adam: multiplied on every touch of the row.
template <int OPT>
__device__ __forceinline__ void step_betas(const apply_params& p, uint32_t row, int lane, float& beta1t,
                                           float& beta2t)
{
  beta1t = beta2t = 0.f;
  if (OPT == WHOLEGRAPH_OPT_LAZY_ADAM) {
    beta1t = __fmul_rn(p.beta12t[static_cast<int64_t>(row) * 2 + 0], p.h.beta1);
    beta2t = __fmul_rn(p.beta12t[static_cast<int64_t>(row) * 2 + 1], p.h.beta2);
    __syncwarp();  // every lane has read the old values before lane 0 overwrites them
    if (lane == 0) {
      p.beta12t[static_cast<int64_t>(row) * 2 + 0] = beta1t;
      p.beta12t[static_cast<int64_t>(row) * 2 + 1] = beta2t;
    }
  }
}

// One warp per distinct row.  Runs of up to kDedupBlock duplicates are summed and applied here;
// longer runs are only registered, with one partial-sum slot per block of kDedupBlock rows.
// VEC = 4: dim, strides and base pointers allow 16-byte accesses; VEC = 1 otherwise.
template <int OPT, typename W, int VEC>
__global__ void __launch_bounds__(kThreads) apply_kernel(const apply_params p)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int runs            = *p.head_count;
  W* weights                = static_cast<W*>(p.weights);

  for (int64_t run = warp_global; run < runs; run += warp_stride) {
    // Heads are in sorted order, so a run ends where the next one starts.
    const int64_t first = p.heads[run];
    const int64_t last  = run + 1 < runs ? p.heads[run + 1] : p.n;
    const uint32_t row  = p.keys[first];
    if (row == p.sentinel) continue;  // ids this rank does not own sort last
    const int64_t len = last - first;
    if (len > kDedupBlock) {
      const int blocks = static_cast<int>((len + kDedupBlock - 1) / kDedupBlock);
      int li = 0, slot = 0;
      if (lane == 0) {
        li               = atomicAdd(p.long_count, 1);
        slot             = atomicAdd(p.slot_count, blocks);
        p.long_first[li] = static_cast<int32_t>(first);
        p.long_len[li]   = static_cast<int32_t>(len);
        p.long_slot[li]  = slot;
      }
      li   = __shfl_sync(0xffffffffu, li, 0);
      slot = __shfl_sync(0xffffffffu, slot, 0);
      for (int b = lane; b < blocks; b += 32) {
        p.slot_run[slot + b]   = li;
        p.slot_block[slot + b] = b;
      }
      continue;
    }
    float beta1t, beta2t;
    step_betas<OPT>(p, row, lane, beta1t, beta2t);
    W* w_row     = weights + static_cast<int64_t>(row) * p.weight_stride;
    float* s_row = p.state != nullptr ? p.state + static_cast<int64_t>(row) * p.state_stride : nullptr;
    w_row        = reinterpret_cast<W*>(current_copy(p.weight_cache, row, lane, reinterpret_cast<char*>(w_row)));
    if (s_row != nullptr)
      s_row = reinterpret_cast<float*>(current_copy(p.state_cache, row, lane, reinterpret_cast<char*>(s_row)));
    for (int c = lane * VEC; c < p.dim; c += 32 * VEC) {
      float acc[VEC];
      sum_rows<VEC>(p, first, last, c, acc);
      update_columns<OPT, W, VEC>(p, w_row, s_row, c, acc, beta1t, beta2t);
    }
  }
}

// One warp per partial-sum slot: block b of a long run, rows [b * kDedupBlock, (b + 1) * kDedupBlock)
// of the run, added in order.
template <int VEC>
__global__ void __launch_bounds__(kThreads) sum_blocks_kernel(const apply_params p)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int slots           = *p.slot_count;
  for (int64_t s = warp_global; s < slots; s += warp_stride) {
    const int li        = p.slot_run[s];
    const int64_t begin = p.long_first[li];
    const int64_t end   = begin + p.long_len[li];
    const int64_t first = begin + static_cast<int64_t>(p.slot_block[s]) * kDedupBlock;
    const int64_t last  = first + kDedupBlock < end ? first + kDedupBlock : end;
    float* out          = p.partial + s * p.dim;
    for (int c = lane * VEC; c < p.dim; c += 32 * VEC) {
      float acc[VEC];
      sum_rows<VEC>(p, first, last, c, acc);
#pragma unroll
      for (int e = 0; e < VEC; e++) out[c + e] = acc[e];
    }
  }
}

// One warp per long run: adds its block sums in block order and applies the optimizer.
template <int OPT, typename W, int VEC>
__global__ void __launch_bounds__(kThreads) apply_long_kernel(const apply_params p)
{
  const int lane            = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warp_stride = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int runs            = *p.long_count;
  W* weights                = static_cast<W*>(p.weights);
  for (int64_t li = warp_global; li < runs; li += warp_stride) {
    const uint32_t row = p.keys[p.long_first[li]];
    const int blocks   = (p.long_len[li] + kDedupBlock - 1) / kDedupBlock;
    const float* part  = p.partial + static_cast<int64_t>(p.long_slot[li]) * p.dim;
    float beta1t, beta2t;
    step_betas<OPT>(p, row, lane, beta1t, beta2t);
    W* w_row     = weights + static_cast<int64_t>(row) * p.weight_stride;
    float* s_row = p.state != nullptr ? p.state + static_cast<int64_t>(row) * p.state_stride : nullptr;
    w_row        = reinterpret_cast<W*>(current_copy(p.weight_cache, row, lane, reinterpret_cast<char*>(w_row)));
    if (s_row != nullptr)
      s_row = reinterpret_cast<float*>(current_copy(p.state_cache, row, lane, reinterpret_cast<char*>(s_row)));
    for (int c = lane * VEC; c < p.dim; c += 32 * VEC) {
      float acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e++) acc[e] = part[c + e];
      for (int b = 1; b < blocks; b += kRowsInFlight) {
        float v[kRowsInFlight][VEC];
#pragma unroll
        for (int u = 0; u < kRowsInFlight; u++) {
          if (b + u < blocks) {
#pragma unroll
            for (int e = 0; e < VEC; e++) v[u][e] = part[static_cast<int64_t>(b + u) * p.dim + c + e];
          }
        }
#pragma unroll
        for (int u = 0; u < kRowsInFlight; u++) {
          if (b + u < blocks) {
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[e] = __fadd_rn(acc[e], v[u][e]);
          }
        }
      }
      update_columns<OPT, W, VEC>(p, w_row, s_row, c, acc, beta1t, beta2t);
    }
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
  size_t long_first, long_len, long_slot, slot_run, slot_block, partial;
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
  l.counters       = off, off += 256;  // head count, long-run count, slot count
  // At most n / block runs are long, and they need at most n / block + (their number) slots.
  const size_t max_long  = cnt / kDedupBlock + 1;
  const size_t max_slots = 2 * max_long;
  l.long_first = off, off += align(max_long * 4);
  l.long_len   = off, off += align(max_long * 4);
  l.long_slot  = off, off += align(max_long * 4);
  l.slot_run   = off, off += align(max_slots * 4);
  l.slot_block = off, off += align(max_slots * 4);
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

template <int OPT, typename W>
void launch_apply(const apply_params& p, bool vec4, int ctas, cudaStream_t stream)
{
  // Long runs are rare and their number is only known on the device: fixed modest grids.
  const int long_ctas = std::min(ctas, 148 * 4);
  if (vec4) {
    apply_kernel<OPT, W, 4><<<ctas, kThreads, 0, stream>>>(p);
    sum_blocks_kernel<4><<<long_ctas, kThreads, 0, stream>>>(p);
    apply_long_kernel<OPT, W, 4><<<long_ctas, kThreads, 0, stream>>>(p);
  } else {
    apply_kernel<OPT, W, 1><<<ctas, kThreads, 0, stream>>>(p);
    sum_blocks_kernel<1><<<long_ctas, kThreads, 0, stream>>>(p);
    apply_long_kernel<OPT, W, 1><<<long_ctas, kThreads, 0, stream>>>(p);
  }
}

template <typename W>
void launch_apply_opt(const apply_params& p, bool vec4, int ctas, cudaStream_t stream)
{
  switch (p.h.type) {
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

void sparse_apply(const sparse_apply_args& a, void* workspace, cudaStream_t stream)
{
  if (a.count == 0 || a.dim == 0) return;
  WGB_EXPECTS(a.count < (int64_t(1) << 31), "gradient list of %ld rows is too long", (long)a.count);
  WGB_EXPECTS(a.local_rows < (int64_t(1) << 32) - 1, "shard of %ld rows is too large", (long)a.local_rows);
  WGB_EXPECTS(a.weight_dtype == WHOLEGRAPH_DT_FLOAT || a.weight_dtype == WHOLEGRAPH_DT_HALF ||
                a.weight_dtype == WHOLEGRAPH_DT_BF16,
              "only float, half and bf16 tables can be trained");
  WGB_EXPECTS(a.hyper.type == WHOLEGRAPH_OPT_SGD || a.state != nullptr, "optimizer state is missing");
  WGB_EXPECTS(a.hyper.type != WHOLEGRAPH_OPT_LAZY_ADAM || a.beta12t != nullptr, "beta12t is missing");
  const workspace_layout l = layout_for(a.count, a.local_rows, a.dim);
  char* ws                 = static_cast<char*>(workspace);
  auto* keys_in            = reinterpret_cast<uint32_t*>(ws + l.keys_in);
  auto* keys_out           = reinterpret_cast<uint32_t*>(ws + l.keys_out);
  auto* pos_in             = reinterpret_cast<int32_t*>(ws + l.pos_in);
  auto* pos_out            = reinterpret_cast<int32_t*>(ws + l.pos_out);
  auto* heads              = reinterpret_cast<int32_t*>(ws + l.heads);
  auto* counters           = reinterpret_cast<int32_t*>(ws + l.counters);
  auto* head_count         = counters;
  const unsigned blocks    = static_cast<unsigned>((a.count + kThreads - 1) / kThreads);

  keys_kernel<<<blocks, kThreads, 0, stream>>>(a.ids, a.ids_are_64 ? 1 : 0, a.count, a.local_start, a.local_rows,
                                               keys_in, pos_in);
  size_t cub_bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(ws + l.cub, cub_bytes, keys_in, keys_out, pos_in, pos_out,
                                                 static_cast<int>(a.count), 0, key_bits(a.local_rows),
                                                 stream));
  WGB_CUDA_CHECK(cudaMemsetAsync(counters, 0, 3 * sizeof(int32_t), stream));
  size_t select_bytes = l.cub_bytes;
  WGB_CUDA_CHECK(cub::DeviceSelect::If(ws + l.cub, select_bytes, thrust::counting_iterator<int>(0), heads,
                                       head_count, static_cast<int>(a.count), is_run_head{keys_out}, stream));

  apply_params p;
  p.keys = keys_out, p.positions = pos_out, p.heads = heads, p.head_count = head_count, p.n = a.count;
  p.sentinel = static_cast<uint32_t>(a.local_rows);
  p.grads = a.grads, p.grad_stride = a.grad_stride, p.dim = static_cast<int>(a.dim);
  p.weights = a.weights, p.weight_stride = a.weight_stride;
  p.state = a.state, p.state_stride = a.state_stride, p.v_offset = a.v_offset, p.beta12t = a.beta12t;
  p.h = a.hyper;
  p.weight_cache = a.weight_cache, p.state_cache = a.state_cache;
  p.long_count = counters + 1, p.slot_count = counters + 2;
  p.long_first = reinterpret_cast<int32_t*>(ws + l.long_first);
  p.long_len   = reinterpret_cast<int32_t*>(ws + l.long_len);
  p.long_slot  = reinterpret_cast<int32_t*>(ws + l.long_slot);
  p.slot_run   = reinterpret_cast<int32_t*>(ws + l.slot_run);
  p.slot_block = reinterpret_cast<int32_t*>(ws + l.slot_block);
  p.partial    = reinterpret_cast<float*>(ws + l.partial);
  const size_t w_es = wholegraph_dtype_get_element_size(a.weight_dtype);
  const bool vec4   = a.dim % 4 == 0 && a.grad_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(a.grads) % 16 == 0 && a.weight_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(a.weights) % (4 * w_es) == 0 &&
                    (a.state == nullptr || (a.state_stride % 4 == 0 && a.v_offset % 4 == 0 &&
                                            reinterpret_cast<uintptr_t>(a.state) % 16 == 0));
  static int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  // One warp per distinct row, grid-stride; the number of rows is only known on the device.
  const int64_t warps_wanted = a.count;
  int ctas = static_cast<int>(std::min<int64_t>((warps_wanted + 7) / 8, static_cast<int64_t>(sm_count) * 8 * 4));
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
