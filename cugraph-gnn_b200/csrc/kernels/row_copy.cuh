// Row copy kernel for sm_100a: gather, scatter and permutation reorder with a fused element
// cast.  One warp owns a tile of 32 list positions: it stages the 32 row ids (and output
// positions) in shared memory with one coalesced load, then walks the tile with several rows
// in flight per lane, every access a single vector of up to 16 bytes.
//
// Semantics follow the reference's gather_func_kernel / scatter_func_kernel
// (cpp/src/wholegraph_tensor_ops/functions/gather_scatter_func.cuh:242-365, :508-587): a
// negative row id skips the position, casts go through fp32 for fp16 / bf16
// (type_caster, :150-197), integer casts truncate.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "row_copy.hpp"

namespace wgb {

constexpr int kRowCopyWarps       = 8;                   // warps per CTA
constexpr int kRowCopyThreads     = kRowCopyWarps * 32;  // threads per CTA
constexpr int kRowCopyTile        = 32;                  // list positions per warp tile

struct row_copy_params {
  const char* src;  // first element of row 0 (storage offset already applied)
  char* dst;
  int64_t src_stride_bytes;
  int64_t dst_stride_bytes;
  const void* indices;
  const int64_t* positions;
  int64_t count;
  int vectors_per_row;  // ceil(dim / EPV)
  int lanes_per_row;    // power of two, 1..32
  int src_select;
  int dst_select;
  int indices_are_64;
  // CHUNKED tables: the BY_INDEX side ignores src / dst and resolves rows through `chunks`;
  // chunk_offset_bytes is that side's storage offset.
  int64_t chunk_offset_bytes;
  chunked_table chunks;
  list_segments segments;
};

// ---- raw vectors of 1..16 bytes ---------------------------------------------------------
template <int BYTES>
struct raw_vec;
template <>
struct raw_vec<1> {
  using type = unsigned char;
};
template <>
struct raw_vec<2> {
  using type = unsigned short;
};
template <>
struct raw_vec<4> {
  using type = unsigned int;
};
template <>
struct raw_vec<8> {
  using type = uint2;
};
template <>
struct raw_vec<16> {
  using type = uint4;
};

// Read-only, no reuse expected: non-coherent path.
template <int BYTES>
__device__ __forceinline__ typename raw_vec<BYTES>::type load_row_vector(const char* p)
{
  return __ldg(reinterpret_cast<const typename raw_vec<BYTES>::type*>(p));
}
template <int BYTES>
__device__ __forceinline__ void store_row_vector(char* p, typename raw_vec<BYTES>::type v)
{
  *reinterpret_cast<typename raw_vec<BYTES>::type*>(p) = v;
}

// ---- element conversion ----------------------------------------------------------------------
template <typename T>
struct wide_of {
  using type = T;
};
template <>
struct wide_of<__half> {
  using type = float;
};
template <>
struct wide_of<__nv_bfloat16> {
  using type = float;
};

template <typename From, typename To>
__device__ __forceinline__ To convert_element(From x)
{
  using wf = typename wide_of<From>::type;
  using wt = typename wide_of<To>::type;
  wf a     = static_cast<wf>(x);  // fp16 / bf16 widen to fp32 exactly
  wt b     = static_cast<wt>(a);  // fp64 -> fp32 rounds to nearest; integers truncate
  return static_cast<To>(b);      // fp32 -> fp16 / bf16 rounds to nearest even
}

// Two fp32 values to one packed fp16x2 / bf16x2 word, round to nearest even: the same result
// as two scalar casts, one instruction instead of two plus a pack.
__device__ __forceinline__ unsigned pack2(float a, float b, __half*)
{
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<unsigned*>(&h);
}
__device__ __forceinline__ unsigned pack2(float a, float b, __nv_bfloat16*)
{
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&h);
}

template <typename From, typename To, int EPV>
struct vector_cast {
  using in_raw  = typename raw_vec<sizeof(From) * EPV>::type;
  using out_raw = typename raw_vec<sizeof(To) * EPV>::type;
  static __device__ __forceinline__ out_raw apply(in_raw v)
  {
    union {
      in_raw raw;
      From e[EPV];
    } a;
    union {
      out_raw raw;
      To e[EPV];
    } b;
    a.raw = v;
    constexpr bool kPacked = (EPV % 2 == 0) && sizeof(typename wide_of<From>::type) == 4 &&
                             (sizeof(To) == 2) && (sizeof(typename wide_of<To>::type) == 4);
    if constexpr (kPacked) {
      // From widens to fp32, To is fp16 / bf16: convert pairs.
      union {
        out_raw raw;
        unsigned w[EPV / 2];
      } c;
#pragma unroll
      for (int i = 0; i < EPV / 2; i++)
        c.w[i] = pack2(static_cast<float>(a.e[2 * i]), static_cast<float>(a.e[2 * i + 1]),
                       static_cast<To*>(nullptr));
      return c.raw;
    } else {
#pragma unroll
      for (int i = 0; i < EPV; i++) b.e[i] = convert_element<From, To>(a.e[i]);
      return b.raw;
    }
  }
};

__device__ __forceinline__ const char* chunked_row(const chunked_table& t, int64_t row,
                                                   int64_t stride_bytes, int64_t offset_bytes)
{
  int r = t.ranks - 1;
  while (r > 0 && t.first_row[r] > row) r--;
  return static_cast<const char*>(t.base[r]) + (row - t.first_row[r]) * stride_bytes + offset_bytes;
}

// IN_BYTES / OUT_BYTES: bytes per vector on each side.  CAST::apply converts one vector.
// Row number on one side of the copy for tile row r.
__device__ __forceinline__ int64_t select_row(int select, int64_t id, int64_t pos, int64_t i)
{
  return select == ROW_BY_INDEX ? id : (select == ROW_BY_POSITION ? pos : i);
}

// ROWS: independent rows every lane keeps in flight per pass.  Addresses are recomputed from
// the staged ids at load and at store time instead of being carried in registers: the kernel
// stays within 64 registers, so 4 CTAs x 8 warps x ROWS rows are outstanding per SM, which is
// what random 256..512-byte rows need to cover HBM latency at full bandwidth.
template <int IN_BYTES, int OUT_BYTES, typename CAST, bool CHUNKED, int ROWS = 6>
__global__ void __launch_bounds__(kRowCopyThreads, 4)
  row_copy_kernel(const row_copy_params p)
{
  __shared__ int64_t s_index[kRowCopyWarps][kRowCopyTile];
  __shared__ int64_t s_position[kRowCopyWarps][kRowCopyTile];
  __shared__ int64_t s_list[kRowCopyWarps][kRowCopyTile];  // array position of each tile row

  const int lane          = threadIdx.x & 31;
  const int warp          = threadIdx.x >> 5;
  const int lpr           = p.lanes_per_row;
  const int sub           = lane / lpr;  // which row of a pass this lane works on
  const int col0          = lane % lpr;  // first vector of the row this lane moves
  const int rows_per_pass = 32 / lpr;
  const bool need_index   = p.src_select == ROW_BY_INDEX || p.dst_select == ROW_BY_INDEX;
  const bool need_pos     = p.src_select == ROW_BY_POSITION || p.dst_select == ROW_BY_POSITION;
  const bool src_chunked  = CHUNKED && p.src_select == ROW_BY_INDEX;
  const bool dst_chunked  = CHUNKED && p.dst_select == ROW_BY_INDEX;

  const int64_t tiles       = (p.count + kRowCopyTile - 1) / kRowCopyTile;
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * kRowCopyWarps + warp;
  const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kRowCopyWarps;

  for (int64_t tile = warp_global; tile < tiles; tile += warp_stride) {
    const int64_t base = tile * kRowCopyTile;
    {
      int64_t i   = base + lane;
      int64_t id  = -1;  // positions past the end behave like skipped rows
      int64_t pos = 0;
      if (i < p.count) {
        if (p.segments.n > 0) {  // logical -> array position
          int s = 0;
          while (s + 1 < p.segments.n && i >= p.segments.prefix[s + 1]) s++;
          i = p.segments.begin[s] + (i - p.segments.prefix[s]);
        }
        id = 0;
        if (need_index)
          id = p.indices_are_64 ? __ldg(static_cast<const int64_t*>(p.indices) + i)
                                : static_cast<int64_t>(__ldg(static_cast<const int*>(p.indices) + i));
        if (need_pos) pos = __ldg(p.positions + i);
      }
      s_index[warp][lane]    = id;
      s_position[warp][lane] = pos;
      s_list[warp][lane]     = i;
    }
    __syncwarp();

    for (int r0 = 0; r0 < kRowCopyTile; r0 += rows_per_pass * ROWS) {
      for (int c = col0; c < p.vectors_per_row; c += lpr) {
        typename raw_vec<IN_BYTES>::type v[ROWS];
        bool live[ROWS];
#pragma unroll
        for (int k = 0; k < ROWS; k++) {
          const int r = r0 + k * rows_per_pass + sub;
          live[k]     = false;
          if (r < kRowCopyTile) {
            const int64_t id = s_index[warp][r];
            live[k]          = id >= 0;
            if (live[k]) {
              const int64_t row = select_row(p.src_select, id, s_position[warp][r], s_list[warp][r]);
              const char* src   = src_chunked
                                    ? chunked_row(p.chunks, row, p.src_stride_bytes, p.chunk_offset_bytes)
                                    : p.src + row * p.src_stride_bytes;
              v[k] = load_row_vector<IN_BYTES>(src + static_cast<int64_t>(c) * IN_BYTES);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < ROWS; k++) {
          if (live[k]) {
            const int r       = r0 + k * rows_per_pass + sub;
            const int64_t row = select_row(p.dst_select, s_index[warp][r], s_position[warp][r], s_list[warp][r]);
            char* dst = dst_chunked ? const_cast<char*>(chunked_row(p.chunks, row, p.dst_stride_bytes,
                                                                    p.chunk_offset_bytes))
                                    : p.dst + row * p.dst_stride_bytes;
            store_row_vector<OUT_BYTES>(dst + static_cast<int64_t>(c) * OUT_BYTES, CAST::apply(v[k]));
          }
        }
      }
    }
    __syncwarp();
  }
}

// Identity "cast" for same-type copies.
template <int BYTES>
struct raw_copy {
  static __device__ __forceinline__ typename raw_vec<BYTES>::type apply(
    typename raw_vec<BYTES>::type v)
  {
    return v;
  }
};

using row_copy_kernel_fn = void (*)(const row_copy_params);

// Kernel for a (from, to, elements-per-vector) triple, or nullptr when the vector would
// exceed 16 bytes.  Defined in the per-family translation units.
row_copy_kernel_fn float_cast_kernel(wholegraph_dtype_t from, wholegraph_dtype_t to, int epv,
                                     bool chunked);
row_copy_kernel_fn int_cast_kernel(wholegraph_dtype_t from, wholegraph_dtype_t to, int epv,
                                   bool chunked);
row_copy_kernel_fn same_type_kernel(int vector_bytes, bool chunked);

}  // namespace wgb
