// Owner side of a distributed gather without host-side counts.
//
// The reference learns on the host how many ids every rank sends to every other rank (a device
// to host copy, a stream synchronisation and a host alltoall, exchange_ids_nccl_func.cu:183-191)
// because NCCL's send / recv need host sizes.  Here the requesters leave their counts and ids in
// a peer-mapped arena and the owner's kernel reads them itself: the grid is sized from an upper
// bound, the real sizes are device data.  Rows are raw byte vectors of up to 16 bytes (the cast
// to the output dtype happens where the requester expands the rows into its output).
#include "serve_rows.hpp"

#include <algorithm>

#include "../common.hpp"
#include "row_copy.cuh"

namespace wgb {

namespace {

constexpr int kWarps   = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kTile    = 32;
constexpr int kRows    = 6;  // rows every lane keeps in flight

struct serve_params {
  int world, me;
  int vectors_per_row, lanes_per_row;
  int64_t capacity;
  const char* shard;
  int64_t first_local_row, local_rows;
  int64_t shard_stride_bytes, row_bytes;
  int interleave;
  int* status;
  serve_region region[kMaxServeRanks];
};

template <int BYTES>
__global__ void __launch_bounds__(kThreads, 4) serve_rows_kernel(const serve_params p)
{
  __shared__ int64_t s_prefix[kMaxServeRanks + 1];  // rows asked by the first k requesters (rotation order)
  __shared__ int64_t s_start[kMaxServeRanks];
  __shared__ int64_t s_id[kWarps][kTile];            // local row, or -1
  __shared__ char* s_dst[kWarps][kTile];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Requester k of the rotation is rank (me + 1 + k) % world: at any moment the owners write to
  // different requesters, and a rank's own rows (a local copy) come last.
  if (threadIdx.x < p.world) {
    const int q          = (p.me + 1 + threadIdx.x) % p.world;
    const int64_t* h     = p.region[q].header;
    int64_t count        = __ldcg(h + p.me);
    const int64_t start  = __ldcg(h + p.world + p.me);
    if (count < 0 || start < 0 || start + count > p.capacity) {
      atomicExch(p.status, 1);
      count = 0;
    }
    s_start[threadIdx.x]      = start;
    s_prefix[threadIdx.x + 1] = count;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_prefix[0] = 0;
    for (int k = 0; k < p.world; k++) s_prefix[k + 1] += s_prefix[k];
  }
  __syncthreads();
  const int64_t total = s_prefix[p.world];

  const int lpr           = p.lanes_per_row;
  const int sub           = lane / lpr;
  const int col0          = lane % lpr;
  const int rows_per_pass = 32 / lpr;
  // Order of the tiles.  Rotation: requester after requester.  Interleaved: tile u of requester k
  // is unit u * world + k, so at every moment an owner's stores spread evenly over all requesters
  // (and every requester receives from all owners at once), whatever the skew between the ranks.
  int64_t tiles = (total + kTile - 1) / kTile;
  if (p.interleave) {
    int64_t longest = 0;
    for (int k = 0; k < p.world; k++) longest = max(longest, s_prefix[k + 1] - s_prefix[k]);
    tiles = (longest + kTile - 1) / kTile * p.world;
  }
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kWarps;

  for (int64_t tile = warp_global; tile < tiles; tile += warp_stride) {
    {
      int k = 0;
      int64_t in_group;  // position within requester k's group
      bool valid;
      if (p.interleave) {
        k        = static_cast<int>(tile % p.world);
        in_group = tile / p.world * kTile + lane;
        valid    = in_group < s_prefix[k + 1] - s_prefix[k];
        if (!__any_sync(0xffffffffu, valid)) continue;
      } else {
        const int64_t i = tile * kTile + lane;
        valid           = i < total;
        if (valid)
          while (k + 1 < p.world && i >= s_prefix[k + 1]) k++;
        in_group = i - s_prefix[k];
      }
      int64_t row = -1;
      char* dst   = nullptr;
      if (valid) {
        const int q      = (p.me + 1 + k) % p.world;
        const int64_t j  = s_start[k] + in_group;
        const int64_t id = __ldcg(p.region[q].ids + j);
        row              = id - p.first_local_row;
        if (row < 0 || row >= p.local_rows) {  // not a row of this shard: never dereferenced
          atomicExch(p.status, 2);
          row = -1;
        }
        dst = p.region[q].rows + j * p.row_bytes;
      }
      s_id[warp][lane]  = row;
      s_dst[warp][lane] = dst;
    }
    __syncwarp();
    for (int r0 = 0; r0 < kTile; r0 += rows_per_pass * kRows) {
      for (int c = col0; c < p.vectors_per_row; c += lpr) {
        typename raw_vec<BYTES>::type v[kRows];
        bool live[kRows];
#pragma unroll
        for (int k = 0; k < kRows; k++) {
          const int r = r0 + k * rows_per_pass + sub;
          live[k]     = false;
          if (r < kTile) {
            const int64_t row = s_id[warp][r];
            live[k]           = row >= 0;
            if (live[k])
              v[k] = load_row_vector<BYTES>(p.shard + row * p.shard_stride_bytes + static_cast<int64_t>(c) * BYTES);
          }
        }
#pragma unroll
        for (int k = 0; k < kRows; k++) {
          if (live[k]) {
            const int r = r0 + k * rows_per_pass + sub;
            store_row_vector<BYTES>(s_dst[warp][r] + static_cast<int64_t>(c) * BYTES, v[k]);
          }
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace

void launch_serve_rows(const serve_rows_args& a, cudaStream_t stream)
{
  WGB_EXPECTS(a.world >= 1 && a.world <= kMaxServeRanks, "world size %d exceeds %d", a.world, kMaxServeRanks);
  WGB_EXPECTS(a.status != nullptr && (a.shard != nullptr || a.local_rows == 0), "incomplete serve arguments");
  if (a.rows_upper_bound <= 0 || a.row_bytes <= 0) return;
  // Widest vector that divides the row, the shard's stride and both first addresses.
  int bytes = 16;
  auto fits = [&](int b) {
    if (a.row_bytes % b != 0 || a.shard_stride_bytes % b != 0) return false;
    if (reinterpret_cast<uintptr_t>(a.shard) % b != 0) return false;
    for (int r = 0; r < a.world; r++)
      if (reinterpret_cast<uintptr_t>(a.region[r].rows) % b != 0) return false;
    return true;
  };
  while (bytes > 1 && !fits(bytes)) bytes /= 2;

  serve_params p;
  p.world = a.world, p.me = a.me;
  p.vectors_per_row = static_cast<int>(a.row_bytes / bytes);
  int lpr           = 1;
  while (lpr < 32 && lpr < p.vectors_per_row) lpr *= 2;
  p.lanes_per_row = lpr;
  p.capacity      = a.capacity;
  p.shard         = static_cast<const char*>(a.shard);
  p.first_local_row = a.first_local_row, p.local_rows = a.local_rows;
  p.shard_stride_bytes = a.shard_stride_bytes, p.row_bytes = a.row_bytes;
  p.status = a.status;
  p.interleave = a.interleave ? 1 : 0;
  for (int r = 0; r < a.world; r++) p.region[r] = a.region[r];

  static int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  // The real number of rows is device data; the grid covers the bound, a few waves at most, and
  // warps without a tile leave at once.
  const int64_t tiles = (a.rows_upper_bound + kTile - 1) / kTile;
  int64_t ctas        = (tiles + kWarps - 1) / kWarps;
  ctas                = std::max<int64_t>(1, std::min<int64_t>(ctas, static_cast<int64_t>(sm_count) * 4 * 8));
  switch (bytes) {
    case 16: serve_rows_kernel<16><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p); break;
    case 8: serve_rows_kernel<8><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p); break;
    case 4: serve_rows_kernel<4><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p); break;
    case 2: serve_rows_kernel<2><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p); break;
    default: serve_rows_kernel<1><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p); break;
  }
  count_kernel_launch();
  WGB_LAUNCH_CHECK(stream);
}

}  // namespace wgb
