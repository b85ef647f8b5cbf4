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
  int tile_rows;  // bulk kernel: rows per tile
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
  const int64_t tiles       = (total + kTile - 1) / kTile;
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kWarps;

  for (int64_t tile = warp_global; tile < tiles; tile += warp_stride) {
    {
      const int64_t i  = tile * kTile + lane;
      const bool valid = i < total;
      int k            = 0;
      if (valid)
        while (k + 1 < p.world && i >= s_prefix[k + 1]) k++;
      const int64_t in_group = i - s_prefix[k];
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


// ---- bulk-copy form -----------------------------------------------------------------------------
// The same service with the copy engines of the SM doing the moving.  A warp owns kBulkStages
// buffers of shared memory.  For a tile of consecutive slots of ONE requester its lanes issue one
// bulk asynchronous load per row (local shard -> shared memory, completion counted in bytes by an
// mbarrier) and, one tile later, ONE bulk store of the whole tile into the requester's region: up
// to 8 KiB of contiguous peer memory per store instead of 512 bytes per warp instruction, no row
// data in registers.  Every wait has a limit; when one runs out the kernel reports it through the
// status word, drains what it has in flight (again with a limit) and returns.
constexpr int kBulkWarps      = 4;
constexpr int kBulkThreads    = kBulkWarps * 32;
constexpr int kBulkStages     = 3;
constexpr int kBulkStageBytes = 8192;
constexpr unsigned kBulkSpins = 1u << 20;  // polls of an mbarrier before giving up (each poll may sleep in hardware)

__device__ __forceinline__ uint32_t shared_address(const void* p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, int arrivals)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbarrier_expect_bytes(uint64_t* bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarrier_poll(uint64_t* bar, uint32_t parity)
{
  uint32_t done;
  asm volatile(
    "{\n"
    ".reg .pred p;\n"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
    "selp.u32 %0, 1, 0, p;\n"
    "}\n"
    : "=r"(done)
    : "r"(shared_address(bar)), "r"(parity)
    : "memory");
  return done != 0;
}
// false: the limit ran out
__device__ __forceinline__ bool mbarrier_wait_bounded(uint64_t* bar, uint32_t parity)
{
  for (unsigned spin = 0; spin < kBulkSpins; spin++)
    if (mbarrier_poll(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_load_row(void* shared_dst, const void* global_src, uint32_t bytes, uint64_t* bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                 shared_address(shared_dst)),
               "l"(__cvta_generic_to_global(global_src)), "r"(bytes), "r"(shared_address(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_tile(void* global_dst, const void* shared_src, uint32_t bytes)
{
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(global_dst)),
               "r"(shared_address(shared_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_sources_read()
{
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }


__global__ void __launch_bounds__(kBulkThreads, 2) serve_rows_bulk_kernel(const serve_params p)
{
  extern __shared__ __align__(128) char s_stage[];  // [warp][stage][kBulkStageBytes]
  __shared__ uint64_t s_bar[kBulkWarps][kBulkStages];
  __shared__ int64_t s_tiles[kMaxServeRanks + 1];  // tiles of the first k requesters (rotation order)
  __shared__ int64_t s_count[kMaxServeRanks];
  __shared__ int64_t s_start[kMaxServeRanks];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int T    = p.tile_rows;
  if (threadIdx.x < p.world) {
    const int q         = (p.me + 1 + threadIdx.x) % p.world;
    const int64_t* h    = p.region[q].header;
    int64_t count       = __ldcg(h + p.me);
    const int64_t start = __ldcg(h + p.world + p.me);
    if (count < 0 || start < 0 || start + count > p.capacity) {
      atomicExch(p.status, 1);
      count = 0;
    }
    s_start[threadIdx.x]     = start;
    s_count[threadIdx.x]     = count;
    s_tiles[threadIdx.x + 1] = (count + T - 1) / T;
  }
  if (lane == 0)
    for (int st = 0; st < kBulkStages; st++) mbarrier_init(&s_bar[warp][st], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0) {
    s_tiles[0] = 0;
    for (int k = 0; k < p.world; k++) s_tiles[k + 1] += s_tiles[k];
  }
  __syncthreads();
  const int64_t tiles       = s_tiles[p.world];
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * kBulkWarps + warp;
  const int64_t warp_stride = static_cast<int64_t>(gridDim.x) * kBulkWarps;
  const uint32_t row_bytes  = static_cast<uint32_t>(p.row_bytes);
  char* my_stage            = s_stage + static_cast<size_t>(warp) * kBulkStages * kBulkStageBytes;
  constexpr unsigned kFull  = 0xffffffffu;

  // A tile of this warp: which requester, which slots, and (per lane) the local row behind a slot.
  auto describe = [&](int64_t tile, int& rows, char*& dst, int64_t& row) {
    int k = 0;
    while (k + 1 < p.world && tile >= s_tiles[k + 1]) k++;
    const int q         = (p.me + 1 + k) % p.world;
    const int64_t first = (tile - s_tiles[k]) * T;  // position in the requester's group
    rows                = static_cast<int>(min(static_cast<int64_t>(T), s_count[k] - first));
    const int64_t j     = s_start[k] + first;
    dst                 = p.region[q].rows + j * p.row_bytes;
    row                 = -1;
    if (lane < rows) {
      row = __ldcg(p.region[q].ids + j + lane) - p.first_local_row;
      if (row < 0 || row >= p.local_rows) {  // not a row of this shard: never dereferenced
        atomicExch(p.status, 2);
        row = -1;
      }
    }
  };
  // The rows of the tile loaded one iteration ago are in shared memory: send them.
  auto send = [&](int it, int rows, char* dst, unsigned present) -> bool {
    const int st = it % kBulkStages;
    char* buf    = my_stage + static_cast<size_t>(st) * kBulkStageBytes;
    // the warp stays together: one lane out of patience ends the walk for all of them
    if (!__all_sync(kFull, mbarrier_wait_bounded(&s_bar[warp][st], (it / kBulkStages) & 1))) {
      atomicExch(p.status, 3);
      return false;
    }
    // A tile with an id that is not this shard's is not sent at all: the status word already says
    // so and the requester's next call fails with it.
    const unsigned whole = rows >= 32 ? kFull : ((1u << rows) - 1u);
    if (lane == 0) {
      if (present == whole) bulk_store_tile(dst, buf, static_cast<uint32_t>(rows) * row_bytes);
      bulk_commit();  // one group per tile, sent or not, so that the buffer bookkeeping stays uniform
    }
    return true;
  };

  int it = 0, prev_rows = 0;
  char* prev_dst        = nullptr;
  unsigned prev_present = 0u;
  bool alive            = true;
  int in_flight         = -1;  // tile whose loads are under way when the loop is left early
  for (int64_t tile = warp_global; tile < tiles; tile += warp_stride, it++) {
    const int st = it % kBulkStages;
    // the store that last read this buffer (two tiles ago in issue order) has read it
    if (it >= kBulkStages && lane == 0) bulk_wait_sources_read<1>();
    __syncwarp();
    int rows;
    char* dst;
    int64_t row;
    describe(tile, rows, dst, row);
    const unsigned present = __ballot_sync(kFull, row >= 0);
    // one arrival per use of the buffer (a tile without a valid row expects no bytes and completes at once)
    if (lane == 0) mbarrier_expect_bytes(&s_bar[warp][st], static_cast<uint32_t>(__popc(present)) * row_bytes);
    __syncwarp();
    if (row >= 0)
      bulk_load_row(my_stage + static_cast<size_t>(st) * kBulkStageBytes + static_cast<size_t>(lane) * row_bytes,
                    p.shard + row * p.shard_stride_bytes, row_bytes, &s_bar[warp][st]);
    if (it > 0 && !send(it - 1, prev_rows, prev_dst, prev_present)) {
      alive   = false;
      in_flight = it;  // this tile's loads were issued
      break;
    }
    prev_rows = rows, prev_dst = dst, prev_present = present;
  }
  if (alive && it > 0) alive = send(it - 1, prev_rows, prev_dst, prev_present);
  // Loads may still be on their way into this warp's buffers: give them the same limit once more
  // before the shared memory goes away.
  if (in_flight >= 0) mbarrier_wait_bounded(&s_bar[warp][in_flight % kBulkStages], (in_flight / kBulkStages) & 1);
  if (lane == 0) bulk_wait_all();
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
  p.tile_rows = kTile;
  for (int r = 0; r < a.world; r++) p.region[r] = a.region[r];

  static int sm_count = [] {
    int dev = 0, n = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
  }();
  if (a.bulk && bytes == 16 && a.row_bytes >= 128 && a.row_bytes <= kBulkStageBytes) {
    // One resident wave of CTAs, every warp walking its tiles with its own three buffers.
    p.tile_rows = static_cast<int>(std::min<int64_t>(32, kBulkStageBytes / a.row_bytes));
    constexpr size_t smem = static_cast<size_t>(kBulkWarps) * kBulkStages * kBulkStageBytes;
    // per device, so set on every launch (a process may drive more than one GPU)
    WGB_CUDA_CHECK(cudaFuncSetAttribute(serve_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    const int64_t tiles = a.rows_upper_bound / p.tile_rows + a.world;
    const int64_t ctas  = std::max<int64_t>(1, std::min<int64_t>((tiles + kBulkWarps - 1) / kBulkWarps,
                                                                  static_cast<int64_t>(sm_count) * 2));
    serve_rows_bulk_kernel<<<static_cast<unsigned>(ctas), kBulkThreads, smem, stream>>>(p);
    count_kernel_launch();
    WGB_LAUNCH_CHECK(stream);
    return;
  }
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
