// Stand-in for the RAFT warp-sort header so that the reference's cache header parses.  The
// class below only has the interface the reference names; it is never executed here (the
// cross-check uses the non-cached optimizer kernels only).
#pragma once
namespace raft {
__device__ inline int laneId() { return threadIdx.x & 31; }
namespace matrix::detail::select::warpsort {
template <int Capacity, bool Ascending, typename T, typename IdxT>
class warp_sort_immediate {
 public:
  __device__ explicit warp_sort_immediate(int) {}
  __device__ void add(T, IdxT) {}
  __device__ void done() {}
  __device__ void store(T*, IdxT*) {}
};
}  // namespace matrix::detail::select::warpsort
}  // namespace raft
