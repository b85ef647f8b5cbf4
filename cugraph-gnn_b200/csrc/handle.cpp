#include "handle.hpp"

#include <cuda.h>
#include <fcntl.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <memory>
#include <string>

#include "common.hpp"

// What backs one handle on this rank.
struct wholegraph_handle_::backing {
  enum kind_t { NONE, CUDA_MALLOC, CUDA_HOST, VMM, SHM, IPC } kind = NONE;
  void* alloc_ptr = nullptr;  // CUDA_MALLOC / CUDA_HOST / IPC(own)
  // VMM
  size_t page = 0, va_size = 0;
  std::vector<CUmemGenericAllocationHandle> mem;  // per rank, 0 = none
  std::vector<size_t> map_off, map_len;           // per rank range inside the VA
  // SHM
  std::string shm_name;
  size_t shm_len = 0;
  bool registered = false;
  // IPC
  std::vector<void*> opened;  // per rank, peers only
};

namespace wgb {

namespace {

// ---- CUDA driver entry points, resolved through the runtime so that the library has no
// link-time dependency on libcuda (it must load on hosts without a driver).
struct driver_api {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                        unsigned long long)                                                = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle)                                     = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                          CUmemAllocationGranularity_flags)                = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) =
    nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t)                                          = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                     unsigned long long)                                                   = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t)                                                = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)            = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                         CUmemAllocationHandleType, unsigned long long)    = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                           CUmemAllocationHandleType)                      = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**)                                       = nullptr;
};

driver_api& drv()
{
  static driver_api api = [] {
    driver_api a;
    auto bind = [](const char* name, void** out) {
      cudaDriverEntryPointQueryResult st;
      cudaError_t e = cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &st);
      if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || *out == nullptr) {
        (void)cudaGetLastError();
        throw cuda_error(std::string("driver entry point unavailable: ") + name);
      }
    };
    bind("cuMemCreate", reinterpret_cast<void**>(&a.MemCreate));
    bind("cuMemRelease", reinterpret_cast<void**>(&a.MemRelease));
    bind("cuMemGetAllocationGranularity", reinterpret_cast<void**>(&a.MemGetAllocationGranularity));
    bind("cuMemAddressReserve", reinterpret_cast<void**>(&a.MemAddressReserve));
    bind("cuMemAddressFree", reinterpret_cast<void**>(&a.MemAddressFree));
    bind("cuMemMap", reinterpret_cast<void**>(&a.MemMap));
    bind("cuMemUnmap", reinterpret_cast<void**>(&a.MemUnmap));
    bind("cuMemSetAccess", reinterpret_cast<void**>(&a.MemSetAccess));
    bind("cuMemExportToShareableHandle", reinterpret_cast<void**>(&a.MemExportToShareableHandle));
    bind("cuMemImportFromShareableHandle",
         reinterpret_cast<void**>(&a.MemImportFromShareableHandle));
    bind("cuGetErrorString", reinterpret_cast<void**>(&a.GetErrorString));
    return a;
  }();
  return api;
}

#define WGB_CU_CHECK(call)                                                                  \
  do {                                                                                      \
    CUresult r__ = (call);                                                                  \
    if (r__ != CUDA_SUCCESS) {                                                              \
      const char* s__ = nullptr;                                                            \
      drv().GetErrorString(r__, &s__);                                                      \
      throw ::wgb::cuda_error(::wgb::format_string("%s:%d driver error %d (%s) in %s", __FILE__, \
                                                   __LINE__, (int)r__, s__ ? s__ : "?", #call)); \
    }                                                                                       \
  } while (0)

// ---- file-descriptor exchange over abstract unix datagram sockets -------------------------
struct fd_exchange {
  int sock = -1;
  uint64_t tag;
  int hid, rank, world;

  static void fill_addr(sockaddr_un* a, socklen_t* len, uint64_t tag, int hid, int rank)
  {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    // Abstract namespace: leading NUL, no file left behind.
    int n = snprintf(a->sun_path + 1, sizeof(a->sun_path) - 1, "wgb-%016llx-%d-%d",
                     static_cast<unsigned long long>(tag), hid, rank);
    *len  = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
  }

  fd_exchange(uint64_t t, int h, int r, int w) : tag(t), hid(h), rank(r), world(w)
  {
    sock = socket(AF_UNIX, SOCK_DGRAM, 0);
    if (sock < 0) throw system_error(std::string("socket: ") + strerror(errno));
    sockaddr_un a;
    socklen_t len;
    fill_addr(&a, &len, tag, hid, rank);
    if (bind(sock, reinterpret_cast<sockaddr*>(&a), len) != 0) {
      int e = errno;
      close(sock);
      throw system_error(std::string("bind: ") + strerror(e));
    }
    timeval tv{30, 0};  // never wait forever for a peer that died
    setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(sock, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  }
  ~fd_exchange()
  {
    if (sock >= 0) close(sock);
  }

  // Non-blocking: false when the peer's queue is full right now.
  bool try_send_fd(int to, int fd)
  {
    sockaddr_un a;
    socklen_t len;
    fill_addr(&a, &len, tag, hid, to);
    int payload = rank;
    iovec iov{&payload, sizeof(payload)};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_name       = &a;
    msg.msg_namelen    = len;
    msg.msg_iov        = &iov;
    msg.msg_iovlen     = 1;
    msg.msg_control    = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c         = CMSG_FIRSTHDR(&msg);
    c->cmsg_level      = SOL_SOCKET;
    c->cmsg_type       = SCM_RIGHTS;
    c->cmsg_len        = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
    if (sendmsg(sock, &msg, MSG_DONTWAIT) >= 0) return true;
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS || errno == EINTR) return false;
    throw system_error(std::string("sendmsg: ") + strerror(errno));
  }

  // Non-blocking: false when nothing has arrived yet.
  bool try_recv_fd(int* from, int* fd)
  {
    int payload = -1;
    iovec iov{&payload, sizeof(payload)};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    msghdr msg{};
    msg.msg_iov        = &iov;
    msg.msg_iovlen     = 1;
    msg.msg_control    = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n          = recvmsg(sock, &msg, MSG_DONTWAIT);
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return false;
      throw system_error(std::string("recvmsg: ") + strerror(errno));
    }
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_type != SCM_RIGHTS) throw system_error("no descriptor in message");
    memcpy(fd, CMSG_DATA(c), sizeof(int));
    *from = payload;
    return true;
  }

  // Sleep until the socket is readable (or writable, when a send is pending), at most `ms`.
  void wait_ready(bool want_write, int ms)
  {
    pollfd p{sock, static_cast<short>(POLLIN | (want_write ? POLLOUT : 0)), 0};
    if (want_write) {
      // A datagram socket is always "writable" even when the peer's queue is full: just nap.
      usleep(1000);
      return;
    }
    poll(&p, 1, ms);
  }
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void alloc_vmm(wholegraph_handle_* h)
{
  auto* b   = h->impl;
  auto* c   = h->comm;
  int W     = c->world_size;
  b->kind   = wholegraph_handle_::backing::VMM;
  CUmemAllocationProp prop{};
  prop.type                 = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type        = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id          = c->dev_id;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t page               = 0;
  WGB_CU_CHECK(drv().MemGetAllocationGranularity(&page, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  // All ranks must tile the range with the same page size.
  std::vector<size_t> pages(W);
  c->host_allgather(&page, pages.data(), sizeof(size_t));
  page    = *std::max_element(pages.begin(), pages.end());
  b->page = page;

  // Page p belongs to the rank whose logical shard contains the page's LAST byte, so the first
  // byte of every shard of at least one page is physically on its own GPU (pointer queries on a
  // shard's base then name the local device); the tail of a shard may sit on the next rank.
  size_t n_pages = round_up(std::max<size_t>(h->total_size, 1), page) / page;
  std::vector<size_t> first(W + 1);
  first[0] = 0;
  for (int r = 1; r < W; r++) first[r] = std::min(n_pages, h->part_offsets[r] / page);
  first[W] = n_pages;
  for (int r = 1; r <= W; r++) first[r] = std::max(first[r], first[r - 1]);
  b->va_size = n_pages * page;
  b->mem.assign(W, 0);
  b->map_off.resize(W);
  b->map_len.resize(W);
  for (int r = 0; r < W; r++) {
    b->map_off[r] = first[r] * page;
    b->map_len[r] = (first[r + 1] - first[r]) * page;
  }

  int me     = c->world_rank;
  int own_fd = -1;
  WGB_DEBUG("vmm handle %d: page %zu, %zu pages, rank %d maps [%zu, +%zu)", h->id, page, n_pages, me,
            b->map_off[me], b->map_len[me]);
  if (b->map_len[me] > 0) {
    WGB_CU_CHECK(drv().MemCreate(&b->mem[me], b->map_len[me], &prop, 0));
    WGB_CU_CHECK(drv().MemExportToShareableHandle(&own_fd, b->mem[me],
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  }
  {
    fd_exchange ex(c->tag, h->id, me, W);
    c->barrier();  // every socket is bound
    // Every rank that holds pages sends its descriptor to every peer; a rank expects one from
    // every peer that holds pages.  Sends and receives are interleaved without blocking, so no
    // chain of full socket queues can stall the exchange, whatever subset of ranks sends.
    int expected = 0;
    for (int r = 0; r < W; r++)
      if (r != me && b->map_len[r] > 0) expected++;
    const int to_send = own_fd >= 0 ? W - 1 : 0;
    int sent = 0, got = 0;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(60);
    while (sent < to_send || got < expected) {
      bool progressed = false;
      if (sent < to_send) {
        const int to = (me + 1 + sent) % W;
        if (ex.try_send_fd(to, own_fd)) {
          sent++;
          progressed = true;
        }
      }
      if (got < expected) {
        int fd = -1, from = -1;
        if (ex.try_recv_fd(&from, &fd)) {
          WGB_EXPECTS(from >= 0 && from < W && from != me && b->mem[from] == 0, "bad sender %d", from);
          WGB_CU_CHECK(drv().MemImportFromShareableHandle(
            &b->mem[from], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
          close(fd);
          got++;
          progressed = true;
        }
      }
      if (!progressed) {
        if (std::chrono::steady_clock::now() > deadline)
          throw system_error("timed out exchanging memory descriptors with the other ranks");
        ex.wait_ready(sent < to_send, 50);
      }
    }
    c->barrier();  // nobody closes a socket that still has senders
  }
  if (own_fd >= 0) close(own_fd);
  WGB_DEBUG("vmm handle %d: descriptors exchanged", h->id);

  CUdeviceptr va = 0;
  WGB_CU_CHECK(drv().MemAddressReserve(&va, b->va_size, page, 0, 0));
  h->global_base = reinterpret_cast<void*>(va);
  for (int r = 0; r < W; r++) {
    if (b->map_len[r] == 0) continue;
    WGB_CU_CHECK(drv().MemMap(va + b->map_off[r], b->map_len[r], 0, b->mem[r], 0));
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id   = c->dev_id;
  acc.flags         = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  WGB_CU_CHECK(drv().MemSetAccess(va, b->va_size, &acc, 1));
  h->local_ptr = static_cast<char*>(h->global_base) + h->part_offsets[me];
  WGB_DEBUG("vmm handle %d: mapped %zu bytes at %p", h->id, b->va_size, h->global_base);
}

void free_vmm(wholegraph_handle_* h)
{
  auto* b = h->impl;
  if (h->global_base != nullptr) {
    CUdeviceptr va = reinterpret_cast<CUdeviceptr>(h->global_base);
    for (size_t r = 0; r < b->mem.size(); r++)
      if (b->map_len[r] > 0 && b->mem[r] != 0) drv().MemUnmap(va + b->map_off[r], b->map_len[r]);
    drv().MemAddressFree(va, b->va_size);
  }
  for (auto m : b->mem)
    if (m != 0) drv().MemRelease(m);
}

void alloc_shm(wholegraph_handle_* h)
{
  auto* b     = h->impl;
  auto* c     = h->comm;
  b->kind     = wholegraph_handle_::backing::SHM;
  b->shm_name = format_string("/wgb-%016llx-%d", static_cast<unsigned long long>(c->tag), h->id);
  b->shm_len  = std::max<size_t>(h->total_size, 1);
  int fd      = -1;
  if (c->world_rank == 0) {
    shm_unlink(b->shm_name.c_str());
    fd = shm_open(b->shm_name.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0) throw system_error(std::string("shm_open: ") + strerror(errno));
    if (ftruncate(fd, static_cast<off_t>(b->shm_len)) != 0) {
      int e = errno;
      close(fd);
      throw system_error(std::string("ftruncate: ") + strerror(e));
    }
  }
  c->barrier();
  if (c->world_rank != 0) {
    fd = shm_open(b->shm_name.c_str(), O_RDWR, 0600);
    if (fd < 0) throw system_error(std::string("shm_open: ") + strerror(errno));
  }
  void* p = mmap(nullptr, b->shm_len, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw system_error(std::string("mmap: ") + strerror(errno));
  b->alloc_ptr = p;
  c->barrier();
  if (c->world_rank == 0) shm_unlink(b->shm_name.c_str());  // mapping keeps it alive
  WGB_CUDA_CHECK(cudaHostRegister(p, b->shm_len, cudaHostRegisterPortable | cudaHostRegisterMapped));
  b->registered = true;
  void* dptr    = nullptr;
  WGB_CUDA_CHECK(cudaHostGetDevicePointer(&dptr, p, 0));
  WGB_EXPECTS(dptr == p, "registered host memory is not addressable at its host address");
  h->global_base = p;
  h->local_ptr   = static_cast<char*>(p) + h->part_offsets[c->world_rank];
}

void alloc_ipc(wholegraph_handle_* h)
{
  auto* b  = h->impl;
  auto* c  = h->comm;
  int W    = c->world_size;
  int me   = c->world_rank;
  b->kind  = wholegraph_handle_::backing::IPC;
  size_t n = std::max<size_t>(h->part_sizes[me], 256);
  WGB_CUDA_CHECK(cudaMalloc(&b->alloc_ptr, n));
  h->local_ptr = b->alloc_ptr;
  h->rank_ptrs.assign(W, nullptr);
  h->rank_ptrs[me] = b->alloc_ptr;
  b->opened.assign(W, nullptr);
  if (W > 1) {
    cudaIpcMemHandle_t mine;
    WGB_CUDA_CHECK(cudaIpcGetMemHandle(&mine, b->alloc_ptr));
    std::vector<cudaIpcMemHandle_t> all(W);
    c->host_allgather(&mine, all.data(), sizeof(mine));
    for (int r = 0; r < W; r++) {
      if (r == me) continue;
      WGB_CUDA_CHECK(cudaIpcOpenMemHandle(&b->opened[r], all[r], cudaIpcMemLazyEnablePeerAccess));
      h->rank_ptrs[r] = b->opened[r];
    }
  }
  WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&h->dev_rank_ptrs), sizeof(void*) * W));
  WGB_CUDA_CHECK(cudaMemcpy(h->dev_rank_ptrs, h->rank_ptrs.data(), sizeof(void*) * W,
                            cudaMemcpyHostToDevice));
}

}  // namespace

void plan_partition(size_t total_size, size_t granularity, int world, const size_t* rank_units,
                    std::vector<size_t>* sizes, std::vector<size_t>* offsets)
{
  sizes->assign(world, 0);
  offsets->assign(world + 1, 0);
  size_t units = total_size / granularity;
  if (rank_units != nullptr) {
    for (int r = 0; r < world; r++) {
      (*sizes)[r]       = rank_units[r] * granularity;
      (*offsets)[r + 1] = (*offsets)[r] + (*sizes)[r];
    }
    return;
  }
  size_t per = (units + world - 1) / world;
  for (int r = 0; r < world; r++) {
    size_t s      = std::min(static_cast<size_t>(r) * per, units);
    size_t e      = std::min(static_cast<size_t>(r + 1) * per, units);
    (*sizes)[r]   = (e - s) * granularity;
    (*offsets)[r] = s * granularity;
  }
  (*offsets)[world] = units * granularity;
}

wholegraph_handle_* create_handle(size_t total_size, wholegraph_comm_* comm,
                                  wholegraph_memory_type_t type,
                                  wholegraph_memory_location_t location, size_t granularity,
                                  size_t* rank_entry_partition)
{
  if (comm == nullptr) throw invalid_input(WHOLEGRAPH_INVALID_INPUT, "comm is null");
  if (granularity == 0 || total_size % granularity != 0)
    throw invalid_input(WHOLEGRAPH_INVALID_VALUE, "total_size is not a multiple of data_granularity");
  if (type != WHOLEGRAPH_MT_CONTINUOUS && type != WHOLEGRAPH_MT_DISTRIBUTED &&
      type != WHOLEGRAPH_MT_CHUNKED)
    throw invalid_input(WHOLEGRAPH_INVALID_INPUT, "memory type not supported");
  if (location != WHOLEGRAPH_ML_DEVICE && location != WHOLEGRAPH_ML_HOST)
    throw invalid_input(WHOLEGRAPH_INVALID_INPUT, "memory location not supported");
  if (type == WHOLEGRAPH_MT_CHUNKED && location != WHOLEGRAPH_ML_DEVICE)
    throw invalid_input(WHOLEGRAPH_NOT_SUPPORTED, "CHUNKED memory is device memory");
  int W = comm->world_size;
  if (rank_entry_partition != nullptr) {
    size_t units = 0;
    for (int r = 0; r < W; r++) {
      if (rank_entry_partition[r] == 0)
        throw invalid_input(WHOLEGRAPH_INVALID_VALUE, "rank_entry_partition holds a zero");
      units += rank_entry_partition[r];
    }
    if (units * granularity != total_size)
      throw invalid_input(WHOLEGRAPH_INVALID_VALUE, "rank_entry_partition does not sum to total_size");
  }
  // All ranks must ask for the same thing (reference: memory_handle.cpp:1408-1414).
  struct {
    size_t total, gran;
    int type, loc, has_part, pad;
  } param;
  memset(&param, 0, sizeof(param));  // compared bytewise: no indeterminate padding
  param.total    = total_size;
  param.gran     = granularity;
  param.type     = type;
  param.loc      = location;
  param.has_part = rank_entry_partition != nullptr ? 1 : 0;
  if (!comm->all_same(&param, sizeof(param)))
    throw comm_error("wholegraph_malloc called with different arguments on different ranks");
  if (rank_entry_partition != nullptr &&
      !comm->all_same(rank_entry_partition, sizeof(size_t) * W))
    throw comm_error("rank_entry_partition differs between ranks");

  std::unique_ptr<wholegraph_handle_> h(new wholegraph_handle_());
  h->comm        = comm;
  h->type        = type;
  h->location    = location;
  h->total_size  = total_size;
  h->granularity = granularity;
  h->impl        = new wholegraph_handle_::backing();
  plan_partition(total_size, granularity, W, rank_entry_partition, &h->part_sizes, &h->part_offsets);
  {
    std::lock_guard<std::mutex> lk(comm->mu);
    h->id = comm->next_handle_id++;
  }
  int me = comm->world_rank;
  try {
    if (type == WHOLEGRAPH_MT_DISTRIBUTED || (type == WHOLEGRAPH_MT_CONTINUOUS && W == 1)) {
      size_t n = std::max<size_t>(h->part_sizes[me], 256);
      if (location == WHOLEGRAPH_ML_DEVICE) {
        h->impl->kind = wholegraph_handle_::backing::CUDA_MALLOC;
        WGB_CUDA_CHECK(cudaMalloc(&h->impl->alloc_ptr, n));
      } else {
        h->impl->kind = wholegraph_handle_::backing::CUDA_HOST;
        WGB_CUDA_CHECK(cudaHostAlloc(&h->impl->alloc_ptr, n, cudaHostAllocPortable | cudaHostAllocMapped));
      }
      h->local_ptr = h->impl->alloc_ptr;
      if (type == WHOLEGRAPH_MT_CONTINUOUS) h->global_base = h->impl->alloc_ptr;
    } else if (type == WHOLEGRAPH_MT_CONTINUOUS) {
      if (location == WHOLEGRAPH_ML_DEVICE)
        alloc_vmm(h.get());
      else
        alloc_shm(h.get());
    } else {
      alloc_ipc(h.get());
    }
  } catch (...) {
    destroy_handle(h.release());
    throw;
  }
  comm->barrier();
  wholegraph_handle_* raw = h.release();
  {
    std::lock_guard<std::mutex> lk(comm->mu);
    comm->handles.insert(raw);
  }
  return raw;
}

void destroy_handle(wholegraph_handle_* h)
{
  if (h == nullptr) return;
  auto* c = h->comm;
  if (c != nullptr) {
    {
      std::lock_guard<std::mutex> lk(c->mu);
      c->handles.erase(h);
    }
    // Nobody may unmap memory a peer's kernel is still reading.
    cudaDeviceSynchronize();
    try {
      c->barrier();
    } catch (...) {
    }
  }
  auto* b = h->impl;
  if (b != nullptr) {
    switch (b->kind) {
      case wholegraph_handle_::backing::CUDA_MALLOC:
        if (b->alloc_ptr) cudaFree(b->alloc_ptr);
        break;
      case wholegraph_handle_::backing::CUDA_HOST:
        if (b->alloc_ptr) cudaFreeHost(b->alloc_ptr);
        break;
      case wholegraph_handle_::backing::VMM: free_vmm(h); break;
      case wholegraph_handle_::backing::SHM:
        if (b->registered) cudaHostUnregister(b->alloc_ptr);
        if (b->alloc_ptr) munmap(b->alloc_ptr, b->shm_len);
        break;
      case wholegraph_handle_::backing::IPC:
        for (void* p : b->opened)
          if (p) cudaIpcCloseMemHandle(p);
        if (c != nullptr) {
          try {
            c->barrier();  // peers closed their views before the owner frees
          } catch (...) {
          }
        }
        if (b->alloc_ptr) cudaFree(b->alloc_ptr);
        if (h->dev_rank_ptrs) cudaFree(h->dev_rank_ptrs);
        break;
      default: break;
    }
    delete b;
  }
  delete h;
}

}  // namespace wgb
