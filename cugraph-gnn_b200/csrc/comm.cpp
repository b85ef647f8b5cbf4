#include "comm.hpp"

#include <dlfcn.h>
#include <fcntl.h>
#include <nccl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <chrono>
#include <thread>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>

#include "common.hpp"
#include "handle.hpp"

namespace wgb {

// NCCL is bound at first use so that the library loads on hosts where only the single-rank
// paths run, and so that a process which already holds an NCCL (e.g. through torch) shares it.
namespace {

struct nccl_api {
  void* lib = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId         = nullptr;
  decltype(&ncclCommInitRank) CommInitRank       = nullptr;
  decltype(&ncclCommDestroy) CommDestroy         = nullptr;
  decltype(&ncclCommAbort) CommAbort             = nullptr;
  decltype(&ncclCommSplit) CommSplit             = nullptr;
  decltype(&ncclGetErrorString) GetErrorString   = nullptr;
  decltype(&ncclCommGetAsyncError) GetAsyncError = nullptr;
  decltype(&ncclGroupStart) GroupStart           = nullptr;
  decltype(&ncclGroupEnd) GroupEnd               = nullptr;
  decltype(&ncclSend) Send                       = nullptr;
  decltype(&ncclRecv) Recv                       = nullptr;
  decltype(&ncclAllGather) AllGather             = nullptr;
  decltype(&ncclAllReduce) AllReduce             = nullptr;
};

nccl_api& nccl_lib()
{
  static nccl_api api = [] {
    nccl_api a;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      a.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.lib != nullptr) break;
    }
    if (a.lib == nullptr) throw comm_error(std::string("cannot load NCCL: ") + dlerror());
#define WGB_BIND(field, sym)                                                     \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.lib, sym));              \
  if (a.field == nullptr) throw comm_error(std::string("NCCL symbol missing: ") + sym)
    WGB_BIND(GetUniqueId, "ncclGetUniqueId");
    WGB_BIND(CommInitRank, "ncclCommInitRank");
    WGB_BIND(CommDestroy, "ncclCommDestroy");
    WGB_BIND(CommAbort, "ncclCommAbort");
    WGB_BIND(CommSplit, "ncclCommSplit");
    WGB_BIND(GetErrorString, "ncclGetErrorString");
    WGB_BIND(GetAsyncError, "ncclCommGetAsyncError");
    WGB_BIND(GroupStart, "ncclGroupStart");
    WGB_BIND(GroupEnd, "ncclGroupEnd");
    WGB_BIND(Send, "ncclSend");
    WGB_BIND(Recv, "ncclRecv");
    WGB_BIND(AllGather, "ncclAllGather");
    WGB_BIND(AllReduce, "ncclAllReduce");
#undef WGB_BIND
    return a;
  }();
  return api;
}

#define WGB_NCCL_CHECK(call)                                                              \
  do {                                                                                    \
    ncclResult_t r__ = (call);                                                            \
    if (r__ != ncclSuccess && r__ != ncclInProgress) {                                    \
      throw ::wgb::comm_error(::wgb::format_string("%s:%d NCCL error %d (%s) in %s", __FILE__, \
                                                   __LINE__, (int)r__,                    \
                                                   ::wgb::nccl_lib().GetErrorString(r__), #call));   \
    }                                                                                     \
  } while (0)

std::mutex g_comm_mu;
std::set<wholegraph_comm_*> g_comms;

uint64_t fnv1a(const void* p, size_t n, uint64_t h = 1469598103934665603ull)
{
  const unsigned char* c = static_cast<const unsigned char*>(p);
  for (size_t i = 0; i < n; i++) {
    h ^= c[i];
    h *= 1099511628211ull;
  }
  return h;
}

}  // namespace
}  // namespace wgb

// One cache line per rank and parity: a sequence number and the posted values.  A rank posting
// call k + 2 overwrites its slot of call k only after it has read everybody's call k + 1, which
// they post after reading call k: two slots per rank are enough.
struct wholegraph_comm_::host_board {
  struct alignas(128) slot {
    uint64_t seq;
    int64_t values[wholegraph_comm_::kBoardValues];
  };
  slot* slots     = nullptr;  // [2][world]
  size_t bytes    = 0;
  uint64_t next   = 1;
};

namespace wgb {
namespace {

void setup_board(wholegraph_comm_* c)
{
  if (c->world_size == 1) return;
  using board_t      = wholegraph_comm_::host_board;
  const size_t bytes = sizeof(board_t::slot) * 2 * static_cast<size_t>(c->world_size);
  const std::string name = format_string("/wgb_board_%016llx", static_cast<unsigned long long>(c->tag));
  void* map = MAP_FAILED;
  int fd    = -1;
  if (c->world_rank == 0) {
    shm_unlink(name.c_str());
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd >= 0 && ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
      close(fd);
      fd = -1;
    }
  }
  c->barrier();  // the segment exists (or rank 0 failed to create it)
  if (c->world_rank != 0) fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd >= 0) {
    map = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
  }
  int ok = map != MAP_FAILED ? 1 : 0;
  std::vector<int> all(c->world_size, 0);
  c->host_allgather(&ok, all.data(), sizeof(int));
  for (int v : all) ok &= v;
  if (c->world_rank == 0) shm_unlink(name.c_str());  // the mappings keep it alive
  if (!ok) {
    if (map != MAP_FAILED) munmap(map, bytes);
    WGB_INFO("no shared host memory between the ranks of this communicator: distributed ops exchange sizes "
             "through the stream");
    return;
  }
  auto* b  = new board_t();
  b->slots = static_cast<board_t::slot*>(map);
  b->bytes = bytes;
  c->board = b;
  // rank 0 created the segment zero-filled; nobody posts before everybody is here
  c->barrier();
}

void destroy_board(wholegraph_comm_* c)
{
  if (c->board == nullptr) return;
  munmap(c->board->slots, c->board->bytes);
  delete c->board;
  c->board = nullptr;
}

void setup_staging(wholegraph_comm_* c)
{
  WGB_CUDA_CHECK(cudaGetDevice(&c->dev_id));
  WGB_CUDA_CHECK(cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking));
  // The exchange stream gets the highest priority: its NCCL kernels need only a few CTAs and
  // must not queue behind the thousands of short CTAs of the copy kernels they overlap with.
  int prio_low = 0, prio_high = 0;
  WGB_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
  WGB_CUDA_CHECK(cudaStreamCreateWithPriority(&c->xchg_stream, cudaStreamNonBlocking, prio_high));
  c->stage_bytes = (size_t(1) << 20) * static_cast<size_t>(c->world_size) * 2;
  if (c->world_size > 1) {
    WGB_CUDA_CHECK(cudaMalloc(&c->dev_stage, c->stage_bytes));
    WGB_CUDA_CHECK(cudaMallocHost(&c->pin_stage, c->stage_bytes));
  }
}

}  // namespace

exchange_tuning tuning_from_environment()
{
  auto flag = [](const char* name, int otherwise) {
    const char* e = getenv(name);
    if (e == nullptr || e[0] == '\0') return otherwise;
    return e[0] == '0' ? 0 : 1;
  };
  exchange_tuning t;
  t.peer_exchange   = flag("WG_PEER_EXCHANGE", t.peer_exchange);
  t.gather_dedup    = flag("WG_GATHER_DEDUP", t.gather_dedup);
  t.gradient_presum = flag("WG_GRADIENT_PRESUM", t.gradient_presum);
  t.peer_gradient   = flag("WG_PEER_GRADIENT", t.peer_gradient);
  t.sync_free       = flag("WG_SYNC_FREE", t.sync_free);
  t.serve_bulk      = flag("WG_SERVE_BULK", t.serve_bulk);
  t.single_rank_exchange = flag("WG_SINGLE_RANK_EXCHANGE", t.single_rank_exchange);
  const char* k     = getenv("WG_EXCHANGE_CHUNKS");
  t.exchange_chunks = k != nullptr ? std::min(std::max(0, atoi(k)), 16) : 0;
  return t;
}

void nccl_get_unique_id(wholegraph_unique_id_t* id)
{
  static_assert(sizeof(ncclUniqueId) <= WHOLEGRAPH_UNIQUE_ID_BYTES, "unique id too small");
  ncclUniqueId nid;
  WGB_NCCL_CHECK(nccl_lib().GetUniqueId(&nid));
  memset(id->internal, 0, sizeof(id->internal));
  memcpy(id->internal, &nid, sizeof(nid));
}

wholegraph_comm_* create_comm(const wholegraph_unique_id_t& id, int rank, int size)
{
  if (size <= 0 || rank < 0 || rank >= size)
    throw invalid_input(WHOLEGRAPH_INVALID_INPUT, format_string("bad rank %d / size %d", rank, size));
  std::unique_ptr<wholegraph_comm_> c(new wholegraph_comm_());
  c->world_rank = rank;
  c->world_size = size;
  c->tag        = fnv1a(id.internal, sizeof(id.internal));
  if (size > 1) {
    ncclUniqueId nid;
    memcpy(&nid, id.internal, sizeof(nid));
    ncclComm_t nc = nullptr;
    WGB_NCCL_CHECK(nccl_lib().CommInitRank(&nc, size, nid, rank));
    c->nccl = nc;
  }
  setup_staging(c.get());
  c->reload_tuning();
  setup_board(c.get());
  wholegraph_comm_* raw = c.release();
  {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    g_comms.insert(raw);
  }
  return raw;
}

wholegraph_comm_* split_comm(wholegraph_comm_* comm, int color, int key)
{
  // Agree on membership first: every rank learns everyone's (color, key).
  struct ck {
    int color, key;
  } mine{color, key};
  std::vector<ck> all(comm->world_size);
  comm->host_allgather(&mine, all.data(), sizeof(ck));
  ncclComm_t nc = nullptr;
  if (comm->world_size > 1) {
    WGB_NCCL_CHECK(nccl_lib().CommSplit(static_cast<ncclComm_t>(comm->nccl),
                                    color < 0 ? NCCL_SPLIT_NOCOLOR : color, key, &nc, nullptr));
  }
  if (color < 0) return nullptr;
  // New rank = position among same-colour ranks ordered by (key, old rank).
  int new_rank = 0, new_size = 0;
  for (int r = 0; r < comm->world_size; r++) {
    if (all[r].color != color) continue;
    new_size++;
    if (all[r].key < key || (all[r].key == key && r < comm->world_rank)) new_rank++;
  }
  std::unique_ptr<wholegraph_comm_> c(new wholegraph_comm_());
  c->world_rank = new_rank;
  c->world_size = new_size;
  uint64_t seed[3] = {comm->tag, static_cast<uint64_t>(color), static_cast<uint64_t>(comm->next_handle_id++)};
  c->tag        = fnv1a(seed, sizeof(seed));
  if (new_size > 1) {
    c->nccl = nc;
  } else if (nc != nullptr) {
    nccl_lib().CommDestroy(nc);
  }
  setup_staging(c.get());
  c->reload_tuning();
  setup_board(c.get());
  wholegraph_comm_* raw = c.release();
  {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    g_comms.insert(raw);
  }
  return raw;
}

void destroy_comm(wholegraph_comm_* comm)
{
  if (comm == nullptr) return;
  {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (g_comms.erase(comm) == 0) return;  // unknown or already destroyed
  }
  // Handles still alive go with the communicator (reference: communicator.cpp:791-810).
  std::vector<wholegraph_handle_*> left;
  {
    std::lock_guard<std::mutex> lk(comm->mu);
    left.assign(comm->handles.begin(), comm->handles.end());
  }
  std::sort(left.begin(), left.end(),
            [](wholegraph_handle_* a, wholegraph_handle_* b) { return a->id < b->id; });
  for (auto* h : left) destroy_handle(h);
  destroy_board(comm);
  if (comm->barrier_word) cudaFree(comm->barrier_word);
  if (comm->status_word) cudaFree(comm->status_word);
  if (comm->status_host) cudaFreeHost(comm->status_host);
  if (comm->arena_idle) cudaEventDestroy(comm->arena_idle);
  if (comm->dev_stage) cudaFree(comm->dev_stage);
  if (comm->pin_stage) cudaFreeHost(comm->pin_stage);
  if (comm->side_stream) cudaStreamDestroy(comm->side_stream);
  if (comm->xchg_stream) cudaStreamDestroy(comm->xchg_stream);
  for (auto e : comm->events) cudaEventDestroy(e);
  if (comm->nccl != nullptr) nccl_lib().CommDestroy(static_cast<ncclComm_t>(comm->nccl));
  delete comm;
}

void destroy_all_comms()
{
  std::vector<wholegraph_comm_*> all;
  {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    all.assign(g_comms.begin(), g_comms.end());
  }
  for (auto* c : all) destroy_comm(c);
}

}  // namespace wgb



cudaEvent_t wholegraph_comm_::event(size_t i)
{
  while (events.size() <= i) {
    cudaEvent_t e = nullptr;
    WGB_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    events.push_back(e);
  }
  return events[i];
}

void wholegraph_comm_::reload_tuning()
{
  const wgb::exchange_tuning mine = wgb::tuning_from_environment();
  // The reference checks the parameters of every collective call the same way
  // (wg_comm_check_all_same, cpp/src/wholegraph/communicator.hpp:220-249).
  if (!all_same(&mine, sizeof(mine)))
    throw wgb::logic_error(
      "the WG_* tuning variables differ between the ranks of a communicator; they select which "
      "collectives an op issues and must be equal everywhere");
  tuning = mine;
}

void wholegraph_comm_::board_exchange(const int64_t* mine, int64_t* all)
{
  if (world_size == 1) {
    memcpy(all, mine, sizeof(int64_t) * kBoardValues);
    return;
  }
  WGB_EXPECTS(board != nullptr, "this communicator has no shared host board");
  const uint64_t seq      = board->next++;
  host_board::slot* mine_ = board->slots + (seq & 1) * world_size + world_rank;
  memcpy(mine_->values, mine, sizeof(int64_t) * kBoardValues);
  __atomic_store_n(&mine_->seq, seq, __ATOMIC_RELEASE);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(60);
  for (int r = 0; r < world_size; r++) {
    host_board::slot* s = board->slots + (seq & 1) * world_size + r;
    unsigned spins      = 0;
    while (__atomic_load_n(&s->seq, __ATOMIC_ACQUIRE) < seq) {
      if (++spins < 2000) continue;
      if ((spins & 1023) == 0 && std::chrono::steady_clock::now() > deadline)
        throw wgb::comm_error(wgb::format_string("rank %d did not reach collective call %llu within 60 s", r,
                                                 static_cast<unsigned long long>(seq)));
      std::this_thread::yield();
    }
    memcpy(all + static_cast<size_t>(r) * kBoardValues, s->values, sizeof(int64_t) * kBoardValues);
  }
}

void wholegraph_comm_::check_async_error()
{
  if (nccl == nullptr) return;
  ncclResult_t st = ncclSuccess;
  WGB_NCCL_CHECK(wgb::nccl_lib().GetAsyncError(static_cast<ncclComm_t>(nccl), &st));
  if (st != ncclSuccess && st != ncclInProgress)
    throw wgb::comm_error(std::string("NCCL asynchronous error: ") + wgb::nccl_lib().GetErrorString(st));
}

void wholegraph_comm_::host_allgather(const void* send, void* recv, size_t bytes)
{
  if (world_size == 1) {
    if (recv != send) memcpy(recv, send, bytes);
    return;
  }
  WGB_EXPECTS(bytes * (world_size + 1) <= stage_bytes, "host_allgather of %zu bytes is too large",
              bytes);
  std::lock_guard<std::mutex> lk(mu);
  char* dsend = static_cast<char*>(dev_stage);
  char* drecv = dsend + bytes;
  memcpy(pin_stage, send, bytes);
  WGB_CUDA_CHECK(cudaMemcpyAsync(dsend, pin_stage, bytes, cudaMemcpyHostToDevice, side_stream));
  WGB_NCCL_CHECK(wgb::nccl_lib().AllGather(dsend, drecv, bytes, ncclInt8,
                                       static_cast<ncclComm_t>(nccl), side_stream));
  WGB_CUDA_CHECK(cudaMemcpyAsync(pin_stage, drecv, bytes * world_size, cudaMemcpyDeviceToHost,
                                 side_stream));
  WGB_CUDA_CHECK(cudaStreamSynchronize(side_stream));
  memcpy(recv, pin_stage, bytes * world_size);
}

void wholegraph_comm_::host_alltoall(const void* send, void* recv, size_t bytes)
{
  if (world_size == 1) {
    if (recv != send) memcpy(recv, send, bytes);
    return;
  }
  size_t total = bytes * world_size;
  WGB_EXPECTS(total * 2 <= stage_bytes, "host_alltoall of %zu bytes is too large", bytes);
  std::lock_guard<std::mutex> lk(mu);
  char* dsend = static_cast<char*>(dev_stage);
  char* drecv = dsend + total;
  memcpy(pin_stage, send, total);
  WGB_CUDA_CHECK(cudaMemcpyAsync(dsend, pin_stage, total, cudaMemcpyHostToDevice, side_stream));
  alltoall(dsend, drecv, bytes, side_stream);
  WGB_CUDA_CHECK(cudaMemcpyAsync(pin_stage, drecv, total, cudaMemcpyDeviceToHost, side_stream));
  WGB_CUDA_CHECK(cudaStreamSynchronize(side_stream));
  memcpy(recv, pin_stage, total);
}

void wholegraph_comm_::barrier()
{
  if (world_size == 1) return;
  std::lock_guard<std::mutex> lk(mu);
  int* d = static_cast<int*>(dev_stage);
  WGB_CUDA_CHECK(cudaMemsetAsync(d, 0, sizeof(int), side_stream));
  WGB_NCCL_CHECK(wgb::nccl_lib().AllReduce(d, d, 1, ncclInt32, ncclSum, static_cast<ncclComm_t>(nccl),
                                       side_stream));
  WGB_CUDA_CHECK(cudaStreamSynchronize(side_stream));
}

bool wholegraph_comm_::all_same(const void* value, size_t bytes)
{
  if (world_size == 1) return true;
  std::vector<char> all(bytes * world_size);
  host_allgather(value, all.data(), bytes);
  for (int r = 1; r < world_size; r++)
    if (memcmp(all.data(), all.data() + r * bytes, bytes) != 0) return false;
  return true;
}

void wholegraph_comm_::alltoallv(const void* send, const int64_t* send_counts,
                                 const int64_t* send_displs, void* recv,
                                 const int64_t* recv_counts, const int64_t* recv_displs,
                                 size_t unit, cudaStream_t stream)
{
  const char* s = static_cast<const char*>(send);
  char* r       = static_cast<char*>(recv);
  if (world_size == 1) {
    if (send_counts[0] > 0)
      WGB_CUDA_CHECK(cudaMemcpyAsync(r + recv_displs[0] * unit, s + send_displs[0] * unit,
                                     send_counts[0] * unit, cudaMemcpyDeviceToDevice, stream));
    return;
  }
  ncclComm_t nc = static_cast<ncclComm_t>(nccl);
  // The self segment never touches NCCL: one local copy.
  if (send_counts[world_rank] > 0)
    WGB_CUDA_CHECK(cudaMemcpyAsync(r + recv_displs[world_rank] * unit,
                                   s + send_displs[world_rank] * unit,
                                   send_counts[world_rank] * unit, cudaMemcpyDeviceToDevice, stream));
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupStart());
  for (int step = 1; step < world_size; step++) {
    int to   = (world_rank + step) % world_size;
    int from = (world_rank - step + world_size) % world_size;
    if (send_counts[to] > 0)
      WGB_NCCL_CHECK(wgb::nccl_lib().Send(s + send_displs[to] * unit, send_counts[to] * unit, ncclInt8,
                                      to, nc, stream));
    if (recv_counts[from] > 0)
      WGB_NCCL_CHECK(wgb::nccl_lib().Recv(r + recv_displs[from] * unit, recv_counts[from] * unit,
                                      ncclInt8, from, nc, stream));
  }
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupEnd());
}

void wholegraph_comm_::exchange(const std::vector<transfer>& sends, const std::vector<transfer>& recvs,
                                cudaStream_t stream)
{
  if (world_size == 1) return;
  ncclComm_t nc = static_cast<ncclComm_t>(nccl);
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupStart());
  for (const auto& t : sends)
    if (t.bytes > 0) WGB_NCCL_CHECK(wgb::nccl_lib().Send(t.ptr, t.bytes, ncclInt8, t.peer, nc, stream));
  for (const auto& t : recvs)
    if (t.bytes > 0) WGB_NCCL_CHECK(wgb::nccl_lib().Recv(t.ptr, t.bytes, ncclInt8, t.peer, nc, stream));
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupEnd());
}

void wholegraph_comm_::sendrecv(const void* send, size_t send_bytes, int to, void* recv,
                                size_t recv_bytes, int from, cudaStream_t stream)
{
  WGB_EXPECTS(world_size > 1, "sendrecv on a single-rank communicator");
  ncclComm_t nc = static_cast<ncclComm_t>(nccl);
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupStart());
  if (send_bytes > 0) WGB_NCCL_CHECK(wgb::nccl_lib().Send(send, send_bytes, ncclInt8, to, nc, stream));
  if (recv_bytes > 0) WGB_NCCL_CHECK(wgb::nccl_lib().Recv(recv, recv_bytes, ncclInt8, from, nc, stream));
  WGB_NCCL_CHECK(wgb::nccl_lib().GroupEnd());
}

void wholegraph_comm_::allgather(const void* send, void* recv, size_t bytes, cudaStream_t stream)
{
  if (world_size == 1) {
    if (recv != send) WGB_CUDA_CHECK(cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, stream));
    return;
  }
  WGB_NCCL_CHECK(wgb::nccl_lib().AllGather(send, recv, bytes, ncclInt8, static_cast<ncclComm_t>(nccl), stream));
}

void wholegraph_comm_::stream_barrier(cudaStream_t stream)
{
  if (world_size == 1) return;
  if (barrier_word == nullptr) {
    WGB_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&barrier_word), 256));
    WGB_CUDA_CHECK(cudaMemset(barrier_word, 0, 256));
  }
  WGB_NCCL_CHECK(wgb::nccl_lib().AllReduce(barrier_word, barrier_word + 32, 1, ncclInt32, ncclSum,
                                       static_cast<ncclComm_t>(nccl), stream));
}

void wholegraph_comm_::alltoall(const void* send, void* recv, size_t bytes, cudaStream_t stream)
{
  std::vector<int64_t> cnt(world_size, 1), dsp(world_size);
  for (int i = 0; i < world_size; i++) dsp[i] = i;
  alltoallv(send, cnt.data(), dsp.data(), recv, cnt.data(), dsp.data(), bytes, stream);
}
