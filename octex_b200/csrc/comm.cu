// NCCL through dlopen: the handful of calls the search needs.

#include "comm.hpp"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <string>

namespace octex_b200::detail {

namespace {

struct nccl_api {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) get_unique_id   = nullptr;
  decltype(&ncclCommInitRank) comm_init_rank = nullptr;
  decltype(&ncclCommDestroy) comm_destroy    = nullptr;
  decltype(&ncclGroupStart) group_start      = nullptr;
  decltype(&ncclGroupEnd) group_end          = nullptr;
  decltype(&ncclSend) send                   = nullptr;
  decltype(&ncclRecv) recv                   = nullptr;
  decltype(&ncclAllGather) all_gather        = nullptr;
  decltype(&ncclGetErrorString) error_string = nullptr;
};

auto api() -> nccl_api&
{
  static nccl_api a;
  static std::once_flag once;
  static std::string failure;
  std::call_once(once, [] {
    // the library a framework in this process already loaded wins (same soname)
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (a.handle == nullptr) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (a.handle == nullptr) {
      failure = std::string("octex: cannot load libnccl.so.2 (") + dlerror() + ")";
      return;
    }
    auto sym = [&](const char* name) {
      void* p = dlsym(a.handle, name);
      if (p == nullptr && failure.empty()) failure = std::string("octex: libnccl lacks ") + name;
      return p;
    };
    a.get_unique_id  = reinterpret_cast<decltype(a.get_unique_id)>(sym("ncclGetUniqueId"));
    a.comm_init_rank = reinterpret_cast<decltype(a.comm_init_rank)>(sym("ncclCommInitRank"));
    a.comm_destroy   = reinterpret_cast<decltype(a.comm_destroy)>(sym("ncclCommDestroy"));
    a.group_start    = reinterpret_cast<decltype(a.group_start)>(sym("ncclGroupStart"));
    a.group_end      = reinterpret_cast<decltype(a.group_end)>(sym("ncclGroupEnd"));
    a.send           = reinterpret_cast<decltype(a.send)>(sym("ncclSend"));
    a.recv           = reinterpret_cast<decltype(a.recv)>(sym("ncclRecv"));
    a.all_gather     = reinterpret_cast<decltype(a.all_gather)>(sym("ncclAllGather"));
    a.error_string   = reinterpret_cast<decltype(a.error_string)>(sym("ncclGetErrorString"));
  });
  if (!failure.empty()) throw error(failure);
  return a;
}

void check(ncclResult_t r, const char* what)
{
  if (r != ncclSuccess)
    throw error(std::string("octex: NCCL ") + what + ": " + api().error_string(r));
}

static_assert(sizeof(ncclUniqueId) == kUniqueIdBytes, "ncclUniqueId size");

}  // namespace

void communicator::unique_id(void* out128)
{
  ncclUniqueId id;
  check(api().get_unique_id(&id), "ncclGetUniqueId");
  std::memcpy(out128, &id, sizeof(id));
}

communicator::communicator(const void* unique_id, int rank, int world, int device)
  : rank_(rank), world_(world), device_(device)
{
  OCTEX_EXPECTS(world >= 1 && rank >= 0 && rank < world, "octex: rank outside world");
  ncclUniqueId id;
  std::memcpy(&id, unique_id, sizeof(id));
  OCTEX_CUDA_TRY(cudaSetDevice(device));
  ncclComm_t c = nullptr;
  check(api().comm_init_rank(&c, world, id, rank), "ncclCommInitRank");
  comm_ = c;
}

communicator::~communicator()
{
  if (comm_ != nullptr) api().comm_destroy(static_cast<ncclComm_t>(comm_));
}

void communicator::group_start() { check(api().group_start(), "ncclGroupStart"); }
void communicator::group_end() { check(api().group_end(), "ncclGroupEnd"); }

void communicator::send(const void* buf, size_t bytes, int peer, cudaStream_t s)
{
  check(api().send(buf, bytes, ncclChar, peer, static_cast<ncclComm_t>(comm_), s), "ncclSend");
}

void communicator::recv(void* buf, size_t bytes, int peer, cudaStream_t s)
{
  check(api().recv(buf, bytes, ncclChar, peer, static_cast<ncclComm_t>(comm_), s), "ncclRecv");
}

void communicator::all_gather(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t s)
{
  check(api().all_gather(send, recv, bytes_per_rank, ncclChar, static_cast<ncclComm_t>(comm_), s),
        "ncclAllGather");
}

}  // namespace octex_b200::detail
