// NCCL reached through dlopen("libnccl.so.2"): the native library links against no NCCL, so it loads on a machine
// without one, and a process that already holds NCCL (PyTorch's bundled copy) shares that copy. Only what the
// `extern:nccl_*` launches need is resolved. Constants follow the public nccl.h (ncclDataType_t, ncclRedOp_t).
// Reference counterpart: crates/kern-runtime/src/nccl.rs:148 (communicator join), :190 (collective).
#pragma once
#include <dlfcn.h>

#include <cstddef>
#include <cstdlib>
#include <stdexcept>
#include <string>

namespace kern {

struct NcclUniqueId { char internal[128]; };

enum class NcclColl { AllReduce, AllGather, ReduceScatter, AllToAll };
enum class NcclElem : int { U8 = 1, I32 = 2, F32 = 7, Bf16 = 9 };      // values of ncclDataType_t

inline size_t nccl_elem_bytes(NcclElem e) { return e == NcclElem::U8 ? 1 : (e == NcclElem::Bf16 ? 2 : 4); }

// `extern:nccl_<coll>_<elem>` parsed; false for any other name.
inline bool parse_nccl_extern(const std::string& entry, NcclColl* coll, NcclElem* elem) {
  const std::string pre = "extern:nccl_";
  if (entry.compare(0, pre.size(), pre) != 0) return false;
  const std::string rest = entry.substr(pre.size());
  const size_t us = rest.find('_');
  if (us == std::string::npos) return false;
  const std::string c = rest.substr(0, us), e = rest.substr(us + 1);
  if (c == "allreduce") *coll = NcclColl::AllReduce;
  else if (c == "allgather") *coll = NcclColl::AllGather;
  else if (c == "reducescatter") *coll = NcclColl::ReduceScatter;
  else if (c == "alltoall") *coll = NcclColl::AllToAll;
  else return false;
  if (e == "f32") *elem = NcclElem::F32;
  else if (e == "bf16") *elem = NcclElem::Bf16;
  else if (e == "i32") *elem = NcclElem::I32;
  else if (e == "u8") *elem = NcclElem::U8;
  else return false;
  return true;
}

class NcclApi {
 public:
  using Comm = void*;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(Comm*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, Comm, void*) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, Comm, void*) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, Comm, void*) = nullptr;
  int (*Send)(const void*, size_t, int, int, Comm, void*) = nullptr;
  int (*Recv)(void*, size_t, int, int, Comm, void*) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;

  // The process-wide table; throws with the loader's message when no NCCL can be found.
  static NcclApi& get() {
    static NcclApi api;
    if (!api.lib_) api.load();
    return api;
  }
  void check(int rc, const char* what) const {
    if (rc != 0) throw std::runtime_error(std::string("nccl: ") + what + ": " + (GetErrorString ? GetErrorString(rc) : "error"));
  }

 private:
  void* lib_ = nullptr;
  void load() {
    const char* env = std::getenv("KERN_NCCL_LIB");
    const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
    std::string why;
    for (const char* n : names) {
      if (!n || !*n) continue;
      lib_ = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (lib_) break;
      why = dlerror();
    }
    if (!lib_) throw std::runtime_error("nccl: no libnccl.so.2 could be loaded (" + why + "); set KERN_NCCL_LIB");
    auto sym = [&](const char* n) {
      void* p = dlsym(lib_, n);
      if (!p) throw std::runtime_error(std::string("nccl: symbol ") + n + " is missing");
      return p;
    };
    GetUniqueId = reinterpret_cast<decltype(GetUniqueId)>(sym("ncclGetUniqueId"));
    CommInitRank = reinterpret_cast<decltype(CommInitRank)>(sym("ncclCommInitRank"));
    CommDestroy = reinterpret_cast<decltype(CommDestroy)>(sym("ncclCommDestroy"));
    AllReduce = reinterpret_cast<decltype(AllReduce)>(sym("ncclAllReduce"));
    AllGather = reinterpret_cast<decltype(AllGather)>(sym("ncclAllGather"));
    ReduceScatter = reinterpret_cast<decltype(ReduceScatter)>(sym("ncclReduceScatter"));
    Send = reinterpret_cast<decltype(Send)>(sym("ncclSend"));
    Recv = reinterpret_cast<decltype(Recv)>(sym("ncclRecv"));
    GroupStart = reinterpret_cast<decltype(GroupStart)>(sym("ncclGroupStart"));
    GroupEnd = reinterpret_cast<decltype(GroupEnd)>(sym("ncclGroupEnd"));
    GetErrorString = reinterpret_cast<decltype(GetErrorString)>(sym("ncclGetErrorString"));
  }
};

}  // namespace kern
