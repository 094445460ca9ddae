// Kernel activity tracing through CUPTI's activity API, reached by dlopen("libcupti.so.12") — the native library links
// against no CUPTI and loads on machines without it. While a trace is on, every kernel launched by this process lands
// as a record {name, start, end (ns, CUPTI clock), stream, grid, block, registers, shared memory}; the records are
// what the per-step trace tables are built from (device time per kernel, without events around every launch).
// Only CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL is enabled: it does not serialise kernels and needs no profiler lock.
// Reference counterpart: crates/kern-runtime/src/trace.rs:343-383 (start), :482-495 (collect), :520-591 (buffers).
#pragma once
#include <cupti.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace kern {

struct KernelRecord {
  std::string name;
  uint64_t start_ns = 0, end_ns = 0;
  uint32_t stream = 0, grid[3] = {0, 0, 0}, block[3] = {0, 0, 0}, registers = 0, shared_bytes = 0;
};

class CuptiTrace {
 public:
  static CuptiTrace& get() {
    static CuptiTrace t;
    return t;
  }
  // false (with the reason) when CUPTI cannot be loaded: the caller falls back to event timing
  bool available(std::string* why = nullptr) {
    std::lock_guard<std::mutex> g(mu_);
    if (!lib_ && !load(why)) return false;
    return true;
  }
  void start() {
    std::string why;
    if (!available(&why)) throw std::runtime_error("cupti: " + why);
    std::lock_guard<std::mutex> g(mu_);
    if (on_) return;
    check(RegisterCallbacks_(&CuptiTrace::requested, &CuptiTrace::completed), "register callbacks");
    check(Enable_(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL), "enable kernel activity");
    on_ = true;
  }
  // Everything recorded since the last collect (flushes CUPTI's buffers; call after synchronising the streams).
  std::vector<KernelRecord> collect() {
    if (lib_) FlushAll_(1);      // CUPTI_ACTIVITY_FLAG_FLUSH_FORCED: also hand over partly filled buffers
    std::lock_guard<std::mutex> g(mu_);
    std::vector<KernelRecord> out;
    out.swap(records_);
    return out;
  }
  std::vector<KernelRecord> stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (!on_) return {};
      on_ = false;
    }
    auto out = collect();
    Disable_(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL);
    return out;
  }
  uint64_t dropped() const { return dropped_; }

 private:
  void* lib_ = nullptr;
  bool on_ = false;
  std::mutex mu_;
  std::vector<KernelRecord> records_;
  uint64_t dropped_ = 0;
  CUptiResult (*RegisterCallbacks_)(CUpti_BuffersCallbackRequestFunc, CUpti_BuffersCallbackCompleteFunc) = nullptr;
  CUptiResult (*Enable_)(CUpti_ActivityKind) = nullptr;
  CUptiResult (*Disable_)(CUpti_ActivityKind) = nullptr;
  CUptiResult (*FlushAll_)(uint32_t) = nullptr;
  CUptiResult (*GetNextRecord_)(uint8_t*, size_t, CUpti_Activity**) = nullptr;
  CUptiResult (*GetNumDropped_)(CUcontext, uint32_t, size_t*) = nullptr;
  CUptiResult (*ResultString_)(CUptiResult, const char**) = nullptr;

  bool load(std::string* why) {
    const char* env = std::getenv("KERN_CUPTI_LIB");
    const char* names[] = {env, "libcupti.so.12", "libcupti.so", "/usr/local/cuda/targets/x86_64-linux/lib/libcupti.so.12",
                           "/usr/local/cuda/extras/CUPTI/lib64/libcupti.so.12"};
    std::string err;
    for (const char* n : names) {
      if (!n || !*n) continue;
      lib_ = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (lib_) break;
      err = dlerror();
    }
    if (!lib_) {
      if (why) *why = "no libcupti could be loaded (" + err + "); set KERN_CUPTI_LIB";
      return false;
    }
    auto sym = [&](const char* n) { return dlsym(lib_, n); };
    RegisterCallbacks_ = reinterpret_cast<decltype(RegisterCallbacks_)>(sym("cuptiActivityRegisterCallbacks"));
    Enable_ = reinterpret_cast<decltype(Enable_)>(sym("cuptiActivityEnable"));
    Disable_ = reinterpret_cast<decltype(Disable_)>(sym("cuptiActivityDisable"));
    FlushAll_ = reinterpret_cast<decltype(FlushAll_)>(sym("cuptiActivityFlushAll"));
    GetNextRecord_ = reinterpret_cast<decltype(GetNextRecord_)>(sym("cuptiActivityGetNextRecord"));
    GetNumDropped_ = reinterpret_cast<decltype(GetNumDropped_)>(sym("cuptiActivityGetNumDroppedRecords"));
    ResultString_ = reinterpret_cast<decltype(ResultString_)>(sym("cuptiGetResultString"));
    if (!RegisterCallbacks_ || !Enable_ || !Disable_ || !FlushAll_ || !GetNextRecord_) {
      if (why) *why = "libcupti lacks the activity API";
      dlclose(lib_);
      lib_ = nullptr;
      return false;
    }
    return true;
  }
  void check(CUptiResult r, const char* what) {
    if (r == CUPTI_SUCCESS) return;
    const char* s = nullptr;
    if (ResultString_) ResultString_(r, &s);
    throw std::runtime_error(std::string("cupti: ") + what + ": " + (s ? s : "error"));
  }
  static constexpr size_t kBuf = 8u << 20;     // 8 MiB per buffer
  static void CUPTIAPI requested(uint8_t** buffer, size_t* size, size_t* max_records) {
    void* p = nullptr;
    if (posix_memalign(&p, 8, kBuf) != 0) p = nullptr;
    *buffer = static_cast<uint8_t*>(p);
    *size = p ? kBuf : 0;
    *max_records = 0;
  }
  static void CUPTIAPI completed(CUcontext ctx, uint32_t stream, uint8_t* buffer, size_t, size_t valid) {
    CuptiTrace& t = get();
    if (buffer && valid) {
      std::lock_guard<std::mutex> g(t.mu_);
      CUpti_Activity* rec = nullptr;
      while (t.GetNextRecord_(buffer, valid, &rec) == CUPTI_SUCCESS) {
        if (rec->kind != CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL && rec->kind != CUPTI_ACTIVITY_KIND_KERNEL) continue;
        const auto* k = reinterpret_cast<const CUpti_ActivityKernel9*>(rec);
        KernelRecord r;
        r.name = k->name ? k->name : "";
        r.start_ns = k->start;
        r.end_ns = k->end;
        r.stream = k->streamId;
        r.grid[0] = (uint32_t)k->gridX; r.grid[1] = (uint32_t)k->gridY; r.grid[2] = (uint32_t)k->gridZ;
        r.block[0] = (uint32_t)k->blockX; r.block[1] = (uint32_t)k->blockY; r.block[2] = (uint32_t)k->blockZ;
        r.registers = k->registersPerThread;
        r.shared_bytes = (uint32_t)k->staticSharedMemory + (uint32_t)k->dynamicSharedMemory;
        t.records_.push_back(std::move(r));
      }
      size_t dropped = 0;
      if (t.GetNumDropped_ && t.GetNumDropped_(ctx, stream, &dropped) == CUPTI_SUCCESS) t.dropped_ += dropped;
    }
    std::free(buffer);
  }
};

}  // namespace kern
