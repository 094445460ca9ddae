// libkern_capture.so — an injection library that writes down how a process launches its kernels, so that a kernel of
// another project can be launched from a manifest without that project's host code:
//
//     CUDA_INJECTION64_PATH=.../libkern_capture.so KERN_CAPTURE_DIR=/some/dir  ./any_cuda_program
//
// writes /some/dir/pid<N>/launches.jsonl, one JSON object per line:
//
//     {"kind":"module", "t_ns", "handle", "sha256", "bytes", "format": "elf"|"fatbin"|"text"}
//     {"kind":"alloc",  "t_ns", "ptr", "bytes"}          {"kind":"free", "t_ns", "ptr"}
//     {"kind":"tensormap", "t_ns", "id", "hex" (the 128 encoded bytes), "dtype", "rank", "address", "dims", "strides",
//      "box", "elem_strides", "interleave", "swizzle", "l2_promotion", "oob_fill"}
//     {"kind":"launch", "t_ns", "symbol", "module" (sha256 or null), "grid", "block", "smem", "cluster", "cooperative",
//      "attrs": {"regs","static_smem","max_dyn_smem","local"}, "params": [{"index","offset","size","hex",
//      "pointers":[{"at","base","offset","bytes"}], "tensormaps":[{"at","id"}]}]}
//
// The staged bytes of every parameter are recorded as the launch call holds them (its offset and size come from the
// driver's own description of the function); an 8-byte word that points into a live allocation is marked with the
// allocation it falls into, and a 128-byte run equal to a descriptor that the process encoded is marked with that
// descriptor's record, wherever in a struct it sits. Module images are hashed, never stored: a manifest pins a module by
// the sha256 of its file, which is what the hash of a loaded image reproduces.
//
// The library subscribes to the driver-API callback domain of the profiling interface, which it opens at run time
// (`KERN_CUPTI_LIB` names the file if the loader cannot find one) and tells calls apart by the name the callback
// carries, so it builds without the interface's headers. `KERN_CAPTURE_SYMBOL` keeps launches whose symbol contains
// the text; `KERN_CAPTURE_MAX` (default 200000) bounds the launch records of one process.
//
// `kern_b200/capture.py` reads the file: `lift` turns one launch into a manifest launch skeleton, `mine` finds forward
// passes, classifies pointers and fits grid and scalar expressions.
// Reference counterpart: tools/kernel-capture/capture.c (what is recorded), tools/kernel-capture/README.md (workflow).
#include <dlfcn.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <cinttypes>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common/sha256.hpp"

namespace {

// ---- the slice of the profiling interface this file uses (layouts are part of its public ABI) ----
struct CallbackData {
  uint32_t site;                  // 0 on entry, 1 on exit
  const char* function_name;      // "cuLaunchKernel", "cuMemAlloc_v2", ...
  const void* params;             // the call's arguments, in order, as a struct
  void* return_value;             // CUresult* on exit
  const char* symbol_name;        // the kernel's name for launches
  void* context;
  uint32_t context_uid;
  uint64_t* correlation_data;
  uint32_t correlation_id;
};
using Callback = void (*)(void* user, int domain, uint32_t id, const void* data);
constexpr int kDomainDriver = 1;

// ---- argument structs of the driver calls that are read (argument order of the public prototypes) ----
struct LaunchKernelArgs { void* f; unsigned gx, gy, gz, bx, by, bz, smem; void* stream; void** params; void** extra; };
struct LaunchCoopArgs { void* f; unsigned gx, gy, gz, bx, by, bz, smem; void* stream; void** params; };
struct LaunchAttr { int id; int pad; unsigned char value[64]; };
struct LaunchConfig { unsigned gx, gy, gz, bx, by, bz, smem; void* stream; LaunchAttr* attrs; unsigned n_attrs; };
struct LaunchExArgs { const LaunchConfig* config; void* f; void** params; void** extra; };
struct ModuleLoadDataArgs { void** module; const void* image; };
struct MemAllocArgs { uint64_t* dptr; size_t bytes; };
struct MemFreeArgs { uint64_t dptr; };
struct AddressReserveArgs { uint64_t* ptr; size_t size; size_t alignment; uint64_t addr; unsigned long long flags; };
struct TensorMapTiledArgs {
  void* map; int dtype; uint32_t rank; void* address; const uint64_t* dims; const uint64_t* strides;
  const uint32_t* box; const uint32_t* elem_strides; int interleave; int swizzle; int l2; int oob;
};
constexpr int kAttrClusterDim = 4, kAttrCooperative = 2;

struct Alloc { uint64_t bytes; };
struct Map { unsigned char bytes[128]; uint64_t id; };

std::mutex g_mu;
FILE* g_out = nullptr;
std::map<uint64_t, Alloc> g_allocs;          // base -> size
std::vector<Map> g_maps;
std::map<void*, std::string> g_modules;      // CUmodule -> sha256
uint64_t g_launches = 0, g_max = 200000, g_map_ids = 0;
const char* g_filter = nullptr;
thread_local bool t_inside = false;

int (*cuFuncGetParamInfo_)(void*, size_t, size_t*, size_t*) = nullptr;
int (*cuFuncGetModule_)(void**, void*) = nullptr;
int (*cuFuncGetAttribute_)(int*, int, void*) = nullptr;
int (*cuFuncGetName_)(const char**, void*) = nullptr;
std::vector<std::pair<size_t, size_t>> g_test_layout;   // stands in for the driver's description where there is no driver

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

std::string hex(const unsigned char* p, size_t n) {
  static const char* x = "0123456789abcdef";
  std::string s(2 * n, '0');
  for (size_t i = 0; i < n; ++i) { s[2 * i] = x[p[i] >> 4]; s[2 * i + 1] = x[p[i] & 15]; }
  return s;
}

std::string quoted(const char* s) {
  std::string o = "\"";
  for (; s && *s; ++s) {
    if (*s == '"' || *s == '\\') { o += '\\'; o += *s; }
    else if ((unsigned char)*s < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", *s); o += b; }
    else o += *s;
  }
  return o + "\"";
}

// How many bytes a module image spans, from its own header, and which kind it is.
size_t image_size(const void* image, const char** format) {
  const unsigned char* p = static_cast<const unsigned char*>(image);
  uint32_t magic;
  memcpy(&magic, p, 4);
  if (magic == 0x466243B1u) {                   // a wrapper {magic, version, const void* data, ...}: follow it
    const void* data;
    memcpy(&data, p + 8, sizeof data);
    return data ? image_size(data, format) : 0;
  }
  if (magic == 0xBA55ED50u) {                   // fat binary: {magic, u16 version, u16 header size, u64 payload size}
    uint16_t header;
    uint64_t payload;
    memcpy(&header, p + 6, 2);
    memcpy(&payload, p + 8, 8);
    *format = "fatbin";
    return (size_t)header + (size_t)payload;
  }
  if (memcmp(p, "\x7f" "ELF", 4) == 0 && p[4] == 2) {   // ELF64: the furthest byte any table or section reaches
    uint64_t shoff, phoff;
    uint16_t shentsize, shnum, phentsize, phnum;
    memcpy(&phoff, p + 0x20, 8);
    memcpy(&shoff, p + 0x28, 8);
    memcpy(&phentsize, p + 0x36, 2);
    memcpy(&phnum, p + 0x38, 2);
    memcpy(&shentsize, p + 0x3A, 2);
    memcpy(&shnum, p + 0x3C, 2);
    uint64_t end = 64;
    if (shoff) end = std::max<uint64_t>(end, shoff + (uint64_t)shentsize * shnum);
    if (phoff) end = std::max<uint64_t>(end, phoff + (uint64_t)phentsize * phnum);
    for (uint16_t i = 0; shoff && i < shnum; ++i) {
      const unsigned char* sh = p + shoff + (uint64_t)i * shentsize;
      uint32_t type;
      uint64_t off, size;
      memcpy(&type, sh + 4, 4);
      memcpy(&off, sh + 0x18, 8);
      memcpy(&size, sh + 0x20, 8);
      if (type != 8) end = std::max(end, off + size);   // 8: a section that occupies no file bytes
    }
    *format = "elf";
    return (size_t)end;
  }
  *format = "text";
  return strnlen(reinterpret_cast<const char*>(p), (size_t)1 << 28);
}

void emit(const std::string& line) {
  if (!g_out) return;
  fputs(line.c_str(), g_out);
  fputc('\n', g_out);
  fflush(g_out);
}

template <typename T>
std::string list_of(const T* v, size_t n) {
  std::string o = "[";
  for (size_t i = 0; v && i < n; ++i) o += (i ? "," : "") + std::to_string((unsigned long long)v[i]);
  return o + "]";
}

void on_module(const void* image, void* handle) {
  if (!image) return;
  const char* format = "?";
  const size_t n = image_size(image, &format);
  uint32_t magic;
  memcpy(&magic, image, 4);
  const void* bytes = image;
  if (magic == 0x466243B1u) memcpy(&bytes, static_cast<const unsigned char*>(image) + 8, sizeof bytes);
  kern::Sha256 h;
  h.update(bytes, n);
  const std::string sha = kern::Sha256::hex(h.finish());
  char b[64];
  snprintf(b, sizeof b, "\"0x%" PRIx64 "\"", (uint64_t)(uintptr_t)handle);
  std::lock_guard<std::mutex> g(g_mu);
  g_modules[handle] = sha;
  emit("{\"kind\":\"module\",\"t_ns\":" + std::to_string(now_ns()) + ",\"handle\":" + b + ",\"sha256\":\"" + sha +
       "\",\"bytes\":" + std::to_string(n) + ",\"format\":\"" + format + "\"}");
}

void on_alloc(uint64_t ptr, uint64_t bytes) {
  char b[160];
  snprintf(b, sizeof b, "{\"kind\":\"alloc\",\"t_ns\":%" PRIu64 ",\"ptr\":\"0x%" PRIx64 "\",\"bytes\":%" PRIu64 "}", now_ns(), ptr, bytes);
  std::lock_guard<std::mutex> g(g_mu);
  g_allocs[ptr] = Alloc{bytes};
  emit(b);
}

void on_free(uint64_t ptr) {
  char b[128];
  snprintf(b, sizeof b, "{\"kind\":\"free\",\"t_ns\":%" PRIu64 ",\"ptr\":\"0x%" PRIx64 "\"}", now_ns(), ptr);
  std::lock_guard<std::mutex> g(g_mu);
  if (g_allocs.erase(ptr)) emit(b);
}

void on_tensormap(const TensorMapTiledArgs& a) {
  if (!a.map || a.rank == 0 || a.rank > 5) return;
  Map m;
  memcpy(m.bytes, a.map, 128);
  char head[256];
  std::lock_guard<std::mutex> g(g_mu);
  m.id = g_map_ids++;
  // a descriptor that is encoded again with the same bytes is the same descriptor
  for (const Map& old : g_maps)
    if (memcmp(old.bytes, m.bytes, 128) == 0) return;
  g_maps.push_back(m);
  snprintf(head, sizeof head, "{\"kind\":\"tensormap\",\"t_ns\":%" PRIu64 ",\"id\":%" PRIu64 ",\"dtype\":%d,\"rank\":%u,\"address\":\"0x%" PRIx64 "\"",
           now_ns(), m.id, a.dtype, a.rank, (uint64_t)(uintptr_t)a.address);
  emit(std::string(head) + ",\"hex\":\"" + hex(m.bytes, 128) + "\",\"dims\":" + list_of(a.dims, a.rank) + ",\"strides\":" +
       list_of(a.strides, a.rank - 1) + ",\"box\":" + list_of(a.box, a.rank) + ",\"elem_strides\":" + list_of(a.elem_strides, a.rank) +
       ",\"interleave\":" + std::to_string(a.interleave) + ",\"swizzle\":" + std::to_string(a.swizzle) + ",\"l2_promotion\":" +
       std::to_string(a.l2) + ",\"oob_fill\":" + std::to_string(a.oob) + "}");
}

// One parameter's bytes with what was recognised inside them. Called with g_mu held.
std::string param_json(size_t index, size_t offset, size_t size, const unsigned char* bytes) {
  std::string o = "{\"index\":" + std::to_string(index) + ",\"offset\":" + std::to_string(offset) + ",\"size\":" + std::to_string(size) +
                  ",\"hex\":\"" + hex(bytes, size) + "\"";
  std::string ptrs, maps;
  std::vector<bool> in_map(size, false);
  for (size_t at = 0; at + 128 <= size; at += 8)
    for (const Map& m : g_maps)
      if (memcmp(bytes + at, m.bytes, 128) == 0) {
        maps += std::string(maps.empty() ? "" : ",") + "{\"at\":" + std::to_string(at) + ",\"id\":" + std::to_string(m.id) + "}";
        for (size_t i = at; i < at + 128; ++i) in_map[i] = true;
        break;
      }
  for (size_t at = 0; at + 8 <= size; at += 8) {
    if (in_map[at]) continue;
    uint64_t v;
    memcpy(&v, bytes + at, 8);
    if (v < 4096) continue;
    auto it = g_allocs.upper_bound(v);
    if (it == g_allocs.begin()) continue;
    --it;
    if (v >= it->first + it->second.bytes) continue;
    char b[160];
    snprintf(b, sizeof b, "{\"at\":%zu,\"base\":\"0x%" PRIx64 "\",\"offset\":%" PRIu64 ",\"bytes\":%" PRIu64 "}", at, it->first,
             v - it->first, it->second.bytes);
    ptrs += std::string(ptrs.empty() ? "" : ",") + b;
  }
  if (!ptrs.empty()) o += ",\"pointers\":[" + ptrs + "]";
  if (!maps.empty()) o += ",\"tensormaps\":[" + maps + "]";
  return o + "}";
}

void on_launch(void* f, const char* symbol, const unsigned* grid, const unsigned* block, unsigned smem, void** params, void** extra,
               const unsigned* cluster, bool cooperative) {
  const char* name = symbol;
  if (!name && cuFuncGetName_) cuFuncGetName_(&name, f);
  if (!name) name = "?";
  if (g_filter && !strstr(name, g_filter)) return;
  // the argument buffer of an `extra`-style launch: {1, buffer, 2, &size, 0}
  const unsigned char* buffer = nullptr;
  size_t buffer_size = 0;
  for (void** e = extra; e && *e; e += 2) {
    if (*e == (void*)1) buffer = static_cast<const unsigned char*>(e[1]);
    if (*e == (void*)2) buffer_size = *static_cast<size_t*>(e[1]);
  }
  std::string ps;
  std::vector<std::pair<size_t, size_t>> layout;
  for (size_t i = 0; cuFuncGetParamInfo_ && i < 512; ++i) {
    size_t off = 0, size = 0;
    if (cuFuncGetParamInfo_(f, i, &off, &size) != 0) break;
    layout.emplace_back(off, size);
  }
  if (!cuFuncGetParamInfo_) layout = g_test_layout;
  void* module = nullptr;
  if (cuFuncGetModule_) cuFuncGetModule_(&module, f);
  int regs = -1, static_smem = -1, max_dyn = -1, local = -1;
  if (cuFuncGetAttribute_) {
    cuFuncGetAttribute_(&static_smem, 1, f);   // shared bytes fixed at compile time
    cuFuncGetAttribute_(&local, 3, f);         // local bytes per thread
    cuFuncGetAttribute_(&regs, 4, f);          // registers per thread
    cuFuncGetAttribute_(&max_dyn, 8, f);       // the dynamic shared size the function was opted into
  }
  std::lock_guard<std::mutex> g(g_mu);
  if (g_launches >= g_max) return;
  ++g_launches;
  for (size_t i = 0; i < layout.size(); ++i) {
    const unsigned char* bytes = nullptr;
    if (params) bytes = static_cast<const unsigned char*>(params[i]);
    else if (buffer && layout[i].first + layout[i].second <= buffer_size) bytes = buffer + layout[i].first;
    if (!bytes) continue;
    ps += (ps.empty() ? "" : ",") + param_json(i, layout[i].first, layout[i].second, bytes);
  }
  auto mod = g_modules.find(module);
  char head[256];
  snprintf(head, sizeof head, "{\"kind\":\"launch\",\"t_ns\":%" PRIu64 ",\"symbol\":", now_ns());
  emit(std::string(head) + quoted(name) + ",\"module\":" + (mod == g_modules.end() ? std::string("null") : "\"" + mod->second + "\"") +
       ",\"grid\":" + list_of(grid, 3) + ",\"block\":" + list_of(block, 3) + ",\"smem\":" + std::to_string(smem) + ",\"cluster\":" +
       (cluster ? list_of(cluster, 3) : std::string("null")) + ",\"cooperative\":" + (cooperative ? "true" : "false") +
       ",\"attrs\":{\"regs\":" + std::to_string(regs) + ",\"static_smem\":" + std::to_string(static_smem) + ",\"max_dyn_smem\":" +
       std::to_string(max_dyn) + ",\"local\":" + std::to_string(local) + "},\"params\":[" + ps + "]}");
}

bool is(const char* name, const char* call) {           // "cuLaunchKernel" also as "cuLaunchKernel_ptsz", "_v2", ...
  const size_t n = strlen(call);
  return strncmp(name, call, n) == 0 && (name[n] == 0 || name[n] == '_');
}

void callback(void*, int domain, uint32_t, const void* data) {
  if (domain != kDomainDriver || t_inside) return;
  const CallbackData& d = *static_cast<const CallbackData*>(data);
  const char* fn = d.function_name;
  if (!fn || fn[0] != 'c' || fn[1] != 'u') return;
  t_inside = true;
  const bool ok = d.site == 1 && d.return_value && *static_cast<int*>(d.return_value) == 0;
  if (d.site == 0) {
    if (is(fn, "cuLaunchKernelEx")) {
      const auto& a = *static_cast<const LaunchExArgs*>(d.params);
      if (a.config) {
        const LaunchConfig& c = *a.config;
        const unsigned grid[3] = {c.gx, c.gy, c.gz}, block[3] = {c.bx, c.by, c.bz};
        unsigned cluster[3] = {0, 0, 0};
        bool has_cluster = false, coop = false;
        for (unsigned i = 0; c.attrs && i < c.n_attrs; ++i) {
          if (c.attrs[i].id == kAttrClusterDim) { memcpy(cluster, c.attrs[i].value, 12); has_cluster = true; }
          if (c.attrs[i].id == kAttrCooperative) { int v; memcpy(&v, c.attrs[i].value, 4); coop = v != 0; }
        }
        on_launch(a.f, d.symbol_name, grid, block, c.smem, a.params, a.extra, has_cluster ? cluster : nullptr, coop);
      }
    } else if (is(fn, "cuLaunchCooperativeKernel")) {
      const auto& a = *static_cast<const LaunchCoopArgs*>(d.params);
      const unsigned grid[3] = {a.gx, a.gy, a.gz}, block[3] = {a.bx, a.by, a.bz};
      on_launch(a.f, d.symbol_name, grid, block, a.smem, a.params, nullptr, nullptr, true);
    } else if (is(fn, "cuLaunchKernel")) {
      const auto& a = *static_cast<const LaunchKernelArgs*>(d.params);
      const unsigned grid[3] = {a.gx, a.gy, a.gz}, block[3] = {a.bx, a.by, a.bz};
      on_launch(a.f, d.symbol_name, grid, block, a.smem, a.params, a.extra, nullptr, false);
    } else if (is(fn, "cuMemFree") || is(fn, "cuMemFreeAsync") || is(fn, "cuMemAddressFree")) {
      on_free(static_cast<const MemFreeArgs*>(d.params)->dptr);
    }
  } else if (ok) {
    if (is(fn, "cuModuleLoadData") || is(fn, "cuModuleLoadDataEx") || is(fn, "cuModuleLoadFatBinary") || is(fn, "cuLibraryLoadData")) {
      const auto& a = *static_cast<const ModuleLoadDataArgs*>(d.params);
      on_module(a.image, a.module ? *a.module : nullptr);
    } else if (is(fn, "cuMemAlloc") || is(fn, "cuMemAllocAsync") || is(fn, "cuMemAllocManaged") || is(fn, "cuMemAllocFromPoolAsync")) {
      const auto& a = *static_cast<const MemAllocArgs*>(d.params);
      if (a.dptr) on_alloc(*a.dptr, a.bytes);
    } else if (is(fn, "cuMemAddressReserve")) {
      const auto& a = *static_cast<const AddressReserveArgs*>(d.params);
      if (a.ptr) on_alloc(*a.ptr, a.size);
    } else if (is(fn, "cuTensorMapEncodeTiled")) {
      on_tensormap(*static_cast<const TensorMapTiledArgs*>(d.params));
    }
  }
  t_inside = false;
}

bool open_output() {
  const char* dir = getenv("KERN_CAPTURE_DIR");
  std::string base = dir && *dir ? dir : "kern_capture";
  mkdir(base.c_str(), 0755);
  base += "/pid" + std::to_string((long)getpid());
  mkdir(base.c_str(), 0755);
  if (g_out) fclose(g_out);
  g_out = fopen((base + "/launches.jsonl").c_str(), "w");
  if (!g_out) { fprintf(stderr, "kern_capture: cannot write under %s\n", base.c_str()); return false; }
  if (const char* m = getenv("KERN_CAPTURE_MAX")) g_max = strtoull(m, nullptr, 10);
  g_filter = getenv("KERN_CAPTURE_SYMBOL");
  if (g_filter && !*g_filter) g_filter = nullptr;
  fprintf(stderr, "kern_capture: writing %s/launches.jsonl\n", base.c_str());
  return true;
}

}  // namespace

// For tests on a machine without a driver: open the output, describe the next launches' parameters, and hand the
// recorder one call as the callback interface would (`params` is the call's argument struct).
extern "C" int kern_capture_open(void) { return open_output() ? 1 : 0; }
extern "C" void kern_capture_layout(const size_t* offsets, const size_t* sizes, size_t n) {
  g_test_layout.clear();
  for (size_t i = 0; i < n; ++i) g_test_layout.emplace_back(offsets[i], sizes[i]);
}
extern "C" void kern_capture_feed(const char* function_name, int site, const void* params, int result, const char* symbol) {
  CallbackData d{};
  d.site = (uint32_t)site;
  d.function_name = function_name;
  d.params = params;
  d.return_value = &result;
  d.symbol_name = symbol;
  callback(nullptr, kDomainDriver, 0, &d);
}

// The driver calls this once, when the process initialises CUDA with CUDA_INJECTION64_PATH naming this file.
extern "C" int InitializeInjection(void) {
  if (!open_output()) return 0;

  if (void* cuda = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL)) {
    cuFuncGetParamInfo_ = reinterpret_cast<decltype(cuFuncGetParamInfo_)>(dlsym(cuda, "cuFuncGetParamInfo"));
    cuFuncGetModule_ = reinterpret_cast<decltype(cuFuncGetModule_)>(dlsym(cuda, "cuFuncGetModule"));
    cuFuncGetAttribute_ = reinterpret_cast<decltype(cuFuncGetAttribute_)>(dlsym(cuda, "cuFuncGetAttribute"));
    cuFuncGetName_ = reinterpret_cast<decltype(cuFuncGetName_)>(dlsym(cuda, "cuFuncGetName"));
  }
  const char* names[] = {getenv("KERN_CUPTI_LIB"), "libcupti.so.12", "libcupti.so", "/usr/local/cuda/targets/x86_64-linux/lib/libcupti.so.12",
                         "/usr/local/cuda/extras/CUPTI/lib64/libcupti.so.12"};
  void* lib = nullptr;
  for (const char* n : names)
    if (n && *n && (lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
  if (!lib) { fprintf(stderr, "kern_capture: no libcupti could be loaded; set KERN_CUPTI_LIB\n"); return 0; }
  auto subscribe = reinterpret_cast<int (*)(void**, Callback, void*)>(dlsym(lib, "cuptiSubscribe"));
  auto enable = reinterpret_cast<int (*)(uint32_t, void*, int)>(dlsym(lib, "cuptiEnableDomain"));
  void* subscriber = nullptr;
  if (!subscribe || !enable || subscribe(&subscriber, callback, nullptr) != 0 || enable(1, subscriber, kDomainDriver) != 0) {
    fprintf(stderr, "kern_capture: the callback interface refused the subscription (another tool may hold it)\n");
    return 0;
  }
  return 1;
}
