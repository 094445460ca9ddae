// Device layer of the native runtime: primary-context binding (shared with PyTorch in the same
// process), module loading, ABI introspection, kernel launch with cluster / programmatic-dependent
// launch attributes, TMA descriptor encoding, plain and VMM allocations, IPC export/import, streams,
// events and graph capture.
// (Reference parity: crates/kern-runtime/src/device.rs:122-352,366-438,629-659 — allocation, VMM,
// import/export, pinned host, events; crates/kern-runtime/src/compile.rs:885-959 — tensor maps;
// crates/kern-runtime/src/exec.rs:726-821 — launch with cluster and PDL attributes.)
#pragma once
#include <array>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "cuda_api.hpp"

namespace kern {

struct LaunchDims {
  unsigned grid[3] = {1, 1, 1};
  unsigned block[3] = {1, 1, 1};
  unsigned cluster[3] = {1, 1, 1};
  unsigned shared_mem = 0;
  bool pdl = false;
};

struct TensorMapSpec {
  // element type code, CUtensorMapDataType numbering:
  // 0 u8, 1 u16, 2 u32, 3 i32, 4 u64, 5 i64, 6 f16, 7 f32, 8 f64, 9 bf16, 10 f32 ftz, 11 tf32
  int dtype = 9;
  std::vector<uint64_t> dims;     // innermost first
  std::vector<uint64_t> strides;  // bytes, dims.size()-1 entries, multiples of 16
  std::vector<uint32_t> box;      // per dim, 1..256
  int swizzle = 0;                // 0 | 32 | 64 | 128 bytes
  int l2_promotion = 0;           // 0 | 64 | 128 | 256 bytes
  bool oob_nan = false;
};

class Device {
 public:
  explicit Device(int gpu) : gpu_(gpu) {
    auto& cu = Cuda::get();
    KERN_CU(cuDeviceGet_(&dev_, gpu));
    KERN_CU(cuDevicePrimaryCtxRetain_(&ctx_, dev_));
    KERN_CU(cuCtxSetCurrent_(ctx_));
    int v = 0;
    cu.cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dev_);
    sm_count_ = v;
    cu.cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, dev_);
    cc_major_ = v;
    cu.cuDeviceGetAttribute_(&v, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, dev_);
    cc_minor_ = v;
  }
  ~Device() {
    // modules are left to the context; releasing the primary context would pull it from under a
    // host framework that shares it
  }
  Device(const Device&) = delete;
  Device& operator=(const Device&) = delete;

  void make_current() const { KERN_CU(cuCtxSetCurrent_(ctx_)); }
  int gpu() const { return gpu_; }
  int sm_count() const { return sm_count_; }
  int cc() const { return cc_major_ * 10 + cc_minor_; }

  // ---- modules ----
  CUmodule load_module(const std::string& image) {
    make_current();
    CUmodule m = nullptr;
    KERN_CU(cuModuleLoadData_(&m, image.data()));
    return m;
  }
  CUfunction function(CUmodule m, const std::string& entry) {
    CUfunction f = nullptr;
    CUresult r = Cuda::get().cuModuleGetFunction_(&f, m, entry.c_str());
    if (r != CUDA_SUCCESS) throw std::runtime_error("entry `" + entry + "` not found in module");
    return f;
  }
  // Entry names by enumeration through the driver (no disassembly, no external tool).
  std::vector<std::string> entries(CUmodule m) {
    auto& cu = Cuda::get();
    unsigned n = 0;
    KERN_CU(cuModuleGetFunctionCount_(&n, m));
    std::vector<CUfunction> fs(n);
    if (n) KERN_CU(cuModuleEnumerateFunctions_(fs.data(), n, m));
    std::vector<std::string> out;
    for (auto f : fs) {
      const char* name = nullptr;
      if (cu.cuFuncGetName_ && cu.cuFuncGetName_(&name, f) == CUDA_SUCCESS && name) out.push_back(name);
    }
    return out;
  }
  // Byte size of every kernel parameter, in order: the ABI the manifest's declared params are
  // checked against at load.
  std::vector<size_t> param_sizes(CUfunction f) {
    std::vector<size_t> out;
    auto& cu = Cuda::get();
    for (size_t i = 0;; ++i) {
      size_t off = 0, sz = 0;
      CUresult r = cu.cuFuncGetParamInfo_(f, i, &off, &sz);
      if (r != CUDA_SUCCESS) break;
      out.push_back(sz);
    }
    return out;
  }

  void launch(CUfunction f, const LaunchDims& d, CUstream stream, void** params) {
    if (d.grid[0] == 0 || d.grid[1] == 0 || d.grid[2] == 0) return;  // an empty grid is a no-op
    auto& cu = Cuda::get();
    if (d.shared_mem > 48 * 1024) {
      auto it = smem_set_.find(f);
      if (it == smem_set_.end() || it->second < d.shared_mem) {
        KERN_CU(cuFuncSetAttribute_(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                    (int)d.shared_mem));
        smem_set_[f] = d.shared_mem;
      }
    }
    CUlaunchConfig cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = d.grid[0]; cfg.gridDimY = d.grid[1]; cfg.gridDimZ = d.grid[2];
    cfg.blockDimX = d.block[0]; cfg.blockDimY = d.block[1]; cfg.blockDimZ = d.block[2];
    cfg.sharedMemBytes = d.shared_mem;
    cfg.hStream = stream;
    CUlaunchAttribute attrs[2];
    unsigned na = 0;
    if (d.cluster[0] * d.cluster[1] * d.cluster[2] > 1) {
      attrs[na].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
      attrs[na].value.clusterDim.x = d.cluster[0];
      attrs[na].value.clusterDim.y = d.cluster[1];
      attrs[na].value.clusterDim.z = d.cluster[2];
      ++na;
    }
    if (d.pdl) {
      attrs[na].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
      attrs[na].value.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cu_check(cu.cuLaunchKernelEx_(&cfg, f, params, nullptr), "cuLaunchKernelEx");
  }

  // ---- TMA descriptors ----
  std::array<uint8_t, 128> encode_tensor_map(uint64_t base, const TensorMapSpec& s) {
    const size_t rank = s.dims.size();
    if (rank < 1 || rank > 5) throw std::runtime_error("tensor map rank must be 1..5");
    if (s.strides.size() + 1 != rank || s.box.size() != rank)
      throw std::runtime_error("tensor map strides/box do not match its rank");
    if (base % 16) throw std::runtime_error("tensor map base address must be 16-byte aligned");
    cuuint64_t dims[5], strides[5];
    cuuint32_t box[5], estr[5];
    for (size_t i = 0; i < rank; ++i) {
      dims[i] = s.dims[i];
      box[i] = s.box[i];
      estr[i] = 1;
      if (s.box[i] < 1 || s.box[i] > 256) throw std::runtime_error("tensor map box extent must be 1..256");
    }
    for (size_t i = 0; i + 1 < rank; ++i) {
      strides[i] = s.strides[i];
      if (s.strides[i] % 16) throw std::runtime_error("tensor map strides must be multiples of 16 bytes");
    }
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    switch (s.swizzle) {
      case 0: break;
      case 32: sw = CU_TENSOR_MAP_SWIZZLE_32B; break;
      case 64: sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
      case 128: sw = CU_TENSOR_MAP_SWIZZLE_128B; break;
      default: throw std::runtime_error("tensor map swizzle must be 0, 32, 64 or 128");
    }
    CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_NONE;
    switch (s.l2_promotion) {
      case 0: break;
      case 64: l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_64B; break;
      case 128: l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_128B; break;
      case 256: l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B; break;
      default: throw std::runtime_error("tensor map l2_promotion must be 0, 64, 128 or 256");
    }
    alignas(64) CUtensorMap tm;
    KERN_CU(cuTensorMapEncodeTiled_(
        &tm, (CUtensorMapDataType)s.dtype, (cuuint32_t)rank, reinterpret_cast<void*>(base), dims,
        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, l2,
        s.oob_nan ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA
                  : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    std::array<uint8_t, 128> out;
    static_assert(sizeof(CUtensorMap) == 128, "CUtensorMap is 128 bytes");
    std::memcpy(out.data(), &tm, 128);
    return out;
  }

  // ---- memory ----
  uint64_t alloc(size_t bytes) {
    make_current();
    CUdeviceptr p = 0;
    KERN_CU(cuMemAlloc_(&p, bytes ? bytes : 16));
    return (uint64_t)p;
  }
  void free(uint64_t p) { if (p) Cuda::get().cuMemFree_((CUdeviceptr)p); }
  std::pair<size_t, size_t> mem_info() {
    size_t f = 0, t = 0;
    KERN_CU(cuMemGetInfo_(&f, &t));
    return {f, t};
  }
  void memset8(uint64_t p, uint8_t v, size_t n, CUstream s) { KERN_CU(cuMemsetD8Async_((CUdeviceptr)p, v, n, s)); }
  void h2d(uint64_t dst, const void* src, size_t n, CUstream s) { KERN_CU(cuMemcpyHtoDAsync_((CUdeviceptr)dst, src, n, s)); }
  void d2h(void* dst, uint64_t src, size_t n, CUstream s) { KERN_CU(cuMemcpyDtoHAsync_(dst, (CUdeviceptr)src, n, s)); }
  void d2d(uint64_t dst, uint64_t src, size_t n, CUstream s) { KERN_CU(cuMemcpyDtoDAsync_((CUdeviceptr)dst, (CUdeviceptr)src, n, s)); }
  // `rows` rows of `width` bytes, device to device (either side may be mapped peer memory), rows `pitch` bytes apart
  void copy_2d(uint64_t dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch, uint64_t width, uint64_t rows, CUstream s) {
    if (rows == 0 || width == 0) return;
    if (rows == 1 || (dst_pitch == width && src_pitch == width)) { d2d(dst, src, width * rows, s); return; }
    CUDA_MEMCPY2D c;
    std::memset(&c, 0, sizeof(c));
    c.srcMemoryType = CU_MEMORYTYPE_DEVICE; c.srcDevice = (CUdeviceptr)src; c.srcPitch = src_pitch;
    c.dstMemoryType = CU_MEMORYTYPE_DEVICE; c.dstDevice = (CUdeviceptr)dst; c.dstPitch = dst_pitch;
    c.WidthInBytes = width; c.Height = rows;
    KERN_CU(cuMemcpy2DAsync_(&c, s));
  }
  void* host_alloc(size_t bytes) {
    void* p = nullptr;
    KERN_CU(cuMemHostAlloc_(&p, bytes ? bytes : 16, CU_MEMHOSTALLOC_PORTABLE));
    return p;
  }
  void host_free(void* p) { if (p) Cuda::get().cuMemFreeHost_(p); }

  // IPC handles for cuMemAlloc memory (64 bytes): the carrier between the one-process-per-GPU ranks of one box.
  // Every state and exported buffer is one cuMemAlloc; there is no cuMemCreate / cuMemMap pool.
  // `offset`: where the exported region starts inside its allocation (a handle names the whole allocation; a runtime
  // with guard bands keeps its payload behind the first band). It travels as eight more bytes after the handle.
  std::string ipc_export(uint64_t p, uint64_t offset = 0) {
    CUipcMemHandle h;
    KERN_CU(cuIpcGetMemHandle_(&h, (CUdeviceptr)p));
    std::string out(reinterpret_cast<const char*>(&h), sizeof(h));
    if (offset) out.append(reinterpret_cast<const char*>(&offset), sizeof(offset));
    return out;
  }
  // The mapped allocation's base; `offset_out` receives the region's offset inside it.
  uint64_t ipc_import(const std::string& handle, uint64_t* offset_out = nullptr) {
    make_current();
    if (handle.size() != sizeof(CUipcMemHandle) && handle.size() != sizeof(CUipcMemHandle) + 8)
      throw std::runtime_error("IPC handle must be 64 bytes (72 with a region offset)");
    CUipcMemHandle h;
    std::memcpy(&h, handle.data(), sizeof(h));
    uint64_t off = 0;
    if (handle.size() > sizeof(h)) std::memcpy(&off, handle.data() + sizeof(h), 8);
    if (off && !offset_out) throw std::runtime_error("this IPC handle carries a region offset the caller does not take");
    if (offset_out) *offset_out = off;
    CUdeviceptr p = 0;
    KERN_CU(cuIpcOpenMemHandle_(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
    return (uint64_t)p;
  }
  void ipc_close(uint64_t p) { Cuda::get().cuIpcCloseMemHandle_((CUdeviceptr)p); }

  // ---- streams, events, graphs ----
  CUstream stream_create() {
    make_current();
    CUstream s = nullptr;
    KERN_CU(cuStreamCreate_(&s, CU_STREAM_NON_BLOCKING));
    return s;
  }
  void stream_sync(CUstream s) { KERN_CU(cuStreamSynchronize_(s)); }
  CUevent event_create(bool timing) {
    CUevent e = nullptr;
    KERN_CU(cuEventCreate_(&e, timing ? CU_EVENT_DEFAULT : CU_EVENT_DISABLE_TIMING));
    return e;
  }
  void event_record(CUevent e, CUstream s) { KERN_CU(cuEventRecord_(e, s)); }
  void stream_wait(CUstream s, CUevent e) { KERN_CU(cuStreamWaitEvent_(s, e, 0)); }
  float event_ms(CUevent a, CUevent b) {
    float ms = 0;
    KERN_CU(cuEventElapsedTime_(&ms, a, b));
    return ms;
  }
  void begin_capture(CUstream s) { KERN_CU(cuStreamBeginCapture_(s, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL)); }
  CUgraphExec end_capture(CUstream s, size_t* nodes = nullptr) {
    CUgraph g = nullptr;
    KERN_CU(cuStreamEndCapture_(s, &g));
    if (nodes) {
      size_t n = 0;
      Cuda::get().cuGraphGetNodes_(g, nullptr, &n);
      *nodes = n;
    }
    CUgraphExec ex = nullptr;
    CUresult r = Cuda::get().cuGraphInstantiateWithFlags_(&ex, g, 0);
    Cuda::get().cuGraphDestroy_(g);
    cu_check(r, "cuGraphInstantiateWithFlags");
    return ex;
  }
  void graph_launch(CUgraphExec g, CUstream s) { KERN_CU(cuGraphLaunch_(g, s)); }
  void graph_destroy(CUgraphExec g) { if (g) Cuda::get().cuGraphExecDestroy_(g); }

 private:
  int gpu_ = 0;
  CUdevice dev_ = 0;
  CUcontext ctx_ = nullptr;
  int sm_count_ = 0, cc_major_ = 0, cc_minor_ = 0;
  std::map<CUfunction, unsigned> smem_set_;
};

}  // namespace kern
