// Runtime: load, allocation, weights (see runtime.hpp). Compilation and execution live in exec.cpp.
#include "runtime.hpp"

#include <algorithm>
#include <cstdio>

#include <cstdio>
#include <cstdlib>

#include <dirent.h>

#include <fstream>
#include <numeric>
#include <sstream>

#include "../common/sha256.hpp"
#include "../manifest/verify.hpp"

namespace kern {

namespace {

std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

std::vector<std::string> list_dir(const std::string& dir, const std::string& suffix) {
  std::vector<std::string> out;
  DIR* d = opendir(dir.c_str());
  if (!d) return out;
  while (dirent* e = readdir(d)) {
    std::string n = e->d_name;
    if (n.size() > suffix.size() && n.compare(n.size() - suffix.size(), suffix.size(), suffix) == 0) out.push_back(dir + "/" + n);
  }
  closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}

uint64_t lcm64(uint64_t a, uint64_t b) { return a / std::gcd(a, b) * b; }

}  // namespace

Runtime::Runtime(Manifest manifest, std::string kernels_dir, int gpu, std::map<std::string, GroupRank> topology,
                 Capacity cap, uint64_t stream)
    : m_(std::move(manifest)), kernels_dir_(std::move(kernels_dir)), topo_(std::move(topology)), cap_(cap) {
  // this rank's place in every group the manifest declares
  for (auto& kv : m_.topology) {
    auto it = topo_.find(kv.first);
    if (it == topo_.end()) {
      if (kv.second == 1) { topo_[kv.first] = GroupRank{0, 1}; continue; }
      throw std::runtime_error("the manifest declares group `" + kv.first + "` but this rank was given no place in it");
    }
    if (it->second.size != kv.second || it->second.index >= kv.second)
      throw std::runtime_error("group `" + kv.first + "`: the manifest declares " + std::to_string(kv.second) +
                               " members, this rank says it is " + std::to_string(it->second.index) + " of " +
                               std::to_string(it->second.size));
  }
  {
    Errors errs;
    // a hosted manifest computes hidden states for its host: no token output is demanded of it
    bool hosted = false;
    for (auto& kv : m_.states) hosted |= kv.second.host.has_value();
    proto_ = protocol_check(m_, !hosted && !m_.cut, errs);
    if (!proto_) { Errors e2; proto_ = protocol_check(m_, false, e2); }
  }
  dev_ = std::make_shared<Device>(gpu);
  if (stream) stream_ = reinterpret_cast<CUstream>(stream);
  else { stream_ = dev_->stream_create(); own_stream_ = true; }
  host_in_ = dev_->event_create(false);
  host_out_ = dev_->event_create(false);
  load_modules();
  allocate();
  if (!awaits_host()) compile_all();
}

Runtime::~Runtime() {
  try {
    dev_->make_current();
    Cuda::get().cuStreamSynchronize_(stream_);
    for (auto& g : graphs_) dev_->graph_destroy(g.second.exec);
    for (auto p : imported_ptrs_) dev_->ipc_close(p);
    for (auto& kv : nccl_comms_) NcclApi::get().CommDestroy(kv.second);
    for (auto& kv : buffers_) if (!kv.second.borrowed && !kv.second.host) dev_->free(kv.second.ptr - guard_);
    for (auto& kv : buffers_) if (!kv.second.borrowed && kv.second.host) dev_->host_free(reinterpret_cast<void*>(kv.second.ptr));
    for (auto& kv : states_) if (!kv.second.borrowed) dev_->free(kv.second.ptr - guard_);
    for (auto& o : scratch_) for (auto& kv : o.second) dev_->free(kv.second.ptr - guard_);
    if (err_word_) dev_->free(err_word_ - guard_);
    if (staging_) dev_->host_free(staging_);
    for (auto s : lane_streams_) Cuda::get().cuStreamDestroy_(s);
    for (auto e : lane_events_) Cuda::get().cuEventDestroy_(e);
    if (host_in_) Cuda::get().cuEventDestroy_(host_in_);
    if (host_out_) Cuda::get().cuEventDestroy_(host_out_);
    if (own_stream_) Cuda::get().cuStreamDestroy_(stream_);
  } catch (...) {
  }
}

uint64_t Runtime::rank(const std::string& group) const {
  auto it = topo_.find(group);
  if (it == topo_.end()) throw std::runtime_error("unknown group `" + group + "`");
  return it->second.index;
}

// The built-in modules (the kernels behind the `extern:` vocabulary) sit beside the package's own cubins, or, for a
// package that brings only its own, in the directory KERN_B200_KERNELS names (the in-tree kernels).
std::string Runtime::builtin_path(const std::string& file) const {
  const std::string here = kernels_dir_ + "/" + file;
  if (FILE* f = std::fopen(here.c_str(), "rb")) { std::fclose(f); return here; }
  if (const char* dir = std::getenv("KERN_B200_KERNELS")) return std::string(dir) + "/" + file;
  return here;
}

// Modules are found by the hash of their bytes: file names are labels. Every *.cubin under the
// kernels directory is hashed once; a manifest module resolves to the file with its sha256.
void Runtime::load_modules() {
  std::map<std::string, std::string> by_hash;   // sha256 -> path
  for (auto& path : list_dir(kernels_dir_, ".cubin")) by_hash[Sha256::hex_of(read_file(path))] = path;
  for (auto& kv : m_.modules) {
    auto it = by_hash.find(kv.second.sha256);
    if (it == by_hash.end())
      throw std::runtime_error("module `" + kv.first + "` (" + kv.second.source + "): no file under " + kernels_dir_ +
                               " has sha256 " + kv.second.sha256);
    modules_[kv.first] = dev_->load_module(read_file(it->second));
    // a checked build's module carries the range table and the failure record
    auto& cu = Cuda::get();
    CUdeviceptr spans = 0, count = 0, fail = 0;
    size_t sb = 0, cb = 0, fb = 0;
    if (cu.cuModuleGetGlobal_ && cu.cuModuleGetGlobal_(&spans, &sb, modules_[kv.first], "kern_spans") == CUDA_SUCCESS &&
        cu.cuModuleGetGlobal_(&count, &cb, modules_[kv.first], "kern_span_count") == CUDA_SUCCESS &&
        cu.cuModuleGetGlobal_(&fail, &fb, modules_[kv.first], "kern_check_fail") == CUDA_SUCCESS)
      checked_.push_back({kv.first, (uint64_t)spans, (uint64_t)count, (uint64_t)fail, (uint64_t)sb / 16});
  }
  // the built-in GEMM serves the `extern:cublaslt_*` / `extern:cublas_*` vocabulary
  bool needs_gemm = false;
  for (auto& okv : m_.ops)
    for (auto& l : okv.second.launches)
      needs_gemm |= l.is_extern && (l.entry.rfind("extern:cublaslt_bf16", 0) == 0 || l.entry.rfind("extern:cublas_bf16", 0) == 0);
  if (needs_gemm) builtin_gemm_ = dev_->load_module(read_file(builtin_path("gemm_bf16.cubin")));
  bool needs_gemm8 = false, needs_mx = false;
  for (auto& okv : m_.ops)
    for (auto& l : okv.second.launches) {
      needs_gemm8 |= l.is_extern && l.entry.rfind("extern:cublaslt_fp8", 0) == 0;
      needs_mx |= l.is_extern && l.entry == "extern:cublaslt_mxfp8_tn";
    }
  if (needs_gemm8) builtin_gemm8_ = dev_->load_module(read_file(builtin_path("gemm_fp8.cubin")));
  if (needs_mx) builtin_gemm_mx_ = dev_->load_module(read_file(builtin_path("gemm_mx.cubin")));
  // a multi-rank manifest runs only modules declared free of cluster-multicast copies
  bool multi = false;
  for (auto& kv : topo_) multi |= kv.second.size >= 2;
  if (multi) {
    Errors errs = verify_manifest(m_, true);
    std::string msg;
    for (auto& e : errs) if (e.find("multicast") != std::string::npos) msg += "\n  - " + e;
    if (!msg.empty()) throw std::runtime_error("refusing to load on 2 or more ranks:" + msg);
  }
}

void Runtime::allocate() {
  const VarMap vmax = m_.vars_at_max();
  // page unit: lcm of the strides of the tables that index a paged state
  page_unit_ = 1;
  for (auto& kv : m_.buffers) {
    const Buffer& b = kv.second;
    if (!b.domain || !b.domain->index_into || b.fill) continue;
    auto st = m_.states.find(*b.domain->index_into);
    if (st != m_.states.end() && st->second.is_paged()) page_unit_ = lcm64(page_unit_, std::max<uint64_t>(1, b.domain->stride));
  }
  guard_ = cap_.guard_bands ? 256 : 0;      // an exported handle carries the band's size as the region's offset
  auto zero_alloc = [&](uint64_t bytes, const std::string& name) {
    const uint64_t pay = (bytes ? bytes : 16);
    const uint64_t padded = (pay + 255) / 256 * 256;      // the trailing band starts 256-byte aligned, right after the payload's last line
    uint64_t p = dev_->alloc(padded + 2 * guard_);
    if (guard_) {
      dev_->memset8(p, 0xA5, guard_, stream_);
      dev_->memset8(p + guard_ + pay, 0xA5, padded - pay + guard_, stream_);
      guards_.push_back({name, p, pay});
    }
    dev_->memset8(p + guard_, 0, pay, stream_);
    return p + guard_;
  };
  err_word_ = zero_alloc(256, "error word");
  for (auto& kv : m_.buffers) {
    const Buffer& b = kv.second;
    auto bytes = b.bytes(vmax);
    if (!bytes) throw std::runtime_error("buffer `" + kv.first + "`: size overflows");
    Allocation a;
    a.bytes = *bytes;
    a.exported = b.export_;
    if (b.host_placement) {
      a.host = true;
      a.ptr = reinterpret_cast<uint64_t>(dev_->host_alloc(a.bytes));
    } else {
      a.ptr = zero_alloc(a.bytes, kv.first);
    }
    buffers_[kv.first] = a;
  }
  for (auto& okv : m_.ops)
    for (auto& skv : okv.second.scratch) {
      Buffer tmp;
      tmp.dtype = skv.second.dtype;
      tmp.shape = skv.second.shape;
      auto bytes = tmp.bytes(vmax);
      if (!bytes) throw std::runtime_error("op `" + okv.first + "` scratch `" + skv.first + "`: size overflows");
      Allocation a;
      a.bytes = *bytes;
      a.ptr = zero_alloc(a.bytes, okv.first + "." + skv.first);
      scratch_[okv.first][skv.first] = a;
    }
  // states: per-sequence and fixed first, then the paged ones share what is asked for (or what is left)
  slots_ = cap_.slots;
  uint64_t token_bytes = 0;
  for (auto& kv : m_.states) {
    const State& s = kv.second;
    StateAlloc a;
    if (!s.is_owned()) { a.borrowed = true; states_[kv.first] = a; continue; }
    if (s.is_per_seq()) {
      a.per_seq = true;
      a.unit_bytes = s.bytes_per_seq;
      a.units = slots_ + 1;
      a.bytes = a.unit_bytes * a.units;
      a.ptr = zero_alloc(a.bytes, kv.first);
    } else if (s.bytes) {
      a.bytes = s.bytes;
      a.ptr = zero_alloc(a.bytes, kv.first);
    } else {
      a.paged = true;
      token_bytes += s.bytes_per_token;
    }
    a.exported = true;   // every state is exportable: peer buffers and pushes may name it
    states_[kv.first] = a;
  }
  if (token_bytes) {
    uint64_t tokens = cap_.tokens;
    if (tokens == 0) {
      Cuda::get().cuStreamSynchronize_(stream_);
      auto info = dev_->mem_info();
      const uint64_t headroom = 1ull << 30;
      const uint64_t avail = info.first > headroom ? (uint64_t)((info.first - headroom) * cap_.memory_fraction) : 0;
      tokens = avail / token_bytes;
    }
    pages_ = tokens / page_unit_;
    if (pages_ == 0) throw std::runtime_error("no room for a single page of the paged states");
    for (auto& kv : m_.states) {
      StateAlloc& a = states_[kv.first];
      if (!a.paged) continue;
      a.unit_bytes = kv.second.bytes_per_token * page_unit_;
      a.units = pages_;
      a.bytes = a.unit_bytes * a.units;
      a.ptr = zero_alloc(a.bytes, kv.first);
    }
  }
}

void Runtime::publish_spans() {
  if (checked_.empty()) return;
  std::vector<std::pair<uint64_t, uint64_t>> spans;
  auto add = [&](uint64_t p, uint64_t bytes) {
    if (p && bytes) spans.push_back({p, p + (bytes + 255) / 256 * 256});
  };
  add(err_word_, 256);
  for (auto& kv : buffers_) add(kv.second.ptr, kv.second.bytes);
  for (auto& o : scratch_) for (auto& kv : o.second) add(kv.second.ptr, kv.second.bytes);
  for (auto& kv : states_) add(kv.second.ptr, kv.second.bytes);
  for (auto& kv : imported_) {          // a peer's copy of an exported buffer is as large as this rank's own
    auto b = m_.buffers.find(kv.first);
    if (b == m_.buffers.end() || !b->second.of) continue;
    auto own = buffers_.find(*b->second.of);
    if (own == buffers_.end()) continue;
    for (uint64_t a : kv.second) add(a, own->second.bytes);
  }
  std::sort(spans.begin(), spans.end());
  std::vector<uint64_t> flat;
  for (auto& s : spans) { flat.push_back(s.first); flat.push_back(s.second); }
  dev_->make_current();
  for (auto& c : checked_) {
    if (spans.size() > c.capacity)
      throw std::runtime_error("checked module `" + c.name + "`: " + std::to_string(spans.size()) + " address ranges, room for " + std::to_string(c.capacity));
    const int32_t n = (int32_t)spans.size();
    dev_->h2d(c.spans, flat.data(), flat.size() * 8, stream_);
    dev_->h2d(c.count, &n, 4, stream_);
  }
  dev_->stream_sync(stream_);
}

std::vector<std::string> Runtime::checked_failures() {
  std::vector<std::string> out;
  if (checked_.empty()) return out;
  dev_->make_current();
  dev_->stream_sync(stream_);
  for (auto& c : checked_) {
    uint64_t rec[2] = {0, 0};
    dev_->d2h(rec, c.fail, 16, stream_);
    dev_->stream_sync(stream_);
    if (rec[0] == 0) continue;
    char buf[160];
    std::snprintf(buf, sizeof buf, "module `%s`: check site %llu caught an access at 0x%llx outside every allocation (skipped)",
                  c.name.c_str(), (unsigned long long)(rec[0] >> 32), (unsigned long long)rec[1]);
    out.push_back(buf);
    const uint64_t zero[2] = {0, 0};
    dev_->h2d(c.fail, zero, 16, stream_);
    dev_->stream_sync(stream_);
  }
  return out;
}

std::vector<std::string> Runtime::check_guards() {
  std::vector<std::string> bad;
  if (!guard_) return bad;
  dev_->make_current();
  dev_->stream_sync(stream_);
  std::vector<uint8_t> band(2 * guard_ + 256);
  for (auto& g : guards_) {
    const uint64_t padded = (g.bytes + 255) / 256 * 256, tail = padded - g.bytes + guard_;
    dev_->d2h(band.data(), g.base, guard_, stream_);
    dev_->d2h(band.data() + guard_, g.base + guard_ + g.bytes, tail, stream_);
    dev_->stream_sync(stream_);
    bool before = true, after = true;
    for (uint64_t i = 0; i < guard_; ++i) before &= band[i] == 0xA5;
    for (uint64_t i = 0; i < tail; ++i) after &= band[guard_ + i] == 0xA5;
    if (!before) bad.push_back(g.name + " (before)");
    if (!after) bad.push_back(g.name + " (after)");
  }
  return bad;
}

bool Runtime::awaits_host() const {
  for (auto& kv : states_) if (kv.second.borrowed && kv.second.ptr == 0) return true;
  return false;
}

// A host engine hands over the memory of every host-declared state: (ptr, dtype, shape, strides).
// Each is checked against its declaration; only then are the programs compiled. Binding again
// replaces every host state, recompiles and drops every captured graph.
void Runtime::bind_host(const std::map<std::string, std::tuple<uint64_t, std::string, std::vector<uint64_t>, std::vector<uint64_t>>>& regions) {
  for (auto& kv : m_.states) {
    if (!kv.second.host) continue;
    auto it = regions.find(kv.first);
    if (it == regions.end()) throw std::runtime_error("host state `" + kv.first + "` was not bound");
    DType dt;
    if (!dtype_parse(std::get<1>(it->second), dt)) throw std::runtime_error("host state `" + kv.first + "`: unknown dtype");
    std::string why;
    auto bytes = kv.second.host->admit(dt, std::get<2>(it->second), std::get<3>(it->second), why);
    if (!bytes) throw std::runtime_error("host state `" + kv.first + "`: " + why);
    StateAlloc& a = states_[kv.first];
    a.ptr = std::get<0>(it->second);
    a.bytes = *bytes;
    a.borrowed = true;
  }
  for (auto& kv : regions)
    if (!m_.states.count(kv.first) || !m_.states.at(kv.first).host)
      throw std::runtime_error("`" + kv.first + "` is not a host state of this manifest");
  for (auto& g : graphs_) dev_->graph_destroy(g.second.exec);
  graphs_.clear();
  compile_all();
}

std::pair<uint64_t, uint64_t> Runtime::region(const std::string& name) const {
  auto b = buffers_.find(name);
  if (b != buffers_.end()) return {b->second.ptr, b->second.bytes};
  auto s = states_.find(name);
  if (s != states_.end()) return {s->second.ptr, s->second.bytes};
  throw std::runtime_error("no buffer or state named `" + name + "`");
}

void Runtime::ensure_staging(size_t bytes) {
  if (bytes <= staging_bytes_) return;
  if (staging_) { Cuda::get().cuStreamSynchronize_(stream_); dev_->host_free(staging_); }
  staging_bytes_ = std::max<size_t>(bytes, 1 << 20);
  staging_ = dev_->host_alloc(staging_bytes_);
}

void Runtime::write_input(const std::string& name, const void* data, size_t bytes, size_t offset) {
  auto it = buffers_.find(name);
  if (it == buffers_.end()) throw std::runtime_error("no buffer named `" + name + "`");
  if (offset + bytes > it->second.bytes) throw std::runtime_error("write past the end of buffer `" + name + "`");
  dev_->make_current();
  dev_->h2d(it->second.ptr + offset, data, bytes, stream_);
}

void Runtime::read_output(const std::string& name, void* out, size_t bytes, size_t offset) {
  auto r = region(name);
  if (offset + bytes > r.second) throw std::runtime_error("read past the end of `" + name + "`");
  dev_->make_current();
  dev_->d2h(out, r.first + offset, bytes, stream_);
  dev_->stream_sync(stream_);
}

void Runtime::synchronize() { dev_->stream_sync(stream_); }

void Runtime::upload(uint64_t dst, const uint8_t* src, size_t bytes) {
  // through pinned staging in 16 MiB pieces so the source pages stream in while the copy engine runs
  const size_t piece = 16u << 20;
  ensure_staging(2 * piece);
  uint8_t* st = static_cast<uint8_t*>(staging_);
  size_t done = 0;
  int half = 0;
  CUevent ev[2] = {dev_->event_create(false), dev_->event_create(false)};
  bool used[2] = {false, false};
  while (done < bytes) {
    const size_t n = std::min(piece, bytes - done);
    if (used[half]) Cuda::get().cuEventSynchronize_(ev[half]);
    std::memcpy(st + half * piece, src + done, n);
    dev_->h2d(dst + done, st + half * piece, n, stream_);
    dev_->event_record(ev[half], stream_);
    used[half] = true;
    done += n;
    half ^= 1;
  }
  dev_->stream_sync(stream_);
  Cuda::get().cuEventDestroy_(ev[0]);
  Cuda::get().cuEventDestroy_(ev[1]);
}

void Runtime::upload_2d(uint64_t dst, size_t dst_pitch, const uint8_t* src, size_t src_pitch, size_t width, size_t rows) {
  if (width == src_pitch && width == dst_pitch) { upload(dst, src, width * rows); return; }
  // gather the rows densely on the host, then one pitched device copy
  const size_t rows_per = std::max<size_t>(1, (16u << 20) / std::max<size_t>(1, width));
  ensure_staging(rows_per * width);
  uint8_t* st = static_cast<uint8_t*>(staging_);
  for (size_t r0 = 0; r0 < rows; r0 += rows_per) {
    const size_t n = std::min(rows_per, rows - r0);
    for (size_t r = 0; r < n; ++r) std::memcpy(st + r * width, src + (r0 + r) * src_pitch, width);
    CUDA_MEMCPY2D cp;
    std::memset(&cp, 0, sizeof cp);
    cp.srcMemoryType = CU_MEMORYTYPE_HOST;
    cp.srcHost = st;
    cp.srcPitch = width;
    cp.dstMemoryType = CU_MEMORYTYPE_DEVICE;
    cp.dstDevice = (CUdeviceptr)(dst + r0 * dst_pitch);
    cp.dstPitch = dst_pitch;
    cp.WidthInBytes = width;
    cp.Height = n;
    KERN_CU(cuMemcpy2DAsync_(&cp, stream_));
    dev_->stream_sync(stream_);
  }
}

// Bind every weight / source buffer from the checkpoint by tensor name: each `bind` segment is a
// tensor (or the member's tensor of a ranked list), optionally a row and a column range, or two
// tensors interleaved in blocks of n rows; segments fill the buffer in order and must fill it exactly.
void Runtime::load_weights(const std::vector<std::string>& paths) {
  if (weights_loaded_) throw std::runtime_error("weights were already loaded into this runtime");
  dev_->make_current();
  Safetensors st(paths);
  for (auto& kv : m_.buffers) {
    const Buffer& b = kv.second;
    if (b.kind != BufferKind::Weight && b.kind != BufferKind::Source) continue;
    const Allocation& dst = buffers_.at(kv.first);
    const uint64_t es = dtype_bytes(b.dtype);
    uint64_t at = 0;
    auto pick = [&](const TensorSource& t) -> const TensorInfo& {
      const std::string& name = t.ranked ? t.tensors.at(rank(t.group)) : t.name;
      const TensorInfo* ti = st.find(name);
      if (!ti) throw std::runtime_error("buffer `" + kv.first + "`: checkpoint has no tensor `" + name + "`");
      DType dt;
      if (!dtype_named(ti->dtype, dt) || dt != b.dtype)
        throw std::runtime_error("buffer `" + kv.first + "`: tensor `" + name + "` is " + ti->dtype + ", the buffer is " + dtype_name(b.dtype));
      return *ti;
    };
    auto range = [&](const std::optional<Ranges>& r, uint64_t whole) -> std::pair<uint64_t, uint64_t> {
      if (!r) return {0, whole};
      auto p = r->ranked ? r->ranges.at(rank(r->group)) : std::make_pair(r->range[0], r->range[1]);
      if (p.second > whole) throw std::runtime_error("buffer `" + kv.first + "`: range end " + std::to_string(p.second) + " is past the tensor's " + std::to_string(whole));
      return p;
    };
    for (auto& seg : b.bind) {
      const TensorInfo& t = pick(seg.tensor);
      const uint64_t rows = t.shape.empty() ? 1 : t.shape[0];
      uint64_t cols = 1;
      for (size_t i = 1; i < t.shape.size(); ++i) cols *= t.shape[i];
      if (rows * cols * es != t.bytes) throw std::runtime_error("tensor for `" + kv.first + "` has inconsistent size");
      auto place = [&](uint64_t need) {
        if (at + need > dst.bytes)
          throw std::runtime_error("buffer `" + kv.first + "`: bound tensors hold more than its " + std::to_string(dst.bytes) + " bytes");
      };
      if (seg.interleave) {
        const TensorInfo& u = pick(seg.interleave->with);
        if (u.shape != t.shape) throw std::runtime_error("buffer `" + kv.first + "`: interleaved tensors differ in shape");
        const uint64_t n = seg.interleave->rows;
        if (rows % n) throw std::runtime_error("buffer `" + kv.first + "`: " + std::to_string(rows) + " rows do not split into blocks of " + std::to_string(n));
        place(2 * t.bytes);
        const uint64_t blk = n * cols * es;
        uint8_t* pd = dst.host ? reinterpret_cast<uint8_t*>(dst.ptr) : nullptr;
        if (pd) {
          for (uint64_t i = 0; i < rows / n; ++i) {
            std::memcpy(pd + at + 2 * i * blk, t.data + i * blk, blk);
            std::memcpy(pd + at + (2 * i + 1) * blk, u.data + i * blk, blk);
          }
        } else {
          upload_2d(dst.ptr + at, 2 * blk, t.data, blk, blk, rows / n);
          upload_2d(dst.ptr + at + blk, 2 * blk, u.data, blk, blk, rows / n);
        }
        at += 2 * t.bytes;
        continue;
      }
      auto rr = range(seg.rows, rows), cr = range(seg.cols, cols);
      const uint64_t nr = rr.second - rr.first, width = (cr.second - cr.first) * es;
      place(nr * width);
      const uint8_t* src = t.data + (rr.first * cols + cr.first) * es;
      if (dst.host) {
        uint8_t* pd = reinterpret_cast<uint8_t*>(dst.ptr) + at;
        for (uint64_t r = 0; r < nr; ++r) std::memcpy(pd + r * width, src + r * cols * es, width);
      } else {
        upload_2d(dst.ptr + at, width, src, cols * es, width, nr);
      }
      at += nr * width;
    }
    if (at != dst.bytes)
      throw std::runtime_error("buffer `" + kv.first + "`: bound tensors hold " + std::to_string(at) + " bytes, the buffer " + std::to_string(dst.bytes));
  }
  weights_loaded_ = true;
  // derive programs run once over the sources, in declaration order
  for (auto& kv : m_.programs)
    if (kv.second.derive) {
      issue(kv.first, m_.vars_at_max(), true);
      synchronize();
    }
}

std::string Runtime::banner() const {
  std::ostringstream o;
  o << "model " << m_.model << " on gpu " << dev_->gpu() << " (" << dev_->sm_count() << " SMs)\n";
  o << "page unit " << page_unit_ << " tokens, " << pages_ << " pages, " << slots_ << " slots\n";
  for (auto& kv : states_) o << "state " << kv.first << " " << kv.second.bytes << " bytes\n";
  uint64_t wb = 0, ob = 0;
  for (auto& kv : buffers_) (m_.buffers.at(kv.first).kind == BufferKind::Weight ? wb : ob) += kv.second.bytes;
  o << "weights " << wb << " bytes, other buffers " << ob << " bytes\n";
  for (auto& okv : m_.ops)
    for (auto& l : okv.second.launches) o << "op " << okv.first << " -> " << (l.is_extern ? "built-in" : l.module) << ":" << l.entry << "\n";
  return o.str();
}

}  // namespace kern
