// The executor: loads a verified manifest onto one GPU, allocates every buffer at its var upper bound
// and every pooled state as one allocation, resolves each launch to a function of a sha256-pinned
// module (ABI checked against the driver's view of the kernel's parameters), compiles every program to
// a flat launch list with its addresses baked in, and replays a program eagerly or as a CUDA graph
// keyed by the call's var values.
// Reference: crates/kern-runtime/src/lib.rs:90-400 (façade), load.rs:84-404, compile.rs:30-959,
// exec.rs:409-821, peers.rs:45-369, lease.rs, derive.rs.
#pragma once
#include <array>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <set>
#include <string>
#include <vector>

#include "../manifest/protocol.hpp"
#include "../manifest/types.hpp"
#include "device.hpp"
#include "push.hpp"
#include "nccl_api.hpp"
#include "safetensors.hpp"

namespace kern {

struct Capacity {
  uint64_t tokens = 0;     // token capacity of the paged states (0: fit what the device has left)
  uint64_t slots = 0;      // per-sequence state slots (excluding the null line)
  double memory_fraction = 0.9;   // of free device memory the paged states may take when tokens == 0
  bool guard_bands = false;       // test mode: a 256-byte canary band before and after every device allocation of the
                                  // runtime (buffers, scratch, states), checked by check_guards(); exported regions
                                  // carry the band's size in their handle, so peers' writes are covered too
};

struct GroupRank {
  uint64_t index = 0, size = 1;
};

struct Allocation {
  uint64_t ptr = 0;
  uint64_t bytes = 0;
  bool exported = false;
  bool host = false;
  bool borrowed = false;   // owned by someone else (host-bound state, resident weights)
};

struct StateAlloc : Allocation {
  uint64_t unit_bytes = 0;   // bytes per page (paged) or per slot (per-sequence); 0 for a fixed state
  uint64_t units = 0;        // pages or slots (including the null line)
  bool paged = false, per_seq = false;
};

// one parameter slot of a compiled launch: a byte image plus the places patched per call
struct Patch {
  uint32_t at = 0, width = 4;
  Expr expr;
};
struct CompiledArg {
  std::vector<uint8_t> image;
  std::vector<Patch> patches;
};

enum class ExternKind { None, GemmBf16, GemmBf16Acc, GemmBf16F32, GemmFp8, GemmFp8F32, GemmMxfp8, Nccl };

struct CompiledLaunch {
  std::string label;           // op name / call label for traces
  size_t call_index = 0;
  CUfunction fn = nullptr;
  ExternKind ext = ExternKind::None;
  uint32_t block[3] = {1, 1, 1};
  Expr grid[3];
  std::optional<Expr> shared_mem;
  uint32_t cluster[3] = {1, 1, 1};
  bool pdl = false;
  std::optional<When> when;
  std::vector<CompiledArg> args;
  uint8_t lane = 0;
  std::vector<uint8_t> after;   // lanes to wait for before the first launch of this call
  bool first_of_call = false;
  // extern GEMM operands
  uint64_t a_ptr = 0, w_ptr = 0, c_ptr = 0;
  uint64_t a_rows = 0, w_rows = 0;
  Expr m, n, k;
  std::optional<Expr> ldc, lda;
  uint64_t sa_ptr = 0, sw_ptr = 0;   // per-tensor f32 scales of an fp8 GEMM (device words)
  // extern collective: send = a_ptr (a_rows bytes behind it), recv = c_ptr (w_rows bytes), count = m (elements per rank)
  NcclColl coll = NcclColl::AllReduce;
  NcclElem elem = NcclElem::F32;
  std::string group;
};

struct CompiledProgram {
  std::string name;
  std::vector<CompiledLaunch> launches;
  std::vector<std::string> vars;   // the vars its launches read: the graph key
  bool graph = false;
  uint8_t lanes = 1;
};

class Runtime {
 public:
  Runtime(Manifest manifest, std::string kernels_dir, int gpu, std::map<std::string, GroupRank> topology, Capacity cap,
          uint64_t stream = 0);
  ~Runtime();
  Runtime(const Runtime&) = delete;

  const Manifest& manifest() const { return m_; }
  const Protocol* protocol() const { return proto_ ? &*proto_ : nullptr; }
  Device& device() { return *dev_; }
  uint64_t stream() const { return (uint64_t)stream_; }
  uint64_t page_unit() const { return page_unit_; }
  uint64_t pages() const { return pages_; }
  uint64_t slots() const { return slots_; }
  uint64_t rank(const std::string& group) const;

  // ---- weights ----
  void load_weights(const std::vector<std::string>& safetensors_paths);
  bool weights_loaded() const { return weights_loaded_; }

  // ---- IO ----
  std::pair<uint64_t, uint64_t> region(const std::string& name) const;   // (device ptr, bytes) of a buffer or state
  void write_input(const std::string& name, const void* data, size_t bytes, size_t offset = 0);
  void read_output(const std::string& name, void* out, size_t bytes, size_t offset = 0);
  void synchronize();

  // ---- execution ----
  void run_once_programs();
  // eager or captured according to the program and `eager`; returns the number of kernel launches issued
  // (a graph replay counts the launches its graph holds)
  size_t issue(const std::string& program, const VarMap& vars, bool eager = false);
  // One eager run with a CUDA event between calls: (call label, op, milliseconds) per call, in order.
  // Serialises the lanes (everything on the main stream); for cost-by-op reports, not for serving.
  struct CallTime {
    std::string label, op;
    float ms = 0;
    size_t launches = 0;
  };
  size_t issue_range(const std::string& program, const VarMap& vars, size_t lo, size_t hi);
  std::vector<CallTime> issue_timed(const std::string& program, const VarMap& vars);
  bool is_captured(const std::string& program, const VarMap& vars) const;
  size_t graphs() const { return graphs_.size(); }
  uint64_t launches_total() const { return launches_total_; }

  // ---- pool support ----
  void zero_slot(int32_t slot);
  void copy_pages(const std::vector<std::pair<int32_t, int32_t>>& pages);
  void copy_slot(int32_t src, int32_t dst);

  // ---- peers ----
  // handles of every exported buffer and state of this rank, keyed by name (64-byte IPC handles)
  std::map<std::string, std::string> export_handles();
  // handles of every member of `group` in member order -> fills each peer buffer of that group
  void connect(const std::string& group, const std::vector<std::map<std::string, std::string>>& members);
  // Names of the allocations whose canary bands no longer hold their pattern ("x (after)", "op.scratch (before)"); empty
  // when guard bands are off. Synchronises the stream.
  std::vector<std::string> check_guards();
  // Checked kernel builds (compiled with KERN_CHECKED): every module of such a build carries a table of the address
  // ranges its kernels may touch, which the runtime fills with every allocation it made or mapped (buffers, scratch,
  // states, peers' regions, bound host states); a checked access outside every range is skipped by the kernel and
  // recorded in the module. `checked_failures` reads the records: one line per module that caught something.
  void publish_spans();
  std::vector<std::string> checked_failures();
  bool checked() const { return !checked_.empty(); }
  bool peers_connected() const;
  // Another process's pool, for pushing pages and slots into it (prefill tier -> decode tier): the owner exports the
  // region of a state, the pusher maps it and copies whole units (a page of a paged state, a slot of a per-sequence one).
  std::string export_region(const std::string& name);
  uint64_t import_region(const std::string& handle);
  void push_unit(const std::string& state, uint64_t dst_base, int64_t src_unit, int64_t dst_unit);
  // strided copies (push.hpp: dealt rows, slot parts) from this runtime's `state`, starting `src_off` bytes in, into mapped
  // memory at `dst_base`; every copy is checked against the state's bytes here and `dst_bytes` there
  void push_copies(const std::string& state, uint64_t src_off, uint64_t dst_base, uint64_t dst_bytes, const std::vector<RowsCopy>& copies);
  void push_bytes(const std::string& name, uint64_t dst_base, uint64_t nbytes);   // the first nbytes of a buffer (a crossing workspace into the next stage's landing buffer)
  std::set<std::string> nccl_groups() const;     // groups named by `extern:nccl_*` launches: each needs connect() first

  // ---- hosted mode ----
  bool awaits_host() const;
  void bind_host(const std::map<std::string, std::tuple<uint64_t, std::string, std::vector<uint64_t>, std::vector<uint64_t>>>& regions);
  size_t enqueue_after(const std::string& program, const VarMap& vars, uint64_t host_stream);

  std::string banner() const;   // every state / buffer size and op -> module resolution

 private:
  Manifest m_;
  std::optional<Protocol> proto_;
  std::string kernels_dir_;
  std::shared_ptr<Device> dev_;
  std::map<std::string, GroupRank> topo_;
  Capacity cap_;
  CUstream stream_ = nullptr;
  bool own_stream_ = false;
  std::vector<CUstream> lane_streams_;
  std::vector<CUevent> lane_events_;
  CUevent host_in_ = nullptr, host_out_ = nullptr;

  std::map<std::string, CUmodule> modules_;
  CUmodule builtin_gemm_ = nullptr;
  CUmodule builtin_gemm8_ = nullptr;     // e4m3 GEMMs behind `extern:cublaslt_fp8_tn[_f32]`
  CUmodule builtin_gemm_mx_ = nullptr;   // block-scaled GEMM behind `extern:cublaslt_mxfp8_tn`
  std::string builtin_path(const std::string& file) const;
  std::map<std::string, CUfunction> gemm_fns_;
  std::map<std::string, Allocation> buffers_;
  std::map<std::string, StateAlloc> states_;
  std::map<std::string, std::map<std::string, Allocation>> scratch_;   // op -> scratch name -> allocation
  std::map<std::string, std::vector<uint64_t>> imported_;             // peer buffer -> mapped addresses
  std::vector<uint64_t> imported_ptrs_;
  struct Guard { std::string name; uint64_t base, bytes; };     // base = start of the leading band; bytes = payload size
  std::vector<Guard> guards_;
  struct CheckedModule { std::string name; uint64_t spans, count, fail; uint64_t capacity; };
  std::vector<CheckedModule> checked_;
  uint64_t guard_ = 0;                                            // band size in bytes (0: off)
  std::map<std::string, void*> nccl_comms_;      // group -> communicator of the `extern:nccl_*` launches
  std::map<std::string, NcclUniqueId> nccl_ids_;  // ids this rank (index 0 of the group) created and offers
  uint64_t page_unit_ = 1, pages_ = 0, slots_ = 0;
  uint64_t err_word_ = 0;
  bool weights_loaded_ = false;
  bool compiled_ = false;

  std::map<std::string, CompiledProgram> programs_;
  struct GraphKey {
    std::string program;
    std::vector<uint64_t> values;
    bool operator<(const GraphKey& o) const { return std::tie(program, values) < std::tie(o.program, o.values); }
  };
  struct GraphEntry {
    CUgraphExec exec = nullptr;
    size_t launches = 0;
  };
  std::map<GraphKey, GraphEntry> graphs_;
  uint64_t launches_total_ = 0;
  void* staging_ = nullptr;
  size_t staging_bytes_ = 0;

  void load_modules();
  void allocate();
  void compile_all();
  CompiledProgram compile_program(const std::string& name, const Program& p);
  void compile_call(CompiledProgram& out, const std::string& pname, const Program& p, size_t ci);
  CompiledArg pointer_arg(uint64_t ptr);
  uint64_t arg_pointer(const Arg& a) const;
  uint64_t arg_extent(const Arg& a) const;
  size_t enqueue(const CompiledProgram& p, const VarMap& vars);
  size_t launch_one(const CompiledLaunch& l, const VarMap& vars, CUstream s);
  size_t launch_gemm(const CompiledLaunch& l, const VarMap& vars, CUstream s);
  size_t launch_nccl(const CompiledLaunch& l, const VarMap& vars, CUstream s);
  void ensure_staging(size_t bytes);
  void upload(uint64_t dst, const uint8_t* src, size_t bytes);
  void upload_2d(uint64_t dst, size_t dst_pitch, const uint8_t* src, size_t src_pitch, size_t width, size_t rows);
};

}  // namespace kern
