// Runtime: program compilation (flat launch lists with baked addresses), launch, graph capture and
// replay, lanes, pool copies, peer import (see runtime.hpp).
#include <cstring>

#include "runtime.hpp"

namespace kern {

namespace {

void put_scalar(std::vector<uint8_t>& img, size_t at, size_t width, DType dt, int64_t i, double f) {
  if (img.size() < at + width) img.resize(at + width, 0);
  if (dt == DType::f32) { float v = (float)f; std::memcpy(&img[at], &v, 4); return; }
  std::memcpy(&img[at], &i, std::min<size_t>(width, 8));   // little-endian truncation
}

Expr const_expr(uint64_t v) { Expr e; e.kind = Expr::Const; e.c = v; return e; }
Expr var_expr(const std::string& v) { Expr e; e.kind = Expr::Var; e.var = v; return e; }

struct GemmPick { int bn; int stages; };
GemmPick pick_gemm_tile(uint64_t m, uint64_t n, int sms, bool allow32) {
  const uint64_t num_m = (m + 127) / 128;
  for (int bn : {256, 128, 64, 32}) {
    if (bn == 32 && !allow32) break;
    if (num_m * ((n + bn - 1) / bn) >= (uint64_t)sms) return {bn, bn == 256 ? 4 : (bn == 128 ? 6 : 8)};
  }
  const int bn = allow32 ? 32 : 64;
  return {bn, 8};
}

}  // namespace

void Runtime::compile_all() {
  programs_.clear();
  uint8_t lanes = 1;
  for (auto& kv : m_.programs) {
    programs_[kv.first] = compile_program(kv.first, kv.second);
    lanes = std::max(lanes, programs_[kv.first].lanes);
  }
  while (lane_streams_.size() + 1 < lanes) {
    lane_streams_.push_back(dev_->stream_create());
    lane_events_.push_back(dev_->event_create(false));
  }
  if (lane_events_.size() < lanes) lane_events_.push_back(dev_->event_create(false));   // one for lane 0
  publish_spans();
  compiled_ = true;
}

uint64_t Runtime::arg_pointer(const Arg& a) const {
  if (a.kind == Arg::Buf) {
    auto it = buffers_.find(a.name);
    if (it == buffers_.end()) throw std::runtime_error("unknown buffer `" + a.name + "`");
    return it->second.ptr + a.offset;
  }
  auto it = states_.find(a.name);
  if (it == states_.end()) throw std::runtime_error("unknown state `" + a.name + "`");
  if (it->second.ptr == 0) throw std::runtime_error("state `" + a.name + "` is the host's and has not been bound");
  return it->second.ptr + a.offset;
}
uint64_t Runtime::arg_extent(const Arg& a) const {
  const uint64_t bytes = a.kind == Arg::Buf ? buffers_.at(a.name).bytes : states_.at(a.name).bytes;
  return bytes > a.offset ? bytes - a.offset : 0;
}
CompiledArg Runtime::pointer_arg(uint64_t ptr) {
  CompiledArg c;
  c.image.resize(8);
  std::memcpy(c.image.data(), &ptr, 8);
  return c;
}

CompiledProgram Runtime::compile_program(const std::string& name, const Program& p) {
  CompiledProgram out;
  out.name = name;
  out.graph = p.graph;
  for (size_t ci = 0; ci < p.calls.size(); ++ci) {
    out.lanes = std::max<uint8_t>(out.lanes, p.calls[ci].lane + 1);
    compile_call(out, name, p, ci);
  }
  std::set<std::string> vs;
  auto add = [&](const Expr& e) { std::vector<std::string> v; e.collect_vars(v); vs.insert(v.begin(), v.end()); };
  for (auto& l : out.launches) {
    for (auto& g : l.grid) add(g);
    if (l.shared_mem) add(*l.shared_mem);
    if (l.when) vs.insert(l.when->var);
    for (auto& a : l.args) for (auto& pt : a.patches) add(pt.expr);
    if (l.ext != ExternKind::None) { add(l.m); add(l.n); add(l.k); if (l.ldc) add(*l.ldc); if (l.lda) add(*l.lda); }
  }
  out.vars.assign(vs.begin(), vs.end());
  return out;
}

void Runtime::compile_call(CompiledProgram& out, const std::string& pname, const Program& p, size_t ci) {
  const Call& c = p.calls[ci];
  const Op& op = m_.ops.at(c.op);
  const std::string where = "program `" + pname + "` call #" + std::to_string(ci) + " (" + c.op + ")";
  bool first = true;
  for (size_t li = 0; li < op.launches.size(); ++li) {
    const Launch& l = op.launches[li];
    const auto& params = op.params_of(l);
    const auto largs = op.args_of(l);
    CompiledLaunch cl;
    cl.label = c.label ? *c.label : c.op;
    cl.call_index = ci;
    cl.lane = c.lane;
    cl.first_of_call = first;
    if (first) cl.after = c.after;
    first = false;
    cl.when = l.when;

    // a launch arg resolved against the call: pointer, scalar image or expression
    auto scalar_of_call = [&](const Arg& a, const ParamType& pt, CompiledArg& ca, size_t at) {
      const size_t w = pt.abi_size();
      switch (a.kind) {
        case Arg::Var: ca.patches.push_back({(uint32_t)at, (uint32_t)w, var_expr(a.name)}); if (ca.image.size() < at + w) ca.image.resize(at + w, 0); break;
        case Arg::ExprK: ca.patches.push_back({(uint32_t)at, (uint32_t)w, a.expr}); if (ca.image.size() < at + w) ca.image.resize(at + w, 0); break;
        case Arg::Rank: put_scalar(ca.image, at, w, pt.dtype, (int64_t)rank(a.name), 0); break;
        case Arg::F32: put_scalar(ca.image, at, w, DType::f32, 0, a.f); break;
        default: put_scalar(ca.image, at, w, pt.dtype, a.i, 0); break;
      }
    };

    if (l.is_extern && parse_nccl_extern(l.entry, &cl.coll, &cl.elem)) {
      // [send, recv, count, rank]: count in elements per rank (the block an all-gather sends and a reduce-scatter
      // receives; per peer for an all-to-all); the rank arg names the group whose communicator carries the call
      if (largs.size() != 4) throw std::runtime_error(where + ": a collective built-in takes [send, recv, count, rank]");
      auto ptr_of = [&](size_t j, uint64_t* extent) {
        if (largs[j].kind == LaunchArg::Scratch) { auto& s = scratch_.at(c.op).at(largs[j].name); *extent = s.bytes; return s.ptr; }
        if (largs[j].kind != LaunchArg::Param) throw std::runtime_error(where + ": collective operand " + std::to_string(j) + " must be a buffer");
        const Arg& a = c.args.at(largs[j].param);
        if (a.kind != Arg::Buf && a.kind != Arg::StateK) throw std::runtime_error(where + ": collective operand " + std::to_string(j) + " must be a buffer");
        *extent = arg_extent(a);
        return arg_pointer(a);
      };
      cl.ext = ExternKind::Nccl;
      cl.a_ptr = ptr_of(0, &cl.a_rows);
      cl.c_ptr = ptr_of(1, &cl.w_rows);
      const LaunchArg& cnt = largs[2];
      if (cnt.kind == LaunchArg::I32 || cnt.kind == LaunchArg::I64) cl.m = const_expr((uint64_t)cnt.i);
      else if (cnt.kind == LaunchArg::Param) {
        const Arg& a = c.args.at(cnt.param);
        if (a.kind == Arg::Var) cl.m = var_expr(a.name);
        else if (a.kind == Arg::ExprK) cl.m = a.expr;
        else if (a.kind == Arg::I32 || a.kind == Arg::I64) cl.m = const_expr((uint64_t)a.i);
        else throw std::runtime_error(where + ": collective count must be an integer");
      } else throw std::runtime_error(where + ": collective count must be an integer");
      cl.n = const_expr(0); cl.k = const_expr(0);
      const LaunchArg& rk = largs[3];
      if (rk.kind == LaunchArg::Rank) cl.group = rk.name;
      else if (rk.kind == LaunchArg::Param && c.args.at(rk.param).kind == Arg::Rank) cl.group = c.args.at(rk.param).name;
      else throw std::runtime_error(where + ": the last arg of a collective built-in is `{rank: <group>}`");
      if (!topo_.count(cl.group)) throw std::runtime_error(where + ": collective over unknown group `" + cl.group + "`");
      out.launches.push_back(std::move(cl));
      continue;
    }
    if (l.is_extern) {
      static const std::pair<const char*, ExternKind> kinds[] = {{"extern:cublaslt_bf16_tn", ExternKind::GemmBf16},
                                                                  {"extern:cublaslt_bf16_tn_acc", ExternKind::GemmBf16Acc},
                                                                  {"extern:cublas_bf16_tn_f32", ExternKind::GemmBf16F32},
                                                                  {"extern:cublaslt_fp8_tn", ExternKind::GemmFp8},
                                                                  {"extern:cublaslt_fp8_tn_f32", ExternKind::GemmFp8F32},
                                                                  {"extern:cublaslt_mxfp8_tn", ExternKind::GemmMxfp8}};
      for (auto& k : kinds) if (l.entry == k.first) cl.ext = k.second;
      if (cl.ext == ExternKind::None)
        throw std::runtime_error(where + ": built-in `" + l.entry + "` is not provided by this runtime");
      const bool mx = cl.ext == ExternKind::GemmMxfp8;     // same argument list as fp8; the scales are UE8M0 atoms
      const bool fp8 = cl.ext == ExternKind::GemmFp8 || cl.ext == ExternKind::GemmFp8F32 || mx;
      // e4m3 operands with per-tensor device scales: [a, w, c, a_scale, w_scale, m, n, k] plus an optional C row stride
      const size_t so = fp8 ? 2 : 0;
      if (fp8 ? (largs.size() < 8 || largs.size() > 9) : (largs.size() < 6 || largs.size() > 8))
        throw std::runtime_error(where + (fp8 ? ": an fp8 GEMM built-in takes [a, w, c, a_scale, w_scale, m, n, k] plus an optional C row stride"
                                              : ": a GEMM built-in takes [a, w, c, m, n, k] plus optional row strides"));
      auto ptr_of = [&](size_t j, uint64_t* extent) {
        if (largs[j].kind == LaunchArg::Scratch) { auto& s = scratch_.at(c.op).at(largs[j].name); if (extent) *extent = s.bytes; return s.ptr; }
        if (largs[j].kind != LaunchArg::Param) throw std::runtime_error(where + ": GEMM operand " + std::to_string(j) + " must be a buffer");
        const Arg& a = c.args.at(largs[j].param);
        if (extent) *extent = arg_extent(a);
        return arg_pointer(a);
      };
      auto expr_of = [&](size_t j) -> Expr {
        const LaunchArg& la = largs[j];
        if (la.kind == LaunchArg::I32 || la.kind == LaunchArg::I64) return const_expr((uint64_t)la.i);
        if (la.kind != LaunchArg::Param) throw std::runtime_error(where + ": GEMM extent " + std::to_string(j) + " must be an integer");
        const Arg& a = c.args.at(la.param);
        if (a.kind == Arg::Var) return var_expr(a.name);
        if (a.kind == Arg::ExprK) return a.expr;
        if (a.kind == Arg::I32 || a.kind == Arg::I64) return const_expr((uint64_t)a.i);
        throw std::runtime_error(where + ": GEMM extent " + std::to_string(j) + " must be an integer");
      };
      uint64_t a_ext = 0, w_ext = 0;
      cl.a_ptr = ptr_of(0, &a_ext);
      cl.w_ptr = ptr_of(1, &w_ext);
      cl.c_ptr = ptr_of(2, nullptr);
      if (fp8) { cl.sa_ptr = ptr_of(3, nullptr); cl.sw_ptr = ptr_of(4, nullptr); }
      cl.m = expr_of(3 + so); cl.n = expr_of(4 + so); cl.k = expr_of(5 + so);
      if (largs.size() >= 7 + so) cl.ldc = expr_of(6 + so);
      if (!fp8 && largs.size() >= 8) cl.lda = expr_of(7);
      cl.a_rows = a_ext;   // bytes available behind the pointers: row counts follow at launch
      cl.w_rows = w_ext;
      if (mx && !gemm_fns_.count("kern_gemm_mxfp8_tn_n128")) {
        for (int bn : {256, 128}) {
          const std::string e = "kern_gemm_mxfp8_tn_n" + std::to_string(bn);
          gemm_fns_[e] = dev_->function(builtin_gemm_mx_, e);
        }
      }
      if (fp8 && !mx && !gemm_fns_.count("kern_gemm_e4m3_tn_n128")) {
        for (const char* epi : {"", "_f32"})
          for (int bn : {256, 128, 64}) {
            const std::string e = std::string("kern_gemm_e4m3_tn") + epi + "_n" + std::to_string(bn);
            gemm_fns_[e] = dev_->function(builtin_gemm8_, e);
          }
      }
      if (!fp8 && !gemm_fns_.count("kern_gemm_bf16_tn_n128")) {
        for (const char* epi : {"", "_acc", "_f32"})
          for (int bn : {256, 128, 64, 32}) {
            if (bn == 32 && std::string(epi) == "_f32") continue;
            const std::string e = std::string("kern_gemm_bf16_tn") + epi + "_n" + std::to_string(bn);
            gemm_fns_[e] = dev_->function(builtin_gemm_, e);
          }
      }
      out.launches.push_back(std::move(cl));
      continue;
    }

    cl.fn = dev_->function(modules_.at(l.module), l.entry);
    // ABI: the driver's view of the kernel's parameters must agree with the declared ones
    {
      auto sizes = dev_->param_sizes(cl.fn);
      bool ok = sizes.size() == params.size();
      for (size_t j = 0; ok && j < sizes.size(); ++j) ok = sizes[j] == params[j].abi_size();
      if (!ok) {
        std::string got, want;
        for (auto s : sizes) got += std::to_string(s) + " ";
        for (auto& pt : params) want += std::to_string(pt.abi_size()) + " ";
        throw std::runtime_error(where + ": entry `" + l.entry + "` takes parameters of bytes [ " + got + "], the manifest declares [ " + want + "]");
      }
    }
    std::memcpy(cl.block, l.block, sizeof cl.block);
    for (int i = 0; i < 3; ++i) cl.grid[i] = l.grid[i];
    cl.shared_mem = l.shared_mem;
    if (l.cluster) for (int i = 0; i < 3; ++i) cl.cluster[i] = (*l.cluster)[i];
    cl.pdl = l.pdl;

    for (size_t j = 0; j < largs.size(); ++j) {
      const LaunchArg& la = largs[j];
      const ParamType& pt = params[j];
      CompiledArg ca;
      switch (la.kind) {
        case LaunchArg::Param: {
          const Arg& a = c.args.at(la.param);
          if (a.kind == Arg::Buf || a.kind == Arg::StateK) ca = pointer_arg(arg_pointer(a));
          else scalar_of_call(a, pt, ca, 0);
          break;
        }
        case LaunchArg::Scratch: ca = pointer_arg(scratch_.at(c.op).at(la.name).ptr); break;
        case LaunchArg::Rank: put_scalar(ca.image, 0, pt.abi_size(), pt.dtype, (int64_t)rank(la.name), 0); break;
        case LaunchArg::F32: put_scalar(ca.image, 0, 4, DType::f32, 0, la.f); break;
        case LaunchArg::I32: case LaunchArg::I64: case LaunchArg::U8: put_scalar(ca.image, 0, pt.abi_size(), pt.dtype, la.i, 0); break;
        case LaunchArg::PackK: {
          ca.image.assign(la.pack.size, 0);
          for (auto& f : la.pack.fields) {
            switch (f.src.kind) {
              case FieldSrc::Param: {
                const Arg& a = c.args.at(f.src.param);
                const ParamType& ipt = op.params.at(f.src.param);
                if (a.kind == Arg::Buf || a.kind == Arg::StateK) { uint64_t p = arg_pointer(a); std::memcpy(&ca.image[f.at], &p, 8); }
                else { ParamType w = ipt; scalar_of_call(a, w, ca, f.at); }
                break;
              }
              case FieldSrc::Scratch: { uint64_t p = scratch_.at(c.op).at(f.src.name).ptr; std::memcpy(&ca.image[f.at], &p, 8); break; }
              case FieldSrc::I32: case FieldSrc::I64: case FieldSrc::U8:
                put_scalar(ca.image, f.at, f.width.value_or(f.src.kind == FieldSrc::I64 ? 8 : (f.src.kind == FieldSrc::U8 ? 1 : 4)), DType::i64, f.src.i, 0);
                break;
              case FieldSrc::F32: put_scalar(ca.image, f.at, 4, DType::f32, 0, f.src.f); break;
              case FieldSrc::Var: ca.patches.push_back({f.at, f.width.value_or(4), var_expr(f.src.name)}); break;
              case FieldSrc::ExprK: ca.patches.push_back({f.at, f.width.value_or(4), f.src.expr}); break;
              case FieldSrc::Rank: put_scalar(ca.image, f.at, f.width.value_or(4), DType::i64, (int64_t)rank(f.src.name), 0); break;
              case FieldSrc::TensorMap: {
                const TensorMapDecl& t = f.src.tmap;
                const Arg& a = c.args.at(t.param);
                TensorMapSpec s;
                s.dtype = t.cu_dtype();
                s.dims = t.dims;
                s.strides = t.strides;
                s.box = t.box;
                s.swizzle = (int)t.swizzle;
                s.l2_promotion = (int)t.l2_promotion;
                s.oob_nan = t.oob_nan;
                if (s.dims.size() > 1 && s.dims.back() == 0) {
                  // the outermost extent spans what lies behind the pointer
                  const uint64_t avail = arg_extent(a);
                  s.dims.back() = std::max<uint64_t>(1, avail / s.strides.back());
                }
                auto tm = dev_->encode_tensor_map(arg_pointer(a), s);
                std::memcpy(&ca.image[f.at], tm.data(), 128);
                break;
              }
            }
          }
          break;
        }
      }
      if (ca.image.size() < pt.abi_size()) ca.image.resize(pt.abi_size(), 0);
      cl.args.push_back(std::move(ca));
    }
    out.launches.push_back(std::move(cl));
  }
}

size_t Runtime::launch_gemm(const CompiledLaunch& l, const VarMap& vars, CUstream s) {
  auto ev = [&](const Expr& e) {
    std::string why;
    auto v = e.eval(vars, &why);
    if (!v) throw std::runtime_error("GEMM extent: " + why);
    return *v;
  };
  const uint64_t m = ev(l.m), n = ev(l.n), k = ev(l.k);
  if (m == 0 || n == 0) return 0;
  const uint64_t ldc = l.ldc ? ev(*l.ldc) : n, lda = l.lda ? ev(*l.lda) : k;
  if (l.ext == ExternKind::GemmMxfp8) {
    // MXFP8 x MXFP8 -> bf16: e4m3 bytes, one UE8M0 scale per 32 elements of K in 128 x 4 atoms of 512 bytes (atom
    // (r / 128, b / 4) at 512 (r / 128 * ceil(k / 128) + b / 4), entry (r % 32) 16 + (r % 128 / 32) 4 + b % 4): the layout
    // the reference's library call takes (crates/kern-runtime/src/cublas.rs:395-400), which is what tcgen05.cp wants.
    if (k % 128) throw std::runtime_error("mxfp8 GEMM `" + l.label + "`: k must be a multiple of 128 (one stage of the block-scaled kernel)");
    const uint64_t tiles_m = (m + 127) / 128;
    const int bn = (n % 256 == 0 && tiles_m * (n / 256) >= (uint64_t)dev_->sm_count() / 2) ? 256 : 128;
    auto tmap8 = [&](uint64_t ptr, uint64_t avail_bytes, uint64_t box_rows) {
      TensorMapSpec sp;
      sp.dtype = 0;
      sp.dims = {k, std::max<uint64_t>(1, avail_bytes / k)};
      sp.strides = {k};
      sp.box = {128, (uint32_t)box_rows};
      sp.swizzle = 128;
      sp.l2_promotion = 256;
      return dev_->encode_tensor_map(ptr, sp);
    };
    alignas(64) std::array<uint8_t, 128> ta = tmap8(l.a_ptr, l.a_rows, 128);
    alignas(64) std::array<uint8_t, 128> tb = tmap8(l.w_ptr, std::min<uint64_t>(l.w_rows, n * k), bn);
    CUfunction fn = gemm_fns_.at("kern_gemm_mxfp8_tn_n" + std::to_string(bn));
    uint64_t c = l.c_ptr, sa = l.sa_ptr, sw = l.sw_ptr, err = err_word_;
    int mi = (int)m, ni = (int)n, ki = (int)k, ldci = (int)ldc;
    void* params[] = {ta.data(), tb.data(), &sa, &sw, &c, &mi, &ni, &ki, &ldci, &err};
    LaunchDims d;
    d.grid[0] = (unsigned)std::min<uint64_t>(tiles_m * ((n + bn - 1) / bn), dev_->sm_count());
    d.block[0] = 192;
    d.shared_mem = 1024 + (bn == 256 ? 4 : 6) * (128 * 128 + bn * 128 + (bn == 256 ? 2048 : 1024)) + 256;
    dev_->launch(fn, d, s, params);
    return 1;
  }
  if (l.ext == ExternKind::GemmFp8 || l.ext == ExternKind::GemmFp8F32) {
    // one byte per element, 128-element K boxes; the tile width as the bf16 picker would choose it (no 32-wide tile)
    const bool f32o = l.ext == ExternKind::GemmFp8F32;
    const uint64_t tiles_m = (m + 127) / 128;
    const int bn = tiles_m * ((n + 255) / 256) >= (uint64_t)dev_->sm_count() ? 256 : (n >= 128 ? 128 : 64);
    if (k % 16) throw std::runtime_error("fp8 GEMM `" + l.label + "`: k must be a multiple of 16");
    auto tmap8 = [&](uint64_t ptr, uint64_t ld, uint64_t avail_bytes, uint64_t box_rows) {
      TensorMapSpec sp;
      sp.dtype = 0;      // CU_TENSOR_MAP_DATA_TYPE_UINT8
      sp.dims = {k, std::max<uint64_t>(1, avail_bytes / ld)};
      sp.strides = {ld};
      sp.box = {128, (uint32_t)box_rows};
      sp.swizzle = 128;
      sp.l2_promotion = 256;
      return dev_->encode_tensor_map(ptr, sp);
    };
    alignas(64) std::array<uint8_t, 128> ta = tmap8(l.a_ptr, k, l.a_rows, 128);
    alignas(64) std::array<uint8_t, 128> tb = tmap8(l.w_ptr, k, std::min<uint64_t>(l.w_rows, n * k), bn);
    CUfunction fn = gemm_fns_.at(std::string("kern_gemm_e4m3_tn") + (f32o ? "_f32" : "") + "_n" + std::to_string(bn));
    uint64_t c = l.c_ptr, r = 0, sa = l.sa_ptr, sw = l.sw_ptr, err = err_word_;
    int mi = (int)m, ni = (int)n, ki = (int)k, ldci = (int)ldc;
    void* params[] = {ta.data(), tb.data(), &c, &r, &sa, &sw, &mi, &ni, &ki, &ldci, &err};
    LaunchDims d;
    d.grid[0] = (unsigned)std::min<uint64_t>(tiles_m * ((n + bn - 1) / bn), dev_->sm_count());
    d.block[0] = 192;
    const int stages = bn == 256 ? 4 : (bn == 128 ? 6 : 8);
    d.shared_mem = 1024 + stages * (128 * 128 + bn * 128) + 256;
    dev_->launch(fn, d, s, params);
    return 1;
  }
  const bool f32 = l.ext == ExternKind::GemmBf16F32;
  const GemmPick pk = pick_gemm_tile(m, n, dev_->sm_count(), !f32);
  // descriptors cover everything behind the pointers, so one encoding serves every row count
  struct Key { uint64_t ptr, ld, rows, box; bool operator<(const Key& o) const { return std::tie(ptr, ld, rows, box) < std::tie(o.ptr, o.ld, o.rows, o.box); } };
  static thread_local std::map<Key, std::array<uint8_t, 128>> cache;
  auto tmap = [&](uint64_t ptr, uint64_t ld, uint64_t avail_bytes, uint64_t box_rows) {
    const uint64_t rows = std::max<uint64_t>(1, avail_bytes / (ld * 2));
    Key key{ptr, ld, rows, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    TensorMapSpec sp;
    sp.dtype = 9;
    sp.dims = {k, rows};
    sp.strides = {ld * 2};
    sp.box = {64, (uint32_t)box_rows};
    sp.swizzle = 128;
    sp.l2_promotion = 256;
    auto tm = dev_->encode_tensor_map(ptr, sp);
    if (cache.size() > 8192) cache.clear();
    cache[key] = tm;
    return tm;
  };
  alignas(64) std::array<uint8_t, 128> ta = tmap(l.a_ptr, lda, l.a_rows, 128);
  alignas(64) std::array<uint8_t, 128> tb = tmap(l.w_ptr, k, std::min<uint64_t>(l.w_rows, n * k * 2), pk.bn);
  const char* epi = l.ext == ExternKind::GemmBf16Acc ? "_acc" : (f32 ? "_f32" : "");
  CUfunction fn = gemm_fns_.at(std::string("kern_gemm_bf16_tn") + epi + "_n" + std::to_string(pk.bn));
  uint64_t c = l.c_ptr, r = l.ext == ExternKind::GemmBf16Acc ? l.c_ptr : 0, err = err_word_;
  int mi = (int)m, ni = (int)n, ki = (int)k, ldci = (int)ldc;
  void* params[] = {ta.data(), tb.data(), &c, &r, &mi, &ni, &ki, &ldci, &err};
  LaunchDims d;
  const uint64_t tiles = ((m + 127) / 128) * ((n + pk.bn - 1) / pk.bn);
  d.grid[0] = (unsigned)std::min<uint64_t>(tiles, dev_->sm_count());
  d.block[0] = 192;
  d.shared_mem = 1024 + pk.stages * (128 * 64 * 2 + pk.bn * 64 * 2) + 256;
  dev_->launch(fn, d, s, params);
  return 1;
}

// One collective on the issuing stream (NCCL calls are capturable, so graph programs may hold them).
size_t Runtime::launch_nccl(const CompiledLaunch& l, const VarMap& vars, CUstream s) {
  std::string why;
  auto cnt = l.m.eval(vars, &why);
  if (!cnt) throw std::runtime_error("collective count of `" + l.label + "`: " + why);
  const uint64_t n = *cnt;
  if (n == 0) return 0;
  const uint64_t world = topo_.at(l.group).size, eb = nccl_elem_bytes(l.elem);
  if (world == 1) {      // a group of one: every collective is a copy, and no communicator exists
    if (l.a_rows < n * eb || l.w_rows < n * eb) throw std::runtime_error("collective `" + l.label + "`: buffers smaller than the count");
    if (l.a_ptr != l.c_ptr) dev_->d2d(l.c_ptr, l.a_ptr, n * eb, s);
    return 1;
  }
  auto it = nccl_comms_.find(l.group);
  if (it == nccl_comms_.end()) throw std::runtime_error("nccl group `" + l.group + "` not joined: connect() it before the first issue");
  uint64_t ins = n, outs = n;
  switch (l.coll) {
    case NcclColl::AllReduce: break;
    case NcclColl::AllGather: outs = n * world; break;
    case NcclColl::ReduceScatter: ins = n * world; break;
    case NcclColl::AllToAll: ins = outs = n * world; break;
  }
  if (l.a_rows < ins * eb || l.w_rows < outs * eb)
    throw std::runtime_error("collective `" + l.label + "`: " + std::to_string(n) + " elements per rank need " + std::to_string(ins * eb) +
                             " B to send and " + std::to_string(outs * eb) + " B to receive; the buffers hold " +
                             std::to_string(l.a_rows) + " B and " + std::to_string(l.w_rows) + " B");
  NcclApi& api = NcclApi::get();
  const void* src = reinterpret_cast<const void*>(l.a_ptr);
  void* dst = reinterpret_cast<void*>(l.c_ptr);
  void* comm = it->second;
  const int dt = (int)l.elem;
  switch (l.coll) {
    case NcclColl::AllReduce: api.check(api.AllReduce(src, dst, n, dt, 0, comm, s), "all-reduce"); break;
    case NcclColl::AllGather: api.check(api.AllGather(src, dst, n, dt, comm, s), "all-gather"); break;
    case NcclColl::ReduceScatter: api.check(api.ReduceScatter(src, dst, n, dt, 0, comm, s), "reduce-scatter"); break;
    case NcclColl::AllToAll: {
      // block p of `send` to peer p, peer p's block into block p of `recv`
      api.check(api.GroupStart(), "group start");
      int rc = 0;
      for (uint64_t p = 0; p < world && rc == 0; ++p) {
        rc = api.Send(static_cast<const uint8_t*>(src) + p * n * eb, n, dt, (int)p, comm, s);
        if (rc == 0) rc = api.Recv(static_cast<uint8_t*>(dst) + p * n * eb, n, dt, (int)p, comm, s);
      }
      const int end = api.GroupEnd();
      api.check(rc, "send/recv");
      api.check(end, "group end");
      break;
    }
  }
  return 1;
}

size_t Runtime::launch_one(const CompiledLaunch& l, const VarMap& vars, CUstream s) {
  if (l.when) {
    auto it = vars.find(l.when->var);
    if (it == vars.end()) throw std::runtime_error("`when` reads var `" + l.when->var + "`, which the call did not set");
    if (!l.when->holds(it->second)) return 0;
  }
  if (l.ext == ExternKind::Nccl) return launch_nccl(l, vars, s);
  if (l.ext != ExternKind::None) return launch_gemm(l, vars, s);
  LaunchDims d;
  for (int i = 0; i < 3; ++i) {
    std::string why;
    auto g = l.grid[i].eval(vars, &why);
    if (!g) throw std::runtime_error("grid of `" + l.label + "`: " + why);
    d.grid[i] = (unsigned)*g;
    d.block[i] = l.block[i];
    d.cluster[i] = l.cluster[i];
  }
  if (d.grid[0] == 0 || d.grid[1] == 0 || d.grid[2] == 0) return 0;
  if (l.shared_mem) {
    auto v = l.shared_mem->eval(vars);
    if (!v) throw std::runtime_error("shared_mem of `" + l.label + "` reads an unset var");
    d.shared_mem = (unsigned)*v;
  }
  d.pdl = l.pdl;
  // materialise the parameter images (64-byte aligned: tensor maps need it)
  size_t total = 0;
  for (auto& a : l.args) total += (a.image.size() + 63) / 64 * 64;
  std::vector<uint8_t> arena(total + 64);
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(arena.data()) + 63) & ~uintptr_t(63));
  std::vector<void*> ptrs(l.args.size());
  size_t off = 0;
  for (size_t j = 0; j < l.args.size(); ++j) {
    const CompiledArg& a = l.args[j];
    std::memcpy(base + off, a.image.data(), a.image.size());
    for (auto& pt : a.patches) {
      std::string why;
      auto v = pt.expr.eval(vars, &why);
      if (!v) throw std::runtime_error("argument of `" + l.label + "`: " + why);
      uint64_t x = *v;
      std::memcpy(base + off + pt.at, &x, std::min<uint32_t>(pt.width, 8));
    }
    ptrs[j] = base + off;
    off += (a.image.size() + 63) / 64 * 64;
  }
  dev_->launch(l.fn, d, s, ptrs.data());
  return 1;
}

size_t Runtime::enqueue(const CompiledProgram& p, const VarMap& vars) {
  dev_->make_current();
  for (auto& v : p.vars) {
    auto it = vars.find(v);
    if (it == vars.end()) throw std::runtime_error("program `" + p.name + "` reads var `" + v + "`, which the call did not set");
    auto decl = m_.vars.find(v);
    if (decl != m_.vars.end() && (it->second < VAR_MIN || it->second > decl->second.max))
      throw std::runtime_error("var `" + v + "` = " + std::to_string(it->second) + " is outside 1.." + std::to_string(decl->second.max));
  }
  auto stream_of = [&](uint8_t lane) { return lane == 0 ? stream_ : lane_streams_.at(lane - 1); };
  size_t n = 0;
  for (auto& l : p.launches) {
    CUstream s = stream_of(l.lane);
    if (l.first_of_call)
      for (uint8_t src : l.after) {
        CUevent e = lane_events_.at(src);
        dev_->event_record(e, stream_of(src));
        dev_->stream_wait(s, e);
      }
    n += launch_one(l, vars, s);
  }
  return n;
}

bool Runtime::is_captured(const std::string& program, const VarMap& vars) const {
  auto it = programs_.find(program);
  if (it == programs_.end()) return false;
  GraphKey key{program, {}};
  for (auto& v : it->second.vars) { auto f = vars.find(v); key.values.push_back(f == vars.end() ? 0 : f->second); }
  return graphs_.count(key) > 0;
}

size_t Runtime::issue(const std::string& program, const VarMap& vars, bool eager) {
  if (!compiled_) throw std::runtime_error("the manifest's host states have not been bound yet");
  auto it = programs_.find(program);
  if (it == programs_.end()) throw std::runtime_error("no program named `" + program + "`");
  const CompiledProgram& p = it->second;
  size_t n;
  if (eager || !p.graph) {
    n = enqueue(p, vars);
  } else {
    GraphKey key{program, {}};
    for (auto& v : p.vars) { auto f = vars.find(v); key.values.push_back(f == vars.end() ? 0 : f->second); }
    auto g = graphs_.find(key);
    if (g == graphs_.end()) {
      dev_->make_current();
      dev_->begin_capture(stream_);
      GraphEntry e;
      try {
        e.launches = enqueue(p, vars);
      } catch (...) {
        CUgraph junk = nullptr;
        Cuda::get().cuStreamEndCapture_(stream_, &junk);
        if (junk) Cuda::get().cuGraphDestroy_(junk);
        throw;
      }
      e.exec = dev_->end_capture(stream_);
      g = graphs_.emplace(key, e).first;
    }
    dev_->graph_launch(g->second.exec, stream_);
    n = g->second.launches;
  }
  launches_total_ += n;
  return n;
}

// Called by a host engine on its own stream: the host's work so far happens-before the program,
// the program happens-before what the host enqueues next. Both edges are events, so the call can be
// recorded into a graph the host is capturing.
size_t Runtime::enqueue_after(const std::string& program, const VarMap& vars, uint64_t host_stream) {
  CUstream hs = reinterpret_cast<CUstream>(host_stream);
  if (hs == stream_) return issue(program, vars, true);
  dev_->event_record(host_in_, hs);
  dev_->stream_wait(stream_, host_in_);
  auto it = programs_.find(program);
  if (it == programs_.end()) throw std::runtime_error("no program named `" + program + "`");
  size_t n = enqueue(it->second, vars);
  dev_->event_record(host_out_, stream_);
  dev_->stream_wait(hs, host_out_);
  launches_total_ += n;
  return n;
}

// Calls [lo, hi) of a program, eagerly and in order on the main stream (lanes are not forked): the harness behind
// activation probes, which read what a call wrote before the next range overwrites it.
size_t Runtime::issue_range(const std::string& program, const VarMap& vars, size_t lo, size_t hi) {
  if (!compiled_) throw std::runtime_error("the manifest's host states have not been bound yet");
  auto it = programs_.find(program);
  if (it == programs_.end()) throw std::runtime_error("no program named `" + program + "`");
  dev_->make_current();
  size_t n = 0;
  for (auto& l : it->second.launches)
    if (l.call_index >= lo && l.call_index < hi) n += launch_one(l, vars, stream_);
  launches_total_ += n;
  return n;
}

std::vector<Runtime::CallTime> Runtime::issue_timed(const std::string& program, const VarMap& vars) {
  if (!compiled_) throw std::runtime_error("the manifest's host states have not been bound yet");
  auto it = programs_.find(program);
  if (it == programs_.end()) throw std::runtime_error("no program named `" + program + "`");
  const CompiledProgram& p = it->second;
  const Program& src = m_.programs.at(program);
  dev_->make_current();
  std::vector<CUevent> evs;
  std::vector<CallTime> out;
  auto mark = [&] { CUevent e = dev_->event_create(true); dev_->event_record(e, stream_); evs.push_back(e); };
  mark();
  size_t call = (size_t)-1;
  for (auto& l : p.launches) {
    if (l.call_index != call) {
      if (call != (size_t)-1) mark();
      call = l.call_index;
      out.push_back({l.label, src.calls[call].op, 0.f, 0});
    }
    out.back().launches += launch_one(l, vars, stream_);
  }
  mark();
  dev_->stream_sync(stream_);
  for (size_t i = 0; i + 1 < evs.size() && i < out.size(); ++i) out[i].ms = dev_->event_ms(evs[i], evs[i + 1]);
  for (auto e : evs) Cuda::get().cuEventDestroy_(e);
  for (auto& c : out) launches_total_ += c.launches;
  return out;
}

void Runtime::run_once_programs() {
  for (auto& kv : m_.programs)
    if (kv.second.once) issue(kv.first, m_.vars_at_max(), true);
  synchronize();
}

// ---- pool support ------------------------------------------------------------------------------------
void Runtime::zero_slot(int32_t slot) {
  for (auto& kv : states_)
    if (kv.second.per_seq && slot >= 0 && (uint64_t)slot < kv.second.units)
      dev_->memset8(kv.second.ptr + (uint64_t)slot * kv.second.unit_bytes, 0, kv.second.unit_bytes, stream_);
}
void Runtime::copy_pages(const std::vector<std::pair<int32_t, int32_t>>& pages) {
  for (auto& kv : states_) {
    if (!kv.second.paged) continue;
    for (auto& p : pages) {
      if (p.first < 0 || p.second < 0 || (uint64_t)p.first >= kv.second.units || (uint64_t)p.second >= kv.second.units)
        throw std::runtime_error("page copy names a page outside the pool");
      dev_->d2d(kv.second.ptr + (uint64_t)p.second * kv.second.unit_bytes, kv.second.ptr + (uint64_t)p.first * kv.second.unit_bytes,
                kv.second.unit_bytes, stream_);
    }
  }
}
void Runtime::copy_slot(int32_t src, int32_t dst) {
  for (auto& kv : states_) {
    if (!kv.second.per_seq) continue;
    if (src < 0 || dst < 0 || (uint64_t)src >= kv.second.units || (uint64_t)dst >= kv.second.units)
      throw std::runtime_error("slot copy names a slot outside the pool");
    dev_->d2d(kv.second.ptr + (uint64_t)dst * kv.second.unit_bytes, kv.second.ptr + (uint64_t)src * kv.second.unit_bytes,
              kv.second.unit_bytes, stream_);
  }
}

// ---- peers -------------------------------------------------------------------------------------------
std::map<std::string, std::string> Runtime::export_handles() {
  std::map<std::string, std::string> out;
  std::set<std::string> wanted;
  for (auto& kv : m_.buffers) if (kv.second.kind == BufferKind::Peer && kv.second.of) wanted.insert(*kv.second.of);
  for (auto& name : wanted) {
    auto r = region(name);
    out[name] = dev_->ipc_export(r.first, guard_);
  }
  // member 0 of every group with `extern:nccl_*` launches creates the communicator's id and offers it
  for (auto& grp : nccl_groups()) {
    if (topo_.at(grp).index != 0) continue;
    auto it = nccl_ids_.find(grp);
    if (it == nccl_ids_.end()) {
      NcclUniqueId id;
      NcclApi::get().check(NcclApi::get().GetUniqueId(&id), "unique id");
      it = nccl_ids_.emplace(grp, id).first;
    }
    out["nccl_id." + grp] = std::string(it->second.internal, sizeof it->second.internal);
  }
  return out;
}

std::set<std::string> Runtime::nccl_groups() const {
  std::set<std::string> out;
  for (auto& p : programs_)
    for (auto& l : p.second.launches)
      if (l.ext == ExternKind::Nccl && topo_.at(l.group).size > 1) out.insert(l.group);
  return out;
}

void Runtime::connect(const std::string& group, const std::vector<std::map<std::string, std::string>>& members) {
  auto g = topo_.find(group);
  if (g == topo_.end()) throw std::runtime_error("unknown group `" + group + "`");
  if (members.size() != g->second.size) throw std::runtime_error("group `" + group + "` has " + std::to_string(g->second.size) + " members, got " + std::to_string(members.size()) + " offers");
  for (auto& kv : m_.buffers) {
    const Buffer& b = kv.second;
    if (b.kind != BufferKind::Peer || !b.group || *b.group != group || !b.of) continue;
    std::vector<uint64_t> addrs(members.size());
    for (size_t r = 0; r < members.size(); ++r) {
      if (r == g->second.index) { addrs[r] = region(*b.of).first; continue; }
      auto h = members[r].find(*b.of);
      if (h == members[r].end()) throw std::runtime_error("member " + std::to_string(r) + " of `" + group + "` did not offer `" + *b.of + "`");
      uint64_t off = 0;
      const uint64_t base = dev_->ipc_import(h->second, &off);
      imported_ptrs_.push_back(base);
      addrs[r] = base + off;
    }
    dev_->h2d(buffers_.at(kv.first).ptr, addrs.data(), addrs.size() * 8, stream_);
    dev_->stream_sync(stream_);
    imported_[kv.first] = addrs;
  }
  publish_spans();
  if (nccl_groups().count(group) && !nccl_comms_.count(group)) {
    // every member calls this with the same offers: member 0's id joins them into one communicator
    auto h = members.at(0).find("nccl_id." + group);
    if (h == members[0].end() || h->second.size() != sizeof(NcclUniqueId))
      throw std::runtime_error("member 0 of `" + group + "` did not offer the communicator id `nccl_id." + group + "`");
    NcclUniqueId id;
    std::memcpy(id.internal, h->second.data(), sizeof id.internal);
    dev_->make_current();
    void* comm = nullptr;
    NcclApi::get().check(NcclApi::get().CommInitRank(&comm, (int)g->second.size, id, (int)g->second.index), "communicator join");
    nccl_comms_[group] = comm;
  }
}

std::string Runtime::export_region(const std::string& name) { return dev_->ipc_export(region(name).first, guard_); }

uint64_t Runtime::import_region(const std::string& handle) {
  uint64_t off = 0;
  const uint64_t p = dev_->ipc_import(handle, &off);
  imported_ptrs_.push_back(p);
  return p + off;
}

void Runtime::push_unit(const std::string& state, uint64_t dst_base, int64_t src_unit, int64_t dst_unit) {
  auto it = states_.find(state);
  if (it == states_.end()) throw std::runtime_error("no state named `" + state + "`");
  const auto& st = it->second;
  if (src_unit < 0 || (uint64_t)src_unit >= st.units || dst_unit < 0)
    throw std::runtime_error("push of `" + state + "` names a unit outside the pool");
  dev_->d2d(dst_base + (uint64_t)dst_unit * st.unit_bytes, st.ptr + (uint64_t)src_unit * st.unit_bytes, st.unit_bytes, stream_);
}

void Runtime::push_copies(const std::string& state, uint64_t src_off, uint64_t dst_base, uint64_t dst_bytes, const std::vector<RowsCopy>& copies) {
  auto it = states_.find(state);
  if (it == states_.end()) throw std::runtime_error("no state named `" + state + "`");
  const auto& st = it->second;
  const uint64_t have = st.units * st.unit_bytes;
  for (const auto& c : copies) {
    if (c.rows == 0 || c.width == 0) continue;
    const uint64_t src_end = src_off + c.src + (c.rows - 1) * c.src_pitch + c.width;
    const uint64_t dst_end = c.dst + (c.rows - 1) * c.dst_pitch + c.width;
    if (src_end > have || dst_end > dst_bytes)
      throw std::runtime_error("push of `" + state + "`: a copy ends at byte " + std::to_string(src_end) + " of " + std::to_string(have) +
                               " here, " + std::to_string(dst_end) + " of " + std::to_string(dst_bytes) + " there");
  }
  for (const auto& c : copies) dev_->copy_2d(dst_base + c.dst, c.dst_pitch, st.ptr + src_off + c.src, c.src_pitch, c.width, c.rows, stream_);
}

void Runtime::push_bytes(const std::string& name, uint64_t dst_base, uint64_t nbytes) {
  auto r = region(name);
  if (nbytes > r.second) throw std::runtime_error("push of `" + name + "`: " + std::to_string(nbytes) + " bytes asked, the region holds " + std::to_string(r.second));
  if (nbytes) dev_->d2d(dst_base, r.first, nbytes, stream_);
}

bool Runtime::peers_connected() const {
  for (auto& kv : m_.buffers)
    if (kv.second.kind == BufferKind::Peer && !imported_.count(kv.first)) return false;
  for (auto& grp : nccl_groups()) if (!nccl_comms_.count(grp)) return false;
  return true;
}

}  // namespace kern
