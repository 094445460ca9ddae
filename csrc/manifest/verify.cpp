// Verifier rule groups (see verify.hpp). One Verifier object carries the "used" sets that the
// unused-declaration rule reads at the end; each rule group is its own method.
#include "verify.hpp"

#include <algorithm>
#include <array>

namespace kern {
namespace {

bool is_paged_owned(const State& s) { return s.is_owned() && s.bytes_per_token > 0; }
const char* state_kind(const State& s) {
  if (!s.is_owned()) return "host";
  if (s.bytes_per_token > 0) return "paged";
  return s.is_per_seq() ? "per-sequence" : "fixed";
}
bool scalar_fits(DType t, uint64_t v) {
  switch (t) {
    case DType::i32: return v <= (uint64_t)INT32_MAX;
    case DType::i64: return v <= (uint64_t)INT64_MAX;
    case DType::u8: return v <= 255;
    default: return false;
  }
}
std::string triple(const uint32_t* v) {
  return "[" + std::to_string(v[0]) + ", " + std::to_string(v[1]) + ", " + std::to_string(v[2]) + "]";
}

struct TmapUse {
  size_t param;
  uint64_t footprint;
  std::string where;
};

class Verifier {
 public:
  Verifier(const Manifest& m, bool strict) : m_(m), vmax_(m.vars_at_max()), vmin_(m.vars_at_min()), strict_(strict) {}

  Errors run() {
    header();
    states();
    shards();
    buffers();
    modules();
    ops();
    programs();
    check_lanes(m_, e_);
    if (strict_) multicast_declarations();
    unused();
    return std::move(e_);
  }

 private:
  const Manifest& m_;
  VarMap vmax_, vmin_;
  bool strict_ = false;
  Errors e_;
  std::set<std::string> used_vars_, used_buffers_, used_states_, used_modules_, used_ops_, used_groups_;
  std::map<std::string, uint64_t> buf_bytes_;
  std::map<std::string, std::vector<TmapUse>> op_tmaps_;
  std::set<std::string> peer_modules_;   // modules with a launch that can receive a peer buffer

  void err(std::string s) { e_.push_back(std::move(s)); }

  std::optional<uint64_t> group(const std::string& g, const std::string& ctx) {
    auto it = m_.topology.find(g);
    if (it != m_.topology.end()) { used_groups_.insert(g); return it->second; }
    err(ctx + (m_.has_topology ? ": unknown topology group `" + g + "`"
                               : ": names group `" + g + "` but the manifest has no topology"));
    return std::nullopt;
  }

  void expr(const Expr& x, const std::string& ctx) {
    switch (x.kind) {
      case Expr::Const: return;
      case Expr::Var:
        if (m_.vars.count(x.var)) used_vars_.insert(x.var); else err(ctx + ": unknown var `" + x.var + "`");
        return;
      case Expr::CeilDiv: if (x.c == 0) err(ctx + ": division by zero"); break;
      case Expr::Mul: if (x.c == 0) err(ctx + ": multiplication by constant zero"); break;
      case Expr::Clamp: if (x.c2 == 0) err(ctx + ": clamp to zero length"); break;
      case Expr::Add: break;
    }
    for (auto& s : x.sub) expr(s, ctx);
  }

  std::optional<uint64_t> shaped_bytes(const std::string& ctx, DType dt, const std::vector<Dim>& shape) {
    unsigned __int128 n = dtype_bytes(dt);
    bool ok = true;
    for (auto& d : shape) {
      uint64_t v = d.c;
      if (d.is_var) {
        auto it = m_.vars.find(d.var);
        if (it == m_.vars.end()) { err(ctx + ": shape names unknown var `" + d.var + "`"); ok = false; continue; }
        used_vars_.insert(d.var);
        v = it->second.max;
      }
      n *= v;
      if (n > UINT64_MAX) { err(ctx + ": size overflows 64 bits at var upper bounds"); return std::nullopt; }
    }
    if (!ok) return std::nullopt;
    return (uint64_t)n;
  }

  // ---- 1, 2, topology, cut, chat ----
  void header() {
    if (m_.schema_version != SCHEMA_VERSION)
      err("unsupported schema_version " + std::to_string(m_.schema_version) + " (this runtime reads " +
          std::to_string(SCHEMA_VERSION) + ")");
    for (auto& kv : m_.vars)
      if (kv.second.max < VAR_MIN) err("var `" + kv.first + "`: max must be >= " + std::to_string(VAR_MIN));
    for (VarAxis ax : {VarAxis::Rows, VarAxis::Groups, VarAxis::Ranks}) {
      std::string names;
      int n = 0;
      for (auto& kv : m_.vars) if (kv.second.axis == ax) { names += (n ? ", `" : "`") + kv.first + "`"; ++n; }
      if (n > 1) err("vars " + names + " all count the `" + axis_name(ax) + "` axis; exactly one var does");
    }
    for (auto& kv : m_.topology)
      if (kv.second == 0) err("topology group `" + kv.first + "`: size must be > 0");
    if (m_.cut && (m_.cut->id.empty() || m_.cut->stages < 2 || m_.cut->stage >= m_.cut->stages))
      err("cut: stage " + std::to_string(m_.cut->stage) + " of " + std::to_string(m_.cut->stages) + " with id `" +
          m_.cut->id + "`; a cut has an id, at least 2 stages and a stage below their count");
    if (m_.tool_parser) {
      const std::string& n = *m_.tool_parser;
      bool ok = !n.empty() && std::all_of(n.begin(), n.end(), [](unsigned char c) {
        return (c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '_'; });
      if (!ok) err("chat.tool_parser `" + n + "`: a parser name is lowercase letters, digits and underscores");
    }
  }

  // ---- 3 ----
  void states() {
    for (auto& kv : m_.states) {
      const State& s = kv.second;
      int set = (s.bytes_per_token > 0) + (s.bytes > 0) + (s.bytes_per_seq > 0);
      const std::string ctx = "state `" + kv.first + "`";
      if (s.host) {
        if (set) { err(ctx + ": a host state is sized by the host; bytes_per_token / bytes / bytes_per_seq must be absent"); continue; }
        const HostTensor& h = *s.host;
        if (h.shape.empty() || h.shape.size() != h.strides.size()) {
          err(ctx + ": host: " + std::to_string(h.shape.size()) + " extents and " + std::to_string(h.strides.size()) +
              " strides; want as many of each, at least one");
          continue;
        }
        if (std::any_of(h.shape.begin() + 1, h.shape.end(), [](uint64_t n) { return n == 0; }))
          err(ctx + ": host: only the outermost extent may be 0 (the host's count)");
        if (std::count(h.strides.begin(), h.strides.end(), 0)) err(ctx + ": host: a zero stride aliases elements");
        if (!h.span(1)) err(ctx + ": host: shape with these strides overflows 64 bits");
      } else if (set == 0) {
        err(ctx + ": one of bytes_per_token / bytes / bytes_per_seq / host must be set");
      } else if (set > 1) {
        err(ctx + ": bytes_per_token, bytes and bytes_per_seq are exclusive");
      }
    }
  }

  // ---- 13 ----
  void shards() {
    const std::string* dealt_state = nullptr;
    const std::string* dealt_group = nullptr;
    for (auto& kv : m_.states) {
      const State& s = kv.second;
      if (!s.shard) continue;
      const std::string ctx = "state `" + kv.first + "`: shard";
      auto w = group(s.shard->group, ctx);
      if (s.shard->by == Shard::Position) {
        if (!is_paged_owned(s)) err(ctx + ": `by: position` deals a paged state, got a " + state_kind(s) + " one");
        else if (!dealt_state) { dealt_state = &kv.first; dealt_group = &s.shard->group; }
      } else {
        if (!(s.is_owned() && s.is_per_seq())) {
          err(ctx + ": `by: heads` splits a per-sequence state, got a " + std::string(state_kind(s)) + " one");
        } else if (w) {
          heads(ctx, s.shard->group, *w, s.bytes_per_seq, s.shard->segments);
        }
      }
    }
    if (!dealt_state) return;
    for (auto& kv : m_.states) {
      if (!is_paged_owned(kv.second)) continue;
      const auto& sh = kv.second.shard;
      if (sh && sh->by == Shard::Position && sh->group == *dealt_group) continue;
      if (sh && sh->by == Shard::Position)
        err("state `" + kv.first + "`: shard deals positions over `" + sh->group + "`, but `" + *dealt_state +
            "` deals them over `" + *dealt_group + "`; the paged states share one page id space, so one group deals them all");
      else
        err("state `" + kv.first + "`: not dealt by position, but `" + *dealt_state + "` is dealt over `" + *dealt_group +
            "`; the paged states share one page id space, so every one is dealt the same way");
    }
    const std::string why = "state `" + *dealt_state + "` deals positions over `" + *dealt_group +
                            "`, so the group runs one replicated batch";
    for (auto& kv : m_.vars)
      if (kv.second.axis == VarAxis::Ranks)
        err("var `" + kv.first + "`: `axis: ranks` gives every member its own rows, but " + why);
    for (auto& kv : m_.buffers)
      if (kv.second.fill && *kv.second.fill == Fill::Blocks)
        err("buffer `" + kv.first + "`: fill `blocks` splits the group's batch into members' blocks, but " + why);
  }
  void heads(const std::string& ctx, const std::string& g, uint64_t w, uint64_t bps,
             const std::vector<std::pair<uint64_t, uint64_t>>& segs) {
    if (segs.empty()) { err(ctx + ": `by: heads` needs at least one segment"); return; }
    unsigned __int128 line = 0;
    for (size_t i = 0; i < segs.size(); ++i) {
      auto [rows, width] = segs[i];
      if (rows == 0 || width == 0)
        err(ctx + ": segment #" + std::to_string(i) + " is " + std::to_string(rows) + " rows of " + std::to_string(width) +
            " bytes, expected neither 0");
      else if (width % w)
        err(ctx + ": segment #" + std::to_string(i) + " rows are " + std::to_string(width) +
            " bytes, expected a multiple of the " + std::to_string(w) + " members of `" + g + "`");
      line += (unsigned __int128)rows * width;
    }
    unsigned __int128 want = (unsigned __int128)w * bps;
    if (line != want)
      err(ctx + ": segments span " + (line > UINT64_MAX ? std::string("more than 2^64") : std::to_string((uint64_t)line)) +
          " bytes, expected the " + std::to_string(w) + " members of `" + g + "` times bytes_per_seq " +
          std::to_string(bps) + " = " + (want > UINT64_MAX ? std::string("more than 2^64") : std::to_string((uint64_t)want)));
  }

  // ---- 4, 11 (peer) ----
  void buffers() {
    for (auto& kv : m_.buffers) {
      const std::string& name = kv.first;
      const Buffer& b = kv.second;
      const std::string ctx = "buffer `" + name + "`";
      if (auto sz = shaped_bytes(ctx, b.dtype, b.shape)) buf_bytes_[name] = *sz;
      if (b.domain) domain(name, b, *b.domain);
      if (b.fill) {
        const bool out = fill_is_output(*b.fill);
        if (b.kind != BufferKind::Input && b.kind != BufferKind::Output)
          err(ctx + ": a fill sits on an input or output, not a " + kind_name(b.kind) + " buffer");
        else if ((b.kind == BufferKind::Output) != out)
          err(ctx + ": fill `" + fill_name(*b.fill) + "` is " + (out ? "read from an output" : "written into an input") +
              " but the buffer is " + kind_name(b.kind));
        auto dts = fill_dtypes(*b.fill);
        if (std::find(dts.begin(), dts.end(), b.dtype) == dts.end()) {
          std::string wants;
          for (size_t i = 0; i < dts.size(); ++i) wants += (i ? " or " : "") + std::string(dtype_name(dts[i]));
          err(ctx + ": fill `" + fill_name(*b.fill) + "` needs an " + wants + " buffer, not " + dtype_name(b.dtype));
        }
      }
      if (b.host_placement) {
        if (b.kind != BufferKind::Weight || b.export_) err(ctx + ": host placement requires a non-exported immutable weight");
        for (auto& s : b.bind)
          if (s.tensor.ranked || (s.rows && s.rows->ranked) || (s.cols && s.cols->ranked) ||
              (s.interleave && s.interleave->with.ranked)) {
            err(ctx + ": shared host weights cannot select tensors, rows or columns by rank");
            break;
          }
      }
      if (b.kind == BufferKind::Source && b.export_) err(ctx + ": a source lives only while weights load; it cannot be exported");
      const bool binds = b.kind == BufferKind::Weight || b.kind == BufferKind::Source;
      if (binds && b.bind.empty()) err(ctx + ": a " + kind_name(b.kind) + " buffer binds at least one checkpoint tensor (`bind`)");
      if (!binds && !b.bind.empty())
        err(ctx + ": `bind` names checkpoint tensors for a weight or a source, not a " + kind_name(b.kind) + " buffer");
      if (binds) for (size_t i = 0; i < b.bind.size(); ++i) segment(ctx + ": bind[" + std::to_string(i) + "]", b.bind[i]);
      if (b.kind == BufferKind::Peer) peer(name, b, ctx);
      else {
        if (b.of) err(ctx + ": `of` only applies to peer buffers");
        if (b.group) err(ctx + ": `group` only applies to peer buffers");
      }
    }
  }
  void tensor_source(const std::string& ctx, const TensorSource& t) {
    if (!t.ranked) { if (t.name.empty()) err(ctx + ": empty tensor name"); return; }
    if (auto n = group(t.group, ctx))
      if (*n != t.tensors.size())
        err(ctx + ": group `" + t.group + "` needs " + std::to_string(*n) + " tensor names, got " + std::to_string(t.tensors.size()));
    for (auto& s : t.tensors) if (s.empty()) { err(ctx + ": empty tensor name"); break; }
  }
  void ranges(const std::string& ctx, const char* axis, const std::optional<Ranges>& r) {
    if (!r) return;
    std::vector<std::pair<uint64_t, uint64_t>> rs;
    if (!r->ranked) rs.emplace_back(r->range[0], r->range[1]);
    else {
      if (auto n = group(r->group, ctx))
        if (*n != r->ranges.size())
          err(ctx + ": group `" + r->group + "` needs " + std::to_string(*n) + " " + axis + " ranges, got " + std::to_string(r->ranges.size()));
      rs = r->ranges;
    }
    for (auto& p : rs)
      if (p.first >= p.second) err(ctx + ": " + axis + " [" + std::to_string(p.first) + ", " + std::to_string(p.second) + ") is empty");
  }
  void segment(const std::string& ctx, const Segment& s) {
    tensor_source(ctx, s.tensor);
    if (s.interleave) {
      tensor_source(ctx, s.interleave->with);
      if (s.interleave->rows == 0) err(ctx + ": interleave blocks of 0 rows");
      if (s.rows || s.cols) err(ctx + ": an interleaved segment takes both tensors whole, not a range");
    }
    ranges(ctx, "rows", s.rows);
    ranges(ctx, "cols", s.cols);
  }
  void peer(const std::string& name, const Buffer& b, const std::string& ctx) {
    if (b.export_) err(ctx + ": a peer buffer cannot itself be exported");
    if (b.dtype != DType::u64) err(ctx + ": a peer buffer holds device addresses, dtype must be u64, not " + std::string(dtype_name(b.dtype)));
    if (b.domain) err(ctx + ": a peer buffer's contents are runtime-filled addresses; it takes no domain");
    if (!b.of) err(ctx + ": a peer buffer must name the exported buffer or state it holds addresses `of`");
    else if (*b.of == name) err(ctx + ": a peer buffer cannot be `of` itself");
    else {
      auto bi = m_.buffers.find(*b.of);
      auto si = m_.states.find(*b.of);
      if (bi != m_.buffers.end() && si != m_.states.end()) err(ctx + ": `of` `" + *b.of + "` is both a buffer and a state");
      else if (bi != m_.buffers.end()) {
        used_buffers_.insert(*b.of);
        if (bi->second.kind == BufferKind::Peer) err(ctx + ": `of` `" + *b.of + "` is itself a peer buffer");
        else if (!bi->second.export_) err(ctx + ": `of` buffer `" + *b.of + "` is not exported");
      } else if (si != m_.states.end()) {
        used_states_.insert(*b.of);
        if (!si->second.is_owned()) err(ctx + ": `of` state `" + *b.of + "` is the host's; only runtime memory is exported");
      } else err(ctx + ": `of` unknown buffer/state `" + *b.of + "`");
    }
    if (!b.group) err(ctx + ": a peer buffer must name the topology `group` its addresses are indexed by");
    else if (auto sz = group(*b.group, ctx)) {
      if (!(b.shape.size() == 1 && !b.shape[0].is_var && b.shape[0].c == *sz))
        err(ctx + ": a peer buffer over group `" + *b.group + "` has shape [" + std::to_string(*sz) + "], one address per member");
    }
  }
  void domain(const std::string& name, const Buffer& b, const Domain& d) {
    const std::string ctx = "buffer `" + name + "` domain";
    const bool fl = dtype_is_float(b.dtype);
    if (d.index_into && (d.min || d.max)) err(ctx + ": `index_into` and `min`/`max` are mutually exclusive");
    if (!d.index_into && !d.min && !d.max && !d.monotone) err(ctx + ": empty (declare bounds, `index_into`, or `monotone`)");
    if (d.stride == 0) err(ctx + ": `stride` must be > 0");
    if (d.stride > 1 && !d.index_into) err(ctx + ": `stride` only applies with `index_into`");
    if (d.index_into) {
      const std::string& t = *d.index_into;
      if (fl) err(ctx + ": a " + std::string(dtype_name(b.dtype)) + " buffer cannot index anything");
      const bool ib = m_.buffers.count(t), is = m_.states.count(t);
      if (!ib && !is) err(ctx + ": `index_into` unknown buffer/state `" + t + "`");
      else if (ib && is) err(ctx + ": `index_into` `" + t + "` is both a buffer and a state");
      else if (is) {
        const State& s = m_.states.at(t);
        if (s.is_per_seq() && s.bytes_per_seq % std::max<uint64_t>(d.stride, 1))
          err(ctx + ": `index_into` per-sequence state `" + t + "` in lines of " + std::to_string(d.stride) +
              " bytes, which do not divide its " + std::to_string(s.bytes_per_seq) + " bytes per sequence");
      } else if (t == name) err(ctx + ": a buffer cannot index itself");
    }
    if (d.monotone && b.shape.size() != 1) err(ctx + ": `monotone` requires a one-dimensional buffer");
    for (auto* bd : {&d.min, &d.max}) {
      if (!*bd) continue;
      const char* which = bd == &d.min ? "min" : "max";
      if ((*bd)->kind == Bound::Float && !fl) err(ctx + ": float `" + which + "` on a " + dtype_name(b.dtype) + " buffer");
      if ((*bd)->kind == Bound::Ex) expr((*bd)->expr, ctx + ": `" + which + "`");
    }
    if (d.min && d.max)
      for (const VarMap* vm : {&vmin_, &vmax_}) {
        auto lo = d.min->eval(*vm), hi = d.max->eval(*vm);
        if (lo && hi && *lo > *hi) { err(ctx + ": min " + std::to_string(*lo) + " > max " + std::to_string(*hi)); break; }
      }
  }

  // ---- 5 ----
  void modules() {
    for (auto& kv : m_.modules) {
      const std::string ctx = "module `" + kv.first + "`";
      const std::string& h = kv.second.sha256;
      if (h.size() != 64 || !std::all_of(h.begin(), h.end(), [](unsigned char c) { return std::isxdigit(c); }))
        err(ctx + ": sha256 `" + h + "` is not 64 hex chars");
      if (kv.second.source.empty()) err(ctx + ": empty source");
      std::string url, why;
      if (registry_ref_parse(kv.second.source, url, why) < 0) err(ctx + ": " + why);
    }
  }

  // ---- 6, 7, 12 ----
  void ops();
  void launch_geometry(const Launch& l, const std::string& ctx);
  void pack_fields(const std::string& oname, const Op& op, const Pack& pk, const std::string& actx,
                   std::vector<bool>& iface_written, std::set<std::string>& s_used, std::set<std::string>& s_written);
  // ---- 8, 9 ----
  void programs();
  void multicast_declarations();
  void unused();
};

void Verifier::launch_geometry(const Launch& l, const std::string& ctx) {
  if (l.entry.empty()) err(ctx + ": empty entry");
  if (l.entry.rfind("extern:", 0) == 0) err(ctx + ": an extern entry has no module or launch geometry");
  if (m_.modules.count(l.module)) used_modules_.insert(l.module); else err(ctx + ": unknown module `" + l.module + "`");
  const uint64_t threads = (uint64_t)l.block[0] * l.block[1] * l.block[2];
  if (!l.block[0] || !l.block[1] || !l.block[2] || threads > Limits::kMaxBlockThreads)
    err(ctx + ": block " + triple(l.block) + " exceeds " + std::to_string(Limits::kMaxBlockThreads) + " threads or has a zero dim");
  if (l.block[2] > Limits::kMaxBlockZ) err(ctx + ": block.z " + std::to_string(l.block[2]) + " > " + std::to_string(Limits::kMaxBlockZ));
  static const char* ax[] = {"x", "y", "z"};
  for (int i = 0; i < 3; ++i) {
    const std::string ectx = ctx + ": grid." + ax[i];
    expr(l.grid[i], ectx);
    std::string why;
    auto v = l.grid[i].eval(vmax_, &why);
    if (!v) { if (why.rfind("unknown var", 0) != 0) err(ectx + ": " + why); continue; }
    if (*v == 0) err(ectx + ": evaluates to 0 at var upper bounds");
    const uint64_t lim = i == 0 ? Limits::kMaxGridX : Limits::kMaxGridYZ;
    if (*v > lim) err(ectx + ": " + std::to_string(*v) + " exceeds CUDA limit " + std::to_string(lim) + " at var upper bounds");
  }
  if (l.shared_mem) {
    expr(*l.shared_mem, ctx + ": shared_mem");
    auto v = l.shared_mem->eval(vmax_);
    if (v && *v > Limits::kMaxDynSharedMem)
      err(ctx + ": shared_mem: " + std::to_string(*v) + " bytes exceeds opt-in limit " + std::to_string(Limits::kMaxDynSharedMem) + " at var upper bounds");
  }
  if (l.cluster) {
    const auto& c = *l.cluster;
    const uint64_t blocks = (uint64_t)c[0] * c[1] * c[2];
    if (!c[0] || !c[1] || !c[2] || blocks > Limits::kMaxClusterBlocks) {
      err(ctx + ": cluster " + triple(c.data()) + " has a zero dim or more than " + std::to_string(Limits::kMaxClusterBlocks) + " blocks");
    } else {
      for (int i = 0; i < 3; ++i)
        for (const VarMap* vm : {&vmax_, &vmin_}) {
          auto v = l.grid[i].eval(*vm);
          if (v && *v % c[i])
            err(ctx + ": grid." + ax[i] + " = " + std::to_string(*v) + " at var " + (vm == &vmax_ ? "upper" : "lower") +
                " bounds is not a multiple of cluster." + ax[i] + " = " + std::to_string(c[i]));
        }
    }
  }
}

void Verifier::pack_fields(const std::string& oname, const Op& op, const Pack& pk, const std::string& actx,
                           std::vector<bool>& iface_written, std::set<std::string>& s_used,
                           std::set<std::string>& s_written) {
  for (auto& e : pk.check(op.params)) err(actx + ": " + e);
  for (size_t k = 0; k < pk.fields.size(); ++k) {
    const Field& f = pk.fields[k];
    const std::string fctx = actx + ": field #" + std::to_string(k);
    auto iface = [&](size_t i) -> const ParamType* {
      if (i < op.params.size()) return &op.params[i];
      err(fctx + ": interface param #" + std::to_string(i) + " out of range (" + std::to_string(op.params.size()) + " interface params)");
      return nullptr;
    };
    switch (f.src.kind) {
      case FieldSrc::Param:
        if (auto* p = iface(f.src.param)) if (p->writes()) iface_written[f.src.param] = true;
        break;
      case FieldSrc::Scratch:
        if (!op.scratch.count(f.src.name)) err(fctx + ": unknown scratch `" + f.src.name + "`");
        else { s_used.insert(f.src.name); s_written.insert(f.src.name); }
        break;
      case FieldSrc::Var:
        if (m_.vars.count(f.src.name)) used_vars_.insert(f.src.name); else err(fctx + ": unknown var `" + f.src.name + "`");
        break;
      case FieldSrc::ExprK: expr(f.src.expr, fctx); break;
      case FieldSrc::Rank: group(f.src.name, fctx); break;
      case FieldSrc::TensorMap: {
        const TensorMapDecl& t = f.src.tmap;
        auto* p = iface(t.param);
        if (!p) break;
        if (!p->is_pointer()) {
          err(fctx + ": tensormap over interface param #" + std::to_string(t.param) + " (`" + p->str() + "`), which is not a buffer or state");
          break;
        }
        for (auto& e : t.check()) err(fctx + ": " + e);
        if (p->writes()) iface_written[t.param] = true;
        auto fp = t.footprint();
        if (t.wrap) { if (fp) err(fctx + ": `wrap` on a tensormap whose strides do not overflow"); }
        else if (fp) op_tmaps_[oname].push_back({t.param, *fp, fctx});
        else err(fctx + ": the tensormap's strides overflow (declare `wrap` if that is the kernel's trick)");
        break;
      }
      default: break;
    }
  }
}

void Verifier::ops() {
  for (auto& okv : m_.ops) {
    const std::string& oname = okv.first;
    const Op& op = okv.second;
    for (size_t i = 0; i < op.params.size(); ++i)
      if (op.params[i].kind == ParamType::Bytes)
        err("op `" + oname + "`: interface param #" + std::to_string(i) +
            " is a byte aggregate; packs are launch-private, the interface takes the buffers and scalars they are assembled from");
    for (auto& skv : op.scratch) shaped_bytes("op `" + oname + "` scratch `" + skv.first + "`", skv.second.dtype, skv.second.shape);
    if (op.launches.empty()) err("op `" + oname + "`: implementation has no launches");

    std::vector<bool> iface_written(op.params.size());
    for (size_t i = 0; i < op.params.size(); ++i)
      iface_written[i] = !(op.params[i].is_pointer() && op.params[i].dir == ParamType::Out);
    std::set<std::string> s_written, s_used;

    for (size_t li = 0; li < op.launches.size(); ++li) {
      const Launch& l = op.launches[li];
      const std::string ctx = "op `" + oname + "` launch #" + std::to_string(li) + " (" + l.entry + ")";
      if (l.when) {
        if (m_.vars.count(l.when->var)) used_vars_.insert(l.when->var); else err(ctx + ": when: unknown var `" + l.when->var + "`");
        if (l.when->min && l.when->max && *l.when->min > *l.when->max)
          err(ctx + ": when: `" + l.when->var + "` range [" + std::to_string(*l.when->min) + ", " + std::to_string(*l.when->max) + "] is empty");
      }
      const auto& params = op.params_of(l);
      if (l.is_extern) {
        if (l.entry.rfind("extern:", 0) != 0) err(ctx + ": a launch without a module must be a runtime built-in (`extern:<name>`)");
        if (l.algo && l.entry != "extern:cublaslt_bf16_tn" && l.entry != "extern:cublaslt_bf16_tn_acc")
          err(ctx + ": `algo` pins a cublaslt_bf16_tn[_acc] launch, not `" + l.entry + "`");
        if (std::any_of(params.begin(), params.end(), [](const ParamType& p) { return p.kind == ParamType::Bytes; }))
          err(ctx + ": an extern launch takes pointers and scalars, not a pack");
      } else {
        launch_geometry(l, ctx);
      }
      const auto args = op.args_of(l);
      if (args.size() != params.size()) {
        err(ctx + ": takes " + std::to_string(params.size()) + " params, got " + std::to_string(args.size()) + " args");
        continue;
      }
      for (size_t j = 0; j < args.size(); ++j) {
        const LaunchArg& a = args[j];
        const ParamType& p = params[j];
        const std::string actx = ctx + ": arg #" + std::to_string(j);
        switch (a.kind) {
          case LaunchArg::Param: {
            if (a.param >= op.params.size()) {
              err(actx + ": interface param #" + std::to_string(a.param) + " out of range (" + std::to_string(op.params.size()) + " interface params)");
              break;
            }
            const ParamType& iface = op.params[a.param];
            bool compat = iface.kind == p.kind &&
                          (iface.kind == ParamType::State || (iface.kind != ParamType::Bytes && iface.dtype == p.dtype));
            if (!compat) { err(actx + ": interface param `" + iface.str() + "` does not match launch param `" + p.str() + "`"); break; }
            if (!iface.is_pointer()) break;
            if (p.writes() && iface.dir == ParamType::In) err(actx + ": launch writes through interface `in` param #" + std::to_string(a.param));
            if (p.reads() && !iface_written[a.param]) err(actx + ": interface `out` param #" + std::to_string(a.param) + " read before any launch wrote it");
            if (p.writes()) iface_written[a.param] = true;
            break;
          }
          case LaunchArg::Scratch: {
            auto it = op.scratch.find(a.name);
            if (it == op.scratch.end()) { err(actx + ": unknown scratch `" + a.name + "`"); break; }
            s_used.insert(a.name);
            if (p.kind != ParamType::Buffer) { err(actx + ": scratch `" + a.name + "` bound to non-buffer param `" + p.str() + "`"); break; }
            if (it->second.dtype != p.dtype)
              err(actx + ": scratch `" + a.name + "` has dtype " + dtype_name(it->second.dtype) + " but param expects " + dtype_name(p.dtype));
            if (p.reads() && !s_written.count(a.name)) err(actx + ": scratch `" + a.name + "` is read before any launch wrote it");
            if (p.writes()) s_written.insert(a.name);
            break;
          }
          case LaunchArg::Rank:
            if (!(p.kind == ParamType::Scalar && (p.dtype == DType::i32 || p.dtype == DType::i64)))
              err(actx + ": a rank binds only to an i32 or i64 param, not `" + p.str() + "`");
            group(a.name, actx);
            break;
          case LaunchArg::PackK:
            if (p.kind != ParamType::Bytes) err(actx + ": a pack binds only to a `bytes<n>` param, not `" + p.str() + "`");
            else if (p.nbytes != a.pack.size) err(actx + ": pack of " + std::to_string(a.pack.size) + " bytes bound to a `" + p.str() + "` param");
            pack_fields(oname, op, a.pack, actx, iface_written, s_used, s_written);
            break;
          default: {
            static const DType want[] = {DType::i32, DType::i32, DType::i32, DType::i64, DType::f32, DType::u8};
            if (!(p.kind == ParamType::Scalar && p.dtype == want[a.kind]))
              err(actx + ": " + a.str() + " does not match launch param `" + p.str() + "`");
          }
        }
      }
    }
    for (size_t i = 0; i < op.params.size(); ++i)
      if (!iface_written[i]) err("op `" + oname + "`: interface `" + op.params[i].str() + "` param #" + std::to_string(i) + " is never written by any launch");
    for (auto& skv : op.scratch)
      if (!s_used.count(skv.first)) err("op `" + oname + "`: scratch `" + skv.first + "` is never used");
  }
}

void Verifier::programs() {
  if (m_.programs.empty()) err("no programs declared");
  std::set<std::string> initially;
  for (auto& kv : m_.buffers) {
    auto k = kv.second.kind;
    if (k == BufferKind::Input || k == BufferKind::Inout || k == BufferKind::Weight || k == BufferKind::Source ||
        k == BufferKind::Carry || k == BufferKind::Peer)
      initially.insert(kv.first);
  }
  std::set<std::string> ever_written;
  for (auto& pkv : m_.programs) {
    const std::string& pname = pkv.first;
    const Program& p = pkv.second;
    const std::string pctx = "program `" + pname + "`";
    if (p.once && p.batch) err(pctx + ": `once` (run after load) and `batch` (driven per step) are exclusive");
    if (p.derive && (p.once || p.batch || p.graph)) err(pctx + ": `derive` (run inside weight loading) excludes `once`, `batch` and `graph`");
    if (p.graph && !p.batch) err(pctx + ": `graph` (captured per call shape) needs a `batch`");
    if (p.batch) {
      if (p.batch->groups == 0) err(pctx + ": batch.groups must be >= 1");
      if (!p.batch->rows.is_var) { if (p.batch->rows.c == 0) err(pctx + ": batch.rows must be >= 1"); }
      else if (m_.vars.count(p.batch->rows.var)) used_vars_.insert(p.batch->rows.var);
      else err(pctx + ": batch.rows names unknown var `" + p.batch->rows.var + "`");
      if (p.batch->context) {
        if (m_.vars.count(*p.batch->context)) used_vars_.insert(*p.batch->context);
        else err(pctx + ": batch.context names unknown var `" + *p.batch->context + "`");
      }
    }
    std::set<std::string> written = initially;
    for (size_t i = 0; i < p.calls.size(); ++i) {
      const Call& c = p.calls[i];
      const std::string ctx = pctx + " call #" + std::to_string(i) + (c.label ? " (" + *c.label + ")" : "");
      auto oit = m_.ops.find(c.op);
      if (oit == m_.ops.end()) { err(ctx + ": unknown op `" + c.op + "`"); continue; }
      used_ops_.insert(c.op);
      const Op& op = oit->second;
      const bool has_extern = std::any_of(op.launches.begin(), op.launches.end(), [](const Launch& l) { return l.is_extern; });
      if (p.derive && std::any_of(op.launches.begin(), op.launches.end(), [](const Launch& l) { return l.entry.rfind("extern:nccl", 0) == 0; }))
        err(ctx + ": a `derive` program runs before any group is joined; op `" + c.op + "` is a collective");
      if (c.args.size() != op.params.size()) {
        err(ctx + ": op `" + c.op + "` takes " + std::to_string(op.params.size()) + " params, got " + std::to_string(c.args.size()) + " args");
        continue;
      }
      for (size_t j = 0; j < c.args.size(); ++j) {
        const Arg& a = c.args[j];
        const ParamType& pt = op.params[j];
        const std::string actx = ctx + ": arg #" + std::to_string(j);
        if (a.kind == Arg::Buf && pt.kind == ParamType::Buffer) {
          used_buffers_.insert(a.name);
          auto bit = m_.buffers.find(a.name);
          if (bit == m_.buffers.end()) { err(actx + ": unknown buffer `" + a.name + "`"); continue; }
          const Buffer& b = bit->second;
          if (b.dtype != pt.dtype)
            err(actx + ": buffer `" + a.name + "` has dtype " + dtype_name(b.dtype) + " but param expects " + dtype_name(pt.dtype));
          auto szit = buf_bytes_.find(a.name);
          if (a.offset > 0) {
            if (a.offset % dtype_bytes(b.dtype))
              err(actx + ": offset " + std::to_string(a.offset) + " into buffer `" + a.name + "` is not " +
                  std::to_string(dtype_bytes(b.dtype)) + "-aligned for " + dtype_name(b.dtype));
            if (szit != buf_bytes_.end() && a.offset >= szit->second)
              err(actx + ": offset " + std::to_string(a.offset) + " is outside buffer `" + a.name + "` (" +
                  std::to_string(szit->second) + " bytes at var upper bounds)");
          }
          if (pt.reads() && !written.count(a.name)) err(actx + ": buffer `" + a.name + "` is read before ever being written");
          auto tm = op_tmaps_.find(c.op);
          if (tm != op_tmaps_.end() && szit != buf_bytes_.end())
            for (auto& t : tm->second) {
              if (t.param != j) continue;
              const uint64_t avail = szit->second > a.offset ? szit->second - a.offset : 0;
              if (t.footprint > avail)
                err(actx + ": " + t.where + " addresses " + std::to_string(t.footprint) + " bytes but buffer `" + a.name +
                    "` has " + std::to_string(avail) + " bytes past offset " + std::to_string(a.offset) + " at var upper bounds");
            }
          if (!p.derive && b.kind == BufferKind::Source)
            err(actx + ": source buffer `" + a.name + "` is read only by a `derive` program; it is gone after load");
          if (p.derive && (b.kind == BufferKind::Input || b.kind == BufferKind::Output || b.kind == BufferKind::Inout || b.kind == BufferKind::Peer))
            err(actx + ": a `derive` program runs inside weight loading, before any " + kind_name(b.kind) + " buffer such as `" + a.name + "` means anything");
          if (b.kind == BufferKind::Peer) {
            if (has_extern)
              err(actx + ": peer buffer `" + a.name + "` passed to op `" + c.op + "`, which has an extern launch; runtime built-ins never receive peer memory");
            for (auto& l : op.launches) if (!l.is_extern) peer_modules_.insert(l.module);
          }
          if (pt.writes()) {
            if (b.kind == BufferKind::Input || b.kind == BufferKind::Weight || b.kind == BufferKind::Source || b.kind == BufferKind::Peer)
              err(actx + ": op writes to read-only " + kind_name(b.kind) + " buffer `" + a.name + "`");
            written.insert(a.name);
            ever_written.insert(a.name);
          }
        } else if (a.kind == Arg::StateK && pt.kind == ParamType::State) {
          used_states_.insert(a.name);
          if (p.derive) err(actx + ": a `derive` program runs inside weight loading, before state `" + a.name + "` holds anything");
          if (!m_.states.count(a.name)) err(actx + ": unknown state `" + a.name + "`");
        } else if (a.kind == Arg::Var && pt.kind == ParamType::Scalar) {
          used_vars_.insert(a.name);
          auto vit = m_.vars.find(a.name);
          if (vit == m_.vars.end()) err(actx + ": unknown var `" + a.name + "`");
          else if (pt.dtype == DType::f32) err(actx + ": var `" + a.name + "` cannot bind to an f32 param");
          else if (!scalar_fits(pt.dtype, vit->second.max))
            err(actx + ": var `" + a.name + "` max " + std::to_string(vit->second.max) + " exceeds " + dtype_name(pt.dtype) + " range");
        } else if (a.kind == Arg::ExprK && pt.kind == ParamType::Scalar) {
          expr(a.expr, actx);
          if (pt.dtype == DType::f32) err(actx + ": an expression cannot bind to an f32 param");
          else if (auto v = a.expr.eval(vmax_))
            if (!scalar_fits(pt.dtype, *v))
              err(actx + ": expression reaches " + std::to_string(*v) + " at var upper bounds, exceeding " + dtype_name(pt.dtype) + " range");
        } else if (a.kind == Arg::Rank && pt.kind == ParamType::Scalar && (pt.dtype == DType::i32 || pt.dtype == DType::i64)) {
          group(a.name, actx);
        } else if (pt.kind == ParamType::Scalar &&
                   ((a.kind == Arg::I32 && pt.dtype == DType::i32) || (a.kind == Arg::I64 && pt.dtype == DType::i64) ||
                    (a.kind == Arg::F32 && pt.dtype == DType::f32) || (a.kind == Arg::U8 && pt.dtype == DType::u8))) {
        } else {
          err(actx + ": " + a.str() + " does not match param `" + pt.str() + "`");
        }
      }
    }
  }
  for (auto& kv : m_.buffers)
    if ((kv.second.kind == BufferKind::Output || kv.second.kind == BufferKind::Carry) && !ever_written.count(kv.first))
      err(std::string(kind_name(kv.second.kind)) + " buffer `" + kv.first + "` is never written by any program");
}

// A launch that can receive a peer buffer, and every kernel module of a manifest whose topology has
// two or more ranks, must come from a module declared `multicast: false` — built from sources that
// pass the no-cluster-multicast lint. This replaces the reference's load-time disassembly scan
// (crates/kern-runtime/src/cubin.rs:273-381) with a declaration the build can vouch for.
void Verifier::multicast_declarations() {
  bool multi = false;
  for (auto& kv : m_.topology) multi |= kv.second >= 2;
  for (auto& kv : m_.modules) {
    const bool needs = peer_modules_.count(kv.first) || (multi && used_modules_.count(kv.first));
    if (needs && !kv.second.multicast_free)
      err("module `" + kv.first + "`: " + (peer_modules_.count(kv.first) ? "a launch of it receives a peer buffer" : "the manifest runs on 2 or more ranks") +
          ", so it must declare `multicast: false` (no cluster-multicast copy may touch peer memory)");
  }
}

void Verifier::unused() {
  for (auto& kv : m_.buffers) if (!used_buffers_.count(kv.first)) err("buffer `" + kv.first + "` is never used by any program");
  for (auto& kv : m_.ops) if (!used_ops_.count(kv.first)) err("op `" + kv.first + "` is never called");
  for (auto& kv : m_.modules) if (!used_modules_.count(kv.first)) err("module `" + kv.first + "` is never launched");
  for (auto& kv : m_.states) if (!used_states_.count(kv.first)) err("state `" + kv.first + "` is never used by any program");
  for (auto& kv : m_.vars) if (!used_vars_.count(kv.first)) err("var `" + kv.first + "` is never used");
  for (auto& kv : m_.topology)
    if (!used_groups_.count(kv.first)) err("topology group `" + kv.first + "` is never used (no peer buffer, shard or rank arg names it)");
}

}  // namespace

Errors verify_manifest(const Manifest& m, bool strict_multicast) { return Verifier(m, strict_multicast).run(); }

bool verify_text(const std::string& text, Manifest& out, Errors& errs) {
  out = parse_manifest_text(text, errs);
  if (!errs.empty()) return false;
  errs = verify_manifest(out);
  return errs.empty();
}

}  // namespace kern
