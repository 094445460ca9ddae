// Projection of the serving protocol out of a verified manifest (see protocol.hpp).
#include "protocol.hpp"

#include <algorithm>
#include <set>

namespace kern {

std::string PAxis::str() const {
  switch (kind) {
    case Rows: return "rows";
    case Groups: return "groups";
    case Ranks: return "ranks";
    default: return "fixed(" + std::to_string(n) + ")";
  }
}

const Forward* Protocol::forward(uint64_t g, bool rows_var, uint64_t r) const {
  for (auto& f : forwards)
    if (f.rows_var == rows_var && (rows_var || f.rows == r) && g <= f.groups) return &f;
  return nullptr;
}
std::vector<uint64_t> Protocol::row_shapes() const {
  std::vector<uint64_t> v;
  for (auto& f : forwards) if (!f.rows_var) v.push_back(f.rows);
  std::sort(v.begin(), v.end());
  return v;
}
const Filled* Protocol::filled(Fill f, PAxis::Kind axis) const {
  for (auto& x : fills) if (x.fill == f && x.axis.kind == axis) return &x;
  return nullptr;
}
const Filled* Protocol::any(Fill f) const {
  for (auto& x : fills) if (x.fill == f) return &x;
  return nullptr;
}
VarMap Protocol::vars(uint64_t g, uint64_t r, uint64_t rk, uint64_t ctx) const {
  VarMap v{{rows.var, r}, {groups.var, g}};
  if (ranks) v[ranks->var] = rk;
  if (context) v[context->var] = ctx;
  return v;
}

namespace {

std::string shape_str(const std::vector<Dim>& s) {
  std::string o = "[";
  for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + (s[i].is_var ? "`" + s[i].var + "`" : std::to_string(s[i].c));
  return o + "]";
}

const char* fill_shape_hint(Fill f) {
  switch (f) {
    case Fill::Token: return "expected [rows], [ranks] (one per row) or [groups] (each sequence's first)";
    case Fill::Position: case Fill::Valid: case Fill::Slot: return "expected [rows]";
    case Fill::CuSeqlens: return "expected [n] with n >= groups + 1";
    case Fill::Tokens: return "expected [groups], [groups, w] or [ranks]";
    case Fill::Error: return "expected i32 [1]";
    case Fill::Blocks: return "expected i32 [members + 1]";
    default: return "expected [groups]";
  }
}

}  // namespace

std::optional<Protocol> protocol_check(const Manifest& m, bool sampled, Errors& errs) {
  const size_t errs_before = errs.size();
  Protocol p;
  auto axis_var = [&](VarAxis a) -> std::optional<PBound> {
    for (auto& kv : m.vars) if (kv.second.axis == a) return PBound{kv.first, kv.second.max};
    return std::nullopt;
  };
  auto rows = axis_var(VarAxis::Rows), groups = axis_var(VarAxis::Groups);
  p.ranks = axis_var(VarAxis::Ranks);
  if (!rows) errs.push_back("no var has `axis: rows`: nothing counts a call's rows");
  if (!groups) errs.push_back("no var has `axis: groups`: nothing counts a call's groups");
  if (!rows || !groups) return std::nullopt;
  p.rows = *rows;
  p.groups = *groups;

  auto classify = [&](const std::string& v) -> std::optional<PAxis> {
    if (v == p.rows.var) return PAxis{PAxis::Rows, 0};
    if (v == p.groups.var) return PAxis{PAxis::Groups, 0};
    if (p.ranks && p.ranks->var == v) return PAxis{PAxis::Ranks, 0};
    return std::nullopt;
  };
  auto axis_of = [&](const std::string& name, const std::string& what, const std::string& v) {
    auto a = classify(v);
    if (!a) errs.push_back(what + " `" + name + "` is over var `" + v + "`, which counts no axis of a call");
    return a;
  };
  auto count_fill = [&](Fill f) { int n = 0; for (auto& kv : m.buffers) n += kv.second.fill && *kv.second.fill == f; return n; };

  // ---- fills ----
  for (auto& kv : m.buffers) {
    const Buffer& b = kv.second;
    if (!b.fill) continue;
    const Fill f = *b.fill;
    const std::string what = std::string("fill `") + fill_name(f) + "`";
    std::optional<PAxis> axis;
    uint64_t width = 1;
    const auto& s = b.shape;
    if (s.size() == 1 && s[0].is_var) axis = axis_of(kv.first, what, s[0].var);
    else if (s.size() == 1) axis = PAxis{PAxis::Fixed, s[0].c};
    else if (s.size() == 2 && s[0].is_var && !s[1].is_var) { axis = axis_of(kv.first, what, s[0].var); width = s[1].c; }
    else {
      errs.push_back("`" + kv.first + "` (" + what + ") is shaped " + shape_str(s) + ", expected [<axis>], [<n>] or [<axis>, w]");
      continue;
    }
    if (!axis) continue;
    const auto k = axis->kind;
    bool ok = false;
    switch (f) {
      case Fill::Token: ok = width == 1 && k != PAxis::Fixed; break;
      case Fill::Position: case Fill::Valid: case Fill::Slot: ok = width == 1 && k == PAxis::Rows; break;
      case Fill::CuSeqlens: ok = k == PAxis::Fixed && axis->n > p.groups.max; break;
      case Fill::Tokens: ok = k == PAxis::Groups || (k == PAxis::Ranks && width == 1); break;
      case Fill::Error: ok = k == PAxis::Fixed && axis->n == 1 && b.dtype == DType::i32; break;
      case Fill::Blocks: ok = k == PAxis::Fixed && axis->n >= 2 && b.dtype == DType::i32; break;
      default: ok = width == 1 && k == PAxis::Groups; break;   // seq_len, count, sampling columns
    }
    if (!ok) {
      errs.push_back("`" + kv.first + "` (" + what + ") is shaped " + shape_str(s) + ": " + fill_shape_hint(f));
      continue;
    }
    p.fills.push_back({kv.first, f, b.dtype, *axis, width});
  }
  for (auto ak : {PAxis::Rows, PAxis::Ranks, PAxis::Groups}) {
    int n = 0;
    for (auto& f : p.fills) n += f.fill == Fill::Token && f.axis.kind == ak;
    if (n > 1) errs.push_back(std::string("fill `token` over ") + PAxis{ak, 0}.str() + " is on " + std::to_string(n) + " buffers, expected one");
  }
  static const Fill kSampling[] = {Fill::Temperature, Fill::TopK, Fill::TopP, Fill::MinP, Fill::Seed};
  for (Fill f : {Fill::Position, Fill::Valid, Fill::CuSeqlens, Fill::Blocks, Fill::Count, Fill::Error, Fill::Temperature,
                 Fill::TopK, Fill::TopP, Fill::MinP, Fill::Seed})
    if (count_fill(f) > 1) errs.push_back(std::string("fill `") + fill_name(f) + "` is on more than one buffer");
  {
    std::string missing;
    int have = 0;
    for (Fill f : kSampling) { if (count_fill(f) == 1) ++have; else missing += std::string(missing.empty() ? "`" : ", `") + fill_name(f) + "`"; }
    if (have && have < 5) errs.push_back("the sampling fills come together, all or none; missing " + missing);
  }
  if (count_fill(Fill::Blocks) == 1 && !p.ranks) errs.push_back("fill `blocks` without a var naming the rows of every rank");

  // ---- tables: inputs without a role whose domain indexes a state ----
  for (auto& kv : m.buffers) {
    const Buffer& b = kv.second;
    if (b.kind != BufferKind::Input || b.fill || !b.domain || !b.domain->index_into) continue;
    auto sit = m.states.find(*b.domain->index_into);
    if (sit == m.states.end()) continue;
    if (b.dtype != DType::i32) {
      errs.push_back("table `" + kv.first + "` is " + dtype_name(b.dtype) + ", the runtime hands out i32 page and line indices");
      continue;
    }
    const auto& s = b.shape;
    if (sit->second.is_per_seq()) {
      const bool two = s.size() == 2 && !s[0].is_var && s[1].is_var;
      const bool three = s.size() == 3 && !s[0].is_var && s[1].is_var && !s[2].is_var;
      if (!two && !three) {
        errs.push_back("line table `" + kv.first + "` is shaped " + shape_str(s) + ", expected [lines, <groups|ranks>] or [lines, <groups|ranks>, w]");
        continue;
      }
      auto axis = axis_of(kv.first, "line table", s[1].var);
      if (!axis) continue;
      if (axis->kind == PAxis::Rows) {
        errs.push_back("line table `" + kv.first + "` has a column per row (`" + s[1].var + "`); lines are per sequence");
        continue;
      }
      p.line_tables.push_back({kv.first, s[0].c, three ? s[2].c : 1, *axis, sit->first, b.domain->stride});
    } else if (s.size() == 2 && s[0].is_var && s[0].var == p.groups.var && !s[1].is_var) {
      p.page_tables.push_back({kv.first, s[1].c, sit->first, b.domain->stride});
    } else {
      errs.push_back("page table `" + kv.first + "` is shaped " + shape_str(s) + ", expected [<groups>, n]");
    }
  }

  // ---- forwards ----
  for (auto& kv : m.programs) {
    const Program& pg = kv.second;
    if (pg.once) p.once.push_back(kv.first);
    if (pg.derive) p.derive.push_back(kv.first);
    if (!pg.batch) continue;
    const Batch& bt = *pg.batch;
    const std::string ctx = "program `" + kv.first + "`";
    Forward fw;
    fw.name = kv.first;
    fw.groups = bt.groups;
    fw.graph = pg.graph;
    if (!bt.rows.is_var) {
      fw.rows = bt.rows.c;
      unsigned __int128 total = (unsigned __int128)bt.groups * bt.rows.c;
      if (total > p.rows.max)
        errs.push_back(ctx + ": " + std::to_string(bt.groups) + " sequences of " + std::to_string(bt.rows.c) + " rows exceed the " +
                       std::to_string(p.rows.max) + " rows `" + p.rows.var + "` allows");
    } else {
      fw.rows_var = true;
      if (bt.rows.var != p.rows.var)
        errs.push_back(ctx + ": batch.rows is var `" + bt.rows.var + "`, but the rows of a call go in `" + p.rows.var + "`");
      if (bt.groups != 1 && count_fill(Fill::CuSeqlens) != 1)
        errs.push_back(ctx + ": rows set per call over " + std::to_string(bt.groups) + " groups needs a `cu_seqlens` fill to split them");
    }
    if (bt.groups > p.groups.max)
      errs.push_back(ctx + ": " + std::to_string(bt.groups) + " groups exceed the " + std::to_string(p.groups.max) + " `" + p.groups.var + "` allows");
    std::set<std::string> written;
    for (auto& c : pg.calls) {
      auto oit = m.ops.find(c.op);
      for (size_t j = 0; j < c.args.size(); ++j)
        if (c.args[j].kind == Arg::Buf && (oit == m.ops.end() || j >= oit->second.params.size() || oit->second.params[j].writes()))
          written.insert(c.args[j].name);
    }
    auto writes = [&](Fill f) {
      std::vector<size_t> out;
      for (size_t i = 0; i < p.fills.size(); ++i) if (p.fills[i].fill == f && written.count(p.fills[i].name)) out.push_back(i);
      return out;
    };
    auto toks = writes(Fill::Tokens);
    if (toks.size() == 1) fw.emits = toks[0];
    else if (toks.size() > 1) errs.push_back(ctx + ": writes " + std::to_string(toks.size()) + " `tokens` outputs; a call hands back one");
    if (fw.emits) {
      const Filled& f = p.fills[*fw.emits];
      const bool ok = fw.rows_var ? f.width == 1 : (f.width == 1 || f.width == fw.rows);
      if (!ok)
        errs.push_back(ctx + ": hands back `" + f.name + "` of " + std::to_string(f.width) + " per sequence, but a call has " +
                       (fw.rows_var ? std::string("a variable number of") : std::to_string(fw.rows)) + " rows per sequence");
    }
    auto cnt = writes(Fill::Count);
    if (cnt.size() == 1) {
      fw.count = cnt[0];
      if (!(fw.emits && p.fills[*fw.emits].width > 1))
        errs.push_back(ctx + ": writes `" + p.fills[cnt[0]].name + "` (fill `count`) but no `tokens` output of several per sequence to count");
    }
    if (bt.context) {
      const std::string& v = *bt.context;
      if (v == p.rows.var || v == p.groups.var)
        errs.push_back(ctx + ": batch.context is `" + v + "`, which sizes the call itself; the context needs its own var");
      auto vit = m.vars.find(v);
      if (vit != m.vars.end()) {
        if (p.context && p.context->var != v)
          errs.push_back(ctx + ": batch.context is `" + v + "`, but `" + p.context->var + "` is the context in another program; one var bounds every context");
        else if (!p.context) p.context = PBound{v, vit->second.max};
      }
    }
    for (auto& o : p.forwards)
      if (o.rows_var == fw.rows_var && (fw.rows_var || o.rows == fw.rows)) {
        errs.push_back(ctx + " and `" + o.name + "` take the same rows per sequence; a row shape names one program, and what differs with the batch is a launch's `when`");
        break;
      }
    p.forwards.push_back(fw);
  }
  if (p.forwards.empty()) errs.push_back("no program declares a `batch`: nothing for a serving loop to drive");
  else if (sampled && std::none_of(p.forwards.begin(), p.forwards.end(), [](const Forward& f) { return f.emits.has_value(); }))
    errs.push_back("no program with a `batch` writes a `tokens` output: no call hands a token back");

  for (auto& kv : m.states) {
    if (!kv.second.shard) continue;
    auto g = m.topology.find(kv.second.shard->group);
    const uint64_t members = g == m.topology.end() ? 0 : g->second;
    if (kv.second.shard->by == Shard::Position) { if (!p.positions) p.positions = std::make_pair(kv.second.shard->group, members); }
    else p.heads[kv.first] = {kv.second.shard->group, members, kv.second.shard->segments};
  }
  if (errs.size() != errs_before) return std::nullopt;
  return p;
}

Json Protocol::to_json() const {
  auto bound = [](const PBound& b) { Json j = Json::object(); j.set("var", Json::str(b.var)); j.set("max", Json::uint(b.max)); return j; };
  auto axis = [](const PAxis& a) {
    if (a.kind != PAxis::Fixed) return Json::str(a.str());
    Json j = Json::object(); j.set("fixed", Json::uint(a.n)); return j;
  };
  Json j = Json::object();
  j.set("rows", bound(rows));
  j.set("groups", bound(groups));
  j.set("ranks", ranks ? bound(*ranks) : Json::null());
  j.set("context", context ? bound(*context) : Json::null());
  Json fs = Json::array();
  for (auto& f : fills) {
    Json o = Json::object();
    o.set("name", Json::str(f.name)); o.set("fill", Json::str(fill_name(f.fill))); o.set("dtype", Json::str(dtype_name(f.dtype)));
    o.set("axis", axis(f.axis)); o.set("width", Json::uint(f.width));
    fs.push(o);
  }
  j.set("fills", fs);
  Json pts = Json::array();
  for (auto& t : page_tables) {
    Json o = Json::object();
    o.set("name", Json::str(t.name)); o.set("width", Json::uint(t.width)); o.set("state", Json::str(t.state)); o.set("stride", Json::uint(t.stride));
    pts.push(o);
  }
  j.set("page_tables", pts);
  Json lts = Json::array();
  for (auto& t : line_tables) {
    Json o = Json::object();
    o.set("name", Json::str(t.name)); o.set("lines", Json::uint(t.lines)); o.set("width", Json::uint(t.width));
    o.set("axis", axis(t.axis)); o.set("state", Json::str(t.state)); o.set("stride", Json::uint(t.stride));
    lts.push(o);
  }
  j.set("line_tables", lts);
  Json fws = Json::array();
  for (auto& f : forwards) {
    Json o = Json::object();
    o.set("name", Json::str(f.name)); o.set("groups", Json::uint(f.groups));
    o.set("rows", f.rows_var ? Json::str("var") : Json::uint(f.rows));
    o.set("emits", f.emits ? Json::str(fills[*f.emits].name) : Json::null());
    o.set("count", f.count ? Json::str(fills[*f.count].name) : Json::null());
    o.set("graph", Json::boolean(f.graph));
    fws.push(o);
  }
  j.set("forwards", fws);
  Json on = Json::array(), dv = Json::array();
  for (auto& s : once) on.push(Json::str(s));
  for (auto& s : derive) dv.push(Json::str(s));
  j.set("once", on);
  j.set("derive", dv);
  Json sh = Json::object();
  if (positions) { Json o = Json::object(); o.set("group", Json::str(positions->first)); o.set("members", Json::uint(positions->second)); sh.set("positions", o); }
  else sh.set("positions", Json::null());
  Json hs = Json::object();
  for (auto& kv : heads) {
    Json o = Json::object(), segs = Json::array();
    o.set("group", Json::str(kv.second.group)); o.set("members", Json::uint(kv.second.members));
    for (auto& s : kv.second.segments) { Json a = Json::array(); a.push(Json::uint(s.first)); a.push(Json::uint(s.second)); segs.push(a); }
    o.set("segments", segs);
    hs.set(kv.first, o);
  }
  sh.set("heads", hs);
  j.set("shards", sh);
  return j;
}

Manifest self_hosted(const Manifest& m, uint64_t) {
  Manifest out = m;
  for (auto& kv : out.states) {
    if (!kv.second.host) continue;
    const HostTensor h = *kv.second.host;
    const uint64_t block = (h.strides.empty() ? 0 : h.strides[0]) * dtype_bytes(h.dtype);
    std::set<uint64_t> strides;
    for (auto& b : m.buffers) {
      const Buffer& bf = b.second;
      if (bf.kind != BufferKind::Input || !bf.domain || !bf.domain->index_into) continue;
      auto sit = m.states.find(*bf.domain->index_into);
      if (sit == m.states.end() || !sit->second.host) continue;
      const HostTensor& o = *sit->second.host;
      if (o.dtype == h.dtype && o.shape == h.shape && o.strides == h.strides) strides.insert(bf.domain->stride);
    }
    State s;
    s.shard = kv.second.shard;
    if (strides.empty()) { s.bytes = block ? block : 1; }                       // nothing indexes it: one fixed block
    else if (strides.count(block) && strides.size() == 1) s.bytes_per_seq = block;   // indexed per line
    else {
      const uint64_t k = *strides.rbegin();
      s.bytes_per_token = k ? std::max<uint64_t>(1, block / k) : block;
    }
    kv.second = s;
  }
  return out;
}

}  // namespace kern
