// JSON -> Manifest. Every object goes through a reader that (1) resolves named constants wherever a
// number is expected, (2) records the keys it consumed so unknown fields are reported with a path.
#include <algorithm>
#include <array>

#include "types.hpp"

namespace kern {
namespace {

struct Ctx {
  Errors& errs;
  const std::map<std::string, Json>* constants;
  void err(const std::string& path, const std::string& msg) { errs.push_back(path + ": " + msg); }
  // a number, or the name of a constant holding one
  const Json* num(const Json& j) const {
    if (j.is_number()) return &j;
    if (j.is_str() && constants) {
      auto it = constants->find(j.s);
      if (it != constants->end()) return &it->second;
    }
    return nullptr;
  }
};

struct Rd {
  const Json& j;
  std::string path;
  Ctx& cx;
  std::vector<const char*> seen;      // keys asked for (string literals): a handful per object
  bool ok;
  Rd(const Json& j_, std::string p, Ctx& c) : j(j_), path(std::move(p)), cx(c), ok(j_.is_obj()) {
    if (!ok) cx.err(path, "expected an object");
  }
  const Json* opt(const char* k) {
    if (!ok) return nullptr;
    seen.push_back(k);
    const Json* v = j.find(k);
    return (v && v->is_null()) ? nullptr : v;
  }
  const Json* req(const char* k) {
    const Json* v = opt(k);
    if (!v && ok) cx.err(path, std::string("missing field `") + k + "`");
    return v;
  }
  std::string at(const char* k) const { return path + "/" + k; }
  void done() {
    if (!ok) return;
    for (auto& kv : j.obj)
      if (std::none_of(seen.begin(), seen.end(), [&](const char* k) { return kv.first == k; }))
        cx.err(path, "unknown field `" + kv.first + "`");
  }
  bool u64(const Json& v, const std::string& p, uint64_t& out) {
    const Json* n = cx.num(v);
    if (n && n->is_uint()) { out = n->u; return true; }
    if (v.is_str() && !n) cx.err(p, "undefined constant `" + v.s + "`");
    else cx.err(p, "expected an unsigned integer");
    return false;
  }
  bool i64(const Json& v, const std::string& p, int64_t& out) {
    const Json* n = cx.num(v);
    if (n && n->fits_i64()) { out = n->as_i64(); return true; }
    cx.err(p, "expected a 64-bit integer");
    return false;
  }
  bool f64(const Json& v, const std::string& p, double& out) {
    const Json* n = cx.num(v);
    if (n) { out = n->d; return true; }
    cx.err(p, "expected a number");
    return false;
  }
  uint64_t get_u64(const char* k, uint64_t dflt, bool required = false) {
    const Json* v = required ? req(k) : opt(k);
    uint64_t out = dflt;
    if (v) u64(*v, at(k), out);
    return out;
  }
  bool get_bool(const char* k) {
    const Json* v = opt(k);
    if (!v) return false;
    if (!v->is_bool()) { cx.err(at(k), "expected true or false"); return false; }
    return v->b;
  }
  std::string get_str(const char* k, bool required = true) {
    const Json* v = required ? req(k) : opt(k);
    if (!v) return "";
    if (!v->is_str()) { cx.err(at(k), "expected a string"); return ""; }
    return v->s;
  }
};

bool parse_u32_triple(const Json& v, const std::string& p, Ctx& cx, uint32_t out[3]) {
  if (!v.is_arr() || v.arr.size() != 3) { cx.err(p, "expected an array of 3 integers"); return false; }
  for (int i = 0; i < 3; ++i) {
    const Json* n = cx.num(v.arr[i]);
    if (!n || !n->is_uint() || n->u > UINT32_MAX) { cx.err(p, "expected an array of 3 unsigned 32-bit integers"); return false; }
    out[i] = (uint32_t)n->u;
  }
  return true;
}

Expr parse_expr(const Json& v, const std::string& p, Ctx& cx) {
  Expr e;
  if (const Json* n = cx.num(v)) {
    if (!n->is_uint()) cx.err(p, "an expression constant is an unsigned integer");
    e.kind = Expr::Const;
    e.c = n->u;
    return e;
  }
  if (v.is_str()) { e.kind = Expr::Var; e.var = v.s; return e; }
  if (!v.is_obj() || v.obj.size() != 1 || !v.obj[0].second.is_arr()) {
    cx.err(p, "expected an integer, a var name, or one of {ceil_div|mul|add|clamp: [...]}");
    return e;
  }
  const std::string& k = v.obj[0].first;
  const auto& a = v.obj[0].second.arr;
  auto cst = [&](size_t i, uint64_t& out) {
    const Json* n = i < a.size() ? cx.num(a[i]) : nullptr;
    if (!n || !n->is_uint()) { cx.err(p + "/" + k, "operand " + std::to_string(i) + " must be an unsigned integer"); return; }
    out = n->u;
  };
  if ((k == "ceil_div" || k == "mul") && a.size() == 2) {
    e.kind = k == "mul" ? Expr::Mul : Expr::CeilDiv;
    e.sub.push_back(parse_expr(a[0], p + "/" + k + "/0", cx));
    cst(1, e.c);
  } else if (k == "add" && a.size() == 2) {
    e.kind = Expr::Add;
    e.sub.push_back(parse_expr(a[0], p + "/add/0", cx));
    e.sub.push_back(parse_expr(a[1], p + "/add/1", cx));
  } else if (k == "clamp" && a.size() == 3) {
    e.kind = Expr::Clamp;
    e.sub.push_back(parse_expr(a[0], p + "/clamp/0", cx));
    cst(1, e.c);
    cst(2, e.c2);
  } else {
    cx.err(p, "unknown expression `" + k + "` or wrong operand count");
  }
  return e;
}

Dim parse_dim(const Json& v, const std::string& p, Ctx& cx) {
  Dim d;
  if (const Json* n = cx.num(v)) {
    if (!n->is_uint()) cx.err(p, "a dimension is an unsigned integer or a var name");
    d.c = n->u;
  } else if (v.is_str()) {
    d.is_var = true;
    d.var = v.s;
  } else {
    cx.err(p, "a dimension is an unsigned integer or a var name");
  }
  return d;
}
std::vector<Dim> parse_shape(const Json* v, const std::string& p, Ctx& cx) {
  std::vector<Dim> out;
  if (!v) return out;
  if (!v->is_arr()) { cx.err(p, "expected an array"); return out; }
  for (size_t i = 0; i < v->arr.size(); ++i) out.push_back(parse_dim(v->arr[i], p + "/" + std::to_string(i), cx));
  return out;
}
bool parse_dtype(const Json* v, const std::string& p, Ctx& cx, DType& out) {
  if (!v) return false;
  if (!v->is_str() || !dtype_parse(v->s, out)) { cx.err(p, "unknown dtype"); return false; }
  return true;
}
std::vector<uint64_t> parse_u64s(const Json* v, const std::string& p, Ctx& cx, Rd& r) {
  std::vector<uint64_t> out;
  if (!v) return out;
  if (!v->is_arr()) { cx.err(p, "expected an array of integers"); return out; }
  for (size_t i = 0; i < v->arr.size(); ++i) {
    uint64_t x = 0;
    r.u64(v->arr[i], p + "/" + std::to_string(i), x);
    out.push_back(x);
  }
  return out;
}

std::vector<ParamType> parse_params(const Json& v, const std::string& p, Ctx& cx) {
  std::vector<ParamType> out;
  if (!v.is_arr()) { cx.err(p, "expected an array of parameter types"); return out; }
  for (size_t i = 0; i < v.arr.size(); ++i) {
    ParamType t;
    if (!v.arr[i].is_str() || !ParamType::parse(v.arr[i].s, t))
      cx.err(p + "/" + std::to_string(i), "invalid parameter type" + (v.arr[i].is_str() ? " `" + v.arr[i].s + "`" : std::string()));
    out.push_back(t);
  }
  return out;
}

TensorSource parse_tensor_source(const Json& v, const std::string& p, Ctx& cx) {
  TensorSource t;
  if (v.is_str()) { t.name = v.s; return t; }
  Rd r(v, p, cx);
  t.ranked = true;
  t.group = r.get_str("group");
  if (const Json* a = r.req("tensors")) {
    if (!a->is_arr()) cx.err(r.at("tensors"), "expected an array of names");
    else for (auto& x : a->arr) { if (x.is_str()) t.tensors.push_back(x.s); else cx.err(r.at("tensors"), "expected a string"); }
  }
  r.done();
  return t;
}
Ranges parse_ranges(const Json& v, const std::string& p, Ctx& cx) {
  Ranges g;
  auto pair = [&](const Json& a, const std::string& pp, uint64_t& lo, uint64_t& hi) {
    const Json* x = a.is_arr() && a.arr.size() == 2 ? cx.num(a.arr[0]) : nullptr;
    const Json* y = x ? cx.num(a.arr[1]) : nullptr;
    if (!x || !y || !x->is_uint() || !y->is_uint()) { cx.err(pp, "expected [begin, end]"); return; }
    lo = x->u; hi = y->u;
  };
  if (v.is_arr()) { pair(v, p, g.range[0], g.range[1]); return g; }
  Rd r(v, p, cx);
  g.ranked = true;
  g.group = r.get_str("group");
  if (const Json* a = r.req("ranges")) {
    if (!a->is_arr()) cx.err(r.at("ranges"), "expected an array of [begin, end]");
    else for (size_t i = 0; i < a->arr.size(); ++i) {
      uint64_t lo = 0, hi = 0;
      pair(a->arr[i], r.at("ranges") + "/" + std::to_string(i), lo, hi);
      g.ranges.emplace_back(lo, hi);
    }
  }
  r.done();
  return g;
}

Bound parse_bound(const Json& v, const std::string& p, Ctx& cx) {
  Bound b;
  const Json* n = cx.num(v);
  if (n && n->fits_i64()) { b.kind = Bound::Int; b.i = n->as_i64(); }
  else if (n) { b.kind = Bound::Float; b.f = n->d; }
  else { b.kind = Bound::Ex; b.expr = parse_expr(v, p, cx); }
  return b;
}

TensorMapDecl parse_tensormap(const Json& v, const std::string& p, Ctx& cx) {
  TensorMapDecl t;
  Rd r(v, p, cx);
  t.param = (size_t)r.get_u64("param", 0, true);
  t.dtype = r.get_str("dtype");
  t.dims = parse_u64s(r.req("dims"), r.at("dims"), cx, r);
  t.strides = parse_u64s(r.opt("strides"), r.at("strides"), cx, r);
  for (uint64_t b : parse_u64s(r.req("box"), r.at("box"), cx, r)) t.box.push_back((uint32_t)std::min<uint64_t>(b, UINT32_MAX));
  t.swizzle = (uint32_t)r.get_u64("swizzle", 0);
  t.l2_promotion = (uint32_t)r.get_u64("l2_promotion", 0);
  t.oob_nan = r.get_bool("oob_nan");
  t.wrap = r.get_bool("wrap");
  r.done();
  return t;
}

// literal sources shared by launch args, pack fields and call args
template <typename T>
bool parse_literal(Rd& r, T& out, int& found) {
  if (const Json* v = r.opt("i32")) {
    int64_t x = 0;
    if (r.i64(*v, r.at("i32"), x) && (x < INT32_MIN || x > INT32_MAX)) r.cx.err(r.at("i32"), "out of range for i32");
    out.i = x; ++found; out.kind = T::I32;
  }
  if (const Json* v = r.opt("i64")) { r.i64(*v, r.at("i64"), out.i); ++found; out.kind = T::I64; }
  if (const Json* v = r.opt("f32")) { r.f64(*v, r.at("f32"), out.f); ++found; out.kind = T::F32; }
  if (const Json* v = r.opt("u8")) {
    int64_t x = 0;
    if (r.i64(*v, r.at("u8"), x) && (x < 0 || x > 255)) r.cx.err(r.at("u8"), "out of range for u8");
    out.i = x; ++found; out.kind = T::U8;
  }
  return found > 0;
}

Pack parse_pack(const Json& v, const std::string& p, Ctx& cx) {
  Pack pk;
  Rd r(v, p, cx);
  pk.size = (uint32_t)r.get_u64("size", 0, true);
  if (const Json* fs = r.req("fields")) {
    if (!fs->is_arr()) cx.err(r.at("fields"), "expected an array");
    else for (size_t i = 0; i < fs->arr.size(); ++i) {
      Field f;
      Rd fr(fs->arr[i], r.at("fields") + "/" + std::to_string(i), cx);
      f.at = (uint32_t)fr.get_u64("at", 0, true);
      if (fr.opt("width")) f.width = (uint32_t)fr.get_u64("width", 0);
      int found = 0;
      parse_literal(fr, f.src, found);
      if (const Json* x = fr.opt("param")) { uint64_t u = 0; fr.u64(*x, fr.at("param"), u); f.src.param = (size_t)u; f.src.kind = FieldSrc::Param; ++found; }
      if (const Json* x = fr.opt("scratch")) { f.src.name = x->is_str() ? x->s : ""; f.src.kind = FieldSrc::Scratch; ++found; }
      if (const Json* x = fr.opt("var")) { f.src.name = x->is_str() ? x->s : ""; f.src.kind = FieldSrc::Var; ++found; }
      if (const Json* x = fr.opt("expr")) { f.src.expr = parse_expr(*x, fr.at("expr"), cx); f.src.kind = FieldSrc::ExprK; ++found; }
      if (const Json* x = fr.opt("rank")) { f.src.name = x->is_str() ? x->s : ""; f.src.kind = FieldSrc::Rank; ++found; }
      if (const Json* x = fr.opt("tensormap")) { f.src.tmap = parse_tensormap(*x, fr.at("tensormap"), cx); f.src.kind = FieldSrc::TensorMap; ++found; }
      if (found != 1) cx.err(fr.path, "a pack field has exactly one source");
      fr.done();
      pk.fields.push_back(std::move(f));
    }
  }
  r.done();
  return pk;
}

std::vector<LaunchArg> parse_launch_args(const Json& v, const std::string& p, Ctx& cx) {
  std::vector<LaunchArg> out;
  if (!v.is_arr()) { cx.err(p, "expected an array of launch args"); return out; }
  for (size_t i = 0; i < v.arr.size(); ++i) {
    LaunchArg a;
    Rd r(v.arr[i], p + "/" + std::to_string(i), cx);
    int found = 0;
    parse_literal(r, a, found);
    if (const Json* x = r.opt("param")) { uint64_t u = 0; r.u64(*x, r.at("param"), u); a.param = (size_t)u; a.kind = LaunchArg::Param; ++found; }
    if (const Json* x = r.opt("scratch")) { a.name = x->is_str() ? x->s : ""; a.kind = LaunchArg::Scratch; ++found; }
    if (const Json* x = r.opt("rank")) { a.name = x->is_str() ? x->s : ""; a.kind = LaunchArg::Rank; ++found; }
    if (const Json* x = r.opt("pack")) { a.pack = parse_pack(*x, r.at("pack"), cx); a.kind = LaunchArg::PackK; ++found; }
    if (found != 1) cx.err(r.path, "a launch arg has exactly one of param|scratch|i32|i64|f32|u8|rank|pack");
    r.done();
    out.push_back(std::move(a));
  }
  return out;
}

Launch parse_launch(const Json& v, const std::string& p, Ctx& cx) {
  Launch l;
  Rd r(v, p, cx);
  l.entry = r.get_str("entry");
  l.is_extern = r.ok && !v.find("module");
  if (const Json* x = r.opt("params")) l.params = parse_params(*x, r.at("params"), cx);
  if (const Json* x = r.opt("when")) {
    When w;
    Rd wr(*x, r.at("when"), cx);
    w.var = wr.get_str("var");
    if (wr.opt("min")) w.min = wr.get_u64("min", 0);
    if (wr.opt("max")) w.max = wr.get_u64("max", 0);
    wr.done();
    l.when = w;
  }
  if (const Json* x = r.opt("args")) l.args = parse_launch_args(*x, r.at("args"), cx);
  if (l.is_extern) {
    if (const Json* x = r.opt("algo")) {
      GemmAlgo g;
      Rd ar(*x, r.at("algo"), cx);
      if (const Json* y = ar.req("id")) ar.i64(*y, ar.at("id"), g.id);
      g.tile = ar.get_u64("tile", 0, true);
      g.stages = ar.get_u64("stages", 0, true);
      if (const Json* y = ar.req("split_k")) ar.i64(*y, ar.at("split_k"), g.split_k);
      g.reduction = ar.get_u64("reduction", 0, true);
      g.swizzle = ar.get_u64("swizzle", 0, true);
      g.custom = ar.get_u64("custom", 0, true);
      g.inner_shape = ar.get_u64("inner_shape", 0, true);
      g.cluster_shape = ar.get_u64("cluster_shape", 0, true);
      ar.done();
      l.algo = g;
    }
  } else {
    l.module = r.get_str("module");
    if (const Json* x = r.req("block")) parse_u32_triple(*x, r.at("block"), cx, l.block);
    if (const Json* x = r.req("grid")) {
      if (!x->is_arr() || x->arr.size() != 3) cx.err(r.at("grid"), "expected an array of 3 expressions");
      else for (int i = 0; i < 3; ++i) l.grid[i] = parse_expr(x->arr[i], r.at("grid") + "/" + std::to_string(i), cx);
    }
    if (const Json* x = r.opt("shared_mem")) l.shared_mem = parse_expr(*x, r.at("shared_mem"), cx);
    if (const Json* x = r.opt("cluster")) {
      uint32_t c[3] = {1, 1, 1};
      if (parse_u32_triple(*x, r.at("cluster"), cx, c)) l.cluster = std::array<uint32_t, 3>{c[0], c[1], c[2]};
    }
    l.pdl = r.get_bool("pdl");
  }
  r.done();
  return l;
}

Arg parse_arg(const Json& v, const std::string& p, Ctx& cx) {
  Arg a;
  Rd r(v, p, cx);
  int found = 0;
  parse_literal(r, a, found);
  if (const Json* x = r.opt("buf")) { a.name = x->is_str() ? x->s : ""; a.kind = Arg::Buf; ++found; a.offset = r.get_u64("offset", 0); }
  if (const Json* x = r.opt("state")) { a.name = x->is_str() ? x->s : ""; a.kind = Arg::StateK; ++found; a.offset = r.get_u64("offset", 0); }
  if (const Json* x = r.opt("var")) { a.name = x->is_str() ? x->s : ""; a.kind = Arg::Var; ++found; }
  if (const Json* x = r.opt("expr")) { a.expr = parse_expr(*x, r.at("expr"), cx); a.kind = Arg::ExprK; ++found; }
  if (const Json* x = r.opt("rank")) { a.name = x->is_str() ? x->s : ""; a.kind = Arg::Rank; ++found; }
  if (found != 1) cx.err(p, "an arg has exactly one of buf|state|var|expr|i32|i64|f32|u8|rank");
  r.done();
  return a;
}

template <typename F>
void each_named(const Json* v, const std::string& p, Ctx& cx, F f) {
  if (!v) return;
  if (!v->is_obj()) { cx.err(p, "expected an object of named entries"); return; }
  for (auto& kv : v->obj) {
    if (kv.first.empty()) cx.err(p, "empty name");
    f(kv.first, kv.second, p + "/" + kv.first);
  }
}

}  // namespace

Manifest parse_manifest(const Json& doc, Errors& errs) {
  Manifest m;
  Ctx cx{errs, nullptr};
  Rd r(doc, "", cx);
  if (!r.ok) return m;
  // constants first: numeric literals by name, not clashing with a var
  if (const Json* c = r.opt("constants")) {
    if (!c->is_obj()) cx.err("/constants", "constants must be an object");
    else for (auto& kv : c->obj) {
      if (kv.first.empty() || !kv.second.is_number()) cx.err("/constants", "constants require nonempty names and numeric literal values");
      else if (doc.find("vars") && doc.find("vars")->find(kv.first)) cx.err("/constants", "constant `" + kv.first + "` conflicts with a var");
      else m.constants[kv.first] = kv.second;
    }
  }
  if (const Json* v = r.req("schema_version")) {
    if (v->is_uint()) m.schema_version = v->u; else cx.err("/schema_version", "expected an integer");
  }
  cx.constants = &m.constants;
  m.model = r.get_str("model");
  if (const Json* c = r.opt("chat")) {
    Rd cr(*c, "/chat", cx);
    m.has_chat = true;
    if (cr.opt("tool_parser")) m.tool_parser = cr.get_str("tool_parser");
    cr.done();
  }
  each_named(r.req("vars"), "/vars", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    Var x;
    Rd vr(v, p, cx);
    x.max = vr.get_u64("max", 0, true);
    if (vr.opt("axis")) {
      std::string a = vr.get_str("axis");
      if (a == "rows") x.axis = VarAxis::Rows; else if (a == "groups") x.axis = VarAxis::Groups;
      else if (a == "ranks") x.axis = VarAxis::Ranks; else cx.err(vr.at("axis"), "axis is one of rows, groups, ranks");
    }
    vr.done();
    m.vars[n] = x;
  });
  if (const Json* t = r.opt("topology")) {
    m.has_topology = true;
    Rd tr(*t, "/topology", cx);
    each_named(tr.req("groups"), "/topology/groups", cx, [&](const std::string& n, const Json& v, const std::string& p) {
      uint64_t s = 0;
      tr.u64(v, p, s);
      m.topology[n] = s;
    });
    tr.done();
  }
  if (const Json* c = r.opt("cut")) {
    Cut x;
    Rd cr(*c, "/cut", cx);
    x.id = cr.get_str("id");
    x.stage = cr.get_u64("stage", 0, true);
    x.stages = cr.get_u64("stages", 0, true);
    cr.done();
    m.cut = x;
  }
  each_named(r.req("states"), "/states", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    State s;
    Rd sr(v, p, cx);
    s.bytes_per_token = sr.get_u64("bytes_per_token", 0);
    s.bytes = sr.get_u64("bytes", 0);
    s.bytes_per_seq = sr.get_u64("bytes_per_seq", 0);
    if (const Json* h = sr.opt("host")) {
      HostTensor t;
      Rd hr(*h, sr.at("host"), cx);
      parse_dtype(hr.req("dtype"), hr.at("dtype"), cx, t.dtype);
      t.shape = parse_u64s(hr.req("shape"), hr.at("shape"), cx, hr);
      t.strides = parse_u64s(hr.req("strides"), hr.at("strides"), cx, hr);
      hr.done();
      s.host = t;
    }
    if (const Json* h = sr.opt("shard")) {
      Shard sh;
      Rd hr(*h, sr.at("shard"), cx);
      std::string by = hr.get_str("by");
      sh.group = hr.get_str("group");
      if (by == "position") sh.by = Shard::Position;
      else if (by == "heads") {
        sh.by = Shard::Heads;
        if (const Json* sg = hr.req("segments")) {
          if (!sg->is_arr()) cx.err(hr.at("segments"), "expected an array of [rows, width]");
          else for (auto& e : sg->arr) {
            const Json* a = e.is_arr() && e.arr.size() == 2 ? cx.num(e.arr[0]) : nullptr;
            const Json* b = a ? cx.num(e.arr[1]) : nullptr;
            if (!a || !b || !a->is_uint() || !b->is_uint()) cx.err(hr.at("segments"), "expected [rows, width]");
            else sh.segments.emplace_back(a->u, b->u);
          }
        }
      } else cx.err(hr.at("by"), "shard is by `position` or by `heads`");
      hr.done();
      s.shard = sh;
    }
    sr.done();
    m.states[n] = std::move(s);
  });
  each_named(r.req("buffers"), "/buffers", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    Buffer b;
    Rd br(v, p, cx);
    parse_dtype(br.req("dtype"), br.at("dtype"), cx, b.dtype);
    b.shape = parse_shape(br.req("shape"), br.at("shape"), cx);
    std::string k = br.get_str("kind");
    static const char* kinds[] = {"input", "output", "inout", "weight", "source", "workspace", "carry", "peer"};
    bool found = false;
    for (int i = 0; i < 8; ++i) if (k == kinds[i]) { b.kind = (BufferKind)i; found = true; }
    if (!found && br.ok) cx.err(br.at("kind"), "unknown buffer kind `" + k + "`");
    if (br.opt("placement")) {
      std::string pl = br.get_str("placement");
      if (pl == "host") b.host_placement = true; else if (pl != "device") cx.err(br.at("placement"), "placement is `device` or `host`");
    }
    if (br.opt("fill")) {
      Fill f;
      std::string fs = br.get_str("fill");
      if (fill_parse(fs, f)) b.fill = f; else cx.err(br.at("fill"), "unknown fill `" + fs + "`");
    }
    if (const Json* d = br.opt("domain")) {
      Domain dm;
      Rd dr(*d, br.at("domain"), cx);
      if (const Json* x = dr.opt("min")) dm.min = parse_bound(*x, dr.at("min"), cx);
      if (const Json* x = dr.opt("max")) dm.max = parse_bound(*x, dr.at("max"), cx);
      if (dr.opt("index_into")) dm.index_into = dr.get_str("index_into");
      dm.stride = dr.get_u64("stride", 1);
      dm.monotone = dr.get_bool("monotone");
      dr.done();
      b.domain = std::move(dm);
    }
    b.export_ = br.get_bool("export");
    if (br.opt("of")) b.of = br.get_str("of");
    if (br.opt("group")) b.group = br.get_str("group");
    if (const Json* bd = br.opt("bind")) {
      if (!bd->is_arr()) cx.err(br.at("bind"), "expected an array of segments");
      else for (size_t i = 0; i < bd->arr.size(); ++i) {
        Segment s;
        Rd sr(bd->arr[i], br.at("bind") + "/" + std::to_string(i), cx);
        if (const Json* t = sr.req("tensor")) s.tensor = parse_tensor_source(*t, sr.at("tensor"), cx);
        if (const Json* x = sr.opt("rows")) s.rows = parse_ranges(*x, sr.at("rows"), cx);
        if (const Json* x = sr.opt("cols")) s.cols = parse_ranges(*x, sr.at("cols"), cx);
        if (const Json* x = sr.opt("interleave")) {
          Interleave il;
          Rd ir(*x, sr.at("interleave"), cx);
          if (const Json* w = ir.req("with")) il.with = parse_tensor_source(*w, ir.at("with"), cx);
          il.rows = ir.get_u64("rows", 0, true);
          ir.done();
          s.interleave = il;
        }
        sr.done();
        b.bind.push_back(std::move(s));
      }
    }
    br.done();
    m.buffers[n] = std::move(b);
  });
  each_named(r.req("modules"), "/modules", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    Module x;
    Rd mr(v, p, cx);
    x.source = mr.get_str("source");
    x.sha256 = mr.get_str("sha256");
    if (const Json* mc = mr.opt("multicast")) {
      if (!mc->is_bool() || mc->b) cx.err(mr.at("multicast"), "the only declarable value is false");
      else x.multicast_free = true;
    }
    mr.done();
    m.modules[n] = x;
  });
  each_named(r.req("ops"), "/ops", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    Op o;
    Rd orr(v, p, cx);
    if (const Json* x = orr.req("params")) o.params = parse_params(*x, orr.at("params"), cx);
    if (const Json* im = orr.req("impl")) {
      Rd ir(*im, orr.at("impl"), cx);
      each_named(ir.opt("scratch"), ir.at("scratch"), cx, [&](const std::string& sn, const Json& sv, const std::string& sp) {
        Scratch s;
        Rd sr(sv, sp, cx);
        parse_dtype(sr.req("dtype"), sr.at("dtype"), cx, s.dtype);
        s.shape = parse_shape(sr.req("shape"), sr.at("shape"), cx);
        sr.done();
        o.scratch[sn] = std::move(s);
      });
      if (const Json* ls = ir.req("launches")) {
        if (!ls->is_arr()) cx.err(ir.at("launches"), "expected an array");
        else for (size_t i = 0; i < ls->arr.size(); ++i)
          o.launches.push_back(parse_launch(ls->arr[i], ir.at("launches") + "/" + std::to_string(i), cx));
      }
      ir.done();
    }
    orr.done();
    m.ops[n] = std::move(o);
  });
  each_named(r.req("programs"), "/programs", cx, [&](const std::string& n, const Json& v, const std::string& p) {
    Program pg;
    Rd pr(v, p, cx);
    if (const Json* b = pr.opt("batch")) {
      Batch bt;
      Rd br(*b, pr.at("batch"), cx);
      bt.groups = br.get_u64("groups", 0, true);
      if (const Json* x = br.req("rows")) bt.rows = parse_dim(*x, br.at("rows"), cx);
      if (br.opt("context")) bt.context = br.get_str("context");
      br.done();
      pg.batch = bt;
    }
    pg.once = pr.get_bool("once");
    pg.derive = pr.get_bool("derive");
    pg.graph = pr.get_bool("graph");
    if (const Json* cs = pr.req("calls")) {
      if (!cs->is_arr()) cx.err(pr.at("calls"), "expected an array");
      else for (size_t i = 0; i < cs->arr.size(); ++i) {
        Call c;
        std::string cp = pr.at("calls") + "/" + std::to_string(i);
        Rd cr(cs->arr[i], cp, cx);
        if (cr.opt("label")) c.label = cr.get_str("label");
        c.op = cr.get_str("op");
        if (const Json* as = cr.req("args")) {
          if (!as->is_arr()) cx.err(cr.at("args"), "expected an array");
          else for (size_t k = 0; k < as->arr.size(); ++k) c.args.push_back(parse_arg(as->arr[k], cr.at("args") + "/" + std::to_string(k), cx));
        }
        uint64_t lane = cr.get_u64("lane", 0);
        if (lane > 255) cx.err(cr.at("lane"), "a lane is 0..255");
        c.lane = (uint8_t)lane;
        for (uint64_t a : parse_u64s(cr.opt("after"), cr.at("after"), cx, cr)) {
          if (a > 255) cx.err(cr.at("after"), "a lane is 0..255");
          c.after.push_back((uint8_t)a);
        }
        cr.done();
        pg.calls.push_back(std::move(c));
      }
    }
    pr.done();
    m.programs[n] = std::move(pg);
    m.program_order.push_back(n);
  });
  r.done();
  return m;
}

Manifest parse_manifest_text(const std::string& text, Errors& errs) {
  Json doc;
  try {
    doc = parse_json(text);
  } catch (const std::exception& e) {
    errs.push_back(e.what());
    return Manifest();
  }
  return parse_manifest(doc, errs);
}

}  // namespace kern
