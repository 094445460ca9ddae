// Manifest -> wire JSON (constants already expanded, defaults omitted), so that derived manifests
// (pipeline stages from `cut`, spliced candidates, self-hosted twins) can be written back out and
// re-read by any consumer of the v7 format.
#include "types.hpp"

namespace kern {
namespace {

Json jstr(const std::string& s) { return Json::str(s); }
Json shape_json(const std::vector<Dim>& s) { Json a = Json::array(); for (auto& d : s) a.push(d.to_json()); return a; }
Json u64s(const std::vector<uint64_t>& v) { Json a = Json::array(); for (auto x : v) a.push(Json::uint(x)); return a; }
Json pair_json(uint64_t a, uint64_t b) { Json j = Json::array(); j.push(Json::uint(a)); j.push(Json::uint(b)); return j; }

Json tensor_source_json(const TensorSource& t) {
  if (!t.ranked) return jstr(t.name);
  Json j = Json::object(), a = Json::array();
  j.set("group", jstr(t.group));
  for (auto& n : t.tensors) a.push(jstr(n));
  j.set("tensors", a);
  return j;
}
Json ranges_json(const Ranges& r) {
  if (!r.ranked) return pair_json(r.range[0], r.range[1]);
  Json j = Json::object(), a = Json::array();
  j.set("group", jstr(r.group));
  for (auto& p : r.ranges) a.push(pair_json(p.first, p.second));
  j.set("ranges", a);
  return j;
}
Json bound_json(const Bound& b) {
  switch (b.kind) {
    case Bound::Int: return Json::sint(b.i);
    case Bound::Float: return Json::number(b.f);
    default: return b.expr.to_json();
  }
}
Json params_json(const std::vector<ParamType>& ps) { Json a = Json::array(); for (auto& p : ps) a.push(jstr(p.str())); return a; }

Json tensormap_json(const TensorMapDecl& t) {
  Json j = Json::object(), box = Json::array();
  j.set("param", Json::uint(t.param));
  j.set("dtype", jstr(t.dtype));
  j.set("dims", u64s(t.dims));
  if (!t.strides.empty()) j.set("strides", u64s(t.strides));
  for (auto b : t.box) box.push(Json::uint(b));
  j.set("box", box);
  if (t.swizzle) j.set("swizzle", Json::uint(t.swizzle));
  if (t.l2_promotion) j.set("l2_promotion", Json::uint(t.l2_promotion));
  if (t.oob_nan) j.set("oob_nan", Json::boolean(true));
  if (t.wrap) j.set("wrap", Json::boolean(true));
  return j;
}
Json pack_json(const Pack& p) {
  Json j = Json::object(), fs = Json::array();
  j.set("size", Json::uint(p.size));
  for (auto& f : p.fields) {
    Json o = Json::object();
    o.set("at", Json::uint(f.at));
    if (f.width) o.set("width", Json::uint(*f.width));
    switch (f.src.kind) {
      case FieldSrc::Param: o.set("param", Json::uint(f.src.param)); break;
      case FieldSrc::Scratch: o.set("scratch", jstr(f.src.name)); break;
      case FieldSrc::I32: o.set("i32", Json::sint(f.src.i)); break;
      case FieldSrc::I64: o.set("i64", Json::sint(f.src.i)); break;
      case FieldSrc::F32: o.set("f32", Json::number(f.src.f)); break;
      case FieldSrc::U8: o.set("u8", Json::sint(f.src.i)); break;
      case FieldSrc::Var: o.set("var", jstr(f.src.name)); break;
      case FieldSrc::ExprK: o.set("expr", f.src.expr.to_json()); break;
      case FieldSrc::Rank: o.set("rank", jstr(f.src.name)); break;
      case FieldSrc::TensorMap: o.set("tensormap", tensormap_json(f.src.tmap)); break;
    }
    fs.push(o);
  }
  j.set("fields", fs);
  return j;
}
Json launch_args_json(const std::vector<LaunchArg>& as) {
  Json a = Json::array();
  for (auto& x : as) {
    Json o = Json::object();
    switch (x.kind) {
      case LaunchArg::Param: o.set("param", Json::uint(x.param)); break;
      case LaunchArg::Scratch: o.set("scratch", jstr(x.name)); break;
      case LaunchArg::I32: o.set("i32", Json::sint(x.i)); break;
      case LaunchArg::I64: o.set("i64", Json::sint(x.i)); break;
      case LaunchArg::F32: o.set("f32", Json::number(x.f)); break;
      case LaunchArg::U8: o.set("u8", Json::sint(x.i)); break;
      case LaunchArg::Rank: o.set("rank", jstr(x.name)); break;
      case LaunchArg::PackK: o.set("pack", pack_json(x.pack)); break;
    }
    a.push(o);
  }
  return a;
}
Json launch_json(const Launch& l) {
  Json j = Json::object();
  if (!l.is_extern) j.set("module", jstr(l.module));
  j.set("entry", jstr(l.entry));
  if (l.params) j.set("params", params_json(*l.params));
  if (!l.is_extern) {
    Json b = Json::array(), g = Json::array();
    for (int i = 0; i < 3; ++i) { b.push(Json::uint(l.block[i])); g.push(l.grid[i].to_json()); }
    j.set("block", b);
    j.set("grid", g);
    if (l.shared_mem) j.set("shared_mem", l.shared_mem->to_json());
    if (l.cluster) { Json c = Json::array(); for (auto v : *l.cluster) c.push(Json::uint(v)); j.set("cluster", c); }
    if (l.pdl) j.set("pdl", Json::boolean(true));
  }
  if (l.when) {
    Json w = Json::object();
    w.set("var", jstr(l.when->var));
    if (l.when->min) w.set("min", Json::uint(*l.when->min));
    if (l.when->max) w.set("max", Json::uint(*l.when->max));
    j.set("when", w);
  }
  if (l.algo) {
    Json a = Json::object();
    a.set("id", Json::sint(l.algo->id)); a.set("tile", Json::uint(l.algo->tile)); a.set("stages", Json::uint(l.algo->stages));
    a.set("split_k", Json::sint(l.algo->split_k)); a.set("reduction", Json::uint(l.algo->reduction));
    a.set("swizzle", Json::uint(l.algo->swizzle)); a.set("custom", Json::uint(l.algo->custom));
    a.set("inner_shape", Json::uint(l.algo->inner_shape)); a.set("cluster_shape", Json::uint(l.algo->cluster_shape));
    j.set("algo", a);
  }
  if (l.args) j.set("args", launch_args_json(*l.args));
  return j;
}
Json arg_json(const Arg& a) {
  Json o = Json::object();
  switch (a.kind) {
    case Arg::Buf: o.set("buf", jstr(a.name)); if (a.offset) o.set("offset", Json::uint(a.offset)); break;
    case Arg::StateK: o.set("state", jstr(a.name)); if (a.offset) o.set("offset", Json::uint(a.offset)); break;
    case Arg::Var: o.set("var", jstr(a.name)); break;
    case Arg::ExprK: o.set("expr", a.expr.to_json()); break;
    case Arg::I32: o.set("i32", Json::sint(a.i)); break;
    case Arg::I64: o.set("i64", Json::sint(a.i)); break;
    case Arg::F32: o.set("f32", Json::number(a.f)); break;
    case Arg::U8: o.set("u8", Json::sint(a.i)); break;
    case Arg::Rank: o.set("rank", jstr(a.name)); break;
  }
  return o;
}

}  // namespace

Json manifest_to_json(const Manifest& m) {
  Json j = Json::object();
  j.set("schema_version", Json::uint(m.schema_version));
  j.set("model", jstr(m.model));
  if (m.has_chat) {
    Json c = Json::object();
    if (m.tool_parser) c.set("tool_parser", jstr(*m.tool_parser));
    j.set("chat", c);
  }
  Json vars = Json::object();
  for (auto& kv : m.vars) {
    Json v = Json::object();
    v.set("max", Json::uint(kv.second.max));
    if (kv.second.axis != VarAxis::None) v.set("axis", jstr(axis_name(kv.second.axis)));
    vars.set(kv.first, v);
  }
  j.set("vars", vars);
  if (m.has_topology) {
    Json t = Json::object(), g = Json::object();
    for (auto& kv : m.topology) g.set(kv.first, Json::uint(kv.second));
    t.set("groups", g);
    j.set("topology", t);
  }
  if (m.cut) {
    Json c = Json::object();
    c.set("id", jstr(m.cut->id)); c.set("stage", Json::uint(m.cut->stage)); c.set("stages", Json::uint(m.cut->stages));
    j.set("cut", c);
  }
  Json states = Json::object();
  for (auto& kv : m.states) {
    const State& s = kv.second;
    Json o = Json::object();
    if (s.bytes_per_token) o.set("bytes_per_token", Json::uint(s.bytes_per_token));
    if (s.bytes) o.set("bytes", Json::uint(s.bytes));
    if (s.bytes_per_seq) o.set("bytes_per_seq", Json::uint(s.bytes_per_seq));
    if (s.host) {
      Json h = Json::object();
      h.set("dtype", jstr(dtype_name(s.host->dtype))); h.set("shape", u64s(s.host->shape)); h.set("strides", u64s(s.host->strides));
      o.set("host", h);
    }
    if (s.shard) {
      Json h = Json::object();
      h.set("by", jstr(s.shard->by == Shard::Position ? "position" : "heads"));
      h.set("group", jstr(s.shard->group));
      if (s.shard->by == Shard::Heads) {
        Json a = Json::array();
        for (auto& p : s.shard->segments) a.push(pair_json(p.first, p.second));
        h.set("segments", a);
      }
      o.set("shard", h);
    }
    states.set(kv.first, o);
  }
  j.set("states", states);
  Json buffers = Json::object();
  for (auto& kv : m.buffers) {
    const Buffer& b = kv.second;
    Json o = Json::object();
    o.set("dtype", jstr(dtype_name(b.dtype)));
    o.set("shape", shape_json(b.shape));
    o.set("kind", jstr(kind_name(b.kind)));
    if (b.host_placement) o.set("placement", jstr("host"));
    if (b.fill) o.set("fill", jstr(fill_name(*b.fill)));
    if (b.domain) {
      Json d = Json::object();
      if (b.domain->min) d.set("min", bound_json(*b.domain->min));
      if (b.domain->max) d.set("max", bound_json(*b.domain->max));
      if (b.domain->index_into) d.set("index_into", jstr(*b.domain->index_into));
      if (b.domain->stride != 1) d.set("stride", Json::uint(b.domain->stride));
      if (b.domain->monotone) d.set("monotone", Json::boolean(true));
      o.set("domain", d);
    }
    if (b.export_) o.set("export", Json::boolean(true));
    if (b.of) o.set("of", jstr(*b.of));
    if (b.group) o.set("group", jstr(*b.group));
    if (!b.bind.empty()) {
      Json a = Json::array();
      for (auto& s : b.bind) {
        Json sj = Json::object();
        sj.set("tensor", tensor_source_json(s.tensor));
        if (s.rows) sj.set("rows", ranges_json(*s.rows));
        if (s.cols) sj.set("cols", ranges_json(*s.cols));
        if (s.interleave) {
          Json il = Json::object();
          il.set("with", tensor_source_json(s.interleave->with));
          il.set("rows", Json::uint(s.interleave->rows));
          sj.set("interleave", il);
        }
        a.push(sj);
      }
      o.set("bind", a);
    }
    buffers.set(kv.first, o);
  }
  j.set("buffers", buffers);
  Json modules = Json::object();
  for (auto& kv : m.modules) {
    Json o = Json::object();
    o.set("source", jstr(kv.second.source));
    o.set("sha256", jstr(kv.second.sha256));
    if (kv.second.multicast_free) o.set("multicast", Json::boolean(false));
    modules.set(kv.first, o);
  }
  j.set("modules", modules);
  Json ops = Json::object();
  for (auto& kv : m.ops) {
    Json o = Json::object(), im = Json::object(), ls = Json::array();
    o.set("params", params_json(kv.second.params));
    if (!kv.second.scratch.empty()) {
      Json sc = Json::object();
      for (auto& s : kv.second.scratch) {
        Json x = Json::object();
        x.set("dtype", jstr(dtype_name(s.second.dtype)));
        x.set("shape", shape_json(s.second.shape));
        sc.set(s.first, x);
      }
      im.set("scratch", sc);
    }
    for (auto& l : kv.second.launches) ls.push(launch_json(l));
    im.set("launches", ls);
    o.set("impl", im);
    ops.set(kv.first, o);
  }
  j.set("ops", ops);
  Json programs = Json::object();
  for (auto& kv : m.programs) {
    const Program& p = kv.second;
    Json o = Json::object(), cs = Json::array();
    if (p.batch) {
      Json b = Json::object();
      b.set("groups", Json::uint(p.batch->groups));
      b.set("rows", p.batch->rows.to_json());
      if (p.batch->context) b.set("context", jstr(*p.batch->context));
      o.set("batch", b);
    }
    if (p.once) o.set("once", Json::boolean(true));
    if (p.derive) o.set("derive", Json::boolean(true));
    if (p.graph) o.set("graph", Json::boolean(true));
    for (auto& c : p.calls) {
      Json cj = Json::object(), as = Json::array();
      if (c.label) cj.set("label", jstr(*c.label));
      cj.set("op", jstr(c.op));
      for (auto& a : c.args) as.push(arg_json(a));
      cj.set("args", as);
      if (c.lane) cj.set("lane", Json::uint(c.lane));
      if (!c.after.empty()) { Json af = Json::array(); for (auto l : c.after) af.push(Json::uint(l)); cj.set("after", af); }
      cs.push(cj);
    }
    o.set("calls", cs);
    programs.set(kv.first, o);
  }
  j.set("programs", programs);
  return j;
}

}  // namespace kern
