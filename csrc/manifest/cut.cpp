// `cut` and candidates (see cut.hpp).
#include "cut.hpp"

#include <algorithm>

#include "verify.hpp"

namespace kern {
namespace {

struct Access {
  const std::string* buf;
  uint64_t offset;
  bool reads, writes;
};

std::vector<Access> accesses(const Manifest& m, const Call& c) {
  std::vector<Access> out;
  auto it = m.ops.find(c.op);
  if (it == m.ops.end()) return out;
  const auto& ps = it->second.params;
  for (size_t i = 0; i < c.args.size() && i < ps.size(); ++i)
    if (c.args[i].kind == Arg::Buf)
      out.push_back({&c.args[i].name, c.args[i].offset, ps[i].is_pointer() ? ps[i].reads() : true,
                     ps[i].is_pointer() && ps[i].writes()});
  return out;
}

std::set<std::string> written_by(const Manifest& m, const std::vector<Call>& calls, size_t lo, size_t hi) {
  std::set<std::string> w;
  for (size_t i = lo; i < hi; ++i) for (auto& a : accesses(m, calls[i])) if (a.writes) w.insert(*a.buf);
  return w;
}

// buffers read by calls[lo..hi) before those calls overwrite them whole (an `out` at offset 0 is
// taken to write the whole buffer)
std::set<std::string> live_into(const Manifest& m, const std::vector<Call>& calls, size_t lo, size_t hi) {
  std::set<std::string> live, killed;
  for (size_t i = lo; i < hi; ++i) {
    auto acc = accesses(m, calls[i]);
    for (auto& a : acc) if (a.reads && !killed.count(*a.buf)) live.insert(*a.buf);
    for (auto& a : acc) if (a.writes && !a.reads && a.offset == 0) killed.insert(*a.buf);
  }
  return live;
}

std::string fnv_id(const Manifest& m, const std::vector<size_t>& at) {
  std::string text = manifest_to_json(m).dump();
  uint64_t h = 0xcbf29ce484222325ull;
  auto mix = [&](uint8_t b) { h = (h ^ b) * 0x00000100000001b3ull; };
  for (unsigned char c : text) mix(c);
  for (size_t a : at) for (int i = 0; i < 8; ++i) mix((uint8_t)((uint64_t)a >> (8 * i)));
  char buf[17];
  snprintf(buf, sizeof buf, "%016llx", (unsigned long long)h);
  return buf;
}

void expr_vars(const Expr& e, std::set<std::string>& out) {
  std::vector<std::string> v;
  e.collect_vars(v);
  out.insert(v.begin(), v.end());
}

// every var a kept declaration names
std::set<std::string> named_vars(const std::map<std::string, Buffer>& buffers, const std::map<std::string, Op>& ops,
                                 const std::map<std::string, Program>& programs) {
  std::set<std::string> s;
  for (auto& kv : buffers) {
    for (auto& d : kv.second.shape) if (d.is_var) s.insert(d.var);
    if (kv.second.domain) {
      if (kv.second.domain->min && kv.second.domain->min->kind == Bound::Ex) expr_vars(kv.second.domain->min->expr, s);
      if (kv.second.domain->max && kv.second.domain->max->kind == Bound::Ex) expr_vars(kv.second.domain->max->expr, s);
    }
  }
  for (auto& kv : ops) {
    for (auto& sc : kv.second.scratch) for (auto& d : sc.second.shape) if (d.is_var) s.insert(d.var);
    for (auto& l : kv.second.launches) {
      for (auto& g : l.grid) expr_vars(g, s);
      if (l.shared_mem) expr_vars(*l.shared_mem, s);
      if (l.when) s.insert(l.when->var);
      if (l.args)
        for (auto& a : *l.args)
          if (a.kind == LaunchArg::PackK)
            for (auto& f : a.pack.fields) {
              if (f.src.kind == FieldSrc::Var) s.insert(f.src.name);
              if (f.src.kind == FieldSrc::ExprK) expr_vars(f.src.expr, s);
            }
    }
  }
  for (auto& kv : programs) {
    if (kv.second.batch) {
      if (kv.second.batch->rows.is_var) s.insert(kv.second.batch->rows.var);
      if (kv.second.batch->context) s.insert(*kv.second.batch->context);
    }
    for (auto& c : kv.second.calls)
      for (auto& a : c.args) {
        if (a.kind == Arg::Var) s.insert(a.name);
        if (a.kind == Arg::ExprK) expr_vars(a.expr, s);
      }
  }
  return s;
}

Manifest build_stage(const Manifest& m, std::map<std::string, Program> programs,
                     const std::map<std::string, BufferKind>& kinds, size_t s, size_t stages, const std::string& id) {
  // once / derive programs: keep, from the back, the calls that produce something this stage reads
  std::set<std::string> needed;
  for (auto& kv : programs) for (auto& c : kv.second.calls) for (auto& a : accesses(m, c)) if (a.reads) needed.insert(*a.buf);
  for (auto& kv : m.programs) {
    if (!kv.second.once && !kv.second.derive) continue;
    std::vector<Call> kept;
    for (auto it = kv.second.calls.rbegin(); it != kv.second.calls.rend(); ++it) {
      auto acc = accesses(m, *it);
      bool feeds = std::any_of(acc.begin(), acc.end(), [&](const Access& a) { return a.writes && needed.count(*a.buf); });
      if (!feeds) continue;
      for (auto& a : acc) if (a.reads) needed.insert(*a.buf);
      Call c = *it;
      c.lane = 0;
      c.after.clear();
      kept.push_back(std::move(c));
    }
    if (kept.empty()) continue;
    std::reverse(kept.begin(), kept.end());
    Program p = kv.second;
    p.calls = std::move(kept);
    programs[kv.first] = std::move(p);
  }
  Manifest out;
  out.schema_version = m.schema_version;
  out.model = m.model;
  out.has_chat = m.has_chat;
  out.tool_parser = m.tool_parser;
  out.cut = Cut{id, (uint64_t)s, (uint64_t)stages};
  for (auto& kv : programs)
    for (auto& c : kv.second.calls) {
      for (auto& a : c.args) {
        if (a.kind == Arg::Buf) { auto b = m.buffers.find(a.name); if (b != m.buffers.end()) out.buffers[a.name] = b->second; }
        if (a.kind == Arg::StateK) { auto st = m.states.find(a.name); if (st != m.states.end()) out.states[a.name] = st->second; }
      }
      auto op = m.ops.find(c.op);
      if (op != m.ops.end()) out.ops[c.op] = op->second;
    }
  for (auto& kv : kinds) {
    auto b = out.buffers.find(kv.first);
    if (b == out.buffers.end()) continue;
    b->second.kind = kv.second;
    b->second.export_ = kv.second != BufferKind::Output;
  }
  // a table whose state this stage dropped indexes a kept state of the same kind instead
  auto kind_of = [](const State& st) { return std::make_tuple(st.bytes_per_token > 0, st.bytes_per_seq, st.is_owned()); };
  for (auto& kv : out.buffers) {
    auto& d = kv.second.domain;
    if (!d || !d->index_into) continue;
    if (out.buffers.count(*d->index_into) || out.states.count(*d->index_into)) continue;
    auto old = m.states.find(*d->index_into);
    const std::string* to = nullptr;
    if (old != m.states.end())
      for (auto& st : out.states) if (kind_of(st.second) == kind_of(old->second)) { to = &st.first; break; }
    if (to) d->index_into = *to; else d.reset();
  }
  for (auto& kv : out.ops)
    for (auto& l : kv.second.launches)
      if (!l.is_extern) { auto md = m.modules.find(l.module); if (md != m.modules.end()) out.modules[l.module] = md->second; }
  auto names = named_vars(out.buffers, out.ops, programs);
  for (auto& kv : m.vars) if (names.count(kv.first)) out.vars[kv.first] = kv.second;
  for (auto& kv : programs) out.program_order.push_back(kv.first);
  out.programs = std::move(programs);
  return out;
}

}  // namespace

std::vector<Manifest> cut_manifest(const Manifest& m, const std::vector<size_t>& at, Errors& errs) {
  const size_t before = errs.size();
  if (m.has_topology) errs.push_back("the manifest has a topology; a cut takes a single-rank manifest");
  if (m.cut) errs.push_back("the manifest is already a stage of a cut");
  bool increasing = !at.empty() && at[0] != 0;
  for (size_t i = 1; i < at.size(); ++i) increasing &= at[i - 1] < at[i];
  if (!increasing) errs.push_back("cut points: at least one, increasing, none at 0");
  std::vector<std::pair<const std::string*, const Program*>> driven;
  for (auto& kv : m.programs) if (kv.second.batch) driven.emplace_back(&kv.first, &kv.second);
  if (driven.empty()) errs.push_back("no program declares a `batch`: nothing to cut");
  if (!at.empty())
    for (auto& d : driven)
      if (at.back() >= d.second->calls.size())
        errs.push_back("program `" + *d.first + "` has " + std::to_string(d.second->calls.size()) +
                       " calls; it cannot be cut before call " + std::to_string(at.back()));
  if (errs.size() != before) return {};

  const size_t stages = at.size() + 1;
  auto lo_of = [&](size_t s) { return s == 0 ? 0 : at[s - 1]; };
  auto hi_of = [&](const Program& p, size_t s) { return s < at.size() ? at[s] : p.calls.size(); };

  std::vector<std::set<std::string>> crossing(at.size());
  for (auto& d : driven) {
    const Program& p = *d.second;
    for (size_t e = 0; e < at.size(); ++e) {
      auto wr = written_by(m, p.calls, 0, at[e]);
      for (auto& b : live_into(m, p.calls, at[e], p.calls.size())) {
        if (!wr.count(b)) continue;
        auto bi = m.buffers.find(b);
        if (bi != m.buffers.end() && bi->second.kind != BufferKind::Workspace)
          errs.push_back("program `" + *d.first + "`: " + kind_name(bi->second.kind) + " buffer `" + b +
                         "` is live across the cut before call " + std::to_string(at[e]) + "; only a workspace travels");
        crossing[e].insert(b);
      }
    }
    for (size_t i = 0; i < at.back() && i < p.calls.size(); ++i)
      for (auto& a : accesses(m, p.calls[i])) {
        auto bi = m.buffers.find(*a.buf);
        // the error word is every stage's own: each keeps it as its output and the head reads them all
        const bool error_word = bi != m.buffers.end() && bi->second.fill && *bi->second.fill == Fill::Error;
        if (a.writes && !error_word && bi != m.buffers.end() &&
            (bi->second.kind == BufferKind::Output || bi->second.kind == BufferKind::Carry))
          errs.push_back("program `" + *d.first + "` call " + std::to_string(i) + " writes " + kind_name(bi->second.kind) +
                         " buffer `" + *a.buf + "` before the last stage; a pipeline's outputs come from its last stage");
      }
  }
  std::vector<std::map<std::string, BufferKind>> kinds(stages);
  for (size_t s = 0; s < stages; ++s) {
    std::set<std::string> arriving = s > 0 ? crossing[s - 1] : std::set<std::string>();
    std::set<std::string> leaving = s < at.size() ? crossing[s] : std::set<std::string>();
    std::set<std::string> touched, written;
    for (auto& d : driven) {
      const Program& p = *d.second;
      for (size_t i = lo_of(s); i < hi_of(p, s); ++i)
        for (auto& a : accesses(m, p.calls[i])) { touched.insert(*a.buf); if (a.writes) written.insert(*a.buf); }
    }
    std::set<std::string> both = arriving;
    both.insert(leaving.begin(), leaving.end());
    for (auto& b : both) {
      kinds[s][b] = arriving.count(b) ? (written.count(b) ? BufferKind::Inout : BufferKind::Input) : BufferKind::Output;
      if (!touched.count(b))
        errs.push_back("stage " + std::to_string(s) + ": `" + b + "` passes through untouched; a stage carries only what it uses");
    }
  }
  std::map<std::pair<std::string, uint64_t>, size_t> owner;
  for (auto& d : driven) {
    const Program& p = *d.second;
    for (size_t s = 0; s < stages; ++s)
      for (size_t i = lo_of(s); i < hi_of(p, s); ++i)
        for (auto& a : p.calls[i].args) {
          if (a.kind != Arg::StateK) continue;
          auto key = std::make_pair(a.name, a.offset);
          auto it = owner.find(key);
          if (it != owner.end() && it->second != s)
            errs.push_back("program `" + *d.first + "`: state `" + a.name + "`+" + std::to_string(a.offset) + " is touched by stages " +
                           std::to_string(it->second) + " and " + std::to_string(s) + "; a state region belongs to one stage");
          owner[key] = s;
        }
  }
  if (errs.size() != before) return {};

  const std::string id = fnv_id(m, at);
  std::vector<Manifest> out;
  for (size_t s = 0; s < stages; ++s) {
    std::map<std::string, Program> programs;
    for (auto& d : driven) {
      Program p = *d.second;
      p.calls.assign(d.second->calls.begin() + lo_of(s), d.second->calls.begin() + hi_of(*d.second, s));
      programs[*d.first] = std::move(p);
    }
    Manifest st = build_stage(m, std::move(programs), kinds[s], s, stages, id);
    for (auto& e : verify_manifest(st)) errs.push_back("stage " + std::to_string(s) + ": " + e);
    out.push_back(std::move(st));
  }
  if (errs.size() != before) return {};
  return out;
}

std::vector<StateUse> state_use(const Manifest& whole, const Manifest& stage) {
  auto regions = [](const Manifest& m, const std::string& st) {
    std::set<uint64_t> r;
    for (auto& kv : m.programs) for (auto& c : kv.second.calls) for (auto& a : c.args)
      if (a.kind == Arg::StateK && a.name == st) r.insert(a.offset);
    return r.size();
  };
  std::vector<StateUse> out;
  for (auto& kv : stage.states) out.push_back({kv.first, regions(stage, kv.first), regions(whole, kv.first)});
  return out;
}

// ---- candidates ------------------------------------------------------------------------------------
namespace {

std::set<std::string> launched(const std::map<std::string, Op>& ops) {
  std::set<std::string> s;
  for (auto& kv : ops) for (auto& l : kv.second.launches) if (!l.is_extern) s.insert(l.module);
  return s;
}
// add `more` into `into`; a name already taken by other bytes is renamed after its hash
std::map<std::string, std::string> adopt(std::map<std::string, Module>& into, const std::map<std::string, Module>& more) {
  std::map<std::string, std::string> names;
  for (auto& kv : more) {
    auto it = into.find(kv.first);
    std::string as = kv.first;
    if (it != into.end() && it->second.sha256 != kv.second.sha256) as = kv.first + "@" + kv.second.sha256.substr(0, 8);
    into.emplace(as, kv.second);
    names[kv.first] = as;
  }
  return names;
}
Op renamed(Op op, const std::map<std::string, std::string>& names) {
  for (auto& l : op.launches) if (!l.is_extern) { auto it = names.find(l.module); if (it != names.end()) l.module = it->second; }
  return op;
}
std::string param_list(const std::vector<ParamType>& ps) {
  std::string s;
  for (size_t i = 0; i < ps.size(); ++i) s += (i ? ", " : "") + ps[i].str();
  return s;
}
bool same_params(const std::vector<ParamType>& a, const std::vector<ParamType>& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i) if (a[i].str() != b[i].str()) return false;
  return true;
}

}  // namespace

Candidate parse_candidate(const std::string& text, Errors& errs) {
  Candidate c;
  Json doc;
  try { doc = parse_json(text); } catch (const std::exception& e) { errs.push_back(e.what()); return c; }
  if (!doc.is_obj()) { errs.push_back("a candidate is an object with `modules` and `ops`"); return c; }
  for (auto& kv : doc.obj)
    if (kv.first != "modules" && kv.first != "ops") errs.push_back("candidate: unknown field `" + kv.first + "`");
  if (!doc.find("ops")) errs.push_back("candidate: missing field `ops`");
  Json full = Json::object();
  full.set("schema_version", Json::uint(SCHEMA_VERSION));
  full.set("model", Json::str("candidate"));
  for (const char* k : {"vars", "states", "buffers", "programs"}) full.set(k, Json::object());
  full.set("modules", doc.find("modules") ? *doc.find("modules") : Json::object());
  full.set("ops", doc.find("ops") ? *doc.find("ops") : Json::object());
  Manifest m = parse_manifest(full, errs);
  c.modules = std::move(m.modules);
  c.ops = std::move(m.ops);
  return c;
}
std::string candidate_to_json(const Candidate& c) {
  Manifest m;
  m.schema_version = SCHEMA_VERSION;
  m.modules = c.modules;
  m.ops = c.ops;
  Json full = manifest_to_json(m), out = Json::object();
  out.set("modules", *full.find("modules"));
  out.set("ops", *full.find("ops"));
  return out.dump(1);
}
Candidate candidate_of(const Manifest& m, const std::vector<std::string>& ops) {
  Candidate c;
  for (auto& n : ops) { auto it = m.ops.find(n); if (it != m.ops.end()) c.ops[n] = it->second; }
  for (auto& mod : launched(c.ops)) { auto it = m.modules.find(mod); if (it != m.modules.end()) c.modules[mod] = it->second; }
  return c;
}

Manifest splice_candidate(const Manifest& m, const Candidate& c, Errors& errs) {
  const size_t before = errs.size();
  if (c.ops.empty()) errs.push_back("no ops");
  for (auto& kv : c.ops) {
    auto have = m.ops.find(kv.first);
    if (have == m.ops.end()) errs.push_back("op `" + kv.first + "`: the manifest has no such op");
    else if (!same_params(have->second.params, kv.second.params))
      errs.push_back("op `" + kv.first + "`: params [" + param_list(kv.second.params) + "] are not the manifest's [" +
                     param_list(have->second.params) + "]");
    for (auto& l : kv.second.launches)
      if (!l.is_extern && !c.modules.count(l.module) && !m.modules.count(l.module))
        errs.push_back("op `" + kv.first + "`: module `" + l.module + "` is in neither the candidate nor the manifest");
  }
  if (errs.size() != before) return Manifest();
  Manifest out = m;
  auto names = adopt(out.modules, c.modules);
  for (auto& kv : c.ops) out.ops[kv.first] = renamed(kv.second, names);
  auto used = launched(out.ops);
  for (auto it = out.modules.begin(); it != out.modules.end();) it = used.count(it->first) ? std::next(it) : out.modules.erase(it);
  for (auto& e : verify_manifest(out)) errs.push_back(e);
  return out;
}
Manifest splice_candidate(const Manifest& m, const std::string& candidate_json, Errors& errs) {
  Candidate c = parse_candidate(candidate_json, errs);
  if (!errs.empty()) return Manifest();
  return splice_candidate(m, c, errs);
}

Candidate tile_candidates(const std::string& op, const std::string& var, const std::vector<Piece>& pieces, Errors& errs) {
  const size_t before = errs.size();
  Candidate out;
  Op imp;
  const std::vector<ParamType>* params = nullptr;
  std::set<std::string> wired;
  for (size_t i = 0; i < pieces.size(); ++i) {
    const Piece& pc = pieces[i];
    auto have_it = pc.from->ops.find(op);
    if (have_it == pc.from->ops.end()) { errs.push_back("piece " + std::to_string(i) + ": no op `" + op + "`"); continue; }
    if (!params) params = &have_it->second.params;
    else if (!same_params(*params, have_it->second.params))
      errs.push_back("piece " + std::to_string(i) + ": op `" + op + "` has other params than piece 0");
    Op have = renamed(have_it->second, adopt(out.modules, pc.from->modules));
    std::map<std::string, std::string> sc_names;
    for (auto& s : have.scratch) {
      auto t = imp.scratch.find(s.first);
      auto same_shape = [](const Scratch& a, const Scratch& b) {
        if (a.dtype != b.dtype || a.shape.size() != b.shape.size()) return false;
        for (size_t k = 0; k < a.shape.size(); ++k)
          if (a.shape[k].is_var != b.shape[k].is_var || a.shape[k].c != b.shape[k].c || a.shape[k].var != b.shape[k].var) return false;
        return true;
      };
      std::string as = (t != imp.scratch.end() && !same_shape(t->second, s.second)) ? s.first + "@" + std::to_string(i) : s.first;
      imp.scratch.emplace(as, s.second);
      sc_names[s.first] = as;
    }
    for (Launch l : have.launches) {
      std::optional<uint64_t> lo = pc.min, hi = pc.max;
      if (l.when) {
        if (l.when->var != var) {
          errs.push_back("piece " + std::to_string(i) + ": op `" + op + "`: launch `" + l.entry + "` runs in a range of `" + l.when->var + "`, not of `" + var + "`");
          continue;
        }
        if (l.when->min) lo = lo ? std::max(*lo, *l.when->min) : *l.when->min;
        if (l.when->max) hi = hi ? std::min(*hi, *l.when->max) : *l.when->max;
      }
      if (lo && hi && *lo > *hi) continue;   // the launch never runs inside this piece
      if (lo && *lo <= 1) lo.reset();        // a var is at least 1: no bound
      if (lo || hi) l.when = When{var, lo, hi}; else l.when.reset();
      if (l.args)
        for (auto& a : *l.args) {
          auto fix = [&](std::string& n) { auto it = sc_names.find(n); if (it != sc_names.end()) n = it->second; wired.insert(n); };
          if (a.kind == LaunchArg::Scratch) fix(a.name);
          if (a.kind == LaunchArg::PackK) for (auto& f : a.pack.fields) if (f.src.kind == FieldSrc::Scratch) fix(f.src.name);
        }
      imp.launches.push_back(std::move(l));
    }
  }
  if (errs.size() == before && imp.launches.empty())
    errs.push_back("op `" + op + "`: no launch of any piece runs in its range of `" + var + "`");
  if (errs.size() != before || !params) return Candidate();
  std::set<std::string> used;
  for (auto& l : imp.launches) if (!l.is_extern) used.insert(l.module);
  for (auto it = out.modules.begin(); it != out.modules.end();) it = used.count(it->first) ? std::next(it) : out.modules.erase(it);
  for (auto it = imp.scratch.begin(); it != imp.scratch.end();) it = wired.count(it->first) ? std::next(it) : imp.scratch.erase(it);
  imp.params = *params;
  out.ops[op] = std::move(imp);
  return out;
}

}  // namespace kern
