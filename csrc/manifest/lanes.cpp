// Lanes rule group: a program's calls may run on side lanes (extra streams) ordered by `after`.
// The check builds the happens-before relation explicitly — every call gets the set of calls that
// are ordered before it (same-lane predecessor plus the latest call of every lane in `after`,
// closed transitively) — and then demands that two calls with no order between them touch no
// common buffer, state or op scratch unless both only read it.
// Reference: crates/kern-manifest/src/lanes.rs:50-185 (same rules, there by vector clocks),
// docs/manifest.md:589-597.
#include <algorithm>

#include "verify.hpp"

namespace kern {
namespace {

struct Touch {
  std::string res;   // "buffer `x`" | "state `x`" | "the scratch of op `x`"
  bool writes;
};

std::vector<Touch> touches(const Manifest& m, const Call& c) {
  std::map<std::string, bool> acc;
  auto it = m.ops.find(c.op);
  if (it == m.ops.end()) return {};
  const Op& op = it->second;
  for (size_t i = 0; i < c.args.size() && i < op.params.size(); ++i) {
    const Arg& a = c.args[i];
    if (a.kind == Arg::Buf) acc["buffer `" + a.name + "`"] |= op.params[i].writes();
    else if (a.kind == Arg::StateK) acc["state `" + a.name + "`"] |= op.params[i].writes();
  }
  if (!op.scratch.empty()) acc["the scratch of op `" + c.op + "`"] = true;
  std::vector<Touch> out;
  for (auto& kv : acc) out.push_back({kv.first, kv.second});
  return out;
}

// why a call may not leave lane 0: it talks to other ranks
std::string cross_rank(const Manifest& m, const Call& c) {
  auto it = m.ops.find(c.op);
  if (it == m.ops.end()) return "";
  for (auto& l : it->second.launches)
    if (l.entry.rfind("extern:nccl", 0) == 0) return "op `" + c.op + "` is a collective";
  std::set<std::string> mapped;
  for (auto& kv : m.buffers) if (kv.second.of) mapped.insert(*kv.second.of);
  for (auto& a : c.args) {
    if (a.kind != Arg::Buf && a.kind != Arg::StateK) continue;
    if (a.kind == Arg::Buf) {
      auto b = m.buffers.find(a.name);
      if (b != m.buffers.end() && b->second.kind == BufferKind::Peer) return "takes peer buffer `" + a.name + "`";
    }
    if (mapped.count(a.name)) return "takes `" + a.name + "`, which a peer buffer maps";
  }
  return "";
}

struct Bits {
  std::vector<uint64_t> w;
  explicit Bits(size_t n = 0) : w((n + 63) / 64) {}
  void set(size_t i) { w[i >> 6] |= 1ull << (i & 63); }
  bool get(size_t i) const { return (w[i >> 6] >> (i & 63)) & 1; }
  void merge(const Bits& o) { for (size_t i = 0; i < w.size(); ++i) w[i] |= o.w[i]; }
};

void check_program(const Manifest& m, const std::string& pname, const Program& p, Errors& errs) {
  const size_t n = p.calls.size();
  bool plain = true;
  for (auto& c : p.calls) plain &= c.lane == 0 && c.after.empty();
  if (plain) return;
  size_t width = 1;
  for (auto& c : p.calls) width = std::max<size_t>(width, c.lane + 1);
  auto ctx = [&](size_t i) {
    const Call& c = p.calls[i];
    return "program `" + pname + "` call #" + std::to_string(i) + " (" + (c.label ? *c.label + ", " : "") + "lane " +
           std::to_string(c.lane) + ")";
  };
  std::vector<Bits> before(n, Bits(n));          // before[i]: calls ordered before call i
  std::vector<long> last(width, -1);             // latest call seen on each lane
  for (size_t i = 0; i < n; ++i) {
    const Call& c = p.calls[i];
    std::set<uint8_t> seen;
    for (uint8_t l : c.after) {
      if (!seen.insert(l).second) errs.push_back(ctx(i) + ": `after` names lane " + std::to_string(l) + " twice");
      else if (l == c.lane) errs.push_back(ctx(i) + ": `after` names its own lane; calls on one lane already run in order");
      else if (l != 0 && (l >= width || last[l] < 0))
        errs.push_back(ctx(i) + ": `after` names lane " + std::to_string(l) + ", which runs no call before it");
    }
    if (c.lane != 0 && last[c.lane] < 0 && c.after.empty())
      errs.push_back(ctx(i) + ": a side lane's first call names the lanes it runs `after`");
    auto join = [&](uint8_t l) {
      if (l < width && last[l] >= 0) {
        before[i].merge(before[(size_t)last[l]]);
        before[i].set((size_t)last[l]);
      }
    };
    join(c.lane);
    for (uint8_t l : c.after) join(l);
    last[c.lane] = (long)i;
    if (c.lane != 0) {
      std::string why = cross_rank(m, c);
      if (!why.empty()) errs.push_back(ctx(i) + ": " + why + "; cross-rank work stays on lane 0");
    }
  }
  if (n) {
    if (p.calls[n - 1].lane != 0) {
      errs.push_back(ctx(n - 1) + ": a program ends on lane 0, after every lane");
    } else {
      for (size_t l = 1; l < width; ++l) {
        size_t total = 0, open = 0;
        long latest = -1;
        for (size_t i = 0; i + 1 < n; ++i)
          if (p.calls[i].lane == l) {
            ++total;
            if (!before[n - 1].get(i)) { ++open; latest = (long)i; }
          }
        if (open)
          errs.push_back("program `" + pname + "`: lane " + std::to_string(l) + " is never joined: " + std::to_string(open) +
                         " of its " + std::to_string(total) + " calls, up to " + ctx((size_t)latest) +
                         ", finish after the program's last call");
      }
    }
  }
  // data races: unordered pairs on different lanes sharing a resource, at least one writing
  std::map<std::string, std::vector<std::pair<size_t, bool>>> by_res;
  for (size_t i = 0; i < n; ++i)
    for (auto& t : touches(m, p.calls[i])) {
      auto& acc = by_res[t.res];
      for (auto& [j, w] : acc) {
        if (p.calls[j].lane == p.calls[i].lane) continue;
        if (!(w || t.writes)) continue;
        if (before[i].get(j)) continue;   // j < i in program order, so only j-before-i can hold
        errs.push_back(ctx(j) + " and " + ctx(i) + " both touch " + t.res + " and neither runs after the other; " +
                       (w ? ctx(j) : ctx(i)) + " writes it");
      }
      acc.emplace_back(i, t.writes);
    }
}

}  // namespace

void check_lanes(const Manifest& m, Errors& errs) {
  std::set<uint8_t> used{0};
  for (auto& kv : m.programs) for (auto& c : kv.second.calls) used.insert(c.lane);
  const uint8_t top = *used.rbegin();
  for (unsigned l = 0; l <= top; ++l)
    if (!used.count((uint8_t)l)) {
      errs.push_back("lanes are numbered densely from 0: lane " + std::to_string(l) + " runs no call, but lane " +
                     std::to_string(top) + " does");
      break;
    }
  for (auto& kv : m.programs) check_program(m, kv.first, kv.second, errs);
}

}  // namespace kern
