// `kern-run`: a manifest executed from C++ alone — no Python, no PyTorch: the manifest library, the pool library and
// the runtime (CUDA driver API by dlopen) behind a single-sequence caller.
//
//   kern-run <manifest.json> --kernels <dir of cubins> [--weights a.safetensors,b.safetensors] --prompt 5,6,7,8
//            [--steps 8] [--chunk N] [--gpu 0] [--capacity TOKENS]
//
// The caller is driven by the manifest's protocol, never by a buffer name: it leases pages (and a state slot) from a
// pool, feeds the prompt in chunks through the ragged forward, then one token per call through the one-row forward,
// filling token / position / slot / seq_len / cu_seqlens / page and line tables / sampling inputs by their fill roles,
// and reads back what the forward emits. Greedy. Prints one JSON line {"tokens": [...], "launches": n, "graphs": n, "ms": t}.
// Reference counterpart: examples/cpp/run.cpp + executor.hpp (a zero-dependency C++ consumer of the package format).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "../manifest/protocol.hpp"
#include "../manifest/verify.hpp"
#include "../pool/pool.hpp"
#include "../runtime/runtime.hpp"

using namespace kern;

namespace {

std::vector<std::string> split(const std::string& s, char c) {
  std::vector<std::string> out;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, c))
    if (!item.empty()) out.push_back(item);
  return out;
}

// one column of int values written in the fill's declared dtype
void write_ints(Runtime& rt, const Filled& f, const std::vector<int64_t>& v) {
  const uint64_t es = dtype_bytes(f.dtype);
  std::vector<uint8_t> raw(v.size() * es);
  for (size_t i = 0; i < v.size(); ++i) {
    if (f.dtype == DType::f32) {
      const float x = (float)v[i];
      std::memcpy(raw.data() + i * es, &x, 4);
    } else if (es == 8) {
      std::memcpy(raw.data() + i * es, &v[i], 8);
    } else if (es == 4) {
      const int32_t x = (int32_t)v[i];
      std::memcpy(raw.data() + i * es, &x, 4);
    } else {
      throw std::runtime_error("fill `" + f.name + "`: a " + std::to_string(es) + "-byte element is not something this caller writes");
    }
  }
  rt.write_input(f.name, raw.data(), raw.size());
}

void write_floats(Runtime& rt, const Filled& f, const std::vector<float>& v) {
  if (f.dtype != DType::f32) throw std::runtime_error("fill `" + f.name + "` is expected to be f32");
  rt.write_input(f.name, v.data(), v.size() * 4);
}

struct Caller {
  Runtime& rt;
  const Protocol& p;
  pool::Pool pool;
  pool::Lease lease;
  uint64_t length = 0;

  Caller(Runtime& r, uint64_t capacity_tokens)
      : rt(r), p(*r.protocol()), pool(r.page_unit(), r.pages(), r.slots(), 0), lease(pool.lease(capacity_tokens)) {
    if (lease.slot() >= 0) rt.zero_slot(lease.slot());
  }

  // feed `toks` (positions length .. length + n) and return the token the call emits (or -1)
  int64_t call(const std::vector<int64_t>& toks, size_t* launches) {
    const uint64_t n = toks.size();
    const Forward* fw = n == 1 ? p.forward(1, false, 1) : nullptr;
    if (!fw) fw = p.chunk();
    if (!fw) throw std::runtime_error("the manifest has no forward that takes " + std::to_string(n) + " rows of one sequence");
    std::vector<int64_t> pos(n), slot(n), ones(n, 1);
    for (uint64_t i = 0; i < n; ++i) {
      pos[i] = (int64_t)(length + i);
      slot[i] = lease.slot_of(length + i);
    }
    for (auto& f : p.fills) {
      switch (f.fill) {
        case Fill::Token: write_ints(rt, f, f.axis.kind == PAxis::Groups ? std::vector<int64_t>{toks[0]} : toks); break;
        case Fill::Position: write_ints(rt, f, pos); break;
        case Fill::Slot: write_ints(rt, f, slot); break;
        case Fill::Valid: write_ints(rt, f, ones); break;
        case Fill::SeqLen: write_ints(rt, f, {(int64_t)(length + n)}); break;
        case Fill::CuSeqlens: write_ints(rt, f, {0, (int64_t)n}); break;
        case Fill::Temperature: write_floats(rt, f, {0.f}); break;      // greedy
        case Fill::TopK: write_ints(rt, f, {0}); break;
        case Fill::TopP: write_floats(rt, f, {1.f}); break;
        case Fill::MinP: write_floats(rt, f, {0.f}); break;
        case Fill::Seed: write_ints(rt, f, {0}); break;
        default: break;      // outputs, and block tables below
      }
    }
    for (auto& t : p.page_tables) {
      const uint64_t per = std::max<uint64_t>(1, t.stride / rt.page_unit());      // pool pages per table entry
      std::vector<int32_t> row(t.width, 0);
      const auto& pg = lease.pages();
      for (uint64_t i = 0, e = 0; i < pg.size() && e < t.width; i += per, ++e) row[e] = per > 1 ? pg[i] / (int32_t)per : pg[i];
      rt.write_input(t.name, row.data(), row.size() * 4);
    }
    for (auto& t : p.line_tables) {
      std::vector<int32_t> rows(t.lines * t.width, 0);      // [lines][1 group][width]: line 0 is the sequence's own slot
      rows[0] = std::max<int32_t>(0, lease.slot());
      rt.write_input(t.name, rows.data(), rows.size() * 4);
    }
    const VarMap vars = p.vars(1, n, n, length + n);
    *launches += rt.issue(fw->name, vars, false);
    length += n;
    if (!fw->emits) return -1;
    const Filled& out = p.fills[*fw->emits];
    int64_t tok = 0;
    if (dtype_bytes(out.dtype) == 8) {
      rt.read_output(out.name, &tok, 8);
    } else {
      int32_t t32 = 0;
      rt.read_output(out.name, &t32, 4);
      tok = t32;
    }
    return tok;
  }
};

int usage() {
  std::fputs("usage: kern-run <manifest.json> --kernels <dir> [--weights a.safetensors,...] --prompt 1,2,3 [--steps 8] [--chunk N]\n"
             "                [--gpu 0] [--capacity TOKENS]\n", stderr);
  return 2;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return usage();
  std::string path = argv[1], kernels, weights, prompt_s;
  uint64_t steps = 8, chunk = 0, capacity = 0;
  int gpu = 0;
  for (int i = 2; i + 1 < argc; i += 2) {
    const std::string k = argv[i], v = argv[i + 1];
    if (k == "--kernels") kernels = v;
    else if (k == "--weights") weights = v;
    else if (k == "--prompt") prompt_s = v;
    else if (k == "--steps") steps = std::stoull(v);
    else if (k == "--chunk") chunk = std::stoull(v);
    else if (k == "--gpu") gpu = std::stoi(v);
    else if (k == "--capacity") capacity = std::stoull(v);
    else return usage();
  }
  if (kernels.empty() || prompt_s.empty()) return usage();
  try {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot read " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    Errors errs;
    Manifest m = parse_manifest_text(ss.str(), errs);
    if (errs.empty()) errs = verify_manifest(m, true);
    if (!errs.empty()) {
      for (auto& e : errs) std::fprintf(stderr, "error: %s\n", e.c_str());
      return 1;
    }
    std::vector<int64_t> prompt;
    for (auto& t : split(prompt_s, ',')) prompt.push_back(std::stoll(t));
    if (prompt.empty()) return usage();
    Capacity cap;
    cap.tokens = capacity ? capacity : 4096;
    cap.slots = 4;
    Runtime rt(std::move(m), kernels, gpu, {}, cap);
    if (!weights.empty()) rt.load_weights(split(weights, ','));
    if (!rt.protocol()) throw std::runtime_error("the manifest projects no serving protocol");
    rt.run_once_programs();
    Caller c(rt, prompt.size() + steps + 1);
    if (!chunk) chunk = rt.protocol()->rows.max;
    size_t launches = 0;
    const auto t0 = std::chrono::steady_clock::now();
    int64_t tok = -1;
    for (size_t at = 0; at < prompt.size(); at += chunk)
      tok = c.call(std::vector<int64_t>(prompt.begin() + at, prompt.begin() + std::min(prompt.size(), at + chunk)), &launches);
    std::vector<int64_t> out{tok};
    while (out.size() < steps) out.push_back(c.call({out.back()}, &launches));
    rt.synchronize();
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    std::printf("{\"tokens\": [");
    for (size_t i = 0; i < out.size(); ++i) std::printf("%s%lld", i ? ", " : "", (long long)out[i]);
    std::printf("], \"launches\": %zu, \"graphs\": %zu, \"ms\": %.3f}\n", launches, rt.graphs(), ms);
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "kern-run: %s\n", e.what());
    return 1;
  }
}
