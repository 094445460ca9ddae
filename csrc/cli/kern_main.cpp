// `kern`: the manifest tools as a native binary with no Python, CUDA or GPU behind them.
//
//   kern verify <manifest.json> [--protocol] [--greedy]     every diagnostic at once; exit 0 clean, 1 otherwise
//   kern cut <manifest.json> --at <i,j,...> --out <dir>      pipeline stage manifests stage0.json, stage1.json, ...
//   kern print <manifest.json>                               the manifest re-serialised (constants expanded)
//
// Reference counterpart: crates/kern-run/src/bin/kern.rs:177 (cut), :231 (verify).
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "../manifest/cut.hpp"
#include "../manifest/protocol.hpp"
#include "../manifest/verify.hpp"

using namespace kern;

namespace {

bool slurp(const std::string& path, std::string& out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::ostringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}

int usage() {
  std::fputs("usage: kern verify <manifest.json> [--protocol] [--greedy]\n"
             "       kern cut <manifest.json> --at <i,j,...> --out <dir>\n"
             "       kern print <manifest.json>\n", stderr);
  return 2;
}

// parse + verify; prints the diagnostics and returns false when there are any
bool load(const std::string& path, Manifest& m, double* ms) {
  std::string text;
  if (!slurp(path, text)) {
    std::fprintf(stderr, "kern: cannot read %s\n", path.c_str());
    return false;
  }
  const auto t0 = std::chrono::steady_clock::now();
  Errors errs;
  m = parse_manifest_text(text, errs);
  if (errs.empty()) errs = verify_manifest(m, true);
  *ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  for (auto& e : errs) std::printf("error: %s\n", e.c_str());
  return errs.empty();
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 3) return usage();
  const std::string cmd = argv[1], path = argv[2];
  Manifest m;
  double ms = 0;
  if (cmd == "verify") {
    bool want_protocol = false, sampled = true;
    for (int i = 3; i < argc; ++i) {
      if (!std::strcmp(argv[i], "--protocol")) want_protocol = true;
      else if (!std::strcmp(argv[i], "--greedy")) sampled = false;
      else return usage();
    }
    if (!load(path, m, &ms)) return 1;
    std::printf("ok: %s  model=%s  programs=%zu ops=%zu buffers=%zu states=%zu  parsed and verified in %.2f ms\n", path.c_str(),
                m.model.c_str(), m.programs.size(), m.ops.size(), m.buffers.size(), m.states.size(), ms);
    if (want_protocol) {
      Errors errs;
      auto pr = protocol_check(m, sampled, errs);
      if (!pr) {
        for (auto& e : errs) std::printf("protocol: %s\n", e.c_str());
        return 1;
      }
      std::printf("%s\n", pr->to_json().dump(1).c_str());
    }
    return 0;
  }
  if (cmd == "print") {
    if (!load(path, m, &ms)) return 1;
    std::printf("%s\n", manifest_to_json(m).dump(1).c_str());
    return 0;
  }
  if (cmd == "cut") {
    std::string at_s, out_dir;
    for (int i = 3; i + 1 < argc; i += 2) {
      if (!std::strcmp(argv[i], "--at")) at_s = argv[i + 1];
      else if (!std::strcmp(argv[i], "--out")) out_dir = argv[i + 1];
      else return usage();
    }
    if (at_s.empty() || out_dir.empty()) return usage();
    std::vector<size_t> at;
    std::stringstream ss(at_s);
    for (std::string tok; std::getline(ss, tok, ',');) at.push_back((size_t)std::stoull(tok));
    if (!load(path, m, &ms)) return 1;
    Errors errs;
    auto stages = cut_manifest(m, at, errs);
    if (!errs.empty()) {
      for (auto& e : errs) std::printf("cut: %s\n", e.c_str());
      return 1;
    }
    for (size_t i = 0; i < stages.size(); ++i) {
      const std::string p = out_dir + "/stage" + std::to_string(i) + ".json";
      std::ofstream f(p);
      if (!f) {
        std::fprintf(stderr, "kern: cannot write %s (does the directory exist?)\n", p.c_str());
        return 1;
      }
      f << manifest_to_json(stages[i]).dump(1) << "\n";
      std::printf("stage %zu: %s  (%zu calls in its largest program)\n", i, p.c_str(), [&] {
        size_t n = 0;
        for (auto& kv : stages[i].programs) n = std::max(n, kv.second.calls.size());
        return n;
      }());
    }
    return 0;
  }
  return usage();
}
