// Whole-manifest verifier: proves a manifest self-consistent without a GPU and reports every problem
// found in one pass list (never stops at the first).
// Reference: crates/kern-manifest/src/verify.rs:69-78 (limits), :174-1105 (rule groups),
// docs/manifest.md:534-601 (the fourteen rule groups in prose).
#pragma once
#include <string>
#include <vector>

#include "types.hpp"

namespace kern {

struct Limits {
  static constexpr uint64_t kMaxGridX = 2147483647ull;
  static constexpr uint64_t kMaxGridYZ = 65535;
  static constexpr uint64_t kMaxBlockThreads = 1024;
  static constexpr uint64_t kMaxBlockZ = 64;
  static constexpr uint64_t kMaxDynSharedMem = 232448;
  static constexpr uint64_t kMaxClusterBlocks = 16;
};

// Every diagnostic for `m`; empty means verified. `strict_multicast` adds the rule that every
// kernel module of a manifest running on 2 or more ranks, and every module a launch of which can
// receive a peer buffer, declares `multicast: false` (the runtime applies it at load).
Errors verify_manifest(const Manifest& m, bool strict_multicast = false);

// Lanes rule group (vector-clock happens-before over `lane` / `after`): appended to errs.
void check_lanes(const Manifest& m, Errors& errs);

// Parse + verify text. Returns true when the manifest is verified; `errs` holds every problem.
bool verify_text(const std::string& text, Manifest& out, Errors& errs);

}  // namespace kern
