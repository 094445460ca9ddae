// Derived manifests: pipeline stages (`cut`) and alternative op implementations (candidates:
// `splice`, `tile`). Both are pure functions over verified manifests; every result verifies as a
// manifest of its own.
// Reference: crates/kern-manifest/src/cut.rs:79-372, crates/kern-manifest/src/candidate.rs:38-300.
#pragma once
#include <string>
#include <vector>

#include "types.hpp"

namespace kern {

// Split a single-rank manifest before each call index in `at` of every program with a `batch`.
// A stage is a function: a workspace live across a cut is an `output` of the stage before and an
// `input` (read only) or `inout` (rewritten in place) of the stage after, exported so the stage
// before can copy into it. States never travel: a (state, offset) region belongs to one stage.
// Returns the stages in order (empty when errs is non-empty).
std::vector<Manifest> cut_manifest(const Manifest& m, const std::vector<size_t>& at, Errors& errs);

// How much of each state a stage uses: (state, regions the stage touches, regions the whole touches).
struct StateUse {
  std::string state;
  size_t stage_regions = 0, whole_regions = 0;
};
std::vector<StateUse> state_use(const Manifest& whole, const Manifest& stage);

// A candidate is the `modules` and `ops` sections of a manifest and nothing else.
struct Candidate {
  std::map<std::string, Module> modules;
  std::map<std::string, Op> ops;
};
Candidate parse_candidate(const std::string& json_text, Errors& errs);
std::string candidate_to_json(const Candidate& c);
// The named ops of a manifest (and the modules they launch) as a candidate.
Candidate candidate_of(const Manifest& m, const std::vector<std::string>& ops);
// Replace the implementations of ops the manifest already has. The interface must match.
Manifest splice_candidate(const Manifest& m, const Candidate& c, Errors& errs);
Manifest splice_candidate(const Manifest& m, const std::string& candidate_json, Errors& errs);

// One implementation assembled from several, each running in its own range [min, max] of `var`.
struct Piece {
  const Candidate* from = nullptr;
  std::optional<uint64_t> min, max;
};
Candidate tile_candidates(const std::string& op, const std::string& var, const std::vector<Piece>& pieces, Errors& errs);

}  // namespace kern
