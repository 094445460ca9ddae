// The serving contract of a verified manifest, projected so that a serving loop never needs a
// buffer, program or var *name*: which var counts rows / groups / ranks / context, which buffer plays
// which fill role (with dtype, axis and width), page and line tables, the forward programs by row
// shape with what they hand back, once / derive program lists, and the state shards.
// Reference: crates/kern-manifest/src/protocol.rs:67-742.
#pragma once
#include <map>
#include <optional>
#include <string>
#include <vector>

#include "types.hpp"

namespace kern {

struct PAxis {
  enum Kind { Rows, Groups, Ranks, Fixed } kind = Fixed;
  uint64_t n = 0;   // Fixed
  bool operator==(const PAxis& o) const { return kind == o.kind && (kind != Fixed || n == o.n); }
  std::string str() const;
};
struct PBound {
  std::string var;
  uint64_t max = 0;
};
struct Filled {
  std::string name;
  Fill fill;
  DType dtype;
  PAxis axis;
  uint64_t width = 1;
};
struct PageTable {
  std::string name;
  uint64_t width = 0;
  std::string state;     // the paged state its domain names
  uint64_t stride = 1;   // tokens per table entry (the page size the kernels assume)
};
struct LineTable {
  std::string name;
  uint64_t lines = 0, width = 1;
  PAxis axis;
  std::string state;
  uint64_t stride = 1;
};
struct Forward {
  std::string name;
  uint64_t groups = 0;
  bool rows_var = false;
  uint64_t rows = 0;               // when !rows_var
  std::optional<size_t> emits;     // index into fills of the `tokens` output it writes
  std::optional<size_t> count;     // index into fills of the `count` output it writes
  bool graph = false;
};
struct ShardHeads {
  std::string group;
  uint64_t members = 0;
  std::vector<std::pair<uint64_t, uint64_t>> segments;
};
struct Protocol {
  PBound rows, groups;
  std::optional<PBound> ranks, context;
  std::vector<Filled> fills;
  std::vector<PageTable> page_tables;
  std::vector<LineTable> line_tables;
  std::vector<Forward> forwards;
  std::vector<std::string> once, derive;
  std::optional<std::pair<std::string, uint64_t>> positions;   // (group, members) of `shard by position`
  std::map<std::string, ShardHeads> heads;

  const Forward* forward(uint64_t groups, bool rows_var, uint64_t rows) const;
  const Forward* chunk() const { return forward(1, true, 0); }
  std::vector<uint64_t> row_shapes() const;
  const Filled* filled(Fill f, PAxis::Kind axis) const;
  const Filled* any(Fill f) const;
  bool samples() const { return any(Fill::Temperature) != nullptr; }
  VarMap vars(uint64_t groups, uint64_t rows, uint64_t ranks, uint64_t context) const;
  Json to_json() const;
};

// Project the protocol of a *verified* manifest. `sampled` demands that some forward hands tokens
// back (a hosted manifest that only computes hidden states is checked with sampled = false).
std::optional<Protocol> protocol_check(const Manifest& m, bool sampled, Errors& errs);

// A hosted manifest (host-owned states) turned into its self-owned twin for benchmarking:
// each host state becomes a `bytes` state of the span its declaration implies for `outer` rows.
// Reference: crates/kern-manifest/src/host.rs:31-81.
Manifest self_hosted(const Manifest& m, uint64_t outer_rows);

}  // namespace kern
