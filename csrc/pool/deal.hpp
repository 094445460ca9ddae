// Dealing positions over a group (decode context parallelism): position p of a sequence lives on
// member p % w at local position p / w. `deal` plans the hand-off of a whole-sequence page table to
// one member as the longest row runs: destination rows contiguous, source rows w apart.
// Reference: crates/kern-pool/src/deal.rs:26-156.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace kern {
namespace pool {

struct Interleave {
  uint64_t w;
  explicit Interleave(uint64_t width) : w(width) {
    if (width == 0) throw std::invalid_argument("a group deals positions over at least one member");
  }
  uint64_t owner(uint64_t p) const { return p % w; }
  uint64_t local(uint64_t p) const { return p / w; }
  // of the first n positions, how many member m holds
  uint64_t len(uint64_t n, uint64_t m) const { return n / w + (m < n % w ? 1 : 0); }
};

struct RowRun {
  int64_t src_row;      // first source row (page id * unit + offset)
  int64_t src_stride;   // rows between consecutive source rows
  int64_t dst_row;      // first destination row
  int64_t rows;
  bool operator==(const RowRun& o) const {
    return src_row == o.src_row && src_stride == o.src_stride && dst_row == o.dst_row && rows == o.rows;
  }
};

struct PagesView {
  const std::vector<int32_t>& ids;
  uint64_t unit;   // rows (token slots) per page
};

// Rows of member m among the first `len` positions of a sequence held in `src` (whole sequence,
// src.unit rows per page) laid into `dst` (the member's local positions, dst.unit rows per page).
// A run continues while both sides stay physically regular: destination row + 1, source row + w.
inline std::vector<RowRun> deal(const PagesView& src, const PagesView& dst, Interleave il, uint64_t m, uint64_t len) {
  if (m >= il.w) throw std::invalid_argument("member is outside the group");
  if (src.unit == 0 || dst.unit == 0) throw std::invalid_argument("a page holds at least one row");
  const uint64_t mine = il.len(len, m);
  if ((len + src.unit - 1) / src.unit > src.ids.size()) throw std::invalid_argument("source page table is shorter than the sequence");
  if ((mine + dst.unit - 1) / dst.unit > dst.ids.size()) throw std::invalid_argument("destination page table is shorter than the member's share");
  for (int32_t id : src.ids) if (id < 0) throw std::invalid_argument("negative source page id");
  for (int32_t id : dst.ids) if (id < 0) throw std::invalid_argument("negative destination page id");
  std::vector<RowRun> runs;
  for (uint64_t j = 0; j < mine; ++j) {
    const uint64_t p = j * il.w + m;
    const int64_t s = (int64_t)src.ids[p / src.unit] * (int64_t)src.unit + (int64_t)(p % src.unit);
    const int64_t d = (int64_t)dst.ids[j / dst.unit] * (int64_t)dst.unit + (int64_t)(j % dst.unit);
    if (!runs.empty()) {
      RowRun& r = runs.back();
      const bool dst_next = d == r.dst_row + r.rows;
      const bool src_next = r.rows == 1 ? s > r.src_row : s == r.src_row + r.rows * r.src_stride;
      if (dst_next && src_next) {
        if (r.rows == 1) r.src_stride = s - r.src_row;
        ++r.rows;
        continue;
      }
    }
    runs.push_back({s, (int64_t)il.w, d, 1});
  }
  return runs;
}

}  // namespace pool
}  // namespace kern
