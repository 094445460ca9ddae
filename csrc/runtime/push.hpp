// The shapes of a push that is not whole pages or whole slots (pure arithmetic, no CUDA):
//
//   dealt rows     a decode tier that shards the context by position (decode context parallelism) takes, per member, the
//                  rows `kern::pool::deal` names: runs of rows a group-width apart in the prefill side's pages, contiguous
//                  in the member's pages. Each run is one strided copy, cut into pieces of at most 64 KiB (one row when a
//                  row is more) so that a copy engine or a gather kernel gets even units of work.
//   slot parts     a decode tier that shards a per-sequence state by heads (tensor parallel) takes, per member, its
//                  columns of every row of every line of the slot. A line is segments back to back, each `rows` rows of
//                  `width` bytes whose leading dimension is the heads; member p holds bytes [p w, (p + 1) w) of every
//                  row, w = width / of, and its own line is the same segments w wide.
//
// Runtime::push_copies runs them as 2-D copies into a mapped peer pool.
// Reference: crates/kern-runtime/src/push.rs:140-254 (Split, Rows), :365-434 (push_slot_part, push_rows).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../pool/deal.hpp"

namespace kern {

struct RowsCopy {
  uint64_t src = 0, dst = 0;            // byte offsets from the start of either side's state (or slot)
  uint64_t width = 0;                   // bytes per row
  uint64_t src_pitch = 0, dst_pitch = 0;
  uint64_t rows = 0;
  bool operator==(const RowsCopy& o) const {
    return src == o.src && dst == o.dst && width == o.width && src_pitch == o.src_pitch && dst_pitch == o.dst_pitch && rows == o.rows;
  }
};

constexpr uint64_t kPushPiece = 1ull << 16;

// A deal's runs as strided copies of `row`-byte rows, in run order.
inline std::vector<RowsCopy> dealt_copies(const std::vector<pool::RowRun>& runs, uint64_t row) {
  if (row == 0) throw std::invalid_argument("a dealt row holds at least one byte");
  const uint64_t most = std::max<uint64_t>(1, kPushPiece / row);
  std::vector<RowsCopy> out;
  for (const auto& r : runs) {
    if (r.rows <= 0 || r.src_row < 0 || r.dst_row < 0 || r.src_stride <= 0) throw std::invalid_argument("a deal's run is empty or negative");
    for (uint64_t i = 0; i < (uint64_t)r.rows; i += most)
      out.push_back({((uint64_t)r.src_row + i * (uint64_t)r.src_stride) * row, ((uint64_t)r.dst_row + i) * row, row,
                     (uint64_t)r.src_stride * row, row, std::min<uint64_t>(most, (uint64_t)r.rows - i)});
  }
  return out;
}

class Split {
 public:
  // segments of (rows, width bytes) in line order, over `of` members
  Split(std::vector<std::pair<uint64_t, uint64_t>> segments, uint64_t of) : seg_(std::move(segments)), of_(of) {
    if (of_ == 0 || seg_.empty()) throw std::invalid_argument("a split needs a segment and a member");
    for (auto& s : seg_)
      if (s.first == 0 || s.second == 0 || s.second % of_ != 0)
        throw std::invalid_argument("split segment of " + std::to_string(s.first) + " rows x " + std::to_string(s.second) +
                                    " bytes: expected non-empty rows that " + std::to_string(of_) + " members divide");
  }
  uint64_t of() const { return of_; }
  uint64_t line() const {
    uint64_t n = 0;
    for (auto& s : seg_) n += s.first * s.second;
    return n;
  }
  // member `part`'s share of a slot of `lines` lines: one strided copy per row of each segment, covering every line
  // (sources a whole line apart, destinations a member's line apart)
  std::vector<RowsCopy> copies(uint64_t lines, uint64_t part) const {
    if (part >= of_) throw std::invalid_argument("part " + std::to_string(part) + " of " + std::to_string(of_));
    const uint64_t ln = line();
    std::vector<RowsCopy> out;
    uint64_t at = 0;
    for (auto& s : seg_) {
      const uint64_t w = s.second / of_;
      for (uint64_t r = 0; r < s.first; ++r) out.push_back({at + r * s.second + part * w, at / of_ + r * w, w, ln, ln / of_, lines});
      at += s.first * s.second;
    }
    return out;
  }

 private:
  std::vector<std::pair<uint64_t, uint64_t>> seg_;
  uint64_t of_;
};

}  // namespace kern
