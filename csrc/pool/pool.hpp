// Host-side accounting of one rank's pooled memory: pages of the paged states (all paged states share
// one page id space) and per-sequence state slots. Pure bookkeeping — no CUDA — so every rank's pool
// reaches the same decisions from the same asks without talking to the others.
//
// Three rules run through every operation: whole pages are shared, a half page is copied to its new
// holder, and the only writer is a lease (a page is frozen the moment a chain node holds it).
//
//   lease(tokens)                 fresh pages, fresh slot (the runtime zeroes it)
//   checkpoint(lease, len)        whole pages join the shared chain; a mid-page len copies the half page
//                                 to the checkpoint; the slot is copied into a new one
//   retire(lease, len)            whole pages into the chain, half page sealed in place, rest returned;
//                                 the slot changes owner (no copy)
//   restore(checkpoint, len, n)   whole pages shared, half page copied to the new lease, slot copied
//   fork(lease, len, n)           the same from a live lease
//
// Reference: crates/kern-pool/src/pages.rs:121-714, store.rs:29-156, docs/pool.md:213-229.
#pragma once
#include <algorithm>
#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace kern {
namespace pool {

struct Denied : std::runtime_error {
  enum Why { Busy, ExceedsRow, ExceedsPool } why;
  Denied(Why w, const std::string& msg) : std::runtime_error(msg), why(w) {}
};

// Free lists; shared by everything that must hand a page or slot back when it dies.
struct Core {
  uint64_t unit = 1;            // tokens per page
  uint64_t total_pages = 0, total_slots = 0, row_pages = 0;   // row_pages: widest page-table row (0 = no bound)
  std::vector<int32_t> free_pages, free_slots;                // stacks; lowest ids handed out first
  void put_page(int32_t p) { free_pages.push_back(p); }
  void put_slot(int32_t s) { free_slots.push_back(s); }
};

// One frozen page of a chain. Holding a node holds every page down to the root.
struct Node {
  int32_t page;
  uint32_t depth;   // pages in the chain up to and including this one
  std::shared_ptr<Node> parent;
  std::shared_ptr<Core> core;
  Node(int32_t p, std::shared_ptr<Node> par, std::shared_ptr<Core> c)
      : page(p), depth(par ? par->depth + 1 : 1), parent(std::move(par)), core(std::move(c)) {}
  ~Node() {
    core->put_page(page);
    // unlink iteratively: a long chain must not recurse through destructors
    std::shared_ptr<Node> p = std::move(parent);
    while (p && p.use_count() == 1) {
      std::shared_ptr<Node> next = std::move(p->parent);
      p.reset();
      p = std::move(next);
    }
  }
  Node(const Node&) = delete;
};

struct SlotOwn {
  int32_t slot;
  std::shared_ptr<Core> core;
  SlotOwn(int32_t s, std::shared_ptr<Core> c) : slot(s), core(std::move(c)) {}
  ~SlotOwn() { core->put_slot(slot); }
  SlotOwn(const SlotOwn&) = delete;
};

// Copies the runtime must execute for an operation to be complete: (source, destination) page ids of
// half pages (only the first `half_tokens` token rows of the page carry data) and one slot pair.
struct Copies {
  std::vector<std::pair<int32_t, int32_t>> pages;
  uint64_t half_tokens = 0;
  std::optional<std::pair<int32_t, int32_t>> slot;
  bool empty() const { return pages.empty() && !slot; }
};

// The bytes of a prefix: `len` tokens held in `pages` = ceil(len / unit) chain pages, plus (for
// stateful models) the recurrent state exactly after token len. Copyable: a copy is one more holder.
struct Checkpoint {
  uint64_t len = 0;
  uint64_t pages = 0;
  std::shared_ptr<Node> chain;
  std::shared_ptr<SlotOwn> slot;
  bool has_slot() const { return (bool)slot; }
  int32_t slot_id() const { return slot ? slot->slot : -1; }
  std::vector<int32_t> page_ids() const {
    std::vector<int32_t> out(chain ? chain->depth : 0);
    for (Node* n = chain.get(); n; n = n->parent.get()) out[n->depth - 1] = n->page;
    return out;
  }
  // usable at `at`: exactly len, or (without a slot) any whole-page length below it
  bool usable_at(uint64_t at, uint64_t unit) const {
    if (at == 0 || at > len) return false;
    if (at == len) return true;
    return !slot && at % unit == 0;
  }
};

// The only thing that writes. Holds shared (frozen) pages, its own pages and a slot for one sequence.
class Lease {
 public:
  Lease() = default;
  Lease(Lease&&) = default;
  Lease& operator=(Lease&& o) {
    if (this != &o) { release(); core_ = std::move(o.core_); chain_ = std::move(o.chain_); shared_ = o.shared_;
                      pages_ = std::move(o.pages_); slot_ = std::move(o.slot_); prefix_ = o.prefix_; o.shared_ = 0; }
    return *this;
  }
  ~Lease() { release(); }
  bool live() const { return (bool)core_; }
  const std::vector<int32_t>& pages() const { return pages_; }     // all page ids in position order
  uint64_t shared_pages() const { return shared_; }
  uint64_t capacity() const { return pages_.size() * core_->unit; }  // tokens the pages hold
  uint64_t prefix() const { return prefix_; }                      // positions already filled at creation
  int32_t slot() const { return slot_ ? slot_->slot : -1; }
  // token slot of position `pos` in the paged states; a position inside a frozen page is refused
  int64_t slot_of(uint64_t pos) const {
    const uint64_t pg = pos / core_->unit;
    if (pg >= pages_.size()) throw std::out_of_range("position is past the lease");
    if (pos < prefix_ || pg < shared_) throw std::logic_error("position lies in a page the lease no longer writes");
    return (int64_t)pages_[pg] * (int64_t)core_->unit + (int64_t)(pos % core_->unit);
  }
  void release() {
    if (!core_) return;
    for (size_t i = shared_; i < pages_.size(); ++i) core_->put_page(pages_[i]);
    pages_.clear();
    chain_.reset();
    slot_.reset();
    core_.reset();
    shared_ = 0;
  }

 private:
  friend class Pool;
  std::shared_ptr<Core> core_;
  std::shared_ptr<Node> chain_;   // top of the shared pages
  uint64_t shared_ = 0;
  std::vector<int32_t> pages_;
  std::shared_ptr<SlotOwn> slot_;
  uint64_t prefix_ = 0;
};

class Pool {
 public:
  // `pages` page ids 0..pages-1; `slots` usable state slots 1..slots (slot 0 is the null line and is
  // never leased); slots == 0 for a model without per-sequence state.
  Pool(uint64_t unit, uint64_t pages, uint64_t slots, uint64_t row_pages = 0) : core_(std::make_shared<Core>()) {
    if (unit == 0) throw std::invalid_argument("page unit must be >= 1");
    core_->unit = unit;
    core_->total_pages = pages;
    core_->total_slots = slots;
    core_->row_pages = row_pages;
    for (uint64_t p = pages; p-- > 0;) core_->free_pages.push_back((int32_t)p);
    for (uint64_t s = slots; s >= 1; --s) core_->free_slots.push_back((int32_t)s);
  }
  uint64_t unit() const { return core_->unit; }
  uint64_t total_pages() const { return core_->total_pages; }
  uint64_t free_pages() const { return core_->free_pages.size(); }
  uint64_t total_slots() const { return core_->total_slots; }
  uint64_t free_slots() const { return core_->free_slots.size(); }
  bool stateful() const { return core_->total_slots > 0; }
  uint64_t pages_for(uint64_t tokens) const { return (tokens + core_->unit - 1) / core_->unit; }

  // can `pages` more pages and (optionally) a slot be had right now?
  bool room(uint64_t pages, bool slot) const {
    return core_->free_pages.size() >= pages && (!slot || !stateful() || !core_->free_slots.empty());
  }

  Lease lease(uint64_t tokens) {
    const uint64_t need = pages_for(tokens);
    check(need, need, true);
    Lease l;
    l.core_ = core_;
    take_pages(l.pages_, need);
    if (stateful()) l.slot_ = take_slot();
    return l;
  }

  // Grow a lease so it holds `tokens` positions in all.
  void extend(Lease& l, uint64_t tokens) {
    const uint64_t want = pages_for(tokens);
    if (want <= l.pages_.size()) return;
    check(want, want - l.pages_.size(), false);
    take_pages(l.pages_, want - l.pages_.size());
  }

  std::pair<Checkpoint, Copies> checkpoint(Lease& l, uint64_t len) {
    if (len == 0 || len > l.capacity()) throw std::invalid_argument("checkpoint length is outside the lease");
    const uint64_t whole = len / core_->unit, half = len % core_->unit;
    check(0, (half ? 1 : 0), true);
    Copies cp;
    freeze(l, whole);
    Checkpoint c;
    c.len = len;
    c.pages = whole + (half ? 1 : 0);
    c.chain = node_at(l.chain_, whole);
    if (half) {
      std::vector<int32_t> fresh;
      take_pages(fresh, 1);
      cp.pages.emplace_back(l.pages_[whole], fresh[0]);
      cp.half_tokens = half;
      c.chain = std::make_shared<Node>(fresh[0], c.chain, core_);
    }
    if (l.slot_) {
      c.slot = take_slot();
      cp.slot = std::make_pair(l.slot_->slot, c.slot->slot);
    }
    return {std::move(c), std::move(cp)};
  }

  Checkpoint retire(Lease&& l, uint64_t len) {
    if (len == 0 || len > l.capacity()) throw std::invalid_argument("retire length is outside the lease");
    const uint64_t whole = len / core_->unit, half = len % core_->unit;
    freeze(l, whole);
    Checkpoint c;
    c.len = len;
    c.pages = whole + (half ? 1 : 0);
    c.chain = node_at(l.chain_, whole);
    if (half) {
      if (whole < l.shared_) throw std::logic_error("retire below the frozen pages of the lease");
      c.chain = std::make_shared<Node>(l.pages_[whole], c.chain, core_);   // sealed in place
      l.pages_[whole] = -1;
    }
    c.slot = std::move(l.slot_);
    // the rest goes back
    for (size_t i = std::max<uint64_t>(l.shared_, whole); i < l.pages_.size(); ++i)
      if (l.pages_[i] >= 0) core_->put_page(l.pages_[i]);
    l.pages_.clear();
    l.chain_.reset();
    l.core_.reset();
    l.shared_ = 0;
    return c;
  }

  std::pair<Lease, Copies> restore(const Checkpoint& c, uint64_t len, uint64_t tokens) {
    if (!c.usable_at(len, core_->unit)) throw std::invalid_argument("checkpoint is not usable at this length");
    return adopt(c.chain, c.slot, len, tokens);
  }

  std::pair<Lease, Copies> fork(Lease& parent, uint64_t len, uint64_t tokens) {
    if (len == 0 || len > parent.capacity()) throw std::invalid_argument("fork length is outside the lease");
    const uint64_t whole = len / core_->unit, half = len % core_->unit;
    // everything the child needs is checked before the parent's pages are frozen
    const uint64_t total = std::max(pages_for(tokens), whole + (half ? 1 : 0));
    check(total, total - whole, true);
    freeze(parent, whole);
    std::shared_ptr<Node> top = node_at(parent.chain_, whole);
    auto out = adopt_from(top, parent.slot_, len, tokens, half ? parent.pages_[whole] : -1);
    return out;
  }

 private:
  std::shared_ptr<Core> core_;

  void check(uint64_t row_total, uint64_t fresh, bool slot) const {
    if (core_->row_pages && row_total > core_->row_pages)
      throw Denied(Denied::ExceedsRow, "the sequence needs " + std::to_string(row_total) + " pages, a table row holds " +
                                           std::to_string(core_->row_pages));
    if (fresh > core_->total_pages)
      throw Denied(Denied::ExceedsPool, "the ask needs " + std::to_string(fresh) + " pages, the pool has " +
                                            std::to_string(core_->total_pages));
    if (fresh > core_->free_pages.size())
      throw Denied(Denied::Busy, "the ask needs " + std::to_string(fresh) + " pages, " +
                                     std::to_string(core_->free_pages.size()) + " are free");
    if (slot && stateful() && core_->free_slots.empty()) throw Denied(Denied::Busy, "no state slot is free");
  }
  void take_pages(std::vector<int32_t>& into, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) { into.push_back(core_->free_pages.back()); core_->free_pages.pop_back(); }
  }
  std::shared_ptr<SlotOwn> take_slot() {
    int32_t s = core_->free_slots.back();
    core_->free_slots.pop_back();
    return std::make_shared<SlotOwn>(s, core_);
  }
  // own pages [shared, upto) of the lease become chain nodes
  void freeze(Lease& l, uint64_t upto) {
    while (l.shared_ < upto) {
      l.chain_ = std::make_shared<Node>(l.pages_[l.shared_], l.chain_, core_);
      ++l.shared_;
    }
  }
  static std::shared_ptr<Node> node_at(std::shared_ptr<Node> top, uint64_t depth) {
    while (top && top->depth > depth) top = top->parent;
    return depth == 0 ? nullptr : top;
  }
  std::pair<Lease, Copies> adopt(const std::shared_ptr<Node>& chain, const std::shared_ptr<SlotOwn>& slot, uint64_t len,
                                 uint64_t tokens) {
    const uint64_t whole = len / core_->unit, half = len % core_->unit;
    const uint64_t total = std::max(pages_for(tokens), whole + (half ? 1 : 0));
    check(total, total - whole, true);
    int32_t half_src = -1;
    if (half) {
      std::shared_ptr<Node> n = node_at(chain, whole + 1);
      if (!n) throw std::logic_error("checkpoint chain is shorter than its length");
      half_src = n->page;
    }
    return adopt_from(node_at(chain, whole), slot, len, tokens, half_src);
  }
  std::pair<Lease, Copies> adopt_from(std::shared_ptr<Node> top, const std::shared_ptr<SlotOwn>& slot, uint64_t len,
                                      uint64_t tokens, int32_t half_src) {
    const uint64_t whole = len / core_->unit, half = len % core_->unit;
    const uint64_t total = std::max(pages_for(tokens), whole + (half ? 1 : 0));
    Lease l;
    l.core_ = core_;
    l.chain_ = top;
    l.shared_ = whole;
    l.prefix_ = len;
    l.pages_.resize(whole);
    for (Node* n = top.get(); n; n = n->parent.get()) l.pages_[n->depth - 1] = n->page;
    take_pages(l.pages_, total - whole);
    Copies cp;
    if (half) {
      cp.pages.emplace_back(half_src, l.pages_[whole]);
      cp.half_tokens = half;
    }
    if (slot) {
      l.slot_ = take_slot();
      cp.slot = std::make_pair(slot->slot, l.slot_->slot);
    } else if (stateful()) {
      l.slot_ = take_slot();
    }
    return {std::move(l), std::move(cp)};
  }
};

}  // namespace pool
}  // namespace kern
