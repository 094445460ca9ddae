// Token-keyed index of kept prefixes (checkpoints) with tiered eviction.
//
// An entry is a token sequence and what was kept for it. A lookup for a prompt returns the longest
// usable prefix over all entries: an entry that carries a recurrent-state slot is usable only at its
// exact length (and only when the prompt starts with all of its tokens); an entry without one is usable
// at any whole-page length of the tokens it shares with the prompt, and at its exact length.
//
// Layout: entries sit in a map ordered lexicographically by key, so the entries sharing the longest
// common prefix with a prompt are the prompt's neighbours in that order; exact-prefix entries (the
// stateful ones) are found through a rolling hash of every prefix of the prompt. Eviction takes
// superseded entries first (a slot-less entry whose every page a longer slot-less entry also holds),
// then the least recently used.
// Reference: crates/kern-pool/src/prefix.rs:51-425 (a radix tree with the same contract).
#pragma once
#include <map>
#include <unordered_map>

#include "pool.hpp"

namespace kern {
namespace pool {

using Tokens = std::vector<int64_t>;

template <typename R>
struct Hit {
  uint64_t len = 0;
  R found;
};

template <typename R = Checkpoint>
class Prefix {
 public:
  explicit Prefix(uint64_t unit) : unit_(unit ? unit : 1) {}
  uint64_t unit() const { return unit_; }
  size_t size() const { return entries_.size(); }

  // keep `r` for `key`; an existing entry under the same key is replaced (its holder dropped)
  void insert(const Tokens& key, R r, bool has_slot, uint64_t len) {
    if (key.empty() || len == 0 || len > key.size()) throw std::invalid_argument("a kept prefix holds at least one token of its key");
    Tokens k(key.begin(), key.begin() + len);
    Entry e{std::move(r), has_slot, len, ++clock_};
    auto it = entries_.find(k);
    if (it != entries_.end()) { unindex(it->first); it->second = std::move(e); }
    else it = entries_.emplace(std::move(k), std::move(e)).first;
    by_hash_[hash_of(it->first, it->first.size())].push_back(&it->first);
  }

  std::optional<Hit<R>> lookup(const Tokens& prompt, uint64_t at_most = UINT64_MAX) {
    const Entry* best = nullptr;
    uint64_t best_len = 0;
    // exact prefixes: any entry whose whole key opens the prompt
    if (!by_hash_.empty()) {
      uint64_t h = kSeed;
      const uint64_t n = std::min<uint64_t>(prompt.size(), at_most);
      for (uint64_t i = 0; i < n; ++i) {
        h = mix(h, prompt[i]);
        if (i + 1 <= best_len) continue;
        auto it = by_hash_.find(h);
        if (it == by_hash_.end()) continue;
        for (const Tokens* k : it->second)
          if (k->size() == i + 1 && std::equal(k->begin(), k->end(), prompt.begin())) {
            best = &entries_.find(*k)->second;
            best_len = i + 1;
          }
      }
    }
    // shared whole pages with a slot-less entry: the neighbours in key order share the most
    auto consider = [&](typename Map::iterator it) {
      if (it == entries_.end() || it->second.has_slot) return;
      const Tokens& k = it->first;
      uint64_t common = 0;
      const uint64_t lim = std::min<uint64_t>({(uint64_t)k.size(), (uint64_t)prompt.size(), at_most});
      while (common < lim && k[common] == prompt[common]) ++common;
      uint64_t usable = common == k.size() ? common : common / unit_ * unit_;
      if (usable > best_len) { best = &it->second; best_len = usable; }
    };
    if (!entries_.empty()) {
      // slot-less neighbours: walk outwards past stateful entries (bounded: they are rare between)
      auto lo = entries_.lower_bound(prompt);
      auto fwd = lo;
      for (int i = 0; i < 8 && fwd != entries_.end(); ++i, ++fwd) consider(fwd);
      auto back = lo;
      for (int i = 0; i < 8 && back != entries_.begin(); ++i) { --back; consider(back); }
    }
    if (!best || best_len == 0) return std::nullopt;
    const_cast<Entry*>(best)->used = ++clock_;
    return Hit<R>{best_len, best->kept};
  }

  // drop the least valuable entry; returns its key (empty when nothing is kept)
  Tokens evict() {
    if (entries_.empty()) return {};
    auto victim = entries_.end();
    // superseded: the next entry in key order extends this key and both are slot-less
    for (auto it = entries_.begin(); it != entries_.end(); ++it) {
      auto nx = std::next(it);
      if (nx == entries_.end() || it->second.has_slot || nx->second.has_slot) continue;
      const Tokens &a = it->first, &b = nx->first;
      if (a.size() <= b.size() && std::equal(a.begin(), a.end(), b.begin()) && (a.size() % unit_ == 0 || a.size() == b.size())) {
        if (victim == entries_.end() || it->second.used < victim->second.used) victim = it;
      }
    }
    if (victim == entries_.end())
      for (auto it = entries_.begin(); it != entries_.end(); ++it)
        if (victim == entries_.end() || it->second.used < victim->second.used) victim = it;
    Tokens key = victim->first;
    unindex(victim->first);
    entries_.erase(victim);
    return key;
  }
  bool remove(const Tokens& key) {
    auto it = entries_.find(key);
    if (it == entries_.end()) return false;
    unindex(it->first);
    entries_.erase(it);
    return true;
  }
  void clear() { by_hash_.clear(); entries_.clear(); }

 private:
  struct Entry {
    R kept;
    bool has_slot;
    uint64_t len;
    uint64_t used;
  };
  using Map = std::map<Tokens, Entry>;
  static constexpr uint64_t kSeed = 0x9E3779B97F4A7C15ull;
  static uint64_t mix(uint64_t h, int64_t t) {
    h ^= (uint64_t)t + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    return h ^ (h >> 33);
  }
  static uint64_t hash_of(const Tokens& k, size_t n) {
    uint64_t h = kSeed;
    for (size_t i = 0; i < n; ++i) h = mix(h, k[i]);
    return h;
  }
  void unindex(const Tokens& k) {
    auto it = by_hash_.find(hash_of(k, k.size()));
    if (it == by_hash_.end()) return;
    auto& v = it->second;
    v.erase(std::remove(v.begin(), v.end(), &k), v.end());
    if (v.empty()) by_hash_.erase(it);
  }
  uint64_t unit_;
  uint64_t clock_ = 0;
  Map entries_;
  std::unordered_map<uint64_t, std::vector<const Tokens*>> by_hash_;
};

}  // namespace pool
}  // namespace kern
