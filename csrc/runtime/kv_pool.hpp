// Paged-KV bookkeeping of the serving runtime: which physical KV block backs which token range of
// which sequence, which blocks hold reusable prompt prefixes, and which of those go first when the
// pool runs dry.
//
// Design (everything is O(1) per block touched; no ordered containers, no scans):
//
//  * KvPool        struct-of-arrays metadata per physical block.  Free blocks form an intrusive
//                  LIFO stack through `link_`; a block that was just released is the next one
//                  handed out, so its pages are still warm in L2 when the next prefill writes them.
//  * PrefixIndex   prompt blocks that are full and immutable are published under a 64-bit *chain
//                  hash*: h_i = mix(h_{i-1}, tokens of block i), h_{-1} = seed.  The hash names the
//                  whole prefix, not a (parent block, tokens) pair, so an entry can never be reached
//                  through a parent that was evicted and recycled for other content.  A hit is
//                  confirmed against the stored token ids and the parent's hash (collisions cost a
//                  miss, never a wrong block).
//                  Eviction order is an intrusive doubly-linked LRU list that holds exactly the
//                  cached blocks no sequence references; the pool tells the index when a cached
//                  block's reference count moves between "cache only" and "in use".  A finished
//                  sequence hands its blocks back tail first, so leaves age before their parents
//                  and a chain is eaten from the end.
//  * SeqBlocks     a sequence's logical -> physical map.
//
// The method names (append / reserve / truncate / release / fork / unshare_tail / adopt_prefix,
// lookup / insert_chain / evict) are the surface the reference exposes for the same bookkeeping
// (crates/model/src/paged.rs); data layout, hashing, and eviction are this file's own.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

namespace kv {

constexpr uint32_t NIL = 0xFFFFFFFFu;

class PrefixIndex;

class KvPool {
 public:
  KvPool(uint32_t num_blocks, uint32_t block_size)
      : bs_(block_size), n_(num_blocks), ref_(num_blocks, 0), link_(num_blocks, NIL) {
    // stack order: block 0 on top, so a fresh pool hands out 0, 1, 2, ...
    for (uint32_t b = num_blocks; b-- > 0;) push_free(b);
  }
  uint32_t block_size() const { return bs_; }
  uint32_t num_blocks() const { return n_; }
  uint32_t free_blocks() const { return n_free_; }
  uint32_t refcount(uint32_t b) const { return ref_[b]; }

  bool alloc(uint32_t* out) {
    if (top_ == NIL) return false;
    const uint32_t b = top_;
    top_ = link_[b];
    --n_free_;
    ref_[b] = 1;
    *out = b;
    return true;
  }
  inline void incref(uint32_t b);
  inline bool decref(uint32_t b);  // false = the block was not referenced (double free)

  void attach(PrefixIndex* ix) { index_ = ix; }
  PrefixIndex* index() const { return index_; }

 private:
  void push_free(uint32_t b) {
    link_[b] = top_;
    top_ = b;
    ++n_free_;
  }
  uint32_t bs_, n_;
  std::vector<uint32_t> ref_;
  std::vector<uint32_t> link_;  // next free block
  uint32_t top_ = NIL, n_free_ = 0;
  PrefixIndex* index_ = nullptr;
};

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 32;
  x *= 0xD6E8FEB86659FD93ull;
  x ^= x >> 32;
  x *= 0xD6E8FEB86659FD93ull;
  x ^= x >> 32;
  return x;
}

// hash of the prefix that ends with `tokens[0..n)` given the hash of everything before it
inline uint64_t chain_hash(uint64_t parent, const uint32_t* tokens, uint32_t n) {
  uint64_t h = parent ^ (0x9E3779B97F4A7C15ull * (n + 1));
  for (uint32_t i = 0; i < n; ++i) h = mix64(h + tokens[i] + 0x632BE59BD9B4E019ull);
  return h;
}

constexpr uint64_t CHAIN_SEED = 0x243F6A8885A308D3ull;

class PrefixIndex {
 public:
  PrefixIndex() = default;
  PrefixIndex(const PrefixIndex&) = delete;
  PrefixIndex& operator=(const PrefixIndex&) = delete;
  // The pool keeps a pointer to its index: an index must be destroyed before its pool.
  ~PrefixIndex() {
    if (pool_ && pool_->index() == this) pool_->attach(nullptr);
  }
  size_t size() const { return map_.size(); }

  // Longest cached chain that is a prefix of `prompt` (whole blocks only, at most `max_tokens`).
  // Blocks that are idle (referenced by the cache alone) become the most recently used.
  std::vector<uint32_t> lookup(const uint32_t* prompt, size_t n, uint32_t bs, size_t max_tokens) {
    std::vector<uint32_t> out;
    uint64_t h = CHAIN_SEED;
    for (size_t i = 0; (i + 1) * bs <= n && (i + 1) * bs <= max_tokens; ++i) {
      const uint64_t parent = h;
      h = chain_hash(parent, prompt + i * bs, bs);
      auto it = map_.find(h);
      if (it == map_.end()) break;
      const uint32_t b = it->second;
      if (parent_[b] != parent || std::memcmp(&tokens_[(size_t)b * bs_], prompt + i * bs, bs * 4u) != 0)
        break;  // a 64-bit collision: treat as a miss
      if (in_lru_[b]) {
        unlink(b);
        push_mru(b);
      }
      out.push_back(b);
    }
    return out;
  }

  // Publish the full prompt blocks blocks[from..) of a sequence.  A prefix that is already cached
  // under another physical block keeps that block (the canonical copy); the sequence's duplicate is
  // simply not indexed.
  void insert_chain(const uint32_t* prompt, size_t n, const std::vector<uint32_t>& blocks, size_t from,
                    KvPool& pool) {
    bind(pool);
    const size_t full = std::min(n / bs_, blocks.size());
    uint64_t h = CHAIN_SEED;
    for (size_t i = 0; i < full; ++i) {
      const uint64_t parent = h;
      h = chain_hash(parent, prompt + i * bs_, bs_);
      if (i < from) continue;
      const uint32_t b = blocks[i];
      if (map_.count(h) || cached_[b]) continue;
      pool.incref(b);  // the cache's own reference (the sequence holds another: not idle yet)
      cached_[b] = 1;
      hash_[b] = h;
      parent_[b] = parent;
      std::memcpy(&tokens_[(size_t)b * bs_], prompt + i * bs_, bs_ * 4u);
      map_.emplace(h, b);
    }
  }

  // Give up to `want` idle cached blocks back to the pool, least recently used first.
  uint32_t evict(uint32_t want, KvPool& pool) {
    bind(pool);
    uint32_t freed = 0;
    while (freed < want && head_ != NIL) {
      const uint32_t b = head_;
      unlink(b);
      map_.erase(hash_[b]);
      cached_[b] = 0;
      pool.decref(b);
      ++freed;
    }
    return freed;
  }

  // Called by the pool after the reference count of block `b` changed to `now`.
  void ref_changed(uint32_t b, uint32_t now, bool rising) {
    if (b >= cached_.size() || !cached_[b]) return;
    if (!rising && now == 1) push_mru(b);          // only the cache holds it: evictable
    else if (rising && now == 2 && in_lru_[b]) unlink(b);  // a sequence adopted it
  }

  void bind(KvPool& pool) {
    if (pool.index() == this && !cached_.empty()) return;
    pool.attach(this);
    pool_ = &pool;
    bs_ = pool.block_size();
    const size_t nb = pool.num_blocks();
    cached_.assign(nb, 0);
    in_lru_.assign(nb, 0);
    hash_.assign(nb, 0);
    parent_.assign(nb, 0);
    prev_.assign(nb, NIL);
    next_.assign(nb, NIL);
    tokens_.assign(nb * bs_, 0);
  }

 private:
  void push_mru(uint32_t b) {
    prev_[b] = tail_;
    next_[b] = NIL;
    if (tail_ != NIL) next_[tail_] = b; else head_ = b;
    tail_ = b;
    in_lru_[b] = 1;
  }
  void unlink(uint32_t b) {
    const uint32_t p = prev_[b], q = next_[b];
    if (p != NIL) next_[p] = q; else head_ = q;
    if (q != NIL) prev_[q] = p; else tail_ = p;
    prev_[b] = next_[b] = NIL;
    in_lru_[b] = 0;
  }
  KvPool* pool_ = nullptr;
  uint32_t bs_ = 0;
  std::unordered_map<uint64_t, uint32_t> map_;  // chain hash -> physical block
  std::vector<uint8_t> cached_, in_lru_;
  std::vector<uint64_t> hash_, parent_;
  std::vector<uint32_t> prev_, next_;           // LRU list over idle cached blocks
  std::vector<uint32_t> tokens_;                // token ids of every cached block, for verification
  uint32_t head_ = NIL, tail_ = NIL;            // head = least recently used
};

inline void KvPool::incref(uint32_t b) {
  ++ref_[b];
  if (index_) index_->ref_changed(b, ref_[b], true);
}
inline bool KvPool::decref(uint32_t b) {
  if (ref_[b] == 0) return false;
  if (--ref_[b] == 0) push_free(b);
  else if (index_) index_->ref_changed(b, ref_[b], false);
  return true;
}

// A sequence's logical -> physical block map.  `len` counts tokens; block i backs tokens
// [i * block_size, (i + 1) * block_size).
struct SeqBlocks {
  std::vector<uint32_t> blocks;
  uint32_t len = 0;

  // one more token: (block, offset) of its slot, or false when the pool is empty
  bool append(KvPool& p, uint32_t* block, uint32_t* offset) {
    const uint32_t off = len % p.block_size();
    if (off == 0 && !grow_to(len / p.block_size() + 1, p)) return false;
    *block = blocks[len / p.block_size()];
    *offset = off;
    ++len;
    return true;
  }
  // back n more tokens; returns the first new position, or -1 when the pool ran out (what was
  // taken stays with the sequence and is returned by release / truncate)
  int64_t reserve(uint32_t n, KvPool& p) {
    const uint32_t start = len;
    if (!grow_to((len + n + p.block_size() - 1) / p.block_size(), p)) return -1;
    len += n;
    return start;
  }
  void truncate(uint32_t new_len, KvPool& p) {
    const size_t keep = (new_len + p.block_size() - 1) / p.block_size();
    while (blocks.size() > keep) {
      p.decref(blocks.back());
      blocks.pop_back();
    }
    len = new_len;
  }
  void release(KvPool& p) { truncate(0, p); }  // tail first: leaves of a cached chain age first
  SeqBlocks fork(KvPool& p) const {
    for (uint32_t b : blocks) p.incref(b);
    return *this;
  }
  // Copy-on-write of a shared tail block: true and (old, fresh) when the caller must copy its rows.
  bool unshare_tail(KvPool& p, uint32_t* old_b, uint32_t* new_b) {
    if (blocks.empty() || p.refcount(blocks.back()) <= 1) return false;
    uint32_t fresh;
    if (!p.alloc(&fresh)) return false;
    *old_b = blocks.back();
    *new_b = fresh;
    p.decref(blocks.back());
    blocks.back() = fresh;
    return true;
  }
  void adopt_prefix(const std::vector<uint32_t>& shared, KvPool& p) {
    for (uint32_t b : shared) {
      p.incref(b);
      blocks.push_back(b);
    }
    len = static_cast<uint32_t>(blocks.size()) * p.block_size();
  }

 private:
  bool grow_to(size_t want, KvPool& p) {
    while (blocks.size() < want) {
      uint32_t b;
      if (!p.alloc(&b)) return false;
      blocks.push_back(b);
    }
    return true;
  }
};

}  // namespace kv
