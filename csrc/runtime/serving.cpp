// Serving runtime: paged KV bookkeeping and the continuous-batching scheduler.
//
//  * kv::KvPool / kv::SeqBlocks / kv::PrefixIndex (kv_pool.hpp) — block pool with an intrusive
//                     free stack, per-sequence block maps, and the chain-hashed prefix index with
//                     its O(1) LRU list of idle cached blocks.
//  * Scheduler      — per step: admit waiting requests FIFO while their whole budget
//                     (prompt + max_new) fits the free blocks and the prefill-token budget
//                     (2 x max_prefill, at least one request) remains, evicting LRU prefix-cache
//                     blocks before giving up; then one batched decode over all running
//                     sequences (a window of k on-device steps when the queue is empty, every
//                     sequence is greedy and there is room); then reap (EOS is not appended,
//                     blocks released, prompt blocks stay cached).
//
// The scheduler does not touch the GPU: `plan()` emits the prefill chunks and the decode batch as
// flat arrays, the Python engine launches the kernels and reports sampled tokens back through
// `commit_*`.  Reference: crates/model/src/serve.rs:262-776 (scheduler semantics).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "kv_pool.hpp"

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

using BlockAllocator = kv::KvPool;
using BlockTable = kv::SeqBlocks;
using PrefixCache = kv::PrefixIndex;

// ------------------------------------------------------------------------------------ scheduler
enum Reject : int { OK = 0, EXCEEDS_CAPACITY = -1, INVALID_TOKEN = -2, POLICY_REJECTED = -3, EMPTY = -4 };
enum SeqState : int { WAITING = 0, RUNNING = 1, FINISHED = 2, CANCELLED = 3 };
enum Finish : int { NONE = 0, STOP = 1, LENGTH = 2 };

struct Seq {
  int64_t id;
  std::vector<uint32_t> prompt;
  std::vector<uint32_t> out;
  uint32_t max_new;
  float temp, top_p;
  uint32_t top_k;
  uint64_t seed;
  bool ignore_eos;
  BlockTable table;
  SeqState state = WAITING;
  Finish finish = NONE;
  uint32_t prefilled = 0;      // prompt tokens whose K/V are stored
  uint32_t prefix_hit = 0;
  uint32_t last_token = 0;     // next decode input
  bool greedy() const { return temp <= 0.f; }
};

struct Config {
  uint32_t num_blocks, block_size, max_batch, max_prefill, max_seq_len, vocab;
  int64_t eos;        // < 0: none
  uint32_t window;    // on-device greedy steps per decode call when idle-queue (>= 1)
  int policy;         // 0 unbounded queue, 1 max queue depth, 2 deadline aware, 3 first-token budget
  double policy_arg;
  int prefix_cache;   // 0/1
};

class Scheduler {
 public:
  explicit Scheduler(const Config& c) : cfg_(c), alloc_(c.num_blocks, c.block_size) {}

  uint32_t blocks_for(uint32_t tokens) const { return (tokens + cfg_.block_size - 1) / cfg_.block_size; }

  int64_t submit(const uint32_t* prompt, uint32_t n, uint32_t max_new, float temp, uint32_t top_k,
                 float top_p, uint64_t seed, int ignore_eos) {
    if (n == 0) return EMPTY;
    for (uint32_t i = 0; i < n; ++i)
      if (prompt[i] >= cfg_.vocab) {
        last_bad_token_ = prompt[i];
        return INVALID_TOKEN;
      }
    const uint64_t need = static_cast<uint64_t>(n) + max_new;
    last_need_ = need;
    if (need > cfg_.max_seq_len || blocks_for(static_cast<uint32_t>(need)) > cfg_.num_blocks)
      return EXCEEDS_CAPACITY;
    if (cfg_.policy == 1 && waiting_.size() >= static_cast<size_t>(cfg_.policy_arg)) return POLICY_REJECTED;
    if (cfg_.policy == 2 && mean_service_ms_ > 0 &&
        static_cast<double>(waiting_.size()) * mean_service_ms_ > cfg_.policy_arg)
      return POLICY_REJECTED;
    // first-token budget: the new request's first token comes after every prompt token that is
    // queued or still being prefilled ahead of it, plus its own; at the measured prefill rate that
    // must fit in policy_arg milliseconds (nothing is rejected before a rate was measured)
    if (cfg_.policy == 3 && prefill_tokens_per_ms_ > 0 &&
        static_cast<double>(pending_prefill_tokens() + n) / prefill_tokens_per_ms_ > cfg_.policy_arg)
      return POLICY_REJECTED;
    auto s = std::make_unique<Seq>();
    s->id = next_id_++;
    s->prompt.assign(prompt, prompt + n);
    s->max_new = max_new;
    s->temp = temp;
    s->top_k = top_k;
    s->top_p = top_p;
    s->seed = seed;
    s->ignore_eos = ignore_eos != 0;
    const int64_t id = s->id;
    waiting_.push_back(id);
    seqs_[id] = std::move(s);
    ++submitted_;
    return id;
  }

  // tokens generated so far are left readable through output(); blocks are freed immediately
  int cancel(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return -1;
    Seq& s = *it->second;
    if (s.state == WAITING) {
      waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    } else if (s.state == RUNNING) {
      running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
      s.table.release(alloc_);
    } else {
      return 0;
    }
    s.state = CANCELLED;
    ++cancelled_;
    return 0;
  }

  bool idle() const { return waiting_.empty() && running_.empty(); }

  // prompt tokens whose K/V are not stored yet: whole prompts in the queue (a prefix-cache hit is
  // only known at admission, so it is not discounted) and the rest of prompts that are mid-prefill
  uint64_t pending_prefill_tokens() const {
    uint64_t t = 0;
    for (int64_t id : waiting_) t += seqs_.at(id)->prompt.size();
    for (int64_t id : running_) {
      const Seq& r = *seqs_.at(id);
      if (r.prefilled < r.prompt.size()) t += r.prompt.size() - r.prefilled;
    }
    return t;
  }

  // ---- step planning ----------------------------------------------------------------------
  struct PrefillItem {
    int64_t id;
    uint32_t start, end;  // prompt positions whose K/V this chunk computes
    bool last;            // chunk reaches the end of the prompt -> first token is sampled
  };
  std::vector<PrefillItem> prefill_plan;
  std::vector<int64_t> decode_plan;
  uint32_t decode_window = 1;
  bool decode_all_greedy = true;
  // what the commits of the current step produced: one entry per sequence that gained tokens or
  // finished, with its new tokens in step_tokens[first, first + n_new)
  struct StepOut {
    int64_t id;
    uint32_t n_new, first;
    int finished;
  };
  std::vector<StepOut> step_out;
  std::vector<uint32_t> step_tokens;

  void plan() {
    prefill_plan.clear();
    decode_plan.clear();
    step_out.clear();
    step_tokens.clear();
    // (1) continue partially prefilled sequences, then admit new ones, under the token budget
    uint32_t budget = prefill_budget_ ? prefill_budget_ : 2 * cfg_.max_prefill;
    bool any = false;
    for (int64_t id : running_) {
      Seq& s = *seqs_[id];
      if (s.prefilled < s.prompt.size()) {
        const uint32_t n = std::min<uint32_t>(cfg_.max_prefill, static_cast<uint32_t>(s.prompt.size()) - s.prefilled);
        if (any && n > budget) break;
        if (!reserve_or_evict(s, n)) break;
        prefill_plan.push_back({id, s.prefilled, s.prefilled + n, s.prefilled + n == s.prompt.size()});
        budget = budget > n ? budget - n : 0;
        any = true;
      }
    }
    // blocks the running sequences may still claim (prompt + max_new each): admission keeps them
    // free, so a sequence that was admitted can always run to its full length
    uint64_t outstanding = 0;
    for (int64_t id : running_) {
      const Seq& r = *seqs_[id];
      const uint32_t full = blocks_for(static_cast<uint32_t>(r.prompt.size()) + r.max_new);
      const uint32_t have = static_cast<uint32_t>(r.table.blocks.size());
      if (full > have) outstanding += full - have;
    }
    // Admission batching: with `admit_batch` > 1 new requests are taken in only once that many
    // slots are free (or nothing runs, or the head of the queue has waited `admit_max_wait`
    // steps), so prefill work arrives in a few large chunks instead of one small one per step.
    ++steps_since_admit_;
    bool admit_now = true;
    if (admit_batch_ > 1 && !running_.empty() && !waiting_.empty()) {
      // a closed-loop client hands over one new request per finished one, so the queue length says
      // nothing: wait until a whole group of slots is free (or the head waited long enough)
      const size_t free_slots = cfg_.max_batch > running_.size() ? cfg_.max_batch - running_.size() : 0;
      admit_now = free_slots >= admit_batch_ || steps_since_admit_ >= admit_max_wait_;
    }
    while (admit_now && !waiting_.empty() && running_.size() < cfg_.max_batch) {
      Seq& s = *seqs_[waiting_.front()];
      const uint32_t total = static_cast<uint32_t>(s.prompt.size()) + s.max_new;
      // prefix-cache hit: adopt shared full blocks (never the whole prompt: the last token must
      // be recomputed to produce logits)
      std::vector<uint32_t> hit;
      if (cfg_.prefix_cache)
        hit = prefix_.lookup(s.prompt.data(), s.prompt.size(), cfg_.block_size, s.prompt.size() - 1);
      const uint32_t need_blocks = blocks_for(total) - static_cast<uint32_t>(hit.size());
      const uint64_t want_free = need_blocks + outstanding;
      if (alloc_.free_blocks() < want_free && cfg_.prefix_cache) {
        // pin the hit while evicting so the eviction cannot take it
        for (uint32_t b : hit) alloc_.incref(b);
        prefix_.evict(static_cast<uint32_t>(want_free - alloc_.free_blocks()), alloc_);
        for (uint32_t b : hit) alloc_.decref(b);
      }
      if (alloc_.free_blocks() < want_free) break;  // FIFO: do not skip ahead
      const uint32_t remaining = static_cast<uint32_t>(s.prompt.size()) - static_cast<uint32_t>(hit.size()) * cfg_.block_size;
      const uint32_t n = std::min(cfg_.max_prefill, remaining);
      if (any && n > budget) break;
      waiting_.pop_front();
      s.table.adopt_prefix(hit, alloc_);
      s.prefix_hit = s.table.len;
      s.prefilled = s.table.len;
      prefix_hit_tokens_ += s.prefix_hit;
      prefix_lookup_tokens_ += s.prompt.size();
      s.table.reserve(n, alloc_);
      outstanding += blocks_for(total) - static_cast<uint32_t>(s.table.blocks.size());
      s.state = RUNNING;
      running_.push_back(s.id);
      steps_since_admit_ = 0;
      prefill_plan.push_back({s.id, s.prefilled, s.prefilled + n, s.prefilled + n == s.prompt.size()});
      budget = budget > n ? budget - n : 0;
      any = true;
    }
    // (2) decode batch: every running sequence whose prompt is fully prefilled and has a token
    bool all_greedy = true;
    for (int64_t id : running_) {
      Seq& s = *seqs_[id];
      if (s.prefilled == s.prompt.size() && !s.out.empty()) {
        decode_plan.push_back(id);
        all_greedy = all_greedy && s.greedy();
      }
    }
    decode_all_greedy = all_greedy;
    decode_window = 1;
    // A window of on-device steps is taken when nobody could be admitted during it anyway: the
    // queue is empty, every slot is taken (the window never outlives a sequence, so no slot frees
    // inside it), or admission is being held back for batching (then at most up to its next turn).
    const bool slots_full = running_.size() >= cfg_.max_batch;
    const bool held = !waiting_.empty() && !admit_now && !slots_full;
    if (cfg_.window > 1 && (waiting_.empty() || slots_full || held) && prefill_plan.empty() && all_greedy &&
        !decode_plan.empty() && alloc_.free_blocks() >= decode_plan.size() * cfg_.window) {
      uint32_t w = cfg_.window;
      if (held)
        w = std::min<uint32_t>(w, admit_max_wait_ > steps_since_admit_ ? admit_max_wait_ - steps_since_admit_ : 1);
      for (int64_t id : decode_plan) {
        Seq& s = *seqs_[id];
        w = std::min<uint32_t>(w, s.max_new - static_cast<uint32_t>(s.out.size()) + 1);
      }
      decode_window = std::max<uint32_t>(1, w);
      steps_since_admit_ += decode_window - 1;   // the window is that many scheduler steps
    }
    // back the positions the decode steps will write
    std::vector<int64_t> ok;
    for (int64_t id : decode_plan) {
      Seq& s = *seqs_[id];
      if (!reserve_or_evict(s, decode_window)) {
        // pool exhausted mid-flight even after dropping cached prefixes: finish the sequence at
        // its current length (and say so in this step's report)
        finish(s, LENGTH);
        record(s, s.out.size());
        continue;
      }
      ok.push_back(id);
    }
    decode_plan.swap(ok);
    ++steps_;
  }

  // A prefill chunk finished; `token` is the first sampled token when the chunk was the last.
  void commit_prefill(int64_t id, uint32_t end, int has_token, uint32_t token) {
    Seq& s = *seqs_.at(id);
    s.prefilled = end;
    if (end == s.prompt.size()) {
      if (cfg_.prefix_cache)
        prefix_.insert_chain(s.prompt.data(), s.prompt.size(), s.table.blocks,
                             s.prefix_hit / cfg_.block_size, alloc_);
      if (has_token) {
        const size_t before = s.out.size();
        push_token(s, token);
        record(s, before);
      }
    }
  }

  // Decode results: `window` tokens per planned sequence, row-major [n, window].
  void commit_decode(const uint32_t* tokens, uint32_t n, uint32_t window) {
    std::vector<int64_t> ids = decode_plan;
    for (uint32_t i = 0; i < n && i < ids.size(); ++i) {
      Seq& s = *seqs_.at(ids[i]);
      uint32_t used = 0;
      const size_t before = s.out.size();
      for (uint32_t w = 0; w < window && s.state == RUNNING; ++w) {
        push_token(s, tokens[i * window + w]);
        ++used;
      }
      if (s.state == RUNNING && used < window) s.table.truncate(s.table.len - (window - used), alloc_);
      record(s, before);
    }
  }

  Seq* get(int64_t id) {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : it->second.get();
  }
  void forget(int64_t id) { seqs_.erase(id); }

  const Config& cfg() const { return cfg_; }
  BlockAllocator& alloc() { return alloc_; }
  PrefixCache& prefix() { return prefix_; }
  size_t n_waiting() const { return waiting_.size(); }
  size_t n_running() const { return running_.size(); }
  uint32_t admit_batch_ = 1, admit_max_wait_ = 64, steps_since_admit_ = 0, prefill_budget_ = 0;
  uint64_t last_need_ = 0, last_bad_token_ = 0;
  uint64_t prefix_hit_tokens_ = 0, prefix_lookup_tokens_ = 0, steps_ = 0, submitted_ = 0, finished_ = 0,
           cancelled_ = 0, generated_ = 0;
  double mean_service_ms_ = 0, prefill_tokens_per_ms_ = 0;

 private:
  // Back `n` more positions of `s`; when the pool is short, evict least-recently-used prefix-cache
  // blocks (they only hold a cache reference) and try once more.
  bool reserve_or_evict(Seq& s, uint32_t n) {
    if (s.table.reserve(n, alloc_) >= 0) return true;
    if (!cfg_.prefix_cache) return false;
    const uint32_t need = blocks_for(s.table.len + n), have = static_cast<uint32_t>(s.table.blocks.size());
    prefix_.evict(need > have ? need - have : 1, alloc_);
    return s.table.reserve(n, alloc_) >= 0;
  }
  void record(const Seq& s, size_t before) {
    const uint32_t n_new = static_cast<uint32_t>(s.out.size() - before);
    if (n_new == 0 && s.state != FINISHED) return;
    step_out.push_back({s.id, n_new, static_cast<uint32_t>(step_tokens.size()), s.state == FINISHED ? 1 : 0});
    step_tokens.insert(step_tokens.end(), s.out.begin() + static_cast<long>(before), s.out.end());
  }
  void finish(Seq& s, Finish why) {
    s.state = FINISHED;
    s.finish = why;
    s.table.release(alloc_);  // prompt blocks indexed by the prefix cache keep the cache's ref
    running_.erase(std::remove(running_.begin(), running_.end(), s.id), running_.end());
    ++finished_;
  }
  void push_token(Seq& s, uint32_t tok) {
    if (s.state != RUNNING) return;
    if (!s.ignore_eos && cfg_.eos >= 0 && tok == static_cast<uint32_t>(cfg_.eos)) {
      finish(s, STOP);  // EOS is not appended
      return;
    }
    s.out.push_back(tok);
    s.last_token = tok;
    ++generated_;
    if (s.out.size() >= s.max_new) finish(s, LENGTH);
  }

  Config cfg_;
  BlockAllocator alloc_;
  PrefixCache prefix_;
  std::unordered_map<int64_t, std::unique_ptr<Seq>> seqs_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_;
  int64_t next_id_ = 1;
};

}  // namespace

// ---- C ABI: allocator / table / prefix cache (used directly by tests and the engine) -----------
BBH_API void* bbh_alloc_new(uint32_t num_blocks, uint32_t block_size) {
  if (num_blocks == 0 || block_size == 0) return nullptr;
  return new BlockAllocator(num_blocks, block_size);
}
BBH_API void bbh_alloc_free(void* a) { delete static_cast<BlockAllocator*>(a); }
BBH_API uint32_t bbh_alloc_free_blocks(void* a) { return static_cast<BlockAllocator*>(a)->free_blocks(); }
BBH_API uint32_t bbh_alloc_refcount(void* a, uint32_t b) { return static_cast<BlockAllocator*>(a)->refcount(b); }
BBH_API int64_t bbh_alloc_alloc(void* a) {
  uint32_t b;
  return static_cast<BlockAllocator*>(a)->alloc(&b) ? static_cast<int64_t>(b) : -1;
}
BBH_API void bbh_alloc_incref(void* a, uint32_t b) { static_cast<BlockAllocator*>(a)->incref(b); }
BBH_API int bbh_alloc_decref(void* a, uint32_t b) { return static_cast<BlockAllocator*>(a)->decref(b) ? 0 : -1; }

BBH_API void* bbh_table_new() { return new BlockTable(); }
BBH_API void bbh_table_free(void* t) { delete static_cast<BlockTable*>(t); }
BBH_API uint32_t bbh_table_len(void* t) { return static_cast<BlockTable*>(t)->len; }
BBH_API uint32_t bbh_table_num_blocks(void* t) { return static_cast<uint32_t>(static_cast<BlockTable*>(t)->blocks.size()); }
BBH_API void bbh_table_blocks(void* t, uint32_t* out) {
  auto& b = static_cast<BlockTable*>(t)->blocks;
  std::memcpy(out, b.data(), b.size() * sizeof(uint32_t));
}
BBH_API int bbh_table_append(void* t, void* a, uint32_t* block, uint32_t* offset) {
  return static_cast<BlockTable*>(t)->append(*static_cast<BlockAllocator*>(a), block, offset) ? 0 : -1;
}
BBH_API int64_t bbh_table_reserve(void* t, void* a, uint32_t n) {
  return static_cast<BlockTable*>(t)->reserve(n, *static_cast<BlockAllocator*>(a));
}
BBH_API void bbh_table_truncate(void* t, void* a, uint32_t n) {
  static_cast<BlockTable*>(t)->truncate(n, *static_cast<BlockAllocator*>(a));
}
BBH_API void bbh_table_release(void* t, void* a) { static_cast<BlockTable*>(t)->release(*static_cast<BlockAllocator*>(a)); }
BBH_API void* bbh_table_fork(void* t, void* a) {
  return new BlockTable(static_cast<BlockTable*>(t)->fork(*static_cast<BlockAllocator*>(a)));
}
BBH_API int bbh_table_unshare_tail(void* t, void* a, uint32_t* old_b, uint32_t* new_b) {
  return static_cast<BlockTable*>(t)->unshare_tail(*static_cast<BlockAllocator*>(a), old_b, new_b) ? 1 : 0;
}
BBH_API void bbh_table_adopt_prefix(void* t, void* a, const uint32_t* blocks, uint32_t n) {
  static_cast<BlockTable*>(t)->adopt_prefix(std::vector<uint32_t>(blocks, blocks + n), *static_cast<BlockAllocator*>(a));
}

BBH_API void* bbh_prefix_new() { return new PrefixCache(); }
BBH_API void bbh_prefix_free(void* p) { delete static_cast<PrefixCache*>(p); }
BBH_API uint64_t bbh_prefix_len(void* p) { return static_cast<PrefixCache*>(p)->size(); }
BBH_API uint32_t bbh_prefix_lookup(void* p, const uint32_t* prompt, uint64_t n, uint32_t bs,
                                   uint64_t max_tokens, uint32_t* out) {
  auto v = static_cast<PrefixCache*>(p)->lookup(prompt, n, bs, max_tokens);
  std::memcpy(out, v.data(), v.size() * sizeof(uint32_t));
  return static_cast<uint32_t>(v.size());
}
BBH_API void bbh_prefix_insert_chain(void* p, void* a, const uint32_t* prompt, uint64_t n,
                                     const uint32_t* blocks, uint32_t nb, uint32_t from) {
  static_cast<PrefixCache*>(p)->insert_chain(prompt, n, std::vector<uint32_t>(blocks, blocks + nb), from,
                                             *static_cast<BlockAllocator*>(a));
}
BBH_API uint32_t bbh_prefix_evict(void* p, void* a, uint32_t want) {
  return static_cast<PrefixCache*>(p)->evict(want, *static_cast<BlockAllocator*>(a));
}

// ---- C ABI: scheduler ---------------------------------------------------------------------------
BBH_API void* bbh_sched_new(uint32_t num_blocks, uint32_t block_size, uint32_t max_batch,
                            uint32_t max_prefill, uint32_t max_seq_len, uint32_t vocab, int64_t eos,
                            uint32_t window, int policy, double policy_arg, int prefix_cache) {
  if (!num_blocks || !block_size || !max_batch || !max_prefill) return nullptr;
  Config c{num_blocks, block_size, max_batch, max_prefill, max_seq_len, vocab, eos,
           window ? window : 1, policy, policy_arg, prefix_cache};
  return new Scheduler(c);
}
BBH_API void bbh_sched_free(void* s) { delete static_cast<Scheduler*>(s); }
BBH_API int64_t bbh_sched_submit(void* s, const uint32_t* prompt, uint32_t n, uint32_t max_new,
                                 float temp, uint32_t top_k, float top_p, uint64_t seed, int ignore_eos) {
  return static_cast<Scheduler*>(s)->submit(prompt, n, max_new, temp, top_k, top_p, seed, ignore_eos);
}
BBH_API uint64_t bbh_sched_last_need(void* s) { return static_cast<Scheduler*>(s)->last_need_; }
BBH_API uint64_t bbh_sched_last_bad_token(void* s) { return static_cast<Scheduler*>(s)->last_bad_token_; }
BBH_API int bbh_sched_cancel(void* s, int64_t id) { return static_cast<Scheduler*>(s)->cancel(id); }
BBH_API int bbh_sched_idle(void* s) { return static_cast<Scheduler*>(s)->idle() ? 1 : 0; }
BBH_API void bbh_sched_plan(void* s, uint32_t* n_prefill, uint32_t* n_decode, uint32_t* window) {
  auto* sc = static_cast<Scheduler*>(s);
  sc->plan();
  *n_prefill = static_cast<uint32_t>(sc->prefill_plan.size());
  *n_decode = static_cast<uint32_t>(sc->decode_plan.size());
  *window = sc->decode_window;
}
// prefill item i: id, [start, end), last flag
BBH_API void bbh_sched_prefill_item(void* s, uint32_t i, int64_t* id, uint32_t* start, uint32_t* end, int* last) {
  auto& it = static_cast<Scheduler*>(s)->prefill_plan[i];
  *id = it.id;
  *start = it.start;
  *end = it.end;
  *last = it.last ? 1 : 0;
}
// decode batch as flat arrays: ids[n], input token[n], position of that token[n] (= len before the
// step), and the block tables padded to max_blocks with -1
BBH_API void bbh_sched_decode_batch(void* s, int64_t* ids, int32_t* tokens, int32_t* positions,
                                    int32_t* block_tables, uint32_t max_blocks) {
  auto* sc = static_cast<Scheduler*>(s);
  for (size_t i = 0; i < sc->decode_plan.size(); ++i) {
    Seq& q = *sc->get(sc->decode_plan[i]);
    ids[i] = q.id;
    tokens[i] = static_cast<int32_t>(q.last_token);
    positions[i] = static_cast<int32_t>(q.table.len - sc->decode_window);
    for (uint32_t b = 0; b < max_blocks; ++b)
      block_tables[i * max_blocks + b] = b < q.table.blocks.size() ? static_cast<int32_t>(q.table.blocks[b]) : -1;
  }
}
BBH_API void bbh_sched_commit_prefill(void* s, int64_t id, uint32_t end, int has_token, uint32_t token) {
  static_cast<Scheduler*>(s)->commit_prefill(id, end, has_token, token);
}
BBH_API void bbh_sched_commit_decode(void* s, const uint32_t* tokens, uint32_t n, uint32_t window) {
  static_cast<Scheduler*>(s)->commit_decode(tokens, n, window);
}
// sequence inspection: state (0 waiting, 1 running, 2 finished, 3 cancelled), finish reason
// (0 none, 1 stop, 2 length), counts; returns -1 for an unknown id
BBH_API int bbh_sched_seq_info(void* s, int64_t id, int* state, int* finish, uint32_t* n_prompt,
                               uint32_t* n_out, uint32_t* prefilled, uint32_t* prefix_hit, float* temp,
                               uint32_t* top_k, float* top_p, uint64_t* seed) {
  Seq* q = static_cast<Scheduler*>(s)->get(id);
  if (!q) return -1;
  *state = q->state;
  *finish = q->finish;
  *n_prompt = static_cast<uint32_t>(q->prompt.size());
  *n_out = static_cast<uint32_t>(q->out.size());
  *prefilled = q->prefilled;
  *prefix_hit = q->prefix_hit;
  *temp = q->temp;
  *top_k = q->top_k;
  *top_p = q->top_p;
  *seed = q->seed;
  return 0;
}
BBH_API void bbh_sched_seq_output(void* s, int64_t id, uint32_t* out) {
  Seq* q = static_cast<Scheduler*>(s)->get(id);
  if (q) std::memcpy(out, q->out.data(), q->out.size() * sizeof(uint32_t));
}
BBH_API void bbh_sched_seq_prompt(void* s, int64_t id, uint32_t* out) {
  Seq* q = static_cast<Scheduler*>(s)->get(id);
  if (q) std::memcpy(out, q->prompt.data(), q->prompt.size() * sizeof(uint32_t));
}
BBH_API uint32_t bbh_sched_seq_table(void* s, int64_t id, int32_t* blocks, uint32_t max_blocks) {
  Seq* q = static_cast<Scheduler*>(s)->get(id);
  if (!q) return 0;
  const uint32_t n = std::min<uint32_t>(max_blocks, static_cast<uint32_t>(q->table.blocks.size()));
  for (uint32_t i = 0; i < n; ++i) blocks[i] = static_cast<int32_t>(q->table.blocks[i]);
  return static_cast<uint32_t>(q->table.blocks.size());
}
BBH_API void bbh_sched_set_admit(void* s, uint32_t batch, uint32_t max_wait_steps) {
  auto* sc = static_cast<Scheduler*>(s);
  sc->admit_batch_ = batch < 1 ? 1 : batch;
  sc->admit_max_wait_ = max_wait_steps < 1 ? 1 : max_wait_steps;
}
BBH_API void bbh_sched_set_prefill_budget(void* s, uint32_t tokens) { static_cast<Scheduler*>(s)->prefill_budget_ = tokens; }
BBH_API int bbh_sched_decode_all_greedy(void* s) { return static_cast<Scheduler*>(s)->decode_all_greedy ? 1 : 0; }
// The current step's results in one call: returns the entry count; fills ids / n_new / finished per
// entry and the new tokens flattened in entry order (`tokens` holds at least `cap_tokens`).
BBH_API uint32_t bbh_sched_step_report(void* s, int64_t* ids, uint32_t* n_new, int32_t* finished,
                                       uint32_t cap_entries, uint32_t* tokens, uint32_t cap_tokens) {
  auto* sc = static_cast<Scheduler*>(s);
  const uint32_t n = static_cast<uint32_t>(sc->step_out.size());
  if (!ids) return n;
  uint32_t t = 0;
  for (uint32_t i = 0; i < n && i < cap_entries; ++i) {
    const auto& e = sc->step_out[i];
    ids[i] = e.id;
    n_new[i] = e.n_new;
    finished[i] = e.finished;
    for (uint32_t k = 0; k < e.n_new && t < cap_tokens; ++k) tokens[t++] = sc->step_tokens[e.first + k];
  }
  return n;
}
BBH_API uint32_t bbh_sched_step_tokens(void* s) { return static_cast<uint32_t>(static_cast<Scheduler*>(s)->step_tokens.size()); }
BBH_API void bbh_sched_forget(void* s, int64_t id) { static_cast<Scheduler*>(s)->forget(id); }
BBH_API void bbh_sched_set_service_ms(void* s, double ms) { static_cast<Scheduler*>(s)->mean_service_ms_ = ms; }
BBH_API void bbh_sched_set_prefill_rate(void* s, double tokens_per_ms) {
  static_cast<Scheduler*>(s)->prefill_tokens_per_ms_ = tokens_per_ms;
}
BBH_API uint64_t bbh_sched_pending_prefill(void* s) { return static_cast<Scheduler*>(s)->pending_prefill_tokens(); }
// stats: [free_blocks, num_blocks, waiting, running, steps, submitted, finished, cancelled,
//         generated, prefix_hit_tokens, prefix_lookup_tokens, prefix_entries]
BBH_API void bbh_sched_stats(void* s, uint64_t* out) {
  auto* sc = static_cast<Scheduler*>(s);
  out[0] = sc->alloc().free_blocks();
  out[1] = sc->cfg().num_blocks;
  out[2] = sc->n_waiting();
  out[3] = sc->n_running();
  out[4] = sc->steps_;
  out[5] = sc->submitted_;
  out[6] = sc->finished_;
  out[7] = sc->cancelled_;
  out[8] = sc->generated_;
  out[9] = sc->prefix_hit_tokens_;
  out[10] = sc->prefix_lookup_tokens_;
  out[11] = sc->prefix().size();
}
