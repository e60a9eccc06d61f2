// Byte-level BPE core: merges are applied to one pre-tokenised word at a time by repeatedly
// fusing the adjacent pair with the lowest merge rank (the GPT-2 / Qwen algorithm), with a
// per-tokenizer word cache.  Vocabulary strings are the byte-to-unicode mapped forms, exactly as
// they appear in a HuggingFace tokenizer.json; the Python face does the regex pre-tokenisation and
// the byte mapping.  Reference: crates/data/src/bpe.rs, crates/data/src/qwen_tokenizer.rs.
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

struct PairHash {
  size_t operator()(const std::pair<int32_t, int32_t>& p) const {
    return std::hash<uint64_t>()((static_cast<uint64_t>(static_cast<uint32_t>(p.first)) << 32) |
                                 static_cast<uint32_t>(p.second));
  }
};

struct Bpe {
  std::unordered_map<std::string, int32_t> vocab;                     // mapped token -> id
  std::vector<std::string> itos;
  std::unordered_map<std::pair<int32_t, int32_t>, std::pair<int32_t, int32_t>, PairHash> merges;
  // (left id, right id) -> (rank, merged id)
  std::unordered_map<std::string, std::vector<int32_t>> cache;
};

// split a UTF-8 string into code points (as byte strings)
std::vector<std::string> utf8_chars(const char* s, size_t n) {
  std::vector<std::string> out;
  size_t i = 0;
  while (i < n) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    size_t len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
    if (i + len > n) len = n - i;
    out.emplace_back(s + i, len);
    i += len;
  }
  return out;
}

}  // namespace

BBH_API void* bbh_bpe_new() { return new Bpe(); }
BBH_API void bbh_bpe_free(void* h) { delete static_cast<Bpe*>(h); }
BBH_API void bbh_bpe_add_token(void* h, const char* tok, int32_t len, int32_t id) {
  auto* b = static_cast<Bpe*>(h);
  std::string s(tok, len);
  b->vocab[s] = id;
  if (static_cast<size_t>(id) >= b->itos.size()) b->itos.resize(id + 1);
  b->itos[id] = s;
}
// merge `rank`: left + right (mapped strings); returns 0 or -1 when a piece is not in the vocab
BBH_API int bbh_bpe_add_merge(void* h, const char* l, int32_t ll, const char* r, int32_t rl, int32_t rank) {
  auto* b = static_cast<Bpe*>(h);
  auto il = b->vocab.find(std::string(l, ll));
  auto ir = b->vocab.find(std::string(r, rl));
  auto im = b->vocab.find(std::string(l, ll) + std::string(r, rl));
  if (il == b->vocab.end() || ir == b->vocab.end() || im == b->vocab.end()) return -1;
  b->merges[{il->second, ir->second}] = {rank, im->second};
  return 0;
}
// Encode one pre-tokenised, byte-mapped word.  Returns the number of ids written (<= cap), or -1
// when a character of the word is not in the vocabulary.
BBH_API int32_t bbh_bpe_encode_word(void* h, const char* word, int32_t len, int32_t* out, int32_t cap) {
  auto* b = static_cast<Bpe*>(h);
  std::string key(word, len);
  auto hit = b->cache.find(key);
  if (hit == b->cache.end()) {
    std::vector<int32_t> ids;
    auto whole = b->vocab.find(key);
    if (whole != b->vocab.end()) {
      ids.push_back(whole->second);
    } else {
      for (auto& ch : utf8_chars(word, len)) {
        auto it = b->vocab.find(ch);
        if (it == b->vocab.end()) return -1;
        ids.push_back(it->second);
      }
      while (ids.size() > 1) {
        int32_t best_rank = std::numeric_limits<int32_t>::max(), best_i = -1, merged = 0;
        for (size_t i = 0; i + 1 < ids.size(); ++i) {
          auto m = b->merges.find({ids[i], ids[i + 1]});
          if (m != b->merges.end() && m->second.first < best_rank) {
            best_rank = m->second.first;
            best_i = static_cast<int32_t>(i);
            merged = m->second.second;
          }
        }
        if (best_i < 0) break;
        ids[best_i] = merged;
        ids.erase(ids.begin() + best_i + 1);
      }
    }
    if (b->cache.size() < (1u << 20)) hit = b->cache.emplace(key, std::move(ids)).first;
    else {
      const int32_t n = static_cast<int32_t>(ids.size());
      if (n > cap) return -2;
      std::memcpy(out, ids.data(), n * sizeof(int32_t));
      return n;
    }
  }
  const auto& ids = hit->second;
  const int32_t n = static_cast<int32_t>(ids.size());
  if (n > cap) return -2;
  std::memcpy(out, ids.data(), n * sizeof(int32_t));
  return n;
}
// Mapped string of a token id; returns its byte length (0 for unknown ids).
BBH_API int32_t bbh_bpe_token(void* h, int32_t id, char* out, int32_t cap) {
  auto* b = static_cast<Bpe*>(h);
  if (id < 0 || static_cast<size_t>(id) >= b->itos.size()) return 0;
  const std::string& s = b->itos[id];
  const int32_t n = static_cast<int32_t>(s.size());
  if (n <= cap) std::memcpy(out, s.data(), n);
  return n;
}
BBH_API int32_t bbh_bpe_vocab_size(void* h) { return static_cast<int32_t>(static_cast<Bpe*>(h)->itos.size()); }
