// Byte-pair-encoding merge loop of the tokenizer (reference: src/tokenizer/tokenizer.h:1-80).
//
// The vocabulary lives on the Python side; this file only sees token ids.  A tokenizer hands over its merge table once as
// (left id, right id, merged id) triples in rank order; encoding a piece then starts from the ids of its single symbols and
// repeatedly replaces the adjacent pair of lowest rank (every occurrence, left to right) until no pair of the piece has a
// rank.  Pieces are short (a word), so the loop is a plain scan over a small vector; the table is one hash map.
#include <cstdint>
#include <unordered_map>
#include <utility>
#include <vector>

namespace r4dxb {

struct BpeTable {
  std::unordered_map<uint64_t, std::pair<int32_t, int32_t>> merges;   // (left << 32 | right) -> (rank, merged id)
};

static inline uint64_t PairKey(int32_t a, int32_t b) {
  return (static_cast<uint64_t>(static_cast<uint32_t>(a)) << 32) | static_cast<uint32_t>(b);
}

}  // namespace r4dxb

extern "C" {

void* r4dxb_bpe_new(const int32_t* triples, int64_t n) {
  auto* t = new r4dxb::BpeTable();
  t->merges.reserve(static_cast<size_t>(n) * 2);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t key = r4dxb::PairKey(triples[3 * i], triples[3 * i + 1]);
    if (t->merges.find(key) == t->merges.end()) t->merges.emplace(key, std::make_pair(static_cast<int32_t>(i), triples[3 * i + 2]));
  }
  return t;
}

void r4dxb_bpe_free(void* h) { delete static_cast<r4dxb::BpeTable*>(h); }

/* symbols[n] -> out (room for n ids); returns the number of ids written */
int64_t r4dxb_bpe_encode(const void* h, const int32_t* symbols, int64_t n, int32_t* out) {
  const auto& merges = static_cast<const r4dxb::BpeTable*>(h)->merges;
  std::vector<int32_t> cur(symbols, symbols + n), next;
  while (cur.size() > 1) {
    int32_t best_rank = INT32_MAX, best_a = 0, best_b = 0, best_m = 0;
    for (size_t i = 0; i + 1 < cur.size(); ++i) {
      const auto it = merges.find(r4dxb::PairKey(cur[i], cur[i + 1]));
      if (it != merges.end() && it->second.first < best_rank) {
        best_rank = it->second.first;
        best_a = cur[i];
        best_b = cur[i + 1];
        best_m = it->second.second;
      }
    }
    if (best_rank == INT32_MAX) break;
    next.clear();
    for (size_t i = 0; i < cur.size();) {
      if (i + 1 < cur.size() && cur[i] == best_a && cur[i + 1] == best_b) {
        next.push_back(best_m);
        i += 2;
      } else {
        next.push_back(cur[i]);
        i += 1;
      }
    }
    cur.swap(next);
  }
  for (size_t i = 0; i < cur.size(); ++i) out[i] = cur[i];
  return static_cast<int64_t>(cur.size());
}

}  // extern "C"
