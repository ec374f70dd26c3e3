// Canonical token sampler on the host, plus the exact "row summary" sampler and the HF repetition
// penalty.
//
// One definition of "the sampled token" (reference semantics: docs/sampling.md:33-62,
// src/kernels/include/r4dx/kernels/sampler.hpp, summary_sampler.hpp):
//   * candidates are ordered by RAW logit descending, ties toward the lower token id (a strict
//     total order that does not depend on the temperature);
//   * filters in order: temperature (division) -> top_k -> min_p (against the untruncated maximum
//     probability) -> top_p (shortest canonical prefix whose mass reaches top_p x the surviving mass);
//   * the token is the first one whose cumulative mass exceeds u x (kept mass), accumulated in double;
//   * one 64-bit Mersenne-twister draw per emitted token.
// The summary path sees only the top-K raw logits + ids and the log-sum-exp of the scaled row (what
// the device kernel returns) and either returns exactly the token the full-row path would return
// or reports that it cannot prove it (-1), in which case the caller falls back to the full row.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <random>
#include <vector>

namespace r4dxb {

struct SampleParams {
  float temperature;
  int top_k;
  float top_p;
  float min_p;
};

struct Order {
  const float* l;
  bool operator()(int32_t a, int32_t b) const { return l[a] > l[b] || (l[a] == l[b] && a < b); }
};

static int32_t ArgmaxLowest(const float* l, int64_t n) {
  int64_t best = 0;
  for (int64_t i = 1; i < n; ++i)
    if (l[i] > l[best]) best = i;
  return static_cast<int32_t>(best);
}

// Walks a canonical prefix.  probs[i] = probability of the i-th canonical candidate (relative to the
// FULL row), n = entries known, `complete` = the prefix is the whole vocabulary.  tail_mass = 1 - sum
// of the whole row beyond the prefix (known exactly only through lse; here passed as 1 - sum(probs)
// clipped at 0).  Returns the index into the prefix, or -1 when the answer depends on unknown entries.
static int WalkPrefix(const double* probs, int n, bool complete, const SampleParams& sp, double u) {
  if (n <= 0) return -1;
  const double pmax = probs[0];
  // length allowed by top_k
  int limit = n;
  bool limit_known = complete;
  if (sp.top_k > 0) {
    if (sp.top_k <= n) { limit = sp.top_k; limit_known = true; }
  }
  // min_p: keep p >= min_p * pmax; the canonical order is non-increasing in p
  if (sp.min_p > 0.f) {
    const double thr = static_cast<double>(sp.min_p) * pmax;
    int k = 0;
    while (k < limit && probs[k] >= thr) ++k;
    if (k < limit) { limit = k; limit_known = true; }   // boundary found inside the known prefix
    if (limit < 1) limit = 1;
  }
  // surviving mass before top_p
  double mass = 0.0;
  for (int i = 0; i < limit; ++i) mass += probs[i];
  if (!limit_known) {
    // the surviving set extends beyond what we can see: its mass is only known when no filter cuts
    // it (then it is the whole row, mass 1)
    if (sp.top_k > 0 || sp.min_p > 0.f) return -1;
    mass = 1.0;
  }
  // top_p: shortest prefix reaching top_p * mass
  int keep = limit;
  bool keep_known = limit_known;
  if (sp.top_p < 1.0f) {
    const double need = static_cast<double>(sp.top_p) * mass;
    double cum = 0.0;
    int k = 0;
    while (k < limit) {
      cum += probs[k];
      ++k;
      if (cum >= need) break;
    }
    if (cum >= need) { keep = k; keep_known = true; }
    else if (!limit_known) return -1;
  }
  double kept = 0.0;
  if (keep_known) {
    for (int i = 0; i < keep; ++i) kept += probs[i];
  } else {
    kept = 1.0;   // nothing was cut: the whole row
  }
  const double target = u * kept;
  double cum = 0.0;
  const int visible = keep_known ? keep : n;
  for (int i = 0; i < visible; ++i) {
    cum += probs[i];
    if (target < cum) return i;
  }
  if (keep_known) return keep - 1;   // rounding left the target at the very end of the kept set
  return -1;                         // the draw lands beyond the visible prefix
}

int32_t SampleCanonical(const float* logits, int64_t vocab, const SampleParams& sp, double u) {
  if (vocab <= 0) return -1;
  if (sp.temperature <= 0.f) return ArgmaxLowest(logits, vocab);
  const double inv_t = 1.0 / static_cast<double>(sp.temperature);
  float mx = logits[0];
  for (int64_t i = 1; i < vocab; ++i) mx = std::max(mx, logits[i]);
  double Z = 0.0;
  for (int64_t i = 0; i < vocab; ++i) Z += std::exp((static_cast<double>(logits[i]) - mx) * inv_t);
  std::vector<int32_t> idx;
  std::vector<double> probs;
  const Order order{logits};
  for (int64_t m = 64;; m *= 8) {
    const int64_t mm = std::min<int64_t>(m, vocab);
    idx.resize(static_cast<size_t>(vocab));
    std::iota(idx.begin(), idx.end(), 0);
    if (mm < vocab) {
      std::nth_element(idx.begin(), idx.begin() + mm, idx.end(), order);
      idx.resize(static_cast<size_t>(mm));
    }
    std::sort(idx.begin(), idx.end(), order);
    probs.resize(idx.size());
    for (size_t i = 0; i < idx.size(); ++i) probs[i] = std::exp((static_cast<double>(logits[idx[i]]) - mx) * inv_t) / Z;
    const int r = WalkPrefix(probs.data(), static_cast<int>(idx.size()), mm == vocab, sp, u);
    if (r >= 0) return idx[static_cast<size_t>(r)];
    if (mm == vocab) return idx.back();
  }
}

// top_logits / top_ids: K entries in canonical order; lse = log sum exp(logit / temperature) over the row.
int32_t SampleFromSummary(const float* top_logits, const int32_t* top_ids, int K, double lse, const SampleParams& sp, double u) {
  if (K <= 0) return -1;
  if (sp.temperature <= 0.f) return top_ids[0];
  const double inv_t = 1.0 / static_cast<double>(sp.temperature);
  std::vector<double> probs(static_cast<size_t>(K));
  for (int i = 0; i < K; ++i) probs[static_cast<size_t>(i)] = std::exp(static_cast<double>(top_logits[i]) * inv_t - lse);
  const int r = WalkPrefix(probs.data(), K, false, sp, u);
  return r < 0 ? -1 : top_ids[r];
}

// HF rule on the distinct ids already seen: positive logits are divided, negative ones multiplied.
void RepetitionPenalty(float* logits, int64_t vocab, const int32_t* seen, int64_t n_seen, float penalty) {
  if (penalty == 1.0f) return;
  std::vector<int32_t> ids(seen, seen + n_seen);
  std::sort(ids.begin(), ids.end());
  ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
  for (int32_t id : ids) {
    if (id < 0 || id >= vocab) continue;
    float& v = logits[id];
    v = v > 0.f ? v / penalty : v * penalty;
  }
}

struct Rng {
  std::mt19937_64 eng;
  explicit Rng(uint64_t seed) : eng(seed) {}
  double Next() { return static_cast<double>(eng() >> 11) * (1.0 / 9007199254740992.0); }
};

}  // namespace r4dxb

namespace r4dxb {

// Selector-lattice walk of the block drafter (greedy chain).  For block position t = 1 .. rows-1 the candidates are
// the row's top-`cands` tokens with unary scores (their logits); the pairwise term couples a candidate to the token
// chosen at the previous position through two rank-R codebooks and the row's gate:
//   score[b] = unary[t][b] + sum_r succ[cand[t][b]][r] * pred[prev][r] * gate[t][r]
// The chain stops early when the chosen candidate's share of the row's softmax (over the candidates, after the
// pairwise term) drops below p_min; a chain shorter than n_min is discarded (reference: docs/dflash2.md:162-186).
int DflashSelect(const int32_t* cand, const float* unary, const float* gate, const float* succ, const float* pred, int rows,
                 int cands, int rank, int64_t vocab, int32_t anchor, float p_min, int n_min, int32_t* out) {
  int n = 0;
  int32_t prev = anchor;
  std::vector<double> score(cands);
  for (int t = 1; t < rows; ++t) {
    double best = -1e300, mx = -1e300;
    int bi = 0;
    for (int b = 0; b < cands; ++b) {
      const int32_t id = cand[t * cands + b];
      double pair = 0.0;
      if (id >= 0 && id < vocab && prev >= 0 && prev < vocab)
        for (int r = 0; r < rank; ++r)
          pair += static_cast<double>(succ[static_cast<int64_t>(id) * rank + r]) * pred[static_cast<int64_t>(prev) * rank + r] *
                  gate[t * rank + r];
      score[b] = unary[t * cands + b] + pair;
      if (score[b] > best || (score[b] == best && id < cand[t * cands + bi])) { best = score[b]; bi = b; }
      mx = std::max(mx, score[b]);
    }
    double z = 0.0;
    for (int b = 0; b < cands; ++b) z += std::exp(score[b] - mx);
    if (std::exp(best - mx) / z < p_min) break;
    out[n++] = cand[t * cands + bi];
    prev = out[n - 1];
  }
  return n < n_min ? 0 : n;
}

}  // namespace r4dxb

extern "C" {

void* r4dxb_rng_new(uint64_t seed) { return new r4dxb::Rng(seed); }
void r4dxb_rng_free(void* r) { delete static_cast<r4dxb::Rng*>(r); }
double r4dxb_rng_next(void* r) { return static_cast<r4dxb::Rng*>(r)->Next(); }

int32_t r4dxb_sample_canonical(const float* logits, int64_t vocab, float temperature, int top_k, float top_p, float min_p,
                               double u) {
  r4dxb::SampleParams sp{temperature, top_k, top_p, min_p};
  return r4dxb::SampleCanonical(logits, vocab, sp, u);
}

int32_t r4dxb_sample_from_summary(const float* top_logits, const int32_t* top_ids, int K, double lse, float temperature,
                                  int top_k, float top_p, float min_p, double u) {
  r4dxb::SampleParams sp{temperature, top_k, top_p, min_p};
  return r4dxb::SampleFromSummary(top_logits, top_ids, K, lse, sp, u);
}

void r4dxb_repetition_penalty(float* logits, int64_t vocab, const int32_t* seen, int64_t n_seen, float penalty) {
  r4dxb::RepetitionPenalty(logits, vocab, seen, n_seen, penalty);
}

int r4dxb_dflash_select(const int32_t* cand, const float* unary, const float* gate, const float* succ, const float* pred,
                        int rows, int cands, int rank, int64_t vocab, int32_t anchor, float p_min, int n_min, int32_t* out) {
  if (rows < 1 || cands < 1 || rank < 0) return -1;
  return r4dxb::DflashSelect(cand, unary, gate, succ, pred, rows, cands, rank, vocab, anchor, p_min, n_min, out);
}

}  // extern "C"
