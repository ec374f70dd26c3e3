// Trellis-coded weights on the host: code book, tile decode, tail-biting Viterbi encoder and the
// Hadamard regularisation around it.  This is the CPU twin of the CUDA decode kernels and the
// quantizer used by the converter (the reference splits this between a Python oracle and a
// native Viterbi: reference tools/reference/trellis_quant.py:69-110, tools/reference/trellis_viterbi.hip).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <thread>
#include <vector>

#include "half_util.hpp"
#include "r4dxb_trellis.h"

namespace r4dxb {

// ---- code book --------------------------------------------------------------------------------
static inline uint32_t ByteSum(uint32_t x) { return (x & 0xFF) + ((x >> 8) & 0xFF) + ((x >> 16) & 0xFF) + (x >> 24); }

uint16_t TrellisCodeF16(uint32_t state) {
  static const float kinv = F16ToFloat(R4DXB_TRELLIS_SCALE_F16), kbias = F16ToFloat(R4DXB_TRELLIS_BIAS_F16);
  const uint32_t bs = ByteSum((state & 0xFFFFu) * R4DXB_TRELLIS_MUL);
  // product and sum are exact in fp32 (22 significant bits), so this is one rounding, like an fp16 FMA
  const float prod = static_cast<float>(1024u + bs) * kinv;
  return FloatToF16(prod + kbias);
}

const float* TrellisCodebookF32() {
  static const std::vector<float> cb = [] {
    std::vector<float> t(1u << 16);
    for (uint32_t s = 0; s < (1u << 16); ++s) t[s] = F16ToFloat(TrellisCodeF16(s));
    return t;
  }();
  return cb.data();
}

// ---- decode -----------------------------------------------------------------------------------
// 16-bit state of position p of one tile ring (8*kb words).
uint32_t TrellisState(const uint32_t* w, int kb, int p) {
  const int R = 256 * kb, nw = 8 * kb;
  int start = (kb * (p + 1) - 16) % R;
  if (start < 0) start += R;
  const int i0 = start >> 5, off = start & 31, i1 = (i0 + 1) % nw;
  const uint64_t both = (static_cast<uint64_t>(w[i0]) << 32) | w[i1];
  return static_cast<uint32_t>(both >> (48 - off)) & 0xFFFFu;
}

// Packed words -> Q [N, K] as fp16 bits (row-major, K contiguous).
void TrellisDecode(const uint32_t* words, int64_t N, int64_t K, int kb, uint16_t* q_out) {
  const int64_t tiles_n = N / 16, tiles_k = K / 16;
  for (int64_t tn = 0; tn < tiles_n; ++tn)
    for (int64_t tk = 0; tk < tiles_k; ++tk) {
      const uint32_t* w = words + TrellisTileWordIndex(K, kb, tn, tk);
      for (int p = 0; p < 256; ++p) {
        const int64_t n = tn * 16 + p / 16, k = tk * 16 + p % 16;
        q_out[n * K + k] = TrellisCodeF16(TrellisState(w, kb, p));
      }
    }
}

// ---- Viterbi ----------------------------------------------------------------------------------
namespace {

struct ViterbiScratch {
  std::vector<float> cost_a, cost_b, m;
  std::vector<uint8_t> bp;   // [256][T] argmin of the bits shifted out
  explicit ViterbiScratch(int kb)
      : cost_a(1u << 16), cost_b(1u << 16), m(size_t(1) << (16 - kb)), bp(size_t(256) << (16 - kb)) {}
};

// One Viterbi pass over 256 values.  overlap < 0: unconstrained ends.  Otherwise state_0 >> kb and
// state_255 & (T-1) are both forced to `overlap` (tail-biting).  Returns the total squared error
// and fills states[256].
float ViterbiPass(const float* w, int kb, int overlap, ViterbiScratch& sc, uint16_t* states) {
  const float* cb = TrellisCodebookF32();
  const int T = 1 << (16 - kb), nh = 1 << kb;
  const float inf = std::numeric_limits<float>::infinity();
  float* prev = sc.cost_a.data();
  float* cur = sc.cost_b.data();
  {
    const float x = w[0];
    for (int s = 0; s < 65536; ++s) {
      const float d = x - cb[s];
      prev[s] = d * d;
    }
    if (overlap >= 0)
      for (int s = 0; s < 65536; ++s)
        if ((s >> kb) != overlap) prev[s] = inf;
  }
  float* m = sc.m.data();
  for (int p = 1; p < 256; ++p) {
    uint8_t* bp = sc.bp.data() + size_t(p) * T;
    // m[t] = min over the kb bits h that fall off the top: predecessor = h * T + t
    for (int t = 0; t < T; ++t) { m[t] = prev[t]; bp[t] = 0; }
    for (int h = 1; h < nh; ++h) {
      const float* row = prev + size_t(h) * T;
      for (int t = 0; t < T; ++t) {
        const bool lt = row[t] < m[t];
        m[t] = lt ? row[t] : m[t];
        bp[t] = lt ? static_cast<uint8_t>(h) : bp[t];
      }
    }
    const float x = w[p];
    for (int t = 0; t < T; ++t) {
      const float base = m[t];
      const int s0 = t << kb;
      for (int b = 0; b < nh; ++b) {
        const float d = x - cb[s0 + b];
        cur[s0 + b] = base + d * d;
      }
    }
    std::swap(prev, cur);
  }
  // best end state
  int best = 0;
  float best_cost = inf;
  if (overlap >= 0) {
    for (int h = 0; h < nh; ++h) {
      const int s = h * T + overlap;
      if (prev[s] < best_cost) { best_cost = prev[s]; best = s; }
    }
  } else {
    for (int s = 0; s < 65536; ++s)
      if (prev[s] < best_cost) { best_cost = prev[s]; best = s; }
  }
  int s = best;
  for (int p = 255; p >= 1; --p) {
    states[p] = static_cast<uint16_t>(s);
    const int t = s >> kb;
    s = (static_cast<int>(sc.bp[size_t(p) * T + t]) << (16 - kb)) | t;
  }
  states[0] = static_cast<uint16_t>(s);
  return best_cost;
}

void StatesToRing(const uint16_t* states, int kb, uint32_t* words) {
  const int nw = 8 * kb;
  for (int i = 0; i < nw; ++i) words[i] = 0;
  for (int p = 0; p < 256; ++p) {
    const uint32_t bits = states[p] & ((1u << kb) - 1u);
    for (int b = 0; b < kb; ++b) {
      const int pos = kb * p + b;                 // stream bit index, MSB first inside the kb group
      const uint32_t bit = (bits >> (kb - 1 - b)) & 1u;
      words[pos >> 5] |= bit << (31 - (pos & 31));
    }
  }
}

}  // namespace

// Encodes 256 values (position order) into a tail-biting ring; returns the squared error.  With ``q_out`` the decoded
// value of every position (what the kernels will read back) is returned too.
float TrellisEncodeTile(const float* w, int kb, uint32_t* words, ViterbiScratch& sc, float* q_out) {
  uint16_t states[256];
  float rot[256];
  for (int i = 0; i < 256; ++i) rot[i] = w[(i + 128) & 255];
  ViterbiPass(rot, kb, -1, sc, states);
  // rotated position 127 is original position 255: its low bits are the ring's wrap-around overlap
  const int overlap = states[127] & ((1 << (16 - kb)) - 1);
  const float err = ViterbiPass(w, kb, overlap, sc, states);
  StatesToRing(states, kb, words);
  if (q_out)
    for (int p = 0; p < 256; ++p) q_out[p] = F16ToFloat(TrellisCodeF16(states[p]));
  return err;
}

float TrellisEncodeTile(const float* w, int kb, uint32_t* words, ViterbiScratch& sc) {
  return TrellisEncodeTile(w, kb, words, sc, nullptr);
}

// ---- Hadamard ---------------------------------------------------------------------------------
static void Fwht128(float* v, int stride) {
  for (int h = 1; h < 128; h <<= 1)
    for (int i = 0; i < 128; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const float a = v[size_t(j) * stride], b = v[size_t(j + h) * stride];
        v[size_t(j) * stride] = a + b;
        v[size_t(j + h) * stride] = a - b;
      }
}

static uint64_t SplitMix(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <class F>
static void ParallelFor(int64_t n, int threads, F fn) {
  threads = std::max(1, std::min<int>(threads, static_cast<int>(n)));
  if (threads == 1) { for (int64_t i = 0; i < n; ++i) fn(i, 0); return; }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&, t] {
      for (;;) {
        const int64_t i = next.fetch_add(1);
        if (i >= n) break;
        fn(i, t);
      }
    });
  for (auto& th : pool) th.join();
}

// Quantizes W [N, K] (fp32, row-major) to the trellis layout.
//   suh_out [K], svh_out [N]: fp16 bits.  words_out: TrellisPackedWords(N, K, kb).
// Regularisation: D = H_N diag(1/svh) W diag(1/suh) H_K with random signs in suh/svh (seeded), the
// per-input-channel RMS folded into suh and the global RMS of the rotated matrix into svh, so D is
// close to unit-variance Gaussian, which is what the code book covers.
// Returns the relative squared error ||Q - D||^2 / ||D||^2.
// Regularisation shared by the plain and the error-compensated quantizer: fills D [N, K] with the rotated, unit-variance
// matrix, su [K] / sv [N] with the signed scales (su already rounded through fp16) and writes suh / svh.
static void TrellisRegularize(const float* W, int64_t N, int64_t K, uint64_t seed, int threads, std::vector<float>& D,
                              std::vector<float>& su, std::vector<float>& sv, uint16_t* suh_out, uint16_t* svh_out) {
  D.resize(static_cast<size_t>(N) * K);
  su.resize(K);
  sv.resize(N);
  uint64_t rng = seed * 0x2545F4914F6CDD1Dull + 0x1234567ull;
  // per-input-channel scale
  for (int64_t k = 0; k < K; ++k) {
    double ss = 0;
    for (int64_t n = 0; n < N; ++n) ss += double(W[n * K + k]) * W[n * K + k];
    su[k] = static_cast<float>(std::sqrt(ss / N));
  }
  double mean_su = 0;
  for (int64_t k = 0; k < K; ++k) mean_su += su[k];
  mean_su = mean_su / K;
  for (int64_t k = 0; k < K; ++k) {
    float s = (mean_su > 0 && su[k] > 0) ? static_cast<float>(su[k] / mean_su) : 1.0f;
    s = std::min(std::max(s, 1.0f / 16), 16.0f);
    if (SplitMix(rng) & 1) s = -s;
    su[k] = F16ToFloat(FloatToF16(s));
  }
  for (int64_t n = 0; n < N; ++n) sv[n] = (SplitMix(rng) & 1) ? -1.0f : 1.0f;
  const float inv_sqrt = 1.0f / std::sqrt(128.0f);
  // rows: divide by suh, Hadamard along K
  ParallelFor(N, threads, [&](int64_t n, int) {
    float* row = D.data() + n * K;
    for (int64_t k = 0; k < K; ++k) row[k] = W[n * K + k] / su[k] * sv[n];
    for (int64_t b = 0; b < K; b += 128) {
      Fwht128(row + b, 1);
      for (int i = 0; i < 128; ++i) row[b + i] *= inv_sqrt;
    }
  });
  // columns: Hadamard along N
  ParallelFor(N / 128, threads, [&](int64_t nb, int) {
    for (int64_t k = 0; k < K; ++k) {
      float* col = D.data() + nb * 128 * K + k;
      Fwht128(col, static_cast<int>(K));
      for (int i = 0; i < 128; ++i) col[size_t(i) * K] *= inv_sqrt;
    }
  });
  double ss = 0;
  for (size_t i = 0; i < D.size(); ++i) ss += double(D[i]) * D[i];
  const float sigma = static_cast<float>(std::sqrt(ss / D.size()));
  const float sigma_h = F16ToFloat(FloatToF16(sigma > 0 ? sigma : 1.0f));
  for (int64_t n = 0; n < N; ++n) svh_out[n] = FloatToF16(sv[n] * sigma_h);
  for (int64_t k = 0; k < K; ++k) suh_out[k] = FloatToF16(su[k]);
  const float inv_sigma = 1.0f / sigma_h;
  for (size_t i = 0; i < D.size(); ++i) D[i] *= inv_sigma;
}

double TrellisQuantize(const float* W, int64_t N, int64_t K, int kb, uint64_t seed, int threads,
                       uint32_t* words_out, uint16_t* suh_out, uint16_t* svh_out) {
  std::vector<float> D, su, sv;
  TrellisRegularize(W, N, K, seed, threads, D, su, sv, suh_out, svh_out);
  const int64_t tiles_k = K / 16, tiles = (N / 16) * tiles_k;
  std::vector<std::unique_ptr<ViterbiScratch>> scratch;
  const int nthreads = std::max(1, threads);
  for (int t = 0; t < nthreads; ++t) scratch.emplace_back(new ViterbiScratch(kb));
  std::vector<double> err(nthreads, 0.0);
  ParallelFor(tiles, nthreads, [&](int64_t ti, int tid) {
    const int64_t tn = ti / tiles_k, tk = ti % tiles_k;
    float vals[256];
    for (int p = 0; p < 256; ++p) vals[p] = D[(tn * 16 + p / 16) * K + tk * 16 + p % 16];
    err[tid] += TrellisEncodeTile(vals, kb, words_out + TrellisTileWordIndex(K, kb, tn, tk), *scratch[tid]);
  });
  double e = 0;
  for (double v : err) e += v;
  return e / double(D.size());   // D / sigma has unit mean square
}

// Error-compensated quantization (block LDLQ, the trellis counterpart of GPTQ; reference: the converter's --ldlq mode,
// src/convert/main.cpp:1-30, and the oracle's block-LDL step, tools/reference/trellis_quant.py:1-110).
//
// The code matrix Q multiplies x' = H_K (suh * x), so the layer's proxy loss tr((D - Q) H' (D - Q)^T) uses the Hessian
// in that basis, H' = H_K diag(suh) Hess diag(suh) H_K (damped by `damp` x its mean diagonal).  With the block LDL
// factorisation H' = L B L^T (L unit lower triangular in 16-column blocks, from a blocked Cholesky), the tile columns are
// encoded from the last to the first and each one first absorbs the error already made to its right:
//     target[:, k] = D[:, k] + sum_{j > k} (D[:, j] - Q[:, j]) L[j, k]
// Every target tile goes through the same Viterbi search as the plain quantizer; row tiles of one tile column are
// independent and run on the thread pool.  Work is K^3 / 3 for the factorisation plus N K^2 / 2 for the feedback.
// Results do not depend on the thread count (each output element is produced by one thread in a fixed order).
// Returns the relative squared error of Q against D; *proxy_out = tr(E H' E^T) / tr(D H' D^T).
double TrellisQuantizeLdlq(const float* W, const float* Hess, int64_t N, int64_t K, int kb, uint64_t seed, int threads,
                           float damp, uint32_t* words_out, uint16_t* suh_out, uint16_t* svh_out, double* proxy_out) {
  std::vector<float> D, su, sv;
  TrellisRegularize(W, N, K, seed, threads, D, su, sv, suh_out, svh_out);
  const float inv_sqrt = 1.0f / std::sqrt(128.0f);
  // H' = R Hess R^T, R = H_K diag(su)
  std::vector<float> Hr(static_cast<size_t>(K) * K);
  ParallelFor(K, threads, [&](int64_t i, int) {
    float* row = Hr.data() + i * K;
    for (int64_t j = 0; j < K; ++j) row[j] = Hess[i * K + j] * su[i] * su[j];
    for (int64_t b = 0; b < K; b += 128) {
      Fwht128(row + b, 1);
      for (int t = 0; t < 128; ++t) row[b + t] *= inv_sqrt;
    }
  });
  ParallelFor(K, threads, [&](int64_t j, int) {
    for (int64_t b = 0; b < K; b += 128) {
      float* col = Hr.data() + b * K + j;
      Fwht128(col, static_cast<int>(K));
      for (int t = 0; t < 128; ++t) col[size_t(t) * K] *= inv_sqrt;
    }
  });
  double mean_diag = 0;
  for (int64_t i = 0; i < K; ++i) mean_diag += Hr[i * K + i];
  mean_diag /= K;
  if (!(mean_diag > 0)) mean_diag = 1.0;
  for (int64_t i = 0; i < K; ++i) Hr[i * K + i] += static_cast<float>(damp * mean_diag);
  std::vector<float> Hkeep;
  if (proxy_out) Hkeep = Hr;                       // the factorisation overwrites Hr's lower triangle
  // blocked right-looking Cholesky on the lower triangle (block 16), then L <- L diag-block^-1 (unit block diagonal)
  constexpr int B = 16;
  const int64_t nb = K / B;
  auto blk = [&](int64_t bi, int64_t bj) { return Hr.data() + bi * B * K + bj * B; };
  for (int64_t j = 0; j < nb; ++j) {
    float* A = blk(j, j);
    for (int c = 0; c < B; ++c) {                  // unblocked Cholesky of the diagonal block
      double d = A[c * K + c];
      for (int t = 0; t < c; ++t) d -= double(A[c * K + t]) * A[c * K + t];
      d = std::sqrt(d > 1e-20 ? d : 1e-20);
      A[c * K + c] = static_cast<float>(d);
      for (int r = c + 1; r < B; ++r) {
        double v = A[r * K + c];
        for (int t = 0; t < c; ++t) v -= double(A[r * K + t]) * A[c * K + t];
        A[r * K + c] = static_cast<float>(v / d);
      }
    }
    // panel: A_ij <- A_ij A_jj^-T, then trailing update of block row i: A_ik -= A_ij A_kj^T for j < k <= i
    ParallelFor(nb - j - 1, threads, [&](int64_t ii, int) {
      float* P = blk(j + 1 + ii, j);
      for (int r = 0; r < B; ++r)
        for (int c = 0; c < B; ++c) {
          double v = P[r * K + c];
          for (int t = 0; t < c; ++t) v -= double(P[r * K + t]) * A[c * K + t];
          P[r * K + c] = static_cast<float>(v / A[c * K + c]);
        }
    });
    ParallelFor(nb - j - 1, threads, [&](int64_t ii, int) {
      const int64_t i = j + 1 + ii;
      const float* Pi = blk(i, j);
      for (int64_t k = j + 1; k <= i; ++k) {
        const float* Pk = blk(k, j);
        float* T = blk(i, k);
        for (int r = 0; r < B; ++r)
          for (int c = 0; c < B; ++c) {
            float acc = 0.f;
            for (int t = 0; t < B; ++t) acc += Pi[r * K + t] * Pk[c * K + t];
            T[r * K + c] -= acc;
          }
      }
    });
  }
  ParallelFor(nb, threads, [&](int64_t j, int) {    // column block j: X A_jj = L_ij  (A_jj lower triangular)
    const float* A = blk(j, j);
    for (int64_t i = j + 1; i < nb; ++i) {
      float* P = blk(i, j);
      for (int r = 0; r < B; ++r)
        for (int c = B - 1; c >= 0; --c) {
          double v = P[r * K + c];
          for (int t = c + 1; t < B; ++t) v -= double(P[r * K + t]) * A[t * K + c];
          P[r * K + c] = static_cast<float>(v / A[c * K + c]);
        }
    }
  });
  // LDLQ sweep, last tile column first.  E holds D - Q for the columns already encoded.
  std::vector<float> E(static_cast<size_t>(N) * K, 0.f);
  const int nthreads = std::max(1, threads);
  std::vector<std::unique_ptr<ViterbiScratch>> scratch;
  for (int t = 0; t < nthreads; ++t) scratch.emplace_back(new ViterbiScratch(kb));
  std::vector<double> err(nthreads, 0.0);
  for (int64_t tk = nb - 1; tk >= 0; --tk) {
    ParallelFor(N / 16, nthreads, [&](int64_t tn, int tid) {
      float vals[256], q[256];
      for (int r = 0; r < 16; ++r) {
        const float* e = E.data() + (tn * 16 + r) * K;
        float acc[16];
        for (int c = 0; c < 16; ++c) acc[c] = 0.f;
        for (int64_t j = (tk + 1) * B; j < K; ++j) {
          const float ev = e[j];
          const float* l = Hr.data() + j * K + tk * B;
          for (int c = 0; c < 16; ++c) acc[c] += ev * l[c];
        }
        for (int c = 0; c < 16; ++c) vals[r * 16 + c] = D[(tn * 16 + r) * K + tk * 16 + c] + acc[c];
      }
      TrellisEncodeTile(vals, kb, words_out + TrellisTileWordIndex(K, kb, tn, tk), *scratch[tid], q);
      for (int r = 0; r < 16; ++r)
        for (int c = 0; c < 16; ++c) {
          const size_t at = (tn * 16 + r) * K + tk * 16 + c;
          const float d = D[at] - q[r * 16 + c];
          E[at] = d;
          err[tid] += double(d) * d;
        }
    });
  }
  if (proxy_out) {
    std::vector<double> num(nthreads, 0.0), den(nthreads, 0.0);
    ParallelFor(N, nthreads, [&](int64_t n, int tid) {
      const float* e = E.data() + n * K;
      const float* d = D.data() + n * K;
      for (int64_t i = 0; i < K; ++i) {
        const float* h = Hkeep.data() + i * K;
        double ae = 0, ad = 0;
        for (int64_t j = 0; j < K; ++j) { ae += double(h[j]) * e[j]; ad += double(h[j]) * d[j]; }
        num[tid] += ae * e[i];
        den[tid] += ad * d[i];
      }
    });
    double a = 0, b = 0;
    for (int t = 0; t < nthreads; ++t) { a += num[t]; b += den[t]; }
    *proxy_out = b > 0 ? a / b : 0.0;
  }
  double e = 0;
  for (double v : err) e += v;
  return e / double(D.size());
}

// Dequantizes to the effective dense weight W_eff [N, K] fp32 = diag(svh) H_N Q H_K diag(suh).
void TrellisReconstruct(const uint32_t* words, const uint16_t* suh, const uint16_t* svh, int64_t N, int64_t K,
                        int kb, int threads, float* W_out) {
  std::vector<uint16_t> q(static_cast<size_t>(N) * K);
  TrellisDecode(words, N, K, kb, q.data());
  const float inv_sqrt = 1.0f / std::sqrt(128.0f);
  ParallelFor(N, threads, [&](int64_t n, int) {
    float* row = W_out + n * K;
    for (int64_t k = 0; k < K; ++k) row[k] = F16ToFloat(q[n * K + k]);
    for (int64_t b = 0; b < K; b += 128) {
      Fwht128(row + b, 1);
      for (int i = 0; i < 128; ++i) row[b + i] *= inv_sqrt * F16ToFloat(suh[b + i]);
    }
  });
  ParallelFor(N / 128, threads, [&](int64_t nb, int) {
    for (int64_t k = 0; k < K; ++k) {
      float* col = W_out + nb * 128 * K + k;
      Fwht128(col, static_cast<int>(K));
      for (int i = 0; i < 128; ++i) col[size_t(i) * K] *= inv_sqrt * F16ToFloat(svh[nb * 128 + i]);
    }
  });
}

// Fills a packed tensor with pseudo-random rings (every bit pattern is a valid code sequence whose
// values are near unit-variance Gaussian): synthetic weights for benchmarks.
void TrellisRandomFill(uint32_t* words, int64_t n_words, uint64_t seed) {
  uint64_t s = seed;
  for (int64_t i = 0; i + 1 < n_words; i += 2) {
    const uint64_t r = SplitMix(s);
    words[i] = static_cast<uint32_t>(r);
    words[i + 1] = static_cast<uint32_t>(r >> 32);
  }
  if (n_words & 1) words[n_words - 1] = static_cast<uint32_t>(SplitMix(s));
}

}  // namespace r4dxb

// ---- C ABI ------------------------------------------------------------------------------------
extern "C" {

uint16_t r4dxb_trellis_code_f16(uint32_t state) { return r4dxb::TrellisCodeF16(state); }

void r4dxb_trellis_decode(const uint32_t* words, int64_t N, int64_t K, int kb, uint16_t* q_out) {
  r4dxb::TrellisDecode(words, N, K, kb, q_out);
}

int64_t r4dxb_trellis_packed_words(int64_t N, int64_t K, int kb) { return r4dxb::TrellisPackedWords(N, K, kb); }

double r4dxb_trellis_quantize(const float* W, int64_t N, int64_t K, int kb, uint64_t seed, int threads,
                              uint32_t* words_out, uint16_t* suh_out, uint16_t* svh_out) {
  if (N % 128 || K % 128 || kb < 3 || kb > 5) return -1.0;
  return r4dxb::TrellisQuantize(W, N, K, kb, seed, threads, words_out, suh_out, svh_out);
}

/* Hess: [K, K] fp32 second-moment matrix of the layer's inputs (symmetric).  proxy_out may be null. */
double r4dxb_trellis_quantize_ldlq(const float* W, const float* Hess, int64_t N, int64_t K, int kb, uint64_t seed, int threads,
                                   float damp, uint32_t* words_out, uint16_t* suh_out, uint16_t* svh_out, double* proxy_out) {
  if (N % 128 || K % 128 || kb < 3 || kb > 5 || !(damp >= 0)) return -1.0;
  return r4dxb::TrellisQuantizeLdlq(W, Hess, N, K, kb, seed, threads, damp, words_out, suh_out, svh_out, proxy_out);
}

void r4dxb_trellis_reconstruct(const uint32_t* words, const uint16_t* suh, const uint16_t* svh, int64_t N,
                               int64_t K, int kb, int threads, float* W_out) {
  r4dxb::TrellisReconstruct(words, suh, svh, N, K, kb, threads, W_out);
}

float r4dxb_trellis_encode_tile(const float* vals256, int kb, uint32_t* words_out) {
  r4dxb::ViterbiScratch sc(kb);
  return r4dxb::TrellisEncodeTile(vals256, kb, words_out, sc);
}

void r4dxb_trellis_random_fill(uint32_t* words, int64_t n_words, uint64_t seed) {
  r4dxb::TrellisRandomFill(words, n_words, seed);
}

}  // extern "C"
