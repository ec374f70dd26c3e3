// Hashed n-gram embedding table: row ids on the host and the row reader of the table file.
//
// The table file ("sidecar") is a 4096-byte header followed by `rows` rows of `row_bytes` bytes in row-id order
// (reference: src/model/qwen4exp/include/r4dx/model/qwen4exp/ngram_sidecar.h:8-35 gives the header fields and their
// offsets; ngram_ids.h:8-20 the hash).  Every token owns `heads` rows: the first half hash the 2-gram (token, previous
// token), the second half the 3-gram, each head modulo its own prime plus its own row offset.  History before the most
// recent end-of-sequence token reads as that token.
//
// The B200 design keeps the whole table in device memory when it fits (95 GiB of 180) and computes the ids in the gather
// kernel; this file serves the other two placements (rows read from pinned host memory or from the file) and the tools.
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

extern "C" {

// ids_out [n][heads] int64.  history[2] = the two tokens before tokens[0] (oldest first), updated to the last two tokens fed.
// Returns 0, or 1 when a token is negative or so large that a product would overflow (nothing is written then).
int r4dxb_ngram_ids(const int32_t* tokens, int64_t n, int64_t* history, const int64_t* mult, const uint64_t* primes,
                    const uint64_t* offsets, int heads, int64_t eos, int64_t* ids_out) {
  if (n < 0 || heads < 2 || heads % 2) return 1;
  int64_t max_token = std::numeric_limits<int64_t>::max();
  for (int i = 0; i < 3; ++i) {
    if (mult[i] <= 0) return 1;
    max_token = std::min(max_token, std::numeric_limits<int64_t>::max() / mult[i]);
  }
  for (int64_t i = 0; i < n; ++i)
    if (tokens[i] < 0 || tokens[i] > max_token) return 1;
  if (eos < 0 || eos > max_token) return 1;
  int64_t a = history[0], b = history[1];
  const int half = heads / 2;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t t = tokens[i];
    const int64_t s1 = b;                                   // an end-of-sequence token stands for itself
    const int64_t s2 = (b == eos || a == eos) ? eos : a;    // anything before the most recent one reads as it
    const uint64_t bi = static_cast<uint64_t>(t * mult[0]) ^ static_cast<uint64_t>(s1 * mult[1]);
    const uint64_t tri = bi ^ static_cast<uint64_t>(s2 * mult[2]);
    int64_t* out = ids_out + i * heads;
    for (int h = 0; h < half; ++h) out[h] = static_cast<int64_t>(bi % primes[h] + offsets[h]);
    for (int h = half; h < heads; ++h) out[h] = static_cast<int64_t>(tri % primes[h] + offsets[h]);
    a = b;
    b = t;
  }
  history[0] = a;
  history[1] = b;
  return 0;
}

// Reads `count` rows (ids[i] -> dst + i * row_bytes) from an open table file with positioned reads spread over
// `threads` threads.  Returns 0, or 1 + the index of the first row that could not be read in full (a short or failed read
// never leaves a silent zero row: the caller fails the request).
int64_t r4dxb_ngram_read_rows(int fd, const int64_t* ids, int64_t count, int64_t total_rows, int row_bytes, int64_t header_bytes,
                              void* dst, int threads) {
  if (count <= 0) return 0;
  std::atomic<int64_t> next{0}, bad{-1};
  auto work = [&]() {
    for (;;) {
      const int64_t i = next.fetch_add(1);
      if (i >= count) return;
      int64_t got = 0;
      if (ids[i] >= 0 && ids[i] < total_rows) {
        char* out = static_cast<char*>(dst) + i * row_bytes;
        const off_t at = static_cast<off_t>(header_bytes + ids[i] * row_bytes);
        while (got < row_bytes) {
          const ssize_t r = pread(fd, out + got, static_cast<size_t>(row_bytes - got), at + got);
          if (r <= 0) break;
          got += r;
        }
      }
      if (got != row_bytes) {
        int64_t seen = bad.load();
        while ((seen < 0 || i < seen) && !bad.compare_exchange_weak(seen, i)) {
        }
      }
    }
  };
  const int nt = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(threads, count)));
  if (nt == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& t : pool) t.join();
  }
  return bad.load() < 0 ? 0 : 1 + bad.load();
}

// The same for a file opened with O_DIRECT (rows never pass through, or evict, the page cache: the full table is 95 GiB and is
// read ~16 rows per token).  Direct reads need sector-aligned offsets, sizes and buffers, so each row is fetched as the
// aligned span that contains it (one or two 4 KiB sectors for a 320-byte row) into a per-thread aligned buffer.
int64_t r4dxb_ngram_read_rows_direct(int fd, const int64_t* ids, int64_t count, int64_t total_rows, int row_bytes,
                                     int64_t header_bytes, int64_t file_bytes, void* dst, int threads) {
  if (count <= 0) return 0;
  constexpr int64_t kSector = 4096;
  std::atomic<int64_t> next{0}, bad{-1};
  auto work = [&]() {
    void* raw = nullptr;
    const int64_t cap = ((row_bytes + kSector - 1) / kSector + 1) * kSector;
    if (posix_memalign(&raw, kSector, static_cast<size_t>(cap)) != 0) raw = nullptr;
    for (;;) {
      const int64_t i = next.fetch_add(1);
      if (i >= count) break;
      bool ok = false;
      if (raw != nullptr && ids[i] >= 0 && ids[i] < total_rows) {
        const int64_t at = header_bytes + ids[i] * row_bytes;
        const int64_t lo = at / kSector * kSector;
        const int64_t hi = std::min<int64_t>((at + row_bytes + kSector - 1) / kSector * kSector, (file_bytes + kSector - 1) / kSector * kSector);
        int64_t got = 0;
        while (got < hi - lo) {
          const ssize_t r = pread(fd, static_cast<char*>(raw) + got, static_cast<size_t>(hi - lo - got), static_cast<off_t>(lo + got));
          if (r <= 0) break;                       // (the last sector of the file comes back short: fine if it covers the row)
          got += r;
        }
        if (lo + got >= at + row_bytes) {
          std::memcpy(static_cast<char*>(dst) + i * row_bytes, static_cast<char*>(raw) + (at - lo), static_cast<size_t>(row_bytes));
          ok = true;
        }
      }
      if (!ok) {
        int64_t seen = bad.load();
        while ((seen < 0 || i < seen) && !bad.compare_exchange_weak(seen, i)) {
        }
      }
    }
    free(raw);
  };
  const int nt = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(threads, count)));
  if (nt == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& t : pool) t.join();
  }
  return bad.load() < 0 ? 0 : 1 + bad.load();
}

}  // extern "C"
