// Weight container: a safetensors-compatible shell (8-byte little-endian header length, JSON
// header, raw tensor bytes) with a `__metadata__` object carrying the model config and the
// quantization description (reference format: docs/container-format.md:6-48).  Reader = mmap;
// writer = two-phase (plan every tensor first, then stream the bytes) into `<path>.partial`,
// fsync, rename -- the model is never held in memory twice.
#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace r4dxb {

struct TensorEntry {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;   // relative to the data section
};

// ---- minimal JSON (objects, arrays, strings, integers) for the header ---------------------------
struct JsonCursor {
  const char* p;
  const char* e;
  bool ok = true;
  void Ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool Eat(char c) { Ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string Str() {
    std::string s;
    Ws();
    if (p >= e || *p != '"') { ok = false; return s; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': s += '\n'; break;
          case 't': s += '\t'; break;
          case 'r': s += '\r'; break;
          case 'b': s += '\b'; break;
          case 'f': s += '\f'; break;
          case 'u': {
            unsigned v = 0;
            for (int i = 1; i <= 4 && p + i < e; ++i) {
              const char c = p[i];
              v = v * 16 + (c <= '9' ? c - '0' : (c | 32) - 'a' + 10);
            }
            p += 4;
            if (v < 0x80) s += static_cast<char>(v);
            else if (v < 0x800) { s += static_cast<char>(0xC0 | (v >> 6)); s += static_cast<char>(0x80 | (v & 63)); }
            else { s += static_cast<char>(0xE0 | (v >> 12)); s += static_cast<char>(0x80 | ((v >> 6) & 63)); s += static_cast<char>(0x80 | (v & 63)); }
            break;
          }
          default: s += *p;
        }
        ++p;
      } else {
        s += *p++;
      }
    }
    if (p < e) ++p; else ok = false;
    return s;
  }
  int64_t Int() {
    Ws();
    bool neg = false;
    if (p < e && *p == '-') { neg = true; ++p; }
    int64_t v = 0;
    if (p >= e || *p < '0' || *p > '9') ok = false;
    while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
    return neg ? -v : v;
  }
  // skips any value
  void Skip() {
    Ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { Str(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = (open == '{') ? '}' : ']';
      ++p;
      if (Eat(close)) return;
      do {
        if (open == '{') { Str(); if (!Eat(':')) { ok = false; return; } }
        Skip();
      } while (ok && Eat(','));
      if (!Eat(close)) ok = false;
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

static std::string JsonEscape(const std::string& s) {
  std::string o;
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\t': o += "\\t"; break;
      case '\r': o += "\\r"; break;
      default:
        if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += static_cast<char>(c);
    }
  }
  return o;
}

class ContainerReader {
 public:
  std::string error;
  std::vector<TensorEntry> tensors;
  std::map<std::string, std::string> metadata;
  std::map<std::string, size_t> index;
  const uint8_t* data = nullptr;   // start of the data section
  uint64_t data_size = 0;

  bool Open(const char* path) {
    fd_ = ::open(path, O_RDONLY);
    if (fd_ < 0) { error = std::string("open failed: ") + std::strerror(errno); return false; }
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) { error = "file too small"; return false; }
    size_ = static_cast<uint64_t>(st.st_size);
    map_ = static_cast<uint8_t*>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
    if (map_ == MAP_FAILED) { map_ = nullptr; error = "mmap failed"; return false; }
    uint64_t hlen;
    std::memcpy(&hlen, map_, 8);
    if (hlen > size_ - 8) { error = "header length exceeds file"; return false; }
    JsonCursor c{reinterpret_cast<const char*>(map_ + 8), reinterpret_cast<const char*>(map_ + 8 + hlen)};
    data = map_ + 8 + hlen;
    data_size = size_ - 8 - hlen;
    if (!c.Eat('{')) { error = "header is not an object"; return false; }
    if (!c.Eat('}')) {
      do {
        const std::string key = c.Str();
        if (!c.Eat(':')) { error = "bad header"; return false; }
        if (key == "__metadata__") {
          if (!c.Eat('{')) { error = "bad metadata"; return false; }
          if (!c.Eat('}')) {
            do {
              const std::string k = c.Str();
              if (!c.Eat(':')) { error = "bad metadata"; return false; }
              metadata[k] = c.Str();
            } while (c.ok && c.Eat(','));
            if (!c.Eat('}')) { error = "bad metadata"; return false; }
          }
        } else {
          TensorEntry t;
          t.name = key;
          if (!c.Eat('{')) { error = "bad tensor entry"; return false; }
          do {
            const std::string f = c.Str();
            if (!c.Eat(':')) { error = "bad tensor entry"; return false; }
            if (f == "dtype") t.dtype = c.Str();
            else if (f == "shape") {
              if (!c.Eat('[')) { error = "bad shape"; return false; }
              if (!c.Eat(']')) { do t.shape.push_back(c.Int()); while (c.Eat(',')); if (!c.Eat(']')) { error = "bad shape"; return false; } }
            } else if (f == "data_offsets") {
              if (!c.Eat('[')) { error = "bad offsets"; return false; }
              t.begin = static_cast<uint64_t>(c.Int());
              c.Eat(',');
              t.end = static_cast<uint64_t>(c.Int());
              if (!c.Eat(']')) { error = "bad offsets"; return false; }
            } else c.Skip();
          } while (c.ok && c.Eat(','));
          if (!c.Eat('}')) { error = "bad tensor entry"; return false; }
          if (t.end < t.begin || t.end > data_size) { error = "tensor " + t.name + " out of bounds"; return false; }
          if (t.name.rfind("__pad", 0) != 0) {
            index[t.name] = tensors.size();
            tensors.push_back(std::move(t));
          }
        }
      } while (c.ok && c.Eat(','));
    }
    if (!c.ok) { error = "header parse error"; return false; }
    return true;
  }
  ~ContainerReader() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
  }

 private:
  int fd_ = -1;
  uint8_t* map_ = nullptr;
  uint64_t size_ = 0;
};

class ContainerWriter {
 public:
  std::string error;
  explicit ContainerWriter(const char* path) : path_(path) {}
  void SetMeta(const char* k, const char* v) { meta_[k] = v; }
  // phase 1
  int Plan(const char* name, const char* dtype, const int64_t* shape, int rank, uint64_t nbytes) {
    if (begun_) { error = "Plan after Begin"; return -1; }
    TensorEntry t;
    t.name = name;
    t.dtype = dtype;
    t.shape.assign(shape, shape + rank);
    // every tensor starts on a 256-byte boundary of the data section (TMA / vector-load friendly);
    // the gap is an explicit U8 padding tensor so that the file stays a valid safetensors file
    const uint64_t aligned = (cursor_ + 255) & ~uint64_t(255);
    if (aligned != cursor_) {
      TensorEntry pad;
      pad.name = "__pad" + std::to_string(plan_.size());
      pad.dtype = "U8";
      pad.shape = {static_cast<int64_t>(aligned - cursor_)};
      pad.begin = cursor_;
      pad.end = aligned;
      pad_.push_back(true);
      plan_.push_back(std::move(pad));
    }
    cursor_ = aligned;
    pad_.push_back(false);
    t.begin = cursor_;
    t.end = cursor_ + nbytes;
    cursor_ = t.end;
    plan_.push_back(std::move(t));
    user_index_.push_back(static_cast<int>(plan_.size()) - 1);
    return static_cast<int>(user_index_.size()) - 1;
  }
  // phase 2
  bool Begin() {
    std::string h = "{\"__metadata__\":{";
    bool first = true;
    for (auto& kv : meta_) {
      if (!first) h += ",";
      first = false;
      h += "\"" + JsonEscape(kv.first) + "\":\"" + JsonEscape(kv.second) + "\"";
    }
    h += "}";
    for (auto& t : plan_) {
      h += ",\"" + JsonEscape(t.name) + "\":{\"dtype\":\"" + t.dtype + "\",\"shape\":[";
      for (size_t i = 0; i < t.shape.size(); ++i) h += (i ? "," : "") + std::to_string(t.shape[i]);
      h += "],\"data_offsets\":[" + std::to_string(t.begin) + "," + std::to_string(t.end) + "]}";
    }
    h += "}";
    while ((8 + h.size()) % 256) h += ' ';     // data section starts 256-byte aligned in the file
    partial_ = path_ + ".partial";
    fp_ = std::fopen(partial_.c_str(), "wb");
    if (!fp_) { error = "cannot create " + partial_; return false; }
    const uint64_t hlen = h.size();
    std::fwrite(&hlen, 8, 1, fp_);
    std::fwrite(h.data(), 1, h.size(), fp_);
    written_ = 0;
    next_ = 0;
    begun_ = true;
    return true;
  }
  bool Write(int idx, const void* bytes, uint64_t nbytes) {
    if (!begun_ || idx != next_ || idx >= static_cast<int>(user_index_.size())) { error = "tensors must be written in plan order"; return false; }
    const TensorEntry& t = plan_[user_index_[idx]];
    if (nbytes != t.end - t.begin) { error = "size mismatch for " + t.name; return false; }
    static const char zeros[256] = {0};
    while (written_ < t.begin) {
      const uint64_t n = std::min<uint64_t>(256, t.begin - written_);
      std::fwrite(zeros, 1, n, fp_);
      written_ += n;
    }
    if (std::fwrite(bytes, 1, nbytes, fp_) != nbytes) { error = "short write"; return false; }
    written_ += nbytes;
    ++next_;
    return true;
  }
  bool Finish() {
    if (!begun_ || next_ != static_cast<int>(user_index_.size())) { error = "not every planned tensor was written"; return false; }
    std::fflush(fp_);
    fsync(fileno(fp_));
    std::fclose(fp_);
    fp_ = nullptr;
    if (std::rename(partial_.c_str(), path_.c_str()) != 0) { error = "rename failed"; return false; }
    return true;
  }
  ~ContainerWriter() {
    if (fp_) { std::fclose(fp_); std::remove(partial_.c_str()); }
  }

 private:
  std::string path_, partial_;
  std::map<std::string, std::string> meta_;
  std::vector<TensorEntry> plan_;
  std::vector<bool> pad_;
  std::vector<int> user_index_;
  uint64_t cursor_ = 0, written_ = 0;
  int next_ = 0;
  bool begun_ = false;
  FILE* fp_ = nullptr;
};

}  // namespace r4dxb

extern "C" {

void* r4dxb_container_open(const char* path, char* err, int err_len) {
  auto* r = new r4dxb::ContainerReader();
  if (!r->Open(path)) {
    if (err && err_len > 0) std::snprintf(err, err_len, "%s", r->error.c_str());
    delete r;
    return nullptr;
  }
  return r;
}
void r4dxb_container_close(void* h) { delete static_cast<r4dxb::ContainerReader*>(h); }
int64_t r4dxb_container_count(void* h) { return static_cast<int64_t>(static_cast<r4dxb::ContainerReader*>(h)->tensors.size()); }
const char* r4dxb_container_name(void* h, int64_t i) { return static_cast<r4dxb::ContainerReader*>(h)->tensors[i].name.c_str(); }
const char* r4dxb_container_dtype(void* h, int64_t i) { return static_cast<r4dxb::ContainerReader*>(h)->tensors[i].dtype.c_str(); }
int r4dxb_container_rank(void* h, int64_t i) { return static_cast<int>(static_cast<r4dxb::ContainerReader*>(h)->tensors[i].shape.size()); }
int64_t r4dxb_container_dim(void* h, int64_t i, int d) { return static_cast<r4dxb::ContainerReader*>(h)->tensors[i].shape[d]; }
const void* r4dxb_container_data(void* h, int64_t i) {
  auto* r = static_cast<r4dxb::ContainerReader*>(h);
  return r->data + r->tensors[i].begin;
}
uint64_t r4dxb_container_nbytes(void* h, int64_t i) {
  auto& t = static_cast<r4dxb::ContainerReader*>(h)->tensors[i];
  return t.end - t.begin;
}
int64_t r4dxb_container_find(void* h, const char* name) {
  auto* r = static_cast<r4dxb::ContainerReader*>(h);
  auto it = r->index.find(name);
  return it == r->index.end() ? -1 : static_cast<int64_t>(it->second);
}
int64_t r4dxb_container_meta_count(void* h) { return static_cast<int64_t>(static_cast<r4dxb::ContainerReader*>(h)->metadata.size()); }
const char* r4dxb_container_meta_key(void* h, int64_t i) {
  auto it = static_cast<r4dxb::ContainerReader*>(h)->metadata.begin();
  std::advance(it, i);
  return it->first.c_str();
}
const char* r4dxb_container_meta_get(void* h, const char* key) {
  auto* r = static_cast<r4dxb::ContainerReader*>(h);
  auto it = r->metadata.find(key);
  return it == r->metadata.end() ? nullptr : it->second.c_str();
}

void* r4dxb_writer_new(const char* path) { return new r4dxb::ContainerWriter(path); }
void r4dxb_writer_free(void* w) { delete static_cast<r4dxb::ContainerWriter*>(w); }
void r4dxb_writer_meta(void* w, const char* k, const char* v) { static_cast<r4dxb::ContainerWriter*>(w)->SetMeta(k, v); }
int r4dxb_writer_plan(void* w, const char* name, const char* dtype, const int64_t* shape, int rank, uint64_t nbytes) {
  return static_cast<r4dxb::ContainerWriter*>(w)->Plan(name, dtype, shape, rank, nbytes);
}
int r4dxb_writer_begin(void* w) { return static_cast<r4dxb::ContainerWriter*>(w)->Begin() ? 0 : -1; }
int r4dxb_writer_write(void* w, int idx, const void* bytes, uint64_t nbytes) {
  return static_cast<r4dxb::ContainerWriter*>(w)->Write(idx, bytes, nbytes) ? 0 : -1;
}
int r4dxb_writer_finish(void* w) { return static_cast<r4dxb::ContainerWriter*>(w)->Finish() ? 0 : -1; }
const char* r4dxb_writer_error(void* w) { return static_cast<r4dxb::ContainerWriter*>(w)->error.c_str(); }

}  // extern "C"
