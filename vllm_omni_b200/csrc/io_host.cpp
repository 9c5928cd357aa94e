// Host-side I/O and tracing pieces (no CUDA kernels):
//
//  * safetensors reader: the file is memory-mapped, its JSON header is parsed here (a flat object
//    of {name: {dtype, shape, data_offsets}} plus an optional "__metadata__" string map), and byte
//    ranges are copied by a pool of threads into caller-owned (pinned) host buffers, so that the
//    page faults of a cold checkpoint overlap and each rank can pull only its own row slices.
//    The reference loads through the safetensors Python package with one thread per shard
//    (vllm_omni/diffusion/model_loader/diffusers_loader.py:1-280).
//  * NVTX ranges (push / pop / mark) for stage, step and block boundaries.  NVTX v3 is header-only
//    and resolves the tools library at run time, so these are no-ops without a profiler attached.
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define OMNI_HAVE_NVTX 1
#else
#define OMNI_HAVE_NVTX 0
#endif

namespace {

struct TensorInfo {
  std::string name;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;      // byte range inside the data section
};

struct StFile {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t bytes = 0;
  size_t data_off = 0;               // start of the data section
  std::vector<TensorInfo> tensors;
  std::string metadata_json;         // raw text of the "__metadata__" object ("" if absent)
  std::string error;
};

// ---- a JSON reader for exactly the header's shape (objects, arrays, strings, integers)
struct Cursor {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool peek(char c) { ws(); return p < e && *p == c; }
  std::string str() {
    std::string s;
    ws();
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
          case 'u': {                                   // \uXXXX: keep BMP code points as UTF-8
            unsigned v = 0;
            for (int i = 1; i <= 4 && p + i < e; ++i) {
              char c = p[i];
              v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) - 'a' + 10);
            }
            p += 4;
            if (v < 0x80) s += (char)v;
            else if (v < 0x800) { s += (char)(0xC0 | (v >> 6)); s += (char)(0x80 | (v & 0x3F)); }
            else { s += (char)(0xE0 | (v >> 12)); s += (char)(0x80 | ((v >> 6) & 0x3F)); s += (char)(0x80 | (v & 0x3F)); }
            break;
          }
          default: s += *p;
        }
        ++p;
      } else {
        s += *p++;
      }
    }
    if (p >= e) { ok = false; return s; }
    ++p;
    return s;
  }
  int64_t integer() {
    ws();
    bool neg = false;
    if (p < e && *p == '-') { neg = true; ++p; }
    if (p >= e || *p < '0' || *p > '9') { ok = false; return 0; }
    int64_t v = 0;
    while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
    return neg ? -v : v;
  }
  // skips any value; returns its raw text
  std::string skip() {
    ws();
    const char* s = p;
    if (p >= e) { ok = false; return ""; }
    if (*p == '"') { str(); }
    else if (*p == '{' || *p == '[') {
      char open = *p, close = open == '{' ? '}' : ']';
      int depth = 0;
      while (p < e) {
        if (*p == '"') { str(); continue; }
        if (*p == open) ++depth;
        else if (*p == close && --depth == 0) { ++p; break; }
        ++p;
      }
    } else {
      while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
    }
    return std::string(s, p);
  }
};

bool parse_header(StFile& f, const char* js, size_t n) {
  Cursor c{js, js + n};
  if (!c.eat('{')) return false;
  if (c.peek('}')) return true;
  do {
    std::string name = c.str();
    if (!c.ok || !c.eat(':')) return false;
    if (name == "__metadata__") { f.metadata_json = c.skip(); continue; }
    TensorInfo t;
    t.name = name;
    if (!c.eat('{')) return false;
    do {
      std::string k = c.str();
      if (!c.ok || !c.eat(':')) return false;
      if (k == "dtype") t.dtype = c.str();
      else if (k == "shape") {
        if (!c.eat('[')) return false;
        if (!c.peek(']')) do { t.shape.push_back(c.integer()); } while (c.eat(','));
        if (!c.eat(']')) return false;
      } else if (k == "data_offsets") {
        if (!c.eat('[')) return false;
        t.begin = (uint64_t)c.integer();
        if (!c.eat(',')) return false;
        t.end = (uint64_t)c.integer();
        if (!c.eat(']')) return false;
      } else c.skip();
    } while (c.ok && c.eat(','));
    if (!c.ok || !c.eat('}')) return false;
    f.tensors.push_back(std::move(t));
  } while (c.ok && c.eat(','));
  return c.ok && c.eat('}');
}

}  // namespace

extern "C" {

// Opens and validates a safetensors file.  Returns a handle (never null); check omni_st_error().
void* omni_st_open(const char* path) {
  auto* f = new StFile();
  f->fd = ::open(path, O_RDONLY);
  if (f->fd < 0) { f->error = std::string("cannot open ") + path; return f; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) { f->error = "file too small for a safetensors header"; return f; }
  f->bytes = (size_t)st.st_size;
  void* m = mmap(nullptr, f->bytes, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { f->error = "mmap failed"; return f; }
  f->map = static_cast<uint8_t*>(m);
  uint64_t hlen;
  memcpy(&hlen, f->map, 8);
  if (hlen > f->bytes - 8) { f->error = "header length exceeds the file"; return f; }
  f->data_off = 8 + (size_t)hlen;
  if (!parse_header(*f, reinterpret_cast<const char*>(f->map + 8), (size_t)hlen)) { f->error = "malformed header"; return f; }
  for (auto& t : f->tensors)
    if (t.end < t.begin || f->data_off + t.end > f->bytes) { f->error = "tensor " + t.name + " lies outside the file"; break; }
  return f;
}

const char* omni_st_error(void* h) { return static_cast<StFile*>(h)->error.c_str(); }
int omni_st_count(void* h) { return (int)static_cast<StFile*>(h)->tensors.size(); }
const char* omni_st_metadata(void* h) { return static_cast<StFile*>(h)->metadata_json.c_str(); }
const uint8_t* omni_st_data(void* h) { auto* f = static_cast<StFile*>(h); return f->map ? f->map + f->data_off : nullptr; }

// Tensor i: name / dtype are valid until close; shape has up to 8 entries.  Returns ndim, or -1.
int omni_st_info(void* h, int i, const char** name, const char** dtype, int64_t* shape, uint64_t* begin, uint64_t* end) {
  auto* f = static_cast<StFile*>(h);
  if (i < 0 || i >= (int)f->tensors.size()) return -1;
  const TensorInfo& t = f->tensors[i];
  *name = t.name.c_str();
  *dtype = t.dtype.c_str();
  *begin = t.begin;
  *end = t.end;
  int nd = (int)std::min<size_t>(t.shape.size(), 8);
  for (int d = 0; d < nd; ++d) shape[d] = t.shape[d];
  return nd;
}

// Copies n byte ranges [offsets[i], offsets[i] + sizes[i]) of the data section to dst[i] with up to
// `threads` workers; large ranges are cut into 8 MiB pieces so that one big tensor is also spread
// over the pool.  Returns 0, or -1 for a range outside the file.
int omni_st_read(void* h, int n, const uint64_t* offsets, const uint64_t* sizes, void* const* dst, int threads) {
  auto* f = static_cast<StFile*>(h);
  if (!f->map) return -1;
  const size_t data_bytes = f->bytes - f->data_off;
  struct Piece { const uint8_t* s; uint8_t* d; size_t n; };
  std::vector<Piece> pieces;
  const size_t kPiece = 8u << 20;
  for (int i = 0; i < n; ++i) {
    if (offsets[i] + sizes[i] > data_bytes) return -1;
    const uint8_t* s = f->map + f->data_off + offsets[i];
    uint8_t* d = static_cast<uint8_t*>(dst[i]);
    for (size_t o = 0; o < sizes[i]; o += kPiece) pieces.push_back({s + o, d + o, std::min(kPiece, (size_t)sizes[i] - o)});
  }
  int nt = std::max(1, std::min<int>(threads, (int)pieces.size()));
  std::atomic<size_t> next{0};
  auto work = [&]() {
    for (size_t k = next.fetch_add(1); k < pieces.size(); k = next.fetch_add(1)) memcpy(pieces[k].d, pieces[k].s, pieces[k].n);
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < nt; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  return 0;
}

void omni_st_close(void* h) {
  auto* f = static_cast<StFile*>(h);
  if (f->map) munmap(f->map, f->bytes);
  if (f->fd >= 0) ::close(f->fd);
  delete f;
}

// ---- NVTX ranges
int omni_nvtx_available() { return OMNI_HAVE_NVTX; }
void omni_nvtx_push(const char* name) {
#if OMNI_HAVE_NVTX
  nvtxRangePushA(name);
#else
  (void)name;
#endif
}
void omni_nvtx_pop() {
#if OMNI_HAVE_NVTX
  nvtxRangePop();
#endif
}
void omni_nvtx_mark(const char* name) {
#if OMNI_HAVE_NVTX
  nvtxMarkA(name);
#else
  (void)name;
#endif
}

}  // extern "C"
