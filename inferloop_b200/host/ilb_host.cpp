// Host runtime of the engine in C++: what runs on the CPU for every model load and every
// step, behind a flat C interface that Python loads with ctypes.
//
//   st_*      the safetensors container: the file is mapped read-only, its header parsed
//             and checked here (header length, JSON, duplicate names, shape x dtype against
//             the byte range, tensors tiling the payload without overlap, gap or trailing
//             bytes); tensors are handed out as (pointer, length) views of the mapping.
//             The reference's checks: crates/model/package/src/storage/safetensors.rs:220-314.
//   pool_*    a page pool: every page free or held by exactly one owner, freeing twice or
//             by a stranger is an error (the reference's block pool with checked leases:
//             crates/engine/state/src/blocks.rs:8-28, :70-82, :208-225).
//   slots_*   one fixed-size state slot per live request
//             (crates/backend/cuda/src/resident/slot_batch.rs:364-403).
//   ledger_*  the cache manager's bookkeeping: page groups with a pool and per-request block
//             tables each, request lengths, slots; pages are taken per step, all groups or
//             none (crates/engine/state/src/logical/reservation.rs:106-158), given back at
//             the end or when a window has passed them.
//   step_*    packs the integer arrays of one step (tokens, positions, sequence of each
//             token, offsets, lengths, slots, wanted rows, block tables) into the pinned
//             staging buffer, each array on a 16-byte boundary.
//
// Every function returns 0 (or a count) on success and a negative code otherwise; the
// message is kept per thread and read with ilb_host_last_error().
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#define ILB_API extern "C" __attribute__((visibility("default")))

namespace {

enum Code : int { kOk = 0, kInvalid = -1, kOutOfPages = -2, kOutOfSlots = -3, kLedger = -4, kFormat = -5, kIo = -6 };

thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

// ------------------------------------------------------------------ JSON (the header of a safetensors file)
struct Json {
  const char* p;
  const char* end;
  std::string err;

  void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
  bool fail_at(const char* what) { if (err.empty()) err = std::string(what) + " at byte " + std::to_string((long long)(p - begin)); return false; }
  const char* begin;

  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += (char)cp;
    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
  }
  bool hex4(uint32_t& v) {
    if (end - p < 4) return fail_at("short \\u escape");
    v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
      else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
      else return fail_at("bad \\u escape");
    }
    return true;
  }
  bool string(std::string& out) {
    ws();
    if (p >= end || *p != '"') return fail_at("expected a string");
    ++p;
    out.clear();
    while (p < end) {
      const unsigned char c = (unsigned char)*p++;
      if (c == '"') return true;
      if (c < 0x20) return fail_at("control character in string");
      if (c != '\\') { out += (char)c; continue; }
      if (p >= end) break;
      const char e = *p++;
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          uint32_t cp = 0;
          if (!hex4(cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00) {            // a surrogate pair
            if (end - p < 6 || p[0] != '\\' || p[1] != 'u') return fail_at("lone surrogate");
            p += 2;
            uint32_t lo = 0;
            if (!hex4(lo)) return false;
            if (lo < 0xDC00 || lo > 0xDFFF) return fail_at("bad surrogate pair");
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
            return fail_at("lone surrogate");
          }
          utf8(out, cp);
          break;
        }
        default: return fail_at("bad escape");
      }
    }
    return fail_at("unterminated string");
  }
  // A non-negative integer that fits 63 bits, nothing else (no sign, fraction or exponent).
  bool uint63(long long& v) {
    ws();
    if (p >= end || *p < '0' || *p > '9') return fail_at("expected a non-negative integer");
    if (*p == '0' && p + 1 < end && p[1] >= '0' && p[1] <= '9') return fail_at("leading zero");
    unsigned long long acc = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (acc > (0x7FFFFFFFFFFFFFFFull - 9) / 10) return fail_at("integer too large");
      acc = acc * 10 + (unsigned)(*p - '0');
      ++p;
    }
    if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail_at("expected an integer");
    v = (long long)acc;
    return true;
  }
  bool literal(const char* word) {
    const size_t n = strlen(word);
    if ((size_t)(end - p) < n || memcmp(p, word, n) != 0) return fail_at("bad literal");
    p += n;
    return true;
  }
  // Any value, skipped; `depth` bounds the nesting.
  bool skip(int depth = 0) {
    if (depth > 64) return fail_at("nesting too deep");
    ws();
    if (p >= end) return fail_at("unexpected end");
    const char c = *p;
    if (c == '"') { std::string s; return string(s); }
    if (c == '{') {
      ++p; ws();
      if (p < end && *p == '}') { ++p; return true; }
      for (;;) {
        std::string k;
        if (!string(k)) return false;
        ws();
        if (p >= end || *p != ':') return fail_at("expected ':'");
        ++p;
        if (!skip(depth + 1)) return false;
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail_at("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p; ws();
      if (p < end && *p == ']') { ++p; return true; }
      for (;;) {
        if (!skip(depth + 1)) return false;
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail_at("expected ',' or ']'");
      }
    }
    if (c == 't') return literal("true");
    if (c == 'f') return literal("false");
    if (c == 'n') return literal("null");
    if (c == '-' || (c >= '0' && c <= '9')) {
      if (c == '-') ++p;
      if (p >= end || *p < '0' || *p > '9') return fail_at("bad number");
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) ++p;
      return true;
    }
    return fail_at("unexpected character");
  }
};

// ------------------------------------------------------------------ safetensors
constexpr long long kMaxHeaderBytes = 16ll << 20;      // storage/safetensors.rs:14

struct StEntry {
  std::string name, dtype;
  std::vector<long long> shape;
  long long begin = 0, end = 0;
};

struct StFile {
  int fd = -1;
  size_t size = 0;
  const uint8_t* map = nullptr;
  long long data_start = 0;
  std::vector<StEntry> entries;
  std::string metadata;                                 // raw JSON of "__metadata__", or empty
  ~StFile() {
    if (map != nullptr && size > 0) munmap(const_cast<uint8_t*>(map), size);
    if (fd >= 0) close(fd);
  }
};

int dtype_width(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

// Well-formed UTF-8 (RFC 3629: no overlong forms, no surrogates, nothing past U+10FFFF); the
// offset of the first byte that is not, or -1.  JSON text is UTF-8 (RFC 8259 section 8.1), and a
// tensor's name reaches the caller as a string.
long long first_bad_utf8(const unsigned char* s, long long n) {
  long long i = 0;
  while (i < n) {
    const unsigned char c = s[i];
    int more;
    uint32_t cp, low;
    if (c < 0x80) { ++i; continue; }
    else if (c >= 0xC2 && c <= 0xDF) { more = 1; cp = c & 0x1F; low = 0x80; }
    else if (c >= 0xE0 && c <= 0xEF) { more = 2; cp = c & 0x0F; low = 0x800; }
    else if (c >= 0xF0 && c <= 0xF4) { more = 3; cp = c & 0x07; low = 0x10000; }
    else return i;
    if (i + more >= n) return i;
    for (int k = 1; k <= more; ++k) {
      if ((s[i + k] & 0xC0) != 0x80) return i;
      cp = (cp << 6) | (s[i + k] & 0x3F);
    }
    if (cp < low || cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) return i;
    i += more + 1;
  }
  return -1;
}

int st_parse(StFile& f, const char* path) {
  if (f.size < 8) return fail(kFormat, "%s: file is shorter than its 8-byte length field", path);
  unsigned long long n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | f.map[i];
  if (n > (unsigned long long)kMaxHeaderBytes) return fail(kFormat, "%s: header of %llu bytes exceeds %lld", path, n, kMaxHeaderBytes);
  if (8 + n > f.size) return fail(kFormat, "%s: header length %llu runs past the end of the file", path, n);
  f.data_start = 8 + (long long)n;
  const long long payload = (long long)f.size - f.data_start;
  const long long bad = first_bad_utf8(f.map + 8, (long long)n);
  if (bad >= 0) return fail(kFormat, "%s: header is not valid UTF-8 at byte %lld", path, bad);
  Json j;
  j.begin = j.p = reinterpret_cast<const char*>(f.map + 8);
  j.end = j.p + n;
  j.ws();
  if (j.p >= j.end || *j.p != '{') return fail(kFormat, "%s: header must be a JSON object", path);
  ++j.p;
  std::unordered_set<std::string> seen;
  j.ws();
  bool first = true;
  if (j.p < j.end && *j.p == '}') { ++j.p; first = false; }
  else {
    for (;;) {
      std::string name;
      if (!j.string(name)) return fail(kFormat, "%s: header is not valid JSON: %s", path, j.err.c_str());
      j.ws();
      if (j.p >= j.end || *j.p != ':') return fail(kFormat, "%s: header is not valid JSON: expected ':' after %s", path, name.c_str());
      ++j.p;
      if (!seen.insert(name).second) return fail(kFormat, "%s: duplicate tensor name '%s' in header", path, name.c_str());
      if (name == "__metadata__") {
        j.ws();
        const char* from = j.p;
        if (!j.skip()) return fail(kFormat, "%s: header is not valid JSON: %s", path, j.err.c_str());
        f.metadata.assign(from, j.p);
      } else {
        StEntry e;
        e.name = name;
        j.ws();
        if (j.p >= j.end || *j.p != '{') return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
        ++j.p;
        bool has_dtype = false, has_shape = false, has_off = false;
        j.ws();
        if (j.p < j.end && *j.p == '}') ++j.p;
        else for (;;) {
          std::string key;
          if (!j.string(key)) return fail(kFormat, "%s: header is not valid JSON: %s", path, j.err.c_str());
          j.ws();
          if (j.p >= j.end || *j.p != ':') return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
          ++j.p;
          if (key == "dtype") {
            if (!j.string(e.dtype)) return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
            has_dtype = true;
          } else if (key == "shape" || key == "data_offsets") {
            std::vector<long long> v;
            j.ws();
            if (j.p >= j.end || *j.p != '[') return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
            ++j.p; j.ws();
            if (j.p < j.end && *j.p == ']') ++j.p;
            else for (;;) {
              long long x;
              if (!j.uint63(x)) return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
              v.push_back(x);
              j.ws();
              if (j.p < j.end && *j.p == ',') { ++j.p; continue; }
              if (j.p < j.end && *j.p == ']') { ++j.p; break; }
              return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
            }
            if (key == "shape") { e.shape = v; has_shape = true; }
            else {
              if (v.size() != 2) return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
              e.begin = v[0]; e.end = v[1]; has_off = true;
            }
          } else if (!j.skip()) {
            return fail(kFormat, "%s: header is not valid JSON: %s", path, j.err.c_str());
          }
          j.ws();
          if (j.p < j.end && *j.p == ',') { ++j.p; continue; }
          if (j.p < j.end && *j.p == '}') { ++j.p; break; }
          return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
        }
        if (!has_dtype || !has_shape || !has_off) return fail(kFormat, "%s: malformed entry for '%s'", path, name.c_str());
        const int width = dtype_width(e.dtype);
        if (width == 0) return fail(kFormat, "%s: %s: unsupported dtype %s", path, name.c_str(), e.dtype.c_str());
        if (e.end < e.begin || e.end > payload)
          return fail(kFormat, "%s: %s: offsets [%lld, %lld) outside payload", path, name.c_str(), e.begin, e.end);
        unsigned long long count = 1, span = 1;     // elements; the same with empty dimensions counted as one (what strides are made of)
        bool over = false;
        for (long long s : e.shape) {
          if (s != 0 && count > 0x7FFFFFFFFFFFFFFFull / (unsigned long long)s) over = true;
          count *= (unsigned long long)s;
          const unsigned long long d = s > 0 ? (unsigned long long)s : 1ull;
          if (span > 0x7FFFFFFFFFFFFFFFull / d) over = true;       // [0, 2^62, 2^62] holds nothing, and no tensor library can stride it
          span *= d;
        }
        if (over || count > 0x7FFFFFFFFFFFFFFFull / (unsigned)width || (long long)(count * width) != e.end - e.begin) {
          std::string shp = "[";
          for (size_t i = 0; i < e.shape.size(); ++i) shp += (i ? ", " : "") + std::to_string(e.shape[i]);
          shp += "]";
          return fail(kFormat, "%s: %s: shape %s of %s needs %llu bytes, entry spans %lld", path, name.c_str(), shp.c_str(),
                      e.dtype.c_str(), over ? 0ull : count * width, e.end - e.begin);
        }
        f.entries.push_back(std::move(e));
      }
      j.ws();
      if (j.p < j.end && *j.p == ',') { ++j.p; continue; }
      if (j.p < j.end && *j.p == '}') { ++j.p; break; }
      return fail(kFormat, "%s: header is not valid JSON: expected ',' or '}'", path);
    }
  }
  (void)first;
  j.ws();
  if (j.p != j.end) return fail(kFormat, "%s: header is not valid JSON: text after the object", path);
  // the tensors tile the payload
  std::vector<const StEntry*> order;
  for (const auto& e : f.entries) order.push_back(&e);
  std::sort(order.begin(), order.end(), [](const StEntry* a, const StEntry* b) {
    return a->begin != b->begin ? a->begin < b->begin : a->end < b->end;
  });
  long long cursor = 0;
  for (const StEntry* e : order) {
    if (e->begin < cursor) return fail(kFormat, "%s: %s overlaps the tensor before it", path, e->name.c_str());
    if (e->begin > cursor) return fail(kFormat, "%s: gap of %lld bytes before %s", path, e->begin - cursor, e->name.c_str());
    cursor = e->end;
  }
  if (cursor != payload) return fail(kFormat, "%s: %lld trailing bytes after the last tensor", path, payload - cursor);
  return kOk;
}

// ------------------------------------------------------------------ page pool
struct Pool {
  int num_pages;
  std::vector<int> free_;                     // last freed, first reused
  std::vector<long long> owner;               // -1: free
  std::vector<char> ever_used;
  long long allocations = 0, reuses = 0;

  explicit Pool(int n) : num_pages(n), owner((size_t)n, -1), ever_used((size_t)n, 0) {
    free_.reserve((size_t)n);
    for (int p = n - 1; p >= 0; --p) free_.push_back(p);
  }
  int take(long long who, int count, int* out) {
    if (who < 0) return fail(kInvalid, "owner must not be negative");
    if (count < 0) return fail(kInvalid, "negative page count");
    if ((size_t)count > free_.size()) return fail(kOutOfPages, "need %d pages, %zu free of %d", count, free_.size(), num_pages);
    for (int i = 0; i < count; ++i) {
      const int p = free_.back();
      if (owner[(size_t)p] >= 0) return fail(kLedger, "free list held page %d, which %lld owns", p, owner[(size_t)p]);
      free_.pop_back();
      owner[(size_t)p] = who;
      ++allocations;
      if (ever_used[(size_t)p]) ++reuses;
      ever_used[(size_t)p] = 1;
      out[i] = p;
    }
    return count;
  }
  int give_back(long long who, const int* pages, int n) {
    for (int i = 0; i < n; ++i) {
      const int p = pages[i];
      if (p < 0 || p >= num_pages) return fail(kLedger, "page %d is outside the pool of %d", p, num_pages);
      if (owner[(size_t)p] < 0) return fail(kLedger, "page %d freed twice (by %lld)", p, who);
      if (owner[(size_t)p] != who) return fail(kLedger, "page %d belongs to %lld, not %lld", p, owner[(size_t)p], who);
    }
    std::unordered_set<int> once(pages, pages + n);
    if ((int)once.size() != n) return fail(kLedger, "%lld returns a page twice in one call", who);
    // pushed last to first, so that whoever takes these pages next gets them in the order
    // they are given back in: a block table that came back ascending goes out ascending, and
    // the attention kernels fetch a run of pages that follow one another as one box
    for (int i = n - 1; i >= 0; --i) { owner[(size_t)pages[i]] = -1; free_.push_back(pages[i]); }
    return kOk;
  }
  int check() const {
    std::vector<char> is_free((size_t)num_pages, 0);
    for (int p : free_) {
      if (p < 0 || p >= num_pages) return fail(kLedger, "the free list holds page %d, outside the pool", p);
      if (is_free[(size_t)p]) return fail(kLedger, "a page is on the free list twice");
      is_free[(size_t)p] = 1;
    }
    for (int p = 0; p < num_pages; ++p) {
      const bool owned = owner[(size_t)p] >= 0;
      if (owned == (bool)is_free[(size_t)p])
        return fail(kLedger, "page %d is %s", p, owned ? "both owned and free" : "neither owned nor free");
    }
    return kOk;
  }
};

struct Slots {
  int num_slots;
  std::vector<int> free_;
  std::vector<long long> holder;
  std::unordered_map<long long, int> slot_of;

  explicit Slots(int n) : num_slots(n), holder((size_t)n, -1) {
    for (int s = n - 1; s >= 0; --s) free_.push_back(s);
  }
  int take(long long who) {
    if (slot_of.count(who)) return fail(kInvalid, "%lld already holds slot %d", who, slot_of[who]);
    if (free_.empty()) return fail(kOutOfSlots, "all %d state slots are in use", num_slots);
    const int s = free_.back();
    free_.pop_back();
    holder[(size_t)s] = who;
    slot_of[who] = s;
    return s;
  }
  int give_back(long long who) {
    auto it = slot_of.find(who);
    if (it == slot_of.end()) return fail(kInvalid, "%lld holds no slot", who);
    const int s = it->second;
    slot_of.erase(it);
    holder[(size_t)s] = -1;
    free_.push_back(s);
    return s;
  }
  int check() const {
    std::vector<char> is_free((size_t)num_slots, 0);
    for (int s : free_) {
      if (is_free[(size_t)s]) return fail(kLedger, "a slot is on the free list twice");
      is_free[(size_t)s] = 1;
    }
    for (int s = 0; s < num_slots; ++s)
      if ((holder[(size_t)s] >= 0) == (bool)is_free[(size_t)s]) return fail(kLedger, "slot %d is misaccounted", s);
    for (const auto& kv : slot_of)
      if (holder[(size_t)kv.second] != kv.first) return fail(kLedger, "slot %d of %lld is recorded for %lld", kv.second, kv.first, holder[(size_t)kv.second]);
    return kOk;
  }
};

// ------------------------------------------------------------------ ledger
struct Group {
  int window;                                   // keys a token may look back over, or -1 for all
  Pool pool;
  std::unordered_map<long long, std::vector<int>> tables;
  Group(int w, int pages) : window(w), pool(pages) {}
};

struct Ledger {
  int page_size;
  std::vector<Group> groups;
  Slots slots;
  std::unordered_map<long long, long long> length;
  long long begun = 0, released = 0, window_pages_released = 0;

  // Every group has a pool of its own size: a group whose layers read a window of the keys
  // needs fewer pages than one that keeps them all.
  Ledger(int n_groups, const int* windows, const int* num_pages, int page_size_, int max_requests)
      : page_size(page_size_), slots(max_requests) {
    groups.reserve((size_t)n_groups);
    for (int g = 0; g < n_groups; ++g) groups.emplace_back(windows[g], num_pages[g]);
  }
  long long blocks_for(long long tokens) const { return (tokens + page_size - 1) / page_size; }
  // Blocks below this index hold only keys that no present or future token reads.
  long long first_needed_block(const Group& g, long long first_query_pos) const {
    if (g.window < 0) return 0;
    const long long oldest = std::max(0ll, first_query_pos - g.window + 1);
    return oldest / page_size;
  }
  int pages_needed(long long req, long long new_length, int* out) const {
    auto it = length.find(req);
    if (it == length.end()) return fail(kInvalid, "request %lld is not live", req);
    const long long cur = it->second;
    for (size_t gi = 0; gi < groups.size(); ++gi) {
      const Group& g = groups[gi];
      const std::vector<int>& table = g.tables.at(req);
      const long long want = blocks_for(new_length);
      const long long first = std::min<long long>(first_needed_block(g, cur), (long long)table.size());
      long long releasable = 0;
      for (long long b = 0; b < first; ++b) releasable += table[(size_t)b] >= 0;
      out[gi] = (int)(std::max(0ll, want - (long long)table.size()) - releasable);
    }
    return kOk;
  }
  int ensure(long long req, long long new_length) {
    auto it = length.find(req);
    if (it == length.end()) return fail(kInvalid, "request %lld is not live", req);
    const long long cur = it->second;
    if (new_length < cur) return fail(kInvalid, "request %lld cannot shrink from %lld to %lld", req, cur, new_length);
    for (Group& g : groups) {                   // first give back what a window has passed
      std::vector<int>& table = g.tables[req];
      const long long first = std::min<long long>(first_needed_block(g, cur), (long long)table.size());
      std::vector<int> gone;
      for (long long b = 0; b < first; ++b) if (table[(size_t)b] >= 0) gone.push_back(table[(size_t)b]);
      if (!gone.empty()) {
        const int rc = g.pool.give_back(req, gone.data(), (int)gone.size());
        if (rc) return rc;
        for (long long b = 0; b < first; ++b) table[(size_t)b] = -1;
        window_pages_released += (long long)gone.size();
      }
    }
    const long long want = blocks_for(new_length);
    for (size_t gi = 0; gi < groups.size(); ++gi) {
      const Group& g = groups[gi];
      const long long extra = want - (long long)g.tables.at(req).size();
      if (extra > (long long)g.pool.free_.size())
        return fail(kOutOfPages, "request %lld needs %lld more pages in group %zu, %zu free of %d", req, extra, gi,
                    g.pool.free_.size(), g.pool.num_pages);
    }
    for (Group& g : groups) {
      std::vector<int>& table = g.tables[req];
      const long long extra = want - (long long)table.size();
      if (extra > 0) {
        const size_t old = table.size();
        table.resize(old + (size_t)extra);
        const int rc = g.pool.take(req, (int)extra, table.data() + old);
        if (rc < 0) { table.resize(old); return rc; }
      }
    }
    return kOk;
  }
  int commit(long long req, long long new_length) {
    auto it = length.find(req);
    if (it == length.end()) return fail(kInvalid, "request %lld is not live", req);
    const long long want = blocks_for(new_length);
    for (size_t gi = 0; gi < groups.size(); ++gi)
      if ((long long)groups[gi].tables.at(req).size() < want)
        return fail(kLedger, "request %lld commits %lld tokens but holds %zu blocks in group %zu", req, new_length,
                    groups[gi].tables.at(req).size(), gi);
    if (new_length < it->second) return fail(kInvalid, "commit cannot shrink a request");
    it->second = new_length;
    return kOk;
  }
  int begin(long long req) {
    if (length.count(req)) return fail(kInvalid, "request %lld is already live", req);
    const int slot = slots.take(req);
    if (slot < 0) return slot;
    length[req] = 0;
    for (Group& g : groups) g.tables[req] = {};
    ++begun;
    return slot;
  }
  int release(long long req) {
    if (!length.count(req)) return fail(kInvalid, "request %lld is not live", req);
    for (Group& g : groups) {
      std::vector<int> held;
      for (int p : g.tables[req]) if (p >= 0) held.push_back(p);
      const int rc = g.pool.give_back(req, held.data(), (int)held.size());
      if (rc) return rc;
      g.tables.erase(req);
    }
    const int rc = slots.give_back(req);
    if (rc < 0) return rc;
    length.erase(req);
    ++released;
    return kOk;
  }
  int check() const {
    for (size_t gi = 0; gi < groups.size(); ++gi) {
      const Group& g = groups[gi];
      const int rc = g.pool.check();
      if (rc) return rc;
      std::unordered_map<int, long long> seen;
      for (const auto& kv : g.tables)
        for (int p : kv.second) {
          if (p < 0) continue;
          auto it = seen.find(p);
          if (it != seen.end()) return fail(kLedger, "page %d of group %zu is in the tables of %lld and %lld", p, gi, it->second, kv.first);
          seen[p] = kv.first;
          if (p >= g.pool.num_pages || g.pool.owner[(size_t)p] != kv.first)
            return fail(kLedger, "page %d is in the table of %lld but owned by %lld", p, kv.first,
                        p < g.pool.num_pages ? g.pool.owner[(size_t)p] : -1ll);
        }
      const long long held = g.pool.num_pages - (long long)g.pool.free_.size();
      if (held != (long long)seen.size())
        return fail(kLedger, "group %zu: %lld pages held, %zu in tables (a page is lost)", gi, held, seen.size());
    }
    return slots.check();
  }
};

}  // namespace

ILB_API const char* ilb_host_last_error() { return g_error.c_str(); }

// ------------------------------------------------------------------ safetensors, C interface
ILB_API int ilb_st_open(const char* path, void** out) {
  *out = nullptr;
  StFile* f = new StFile();
  f->fd = open(path, O_RDONLY | O_CLOEXEC);
  if (f->fd < 0) { delete f; return fail(kIo, "%s: cannot open", path); }
  struct stat st;
  if (fstat(f->fd, &st) != 0) { delete f; return fail(kIo, "%s: cannot stat", path); }
  f->size = (size_t)st.st_size;
  if (f->size > 0) {
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { f->map = nullptr; delete f; return fail(kIo, "%s: cannot map", path); }
    f->map = static_cast<const uint8_t*>(m);
  }
  const int rc = st_parse(*f, path);
  if (rc) { delete f; return rc; }
  *out = f;
  return kOk;
}
ILB_API int ilb_st_count(void* h) { return (int)static_cast<StFile*>(h)->entries.size(); }
ILB_API int ilb_st_entry(void* h, int i, const char** name, const char** dtype, int* ndim, const long long** shape,
                         long long* begin, long long* end) {
  StFile* f = static_cast<StFile*>(h);
  if (i < 0 || (size_t)i >= f->entries.size()) return fail(kInvalid, "no tensor %d", i);
  const StEntry& e = f->entries[(size_t)i];
  *name = e.name.c_str(); *dtype = e.dtype.c_str(); *ndim = (int)e.shape.size();
  *shape = e.shape.data(); *begin = e.begin; *end = e.end;
  return kOk;
}
ILB_API const void* ilb_st_payload(void* h) { StFile* f = static_cast<StFile*>(h); return f->map ? f->map + f->data_start : nullptr; }
ILB_API long long ilb_st_data_start(void* h) { return static_cast<StFile*>(h)->data_start; }
ILB_API const char* ilb_st_metadata(void* h) { return static_cast<StFile*>(h)->metadata.c_str(); }
ILB_API void ilb_st_close(void* h) { delete static_cast<StFile*>(h); }

// ------------------------------------------------------------------ pool and slots, C interface
ILB_API int ilb_pool_new(int num_pages, void** out) {
  *out = nullptr;
  if (num_pages <= 0) return fail(kInvalid, "a page pool needs at least one page");
  *out = new Pool(num_pages);
  return kOk;
}
ILB_API void ilb_pool_free(void* h) { delete static_cast<Pool*>(h); }
ILB_API int ilb_pool_take(void* h, long long owner, int count, int* out) { return static_cast<Pool*>(h)->take(owner, count, out); }
ILB_API int ilb_pool_give_back(void* h, long long owner, const int* pages, int n) { return static_cast<Pool*>(h)->give_back(owner, pages, n); }
ILB_API int ilb_pool_check(void* h) { return static_cast<Pool*>(h)->check(); }
ILB_API int ilb_pool_num_free(void* h) { return (int)static_cast<Pool*>(h)->free_.size(); }
ILB_API long long ilb_pool_owner_of(void* h, int page) {
  Pool* p = static_cast<Pool*>(h);
  return (page >= 0 && page < p->num_pages) ? p->owner[(size_t)page] : -1;
}
ILB_API void ilb_pool_counters(void* h, long long* out) { Pool* p = static_cast<Pool*>(h); out[0] = p->allocations; out[1] = p->reuses; }

ILB_API int ilb_slots_new(int num_slots, void** out) {
  *out = nullptr;
  if (num_slots <= 0) return fail(kInvalid, "a slot pool needs at least one slot");
  *out = new Slots(num_slots);
  return kOk;
}
ILB_API void ilb_slots_free(void* h) { delete static_cast<Slots*>(h); }
ILB_API int ilb_slots_take(void* h, long long owner) { return static_cast<Slots*>(h)->take(owner); }
ILB_API int ilb_slots_give_back(void* h, long long owner) { return static_cast<Slots*>(h)->give_back(owner); }
ILB_API int ilb_slots_slot_of(void* h, long long owner) {
  Slots* s = static_cast<Slots*>(h);
  auto it = s->slot_of.find(owner);
  return it == s->slot_of.end() ? fail(kInvalid, "%lld holds no slot", owner) : it->second;
}
ILB_API int ilb_slots_num_free(void* h) { return (int)static_cast<Slots*>(h)->free_.size(); }
ILB_API int ilb_slots_check(void* h) { return static_cast<Slots*>(h)->check(); }

// ------------------------------------------------------------------ ledger, C interface
// num_pages: one entry per group.
ILB_API int ilb_ledger_new(int n_groups, const int* windows, const int* num_pages, int page_size, int max_requests, void** out) {
  *out = nullptr;
  if (page_size <= 0) return fail(kInvalid, "page_size must be positive");
  if (n_groups < 0) return fail(kInvalid, "a negative number of page groups");
  for (int g = 0; g < n_groups; ++g)
    if (num_pages[g] <= 0) return fail(kInvalid, "a page pool needs at least one page");
  if (max_requests <= 0) return fail(kInvalid, "a slot pool needs at least one slot");
  *out = new Ledger(n_groups, windows, num_pages, page_size, max_requests);
  return kOk;
}
ILB_API void ilb_ledger_free(void* h) { delete static_cast<Ledger*>(h); }
ILB_API int ilb_ledger_begin(void* h, long long req) { return static_cast<Ledger*>(h)->begin(req); }
ILB_API int ilb_ledger_has(void* h, long long req) { return static_cast<Ledger*>(h)->length.count(req) ? 1 : 0; }
ILB_API long long ilb_ledger_length(void* h, long long req) {
  Ledger* l = static_cast<Ledger*>(h);
  auto it = l->length.find(req);
  return it == l->length.end() ? (long long)fail(kInvalid, "request %lld is not live", req) : it->second;
}
ILB_API int ilb_ledger_slot_of(void* h, long long req) { return ilb_slots_slot_of(&static_cast<Ledger*>(h)->slots, req); }
ILB_API int ilb_ledger_pages_needed(void* h, long long req, long long new_length, int* out) { return static_cast<Ledger*>(h)->pages_needed(req, new_length, out); }
ILB_API int ilb_ledger_ensure(void* h, long long req, long long new_length) { return static_cast<Ledger*>(h)->ensure(req, new_length); }
ILB_API int ilb_ledger_commit(void* h, long long req, long long new_length) { return static_cast<Ledger*>(h)->commit(req, new_length); }
ILB_API int ilb_ledger_release(void* h, long long req) { return static_cast<Ledger*>(h)->release(req); }
ILB_API int ilb_ledger_check(void* h) { return static_cast<Ledger*>(h)->check(); }
ILB_API int ilb_ledger_table_len(void* h, int group, long long req) {
  Ledger* l = static_cast<Ledger*>(h);
  if (group < 0 || (size_t)group >= l->groups.size()) return fail(kInvalid, "no page group %d", group);
  auto it = l->groups[(size_t)group].tables.find(req);
  if (it == l->groups[(size_t)group].tables.end()) return fail(kInvalid, "request %lld is not live", req);
  return (int)it->second.size();
}
ILB_API int ilb_ledger_table(void* h, int group, long long req, int* out, int cap) {
  Ledger* l = static_cast<Ledger*>(h);
  const int n = ilb_ledger_table_len(h, group, req);
  if (n < 0) return n;
  if (n > cap) return fail(kInvalid, "table of %d blocks does not fit %d", n, cap);
  const std::vector<int>& t = l->groups[(size_t)group].tables[req];
  std::copy(t.begin(), t.end(), out);
  return n;
}
ILB_API void* ilb_ledger_pool(void* h, int group) { return &static_cast<Ledger*>(h)->groups[(size_t)group].pool; }
ILB_API void* ilb_ledger_slots(void* h) { return &static_cast<Ledger*>(h)->slots; }
ILB_API void ilb_ledger_stats(void* h, long long* out) {
  Ledger* l = static_cast<Ledger*>(h);
  out[0] = l->begun; out[1] = l->released; out[2] = l->window_pages_released; out[3] = (long long)l->length.size();
}

// ------------------------------------------------------------------ checks before a step changes anything
// req[i] < 0 stands for a request that is not live yet (length 0).  Nothing is changed.
ILB_API int ilb_step_check(void* h, int n, const long long* req, const int* n_tok, const int* tok, const int* n_want,
                           const int* want, long long vocab, long long max_positions) {
  Ledger* l = static_cast<Ledger*>(h);
  if (n <= 0) return fail(kInvalid, "a step needs at least one entry");
  std::unordered_set<long long> seen;
  long long ti = 0, wi = 0;
  for (int i = 0; i < n; ++i) {
    if (req[i] >= 0 && !seen.insert(req[i]).second) return fail(kInvalid, "request #%d appears twice in one step", i);
    if (n_tok[i] <= 0) return fail(kInvalid, "request #%d brings no tokens", i);
    for (int k = 0; k < n_want[i]; ++k) {
      const int w = want[wi + k];
      if (w < 0 || w >= n_tok[i]) return fail(kInvalid, "request #%d: wanted place %d is outside its %d tokens", i, w, n_tok[i]);
    }
    for (int k = 0; k < n_tok[i]; ++k) {
      const int id = tok[ti + k];
      if (id < 0 || id >= vocab) return fail(kInvalid, "request #%d: token %d is outside the vocabulary of %lld", i, id, vocab);
    }
    long long cur = 0;
    if (req[i] >= 0) {
      auto it = l->length.find(req[i]);
      if (it == l->length.end()) return fail(kInvalid, "request #%d is not live", i);
      cur = it->second;
    }
    if (cur + n_tok[i] > max_positions)
      return fail(kInvalid, "request #%d would reach %lld tokens; the model's limit is %lld", i, cur + n_tok[i], max_positions);
    ti += n_tok[i]; wi += n_want[i];
  }
  return kOk;
}

// Whether every group has the pages that these entries would take (1) or not (0).
ILB_API int ilb_step_fits(void* h, int n, const long long* req, const int* n_tok) {
  Ledger* l = static_cast<Ledger*>(h);
  std::vector<long long> need(l->groups.size(), 0);
  std::vector<int> per(l->groups.size() ? l->groups.size() : 1, 0);
  for (int i = 0; i < n; ++i) {
    if (req[i] >= 0) {
      auto it = l->length.find(req[i]);
      if (it == l->length.end()) return fail(kInvalid, "request #%d is not live", i);
      const int rc = l->pages_needed(req[i], it->second + n_tok[i], per.data());
      if (rc) return rc;
      for (size_t g = 0; g < need.size(); ++g) need[g] += per[g];
    } else {
      for (size_t g = 0; g < need.size(); ++g) need[g] += l->blocks_for(n_tok[i]);
    }
  }
  for (size_t g = 0; g < need.size(); ++g)
    if (need[g] > (long long)l->groups[g].pool.free_.size()) return 0;
  return 1;
}

// ------------------------------------------------------------------ the arrays of one step
// Entries i = 0..n-1: request req[i] brings n_tok[i] tokens (tok, concatenated) and wants the
// logits at n_want[i] of them (want, concatenated, indices into its own tokens).  Every
// request must be live and hold the pages that cover its new tokens (ledger_ensure).
// `pad_seqs` one-token dummy sequences follow (token 0, position 0, no pages, slot -1).
// Layout in `out` (int32, every array starting on a multiple of 4 elements):
//   tokens[T] positions[T] seq_of_token[T] cu_q[S+1] kv_len[S] slots[S] logit_rows[R]
//   then one block table [S][max_blocks] per page group, missing entries -1.
// offsets[0..6+n_groups] receive where each array starts; returns the elements used.
ILB_API long long ilb_step_build(void* h, int n, const long long* req, const int* n_tok, const int* tok, const int* n_want,
                                 const int* want, int pad_seqs, int max_blocks, long long vocab, long long max_positions,
                                 int* out, long long cap, long long* offsets) {
  Ledger* l = static_cast<Ledger*>(h);
  if (n <= 0) return fail(kInvalid, "a step needs at least one entry");
  long long T = 0, R = 0;
  std::unordered_set<long long> seen;
  for (int i = 0; i < n; ++i) {
    if (!seen.insert(req[i]).second) return fail(kInvalid, "request #%d appears twice in one step", i);
    if (n_tok[i] <= 0) return fail(kInvalid, "request #%d brings no tokens", i);
    auto it = l->length.find(req[i]);
    if (it == l->length.end()) return fail(kInvalid, "request #%d is not live", i);
    if (it->second + n_tok[i] > max_positions)
      return fail(kInvalid, "request #%d would reach %lld tokens; the model's limit is %lld", i, it->second + n_tok[i], max_positions);
    T += n_tok[i];
    R += n_want[i];
  }
  const long long S = n + pad_seqs;
  T += pad_seqs;
  R += pad_seqs;
  auto pad4 = [](long long x) { return (x + 3) / 4 * 4; };
  const size_t n_groups = l->groups.size();
  long long off = 0;
  const long long sizes[7] = {T, T, T, S + 1, S, S, R};
  for (int a = 0; a < 7; ++a) { offsets[a] = off; off += pad4(sizes[a]); }
  for (size_t g = 0; g < n_groups; ++g) { offsets[7 + g] = off; off += pad4(S * (long long)max_blocks); }
  if (off > cap) return fail(kInvalid, "the step needs %lld staging elements, the buffer holds %lld", off, cap);
  int* tokens = out + offsets[0];
  int* positions = out + offsets[1];
  int* seq_of = out + offsets[2];
  int* cu_q = out + offsets[3];
  int* kv_len = out + offsets[4];
  int* slots = out + offsets[5];
  int* rows = out + offsets[6];
  long long t = 0, r = 0, ti = 0, wi = 0;
  cu_q[0] = 0;
  for (int i = 0; i < n; ++i) {
    const long long cur = l->length[req[i]];
    for (int k = 0; k < n_tok[i]; ++k) {
      const int id = tok[ti + k];
      if (id < 0 || id >= vocab) return fail(kInvalid, "request #%d: token %d is outside the vocabulary of %lld", i, id, vocab);
      tokens[t + k] = id;
      positions[t + k] = (int)(cur + k);
      seq_of[t + k] = i;
    }
    for (int k = 0; k < n_want[i]; ++k) {
      const int w = want[wi + k];
      if (w < 0 || w >= n_tok[i]) return fail(kInvalid, "request #%d: wanted place %d is outside its %d tokens", i, w, n_tok[i]);
      rows[r++] = (int)(t + w);
    }
    cu_q[i + 1] = (int)(t + n_tok[i]);
    kv_len[i] = (int)(cur + n_tok[i]);
    slots[i] = l->slots.slot_of.at(req[i]);
    t += n_tok[i]; ti += n_tok[i]; wi += n_want[i];
  }
  for (long long s = n; s < S; ++s) {           // padding
    tokens[t] = 0; positions[t] = 0; seq_of[t] = (int)s;
    cu_q[s + 1] = (int)(t + 1);
    kv_len[s] = 0; slots[s] = -1;
    rows[r++] = (int)t;
    ++t;
  }
  for (size_t g = 0; g < n_groups; ++g) {
    int* tb = out + offsets[7 + g];
    std::fill(tb, tb + S * (long long)max_blocks, -1);
    for (int i = 0; i < n; ++i) {
      const std::vector<int>& row = l->groups[g].tables.at(req[i]);
      if ((long long)row.size() > max_blocks)
        return fail(kInvalid, "a request holds %zu blocks, the table is %d wide", row.size(), max_blocks);
      std::copy(row.begin(), row.end(), tb + (long long)i * max_blocks);
    }
  }
  return off;
}

// One call for the commonest step: every request live and bringing exactly one token whose
// logits are wanted.  Checks, takes the pages (all or none) and packs the arrays.
ILB_API long long ilb_step_decode(void* h, int n, const long long* req, const int* tok, int pad_seqs, int max_blocks,
                                  long long vocab, long long max_positions, int* out, long long cap, long long* offsets) {
  Ledger* l = static_cast<Ledger*>(h);
  if (n <= 0) return fail(kInvalid, "a step needs at least one entry");
  std::vector<int> ones((size_t)n, 1), zeros((size_t)n, 0);
  int rc = ilb_step_check(h, n, req, ones.data(), tok, ones.data(), zeros.data(), vocab, max_positions);
  if (rc) return rc;
  for (int i = 0; i < n; ++i)
    if (req[i] < 0) return fail(kInvalid, "request #%d is not live", i);
  rc = ilb_step_fits(h, n, req, ones.data());
  if (rc < 0) return rc;
  if (rc == 0) return fail(kOutOfPages, "step of %d tokens does not fit the free pages", n);
  for (int i = 0; i < n; ++i) {
    rc = l->ensure(req[i], l->length[req[i]] + 1);
    if (rc) return rc;
  }
  return ilb_step_build(h, n, req, ones.data(), tok, ones.data(), zeros.data(), pad_seqs, max_blocks, vocab, max_positions,
                        out, cap, offsets);
}

// Every request's committed length grows by its token count (after the step has run).
ILB_API int ilb_step_commit(void* h, int n, const long long* req, const int* n_tok) {
  Ledger* l = static_cast<Ledger*>(h);
  for (int i = 0; i < n; ++i) {
    auto it = l->length.find(req[i]);
    if (it == l->length.end()) return fail(kInvalid, "request #%d is not live", i);
    const int rc = l->commit(req[i], it->second + n_tok[i]);
    if (rc) return rc;
  }
  return kOk;
}

// ------------------------------------------------------------------ the scheduler
// Continuous batching above the step function: each plan() builds ONE step under a token
// budget and a sequence cap.  Decoding requests bring one token each (oldest first; one that
// cannot get its next page preempts the youngest running request that is not yet in the plan,
// by recompute: pages and slot returned, back to the head of the waiting queue); then prompt
// portions of running requests, then new arrivals first come first served.  A portion is
// granted whole if the budget funds it, or the remainder if that is at least half a portion
// (crates/engine/scheduler/src/policy/packing.rs:328-347); what the free pages cannot hold is
// shrunk to what they can.  Requests are known by the ledger's numbers; token values never
// come here, only counts.  Reference: crates/engine/scheduler/src/preemption.rs:59-119,
// crates/engine/runtime/src/pipeline/scheduling/{ready.rs:105-117, preemption.rs:67-76}.
namespace {

constexpr int kCapacity = -7;

struct SReq { long long prompt_len = 0, generated = 0, max_new = 0, arrival = 0; int preemptions = 0; };
struct Work { long long id, start, count; int samples; };

struct Sched {
  Ledger* l;
  long long max_num_seqs, max_batched, chunk, max_model_len;
  long long token_multiple = 1;                // a whole portion beside other work is trimmed so that the step's tokens are a multiple of this
  std::vector<long long> waiting;              // front = index 0
  std::vector<long long> running;              // admission order
  std::unordered_map<long long, SReq> reqs;
  long long arrivals = 0, steps = 0, preemptions = 0, admitted = 0, finished = 0;
  std::vector<Work> work;
  std::vector<long long> preempted;

  long long total_len(long long id) const { const SReq& r = reqs.at(id); return r.prompt_len + r.generated; }
  bool live(long long id) const { return l->length.count(id) != 0; }
  long long computed(long long id) const { auto it = l->length.find(id); return it == l->length.end() ? 0 : it->second; }
  bool is_decode(long long id) const { return computed(id) == total_len(id) - 1; }
  bool planned(long long id) const { for (const Work& w : work) if (w.id == id) return true; return false; }
  void pages_for(long long id, long long new_len, std::vector<long long>& need) const {
    need.assign(l->groups.size(), 0);
    if (live(id)) {
      std::vector<int> per(l->groups.size() ? l->groups.size() : 1, 0);
      l->pages_needed(id, new_len, per.data());
      for (size_t g = 0; g < need.size(); ++g) need[g] = per[g];
    } else {
      for (size_t g = 0; g < need.size(); ++g) need[g] = l->blocks_for(new_len);
    }
  }
  void held(long long id, std::vector<long long>& out) const {
    out.assign(l->groups.size(), 0);
    if (!live(id)) return;
    for (size_t g = 0; g < out.size(); ++g)
      for (int p : l->groups[g].tables.at(id)) out[g] += p >= 0;
  }
  void preempt(long long victim) {
    if (live(victim)) l->release(victim);
    running.erase(std::find(running.begin(), running.end(), victim));
    reqs[victim].preemptions += 1;
    waiting.insert(waiting.begin(), victim);   // it keeps its place ahead of newer arrivals
    preempted.push_back(victim);
    ++preemptions;
  }
  void fill() {
    long long budget = max_batched;
    const size_t G = l->groups.size();
    std::vector<long long> free_(G), need, hold;
    for (size_t g = 0; g < G; ++g) free_[g] = (long long)l->groups[g].pool.free_.size();
    auto fits = [&](const std::vector<long long>& n) { for (size_t g = 0; g < G; ++g) if (n[g] > free_[g]) return false; return true; };
    auto charge = [&](const std::vector<long long>& n) { for (size_t g = 0; g < G; ++g) free_[g] -= n[g]; };
    // 1. decoding requests, oldest first; a blocked one preempts the youngest running
    std::vector<long long> decoders;
    for (long long id : running) if (is_decode(id)) decoders.push_back(id);
    for (long long id : decoders) {
      if (std::find(running.begin(), running.end(), id) == running.end()) continue;   // became a victim meanwhile
      if (budget <= 0 || (long long)work.size() >= max_num_seqs) break;
      pages_for(id, total_len(id), need);
      while (!fits(need)) {
        long long victim = -1;
        for (auto it = running.rbegin(); it != running.rend(); ++it)
          if (*it != id && !planned(*it)) { victim = *it; break; }
        if (victim < 0) break;
        held(victim, hold);
        preempt(victim);
        for (size_t g = 0; g < G; ++g) free_[g] += hold[g];
      }
      if (!fits(need)) continue;               // waits; something else may finish first
      charge(need);
      work.push_back({id, total_len(id) - 1, 1, 1});
      budget -= 1;
    }
    // 2. prompt portions: requests already running, then new arrivals in order
    auto grant = [&](long long id, Work& w) {
      const long long done = computed(id);
      const long long portion = std::min(chunk, total_len(id) - done);
      long long count;
      if (budget >= portion) count = portion;
      else if (budget >= 1 && budget * 2 >= portion) count = budget;
      else return false;
      // The matrix kernels work on tiles of `token_multiple` tokens: a whole portion that
      // rides beside other work (decode tokens, another portion) would push the step a few
      // tokens past a tile edge and cost a whole tile more.  It is trimmed to the edge, as
      // long as at least half a portion stays (the same floor as above); the prompt's tail
      // is never trimmed.
      if (token_multiple > 1 && portion == chunk) {
        const long long used = max_batched - budget;
        const long long edge = (used + count) / token_multiple * token_multiple;
        if (used > 0 && edge < used + count && (edge - used) * 2 >= portion) count = edge - used;
      }
      pages_for(id, done + count, need);
      if (!fits(need)) {
        // take what the free pages can hold, if that is still progress
        long long room = done + count;
        if (G > 0) {
          room = -1;
          for (size_t g = 0; g < G; ++g) {
            const long long have = live(id) ? (long long)l->groups[g].tables.at(id).size() : 0;
            const long long r = (have + free_[g]) * l->page_size;
            room = room < 0 ? r : std::min(room, r);
          }
        }
        count = std::min(count, room - done);
        if (count <= 0) return false;
        pages_for(id, done + count, need);
        if (!fits(need)) return false;
      }
      charge(need);
      budget -= count;
      w = {id, done, count, done + count == total_len(id) ? 1 : 0};
      return true;
    };
    const std::vector<long long> snapshot = running;
    for (long long id : snapshot) {
      if (planned(id) || is_decode(id)) continue;
      if (budget <= 0 || (long long)work.size() >= max_num_seqs) break;
      Work w;
      if (grant(id, w)) work.push_back(w);
    }
    for (;;) {
      if (waiting.empty() || budget <= 0 || (long long)work.size() >= max_num_seqs || (long long)running.size() >= max_num_seqs) break;
      long long fresh = 0;
      for (const Work& w : work) fresh += !live(w.id);
      if ((long long)l->slots.free_.size() <= fresh) break;
      const long long id = waiting.front();
      if (std::find(preempted.begin(), preempted.end(), id) != preempted.end() && !running.empty())
        break;                                  // a victim of this very step waits for the next one
      Work w;
      if (!grant(id, w)) break;                 // first come first served: nobody overtakes the head
      waiting.erase(waiting.begin());
      running.push_back(id);
      ++admitted;
      work.push_back(w);
    }
  }
  int plan() {
    work.clear();
    preempted.clear();
    for (;;) {
      fill();
      if (!work.empty() || running.empty()) break;
      if (running.size() == 1)
        return fail(kCapacity, "request #%lld cannot grow: the cache is too small for it alone", running[0]);
      preempt(running.back());
    }
    if (work.empty() && !waiting.empty() && running.empty())
      return fail(kCapacity, "request #%lld cannot start: the cache is too small for it alone", waiting.front());
    if (!work.empty()) ++steps;
    return kOk;
  }
};

}  // namespace

ILB_API int ilb_sched_new(void* ledger, long long max_num_seqs, long long max_batched, long long chunk, long long max_model_len,
                          void** out) {
  *out = nullptr;
  if (max_num_seqs <= 0 || max_batched <= 0 || chunk <= 0 || max_model_len <= 0) return fail(kInvalid, "scheduler limits must be positive");
  Sched* s = new Sched();
  s->l = static_cast<Ledger*>(ledger);
  s->max_num_seqs = max_num_seqs; s->max_batched = max_batched; s->chunk = chunk; s->max_model_len = max_model_len;
  *out = s;
  return kOk;
}
ILB_API void ilb_sched_free(void* h) { delete static_cast<Sched*>(h); }

// A new request: `id` is the ledger's number for it.  `generated` tokens it already has
// (0 for a fresh one).
ILB_API int ilb_sched_add(void* h, long long id, long long prompt_len, long long max_new) {
  Sched* s = static_cast<Sched*>(h);
  if (max_new <= 0) return fail(kInvalid, "max_new_tokens must be positive");
  if (prompt_len <= 0) return fail(kInvalid, "empty input");
  if (std::find(s->waiting.begin(), s->waiting.end(), id) != s->waiting.end() ||
      std::find(s->running.begin(), s->running.end(), id) != s->running.end())
    return fail(kInvalid, "request #%lld is already queued", id);
  const long long total = prompt_len + max_new;
  if (total > s->max_model_len)
    // reserved tokens = prompt + max_new_tokens must fit the context (crates/engine/workloads/src/native.rs:91-111)
    return fail(kInvalid, "request #%lld: prompt %lld + max_new_tokens %lld exceeds max_model_len %lld", id, prompt_len, max_new,
                s->max_model_len);
  const long long pages = s->l->blocks_for(total);
  for (size_t g = 0; g < s->l->groups.size(); ++g) {
    const Group& grp = s->l->groups[g];
    long long reach = pages;
    if (grp.window >= 0) reach = std::min(pages, s->l->blocks_for(grp.window + s->chunk) + 1);
    if (reach > grp.pool.num_pages)
      return fail(kCapacity, "request #%lld needs %lld pages of group %zu, the pool has %d", id, reach, g, grp.pool.num_pages);
  }
  SReq r;
  r.prompt_len = prompt_len; r.max_new = max_new; r.arrival = s->arrivals++;
  s->reqs[id] = r;
  s->waiting.push_back(id);
  return kOk;
}

// One step.  work receives (id, start, count, samples) per entry, preempted the requests that
// lost their pages (they are waiting again).  Returns 0, or the capacity code when a request
// cannot run even alone.
ILB_API int ilb_sched_plan(void* h, long long* work, int cap, int* n_work, long long* preempted, int* n_preempted) {
  Sched* s = static_cast<Sched*>(h);
  const int rc = s->plan();
  // victims are reported whether or not the plan stands: their pages are gone either way
  *n_preempted = (int)std::min<size_t>(s->preempted.size(), (size_t)cap);
  for (int i = 0; i < *n_preempted; ++i) preempted[i] = s->preempted[(size_t)i];
  *n_work = 0;
  if (rc) return rc;
  if ((int)s->work.size() > cap) return fail(kInvalid, "the plan has %zu entries, room for %d", s->work.size(), cap);
  *n_work = (int)s->work.size();
  for (int i = 0; i < *n_work; ++i) {
    const Work& w = s->work[(size_t)i];
    work[4 * i] = w.id; work[4 * i + 1] = w.start; work[4 * i + 2] = w.count; work[4 * i + 3] = w.samples;
  }
  return kOk;
}

// A token was drawn for a running request (`stop`: it is one of its stop tokens).  Returns
// 0 (goes on), 1 (ended on the stop token) or 2 (ended on a length limit); an ended request's
// pages and slot are released here.
ILB_API int ilb_sched_token(void* h, long long id, int stop) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end() || std::find(s->running.begin(), s->running.end(), id) == s->running.end())
    return fail(kInvalid, "request #%lld is not running", id);
  SReq& r = it->second;
  r.generated += 1;
  int reason = 0;
  if (stop) reason = 1;
  else if (r.generated >= r.max_new) reason = 2;
  else if (r.prompt_len + r.generated >= s->max_model_len) reason = 2;
  if (reason) {
    s->running.erase(std::find(s->running.begin(), s->running.end(), id));
    if (s->live(id)) s->l->release(id);
    s->reqs.erase(it);
    ++s->finished;
  }
  return reason;
}

// Returns 1 if the request was known (running or waiting) and is now gone, 0 otherwise.
ILB_API int ilb_sched_abort(void* h, long long id) {
  Sched* s = static_cast<Sched*>(h);
  auto r = std::find(s->running.begin(), s->running.end(), id);
  if (r != s->running.end()) {
    s->running.erase(r);
    if (s->live(id)) s->l->release(id);
    s->reqs.erase(id);
    return 1;
  }
  auto w = std::find(s->waiting.begin(), s->waiting.end(), id);
  if (w != s->waiting.end()) { s->waiting.erase(w); s->reqs.erase(id); return 1; }
  return 0;
}

// which: 0 waiting, 1 running.  Copies up to cap ids in order; returns how many there are.
ILB_API int ilb_sched_list(void* h, int which, long long* out, int cap) {
  Sched* s = static_cast<Sched*>(h);
  const std::vector<long long>& v = which == 0 ? s->waiting : s->running;
  for (size_t i = 0; i < v.size() && (int)i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}
ILB_API void ilb_sched_stats(void* h, long long* out) {
  Sched* s = static_cast<Sched*>(h);
  out[0] = s->steps; out[1] = s->preemptions; out[2] = s->admitted; out[3] = s->finished;
  out[4] = (long long)s->waiting.size(); out[5] = (long long)s->running.size();
}
ILB_API void ilb_sched_count_step(void* h) { static_cast<Sched*>(h)->steps += 1; }
ILB_API int ilb_sched_preemptions_of(void* h, long long id) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? 0 : it->second.preemptions;
}
ILB_API int ilb_sched_set_token_multiple(void* h, long long multiple) {
  if (multiple <= 0) return fail(kInvalid, "the token multiple must be positive");
  static_cast<Sched*>(h)->token_multiple = multiple;
  return kOk;
}
ILB_API int ilb_sched_set_limits(void* h, long long max_num_seqs, long long max_batched, long long chunk, long long max_model_len) {
  if (max_num_seqs <= 0 || max_batched <= 0 || chunk <= 0 || max_model_len <= 0) return fail(kInvalid, "scheduler limits must be positive");
  Sched* s = static_cast<Sched*>(h);
  s->max_num_seqs = max_num_seqs; s->max_batched = max_batched; s->chunk = chunk; s->max_model_len = max_model_len;
  return kOk;
}
