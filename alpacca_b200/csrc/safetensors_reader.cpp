// Reader of safetensors files: maps the file, parses and checks its table of tensors, and hands
// out the table and the address of the data.  The counterpart in the reference is the GGUF reader
// (alpacca/gguf.py:82-194: mmap, header, tensor table name -> shape, dtype, offset, zero-copy
// tensor_bytes); here it is native code behind a C interface (ctypes on the Python side).
//
// File layout: 8 bytes little-endian header length N, N bytes of JSON
//   { "tensor name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ...,
//     "__metadata__": {"key": "value", ...} }
// then the data section; offsets count from its start.
//
// Everything is checked before the first tensor is read: header length against the file size,
// JSON syntax, known dtypes, offsets inside the data section, byte counts against shapes.
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <utility>
#include <vector>

#define ST_API extern "C" __attribute__((visibility("default")))

namespace {

struct Entry {
  std::string name, dtype;
  std::vector<long long> shape;
  long long begin = 0, end = 0;
};

struct File {
  int fd = -1;
  void* map = nullptr;
  size_t size = 0;
  size_t data_start = 0;
  std::vector<Entry> entries;
  std::vector<std::pair<std::string, std::string>> metadata;
};

int item_size(const std::string& dt) {
  if (dt == "F64" || dt == "I64" || dt == "U64") return 8;
  if (dt == "F32" || dt == "I32" || dt == "U32") return 4;
  if (dt == "F16" || dt == "BF16" || dt == "I16" || dt == "U16") return 2;
  if (dt == "I8" || dt == "U8" || dt == "BOOL") return 1;
  return 0;
}

// A parser for the JSON that such headers hold: objects, arrays, strings, integers.
struct Parser {
  const char* p;
  const char* end;
  std::string err;

  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool fail(const char* what) { if (err.empty()) err = std::string("header is not JSON: ") + what; return false; }
  bool expect(char c) {
    ws();
    if (p >= end || *p != c) return fail((std::string("expected '") + c + "'").c_str());
    ++p;
    return true;
  }
  bool peek(char c) { ws(); return p < end && *p == c; }

  bool string(std::string& out) {
    ws();
    if (p >= end || *p != '"') return fail("expected a string");
    ++p;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("unfinished escape");
        switch (*p) {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'n': out += '\n'; break;
          case 'r': out += '\r'; break;
          case 't': out += '\t'; break;
          case 'u': {
            if (end - p < 5) return fail("unfinished \\u escape");
            unsigned v = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p[i];
              v <<= 4;
              if (c >= '0' && c <= '9') v |= c - '0';
              else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
              else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
              else return fail("bad \\u escape");
            }
            p += 4;
            if (v < 0x80) out += (char)v;
            else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
            else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
            break;
          }
          default: return fail("unknown escape");
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end) return fail("unfinished string");
    ++p;
    return true;
  }

  bool integer(long long& out) {
    ws();
    const char* s = p;
    if (p < end && *p == '-') ++p;
    if (p >= end || *p < '0' || *p > '9') return fail("expected an integer");
    long long v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (INT64_MAX - 9) / 10) return fail("integer too large");
      v = v * 10 + (*p++ - '0');
    }
    if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail("expected an integer, found a fraction");
    out = (*s == '-') ? -v : v;
    return true;
  }

  bool int_array(std::vector<long long>& out) {
    if (!expect('[')) return false;
    out.clear();
    if (peek(']')) { ++p; return true; }
    for (;;) {
      long long v;
      if (!integer(v)) return false;
      out.push_back(v);
      if (peek(',')) { ++p; continue; }
      return expect(']');
    }
  }

  // skips any value (used for keys this reader does not know); nesting is bounded, so that a
  // header made of brackets cannot exhaust the stack
  static constexpr int MAX_DEPTH = 64;
  bool skip(int depth = 0) {
    ws();
    if (p >= end) return fail("unexpected end");
    if (*p == '"') { std::string s; return string(s); }
    if (*p == '{' || *p == '[') {
      if (depth >= MAX_DEPTH) return fail("values nested deeper than 64 levels");
      const char open = *p, close = (open == '{') ? '}' : ']';
      ++p;
      if (peek(close)) { ++p; return true; }
      for (;;) {
        if (open == '{') { std::string k; if (!string(k) || !expect(':')) return false; }
        if (!skip(depth + 1)) return false;
        if (peek(',')) { ++p; continue; }
        return expect(close);
      }
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;     // number, true, false, null
    return true;
  }
};

bool parse_header(File& f, const char* text, size_t len, std::string& err) {
  Parser ps{text, text + len, {}};
  if (!ps.expect('{')) { err = ps.err; return false; }
  if (ps.peek('}')) return true;
  for (;;) {
    std::string key;
    if (!ps.string(key) || !ps.expect(':')) { err = ps.err; return false; }
    if (key == "__metadata__") {
      if (ps.peek('{')) {
        ++ps.p;
        if (ps.peek('}')) { ++ps.p; }
        else for (;;) {
          std::string k, v;
          if (!ps.string(k) || !ps.expect(':')) { err = ps.err; return false; }
          if (ps.peek('"')) { if (!ps.string(v)) { err = ps.err; return false; } }
          else if (!ps.skip()) { err = ps.err; return false; }
          f.metadata.emplace_back(k, v);
          if (ps.peek(',')) { ++ps.p; continue; }
          if (!ps.expect('}')) { err = ps.err; return false; }
          break;
        }
      } else if (!ps.skip()) { err = ps.err; return false; }
    } else {
      Entry e;
      e.name = key;
      bool has_dtype = false, has_shape = false, has_off = false;
      if (!ps.expect('{')) { err = "malformed entry for tensor " + key; return false; }
      if (!ps.peek('}')) for (;;) {
        std::string k;
        if (!ps.string(k) || !ps.expect(':')) { err = "malformed entry for tensor " + key; return false; }
        if (k == "dtype") { if (!ps.string(e.dtype)) { err = "malformed entry for tensor " + key; return false; } has_dtype = true; }
        else if (k == "shape") { if (!ps.int_array(e.shape)) { err = "malformed entry for tensor " + key; return false; } has_shape = true; }
        else if (k == "data_offsets") {
          std::vector<long long> o;
          if (!ps.int_array(o) || o.size() != 2) { err = "malformed entry for tensor " + key; return false; }
          e.begin = o[0]; e.end = o[1]; has_off = true;
        } else if (!ps.skip()) { err = ps.err; return false; }
        if (ps.peek(',')) { ++ps.p; continue; }
        break;
      }
      if (!ps.expect('}') || !has_dtype || !has_shape || !has_off) { err = "malformed entry for tensor " + key; return false; }
      f.entries.push_back(std::move(e));
    }
    if (ps.peek(',')) { ++ps.p; continue; }
    if (!ps.expect('}')) { err = ps.err; return false; }
    break;
  }
  ps.ws();
  return true;
}

void set_err(char* buf, int n, const std::string& msg) {
  if (buf && n > 0) { snprintf(buf, (size_t)n, "%s", msg.c_str()); }
}

}  // namespace

// Opens and checks a file; nullptr on failure with the reason in `err`.
ST_API void* st_open(const char* path, char* err, int err_len) {
  File* f = new File();
  auto bail = [&](const std::string& msg) -> void* {
    set_err(err, err_len, msg);
    if (f->map && f->map != MAP_FAILED) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
    return nullptr;
  };
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) return bail(std::string("cannot open: ") + strerror(errno));
  struct stat st;
  if (fstat(f->fd, &st) != 0) return bail(std::string("cannot stat: ") + strerror(errno));
  f->size = (size_t)st.st_size;
  if (f->size < 8) return bail("too short to be a safetensors file (" + std::to_string(f->size) + " bytes)");
  f->map = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (f->map == MAP_FAILED) { f->map = nullptr; return bail(std::string("cannot map: ") + strerror(errno)); }
  const unsigned char* b = static_cast<const unsigned char*>(f->map);
  unsigned long long hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | b[i];
  if (hlen > f->size - 8)
    return bail("header length " + std::to_string(hlen) + " exceeds the file (" + std::to_string(f->size) + " bytes)");
  f->data_start = 8 + (size_t)hlen;
  std::string perr;
  if (!parse_header(*f, reinterpret_cast<const char*>(b + 8), (size_t)hlen, perr)) return bail(perr);
  const long long data_len = (long long)(f->size - f->data_start);
  for (const Entry& e : f->entries) {
    const int isz = item_size(e.dtype);
    if (!isz) return bail("tensor " + e.name + " has unsupported dtype " + e.dtype);
    long long n = 1;
    for (long long s : e.shape) {
      if (s < 0) return bail("tensor " + e.name + " has a negative size");
      // the element count times the item size must stay a valid byte count: a product that
      // wrapped around could equal end - begin and pass the comparison below
      if (s > 0 && n > (INT64_MAX / isz) / s)
        return bail("tensor " + e.name + " has a shape whose byte count does not fit 63 bits");
      n *= s;
    }
    if (e.begin < 0 || e.end < e.begin || e.end > data_len)
      return bail("tensor " + e.name + " lies outside the file (offsets " + std::to_string(e.begin) + ".." +
                  std::to_string(e.end) + ", data section " + std::to_string(data_len) + " bytes)");
    if (e.end - e.begin != n * isz)
      return bail("tensor " + e.name + " of dtype " + e.dtype + " needs " + std::to_string(n * isz) + " bytes, has " +
                  std::to_string(e.end - e.begin));
  }
  return f;
}

ST_API int st_count(void* h) { return (int)static_cast<File*>(h)->entries.size(); }

// Entry i: its name and dtype (valid until st_close), shape (up to `max_dims` sizes, returns the rank) and offsets.
ST_API int st_entry(void* h, int i, const char** name, const char** dtype, long long* shape, int max_dims,
                    long long* begin, long long* end) {
  File* f = static_cast<File*>(h);
  if (i < 0 || i >= (int)f->entries.size()) return -1;
  const Entry& e = f->entries[i];
  *name = e.name.c_str();
  *dtype = e.dtype.c_str();
  for (int d = 0; d < (int)e.shape.size() && d < max_dims; ++d) shape[d] = e.shape[d];
  *begin = e.begin;
  *end = e.end;
  return (int)e.shape.size();
}

ST_API int st_metadata_count(void* h) { return (int)static_cast<File*>(h)->metadata.size(); }
ST_API void st_metadata(void* h, int i, const char** key, const char** value) {
  File* f = static_cast<File*>(h);
  *key = f->metadata[i].first.c_str();
  *value = f->metadata[i].second.c_str();
}

// Address of the data section (read-only mapping) and its length.
ST_API const void* st_data(void* h) {
  File* f = static_cast<File*>(h);
  return static_cast<const unsigned char*>(f->map) + f->data_start;
}
ST_API long long st_data_len(void* h) {
  File* f = static_cast<File*>(h);
  return (long long)(f->size - f->data_start);
}

ST_API void st_close(void* h) {
  File* f = static_cast<File*>(h);
  if (!f) return;
  if (f->map) munmap(f->map, f->size);
  if (f->fd >= 0) close(f->fd);
  delete f;
}
