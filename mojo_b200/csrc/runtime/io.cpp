// Memory-mapped checkpoint files and the safetensors header (see b2/io.h).
#include "b2/io.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <stdexcept>

#include "b2/runtime.h"

namespace b2 {
namespace io {

// ---- MappedFile -----------------------------------------------------------------------------------
std::shared_ptr<MappedFile> MappedFile::open(const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) throw std::runtime_error("cannot open " + path + ": " + std::strerror(errno));
  struct stat st;
  if (::fstat(fd, &st) != 0) {
    const int e = errno;
    ::close(fd);
    throw std::runtime_error("cannot stat " + path + ": " + std::strerror(e));
  }
  std::shared_ptr<MappedFile> f(new MappedFile());
  f->path_ = path;
  f->size_ = static_cast<size_t>(st.st_size);
  if (f->size_ > 0) {
    void* p = ::mmap(nullptr, f->size_, PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) {
      const int e = errno;
      ::close(fd);
      throw std::runtime_error("cannot map " + path + ": " + std::strerror(e));
    }
    f->data_ = static_cast<const uint8_t*>(p);
  }
  ::close(fd);  // the mapping keeps the file alive
  return f;
}

MappedFile::~MappedFile() {
  if (data_ != nullptr) ::munmap(const_cast<uint8_t*>(data_), size_);
}

void MappedFile::will_need(size_t offset, size_t n) const {
  if (data_ == nullptr || offset >= size_) return;
  n = std::min(n, size_ - offset);
  const size_t page = static_cast<size_t>(::sysconf(_SC_PAGESIZE));
  const size_t lo = offset / page * page;
  ::madvise(const_cast<uint8_t*>(data_) + lo, n + (offset - lo), MADV_WILLNEED);
}

// ---- a JSON reader for exactly what a safetensors header contains ---------------------------------
namespace {

struct Cursor {
  const char* p;
  const char* end;
  [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("safetensors header: ") + what); }
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool peek(char c) {
    ws();
    return p < end && *p == c;
  }
  void expect(char c) {
    ws();
    if (p >= end || *p != c) fail("unexpected character");
    ++p;
  }
  static void put_utf8(std::string& out, unsigned cp) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  unsigned hex4() {
    if (end - p < 4) fail("truncated \\u escape");
    unsigned v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= static_cast<unsigned>(c - '0');
      else if (c >= 'a' && c <= 'f') v |= static_cast<unsigned>(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= static_cast<unsigned>(c - 'A' + 10);
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string string() {
    expect('"');
    std::string out;
    while (true) {
      if (p >= end) fail("unterminated string");
      const char c = *p++;
      if (c == '"') break;
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (p >= end) fail("unterminated escape");
      const char e = *p++;
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          unsigned cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
            p += 2;
            const unsigned lo = hex4();
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          put_utf8(out, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return out;
  }
  uint64_t uint() {
    ws();
    if (p >= end || *p < '0' || *p > '9') fail("expected a non-negative integer");
    uint64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      const uint64_t d = static_cast<uint64_t>(*p - '0');
      if (v > (UINT64_MAX - d) / 10) fail("integer overflow");
      v = v * 10 + d;
      ++p;
    }
    return v;
  }
  // Skips any JSON value (used for keys this reader does not know).
  void skip_value() {
    ws();
    if (p >= end) fail("truncated");
    if (*p == '"') { string(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (peek(close)) { ++p; return; }
      while (true) {
        if (open == '{') { string(); expect(':'); }
        skip_value();
        if (peek(',')) { ++p; continue; }
        expect(close);
        return;
      }
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;  // number, true, false, null
  }
};

}  // namespace

int dtype_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

SafetensorsFile::SafetensorsFile(const std::string& path) : file_(MappedFile::open(path)) {
  const size_t size = file_->size();
  if (size < 8) throw std::runtime_error(path + ": too short for a safetensors file");
  uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | file_->data()[i];  // little-endian u64
  if (hlen > size - 8) throw std::runtime_error(path + ": header length runs past the end of the file");
  data_start_ = 8 + static_cast<size_t>(hlen);
  const size_t data_bytes = size - data_start_;
  Cursor c{reinterpret_cast<const char*>(file_->data()) + 8, reinterpret_cast<const char*>(file_->data()) + data_start_};
  c.expect('{');
  if (!c.peek('}')) {
    while (true) {
      const std::string name = c.string();
      c.expect(':');
      if (name == "__metadata__") {
        c.expect('{');
        if (!c.peek('}')) {
          while (true) {
            const std::string k = c.string();
            c.expect(':');
            if (c.peek('"')) metadata_[k] = c.string();
            else c.skip_value();
            if (c.peek(',')) { ++c.p; continue; }
            break;
          }
        }
        c.expect('}');
      } else {
        TensorInfo t;
        bool have_dtype = false, have_shape = false, have_off = false;
        c.expect('{');
        while (true) {
          const std::string k = c.string();
          c.expect(':');
          if (k == "dtype") {
            t.dtype = c.string();
            have_dtype = true;
          } else if (k == "shape") {
            c.expect('[');
            if (!c.peek(']')) {
              while (true) {
                t.shape.push_back(static_cast<int64_t>(c.uint()));
                if (c.peek(',')) { ++c.p; continue; }
                break;
              }
            }
            c.expect(']');
            have_shape = true;
          } else if (k == "data_offsets") {
            c.expect('[');
            t.begin = c.uint();
            c.expect(',');
            t.end = c.uint();
            c.expect(']');
            have_off = true;
          } else {
            c.skip_value();
          }
          if (c.peek(',')) { ++c.p; continue; }
          break;
        }
        c.expect('}');
        if (!have_dtype || !have_shape || !have_off) throw std::runtime_error(path + ": tensor '" + name + "' lacks dtype, shape or data_offsets");
        if (t.begin > t.end || t.end > data_bytes) throw std::runtime_error(path + ": tensor '" + name + "' lies outside the file");
        const int esz = dtype_size(t.dtype);
        if (esz > 0) {
          uint64_t n = static_cast<uint64_t>(esz);
          for (int64_t d : t.shape) n *= static_cast<uint64_t>(d);
          if (n != t.end - t.begin) throw std::runtime_error(path + ": tensor '" + name + "': byte range does not match shape and dtype");
        }
        if (tensors_.emplace(name, std::move(t)).second) names_.push_back(name);
      }
      if (c.peek(',')) { ++c.p; continue; }
      break;
    }
  }
  c.expect('}');
  // file order = order of the data, which is what a sequential reader wants
  std::sort(names_.begin(), names_.end(), [this](const std::string& a, const std::string& b) { return tensors_.at(a).begin < tensors_.at(b).begin; });
}

const TensorInfo& SafetensorsFile::info(const std::string& name) const { return tensors_.at(name); }

const uint8_t* SafetensorsFile::tensor_data(const std::string& name) const { return file_->data() + data_start_ + tensors_.at(name).begin; }

// ---- parallel copy --------------------------------------------------------------------------------
void parallel_copy(void* dst, const void* src, size_t n, int max_threads) {
  constexpr size_t kChunk = 8u << 20;
  if (n <= kChunk) {
    std::memcpy(dst, src, n);
    return;
  }
  rt::WorkerPool& pool = rt::Context::instance().pool();
  int64_t chunks = static_cast<int64_t>((n + kChunk - 1) / kChunk);
  size_t chunk = kChunk;
  if (max_threads > 0 && chunks > max_threads * 4) {  // fewer, larger pieces when the caller wants little parallelism
    chunks = max_threads * 4;
    chunk = (n + static_cast<size_t>(chunks) - 1) / static_cast<size_t>(chunks);
    chunk = (chunk + 4095) / 4096 * 4096;
    chunks = static_cast<int64_t>((n + chunk - 1) / chunk);
  }
  auto* d = static_cast<uint8_t*>(dst);
  const auto* s = static_cast<const uint8_t*>(src);
  pool.parallel_for(chunks, [=](int64_t i) {
    const size_t off = static_cast<size_t>(i) * chunk;
    std::memcpy(d + off, s + off, std::min(chunk, n - off));
  });
}

}  // namespace io
}  // namespace b2
