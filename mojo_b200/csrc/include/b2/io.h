// Checkpoint file access: read-only memory maps and the safetensors container format.
//
// The reference reads files through a closed buffered layer (`FileHandle.read/read_bytes/seek`,
// stdlib/src/builtin/file.mojo:71-498 over KGEN_CompilerRT_IO_File*). Weights are tens of gigabytes that are read
// once and copied to the device, so this runtime maps the file instead and lets a worker pool fault pages in and
// copy in parallel (`parallel_copy`): nothing is buffered twice, and a tensor can also be handed out as a view of
// the mapping with no copy at all.
//
// safetensors layout: u64 little-endian header length N, N bytes of JSON
//   {"name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {...}}
// followed by the tensor bytes; offsets are relative to the end of the header.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace b2 {
namespace io {

class MappedFile {
 public:
  // Throws std::runtime_error (with the path and errno text) when the file cannot be opened or mapped.
  static std::shared_ptr<MappedFile> open(const std::string& path);
  ~MappedFile();
  MappedFile(const MappedFile&) = delete;
  MappedFile& operator=(const MappedFile&) = delete;

  const uint8_t* data() const { return data_; }
  size_t size() const { return size_; }
  const std::string& path() const { return path_; }
  // Hint that [offset, offset + n) is about to be read front to back.
  void will_need(size_t offset, size_t n) const;

 private:
  MappedFile() = default;
  const uint8_t* data_ = nullptr;
  size_t size_ = 0;
  std::string path_;
};

struct TensorInfo {
  std::string dtype;            // as spelled in the file: "BF16", "F32", "F8_E4M3", "I64", ...
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range relative to the start of the data section
  size_t nbytes() const { return static_cast<size_t>(end - begin); }
};

// Bytes per element of a safetensors dtype string; 0 for an unknown one.
int dtype_size(const std::string& dtype);

class SafetensorsFile {
 public:
  // Throws std::runtime_error on a malformed header, on offsets outside the file, or when a tensor's byte range does
  // not match its shape and dtype.
  explicit SafetensorsFile(const std::string& path);

  const std::vector<std::string>& names() const { return names_; }   // in file order
  bool has(const std::string& name) const { return tensors_.count(name) != 0; }
  const TensorInfo& info(const std::string& name) const;              // throws std::out_of_range
  const uint8_t* tensor_data(const std::string& name) const;          // into the mapping
  const std::unordered_map<std::string, std::string>& metadata() const { return metadata_; }
  const std::shared_ptr<MappedFile>& file() const { return file_; }

 private:
  std::shared_ptr<MappedFile> file_;
  size_t data_start_ = 0;
  std::vector<std::string> names_;
  std::unordered_map<std::string, TensorInfo> tensors_;
  std::unordered_map<std::string, std::string> metadata_;
};

// memcpy of n bytes split into chunks over the process worker pool (at most `max_threads` at a time, 0 = all).
// For a cold mapping the page faults, which dominate, proceed in parallel.
void parallel_copy(void* dst, const void* src, size_t n, int max_threads = 0);

}  // namespace io
}  // namespace b2
