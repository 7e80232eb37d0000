#include "gguf_reader.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace pk {
namespace {

struct TypeInfo {
  uint32_t id;
  const char* name;
  uint32_t block, bytes;
};
// ids and block geometry of the public ggml type table
const TypeInfo kTypes[] = {
    {0, "f32", 1, 4},      {1, "f16", 1, 2},       {2, "q4_0", 32, 18},    {3, "q4_1", 32, 20},   {6, "q5_0", 32, 22},
    {7, "q5_1", 32, 24},   {8, "q8_0", 32, 34},    {9, "q8_1", 32, 36},    {10, "q2_k", 256, 84}, {11, "q3_k", 256, 110},
    {12, "q4_k", 256, 144}, {13, "q5_k", 256, 176}, {14, "q6_k", 256, 210}, {15, "q8_k", 256, 292}, {16, "iq2_xxs", 256, 66},
    {17, "iq2_xs", 256, 74}, {18, "iq3_xxs", 256, 98}, {19, "iq1_s", 256, 50}, {20, "iq4_nl", 32, 18}, {21, "iq3_s", 256, 110},
    {22, "iq2_s", 256, 82}, {23, "iq4_xs", 256, 136}, {24, "i8", 1, 1},      {25, "i16", 1, 2},     {26, "i32", 1, 4},
    {27, "i64", 1, 8},     {28, "f64", 1, 8},      {29, "iq1_m", 256, 56}, {30, "bf16", 1, 2},    {39, "mxfp4", 32, 17},
};

class Cursor {
 public:
  Cursor(const uint8_t* p, uint64_t n) : p_(p), n_(n) {}
  template <class T>
  T get() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p_ + off_, sizeof(T));
    off_ += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t len = get<uint64_t>();
    need(len);
    std::string s((const char*)p_ + off_, (size_t)len);
    off_ += len;
    return s;
  }
  uint64_t offset() const { return off_; }
  uint64_t remaining() const { return n_ - off_; }

 private:
  // written so that a huge `k` from an untrusted file cannot wrap around
  void need(uint64_t k) const {
    if (k > n_ - off_) throw std::runtime_error("gguf: truncated file");
  }
  const uint8_t* p_;
  uint64_t n_, off_ = 0;
};

Json read_value(Cursor& c, uint32_t type, int depth) {
  switch (type) {
    case 0: return Json((int64_t)c.get<uint8_t>());
    case 1: return Json((int64_t)c.get<int8_t>());
    case 2: return Json((int64_t)c.get<uint16_t>());
    case 3: return Json((int64_t)c.get<int16_t>());
    case 4: return Json((int64_t)c.get<uint32_t>());
    case 5: return Json((int64_t)c.get<int32_t>());
    case 6: return Json((double)c.get<float>());
    case 7: return Json(c.get<uint8_t>() != 0);
    case 8: return Json(c.str());
    case 9: {
      if (depth > 4) throw std::runtime_error("gguf: arrays nested too deeply");
      const uint32_t et = c.get<uint32_t>();
      const uint64_t n = c.get<uint64_t>();
      // every element takes at least one byte: a count beyond the bytes left is a corrupt file, not a reservation
      if (n > c.remaining()) throw std::runtime_error("gguf: array length exceeds the file");
      Json arr = Json::array();
      arr.items().reserve((size_t)n);
      for (uint64_t i = 0; i < n; ++i) arr.push_back(read_value(c, et, depth + 1));
      return arr;
    }
    case 10: return Json((int64_t)c.get<uint64_t>());
    case 11: return Json((int64_t)c.get<int64_t>());
    case 12: return Json(c.get<double>());
    default: throw std::runtime_error("gguf: unknown metadata value type " + std::to_string(type));
  }
}

}  // namespace

uint64_t GgufTensor::elements() const {
  uint64_t n = 1;
  for (uint64_t d : dims) {
    if (d != 0 && n > UINT64_MAX / d) throw std::runtime_error("gguf: tensor " + name + " has more elements than fit 64 bits");
    n *= d;
  }
  return n;
}

const char* ggml_type_name(uint32_t type) {
  for (const auto& t : kTypes)
    if (t.id == type) return t.name;
  return "unknown";
}

std::pair<uint32_t, uint32_t> ggml_type_block(uint32_t type) {
  for (const auto& t : kTypes)
    if (t.id == type) return {t.block, t.bytes};
  return {0, 0};
}

void GgufFile::release() {
  if (base_) munmap((void*)base_, size_);
  if (fd_ >= 0) ::close(fd_);
  base_ = nullptr;
  fd_ = -1;
}

GgufFile::GgufFile(const std::string& path) : path_(path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("gguf: cannot open " + path);
  // a constructor that throws does not run the destructor: the descriptor and the mapping are released here
  try {
    parse(path);
  } catch (...) {
    release();
    throw;
  }
}

void GgufFile::parse(const std::string& path) {
  struct stat st;
  if (fstat(fd_, &st) != 0) throw std::runtime_error("gguf: cannot stat " + path);
  size_ = (uint64_t)st.st_size;
  if (size_ < 24) throw std::runtime_error("gguf: file too small: " + path);
  void* m = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
  if (m == MAP_FAILED) throw std::runtime_error("gguf: mmap failed for " + path);
  base_ = (const uint8_t*)m;
  Cursor c(base_, size_);
  if (c.get<uint32_t>() != 0x46554747u) throw std::runtime_error("gguf: bad magic in " + path);
  version_ = c.get<uint32_t>();
  if (version_ < 2 || version_ > 3) throw std::runtime_error("gguf: unsupported version " + std::to_string(version_));
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = c.str();
    const uint32_t type = c.get<uint32_t>();
    meta_[key] = read_value(c, type, 0);
  }
  alignment_ = (uint64_t)meta_.get_int("general.alignment", 32);
  if (alignment_ == 0 || (alignment_ & (alignment_ - 1))) throw std::runtime_error("gguf: alignment is not a power of two");
  // a tensor entry takes at least 24 bytes (name length, rank, type, offset)
  if (n_tensors > c.remaining() / 24) throw std::runtime_error("gguf: tensor count exceeds the file");
  tensors_.reserve((size_t)n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    GgufTensor t;
    t.name = c.str();
    const uint32_t nd = c.get<uint32_t>();
    if (nd > 8) throw std::runtime_error("gguf: tensor rank too large");
    for (uint32_t d = 0; d < nd; ++d) t.dims.push_back(c.get<uint64_t>());
    t.type = c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    const auto blk = ggml_type_block(t.type);
    if (blk.first == 0) throw std::runtime_error("gguf: tensor " + t.name + " has unknown type " + std::to_string(t.type));
    if (t.dims.empty() || t.dims[0] % blk.first) throw std::runtime_error("gguf: tensor " + t.name + " row is not a whole number of blocks");
    const uint64_t blocks = t.elements() / blk.first;
    if (blocks > UINT64_MAX / blk.second) throw std::runtime_error("gguf: tensor " + t.name + " is larger than 64 bits of bytes");
    t.nbytes = blocks * blk.second;
    index_[t.name] = tensors_.size();
    tensors_.push_back(std::move(t));
  }
  data_offset_ = (c.offset() + alignment_ - 1) / alignment_ * alignment_;
  if (data_offset_ > size_) {
    if (!tensors_.empty()) throw std::runtime_error("gguf: the data section starts past the end of the file");
    data_offset_ = size_;
  }
  const uint64_t data_bytes = size_ - data_offset_;
  for (const auto& t : tensors_) {
    if (t.offset % alignment_) throw std::runtime_error("gguf: tensor " + t.name + " is not aligned");
    // subtraction form: an offset near 2^64 cannot wrap the sum back into range
    if (t.offset > data_bytes || t.nbytes > data_bytes - t.offset)
      throw std::runtime_error("gguf: tensor " + t.name + " runs past the end of the file");
  }
}

GgufFile::~GgufFile() { release(); }

const GgufTensor* GgufFile::find(const std::string& name) const {
  auto it = index_.find(name);
  return it == index_.end() ? nullptr : &tensors_[it->second];
}

}  // namespace pk
