#include "safetensors.hpp"

#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <set>
#include <sstream>
#include <stdexcept>

#include "json.hpp"

namespace pk {

const char* st_dtype_name(StDtype d) {
  switch (d) {
    case StDtype::F32: return "F32";
    case StDtype::F16: return "F16";
    case StDtype::BF16: return "BF16";
    case StDtype::F8_E4M3: return "F8_E4M3";
    case StDtype::F8_E5M2: return "F8_E5M2";
    case StDtype::I8: return "I8";
    case StDtype::U8: return "U8";
    case StDtype::I32: return "I32";
    case StDtype::I64: return "I64";
    case StDtype::F8_E8M0: return "F8_E8M0";
    default: return "?";
  }
}

size_t st_dtype_size(StDtype d) {
  switch (d) {
    case StDtype::F32: case StDtype::I32: return 4;
    case StDtype::F16: case StDtype::BF16: return 2;
    case StDtype::I64: return 8;
    case StDtype::Unknown: return 0;
    default: return 1;
  }
}

static StDtype parse_dtype(const std::string& s) {
  if (s == "F32") return StDtype::F32;
  if (s == "F16") return StDtype::F16;
  if (s == "BF16") return StDtype::BF16;
  if (s == "F8_E4M3") return StDtype::F8_E4M3;
  if (s == "F8_E5M2") return StDtype::F8_E5M2;
  if (s == "I8") return StDtype::I8;
  if (s == "U8") return StDtype::U8;
  if (s == "I32") return StDtype::I32;
  if (s == "I64") return StDtype::I64;
  if (s == "F8_E8M0") return StDtype::F8_E8M0;
  return StDtype::Unknown;
}

MappedFile::MappedFile(const std::string& path) : path_(path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("cannot open " + path);
  struct stat st;
  if (fstat(fd_, &st) != 0) {
    ::close(fd_);
    throw std::runtime_error("cannot stat " + path);
  }
  size_ = (size_t)st.st_size;
  if (size_ > 0) {
    void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (p == MAP_FAILED) {
      ::close(fd_);
      throw std::runtime_error("cannot mmap " + path);
    }
    data_ = (const uint8_t*)p;
  }
}

MappedFile::~MappedFile() {
  if (data_) munmap((void*)data_, size_);
  if (fd_ >= 0) ::close(fd_);
}

SafetensorsFile::SafetensorsFile(const std::string& path) : file_(new MappedFile(path)) {
  const uint8_t* base = file_->data();
  const size_t size = file_->size();
  if (size < 8) throw std::runtime_error("safetensors: file too small: " + path);
  uint64_t header_len = 0;
  memcpy(&header_len, base, 8);
  if (header_len > size - 8) throw std::runtime_error("safetensors: bad header length: " + path);
  const Json header = Json::parse((const char*)base + 8, (size_t)header_len);
  const uint8_t* payload = base + 8 + header_len;
  const size_t payload_size = size - 8 - (size_t)header_len;
  for (const auto& kv : header.members()) {
    if (kv.first == "__metadata__") {
      if (kv.second.is_object())
        for (const auto& m : kv.second.members())
          if (m.second.is_string()) metadata_[m.first] = m.second.as_string();
      continue;
    }
    StTensor t;
    t.name = kv.first;
    t.dtype = parse_dtype(kv.second.at("dtype").as_string());
    // dimensions of an untrusted header: non-negative, and their product (times the element size) must not wrap
    uint64_t count = 1;
    for (const auto& d : kv.second.at("shape").items()) {
      const int64_t dim = d.as_int();
      if (dim < 0) throw std::runtime_error("safetensors: negative dimension in " + t.name);
      if (dim != 0 && count > (uint64_t)1 << 60) throw std::runtime_error("safetensors: shape too large for " + t.name);
      if (dim != 0 && count > ((uint64_t)1 << 60) / (uint64_t)dim) throw std::runtime_error("safetensors: shape too large for " + t.name);
      count *= (uint64_t)dim;
      t.shape.push_back(dim);
    }
    const auto& off = kv.second.at("data_offsets").items();
    if (off.size() != 2) throw std::runtime_error("safetensors: bad offsets for " + t.name);
    const uint64_t b = (uint64_t)off[0].as_int(), e = (uint64_t)off[1].as_int();
    if (e < b || e > payload_size) throw std::runtime_error("safetensors: offsets out of range for " + t.name);
    t.data = payload + b;
    t.nbytes = (size_t)(e - b);
    const size_t expect = (size_t)t.numel() * st_dtype_size(t.dtype);
    if (t.dtype != StDtype::Unknown && expect != t.nbytes)
      throw std::runtime_error("safetensors: size mismatch for " + t.name);
    tensors_[t.name] = std::move(t);
  }
}

static bool is_dir(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
static bool file_exists(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

SafetensorsModel::SafetensorsModel(const std::string& path) {
  std::vector<std::string> shard_paths;
  if (is_dir(path)) {
    const std::string index = path + "/model.safetensors.index.json";
    if (file_exists(index)) {
      std::ifstream in(index);
      std::stringstream ss;
      ss << in.rdbuf();
      const Json j = Json::parse(ss.str());
      std::set<std::string> uniq;
      for (const auto& kv : j.at("weight_map").members()) uniq.insert(kv.second.as_string());
      for (const auto& f : uniq) shard_paths.push_back(path + "/" + f);
    } else {
      DIR* d = opendir(path.c_str());
      if (!d) throw std::runtime_error("cannot list " + path);
      while (dirent* e = readdir(d)) {
        const std::string n = e->d_name;
        if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") shard_paths.push_back(path + "/" + n);
      }
      closedir(d);
      std::sort(shard_paths.begin(), shard_paths.end());
    }
  } else {
    shard_paths.push_back(path);
  }
  if (shard_paths.empty()) throw std::runtime_error("no safetensors files under " + path);
  for (const auto& sp : shard_paths) {
    files_.emplace_back(new SafetensorsFile(sp));
    for (const auto& kv : files_.back()->tensors()) lookup_[kv.first] = &kv.second;
  }
}

const StTensor* SafetensorsModel::find(const std::string& name) const {
  auto it = lookup_.find(name);
  return it == lookup_.end() ? nullptr : it->second;
}

const StTensor& SafetensorsModel::get(const std::string& name) const {
  const StTensor* t = find(name);
  if (!t) throw std::runtime_error("safetensors: missing tensor " + name);
  return *t;
}

std::vector<std::string> SafetensorsModel::names() const {
  std::vector<std::string> out;
  for (const auto& kv : lookup_) out.push_back(kv.first);
  return out;
}

}  // namespace pk
