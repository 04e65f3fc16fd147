// Byte buffers that make up a message: pack / unpack of PODs, vectors, strings and raw or
// device memory (role of the reference's src/common/portable-bytes.hpp:52-130 and
// src/common/zmq-portable-bytes.hpp:40-98; here a frame owns a plain std::vector).
#pragma once
#include <stdint.h>
#include <string.h>

#include <string>
#include <vector>

#include "core/common_util.hpp"

namespace geeps_b200 {

class PortableBytes {
 public:
  PortableBytes() {}
  explicit PortableBytes(size_t n) : buf_(n) {}
  size_t size() const { return buf_.size(); }
  char* data() { return buf_.data(); }
  const char* data() const { return buf_.data(); }
  void resize(size_t n) { buf_.resize(n); }

  template <class T> void pack(const T& pod) { buf_.resize(sizeof(T)); memcpy(buf_.data(), &pod, sizeof(T)); }
  template <class T> bool unpack(T* pod) const {
    if (buf_.size() < sizeof(T)) return false;
    memcpy(pod, buf_.data(), sizeof(T));
    return true;
  }
  template <class T> void pack_vector(const std::vector<T>& v) {
    buf_.resize(v.size() * sizeof(T));
    if (!v.empty()) memcpy(buf_.data(), v.data(), buf_.size());
  }
  template <class T> void unpack_vector(std::vector<T>* v) const {
    v->resize(buf_.size() / sizeof(T));
    if (!v->empty()) memcpy(v->data(), buf_.data(), v->size() * sizeof(T));
  }
  void pack_string(const std::string& s) { buf_.assign(s.begin(), s.end()); }
  std::string unpack_string() const { return std::string(buf_.begin(), buf_.end()); }
  void pack_memory(const void* p, size_t n) { buf_.resize(n); if (n) memcpy(buf_.data(), p, n); }
  // concatenation of two sources (host-cached part followed by the device-cached part)
  void pack_memory(const void* p0, size_t n0, const void* p1, size_t n1) {
    buf_.resize(n0 + n1);
    if (n0) memcpy(buf_.data(), p0, n0);
    if (n1) memcpy(buf_.data() + n0, p1, n1);
  }
  // device memory straight into the frame (synchronous D2H on `stream`)
  void pack_gpu_memory(const void* dev, size_t n, void* stream) {
    buf_.resize(n);
    Mem::copy(buf_.data(), MEM_HOST, dev, MEM_DEVICE, n, stream, true);
  }
  uint32_t cmd() const { uint32_t c = 0xffffffffu; if (buf_.size() >= 4) memcpy(&c, buf_.data(), 4); return c; }

 private:
  std::vector<char> buf_;
};

typedef std::vector<PortableBytes> Message;

inline size_t message_bytes(const Message& m) {
  size_t n = 0;
  for (const PortableBytes& f : m) n += f.size();
  return n;
}

}  // namespace geeps_b200
