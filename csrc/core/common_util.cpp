#include "common_util.hpp"

#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>

namespace geeps_b200 {

bool Mem::cuda_available() {
  static int cached = -1;
  if (cached < 0) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    cached = n > 0 ? 1 : 0;
  }
  return cached == 1;
}

void* malloc_host_pinned(size_t bytes, int max_tries) {
  void* p = nullptr;
  for (int i = 0; i < max_tries; ++i) {
    cudaError_t e = cudaMallocHost(&p, bytes);
    if (e == cudaSuccess) return p;
    cudaGetLastError();
    std::this_thread::sleep_for(std::chrono::milliseconds(50 << i));
  }
  return nullptr;
}

void* Mem::alloc(MemType type, size_t bytes, std::string* err) {
  if (bytes == 0) return nullptr;
  void* p = nullptr;
  if (type == MEM_HOST || (type == MEM_PINNED && !cuda_available())) {
    if (posix_memalign(&p, 256, bytes) != 0) p = nullptr;
    if (!p && err) *err = "host allocation of " + std::to_string(bytes) + " bytes failed";
    return p;
  }
  if (type == MEM_PINNED) {
    p = malloc_host_pinned(bytes);
    if (!p && err) *err = "pinned host allocation of " + std::to_string(bytes) + " bytes failed";
    return p;
  }
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (err) *err = std::string("cudaMalloc(") + std::to_string(bytes) + "): " + cudaGetErrorString(e);
    return nullptr;
  }
  return p;
}

void Mem::free(MemType type, void* p) {
  if (!p) return;
  if (type == MEM_HOST || (type == MEM_PINNED && !cuda_available())) ::free(p);
  else if (type == MEM_PINNED) cudaFreeHost(p);
  else cudaFree(p);
}

void Mem::zero(MemType type, void* p, size_t bytes, void* stream) {
  if (!p || !bytes) return;
  if (type == MEM_DEVICE) cudaMemsetAsync(p, 0, bytes, (cudaStream_t)stream);
  else memset(p, 0, bytes);
}

void Mem::copy(void* dst, MemType dt, const void* src, MemType st, size_t bytes, void* stream, bool sync) {
  if (!bytes) return;
  if (dt != MEM_DEVICE && st != MEM_DEVICE) { memcpy(dst, src, bytes); return; }
  cudaMemcpyKind kind = (dt == MEM_DEVICE && st == MEM_DEVICE) ? cudaMemcpyDeviceToDevice
                        : dt == MEM_DEVICE ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
  cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream);
  if (sync) cudaStreamSynchronize((cudaStream_t)stream);
}

void Mem::stream_sync(void* stream) {
  if (cuda_available()) cudaStreamSynchronize((cudaStream_t)stream);
}

void DataStorage::init(size_t rows, MemType type) {
  release();
  type_ = type;
  rows_ = rows;
  row_keys.assign(rows, RowKey());
  if (rows) {
    std::string err;
    ptr_ = static_cast<RowData*>(Mem::alloc(type, rows * sizeof(RowData), &err));
    if (!ptr_) { fprintf(stderr, "[geeps] DataStorage: %s\n", err.c_str()); rows_ = 0; row_keys.clear(); }
  }
}

void DataStorage::init_from(const DataStorage& other) {
  init(other.size(), other.type());
  row_keys = other.row_keys;
  Mem::copy(ptr_, type_, other.data(), other.type(), bytes());
}

void DataStorage::release() {
  if (ptr_) Mem::free(type_, ptr_);
  ptr_ = nullptr;
  rows_ = 0;
}

void DataStorage::zerofy(void* stream) { Mem::zero(type_, ptr_, bytes(), stream); }

// ---------------- SimpleCacheHelper: FIFO ring ----------------
size_t SimpleCacheHelper::get(size_t count, bool /*wait*/, int /*tag*/) {
  if (count == 0 || count > size_) return (size_t)-1;
  size_t skip = 0;
  size_t start = head_;
  if (head_ + count > size_) {  // does not fit before the end: skip the tail fragment
    skip = size_ - head_;
    start = 0;
  }
  if (used_ + skip + count > size_) return (size_t)-1;
  fifo_.push_back({start, count, skip});
  head_ = (start + count) % size_;
  used_ += skip + count;
  last_alloc_start_ = start;
  return start;
}

void SimpleCacheHelper::put(size_t start, size_t count) {
  // frees must come in allocation order
  if (fifo_.empty() || fifo_.front().start != start || fifo_.front().count != count) {
    fprintf(stderr, "[geeps] SimpleCacheHelper: out-of-order free(%zu,%zu)\n", start, count);
    return;
  }
  used_ -= fifo_.front().skip + count;
  tail_ = (start + count) % size_;
  fifo_.erase(fifo_.begin());
}

// ---------------- MultithreadedCacheHelper: next-fit over an ordered block map ----------------
void MultithreadedCacheHelper::init(size_t size) {
  std::lock_guard<std::mutex> lk(mu_);
  size_ = size;
  used_ = 0;
  cursor_ = 0;
  blocks_.clear();
}

size_t MultithreadedCacheHelper::used() const {
  std::lock_guard<std::mutex> lk(mu_);
  return used_;
}

size_t MultithreadedCacheHelper::try_get_locked(size_t count, int tag) {
  if (count == 0 || count > size_) return (size_t)-1;
  // candidate starts: the cursor, then the end of every block after it, then from 0 (wrap)
  for (int pass = 0; pass < 2; ++pass) {
    size_t pos = pass == 0 ? cursor_ : 0;
    const size_t limit = pass == 0 ? size_ : cursor_ + count > size_ ? size_ : cursor_ + count;
    while (pos + count <= limit) {
      // first block that ends after pos
      auto it = blocks_.upper_bound(pos);
      if (it != blocks_.begin()) {
        auto prev = std::prev(it);
        if (prev->first + prev->second.size > pos) { pos = prev->first + prev->second.size; continue; }
      }
      if (it != blocks_.end() && it->first < pos + count) { pos = it->first + it->second.size; continue; }
      blocks_[pos] = Block{count, tag};
      used_ += count;
      cursor_ = pos + count >= size_ ? 0 : pos + count;
      return pos;
    }
  }
  return (size_t)-1;
}

size_t MultithreadedCacheHelper::get(size_t count, bool wait, int tag, size_t budget_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  const double t0 = now_seconds();
  for (;;) {
    size_t s = try_get_locked(count, tag);
    if (s != (size_t)-1 || !wait) return s;
    double wait_ms = kWatchdogSeconds * 1000.0;
    if (budget_ms) {
      const double left = (double)budget_ms - (now_seconds() - t0) * 1000.0;
      if (left <= 0) return (size_t)-1;
      if (left < wait_ms) wait_ms = left;
    }
    if (cv_.wait_for(lk, std::chrono::microseconds((long long)(wait_ms * 1000))) == std::cv_status::timeout &&
        wait_ms >= kWatchdogSeconds * 1000.0) {
      fprintf(stderr, "[geeps] staging pool: tag %d still waiting for %zu rows (%zu of %zu used)\n", tag, count,
              used_, size_);
    }
  }
}

void MultithreadedCacheHelper::put(size_t start, size_t count) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = blocks_.find(start);
    if (it == blocks_.end() || it->second.size != count) {
      fprintf(stderr, "[geeps] staging pool: bad free(%zu,%zu)\n", start, count);
      return;
    }
    used_ -= count;
    blocks_.erase(it);
  }
  cv_.notify_all();
}

std::string MultithreadedCacheHelper::describe() const {
  std::lock_guard<std::mutex> lk(mu_);
  std::string s = "{size:" + std::to_string(size_) + ",used:" + std::to_string(used_) + ",blocks:[";
  for (auto& kv : blocks_)
    s += "(" + std::to_string(kv.first) + "," + std::to_string(kv.second.size) + "," + std::to_string(kv.second.tag) + ")";
  return s + "]}";
}

}  // namespace geeps_b200
