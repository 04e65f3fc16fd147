// Storage and allocation utilities of the runtime.
//
//   DataStorage              typed row buffer in host, pinned-host or device memory with its row keys
//   GpuCache<Helper>         one slab + pluggable sub-allocator returning row pointers
//   SimpleCacheHelper        single-thread FIFO ring sub-allocator
//   MultithreadedCacheHelper thread-safe next-fit sub-allocator with blocking, bounded get()
//
// Same roles as the reference's src/common/common-util.hpp:57-558; the implementation differs:
// waits are bounded and report, device memory is reached through a small MemoryBackend so the
// whole runtime also runs on a machine without a GPU.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "geeps-user-defined-types.hpp"
#include "internal_config.hpp"

namespace geeps_b200 {

inline iter_t clock_min(const std::vector<iter_t>& clocks) {
  iter_t m = kBigIter;
  for (iter_t c : clocks) m = c < m ? c : m;
  return clocks.empty() ? kInitialDataAge : m;
}
inline iter_t clock_max(const std::vector<iter_t>& clocks) {
  iter_t m = kInitialDataAge;
  for (iter_t c : clocks) m = c > m ? c : m;
  return m;
}
inline size_t get_nearest_power2(size_t n) {
  size_t p = 1;
  while (p < n) p <<= 1;
  return p;
}

struct RowKey {
  uint64_t table;
  uint64_t row;
  RowKey(uint64_t t = 0, uint64_t r = 0) : table(t), row(r) {}
  bool operator==(const RowKey& o) const { return table == o.table && row == o.row; }
};

enum MemType { MEM_HOST = 0, MEM_PINNED = 1, MEM_DEVICE = 2 };

// Thin wrapper over the CUDA runtime so that host-only processes never touch it.
struct Mem {
  static bool cuda_available();
  static void* alloc(MemType type, size_t bytes, std::string* err = nullptr);
  static void free(MemType type, void* p);
  static void zero(MemType type, void* p, size_t bytes, void* stream = nullptr);
  // kind is deduced from the two memory types; async on `stream` when one side is device memory
  static void copy(void* dst, MemType dt, const void* src, MemType st, size_t bytes, void* stream = nullptr,
                   bool sync = true);
  static void stream_sync(void* stream);
};
// cudaMallocHost with a bounded number of retries (the reference's mallocHost retries forever,
// src/common/common-util.hpp:84-95).
void* malloc_host_pinned(size_t bytes, int max_tries = 8);

class DataStorage {
 public:
  DataStorage() : type_(MEM_HOST), rows_(0), ptr_(nullptr) {}
  ~DataStorage() { release(); }
  DataStorage(const DataStorage&) = delete;
  DataStorage& operator=(const DataStorage&) = delete;
  DataStorage(DataStorage&& o) noexcept : row_keys(std::move(o.row_keys)), type_(o.type_), rows_(o.rows_), ptr_(o.ptr_) {
    o.ptr_ = nullptr; o.rows_ = 0;
  }
  DataStorage& operator=(DataStorage&& o) noexcept {
    if (this != &o) {
      release();
      row_keys = std::move(o.row_keys); type_ = o.type_; rows_ = o.rows_; ptr_ = o.ptr_;
      o.ptr_ = nullptr; o.rows_ = 0;
    }
    return *this;
  }
  void init(size_t rows, MemType type);
  void init_from(const DataStorage& other);   // same size/type, copies keys and data
  void release();
  void zerofy(void* stream = nullptr);
  RowData* data() const { return ptr_; }
  float* floats() const { return reinterpret_cast<float*>(ptr_); }
  size_t size() const { return rows_; }
  size_t bytes() const { return rows_ * sizeof(RowData); }
  MemType type() const { return type_; }
  std::vector<RowKey> row_keys;
 private:
  MemType type_;
  size_t rows_;
  RowData* ptr_;
};

// ---------------- sub-allocators over a row range [0, size) ----------------
class SimpleCacheHelper {
 public:
  void init(size_t size) { size_ = size; head_ = tail_ = used_ = 0; last_alloc_start_ = 0; }
  size_t size() const { return size_; }
  size_t used() const { return used_; }
  // FIFO ring: returns the start row or (size_t)-1 if `count` rows are not free right now.
  size_t get(size_t count, bool wait = false, int tag = 0);
  void put(size_t start, size_t count);
 private:
  size_t size_ = 0, head_ = 0, tail_ = 0, used_ = 0, last_alloc_start_ = 0;
  struct Seg { size_t start, count, skip; };
  std::vector<Seg> fifo_;
};

class MultithreadedCacheHelper {
 public:
  struct Block { size_t size; int tag; };
  void init(size_t size);
  size_t size() const { return size_; }
  size_t used() const;
  // Next-fit search from the last allocation.  With wait=true blocks until space appears, logging who
  // is waiting every kWatchdogSeconds; gives up after budget_ms (0 = never) and returns (size_t)-1.
  size_t get(size_t count, bool wait, int tag = 0, size_t budget_ms = 0);
  void put(size_t start, size_t count);
  std::string describe() const;
 private:
  size_t try_get_locked(size_t count, int tag);
  size_t size_ = 0, used_ = 0, cursor_ = 0;
  std::map<size_t, Block> blocks_;   // start -> block, ordered
  mutable std::mutex mu_;
  std::condition_variable cv_;
};

template <class Helper>
class GpuCache {
 public:
  GpuCache() : type_(MEM_DEVICE), base_(nullptr), rows_(0) {}
  ~GpuCache() { clear(); }
  bool init(size_t rows, MemType type = MEM_DEVICE, std::string* err = nullptr) {
    clear();
    type_ = type;
    rows_ = rows;
    if (rows) {
      base_ = static_cast<RowData*>(Mem::alloc(type, rows * sizeof(RowData), err));
      if (!base_) { rows_ = 0; return false; }
    }
    helper.init(rows);
    return true;
  }
  void clear() {
    if (base_) Mem::free(type_, base_);
    base_ = nullptr;
    rows_ = 0;
  }
  RowData* get(size_t count, bool wait, int tag = 0) {
    size_t s = helper.get(count, wait, tag);
    return s == (size_t)-1 ? nullptr : base_ + s;
  }
  void put(RowData* p, size_t count) { helper.put((size_t)(p - base_), count); }
  RowData* at(size_t row) const { return base_ + row; }
  size_t size() const { return rows_; }
  RowData* base() const { return base_; }
  Helper helper;
 private:
  MemType type_;
  RowData* base_;
  size_t rows_;
};

inline double now_seconds() {
  using namespace std::chrono;
  return duration_cast<duration<double>>(steady_clock::now().time_since_epoch()).count();
}

}  // namespace geeps_b200
