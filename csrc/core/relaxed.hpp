// Statistics counters that one thread writes while another serialises them.
#pragma once
#include <atomic>
#include <ostream>

namespace geeps_b200 {

// A counter that one thread (application, push worker, decoder, server) updates while GetStats() reads it from
// another: relaxed atomic load / store, single writer per field, so += needs no read-modify-write instruction.
template <typename T>
struct Relaxed {
  std::atomic<T> v;
  Relaxed(T x = T()) : v(x) {}
  Relaxed(const Relaxed& o) : v(o.get()) {}
  Relaxed& operator=(const Relaxed& o) { set(o.get()); return *this; }
  T get() const { return v.load(std::memory_order_relaxed); }
  void set(T x) { v.store(x, std::memory_order_relaxed); }
  operator T() const { return get(); }
  Relaxed& operator=(T x) { set(x); return *this; }
  Relaxed& operator+=(T x) { set(get() + x); return *this; }
  Relaxed& operator++() { set(get() + 1); return *this; }
  T operator++(int) { T old = get(); set(old + 1); return old; }
};
template <typename T>
std::ostream& operator<<(std::ostream& o, const Relaxed<T>& r) { return o << r.get(); }

}  // namespace geeps_b200
