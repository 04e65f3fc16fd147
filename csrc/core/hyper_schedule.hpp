// Optimizer hyper-parameters as a function of the clock.  The shard-side optimizer (momentum SGD with weight decay)
// reads its learning rate, momentum and weight decay from here, keyed by the clock of the updates it applies, so a
// worker can change them while training runs (a learning-rate policy) and every shard switches at the same clock:
// all workers make the same set() call in the same iteration, and the values hold for the updates of that
// iteration and all later ones.  The reference's server only adds (src/server/tablet-server.cpp:119-134); its
// learning-rate policy lived in the solver of the absent Caffe application.
#pragma once
#include <mutex>
#include <vector>

#include "geeps-user-defined-types.hpp"

namespace geeps_b200 {

class HyperSchedule {
 public:
  struct Entry {
    iter_t from_clock;
    float lr, momentum, weight_decay;
  };
  HyperSchedule(float lr, float momentum, float weight_decay) {
    entries_.push_back(Entry{-(1 << 30), lr, momentum, weight_decay});
  }
  // The values for updates of clock >= from_clock.  A call for a clock at or before an earlier call's replaces it
  // (and what came after it): the schedule stays sorted and the latest call wins.
  void set(iter_t from_clock, float lr, float momentum, float weight_decay) {
    std::lock_guard<std::mutex> g(mu_);
    while (entries_.size() > 1 && entries_.back().from_clock >= from_clock) entries_.pop_back();
    const Entry& b = entries_.back();
    if (b.lr == lr && b.momentum == momentum && b.weight_decay == weight_decay) return;   // nothing changes
    entries_.push_back(Entry{from_clock, lr, momentum, weight_decay});
  }
  Entry at(iter_t clock) const {
    std::lock_guard<std::mutex> g(mu_);
    size_t i = entries_.size() - 1;
    while (i > 0 && entries_[i].from_clock > clock) --i;
    return entries_[i];
  }
  size_t size() const {
    std::lock_guard<std::mutex> g(mu_);
    return entries_.size();
  }

 private:
  mutable std::mutex mu_;
  std::vector<Entry> entries_;
};

}  // namespace geeps_b200
