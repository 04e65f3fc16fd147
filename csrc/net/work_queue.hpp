// In-process command queue with a worker thread and a callback table keyed by command id
// (roles of the reference's WorkPusher / WorkPuller / BackgroundWorker,
// src/common/work-pusher.cpp:36-53, work-puller.cpp:36-57, background-worker.cpp:36-67,
// which ride on ZeroMQ inproc sockets; here a mutex-protected deque).
#pragma once
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string.h>
#include <thread>
#include <vector>

#include "core/internal_config.hpp"

namespace geeps_b200 {

struct WorkItem {
  unsigned cmd = 0;
  std::vector<char> args;
};

class WorkQueue {
 public:
  void push(WorkItem&& w) {
    { std::lock_guard<std::mutex> lk(mu_); q_.push_back(std::move(w)); }
    cv_.notify_one();
  }
  WorkItem pull() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return !q_.empty(); });
    WorkItem w = std::move(q_.front());
    q_.pop_front();
    return w;
  }
  size_t pending() { std::lock_guard<std::mutex> lk(mu_); return q_.size(); }
 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<WorkItem> q_;
};

class WorkPusher {
 public:
  explicit WorkPusher(WorkQueue* q) : q_(q) {}
  template <class T> void push_work(unsigned cmd, const T& args) {
    WorkItem w;
    w.cmd = cmd;
    w.args.resize(sizeof(T));
    memcpy(w.args.data(), &args, sizeof(T));
    q_->push(std::move(w));
  }
  void push_work(unsigned cmd) { WorkItem w; w.cmd = cmd; q_->push(std::move(w)); }
 private:
  WorkQueue* q_;
};

class WorkPuller {
 public:
  explicit WorkPuller(WorkQueue* q) : q_(q) {}
  // blocks; returns false on the stop command
  bool pull_work(unsigned* cmd, std::vector<char>* args) {
    WorkItem w = q_->pull();
    *cmd = w.cmd;
    *args = std::move(w.args);
    return w.cmd != kStopCmd;
  }
 private:
  WorkQueue* q_;
};

class BackgroundWorker {
 public:
  typedef std::function<void(std::vector<char>&)> Callback;
  BackgroundWorker() : pusher_(&queue_), puller_(&queue_) {}
  ~BackgroundWorker() { stop(); }
  void add_callback(unsigned cmd, Callback cb) { callbacks_[cmd] = cb; }
  WorkPusher* pusher() { return &pusher_; }
  void start() {
    if (thread_.joinable()) return;
    thread_ = std::thread([this] {
      unsigned cmd;
      std::vector<char> args;
      while (puller_.pull_work(&cmd, &args)) {
        auto it = callbacks_.find(cmd);
        if (it != callbacks_.end()) it->second(args);
      }
    });
  }
  void stop() {
    if (!thread_.joinable()) return;
    pusher_.push_work(kStopCmd);
    thread_.join();
  }
  size_t pending() { return queue_.pending(); }
 private:
  WorkQueue queue_;
  WorkPusher pusher_;
  WorkPuller puller_;
  std::map<unsigned, Callback> callbacks_;
  std::thread thread_;
};

}  // namespace geeps_b200
