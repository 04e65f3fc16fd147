// ClientLib background machinery: the plan-driven swapper for host-resident local rows (prefetch
// one access ahead and evict on a side stream), per-table clock signalling through the push worker,
// the heartbeat failure detector and the host barrier.
//
// The reference runs two threads per application thread for this (alloc_worker_entry /
// reclaim_worker_entry, src/client/clientlib-bg-access.cpp:83-573) with a condition variable per
// buffer slot; here buffers have fixed offsets from the plan and ordering is expressed with CUDA
// events between the application's stream and the swap stream.
#include <cuda_runtime.h>
#include <stdio.h>

#include "clientlib.hpp"

namespace geeps_b200 {

namespace {
struct IterateArgs { iter_t clock; uint table_id; int is_init; };
bool overlaps(const OpInfo& a, const OpInfo& b) {
  return a.staging_offset < b.staging_offset + b.rows.size() && b.staging_offset < a.staging_offset + a.rows.size();
}
bool is_pre(OpType t) { return t == OP_READ || t == OP_PRE_UPDATE || t == OP_LOCAL_ACCESS; }
}  // namespace

// ---------------- swapper ----------------
void ClientLib::swap_init() {
  const size_t n = plan_.ops.size();
  fetch_done_ev_.assign(n, nullptr);
  release_ev_.assign(n, nullptr);
  fetch_issued_clock_.assign(n, -1);
  accessed_clock_.assign(n, -1);
  released_clock_.assign(n, -1);
  if (!gpu_) return;
  for (size_t i = 0; i < n; ++i) {
    if (!is_pre(plan_.ops[i].type) || !plan_.ops[i].needs_staging) continue;
    cudaEvent_t a, b;
    cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
    fetch_done_ev_[i] = a;
    release_ev_[i] = b;
  }
}

// H2D of a host-resident local batch into its staging buffer on the swap stream, after every
// earlier user of an overlapping staging region has released it.
void ClientLib::swap_issue_fetch(int h) {
  const OpInfo& op = plan_.ops[h];
  for (size_t j = 0; j < plan_.ops.size(); ++j) {
    const OpInfo& o = plan_.ops[j];
    if ((int)j == h || !is_pre(o.type) || !o.needs_staging || !overlaps(o, op)) continue;
    if (released_clock_[j] >= 0 && release_ev_[j])
      cudaStreamWaitEvent((cudaStream_t)swap_stream_, (cudaEvent_t)release_ev_[j], 0);
  }
  if (released_clock_[h] >= 0) cudaStreamWaitEvent((cudaStream_t)swap_stream_, (cudaEvent_t)release_ev_[h], 0);
  const size_t bytes = op.rows.size() * sizeof(RowData);
  cudaMemcpyAsync(staging_ptr(op), local_.cpu.data() + op.store_offset, bytes, cudaMemcpyHostToDevice,
                  (cudaStream_t)swap_stream_);
  cudaEventRecord((cudaEvent_t)fetch_done_ev_[h], (cudaStream_t)swap_stream_);
  fetch_issued_clock_[h] = clock_;
  stats_.swap_h2d_bytes += bytes;
}

// `stream` may write the staging region of access h once every earlier user of an overlapping region has
// released it (an eviction copy to the host releases on the swap stream).
void ClientLib::swap_wait_region_free(int h, void* stream) {
  if (!gpu_) return;
  const OpInfo& op = plan_.ops[h];
  for (size_t j = 0; j < plan_.ops.size(); ++j) {
    const OpInfo& o = plan_.ops[j];
    if (!is_pre(o.type) || !o.needs_staging || !release_ev_[j] || released_clock_[j] < 0) continue;
    if ((int)j != h && !overlaps(o, op)) continue;
    cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)release_ev_[j], 0);
  }
}

// A later fetch may start now if no access that is live now, or that comes between now and the
// target, uses an overlapping staging region.
bool ClientLib::swap_can_prefetch(int current, int target) const {
  const OpInfo& t = plan_.ops[target];
  for (int j = 0; j < (int)plan_.ops.size(); ++j) {
    const OpInfo& o = plan_.ops[j];
    if (j == target || !is_pre(o.type) || !o.needs_staging || o.one_off || !overlaps(o, t)) continue;
    const bool live = accessed_clock_[j] == clock_ && released_clock_[j] != clock_;
    const bool between = j > current && j < target;
    if (live || between) return false;
  }
  return true;
}

void ClientLib::swap_prefetch_after(int h) {
  if (!started_) return;
  for (int j = h + 1; j < plan_.clock_handle; ++j) {
    const OpInfo& o = plan_.ops[j];
    if (o.type != OP_LOCAL_ACCESS || !o.needs_staging || !o.fetch) continue;
    if (fetch_issued_clock_[j] != clock_ && swap_can_prefetch(h, j)) swap_issue_fetch(j);
    break;   // look one fetch ahead
  }
}

void ClientLib::swap_release(int pre_handle, void* stream, bool) {
  if (!gpu_ || !release_ev_[pre_handle]) return;
  cudaEventRecord((cudaEvent_t)release_ev_[pre_handle], (cudaStream_t)stream);
  released_clock_[pre_handle] = clock_;
}

// ---------------- clock signalling ----------------
// "Signal clock c of table t": this worker's updates of clock c are complete.  On the host-staged
// path the push worker sends them; on NVLINK the push kernels are enqueued right here.
void ClientLib::clock_table(iter_t signalled_clock, uint table_id, bool is_init, bool synchronous, void* stream) {
  auto it = tables_.find(table_id);
  if (it == tables_.end()) return;
  CachedTable& ct = *it->second;
  if (signalled_clock <= ct.signalled_clock) return;
  ct.signalled_clock = signalled_clock;
  if (nvlink_) {
    // the announcement has to follow the application's update writes in stream order
    void* st = stream ? stream : (ct.last_stream ? ct.last_stream : default_stream_);
    fabric_push(signalled_clock, table_id, is_init, st);
    return;
  }
  if (synchronous) { push_updates_param_cache(signalled_clock, table_id, is_init); return; }
  IterateArgs a{signalled_clock, table_id, is_init ? 1 : 0};
  bg_workers_[channel_of(table_id) % bg_workers_.size()]->pusher()->push_work(kIterateCmd, a);
}

void ClientLib::clock_all(iter_t signalled_clock, bool is_init) {
  for (auto& kv : tables_) clock_table(signalled_clock, kv.first, is_init, true, nullptr);
}

void ClientLib::cbk_iterate(std::vector<char>& args) {
  if (args.size() < sizeof(IterateArgs)) return;
  IterateArgs a;
  memcpy(&a, args.data(), sizeof(a));
  const double t0 = now_seconds();
  push_updates_param_cache(a.clock, a.table_id, a.is_init != 0);
  stats_.iterate_time += now_seconds() - t0;
}

// ---------------- failure detection ----------------
void ClientLib::heartbeat_loop() {
  uint64_t counter = 0;
  const double timeout_s = (double)config_.heartbeat_timeout_ms / 1000.0;
  {
    std::lock_guard<std::mutex> lk(peers_mu_);
    for (double& t : last_heartbeat_) t = now_seconds();
  }
  while (!stop_heartbeat_) {
    if (!skip_heartbeats_ && encoder_) encoder_->heartbeat(++counter, clock_);
    {
      std::lock_guard<std::mutex> lk(peers_mu_);
      const double now = now_seconds();
      for (uint r = 0; r < num_processes_; ++r) {
        if (r == process_id_ || peer_dead_[r]) continue;
        if (now - last_heartbeat_[r] > timeout_s && !shut_down_) {
          peer_dead_[r] = 1;
          set_error(ERR_PEER_LOST, "no heartbeat from worker " + std::to_string(r) + " for " +
                                       std::to_string((int)timeout_s) + " s");
        }
      }
    }
    for (int i = 0; i < 10 && !stop_heartbeat_; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

bool ClientLib::host_barrier(int timeout_ms) {
  uint epoch;
  {
    std::lock_guard<std::mutex> lk(global_mu_);
    epoch = ++barrier_epoch_;
  }
  encoder_->barrier(epoch);
  std::unique_lock<std::mutex> lk(global_mu_);
  return global_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] {
    if (error_code_.load()) return true;
    for (uint r = 0; r < num_processes_; ++r)
      if (barrier_seen_[r] < epoch) return false;
    return true;
  });
}

}  // namespace geeps_b200
