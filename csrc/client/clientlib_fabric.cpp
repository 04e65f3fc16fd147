// ClientLib NVLINK transport: every rank owns one device arena with the same layout (parameter
// cache, bf16 compute copy, update ring, shard master + momentum, clock flags per table), maps the
// other ranks' arenas through CUDA IPC (handles travel over the TCP control plane), and drives the
// sm_100a push / apply / publish kernels of kernels/ps_fabric.cu.
//
// This path replaces, per clock and table, the reference's D2H + ZeroMQ push
// (src/client/clientlib-data.cpp:436-522), the host apply (src/server/tablet-server.cpp:119-134), the
// whole-shard broadcast (src/server/tablet-server.cpp:147-163) and the pinned-bounce install
// (src/client/clientlib-data.cpp:110-151).  Peer memory is only touched with plain loads/stores and
// flag words; no TMA and no multicast object is involved.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "clientlib.hpp"
#include "kernels/kernels.h"

namespace geeps_b200 {

namespace {
struct IpcBlob {
  uint32_t pid;
  int32_t device;
  cudaIpcMemHandle_t handle;
  uint64_t raw_ptr;
  uint64_t bytes;
  int32_t phase;        // 0: capability round (can this rank use the multicast arena?), 1: handle round
  int32_t mc_capable;
};
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
constexpr size_t kFlagBytes = 256;
constexpr size_t kPushReadyOff = 0, kDataAgeOff = 32, kGlobalClockOff = 64, kCtaCounterOff = 68, kPublishBeginOff = 96;
constexpr size_t kPushTimingRing = 64;
constexpr size_t kPullCounterOff = 72;    // per table: scratch counter of the pull kernel (beside the push kernel's)
constexpr size_t kDeviceClockOff = 64;    // inside the 256-byte status area, after the 4 status words
}  // namespace

float* ClientLib::fabric_cache_ptr(uint table_id, int rank) const {
  return reinterpret_cast<float*>(fabric_.peer_base[rank] + fabric_.tables[table_id].cache_off);
}

float* ClientLib::fabric_ring_ptr(uint table_id, int rank, iter_t clock) const {
  const TableArena& ta = fabric_.tables[table_id];
  const size_t slot = (size_t)(clock % ta.ring_slots);
  return reinterpret_cast<float*>(fabric_.peer_base[rank] + ta.ring_off + slot * ta.rows * kRowBytes);
}

bool ClientLib::fabric_setup(std::string* err) {
  // ---- layout (identical on every rank: it only depends on the plan) ----
  size_t off = 0;
  fabric_.tables.assign(config_.num_tables, TableArena());
  for (auto& kv : plan_.tables) {
    const TablePlan& tp = kv.second;
    TableArena& ta = fabric_.tables[tp.table_id];
    ta.rows = tp.rows.size();
    ta.ring_slots = tp.num_oplog_entries;
    for (const ShardRange& r : tp.shard_ranges) ta.max_owned = std::max(ta.max_owned, r.count);
    ta.pull = tp.pull;
    if (!ta.pull) {
      ta.cache_off = off; off = align_up(off + ta.rows * kRowBytes, 256);
      if (config_.bf16_compute_cache) { ta.cache16_off = off; off = align_up(off + ta.rows * kRowBytes / 2, 256); }
    } else {
      // uncached: the shard keeps a bf16 copy of the rows it owns; the worker only has room for the fp32 tail
      if (config_.bf16_compute_cache) { ta.master16_off = off; off = align_up(off + ta.max_owned * kRowBytes / 2, 256); }
      ta.tail_from = tp.table_id < config_.table_fp32_from_row.size() ? config_.table_fp32_from_row[tp.table_id] : 0;
      if (ta.tail_from > ta.rows) ta.tail_from = ta.rows;
      ta.tail_rows = ta.tail_from > 0 ? ta.rows - ta.tail_from : 0;     // 0: no split, a generic Read pulls everything
      if (ta.tail_rows) { ta.tail_off = off; off = align_up(off + ta.tail_rows * kRowBytes, 256); }
    }
    ta.ring_off = off; off = align_up(off + (size_t)ta.ring_slots * ta.rows * kRowBytes, 256);
    ta.master_off = off; off = align_up(off + ta.max_owned * kRowBytes, 256);
    ta.momentum_off = off; off = align_up(off + ta.max_owned * kRowBytes, 256);
    ta.flags_off = off; off += kFlagBytes;
  }
  fabric_.status_off = off;
  off += 256;
  fabric_.bytes = off;
  int my_device = 0;
  cudaGetDevice(&my_device);
  // every rank sends one blob per round; a round is complete when all blobs of that phase are in
  auto exchange = [&](const IpcBlob& mine_blob, std::vector<IpcBlob>* all) -> bool {
    std::vector<char> blob(sizeof(IpcBlob));
    memcpy(blob.data(), &mine_blob, sizeof(IpcBlob));
    const uint round = (uint)mine_blob.phase;
    encoder_->ipc_exchange(blob, round);
    std::unique_lock<std::mutex> lk(global_mu_);
    const bool got = global_cv_.wait_for(lk, std::chrono::seconds(120), [&] {
      if (error_code_.load() != 0) return true;
      for (uint r = 0; r < num_processes_; ++r) {
        auto it = ipc_blobs_.find(r + kIpcRoundStride * round);
        if (it == ipc_blobs_.end() || it->second.size() != sizeof(IpcBlob)) return false;
      }
      return true;
    });
    if (!got || error_code_.load()) return false;
    all->assign(num_processes_, IpcBlob());
    for (uint r = 0; r < num_processes_; ++r)
      memcpy(&(*all)[r], ipc_blobs_[r + kIpcRoundStride * round].data(), sizeof(IpcBlob));
    return true;
  };
  // ---- multicast arena (optional): agree first, so that either every rank uses it or none does ----
  bool use_mc = false;
  if (config_.use_multicast && num_processes_ > 1) {
    std::string mc_err;
    IpcBlob cap;
    memset(&cap, 0, sizeof(cap));
    cap.pid = (uint32_t)getpid();
    cap.device = my_device;
    cap.bytes = fabric_.bytes;
    cap.phase = 0;
    cap.mc_capable = MulticastArena::device_supported(my_device) && fabric_.mc.allocate(fabric_.bytes, my_device, &mc_err);
    if (!cap.mc_capable) fprintf(stderr, "[geeps worker %u] multicast arena not available: %s\n", process_id_, mc_err.c_str());
    std::vector<IpcBlob> all;
    if (!exchange(cap, &all)) { *err = "timed out agreeing on the multicast arena with the other ranks"; return false; }
    use_mc = true;
    for (uint r = 0; r < num_processes_; ++r) {
      use_mc = use_mc && all[r].mc_capable != 0 && all[r].bytes == fabric_.bytes;
      for (uint q = 0; q < r; ++q) use_mc = use_mc && all[q].pid != all[r].pid;     // one process per rank only
    }
    if (!use_mc) fabric_.mc.release();
  }
  if (use_mc) {
    const std::string tag = std::to_string(ServerThreadEntry::port_for(config_, 0, 0));
    std::string mc_err;
    // Nothing is bound before every rank has come this far without an error: up to the bind a failing rank can
    // still leave and the others fall into their timeouts with plain memory.
    bool ok = fabric_.mc.listen(tag, (int)process_id_, &mc_err);
    ok = host_barrier(120000) && ok && error_code_.load() == 0;
    ok = ok && fabric_.mc.send_handles(tag, (int)process_id_, (int)num_processes_, &mc_err);
    ok = ok && fabric_.mc.receive_and_map((int)process_id_, (int)num_processes_, &mc_err);
    if (!ok) set_error(ERR_TRANSPORT, "multicast arena: " + mc_err);
    if (!host_barrier(120000) || error_code_.load()) { *err = "multicast arena setup failed: " + mc_err; return false; }
    if (!fabric_.mc.bind_and_map(&mc_err)) { *err = "multicast arena: " + mc_err; return false; }
    fabric_.use_mc = true;
    fabric_.base = fabric_.mc.base();
    fabric_.mc_base = fabric_.mc.multicast_base();
    fabric_.peer_base.assign(num_processes_, nullptr);
    for (uint r = 0; r < num_processes_; ++r) fabric_.peer_base[r] = fabric_.mc.peer((int)r);
    cudaMemset(fabric_.base, 0, fabric_.bytes);
    cudaDeviceSynchronize();
    if (!host_barrier(120000) || error_code_.load()) { *err = "barrier after multicast binding failed"; return false; }
  }
  void* base = fabric_.base;
  cudaError_t e = cudaSuccess;
  if (!use_mc) {
    e = cudaMalloc(&base, fabric_.bytes);
    if (e != cudaSuccess) { *err = std::string("arena cudaMalloc: ") + cudaGetErrorString(e); cudaGetLastError(); return false; }
    cudaMemset(base, 0, fabric_.bytes);
    cudaDeviceSynchronize();
    fabric_.base = static_cast<char*>(base);
    fabric_.peer_base.assign(num_processes_, nullptr);
    fabric_.peer_base[process_id_] = fabric_.base;
  }

  // ---- exchange arena handles over the control plane ----
  if (num_processes_ > 1 && !use_mc) {
    IpcBlob mine;
    memset(&mine, 0, sizeof(mine));
    mine.pid = (uint32_t)getpid();
    mine.phase = 1;
    cudaGetDevice(&mine.device);
    mine.raw_ptr = (uint64_t)(uintptr_t)base;
    mine.bytes = fabric_.bytes;
    e = cudaIpcGetMemHandle(&mine.handle, base);
    if (e != cudaSuccess) { *err = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e); cudaGetLastError(); return false; }
    std::vector<IpcBlob> all;
    if (!exchange(mine, &all)) { *err = "timed out exchanging arena handles with the other ranks"; return false; }
    for (uint r = 0; r < num_processes_; ++r) {
      if (r == process_id_) continue;
      const IpcBlob theirs = all[r];
      if (theirs.bytes != fabric_.bytes) { *err = "rank " + std::to_string(r) + " compiled a different plan"; return false; }
      if (theirs.pid == mine.pid) {
        // ranks living in one process (threads): plain pointers, peer access enabled explicitly
        if (theirs.device != mine.device) {
          cudaError_t pe = cudaDeviceEnablePeerAccess(theirs.device, 0);
          if (pe != cudaSuccess && pe != cudaErrorPeerAccessAlreadyEnabled) {
            *err = std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(pe);
            cudaGetLastError();
            return false;
          }
          cudaGetLastError();
        }
        fabric_.peer_base[r] = reinterpret_cast<char*>((uintptr_t)theirs.raw_ptr);
      } else {
        void* p = nullptr;
        e = cudaIpcOpenMemHandle(&p, theirs.handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { *err = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e); cudaGetLastError(); return false; }
        fabric_.peer_base[r] = static_cast<char*>(p);
      }
    }
    if (!host_barrier(120000) || error_code_.load()) { *err = "barrier after arena mapping failed"; return false; }
  }
  {
    // One comm stream at the lowest priority: the application's stream (created with a higher priority by
    // the caller, if it wants) gets its CTAs dispatched first, the pushes fill in behind.  Several lanes
    // (small tables ahead of the large fully-connected ones) were measured and were not faster.
    int prio_lo = 0, prio_hi = 0;     // numerically lowest = greatest priority
    cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    cudaStream_t cs;
    cudaStreamCreateWithPriority(&cs, cudaStreamNonBlocking, prio_lo);
    fabric_.comm_lanes.assign(1, cs);
    fabric_.comm_stream = cs;
    // one comm lane (stream) per comm channel; a table's pushes always ride the lane of its channel
    for (uint c = 1; c < num_channels(); ++c) {
      cudaStream_t lane;
      cudaStreamCreateWithPriority(&lane, cudaStreamNonBlocking, prio_lo);
      fabric_.comm_lanes.push_back(lane);
    }
    for (size_t t = 0; t < fabric_.tables.size(); ++t) fabric_.tables[t].comm_lane = (int)channel_of((uint)t);
    if (const char* e = getenv("GEEPS_PUSH_CTAS")) fabric_.push_ctas = atoi(e);
    if (const char* e = getenv("GEEPS_TIMELINE")) fabric_.timeline = atoi(e) != 0;
  }
  cudaHostAlloc(reinterpret_cast<void**>(&fabric_.host_status), 4 * sizeof(int), cudaHostAllocDefault);
  memset(fabric_.host_status, 0, 4 * sizeof(int));
  fabric_.active = true;
  return true;
}

void ClientLib::fabric_teardown() {
  if (!fabric_.base) return;
  cudaDeviceSynchronize();
  if (num_processes_ > 1 && error_code_.load() != 0) {
    // This rank leaves on an error without the closing barrier: healthy peers may still have kernels in flight
    // that store into this arena through their mappings, and freeing exported memory under them is undefined.
    // The arena and the mappings stay until the process exits (the driver reclaims them then).
    fabric_.active = false;
    return;
  }
  const uint32_t pid = (uint32_t)getpid();
  for (uint r = 0; r < num_processes_ && !fabric_.use_mc; ++r) {
    if (r == process_id_ || !fabric_.peer_base[r]) continue;
    bool same_process = false;
    {
      std::lock_guard<std::mutex> lk(global_mu_);
      std::vector<char>& blob = ipc_blobs_[r + kIpcRoundStride * 1];
      if (blob.size() == sizeof(IpcBlob)) {
        IpcBlob b;
        memcpy(&b, blob.data(), sizeof(b));
        same_process = b.pid == pid;
      }
    }
    if (!same_process) cudaIpcCloseMemHandle(fabric_.peer_base[r]);
  }
  for (Fabric::PushTiming& pt : fabric_.push_timing) {
    if (pt.begin) cudaEventDestroy((cudaEvent_t)pt.begin);
    if (pt.end) cudaEventDestroy((cudaEvent_t)pt.end);
  }
  fabric_.push_timing.clear();
  for (void* e : fabric_.table_events) if (e) cudaEventDestroy((cudaEvent_t)e);
  fabric_.table_events.clear();
  if (fabric_.join_event) { cudaEventDestroy((cudaEvent_t)fabric_.join_event); fabric_.join_event = nullptr; }
  for (void* cs : fabric_.comm_lanes) cudaStreamDestroy((cudaStream_t)cs);
  fabric_.comm_lanes.clear();
  fabric_.comm_stream = nullptr;
  if (fabric_.host_status) cudaFreeHost(fabric_.host_status);
  // the ranks left their last clock together (closing barrier in shutdown()): nothing uses the mappings any more
  if (fabric_.use_mc) fabric_.mc.release();
  else cudaFree(fabric_.base);
  fabric_.use_mc = false;
  fabric_.mc_base = nullptr;
  fabric_.base = nullptr;
  fabric_.active = false;
}

// Device-side SSP wait: the stream stalls (bounded) until every shard stamped data_age >= needed+1.
void ClientLib::fabric_wait_data_age(CachedTable& ct, uint table_id, iter_t needed_age, void* stream) {
  const iter_t stamp = needed_age + 1;
  if (stamp <= 0 || stamp <= ct.waited_floor) return;
  // a wait kernel orders only the stream it was enqueued on: another stream that touches the table in the same
  // clock needs its own
  std::pair<void*, iter_t>* mine = nullptr;
  for (auto& w : ct.waited_by_stream) if (w.first == stream) mine = &w;
  if (mine && stamp <= mine->second) return;
  const TableArena& ta = fabric_.tables[table_id];
  const int* flags = reinterpret_cast<const int*>(fabric_.base + ta.flags_off + kDataAgeOff);
  geeps_flag_wait_rel(flags, (int)num_processes_, stamp_arg(stamp), clock_ref(),
                      (unsigned long long)config_.device_wait_budget_us * 1000ull,
                      reinterpret_cast<int*>(fabric_.base + fabric_.status_off), stream);
  if (mine) mine->second = stamp; else ct.waited_by_stream.emplace_back(stream, stamp);
  stats_.device_waits_enqueued++;
}

// Push of (clock, table): announce "my update is complete" to every shard on the application's
// stream, then - on the comm stream - wait for all workers' announcements and run the fused
// reduce + apply + publish kernel for the rows this rank owns.
void ClientLib::fabric_push(iter_t clock, uint table_id, bool is_init, void* stream) {
  CachedTable& ct = *tables_[table_id];
  const TableArena& ta = fabric_.tables[table_id];
  const int stamp = clock + 1;
  int* status = reinterpret_cast<int*>(fabric_.base + fabric_.status_off);
  if (!withhold_push_signal_) {
    GeepsFlagList list;
    memset(&list, 0, sizeof(list));
    list.n = (int)num_processes_;
    for (uint r = 0; r < num_processes_; ++r)
      list.ptr[r] = reinterpret_cast<int*>(fabric_.peer_base[r] + ta.flags_off + kPushReadyOff);
    geeps_flag_signal_rel(&list, (int)process_id_, stamp_arg(stamp), clock_ref(), stream);
  }
  // The comm stream does not even start waiting before this worker's own announcement has run: the host
  // enqueues a whole step ahead of the GPU, and a wait kernel that started right away would sit spinning on
  // an SM through the entire forward pass, next to the compute kernels.
  if (fabric_.table_events.size() <= table_id) fabric_.table_events.resize(table_id + 1, nullptr);
  if (!fabric_.table_events[table_id]) {
    cudaEvent_t e;
    cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    fabric_.table_events[table_id] = e;
  }
  cudaEventRecord((cudaEvent_t)fabric_.table_events[table_id], (cudaStream_t)stream);
  cudaStreamWaitEvent((cudaStream_t)fabric_.comm_lanes[ta.comm_lane], (cudaEvent_t)fabric_.table_events[table_id], 0);
  void* cs = fabric_.comm_lanes[ta.comm_lane];
  Fabric::TimelineRec rec = {table_id, (int)clock, nullptr, nullptr, nullptr};
  const bool timed = fabric_.timeline && !is_init && fabric_.timeline_recs.size() < 4096;
  if (timed) {
    cudaEvent_t e0, e1, e2;
    cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
    rec.handed = e0; rec.arrived = e1; rec.applied = e2;
    if (!fabric_.timeline_origin) {
      cudaEvent_t o;
      cudaEventCreate(&o);
      cudaEventRecord(o, (cudaStream_t)stream);
      fabric_.timeline_origin = o;
    }
    cudaEventRecord(e0, (cudaStream_t)stream);
  }
  const unsigned long long budget = (unsigned long long)config_.device_wait_budget_us * 1000ull;
  if (config_.read_my_writes && ct.plan->slack > 0) {
    // readers that merge their own pending updates need to know when a publish is in progress: mark its begin on
    // every worker before the first row is stored (the data_age stamp after the last row marks its end)
    GeepsFlagList begin;
    memset(&begin, 0, sizeof(begin));
    begin.n = (int)num_processes_;
    for (uint r = 0; r < num_processes_; ++r)
      begin.ptr[r] = reinterpret_cast<int*>(fabric_.peer_base[r] + ta.flags_off + kPublishBeginOff);
    geeps_flag_wait_signal_rel(reinterpret_cast<const int*>(fabric_.base + ta.flags_off + kPushReadyOff),
                               (int)num_processes_, stamp_arg(stamp), clock_ref(), budget, status, &begin,
                               (int)process_id_, cs);
  } else {
    geeps_flag_wait_rel(reinterpret_cast<const int*>(fabric_.base + ta.flags_off + kPushReadyOff), (int)num_processes_,
                        stamp_arg(stamp), clock_ref(), budget, status, cs);
  }
  // device time of the push kernel itself (the wait for the other workers is not part of it)
  Fabric::PushTiming* pt = nullptr;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing((cudaStream_t)cs, &capturing);
  if (!is_init && capturing == cudaStreamCaptureStatusNone) {   // an event recorded under capture cannot be queried
    if (fabric_.push_timing.empty()) fabric_.push_timing.resize(kPushTimingRing);
    pt = &fabric_.push_timing[fabric_.push_timing_next++ % kPushTimingRing];
    if (!pt->begin) {
      cudaEvent_t a, b;
      cudaEventCreate(&a); cudaEventCreate(&b);
      pt->begin = a; pt->end = b;
    }
    pt->table_bytes = ta.rows * kRowBytes;
    pt->armed = true;
    cudaEventRecord((cudaEvent_t)pt->begin, (cudaStream_t)cs);
  }
  GeepsPushApplyParams p;
  memset(&p, 0, sizeof(p));
  for (uint r = 0; r < num_processes_; ++r) {
    p.upd[r] = fabric_ring_ptr(table_id, (int)r, clock);
    p.cache[r] = ta.pull ? nullptr : fabric_cache_ptr(table_id, (int)r);
    p.cache16[r] = (config_.bf16_compute_cache && !ta.pull) ? (void*)(fabric_.peer_base[r] + ta.cache16_off) : nullptr;
    p.data_age[r] = reinterpret_cast<int*>(fabric_.peer_base[r] + ta.flags_off + kDataAgeOff);
  }
  p.master16 = (ta.pull && config_.bf16_compute_cache) ? (void*)(fabric_.base + ta.master16_off) : nullptr;
  // The switch path moves fewer bytes per link once there are several peers (each row crosses a link once instead
  // of once per peer) but a row's round trip is longer: measured, it wins from 4 ranks on for tables of tens of MB,
  // and loses for small tables and for 2 ranks (GEEPS_MC_MIN_MB / GEEPS_MC_MIN_RANKS move the thresholds).
  static const long long mc_min_bytes = (getenv("GEEPS_MC_MIN_MB") ? atoll(getenv("GEEPS_MC_MIN_MB")) : 32) << 20;
  static const int mc_min_ranks = getenv("GEEPS_MC_MIN_RANKS") ? atoi(getenv("GEEPS_MC_MIN_RANKS")) : 4;
  if (fabric_.use_mc && fabric_.mc_base != nullptr && (long long)(ta.rows * kRowBytes) >= mc_min_bytes &&
      (int)num_processes_ >= mc_min_ranks) {
    // through the multicast view: one in-switch reduction per row instead of a load per worker, one store per
    // row instead of a store per worker
    const size_t slot = (size_t)(clock % ta.ring_slots);
    p.upd_mc = reinterpret_cast<const float*>(fabric_.mc_base + ta.ring_off + slot * ta.rows * kRowBytes);
    if (!ta.pull) {
      p.cache_mc = reinterpret_cast<float*>(fabric_.mc_base + ta.cache_off);
      p.cache16_mc = config_.bf16_compute_cache ? (void*)(fabric_.mc_base + ta.cache16_off) : nullptr;
    }
  }
  const ShardRange& own = ct.plan->shard_ranges[process_id_];
  p.master = reinterpret_cast<float*>(fabric_.base + ta.master_off);
  p.momentum = reinterpret_cast<float*>(fabric_.base + ta.momentum_off);
  p.push_ready = nullptr;   // already awaited by the one-warp wait kernel above, which occupies no SM worth of CTAs
  p.global_clock = reinterpret_cast<int*>(fabric_.base + ta.flags_off + kGlobalClockOff);
  p.cta_counter = reinterpret_cast<int*>(fabric_.base + ta.flags_off + kCtaCounterOff);
  p.status = status;
  p.n_owned = (long long)own.count;
  p.row_start = (long long)own.start;
  p.row_stride = (long long)own.stride;
  p.total_rows = (long long)ta.rows;
  p.wait_budget_ns = budget;
  p.n_ranks = (int)num_processes_;
  p.rank = (int)process_id_;
  p.clock_stamp = stamp_arg(stamp);
  p.clock_ref = clock_ref();
  p.mode = is_init ? GEEPS_TABLE_ADDITIVE : ct.mode;
  p.publish = 1;
  const HyperSchedule::Entry hyper = hyper_->at(clock);      // the values in force for the updates of this clock
  p.lr = hyper.lr;
  p.momentum_coef = hyper.momentum;
  p.weight_decay = hyper.weight_decay;
  p.grad_scale = config_.grad_scale;
  p.fp32_from_row = (!is_init && config_.bf16_compute_cache && table_id < config_.table_fp32_from_row.size())
                        ? (long long)config_.table_fp32_from_row[table_id] : 0;
  if (timed) cudaEventRecord((cudaEvent_t)rec.arrived, (cudaStream_t)cs);
  geeps_ps_push_apply(&p, fabric_.push_ctas, cs);
  if (pt) cudaEventRecord((cudaEvent_t)pt->end, (cudaStream_t)cs);
  if (timed) {
    cudaEventRecord((cudaEvent_t)rec.applied, (cudaStream_t)cs);
    fabric_.timeline_recs.push_back(rec);
  }
  bg_stats_.nr_push++;
  bg_stats_.bytes_pushed += ta.rows * kRowBytes;
}

// Sum the device time of the pushes in the timing ring that have completed since the last call.
void ClientLib::fabric_collect_push_timing() {
  if (!fabric_.active) return;
  for (Fabric::PushTiming& pt : fabric_.push_timing) {
    if (!pt.armed || cudaEventQuery((cudaEvent_t)pt.end) != cudaSuccess) { cudaGetLastError(); continue; }
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, (cudaEvent_t)pt.begin, (cudaEvent_t)pt.end) == cudaSuccess) {
      bg_stats_.device_push_ms += ms;
      bg_stats_.device_push_bytes += pt.table_bytes;
      bg_stats_.device_push_samples++;
    } else {
      cudaGetLastError();
    }
    pt.armed = false;
  }
}

// Staged Read with read-my-updates: the worker's private copy = cache rows + its own updates that the owning
// shards have not published yet (additive tables: the updates themselves; optimizer tables: the plain gradient
// step -lr * grad_scale * g as a provisional value).  Counterpart of the reference's replay of the oplog onto
// freshly received rows (src/client/clientlib-data.cpp:132-150), done at read time because here the shards write
// the cache in place.
void ClientLib::fabric_read_rmw(const OpInfo& op, RowData* dst, void* stream) {
  CachedTable& ct = *tables_[(uint)op.table];
  const TableArena& ta = fabric_.tables[op.table];
  GeepsRmwReadParams p;
  memset(&p, 0, sizeof(p));
  p.dst = reinterpret_cast<float*>(dst);
  p.cache = fabric_cache_ptr((uint)op.table, (int)process_id_);
  p.ring = reinterpret_cast<const float*>(fabric_.base + ta.ring_off);
  p.index = op_index_dev_[&op - &plan_.ops[0]];
  p.data_age = reinterpret_cast<const int*>(fabric_.base + ta.flags_off + kDataAgeOff);
  p.publish_begin = reinterpret_cast<const int*>(fabric_.base + ta.flags_off + kPublishBeginOff);
  p.status = reinterpret_cast<int*>(fabric_.base + fabric_.status_off);
  p.num_rows = (long long)op.rows.size();
  p.num_vals_limit = (long long)op.num_vals_limit;
  p.dst_rows = (long long)op.rows.size();
  p.total_rows = (long long)ta.rows;
  p.wait_budget_ns = (unsigned long long)config_.device_wait_budget_us * 1000ull;
  p.n_ranks = (int)num_processes_;
  p.partition_kind = config_.partitioner;
  p.partition_per = (long long)ct.plan->partition_per;
  p.ring_slots = ta.ring_slots;
  p.clock = stamp_arg(clock_);
  p.clock_ref = clock_ref();
  p.additive_below_clock = bootstrap_init_pushed_ ? (int)kInitialClock + 1 : 0;
  p.alpha = ct.mode == GeePsConfig::TABLE_SGD_MOMENTUM ? -hyper_->at(clock_).lr * config_.grad_scale : 1.f;
  geeps_row_gather_rmw(&p, stream);
  bg_stats_.nr_rmw_replay++;
}

// ---- device-resident clock and replayed iterations ----
// With the device clock on, every stamp a launch carries is relative to a clock word in device memory that a
// one-thread kernel advances at the end of each iteration, after the comm streams have joined the application's
// stream.  An iteration's launches then contain nothing that changes from one clock to the next (for a fixed phase
// of the update ring), so the application can capture them once in a CUDA graph and replay the graph;
// advance_replayed_iteration() does the host-side bookkeeping of such a replay.
bool ClientLib::enable_device_clock() {
  if (!nvlink_ || !fabric_.active) { set_error(ERR_ORDER, "the device clock needs the NVLINK transport after FinishVirtualIteration"); return false; }
  if (device_clock_) return true;
  cudaDeviceSynchronize();
  const int now = (int)clock_;
  cudaMemcpy(fabric_.base + fabric_.status_off + kDeviceClockOff, &now, sizeof(int), cudaMemcpyHostToDevice);
  device_clock_ = reinterpret_cast<int*>(fabric_.base + fabric_.status_off + kDeviceClockOff);
  return true;
}

// End of an iteration in device-clock mode: everything the iteration put on the comm streams completes before
// the clock word moves (a push kernel that ran after the advance would read the next clock's value).
void ClientLib::fabric_end_iteration_device_clock() {
  cudaStream_t app = (cudaStream_t)(last_app_stream_ ? last_app_stream_ : default_stream_);
  if (!fabric_.join_event) {
    cudaEvent_t e;
    cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    fabric_.join_event = e;
  }
  for (void* cs : fabric_.comm_lanes) {
    cudaEventRecord((cudaEvent_t)fabric_.join_event, (cudaStream_t)cs);
    cudaStreamWaitEvent(app, (cudaEvent_t)fabric_.join_event, 0);
  }
  geeps_clock_advance(device_clock_, app);
}

void ClientLib::advance_replayed_iteration() {
  if (!device_clock_ || !started_) { set_error(ERR_ORDER, "advance_replayed_iteration without the device clock"); return; }
  for (auto& kv : tables_) {
    CachedTable& ct = *kv.second;
    ct.signalled_clock = clock_;
    for (auto& w : ct.waited_by_stream) w.second += 1;
    if (ct.ring_zeroed_clock == clock_ - 1) ct.ring_zeroed_clock = clock_;
    bg_stats_.nr_push++;
    bg_stats_.bytes_pushed += ct.plan->rows.size() * kRowBytes;
  }
  for (int h = 0; h < plan_.clock_handle; ++h) {
    const OpInfo& op = plan_.ops[h];
    accessed_clock_[h] = clock_;
    if (op.type == OP_READ) { stats_.nr_read++; stats_.rows_read += op.rows.size(); }
    else if (op.type == OP_POST_READ) stats_.nr_postread++;
    else if (op.type == OP_PRE_UPDATE) stats_.nr_preupdate++;
    else if (op.type == OP_UPDATE) { stats_.nr_update++; stats_.rows_updated += plan_.ops[op.prestep].rows.size(); }
  }
  clock_++;
  last_handle_ = -1;
  stats_.nr_clock++;
  stats_.nr_replayed_clocks++;
  // the replayed graph refreshed the pinned mirror of the status block: look at it without enqueuing anything
  if (fabric_.host_status[0] != 0) {
    const int code = fabric_.host_status[0];
    if (code == 1) stats_.device_wait_timeouts++;
    set_error(code == 1 ? ERR_DEVICE_TIMEOUT : ERR_CUDA,
              std::string(code == 1 ? "device-side wait expired" : "device-side check failed") + " (kernel " +
                  std::to_string(fabric_.host_status[1]) + ", detail " + std::to_string(fabric_.host_status[2]) +
                  ", seen " + std::to_string(fabric_.host_status[3]) + ")");
  }
}

// Rows [row_from, end) of an uncached table, fetched from the master rows of the shards that own them into `dst`
// (row row_from lands at dst[0]).  The stream has already waited for the table's freshness condition, and a
// shard stamps data_age only after its master rows are written, so the kernel needs no wait of its own.
void ClientLib::fabric_pull_rows(uint table_id, RowData* dst, size_t row_from, void* stream) {
  CachedTable& ct = *tables_[table_id];
  const TableArena& ta = fabric_.tables[table_id];
  GeepsPullParams p;
  memset(&p, 0, sizeof(p));
  for (uint s = 0; s < num_processes_; ++s) {
    const ShardRange& r = ct.plan->shard_ranges[s];
    p.master[s] = reinterpret_cast<const float*>(fabric_.peer_base[s] + ta.master_off);
    p.global_clock[s] = nullptr;
    p.n_owned[s] = (long long)r.count;
    p.row_start[s] = (long long)r.start;
    p.row_stride[s] = (long long)r.stride;
  }
  p.cache = reinterpret_cast<float*>(dst);
  p.cache16 = nullptr;
  p.data_age_local = nullptr;
  p.cta_counter = reinterpret_cast<int*>(fabric_.base + ta.flags_off + kPullCounterOff);
  p.status = reinterpret_cast<int*>(fabric_.base + fabric_.status_off);
  p.total_rows = (long long)ta.rows;
  p.wait_budget_ns = (unsigned long long)config_.device_wait_budget_us * 1000ull;
  p.n_ranks = (int)num_processes_;
  p.rank = (int)process_id_;
  p.needed_stamp = 0;
  p.row_from = (long long)row_from;
  p.row_base = (long long)row_from;
  geeps_ps_pull(&p, 0, stream);
  stats_.rows_pulled += ta.rows - row_from;
}

// Errors recorded by kernels (expired waits, failed bounds checks) surface here.  The device block
// is mirrored into pinned memory asynchronously, so a problem is seen at most one clock late
// without ever synchronising the streams.
bool ClientLib::fabric_check_status(bool sync) {
  if (!fabric_.active) return true;
  bool ok = true;
  if (sync)   // the caller has synchronised the streams: read the block itself
    cudaMemcpy(fabric_.host_status, fabric_.base + fabric_.status_off, 4 * sizeof(int), cudaMemcpyDeviceToHost);
  if (fabric_.host_status[0] != 0) {
    ok = false;
    const int code = fabric_.host_status[0];
    if (code == 1) stats_.device_wait_timeouts++;
    set_error(code == 1 ? ERR_DEVICE_TIMEOUT : ERR_CUDA,
              std::string(code == 1 ? "device-side wait expired" : "device-side check failed") + " (kernel " +
                  std::to_string(fabric_.host_status[1]) + ", detail " + std::to_string(fabric_.host_status[2]) +
                  ", seen " + std::to_string(fabric_.host_status[3]) + ")");
  }
  cudaMemcpyAsync(fabric_.host_status, fabric_.base + fabric_.status_off, 4 * sizeof(int), cudaMemcpyDeviceToHost,
                  (cudaStream_t)fabric_.comm_stream);
  return ok;
}

// Milliseconds since the first recorded push, per (table, clock): update handed over on the application's
// stream / all workers' updates arrived / apply + publish finished.  Synchronises the device.
std::string ClientLib::fabric_timeline_json() {
  if (!fabric_.active || !fabric_.timeline || fabric_.timeline_recs.empty()) return "[]";
  cudaDeviceSynchronize();
  std::string out = "[";
  bool first = true;
  for (const Fabric::TimelineRec& r : fabric_.timeline_recs) {
    float a = 0, b = 0, c = 0;
    cudaEvent_t o = (cudaEvent_t)fabric_.timeline_origin;
    if (cudaEventElapsedTime(&a, o, (cudaEvent_t)r.handed) != cudaSuccess ||
        cudaEventElapsedTime(&b, o, (cudaEvent_t)r.arrived) != cudaSuccess ||
        cudaEventElapsedTime(&c, o, (cudaEvent_t)r.applied) != cudaSuccess) { cudaGetLastError(); continue; }
    char buf[160];
    snprintf(buf, sizeof(buf), "%s{\"table\":%u,\"clock\":%d,\"handed\":%.4f,\"arrived\":%.4f,\"applied\":%.4f}",
             first ? "" : ",", r.table, r.clock, a, b, c);
    out += buf;
    first = false;
  }
  return out + "]";
}

}  // namespace geeps_b200
