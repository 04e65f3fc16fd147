// ClientLib data path: parameter-cache reads (with the SSP wait), update logging, the host-staged
// push to the tablet servers, installation of received rows with read-my-writes replay, and the
// copies of host-resident worker-local rows.  Counterpart of the reference's
// src/client/clientlib-data.cpp:51-600.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "clientlib.hpp"
#include "kernels/kernels.h"

namespace geeps_b200 {

namespace {
const long long kNoLimit = (long long)1 << 62;
}

// Wait (host side) until the cached table is fresh enough for a read in `clock` with `slack`:
// data_age >= clock - slack - 1 (the reference's admission rule,
// src/client/clientlib-bg-access.cpp:283 and src/client/clientlib-data.cpp:205), then gather.
bool ClientLib::read_row_batch_param_cache(const OpInfo& op, RowData* dst, void* stream) {
  CachedTable& ct = *tables_[(uint)op.table];
  const size_t n = op.rows.size();
  if (nvlink_ && ct.plan->pull) {
    // uncached table: fetch every row from the shard that owns it (the caller enqueued the freshness wait)
    fabric_pull_rows((uint)op.table, dst, 0, stream);
    return true;
  }
  if (nvlink_ && config_.read_my_writes && ct.plan->slack > 0) {
    fabric_read_rmw(op, dst, stream);
    return true;
  }
  if (nvlink_) {
    // device wait already enqueued by the caller; gather from the local arena cache
    const void* idx = op_index_dev_[&op - &plan_.ops[0]];
    geeps_row_gather(reinterpret_cast<float*>(dst), fabric_cache_ptr((uint)op.table, (int)process_id_), idx,
                     (long long)n, 0, 0, (long long)op.num_vals_limit, (long long)n, (long long)ct.plan->rows.size(),
                     fabric_.base ? reinterpret_cast<int*>(fabric_.base + fabric_.status_off) : nullptr, stream);
    return true;
  }
  const iter_t needed = clock_ - op.slack - 1;
  std::unique_lock<std::mutex> lk(ct.mu);
  const double t0 = now_seconds();
  double last_report = t0;
  while (ct.data_age < needed) {
    if (error_code_.load()) return false;
    ct.cv.wait_for(lk, std::chrono::milliseconds(200));
    const double now = now_seconds();
    if (now - last_report > kWatchdogSeconds) {
      last_report = now;
      fprintf(stderr, "[geeps worker %u] read of table %zu at clock %d still waits for data age %d (have %d)\n",
              process_id_, op.table, clock_, needed, ct.data_age);
    }
    if (config_.host_wait_budget_ms && (now - t0) * 1000.0 > (double)config_.host_wait_budget_ms) {
      stats_.host_wait_timeouts++;
      lk.unlock();
      set_error(ERR_HOST_TIMEOUT, "read of table " + std::to_string(op.table) + " at clock " + std::to_string(clock_) +
                                      " timed out waiting for data age " + std::to_string(needed));
      return false;
    }
  }
  stats_.read_wait_time += now_seconds() - t0;
  if (ct.data_age < kBigIter) {
    const int staleness = std::max(0, (int)(clock_ - 1 - ct.data_age));
    stats_.staleness_hist[std::min(staleness, 7)]++;
    stats_.max_staleness = std::max(stats_.max_staleness.get(), staleness);
  }
  const size_t op_idx = &op - &plan_.ops[0];
  if (op.location == LOC_GPU) {
    geeps_row_gather(reinterpret_cast<float*>(dst), ct.gpu.data_cache.floats(), op_index_dev_[op_idx], (long long)n, 0, 0,
                     (long long)op.num_vals_limit, (long long)n, (long long)ct.gpu.data_cache.size(), row_status(), stream);
    cudaStreamSynchronize((cudaStream_t)stream);   // the receiver may overwrite the cache once the lock drops
  } else if (gpu_) {
    // host-cached rows on a GPU worker: gather on the host into pinned staging, then H2D
    if (host_stage_.size() < n) host_stage_.init(std::max(n, plan_.max_access_rows), MEM_PINNED);
    assign_rows_to_double_index_cpu(host_stage_.data(), ct.cpu.data_cache.data(), op.index.data(), n, 0, 0, op.num_vals_limit);
    Mem::copy(dst, MEM_DEVICE, host_stage_.data(), MEM_PINNED, n * sizeof(RowData), stream, true);
    stats_.swap_h2d_bytes += n * sizeof(RowData);
  } else {
    assign_rows_to_double_index_cpu(dst, ct.cpu.data_cache.data(), op.index.data(), n, 0, 0, op.num_vals_limit);
  }
  return true;
}

// Called with ct.mu held.  The wait for a free entry happens with the lock released: the push
// worker needs the same lock to recycle entries.
FlatOps* ClientLib::create_oplog_entry(CachedTable& ct, ParamCache& pc, MemType, iter_t clock, void* stream) {
  auto it = pc.oplog.find(clock);
  if (it != pc.oplog.end()) return it->second;
  ct.mu.unlock();
  FlatOps* e = pc.pool.get(config_.host_wait_budget_ms);
  ct.mu.lock();
  if (!e) { set_error(ERR_HOST_TIMEOUT, "no free oplog entry for table " + std::to_string(ct.plan->table_id)); return nullptr; }
  e->data.zerofy(stream);
  if (e->data.type() == MEM_DEVICE) cudaStreamSynchronize((cudaStream_t)stream);
  e->flag = FlatOps::INC;
  e->clock = clock;
  e->rmw_alpha = rmw_alpha_for(ct, clock);
  pc.oplog[clock] = e;
  return e;
}

// What a logged update of `clock` contributes to this worker's own view of the rows under read-my-writes.
// Additive tables (and the initial values pushed during bootstrap, which every table adds): the update itself,
// exactly what the shard will add (src/client/clientlib-data.cpp:389-394 of the reference).  Optimizer tables:
// the shard's momentum step depends on the other workers' gradients, so the worker applies the plain gradient
// step -lr * grad_scale * g as a provisional value; the shard's rows replace it when they arrive, and updates
// the shard had not yet seen are re-applied the same way.
float ClientLib::rmw_alpha_for(const CachedTable& ct, iter_t clock) const {
  const bool is_init = !started_ && clock == kInitialClock;
  if (ct.mode == GeePsConfig::TABLE_SGD_MOMENTUM && !is_init) return -hyper_->at(clock).lr * config_.grad_scale;
  return 1.f;
}

// Fold an application update buffer into this clock's update log (and, with read-my-writes, into
// the cache so that the worker's own next read sees it).
void ClientLib::update_batch_param_cache(const OpInfo& pre, const RowOpVal* src, void* stream) {
  CachedTable& ct = *tables_[(uint)pre.table];
  const size_t n = pre.rows.size();
  const size_t op_idx = &pre - &plan_.ops[0];
  if (nvlink_) {
    float* ring = fabric_ring_ptr((uint)pre.table, (int)process_id_, clock_);
    geeps_row_scatter_add(ring, reinterpret_cast<const float*>(src), op_index_dev_[op_idx], (long long)n, 0, 0,
                          (long long)pre.num_vals_limit, (long long)ct.plan->rows.size(), (long long)n,
                          reinterpret_cast<int*>(fabric_.base + fabric_.status_off), stream);
    return;
  }
  std::lock_guard<std::mutex> lk(ct.mu);
  if (pre.location == LOC_GPU) {
    FlatOps* e = create_oplog_entry(ct, ct.gpu, MEM_DEVICE, clock_, stream);
    if (!e) return;
    geeps_row_scatter_add(e->data.floats(), reinterpret_cast<const float*>(src), op_index_dev_[op_idx], (long long)n, 0, 0,
                          (long long)pre.num_vals_limit, (long long)e->data.size(), (long long)n, row_status(), stream);
    if (config_.read_my_writes)
      geeps_row_scatter_axpy(ct.gpu.data_cache.floats(), reinterpret_cast<const float*>(src), op_index_dev_[op_idx],
                             (long long)n, 0, 0, (long long)pre.num_vals_limit, (long long)ct.gpu.data_cache.size(),
                             (long long)n, e->rmw_alpha, row_status(), stream);
    cudaStreamSynchronize((cudaStream_t)stream);
  } else {
    const RowOpVal* host_src = src;
    if (gpu_) {  // staging is device memory but this part of the cache lives on the host
      if (host_stage_.size() < n) host_stage_.init(std::max(n, plan_.max_access_rows), MEM_PINNED);
      Mem::copy(host_stage_.data(), MEM_PINNED, src, MEM_DEVICE, n * sizeof(RowData), stream, true);
      stats_.swap_d2h_bytes += n * sizeof(RowData);
      host_src = host_stage_.data();
    }
    FlatOps* e = create_oplog_entry(ct, ct.cpu, MEM_HOST, clock_, stream);
    if (!e) return;
    add_rows_from_double_index_cpu(e->data.data(), host_src, pre.index.data(), n, 0, 0, pre.num_vals_limit);
    if (config_.read_my_writes)
      axpy_rows_from_double_index_cpu(ct.cpu.data_cache.data(), host_src, pre.index.data(), n, 0, 0, pre.num_vals_limit,
                                      e->rmw_alpha);
  }
}

void ClientLib::reclaim_oplog(CachedTable& ct, iter_t up_to_clock) {
  for (ParamCache* pc : {&ct.gpu, &ct.cpu}) {
    for (auto it = pc->oplog.begin(); it != pc->oplog.end() && it->first <= up_to_clock;) {
      pc->pool.put(it->second);
      it = pc->oplog.erase(it);
      bg_stats_.nr_oplog_reclaimed++;
    }
  }
}

// Send this worker's updates of (clock, table) to every server shard, or a bare clock message when
// the table was not updated (host-staged path).
void ClientLib::push_updates_param_cache(iter_t clock, uint table_id, bool is_init) {
  const double t0 = now_seconds();
  CachedTable& ct = *tables_[table_id];
  FlatOps* ge = nullptr;
  FlatOps* ce = nullptr;
  {
    std::lock_guard<std::mutex> lk(ct.mu);
    auto g = ct.gpu.oplog.find(clock);
    if (g != ct.gpu.oplog.end()) ge = g->second;
    auto c = ct.cpu.oplog.find(clock);
    if (c != ct.cpu.oplog.end()) ce = c->second;
  }
  if (!ge && !ce) {
    enc(table_id)->clock_broadcast(clock, table_id);
    bg_stats_.nr_clock_only++;
    return;
  }
  std::lock_guard<std::mutex> sl(send_mu_);
  const RowOpVal* gpu_host = nullptr;
  if (ge) {
    if (gpu_) {
      const double t1 = now_seconds();
      Mem::copy(send_buffer_.data(), MEM_PINNED, ge->data.data(), MEM_DEVICE, ge->data.bytes(), swap_stream_, true);
      bg_stats_.push_d2h_time += now_seconds() - t1;
      gpu_host = send_buffer_.data();
    } else {
      gpu_host = ge->data.data();
    }
  }
  const double t2 = now_seconds();
  std::vector<RowOpVal> assembled;
  for (uint s = 0; s < num_processes_; ++s) {
    const ShardRows& sr = ct.shards[s];
    const size_t n = sr.is_gpu.size();
    if (n == 0) { enc(table_id)->clock_to(s, clock, table_id); continue; }
    assembled.resize(n);
    size_t gi = 0, ci = 0;
    for (size_t k = 0; k < n; ++k) {
      const RowOpVal* src = nullptr;
      if (sr.is_gpu[k]) { if (gpu_host) src = gpu_host + sr.gpu_slots[gi]; ++gi; }
      else { if (ce) src = ce->data.data() + sr.cpu_slots[ci]; ++ci; }
      if (src) memcpy(&assembled[k], src, sizeof(RowOpVal)); else memset(&assembled[k], 0, sizeof(RowOpVal));
    }
    if (!enc(table_id)->clock_with_updates_batch(s, clock, table_id, sr.keys.data(), assembled.data(), n, is_init))
      set_error(ERR_TRANSPORT, "cannot reach tablet-" + std::to_string(s));
    bg_stats_.bytes_pushed += n * sizeof(RowOpVal);
  }
  bg_stats_.push_send_time += now_seconds() - t2;
  if (!config_.read_my_writes) {
    // nothing will replay this entry: recycle it now
    std::lock_guard<std::mutex> lk(ct.mu);
    reclaim_oplog(ct, clock);
  }
  bg_stats_.nr_push++;
  bg_stats_.push_time += now_seconds() - t0;
}

void ClientLib::recv_row_batch_cpu(CachedTable& ct, uint server_id, const RowData* rows, iter_t self_clock) {
  const ShardRows& sr = ct.shards[server_id];
  size_t ci = 0;
  for (size_t k = 0; k < sr.is_gpu.size(); ++k) {
    if (sr.is_gpu[k]) continue;
    RowData* dst = ct.cpu.data_cache.data() + sr.cpu_slots[ci++];
    memcpy(dst, rows + k, sizeof(RowData));
  }
  if (!config_.read_my_writes) return;
  // replay this worker's own updates the server had not seen when it sent the rows
  for (auto& kv : ct.cpu.oplog) {
    if (kv.first <= self_clock) continue;
    for (size_t slot : sr.cpu_slots)
      cpu_axpy(ROW_DATA_SIZE, kv.second->rmw_alpha, kv.second->data.data()[slot].data, ct.cpu.data_cache.data()[slot].data);
    bg_stats_.nr_rmw_replay++;
  }
}

void ClientLib::recv_row_batch_gpu(CachedTable& ct, uint server_id, const RowData* rows, iter_t self_clock) {
  const ShardRows& sr = ct.shards[server_id];
  const size_t ng = sr.gpu_slots.size();
  if (!ng) return;
  const double t0 = now_seconds();
  std::unique_lock<std::mutex> bounce(recv_mu_, std::defer_lock);
  if (gpu_) bounce.lock();      // one pinned receive buffer and one swap stream for all channels
  if (!gpu_) {
    size_t gi = 0;
    for (size_t k = 0; k < sr.is_gpu.size(); ++k)
      if (sr.is_gpu[k]) memcpy(ct.gpu.data_cache.data() + sr.gpu_slots[gi++], rows + k, sizeof(RowData));
  } else {
    // compact the shard's device-cached rows into pinned memory, then one H2D (+ scatter if strided)
    size_t gi = 0;
    for (size_t k = 0; k < sr.is_gpu.size(); ++k)
      if (sr.is_gpu[k]) memcpy(recv_buffer_.data() + gi++, rows + k, sizeof(RowData));
    if (sr.gpu_contiguous) {
      Mem::copy(ct.gpu.data_cache.data() + sr.gpu_slots[0], MEM_DEVICE, recv_buffer_.data(), MEM_PINNED,
                ng * sizeof(RowData), swap_stream_, true);
    } else {
      if (recv_dev_.size() < ng) recv_dev_.init(recv_buffer_.size(), MEM_DEVICE);
      Mem::copy(recv_dev_.data(), MEM_DEVICE, recv_buffer_.data(), MEM_PINNED, ng * sizeof(RowData), swap_stream_, false);
      geeps_row_scatter(ct.gpu.data_cache.floats(), recv_dev_.floats(), sr.gpu_index_dev, (long long)ng, 0, 0, kNoLimit,
                        (long long)ct.gpu.data_cache.size(), (long long)ng, row_status(), swap_stream_);
      cudaStreamSynchronize((cudaStream_t)swap_stream_);
    }
  }
  bg_stats_.recv_h2d_time += now_seconds() - t0;
  if (!config_.read_my_writes) return;
  for (auto& kv : ct.gpu.oplog) {
    if (kv.first <= self_clock) continue;
    if (!gpu_) {
      for (size_t slot : sr.gpu_slots)
        cpu_axpy(ROW_DATA_SIZE, kv.second->rmw_alpha, kv.second->data.data()[slot].data, ct.gpu.data_cache.data()[slot].data);
    } else if (sr.gpu_contiguous) {
      geeps_axpy(ct.gpu.data_cache.floats() + sr.gpu_slots[0] * ROW_DATA_SIZE,
                 kv.second->data.floats() + sr.gpu_slots[0] * ROW_DATA_SIZE, kv.second->rmw_alpha, (long long)(ng * ROW_DATA_SIZE),
                 swap_stream_);
    } else {
      for (size_t slot : sr.gpu_slots)
        geeps_axpy(ct.gpu.data_cache.floats() + slot * ROW_DATA_SIZE, kv.second->data.floats() + slot * ROW_DATA_SIZE,
                   kv.second->rmw_alpha, ROW_DATA_SIZE, swap_stream_);
    }
    bg_stats_.nr_rmw_replay++;
  }
  if (gpu_) cudaStreamSynchronize((cudaStream_t)swap_stream_);
}

// Host-resident worker-local rows -> staging buffer (H2D on the swap stream; the caller's stream
// waits for the copy) and back.
void ClientLib::read_batch_local(const OpInfo& op, RowData* staging, void* stream) {
  const size_t bytes = op.rows.size() * sizeof(RowData);
  const RowData* src = local_.cpu.data() + op.store_offset;
  if (!gpu_) { memcpy(staging, src, bytes); return; }
  const int h = (int)(&op - &plan_.ops[0]);
  if (fetch_issued_clock_[h] != clock_) swap_issue_fetch(h);
  cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)fetch_done_ev_[h], 0);
  swap_prefetch_after(h);
  stats_.rows_fetched += op.rows.size();
}

void ClientLib::update_batch_local(const OpInfo& pre, const RowData* staging, void* stream) {
  const size_t bytes = pre.rows.size() * sizeof(RowData);
  RowData* dst = local_.cpu.data() + pre.store_offset;
  if (!gpu_) { memcpy(dst, staging, bytes); return; }
  // evict on the swap stream once the application's work on `stream` that produced the rows is done
  const int h = (int)(&pre - &plan_.ops[0]);
  cudaEventRecord((cudaEvent_t)release_ev_[h], (cudaStream_t)stream);
  cudaStreamWaitEvent((cudaStream_t)swap_stream_, (cudaEvent_t)release_ev_[h], 0);
  cudaMemcpyAsync(dst, staging, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)swap_stream_);
  cudaEventRecord((cudaEvent_t)release_ev_[h], (cudaStream_t)swap_stream_);
  released_clock_[h] = clock_;
  stats_.swap_d2h_bytes += bytes;
  stats_.rows_kept += pre.rows.size();
}

}  // namespace geeps_b200
