// ClientLib: FinishVirtualIteration - compile the recorded sequence and realise the plan
// (allocate worker-local storage, parameter caches, oplog pools, the staging pool, bounce
// buffers, device copies of the gather indices, and - on the NVLINK transport - the peer-mapped
// arena).  Counterpart of the reference's src/client/clientlib-viter.cpp:120-883, whose planning
// half lives in core/plan_compile.cpp.
#include <cuda_runtime.h>
#include <stdio.h>

#include "clientlib.hpp"

namespace geeps_b200 {

void ClientLib::finish_virtual_iteration() {
  const double t0 = now_seconds();
  if (vi_finished_) { set_error(ERR_ORDER, "FinishVirtualIteration called twice"); return; }
  plan_ = compiler_->compile();
  if (!plan_.ok()) { set_error(ERR_PLAN, plan_.error); return; }
  for (const std::string& w : plan_.warnings) fprintf(stderr, "[geeps worker %u] plan: %s\n", process_id_, w.c_str());
  if (nvlink_ && plan_.cpu_param_rows > 0) {
    set_error(ERR_PLAN, "NVLINK transport needs the whole parameter cache in GPU memory; raise gpu_memory_capacity or use TCP");
    return;
  }
  if (!vi_create_storage()) return;
  stats_.gpu_memory_capacity_rows = plan_.capacity_rows;
  stats_.staging_rows = plan_.staging_rows * plan_.staging_copies;
  stats_.gpu_local_rows = plan_.gpu_local_rows;
  stats_.cpu_local_rows = plan_.cpu_local_rows;
  stats_.gpu_param_rows = plan_.gpu_param_rows;
  stats_.cpu_param_rows = plan_.cpu_param_rows;
  vi_finished_ = true;
  stats_.vi_time += now_seconds() - t0;
}

void ClientLib::vi_build_shard_rows(CachedTable& ct) {
  const TablePlan& tp = *ct.plan;
  ct.shards.assign(num_processes_, ShardRows());
  for (uint s = 0; s < num_processes_; ++s) {
    const ShardRange& r = tp.shard_ranges[s];
    ShardRows& sr = ct.shards[s];
    for (size_t k = 0; k < r.count; ++k) {
      const size_t idx = r.start + k * r.stride;
      const bool g = tp.location[idx] == LOC_GPU;
      sr.is_gpu.push_back(g ? 1 : 0);
      (g ? sr.gpu_slots : sr.cpu_slots).push_back(tp.slot[idx]);
      sr.keys.push_back(RowKey(tp.table_id, tp.rows[idx]));
    }
    for (size_t k = 1; k < sr.gpu_slots.size(); ++k)
      if (sr.gpu_slots[k] != sr.gpu_slots[k - 1] + 1) sr.gpu_contiguous = false;
    if (gpu_ && !nvlink_ && !sr.gpu_slots.empty() && !sr.gpu_contiguous) {
      std::vector<DoubleIndex> idx;
      for (size_t k = 0; k < sr.gpu_slots.size(); ++k) idx.push_back(DoubleIndex((int64_t)k, (int64_t)sr.gpu_slots[k]));
      cudaMalloc(&sr.gpu_index_dev, idx.size() * sizeof(DoubleIndex));
      cudaMemcpy(sr.gpu_index_dev, idx.data(), idx.size() * sizeof(DoubleIndex), cudaMemcpyHostToDevice);
    }
  }
}

bool ClientLib::vi_create_storage() {
  const MemType dev = gpu_ ? MEM_DEVICE : MEM_HOST;
  const MemType host = (gpu_ && config_.pinned_cpu_memory) ? MEM_PINNED : MEM_HOST;
  // worker-local rows: resident part and host part (pinned so that swaps are true async copies)
  if (plan_.gpu_local_rows) { local_.gpu.init(plan_.gpu_local_rows, dev); local_.gpu.zerofy(default_stream_); }
  if (plan_.cpu_local_rows) { local_.cpu.init(plan_.cpu_local_rows, host); local_.cpu.zerofy(); }
  if ((plan_.gpu_local_rows && !local_.gpu.data()) || (plan_.cpu_local_rows && !local_.cpu.data())) {
    set_error(ERR_MEMORY, "cannot allocate worker-local storage");
    return false;
  }
  // staging pool: fixed offsets from the plan, `staging_copies` copies selected by clock parity
  const size_t staging_total = plan_.staging_rows * (size_t)plan_.staging_copies;
  std::string err;
  if (staging_total && !thread_cache_.init(staging_total, dev, &err)) {
    set_error(ERR_MEMORY, "staging pool: " + err);
    return false;
  }
  // parameter caches + oplog pools per table
  size_t biggest_gpu_table = 0, biggest_shard = 0;
  for (auto& kv : plan_.tables) {
    TablePlan& tp = kv.second;
    std::unique_ptr<CachedTable> ct(new CachedTable());
    ct->plan = &tp;
    ct->mode = tp.table_id < config_.table_modes.size() ? config_.table_modes[tp.table_id] : config_.table_mode;
    ct->per_server_data_age.assign(num_processes_, kInitialDataAge);
    ct->server_clock.assign(num_processes_, kInitialDataAge);
    if (!nvlink_) {
      if (tp.gpu_rows) {
        ct->gpu.data_cache.init(tp.gpu_rows, dev);
        ct->gpu.data_cache.zerofy(default_stream_);
        ct->gpu.pool.init((size_t)tp.num_oplog_entries, tp.gpu_rows, dev);
      }
      if (tp.cpu_rows) {
        ct->cpu.data_cache.init(tp.cpu_rows, MEM_HOST);
        ct->cpu.data_cache.zerofy();
        ct->cpu.pool.init((size_t)tp.num_oplog_entries, tp.cpu_rows, MEM_HOST);
      }
    }
    vi_build_shard_rows(*ct);
    // shards that own no row of this table never send data: they are always "fresh"
    for (uint s = 0; s < num_processes_; ++s)
      if (tp.shard_ranges[s].count == 0) ct->per_server_data_age[s] = kBigIter;
    biggest_gpu_table = std::max(biggest_gpu_table, tp.gpu_rows);
    for (const ShardRange& r : tp.shard_ranges) biggest_shard = std::max(biggest_shard, r.count);
    tables_[(uint)tp.table_id] = std::move(ct);
  }
  if (gpu_ && !nvlink_) {
    // pinned bounce buffers of the host-staged path, sized for the biggest table / shard
    if (biggest_gpu_table) send_buffer_.init(biggest_gpu_table, MEM_PINNED);
    if (biggest_shard) recv_buffer_.init(biggest_shard, MEM_PINNED);
  }
  // device copies of the per-op gather indices (only ops that go through staging need them)
  op_index_dev_.assign(plan_.ops.size(), nullptr);
  if (gpu_) {
    for (size_t i = 0; i < plan_.ops.size(); ++i) {
      const OpInfo& op = plan_.ops[i];
      if (op.local || op.direct || op.index.empty()) continue;
      if (op.location != LOC_GPU) continue;
      cudaMalloc(&op_index_dev_[i], op.index.size() * sizeof(DoubleIndex));
      cudaMemcpy(op_index_dev_[i], op.index.data(), op.index.size() * sizeof(DoubleIndex), cudaMemcpyHostToDevice);
    }
    cudaStreamSynchronize((cudaStream_t)default_stream_);
  }
  for (const OpInfo& op : plan_.ops)
    if (op.type == OP_PRE_UPDATE && !op.local && !op.direct) tables_[(uint)op.table]->has_indirect_updates = true;
  swap_init();
  op_time_.assign(plan_.ops.size(), 0.0);
  op_calls_.assign(plan_.ops.size(), 0);
  if (gpu_ && !nvlink_) {
    // status block for the row kernels of the host-staged path (failed bounds checks land here)
    cudaMalloc(reinterpret_cast<void**>(&row_status_dev_), 4 * sizeof(int));
    cudaMemset(row_status_dev_, 0, 4 * sizeof(int));
    cudaHostAlloc(reinterpret_cast<void**>(&row_status_host_), 4 * sizeof(int), cudaHostAllocDefault);
  }
  if (nvlink_) {
    if (!fabric_setup(&err)) { set_error(ERR_TRANSPORT, "NVLINK fabric: " + err); return false; }
  }
  return true;
}

}  // namespace geeps_b200
