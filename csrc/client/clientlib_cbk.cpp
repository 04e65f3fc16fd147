// ClientLib callbacks run by the router handler threads: installation of received rows, server
// clock bookkeeping, stats replies and the membership / control messages
// (role of the reference's src/client/clientlib-cbk.cpp:51-111).
#include <stdio.h>

#include <algorithm>
#include <chrono>
#include <string.h>

#include "clientlib.hpp"

namespace geeps_b200 {

void ClientLib::find_row_cbk(uint64_t table, uint64_t row, uint server_id) {
  // placement answers go to whoever asked (locate_row); the data path uses the static partitioner
  {
    std::lock_guard<std::mutex> lk(global_mu_);
    located_[{table, row}] = (int)server_id;
  }
  global_cv_.notify_all();
}

int ClientLib::locate_row(uint64_t table, uint64_t row, uint metadata_server, int timeout_ms) {
  if (!encoder_ || metadata_server >= num_processes_) return -1;
  {
    std::lock_guard<std::mutex> lk(global_mu_);
    located_.erase({table, row});
  }
  encoder_->find_row(table, row, metadata_server);
  std::unique_lock<std::mutex> lk(global_mu_);
  const bool got = global_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                                       [&] { return located_.count({table, row}) > 0 || error_code_.load() != 0; });
  if (!got || !located_.count({table, row})) return -1;
  return located_[{table, row}];
}

void ClientLib::report_access(uint metadata_server, uint64_t table, uint64_t row, uint32_t nread, uint32_t nwrite) {
  if (!encoder_ || metadata_server >= num_processes_) return;
  std::vector<access_info_t> infos(1);
  infos[0].table = table; infos[0].row = row; infos[0].nread = nread; infos[0].nwrite = nwrite;
  encoder_->add_access_info(metadata_server, infos);
}

void ClientLib::recv_row_batch_cbk(uint server_id, uint table_id, iter_t data_age, iter_t self_clock, const RowKey*,
                                   const RowData* rows, size_t num_rows) {
  const double t0 = now_seconds();
  auto it = tables_.find(table_id);
  if (it == tables_.end() || server_id >= num_processes_) return;
  CachedTable& ct = *it->second;
  std::unique_lock<std::mutex> lk(ct.mu);
  bg_stats_.recv_wait_lock_time += now_seconds() - t0;
  if (num_rows != ct.shards[server_id].is_gpu.size()) {
    lk.unlock();
    set_error(ERR_PROTOCOL, "tablet-" + std::to_string(server_id) + " sent " + std::to_string(num_rows) +
                                " rows for a shard of " + std::to_string(ct.shards[server_id].is_gpu.size()));
    return;
  }
  if (data_age <= ct.per_server_data_age[server_id]) {
    // stale or duplicate delivery: never install older data over newer
    lk.unlock();
    set_error(ERR_PROTOCOL, "stale row batch from tablet-" + std::to_string(server_id) + " (age " +
                                std::to_string(data_age) + ")");
    return;
  }
  // Own updates newer than this are not in the rows just received and are replayed (read-my-writes).  An additive
  // shard applies an update on arrival, so everything up to self_clock is in; an optimizer shard steps once per
  // global clock, so only clocks up to data_age are.
  const iter_t replay_after = ct.mode == GeePsConfig::TABLE_SGD_MOMENTUM ? std::min(data_age, self_clock) : self_clock;
  recv_row_batch_cpu(ct, server_id, rows, replay_after);
  recv_row_batch_gpu(ct, server_id, rows, replay_after);
  ct.per_server_data_age[server_id] = data_age;
  ct.data_age = clock_min(ct.per_server_data_age);
  bg_stats_.nr_recv++;
  bg_stats_.bytes_received += num_rows * sizeof(RowData);
  bg_stats_.recv_time += now_seconds() - t0;
  lk.unlock();
  ct.cv.notify_all();
}

void ClientLib::server_clock_cbk(uint server_id, uint table_id, iter_t clock) {
  auto it = tables_.find(table_id);
  if (it == tables_.end() || server_id >= num_processes_) return;
  CachedTable& ct = *it->second;
  std::lock_guard<std::mutex> lk(ct.mu);
  if (clock > ct.server_clock[server_id]) ct.server_clock[server_id] = clock;
  std::vector<iter_t> active;
  for (uint s = 0; s < num_processes_; ++s)
    if (!ct.shards[s].is_gpu.empty()) active.push_back(ct.server_clock[s]);
  const iter_t m = clock_min(active);
  if (m > ct.server_clock_min) {
    ct.server_clock_min = m;
    // every shard has applied our updates up to m: those log entries can be recycled
    reclaim_oplog(ct, m);
  }
}

void ClientLib::get_stats_cbk(uint server_id, const std::string& stats) {
  { std::lock_guard<std::mutex> lk(global_mu_); server_stats_[server_id] = stats; }
  global_cv_.notify_all();
}

void ClientLib::peer_lost_cbk(const std::string& who) {
  if (shut_down_) return;
  set_error(ERR_PEER_LOST, "connection to " + who + " was lost");
}

void ClientLib::heartbeat_cbk(uint id, uint64_t, iter_t clock) {
  if (id >= num_processes_) return;
  std::lock_guard<std::mutex> lk(peers_mu_);
  last_heartbeat_[id] = now_seconds();
  peer_clock_[id] = clock;
}

void ClientLib::barrier_cbk(uint id, uint epoch) {
  { std::lock_guard<std::mutex> lk(global_mu_); if (barrier_seen_[id] < epoch) barrier_seen_[id] = epoch; }
  global_cv_.notify_all();
}

void ClientLib::ipc_exchange_cbk(const Message& msg) {
  ipc_exchange_msg_t h;
  if (msg.size() < 2 || !msg[0].unpack(&h)) return;
  {
    std::lock_guard<std::mutex> lk(global_mu_);
    ipc_blobs_[h.id + kIpcRoundStride * h.table_id].assign(msg[1].data(), msg[1].data() + msg[1].size());
  }
  global_cv_.notify_all();
}

}  // namespace geeps_b200
