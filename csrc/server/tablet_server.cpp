#include "tablet_server.hpp"

#include <stdio.h>

#include <sstream>

#include "server_encoder_decoder.hpp"

namespace geeps_b200 {

std::string TabletStats::to_json() const {
  std::ostringstream o;
  o << "{\"nr_update\":" << nr_update << ",\"nr_local_update\":" << nr_local_update << ",\"nr_rows\":" << nr_rows
    << ",\"nr_clock\":" << nr_clock << ",\"nr_broadcast\":" << nr_broadcast << ",\"nr_errors\":" << nr_errors
    << ",\"apply_time\":" << apply_time << ",\"clock_time\":" << clock_time << ",\"send_time\":" << send_time << "}";
  return o.str();
}

TabletStorage::TabletStorage(uint channel_id, uint num_channels, uint process_id, uint num_processes,
                             std::shared_ptr<ServerClientEncode> communicator, const GeePsConfig& config)
    : channel_id_(channel_id), num_channels_(num_channels), process_id_(process_id),
      num_processes_(num_processes), communicator_(communicator), config_(config) {
  tables_.resize(config.num_tables);
  for (size_t t = 0; t < tables_.size(); ++t) {
    tables_[t].vec_clock.assign(num_processes, -1);
    tables_[t].global_clock = -1;
    tables_[t].mode = t < config.table_modes.size() ? config.table_modes[t] : config.table_mode;
  }
  optimizer.lr = config.learning_rate;
  optimizer.momentum = config.momentum;
  optimizer.weight_decay = config.weight_decay;
  optimizer.grad_scale = config.grad_scale;
  hyper.reset(new HyperSchedule(config.learning_rate, config.momentum, config.weight_decay));
}

bool TabletStorage::fail(const std::string& what) {
  last_error_ = what;
  stats_.nr_errors++;
  fprintf(stderr, "[geeps tablet-%u] %s\n", process_id_, what.c_str());
  return false;
}

bool TabletStorage::update_row_batch(uint client_id, iter_t clock, uint table_id, const RowKey* keys,
                                     const RowOpVal* updates, size_t batch_size, bool is_init) {
  const double t0 = now_seconds();
  if (table_id >= tables_.size()) return fail("update for unknown table " + std::to_string(table_id));
  if (client_id >= num_processes_) return fail("update from unknown client " + std::to_string(client_id));
  DataTable& t = tables_[table_id];
  if (clock != t.vec_clock[client_id] + 1)
    return fail("client " + std::to_string(client_id) + " sent updates of clock " + std::to_string(clock) +
                " for table " + std::to_string(table_id) + " but its last clock is " + std::to_string(t.vec_clock[client_id]));
  if (!t.created) {
    // the first batch defines the shard's rows of this table
    t.store.init(batch_size, MEM_HOST);
    t.store.zerofy();
    if (keys) for (size_t i = 0; i < batch_size; ++i) t.store.row_keys[i] = keys[i];
    if (t.mode == GeePsConfig::TABLE_SGD_MOMENTUM) { t.momentum.init(batch_size, MEM_HOST); t.momentum.zerofy(); }
    t.row_count = batch_size;
    t.created = true;
    stats_.nr_rows += batch_size;
  }
  if (batch_size != t.row_count)
    return fail("batch of " + std::to_string(batch_size) + " rows for a shard of " + std::to_string(t.row_count));
  if (t.mode == GeePsConfig::TABLE_SGD_MOMENTUM && !is_init) {
    std::unique_ptr<DataStorage>& acc = t.pending[clock];
    if (!acc) { acc.reset(new DataStorage()); acc->init(t.row_count, MEM_HOST); acc->zerofy(); }
    add_row_batch(acc->data(), updates, t.row_count);
  } else {
    apply_updates(t, updates, batch_size);
  }
  stats_.nr_update++;
  if (client_id == process_id_) stats_.nr_local_update++;
  stats_.apply_time += now_seconds() - t0;
  return true;
}

void TabletStorage::apply_updates(DataTable& t, const RowOpVal* updates, size_t n) {
  add_row_batch(t.store.data(), updates, n);   // master += update
}

void TabletStorage::process_pending_reads(uint client_id, uint table_id) {
  DataTable& t = tables_[table_id];
  communicator_->read_row_batch_reply(client_id, table_id, t.global_clock, t.vec_clock[client_id],
                                      t.store.row_keys.data(), t.store.data(), t.row_count);
}

void TabletStorage::process_multiclient_pending_reads(uint table_id) {
  // rotate the first receiver so that no worker is always served last
  for (uint k = 0; k < num_processes_; ++k) process_pending_reads((start_client_ + k) % num_processes_, table_id);
  start_client_ = (start_client_ + 1) % num_processes_;
  stats_.nr_broadcast++;
}

bool TabletStorage::clock(uint client_id, iter_t clock, uint table_id) {
  const double t0 = now_seconds();
  if (table_id >= tables_.size() || client_id >= num_processes_) return fail("clock for unknown table/client");
  DataTable& t = tables_[table_id];
  if (clock != t.vec_clock[client_id] + 1)
    return fail("client " + std::to_string(client_id) + " signalled clock " + std::to_string(clock) + " after " +
                std::to_string(t.vec_clock[client_id]));
  t.vec_clock[client_id] = clock;
  const iter_t new_global = clock_min(t.vec_clock);
  stats_.nr_clock++;
  if (new_global != t.global_clock) {
    if (new_global != t.global_clock + 1) return fail("global clock jumped");
    t.global_clock = new_global;
    if (t.mode == GeePsConfig::TABLE_SGD_MOMENTUM) {
      auto it = t.pending.find(new_global);
      if (it != t.pending.end()) {   // every worker's update of this clock is in: one optimizer step
        const HyperSchedule::Entry h = hyper->at(new_global);
        optimizer.lr = h.lr; optimizer.momentum = h.momentum; optimizer.weight_decay = h.weight_decay;
        cpu_sgd_momentum(t.row_count * ROW_DATA_SIZE, t.store.floats(), t.momentum.floats(), it->second->floats(),
                         optimizer);
        t.pending.erase(it);
      }
    }
    const double t1 = now_seconds();
    if (t.created) process_multiclient_pending_reads(table_id);
    stats_.send_time += now_seconds() - t1;
  }
  stats_.clock_time += now_seconds() - t0;
  return true;
}

std::string TabletStorage::get_stats() const {
  return stats_.to_json();
}

}  // namespace geeps_b200
