// Server shard on the host ("tablet server"): master copy of this shard's rows of every table,
// one vector clock per table, update application and the broadcast of fresh rows when the
// table's global clock (min over workers) advances.
//
// Same responsibilities as the reference's TabletStorage (src/server/tablet-server.cpp:57-228).
// Differences: an optimizer-table mode that sums the workers' updates of a clock and applies
// momentum SGD once when every worker has signalled that clock; protocol violations (clock
// gaps, size mismatches) are counted and reported instead of aborting the process; snapshots.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "core/common_util.hpp"
#include "core/hyper_schedule.hpp"
#include "core/relaxed.hpp"
#include "core/row_op_util.hpp"
#include "geeps.hpp"

namespace geeps_b200 {

class ServerClientEncode;

struct TabletStats {
  // written by the shard's server thread, read by GetStats() on the application thread
  Relaxed<uint64_t> nr_update = 0, nr_local_update = 0, nr_rows = 0, nr_clock = 0, nr_broadcast = 0, nr_errors = 0;
  Relaxed<double> apply_time = 0, clock_time = 0, send_time = 0;
  std::string to_json() const;
};

class TabletStorage {
 public:
  struct DataTable {
    std::vector<iter_t> vec_clock;
    iter_t global_clock = -1;
    size_t row_count = 0;
    bool created = false;
    int mode = GeePsConfig::TABLE_ADDITIVE;
    DataStorage store;                 // master rows (host memory)
    DataStorage momentum;              // optimizer tables only
    std::map<iter_t, std::unique_ptr<DataStorage>> pending;  // per-clock sums (optimizer tables)
  };

  TabletStorage(uint channel_id, uint num_channels, uint process_id, uint num_processes,
                std::shared_ptr<ServerClientEncode> communicator, const GeePsConfig& config);
  // Updates for this shard's rows from one worker for one clock.  `keys` may be null after the
  // table exists (the row order is then the order of the first batch).
  bool update_row_batch(uint client_id, iter_t clock, uint table_id, const RowKey* keys, const RowOpVal* updates,
                        size_t batch_size, bool is_init);
  bool clock(uint client_id, iter_t clock, uint table_id);
  std::string get_stats() const;
  const DataTable* table(uint table_id) const { return table_id < tables_.size() ? &tables_[table_id] : nullptr; }
  DataTable* mutable_table(uint table_id) { return table_id < tables_.size() ? &tables_[table_id] : nullptr; }
  size_t num_tables() const { return tables_.size(); }
  uint process_id() const { return process_id_; }
  const std::string& last_error() const { return last_error_; }
  OptimizerParams optimizer;
  // learning rate, momentum and weight decay by clock; the worker side of the process shares the object and
  // changes it (set before the handler thread starts; a schedule of its own, built from the config, otherwise)
  std::shared_ptr<HyperSchedule> hyper;

 private:
  void apply_updates(DataTable& t, const RowOpVal* updates, size_t n);
  void process_pending_reads(uint client_id, uint table_id);
  void process_multiclient_pending_reads(uint table_id);
  bool fail(const std::string& what);

  uint channel_id_, num_channels_, process_id_, num_processes_;
  std::shared_ptr<ServerClientEncode> communicator_;
  GeePsConfig config_;
  std::vector<DataTable> tables_;
  uint start_client_ = 0;
  TabletStats stats_;
  std::string last_error_;
};

}  // namespace geeps_b200
