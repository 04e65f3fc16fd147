// Counters and timers of a worker, serialised as JSON by GeePs::GetStats()
// (role of the reference's src/client/stats-tracker.hpp:44-398; only fields that are actually
// maintained are kept, plus device-side and NVLink-path figures).
#pragma once
#include <stdint.h>

#include <atomic>
#include <sstream>
#include <string>

#include "core/relaxed.hpp"

namespace geeps_b200 {

struct Stats {
  // plan
  Relaxed<size_t> gpu_memory_capacity_rows = 0, staging_rows = 0, gpu_local_rows = 0, cpu_local_rows = 0;
  Relaxed<size_t> gpu_param_rows = 0, cpu_param_rows = 0;
  // foreground (application thread)
  Relaxed<uint64_t> nr_read = 0, nr_postread = 0, nr_preupdate = 0, nr_update = 0, nr_localaccess = 0, nr_clock = 0;
  Relaxed<uint64_t> rows_read = 0, rows_updated = 0, rows_fetched = 0, rows_kept = 0;
  Relaxed<double> read_time = 0, read_wait_time = 0, postread_time = 0, preupdate_time = 0, update_time = 0;
  Relaxed<double> localaccess_time = 0, clock_time = 0, vi_time = 0;
  Relaxed<uint64_t> staleness_hist[8];   // observed (clock-1 - data_age) per read
  Relaxed<int> max_staleness = 0;
  Relaxed<uint64_t> swap_h2d_bytes = 0, swap_d2h_bytes = 0;
  Relaxed<uint64_t> device_wait_timeouts = 0, host_wait_timeouts = 0;
  Relaxed<uint64_t> device_waits_enqueued = 0;   // data_age wait kernels put on application streams
  Relaxed<uint64_t> nr_replayed_clocks = 0;      // iterations whose launches came from a replayed CUDA graph
  Relaxed<uint64_t> nr_read_pull = 0, rows_pulled = 0;   // uncached tables: ReadPull calls; rows fetched from the shards
  Relaxed<double> iterate_time = 0;

  std::string to_json() const {
    std::ostringstream o;
    o << "{\"gpu_memory_capacity_rows\":" << (long long)gpu_memory_capacity_rows.get() << ",\"staging_rows\":" << staging_rows
      << ",\"gpu_local_rows\":" << gpu_local_rows << ",\"cpu_local_rows\":" << cpu_local_rows
      << ",\"gpu_param_rows\":" << gpu_param_rows << ",\"cpu_param_rows\":" << cpu_param_rows
      << ",\"nr_read\":" << nr_read << ",\"nr_postread\":" << nr_postread << ",\"nr_preupdate\":" << nr_preupdate
      << ",\"nr_update\":" << nr_update << ",\"nr_localaccess\":" << nr_localaccess << ",\"nr_clock\":" << nr_clock
      << ",\"rows_read\":" << rows_read << ",\"rows_updated\":" << rows_updated << ",\"rows_fetched\":" << rows_fetched
      << ",\"rows_kept\":" << rows_kept << ",\"read_time\":" << read_time << ",\"read_wait_time\":" << read_wait_time
      << ",\"postread_time\":" << postread_time << ",\"preupdate_time\":" << preupdate_time
      << ",\"update_time\":" << update_time << ",\"localaccess_time\":" << localaccess_time
      << ",\"clock_time\":" << clock_time << ",\"vi_time\":" << vi_time << ",\"iterate_time\":" << iterate_time
      << ",\"max_staleness\":" << max_staleness << ",\"staleness_hist\":[";
    for (int i = 0; i < 8; ++i) o << (i ? "," : "") << staleness_hist[i];
    o << "],\"swap_h2d_bytes\":" << swap_h2d_bytes << ",\"swap_d2h_bytes\":" << swap_d2h_bytes
      << ",\"device_wait_timeouts\":" << device_wait_timeouts << ",\"host_wait_timeouts\":" << host_wait_timeouts
      << ",\"device_waits_enqueued\":" << device_waits_enqueued << ",\"nr_replayed_clocks\":" << nr_replayed_clocks
      << ",\"nr_read_pull\":" << nr_read_pull << ",\"rows_pulled\":" << rows_pulled << "}";
    return o.str();
  }
};

struct BgthreadStats {
  Relaxed<uint64_t> nr_push = 0, nr_clock_only = 0, nr_recv = 0, nr_rmw_replay = 0, nr_oplog_reclaimed = 0;
  Relaxed<uint64_t> bytes_pushed = 0, bytes_received = 0;
  Relaxed<double> push_time = 0, push_d2h_time = 0, push_send_time = 0, recv_time = 0, recv_h2d_time = 0, recv_wait_lock_time = 0;
  // device time and table bytes of completed push kernels (reduce + apply + publish), NVLINK transport
  Relaxed<double> device_push_ms = 0;
  Relaxed<uint64_t> device_push_bytes = 0, device_push_samples = 0;
  std::string to_json() const {
    std::ostringstream o;
    o << "{\"nr_push\":" << nr_push << ",\"nr_clock_only\":" << nr_clock_only << ",\"nr_recv\":" << nr_recv
      << ",\"nr_rmw_replay\":" << nr_rmw_replay << ",\"nr_oplog_reclaimed\":" << nr_oplog_reclaimed
      << ",\"bytes_pushed\":" << bytes_pushed << ",\"bytes_received\":" << bytes_received
      << ",\"push_time\":" << push_time << ",\"push_d2h_time\":" << push_d2h_time << ",\"push_send_time\":" << push_send_time
      << ",\"recv_time\":" << recv_time << ",\"recv_h2d_time\":" << recv_h2d_time
      << ",\"recv_wait_lock_time\":" << recv_wait_lock_time << ",\"device_push_ms\":" << device_push_ms
      << ",\"device_push_bytes\":" << device_push_bytes << ",\"device_push_samples\":" << device_push_samples
      << ",\"device_push_gb_per_s\":"
      << (device_push_ms.get() > 0 ? (double)device_push_bytes.get() / (device_push_ms.get() * 1e6) : 0.0) << "}";
    return o.str();
  }
};

}  // namespace geeps_b200
