// Table snapshots (checkpoint / resume).  The reference has no checkpoint code (only an unused
// serialisation hook, include/geeps-user-defined-types.hpp:66-69 of the reference); the layout here
// mirrors a server shard's in-memory table - row keys, rows, optimizer state, clocks - one file set
// per (table, shard) so shards write in parallel and a different world size can re-shard on load:
//
//   <dir>/snapshot.<clock>/MANIFEST.<shard>.json       world size, partitioner, clock, per-table row counts
//   <dir>/snapshot.<clock>/table<T>.shard<S>.keys      (u64 table, u64 row) x n
//   <dir>/snapshot.<clock>/table<T>.shard<S>.rows      fp32[n][128]
//   <dir>/snapshot.<clock>/table<T>.shard<S>.mom       fp32[n][128]   (optimizer tables)
//   <dir>/snapshot.<clock>/table<T>.shard<S>.clock     i32 global_clock, i32 vec_clock[workers]
//   <dir>/snapshot.<clock>/worker<W>.local             worker-local rows (resident part then host part)
//   <dir>/LATEST                                       clock of the newest complete snapshot
//
// A snapshot is taken at a clock boundary after every update of earlier clocks has been applied.
#include <cuda_runtime.h>
#include <dirent.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>

#include <fstream>
#include <sstream>

#include "clientlib.hpp"
#include "kernels/kernels.h"

namespace geeps_b200 {

namespace {
bool write_file(const std::string& path, const void* p, size_t n) {
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) return false;
  if (n) f.write(static_cast<const char*>(p), (std::streamsize)n);
  return (bool)f;
}
bool read_file(const std::string& path, std::vector<char>* out) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) return false;
  const std::streamsize n = f.tellg();
  f.seekg(0);
  out->resize((size_t)n);
  if (n) f.read(out->data(), n);
  return (bool)f;
}
long long json_int(const std::string& s, const std::string& key, long long def) {
  const size_t p = s.find("\"" + key + "\":");
  if (p == std::string::npos) return def;
  return atoll(s.c_str() + p + key.size() + 3);
}
}  // namespace

bool ClientLib::save_snapshot(const std::string& dir) {
  if (!vi_finished_) { set_error(ERR_SNAPSHOT, "snapshot before FinishVirtualIteration"); return false; }
  const iter_t cut = clock_ - 1;   // every update of clocks <= cut is in the snapshot
  // 1. wait until all of them are applied everywhere
  for (auto& kv : tables_) {
    CachedTable& ct = *kv.second;
    if (nvlink_) {
      fabric_wait_data_age(ct, kv.first, cut, default_stream_);
    } else {
      std::unique_lock<std::mutex> lk(ct.mu);
      const bool ok = ct.cv.wait_for(lk, std::chrono::seconds(120), [&] { return ct.data_age >= cut || error_code_.load(); });
      if (!ok || error_code_.load()) { lk.unlock(); set_error(ERR_SNAPSHOT, "snapshot: updates did not settle"); return false; }
    }
  }
  if (gpu_) { cudaStreamSynchronize((cudaStream_t)default_stream_); if (nvlink_) for (void* cs : fabric_.comm_lanes) cudaStreamSynchronize((cudaStream_t)cs); }
  if (num_processes_ > 1 && !host_barrier(120000)) { set_error(ERR_SNAPSHOT, "snapshot barrier timed out"); return false; }
  // 2. write this shard
  ::mkdir(dir.c_str(), 0777);
  const std::string sdir = dir + "/snapshot." + std::to_string(clock_);
  ::mkdir(sdir.c_str(), 0777);
  bool ok = true;
  std::ostringstream man;
  const HyperSchedule::Entry hyper = hyper_->at(clock_);
  man << "{\"clock\":" << clock_ << ",\"world_size\":" << num_processes_ << ",\"shard\":" << process_id_
      << ",\"partitioner\":" << config_.partitioner << ",\"num_tables\":" << config_.num_tables
      << ",\"row_floats\":128,\"dtype\":\"fp32\",\"learning_rate\":" << hyper.lr
      << ",\"momentum\":" << hyper.momentum << ",\"weight_decay\":" << hyper.weight_decay << ",\"tables\":[";
  bool first = true;
  for (auto& kv : tables_) {
    CachedTable& ct = *kv.second;
    const uint t = kv.first;
    const ShardRows& sr = ct.shards[process_id_];
    const size_t n = sr.keys.size();
    const std::string base = sdir + "/table" + std::to_string(t) + ".shard" + std::to_string(process_id_);
    std::vector<RowData> rows(n), mom;
    std::vector<int32_t> clocks;
    bool has_mom = false;
    if (nvlink_) {
      const TableArena& ta = fabric_.tables[t];
      if (n) cudaMemcpy(rows.data(), fabric_.base + ta.master_off, n * sizeof(RowData), cudaMemcpyDeviceToHost);
      if (ct.mode == GeePsConfig::TABLE_SGD_MOMENTUM) {
        mom.resize(n);
        has_mom = true;
        if (n) cudaMemcpy(mom.data(), fabric_.base + ta.momentum_off, n * sizeof(RowData), cudaMemcpyDeviceToHost);
      }
      clocks.push_back(cut);
      for (uint w = 0; w < num_processes_; ++w) clocks.push_back(cut);
    } else {
      const TabletStorage::DataTable* dt = srv(t)->storage()->table(t);
      if (dt && dt->created && dt->row_count == n) {
        if (n) memcpy(rows.data(), dt->store.data(), n * sizeof(RowData));
        if (dt->mode == GeePsConfig::TABLE_SGD_MOMENTUM) { mom.resize(n); has_mom = true; if (n) memcpy(mom.data(), dt->momentum.data(), n * sizeof(RowData)); }
        clocks.push_back(dt->global_clock);
        for (iter_t c : dt->vec_clock) clocks.push_back(c);
      } else if (n) {
        ok = false;
      }
    }
    ok = write_file(base + ".keys", sr.keys.data(), n * sizeof(RowKey)) && ok;
    ok = write_file(base + ".rows", rows.data(), n * sizeof(RowData)) && ok;
    if (has_mom) ok = write_file(base + ".mom", mom.data(), n * sizeof(RowData)) && ok;
    ok = write_file(base + ".clock", clocks.data(), clocks.size() * sizeof(int32_t)) && ok;
    man << (first ? "" : ",") << "{\"table_id\":" << t << ",\"rows\":" << ct.plan->rows.size() << ",\"shard_rows\":" << n
        << ",\"mode\":" << ct.mode << "}";
    first = false;
  }
  man << "]}";
  {
    // worker-local rows that survive across clocks
    std::vector<RowData> loc(local_.gpu.size() + local_.cpu.size());
    if (local_.gpu.size()) Mem::copy(loc.data(), MEM_HOST, local_.gpu.data(), local_.gpu.type(), local_.gpu.bytes(), default_stream_, true);
    if (local_.cpu.size()) memcpy(loc.data() + local_.gpu.size(), local_.cpu.data(), local_.cpu.bytes());
    ok = write_file(sdir + "/worker" + std::to_string(process_id_) + ".local", loc.data(), loc.size() * sizeof(RowData)) && ok;
  }
  const std::string m = man.str();
  ok = write_file(sdir + "/MANIFEST." + std::to_string(process_id_) + ".json", m.data(), m.size()) && ok;
  // 3. nobody resumes pushing before every shard is on disk
  if (num_processes_ > 1 && !host_barrier(120000)) ok = false;
  if (ok && process_id_ == 0) {
    const std::string latest = std::to_string(clock_);
    write_file(dir + "/LATEST", latest.data(), latest.size());
  }
  if (!ok) set_error(ERR_SNAPSHOT, "snapshot to " + sdir + " failed");
  return ok;
}

bool ClientLib::load_snapshot(const std::string& dir) {
  if (!vi_finished_) { set_error(ERR_SNAPSHOT, "LoadSnapshot needs the plan: call FinishVirtualIteration first"); return false; }
  std::vector<char> buf;
  if (!read_file(dir + "/LATEST", &buf)) { set_error(ERR_SNAPSHOT, "no LATEST in " + dir); return false; }
  const iter_t snap_clock = atoi(std::string(buf.begin(), buf.end()).c_str());
  const std::string sdir = dir + "/snapshot." + std::to_string(snap_clock);
  if (!read_file(sdir + "/MANIFEST.0.json", &buf)) { set_error(ERR_SNAPSHOT, "no manifest in " + sdir); return false; }
  const std::string man(buf.begin(), buf.end());
  const int old_world = (int)json_int(man, "world_size", 1);
  const iter_t cut = snap_clock - 1;
  for (auto& kv : tables_) {
    CachedTable& ct = *kv.second;
    const uint t = kv.first;
    const TablePlan& tp = *ct.plan;
    // gather the whole table (rows + momentum) from every old shard, keyed by row id
    std::vector<RowData> full(tp.rows.size()), full_mom(tp.rows.size());
    bool any_mom = false;
    size_t seen = 0;
    for (int s = 0; s < old_world; ++s) {
      const std::string base = sdir + "/table" + std::to_string(t) + ".shard" + std::to_string(s);
      std::vector<char> kb, rb, mb;
      if (!read_file(base + ".keys", &kb) || !read_file(base + ".rows", &rb)) { set_error(ERR_SNAPSHOT, "missing " + base); return false; }
      const bool hm = read_file(base + ".mom", &mb);
      const size_t n = kb.size() / sizeof(RowKey);
      const RowKey* keys = reinterpret_cast<const RowKey*>(kb.data());
      for (size_t i = 0; i < n; ++i) {
        auto it = tp.row_to_idx.find((size_t)keys[i].row);
        if (it == tp.row_to_idx.end()) continue;
        memcpy(&full[it->second], rb.data() + i * sizeof(RowData), sizeof(RowData));
        if (hm && mb.size() >= (i + 1) * sizeof(RowData)) { memcpy(&full_mom[it->second], mb.data() + i * sizeof(RowData), sizeof(RowData)); any_mom = true; }
        ++seen;
      }
    }
    if (seen != tp.rows.size()) { set_error(ERR_SNAPSHOT, "snapshot of table " + std::to_string(t) + " does not cover the planned rows"); return false; }
    // this rank's shard under the current partitioning
    const ShardRange& own = tp.shard_ranges[process_id_];
    std::vector<RowData> mine(own.count), mine_mom(own.count);
    for (size_t k = 0; k < own.count; ++k) { mine[k] = full[own.start + k * own.stride]; mine_mom[k] = full_mom[own.start + k * own.stride]; }
    if (nvlink_) {
      const TableArena& ta = fabric_.tables[t];
      if (!ta.pull) {
        cudaMemcpy(fabric_.base + ta.cache_off, full.data(), full.size() * sizeof(RowData), cudaMemcpyHostToDevice);
        if (config_.bf16_compute_cache)
          geeps_f32_to_bf16(reinterpret_cast<const float*>(fabric_.base + ta.cache_off), fabric_.base + ta.cache16_off,
                            (long long)(full.size() * ROW_DATA_SIZE), default_stream_);
      }
      if (own.count) cudaMemcpy(fabric_.base + ta.master_off, mine.data(), own.count * sizeof(RowData), cudaMemcpyHostToDevice);
      if (ta.pull && config_.bf16_compute_cache && own.count)   // uncached table: the shard's bf16 copy of its rows
        geeps_f32_to_bf16(reinterpret_cast<const float*>(fabric_.base + ta.master_off), fabric_.base + ta.master16_off,
                          (long long)(own.count * ROW_DATA_SIZE), default_stream_);
      if (own.count && any_mom) cudaMemcpy(fabric_.base + ta.momentum_off, mine_mom.data(), own.count * sizeof(RowData), cudaMemcpyHostToDevice);
      std::vector<int> flags(kRowFloats / 2, 0);
      for (int i = 0; i < 8; ++i) { flags[i] = snap_clock; flags[8 + i] = snap_clock; }   // push_ready, data_age stamps
      flags[16] = snap_clock;                                                              // global clock stamp
      for (int i = 0; i < 8; ++i) flags[24 + i] = snap_clock;                              // publish-begin stamps
      cudaMemcpy(fabric_.base + ta.flags_off, flags.data(), 128, cudaMemcpyHostToDevice);
      ct.waited_floor = snap_clock;
      ct.waited_by_stream.clear();
      cudaStreamSynchronize((cudaStream_t)default_stream_);
    } else {
      TabletStorage::DataTable* dt = srv(t)->storage()->mutable_table(t);
      dt->store.init(own.count, MEM_HOST);
      if (own.count) memcpy(dt->store.data(), mine.data(), own.count * sizeof(RowData));
      dt->store.row_keys = ct.shards[process_id_].keys;
      if (dt->mode == GeePsConfig::TABLE_SGD_MOMENTUM) {
        dt->momentum.init(own.count, MEM_HOST);
        if (own.count) memcpy(dt->momentum.data(), mine_mom.data(), own.count * sizeof(RowData));
      }
      dt->row_count = own.count;
      dt->created = own.count > 0;
      dt->vec_clock.assign(num_processes_, cut);
      dt->global_clock = cut;
      dt->pending.clear();
      std::lock_guard<std::mutex> lk(ct.mu);
      for (size_t idx = 0; idx < tp.rows.size(); ++idx) {
        DataStorage& part = tp.location[idx] == LOC_GPU ? ct.gpu.data_cache : ct.cpu.data_cache;
        Mem::copy(part.data() + tp.slot[idx], part.type(), &full[idx], MEM_HOST, sizeof(RowData), default_stream_, false);
      }
      if (gpu_) cudaStreamSynchronize((cudaStream_t)default_stream_);
      for (uint s = 0; s < num_processes_; ++s)
        if (tp.shard_ranges[s].count) ct.per_server_data_age[s] = cut;
      ct.data_age = clock_min(ct.per_server_data_age);
      ct.server_clock.assign(num_processes_, cut);
      ct.server_clock_min = cut;
    }
    ct.signalled_clock = cut;
  }
  if (read_file(sdir + "/worker" + std::to_string(process_id_) + ".local", &buf) &&
      buf.size() == (local_.gpu.size() + local_.cpu.size()) * sizeof(RowData)) {
    if (local_.gpu.size()) Mem::copy(local_.gpu.data(), local_.gpu.type(), buf.data(), MEM_HOST, local_.gpu.bytes(), default_stream_, true);
    if (local_.cpu.size()) memcpy(local_.cpu.data(), buf.data() + local_.gpu.bytes(), local_.cpu.bytes());
  }
  clock_ = snap_clock;
  if (num_processes_ > 1 && !host_barrier(120000)) { set_error(ERR_SNAPSHOT, "barrier after LoadSnapshot timed out"); return false; }
  return error_code_.load() == 0;
}

}  // namespace geeps_b200
