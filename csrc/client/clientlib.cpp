// ClientLib: construction, communication bring-up, foreground access calls.
#include "clientlib.hpp"

#include <cuda_runtime.h>
#include <stdio.h>
#include <unistd.h>

#include <string.h>

#include <fstream>

namespace geeps_b200 {

// ---------------- OpMemBufferPool ----------------
void OpMemBufferPool::init(size_t entries, size_t rows, MemType type) {
  std::lock_guard<std::mutex> lk(mu_);
  all_.clear();
  free_.clear();
  for (size_t i = 0; i < entries; ++i) {
    all_.emplace_back(new FlatOps());
    all_.back()->data.init(rows, type);
    free_.push_back(all_.back().get());
  }
}

FlatOps* OpMemBufferPool::get(size_t budget_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  const double t0 = now_seconds();
  while (free_.empty()) {
    double wait_ms = kWatchdogSeconds * 1000.0;
    if (budget_ms) {
      const double left = (double)budget_ms - (now_seconds() - t0) * 1000.0;
      if (left <= 0) return nullptr;
      if (left < wait_ms) wait_ms = left;
    }
    if (cv_.wait_for(lk, std::chrono::microseconds((long long)(wait_ms * 1000))) == std::cv_status::timeout &&
        wait_ms >= kWatchdogSeconds * 1000.0)
      fprintf(stderr, "[geeps] oplog pool: all %zu entries in flight, still waiting\n", all_.size());
  }
  FlatOps* e = free_.front();
  free_.erase(free_.begin());
  return e;
}

void OpMemBufferPool::put(FlatOps* e) {
  { std::lock_guard<std::mutex> lk(mu_); e->flag = FlatOps::NONE; e->clock = -1; free_.push_back(e); }
  cv_.notify_all();
}

// ---------------- construction ----------------
ClientLib::ClientLib(uint process_id, const GeePsConfig& config) : process_id_(process_id), config_(config) {
  num_processes_ = config.num_workers_override > 0 ? (uint)config.num_workers_override
                                                   : (uint)(config.host_list.empty() ? 1 : config.host_list.size());
  gpu_ = config.device == GeePsConfig::DEVICE_CUDA && Mem::cuda_available();
  if (config.device == GeePsConfig::DEVICE_CUDA && !gpu_)
    fprintf(stderr, "[geeps] no CUDA device visible: caches and staging live in host memory\n");
  nvlink_ = gpu_ && config.transport == GeePsConfig::TRANSPORT_NVLINK;
  if (config.transport == GeePsConfig::TRANSPORT_NVLINK && !gpu_)
    set_error(ERR_TRANSPORT, "NVLINK transport needs a CUDA device");
  if (gpu_) {
    if (config.cuda_device >= 0) cudaSetDevice(config.cuda_device);
    cudaStream_t s0, s1;
    cudaStreamCreateWithFlags(&s0, cudaStreamNonBlocking);
    cudaStreamCreateWithFlags(&s1, cudaStreamNonBlocking);
    default_stream_ = s0;
    swap_stream_ = s1;
  }
  PlanConfig pc;
  pc.gpu_memory_capacity = config.gpu_memory_capacity;
  pc.mm_warning_level = config.mm_warning_level;
  pc.read_my_writes = config.read_my_writes;
  pc.num_shards = (int)num_processes_;
  pc.partitioner = config.partitioner;
  pc.num_tables = config.num_tables;
  pc.device_is_gpu = gpu_;
  pc.allow_direct = nvlink_;
  pc.update_ring = nvlink_;
  pc.partition_align = config.table_partition_align;
  for (int v : config.table_pull) pc.pull_tables.push_back(nvlink_ && v ? 1 : 0);
  compiler_.reset(new PlanCompiler(pc));
  hyper_.reset(new HyperSchedule(config.learning_rate, config.momentum, config.weight_decay));
  last_heartbeat_.assign(num_processes_, now_seconds());
  peer_clock_.assign(num_processes_, 0);
  peer_dead_.assign(num_processes_, 0);
  std::string err;
  if (!init_comm(&err)) set_error(ERR_TRANSPORT, err);
}

ClientLib::~ClientLib() {
  shutdown();
  for (void* p : op_index_dev_) if (p) cudaFree(p);
  for (auto& kv : tables_)
    for (ShardRows& sr : kv.second->shards) if (sr.gpu_index_dev) cudaFree(sr.gpu_index_dev);
  fabric_teardown();
  if (row_status_dev_) cudaFree(row_status_dev_);
  if (row_status_host_) cudaFreeHost(row_status_host_);
  if (default_stream_) cudaStreamDestroy((cudaStream_t)default_stream_);
  if (swap_stream_) cudaStreamDestroy((cudaStream_t)swap_stream_);
}

void ClientLib::set_error(int code, const std::string& what) {
  int expected = 0;
  if (error_code_.compare_exchange_strong(expected, code)) {
    std::lock_guard<std::mutex> lk(error_mu_);
    error_text_ = what;
    fprintf(stderr, "[geeps worker %u] error %d: %s\n", process_id_, code, what.c_str());
  }
  // wake every host-side waiter so that it can observe the error
  for (auto& kv : tables_) kv.second->cv.notify_all();
  global_cv_.notify_all();
}

// Takes effect for the updates of the iteration in progress (pushed by its Clock call under the number clock_) and
// all later ones.  The TCP shard of this process applies an update of clock c only after this worker's own push of
// clock c, which comes after this call, so the shard always finds the entry; the NVLINK push reads it when it
// launches.  Steps captured in a CUDA graph carry the values of the time of capture: capture again after a change.
void ClientLib::set_hyper_params(float lr, float momentum, float weight_decay) {
  hyper_->set(clock_, lr, momentum, weight_decay);
}

std::string ClientLib::last_error_string() {
  std::lock_guard<std::mutex> lk(error_mu_);
  return error_text_;
}

// One comm channel: a server shard bound to port_for(process, c), a client router connected to every other
// process's shard of the same channel, codec objects and the handler thread.
bool ClientLib::open_channel(uint c, std::unique_ptr<ServerThreadEntry>* server, std::shared_ptr<RouterHandler>* router,
                             std::unique_ptr<ClientServerEncode>* encoder, std::unique_ptr<ServerClientDecode>* decoder,
                             std::string* err) {
  const uint nch = config_.num_comm_channels ? config_.num_comm_channels : 1;
  server->reset(new ServerThreadEntry(c, nch, process_id_, num_processes_, config_));
  (*server)->hyper_schedule = hyper_;
  ClientLib* self = this;
  if (c == 0) {
    (*server)->control_hook = [self](const std::string& src, Message& msg) {
      switch (msg[0].cmd()) {
        case CMD_HEARTBEAT: { heartbeat_msg_t h; if (msg[0].unpack(&h)) self->heartbeat_cbk(h.id, h.counter, h.clock); break; }
        case CMD_BARRIER: { barrier_msg_t h; if (msg[0].unpack(&h)) self->barrier_cbk(h.id, h.epoch); break; }
        case CMD_IPC_EXCHANGE: self->ipc_exchange_cbk(msg); break;
        case CMD_PEER_LOST: self->peer_lost_cbk(src); break;
        default: break;
      }
    };
  } else {
    // a data channel that loses a peer reports it like the control channel does
    (*server)->control_hook = [self](const std::string& src, Message& msg) {
      if (msg[0].cmd() == CMD_PEER_LOST) self->peer_lost_cbk(src);
    };
  }
  if (!(*server)->start(err)) return false;
  router->reset(new RouterHandler("client-" + std::to_string(process_id_)));
  if (config_.local_opt) {
    (*router)->set_local_peer((*server)->router().get());
    (*server)->router()->set_local_peer(router->get());
  }
  for (uint s = 0; s < num_processes_; ++s) {
    if (config_.local_opt && s == process_id_) continue;
    const std::string host = s < config_.host_list.size() ? config_.host_list[s] : "127.0.0.1";
    const unsigned port = ServerThreadEntry::port_for(config_, s, c);
    if (!(*router)->connect_to("tablet-" + std::to_string(s), host, port, 60000, err)) return false;
  }
  encoder->reset(new ClientServerEncode(*router, num_processes_, process_id_, config_));
  decoder->reset(new ServerClientDecode(this));
  ServerClientDecode* dec = decoder->get();
  (*router)->start_handler_thread([dec](const std::string& src, Message& msg) { dec->router_callback(src, msg); });
  return true;
}

bool ClientLib::init_comm(std::string* err) {
  // every process hosts a server shard per channel (channel 0 carries the control plane as well)
  if (!open_channel(0, &server_, &router_, &encoder_, &decoder_, err)) return false;
  ClientLib* self = this;
  const uint nch = config_.num_comm_channels ? config_.num_comm_channels : 1;
  for (uint c = 1; c < nch; ++c) {
    extra_channels_.emplace_back();
    Channel& ch = extra_channels_.back();
    if (!open_channel(c, &ch.server, &ch.router, &ch.encoder, &ch.decoder, err)) return false;
  }
  for (uint c = 0; c < nch; ++c) {
    bg_workers_.emplace_back(new BackgroundWorker());
    bg_workers_.back()->add_callback(kIterateCmd, [self](std::vector<char>& args) { self->cbk_iterate(args); });
    bg_workers_.back()->start();
  }
  if (num_processes_ > 1) heartbeat_thread_ = std::thread([self] { self->heartbeat_loop(); });
  return true;
}

void ClientLib::shutdown() {
  if (shut_down_) return;
  shut_down_ = true;
  if (gpu_) cudaDeviceSynchronize();
  for (auto& w : bg_workers_) w->stop();
  // leave together: a rank that tears its sockets down early would look like a failure to the rest
  if (num_processes_ > 1 && error_code_.load() == 0) host_barrier(10000);
  stop_heartbeat_ = true;
  if (heartbeat_thread_.joinable()) heartbeat_thread_.join();
  if (router_) router_->stop_handler_thread();
  if (server_) server_->stop();
  for (Channel& ch : extra_channels_) {
    if (ch.router) ch.router->stop_handler_thread();
    if (ch.server) ch.server->stop();
  }
}

// ---------------- virtual iteration (recording) ----------------
int ClientLib::virtual_read_batch(size_t table, const std::vector<size_t>& rows, int slack) {
  OpInfo op; op.type = OP_READ; op.table = table; op.rows = rows; op.slack = slack;
  return compiler_->record(op);
}
int ClientLib::virtual_postread_batch(int prestep) {
  OpInfo op; op.type = OP_POST_READ; op.prestep = prestep;
  return compiler_->record(op);
}
int ClientLib::virtual_preupdate_batch(size_t table, const std::vector<size_t>& rows) {
  OpInfo op; op.type = OP_PRE_UPDATE; op.table = table; op.rows = rows;
  return compiler_->record(op);
}
int ClientLib::virtual_update_batch(int prestep) {
  OpInfo op; op.type = OP_UPDATE; op.prestep = prestep;
  return compiler_->record(op);
}
int ClientLib::virtual_localaccess_batch(const std::vector<size_t>& rows, bool fetch) {
  OpInfo op; op.type = OP_LOCAL_ACCESS; op.table = kLocalTableId; op.rows = rows; op.local = true; op.fetch = fetch;
  return compiler_->record(op);
}
int ClientLib::virtual_postlocalaccess_batch(int prestep, bool keep) {
  OpInfo op; op.type = OP_POST_LOCAL_ACCESS; op.prestep = prestep; op.local = true; op.keep = keep;
  return compiler_->record(op);
}
int ClientLib::virtual_clock() {
  OpInfo op; op.type = OP_CLOCK;
  return compiler_->record(op);
}

// ---------------- foreground access ----------------
bool ClientLib::check_order(int handle, OpType want) {
  if (!vi_finished_ || handle < 0 || handle >= (int)plan_.ops.size() || plan_.ops[handle].type != want) {
    set_error(ERR_ORDER, "handle " + std::to_string(handle) + " is not a valid handle for this call");
    return false;
  }
  if (started_ && !plan_.ops[handle].one_off) {
    // after StartIterations the calls must come in exactly the declared order
    if (handle != last_handle_ + 1) {
      set_error(ERR_ORDER, "call with handle " + std::to_string(handle) + " after handle " +
                               std::to_string(last_handle_) + " breaks the declared order");
      return false;
    }
    last_handle_ = handle;
  }
  return true;
}

RowData* ClientLib::staging_ptr(const OpInfo& op) {
  const size_t copy = plan_.staging_copies > 1 ? (size_t)(clock_ & 1) : 0;
  return thread_cache_.at(copy * plan_.staging_rows + op.staging_offset);
}

bool ClientLib::read_batch(int handle, RowData** buf, void* stream, bool async) {
  const double t0 = now_seconds();
  *buf = nullptr;
  if (!check_order(handle, OP_READ)) return false;
  const OpInfo& op = plan_.ops[handle];
  void* st = op_stream(stream);
  last_app_stream_ = st;
  bool ok = true;
  if (nvlink_) {
    CachedTable& ct = *tables_[(uint)op.table];
    fabric_wait_data_age(ct, (uint)op.table, clock_ - op.slack - 1, st);
    if (op.direct) {
      *buf = reinterpret_cast<RowData*>(fabric_cache_ptr((uint)op.table, (int)process_id_)) + op.store_offset;
    } else {
      *buf = staging_ptr(op);
      ok = read_row_batch_param_cache(op, *buf, st);
    }
    if (!async) { cudaStreamSynchronize((cudaStream_t)st); ok = fabric_check_status(true) && ok; }
  } else {
    *buf = staging_ptr(op);
    ok = read_row_batch_param_cache(op, *buf, st);
  }
  accessed_clock_[handle] = clock_;
  stats_.nr_read++;
  stats_.rows_read += op.rows.size();
  stats_.read_time += now_seconds() - t0;
  op_account(handle, t0);
  return ok && error_code_.load() == 0;
}

// ReadPull of an uncached table: the freshness wait and the fp32 tail (rows from table_fp32_from_row on) are
// enqueued here; the leading rows are described, not copied - the caller's kernel reads them from the shards.
bool ClientLib::read_pull(int handle, GeePs::PullInfo* info, void* stream) {
  const double t0 = now_seconds();
  memset(info, 0, sizeof(*info));
  if (!check_order(handle, OP_READ)) return false;
  const OpInfo& op = plan_.ops[handle];
  if (!nvlink_ || !fabric_.active || op.table >= fabric_.tables.size() || !fabric_.tables[op.table].pull) {
    set_error(ERR_ORDER, "ReadPull on a table that is not an uncached (pull) table of the NVLINK transport");
    return false;
  }
  void* st = op_stream(stream);
  last_app_stream_ = st;
  CachedTable& ct = *tables_[(uint)op.table];
  const TableArena& ta = fabric_.tables[op.table];
  fabric_wait_data_age(ct, (uint)op.table, clock_ - op.slack - 1, st);
  if (ta.tail_rows) fabric_pull_rows((uint)op.table, reinterpret_cast<RowData*>(fabric_.base + ta.tail_off), ta.tail_from, st);
  info->num_shards = (int)num_processes_;
  for (uint s = 0; s < num_processes_ && s < 8; ++s) {
    const ShardRange& r = ct.plan->shard_ranges[s];
    info->shard_bf16[s] = config_.bf16_compute_cache ? fabric_.peer_base[s] + ta.master16_off : nullptr;
    info->shard_fp32[s] = reinterpret_cast<const float*>(fabric_.peer_base[s] + ta.master_off);
    info->row_start[s] = (long long)r.start;
    info->row_count[s] = (long long)r.count;
  }
  info->tail = ta.tail_rows ? reinterpret_cast<RowData*>(fabric_.base + ta.tail_off) : nullptr;
  info->tail_from_row = (long long)ta.tail_from;
  info->tail_rows = (long long)ta.tail_rows;
  accessed_clock_[handle] = clock_;
  stats_.nr_read++;
  stats_.nr_read_pull++;
  stats_.rows_read += op.rows.size();
  stats_.read_time += now_seconds() - t0;
  op_account(handle, t0);
  return error_code_.load() == 0;
}

void* ClientLib::read_bf16(int handle) {
  if (!nvlink_ || !config_.bf16_compute_cache || handle < 0 || handle >= (int)plan_.ops.size()) return nullptr;
  const OpInfo& op = plan_.ops[handle];
  if (op.type != OP_READ || !op.direct) return nullptr;
  const TableArena& ta = fabric_.tables[op.table];
  return fabric_.base + ta.cache16_off + op.store_offset * (size_t)kRowFloats * 2;
}

void ClientLib::postread_batch(int handle) { postread_batch(handle, nullptr); }

void ClientLib::postread_batch(int handle, void* stream) {
  const double t0 = now_seconds();
  if (!check_order(handle, OP_POST_READ)) return;
  swap_release(plan_.ops[handle].prestep, op_stream(stream), false);
  stats_.nr_postread++;
  stats_.postread_time += now_seconds() - t0;
  op_account(handle, t0);
}

void ClientLib::preupdate_batch(int handle, RowOpVal** buf, void* stream) {
  const double t0 = now_seconds();
  *buf = nullptr;
  if (!check_order(handle, OP_PRE_UPDATE)) return;
  const OpInfo& op = plan_.ops[handle];
  if (nvlink_) {
    // the ring slot of this clock is free again once every shard consumed clock - (slack+1):
    // the same condition a read of this clock waits for
    CachedTable& ct = *tables_[(uint)op.table];
    ct.last_stream = op_stream(stream);
    fabric_wait_data_age(ct, (uint)op.table, clock_ - ct.plan->slack - 1, op_stream(stream));
    if (ct.has_indirect_updates && ct.ring_zeroed_clock != clock_) {
      // staged updates are accumulated into the ring slot: it has to start the clock at zero
      cudaMemsetAsync(fabric_ring_ptr((uint)op.table, (int)process_id_, clock_), 0, ct.plan->rows.size() * kRowBytes,
                      (cudaStream_t)op_stream(stream));
      ct.ring_zeroed_clock = clock_;
    }
    if (op.direct) {
      *buf = reinterpret_cast<RowOpVal*>(fabric_ring_ptr((uint)op.table, (int)process_id_, clock_)) + op.store_offset;
      stats_.nr_preupdate++;
      stats_.preupdate_time += now_seconds() - t0;
      op_account(handle, t0);
      return;
    }
  }
  *buf = staging_ptr(op);
  accessed_clock_[handle] = clock_;
  swap_wait_region_free(handle, op_stream(stream));
  stats_.nr_preupdate++;
  stats_.preupdate_time += now_seconds() - t0;
  op_account(handle, t0);
}

void ClientLib::update_batch(int handle, void* stream, bool async) {
  const double t0 = now_seconds();
  if (!check_order(handle, OP_UPDATE)) return;
  const OpInfo& op = plan_.ops[handle];
  const OpInfo& pre = plan_.ops[op.prestep];
  void* st = op_stream(stream);
  if (!pre.direct) { update_batch_param_cache(pre, staging_ptr(pre), st); swap_release(op.prestep, st, false); }
  stats_.nr_update++;
  stats_.rows_updated += pre.rows.size();
  // after StartIterations the last write of a table in the clock signals that table's clock at
  // once, so its push overlaps the rest of the iteration; during bootstrap Clock() signals all
  last_app_stream_ = st;
  if (!pre.local) tables_[(uint)op.table]->last_stream = st;
  if (started_ && op.table_last_write) clock_table(clock_, (uint)op.table, false, false, st);
  // the blocking form returns once the update buffer may be reused by the host (the reference's Update returns
  // after the buffer was folded into the oplog); the asynchronous form leaves that to stream order
  if (!async && gpu_) cudaStreamSynchronize((cudaStream_t)st);
  stats_.update_time += now_seconds() - t0;
  op_account(handle, t0);
}

bool ClientLib::localaccess_batch(int handle, RowData** buf, void* stream) {
  const double t0 = now_seconds();
  *buf = nullptr;
  if (!check_order(handle, OP_LOCAL_ACCESS)) return false;
  const OpInfo& op = plan_.ops[handle];
  if (op.direct) {
    *buf = (op.location == LOC_GPU ? local_.gpu.data() : local_.cpu.data()) + op.store_offset;
  } else {
    *buf = staging_ptr(op);
    accessed_clock_[handle] = clock_;
    if (op.fetch) read_batch_local(op, *buf, op_stream(stream));
    else swap_wait_region_free(handle, op_stream(stream));   // rows produced in place: the region's previous
                                                             // contents may still be on their way to the host
  }
  stats_.nr_localaccess++;
  stats_.localaccess_time += now_seconds() - t0;
  op_account(handle, t0);
  return true;
}

void ClientLib::postlocalaccess_batch(int handle, void* stream) {
  const double t0 = now_seconds();
  if (!check_order(handle, OP_POST_LOCAL_ACCESS)) return;
  const OpInfo& op = plan_.ops[handle];
  const OpInfo& pre = plan_.ops[op.prestep];
  if (!pre.direct) {
    if (op.keep) update_batch_local(pre, staging_ptr(pre), op_stream(stream));
    else swap_release(op.prestep, op_stream(stream), false);
  }
  stats_.localaccess_time += now_seconds() - t0;
  op_account(handle, t0);
}

void ClientLib::start_opseq() {
  if (!vi_finished_) { set_error(ERR_ORDER, "StartIterations before FinishVirtualIteration"); return; }
  started_ = true;
  last_handle_ = -1;
}

void ClientLib::iterate() {
  const double t0 = now_seconds();
  if (!vi_finished_) { set_error(ERR_ORDER, "Clock before FinishVirtualIteration"); return; }
  if (started_ && last_handle_ != plan_.clock_handle - 1)
    set_error(ERR_ORDER, "Clock called before all declared accesses of the iteration");
  if (!started_) {   // bootstrap: signal every table now
    if (clock_ == kInitialClock) bootstrap_init_pushed_ = true;
    clock_all(clock_, clock_ == kInitialClock);
  }
  clock_++;
  last_handle_ = -1;
  stats_.nr_clock++;
  if (nvlink_) fabric_check_status();
  else check_row_status();
  if (device_clock_) fabric_end_iteration_device_clock();
  if (config_.snapshot_interval > 0 && !config_.snapshot_dir.empty() && clock_ % config_.snapshot_interval == 0)
    save_snapshot(config_.snapshot_dir);
  if (config_.log_interval > 0 && clock_ % config_.log_interval == 0) {
    fabric_collect_push_timing();
    fprintf(stderr, "[geeps worker %u] clock %d stats %s bgthread %s\n", process_id_, clock_, stats_.to_json().c_str(),
            bg_stats_.to_json().c_str());
    dump_op_times();
  }
  stats_.clock_time += now_seconds() - t0;
}

void ClientLib::op_account(int handle, double t0) {
  if (handle < 0 || (size_t)handle >= op_time_.size()) return;
  op_time_[handle] += now_seconds() - t0;
  op_calls_[handle]++;
}

// Host time spent inside each declared access since the last dump, one line per handle (what the reference prints
// per operation every log_interval clocks: src/client/clientlib-bg-access.cpp:544-573).
void ClientLib::dump_op_times() {
  static const char* names[] = {"read", "post_read", "pre_update", "update", "local_access", "post_local_access", "clock"};
  for (size_t h = 0; h < op_time_.size(); ++h) {
    if (!op_calls_[h]) continue;
    const OpInfo& op = plan_.ops[h];
    const OpInfo& pre = (op.prestep >= 0 && (size_t)op.prestep < plan_.ops.size()) ? plan_.ops[op.prestep] : op;
    fprintf(stderr, "[geeps worker %u] op %zu %s table %lld rows %zu %s: calls %llu, %.3f ms total, %.1f us per call\n",
            process_id_, h, (int)op.type >= 0 && (int)op.type < 7 ? names[(int)op.type] : "?",
            pre.local ? -1LL : (long long)pre.table, pre.rows.size(),
            pre.direct ? "direct" : (pre.location == LOC_GPU ? "staged" : "staged from host"),
            (unsigned long long)op_calls_[h], op_time_[h] * 1e3, op_time_[h] * 1e6 / (double)op_calls_[h]);
    op_time_[h] = 0;
    op_calls_[h] = 0;
  }
}

// Row kernels of the host-staged GPU path report failed bounds checks into a device block; mirror it.
bool ClientLib::check_row_status() {
  if (!row_status_dev_) return true;
  cudaMemcpy(row_status_host_, row_status_dev_, 4 * sizeof(int), cudaMemcpyDeviceToHost);
  if (row_status_host_[0] == 0) return true;
  set_error(ERR_CUDA, "row kernel check failed (kernel " + std::to_string(row_status_host_[1]) + ", detail " +
                          std::to_string(row_status_host_[2]) + ", seen " + std::to_string(row_status_host_[3]) + ")");
  return false;
}

std::string ClientLib::json_stats() {
  fabric_collect_push_timing();
  // ask the co-located shard for its counters and wait (bounded) for the reply
  {
    std::lock_guard<std::mutex> lk(global_mu_);
    server_stats_.erase(process_id_);
  }
  if (encoder_) encoder_->get_stats(process_id_);
  std::string server_json = "{}";
  {
    std::unique_lock<std::mutex> lk(global_mu_);
    global_cv_.wait_for(lk, std::chrono::seconds(5), [&] { return server_stats_.count(process_id_) > 0; });
    if (server_stats_.count(process_id_)) server_json = server_stats_[process_id_];
  }
  std::string out = "{\"process_id\":" + std::to_string(process_id_) + ",\"clock\":" + std::to_string(clock_) +
                    ",\"comm_channels\":" + std::to_string(num_channels()) +
                    ",\"multicast\":" + (fabric_.use_mc ? "true" : "false") +
                    ",\"transport\":\"" + (nvlink_ ? "nvlink" : "tcp") + "\",\"device\":\"" + (gpu_ ? "cuda" : "cpu") +
                    "\",\"client\":" + stats_.to_json() + ",\"bgthread\":" + bg_stats_.to_json() +
                    ",\"router\":" + (router_ ? router_->stats.to_json() : std::string("{}")) +
                    ",\"server_router\":" + (server_ ? server_->router()->stats.to_json() : std::string("{}")) +
                    ",\"channels\":[";
  for (uint c = 0; c < num_channels(); ++c) {
    RouterHandler* cr = c == 0 ? router_.get() : extra_channels_[c - 1].router.get();
    ServerThreadEntry* sv = c == 0 ? server_.get() : extra_channels_[c - 1].server.get();
    out += std::string(c ? "," : "") + "{\"channel\":" + std::to_string(c) + ",\"port\":" +
           std::to_string(ServerThreadEntry::port_for(config_, process_id_, c)) + ",\"router\":" +
           (cr ? cr->stats.to_json() : std::string("{}")) + ",\"server_router\":" +
           (sv ? sv->router()->stats.to_json() : std::string("{}")) + ",\"storage\":" +
           (sv ? sv->storage()->get_stats() : std::string("{}")) + "}";
  }
  out += "],\"push_timeline\":" + fabric_timeline_json() + ",\"server\":" + server_json + "}";
  if (!config_.output_dir.empty()) {
    std::ofstream f(config_.output_dir + "/json_stats." + std::to_string(process_id_), std::ios::app);
    f << out << "\n";
  }
  return out;
}

}  // namespace geeps_b200
