// Worker-side runtime behind the GeePs facade.
//
// One instance per process = one worker plus (through ServerThreadEntry or the device shard) one
// server shard.  It records the virtual iteration, compiles it into a Plan, owns the parameter
// caches / oplogs / staging pool / worker-local storage, executes the foreground access calls and
// runs the background machinery: a push worker per channel, the decoder callbacks that install
// fresh rows, the swapper for host-resident local data, and a heartbeat-based failure detector.
//
// Two data paths share everything above them:
//   TCP     host-staged messages to the tablet servers (same data path as the reference:
//           src/client/clientlib-data.cpp:436-522 push, :51-151 receive)
//   NVLINK  device-resident shards; update push / apply / publish are sm_100a kernels over
//           peer-mapped memory and the SSP clocks are device flags (kernels/ps_fabric.cu)
//
// Counterpart of the reference's ClientLib (src/client/clientlib.hpp:419-602 and the five
// clientlib-*.cpp files); it is an ordinary object, not a process-wide singleton.
#pragma once
#include <atomic>
#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "core/common_util.hpp"
#include "core/plan.hpp"
#include "encoder_decoder.hpp"
#include "geeps.hpp"
#include "multicast_arena.hpp"
#include "net/router_handler.hpp"
#include "net/work_queue.hpp"
#include "server/server_entry.hpp"
#include "stats_tracker.hpp"

namespace geeps_b200 {

enum GeepsError {
  ERR_NONE = 0, ERR_PLAN = 1, ERR_ORDER = 2, ERR_HOST_TIMEOUT = 3, ERR_DEVICE_TIMEOUT = 4, ERR_PEER_LOST = 5,
  ERR_PROTOCOL = 6, ERR_TRANSPORT = 7, ERR_MEMORY = 8, ERR_CUDA = 9, ERR_SNAPSHOT = 10,
};

// One per-clock update log of a table part (GPU or host)
struct FlatOps {
  enum Flag { NONE = 0, INC = 1 };
  DataStorage data;
  Flag flag = NONE;
  iter_t clock = -1;
  // read-my-writes: what one unit of this logged update adds to the worker's own view of the rows until the
  // shard's answer replaces it (1 for additive tables and initial values; -lr * grad_scale, the plain gradient
  // step, for optimizer tables, whose real step only the shard can compute)
  float rmw_alpha = 1.f;
};

// Fixed pool of pre-allocated oplog entries handed out in FIFO order; get() blocks (bounded) when
// all entries are in flight.
class OpMemBufferPool {
 public:
  void init(size_t entries, size_t rows, MemType type);
  FlatOps* get(size_t budget_ms);
  void put(FlatOps* e);
  size_t size() const { return all_.size(); }
 private:
  std::vector<std::unique_ptr<FlatOps>> all_;
  std::vector<FlatOps*> free_;
  std::mutex mu_;
  std::condition_variable cv_;
};

struct ShardRows {                 // the rows of one table that one server shard owns, as seen by a worker
  std::vector<size_t> gpu_slots, cpu_slots;   // cache slots in shard order, split by cache part
  std::vector<char> is_gpu;                   // per shard row: which part
  std::vector<RowKey> keys;
  bool gpu_contiguous = true;
  void* gpu_index_dev = nullptr;              // device DoubleIndex (position in shard's gpu rows, slot)
};

struct ParamCache {
  DataStorage data_cache;
  std::map<iter_t, FlatOps*> oplog;
  OpMemBufferPool pool;
};

struct CachedTable {
  TablePlan* plan = nullptr;
  ParamCache gpu, cpu;
  iter_t data_age = kInitialDataAge;
  std::vector<iter_t> per_server_data_age;
  std::vector<iter_t> server_clock;
  iter_t server_clock_min = kInitialDataAge;
  std::vector<ShardRows> shards;
  iter_t signalled_clock = -1;         // last clock this worker signalled for the table
  // NVLINK: data_age stamps for which a device wait has already been enqueued, per application stream (a wait
  // only orders the stream it runs on), and a floor that holds for every stream (set where the host itself
  // synchronised the device, e.g. after LoadSnapshot)
  std::vector<std::pair<void*, iter_t>> waited_by_stream;
  iter_t waited_floor = -1;
  int mode = 0;
  bool has_indirect_updates = false;   // some PreUpdate of this table goes through staging
  iter_t ring_zeroed_clock = -1;       // NVLINK: clock whose ring slot has been zeroed
  void* last_stream = nullptr;         // stream of the application's latest PreUpdate/Update on this table
  std::mutex mu;
  std::condition_variable cv;
};

// NVLINK transport: one device arena per rank with an identical layout on every rank, so a peer's
// buffer is peer_base + the same offset.
struct TableArena {
  size_t cache_off = 0, cache16_off = 0, ring_off = 0, master_off = 0, momentum_off = 0, flags_off = 0;
  size_t master16_off = 0, tail_off = 0;  // uncached tables: the shard's bf16 copy of its rows; this worker's fp32 tail
  size_t tail_from = 0, tail_rows = 0;
  bool pull = false;                      // uncached: no cache / cache16 regions
  size_t rows = 0, max_owned = 0;
  int ring_slots = 1;
  int comm_lane = 0;                      // which comm stream carries this table's pushes
};
struct Fabric {
  bool active = false;
  MulticastArena mc;                      // arena allocated through the VMM API and bound to a multicast object
  bool use_mc = false;                    //   ... in use: base / peer_base / mc_base come from it
  char* mc_base = nullptr;                // multicast view of the arena (same offsets), or null
  char* base = nullptr;                   // local arena
  size_t bytes = 0;
  std::vector<char*> peer_base;           // per rank (own rank: base)
  std::vector<TableArena> tables;         // by table id
  size_t status_off = 0;
  void* comm_stream = nullptr;            // lane 0 (also used for the status mirror)
  // comm streams by lane; a table's pushes always use the same lane (one lane today)
  std::vector<void*> comm_lanes;
  int push_ctas = 0;                      // CTA cap of the push kernel (0 = its default of 4 per SM)
  // Device timeline of the pushes (GEEPS_TIMELINE=1): per (table, clock) an event on the application's
  // stream when the update was handed over, and events on the comm stream when every worker's update had
  // arrived and when the reduce + apply + publish kernel finished.  Reported in the stats JSON.
  struct TimelineRec { unsigned table; int clock; void* handed; void* arrived; void* applied; };
  bool timeline = false;
  void* timeline_origin = nullptr;
  std::vector<TimelineRec> timeline_recs;
  void* push_done_event = nullptr;
  // Device time of the latest pushes: a ring of event pairs around the reduce + apply + publish kernel on the comm
  // stream, summed by GetStats() over the pairs that have completed (device_push_ms / device_push_gb_per_s).
  struct PushTiming { void* begin = nullptr; void* end = nullptr; size_t table_bytes = 0; bool armed = false; };
  std::vector<PushTiming> push_timing;
  size_t push_timing_next = 0;
  std::vector<void*> table_events;
  void* join_event = nullptr;             // device-clock mode: comm lanes -> application stream at the end of a clock
  int* host_status = nullptr;             // pinned mirror of the device status block
};

struct LocalStore {
  DataStorage gpu, cpu;        // resident and host-resident worker-local rows
};

class ClientLib {
 public:
  ClientLib(uint process_id, const GeePsConfig& config);
  ~ClientLib();

  // ---- virtual iteration ----
  int virtual_read_batch(size_t table, const std::vector<size_t>& rows, int slack);
  int virtual_postread_batch(int prestep);
  int virtual_preupdate_batch(size_t table, const std::vector<size_t>& rows);
  int virtual_update_batch(int prestep);
  int virtual_localaccess_batch(const std::vector<size_t>& rows, bool fetch);
  int virtual_postlocalaccess_batch(int prestep, bool keep);
  int virtual_clock();
  void finish_virtual_iteration();

  // ---- real access ----
  bool read_batch(int handle, RowData** buf, void* stream, bool async);
  void postread_batch(int handle);
  void preupdate_batch(int handle, RowOpVal** buf, void* stream);
  void update_batch(int handle, void* stream, bool async);
  bool localaccess_batch(int handle, RowData** buf, void* stream);
  void postlocalaccess_batch(int handle, void* stream);
  void postread_batch(int handle, void* stream);
  void iterate();
  void start_opseq();
  void* read_bf16(int handle);
  bool read_pull(int handle, GeePs::PullInfo* info, void* stream);
  // device-resident clock (NVLINK transport): see clientlib_fabric.cpp
  bool enable_device_clock();
  void advance_replayed_iteration();
  int* device_clock_ptr() const { return device_clock_; }

  void shutdown();
  std::string json_stats();
  std::string fabric_timeline_json();
  bool save_snapshot(const std::string& dir);
  bool load_snapshot(const std::string& dir);
  std::string plan_json() const { return plan_.to_json(); }
  iter_t current_clock() const { return clock_; }
  // Learning rate, momentum and weight decay of the shard-side optimizer for the updates of the current iteration
  // and all later ones.  Every worker makes the same call in the same iteration.
  void set_hyper_params(float lr, float momentum, float weight_decay);
  HyperSchedule::Entry hyper_params() const { return hyper_->at(clock_); }
  int last_error() const { return error_code_.load(); }
  std::string last_error_string();
  const Plan& plan() const { return plan_; }
  uint process_id() const { return process_id_; }
  uint num_processes() const { return num_processes_; }
  // test hooks (host-side fault injection)
  RouterHandler* client_router() { return router_.get(); }
  ServerThreadEntry* server() { return server_.get(); }
  void inject_skip_heartbeats(bool on) { skip_heartbeats_ = on; }
  void inject_withhold_push_signal(bool on) { withhold_push_signal_ = on; }

  // ---- decoder callbacks (router handler thread) ----
  void recv_row_batch_cbk(uint server_id, uint table_id, iter_t data_age, iter_t self_clock, const RowKey* keys,
                          const RowData* rows, size_t num_rows);
  void server_clock_cbk(uint server_id, uint table_id, iter_t clock);
  void get_stats_cbk(uint server_id, const std::string& stats);
  void find_row_cbk(uint64_t table, uint64_t row, uint server_id);
  // Placement service of the shards (the reference's MetadataServer protocol: FIND_ROW / ADD_ACCESS_INFO,
  // src/server/metadata-server.cpp:44-170): ask shard `metadata_server` which shard it places (table, row) on
  // under the configured pp_policy; -1 if no answer arrives within timeout_ms.  The data path itself uses the
  // static partitioner.
  int locate_row(uint64_t table, uint64_t row, uint metadata_server, int timeout_ms);
  void report_access(uint metadata_server, uint64_t table, uint64_t row, uint32_t nread, uint32_t nwrite);
  void peer_lost_cbk(const std::string& who);
  void heartbeat_cbk(uint id, uint64_t counter, iter_t clock);
  void barrier_cbk(uint id, uint epoch);
  void ipc_exchange_cbk(const Message& msg);

 private:
  friend class ServerClientDecode;
  void set_error(int code, const std::string& what);
  bool init_comm(std::string* err);
  bool check_order(int handle, OpType want);
  RowData* staging_ptr(const OpInfo& op);
  void* op_stream(void* stream) const { return stream ? stream : default_stream_; }

  // plan realisation (clientlib_viter.cpp)
  bool vi_create_storage();
  void vi_build_shard_rows(CachedTable& ct);
  // data path (clientlib_data.cpp)
  bool read_row_batch_param_cache(const OpInfo& op, RowData* dst, void* stream);
  void update_batch_param_cache(const OpInfo& op, const RowOpVal* src, void* stream);
  FlatOps* create_oplog_entry(CachedTable& ct, ParamCache& pc, MemType type, iter_t clock, void* stream);
  void push_updates_param_cache(iter_t clock, uint table_id, bool is_init);
  void reclaim_oplog(CachedTable& ct, iter_t up_to_clock);
  float rmw_alpha_for(const CachedTable& ct, iter_t clock) const;
  int* row_status() const { return nvlink_ ? (fabric_.base ? reinterpret_cast<int*>(fabric_.base + fabric_.status_off) : nullptr)
                                           : row_status_dev_; }
  void recv_row_batch_gpu(CachedTable& ct, uint server_id, const RowData* rows, iter_t self_clock);
  void recv_row_batch_cpu(CachedTable& ct, uint server_id, const RowData* rows, iter_t self_clock);
  void read_batch_local(const OpInfo& op, RowData* staging, void* stream);
  void update_batch_local(const OpInfo& op, const RowData* staging, void* stream);
  // swapper (clientlib_bg.cpp)
  void swap_init();
  void swap_issue_fetch(int handle);
  void swap_wait_region_free(int handle, void* stream);
  bool swap_can_prefetch(int current, int target) const;
  void swap_prefetch_after(int handle);
  void swap_release(int pre_handle, void* stream, bool after_swap_stream);
  // background (clientlib_bg.cpp)
  void clock_table(iter_t signalled_clock, uint table_id, bool is_init, bool synchronous, void* stream);
  void clock_all(iter_t signalled_clock, bool is_init);
  void cbk_iterate(std::vector<char>& args);
  void heartbeat_loop();
  bool host_barrier(int timeout_ms);
  // NVLINK path (clientlib_fabric.cpp)
  bool fabric_setup(std::string* err);
  void fabric_teardown();
  void fabric_wait_data_age(CachedTable& ct, uint table_id, iter_t needed_age, void* stream);
  void fabric_push(iter_t clock, uint table_id, bool is_init, void* stream);
  bool fabric_check_status(bool sync = false);
  void fabric_end_iteration_device_clock();
  int stamp_arg(iter_t stamp) const { return device_clock_ ? (int)(stamp - clock_) : (int)stamp; }
  const int* clock_ref() const { return device_clock_; }
  void fabric_read_rmw(const OpInfo& op, RowData* dst, void* stream);
  void fabric_pull_rows(uint table_id, RowData* dst, size_t row_from, void* stream);
  float* fabric_cache_ptr(uint table_id, int rank) const;
  float* fabric_ring_ptr(uint table_id, int rank, iter_t clock) const;

  uint process_id_, num_processes_;
  GeePsConfig config_;
  bool gpu_ = false;            // caches and staging in device memory
  bool nvlink_ = false;
  void* default_stream_ = nullptr;
  void* swap_stream_ = nullptr;

  // recording + plan
  std::unique_ptr<PlanCompiler> compiler_;
  Plan plan_;
  bool vi_finished_ = false, started_ = false, shut_down_ = false;
  int* device_clock_ = nullptr;          // device word holding clock_ (device-clock mode), else null
  void* last_app_stream_ = nullptr;      // stream of the application's latest access call
  bool bootstrap_init_pushed_ = false;   // clock 0 was signalled before StartIterations: its updates are initial values
  iter_t clock_ = kInitialClock;
  std::shared_ptr<HyperSchedule> hyper_;
  int last_handle_ = -1;

  // storage
  std::map<uint, std::unique_ptr<CachedTable>> tables_;
  LocalStore local_;
  GpuCache<MultithreadedCacheHelper> thread_cache_;   // staging pool (device or host memory)
  DataStorage send_buffer_, recv_buffer_;             // pinned bounce buffers for the TCP path on a GPU
  DataStorage host_stage_;                            // pinned staging for host-cached rows read on a GPU
  DataStorage recv_dev_;                              // device staging for strided shard installs
  // swapper state: per-op events and the clock in which the op's fetch was issued
  std::vector<void*> fetch_done_ev_, release_ev_;
  std::vector<iter_t> fetch_issued_clock_, accessed_clock_, released_clock_;
  std::mutex send_mu_, recv_mu_;    // the pinned bounce buffers are shared by the channels' push / receive threads
  std::vector<void*> op_index_dev_;                   // per op: device copy of its gather index

  // communication
  // Channel 0: the control plane (heartbeats, barriers, handle exchange, placement service) and the tables with
  // id % channels == 0.  Every further channel is a full stack of its own - server shard on its own port, client
  // router with its own connections and reader threads, codec, push worker - and carries the tables with
  // id % channels == its index (the reference's comm channels: src/client/clientlib.cpp:72-158, :216-224).
  std::unique_ptr<ServerThreadEntry> server_;
  std::shared_ptr<RouterHandler> router_;
  std::unique_ptr<ClientServerEncode> encoder_;
  std::unique_ptr<ServerClientDecode> decoder_;
  struct Channel {
    std::unique_ptr<ServerThreadEntry> server;
    std::shared_ptr<RouterHandler> router;
    std::unique_ptr<ClientServerEncode> encoder;
    std::unique_ptr<ServerClientDecode> decoder;
  };
  std::vector<Channel> extra_channels_;     // channels 1 .. K-1
  uint num_channels() const { return (uint)extra_channels_.size() + 1; }
  uint channel_of(uint table_id) const { return table_id % num_channels(); }
  ClientServerEncode* enc(uint table_id) {
    const uint c = channel_of(table_id);
    return c == 0 ? encoder_.get() : extra_channels_[c - 1].encoder.get();
  }
  ServerThreadEntry* srv(uint table_id) {
    const uint c = channel_of(table_id);
    return c == 0 ? server_.get() : extra_channels_[c - 1].server.get();
  }
  bool open_channel(uint c, std::unique_ptr<ServerThreadEntry>* server, std::shared_ptr<RouterHandler>* router,
                    std::unique_ptr<ClientServerEncode>* encoder, std::unique_ptr<ServerClientDecode>* decoder,
                    std::string* err);
  std::vector<std::unique_ptr<BackgroundWorker>> bg_workers_;   // one per comm channel
  Fabric fabric_;

  // failure detection
  std::thread heartbeat_thread_;
  std::atomic<bool> stop_heartbeat_{false};
  std::atomic<bool> skip_heartbeats_{false}, withhold_push_signal_{false};
  std::mutex peers_mu_;
  std::vector<double> last_heartbeat_;
  std::vector<iter_t> peer_clock_;
  std::vector<char> peer_dead_;
  std::condition_variable global_cv_;
  std::map<std::pair<uint64_t, uint64_t>, int> located_;   // answers to locate_row (guarded by global_mu_)
  std::mutex global_mu_;
  std::map<uint, uint> barrier_seen_;      // rank -> last epoch seen
  uint barrier_epoch_ = 0;
  static constexpr uint kIpcRoundStride = 1u << 16;      // key of ipc_blobs_: rank + kIpcRoundStride * round
  std::map<uint, std::vector<char>> ipc_blobs_;
  std::map<uint, std::string> server_stats_;

  std::atomic<int> error_code_{0};
  std::mutex error_mu_;
  std::string error_text_;

  Stats stats_;
  BgthreadStats bg_stats_;
  // host time and call count of every declared access (indexed by handle), printed every log_interval clocks
  std::vector<double> op_time_;
  std::vector<uint64_t> op_calls_;
  void op_account(int handle, double t0);
  void dump_op_times();
  void fabric_collect_push_timing();
  int* row_status_dev_ = nullptr;      // status block of the row kernels on the host-staged GPU path
  int* row_status_host_ = nullptr;     // its pinned mirror
  bool check_row_status();
};

}  // namespace geeps_b200
