#ifndef GEEPS_B200_GEEPS_HPP_
#define GEEPS_B200_GEEPS_HPP_
// Public C++ API of the B200-native GPU parameter server.
//
// The class and the first thirteen GeePsConfig fields are source-compatible with the
// reference's include/geeps.hpp:42-98: an application written against that header compiles
// against this one.  Everything after `read_my_writes` in the config, the *Async calls, the
// snapshot calls and the error accessors are additions.
//
// Life cycle: construct -> Virtual* calls (declare one iteration's accesses, get handles) ->
// FinishVirtualIteration() (compiles the memory + communication plan) -> optional bootstrap
// accesses in any order + Clock() -> StartIterations() -> the declared accesses in exactly the
// declared order, every clock.
#include <limits>
#include <string>
#include <vector>

#include "geeps-user-defined-types.hpp"

using std::string;
using std::vector;

struct GeePsConfig {
  uint num_tables;
  std::vector<std::string> host_list;
  std::vector<uint> port_list;   /* per-process TCP port (honoured; lets several processes share a host) */
  uint tcp_base_port;
  uint num_comm_channels;
  std::string output_dir;
  iter_t log_interval;
  int pp_policy;
  int local_opt;
  size_t gpu_memory_capacity;
  int mm_warning_level;
      /* 0: no warning
       * 1: guarantee double buffering for the staging pool
       * 2: make sure all local data is in GPU memory
       * 3: make sure the whole parameter cache is in GPU memory */
  int pinned_cpu_memory;
  int read_my_writes;

  /* ---- additions ---- */
  enum Device { DEVICE_CPU = 0, DEVICE_CUDA = 1 };
  enum Transport { TRANSPORT_TCP = 0, TRANSPORT_NVLINK = 1 };
  enum Partitioner { PARTITION_RANGE = 0, PARTITION_ROUND_ROBIN = 1 };
  enum TableMode { TABLE_ADDITIVE = 0, TABLE_SGD_MOMENTUM = 1 };
  int device;                 /* where caches and staging live */
  int cuda_device;            /* CUDA ordinal for DEVICE_CUDA (-1: current device) */
  int transport;              /* TCP: host-staged messages; NVLINK: in-kernel peer loads/stores */
  int partitioner;
  int table_mode;             /* default mode of every table */
  std::vector<int> table_modes;  /* optional per-table override */
  /* NVLINK transport with bf16_compute_cache: rows of table t below table_fp32_from_row[t] are published to the
     workers' bf16 caches only - their fp32 cache rows (what Read returns) are not refreshed.  For tables whose
     leading rows (weights) are consumed through ReadBf16 only; default: every row also in fp32. */
  std::vector<size_t> table_fp32_from_row;
  /* NVLINK transport, per table: 1 = the table is uncached ("pull" table).  Workers keep no copy of its rows: the
     owning shards hold the fp32 master rows (and a bf16 copy with bf16_compute_cache) and a Read fetches the whole
     table from them over NVLink into the staging pool - the device-side form of a parameter cache that does not
     fit the GPU budget.  ReadPull gives a consumer (a GEMM that pulls while it computes) the shard pointers. */
  std::vector<int> table_pull;
  /* per table: the range partition hands out rows in groups of this many (0 / 1: single rows), so that a matrix
     row spanning several 128-float table rows never straddles two shards */
  std::vector<size_t> table_partition_align;
  /* NVLINK transport: allocate the arena through the virtual-memory API, bind it to an NVSwitch multicast object and
     let the push kernel reduce (multimem.ld_reduce) and publish (multimem.st) through it.  Falls back to peer loads
     and stores when a device lacks multicast support.  Sums are then added inside the switch, in an order the
     switch chooses; the peer-load kernel adds in rank order. */
  int use_multicast;
  float learning_rate, momentum, weight_decay;
  float grad_scale;           /* multiplies the reduced update before the optimizer (e.g. 1/workers) */
  int bf16_compute_cache;     /* also keep a bf16 copy of the parameter cache (NVLINK transport) */
  size_t device_wait_budget_us;  /* bound of every device-side flag wait */
  size_t host_wait_budget_ms;    /* bound of every host-side blocking wait (0 = wait forever, log every 12 s) */
  size_t heartbeat_timeout_ms;   /* a peer silent for this long is declared lost */
  std::string snapshot_dir;
  iter_t snapshot_interval;
  int num_workers_override;   /* 0: one worker per host_list entry */

  GeePsConfig() :
    num_tables(1),
    tcp_base_port(9090),
    num_comm_channels(1),
    output_dir(""), log_interval(0),
    pp_policy(0), local_opt(1),
    gpu_memory_capacity(std::numeric_limits<size_t>::max()),
    mm_warning_level(1),
    pinned_cpu_memory(1),
    read_my_writes(0),
    device(DEVICE_CUDA), cuda_device(-1), transport(TRANSPORT_TCP),
    partitioner(PARTITION_RANGE), table_mode(TABLE_ADDITIVE), use_multicast(0),
    learning_rate(0.01f), momentum(0.9f), weight_decay(0.f), grad_scale(1.f),
    bf16_compute_cache(0),
    device_wait_budget_us(30u * 1000u * 1000u), host_wait_budget_ms(0), heartbeat_timeout_ms(30000),
    snapshot_dir(""), snapshot_interval(0), num_workers_override(0) {}
};

namespace geeps_b200 { class ClientLib; }

class GeePs {
 public:
  GeePs(uint process_id, const GeePsConfig& config);
  ~GeePs();
  void Shutdown();
  std::string GetStats();
  void StartIterations();

  /* Interfaces for virtual iteration */
  int VirtualRead(size_t table_id, const vector<size_t>& row_ids, int slack);
  int VirtualPostRead(int prestep_handle);
  int VirtualPreUpdate(size_t table_id, const vector<size_t>& row_ids);
  int VirtualUpdate(int prestep_handle);
  int VirtualLocalAccess(const vector<size_t>& row_ids, bool fetch);
  int VirtualPostLocalAccess(int prestep_handle, bool keep);
  int VirtualClock();
  void FinishVirtualIteration();

  /* Interfaces for real access */
  bool Read(int handle, RowData **buffer_ptr);
  void PostRead(int handle);
  void PreUpdate(int handle, RowOpVal **buffer_ptr);
  void Update(int handle);
  bool LocalAccess(int handle, RowData **buffer_ptr);
  void PostLocalAccess(int handle);
  void Clock();

  /* ---- additions ---- */
  /* Stream-aware variants: enqueue the work (and any device-side SSP wait) on `cuda_stream`
   * and return without synchronising the host. */
  bool ReadAsync(int handle, RowData **buffer_ptr, void *cuda_stream);
  void UpdateAsync(int handle, void *cuda_stream);
  /* bf16 view of a Read buffer when bf16_compute_cache is on and the batch is cache-contiguous */
  void *ReadBf16(int handle);
  /* 0 when healthy; otherwise the first error (expired wait, dead peer, ...) and its text */
  int LastError() const;
  std::string LastErrorString() const;
  /* Table snapshots: rows, optimizer momentum and clocks.  The hyper-parameters of a resumed run come from its
   * config and its own SetHyperParams calls (the manifest records the values in force for reference). */
  bool SaveSnapshot(const std::string& dir);
  bool LoadSnapshot(const std::string& dir);
  /* The compiled plan as JSON (placement, offsets, indices, per-shard ranges) */
  std::string PlanJson() const;
  iter_t CurrentClock() const;
  /* Optimizer tables: learning rate, momentum and weight decay of the shard-side optimizer for the updates of the
   * iteration in progress and all later ones (a learning-rate policy calls this between iterations).  Every worker
   * makes the same call in the same iteration, so all shards switch at the same clock.  Iterations captured in a
   * CUDA graph keep the values of the time of capture. */
  void SetHyperParams(float learning_rate, float momentum, float weight_decay);
  void GetHyperParams(float* learning_rate, float* momentum, float* weight_decay) const;
  /* NVLINK transport: keep the clock in a device word, so that the launches of one iteration carry no value that
   * changes from clock to clock and can be captured in a CUDA graph (one graph per phase of the update ring, i.e.
   * per clock modulo slack + 1).  From then on Clock() joins the runtime's streams into the stream of the latest
   * access call and advances the device word there.  After replaying a captured iteration, call
   * AdvanceReplayedClock() instead of repeating the access calls.  DeviceClockPtr() is the device word (an int that
   * kernels of the application may read, e.g. to derive per-step random seeds). */
  bool EnableDeviceClock();
  void AdvanceReplayedClock();
  const int* DeviceClockPtr() const;
  /* Uncached (pull) tables.  ReadPull stands in for Read in the declared sequence: it orders `cuda_stream` after
   * the table's freshness condition, fetches the rows from `table_fp32_from_row` on (fp32, e.g. biases) into a
   * private buffer, and describes where the leading rows live on the shards so that the caller's kernel can read
   * them in place: shard s holds rows [row_start[s], row_start[s] + row_count[s]) as bf16 at shard_bf16[s] (a peer
   * pointer, 128 values per row) and as fp32 at shard_fp32[s]. */
  struct PullInfo {
    const void* shard_bf16[8];
    const float* shard_fp32[8];
    long long row_start[8], row_count[8];
    int num_shards;
    RowData* tail;              /* rows [tail_from_row, end) in fp32, private to this worker */
    long long tail_from_row, tail_rows;
  };
  bool ReadPull(int handle, PullInfo* info, void* cuda_stream);
  geeps_b200::ClientLib* impl() { return impl_; }

 private:
  GeePs(const GeePs&);
  GeePs& operator=(const GeePs&);
  geeps_b200::ClientLib* impl_;
};

#endif  // GEEPS_B200_GEEPS_HPP_
