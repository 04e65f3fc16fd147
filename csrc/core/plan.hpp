// Access-plan compiler ("virtual iteration" -> static memory and communication plan).
//
// Input: the op sequence one iteration will issue (Read / PostRead / PreUpdate / Update /
// LocalAccess / PostLocalAccess / Clock) and a GPU memory budget.  Output, all decided on the
// host before the first real clock:
//   * which worker-local row batches stay resident in GPU memory and which live in (pinned)
//     host memory and are swapped through the staging pool,
//   * which parameter batches are cached in GPU memory and which in host memory,
//   * a static offset in the staging pool for every access that needs a buffer (interval
//     colouring over the op sequence, two copies for double buffering across clocks),
//   * per-op gather indices (buffer position -> cache position), whether the op can be served
//     zero-copy straight from the cache, and which Update is the last write of its table,
//   * per-table row lists and per-shard ranges.
//
// Covers the same decisions as the reference's src/client/clientlib-viter.cpp:120-883
// (vi_create_local_storage, vi_decide_param_cache, vi_create_thread_cache,
// vi_process_channel_table_finalize, vi_thread_finalize, vi_create_double_index) with the same
// budget rules (gpu_memory_capacity, mm_warning_level 1/2/3, 2x peak staging); because the
// sequence is cyclic and known, buffers get fixed offsets instead of a run-time allocator.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "partitioner.hpp"
#include "row_op_util.hpp"

namespace geeps_b200 {

enum OpType {
  OP_READ = 0, OP_POST_READ = 1, OP_PRE_UPDATE = 2, OP_UPDATE = 3,
  OP_LOCAL_ACCESS = 4, OP_POST_LOCAL_ACCESS = 5, OP_CLOCK = 6
};
enum DataLocation { LOC_UNKNOWN = 0, LOC_GPU = 1, LOC_CPU = 2 };

struct OpInfo {
  // ---- recorded ----
  OpType type = OP_CLOCK;
  size_t table = 0;
  std::vector<size_t> rows;
  int slack = 0;
  int prestep = -1;        // handle of the matching pre-op (post ops only)
  bool local = false;      // worker-private rows (LocalAccess family)
  bool fetch = false;      // LocalAccess: contents needed (H2D when CPU-resident)
  bool keep = false;       // PostLocalAccess: contents must survive (D2H when CPU-resident)
  // ---- planned ----
  int post = -1;                 // handle of the matching post-op (pre ops only)
  bool one_off = false;          // recorded after the Clock: not repeated
  size_t num_vals_limit = 0;     // rows * 128
  DataLocation location = LOC_UNKNOWN;   // of the backing data (param cache part or local storage)
  bool direct = false;           // served zero-copy from the cache / resident local storage
  bool needs_staging = false;
  size_t staging_offset = 0;     // rows, inside one copy of the staging pool
  size_t store_offset = 0;       // first row in the backing storage (local storage or cache slot)
  bool contiguous = false;       // the batch is one ascending run of cache slots
  bool table_last_write = false; // Update: last write of its table before the Clock
  bool last_access_of_batch = false;  // PostLocalAccess: last post-access of its batch in the iteration
  std::vector<DoubleIndex> index;     // (position in batch, cache slot) for non-local pre ops
};

struct TablePlan {
  size_t table_id = 0;
  std::vector<size_t> rows;            // sorted unique row ids = cache index -> row id
  std::map<size_t, size_t> row_to_idx; // row id -> cache index
  std::vector<int> location;           // per cache index: LOC_GPU / LOC_CPU
  std::vector<size_t> slot;            // per cache index: position inside the GPU or CPU part
  size_t gpu_rows = 0, cpu_rows = 0;
  int slack = 0;
  int num_oplog_entries = 1;
  std::vector<ShardRange> shard_ranges;  // over the cache index space
  size_t partition_per = 0;              // rows per shard of the range partition (alignment included)
  bool pull = false;                     // uncached: reads are fetched from the owning shards
  bool written = false;
};

struct PlanConfig {
  size_t gpu_memory_capacity = (size_t)-1;   // bytes
  int mm_warning_level = 1;
  int read_my_writes = 0;
  int num_shards = 1;
  int partitioner = PARTITION_RANGE;
  size_t num_tables = 1;
  bool device_is_gpu = true;     // false: everything is host memory, the budget is not enforced
  bool allow_direct = false;     // zero-copy param access (NVLINK transport)
  bool update_ring = false;      // update staging is a ring of slack+1 slots (NVLINK transport)
  // per table (by id; missing entries = default): rows per alignment group of the range partition, and whether the
  // table is kept uncached ("pull" tables: no worker-side copy, a Read fetches the rows from the owning shards)
  std::vector<size_t> partition_align;
  std::vector<char> pull_tables;
};

struct Plan {
  std::vector<OpInfo> ops;
  std::map<size_t, TablePlan> tables;
  int clock_handle = -1;
  size_t capacity_rows = 0;
  size_t peak_staging_rows = 0;     // max rows simultaneously staged
  size_t staging_rows = 0;          // size of ONE copy of the staging pool (>= peak)
  int staging_copies = 2;           // 2 = double buffered across clocks
  size_t gpu_local_rows = 0, cpu_local_rows = 0;
  size_t gpu_param_rows = 0, cpu_param_rows = 0;
  size_t uncached_param_rows = 0;   // rows of pull tables: no worker-side cache, fetched from the shards per Read
  size_t max_access_rows = 0;
  int pf_slack = 0;
  std::vector<std::string> warnings;
  std::string error;                // non-empty: the plan violates the requested mm_warning_level
  bool ok() const { return error.empty(); }
  size_t gpu_rows_total() const;
  std::string to_json() const;
};

class PlanCompiler {
 public:
  explicit PlanCompiler(const PlanConfig& cfg) : cfg_(cfg) {}
  // Recording: returns the handle (index in the sequence)
  int record(const OpInfo& op) { ops_.push_back(op); return (int)ops_.size() - 1; }
  size_t num_ops() const { return ops_.size(); }
  const OpInfo& op(int h) const { return ops_[h]; }
  Plan compile() const;

 private:
  PlanConfig cfg_;
  std::vector<OpInfo> ops_;
};

}  // namespace geeps_b200
