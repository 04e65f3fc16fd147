// Flat C API over the C++ runtime for the Python layer (ctypes) and for tests: the GeePs facade,
// the stand-alone plan compiler, the partitioner, the allocators and the host row-op oracle.
#include <cuda_runtime.h>
#include <string.h>

#include <string>
#include <vector>

#include "client/clientlib.hpp"
#include "core/common_util.hpp"
#include "core/partitioner.hpp"
#include "core/plan.hpp"
#include "core/row_op_util.hpp"
#include "geeps.hpp"

using namespace geeps_b200;

namespace {
int copy_out(const std::string& s, char* buf, int cap) {
  if (buf && cap > 0) {
    const int n = (int)s.size() < cap - 1 ? (int)s.size() : cap - 1;
    memcpy(buf, s.data(), (size_t)n);
    buf[n] = 0;
  }
  return (int)s.size() + 1;   // capacity needed
}
std::vector<size_t> rows_of(const long long* rows, int n) {
  std::vector<size_t> v((size_t)n);
  for (int i = 0; i < n; ++i) v[i] = (size_t)rows[i];
  return v;
}
}  // namespace

extern "C" {

// ---------------- config ----------------
void* geeps_config_new() { return new GeePsConfig(); }
void geeps_config_delete(void* c) { delete static_cast<GeePsConfig*>(c); }
void geeps_config_add_host(void* c, const char* host, int port) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  cfg->host_list.push_back(host);
  if (port > 0) cfg->port_list.push_back((uint)port);
}
int geeps_config_set(void* c, const char* key, double v) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  const std::string k(key);
  if (k == "num_tables") cfg->num_tables = (uint)v;
  else if (k == "tcp_base_port") cfg->tcp_base_port = (uint)v;
  else if (k == "num_comm_channels") cfg->num_comm_channels = (uint)v;
  else if (k == "log_interval") cfg->log_interval = (iter_t)v;
  else if (k == "pp_policy") cfg->pp_policy = (int)v;
  else if (k == "local_opt") cfg->local_opt = (int)v;
  else if (k == "gpu_memory_capacity") cfg->gpu_memory_capacity = v < 0 ? (size_t)-1 : (size_t)v;
  else if (k == "mm_warning_level") cfg->mm_warning_level = (int)v;
  else if (k == "pinned_cpu_memory") cfg->pinned_cpu_memory = (int)v;
  else if (k == "read_my_writes") cfg->read_my_writes = (int)v;
  else if (k == "device") cfg->device = (int)v;
  else if (k == "cuda_device") cfg->cuda_device = (int)v;
  else if (k == "transport") cfg->transport = (int)v;
  else if (k == "partitioner") cfg->partitioner = (int)v;
  else if (k == "table_mode") cfg->table_mode = (int)v;
  else if (k == "learning_rate") cfg->learning_rate = (float)v;
  else if (k == "momentum") cfg->momentum = (float)v;
  else if (k == "weight_decay") cfg->weight_decay = (float)v;
  else if (k == "grad_scale") cfg->grad_scale = (float)v;
  else if (k == "bf16_compute_cache") cfg->bf16_compute_cache = (int)v;
  else if (k == "use_multicast") cfg->use_multicast = (int)v;
  else if (k == "device_wait_budget_us") cfg->device_wait_budget_us = (size_t)v;
  else if (k == "host_wait_budget_ms") cfg->host_wait_budget_ms = (size_t)v;
  else if (k == "heartbeat_timeout_ms") cfg->heartbeat_timeout_ms = (size_t)v;
  else if (k == "snapshot_interval") cfg->snapshot_interval = (iter_t)v;
  else if (k == "num_workers_override") cfg->num_workers_override = (int)v;
  else return -1;
  return 0;
}
int geeps_config_set_str(void* c, const char* key, const char* v) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  const std::string k(key);
  if (k == "output_dir") cfg->output_dir = v;
  else if (k == "snapshot_dir") cfg->snapshot_dir = v;
  else return -1;
  return 0;
}
void geeps_config_set_table_mode(void* c, int table, int mode) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  if ((int)cfg->table_modes.size() <= table) cfg->table_modes.resize((size_t)table + 1, cfg->table_mode);
  cfg->table_modes[(size_t)table] = mode;
}
void geeps_config_set_table_pull(void* c, int table, int pull) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  if ((int)cfg->table_pull.size() <= table) cfg->table_pull.resize((size_t)table + 1, 0);
  cfg->table_pull[(size_t)table] = pull;
}
void geeps_config_set_table_partition_align(void* c, int table, long long rows) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  if ((int)cfg->table_partition_align.size() <= table) cfg->table_partition_align.resize((size_t)table + 1, 1);
  cfg->table_partition_align[(size_t)table] = rows > 0 ? (size_t)rows : 1;
}
void geeps_config_set_table_fp32_from_row(void* c, int table, long long row) {
  GeePsConfig* cfg = static_cast<GeePsConfig*>(c);
  if ((int)cfg->table_fp32_from_row.size() <= table) cfg->table_fp32_from_row.resize((size_t)table + 1, 0);
  cfg->table_fp32_from_row[(size_t)table] = (size_t)row;
}

// ---------------- GeePs facade ----------------
void* geeps_new(unsigned process_id, void* config) { return new GeePs(process_id, *static_cast<GeePsConfig*>(config)); }
void geeps_delete(void* g) { delete static_cast<GeePs*>(g); }
void geeps_shutdown(void* g) { static_cast<GeePs*>(g)->Shutdown(); }
int geeps_virtual_read(void* g, long long table, const long long* rows, int n, int slack) {
  return static_cast<GeePs*>(g)->VirtualRead((size_t)table, rows_of(rows, n), slack);
}
int geeps_virtual_post_read(void* g, int prestep) { return static_cast<GeePs*>(g)->VirtualPostRead(prestep); }
int geeps_virtual_pre_update(void* g, long long table, const long long* rows, int n) {
  return static_cast<GeePs*>(g)->VirtualPreUpdate((size_t)table, rows_of(rows, n));
}
int geeps_virtual_update(void* g, int prestep) { return static_cast<GeePs*>(g)->VirtualUpdate(prestep); }
int geeps_virtual_local_access(void* g, const long long* rows, int n, int fetch) {
  return static_cast<GeePs*>(g)->VirtualLocalAccess(rows_of(rows, n), fetch != 0);
}
int geeps_virtual_post_local_access(void* g, int prestep, int keep) {
  return static_cast<GeePs*>(g)->VirtualPostLocalAccess(prestep, keep != 0);
}
int geeps_virtual_clock(void* g) { return static_cast<GeePs*>(g)->VirtualClock(); }
void geeps_finish_virtual_iteration(void* g) { static_cast<GeePs*>(g)->FinishVirtualIteration(); }
void geeps_start_iterations(void* g) { static_cast<GeePs*>(g)->StartIterations(); }

int geeps_read(void* g, int handle, void** buf, void* stream, int async) {
  RowData* p = nullptr;
  const bool ok = static_cast<GeePs*>(g)->impl()->read_batch(handle, &p, stream, async != 0);
  *buf = p;
  return ok ? 1 : 0;
}
void geeps_post_read(void* g, int handle, void* stream) { static_cast<GeePs*>(g)->impl()->postread_batch(handle, stream); }
void geeps_pre_update(void* g, int handle, void** buf, void* stream) {
  RowOpVal* p = nullptr;
  static_cast<GeePs*>(g)->impl()->preupdate_batch(handle, &p, stream);
  *buf = p;
}
void geeps_update(void* g, int handle, void* stream, int async) {
  static_cast<GeePs*>(g)->impl()->update_batch(handle, stream, async != 0);
}
int geeps_local_access(void* g, int handle, void** buf, void* stream) {
  RowData* p = nullptr;
  const bool ok = static_cast<GeePs*>(g)->impl()->localaccess_batch(handle, &p, stream);
  *buf = p;
  return ok ? 1 : 0;
}
void geeps_post_local_access(void* g, int handle, void* stream) {
  static_cast<GeePs*>(g)->impl()->postlocalaccess_batch(handle, stream);
}
void geeps_clock(void* g) { static_cast<GeePs*>(g)->Clock(); }
int geeps_read_pull(void* g, int handle, void* info, void* stream) {
  return static_cast<GeePs*>(g)->ReadPull(handle, static_cast<GeePs::PullInfo*>(info), stream) ? 1 : 0;
}
void* geeps_read_bf16(void* g, int handle) { return static_cast<GeePs*>(g)->ReadBf16(handle); }
int geeps_enable_device_clock(void* g) { return static_cast<GeePs*>(g)->EnableDeviceClock() ? 1 : 0; }
void geeps_advance_replayed_clock(void* g) { static_cast<GeePs*>(g)->AdvanceReplayedClock(); }
const void* geeps_device_clock_ptr(void* g) { return static_cast<GeePs*>(g)->DeviceClockPtr(); }

// ---- stream fork / join for independent branches of a network (Inception modules) ----
void* geeps_event_new() {
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return e;
}
void geeps_event_delete(void* e) { if (e) cudaEventDestroy((cudaEvent_t)e); }
// work enqueued on `to` after this call starts only when everything enqueued on `from` so far has finished
int geeps_stream_order(void* from, void* to, void* event) {
  cudaError_t e = cudaEventRecord((cudaEvent_t)event, (cudaStream_t)from);
  if (e == cudaSuccess) e = cudaStreamWaitEvent((cudaStream_t)to, (cudaEvent_t)event, 0);
  return (int)e;
}

// ---- CUDA graph helpers: capture what is enqueued on `stream` (and on every stream that joins it through
// events) between begin and end, instantiate it, replay it ----
int geeps_graph_begin(void* stream) {
  return (int)cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeRelaxed);
}
int geeps_graph_end(void* stream, void** exec_out, long long* num_nodes) {
  *exec_out = nullptr;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &graph);
  if (e != cudaSuccess || graph == nullptr) { cudaGetLastError(); return e != cudaSuccess ? (int)e : (int)cudaErrorUnknown; }
  size_t n = 0;
  cudaGraphGetNodes(graph, nullptr, &n);
  if (num_nodes) *num_nodes = (long long)n;
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  *exec_out = exec;
  return 0;
}
int geeps_graph_launch(void* exec, void* stream) { return (int)cudaGraphLaunch((cudaGraphExec_t)exec, (cudaStream_t)stream); }
void geeps_graph_destroy(void* exec) { if (exec) cudaGraphExecDestroy((cudaGraphExec_t)exec); }

int geeps_current_clock(void* g) { return static_cast<GeePs*>(g)->CurrentClock(); }
void geeps_set_hyper_params(void* g, float lr, float momentum, float weight_decay) {
  static_cast<GeePs*>(g)->SetHyperParams(lr, momentum, weight_decay);
}
void geeps_get_hyper_params(void* g, float* out3) {
  static_cast<GeePs*>(g)->GetHyperParams(out3, out3 + 1, out3 + 2);
}
int geeps_last_error(void* g) { return static_cast<GeePs*>(g)->LastError(); }
int geeps_last_error_string(void* g, char* buf, int cap) { return copy_out(static_cast<GeePs*>(g)->LastErrorString(), buf, cap); }
int geeps_get_stats(void* g, char* buf, int cap) { return copy_out(static_cast<GeePs*>(g)->GetStats(), buf, cap); }
int geeps_plan_json(void* g, char* buf, int cap) { return copy_out(static_cast<GeePs*>(g)->PlanJson(), buf, cap); }
int geeps_save_snapshot(void* g, const char* dir) { return static_cast<GeePs*>(g)->SaveSnapshot(dir) ? 1 : 0; }
int geeps_load_snapshot(void* g, const char* dir) { return static_cast<GeePs*>(g)->LoadSnapshot(dir) ? 1 : 0; }
// host-side fault injection for tests: 0 = stop sending heartbeats, 1 = withhold the push-ready flag,
// 2 = drop the next `value` inbound row batches at the client router
int geeps_locate_row(void* g, long long table, long long row, int metadata_server, int timeout_ms) {
  return static_cast<GeePs*>(g)->impl()->locate_row((uint64_t)table, (uint64_t)row, (uint)metadata_server, timeout_ms);
}
void geeps_report_access(void* g, int metadata_server, long long table, long long row, int nread, int nwrite) {
  static_cast<GeePs*>(g)->impl()->report_access((uint)metadata_server, (uint64_t)table, (uint64_t)row, (uint32_t)nread,
                                                (uint32_t)nwrite);
}
void geeps_inject(void* g, int what, int value) {
  ClientLib* lib = static_cast<GeePs*>(g)->impl();
  if (what == 0) lib->inject_skip_heartbeats(value != 0);
  else if (what == 1) lib->inject_withhold_push_signal(value != 0);
  else if (what == 2) lib->client_router()->drop_inbound(CMD_READ_ROW_BATCH, value);
}

// ---------------- stand-alone plan compiler ----------------
void* geeps_planner_new(long long capacity_bytes, int mm_warning_level, int read_my_writes, int num_shards,
                        int partitioner, int num_tables, int device_is_gpu, int allow_direct, int update_ring) {
  PlanConfig pc;
  pc.gpu_memory_capacity = capacity_bytes < 0 ? (size_t)-1 : (size_t)capacity_bytes;
  pc.mm_warning_level = mm_warning_level;
  pc.read_my_writes = read_my_writes;
  pc.num_shards = num_shards;
  pc.partitioner = partitioner;
  pc.num_tables = (size_t)num_tables;
  pc.device_is_gpu = device_is_gpu != 0;
  pc.allow_direct = allow_direct != 0;
  pc.update_ring = update_ring != 0;
  return new PlanCompiler(pc);
}
void geeps_planner_delete(void* p) { delete static_cast<PlanCompiler*>(p); }
int geeps_planner_record(void* p, int type, long long table, const long long* rows, int n, int slack, int prestep,
                         int fetch, int keep) {
  OpInfo op;
  op.type = (OpType)type;
  op.table = (size_t)table;
  op.rows = rows_of(rows, n);
  op.slack = slack;
  op.prestep = prestep;
  op.fetch = fetch != 0;
  op.keep = keep != 0;
  op.local = type == OP_LOCAL_ACCESS || type == OP_POST_LOCAL_ACCESS;
  return static_cast<PlanCompiler*>(p)->record(op);
}
int geeps_planner_compile_json(void* p, char* buf, int cap) {
  return copy_out(static_cast<PlanCompiler*>(p)->compile().to_json(), buf, cap);
}

// ---------------- partitioner ----------------
void geeps_partition_range(int kind, long long num_rows, int num_shards, int shard, long long* out3) {
  ShardRange r = Partitioner(kind, (size_t)num_rows, (size_t)num_shards).range_of((size_t)shard);
  out3[0] = (long long)r.start; out3[1] = (long long)r.stride; out3[2] = (long long)r.count;
}
void geeps_partition_range_aligned(int kind, long long num_rows, int num_shards, int shard, long long align,
                                   long long* out3) {
  ShardRange r = Partitioner(kind, (size_t)num_rows, (size_t)num_shards, (size_t)align).range_of((size_t)shard);
  out3[0] = (long long)r.start; out3[1] = (long long)r.stride; out3[2] = (long long)r.count;
}
int geeps_partition_shard_of(int kind, long long num_rows, int num_shards, long long i) {
  return (int)Partitioner(kind, (size_t)num_rows, (size_t)num_shards).shard_of((size_t)i);
}

// ---------------- allocators ----------------
void* geeps_mtcache_new(long long size) { auto* h = new MultithreadedCacheHelper(); h->init((size_t)size); return h; }
void geeps_mtcache_delete(void* h) { delete static_cast<MultithreadedCacheHelper*>(h); }
long long geeps_mtcache_get(void* h, long long count, int wait, int tag, long long budget_ms) {
  const size_t s = static_cast<MultithreadedCacheHelper*>(h)->get((size_t)count, wait != 0, tag, (size_t)budget_ms);
  return s == (size_t)-1 ? -1 : (long long)s;
}
void geeps_mtcache_put(void* h, long long start, long long count) {
  static_cast<MultithreadedCacheHelper*>(h)->put((size_t)start, (size_t)count);
}
long long geeps_mtcache_used(void* h) { return (long long)static_cast<MultithreadedCacheHelper*>(h)->used(); }
void* geeps_ringcache_new(long long size) { auto* h = new SimpleCacheHelper(); h->init((size_t)size); return h; }
void geeps_ringcache_delete(void* h) { delete static_cast<SimpleCacheHelper*>(h); }
long long geeps_ringcache_get(void* h, long long count) {
  const size_t s = static_cast<SimpleCacheHelper*>(h)->get((size_t)count);
  return s == (size_t)-1 ? -1 : (long long)s;
}
void geeps_ringcache_put(void* h, long long start, long long count) {
  static_cast<SimpleCacheHelper*>(h)->put((size_t)start, (size_t)count);
}

// ---------------- host oracle ----------------
void geeps_cpu_row_gather(float* y, const float* x, const long long* index, long long n, long long off0, long long off1,
                          long long limit) {
  assign_rows_to_double_index_cpu(reinterpret_cast<RowData*>(y), reinterpret_cast<const RowData*>(x),
                                  reinterpret_cast<const DoubleIndex*>(index), (size_t)n, (size_t)off0, (size_t)off1,
                                  (size_t)limit);
}
void geeps_cpu_row_scatter(float* y, const float* x, const long long* index, long long n, long long off0,
                           long long off1, long long limit) {
  assign_rows_from_double_index_cpu(reinterpret_cast<RowData*>(y), reinterpret_cast<const RowData*>(x),
                                    reinterpret_cast<const DoubleIndex*>(index), (size_t)n, (size_t)off0, (size_t)off1,
                                    (size_t)limit);
}
void geeps_cpu_row_scatter_add(float* y, const float* x, const long long* index, long long n, long long off0,
                               long long off1, long long limit) {
  add_rows_from_double_index_cpu(reinterpret_cast<RowData*>(y), reinterpret_cast<const RowData*>(x),
                                 reinterpret_cast<const DoubleIndex*>(index), (size_t)n, (size_t)off0, (size_t)off1,
                                 (size_t)limit);
}
void geeps_cpu_sgd_momentum(long long n, float* p, float* v, const float* g, float lr, float momentum,
                            float weight_decay, float grad_scale) {
  OptimizerParams o;
  o.lr = lr; o.momentum = momentum; o.weight_decay = weight_decay; o.grad_scale = grad_scale;
  cpu_sgd_momentum((size_t)n, p, v, g, o);
}
int geeps_cuda_available() { return Mem::cuda_available() ? 1 : 0; }

}  // extern "C"
