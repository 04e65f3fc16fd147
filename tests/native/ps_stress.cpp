// Multi-worker stress of the host runtime inside ONE process, meant to run under ThreadSanitizer /
// AddressSanitizer: W application threads, each with its own GeePs instance (worker + server shard) on host
// memory over TCP loopback.  Every clock every worker reads the table (SSP, slack given on the command line),
// checks the staleness bound, adds 1.0 to every element and keeps a worker-local batch through
// LocalAccess / PostLocalAccess.  With a fifth argument "sgd" the table is an optimizer table (momentum SGD on the
// shard), every worker changes the learning rate / momentum / weight decay every few clocks through
// SetHyperParams while the shards apply earlier clocks, and the final table is compared with the recurrence.
// Exit code 0 = all values and bounds held.
//
// The reference has no tests (its only program is apps/helloworld/helloworld.cpp, which never checks a value).
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "geeps.hpp"

namespace {
std::atomic<int> failures{0};

void worker(int rank, int world, int base_port, int rows, int clocks, int slack, bool sgd) {
  GeePsConfig cfg;
  cfg.device = GeePsConfig::DEVICE_CPU;
  cfg.transport = GeePsConfig::TRANSPORT_TCP;
  for (int r = 0; r < world; ++r) {
    cfg.host_list.push_back("127.0.0.1");
    cfg.port_list.push_back(base_port + 10 * r);
  }
  cfg.heartbeat_timeout_ms = 60000;
  cfg.host_wait_budget_ms = 60000;
  if (sgd) {
    cfg.table_mode = GeePsConfig::TABLE_SGD_MOMENTUM;
    cfg.learning_rate = 0.5f; cfg.momentum = 0.5f; cfg.weight_decay = 0.f;
    cfg.grad_scale = 1.f / (float)world;
  }
  GeePs ps(rank, cfg);
  std::vector<size_t> ids(rows), local_ids(8);
  for (int i = 0; i < rows; ++i) ids[i] = i;
  for (int i = 0; i < 8; ++i) local_ids[i] = 1000000 + i;
  const int h_read = ps.VirtualRead(0, ids, slack);
  const int h_loc = ps.VirtualLocalAccess(local_ids, true);
  const int h_pre = ps.VirtualPreUpdate(0, ids);
  const int h_postloc = ps.VirtualPostLocalAccess(h_loc, true);
  const int h_postread = ps.VirtualPostRead(h_read);
  const int h_upd = ps.VirtualUpdate(h_pre);
  ps.VirtualClock();
  ps.FinishVirtualIteration();
  // bootstrap: initial values (zeros) from every worker
  RowOpVal* ub = nullptr;
  ps.PreUpdate(h_pre, &ub);
  for (int i = 0; i < rows; ++i) ub[i].init();
  ps.Update(h_upd);
  ps.Clock();
  ps.StartIterations();
  // optimizer mode: the expected parameter value, stepped with the values in force at every clock
  double p_exp = 0.0, v_exp = 0.0;
  float lr = cfg.learning_rate, mom = cfg.momentum, wd = cfg.weight_decay;
  for (int c = 0; c < clocks; ++c) {
    if (sgd && c % 3 == 1) {   // every worker makes the same call before the same clock
      lr = 0.5f / (float)(1 + c); mom = (c % 2) ? 0.25f : 0.75f; wd = (c % 5 == 0) ? 0.125f : 0.f;
      ps.SetHyperParams(lr, mom, wd);
      float a = 0, b = 0, d = 0;
      ps.GetHyperParams(&a, &b, &d);
      if (a != lr || b != mom || d != wd) { ++failures; fprintf(stderr, "rank %d: hyper-parameters read back differ\n", rank); }
    }
    RowData* rb = nullptr;
    if (!ps.Read(h_read, &rb) || rb == nullptr) { ++failures; fprintf(stderr, "rank %d: read failed: %s\n", rank, ps.LastErrorString().c_str()); return; }
    // clock c reads at least every update of clocks <= c - slack - 1 and at most those of clocks <= c + slack
    if (sgd) {
      // slack 0 in this mode: the read of clock c holds exactly the updates of clocks < c
      if (std::fabs((double)rb[0].data[0] - p_exp) > 1e-3 * (1.0 + std::fabs(p_exp)) ||
          std::fabs((double)rb[rows - 1].data[77] - p_exp) > 1e-3 * (1.0 + std::fabs(p_exp))) {
        ++failures; fprintf(stderr, "rank %d clock %d: read %.6f, expected %.6f\n", rank, c, rb[0].data[0], p_exp);
      }
      v_exp = (double)mom * v_exp + (double)lr * (1.0 + (double)wd * p_exp);     // mean gradient 1.0
      p_exp -= v_exp;
    }
    const float v = rb[0].data[0], lo = sgd ? -1e30f : (float)world * (float)(c - slack > 0 ? c - slack : 0), hi = sgd ? 1e30f : (float)world * (float)(c + slack + 1);
    if (v < lo - 0.5f || v > hi + 0.5f) { ++failures; fprintf(stderr, "rank %d clock %d: read %.1f outside [%.1f, %.1f]\n", rank, c, v, lo, hi); }
    for (int i = 1; i < rows; ++i)
      if (rb[i].data[5] < lo - 0.5f || rb[i].data[5] > hi + 0.5f) { ++failures; break; }
    RowData* lb = nullptr;
    ps.LocalAccess(h_loc, &lb);
    if (c > 0 && lb[3].data[7] != (float)c) { ++failures; fprintf(stderr, "rank %d clock %d: local batch holds %.1f\n", rank, c, lb[3].data[7]); }
    for (int i = 0; i < 8; ++i) for (int k = 0; k < ROW_DATA_SIZE; ++k) lb[i].data[k] = (float)(c + 1);
    ps.PreUpdate(h_pre, &ub);
    for (int i = 0; i < rows; ++i) for (int k = 0; k < ROW_DATA_SIZE; ++k) ub[i].data[k] = 1.0f;
    ps.PostLocalAccess(h_postloc);
    ps.PostRead(h_postread);
    ps.Update(h_upd);
    ps.Clock();
    if (ps.LastError() != 0) { ++failures; fprintf(stderr, "rank %d: %s\n", rank, ps.LastErrorString().c_str()); return; }
  }
  const std::string stats = ps.GetStats();
  if (stats.find("\"clock\"") == std::string::npos) ++failures;
  ps.Shutdown();
}
}  // namespace

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 3;
  const int slack = argc > 2 ? atoi(argv[2]) : 1;
  const int clocks = argc > 3 ? atoi(argv[3]) : 30;
  const int base_port = argc > 4 ? atoi(argv[4]) : 21000;
  const bool sgd = argc > 5 && std::string(argv[5]) == "sgd";
  if (sgd && slack != 0) { fprintf(stderr, "the sgd mode checks exact values: slack must be 0\n"); return 2; }
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(worker, r, world, base_port, 48, clocks, slack, sgd);
  for (auto& t : th) t.join();
  printf("ps_stress: world %d slack %d clocks %d%s failures %d\n", world, slack, clocks, sgd ? " sgd" : "", failures.load());
  return failures.load() ? 1 : 0;
}
