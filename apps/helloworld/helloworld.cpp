// Smallest complete program against the public C++ API: one process, one table, one row, BSP.
// Same flow as the reference's demo (apps/helloworld/helloworld.cpp:10-71 of the reference) - virtual
// iteration, one bootstrap update, ten clocks of Read / PreUpdate / PostRead / Update / Clock - but this
// one writes values and checks them: every clock adds 1.0 to the row, so clock c reads c.
//
//   ./helloworld            uses the GPU when one is visible, host memory otherwise
//   ./helloworld cpu        forces host memory
#include <cuda_runtime.h>

#include <cstring>
#include <iostream>
#include <vector>

#include "geeps.hpp"

using std::cout;
using std::endl;
using std::vector;

static void fill(RowOpVal* buf, bool on_gpu, float v) {
  RowOpVal host;
  for (int i = 0; i < ROW_DATA_SIZE; ++i) host.data[i] = v;
  if (on_gpu) cudaMemcpy(buf, &host, sizeof(host), cudaMemcpyHostToDevice);
  else memcpy(buf, &host, sizeof(host));
}
static float first(const RowData* buf, bool on_gpu) {
  float v = 0;
  if (on_gpu) cudaMemcpy(&v, buf, sizeof(float), cudaMemcpyDeviceToHost);
  else v = buf->data[0];
  return v;
}

int main(int argc, char** argv) {
  GeePsConfig geeps_config;
  geeps_config.host_list.push_back("localhost");
  geeps_config.gpu_memory_capacity = (size_t)1 << 32;   /* 4 GB budget */
  int ndev = 0;
  const bool force_cpu = argc > 1 && std::string(argv[1]) == "cpu";
  if (force_cpu || cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    geeps_config.device = GeePsConfig::DEVICE_CPU;
  }
  const bool on_gpu = geeps_config.device == GeePsConfig::DEVICE_CUDA;
  GeePs* geeps = new GeePs(0, geeps_config);

  size_t table_id = 0;
  int slack = 0; /* BSP */
  vector<size_t> row_ids;
  row_ids.push_back(0);

  /* virtual iteration: declare one clock's accesses */
  int read_handle = geeps->VirtualRead(table_id, row_ids, slack);
  int preupdate_handle = geeps->VirtualPreUpdate(table_id, row_ids);
  int postread_handle = geeps->VirtualPostRead(read_handle);
  int update_handle = geeps->VirtualUpdate(preupdate_handle);
  geeps->VirtualClock();
  geeps->FinishVirtualIteration();

  /* bootstrap: the first update carries the initial values (zeros here) */
  RowOpVal* update_buffer;
  geeps->PreUpdate(preupdate_handle, &update_buffer);
  fill(update_buffer, on_gpu, 0.f);
  geeps->Update(update_handle);
  geeps->Clock();

  geeps->StartIterations();
  bool ok = true;
  for (int clock = 0; clock < 10; clock++) {
    RowData* read_buffer;
    geeps->Read(read_handle, &read_buffer);
    const float seen = first(read_buffer, on_gpu);
    ok = ok && seen == (float)clock;
    geeps->PreUpdate(preupdate_handle, &update_buffer);
    fill(update_buffer, on_gpu, 1.f);
    geeps->PostRead(postread_handle);
    geeps->Update(update_handle);
    geeps->Clock();
  }
  if (geeps->LastError()) { cout << "error: " << geeps->LastErrorString() << endl; ok = false; }
  geeps->Shutdown();
  delete geeps;
  cout << (ok ? "Finished \"training\", hello world!" : "helloworld FAILED") << " (" << (on_gpu ? "cuda" : "cpu") << ")\n";
  return ok ? 0 : 1;
}
