// GeePs facade: forwards to a ClientLib instance (the reference's facade forwards to a process-wide
// singleton: src/client/geeps.cpp:41-132).
#include "geeps.hpp"

#include "clientlib.hpp"

using geeps_b200::ClientLib;

GeePs::GeePs(uint process_id, const GeePsConfig& config) : impl_(new ClientLib(process_id, config)) {}
GeePs::~GeePs() { delete impl_; }
void GeePs::Shutdown() { impl_->shutdown(); }
std::string GeePs::GetStats() { return impl_->json_stats(); }
void GeePs::StartIterations() { impl_->start_opseq(); }

int GeePs::VirtualRead(size_t table_id, const vector<size_t>& row_ids, int slack) {
  return impl_->virtual_read_batch(table_id, row_ids, slack);
}
int GeePs::VirtualPostRead(int prestep_handle) { return impl_->virtual_postread_batch(prestep_handle); }
int GeePs::VirtualPreUpdate(size_t table_id, const vector<size_t>& row_ids) {
  return impl_->virtual_preupdate_batch(table_id, row_ids);
}
int GeePs::VirtualUpdate(int prestep_handle) { return impl_->virtual_update_batch(prestep_handle); }
int GeePs::VirtualLocalAccess(const vector<size_t>& row_ids, bool fetch) {
  return impl_->virtual_localaccess_batch(row_ids, fetch);
}
int GeePs::VirtualPostLocalAccess(int prestep_handle, bool keep) {
  return impl_->virtual_postlocalaccess_batch(prestep_handle, keep);
}
int GeePs::VirtualClock() { return impl_->virtual_clock(); }
void GeePs::FinishVirtualIteration() { impl_->finish_virtual_iteration(); }

bool GeePs::Read(int handle, RowData** buffer_ptr) { return impl_->read_batch(handle, buffer_ptr, nullptr, false); }
void GeePs::PostRead(int handle) { impl_->postread_batch(handle); }
void GeePs::PreUpdate(int handle, RowOpVal** buffer_ptr) { impl_->preupdate_batch(handle, buffer_ptr, nullptr); }
void GeePs::Update(int handle) { impl_->update_batch(handle, nullptr, false); }
bool GeePs::LocalAccess(int handle, RowData** buffer_ptr) { return impl_->localaccess_batch(handle, buffer_ptr, nullptr); }
void GeePs::PostLocalAccess(int handle) { impl_->postlocalaccess_batch(handle, nullptr); }
void GeePs::Clock() { impl_->iterate(); }

bool GeePs::ReadAsync(int handle, RowData** buffer_ptr, void* cuda_stream) {
  return impl_->read_batch(handle, buffer_ptr, cuda_stream, true);
}
void GeePs::UpdateAsync(int handle, void* cuda_stream) { impl_->update_batch(handle, cuda_stream, true); }
void* GeePs::ReadBf16(int handle) { return impl_->read_bf16(handle); }
int GeePs::LastError() const { return impl_->last_error(); }
std::string GeePs::LastErrorString() const { return impl_->last_error_string(); }
bool GeePs::SaveSnapshot(const std::string& dir) { return impl_->save_snapshot(dir); }
bool GeePs::LoadSnapshot(const std::string& dir) { return impl_->load_snapshot(dir); }
std::string GeePs::PlanJson() const { return impl_->plan_json(); }
bool GeePs::ReadPull(int handle, PullInfo* info, void* cuda_stream) { return impl_->read_pull(handle, info, cuda_stream); }
bool GeePs::EnableDeviceClock() { return impl_->enable_device_clock(); }
void GeePs::AdvanceReplayedClock() { impl_->advance_replayed_iteration(); }
const int* GeePs::DeviceClockPtr() const { return impl_->device_clock_ptr(); }
iter_t GeePs::CurrentClock() const { return impl_->current_clock(); }
void GeePs::SetHyperParams(float learning_rate, float momentum, float weight_decay) {
  impl_->set_hyper_params(learning_rate, momentum, weight_decay);
}
void GeePs::GetHyperParams(float* learning_rate, float* momentum, float* weight_decay) const {
  const geeps_b200::HyperSchedule::Entry h = impl_->hyper_params();
  if (learning_rate) *learning_rate = h.lr;
  if (momentum) *momentum = h.momentum;
  if (weight_decay) *weight_decay = h.weight_decay;
}
