#include "metadata_server.hpp"

#include <algorithm>
#include <sstream>

#include "server_encoder_decoder.hpp"

namespace geeps_b200 {

MetadataServer::MetadataServer(uint server_id, uint num_servers, std::shared_ptr<ServerClientEncode> communicator,
                               const GeePsConfig& config)
    : server_id_(server_id), num_servers_(num_servers ? num_servers : 1), communicator_(communicator),
      policy_(config.pp_policy), load_(num_servers_, 0) {}

void MetadataServer::add_access_info(uint client_id, const std::vector<access_info_t>& infos) {
  for (const access_info_t& a : infos) {
    RowInfo& r = rows_[{a.table, a.row}];
    if (r.access.size() < num_servers_) r.access.resize(num_servers_, 0);
    if (client_id < num_servers_) r.access[client_id] += a.nread + a.nwrite;
    if (policy_ == 2 && r.owner < 0) { r.owner = (int)(client_id % num_servers_); load_[r.owner]++; }
  }
}

void MetadataServer::decide_data_assignment() {
  if (decided_ || policy_ != 3) { decided_ = true; serve_pending_requests(); return; }
  // most frequent accessor wins unless it already owns more than its fair share
  const uint64_t fair = rows_.size() / num_servers_ + 1;
  for (auto& kv : rows_) {
    RowInfo& r = kv.second;
    if (r.owner >= 0) continue;
    std::vector<uint> order(num_servers_);
    for (uint s = 0; s < num_servers_; ++s) order[s] = s;
    std::stable_sort(order.begin(), order.end(), [&](uint a, uint b) {
      const uint32_t ca = a < r.access.size() ? r.access[a] : 0, cb = b < r.access.size() ? r.access[b] : 0;
      return ca > cb;
    });
    for (uint s : order)
      if (load_[s] < fair) { r.owner = (int)s; break; }
    if (r.owner < 0) r.owner = (int)order[0];
    load_[r.owner]++;
  }
  decided_ = true;
  serve_pending_requests();
}

uint MetadataServer::owner_of(uint64_t table, uint64_t row) const {
  auto it = rows_.find({table, row});
  if (it != rows_.end() && it->second.owner >= 0) return (uint)it->second.owner;
  return (uint)(row % num_servers_);   // policy 1 and the default: hash
}

void MetadataServer::find_row(uint client_id, uint64_t table, uint64_t row) {
  nr_requests_++;
  if (policy_ == 3 && !decided_) { pending_.push_back({client_id, table, row}); return; }
  if (policy_ == 2) {
    RowInfo& r = rows_[{table, row}];
    if (r.owner < 0) { r.owner = (int)(client_id % num_servers_); load_[r.owner]++; }
  }
  communicator_->find_row(client_id, table, row, owner_of(table, row));
}

void MetadataServer::serve_pending_requests() {
  for (const Pending& p : pending_) communicator_->find_row(p.client, p.table, p.row, owner_of(p.table, p.row));
  pending_.clear();
}

void MetadataServer::reply_stats(uint client_id, const std::string& stats) { communicator_->get_stats(client_id, stats); }

std::string MetadataServer::get_stats() const {
  std::ostringstream o;
  o << "{\"policy\":" << policy_ << ",\"rows_tracked\":" << rows_.size() << ",\"nr_requests\":" << nr_requests_ << "}";
  return o.str();
}

}  // namespace geeps_b200
