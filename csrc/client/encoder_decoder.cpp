#include "encoder_decoder.hpp"

#include "clientlib.hpp"

namespace geeps_b200 {

ClientServerEncode::ClientServerEncode(std::shared_ptr<RouterHandler> router, uint num_servers, uint client_id,
                                       const GeePsConfig& config)
    : router_(router), num_servers_(num_servers), client_id_(client_id), config_(config) {}

std::string ClientServerEncode::server_name(uint server_id) const {
  if (config_.local_opt && server_id == client_id_) return "local";
  return "tablet-" + std::to_string(server_id);
}

std::vector<std::string> ClientServerEncode::all_servers() const {
  std::vector<std::string> v;
  for (uint s = 0; s < num_servers_; ++s) v.push_back(server_name(s));
  return v;
}

void ClientServerEncode::find_row(uint64_t table, uint64_t row, uint metadata_server_id) {
  Message msg(1);
  cs_find_row_msg_t h{CMD_FIND_ROW, client_id_, table, row};
  msg[0].pack(h);
  router_->send_to(server_name(metadata_server_id), std::move(msg));
}

void ClientServerEncode::clock_to(uint server_id, iter_t clock, uint table_id) {
  Message msg(1);
  cs_clock_msg_t h{CMD_CLOCK, client_id_, clock, table_id};
  msg[0].pack(h);
  router_->send_to(server_name(server_id), std::move(msg));
}

void ClientServerEncode::clock_broadcast(iter_t clock, uint table_id) {
  for (uint s = 0; s < num_servers_; ++s) clock_to(s, clock, table_id);
}

bool ClientServerEncode::clock_with_updates_batch(uint server_id, iter_t clock, uint table_id, const RowKey* keys,
                                                  const RowOpVal* rows, size_t num_rows, bool is_init) {
  return clock_with_updates_batch(server_id, clock, table_id, keys, rows, num_rows, nullptr, 0, is_init);
}

bool ClientServerEncode::clock_with_updates_batch(uint server_id, iter_t clock, uint table_id, const RowKey* keys,
                                                  const RowOpVal* rows0, size_t n0, const RowOpVal* rows1, size_t n1,
                                                  bool is_init) {
  Message msg(3);
  cs_clock_with_updates_batch_msg_t h{CMD_CLOCK_WITH_UPDATES_BATCH, client_id_, clock, table_id, (uint64_t)(n0 + n1),
                                      is_init ? 1u : 0u};
  msg[0].pack(h);
  msg[1].pack_memory(keys, (n0 + n1) * sizeof(RowKey));
  msg[2].pack_memory(rows0, n0 * sizeof(RowOpVal), rows1, n1 * sizeof(RowOpVal));
  return router_->send_to(server_name(server_id), std::move(msg));
}

void ClientServerEncode::add_access_info(uint metadata_server_id, const std::vector<access_info_t>& infos) {
  Message msg(2);
  cs_add_access_info_msg_t h{CMD_ADD_ACCESS_INFO, client_id_, (uint64_t)infos.size()};
  msg[0].pack(h);
  msg[1].pack_vector(infos);
  router_->send_to(server_name(metadata_server_id), std::move(msg));
}

void ClientServerEncode::get_stats(uint server_id) {
  Message msg(1);
  cs_get_stats_msg_t h{CMD_GET_STATS, client_id_};
  msg[0].pack(h);
  router_->send_to(server_name(server_id), std::move(msg));
}

void ClientServerEncode::heartbeat(uint64_t counter, iter_t clock) {
  for (uint s = 0; s < num_servers_; ++s) {
    if (s == client_id_) continue;
    Message msg(1);
    heartbeat_msg_t h{CMD_HEARTBEAT, client_id_, counter, clock};
    msg[0].pack(h);
    router_->send_to("tablet-" + std::to_string(s), std::move(msg));
  }
}

void ClientServerEncode::barrier(uint epoch) {
  for (uint s = 0; s < num_servers_; ++s) {
    Message msg(1);
    barrier_msg_t h{CMD_BARRIER, client_id_, epoch};
    msg[0].pack(h);
    router_->send_to(server_name(s), std::move(msg));
  }
}

void ClientServerEncode::ipc_exchange(const std::vector<char>& blob, uint32_t round) {
  for (uint s = 0; s < num_servers_; ++s) {
    Message msg(2);
    ipc_exchange_msg_t h{CMD_IPC_EXCHANGE, client_id_, round, 1};
    msg[0].pack(h);
    msg[1].pack_memory(blob.data(), blob.size());
    router_->send_to(server_name(s), std::move(msg));
  }
}

void ClientServerEncode::shutdown_notice() {
  for (uint s = 0; s < num_servers_; ++s) {
    Message msg(1);
    MsgHeader h{CMD_SHUTDOWN};
    msg[0].pack(h);
    router_->send_to(server_name(s), std::move(msg));
  }
}

// ---------------- decoder ----------------
void ServerClientDecode::read_row_batch(Message& msg) {
  sc_read_row_batch_msg_t h;
  if (msg.size() < 3 || !msg[0].unpack(&h)) return;
  if (msg[2].size() != h.num_rows * sizeof(RowData)) return;
  // clock bookkeeping first (may recycle oplog entries), then install the rows
  lib_->server_clock_cbk(h.server_id, h.table_id, h.data_age);
  lib_->recv_row_batch_cbk(h.server_id, h.table_id, h.data_age, h.self_clock,
                           reinterpret_cast<const RowKey*>(msg[1].data()),
                           reinterpret_cast<const RowData*>(msg[2].data()), h.num_rows);
}

void ServerClientDecode::clock(Message& msg) {
  sc_clock_msg_t h;
  if (!msg[0].unpack(&h)) return;
  lib_->server_clock_cbk(h.server_id, h.table_id, h.clock);
}

void ServerClientDecode::get_stats(Message& msg) {
  sc_get_stats_msg_t h;
  if (msg.size() < 2 || !msg[0].unpack(&h)) return;
  lib_->get_stats_cbk(h.server_id, msg[1].unpack_string());
}

void ServerClientDecode::find_row(Message& msg) {
  sc_find_row_msg_t h;
  if (!msg[0].unpack(&h)) return;
  lib_->find_row_cbk(h.table, h.row, h.server_id);
}

void ServerClientDecode::decode_msg(const std::string& src, Message& msg) {
  if (msg.empty()) return;
  switch (msg[0].cmd()) {
    case CMD_READ_ROW_BATCH: read_row_batch(msg); break;
    case CMD_SERVER_CLOCK: clock(msg); break;
    case CMD_GET_STATS: get_stats(msg); break;
    case CMD_FIND_ROW: find_row(msg); break;
    case CMD_PEER_LOST: lib_->peer_lost_cbk(src); break;
    default: break;
  }
}

}  // namespace geeps_b200
