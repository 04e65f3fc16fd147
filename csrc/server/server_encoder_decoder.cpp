#include "server_encoder_decoder.hpp"

#include "metadata_server.hpp"
#include "tablet_server.hpp"

namespace geeps_b200 {

ServerClientEncode::ServerClientEncode(std::shared_ptr<RouterHandler> router, uint num_clients, uint server_id,
                                       const GeePsConfig& config)
    : router_(router), num_clients_(num_clients), server_id_(server_id), config_(config) {}

std::string ServerClientEncode::client_name(uint client_id) const {
  if (config_.local_opt && client_id == server_id_) return "local";
  return "client-" + std::to_string(client_id);
}

void ServerClientEncode::clock(uint table_id, iter_t clock) {
  for (uint c = 0; c < num_clients_; ++c) {
    Message msg(1);
    sc_clock_msg_t h{CMD_SERVER_CLOCK, server_id_, clock, table_id};
    msg[0].pack(h);
    router_->send_to(client_name(c), std::move(msg));
  }
}

void ServerClientEncode::find_row(uint client_id, uint64_t table, uint64_t row, uint server_id) {
  Message msg(1);
  sc_find_row_msg_t h{CMD_FIND_ROW, table, row, server_id};
  msg[0].pack(h);
  router_->send_to(client_name(client_id), std::move(msg));
}

void ServerClientEncode::read_row_batch_reply(uint client_id, uint table_id, iter_t data_age, iter_t self_clock,
                                              const RowKey* keys, const RowData* rows, size_t num_rows) {
  Message msg(3);
  sc_read_row_batch_msg_t h{CMD_READ_ROW_BATCH, server_id_, table_id, data_age, self_clock, (uint64_t)num_rows};
  msg[0].pack(h);
  msg[1].pack_memory(keys, num_rows * sizeof(RowKey));
  msg[2].pack_memory(rows, num_rows * sizeof(RowData));
  router_->send_to(client_name(client_id), std::move(msg));
}

void ServerClientEncode::get_stats(uint client_id, const std::string& stats) {
  Message msg(2);
  sc_get_stats_msg_t h{CMD_GET_STATS, server_id_};
  msg[0].pack(h);
  msg[1].pack_string(stats);
  router_->send_to(client_name(client_id), std::move(msg));
}

ClientServerDecode::ClientServerDecode(std::shared_ptr<TabletStorage> storage, std::shared_ptr<MetadataServer> metadata)
    : storage_(storage), metadata_(metadata) {}

void ClientServerDecode::find_row(const std::string&, Message& msg) {
  cs_find_row_msg_t h;
  if (!msg[0].unpack(&h)) return;
  metadata_->find_row(h.client_id, h.table, h.row);
}

void ClientServerDecode::clock(const std::string&, Message& msg) {
  cs_clock_msg_t h;
  if (!msg[0].unpack(&h)) return;
  storage_->clock(h.client_id, h.clock, h.table_id);
}

void ClientServerDecode::clock_with_updates_batch(const std::string&, Message& msg) {
  cs_clock_with_updates_batch_msg_t h;
  if (msg.size() < 3 || !msg[0].unpack(&h)) return;
  if (msg[2].size() != h.num_rows * sizeof(RowOpVal)) { unknown_commands++; return; }
  const RowKey* keys = msg[1].size() == h.num_rows * sizeof(RowKey) ? reinterpret_cast<const RowKey*>(msg[1].data()) : nullptr;
  // apply first, then advance the clock (the broadcast that may follow must contain this update)
  if (storage_->update_row_batch(h.client_id, h.clock, h.table_id, keys,
                                 reinterpret_cast<const RowOpVal*>(msg[2].data()), h.num_rows, h.is_init != 0))
    storage_->clock(h.client_id, h.clock, h.table_id);
}

void ClientServerDecode::add_access_info(const std::string&, Message& msg) {
  cs_add_access_info_msg_t h;
  if (msg.size() < 2 || !msg[0].unpack(&h)) return;
  std::vector<access_info_t> infos;
  msg[1].unpack_vector(&infos);
  metadata_->add_access_info(h.client_id, infos);
}

void ClientServerDecode::get_stats(const std::string&, Message& msg) {
  cs_get_stats_msg_t h;
  if (!msg[0].unpack(&h)) return;
  // reply goes through the storage's communicator via the metadata server's encoder
  metadata_->decide_data_assignment();
  std::string s = "{\"storage\":" + storage_->get_stats() + ",\"metadata\":" + metadata_->get_stats() + "}";
  metadata_->reply_stats(h.client_id, s);
}

void ClientServerDecode::decode_msg(const std::string& src, Message& msg) {
  if (msg.empty()) return;
  switch (msg[0].cmd()) {
    case CMD_FIND_ROW: find_row(src, msg); break;
    case CMD_CLOCK: clock(src, msg); break;
    case CMD_CLOCK_WITH_UPDATES_BATCH: clock_with_updates_batch(src, msg); break;
    case CMD_ADD_ACCESS_INFO: add_access_info(src, msg); break;
    case CMD_GET_STATS: get_stats(src, msg); break;
    case CMD_PEER_LOST:
    case CMD_SHUTDOWN:
    case CMD_HEARTBEAT:
    case CMD_BARRIER:
    case CMD_IPC_EXCHANGE:
      if (control_hook) control_hook(src, msg);
      break;
    default: unknown_commands++;
  }
}

}  // namespace geeps_b200
