// Server side of the message codec: decode worker -> shard commands, encode replies
// (role of the reference's src/server/server-encoder-decoder.cpp:69-266).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "geeps.hpp"
#include "net/router_handler.hpp"
#include "net/wire_protocol.hpp"

namespace geeps_b200 {

class TabletStorage;
class MetadataServer;

class ServerClientEncode {
 public:
  ServerClientEncode(std::shared_ptr<RouterHandler> router, uint num_clients, uint server_id,
                     const GeePsConfig& config);
  void clock(uint table_id, iter_t clock);                       // clock-only broadcast to every client
  void find_row(uint client_id, uint64_t table, uint64_t row, uint server_id);
  // header + keys + rows of one table shard to one client
  void read_row_batch_reply(uint client_id, uint table_id, iter_t data_age, iter_t self_clock,
                            const RowKey* keys, const RowData* rows, size_t num_rows);
  void get_stats(uint client_id, const std::string& stats);
  std::string client_name(uint client_id) const;
 private:
  std::shared_ptr<RouterHandler> router_;
  uint num_clients_, server_id_;
  GeePsConfig config_;
};

class ClientServerDecode {
 public:
  ClientServerDecode(std::shared_ptr<TabletStorage> storage, std::shared_ptr<MetadataServer> metadata);
  void find_row(const std::string& src, Message& msg);
  void clock(const std::string& src, Message& msg);
  void clock_with_updates_batch(const std::string& src, Message& msg);
  void add_access_info(const std::string& src, Message& msg);
  void get_stats(const std::string& src, Message& msg);
  void decode_msg(const std::string& src, Message& msg);
  void router_callback(const std::string& src, Message& msg) { decode_msg(src, msg); }
  // membership / control messages (heartbeat, barrier, CUDA IPC exchange, peer loss) go to the
  // co-located worker runtime through this hook
  std::function<void(const std::string&, Message&)> control_hook;
  uint64_t unknown_commands = 0;
 private:
  std::shared_ptr<TabletStorage> storage_;
  std::shared_ptr<MetadataServer> metadata_;
};

}  // namespace geeps_b200
