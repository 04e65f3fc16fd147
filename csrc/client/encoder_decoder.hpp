// Worker side of the message codec: encode worker -> shard commands, decode replies and hand
// them to the ClientLib callbacks (role of the reference's src/client/encoder-decoder.cpp:48-333).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "geeps.hpp"
#include "net/router_handler.hpp"
#include "net/wire_protocol.hpp"

namespace geeps_b200 {

class ClientLib;

class ClientServerEncode {
 public:
  ClientServerEncode(std::shared_ptr<RouterHandler> router, uint num_servers, uint client_id,
                     const GeePsConfig& config);
  std::string server_name(uint server_id) const;
  std::vector<std::string> all_servers() const;
  void find_row(uint64_t table, uint64_t row, uint metadata_server_id);
  void clock_broadcast(iter_t clock, uint table_id);
  void clock_to(uint server_id, iter_t clock, uint table_id);
  // one source: `rows` holds the shard's updates in shard order
  bool clock_with_updates_batch(uint server_id, iter_t clock, uint table_id, const RowKey* keys,
                                const RowOpVal* rows, size_t num_rows, bool is_init);
  // two sources: host-cached part followed by the device-cached part (already copied to the host)
  bool clock_with_updates_batch(uint server_id, iter_t clock, uint table_id, const RowKey* keys,
                                const RowOpVal* rows0, size_t n0, const RowOpVal* rows1, size_t n1, bool is_init);
  void add_access_info(uint metadata_server_id, const std::vector<access_info_t>& infos);
  void get_stats(uint server_id);
  void heartbeat(uint64_t counter, iter_t clock);
  void barrier(uint epoch);
  // `round` distinguishes successive exchanges (a fast rank may start the next one before a slow rank has read
  // the previous one): the receiver keeps one blob per (rank, round)
  void ipc_exchange(const std::vector<char>& blob, uint32_t round = 0);
  void shutdown_notice();
 private:
  std::shared_ptr<RouterHandler> router_;
  uint num_servers_, client_id_;
  GeePsConfig config_;
};

class ServerClientDecode {
 public:
  explicit ServerClientDecode(ClientLib* lib) : lib_(lib) {}
  void read_row_batch(Message& msg);
  void clock(Message& msg);
  void get_stats(Message& msg);
  void find_row(Message& msg);
  void decode_msg(const std::string& src, Message& msg);
  void router_callback(const std::string& src, Message& msg) { decode_msg(src, msg); }
 private:
  ClientLib* lib_;
};

// Control-plane messages that arrive on a process's *server* router (heartbeats, barriers, CUDA IPC
// handles) are forwarded to the co-located ClientLib through this hook.
typedef void (*ControlHook)(void* lib, const std::string& src, Message& msg);

}  // namespace geeps_b200
