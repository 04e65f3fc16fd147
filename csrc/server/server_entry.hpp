// Brings up one server shard of a process: router bound to the shard's TCP port, codec,
// tablet storage, metadata server (role of the reference's src/server/server-entry.cpp:51-88).
#pragma once
#include <functional>
#include <memory>
#include <string>

#include "geeps.hpp"
#include "metadata_server.hpp"
#include "net/router_handler.hpp"
#include "server_encoder_decoder.hpp"
#include "tablet_server.hpp"

namespace geeps_b200 {

class ServerThreadEntry {
 public:
  ServerThreadEntry(uint channel_id, uint num_channels, uint process_id, uint num_processes,
                    const GeePsConfig& config);
  ~ServerThreadEntry();
  // Binds, builds the components and starts the handler thread.  false + err on failure.
  bool start(std::string* err);
  void stop();
  // Handler for the control-plane messages that reach this shard (heartbeats, barriers, handle exchange, lost
  // peers).  Set it before start(): a peer may deliver such a message the moment the port is bound.
  std::function<void(const std::string&, Message&)> control_hook;
  // Optimizer hyper-parameters by clock, shared with the worker side of the process (set before start()).
  std::shared_ptr<HyperSchedule> hyper_schedule;
  static unsigned port_for(const GeePsConfig& config, uint process_id, uint channel_id);
  std::shared_ptr<RouterHandler> router() { return router_; }
  std::shared_ptr<TabletStorage> storage() { return storage_; }
  std::shared_ptr<MetadataServer> metadata() { return metadata_; }
  std::shared_ptr<ClientServerDecode> decoder() { return decoder_; }
 private:
  uint channel_id_, num_channels_, process_id_, num_processes_;
  GeePsConfig config_;
  std::shared_ptr<RouterHandler> router_;
  std::shared_ptr<ServerClientEncode> encoder_;
  std::shared_ptr<TabletStorage> storage_;
  std::shared_ptr<MetadataServer> metadata_;
  std::shared_ptr<ClientServerDecode> decoder_;
};

}  // namespace geeps_b200
