#include "server_entry.hpp"

namespace geeps_b200 {

ServerThreadEntry::ServerThreadEntry(uint channel_id, uint num_channels, uint process_id, uint num_processes,
                                     const GeePsConfig& config)
    : channel_id_(channel_id), num_channels_(num_channels), process_id_(process_id),
      num_processes_(num_processes), config_(config) {}

ServerThreadEntry::~ServerThreadEntry() { stop(); }

unsigned ServerThreadEntry::port_for(const GeePsConfig& config, uint process_id, uint channel_id) {
  // port_list gives every process its own base port, so several processes can share one host
  const unsigned base = process_id < config.port_list.size() ? config.port_list[process_id] : config.tcp_base_port;
  return base + channel_id;
}

bool ServerThreadEntry::start(std::string* err) {
  router_.reset(new RouterHandler("tablet-" + std::to_string(process_id_)));
  if (!router_->bind("*", port_for(config_, process_id_, channel_id_), err)) return false;
  encoder_.reset(new ServerClientEncode(router_, num_processes_, process_id_, config_));
  storage_.reset(new TabletStorage(channel_id_, num_channels_, process_id_, num_processes_, encoder_, config_));
  if (hyper_schedule) storage_->hyper = hyper_schedule;
  metadata_.reset(new MetadataServer(process_id_, num_processes_, encoder_, config_));
  decoder_.reset(new ClientServerDecode(storage_, metadata_));
  decoder_->control_hook = control_hook;
  std::shared_ptr<ClientServerDecode> dec = decoder_;
  router_->start_handler_thread([dec](const std::string& src, Message& msg) { dec->router_callback(src, msg); });
  return true;
}

void ServerThreadEntry::stop() {
  if (router_) router_->stop_handler_thread();
}

}  // namespace geeps_b200
