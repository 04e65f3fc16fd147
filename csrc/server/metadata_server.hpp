// Row -> server placement service with three policies: 1 hash (row mod servers), 2 first
// toucher, 3 most frequent accessor with load balancing.  The reference carries this component
// as dead code (its find_row begins with CHECK(0): src/server/metadata-server.cpp:119-170); here
// it is live and answers FIND_ROW requests, while the data path uses the static partitioner.
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "geeps.hpp"
#include "net/wire_protocol.hpp"

namespace geeps_b200 {

class ServerClientEncode;

class MetadataServer {
 public:
  MetadataServer(uint server_id, uint num_servers, std::shared_ptr<ServerClientEncode> communicator,
                 const GeePsConfig& config);
  void add_access_info(uint client_id, const std::vector<access_info_t>& infos);
  void find_row(uint client_id, uint64_t table, uint64_t row);
  // decide the placement of every row seen so far (policy 3) and answer queued requests
  void decide_data_assignment();
  uint owner_of(uint64_t table, uint64_t row) const;
  std::string get_stats() const;
  void reply_stats(uint client_id, const std::string& stats);
 private:
  struct RowInfo { std::vector<uint32_t> access; int owner = -1; };
  void serve_pending_requests();
  uint server_id_, num_servers_;
  std::shared_ptr<ServerClientEncode> communicator_;
  int policy_;
  std::map<std::pair<uint64_t, uint64_t>, RowInfo> rows_;
  struct Pending { uint client; uint64_t table, row; };
  std::vector<Pending> pending_;
  std::vector<uint64_t> load_;
  bool decided_ = false;
  uint64_t nr_requests_ = 0;
};

}  // namespace geeps_b200
