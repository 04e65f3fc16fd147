// Message schema between workers ("clients") and server shards ("tablets") on the TCP path.
// One message = a header frame (one of the POD structs below) followed by payload frames.
// The commands cover the reference's set (src/common/wire-protocol.hpp:42-135) and add the
// control-plane messages the B200 runtime needs (membership, heartbeats, CUDA IPC exchange,
// snapshots, barrier).
#pragma once
#include <stdint.h>

#include "core/common_util.hpp"

namespace geeps_b200 {

enum Command : uint32_t {
  CMD_FIND_ROW = 0,
  CMD_READ_ROW_BATCH = 1,          // server -> client: rows of one shard of one table
  CMD_CLOCK = 2,                   // client -> server: clock of (table) advanced, no updates
  CMD_CLOCK_WITH_UPDATES_BATCH = 3,// client -> server: updates of this shard's rows + clock
  CMD_ADD_ACCESS_INFO = 4,
  CMD_GET_STATS = 5,
  CMD_SHUTDOWN = 6,
  CMD_SERVER_CLOCK = 7,            // server -> client: clock-only notification
  CMD_HELLO = 8,                   // first message on a connection: carries the sender identity
  CMD_IPC_EXCHANGE = 9,            // CUDA IPC handles of a rank's peer-visible buffers
  CMD_HEARTBEAT = 10,
  CMD_BARRIER = 11,
  CMD_SNAPSHOT = 12,
  CMD_PEER_LOST = 13,              // synthesised locally when a connection drops
};

#pragma pack(push, 1)
struct MsgHeader { uint32_t cmd; };
struct cs_find_row_msg_t { uint32_t cmd; uint32_t client_id; uint64_t table; uint64_t row; };
struct sc_find_row_msg_t { uint32_t cmd; uint64_t table; uint64_t row; uint32_t server_id; };
struct cs_clock_msg_t { uint32_t cmd; uint32_t client_id; int32_t clock; uint32_t table_id; };
struct cs_clock_with_updates_batch_msg_t {
  uint32_t cmd; uint32_t client_id; int32_t clock; uint32_t table_id; uint64_t num_rows;
  uint32_t is_init;   // 1: bootstrap values, always applied additively
};
struct cs_add_access_info_msg_t { uint32_t cmd; uint32_t client_id; uint64_t num_entries; };
struct cs_get_stats_msg_t { uint32_t cmd; uint32_t client_id; };
struct sc_clock_msg_t { uint32_t cmd; uint32_t server_id; int32_t clock; uint32_t table_id; };
struct sc_read_row_batch_msg_t {
  uint32_t cmd; uint32_t server_id; uint32_t table_id; int32_t data_age; int32_t self_clock; uint64_t num_rows;
};
struct sc_get_stats_msg_t { uint32_t cmd; uint32_t server_id; };
struct hello_msg_t { uint32_t cmd; uint32_t id; uint32_t is_server; };
struct heartbeat_msg_t { uint32_t cmd; uint32_t id; uint64_t counter; int32_t clock; };
struct barrier_msg_t { uint32_t cmd; uint32_t id; uint32_t epoch; };
struct ipc_exchange_msg_t { uint32_t cmd; uint32_t id; uint32_t table_id; uint32_t num_handles; };
struct access_info_t { uint64_t table; uint64_t row; uint32_t nread; uint32_t nwrite; };
#pragma pack(pop)

}  // namespace geeps_b200
