// Message router over TCP: every node owns one RouterHandler with an identity
// ("client-<i>" or "tablet-<i>"), optionally listens on a port, connects to peers, and delivers
// inbound messages to a single handler thread.  A co-located peer is reachable under the name
// "local" without touching a socket.
//
// Role of the reference's RouterHandler (src/common/router-handler.cpp:70-291: one ZeroMQ ROUTER
// socket + inproc funnels polled by one thread).  This one is plain POSIX sockets with
// length-prefixed frames, bounded connect retries, and a CMD_PEER_LOST notification instead of a
// silent exit when a connection drops.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "portable_bytes.hpp"

namespace geeps_b200 {

struct RouterStats {
  std::atomic<uint64_t> total_send{0}, total_local_send{0}, total_receive{0}, total_local_receive{0};
  std::atomic<uint64_t> msgs_sent{0}, msgs_received{0};
  std::string to_json() const;
};

class RouterHandler {
 public:
  typedef std::function<void(const std::string& src, Message& msg)> RecvCallback;

  explicit RouterHandler(const std::string& identity);
  ~RouterHandler();

  const std::string& identity() const { return identity_; }
  // Listen on host:port (host "" or "*" = all interfaces).
  bool bind(const std::string& host, unsigned port, std::string* err);
  // Connect to a listening peer and register the connection under `peer_identity`.
  bool connect_to(const std::string& peer_identity, const std::string& host, unsigned port, int timeout_ms,
                  std::string* err);
  // Pair two routers of one process; each then reaches the other as "local".
  void set_local_peer(RouterHandler* peer) { local_peer_ = peer; }

  // Thread-safe.  Returns false if the destination is unknown or the connection is gone.
  bool send_to(const std::string& dest, Message&& msg);
  bool send_to(const std::vector<std::string>& dests, const Message& msg);
  bool has_peer(const std::string& name);
  std::vector<std::string> peers();

  void start_handler_thread(RecvCallback cb);
  void stop_handler_thread();
  // test hook: drop (do not deliver) the next `n` inbound messages whose command equals `cmd`
  void drop_inbound(uint32_t cmd, int n) { drop_cmd_ = cmd; drop_left_ = n; }

  RouterStats stats;

 private:
  struct Conn {
    int fd = -1;
    std::string peer;
    std::mutex write_mu;
    std::thread reader;
    std::atomic<bool> alive{true};
  };
  void accept_loop();
  void reader_loop(std::shared_ptr<Conn> c);
  void enqueue(const std::string& src, Message&& msg, bool local);
  void register_conn(std::shared_ptr<Conn> c);
  bool write_message(Conn* c, const Message& msg);

  std::string identity_;
  std::atomic<int> listen_fd_{-1};   // read by the accept thread, closed by the destructor
  std::thread accept_thread_;
  std::atomic<bool> stopping_{false};
  RouterHandler* local_peer_ = nullptr;

  std::mutex conns_mu_;
  std::map<std::string, std::shared_ptr<Conn>> conns_;
  std::vector<std::shared_ptr<Conn>> all_conns_;

  std::mutex q_mu_;
  std::condition_variable q_cv_;
  std::deque<std::pair<std::string, Message>> inbound_;
  std::thread handler_thread_;
  bool handler_running_ = false;
  std::atomic<uint32_t> drop_cmd_{0xffffffffu};
  std::atomic<int> drop_left_{0};
};

}  // namespace geeps_b200
