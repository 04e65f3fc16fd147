#include "router_handler.hpp"

#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <sstream>

#include "wire_protocol.hpp"

namespace geeps_b200 {

namespace { constexpr uint64_t kMaxFrameBytes = 1ull << 34; }   // 16 GiB: above any table shard


namespace {

bool write_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    p += w; n -= (size_t)w;
  }
  return true;
}
bool read_all(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) { if (errno == EINTR) continue; return false; }
    p += r; n -= (size_t)r;
  }
  return true;
}
void tune_socket(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 8 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

}  // namespace

std::string RouterStats::to_json() const {
  std::ostringstream o;
  o << "{\"total_send\":" << total_send.load() << ",\"total_local_send\":" << total_local_send.load()
    << ",\"total_receive\":" << total_receive.load() << ",\"total_local_receive\":" << total_local_receive.load()
    << ",\"msgs_sent\":" << msgs_sent.load() << ",\"msgs_received\":" << msgs_received.load() << "}";
  return o.str();
}

RouterHandler::RouterHandler(const std::string& identity) : identity_(identity) {}

RouterHandler::~RouterHandler() {
  stop_handler_thread();
  stopping_ = true;
  const int lfd = listen_fd_.load();
  if (lfd >= 0) ::shutdown(lfd, SHUT_RDWR);         // wakes the accept thread
  if (accept_thread_.joinable()) accept_thread_.join();
  if (lfd >= 0) { ::close(lfd); listen_fd_ = -1; }
  std::vector<std::shared_ptr<Conn>> cs;
  { std::lock_guard<std::mutex> lk(conns_mu_); cs = all_conns_; }
  for (auto& c : cs) { c->alive = false; if (c->fd >= 0) ::shutdown(c->fd, SHUT_RDWR); }
  for (auto& c : cs) { if (c->reader.joinable()) c->reader.join(); if (c->fd >= 0) ::close(c->fd); c->fd = -1; }
}

bool RouterHandler::bind(const std::string& host, unsigned port, std::string* err) {
  const int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (lfd < 0) { if (err) *err = "socket() failed"; return false; }
  listen_fd_ = lfd;
  int one = 1;
  setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr;
  memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_port = htons((uint16_t)port);
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  if (!host.empty() && host != "*" && inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1)
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
  int rc = -1;
  for (int attempt = 0; attempt < 30 && rc != 0; ++attempt) {   // a port in TIME_WAIT frees up within seconds
    rc = ::bind(lfd, (sockaddr*)&addr, sizeof(addr));
    if (rc != 0) std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  if (rc != 0 || ::listen(lfd, 64) != 0) {
    if (err) *err = "bind/listen on port " + std::to_string(port) + " failed: " + strerror(errno);
    ::close(lfd);
    listen_fd_ = -1;
    return false;
  }
  accept_thread_ = std::thread([this] { accept_loop(); });
  return true;
}

void RouterHandler::accept_loop() {
  const int lfd = listen_fd_.load();
  while (!stopping_) {
    int fd = ::accept(lfd, nullptr, nullptr);
    if (fd < 0) { if (stopping_) return; if (errno == EINTR) continue; return; }
    tune_socket(fd);
    uint32_t len = 0;
    if (!read_all(fd, &len, 4) || len > 256) { ::close(fd); continue; }
    std::string peer(len, 0);
    if (!read_all(fd, &peer[0], len)) { ::close(fd); continue; }
    auto c = std::make_shared<Conn>();
    c->fd = fd;
    c->peer = peer;
    register_conn(c);
  }
}

void RouterHandler::register_conn(std::shared_ptr<Conn> c) {
  {
    std::lock_guard<std::mutex> lk(conns_mu_);
    conns_[c->peer] = c;
    all_conns_.push_back(c);
  }
  c->reader = std::thread([this, c] { reader_loop(c); });
}

bool RouterHandler::connect_to(const std::string& peer_identity, const std::string& host, unsigned port,
                               int timeout_ms, std::string* err) {
  addrinfo hints, *res = nullptr;
  memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  const std::string h = (host == "localhost") ? "127.0.0.1" : host;
  if (getaddrinfo(h.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) {
    if (err) *err = "cannot resolve " + host;
    return false;
  }
  const auto t0 = std::chrono::steady_clock::now();
  int fd = -1;
  for (;;) {
    fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) == 0) break;
    if (fd >= 0) ::close(fd);
    fd = -1;
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (ms > timeout_ms) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
  freeaddrinfo(res);
  if (fd < 0) {
    if (err) *err = "connect to " + host + ":" + std::to_string(port) + " timed out";
    return false;
  }
  tune_socket(fd);
  const uint32_t len = (uint32_t)identity_.size();
  if (!write_all(fd, &len, 4) || !write_all(fd, identity_.data(), len)) {
    ::close(fd);
    if (err) *err = "handshake with " + host + " failed";
    return false;
  }
  auto c = std::make_shared<Conn>();
  c->fd = fd;
  c->peer = peer_identity;
  register_conn(c);
  return true;
}

bool RouterHandler::write_message(Conn* c, const Message& msg) {
  std::lock_guard<std::mutex> lk(c->write_mu);
  if (!c->alive) return false;
  std::vector<uint64_t> head(1 + msg.size());
  head[0] = msg.size();
  for (size_t i = 0; i < msg.size(); ++i) head[1 + i] = msg[i].size();
  if (!write_all(c->fd, head.data(), head.size() * 8)) { c->alive = false; return false; }
  for (const PortableBytes& f : msg)
    if (f.size() && !write_all(c->fd, f.data(), f.size())) { c->alive = false; return false; }
  return true;
}

void RouterHandler::reader_loop(std::shared_ptr<Conn> c) {
  for (;;) {
    uint64_t nframes = 0;
    if (!read_all(c->fd, &nframes, 8) || nframes > 64) break;
    std::vector<uint64_t> lens(nframes);
    if (nframes && !read_all(c->fd, lens.data(), nframes * 8)) break;
    Message msg(nframes);
    bool ok = true;
    // a length no sender of this protocol produces (the largest frame is one table shard) is treated as a
    // corrupt or hostile stream: the peer is dropped instead of the allocation being attempted
    for (size_t i = 0; i < nframes && ok; ++i) ok = lens[i] <= kMaxFrameBytes;
    for (size_t i = 0; i < nframes && ok; ++i) {
      msg[i].resize(lens[i]);
      ok = lens[i] == 0 || read_all(c->fd, msg[i].data(), lens[i]);
    }
    if (!ok) break;
    stats.total_receive += message_bytes(msg);
    enqueue(c->peer, std::move(msg), false);
  }
  c->alive = false;
  if (!stopping_) {
    Message lost(1);
    MsgHeader h{CMD_PEER_LOST};
    lost[0].pack(h);
    enqueue(c->peer, std::move(lost), false);
  }
}

void RouterHandler::enqueue(const std::string& src, Message&& msg, bool local) {
  if (!msg.empty() && drop_left_ > 0 && msg[0].cmd() == drop_cmd_.load()) { --drop_left_; return; }
  if (local) stats.total_local_receive += message_bytes(msg);
  stats.msgs_received++;
  { std::lock_guard<std::mutex> lk(q_mu_); inbound_.emplace_back(src, std::move(msg)); }
  q_cv_.notify_one();
}

bool RouterHandler::send_to(const std::string& dest, Message&& msg) {
  const size_t bytes = message_bytes(msg);
  if (dest == "local") {
    if (!local_peer_) return false;
    stats.total_send += bytes;
    stats.total_local_send += bytes;
    stats.msgs_sent++;
    local_peer_->enqueue("local", std::move(msg), true);
    return true;
  }
  std::shared_ptr<Conn> c;
  {
    std::lock_guard<std::mutex> lk(conns_mu_);
    auto it = conns_.find(dest);
    if (it == conns_.end()) return false;
    c = it->second;
  }
  if (!write_message(c.get(), msg)) return false;
  stats.total_send += bytes;
  stats.msgs_sent++;
  return true;
}

bool RouterHandler::send_to(const std::vector<std::string>& dests, const Message& msg) {
  bool ok = true;
  for (const std::string& d : dests) {
    Message copy = msg;
    ok = send_to(d, std::move(copy)) && ok;
  }
  return ok;
}

bool RouterHandler::has_peer(const std::string& name) {
  if (name == "local") return local_peer_ != nullptr;
  std::lock_guard<std::mutex> lk(conns_mu_);
  auto it = conns_.find(name);
  return it != conns_.end() && it->second->alive;
}

std::vector<std::string> RouterHandler::peers() {
  std::lock_guard<std::mutex> lk(conns_mu_);
  std::vector<std::string> v;
  for (auto& kv : conns_) v.push_back(kv.first);
  return v;
}

void RouterHandler::start_handler_thread(RecvCallback cb) {
  if (handler_running_) return;
  handler_running_ = true;
  handler_thread_ = std::thread([this, cb] {
    for (;;) {
      std::pair<std::string, Message> item;
      {
        std::unique_lock<std::mutex> lk(q_mu_);
        q_cv_.wait(lk, [&] { return !inbound_.empty() || !handler_running_; });
        if (inbound_.empty()) return;
        item = std::move(inbound_.front());
        inbound_.pop_front();
      }
      cb(item.first, item.second);
    }
  });
}

void RouterHandler::stop_handler_thread() {
  {
    std::lock_guard<std::mutex> lk(q_mu_);
    if (!handler_running_) return;
    handler_running_ = false;
  }
  q_cv_.notify_all();
  if (handler_thread_.joinable()) handler_thread_.join();
}

}  // namespace geeps_b200
