// Lighthouse: the global quorum service.  Tracks heartbeats and pending participants,
// recomputes the quorum on a periodic tick and on every join, and wakes all blocked
// `Quorum` calls when a quorum forms.  Also serves a small HTML dashboard
// (`/`, `/status`, `POST /replica/<id>/kill`) on the same port.
// Behavioural counterpart of src/lighthouse.rs:57-566 in the reference.
#pragma once

#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>

#include "net.h"
#include "quorum.h"

namespace ftcp {

class Lighthouse {
 public:
  explicit Lighthouse(LighthouseOpt opt);
  ~Lighthouse();
  std::string address() const;  // "http://<hostname>:<port>"
  int port() const { return server_->port(); }
  void shutdown();

  // exposed for tests
  Quorum handle_quorum(const QuorumMember& requester, TimePoint deadline);
  void handle_heartbeat(const std::string& replica_id);

 private:
  std::string rpc(uint8_t method, const std::string& body, TimePoint deadline);
  HttpResponse http(const HttpRequest& req);
  void tick_locked();
  void tick_loop();
  std::string render_status();
  std::string render_metrics();  // Prometheus text exposition, served at /metrics
  void prune_heartbeats_locked(TimePoint now);

  LighthouseOpt opt_;
  std::mutex mu_;
  std::condition_variable cv_;
  LighthouseState state_;
  std::deque<std::pair<uint64_t, Quorum>> history_;  // recently issued quorums (seq, quorum)
  uint64_t seq_ = 0;
  uint64_t quorum_requests_ = 0;  // counters for /metrics
  uint64_t heartbeats_received_ = 0;
  uint64_t ticks_ = 0;
  std::string last_reason_;
  bool stop_ = false;
  std::unique_ptr<Server> server_;
  std::thread tick_thread_;
};

}  // namespace ftcp
