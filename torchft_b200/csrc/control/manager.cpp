#include "manager.h"

#include <algorithm>
#include <cstdlib>

#include "log.h"

namespace ftcp {

namespace {
// "<id>:<uuid>" -> "<id>" for log prefixes
std::string short_id(const std::string& replica_id) {
  const size_t p = replica_id.find(':');
  return p == std::string::npos ? replica_id : replica_id.substr(0, p);
}
}  // namespace

ManagerServer::ManagerServer(std::string replica_id, std::string lighthouse_addr, std::string hostname,
                             const std::string& bind, std::string store_addr, uint64_t world_size,
                             Millis heartbeat_interval, Millis connect_timeout, int64_t quorum_retries)
    : replica_id_(std::move(replica_id)),
      lighthouse_addr_(std::move(lighthouse_addr)),
      hostname_(std::move(hostname)),
      store_addr_(std::move(store_addr)),
      world_size_(world_size),
      heartbeat_interval_(heartbeat_interval),
      connect_timeout_(connect_timeout),
      quorum_retries_(quorum_retries) {
  // fail early (TimeoutError) when the lighthouse is unreachable
  { Client probe(lighthouse_addr_, connect_timeout_); }
  server_ = std::make_unique<Server>(bind, [this](uint8_t m, const std::string& b, TimePoint d) { return rpc(m, b, d); });
  server_->set_thread_tag("ftb-manager");
  server_->start();
  heartbeat_thread_ = std::thread([this] { heartbeat_loop(); });
  log_info("manager", "[Replica " + short_id(replica_id_) + "] Manager listening on " + address());
}

ManagerServer::~ManagerServer() { shutdown(); }

std::string ManagerServer::address() const { return "http://" + hostname_ + ":" + std::to_string(server_->port()); }

void ManagerServer::shutdown() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (stop_) return;
    stop_ = true;
  }
  cv_.notify_all();
  if (heartbeat_thread_.joinable()) heartbeat_thread_.join();
  server_->shutdown();
  std::vector<std::thread> threads;
  {
    std::lock_guard<std::mutex> g(mu_);
    threads.swap(round_threads_);
  }
  for (auto& t : threads)
    if (t.joinable()) t.join();
}

void ManagerServer::heartbeat_loop() {
  set_thread_name("ftb-manager-hb");
  std::unique_ptr<Client> client;
  std::unique_lock<std::mutex> lk(mu_);
  while (!stop_) {
    lk.unlock();
    try {
      if (!client) client = std::make_unique<Client>(lighthouse_addr_, connect_timeout_);
      client->call(kLighthouseHeartbeat, encode_str1(replica_id_), std::max(Millis(1000), heartbeat_interval_ * 10));
    } catch (const std::exception& e) {
      log_info("manager", "[Replica " + short_id(replica_id_) + "] Failed to send heartbeat to lighthouse: " + e.what());
      client.reset();
    }
    lk.lock();
    cv_.wait_for(lk, heartbeat_interval_, [this] { return stop_; });
  }
}

void ManagerServer::run_lighthouse_round(uint64_t round, QuorumMember requester, Millis timeout) {
  log_info("manager", "[Replica " + short_id(replica_id_) + "] All workers joined - starting quorum");
  const std::string body = encode_msg1(requester.encode());
  std::optional<Quorum> result;
  std::string error;
  bool timed_out = false;
  for (int64_t attempt = 0;; ++attempt) {
    Millis sleep_ms(100);
    try {
      Client c(lighthouse_addr_, std::min(connect_timeout_, timeout));
      const std::string resp = c.call(kLighthouseQuorum, body, timeout);
      Reader r(resp);
      int f, wt;
      while (r.next(&f, &wt)) {
        if (f == 1 && wt == 2) result = Quorum::decode(r.bytes());
        else r.skip(wt);
      }
      if (!result) throw RpcError("missing quorum");
      break;
    } catch (const TimeoutError& e) {
      error = e.what();
      timed_out = true;
      log_info("manager", "[Replica " + short_id(replica_id_) + "] lighthouse quorum timeout. error: " + error);
    } catch (const std::exception& e) {
      error = e.what();
      timed_out = false;
      log_info("manager", "[Replica " + short_id(replica_id_) + "] lighthouse quorum failed. error: " + error);
      sleep_ms = std::max(Millis(100), Millis(timeout.count() / std::max<int64_t>(quorum_retries_ + 1, 1)));
    }
    if (attempt >= quorum_retries_) {
      error = "lighthouse quorum failed after " + std::to_string(attempt) + " retries: " + error;
      break;
    }
    std::unique_lock<std::mutex> lk(mu_);
    if (cv_.wait_for(lk, sleep_ms, [this] { return stop_; })) {
      error = "manager shutting down";
      break;
    }
  }
  std::lock_guard<std::mutex> g(mu_);
  round_quorum_ = result;
  round_error_ = result ? std::string() : error;
  round_timeout_ = !result && timed_out;
  done_round_ = round;
  cv_.notify_all();
}

ManagerQuorumResponse ManagerServer::handle_quorum(const ManagerQuorumRequest& req, TimePoint deadline) {
  std::unique_lock<std::mutex> lk(mu_);
  log_info("manager", "[Replica " + short_id(replica_id_) + "] Start quorum for group_rank " + std::to_string(req.group_rank));
  checkpoint_metadata_[req.group_rank] = req.checkpoint_metadata;
  joined_.insert(req.group_rank);
  const uint64_t my_round = round_ + 1;  // the round being collected
  if (joined_.size() == world_size_) {
    joined_.clear();
    round_ = my_round;
    QuorumMember me;
    me.replica_id = replica_id_;
    me.address = address();
    me.store_address = store_addr_;
    me.step = req.step;
    me.world_size = world_size_;
    me.shrink_only = req.shrink_only;
    me.commit_failures = req.commit_failures;
    const Millis timeout = std::max(Millis(1), std::chrono::duration_cast<Millis>(deadline - Clock::now()));
    // finished round threads are reaped lazily
    if (round_threads_.size() > 8) {
      std::vector<std::thread> old;
      old.swap(round_threads_);
      lk.unlock();
      for (auto& t : old)
        if (t.joinable()) t.join();
      lk.lock();
    }
    round_threads_.emplace_back([this, my_round, me, timeout] { run_lighthouse_round(my_round, me, timeout); });
  }
  while (done_round_ < my_round && !stop_) {
    if (cv_.wait_until(lk, deadline) == std::cv_status::timeout && done_round_ < my_round) {
      joined_.erase(req.group_rank);
      throw TimeoutError("manager quorum deadline exceeded for group_rank " + std::to_string(req.group_rank));
    }
  }
  if (stop_ && done_round_ < my_round) throw RpcError("manager shutting down");
  if (done_round_ != my_round || !round_quorum_) {
    const std::string err = round_error_.empty() ? std::string("quorum round superseded") : round_error_;
    if (round_timeout_) throw TimeoutError(err);
    throw RpcError(err);
  }
  const Quorum q = *round_quorum_;
  lk.unlock();
  log_info("manager", "[Replica " + short_id(replica_id_) + "] Finished quorum for group_rank " + std::to_string(req.group_rank));
  return compute_quorum_results(replica_id_, req.group_rank, q, req.init_sync);
}

bool ManagerServer::handle_should_commit(const ShouldCommitRequest& req, TimePoint deadline) {
  std::unique_lock<std::mutex> lk(mu_);
  // Votes of one round must be about one step.  The reference merges whatever arrives
  // (src/manager.rs:440-478 never looks at `step`); ranks that drifted apart would then commit
  // different steps together.  Here a vote for another step than the round's first vote counts
  // as a failure, so the whole group declines and retries.
  if (commit_votes_.empty()) {
    commit_step_ = req.step;
  } else if (req.step != commit_step_) {
    log_warn("manager", "[Replica " + short_id(replica_id_) + "] should_commit: group_rank " + std::to_string(req.group_rank) +
                            " votes for step " + std::to_string(req.step) + " while the round is about step " +
                            std::to_string(commit_step_) + "; declining the commit");
    commit_failures_.insert(req.group_rank);
  }
  if (!req.should_commit) commit_failures_.insert(req.group_rank);
  commit_votes_.insert(req.group_rank);
  const uint64_t my_round = commit_round_ + 1;
  if (commit_votes_.size() == world_size_) {
    commit_decision_ = commit_failures_.empty();
    log_info("manager", "[Replica " + short_id(replica_id_) + "] should_commit completed should_commit=" +
                            (commit_decision_ ? "true" : "false"));
    commit_votes_.clear();
    commit_failures_.clear();
    commit_round_ = my_round;
    commit_done_round_ = my_round;
    cv_.notify_all();
    return commit_decision_;
  }
  while (commit_done_round_ < my_round && !stop_) {
    if (cv_.wait_until(lk, deadline) == std::cv_status::timeout && commit_done_round_ < my_round) {
      commit_votes_.erase(req.group_rank);
      commit_failures_.erase(req.group_rank);
      throw TimeoutError("should_commit deadline exceeded for group_rank " + std::to_string(req.group_rank));
    }
  }
  if (commit_done_round_ < my_round) throw RpcError("manager shutting down");
  return commit_decision_;
}

std::string ManagerServer::rpc(uint8_t method, const std::string& body, TimePoint deadline) {
  switch (method) {
    case kManagerQuorum:
      return handle_quorum(ManagerQuorumRequest::decode(body), deadline).encode();
    case kManagerCheckpointMetadata: {
      const int64_t rank = decode_i64_1(body);
      std::lock_guard<std::mutex> g(mu_);
      auto it = checkpoint_metadata_.find(rank);
      if (it == checkpoint_metadata_.end()) throw RpcError("rank not found");
      return encode_str1(it->second);
    }
    case kManagerShouldCommit: {
      const bool d = handle_should_commit(ShouldCommitRequest::decode(body), deadline);
      Writer w;
      w.boolean(1, d);
      return w.take();
    }
    case kManagerKill:
      log_warn("manager", "got kill request: " + decode_str1(body));
      std::_Exit(1);
    default:
      throw RpcError("manager: unknown method " + std::to_string(method));
  }
}

}  // namespace ftcp
