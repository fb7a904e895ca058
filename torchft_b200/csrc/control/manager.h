// Manager server: one per replica group (hosted by the group's rank 0).  Collects the
// quorum requests of the group's `world_size` ranks into a single lighthouse request,
// hands every rank its own view of the result (ranks, store, recovery assignments),
// runs the should_commit vote as a barrier, keeps per-rank checkpoint metadata, sends
// heartbeats to the lighthouse, and exits the process on `Kill`.
// Behavioural counterpart of src/manager.rs:68-486 in the reference, with two holes
// closed: a failed lighthouse round is reported to every waiting rank instead of
// leaving them to time out, and a round's result is tagged so late callers of an old
// round cannot consume a newer result.
#pragma once

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <thread>

#include "net.h"
#include "quorum.h"

namespace ftcp {

class ManagerServer {
 public:
  ManagerServer(std::string replica_id, std::string lighthouse_addr, std::string hostname, const std::string& bind,
                std::string store_addr, uint64_t world_size, Millis heartbeat_interval, Millis connect_timeout,
                int64_t quorum_retries);
  ~ManagerServer();
  std::string address() const;
  void shutdown();

 private:
  std::string rpc(uint8_t method, const std::string& body, TimePoint deadline);
  ManagerQuorumResponse handle_quorum(const ManagerQuorumRequest& req, TimePoint deadline);
  bool handle_should_commit(const ShouldCommitRequest& req, TimePoint deadline);
  void heartbeat_loop();
  void run_lighthouse_round(uint64_t round, QuorumMember requester, Millis timeout);

  const std::string replica_id_, lighthouse_addr_, hostname_, store_addr_;
  const uint64_t world_size_;
  const Millis heartbeat_interval_, connect_timeout_;
  const int64_t quorum_retries_;

  std::mutex mu_;
  std::condition_variable cv_;
  bool stop_ = false;
  std::map<int64_t, std::string> checkpoint_metadata_;
  // quorum rounds
  std::set<int64_t> joined_;
  uint64_t round_ = 0;       // round currently collecting ranks
  uint64_t done_round_ = 0;  // last round with a result
  std::optional<Quorum> round_quorum_;
  std::string round_error_;
  bool round_timeout_ = false;
  // should_commit rounds
  std::set<int64_t> commit_votes_, commit_failures_;
  uint64_t commit_round_ = 0, commit_done_round_ = 0;
  bool commit_decision_ = false;
  int64_t commit_step_ = 0;  // step the current should_commit round is about (set by its first vote)

  std::unique_ptr<Server> server_;
  std::thread heartbeat_thread_;
  std::vector<std::thread> round_threads_;
};

}  // namespace ftcp
