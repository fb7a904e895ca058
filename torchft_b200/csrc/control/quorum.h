// Pure quorum mathematics of the control plane (no I/O, no clocks of its own):
//  * quorum_compute          -- lighthouse membership decision (src/lighthouse.rs:141-269)
//  * quorum_changed          -- did the set of replica ids change (src/lighthouse.rs:133-138)
//  * compute_quorum_results  -- per-rank view of a quorum: ranks, primary store, recovery
//                               assignments (src/manager.rs:489-624)
#pragma once

#include <map>
#include <optional>
#include <string>
#include <vector>

#include "net.h"
#include "wire.h"

namespace ftcp {

struct LighthouseOpt {
  std::string bind = "[::]:29510";
  int64_t join_timeout_ms = 60000;
  uint64_t min_replicas = 1;
  int64_t quorum_tick_ms = 100;
  int64_t heartbeat_timeout_ms = 5000;
};

struct ParticipantDetails {
  TimePoint joined;
  QuorumMember member;
};

struct LighthouseState {
  std::map<std::string, ParticipantDetails> participants;
  std::optional<Quorum> prev_quorum;
  int64_t quorum_id = 0;
  std::map<std::string, TimePoint> heartbeats;
};

bool quorum_changed(const std::vector<QuorumMember>& a, const std::vector<QuorumMember>& b);

// Returns the members of the new quorum (sorted by replica id) or nullopt, plus a
// human-readable explanation of the decision.
std::pair<std::optional<std::vector<QuorumMember>>, std::string> quorum_compute(TimePoint now,
                                                                                const LighthouseState& state,
                                                                                const LighthouseOpt& opt);

// Throws RpcError when `replica_id` is not a member of `quorum`.
ManagerQuorumResponse compute_quorum_results(const std::string& replica_id, int64_t group_rank, const Quorum& quorum,
                                             bool init_sync);

}  // namespace ftcp
