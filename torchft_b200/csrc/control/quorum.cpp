#include "quorum.h"

#include <algorithm>
#include <set>
#include <sstream>

namespace ftcp {

bool quorum_changed(const std::vector<QuorumMember>& a, const std::vector<QuorumMember>& b) {
  if (a.size() != b.size()) return true;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].replica_id != b[i].replica_id) return true;
  return false;
}

std::pair<std::optional<std::vector<QuorumMember>>, std::string> quorum_compute(TimePoint now,
                                                                                const LighthouseState& state,
                                                                                const LighthouseOpt& opt) {
  // A replica is healthy while its last heartbeat is younger than the expiry.
  std::set<std::string> healthy;
  for (const auto& [id, last] : state.heartbeats)
    if (now - last < Millis(opt.heartbeat_timeout_ms)) healthy.insert(id);

  // std::map iteration gives the replica-id ordering the protocol requires.
  std::vector<const ParticipantDetails*> joined;
  for (const auto& [id, det] : state.participants)
    if (healthy.count(id)) joined.push_back(&det);

  std::vector<QuorumMember> candidates;
  bool shrink_only = false;
  for (const auto* d : joined) {
    candidates.push_back(d->member);
    shrink_only = shrink_only || d->member.shrink_only;
  }

  std::ostringstream meta;
  meta << "[" << joined.size() << "/" << state.participants.size() << " participants healthy][" << healthy.size()
       << " heartbeating][shrink_only=" << (shrink_only ? "true" : "false") << "]";

  if (state.prev_quorum) {
    std::set<std::string> prev_ids;
    for (const auto& p : state.prev_quorum->participants) prev_ids.insert(p.replica_id);
    if (shrink_only) {
      candidates.erase(std::remove_if(candidates.begin(), candidates.end(),
                                      [&](const QuorumMember& m) { return !prev_ids.count(m.replica_id); }),
                       candidates.end());
    }
    // Fast path: everybody of the previous quorum is back (new joiners ride along).
    bool all_back = true;
    for (const auto& id : prev_ids) {
      auto it = state.participants.find(id);
      if (it == state.participants.end() || !healthy.count(id)) {
        all_back = false;
        break;
      }
    }
    if (all_back) return {candidates, "Fast quorum found! " + meta.str()};
  }

  if (joined.size() < opt.min_replicas) {
    std::ostringstream s;
    s << "New quorum not ready, only have " << joined.size() << " participants, need min_replicas " << opt.min_replicas
      << " " << meta.str();
    return {std::nullopt, s.str()};
  }

  // Split-brain guard: strictly more than half of everything that is heartbeating.
  if (joined.size() <= healthy.size() / 2) {
    std::ostringstream s;
    s << "New quorum not ready, only have " << joined.size() << " participants, need at least half of "
      << healthy.size() << " healthy workers " << meta.str();
    return {std::nullopt, s.str()};
  }

  const bool everyone_joined = joined.size() == healthy.size();
  TimePoint first = now;
  for (const auto* d : joined) first = std::min(first, d->joined);
  if (!everyone_joined && now - first < Millis(opt.join_timeout_ms)) {
    std::ostringstream s;
    s << "Valid quorum with " << joined.size() << " participants, waiting for " << (healthy.size() - joined.size())
      << " healthy but not participating stragglers due to join timeout " << meta.str();
    return {std::nullopt, s.str()};
  }
  return {candidates, "Valid quorum found " + meta.str()};
}

ManagerQuorumResponse compute_quorum_results(const std::string& replica_id, int64_t group_rank, const Quorum& quorum,
                                             bool init_sync) {
  std::vector<QuorumMember> members = quorum.participants;
  std::stable_sort(members.begin(), members.end(),
                   [](const QuorumMember& a, const QuorumMember& b) { return a.replica_id < b.replica_id; });
  const size_t n = members.size();
  size_t me = n;
  for (size_t i = 0; i < n; ++i)
    if (members[i].replica_id == replica_id) {
      me = i;
      break;
    }
  if (me == n) throw RpcError("replica " + replica_id + " not participating in returned quorum");

  int64_t max_step = members[0].step;
  int64_t max_failures = 0;
  for (const auto& m : members) {
    max_step = std::max(max_step, m.step);
    max_failures = std::max(max_failures, m.commit_failures);
  }
  std::vector<size_t> at_max;
  for (size_t i = 0; i < n; ++i)
    if (members[i].step == max_step) at_max.push_back(i);

  ManagerQuorumResponse r;
  for (size_t i = 0; i < at_max.size(); ++i)
    if (at_max[i] == me) r.max_replica_rank = static_cast<int64_t>(i);

  // One store per replica group; ranks of a group spread over the up-to-date replicas.
  const size_t primary = at_max[static_cast<size_t>(group_rank) % at_max.size()];

  // At step 0 with init_sync everybody but the primary pulls the primary's weights.
  const bool force_recover = init_sync && max_step == 0;
  std::vector<size_t> behind, current;
  for (size_t i = 0; i < n; ++i) {
    const bool recovering = members[i].step != max_step || (force_recover && i != primary);
    (recovering ? behind : current).push_back(i);
  }
  // Stripe recovering replicas over the up-to-date ones, offset by the local rank so the
  // ranks of one group fetch from different sources.
  for (size_t i = 0; i < behind.size(); ++i) {
    const size_t src = current[(i + static_cast<size_t>(group_rank)) % current.size()];
    if (src == me) r.recover_dst_replica_ranks.push_back(static_cast<int64_t>(behind[i]));
    if (behind[i] == me) r.recover_src_replica_rank = static_cast<int64_t>(src);
  }
  r.heal = r.recover_src_replica_rank.has_value();
  if (r.heal) r.recover_src_manager_address = members[static_cast<size_t>(*r.recover_src_replica_rank)].address;
  r.quorum_id = quorum.quorum_id;
  r.store_address = members[primary].store_address;
  r.max_step = max_step;
  r.max_world_size = static_cast<int64_t>(at_max.size());
  r.replica_rank = static_cast<int64_t>(me);
  r.replica_world_size = static_cast<int64_t>(n);
  r.commit_failures = max_failures;
  return r;
}

}  // namespace ftcp
