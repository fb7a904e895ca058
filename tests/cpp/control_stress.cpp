// Concurrency stress of the control plane, meant to be built with -fsanitize=thread or
// -fsanitize=address: one lighthouse, three replica groups of two ranks each running quorum +
// should_commit rounds from their own threads, a fourth group that joins and leaves in the
// middle, dashboard requests and heartbeats in the background.  Exits non-zero when the ranks of
// one step disagree on the quorum or on the commit decision.
#include <atomic>
#include <cstdio>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "lighthouse.h"
#include "manager.h"

using namespace ftcp;

namespace {

std::mutex g_mu;
std::map<int64_t, std::map<std::string, int64_t>> g_quorum_of_step;  // step -> replica -> quorum id
std::atomic<int> g_failures{0};

void fail(const char* what, int64_t step) {
  std::fprintf(stderr, "MISMATCH: %s at step %lld\n", what, static_cast<long long>(step));
  g_failures.fetch_add(1);
}

void rank_loop(const std::string& replica, const std::string& manager_addr, int rank, int steps, bool dissent) {
  Client c(manager_addr, Millis(5000));
  for (int step = 0; step < steps; ++step) {
    ManagerQuorumRequest req;
    req.group_rank = rank;
    req.step = step;
    req.checkpoint_metadata = "meta-" + replica + "-" + std::to_string(rank);
    req.init_sync = false;
    ManagerQuorumResponse r = ManagerQuorumResponse::decode(c.call(kManagerQuorum, req.encode(), Millis(20000)));
    {
      std::lock_guard<std::mutex> l(g_mu);
      auto& seen = g_quorum_of_step[step];
      auto it = seen.find(replica);
      if (it == seen.end())
        seen[replica] = r.quorum_id;
      else if (it->second != r.quorum_id)
        fail("ranks of one replica saw different quorum ids", step);
    }
    ShouldCommitRequest v;
    v.group_rank = rank;
    v.step = step;
    v.should_commit = !(dissent && rank == 1 && step % 5 == 3);
    const bool decision = decode_i64_1(c.call(kManagerShouldCommit, v.encode(), Millis(20000))) != 0;
    const bool expect = !(dissent && step % 5 == 3);
    if (decision != expect) fail("commit decision", step);
    (void)decode_str1(c.call(kManagerCheckpointMetadata, encode_i64_1(1 - rank), Millis(5000)));
  }
}

}  // namespace

int main() {
  LighthouseOpt opt;
  opt.bind = "[::]:0";
  opt.min_replicas = 3;
  opt.join_timeout_ms = 50;
  opt.quorum_tick_ms = 5;
  opt.heartbeat_timeout_ms = 2000;
  Lighthouse lh(opt);
  const std::string lh_addr = "http://127.0.0.1:" + std::to_string(lh.port());

  const int steps = 25;
  std::vector<std::unique_ptr<ManagerServer>> managers;
  for (int g = 0; g < 3; ++g) {
    managers.emplace_back(new ManagerServer("rep" + std::to_string(g), lh_addr, "127.0.0.1", "[::]:0",
                                            "store" + std::to_string(g) + ":1234", 2, Millis(20), Millis(5000), 2));
  }
  std::vector<std::thread> threads;
  for (int g = 0; g < 3; ++g)
    for (int r = 0; r < 2; ++r)
      threads.emplace_back(rank_loop, "rep" + std::to_string(g), managers[g]->address(), r, steps, g == 1);

  // a fourth group that comes and goes while the others are running
  std::thread churn([&] {
    for (int k = 0; k < 3; ++k) {
      std::this_thread::sleep_for(Millis(60));
      ManagerServer extra("extra" + std::to_string(k), lh_addr, "127.0.0.1", "[::]:0", "storeX:1", 1, Millis(20), Millis(5000), 0);
      try {
        Client c(extra.address(), Millis(2000));
        ManagerQuorumRequest req;
        req.group_rank = 0;
        req.step = 0;
        req.init_sync = false;
        (void)c.call(kManagerQuorum, req.encode(), Millis(3000));
      } catch (const std::exception&) {
        // it may time out when the others are between rounds; joining and leaving is the point
      }
      extra.shutdown();
    }
  });
  // background traffic: explicit heartbeats of an unknown replica
  std::atomic<bool> stop{false};
  std::thread pinger([&] {
    Client c(lh_addr, Millis(2000));
    while (!stop.load()) {
      try {
        (void)c.call(kLighthouseHeartbeat, encode_str1("observer"), Millis(1000));
      } catch (const std::exception&) {
      }
      std::this_thread::sleep_for(Millis(3));
    }
  });

  for (auto& t : threads) t.join();
  churn.join();
  stop.store(true);
  pinger.join();
  for (auto& m : managers) m->shutdown();
  lh.shutdown();
  if (g_failures.load() != 0) return 1;
  std::printf("control stress ok: %d steps x 3 replica groups x 2 ranks\n", steps);
  return 0;
}
