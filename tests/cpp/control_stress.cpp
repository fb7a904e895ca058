// Concurrency stress of the control plane, meant to be built with -fsanitize=thread or
// -fsanitize=address: one lighthouse, three replica groups of two ranks each running quorum +
// should_commit rounds from their own threads, a fourth group that joins and leaves in the
// middle, dashboard requests and heartbeats in the background.  Exits non-zero when the ranks of
// one step disagree on the quorum or on the commit decision.  A last stage throws malformed input
// (garbage, truncated frames, absurd lengths, random bodies for every method) at both servers,
// which must keep answering; under the sanitizers any bad read in the decoders shows up there.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstring>
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

// ---- malformed input ------------------------------------------------------------------------
uint32_t g_lcg = 12345;
uint32_t rnd() { return g_lcg = g_lcg * 1664525u + 1013904223u; }

void poke(int port, const std::string& payload) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(static_cast<uint16_t>(port));
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  timeval tv{0, 20000};
  ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) {
    if (!payload.empty()) (void)!::send(fd, payload.data(), payload.size(), MSG_NOSIGNAL);
    char buf[512];
    (void)!::recv(fd, buf, sizeof(buf), 0);
  }
  ::close(fd);
}

std::string frame(uint8_t method, const std::string& body, uint32_t announced) {
  std::string f = "FTB2";
  for (int i = 0; i < 4; ++i) f.push_back(static_cast<char>((announced >> (8 * i)) & 0xff));
  f.push_back(static_cast<char>(method));
  const uint64_t timeout_ms = 30;
  for (int i = 0; i < 8; ++i) f.push_back(static_cast<char>((timeout_ms >> (8 * i)) & 0xff));
  return f + body;
}

std::string random_bytes(size_t n) {
  std::string s(n, '\0');
  for (auto& c : s) c = static_cast<char>(rnd() >> 24);
  return s;
}

void malformed_input(int port) {
  poke(port, "");
  poke(port, random_bytes(3));
  poke(port, random_bytes(64));
  poke(port, "FTB2" + random_bytes(5));
  poke(port, frame(1, "", 0xFFFFFFFFu));
  poke(port, frame(1, "abc", 1u << 20));
  poke(port, "GET /" + std::string(70000, 'a') + " HTTP/1.1\r\n\r\n");
  poke(port, "POST /replica/%zz/kill HTTP/1.1\r\nContent-Length: 99999999999\r\n\r\n");
  const size_t sizes[] = {0, 1, 2, 7, 33, 200, 4096};
  for (int method = 0; method < 12; ++method)
    for (int k = 0; k < 8; ++k) {
      const std::string body = random_bytes(sizes[rnd() % 7]);
      poke(port, frame(static_cast<uint8_t>(method), body, static_cast<uint32_t>(body.size())));
    }
  ManagerQuorumRequest good;
  good.group_rank = 1;
  good.step = 7;
  good.checkpoint_metadata = "some metadata";
  const std::string enc = good.encode();
  for (size_t cut = 0; cut < enc.size(); ++cut)
    for (int method = 1; method <= 6; ++method)
      poke(port, frame(static_cast<uint8_t>(method), enc.substr(0, cut), static_cast<uint32_t>(cut)));
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
  // malformed input against the lighthouse and one manager; both must still answer afterwards
  {
    ManagerServer probe("probe", lh_addr, "127.0.0.1", "[::]:0", "storeP:1", 1, Millis(20), Millis(5000), 0);
    const std::string paddr = probe.address();
    malformed_input(lh.port());
    malformed_input(std::stoi(paddr.substr(paddr.rfind(':') + 1)));
    try {
      Client c(lh_addr, Millis(2000));
      (void)c.call(kLighthouseHeartbeat, encode_str1("observer"), Millis(2000));
      Client m(paddr, Millis(2000));
      ShouldCommitRequest v;  // a group of one rank: the vote returns at once
      v.group_rank = 0;
      v.step = 0;
      v.should_commit = true;
      if (decode_i64_1(m.call(kManagerShouldCommit, v.encode(), Millis(2000))) == 0) fail("vote after malformed input", 0);
    } catch (const std::exception& e) {
      std::fprintf(stderr, "MISMATCH: server unusable after malformed input: %s\n", e.what());
      g_failures.fetch_add(1);
    }
    probe.shutdown();
  }
  for (auto& m : managers) m->shutdown();
  lh.shutdown();
  if (g_failures.load() != 0) return 1;
  std::printf("control stress ok: %d steps x 3 replica groups x 2 ranks\n", steps);
  return 0;
}
