#include "lighthouse.h"

#include <algorithm>
#include <cstdio>
#include <ctime>
#include <sstream>

#include "log.h"

namespace ftcp {

namespace {

std::string html_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    switch (c) {
      case '<': o += "&lt;"; break;
      case '>': o += "&gt;"; break;
      case '&': o += "&amp;"; break;
      case '"': o += "&quot;"; break;
      default: o += c;
    }
  }
  return o;
}

const char* kIndexHtml = R"HTML(<!doctype html>
<html><head><meta charset="utf-8"><title>Lighthouse Dashboard - torchft_b200</title>
<style>
 body { font-family: sans-serif; margin: 1.5em; }
 .member { display: inline-block; border: 1px solid #888; border-radius: 4px; padding: 8px; margin: 4px; }
 .member.recovering { background: orange; }
 .heartbeat.old { color: red; }
</style></head>
<body>
<h1>Lighthouse Dashboard - torchft_b200</h1>
<div id="status">loading...</div>
<script>
async function refresh() {
  try { const r = await fetch('/status'); document.getElementById('status').innerHTML = await r.text(); } catch (e) {}
}
async function kill(id) { await fetch('/replica/' + encodeURIComponent(id) + '/kill', {method: 'POST'}); refresh(); }
refresh(); setInterval(refresh, 1000);
</script>
</body></html>
)HTML";

}  // namespace

Lighthouse::Lighthouse(LighthouseOpt opt) : opt_(std::move(opt)) {
  server_ = std::make_unique<Server>(
      opt_.bind, [this](uint8_t m, const std::string& b, TimePoint d) { return rpc(m, b, d); },
      [this](const HttpRequest& r) { return http(r); });
  server_->set_thread_tag("ftb-lighths");
  server_->start();
  tick_thread_ = std::thread([this] { tick_loop(); });
  log_info("lighthouse", "listening on " + address());
}

Lighthouse::~Lighthouse() { shutdown(); }

std::string Lighthouse::address() const { return "http://" + local_hostname() + ":" + std::to_string(server_->port()); }

void Lighthouse::shutdown() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (stop_) return;
    stop_ = true;
  }
  cv_.notify_all();
  if (tick_thread_.joinable()) tick_thread_.join();
  server_->shutdown();
}

void Lighthouse::tick_loop() {
  set_thread_name("ftb-lighths-tick");
  std::unique_lock<std::mutex> lk(mu_);
  while (!stop_) {
    tick_locked();
    cv_.wait_for(lk, Millis(opt_.quorum_tick_ms), [this] { return stop_; });
  }
}

// Replica ids are fresh on every process start, so a long job with many restarts would otherwise collect an
// unbounded number of dead entries.  Entries stay long enough for the dashboard to show them as stale.
void Lighthouse::prune_heartbeats_locked(TimePoint now) {
  const auto keep = std::max<int64_t>(600000, 100 * static_cast<int64_t>(opt_.heartbeat_timeout_ms));
  for (auto it = state_.heartbeats.begin(); it != state_.heartbeats.end();) {
    if (now - it->second > Millis(keep) && state_.participants.find(it->first) == state_.participants.end())
      it = state_.heartbeats.erase(it);
    else
      ++it;
  }
}

void Lighthouse::tick_locked() {
  if ((++ticks_ & 1023) == 0) prune_heartbeats_locked(Clock::now());
  auto [members, reason] = quorum_compute(Clock::now(), state_, opt_);
  if (reason != last_reason_) {
    log_info("lighthouse", "Quorum status: " + reason);
    last_reason_ = reason;
  }
  if (!members) return;
  bool failures = false;
  for (const auto& m : *members) failures = failures || m.commit_failures > 0;
  if (!state_.prev_quorum || quorum_changed(*members, state_.prev_quorum->participants)) {
    state_.quorum_id += 1;
    log_info("lighthouse", "Detected quorum change, bumping quorum_id to " + std::to_string(state_.quorum_id));
  } else if (failures) {
    state_.quorum_id += 1;
    log_info("lighthouse", "Detected commit failures, bumping quorum_id to " + std::to_string(state_.quorum_id));
  }
  Quorum q;
  q.quorum_id = state_.quorum_id;
  q.participants = std::move(*members);
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  q.created_seconds = ts.tv_sec;
  q.created_nanos = static_cast<int32_t>(ts.tv_nsec);
  state_.prev_quorum = q;
  state_.participants.clear();  // every member has to ask again for the next step
  history_.emplace_back(++seq_, std::move(q));
  while (history_.size() > 16) history_.pop_front();
  cv_.notify_all();
}

Quorum Lighthouse::handle_quorum(const QuorumMember& requester, TimePoint deadline) {
  std::unique_lock<std::mutex> lk(mu_);
  const std::string& id = requester.replica_id;
  ++quorum_requests_;
  log_info("lighthouse", "Received quorum request for replica " + id);
  auto join = [&] {
    const TimePoint now = Clock::now();
    state_.heartbeats[id] = now;  // a quorum request counts as a heartbeat
    state_.participants[id] = ParticipantDetails{now, requester};
  };
  join();
  uint64_t seen = seq_;
  tick_locked();
  while (true) {
    for (const auto& [s, q] : history_) {
      if (s <= seen) continue;
      seen = s;
      for (const auto& p : q.participants)
        if (p.replica_id == id) return q;
      // a quorum formed without us (e.g. a shrink-only round): register for the next one
      state_.heartbeats[id] = Clock::now();
      state_.participants[id] = ParticipantDetails{Clock::now(), requester};
      log_info("lighthouse", "Replica " + id + " not in quorum, retrying");
    }
    if (stop_) throw RpcError("lighthouse shutting down");
    if (cv_.wait_until(lk, deadline) == std::cv_status::timeout && seen == seq_)
      throw TimeoutError("lighthouse quorum deadline exceeded for replica " + id);
  }
}

void Lighthouse::handle_heartbeat(const std::string& replica_id) {
  std::lock_guard<std::mutex> g(mu_);
  ++heartbeats_received_;
  state_.heartbeats[replica_id] = Clock::now();
}

std::string Lighthouse::rpc(uint8_t method, const std::string& body, TimePoint deadline) {
  switch (method) {
    case kLighthouseQuorum: {
      // LighthouseQuorumRequest { QuorumMember requester = 1; }
      Reader r(body);
      int f, wt;
      std::optional<QuorumMember> req;
      while (r.next(&f, &wt)) {
        if (f == 1 && wt == 2) req = QuorumMember::decode(r.bytes());
        else r.skip(wt);
      }
      if (!req) throw RpcError("missing requester");
      return encode_msg1(handle_quorum(*req, deadline).encode());
    }
    case kLighthouseHeartbeat:
      handle_heartbeat(decode_str1(body));
      return std::string();
    default:
      throw RpcError("lighthouse: unknown method " + std::to_string(method));
  }
}

std::string Lighthouse::render_status() {
  std::lock_guard<std::mutex> g(mu_);
  const TimePoint now = Clock::now();
  auto [unused, reason] = quorum_compute(now, state_, opt_);
  (void)unused;
  std::ostringstream o;
  o << "Current quorum_id: " << state_.quorum_id << " <br>\nNext quorum status: " << html_escape(reason) << "\n";
  o << "<h3>Previous Quorum</h3>\n";
  if (state_.prev_quorum) {
    const Quorum& q = *state_.prev_quorum;
    int64_t max_step = -1;
    for (const auto& p : q.participants) max_step = std::max(max_step, p.step);
    timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    const double age = (ts.tv_sec - q.created_seconds) + (ts.tv_nsec - q.created_nanos) * 1e-9;
    o << "Previous quorum id: " << q.quorum_id << " <br>\nNum participants: " << q.participants.size()
      << " <br>\nQuorum age: " << age << "s\n<div>\n";
    for (const auto& p : q.participants) {
      o << "<div class=\"member" << (p.step != max_step ? " recovering" : "") << "\">\n  <b>" << html_escape(p.replica_id)
        << "</b> <br/>\n  Step: " << p.step << " <br/>\n  Manager: " << html_escape(p.address)
        << " <br/>\n  TCPStore: " << html_escape(p.store_address) << " <br/>\n  World size: " << p.world_size
        << " <br/>\n  <button onclick=\"kill('" << html_escape(p.replica_id) << "')\">Kill</button>\n</div>\n";
    }
    o << "</div>\n";
  }
  o << "<h2>Heartbeats</h2>\n<ul>\n";
  for (const auto& [id, last] : state_.heartbeats) {
    const double age = std::chrono::duration<double>(now - last).count();
    const bool old = now - last >= Millis(opt_.heartbeat_timeout_ms);
    o << "  <li class=\"heartbeat" << (old ? " old" : "") << "\">" << html_escape(id) << ": seen " << age << "s ago</li>\n";
  }
  o << "</ul>\n";
  return o.str();
}

namespace {
std::string label_escape(const std::string& v) {
  std::string o;
  for (char c : v) {
    if (c == '\\' || c == '"') o += '\\';
    if (c == '\n') {
      o += "\\n";
      continue;
    }
    o += c;
  }
  return o;
}
}  // namespace

std::string Lighthouse::render_metrics() {
  std::lock_guard<std::mutex> g(mu_);
  const TimePoint now = Clock::now();
  size_t healthy = 0;
  for (const auto& [id, last] : state_.heartbeats)
    if (now - last < Millis(opt_.heartbeat_timeout_ms)) ++healthy;
  std::ostringstream o;
  auto gauge = [&](const char* name, const char* help, double v) {
    o << "# HELP " << name << ' ' << help << "\n# TYPE " << name << " gauge\n" << name << ' ' << v << "\n";
  };
  auto counter = [&](const char* name, const char* help, uint64_t v) {
    o << "# HELP " << name << ' ' << help << "\n# TYPE " << name << " counter\n" << name << ' ' << v << "\n";
  };
  gauge("torchft_lighthouse_quorum_id", "Identifier of the latest quorum.", static_cast<double>(state_.quorum_id));
  gauge("torchft_lighthouse_quorum_participants", "Replica groups in the latest quorum.",
        state_.prev_quorum ? static_cast<double>(state_.prev_quorum->participants.size()) : 0.0);
  gauge("torchft_lighthouse_pending_participants", "Replica groups that have asked for the next quorum.",
        static_cast<double>(state_.participants.size()));
  gauge("torchft_lighthouse_healthy_replicas", "Replica groups with a heartbeat younger than the timeout.",
        static_cast<double>(healthy));
  gauge("torchft_lighthouse_known_replicas", "Replica ids with a recorded heartbeat.", static_cast<double>(state_.heartbeats.size()));
  counter("torchft_lighthouse_quorums_issued_total", "Quorums issued since start.", seq_);
  counter("torchft_lighthouse_quorum_requests_total", "Quorum requests received since start.", quorum_requests_);
  counter("torchft_lighthouse_heartbeats_total", "Explicit heartbeats received since start.", heartbeats_received_);
  if (state_.prev_quorum) {
    o << "# HELP torchft_lighthouse_replica_step Step reported by each member of the latest quorum.\n"
      << "# TYPE torchft_lighthouse_replica_step gauge\n";
    for (const auto& p : state_.prev_quorum->participants)
      o << "torchft_lighthouse_replica_step{replica=\"" << label_escape(p.replica_id) << "\"} " << p.step << "\n";
  }
  o << "# HELP torchft_lighthouse_heartbeat_age_seconds Seconds since each replica was last heard from.\n"
    << "# TYPE torchft_lighthouse_heartbeat_age_seconds gauge\n";
  for (const auto& [id, last] : state_.heartbeats)
    o << "torchft_lighthouse_heartbeat_age_seconds{replica=\"" << label_escape(id) << "\"} "
      << std::chrono::duration<double>(now - last).count() << "\n";
  return o.str();
}

HttpResponse Lighthouse::http(const HttpRequest& req) {
  HttpResponse resp;
  if (req.method == "GET" && (req.path == "/" || req.path == "/index.html")) {
    resp.body = kIndexHtml;
    return resp;
  }
  if (req.method == "GET" && req.path == "/status") {
    resp.body = render_status();
    return resp;
  }
  if (req.method == "GET" && req.path == "/metrics") {
    resp.body = render_metrics();
    resp.content_type = "text/plain; version=0.0.4";
    return resp;
  }
  const std::string prefix = "/replica/", suffix = "/kill";
  if (req.method == "POST" && req.path.rfind(prefix, 0) == 0 && req.path.size() > prefix.size() + suffix.size() &&
      req.path.compare(req.path.size() - suffix.size(), suffix.size(), suffix) == 0) {
    std::string id = req.path.substr(prefix.size(), req.path.size() - prefix.size() - suffix.size());
    // minimal percent-decoding (replica ids contain ':' and '-')
    std::string dec;
    for (size_t i = 0; i < id.size(); ++i) {
      if (id[i] == '%' && i + 2 < id.size() + 0 && isxdigit(id[i + 1]) && isxdigit(id[i + 2])) {
        dec += static_cast<char>(std::stoi(id.substr(i + 1, 2), nullptr, 16));
        i += 2;
      } else {
        dec += id[i];
      }
    }
    std::string addr;
    {
      std::lock_guard<std::mutex> g(mu_);
      if (state_.prev_quorum)
        for (const auto& p : state_.prev_quorum->participants)
          if (p.replica_id == dec) addr = p.address;
    }
    if (addr.empty()) {
      resp.code = 500;
      resp.body = "Something went wrong: failed to find replica";
      return resp;
    }
    try {
      Client c(addr, Millis(10000));
      c.call(kManagerKill, encode_str1("killed from dashboard"), Millis(10000));
    } catch (const std::exception& e) {
      // the manager exits inside the handler, so a closed connection is the expected outcome
    }
    resp.body = "ok";
    return resp;
  }
  resp.code = 404;
  resp.body = "not found";
  return resp;
}

}  // namespace ftcp
