#include "net.h"

#include "log.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <signal.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstring>
#include <random>

namespace ftcp {

namespace {

int remaining_ms(TimePoint deadline) {
  auto d = std::chrono::duration_cast<Millis>(deadline - Clock::now()).count();
  if (d < 0) return 0;
  if (d > 3600 * 1000) return 3600 * 1000;
  return static_cast<int>(d);
}

void set_nonblocking(int fd, bool nb) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, nb ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}

void tune(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
  int idle = 60, intvl = 20, cnt = 3;  // keepalive probes comparable to the 60 s / 20 s HTTP2 pings of the reference
  setsockopt(fd, IPPROTO_TCP, TCP_KEEPIDLE, &idle, sizeof(idle));
  setsockopt(fd, IPPROTO_TCP, TCP_KEEPINTVL, &intvl, sizeof(intvl));
  setsockopt(fd, IPPROTO_TCP, TCP_KEEPCNT, &cnt, sizeof(cnt));
}

void put_u32(std::string& s, uint32_t v) {
  char b[4];
  for (int i = 0; i < 4; ++i) b[i] = static_cast<char>((v >> (8 * i)) & 0xFF);
  s.append(b, 4);
}
void put_u64(std::string& s, uint64_t v) {
  char b[8];
  for (int i = 0; i < 8; ++i) b[i] = static_cast<char>((v >> (8 * i)) & 0xFF);
  s.append(b, 8);
}
uint32_t get_u32(const char* p) {
  uint32_t v = 0;
  for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(static_cast<uint8_t>(p[i])) << (8 * i);
  return v;
}
uint64_t get_u64(const char* p) {
  uint64_t v = 0;
  for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(static_cast<uint8_t>(p[i])) << (8 * i);
  return v;
}

constexpr uint32_t kMaxFrame = 64u << 20;

}  // namespace

void parse_address(const std::string& addr_in, std::string* host, int* port) {
  std::string addr = addr_in;
  for (const char* scheme : {"http://", "https://", "tcp://"}) {
    if (addr.rfind(scheme, 0) == 0) addr = addr.substr(strlen(scheme));
  }
  while (!addr.empty() && addr.back() == '/') addr.pop_back();
  const size_t colon = addr.rfind(':');
  if (colon == std::string::npos) throw RpcError("address has no port: " + addr_in);
  std::string h = addr.substr(0, colon);
  if (!h.empty() && h.front() == '[' && h.back() == ']') h = h.substr(1, h.size() - 2);
  *host = h;
  try {
    *port = std::stoi(addr.substr(colon + 1));
  } catch (...) {
    throw RpcError("bad port in address: " + addr_in);
  }
}

Millis Backoff::next() {
  static thread_local std::mt19937 rng(std::random_device{}());
  if (current.count() == 0) current = initial;
  else current = std::min(max, Millis(static_cast<int64_t>(current.count() * factor)));
  std::uniform_int_distribution<int64_t> j(0, jitter.count());
  return current + Millis(j(rng));
}

void close_fd(int fd) {
  if (fd >= 0) ::close(fd);
}

static int try_connect_once(const std::string& host, int port, TimePoint deadline, std::string* err) {
  addrinfo hints{};
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  addrinfo* res = nullptr;
  std::string h = host;
  if (h.empty() || h == "::" || h == "0.0.0.0") h = "localhost";
  const std::string ps = std::to_string(port);
  int rc = getaddrinfo(h.c_str(), ps.c_str(), &hints, &res);
  if (rc != 0) {
    *err = std::string("getaddrinfo(") + h + "): " + gai_strerror(rc);
    return -1;
  }
  int fd = -1;
  for (addrinfo* ai = res; ai != nullptr; ai = ai->ai_next) {
    fd = ::socket(ai->ai_family, ai->ai_socktype | SOCK_CLOEXEC, ai->ai_protocol);
    if (fd < 0) continue;
    set_nonblocking(fd, true);
    rc = ::connect(fd, ai->ai_addr, ai->ai_addrlen);
    if (rc != 0 && errno == EINPROGRESS) {
      pollfd pfd{fd, POLLOUT, 0};
      rc = ::poll(&pfd, 1, std::max(1, remaining_ms(deadline)));
      if (rc > 0) {
        int soerr = 0;
        socklen_t len = sizeof(soerr);
        getsockopt(fd, SOL_SOCKET, SO_ERROR, &soerr, &len);
        rc = soerr == 0 ? 0 : -1;
        if (soerr) errno = soerr;
      } else {
        rc = -1;
        if (errno == 0) errno = ETIMEDOUT;
      }
    }
    if (rc == 0) break;
    *err = std::string("connect: ") + strerror(errno);
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd >= 0) tune(fd);
  return fd;
}

int connect_with_deadline(const std::string& addr, TimePoint deadline) {
  std::string host;
  int port;
  parse_address(addr, &host, &port);
  Backoff bo;
  std::string err;
  while (true) {
    int fd = try_connect_once(host, port, deadline, &err);
    if (fd >= 0) return fd;
    const Millis wait = bo.next();
    if (Clock::now() + wait >= deadline) throw TimeoutError("timed out connecting to " + addr + ": " + err);
    std::this_thread::sleep_for(wait);
  }
}

bool send_all(int fd, const char* p, size_t n, TimePoint deadline) {
  while (n > 0) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w > 0) {
      p += w;
      n -= static_cast<size_t>(w);
      continue;
    }
    if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) {
      pollfd pfd{fd, POLLOUT, 0};
      int ms = remaining_ms(deadline);
      if (ms == 0) return false;
      ::poll(&pfd, 1, ms);
      continue;
    }
    return false;
  }
  return true;
}

bool recv_all(int fd, char* p, size_t n, TimePoint deadline) {
  while (n > 0) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r > 0) {
      p += r;
      n -= static_cast<size_t>(r);
      continue;
    }
    if (r == 0) return false;
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) {
      pollfd pfd{fd, POLLIN, 0};
      int ms = remaining_ms(deadline);
      if (ms == 0) return false;
      ::poll(&pfd, 1, ms);
      continue;
    }
    return false;
  }
  return true;
}

std::string local_hostname() {
  char buf[256];
  if (gethostname(buf, sizeof(buf)) != 0) return "localhost";
  buf[255] = 0;
  return buf;
}

// ------------------------------------------------------------------------------------ Server

Server::Server(const std::string& bind, RpcHandler rpc, HttpHandler http) : rpc_(std::move(rpc)), http_(std::move(http)) {
  std::string host;
  int port;
  parse_address(bind, &host, &port);
  // dual-stack IPv6 listener; falls back to IPv4 when IPv6 is unavailable
  int fd = ::socket(AF_INET6, SOCK_STREAM | SOCK_CLOEXEC, 0);
  bool v6 = fd >= 0;
  if (v6) {
    int zero = 0, one = 1;
    setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, &zero, sizeof(zero));
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in6 a{};
    a.sin6_family = AF_INET6;
    a.sin6_addr = in6addr_any;
    a.sin6_port = htons(static_cast<uint16_t>(port));
    if (::bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
      ::close(fd);
      fd = -1;
      v6 = false;
    }
  }
  if (!v6) {
    fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) throw RpcError("socket() failed");
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(INADDR_ANY);
    a.sin_port = htons(static_cast<uint16_t>(port));
    if (::bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
      ::close(fd);
      throw RpcError("bind(" + bind + ") failed: " + strerror(errno));
    }
  }
  if (::listen(fd, 1024) != 0) {
    ::close(fd);
    throw RpcError("listen failed");
  }
  sockaddr_storage ss{};
  socklen_t len = sizeof(ss);
  getsockname(fd, reinterpret_cast<sockaddr*>(&ss), &len);
  port_ = ntohs(ss.ss_family == AF_INET6 ? reinterpret_cast<sockaddr_in6*>(&ss)->sin6_port
                                         : reinterpret_cast<sockaddr_in*>(&ss)->sin_port);
  listen_fd_ = fd;
}

Server::~Server() { shutdown(); }

void Server::start() {
  accept_thread_ = std::thread([this] {
    set_thread_name(tag_ + "-acc");
    accept_loop();
  });
}

void Server::shutdown() {
  if (stop_.exchange(true)) {
    if (accept_thread_.joinable() && std::this_thread::get_id() != accept_thread_.get_id()) accept_thread_.join();
    return;
  }
  if (listen_fd_ >= 0) ::shutdown(listen_fd_, SHUT_RDWR);
  {
    std::lock_guard<std::mutex> g(mu_);
    for (int fd : conns_) ::shutdown(fd, SHUT_RDWR);
  }
  if (accept_thread_.joinable()) accept_thread_.join();
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
  // connection threads are detached; wait for them to leave the handlers
  for (int i = 0; i < 500 && active_.load() > 0; ++i) std::this_thread::sleep_for(Millis(10));
}

void Server::accept_loop() {
  while (!stop_.load()) {
    pollfd pfd{listen_fd_, POLLIN, 0};
    int rc = ::poll(&pfd, 1, 100);
    if (rc <= 0) continue;
    int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) continue;
    tune(fd);
    {
      std::lock_guard<std::mutex> g(mu_);
      conns_.insert(fd);
    }
    active_.fetch_add(1);
    std::thread([this, fd] {
      set_thread_name(tag_ + "-conn");
      try {
        serve(fd);
      } catch (...) {
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        conns_.erase(fd);
      }
      ::close(fd);
      active_.fetch_sub(1);
    }).detach();
  }
}

void Server::serve(int fd) {
  const TimePoint forever = Clock::now() + std::chrono::hours(24 * 365);
  while (!stop_.load()) {
    char magic[4];
    if (!recv_all(fd, magic, 4, forever)) return;
    if (memcmp(magic, "FTB2", 4) != 0) {
      serve_http(fd, std::string(magic, 4));
      return;
    }
    char hdr[13];
    if (!recv_all(fd, hdr, 13, forever)) return;
    const uint32_t len = get_u32(hdr);
    const uint8_t method = static_cast<uint8_t>(hdr[4]);
    const uint64_t timeout_ms = get_u64(hdr + 5);
    if (len > kMaxFrame) return;
    std::string body(len, '\0');
    if (len && !recv_all(fd, body.data(), len, Clock::now() + Millis(30000))) return;
    const TimePoint deadline = Clock::now() + Millis(std::min<uint64_t>(timeout_ms, 24ull * 3600 * 1000));
    std::string out;
    uint8_t status = kOk;
    try {
      out = rpc_(method, body, deadline);
    } catch (const TimeoutError& e) {
      status = kTimeout;
      out = e.what();
    } catch (const std::exception& e) {
      status = kError;
      out = e.what();
    }
    std::string frame;
    put_u32(frame, static_cast<uint32_t>(out.size()));
    frame.push_back(static_cast<char>(status));
    frame.append(out);
    if (!send_all(fd, frame.data(), frame.size(), Clock::now() + Millis(30000))) return;
  }
}

void Server::serve_http(int fd, std::string buf) {
  const TimePoint deadline = Clock::now() + Millis(5000);
  // read until end of headers
  while (buf.find("\r\n\r\n") == std::string::npos && buf.size() < 65536) {
    char c[1024];
    pollfd pfd{fd, POLLIN, 0};
    if (::poll(&pfd, 1, remaining_ms(deadline)) <= 0) return;
    ssize_t r = ::recv(fd, c, sizeof(c), 0);
    if (r <= 0) return;
    buf.append(c, static_cast<size_t>(r));
  }
  const size_t hend = buf.find("\r\n\r\n");
  if (hend == std::string::npos) return;
  HttpRequest req;
  const size_t sp1 = buf.find(' ');
  const size_t sp2 = buf.find(' ', sp1 + 1);
  if (sp1 == std::string::npos || sp2 == std::string::npos) return;
  req.method = buf.substr(0, sp1);
  req.path = buf.substr(sp1 + 1, sp2 - sp1 - 1);
  size_t content_len = 0;
  {
    std::string lower = buf.substr(0, hend);
    for (auto& ch : lower) ch = static_cast<char>(tolower(ch));
    const size_t p = lower.find("content-length:");
    if (p != std::string::npos) content_len = static_cast<size_t>(atoll(lower.c_str() + p + 15));
  }
  req.body = buf.substr(hend + 4);
  while (req.body.size() < content_len && content_len < (1u << 20)) {
    char c[1024];
    pollfd pfd{fd, POLLIN, 0};
    if (::poll(&pfd, 1, remaining_ms(deadline)) <= 0) break;
    ssize_t r = ::recv(fd, c, sizeof(c), 0);
    if (r <= 0) break;
    req.body.append(c, static_cast<size_t>(r));
  }
  HttpResponse resp;
  if (http_) {
    try {
      resp = http_(req);
    } catch (const std::exception& e) {
      resp.code = 500;
      resp.body = std::string("Something went wrong: ") + e.what();
    }
  } else {
    resp.code = 404;
    resp.body = "not found";
  }
  const char* reason = resp.code == 200 ? "OK" : resp.code == 404 ? "Not Found" : resp.code == 400 ? "Bad Request" : "Error";
  std::string out = "HTTP/1.1 " + std::to_string(resp.code) + " " + reason + "\r\nContent-Type: " + resp.content_type +
                    "\r\nContent-Length: " + std::to_string(resp.body.size()) + "\r\nConnection: close\r\n\r\n" + resp.body;
  send_all(fd, out.data(), out.size(), Clock::now() + Millis(5000));
}

// ------------------------------------------------------------------------------------ Client

Client::Client(std::string addr, Millis connect_timeout) : addr_(std::move(addr)), connect_timeout_(connect_timeout) {
  std::lock_guard<std::mutex> g(mu_);
  ensure_connected(Clock::now() + connect_timeout_);
}

Client::~Client() { close(); }

void Client::close() {
  std::lock_guard<std::mutex> g(mu_);
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

void Client::ensure_connected(TimePoint deadline) {
  if (fd_ >= 0) return;
  fd_ = connect_with_deadline(addr_, deadline);
}

std::string Client::call(uint8_t method, const std::string& body, Millis timeout) {
  std::lock_guard<std::mutex> g(mu_);
  const TimePoint deadline = Clock::now() + timeout;
  ensure_connected(std::min(deadline, Clock::now() + connect_timeout_));
  std::string frame("FTB2", 4);
  put_u32(frame, static_cast<uint32_t>(body.size()));
  frame.push_back(static_cast<char>(method));
  put_u64(frame, static_cast<uint64_t>(std::max<int64_t>(0, timeout.count())));
  frame.append(body);
  auto fail = [&](const std::string& what, bool timed_out) {
    ::close(fd_);
    fd_ = -1;
    if (timed_out) throw TimeoutError(what);
    throw RpcError(what);
  };
  if (!send_all(fd_, frame.data(), frame.size(), deadline)) {
    // stale connection (server restarted): retry once on a fresh socket
    ::close(fd_);
    fd_ = -1;
    ensure_connected(std::min(deadline, Clock::now() + connect_timeout_));
    if (!send_all(fd_, frame.data(), frame.size(), deadline)) fail("send to " + addr_ + " failed", Clock::now() >= deadline);
  }
  // small grace period so a server-side timeout message can still arrive
  const TimePoint rdl = deadline + Millis(200);
  char hdr[5];
  if (!recv_all(fd_, hdr, 5, rdl)) {
    const bool to = Clock::now() >= deadline;
    fail(to ? "deadline exceeded waiting for " + addr_ : "connection to " + addr_ + " closed", to);
  }
  const uint32_t len = get_u32(hdr);
  const uint8_t status = static_cast<uint8_t>(hdr[4]);
  if (len > kMaxFrame) fail("oversized response", false);
  std::string out(len, '\0');
  if (len && !recv_all(fd_, out.data(), len, rdl + Millis(5000))) fail("truncated response from " + addr_, false);
  if (status == kTimeout) throw TimeoutError(out);
  if (status != kOk) throw RpcError(out);
  return out;
}

}  // namespace ftcp
