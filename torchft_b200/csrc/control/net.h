// TCP plumbing of the control plane: listener, framed RPC server (thread per
// connection), RPC client with deadlines and reconnect-with-backoff.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "wire.h"

namespace ftcp {

using Clock = std::chrono::steady_clock;
using TimePoint = Clock::time_point;
using Millis = std::chrono::milliseconds;

struct TimeoutError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct RpcError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// "host:port", "[v6]:port" or "http://host:port" -> (host, port)
void parse_address(const std::string& addr, std::string* host, int* port);

// Exponential backoff used for (re)connects: 100 ms growing x1.5 up to 10 s with up to
// 100 ms of jitter (mirrors the policy of src/retry.rs:8-43 and src/net.rs:24-36).
struct Backoff {
  Millis initial{100}, max{10000};
  double factor = 1.5;
  Millis jitter{100};
  Millis current{0};
  Millis next();
};

int connect_with_deadline(const std::string& addr, TimePoint deadline);  // throws TimeoutError / RpcError
bool send_all(int fd, const char* p, size_t n, TimePoint deadline);
bool recv_all(int fd, char* p, size_t n, TimePoint deadline);  // false on EOF/timeout
void close_fd(int fd);

struct HttpRequest {
  std::string method, path, body;
};
struct HttpResponse {
  int code = 200;
  std::string content_type = "text/html; charset=utf-8";
  std::string body;
};

// Framed RPC + minimal HTTP/1.1 on one listening socket.
class Server {
 public:
  using RpcHandler = std::function<std::string(uint8_t method, const std::string& body, TimePoint deadline)>;
  using HttpHandler = std::function<HttpResponse(const HttpRequest&)>;

  Server(const std::string& bind, RpcHandler rpc, HttpHandler http = nullptr);
  ~Server();
  void start();
  void shutdown();
  int port() const { return port_; }
  bool stopping() const { return stop_.load(); }
  // Prefix of the names of the accept and connection threads; call before start().
  void set_thread_tag(std::string tag) { tag_ = std::move(tag); }

 private:
  void accept_loop();
  void serve(int fd);
  void serve_http(int fd, std::string first);

  RpcHandler rpc_;
  HttpHandler http_;
  int listen_fd_ = -1;
  int port_ = 0;
  std::atomic<bool> stop_{false};
  std::thread accept_thread_;
  std::mutex mu_;
  std::set<int> conns_;
  std::atomic<int> active_{0};
  std::string tag_ = "ftb-rpc";
};

// One reusable connection; calls are serialised.  A call that times out or fails closes
// the connection; the next call reconnects.
class Client {
 public:
  Client(std::string addr, Millis connect_timeout);
  ~Client();
  // Throws TimeoutError when the deadline passes (or the server reports one), RpcError otherwise.
  std::string call(uint8_t method, const std::string& body, Millis timeout);
  const std::string& addr() const { return addr_; }
  void close();

 private:
  void ensure_connected(TimePoint deadline);
  std::string addr_;
  Millis connect_timeout_;
  std::mutex mu_;
  int fd_ = -1;
};

std::string local_hostname();

}  // namespace ftcp
