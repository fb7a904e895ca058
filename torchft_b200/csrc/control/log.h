// Minimal leveled logger for the control plane (stderr).  Level from the
// FTB200_LOG (or RUST_LOG, honoured for drop-in compatibility) environment variable:
// error, warn, info (default: warn), debug.
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include <pthread.h>

namespace ftcp {

inline int log_level() {
  static int lvl = [] {
    const char* e = getenv("FTB200_LOG");
    if (e == nullptr) e = getenv("RUST_LOG");
    if (e == nullptr) return 1;
    if (!strcasecmp(e, "error")) return 0;
    if (!strcasecmp(e, "warn")) return 1;
    if (!strcasecmp(e, "info")) return 2;
    if (!strcasecmp(e, "debug") || !strcasecmp(e, "trace")) return 3;
    return 1;
  }();
  return lvl;
}

inline void log_at(int lvl, const char* name, const std::string& who, const std::string& msg) {
  if (lvl > log_level()) return;
  const auto now = std::chrono::system_clock::now().time_since_epoch();
  const double t = std::chrono::duration<double>(now).count();
  fprintf(stderr, "[%.3f %s torchft_b200::%s] %s\n", t, name, who.c_str(), msg.c_str());
}

// Names the calling thread (shown by ps -L, top -H, gdb and py-spy); the kernel keeps 15 characters.
inline void set_thread_name(const std::string& name) { pthread_setname_np(pthread_self(), name.substr(0, 15).c_str()); }

inline void log_error(const std::string& who, const std::string& msg) { log_at(0, "ERROR", who, msg); }
inline void log_warn(const std::string& who, const std::string& msg) { log_at(1, "WARN", who, msg); }
inline void log_info(const std::string& who, const std::string& msg) { log_at(2, "INFO", who, msg); }

}  // namespace ftcp
