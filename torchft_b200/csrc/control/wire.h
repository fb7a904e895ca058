// Wire format of the control plane.
//
// Messages use proto3 field encoding (varint and length-delimited wire types) with the
// field numbers of the reference schema (proto/torchft.proto:37-121), so a message body
// produced here is byte-compatible with that schema.  The transport differs from gRPC:
// a request is one frame
//     magic "FTB2" | u32 body_len | u8 method | u64 timeout_ms | body
// and a response is
//     u32 body_len | u8 status | body      (status 0 ok, 1 error text, 2 timeout text)
// both over a plain TCP connection that is reused across calls.  The timeout in the
// request header plays the role of the `grpc-timeout` header (src/timeout.rs:20-63).
#pragma once

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace ftcp {

enum Method : uint8_t {
  kLighthouseQuorum = 1,
  kLighthouseHeartbeat = 2,
  kManagerQuorum = 10,
  kManagerCheckpointMetadata = 11,
  kManagerShouldCommit = 12,
  kManagerKill = 13,
};

enum Status : uint8_t { kOk = 0, kError = 1, kTimeout = 2 };

struct WireError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Writer {
 public:
  void varint(uint64_t v) {
    while (v >= 0x80) {
      buf_.push_back(static_cast<char>((v & 0x7F) | 0x80));
      v >>= 7;
    }
    buf_.push_back(static_cast<char>(v));
  }
  void tag(int field, int wt) { varint((static_cast<uint64_t>(field) << 3) | wt); }
  void i64(int field, int64_t v) {
    if (v == 0) return;
    tag(field, 0);
    varint(static_cast<uint64_t>(v));
  }
  void i64_always(int field, int64_t v) {
    tag(field, 0);
    varint(static_cast<uint64_t>(v));
  }
  void boolean(int field, bool v) {
    if (!v) return;
    tag(field, 0);
    varint(1);
  }
  void str(int field, const std::string& s) {
    if (s.empty()) return;
    tag(field, 2);
    varint(s.size());
    buf_.append(s);
  }
  void msg(int field, const std::string& body) {
    tag(field, 2);
    varint(body.size());
    buf_.append(body);
  }
  std::string take() { return std::move(buf_); }

 private:
  std::string buf_;
};

class Reader {
 public:
  Reader(const char* p, size_t n) : p_(p), end_(p + n) {}
  explicit Reader(const std::string& s) : Reader(s.data(), s.size()) {}
  bool done() const { return p_ >= end_; }
  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (true) {
      if (p_ >= end_) throw WireError("truncated varint");
      const uint8_t b = static_cast<uint8_t>(*p_++);
      v |= static_cast<uint64_t>(b & 0x7F) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
      if (shift > 63) throw WireError("varint too long");
    }
    return v;
  }
  // Returns false at end of buffer; otherwise the next field number and wire type.
  bool next(int* field, int* wt) {
    if (done()) return false;
    const uint64_t t = varint();
    *field = static_cast<int>(t >> 3);
    *wt = static_cast<int>(t & 7);
    return true;
  }
  std::string bytes() {
    const uint64_t n = varint();
    if (n > static_cast<uint64_t>(end_ - p_)) throw WireError("truncated bytes");
    std::string s(p_, p_ + n);
    p_ += n;
    return s;
  }
  void skip(int wt) {
    switch (wt) {
      case 0: varint(); break;
      case 1: advance(8); break;
      case 2: bytes(); break;
      case 5: advance(4); break;
      default: throw WireError("unsupported wire type");
    }
  }

 private:
  void advance(size_t n) {
    if (n > static_cast<size_t>(end_ - p_)) throw WireError("truncated");
    p_ += n;
  }
  const char* p_;
  const char* end_;
};

// ------------------------------------------------------------------------------------ messages

struct QuorumMember {
  std::string replica_id;
  std::string address;
  std::string store_address;
  int64_t step = 0;
  uint64_t world_size = 0;
  bool shrink_only = false;
  int64_t commit_failures = 0;
  std::string data;  // user JSON

  std::string encode() const {
    Writer w;
    w.str(1, replica_id);
    w.str(2, address);
    w.str(3, store_address);
    w.i64(4, step);
    w.i64(5, static_cast<int64_t>(world_size));
    w.boolean(6, shrink_only);
    w.str(7, data);
    w.i64(8, commit_failures);
    return w.take();
  }
  static QuorumMember decode(const std::string& s) {
    QuorumMember m;
    Reader r(s);
    int f, wt;
    while (r.next(&f, &wt)) {
      switch (f) {
        case 1: m.replica_id = r.bytes(); break;
        case 2: m.address = r.bytes(); break;
        case 3: m.store_address = r.bytes(); break;
        case 4: m.step = static_cast<int64_t>(r.varint()); break;
        case 5: m.world_size = r.varint(); break;
        case 6: m.shrink_only = r.varint() != 0; break;
        case 7: m.data = r.bytes(); break;
        case 8: m.commit_failures = static_cast<int64_t>(r.varint()); break;
        default: r.skip(wt);
      }
    }
    return m;
  }
};

struct Quorum {
  int64_t quorum_id = 0;
  std::vector<QuorumMember> participants;
  int64_t created_seconds = 0;
  int32_t created_nanos = 0;

  std::string encode() const {
    Writer w;
    w.i64(1, quorum_id);
    for (const auto& p : participants) w.msg(2, p.encode());
    Writer ts;
    ts.i64(1, created_seconds);
    ts.i64(2, created_nanos);
    w.msg(3, ts.take());
    return w.take();
  }
  static Quorum decode(const std::string& s) {
    Quorum q;
    Reader r(s);
    int f, wt;
    while (r.next(&f, &wt)) {
      switch (f) {
        case 1: q.quorum_id = static_cast<int64_t>(r.varint()); break;
        case 2: q.participants.push_back(QuorumMember::decode(r.bytes())); break;
        case 3: {
          const std::string t = r.bytes();
          Reader tr(t);
          int tf, twt;
          while (tr.next(&tf, &twt)) {
            if (tf == 1) q.created_seconds = static_cast<int64_t>(tr.varint());
            else if (tf == 2) q.created_nanos = static_cast<int32_t>(tr.varint());
            else tr.skip(twt);
          }
          break;
        }
        default: r.skip(wt);
      }
    }
    return q;
  }
};

struct ManagerQuorumRequest {
  int64_t group_rank = 0;
  int64_t step = 0;
  std::string checkpoint_metadata;
  bool shrink_only = false;
  bool init_sync = true;
  int64_t commit_failures = 0;

  std::string encode() const {
    Writer w;
    w.i64(1, group_rank);
    w.i64(2, step);
    w.str(3, checkpoint_metadata);
    w.boolean(4, shrink_only);
    w.boolean(5, init_sync);
    w.i64(6, commit_failures);
    return w.take();
  }
  static ManagerQuorumRequest decode(const std::string& s) {
    ManagerQuorumRequest m;
    m.init_sync = false;  // proto3 default when the field is absent
    Reader r(s);
    int f, wt;
    while (r.next(&f, &wt)) {
      switch (f) {
        case 1: m.group_rank = static_cast<int64_t>(r.varint()); break;
        case 2: m.step = static_cast<int64_t>(r.varint()); break;
        case 3: m.checkpoint_metadata = r.bytes(); break;
        case 4: m.shrink_only = r.varint() != 0; break;
        case 5: m.init_sync = r.varint() != 0; break;
        case 6: m.commit_failures = static_cast<int64_t>(r.varint()); break;
        default: r.skip(wt);
      }
    }
    return m;
  }
};

struct ManagerQuorumResponse {
  int64_t quorum_id = 0;
  std::string recover_src_manager_address;
  std::optional<int64_t> recover_src_replica_rank;
  std::vector<int64_t> recover_dst_replica_ranks;
  std::string store_address;
  int64_t max_step = 0;
  std::optional<int64_t> max_replica_rank;
  int64_t max_world_size = 0;
  int64_t replica_rank = 0;
  int64_t replica_world_size = 0;
  bool heal = false;
  int64_t commit_failures = 0;

  std::string encode() const {
    Writer w;
    w.i64(1, quorum_id);
    w.str(2, recover_src_manager_address);
    if (recover_src_replica_rank) w.i64_always(3, *recover_src_replica_rank);
    for (int64_t d : recover_dst_replica_ranks) w.i64_always(4, d);
    w.str(5, store_address);
    w.i64(6, max_step);
    if (max_replica_rank) w.i64_always(7, *max_replica_rank);
    w.i64(8, max_world_size);
    w.i64(9, replica_rank);
    w.i64(10, replica_world_size);
    w.boolean(11, heal);
    w.i64(12, commit_failures);
    return w.take();
  }
  static ManagerQuorumResponse decode(const std::string& s) {
    ManagerQuorumResponse m;
    Reader r(s);
    int f, wt;
    while (r.next(&f, &wt)) {
      switch (f) {
        case 1: m.quorum_id = static_cast<int64_t>(r.varint()); break;
        case 2: m.recover_src_manager_address = r.bytes(); break;
        case 3: m.recover_src_replica_rank = static_cast<int64_t>(r.varint()); break;
        case 4:
          if (wt == 2) {  // packed
            const std::string packed = r.bytes();
            Reader pr(packed);
            while (!pr.done()) m.recover_dst_replica_ranks.push_back(static_cast<int64_t>(pr.varint()));
          } else {
            m.recover_dst_replica_ranks.push_back(static_cast<int64_t>(r.varint()));
          }
          break;
        case 5: m.store_address = r.bytes(); break;
        case 6: m.max_step = static_cast<int64_t>(r.varint()); break;
        case 7: m.max_replica_rank = static_cast<int64_t>(r.varint()); break;
        case 8: m.max_world_size = static_cast<int64_t>(r.varint()); break;
        case 9: m.replica_rank = static_cast<int64_t>(r.varint()); break;
        case 10: m.replica_world_size = static_cast<int64_t>(r.varint()); break;
        case 11: m.heal = r.varint() != 0; break;
        case 12: m.commit_failures = static_cast<int64_t>(r.varint()); break;
        default: r.skip(wt);
      }
    }
    return m;
  }
};

struct ShouldCommitRequest {
  bool should_commit = false;
  int64_t group_rank = 0;
  int64_t step = 0;
  std::string encode() const {
    Writer w;
    w.boolean(1, should_commit);
    w.i64(2, group_rank);
    w.i64(3, step);
    return w.take();
  }
  static ShouldCommitRequest decode(const std::string& s) {
    ShouldCommitRequest m;
    Reader r(s);
    int f, wt;
    while (r.next(&f, &wt)) {
      switch (f) {
        case 1: m.should_commit = r.varint() != 0; break;
        case 2: m.group_rank = static_cast<int64_t>(r.varint()); break;
        case 3: m.step = static_cast<int64_t>(r.varint()); break;
        default: r.skip(wt);
      }
    }
    return m;
  }
};

// Single-field helpers (field 1) for the small request/response messages.
inline std::string encode_str1(const std::string& s) {
  Writer w;
  w.str(1, s);
  return w.take();
}
inline std::string decode_str1(const std::string& body) {
  Reader r(body);
  int f, wt;
  std::string out;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == 2) out = r.bytes();
    else r.skip(wt);
  }
  return out;
}
inline std::string encode_i64_1(int64_t v) {
  Writer w;
  w.i64(1, v);
  return w.take();
}
inline int64_t decode_i64_1(const std::string& body) {
  Reader r(body);
  int f, wt;
  int64_t out = 0;
  while (r.next(&f, &wt)) {
    if (f == 1 && wt == 0) out = static_cast<int64_t>(r.varint());
    else r.skip(wt);
  }
  return out;
}
inline std::string encode_msg1(const std::string& inner) {
  Writer w;
  w.msg(1, inner);
  return w.take();
}

}  // namespace ftcp
