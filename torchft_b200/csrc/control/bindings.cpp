// pybind11 module `torchft_b200._ftcp`: Python surface of the C++ control plane.
// Class and method names follow torchft/_torchft.pyi of the reference so that the
// Python layers above can be written against the same contract.  Every blocking call
// releases the GIL; deadline expiry surfaces as Python `TimeoutError`, every other
// control-plane failure as `RuntimeError` (the mapping of src/lib.rs:670-694).
#include <pybind11/chrono.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <csignal>
#include <cstring>
#include <iostream>

#include "lighthouse.h"
#include "log.h"
#include "manager.h"
#include "quorum.h"

namespace py = pybind11;
using namespace ftcp;

namespace {

Millis to_ms(std::chrono::duration<double> d) { return Millis(static_cast<int64_t>(d.count() * 1000.0)); }

struct PyQuorumMember {
  std::string replica_id, address, store_address;
  int64_t step = 0;
  uint64_t world_size = 0;
  bool shrink_only = false;
  int64_t commit_failures = 0;
  py::object data = py::none();
};

struct PyTimestamp {
  int64_t seconds = 0;
  int32_t nanos = 0;
};

struct PyQuorum {
  int64_t quorum_id = 0;
  std::vector<PyQuorumMember> participants;
  PyTimestamp created;
};

PyQuorumMember to_py(const QuorumMember& m) {
  PyQuorumMember p;
  p.replica_id = m.replica_id;
  p.address = m.address;
  p.store_address = m.store_address;
  p.step = m.step;
  p.world_size = m.world_size;
  p.shrink_only = m.shrink_only;
  p.commit_failures = m.commit_failures;
  if (!m.data.empty()) {
    try {
      p.data = py::module_::import("json").attr("loads")(m.data);
    } catch (py::error_already_set&) {
      p.data = py::none();
    }
  }
  return p;
}

QuorumMember from_py(const PyQuorumMember& p) {
  QuorumMember m;
  m.replica_id = p.replica_id;
  m.address = p.address;
  m.store_address = p.store_address;
  m.step = p.step;
  m.world_size = p.world_size;
  m.shrink_only = p.shrink_only;
  m.commit_failures = p.commit_failures;
  if (!p.data.is_none()) m.data = py::module_::import("json").attr("dumps")(p.data).cast<std::string>();
  return m;
}

PyQuorum to_py(const Quorum& q) {
  PyQuorum p;
  p.quorum_id = q.quorum_id;
  for (const auto& m : q.participants) p.participants.push_back(to_py(m));
  p.created.seconds = q.created_seconds;
  p.created.nanos = q.created_nanos;
  return p;
}

class PyManagerClient {
 public:
  PyManagerClient(const std::string& addr, std::chrono::duration<double> connect_timeout) {
    py::gil_scoped_release nogil;
    client_ = std::make_unique<Client>(addr, to_ms(connect_timeout));
  }
  ManagerQuorumResponse quorum(int64_t group_rank, int64_t step, const std::string& checkpoint_metadata, bool shrink_only,
                               std::chrono::duration<double> timeout, bool init_sync, int64_t commit_failures) {
    ManagerQuorumRequest req;
    req.group_rank = group_rank;
    req.step = step;
    req.checkpoint_metadata = checkpoint_metadata;
    req.shrink_only = shrink_only;
    req.init_sync = init_sync;
    req.commit_failures = commit_failures;
    py::gil_scoped_release nogil;
    return ManagerQuorumResponse::decode(client_->call(kManagerQuorum, req.encode(), to_ms(timeout)));
  }
  std::string checkpoint_metadata(int64_t rank, std::chrono::duration<double> timeout) {
    py::gil_scoped_release nogil;
    return decode_str1(client_->call(kManagerCheckpointMetadata, encode_i64_1(rank), to_ms(timeout)));
  }
  bool should_commit(int64_t group_rank, int64_t step, bool vote, std::chrono::duration<double> timeout) {
    ShouldCommitRequest req;
    req.group_rank = group_rank;
    req.step = step;
    req.should_commit = vote;
    py::gil_scoped_release nogil;
    return decode_i64_1(client_->call(kManagerShouldCommit, req.encode(), to_ms(timeout))) != 0;
  }
  void kill(const std::string& msg, std::chrono::duration<double> timeout) {
    py::gil_scoped_release nogil;
    try {
      client_->call(kManagerKill, encode_str1(msg), to_ms(timeout));
    } catch (const RpcError&) {
      // the server exits inside the handler
    }
  }

 private:
  std::unique_ptr<Client> client_;
};

class PyLighthouseClient {
 public:
  PyLighthouseClient(const std::string& addr, std::chrono::duration<double> connect_timeout) {
    py::gil_scoped_release nogil;
    client_ = std::make_unique<Client>(addr, to_ms(connect_timeout));
  }
  PyQuorum quorum(const std::string& replica_id, std::chrono::duration<double> timeout, py::object address,
                  py::object store_address, py::object step, py::object world_size, py::object shrink_only,
                  py::object data) {
    QuorumMember m;
    m.replica_id = replica_id;
    if (!address.is_none()) m.address = address.cast<std::string>();
    if (!store_address.is_none()) m.store_address = store_address.cast<std::string>();
    if (!step.is_none()) m.step = step.cast<int64_t>();
    if (!world_size.is_none()) m.world_size = world_size.cast<uint64_t>();
    if (!shrink_only.is_none()) m.shrink_only = shrink_only.cast<bool>();
    if (!data.is_none()) m.data = py::module_::import("json").attr("dumps")(data).cast<std::string>();
    std::string resp;
    {
      py::gil_scoped_release nogil;
      resp = client_->call(kLighthouseQuorum, encode_msg1(m.encode()), to_ms(timeout));
    }
    Reader r(resp);
    int f, wt;
    Quorum q;
    while (r.next(&f, &wt)) {
      if (f == 1 && wt == 2) q = Quorum::decode(r.bytes());
      else r.skip(wt);
    }
    return to_py(q);
  }
  void heartbeat(const std::string& replica_id, std::chrono::duration<double> timeout) {
    py::gil_scoped_release nogil;
    client_->call(kLighthouseHeartbeat, encode_str1(replica_id), to_ms(timeout));
  }

 private:
  std::unique_ptr<Client> client_;
};

int lighthouse_main(std::vector<std::string> argv) {
  LighthouseOpt opt;
  bool have_min = false;
  auto need = [&](size_t i) {
    if (i + 1 >= argv.size()) throw std::runtime_error("missing value for " + argv[i]);
    return argv[i + 1];
  };
  for (size_t i = 1; i < argv.size(); ++i) {
    std::string a = argv[i], v;
    const size_t eq = a.find('=');
    bool inline_val = false;
    if (a.rfind("--", 0) == 0 && eq != std::string::npos) {
      v = a.substr(eq + 1);
      a = a.substr(0, eq);
      inline_val = true;
    }
    auto val = [&] {
      if (inline_val) return v;
      std::string r = need(i);
      ++i;
      return r;
    };
    if (a == "--bind") opt.bind = val();
    else if (a == "--join_timeout_ms" || a == "--join-timeout-ms") opt.join_timeout_ms = std::stoll(val());
    else if (a == "--min_replicas" || a == "--min-replicas") { opt.min_replicas = std::stoull(val()); have_min = true; }
    else if (a == "--quorum_tick_ms" || a == "--quorum-tick-ms") opt.quorum_tick_ms = std::stoll(val());
    else if (a == "--heartbeat_timeout_ms" || a == "--heartbeat-timeout-ms") opt.heartbeat_timeout_ms = std::stoll(val());
    else if (a == "-h" || a == "--help") {
      std::cout << "torchft_b200 lighthouse\n  --bind <addr> (default [::]:29510)\n  --min_replicas <n> (required)\n"
                   "  --join_timeout_ms <ms> (default 60000)\n  --quorum_tick_ms <ms> (default 100)\n"
                   "  --heartbeat_timeout_ms <ms> (default 5000)\n";
      return 0;
    } else {
      throw std::runtime_error("unknown argument " + a);
    }
  }
  if (!have_min) throw std::runtime_error("--min_replicas is required");
  Lighthouse lh(opt);
  std::cout << "lighthouse listening on " << lh.address() << std::endl;
  // run until interrupted; SIGINT keeps its default disposition so Ctrl-C ends the process
  std::signal(SIGINT, SIG_DFL);
  while (true) std::this_thread::sleep_for(std::chrono::seconds(3600));
  return 0;
}

}  // namespace

PYBIND11_MODULE(_ftcp, m) {
  m.doc() = "torchft_b200 control plane (C++): lighthouse, manager server/client, quorum math";

  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const TimeoutError& e) {
      PyErr_SetString(PyExc_TimeoutError, e.what());
    } catch (const RpcError& e) {
      PyErr_SetString(PyExc_RuntimeError, e.what());
    } catch (const WireError& e) {
      PyErr_SetString(PyExc_RuntimeError, e.what());
    }
  });

  py::class_<ManagerQuorumResponse>(m, "QuorumResult", R"doc(What one rank learns from a quorum round.

Args (all read/write attributes; the constructor takes none):
    quorum_id: changes whenever the set of replica groups changes or a member reported failed commits
    replica_rank, replica_world_size: this group's index among the quorum's groups and their number
    recover_src_manager_address, recover_src_replica_rank: where a group that is behind fetches its state
    recover_dst_replica_ranks: groups this rank must serve state to
    store_address: store on which the replica process group of this quorum rendezvouses
    max_step, max_replica_rank, max_world_size: the most advanced step, this group's index among the groups
        at that step (None when behind) and their number
    heal: True when this group must fetch state before it can contribute
    commit_failures: largest number of consecutive failed commits reported by a member
)doc")
      .def(py::init<>())
      .def_readwrite("quorum_id", &ManagerQuorumResponse::quorum_id)
      .def_readwrite("replica_rank", &ManagerQuorumResponse::replica_rank)
      .def_readwrite("replica_world_size", &ManagerQuorumResponse::replica_world_size)
      .def_readwrite("recover_src_manager_address", &ManagerQuorumResponse::recover_src_manager_address)
      .def_readwrite("recover_src_replica_rank", &ManagerQuorumResponse::recover_src_replica_rank)
      .def_readwrite("recover_dst_replica_ranks", &ManagerQuorumResponse::recover_dst_replica_ranks)
      .def_readwrite("store_address", &ManagerQuorumResponse::store_address)
      .def_readwrite("max_step", &ManagerQuorumResponse::max_step)
      .def_readwrite("max_replica_rank", &ManagerQuorumResponse::max_replica_rank)
      .def_readwrite("max_world_size", &ManagerQuorumResponse::max_world_size)
      .def_readwrite("heal", &ManagerQuorumResponse::heal)
      .def_readwrite("commit_failures", &ManagerQuorumResponse::commit_failures);

  py::class_<PyQuorumMember>(m, "QuorumMember", R"doc(One replica group as the lighthouse sees it.

Args:
    replica_id: unique name of the group (a fresh suffix per process start)
    address: address of the group's manager server
    store_address: address of the group's store
    step: committed steps of the group
    world_size: ranks in the group
    shrink_only: the group asks that the next quorum does not grow
    data: free-form dict that is carried through the quorum as JSON
    commit_failures: consecutive failed commits the group reports
)doc")
      .def(py::init([](std::string replica_id, std::string address, std::string store_address, int64_t step,
                       uint64_t world_size, bool shrink_only, py::object data, int64_t commit_failures) {
             PyQuorumMember q;
             q.replica_id = std::move(replica_id);
             q.address = std::move(address);
             q.store_address = std::move(store_address);
             q.step = step;
             q.world_size = world_size;
             q.shrink_only = shrink_only;
             q.data = std::move(data);
             q.commit_failures = commit_failures;
             return q;
           }),
           py::arg("replica_id"), py::arg("address") = "", py::arg("store_address") = "", py::arg("step") = 0,
           py::arg("world_size") = 0, py::arg("shrink_only") = false, py::arg("data") = py::none(),
           py::arg("commit_failures") = 0)
      .def_readwrite("replica_id", &PyQuorumMember::replica_id)
      .def_readwrite("address", &PyQuorumMember::address)
      .def_readwrite("store_address", &PyQuorumMember::store_address)
      .def_readwrite("step", &PyQuorumMember::step)
      .def_readwrite("world_size", &PyQuorumMember::world_size)
      .def_readwrite("shrink_only", &PyQuorumMember::shrink_only)
      .def_readwrite("commit_failures", &PyQuorumMember::commit_failures)
      .def_readwrite("data", &PyQuorumMember::data);

  py::class_<PyTimestamp>(m, "Timestamp", R"doc(Wall-clock time of an event.

Args (attributes):
    seconds: seconds since the Unix epoch
    nanos: nanoseconds within the second
)doc")
      .def(py::init<>())
      .def_readwrite("seconds", &PyTimestamp::seconds)
      .def_readwrite("nanos", &PyTimestamp::nanos);

  py::class_<PyQuorum>(m, "Quorum", R"doc(A quorum as issued by the lighthouse.

Args (attributes):
    quorum_id: identifier of the quorum
    participants: list of QuorumMember, sorted by replica_id
    created: Timestamp of the decision
)doc")
      .def(py::init<>())
      .def_readwrite("quorum_id", &PyQuorum::quorum_id)
      .def_readwrite("participants", &PyQuorum::participants)
      .def_readwrite("created", &PyQuorum::created);

  py::class_<PyManagerClient>(m, "ManagerClient", R"doc(Client of a replica group's manager server, one per rank.

Args:
    addr: address of the manager server, e.g. http://host:port
    connect_timeout: timedelta bound on establishing the connection

A call whose deadline passes raises TimeoutError, any other failure RuntimeError; the GIL is released while a call blocks.
)doc")
      .def(py::init<const std::string&, std::chrono::duration<double>>(), py::arg("addr"), py::arg("connect_timeout"))
      .def("_quorum", &PyManagerClient::quorum, py::arg("group_rank"), py::arg("step"), py::arg("checkpoint_metadata"),
           py::arg("shrink_only"), py::arg("timeout"), py::arg("init_sync") = true, py::arg("commit_failures") = 0)
      .def("_checkpoint_metadata", &PyManagerClient::checkpoint_metadata, py::arg("rank"), py::arg("timeout"))
      .def("should_commit", &PyManagerClient::should_commit, py::arg("group_rank"), py::arg("step"),
           py::arg("should_commit"), py::arg("timeout"))
      .def("_kill", &PyManagerClient::kill, py::arg("msg"), py::arg("timeout"));

  py::class_<ManagerServer>(m, "ManagerServer", R"doc(The per-group manager server (hosted by the group's rank 0): gathers the quorum requests of the group's
ranks into one lighthouse request, hands each rank its share of the answer, runs the commit barrier, keeps the ranks'
checkpoint metadata and sends heartbeats.

Args:
    replica_id: name of the replica group
    lighthouse_addr: address of the lighthouse
    hostname: host name other groups use to reach this server
    bind: address to listen on, e.g. [::]:0
    store_addr: address of the group's store, published to the other groups
    world_size: ranks in the group
    heartbeat_interval: timedelta between heartbeats to the lighthouse
    connect_timeout: timedelta bound on connecting to the lighthouse
    quorum_retries: extra attempts at the lighthouse inside one quorum call
)doc")
      .def(py::init([](const std::string& replica_id, const std::string& lighthouse_addr, const std::string& hostname,
                       const std::string& bind, const std::string& store_addr, uint64_t world_size,
                       std::chrono::duration<double> heartbeat_interval, std::chrono::duration<double> connect_timeout,
                       int64_t quorum_retries) {
             py::gil_scoped_release nogil;
             return std::make_unique<ManagerServer>(replica_id, lighthouse_addr, hostname, bind, store_addr, world_size,
                                                    to_ms(heartbeat_interval), to_ms(connect_timeout), quorum_retries);
           }),
           py::arg("replica_id"), py::arg("lighthouse_addr"), py::arg("hostname"), py::arg("bind"), py::arg("store_addr"),
           py::arg("world_size"), py::arg("heartbeat_interval"), py::arg("connect_timeout"), py::arg("quorum_retries") = 0)
      .def("address", &ManagerServer::address)
      .def("shutdown", &ManagerServer::shutdown, py::call_guard<py::gil_scoped_release>());

  py::class_<Lighthouse>(m, "LighthouseServer", R"doc(The job-wide quorum service, with the dashboard on the same port.

Args:
    bind: address to listen on, e.g. [::]:29510
    min_replicas: smallest number of groups a quorum may have
    join_timeout_ms: how long a quorum waits for healthy groups that have not asked yet (default 100)
    quorum_tick_ms: period of the background quorum check (default 100)
    heartbeat_timeout_ms: silence after which a group no longer counts as healthy (default 5000)
)doc")
      .def(py::init([](const std::string& bind, uint64_t min_replicas, std::optional<int64_t> join_timeout_ms,
                       std::optional<int64_t> quorum_tick_ms, std::optional<int64_t> heartbeat_timeout_ms) {
             LighthouseOpt opt;
             opt.bind = bind;
             opt.min_replicas = min_replicas;
             opt.join_timeout_ms = join_timeout_ms.value_or(100);
             opt.quorum_tick_ms = quorum_tick_ms.value_or(100);
             opt.heartbeat_timeout_ms = heartbeat_timeout_ms.value_or(5000);
             py::gil_scoped_release nogil;
             return std::make_unique<Lighthouse>(opt);
           }),
           py::arg("bind"), py::arg("min_replicas"), py::arg("join_timeout_ms") = py::none(),
           py::arg("quorum_tick_ms") = py::none(), py::arg("heartbeat_timeout_ms") = py::none())
      .def("address", &Lighthouse::address)
      .def("shutdown", &Lighthouse::shutdown, py::call_guard<py::gil_scoped_release>());

  py::class_<PyLighthouseClient>(m, "LighthouseClient", R"doc(Direct client of the lighthouse, for launchers and tools that take part in quorums without a manager.

Args:
    addr: address of the lighthouse, e.g. http://host:29510
    connect_timeout: timedelta bound on establishing the connection
)doc")
      .def(py::init<const std::string&, std::chrono::duration<double>>(), py::arg("addr"), py::arg("connect_timeout"))
      .def("quorum", &PyLighthouseClient::quorum, py::arg("replica_id"), py::arg("timeout"),
           py::arg("address") = py::none(), py::arg("store_address") = py::none(), py::arg("step") = py::none(),
           py::arg("world_size") = py::none(), py::arg("shrink_only") = py::none(), py::arg("data") = py::none())
      .def("heartbeat", &PyLighthouseClient::heartbeat, py::arg("replica_id"),
           py::arg("timeout") = std::chrono::duration<double>(5.0));

  m.def(
      "lighthouse_main",
      [](std::optional<std::vector<std::string>> argv) {
        std::vector<std::string> args;
        if (argv) args = *argv;
        else args = py::module_::import("sys").attr("argv").cast<std::vector<std::string>>();
        py::gil_scoped_release nogil;
        return lighthouse_main(args);
      },
      py::arg("argv") = py::none(),
      R"doc(Run a lighthouse until it is interrupted; returns the process exit code.

Args:
    argv: program name followed by --bind, --min_replicas, --join_timeout_ms, --quorum_tick_ms,
        --heartbeat_timeout_ms (sys.argv when None)
)doc");

  // ---- pure functions, exposed for table-driven tests of the quorum mathematics ----
  m.def(
      "quorum_compute",
      [](double now_s, const std::vector<std::pair<PyQuorumMember, double>>& participants,
         const std::map<std::string, double>& heartbeats, std::optional<PyQuorum> prev_quorum, uint64_t min_replicas,
         int64_t join_timeout_ms, int64_t heartbeat_timeout_ms) {
        // times are seconds on an arbitrary axis; mapped onto the steady clock
        const TimePoint base = Clock::now();
        auto tp = [&](double s) { return base + std::chrono::duration_cast<Clock::duration>(std::chrono::duration<double>(s - now_s)); };
        LighthouseState st;
        for (const auto& [mem, joined] : participants) st.participants[mem.replica_id] = ParticipantDetails{tp(joined), from_py(mem)};
        for (const auto& [id, t] : heartbeats) st.heartbeats[id] = tp(t);
        if (prev_quorum) {
          Quorum q;
          q.quorum_id = prev_quorum->quorum_id;
          for (const auto& p : prev_quorum->participants) q.participants.push_back(from_py(p));
          st.prev_quorum = q;
        }
        LighthouseOpt opt;
        opt.min_replicas = min_replicas;
        opt.join_timeout_ms = join_timeout_ms;
        opt.heartbeat_timeout_ms = heartbeat_timeout_ms;
        auto [members, reason] = quorum_compute(base, st, opt);
        py::object out = py::none();
        if (members) {
          std::vector<PyQuorumMember> v;
          for (const auto& mm : *members) v.push_back(to_py(mm));
          out = py::cast(v);
        }
        return py::make_tuple(out, reason);
      },
      py::arg("now"), py::arg("participants"), py::arg("heartbeats"), py::arg("prev_quorum") = py::none(),
      py::arg("min_replicas") = 1, py::arg("join_timeout_ms") = 60000, py::arg("heartbeat_timeout_ms") = 5000);

  m.def(
      "compute_quorum_results",
      [](const std::string& replica_id, int64_t group_rank, const PyQuorum& quorum, bool init_sync) {
        Quorum q;
        q.quorum_id = quorum.quorum_id;
        for (const auto& p : quorum.participants) q.participants.push_back(from_py(p));
        return compute_quorum_results(replica_id, group_rank, q, init_sync);
      },
      py::arg("replica_id"), py::arg("group_rank"), py::arg("quorum"), py::arg("init_sync") = true);

  m.def("quorum_changed", [](const std::vector<PyQuorumMember>& a, const std::vector<PyQuorumMember>& b) {
    std::vector<QuorumMember> ca, cb;
    for (const auto& x : a) ca.push_back(from_py(x));
    for (const auto& x : b) cb.push_back(from_py(x));
    return quorum_changed(ca, cb);
  });
}
