// Native executor: replays a static op graph once per serving iteration.
//
// An op is a kernel entry point of libnanoflow_kernels.so in the uniform
// `int fn(const void* params, cudaStream_t)` form, a copy of its parameter block, the stream class
// it runs on, the ops whose completion (or start) it waits for, and a list of patches: integer
// fields of the parameter block that are overwritten from the iteration's symbol table right
// before the launch (token counts, request ranges, staging-slot pointers). A worker thread bound to
// the GPU issues the iteration, so the Python scheduler forms the next batch while this one is
// being launched; `wait(ticket)` blocks until the GPU has finished that iteration.
//
// Dependencies across streams are CUDA events; ops on one stream rely on stream order. The seven
// stream classes (gemm, attn, net, other, copy, attn2, net2) fork from and join back into the caller's main
// stream, so consecutive iterations stay ordered and torch work queued on that stream composes.
//
// Graph mode (set_graph_mode): after two plain iterations the same issue sequence is recorded by
// stream capture on a private stream, the executable graph of the previous iteration is updated
// in place with the new parameters (cudaGraphExecUpdate; re-instantiated if the topology changed)
// and launched on the main stream as one unit. The parameter blocks are passed by value, so an
// iteration whose token counts differ is still one update, not a rebuild.
//
// This takes the place of the reference's per-GPU Worker thread + hand-written Pipeline::run
// (pipeline/src/computeBound.cu:163-193, :255-290; pipeline/src/pipeline.cu:599-789) and of its
// OperatorWrapper run/wait/wait_for_start event plumbing (pipeline/include/operatorWrapper.cuh:98-144).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#ifdef NF_HOST_CUDA
#include "host_cuda.h"   // host-only build: the runtime calls are logged instead of made
#else
#include <cuda_runtime.h>
#endif

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

constexpr int kNumStreamClasses = 7;
constexpr int kTickets = 8;

using LaunchFn = int (*)(const void*, cudaStream_t);

struct Patch {
  uint32_t offset;
  uint32_t sym;
  uint32_t nbytes;  // 4 or 8
};

struct Op {
  std::string name;
  LaunchFn fn = nullptr;
  std::vector<uint8_t> params;
  int stream_class = 0;
  std::vector<int> deps;
  std::vector<int> after_start;
  std::vector<Patch> patches;
  cudaEvent_t end_event = nullptr;
  cudaEvent_t start_event = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;  // timing (only in timed runs)
};

struct Job {
  uint64_t ticket;
  std::vector<int64_t> syms;
  bool timed;
};

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

class Executor {
 public:
  Executor(uintptr_t main_stream, int device, bool single_stream, int num_symbols)
      : main_(reinterpret_cast<cudaStream_t>(main_stream)), device_(device),
        single_stream_(single_stream), num_symbols_(num_symbols) {
    check(cudaSetDevice(device_), "cudaSetDevice");
    for (int i = 0; i < kNumStreamClasses; ++i) {
      if (single_stream_) {
        streams_[i] = main_;
      } else {
        check(cudaStreamCreateWithFlags(&streams_[i], cudaStreamNonBlocking), "cudaStreamCreate");
      }
      check(cudaEventCreateWithFlags(&join_[i], cudaEventDisableTiming), "cudaEventCreate");
    }
    check(cudaEventCreateWithFlags(&fork_, cudaEventDisableTiming), "cudaEventCreate");
    for (int i = 0; i < kTickets; ++i)
      check(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming), "cudaEventCreate");
    worker_ = std::thread([this] { this->loop(); });
  }

  ~Executor() { close(); }

  void close() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
    cudaSetDevice(device_);
    for (auto& op : ops_) {
      if (op.end_event) cudaEventDestroy(op.end_event);
      if (op.start_event) cudaEventDestroy(op.start_event);
      if (op.t0) cudaEventDestroy(op.t0);
      if (op.t1) cudaEventDestroy(op.t1);
    }
    if (exec_) cudaGraphExecDestroy(exec_);
    if (cap_) cudaStreamDestroy(cap_);
    if (!single_stream_)
      for (int i = 0; i < kNumStreamClasses; ++i) cudaStreamDestroy(streams_[i]);
    for (int i = 0; i < kNumStreamClasses; ++i) cudaEventDestroy(join_[i]);
    cudaEventDestroy(fork_);
    for (int i = 0; i < kTickets; ++i) cudaEventDestroy(done_[i]);
  }

  int add_op(const std::string& name, uintptr_t fn, const py::bytes& params, int stream_class,
             const std::vector<int>& deps, const std::vector<int>& after_start,
             const std::vector<std::tuple<int, int, int>>& patches) {
    if (frozen_) throw std::runtime_error("add_op after the first run");
    if (stream_class < 0 || stream_class >= kNumStreamClasses) throw std::runtime_error("bad stream class");
    Op op;
    op.name = name;
    op.fn = reinterpret_cast<LaunchFn>(fn);
    std::string raw = params;
    op.params.assign(raw.begin(), raw.end());
    op.stream_class = stream_class;
    const int idx = static_cast<int>(ops_.size());
    for (int d : deps) {
      if (d < 0 || d >= idx) throw std::runtime_error("dependency must be an earlier op");
      op.deps.push_back(d);
    }
    for (int d : after_start) {
      if (d < 0 || d >= idx) throw std::runtime_error("dependency must be an earlier op");
      op.after_start.push_back(d);
    }
    for (auto& t : patches) {
      Patch p{static_cast<uint32_t>(std::get<0>(t)), static_cast<uint32_t>(std::get<1>(t)),
              static_cast<uint32_t>(std::get<2>(t))};
      if ((p.nbytes != 4 && p.nbytes != 8) || p.offset + p.nbytes > op.params.size() ||
          static_cast<int>(p.sym) >= num_symbols_)
        throw std::runtime_error("bad patch for op " + name);
      op.patches.push_back(p);
    }
    ops_.push_back(std::move(op));
    return idx;
  }

  // Create the events the dependency edges need. Called once, before the first run.
  void freeze() {
    if (frozen_) return;
    check(cudaSetDevice(device_), "cudaSetDevice");
    for (auto& op : ops_) {
      for (int d : op.deps)
        if (!single_stream_ && ops_[d].stream_class != op.stream_class && !ops_[d].end_event)
          check(cudaEventCreateWithFlags(&ops_[d].end_event, cudaEventDisableTiming), "cudaEventCreate");
      for (int d : op.after_start)
        if (!single_stream_ && !ops_[d].start_event)
          check(cudaEventCreateWithFlags(&ops_[d].start_event, cudaEventDisableTiming), "cudaEventCreate");
    }
    frozen_ = true;
  }

  uint64_t submit(const std::vector<int64_t>& syms, bool timed) {
    if (static_cast<int>(syms.size()) != num_symbols_) throw std::runtime_error("symbol table size mismatch");
    freeze();
    std::unique_lock<std::mutex> lk(mu_);
    if (!error_.empty()) throw std::runtime_error(error_);
    if (next_ticket_ - completed_waits_ >= kTickets) throw std::runtime_error("too many iterations in flight");
    const uint64_t t = next_ticket_++;
    queue_.push_back(Job{t, syms, timed});
    lk.unlock();
    cv_.notify_all();
    return t;
  }

  // Block until iteration `ticket` has been issued and the GPU has finished it.
  void wait(uint64_t ticket) {
    {
      py::gil_scoped_release nogil;
      std::unique_lock<std::mutex> lk(mu_);
      issued_cv_.wait(lk, [&] { return issued_ > ticket || !error_.empty() || stop_; });
      if (error_.empty() && !stop_) {
        lk.unlock();
        cudaSetDevice(device_);
        cudaError_t e = cudaEventSynchronize(done_[ticket % kTickets]);
        lk.lock();
        if (e != cudaSuccess && error_.empty()) error_ = std::string("cudaEventSynchronize: ") + cudaGetErrorString(e);
      }
      completed_waits_ = std::max(completed_waits_, ticket + 1);
    }
    std::lock_guard<std::mutex> lk(mu_);
    if (!error_.empty()) throw std::runtime_error(error_);
  }

  // Per-op (name, stream class, start_us, end_us) of the last timed iteration; call after wait().
  std::vector<std::tuple<std::string, int, double, double>> timeline() {
    std::vector<std::tuple<std::string, int, double, double>> out;
    cudaSetDevice(device_);
    cudaEvent_t base = nullptr;
    for (auto& op : ops_)
      if (op.t0) { base = op.t0; break; }
    if (!base) return out;
    for (auto& op : ops_) {
      if (!op.t0 || !op.t1) continue;
      float a = 0.f, b = 0.f;
      if (cudaEventElapsedTime(&a, base, op.t0) != cudaSuccess) continue;
      if (cudaEventElapsedTime(&b, base, op.t1) != cudaSuccess) continue;
      out.emplace_back(op.name, op.stream_class, a * 1e3, b * 1e3);
    }
    return out;
  }

  void set_graph_mode(bool on) { graph_mode_ = on; }
  uint64_t graph_launches() const { return graph_launches_.load(); }
  uint64_t graph_rebuilds() const { return graph_rebuilds_.load(); }

  int num_ops() const { return static_cast<int>(ops_.size()); }
  uint64_t launches() const { return launches_.load(); }

 private:
  void loop() {
    cudaSetDevice(device_);
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !queue_.empty(); });
        if (stop_ && queue_.empty()) return;
        job = std::move(queue_.front());
        queue_.pop_front();
      }
      std::string err;
      try {
        issue(job);
      } catch (const std::exception& e) {
        err = e.what();
      }
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (!err.empty() && error_.empty()) error_ = err;
        issued_ = job.ticket + 1;
      }
      issued_cv_.notify_all();
    }
  }

  void issue(const Job& job) {
    if (graph_mode_ && !job.timed && plain_iterations_ >= 2) {
      issue_graph(job);
    } else {
      issue_ops(job, main_);
      ++plain_iterations_;
    }
    check(cudaEventRecord(done_[job.ticket % kTickets], main_), "record(done)");
  }

  // Record the iteration on the capture stream and run it on the main stream as one graph launch.
  void issue_graph(const Job& job) {
    if (!cap_) check(cudaStreamCreateWithFlags(&cap_, cudaStreamNonBlocking), "cudaStreamCreate(capture)");
    check(cudaStreamBeginCapture(cap_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    cudaGraph_t graph = nullptr;
    try {
      issue_ops(job, cap_);
    } catch (...) {
      cudaStreamEndCapture(cap_, &graph);
      if (graph) cudaGraphDestroy(graph);
      throw;
    }
    check(cudaStreamEndCapture(cap_, &graph), "cudaStreamEndCapture");
    bool ok = false;
    if (exec_) {
      cudaGraphExecUpdateResultInfo info;
      ok = cudaGraphExecUpdate(exec_, graph, &info) == cudaSuccess;
      if (!ok) {
        (void)cudaGetLastError();
        cudaGraphExecDestroy(exec_);
        exec_ = nullptr;
      }
    }
    if (!ok) {
      cudaError_t e = cudaGraphInstantiate(&exec_, graph, 0);
      if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        exec_ = nullptr;
        check(e, "cudaGraphInstantiate");
      }
      graph_rebuilds_.fetch_add(1);
    }
    cudaGraphDestroy(graph);
    check(cudaGraphLaunch(exec_, main_), "cudaGraphLaunch");
    graph_launches_.fetch_add(1);
  }

  // The iteration's launches, forked from and joined back into `origin`.
  void issue_ops(const Job& job, cudaStream_t origin) {
    if (!single_stream_) {
      check(cudaEventRecord(fork_, origin), "cudaEventRecord(fork)");
      for (int i = 0; i < kNumStreamClasses; ++i) check(cudaStreamWaitEvent(streams_[i], fork_, 0), "wait(fork)");
    }
    bool used[kNumStreamClasses] = {};
    for (auto& op : ops_) {
      cudaStream_t st = single_stream_ ? origin : streams_[op.stream_class];
      used[op.stream_class] = true;
      for (const Patch& p : op.patches) {
        const int64_t v = job.syms[p.sym];
        if (p.nbytes == 4) {
          const int32_t v32 = static_cast<int32_t>(v);
          std::memcpy(op.params.data() + p.offset, &v32, 4);
        } else {
          std::memcpy(op.params.data() + p.offset, &v, 8);
        }
      }
      if (!single_stream_) {
        for (int d : op.deps)
          if (ops_[d].end_event && ops_[d].stream_class != op.stream_class)
            check(cudaStreamWaitEvent(st, ops_[d].end_event, 0), "wait(dep)");
        for (int d : op.after_start)
          if (ops_[d].start_event) check(cudaStreamWaitEvent(st, ops_[d].start_event, 0), "wait(start)");
      }
      if (op.start_event) check(cudaEventRecord(op.start_event, st), "record(start)");
      if (job.timed) {
        if (!op.t0) {
          check(cudaEventCreate(&op.t0), "cudaEventCreate");
          check(cudaEventCreate(&op.t1), "cudaEventCreate");
        }
        check(cudaEventRecord(op.t0, st), "record(t0)");
      }
#ifdef NF_HOST_CUDA
      host_cuda::note_launch(st, static_cast<int>(&op - ops_.data()), op.params);
#endif
      const int rc = op.fn(op.params.data(), st);
      if (rc != 0) throw std::runtime_error("op " + op.name + " rejected its arguments (code " + std::to_string(rc) + ")");
      launches_.fetch_add(1);
      if (job.timed) check(cudaEventRecord(op.t1, st), "record(t1)");
      if (op.end_event) check(cudaEventRecord(op.end_event, st), "record(end)");
    }
    if (!single_stream_) {
      for (int i = 0; i < kNumStreamClasses; ++i) {
        if (!used[i] && origin == main_) continue;   // under capture every forked stream must join back
        check(cudaEventRecord(join_[i], streams_[i]), "record(join)");
        check(cudaStreamWaitEvent(origin, join_[i], 0), "wait(join)");
      }
    }
  }

  cudaStream_t main_;
  int device_;
  bool single_stream_;
  int num_symbols_;
  cudaStream_t streams_[kNumStreamClasses];
  cudaEvent_t join_[kNumStreamClasses];
  cudaEvent_t fork_ = nullptr;
  cudaEvent_t done_[kTickets];
  std::vector<Op> ops_;
  bool frozen_ = false;

  std::mutex mu_;
  std::condition_variable cv_, issued_cv_;
  std::deque<Job> queue_;
  uint64_t next_ticket_ = 0, issued_ = 0, completed_waits_ = 0;
  bool stop_ = false;
  std::string error_;
  std::thread worker_;
  std::atomic<uint64_t> launches_{0};
  bool graph_mode_ = false;
  int plain_iterations_ = 0;
  cudaStream_t cap_ = nullptr;
  cudaGraphExec_t exec_ = nullptr;
  std::atomic<uint64_t> graph_launches_{0}, graph_rebuilds_{0};
};

}  // namespace

#ifndef NF_EXECUTOR_MODULE
#define NF_EXECUTOR_MODULE _executor
#endif

PYBIND11_MODULE(NF_EXECUTOR_MODULE, m) {
  m.doc() = "Native op-graph executor (one worker thread per GPU)";
#ifdef NF_HOST_CUDA
  // Host-only build: the log of runtime calls, and a launch function that does nothing.
  m.attr("host_only") = true;
  m.def("noop_fn", [] { return reinterpret_cast<uintptr_t>(&host_cuda::noop_launch); });
  m.def("failing_fn", [] { return reinterpret_cast<uintptr_t>(&host_cuda::failing_launch); });
  m.def("host_log", [] {
    std::lock_guard<std::mutex> lk(host_cuda::state().mu);
    py::list out;
    for (const auto& r : host_cuda::state().log)
      out.append(py::make_tuple(r.kind, r.stream, r.event, r.op, r.captured, py::bytes(r.params)));
    return out;
  });
  m.def("host_log_clear", [] {
    std::lock_guard<std::mutex> lk(host_cuda::state().mu);
    host_cuda::state().log.clear();
  });
  m.def("fail_next_graph_update", [] {
    std::lock_guard<std::mutex> lk(host_cuda::state().mu);
    host_cuda::state().fail_next_update = true;
  });
#endif
  py::class_<Executor>(m, "Executor")
      .def(py::init<uintptr_t, int, bool, int>(), py::arg("main_stream"), py::arg("device"),
           py::arg("single_stream"), py::arg("num_symbols"))
      .def("add_op", &Executor::add_op)
      .def("freeze", &Executor::freeze)
      .def("submit", &Executor::submit, py::arg("syms"), py::arg("timed") = false)
      .def("wait", &Executor::wait)
      .def("timeline", &Executor::timeline)
      .def("num_ops", &Executor::num_ops)
      .def("launches", &Executor::launches)
      .def("set_graph_mode", &Executor::set_graph_mode)
      .def("graph_launches", &Executor::graph_launches)
      .def("graph_rebuilds", &Executor::graph_rebuilds)
      .def("close", &Executor::close);
}
