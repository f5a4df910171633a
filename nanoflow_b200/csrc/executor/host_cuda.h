// Stand-in for the CUDA runtime calls the executor makes, for a host-only build of the same source
// (-DNF_HOST_CUDA). Nothing runs on a device: every stream / event / graph call is appended to a
// process-wide log (kind, stream id, event id, op index, parameter bytes at launch), which a test
// turns back into the happens-before relation the calls imply and compares with the op graph's
// dependencies. Stream capture follows the runtime's rule that a stream which waits on an event
// recorded in a capturing stream joins the capture, so unjoined forks show up in the log.
//
// The reference has no host-only mode for its worker threads (pipeline/src/computeBound.cu:163-193);
// its event plumbing (pipeline/include/operatorWrapper.cuh:98-144) is only exercised on GPUs.
#pragma once

#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

enum cudaError_t { cudaSuccess = 0, cudaErrorInvalidValue = 1, cudaErrorGraphExecUpdateFailure = 910 };

struct HostStream {
  int id;
  bool capturing;
};
struct HostEvent {
  int id;
  bool captured;
  long long seq;
};
struct HostGraph {
  int nodes;
};
struct HostGraphExec {
  int nodes;
};
using cudaStream_t = HostStream*;
using cudaEvent_t = HostEvent*;
using cudaGraph_t = HostGraph*;
using cudaGraphExec_t = HostGraphExec*;
struct cudaGraphExecUpdateResultInfo {
  int result;
};
enum cudaStreamCaptureMode { cudaStreamCaptureModeGlobal = 0, cudaStreamCaptureModeThreadLocal = 1 };
constexpr unsigned int cudaStreamNonBlocking = 1u;
constexpr unsigned int cudaEventDisableTiming = 2u;

namespace host_cuda {

enum Kind {
  kLaunch = 0,
  kEventRecord = 1,
  kStreamWait = 2,
  kBeginCapture = 3,
  kEndCapture = 4,
  kGraphInstantiate = 5,
  kGraphUpdate = 6,
  kGraphLaunch = 7,
  kEventSync = 8,
};

struct Record {
  int kind;
  int stream;     // 0 = the caller's main stream (a null handle)
  int event;      // -1 when the call has none
  int op;         // op index for launches, node count for graph calls, else -1
  bool captured;  // issued into a stream capture instead of being run
  std::string params;
};

struct State {
  std::mutex mu;
  std::vector<Record> log;
  std::vector<HostStream*> streams;   // every live stream but the main one
  HostStream main{0, false};
  int next_stream = 1, next_event = 0;
  long long seq = 0;
  int captured_nodes = 0;
  bool fail_next_update = false;
};

inline State& state() {
  static State s;
  return s;
}
inline HostStream* resolve(cudaStream_t s) { return s ? s : &state().main; }

inline void push(int kind, cudaStream_t s, int event, int op, const std::string& params = std::string()) {
  State& st = state();
  HostStream* hs = resolve(s);
  if (hs->capturing && (kind == kLaunch || kind == kEventRecord || kind == kStreamWait)) ++st.captured_nodes;
  st.log.push_back(Record{kind, hs->id, event, op, hs->capturing, params});
  ++st.seq;
}

inline void note_launch(cudaStream_t s, int op, const std::vector<uint8_t>& params) {
  std::lock_guard<std::mutex> lk(state().mu);
  push(kLaunch, s, -1, op, std::string(params.begin(), params.end()));
}

inline int noop_launch(const void*, cudaStream_t) { return 0; }
inline int failing_launch(const void*, cudaStream_t) { return 3; }   // an op that rejects its arguments

}  // namespace host_cuda

inline const char* cudaGetErrorString(cudaError_t e) {
  return e == cudaSuccess ? "no error" : (e == cudaErrorGraphExecUpdateFailure ? "graph update failed" : "invalid value");
}
inline cudaError_t cudaGetLastError() { return cudaSuccess; }
inline cudaError_t cudaSetDevice(int) { return cudaSuccess; }

inline cudaError_t cudaStreamCreateWithFlags(cudaStream_t* s, unsigned int) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  *s = new HostStream{host_cuda::state().next_stream++, false};
  host_cuda::state().streams.push_back(*s);
  return cudaSuccess;
}
inline cudaError_t cudaStreamCreate(cudaStream_t* s) { return cudaStreamCreateWithFlags(s, 0); }
inline cudaError_t cudaStreamDestroy(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  auto& v = host_cuda::state().streams;
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i] == s) {
      v.erase(v.begin() + static_cast<long>(i));
      break;
    }
  delete s;
  return cudaSuccess;
}
inline cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned int) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  *e = new HostEvent{host_cuda::state().next_event++, false, -1};
  return cudaSuccess;
}
inline cudaError_t cudaEventCreate(cudaEvent_t* e) { return cudaEventCreateWithFlags(e, 0); }
inline cudaError_t cudaEventDestroy(cudaEvent_t e) {
  delete e;
  return cudaSuccess;
}
inline cudaError_t cudaEventRecord(cudaEvent_t e, cudaStream_t s) {
  if (!e) return cudaErrorInvalidValue;
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  e->captured = host_cuda::resolve(s)->capturing;
  e->seq = host_cuda::state().seq;
  host_cuda::push(host_cuda::kEventRecord, s, e->id, -1);
  return cudaSuccess;
}
inline cudaError_t cudaStreamWaitEvent(cudaStream_t s, cudaEvent_t e, unsigned int) {
  if (!e) return cudaErrorInvalidValue;
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  if (e->captured) host_cuda::resolve(s)->capturing = true;   // the waiting stream joins the capture
  host_cuda::push(host_cuda::kStreamWait, s, e->id, -1);
  return cudaSuccess;
}
inline cudaError_t cudaEventSynchronize(cudaEvent_t e) {
  if (!e) return cudaErrorInvalidValue;
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  host_cuda::state().log.push_back(host_cuda::Record{host_cuda::kEventSync, -1, e->id, -1, false, std::string()});
  return cudaSuccess;
}
inline cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t a, cudaEvent_t b) {
  if (!a || !b || a->seq < 0 || b->seq < 0) return cudaErrorInvalidValue;
  *ms = static_cast<float>(b->seq - a->seq) * 1e-3f;   // one log entry counts as a microsecond
  return cudaSuccess;
}

inline cudaError_t cudaStreamBeginCapture(cudaStream_t s, cudaStreamCaptureMode) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  host_cuda::state().captured_nodes = 0;
  host_cuda::push(host_cuda::kBeginCapture, s, -1, -1);
  host_cuda::resolve(s)->capturing = true;
  return cudaSuccess;
}
// Ends the capture on every stream that joined it. Whether all of them had been joined back into the
// origin is for the reader of the log to decide (the runtime refuses the capture otherwise).
inline cudaError_t cudaStreamEndCapture(cudaStream_t s, cudaGraph_t* g) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  host_cuda::state().main.capturing = false;
  for (HostStream* hs : host_cuda::state().streams) hs->capturing = false;
  host_cuda::push(host_cuda::kEndCapture, s, -1, host_cuda::state().captured_nodes);
  *g = new HostGraph{host_cuda::state().captured_nodes};
  return cudaSuccess;
}

inline cudaError_t cudaGraphDestroy(cudaGraph_t g) {
  delete g;
  return cudaSuccess;
}
inline cudaError_t cudaGraphInstantiate(cudaGraphExec_t* x, cudaGraph_t g, unsigned long long) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  *x = new HostGraphExec{g->nodes};
  host_cuda::state().log.push_back(host_cuda::Record{host_cuda::kGraphInstantiate, -1, -1, g->nodes, false, std::string()});
  return cudaSuccess;
}
inline cudaError_t cudaGraphExecUpdate(cudaGraphExec_t x, cudaGraph_t g, cudaGraphExecUpdateResultInfo* info) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  const bool ok = !host_cuda::state().fail_next_update && x->nodes == g->nodes;
  host_cuda::state().fail_next_update = false;
  if (info) info->result = ok ? 0 : 1;
  host_cuda::state().log.push_back(host_cuda::Record{host_cuda::kGraphUpdate, -1, -1, ok ? g->nodes : -1, false, std::string()});
  return ok ? cudaSuccess : cudaErrorGraphExecUpdateFailure;
}
inline cudaError_t cudaGraphExecDestroy(cudaGraphExec_t x) {
  delete x;
  return cudaSuccess;
}
inline cudaError_t cudaGraphLaunch(cudaGraphExec_t x, cudaStream_t s) {
  std::lock_guard<std::mutex> lk(host_cuda::state().mu);
  host_cuda::push(host_cuda::kGraphLaunch, s, -1, x->nodes);
  return cudaSuccess;
}
