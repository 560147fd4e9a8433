// Event-based kernel tracing (counterpart of the reference's
// core/mlu_op_trace.cpp + core/kernel_tracing.cpp, which hook the vendor launch
// call; here each launch site opens a trace::Scope).
#include "core/trace.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "core/logging.h"
#include "mlu_op_trace.h"

namespace mluop {
namespace trace {

namespace {

struct Record {
  const char *name;
  cudaEvent_t start, stop;
  double bytes, flops;
};

struct State {
  std::mutex lock;
  std::vector<Record> records;
  std::vector<cudaEvent_t> spare;
  std::string data_dir;
  std::string unfetched;  // a report that did not fit the caller's buffer
};

std::atomic<int> g_enabled{-1};  // -1: environment not read yet

State &state() {
  static State *s = new State;
  return *s;
}

cudaEvent_t takeEvent(State &s) {
  if (!s.spare.empty()) {
    cudaEvent_t e = s.spare.back();
    s.spare.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return e;
}

std::string summarise(State &s) {
  struct Sum {
    long launches = 0;
    double ms = 0, bytes = 0, flops = 0;
  };
  std::vector<const char *> order;
  std::map<std::string, Sum> sums;
  for (Record &r : s.records) {
    float ms = 0.f;
    if (r.start && r.stop && cudaEventSynchronize(r.stop) == cudaSuccess &&
        cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess) {
      if (!sums.count(r.name)) order.push_back(r.name);
      Sum &u = sums[r.name];
      u.launches += 1;
      u.ms += ms;
      u.bytes += r.bytes;
      u.flops += r.flops;
    } else {
      (void)cudaGetLastError();
    }
    if (r.start) s.spare.push_back(r.start);
    if (r.stop) s.spare.push_back(r.stop);
  }
  s.records.clear();
  std::string out = "name,launches,total_ms,algorithmic_bytes,flops\n";
  char line[512];
  for (const char *name : order) {
    const Sum &u = sums[name];
    std::snprintf(line, sizeof(line), "%s,%ld,%.6f,%.0f,%.0f\n", name, u.launches, u.ms, u.bytes, u.flops);
    out += line;
  }
  return out;
}

void dumpAtExit() {
  State &s = state();
  std::lock_guard<std::mutex> guard(s.lock);
  if (s.data_dir.empty() || s.records.empty()) return;
  const std::string path = s.data_dir + "/mlu_op_kernel.csv";
  const std::string text = summarise(s);
  if (FILE *f = std::fopen(path.c_str(), "w")) {
    std::fputs(text.c_str(), f);
    std::fclose(f);
  }
}

void readEnvironment() {
  const char *on = std::getenv("MLUOP_TRACE_ENABLE_KERNEL");
  const char *dir = std::getenv("MLUOP_TRACE_DATA_DIR");
  int want = (on && std::strcmp(on, "1") == 0) ? 1 : 0;
  int expected = -1;
  if (g_enabled.compare_exchange_strong(expected, want) && dir && *dir) {
    state().data_dir = dir;
    std::atexit(dumpAtExit);
  }
}

}  // namespace

bool enabled() {
  int v = g_enabled.load(std::memory_order_relaxed);
  if (v < 0) {
    readEnvironment();
    v = g_enabled.load(std::memory_order_relaxed);
  }
  return v > 0;
}

Scope::Scope(const char *name, cudaStream_t stream, double bytes, double flops) : slot_(-1), stream_(stream) {
  if (!enabled()) return;
  State &s = state();
  std::lock_guard<std::mutex> guard(s.lock);
  Record r{name, takeEvent(s), takeEvent(s), bytes, flops};
  if (r.start) cudaEventRecord(r.start, stream);
  s.records.push_back(r);
  slot_ = (int)s.records.size() - 1;
}

Scope::~Scope() {
  if (slot_ < 0) return;
  State &s = state();
  std::lock_guard<std::mutex> guard(s.lock);
  if (slot_ < (int)s.records.size() && s.records[slot_].stop) cudaEventRecord(s.records[slot_].stop, stream_);
}

}  // namespace trace
}  // namespace mluop

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelEnable(int enable) {
  (void)mluop::trace::enabled();  // settle the environment first
  mluop::trace::g_enabled.store(enable ? 1 : 0);
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelReset(void) {
  auto &s = mluop::trace::state();
  std::lock_guard<std::mutex> guard(s.lock);
  for (auto &r : s.records) {
    if (r.start) s.spare.push_back(r.start);
    if (r.stop) s.spare.push_back(r.stop);
  }
  s.records.clear();
  s.unfetched.clear();
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelReport(char *buffer, size_t buffer_size, size_t *needed) {
  PARAM_CHECK("[mluOpTraceKernelReport]", buffer != NULL || buffer_size == 0);
  auto &s = mluop::trace::state();
  std::lock_guard<std::mutex> guard(s.lock);
  // A report that did not fit the caller's buffer is kept, so that a caller that asks
  // for the size first and fetches second loses nothing; launches recorded in between
  // are appended as further lines.
  std::string text = s.unfetched;
  if (text.empty() || !s.records.empty()) {
    std::string more = mluop::trace::summarise(s);
    if (!text.empty()) more.erase(0, more.find('\n') + 1);  // one header line only
    text += more;
  }
  if (needed) *needed = text.size() + 1;
  const bool fits = buffer_size >= text.size() + 1;
  if (buffer_size > 0) {
    const size_t n = fits ? text.size() : buffer_size - 1;
    std::memcpy(buffer, text.data(), n);
    buffer[n] = '\0';
  }
  if (fits) {
    s.unfetched.clear();
  } else {
    s.unfetched = text;
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
