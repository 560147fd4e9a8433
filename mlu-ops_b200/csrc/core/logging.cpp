// stderr logger behind the LOG/VLOG macros, and the contiguity test used by
// STRIDE_TENSOR_CHECK (same rule as the reference's core/util.cpp:43).
#include "core/logging.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace mluop {

static int envInt(const char *name, int fallback) {
  const char *v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : fallback;
}

int minLogLevel() {
  static int level = envInt("MLUOP_MIN_LOG_LEVEL", 0);
  return level;
}

int minVlogLevel() {
  static int level = envInt("MLUOP_MIN_VLOG_LEVEL", 0);
  return level;
}

LogLine::LogLine(int level, const char *file, int line) : level_(level) {
  static const char *names[] = {"INFO", "WARNING", "ERROR"};
  const char *base = std::strrchr(file, '/');
  os_ << "[MLUOP][" << names[level] << "][" << (base ? base + 1 : file) << ":" << line << "] ";
}

LogLine::~LogLine() {
  os_ << "\n";
  std::fputs(os_.str().c_str(), stderr);
}

bool isStrideTensor(int dim, const int64_t *dims, const int64_t *strides) {
  int64_t expect = 1;
  for (int i = dim - 1; i >= 0; --i) {
    if (dims[i] != 1 && strides[i] != expect) return true;
    expect *= dims[i];
  }
  return false;
}

}  // namespace mluop
