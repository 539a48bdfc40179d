#include "logger.hpp"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unistd.h>

namespace mscclpp {

namespace {

struct LogState {
  LogLevel level = LogLevel::ERROR;
  unsigned mask = static_cast<unsigned>(LogSubsys::ALL);
  FILE* out = stderr;
  bool ownsFile = false;
  std::mutex mutex;
  bool configured = false;
};

LogState& state() {
  static LogState s;
  return s;
}

const char* levelName(LogLevel l) {
  switch (l) {
    case LogLevel::DEBUG:
      return "DEBUG";
    case LogLevel::INFO:
      return "INFO";
    case LogLevel::WARN:
      return "WARN";
    case LogLevel::ERROR:
      return "ERROR";
    default:
      return "NONE";
  }
}

const char* subsysName(LogSubsys s) {
  switch (s) {
    case LogSubsys::ENV:
      return "ENV";
    case LogSubsys::GPU:
      return "GPU";
    case LogSubsys::NET:
      return "NET";
    case LogSubsys::CONN:
      return "CONN";
    case LogSubsys::EXEC:
      return "EXEC";
    case LogSubsys::NCCL:
      return "NCCL";
    case LogSubsys::ALGO:
      return "ALGO";
    default:
      return "ALL";
  }
}

unsigned subsysFromName(const std::string& n) {
  static const struct {
    const char* name;
    LogSubsys s;
  } table[] = {{"ENV", LogSubsys::ENV},   {"GPU", LogSubsys::GPU},   {"NET", LogSubsys::NET},  {"CONN", LogSubsys::CONN},
               {"EXEC", LogSubsys::EXEC}, {"NCCL", LogSubsys::NCCL}, {"ALGO", LogSubsys::ALGO}, {"ALL", LogSubsys::ALL}};
  for (auto& e : table)
    if (n == e.name) return static_cast<unsigned>(e.s);
  return 0;
}

void configureLocked(LogState& s) {
  const char* lvl = std::getenv("MSCCLPP_LOG_LEVEL");
  if (!lvl) lvl = std::getenv("MSCCLPP_DEBUG");  // legacy spelling
  s.level = LogLevel::ERROR;
  if (lvl) {
    std::string v(lvl);
    for (auto& c : v) c = static_cast<char>(std::toupper(c));
    if (v == "DEBUG" || v == "TRACE") s.level = LogLevel::DEBUG;
    else if (v == "INFO") s.level = LogLevel::INFO;
    else if (v == "WARN") s.level = LogLevel::WARN;
    else if (v == "ERROR") s.level = LogLevel::ERROR;
    else if (v == "NONE") s.level = LogLevel::NONE;
  }
  const char* sub = std::getenv("MSCCLPP_LOG_SUBSYS");
  if (!sub) sub = std::getenv("MSCCLPP_DEBUG_SUBSYS");
  s.mask = static_cast<unsigned>(LogSubsys::ALL);
  if (sub && *sub) {
    std::string v(sub);
    bool invert = false;
    if (v[0] == '^') {
      invert = true;
      v = v.substr(1);
    }
    unsigned m = 0;
    size_t pos = 0;
    while (pos <= v.size()) {
      size_t comma = v.find(',', pos);
      if (comma == std::string::npos) comma = v.size();
      std::string tok = v.substr(pos, comma - pos);
      for (auto& c : tok) c = static_cast<char>(std::toupper(c));
      m |= subsysFromName(tok);
      pos = comma + 1;
    }
    s.mask = invert ? (~m & static_cast<unsigned>(LogSubsys::ALL)) : m;
  }
  const char* file = std::getenv("MSCCLPP_LOG_FILE");
  if (!file) file = std::getenv("MSCCLPP_DEBUG_FILE");
  if (s.ownsFile && s.out) std::fclose(s.out);
  s.out = stderr;
  s.ownsFile = false;
  if (file && *file) {
    // %p -> pid, so that every rank writes its own file
    std::string path(file);
    size_t p = path.find("%p");
    if (p != std::string::npos) path.replace(p, 2, std::to_string(getpid()));
    FILE* f = std::fopen(path.c_str(), "a");
    if (f) {
      s.out = f;
      s.ownsFile = true;
    }
  }
  s.configured = true;
}

}  // namespace

void logReconfigure() {
  LogState& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  configureLocked(s);
}

bool logEnabled(LogLevel level, LogSubsys subsys) {
  LogState& s = state();
  if (!s.configured) {
    std::lock_guard<std::mutex> lock(s.mutex);
    if (!s.configured) configureLocked(s);
  }
  if (static_cast<int>(level) < static_cast<int>(s.level)) return false;
  if (level == LogLevel::ERROR) return true;  // errors ignore the subsystem filter
  return (s.mask & static_cast<unsigned>(subsys)) != 0;
}

void logWrite(LogLevel level, LogSubsys subsys, const char* file, int line, const std::string& message) {
  LogState& s = state();
  using namespace std::chrono;
  auto now = system_clock::now();
  auto us = duration_cast<microseconds>(now.time_since_epoch()).count();
  std::time_t secs = static_cast<std::time_t>(us / 1000000);
  std::tm tm{};
  localtime_r(&secs, &tm);
  char ts[64];
  std::snprintf(ts, sizeof(ts), "%04d-%02d-%02d %02d:%02d:%02d.%06ld", tm.tm_year + 1900, tm.tm_mon + 1, tm.tm_mday,
                tm.tm_hour, tm.tm_min, tm.tm_sec, static_cast<long>(us % 1000000));
  const char* base = std::strrchr(file, '/');
  base = base ? base + 1 : file;
  std::lock_guard<std::mutex> lock(s.mutex);
  std::fprintf(s.out, "%s MSCCLPP %d %s %s %s:%d %s\n", ts, static_cast<int>(getpid()), levelName(level),
               subsysName(subsys), base, line, message.c_str());
  std::fflush(s.out);
}

}  // namespace mscclpp
