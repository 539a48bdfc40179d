// Leveled, subsystem-filtered logger (internal). Line format:
//   <timestamp> MSCCLPP <pid> <LEVEL> <SUBSYS> <file>:<line> <message>
// Controlled by MSCCLPP_LOG_LEVEL / MSCCLPP_LOG_SUBSYS / MSCCLPP_LOG_FILE, read directly from the
// environment (not through Env) so that Env's own start-up dump can be logged.
#pragma once

#include <sstream>
#include <string>

namespace mscclpp {

enum class LogLevel : int { DEBUG = 0, INFO = 1, WARN = 2, ERROR = 3, NONE = 4 };
enum class LogSubsys : unsigned {
  ENV = 1u << 0,
  GPU = 1u << 1,
  NET = 1u << 2,
  CONN = 1u << 3,
  EXEC = 1u << 4,
  NCCL = 1u << 5,
  ALGO = 1u << 6,
  ALL = 0x7fu
};

bool logEnabled(LogLevel level, LogSubsys subsys);
void logWrite(LogLevel level, LogSubsys subsys, const char* file, int line, const std::string& message);
// Re-read MSCCLPP_LOG_* (tests change them at run time).
void logReconfigure();

namespace detail {
inline void logAppend(std::ostringstream&) {}
template <typename T, typename... Rest>
void logAppend(std::ostringstream& os, const T& v, const Rest&... rest) {
  os << v;
  logAppend(os, rest...);
}
template <typename... Args>
std::string logConcat(const Args&... args) {
  std::ostringstream os;
  logAppend(os, args...);
  return os.str();
}
}  // namespace detail

}  // namespace mscclpp

#define MSCCLPP_LOG(level, subsys, ...)                                                              \
  do {                                                                                               \
    if (::mscclpp::logEnabled(level, subsys))                                                        \
      ::mscclpp::logWrite(level, subsys, __FILE__, __LINE__, ::mscclpp::detail::logConcat(__VA_ARGS__)); \
  } while (0)
#define LOG_DEBUG(subsys, ...) MSCCLPP_LOG(::mscclpp::LogLevel::DEBUG, subsys, __VA_ARGS__)
#define LOG_INFO(subsys, ...) MSCCLPP_LOG(::mscclpp::LogLevel::INFO, subsys, __VA_ARGS__)
#define LOG_WARN(subsys, ...) MSCCLPP_LOG(::mscclpp::LogLevel::WARN, subsys, __VA_ARGS__)
#define LOG_ERROR(subsys, ...) MSCCLPP_LOG(::mscclpp::LogLevel::ERROR, subsys, __VA_ARGS__)
// Log at ERROR level, then throw ErrorType(message, code).
#define THROW(subsys, ErrorType, code, ...)                                   \
  do {                                                                        \
    std::string msg__ = ::mscclpp::detail::logConcat(__VA_ARGS__);            \
    LOG_ERROR(subsys, msg__);                                                 \
    throw ErrorType(msg__, code);                                             \
  } while (0)
