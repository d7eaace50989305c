// Header-only levelled logger to stderr (role of backend/src/engine/logger.h:9-64).  Level from
// env STELLATRAIN_LOG = debug|info|warn|error (default info).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>

namespace stc {

enum class LogLevel : int { Debug = 0, Info = 1, Warn = 2, Error = 3 };

class Logger {
 public:
  static Logger& get() {
    static Logger inst;
    return inst;
  }
  LogLevel level() const { return level_; }
  void set_level(LogLevel l) { level_ = l; }
  void write(LogLevel l, const char* tag, const std::string& msg) {
    if (l < level_) return;
    static const char* names[] = {"DEBUG", "INFO", "WARN", "ERROR"};
    std::lock_guard<std::mutex> lk(mu_);
    std::fprintf(stderr, "[%s] %s: %s\n", names[static_cast<int>(l)], tag, msg.c_str());
  }

 private:
  Logger() {
    const char* v = std::getenv("STELLATRAIN_LOG");
    if (!v) return;
    if (!std::strcmp(v, "debug")) level_ = LogLevel::Debug;
    else if (!std::strcmp(v, "warn")) level_ = LogLevel::Warn;
    else if (!std::strcmp(v, "error")) level_ = LogLevel::Error;
  }
  LogLevel level_ = LogLevel::Info;
  std::mutex mu_;
};

}  // namespace stc

#define STC_LOG(lvl_, tag, expr)                                              \
  do {                                                                        \
    if ((lvl_) >= ::stc::Logger::get().level()) {                             \
      std::ostringstream stc_log_os;                                          \
      stc_log_os << expr;                                                     \
      ::stc::Logger::get().write((lvl_), (tag), stc_log_os.str());            \
    }                                                                         \
  } while (0)
#define LOG_DEBUG(tag, expr) STC_LOG(::stc::LogLevel::Debug, tag, expr)
#define LOG_INFO(tag, expr) STC_LOG(::stc::LogLevel::Info, tag, expr)
#define LOG_WARN(tag, expr) STC_LOG(::stc::LogLevel::Warn, tag, expr)
#define LOG_ERROR(tag, expr) STC_LOG(::stc::LogLevel::Error, tag, expr)
