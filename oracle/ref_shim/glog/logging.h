// Minimal stand-in for <glog/logging.h>, used ONLY to compile the unmodified reference
// sources into oracle/_ref/libgs_ref.so (the reference's glog submodule is not vendored).
// Streams to stderr; FATAL and failed CHECKs abort, like glog.
#ifndef GSB_REF_SHIM_GLOG_LOGGING_H_
#define GSB_REF_SHIM_GLOG_LOGGING_H_
#include <cstdlib>
#include <iostream>
#include <sstream>

namespace gsb_ref_shim {
enum Severity { INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };
class LogMessage {
 public:
  LogMessage(const char* file, int line, int sev) : sev_(sev) {
    static const char* names[] = {"I", "W", "E", "F"};
    os_ << names[sev] << " " << file << ":" << line << "] ";
  }
  ~LogMessage() {
    os_ << "\n";
    std::cerr << os_.str();
    if (sev_ == FATAL) std::abort();
  }
  std::ostream& stream() { return os_; }

 private:
  std::ostringstream os_;
  int sev_;
};
struct Voidify {
  void operator&(std::ostream&) {}
};
}  // namespace gsb_ref_shim

#define LOG(sev) ::gsb_ref_shim::LogMessage(__FILE__, __LINE__, ::gsb_ref_shim::sev).stream()
#define CHECK(cond)    \
  (cond) ? (void)0     \
         : ::gsb_ref_shim::Voidify() & LOG(FATAL) << "Check failed: " #cond " "
#define GSB_SHIM_CHECK_OP(a, b, op) CHECK((a)op(b))
#define CHECK_EQ(a, b) GSB_SHIM_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) GSB_SHIM_CHECK_OP(a, b, !=)
#define CHECK_LE(a, b) GSB_SHIM_CHECK_OP(a, b, <=)
#define CHECK_LT(a, b) GSB_SHIM_CHECK_OP(a, b, <)
#define CHECK_GE(a, b) GSB_SHIM_CHECK_OP(a, b, >=)
#define CHECK_GT(a, b) GSB_SHIM_CHECK_OP(a, b, >)
#define CHECK_NOTNULL(p) (p)
#define DCHECK(c) CHECK(c)
#endif
