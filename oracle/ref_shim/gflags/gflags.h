// Minimal stand-in for <gflags/gflags.h> (gflags is not installed on this image) so that the
// reference's walk sources compile unmodified: flags become plain globals that the harness
// sets directly.  Test infrastructure only.
#pragma once
#include <stdint.h>
#include <string>

#define DEFINE_bool(name, val, txt) bool FLAGS_##name = (val)
#define DEFINE_int32(name, val, txt) int32_t FLAGS_##name = (val)
#define DEFINE_uint32(name, val, txt) uint32_t FLAGS_##name = (val)
#define DEFINE_int64(name, val, txt) int64_t FLAGS_##name = (val)
#define DEFINE_uint64(name, val, txt) uint64_t FLAGS_##name = (val)
#define DEFINE_double(name, val, txt) double FLAGS_##name = (val)
#define DEFINE_string(name, val, txt) std::string FLAGS_##name = (val)
#define DECLARE_bool(name) extern bool FLAGS_##name
#define DECLARE_int32(name) extern int32_t FLAGS_##name
#define DECLARE_uint32(name) extern uint32_t FLAGS_##name
#define DECLARE_int64(name) extern int64_t FLAGS_##name
#define DECLARE_uint64(name) extern uint64_t FLAGS_##name
#define DECLARE_double(name) extern double FLAGS_##name
#define DECLARE_string(name) extern std::string FLAGS_##name

namespace gflags {
inline uint32_t ParseCommandLineFlags(int*, char***, bool) { return 1; }
}  // namespace gflags
namespace google = gflags;
