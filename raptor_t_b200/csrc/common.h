// Shared host-side helpers of the raptor_b200 library: status codes, the
// thread-local error message and CUDA call checking.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/raptor_b200.h"

namespace rt {

std::string& last_error_ref();

inline rt_status fail(rt_status code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error_ref() = buf;
  return code;
}

}  // namespace rt

#define RT_CHECK_CUDA(expr)                                                                   \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return rt::fail(RT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                      __FILE__, __LINE__);                                                    \
  } while (0)

#define RT_REQUIRE(cond, code, ...)                  \
  do {                                               \
    if (!(cond)) return rt::fail(code, __VA_ARGS__); \
  } while (0)

#define RT_TRY(expr)                \
  do {                              \
    rt_status _s = (expr);          \
    if (_s != RT_OK) return _s;     \
  } while (0)
