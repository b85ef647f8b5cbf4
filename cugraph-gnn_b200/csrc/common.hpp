// Shared host-side plumbing: logging, error types, and the macros that turn failures into
// return codes at the C boundary (no exception ever crosses it).
// Mirrors the contract of the reference's cpp/src/error.hpp:75-136 and cpp/src/logger.hpp:59-76.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include <wholegraph/wholegraph.h>

namespace wgb {

LogLevel& log_level();
void log_line(LogLevel lvl, const char* file, int line, const char* fmt, ...)
  __attribute__((format(printf, 4, 5)));
std::string format_string(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

struct logic_error : std::logic_error {
  using std::logic_error::logic_error;
};
struct cuda_error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct comm_error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct system_error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct invalid_input : std::runtime_error {
  wholegraph_error_code_t code;
  invalid_input(wholegraph_error_code_t c, const std::string& s) : std::runtime_error(s), code(c) {}
};

// Map the exception in flight to a return code and log it. Call inside `catch (...)`.
wholegraph_error_code_t translate_current_exception(const char* where) noexcept;

// True when WG_DEBUG_SYNC=1: every checked launch is followed by a stream synchronize
// (reference: cpp/src/cuda_macros.cpp:16-56).
bool debug_sync_enabled();
void debug_sync_stream(cudaStream_t s, const char* file, int line);

}  // namespace wgb

#define WGB_LOG(lvl, ...)                                                              \
  do {                                                                                 \
    if ((lvl) <= ::wgb::log_level()) ::wgb::log_line((lvl), __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define WGB_ERROR(...) WGB_LOG(LEVEL_ERROR, __VA_ARGS__)
#define WGB_WARN(...) WGB_LOG(LEVEL_WARN, __VA_ARGS__)
#define WGB_INFO(...) WGB_LOG(LEVEL_INFO, __VA_ARGS__)
#define WGB_DEBUG(...) WGB_LOG(LEVEL_DEBUG, __VA_ARGS__)

// Throwing checks, for code below a try/catch at the C boundary.
#define WGB_EXPECTS(cond, ...)                                                          \
  do {                                                                                  \
    if (!(cond)) {                                                                      \
      throw ::wgb::logic_error(::wgb::format_string("%s:%d (%s) ", __FILE__, __LINE__, #cond) + \
                               ::wgb::format_string(__VA_ARGS__));                      \
    }                                                                                   \
  } while (0)
#define WGB_CHECK(cond) WGB_EXPECTS(cond, "check failed")

#define WGB_CUDA_CHECK(call)                                                            \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      (void)cudaGetLastError();                                                         \
      throw ::wgb::cuda_error(::wgb::format_string(                                     \
        "%s:%d CUDA error %d (%s) in %s", __FILE__, __LINE__, (int)e__, cudaGetErrorString(e__), \
        #call));                                                                        \
    }                                                                                   \
  } while (0)

#define WGB_LAUNCH_CHECK(stream)                        \
  do {                                                  \
    WGB_CUDA_CHECK(cudaGetLastError());                 \
    if (::wgb::debug_sync_enabled())                    \
      ::wgb::debug_sync_stream((stream), __FILE__, __LINE__); \
  } while (0)

// Boundary wrapper: run `body`, return its code or the translated exception.
#define WGB_API_BEGIN try {
#define WGB_API_END(where)                                   \
  }                                                          \
  catch (...) { return ::wgb::translate_current_exception(where); }
