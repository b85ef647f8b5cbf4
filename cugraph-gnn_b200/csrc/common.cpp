#include "common.hpp"

#include <cstring>
#include <new>

namespace wgb {

LogLevel& log_level()
{
  static LogLevel lvl = LEVEL_INFO;
  return lvl;
}

static const char* level_name(LogLevel l)
{
  switch (l) {
    case LEVEL_FATAL: return "FATAL";
    case LEVEL_ERROR: return "ERROR";
    case LEVEL_WARN: return "WARN";
    case LEVEL_INFO: return "INFO";
    case LEVEL_DEBUG: return "DEBUG";
    default: return "TRACE";
  }
}

void log_line(LogLevel lvl, const char* file, int line, const char* fmt, ...)
{
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  fprintf(lvl <= LEVEL_WARN ? stderr : stdout, "[wholegraph %s] %s:%d %s\n", level_name(lvl),
          base ? base + 1 : file, line, buf);
}

std::string format_string(const char* fmt, ...)
{
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return std::string(buf);
}

wholegraph_error_code_t translate_current_exception(const char* where) noexcept
{
  try {
    throw;
  } catch (const invalid_input& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return e.code;
  } catch (const cuda_error& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return WHOLEGRAPH_CUDA_ERROR;
  } catch (const comm_error& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return WHOLEGRAPH_COMMUNICATION_ERROR;
  } catch (const system_error& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return WHOLEGRAPH_SYSTEM_ERROR;
  } catch (const logic_error& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return WHOLEGRAPH_LOGIC_ERROR;
  } catch (const std::bad_alloc&) {
    WGB_ERROR("%s: out of memory", where);
    return WHOLEGRAPH_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    WGB_ERROR("%s: %s", where, e.what());
    return WHOLEGRAPH_UNKNOW_ERROR;
  } catch (...) {
    WGB_ERROR("%s: unknown exception", where);
    return WHOLEGRAPH_UNKNOW_ERROR;
  }
}

bool debug_sync_enabled()
{
  static int v = [] {
    const char* e = getenv("WG_DEBUG_SYNC");
    return (e != nullptr && strcmp(e, "1") == 0) ? 1 : 0;
  }();
  return v == 1;
}

void debug_sync_stream(cudaStream_t s, const char* file, int line)
{
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    throw cuda_error(format_string("%s:%d stream sync after launch failed: %s", file, line,
                                   cudaGetErrorString(e)));
  }
}

}  // namespace wgb
