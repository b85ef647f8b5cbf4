// Stand-in for the RAFT header of the same name, just enough for the reference's error types
// to compile outside its build system.  TEST INFRASTRUCTURE (used only by oracle/ref_kernels.cu).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <exception>
#include <iostream>
#include <memory>
#include <sstream>
#include <vector>
#include <string>
namespace raft {
class exception : public std::exception {
 public:
  explicit exception(const char* m) : msg_(m) {}
  explicit exception(const std::string& m) : msg_(m) {}
  const char* what() const noexcept override { return msg_.c_str(); }

 private:
  std::string msg_;
};
struct logic_error : public exception {
  using exception::exception;
};
}  // namespace raft
