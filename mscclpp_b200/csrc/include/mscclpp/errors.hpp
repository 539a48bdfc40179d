// Error types of the library. Same public names and codes as the reference
// (include/mscclpp/errors.hpp:12-94) so that user code catching mscclpp::Error keeps working.
#pragma once

#include <stdexcept>
#include <string>

namespace mscclpp {

enum class ErrorCode {
  SystemError = 0,    // a system call failed
  InternalError = 1,  // a bug in this library
  RemoteError = 2,    // a peer reported or caused a failure
  InvalidUsage = 3,   // the caller broke an API contract
  Timeout = 4,        // a bounded wait ran out
  Aborted = 5,        // the operation was cancelled through an abort flag
  ExecutorError = 6,  // a plan could not be loaded or executed
};

std::string errorToString(ErrorCode code);

class BaseError : public std::runtime_error {
 public:
  BaseError(const std::string& message, int errorCode);
  explicit BaseError(int errorCode);
  int getErrorCode() const { return errorCode_; }
  const char* what() const noexcept override { return message_.c_str(); }

 protected:
  std::string message_;
  int errorCode_;
};

class Error : public BaseError {
 public:
  Error(const std::string& message, ErrorCode errorCode);
  ErrorCode getErrorCode() const { return static_cast<ErrorCode>(errorCode_); }
};

class SysError : public BaseError {
 public:
  SysError(const std::string& message, int errnoValue);
};

class CudaError : public BaseError {
 public:
  CudaError(const std::string& message, int cudaErrorValue);
};

class CuError : public BaseError {
 public:
  CuError(const std::string& message, int cuResultValue);
};

class IbError : public BaseError {
 public:
  IbError(const std::string& message, int errnoValue);
};

}  // namespace mscclpp

#define MSCCLPP_CUDATHROW(cmd)                                                                                  \
  do {                                                                                                          \
    cudaError_t err__ = (cmd);                                                                                  \
    if (err__ != cudaSuccess) {                                                                                 \
      throw ::mscclpp::CudaError(std::string(#cmd " failed at ") + __FILE__ + ":" + std::to_string(__LINE__), \
                                 static_cast<int>(err__));                                                      \
    }                                                                                                           \
  } while (0)

#define MSCCLPP_CUTHROW(cmd)                                                                                  \
  do {                                                                                                        \
    CUresult err__ = (cmd);                                                                                   \
    if (err__ != CUDA_SUCCESS) {                                                                              \
      throw ::mscclpp::CuError(std::string(#cmd " failed at ") + __FILE__ + ":" + std::to_string(__LINE__), \
                               static_cast<int>(err__));                                                      \
    }                                                                                                         \
  } while (0)
