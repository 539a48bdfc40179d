#include <mscclpp/errors.hpp>

#include <cstring>
#include <cuda_runtime.h>

namespace mscclpp {

std::string errorToString(ErrorCode code) {
  switch (code) {
    case ErrorCode::SystemError:
      return "SystemError";
    case ErrorCode::InternalError:
      return "InternalError";
    case ErrorCode::RemoteError:
      return "RemoteError";
    case ErrorCode::InvalidUsage:
      return "InvalidUsage";
    case ErrorCode::Timeout:
      return "Timeout";
    case ErrorCode::Aborted:
      return "Aborted";
    case ErrorCode::ExecutorError:
      return "ExecutorError";
  }
  return "UnknownError";
}

BaseError::BaseError(const std::string& message, int errorCode)
    : std::runtime_error(message), message_(message), errorCode_(errorCode) {}
BaseError::BaseError(int errorCode) : std::runtime_error(""), errorCode_(errorCode) {}

Error::Error(const std::string& message, ErrorCode errorCode) : BaseError(static_cast<int>(errorCode)) {
  message_ = message + " (mscclpp failure: " + errorToString(errorCode) + ")";
}

SysError::SysError(const std::string& message, int errnoValue) : BaseError(errnoValue) {
  message_ = message + " (system failure: " + std::strerror(errnoValue) + ")";
}

CudaError::CudaError(const std::string& message, int cudaErrorValue) : BaseError(cudaErrorValue) {
  message_ = message + " (CUDA failure: " + cudaGetErrorString(static_cast<cudaError_t>(cudaErrorValue)) + ")";
}

CuError::CuError(const std::string& message, int cuResultValue) : BaseError(cuResultValue) {
  message_ = message + " (CUDA driver failure: CUresult " + std::to_string(cuResultValue) + ")";
}

IbError::IbError(const std::string& message, int errnoValue) : BaseError(errnoValue) {
  message_ = message + " (IB failure: " + std::strerror(errnoValue) + ")";
}

}  // namespace mscclpp
