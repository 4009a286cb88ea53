// Error helpers: every CUDA / NCCL / launcher failure becomes a C++ exception with file:line, so a
// failing call surfaces in Python as RuntimeError instead of ending the process.
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include <sstream>
#include <stdexcept>
#include <string>

namespace hetuCTR {

[[noreturn]] inline void throw_at(const char *file, int line, const std::string &what) {
  std::ostringstream os;
  os << file << ":" << line << ": " << what;
  throw std::runtime_error(os.str());
}

#define HCTR_CUDA(expr)                                                                       \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess)                                                                    \
      ::hetuCTR::throw_at(__FILE__, __LINE__, std::string("CUDA error: ") + cudaGetErrorString(e_) + " in " #expr); \
  } while (0)

// launchers return 0 or a cudaError_t value
#define HCTR_LAUNCH(expr)                                                                     \
  do {                                                                                        \
    int e_ = (expr);                                                                          \
    if (e_ != 0)                                                                              \
      ::hetuCTR::throw_at(__FILE__, __LINE__, std::string("kernel launch failed: ") +         \
                                                   cudaGetErrorString((cudaError_t)e_) + " in " #expr); \
  } while (0)

#define HCTR_NCCL(expr)                                                                       \
  do {                                                                                        \
    ncclResult_t e_ = (expr);                                                                 \
    if (e_ != ncclSuccess)                                                                    \
      ::hetuCTR::throw_at(__FILE__, __LINE__, std::string("NCCL error: ") + ncclGetErrorString(e_) + " in " #expr); \
  } while (0)

#define HCTR_CHECK(cond, msg)                                                 \
  do {                                                                        \
    if (!(cond)) ::hetuCTR::throw_at(__FILE__, __LINE__, std::string(msg));   \
  } while (0)

}  // namespace hetuCTR
