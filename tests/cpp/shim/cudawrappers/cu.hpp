// TEST INFRASTRUCTURE: a small stand-in for the part of the cudawrappers C++ API that callers of
// the reference library use (cu::init, Device, Context, Stream, DeviceMemory, HostMemory, Event),
// written from the public names of those classes, so that the cu:: overloads of <ccglib/...> can
// be compiled and exercised where the real header-only library is not installed.  Real users
// include the real <cudawrappers/cu.hpp>; nothing in the product depends on this file.
#ifndef TESTS_SHIM_CUDAWRAPPERS_CU_HPP_
#define TESTS_SHIM_CUDAWRAPPERS_CU_HPP_

#include <cstddef>
#include <stdexcept>
#include <string>

#include <cuda.h>

namespace cu {

class Error : public std::exception {
public:
  explicit Error(CUresult result) : result_(result) {}
  const char *what() const noexcept override {
    const char *text = nullptr;
    cuGetErrorString(result_, &text);
    return text ? text : "unknown CUDA error";
  }

private:
  CUresult result_;
};

inline void checkCudaCall(CUresult result) {
  if (result != CUDA_SUCCESS) throw Error(result);
}

inline void init(unsigned flags = 0) { checkCudaCall(cuInit(flags)); }

template <typename T> class Wrapper {
public:
  operator T() const { return obj_; }

protected:
  Wrapper() = default;
  explicit Wrapper(T obj) : obj_(obj) {}
  T obj_{};
};

class Device : public Wrapper<CUdevice> {
public:
  explicit Device(int ordinal) { checkCudaCall(cuDeviceGet(&obj_, ordinal)); }  // CUdevice is int
  int getAttribute(CUdevice_attribute attribute) const {
    int value = 0;
    checkCudaCall(cuDeviceGetAttribute(&value, attribute, obj_));
    return value;
  }
  std::string getArch() const {
    return "sm_" + std::to_string(10 * getAttribute(CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR) +
                                  getAttribute(CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR));
  }
};

// Retains the primary context and makes it current, which is what the runtime API shares.
class Context : public Wrapper<CUcontext> {
public:
  Context(unsigned /*flags*/, Device &device) : device_(device) {
    checkCudaCall(cuDevicePrimaryCtxRetain(&obj_, device_));
    checkCudaCall(cuCtxSetCurrent(obj_));
  }
  ~Context() { cuDevicePrimaryCtxRelease(device_); }
  Context(const Context &) = delete;
  Context &operator=(const Context &) = delete;

private:
  CUdevice device_;
};

class HostMemory : public Wrapper<void *> {
public:
  explicit HostMemory(size_t size) : size_(size), owner_(true) {
    checkCudaCall(cuMemHostAlloc(&obj_, size ? size : 1, 0));
  }
  HostMemory(void *ptr, size_t size) : Wrapper(ptr), size_(size), owner_(false) {}
  ~HostMemory() {
    if (owner_) cuMemFreeHost(obj_);
  }
  HostMemory(const HostMemory &) = delete;
  HostMemory &operator=(const HostMemory &) = delete;
  template <typename T> operator T *() { return static_cast<T *>(obj_); }
  size_t size() const { return size_; }

private:
  size_t size_;
  bool owner_;
};

class DeviceMemory : public Wrapper<CUdeviceptr> {
public:
  explicit DeviceMemory(size_t size) : size_(size), owner_(true) {
    checkCudaCall(cuMemAlloc(&obj_, size ? size : 1));
  }
  explicit DeviceMemory(CUdeviceptr ptr, size_t size = 0) : Wrapper(ptr), size_(size), owner_(false) {}
  ~DeviceMemory() {
    if (owner_) cuMemFree(obj_);
  }
  DeviceMemory(const DeviceMemory &) = delete;
  DeviceMemory &operator=(const DeviceMemory &) = delete;
  size_t size() const { return size_; }
  void zero(size_t size) { checkCudaCall(cuMemsetD8(obj_, 0, size)); }
  const void *parameter() const { return &obj_; }

private:
  size_t size_;
  bool owner_;
};

class Event : public Wrapper<CUevent> {
public:
  explicit Event(unsigned flags = CU_EVENT_DEFAULT) { checkCudaCall(cuEventCreate(&obj_, flags)); }
  ~Event() { cuEventDestroy(obj_); }
  Event(const Event &) = delete;
  Event &operator=(const Event &) = delete;
  float elapsedTime(const Event &start) const {
    float ms = 0;
    checkCudaCall(cuEventElapsedTime(&ms, start.obj_, obj_));
    return ms;
  }
  void synchronize() { checkCudaCall(cuEventSynchronize(obj_)); }
};

class Stream : public Wrapper<CUstream> {
public:
  explicit Stream(unsigned flags = CU_STREAM_DEFAULT) : owner_(true) {
    checkCudaCall(cuStreamCreate(&obj_, flags));
  }
  explicit Stream(CUstream stream) : Wrapper(stream), owner_(false) {}
  ~Stream() {
    if (owner_) cuStreamDestroy(obj_);
  }
  Stream(const Stream &) = delete;
  Stream &operator=(const Stream &) = delete;
  void memcpyHtoDAsync(DeviceMemory &dst, const void *src, size_t size) {
    checkCudaCall(cuMemcpyHtoDAsync(dst, src, size, obj_));
  }
  void memcpyDtoHAsync(void *dst, const DeviceMemory &src, size_t size) {
    checkCudaCall(cuMemcpyDtoHAsync(dst, src, size, obj_));
  }
  void memsetAsync(DeviceMemory &dst, unsigned char value, size_t size) {
    checkCudaCall(cuMemsetD8Async(dst, value, size, obj_));
  }
  void record(Event &event) { checkCudaCall(cuEventRecord(event, obj_)); }
  void synchronize() { checkCudaCall(cuStreamSynchronize(obj_)); }

private:
  bool owner_;
};

} // namespace cu
#endif
