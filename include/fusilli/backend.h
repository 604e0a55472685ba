// Backend enum, Handle (device + stream) and Buffer (device memory) over the C ABI of
// libfusilli_b200.so. Same public surface as the reference's include/fusilli/backend/
// {backend.h:42, handle.h:35-176, buffer.h:31-81, runtime.h:532-674}: move-only RAII objects,
// ErrorOr factories, the same size checks and messages. Backend::CUDA is the one executable
// backend of this build; CPU and AMDGPU stay as enumerators so existing code that names them
// compiles, and creating a handle for them fails with NotImplemented (there is no CPU path).
#ifndef FUSILLI_BACKEND_H
#define FUSILLI_BACKEND_H

#include <cstdint>
#include <ostream>
#include <string>
#include <utility>
#include <vector>

#include "../fusilli_b200.h"
#include "error.h"
#include "types.h"

namespace fusilli {

enum class Backend : uint8_t { CPU, AMDGPU, CUDA };

inline std::ostream &operator<<(std::ostream &os, Backend b) {
  return os << (b == Backend::CPU ? "CPU" : b == Backend::AMDGPU ? "AMDGPU" : "CUDA");
}

// fb_status carries the ErrorCode numbering; a failing call's message is thread local.
inline ErrorObject fromStatus(fb_status st) {
  if (st == FB_OK) return ok();
  return ErrorObject(static_cast<ErrorCode>(st), fb_last_error());
}
#define FUSILLI_FB_CALL(expr) FUSILLI_CHECK_ERROR(fusilli::fromStatus(expr))

class Handle {
public:
  static ErrorOr<Handle> create(Backend backend) { return open(backend, 0, 0, false); }
  // A device (and a stream) can be chosen on the device backend only; on any other backend both
  // overloads are InvalidArgument, as in the reference (handle.h:74-98).
  static ErrorOr<Handle> create(Backend backend, int deviceId) {
    FUSILLI_RETURN_ERROR_IF(backend != Backend::CUDA, ErrorCode::InvalidArgument,
                            "Stream can only be set on the CUDA backend");
    return open(backend, deviceId, 0, false);
  }
  // `stream` is a cudaStream_t owned by the caller; work is enqueued on it and never
  // synchronised except by Buffer::read.
  static ErrorOr<Handle> create(Backend backend, int deviceId, uintptr_t stream) {
    return open(backend, deviceId, stream, true);
  }

  Handle(const Handle &) = delete;
  Handle &operator=(const Handle &) = delete;
  Handle(Handle &&o) noexcept : backend_(o.backend_), dev_(std::exchange(o.dev_, nullptr)) {}
  Handle &operator=(Handle &&o) noexcept {
    if (this != &o) {
      reset();
      backend_ = o.backend_;
      dev_ = std::exchange(o.dev_, nullptr);
    }
    return *this;
  }
  ~Handle() { reset(); }

  Backend getBackend() const { return backend_; }
  fb_device *device() const { return dev_; }
  operator fb_device *() const { return dev_; }
  uintptr_t getStream() const { return reinterpret_cast<uintptr_t>(fb_device_stream(dev_)); }
  ErrorObject synchronize() const { return fromStatus(fb_device_sync(dev_)); }

private:
  Handle(Backend b, fb_device *d) : backend_(b), dev_(d) {}
  static ErrorOr<Handle> open(Backend backend, int deviceId, uintptr_t stream, bool streamGiven) {
    FUSILLI_LOG_LABEL_ENDL("INFO: Creating handle for backend: " << backend << " on device: " << deviceId);
    FUSILLI_RETURN_ERROR_IF(backend != Backend::CUDA && streamGiven, ErrorCode::InvalidArgument,
                            "Stream can only be set on the CUDA backend");
    FUSILLI_RETURN_ERROR_IF(backend != Backend::CUDA, ErrorCode::NotImplemented,
                            "Only Backend::CUDA is executable in this build (no CPU or AMDGPU path)");
    fb_device *dev = nullptr;
    FUSILLI_FB_CALL(fb_device_open(deviceId, reinterpret_cast<void *>(stream), &dev));
    return ok(Handle(backend, dev));
  }
  void reset() {
    if (dev_) fb_device_close(dev_);
    dev_ = nullptr;
  }
  Backend backend_ = Backend::CUDA;
  fb_device *dev_ = nullptr;
};

class Buffer {
public:
  // Allocates a device buffer of prod(bufferShape) elements and uploads `bufferData`.
  template <typename T>
  static ErrorOr<Buffer> allocate(const Handle &handle, const std::vector<size_t> &bufferShape,
                                  const std::vector<T> &bufferData) {
    size_t expected = bufferShape.empty() ? 0 : 1;
    for (size_t d : bufferShape) expected *= d;
    FUSILLI_RETURN_ERROR_IF(expected == 0, ErrorCode::RuntimeFailure,
                            "Buffer::allocate failed: cannot allocate a buffer with zero size");
    FUSILLI_RETURN_ERROR_IF(bufferData.size() != expected, ErrorCode::RuntimeFailure,
                            "Buffer::allocate failed: bufferData size (" + std::to_string(bufferData.size()) +
                                ") does not match product of bufferShape dimensions (" +
                                std::to_string(expected) + ")");
    fb_buffer *b = nullptr;
    if constexpr (kIsSubByteElement<T>) {
      // sub-byte elements travel packed (reference runtime.h:556-560)
      const std::vector<uint8_t> packed = T::pack(bufferData);
      FUSILLI_FB_CALL(fb_buffer_alloc(handle.device(), packed.size(), &b));
      Buffer out(b);
      out.shape_ = bufferShape;
      FUSILLI_FB_CALL(fb_buffer_h2d(handle.device(), b, packed.data(), packed.size()));
      return ok(std::move(out));
    } else {
      FUSILLI_FB_CALL(fb_buffer_alloc(handle.device(), expected * sizeof(T), &b));
      Buffer out(b);
      out.shape_ = bufferShape;
      FUSILLI_FB_CALL(fb_buffer_h2d(handle.device(), b, bufferData.data(), expected * sizeof(T)));
      return ok(std::move(out));
    }
  }

  static ErrorOr<Buffer> allocateRaw(const Handle &handle, size_t sizeInBytes) {
    FUSILLI_RETURN_ERROR_IF(sizeInBytes == 0, ErrorCode::RuntimeFailure,
                            "Buffer::allocateRaw failed: cannot allocate zero-size buffer");
    fb_buffer *b = nullptr;
    FUSILLI_FB_CALL(fb_buffer_alloc(handle.device(), sizeInBytes, &b));
    return ok(Buffer(b));
  }

  // Shares an existing buffer object: the import holds its own reference.
  static ErrorOr<Buffer> import(fb_buffer *externalBufferView) {
    FUSILLI_RETURN_ERROR_IF(externalBufferView == nullptr, ErrorCode::RuntimeFailure,
                            "Buffer::import failed as externalBufferView* is NULL");
    FUSILLI_FB_CALL(fb_buffer_retain(externalBufferView));
    return ok(Buffer(externalBufferView));
  }
  // Wraps caller-owned device memory (a cudaMalloc'd pointer); never freed here.
  static ErrorOr<Buffer> import(const Handle &handle, void *devicePtr, size_t sizeInBytes) {
    FUSILLI_RETURN_ERROR_IF(devicePtr == nullptr, ErrorCode::RuntimeFailure,
                            "Buffer::import failed as externalBufferView* is NULL");
    fb_buffer *b = nullptr;
    FUSILLI_FB_CALL(fb_buffer_wrap(handle.device(), devicePtr, sizeInBytes, &b));
    return ok(Buffer(b));
  }
  // The same with the dims of the dense array behind the pointer, which a graph with dynamic dims
  // reads at execute (the reference's imported buffer views carry their shape, runtime.h:596-611).
  static ErrorOr<Buffer> import(const Handle &handle, void *devicePtr, size_t sizeInBytes,
                                const std::vector<size_t> &bufferShape) {
    FUSILLI_ASSIGN_OR_RETURN(Buffer out, import(handle, devicePtr, sizeInBytes));
    out.shape_ = bufferShape;
    return ok(std::move(out));
  }

  // Device -> host copy of the whole buffer; synchronises the handle's stream.
  template <typename T> ErrorObject read(const Handle &handle, std::vector<T> &outData) {
    FUSILLI_RETURN_ERROR_IF(!outData.empty(), ErrorCode::RuntimeFailure,
                            "Buffer::read failed as outData is NOT empty");
    const size_t bytes = fb_buffer_size(buf_);
    if constexpr (kIsSubByteElement<T>) {
      // the element count comes from the shape when there is one, else two per byte
      std::vector<uint8_t> raw(bytes);
      FUSILLI_FB_CALL(fb_buffer_d2h(handle.device(), buf_, raw.data(), bytes));
      size_t count = bytes * 2;
      if (!shape_.empty()) {
        count = 1;
        for (size_t d : shape_) count *= d;
      }
      outData = T::unpack(raw.data(), count);
    } else {
      outData.resize(bytes / sizeof(T));
      FUSILLI_FB_CALL(fb_buffer_d2h(handle.device(), buf_, outData.data(), outData.size() * sizeof(T)));
    }
    return ok();
  }

  operator fb_buffer *() const { return buf_; }
  void *devicePointer() const { return fb_buffer_ptr(buf_); }
  size_t sizeInBytes() const { return fb_buffer_size(buf_); }
  // Dims of the dense (physical order) array the buffer was allocated for; empty when unknown.
  const std::vector<size_t> &getShape() const { return shape_; }
  Buffer &setShape(const std::vector<size_t> &shape) {
    shape_ = shape;
    return *this;
  }

  Buffer(const Buffer &) = delete;
  Buffer &operator=(const Buffer &) = delete;
  Buffer(Buffer &&o) noexcept : buf_(std::exchange(o.buf_, nullptr)), shape_(std::move(o.shape_)) {}
  Buffer &operator=(Buffer &&o) noexcept {
    if (this != &o) {
      if (buf_) fb_buffer_release(buf_);
      buf_ = std::exchange(o.buf_, nullptr);
      shape_ = std::move(o.shape_);
    }
    return *this;
  }
  ~Buffer() {
    if (buf_) fb_buffer_release(buf_);
  }

private:
  explicit Buffer(fb_buffer *b) : buf_(b) {}
  fb_buffer *buf_ = nullptr;
  std::vector<size_t> shape_;
};

} // namespace fusilli

#endif // FUSILLI_BACKEND_H
