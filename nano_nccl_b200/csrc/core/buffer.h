// RAII owners for the CUDA memory kinds the library uses.
//
// Parity: reference src/core/buffer.h:33-214 / buffer.cu — DeviceBuffer (cudaMalloc),
// PinnedBuffer, MappedBuffer (host memory mapped into the device address space, allocated while
// the calling thread prefers the NUMA node of the GPU that will read it), and small mapped u64 /
// u32 arrays used for counters and abort words.  Here the mapped kinds share one untyped base so
// the typed wrappers stay header-only.
#pragma once

#include "core/error.h"

#include <cstddef>
#include <cstdint>
#include <utility>

namespace nano_nccl {

class RawDeviceBuffer {
public:
    RawDeviceBuffer() = default;
    RawDeviceBuffer(int device, std::size_t bytes, bool zero = false);
    ~RawDeviceBuffer();
    RawDeviceBuffer(RawDeviceBuffer&& o) noexcept { swap(o); }
    RawDeviceBuffer& operator=(RawDeviceBuffer&& o) noexcept {
        if (this != &o) { release(); swap(o); }
        return *this;
    }
    RawDeviceBuffer(const RawDeviceBuffer&) = delete;
    RawDeviceBuffer& operator=(const RawDeviceBuffer&) = delete;
    void* data() const noexcept { return ptr_; }
    std::size_t bytes() const noexcept { return bytes_; }
    int device() const noexcept { return device_; }
    void release() noexcept;
    // Forgets the allocation without freeing it (teardown after a failed drain: a kernel may still use it).
    void leak() noexcept { ptr_ = nullptr; bytes_ = 0; }

private:
    void swap(RawDeviceBuffer& o) noexcept {
        std::swap(ptr_, o.ptr_); std::swap(bytes_, o.bytes_); std::swap(device_, o.device_);
    }
    void* ptr_ = nullptr;
    std::size_t bytes_ = 0;
    int device_ = -1;
};

template <typename T>
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(int device, std::size_t count, bool zero = false)
        : raw_(device, count * sizeof(T), zero), count_(count) {}
    T* data() const noexcept { return static_cast<T*>(raw_.data()); }
    std::size_t size() const noexcept { return count_; }
    std::size_t bytes() const noexcept { return raw_.bytes(); }

private:
    RawDeviceBuffer raw_;
    std::size_t count_ = 0;
};

// Page-locked host memory; `mapped` also gives a device-side address for it.
class RawHostBuffer {
public:
    RawHostBuffer() = default;
    // numa_node < 0: no placement preference.
    RawHostBuffer(std::size_t bytes, bool mapped, int numa_node = -1);
    ~RawHostBuffer();
    RawHostBuffer(RawHostBuffer&& o) noexcept { swap(o); }
    RawHostBuffer& operator=(RawHostBuffer&& o) noexcept {
        if (this != &o) { release(); swap(o); }
        return *this;
    }
    RawHostBuffer(const RawHostBuffer&) = delete;
    RawHostBuffer& operator=(const RawHostBuffer&) = delete;
    void* host() const noexcept { return host_; }
    // Device-visible alias of the same bytes for the current device (mapped buffers only).
    void* device_pointer() const;
    std::size_t bytes() const noexcept { return bytes_; }
    void release() noexcept;

private:
    void swap(RawHostBuffer& o) noexcept {
        std::swap(host_, o.host_); std::swap(bytes_, o.bytes_); std::swap(mapped_, o.mapped_);
    }
    void* host_ = nullptr;
    std::size_t bytes_ = 0;
    bool mapped_ = false;
};

template <typename T>
class PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(std::size_t count) : raw_(count * sizeof(T), false), count_(count) {}
    T* data() const noexcept { return static_cast<T*>(raw_.host()); }
    std::size_t size() const noexcept { return count_; }

private:
    RawHostBuffer raw_;
    std::size_t count_ = 0;
};

template <typename T>
class MappedBuffer {
public:
    MappedBuffer() = default;
    MappedBuffer(std::size_t count, int numa_node = -1)
        : raw_(count * sizeof(T), true, numa_node), count_(count) {}
    T* host() const noexcept { return static_cast<T*>(raw_.host()); }
    T* device() const { return static_cast<T*>(raw_.device_pointer()); }
    std::size_t size() const noexcept { return count_; }
    std::size_t bytes() const noexcept { return raw_.bytes(); }

private:
    RawHostBuffer raw_;
    std::size_t count_ = 0;
};

// Zero-initialised counters shared between proxy threads and kernels.
using MappedU64Array = MappedBuffer<std::uint64_t>;
using MappedU32Array = MappedBuffer<std::uint32_t>;

// Host memory that does not need CUDA at all (CPU-only tests of proxies and the host ring use it
// in place of MappedBuffer; the proxies only ever see raw pointers).
template <typename T>
class PlainHostArray {
public:
    PlainHostArray() = default;
    explicit PlainHostArray(std::size_t count) : data_(new T[count]()), count_(count) {}
    ~PlainHostArray() { delete[] data_; }
    PlainHostArray(PlainHostArray&& o) noexcept : data_(o.data_), count_(o.count_) {
        o.data_ = nullptr; o.count_ = 0;
    }
    PlainHostArray& operator=(PlainHostArray&& o) noexcept {
        if (this != &o) { delete[] data_; data_ = o.data_; count_ = o.count_; o.data_ = nullptr; o.count_ = 0; }
        return *this;
    }
    T* data() const noexcept { return data_; }
    std::size_t size() const noexcept { return count_; }

private:
    T* data_ = nullptr;
    std::size_t count_ = 0;
};

}  // namespace nano_nccl
