// Device abstraction of the GPU backend: allocators and the flat Tensor.
//
// Same public surface as the reference's src/device.hpp:9-55 (CPUAllocator,
// NPUAllocator -> GPUAllocator, Tensor with Make*Tensor / to / to_file), with
// the GPU slot the reference leaves empty (src/device_gpu.cpp is a 0-byte file,
// DEV_GPU exists in prebuild/defs.hpp:6) filled in.
#pragma once

#include <cstddef>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "defs.hpp"

class CPUAllocator {
public:
  static CPUAllocator &GetInstance();
  static void *Allocate(size_t size);
  static void Deallocate(void *ptr);
};

// Pooling allocator over cudaMalloc, one pool per device.
//
// Same policy as the reference's NPUAllocator (src/device_npu.cpp:22-67): a
// request is served by the smallest pooled block that is large enough, else by
// the backend; freed blocks go back to the pool; when the bytes obtained from
// the backend exceed the limit, pooled blocks are released smallest first.
// Differences: the pool is an ordered multimap (no list scan, no sort on every
// free), sizes are rounded up to 512 bytes so temporaries of similar size reuse
// one block, it is thread-safe, and the default limit is 64 GiB of a 180 GB part
// (reference: 8 GiB of a 24 GB board).
//
// Like the reference's, the pool is not stream-aware: a block may be handed out
// again as soon as its Tensor dies, so the owner must keep temporaries alive
// until the work that uses them has been ordered before the next user (the
// attention layer runs everything on one stream, which gives that order).
class GPUAllocator {
public:
  struct Stats {
    size_t backend_bytes;  // bytes currently obtained from the backend (in use + pooled)
    size_t pooled_bytes;   // of those, sitting in the pool
    size_t backend_allocs; // backend allocation calls so far
    size_t pool_hits;      // requests served from the pool so far
    size_t backend_frees;
  };
  using BackendAlloc = void *(*)(size_t);
  using BackendFree = void (*)(void *);

  static GPUAllocator &GetInstance();
  static void *Allocate(size_t size);
  static void Deallocate(void *ptr);
  static Stats GetStats();
  static void Trim();                   // release every pooled block of the current device
  static void SetLimit(size_t bytes);   // backend-bytes threshold above which the pool is trimmed
  // Replace cudaMalloc / cudaFree (tests run the pool logic on a host without a GPU).
  static void SetBackend(BackendAlloc alloc_fn, BackendFree free_fn);

private:
  struct Pool {
    std::multimap<size_t, void *> free_blocks;
    std::unordered_map<void *, size_t> ptr_size;
    Stats stats{};
  };
  void *AllocateImpl(size_t size);
  void DeallocateImpl(void *ptr);
  Pool &CurrentPool();

  std::mutex mu_;
  std::map<int, Pool> pools_;
  size_t limit_{64ULL << 30};
  BackendAlloc alloc_fn_{nullptr};
  BackendFree free_fn_{nullptr};
};

class Tensor : public std::enable_shared_from_this<Tensor> {
public:
  Tensor() = default;
  ~Tensor();
  static std::shared_ptr<Tensor> MakeCPUTensor(size_t size, DataType dtype);
  static std::shared_ptr<Tensor> MakeGPUTensor(size_t size, DataType dtype);

  std::shared_ptr<Tensor> to(DeviceType to_dev); // synchronous copy, as the reference's
  void to_file(const char *path);

  void *data_ptr{nullptr};
  size_t data_size{0}; // elements
  DataType data_type{DT_FLOAT16};
  DeviceType dev_type{DEV_CPU};
};
