// GPU allocator and tensor factory: the slot the reference leaves empty
// (src/device_gpu.cpp).  Policy mirrors src/device_npu.cpp:22-77.
#include "device.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>

namespace {
void *cuda_backend_alloc(size_t bytes) {
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "GPUAllocator: cudaMalloc(%zu) failed: %s\n", bytes, cudaGetErrorString(e));
    return nullptr;
  }
  return p;
}
void cuda_backend_free(void *p) { cudaFree(p); }
constexpr size_t kGranule = 512;
} // namespace

GPUAllocator &GPUAllocator::GetInstance() {
  static GPUAllocator instance;
  return instance;
}

void *GPUAllocator::Allocate(size_t size) { return GetInstance().AllocateImpl(size); }
void GPUAllocator::Deallocate(void *ptr) { GetInstance().DeallocateImpl(ptr); }

GPUAllocator::Pool &GPUAllocator::CurrentPool() {
  int dev = 0;
  if (!alloc_fn_) cudaGetDevice(&dev); // a replaced backend has no notion of devices
  return pools_[dev];
}

void *GPUAllocator::AllocateImpl(size_t size) {
  if (size == 0) size = 1;
  size = (size + kGranule - 1) / kGranule * kGranule;
  std::lock_guard<std::mutex> lk(mu_);
  Pool &pool = CurrentPool();
  auto it = pool.free_blocks.lower_bound(size); // smallest pooled block that fits
  if (it != pool.free_blocks.end()) {
    void *p = it->second;
    pool.stats.pooled_bytes -= it->first;
    pool.stats.pool_hits += 1;
    pool.free_blocks.erase(it);
    return p;
  }
  void *p = alloc_fn_ ? alloc_fn_(size) : cuda_backend_alloc(size);
  if (!p) {
    // out of memory: give the pool back and try once more
    for (auto &kv : pool.free_blocks) {
      (free_fn_ ? free_fn_ : cuda_backend_free)(kv.second);
      pool.stats.backend_bytes -= kv.first;
      pool.stats.backend_frees += 1;
      pool.ptr_size.erase(kv.second);
    }
    pool.free_blocks.clear();
    pool.stats.pooled_bytes = 0;
    p = alloc_fn_ ? alloc_fn_(size) : cuda_backend_alloc(size);
    if (!p) return nullptr;
  }
  pool.stats.backend_bytes += size;
  pool.stats.backend_allocs += 1;
  pool.ptr_size[p] = size;
  // over the limit: release pooled blocks, smallest first (src/device_npu.cpp:47-53)
  for (auto fit = pool.free_blocks.begin(); fit != pool.free_blocks.end() && pool.stats.backend_bytes > limit_;) {
    (free_fn_ ? free_fn_ : cuda_backend_free)(fit->second);
    pool.stats.backend_bytes -= fit->first;
    pool.stats.pooled_bytes -= fit->first;
    pool.stats.backend_frees += 1;
    pool.ptr_size.erase(fit->second);
    fit = pool.free_blocks.erase(fit);
  }
  return p;
}

void GPUAllocator::DeallocateImpl(void *ptr) {
  if (!ptr) return;
  std::lock_guard<std::mutex> lk(mu_);
  // the block belongs to the pool of the device it came from
  for (auto &dp : pools_) {
    auto it = dp.second.ptr_size.find(ptr);
    if (it != dp.second.ptr_size.end()) {
      dp.second.free_blocks.emplace(it->second, ptr);
      dp.second.stats.pooled_bytes += it->second;
      return;
    }
  }
  std::fprintf(stderr, "GPUAllocator: pointer %p was not allocated here\n", ptr);
}

GPUAllocator::Stats GPUAllocator::GetStats() {
  GPUAllocator &a = GetInstance();
  std::lock_guard<std::mutex> lk(a.mu_);
  return a.CurrentPool().stats;
}

void GPUAllocator::Trim() {
  GPUAllocator &a = GetInstance();
  std::lock_guard<std::mutex> lk(a.mu_);
  Pool &pool = a.CurrentPool();
  for (auto &kv : pool.free_blocks) {
    (a.free_fn_ ? a.free_fn_ : cuda_backend_free)(kv.second);
    pool.stats.backend_bytes -= kv.first;
    pool.stats.backend_frees += 1;
    pool.ptr_size.erase(kv.second);
  }
  pool.free_blocks.clear();
  pool.stats.pooled_bytes = 0;
}

void GPUAllocator::SetLimit(size_t bytes) {
  GPUAllocator &a = GetInstance();
  std::lock_guard<std::mutex> lk(a.mu_);
  a.limit_ = bytes;
}

void GPUAllocator::SetBackend(BackendAlloc alloc_fn, BackendFree free_fn) {
  GPUAllocator &a = GetInstance();
  std::lock_guard<std::mutex> lk(a.mu_);
  a.alloc_fn_ = alloc_fn;
  a.free_fn_ = free_fn;
  a.pools_.clear();
}

// ---- CPU allocator (src/device_cpu.cpp:5-27) ----------------------------------
CPUAllocator &CPUAllocator::GetInstance() {
  static CPUAllocator instance;
  return instance;
}
void *CPUAllocator::Allocate(size_t size) { return std::malloc(size); }
void CPUAllocator::Deallocate(void *ptr) { std::free(ptr); }

// ---- Tensor (src/device.cpp:6-64, src/device_npu.cpp:70-77) -------------------
std::shared_ptr<Tensor> Tensor::MakeCPUTensor(size_t size, DataType dtype) {
  auto t = std::make_shared<Tensor>();
  t->data_size = size;
  t->data_ptr = CPUAllocator::Allocate(SizeOfTensor(size, dtype));
  t->data_type = dtype;
  t->dev_type = DEV_CPU;
  return t;
}

std::shared_ptr<Tensor> Tensor::MakeGPUTensor(size_t size, DataType dtype) {
  auto t = std::make_shared<Tensor>();
  t->data_size = size;
  t->data_ptr = GPUAllocator::Allocate(SizeOfTensor(size, dtype));
  t->data_type = dtype;
  t->dev_type = DEV_GPU;
  return t;
}

Tensor::~Tensor() {
  switch (dev_type) {
  case DEV_GPU:
    GPUAllocator::Deallocate(data_ptr);
    break;
  case DEV_CPU:
    CPUAllocator::Deallocate(data_ptr);
    break;
  default:
    break;
  }
}

std::shared_ptr<Tensor> Tensor::to(DeviceType to_dev) {
  if (to_dev == dev_type) return shared_from_this();
  const size_t bytes = SizeOfTensor(data_size, data_type);
  if (dev_type == DEV_GPU && to_dev == DEV_CPU) {
    auto r = Tensor::MakeCPUTensor(data_size, data_type);
    cudaMemcpy(r->data_ptr, data_ptr, bytes, cudaMemcpyDeviceToHost);
    return r;
  }
  if (dev_type == DEV_CPU && to_dev == DEV_GPU) {
    auto r = Tensor::MakeGPUTensor(data_size, data_type);
    cudaMemcpy(r->data_ptr, data_ptr, bytes, cudaMemcpyHostToDevice);
    return r;
  }
  return std::shared_ptr<Tensor>();
}

void Tensor::to_file(const char *path) {
  std::shared_ptr<Tensor> host = dev_type == DEV_CPU ? shared_from_this() : to(DEV_CPU);
  std::ofstream ofs(path, std::ios::binary);
  ofs.write(static_cast<const char *>(host->data_ptr), SizeOfTensor(data_size, data_type));
}
