// Device and data type codes shared by every operator of the GPU library.
//
// The numeric values are those of the reference's prebuild/defs.hpp:6-18, so a
// DataType that the reference's model code holds can be passed through
// unchanged (DT_FLOAT16 = 4, DT_BFLOAT16 = 5, DT_FLOAT32 = 6).
#pragma once

#include <cstddef>
#include <cstdint>

enum DeviceType { DEV_CPU = 0, DEV_GPU, DEV_NPU };

enum DataType : int32_t {
  DT_UINT8 = 0,
  DT_INT8,
  DT_UINT32,
  DT_INT32,
  DT_FLOAT16,
  DT_BFLOAT16,
  DT_FLOAT32,
  DT_UINT64,
  DT_INT64,
};

// Bytes taken by `size` elements of `dt` (reference: prebuild/defs.hpp:20-41).
// Unknown types give (size_t)-1, as the reference does.
inline size_t SizeOfTensor(size_t size, DataType dt) {
  switch (dt) {
  case DT_UINT8:
  case DT_INT8:
    return size;
  case DT_FLOAT16:
  case DT_BFLOAT16:
    return size * 2;
  case DT_UINT32:
  case DT_INT32:
  case DT_FLOAT32:
    return size * 4;
  case DT_UINT64:
  case DT_INT64:
    return size * 8;
  }
  return static_cast<size_t>(-1);
}
