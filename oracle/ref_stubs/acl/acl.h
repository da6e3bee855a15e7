// Stand-in for the Ascend runtime header: types and entry points the reference's test
// utilities name.  Nothing here is ever called by the pinned functions.
#pragma once
#include <cstddef>
typedef int aclError;
typedef void *aclrtStream;
typedef unsigned short aclFloat16;
#define ACL_ERROR_NONE 0
enum aclrtMemMallocPolicy { ACL_MEM_MALLOC_HUGE_FIRST = 0 };
enum aclrtMemcpyKind { ACL_MEMCPY_HOST_TO_DEVICE = 1, ACL_MEMCPY_DEVICE_TO_HOST = 2 };
aclError aclrtMalloc(void **ptr, size_t size, aclrtMemMallocPolicy policy);
aclError aclrtFree(void *ptr);
aclError aclrtMemcpy(void *dst, size_t dst_max, const void *src, size_t count, aclrtMemcpyKind kind);
aclError aclrtMemset(void *ptr, size_t max, int value, size_t count);
aclError aclrtCreateStream(aclrtStream *stream);
aclError aclrtDestroyStream(aclrtStream stream);
aclError aclrtSynchronizeStream(aclrtStream stream);
