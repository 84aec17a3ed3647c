// NCCL, bound at run time.  The multi-GPU entry points receive the caller's communicator
// (ncclComm_t as void*) and call a handful of NCCL functions on it.  The library is not
// linked against NCCL: the functions are looked up in the libnccl the process has already
// loaded (the one that created the communicator), or in "libnccl.so.2" of the loader path.
// Only declarations of NCCL's public C API appear here (nccl.h: ncclAllGather,
// ncclBroadcast, ncclGroupStart, ncclGroupEnd, ncclCommCount, ncclCommUserRank).
#pragma once

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stddef.h>

namespace mmbo {

constexpr int kNcclFloat16 = 6;  // ncclFloat16 / ncclHalf of ncclDataType_t
constexpr int kNcclUint8 = 1;    // ncclUint8

struct NcclApi {
  bool tried = false;
  void* handle = nullptr;
  int (*all_gather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*broadcast)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*group_start)() = nullptr;
  int (*group_end)() = nullptr;
  int (*comm_count)(void*, int*) = nullptr;
  int (*comm_user_rank)(void*, int*) = nullptr;
  bool ok() const { return all_gather && broadcast && group_start && group_end && comm_count && comm_user_rank; }
};

inline NcclApi& nccl_api() {
  static NcclApi api;
  if (!api.tried) {
    api.tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the process already uses
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    api.handle = h;
    if (h) {
      api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
      api.broadcast = reinterpret_cast<decltype(api.broadcast)>(dlsym(h, "ncclBroadcast"));
      api.group_start = reinterpret_cast<decltype(api.group_start)>(dlsym(h, "ncclGroupStart"));
      api.group_end = reinterpret_cast<decltype(api.group_end)>(dlsym(h, "ncclGroupEnd"));
      api.comm_count = reinterpret_cast<decltype(api.comm_count)>(dlsym(h, "ncclCommCount"));
      api.comm_user_rank = reinterpret_cast<decltype(api.comm_user_rank)>(dlsym(h, "ncclCommUserRank"));
    }
  }
  return api;
}

}  // namespace mmbo
