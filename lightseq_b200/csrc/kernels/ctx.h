// Internal definition of the opaque ls100_ctx handle.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <mutex>
#include <utility>
#include <unordered_map>

#include "../../../include/ls100.h"

typedef CUresult (*ls100_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                          const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                          CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                          CUtensorMapFloatOOBfill);

struct ls100_tmap_key {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  bool operator==(const ls100_tmap_key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols;
  }
};
struct ls100_tmap_hash {
  size_t operator()(const ls100_tmap_key& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9E3779B97F4A7C15ull;
    h ^= k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.ld + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.box_rows << 32 | k.box_cols) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    return (size_t)h;
  }
};

struct ls100_ctx {
  int device = 0;
  int sm_count = 0;
  int* d_err = nullptr;  // device error word written by bounded waits
  ls100_encode_tiled_fn encode = nullptr;
  std::mutex mu;
  std::unordered_map<ls100_tmap_key, CUtensorMap, ls100_tmap_hash> tmaps;
};

// True unless the environment sets LS100_PDL=0: kernels are then launched with the programmatic
// stream-serialisation attribute so that each kernel's prologue overlaps its predecessor's tail.
bool ls100_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t ls100_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  if (ls100_pdl_enabled()) {
    cfg.attrs = at;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// The same with the CTAs grouped into thread-block clusters of cluster_x along grid.x.
template <typename... KArgs, typename... Args>
inline cudaError_t ls100_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                        unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cluster_x;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = ls100_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// 2-D uint8 tensor map, 128-byte swizzle, box = box_cols (bytes, <=128) x box_rows.
int ls100_get_tmap_u8(ls100_ctx* ctx, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld_bytes,
                      uint32_t box_rows, uint32_t box_cols, CUtensorMap* out);
