// Host-side helpers that build TMA tensor maps without linking libcuda: the encoder is looked up through
// the runtime's driver entry-point query, so the library loads on a machine that has no driver installed
// (the build box) and only needs the driver once a kernel is launched.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace afb {

// Returns 0 on success; a negative value if the encoder is unavailable or rejects the arguments.
// 2-D row-major matrix [rows, cols] of `elem_bytes`-sized elements with row pitch `pitch_bytes`;
// box = [box_rows, box_cols]; swizzle: 0 none, 1 32B, 2 64B, 3 128B.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle);

// 3-D [d2, d1, d0] with d0 innermost (contiguous); strides in bytes for d1 and d2.
int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                 int swizzle);

// Launch with the programmatic-dependent-launch attribute when enabled (afb_set_pdl), plain launch otherwise.
// Only kernels that call griddep_wait() before touching global memory may be launched through this.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// As launch_pdl, with the grid partitioned into thread-block clusters of `cluster` CTAs (grid dimensions must be
// multiples of the cluster dimensions).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster.x;
  attr[1].val.clusterDim.y = cluster.y;
  attr[1].val.clusterDim.z = cluster.z;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

const char* last_error();
void set_last_error(const char* fmt, ...);

}  // namespace afb

#define AFB_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      afb::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return -1;                                                                          \
    }                                                                                     \
  } while (0)
