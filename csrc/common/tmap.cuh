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

// One-time, PER-DEVICE kernel set-up.  The shared-memory opt-in of cudaFuncSetAttribute and the occupancy of a
// kernel belong to the device that is current when they are asked for, so a process that drives several GPUs
// has to repeat them on each.  `state` is a call-site (or template-instantiation) static.
//
// tmem_cols > 0 also checks the tensor-memory residency invariant of the tcgen05 kernels: they allocate their
// TMEM columns BEFORE griddepcontrol.wait, i.e. possibly while CTAs of the preceding kernel still hold theirs,
// and tcgen05.alloc blocks (without a bound) until columns are free.  That can only be safe if every CTA that
// the SM can hold at once gets its columns: resident CTAs x columns <= 512.  A configuration that breaks it is
// rejected here, at launch time, instead of deadlocking on the device.
struct PerDeviceOnce {
  unsigned char done[64];
};
int configure_kernel_once(PerDeviceOnce* state, const void* kernel, size_t dyn_smem_bytes, int threads,
                          int tmem_cols, const char* name);
// Number of SMs of the current device (cached per device).
int device_sm_count();

}  // namespace afb

// Runs configure_kernel_once for `kernel` with a static of its own; returns -1 from the calling launcher on error.
#define AFB_CONFIGURE_KERNEL(kernel, smem, threads, tmem_cols)                                              \
  do {                                                                                                      \
    static afb::PerDeviceOnce _afb_once = {};                                                               \
    if (afb::configure_kernel_once(&_afb_once, reinterpret_cast<const void*>(kernel), (smem), (threads),    \
                                   (tmem_cols), #kernel))                                                   \
      return -1;                                                                                            \
  } while (0)

#define AFB_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      afb::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return -1;                                                                          \
    }                                                                                     \
  } while (0)
