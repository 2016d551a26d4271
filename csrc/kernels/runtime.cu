// Library-wide host runtime: error string, status-word registry, TMA tensor-map encoder lookup.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <vector>

#include "../common/status.cuh"
#include "../common/tmap.cuh"

namespace afb {

namespace {
thread_local char g_err[512] = {0};

std::vector<StatusReader>& readers() {
  static std::vector<StatusReader> r;
  return r;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

CUtensorMapDataType dtype_for(int elem_bytes) {
  switch (elem_bytes) {
    case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case 4: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

CUtensorMapSwizzle swizzle_for(int s) {
  switch (s) {
    case 1: return CU_TENSOR_MAP_SWIZZLE_32B;
    case 2: return CU_TENSOR_MAP_SWIZZLE_64B;
    case 3: return CU_TENSOR_MAP_SWIZZLE_128B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}
}  // namespace

void register_status_reader(StatusReader fn) { readers().push_back(fn); }

namespace {
std::vector<StatusPoisoner>& poisoners() {
  static std::vector<StatusPoisoner> p;
  return p;
}
}  // namespace
void register_status_poisoner(StatusPoisoner fn) { poisoners().push_back(fn); }
int poison_all(int code, int device) {
  // The current device belongs to the calling host thread: a watchdog or timer thread starts on device 0
  // whatever the main thread selected, and the status words are per-device copies.  So the caller names the
  // device (negative = keep the thread's current one) and the write goes to that device's words, on a stream of
  // that device: non-blocking with respect to the default stream, so the writes overtake whatever kernels are
  // queued or spinning on the compute streams.
  if (device >= 0 && cudaSetDevice(device) != cudaSuccess) return -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  static cudaStream_t streams[64] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  cudaStream_t& s = streams[dev];
  if (!s && cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return -1;
  int rc = 0;
  for (auto fn : poisoners()) rc |= fn(code, s);
  if (cudaStreamSynchronize(s) != cudaSuccess) rc = -1;
  return rc;
}

int g_pdl = -1;
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("ANTFLY_B200_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}

const char* last_error() { return g_err; }

int configure_kernel_once(PerDeviceOnce* state, const void* kernel, size_t dyn_smem_bytes, int threads,
                          int tmem_cols, const char* name) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_error("%s: no current CUDA device", name);
    return -1;
  }
  // Racing first calls from two host threads both do the same idempotent set-up and store the same byte.
  if (state->done[dev]) return 0;
  if (dyn_smem_bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dyn_smem_bytes));
    if (e != cudaSuccess) {
      set_last_error("%s: cannot opt in to %zu bytes of shared memory on device %d: %s", name, dyn_smem_bytes, dev,
                     cudaGetErrorString(e));
      return -1;
    }
  }
  if (tmem_cols > 0) {
    int resident = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, threads, dyn_smem_bytes);
    if (e != cudaSuccess) {
      set_last_error("%s: occupancy query failed: %s", name, cudaGetErrorString(e));
      return -1;
    }
    if (resident * tmem_cols > 512) {
      set_last_error("%s: %d resident CTAs x %d tensor-memory columns exceed the 512 columns of an SM; a CTA "
                     "could block in tcgen05.alloc behind dependents parked in griddepcontrol.wait", name, resident,
                     tmem_cols);
      return -1;
    }
  }
  state->done[dev] = 1;
  return 0;
}

int device_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    sms[dev] = n;
  }
  return sms[dev];
}

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  EncodeTiledFn enc = get_encoder();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) {
    set_last_error("TMA operand must be 16-byte aligned with a 16-byte multiple pitch (base=%p pitch=%llu)", base,
                   (unsigned long long)pitch_bytes);
    return -2;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype_for(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(2d) failed with %d (rows=%llu cols=%llu pitch=%llu box=%ux%u)", (int)r,
                   (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows,
                   box_cols);
    return -3;
  }
  return 0;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                 int swizzle) {
  EncodeTiledFn enc = get_encoder();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) {
    set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple strides");
    return -2;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dtype_for(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(3d) failed with %d", (int)r);
    return -3;
  }
  return 0;
}

}  // namespace afb

extern "C" {

const char* afb_last_error() { return afb::last_error(); }

// ORs the status words of every kernel file; clears them when `clear` is non-zero.  Call after a
// synchronise.  Returns a negative value if a word could not be read.
int afb_status_read(int clear) {
  int v = 0;
  for (auto fn : afb::readers()) {
    int s = fn(clear);
    if (s < 0) return -1;
    v |= s;
  }
  return v;
}

// Makes every bounded wait of every kernel file give up at once, including waits of kernels that are running or
// queued right now (a CUDA graph full of cross-GPU hand-offs whose peer will never answer): the timeout code is
// written into each status word from a side stream.  Call before tearing a process down on a watchdog or signal,
// so the GPU drains in microseconds and is idle when the process exits.  afb_status_read(1) clears it again.
int afb_poison_waits() { return afb::poison_all(afb::kStatusPeerFlagTimeout, -1); }
// The same for a named device: for a thread other than the one that launched the work (watchdog timers, signal
// helpers), whose current device is 0 by default.  Leaves `device` current in the calling thread.
int afb_poison_waits_on(int device) { return afb::poison_all(afb::kStatusPeerFlagTimeout, device); }
int afb_device_sm_count() { return afb::device_sm_count(); }

// Programmatic dependent launch on (1) / off (0) for the kernels that support it; default on, or
// ANTFLY_B200_PDL=0 in the environment.
void afb_set_pdl(int on) { afb::g_pdl = on ? 1 : 0; }
int afb_get_pdl() { return afb::pdl_enabled() ? 1 : 0; }

int afb_num_status_words() { return static_cast<int>(afb::readers().size()); }

}  // extern "C"
