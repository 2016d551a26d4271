// Per-translation-unit device status word.  Kernels never trap or spin forever: a bounded wait that
// gives up, or a self-check that finds a bad index, ORs a code into this word and carries on to its normal
// exit.  Each .cu file that includes this header owns one word and registers a reader for it; the host
// entry point afb_status_read() ORs all of them together (and optionally clears them) after a
// synchronise.
#pragma once
#include <cuda_runtime.h>

namespace afb {

enum StatusCode : int {
  kStatusOk = 0,
  kStatusTmaWaitTimeout = 1 << 0,      // consumer waited for a TMA stage that never filled
  kStatusEmptyWaitTimeout = 1 << 1,    // producer waited for a stage that was never released
  kStatusMmaWaitTimeout = 1 << 2,      // epilogue waited for accumulators that never completed
  kStatusDequantWaitTimeout = 1 << 3,  // MMA warp waited for a dequantised stage
  kStatusPeerFlagTimeout = 1 << 4,     // wait on a flag another GPU writes ran out
  kStatusBadIndex = 1 << 5,            // a bounds self-check rejected an index (access skipped)
  kStatusTmemFull = 1 << 6,
  kStatusGridFlagTimeout = 1 << 7,     // wait on a flag another CTA of the same grid writes ran out
};

// Codes that mean "a wait gave up": once one is recorded, later waits of the same library file give up at once.
constexpr int kStatusAnyWaitTimeout = kStatusTmaWaitTimeout | kStatusEmptyWaitTimeout | kStatusMmaWaitTimeout |
                                      kStatusDequantWaitTimeout | kStatusPeerFlagTimeout | kStatusGridFlagTimeout;

typedef int (*StatusReader)(int clear);
// ORs `code` into the file's status word from the host, on `stream`, while kernels may be running.
typedef int (*StatusPoisoner)(int code, cudaStream_t stream);
// Defined in runtime.cu.
void register_status_reader(StatusReader fn);
void register_status_poisoner(StatusPoisoner fn);

}  // namespace afb

static __device__ int g_afb_status = 0;

namespace afb {
__device__ __forceinline__ void status_set(int code) { atomicOr(&g_afb_status, code); }
// Current value of this file's status word (uncached read).
__device__ __forceinline__ int status_peek() { return *reinterpret_cast<volatile int*>(&g_afb_status); }
}  // namespace afb

namespace {
struct AfbStatusRegistration {
  AfbStatusRegistration() {
    afb::register_status_reader(+[](int clear) -> int {
      int v = 0;
      if (cudaMemcpyFromSymbol(&v, g_afb_status, sizeof(int)) != cudaSuccess) return -1;
      if (clear && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_afb_status, &z, sizeof(int));
      }
      return v;
    });
    // Host-side poison: kernels spinning in a bounded wait re-read the word (uncached) and give up at once.
    // The value is written, not OR-ed: the host cannot read-modify-write under a running kernel, and a set
    // timeout code is all the waits look for.
    afb::register_status_poisoner(+[](int code, cudaStream_t stream) -> int {
      static int staged;
      staged = code;
      return cudaMemcpyToSymbolAsync(g_afb_status, &staged, sizeof(int), 0, cudaMemcpyHostToDevice, stream) ==
                     cudaSuccess
                 ? 0
                 : -1;
    });
  }
};
static AfbStatusRegistration g_afb_status_registration;
}  // namespace
