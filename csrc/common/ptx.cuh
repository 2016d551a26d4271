// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the kernels in this tree use:
// mbarrier, TMA (cp.async.bulk.tensor, no cluster multicast anywhere), tcgen05 (alloc / mma / commit /
// ld), shared-memory matrix descriptors and instruction descriptors.
//
// Every wait in here is bounded.  A wait that runs out of iterations records an error code in the
// device-global status word (see status.cuh) and returns false; callers fall through to their normal
// exit path so tensor memory is always released and the context stays usable.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.cuh"

namespace afb {

#ifndef AFB_SPIN_LIMIT
#define AFB_SPIN_LIMIT (1u << 24)
#endif
// Wall-clock limit of one wait on data or a flag that ANOTHER GPU writes.  Long enough for the skew between
// ranks at start-up (graph capture, first-use module loads), short enough that a missing rank costs seconds.
#ifndef AFB_PEER_WAIT_NS
#define AFB_PEER_WAIT_NS 2000000000ull
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Deadline of a cross-GPU wait.  expired() is cheap on most polls (the clock and the status word are looked at
// every 32nd call).  Once any cross-GPU wait of this library file has expired, every later one gives up on its
// first poll: the kernels still queued behind a failure (a whole CUDA graph of them) then drain in microseconds
// instead of serving one limit each, and the host finds the status word set.
struct PeerDeadline {
  uint64_t t0;
  uint32_t polls;
  __device__ __forceinline__ PeerDeadline() : t0(0), polls(0) {}
  __device__ __forceinline__ bool expired() {
    if ((polls++ & 31u) != 0u) return false;
    if (status_peek() & kStatusPeerFlagTimeout) return true;
    const uint64_t now = globaltimer_ns();
    if (t0 == 0) {
      t0 = now | 1ull;
      return false;
    }
    return now - t0 > AFB_PEER_WAIT_NS;
  }
};

// Counters that other GPUs bump (monotonic; never reset, so there is no reset to race with).  The producer's
// stores to this GPU's memory are ordered before its red.release; the consumer's ld.acquire orders its reads
// after them.  The comparison is wrap-safe.
__device__ __forceinline__ int peer_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void peer_red_release_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded: false (status recorded) when the counter has not reached `target` within AFB_PEER_WAIT_NS, or at once
// when an earlier cross-GPU wait of this file already expired or the host poisoned the waits.
__device__ __forceinline__ bool peer_wait_counter(const int* p, int target) {
  PeerDeadline dl;
  for (uint32_t it = 0; it < AFB_SPIN_LIMIT; ++it) {
    if (peer_ld_acquire(p) - target >= 0) return true;
    if (dl.expired()) break;
    __nanosleep(40);
  }
  status_set(kStatusPeerFlagTimeout);
  return false;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false (and records `code`) when the limit is hit: an iteration cap, a wall-clock limit
// (AFB_LOCAL_WAIT_NS, looked at every 64th poll), or -- so that whatever is queued behind a failure drains at
// once -- a wait-timeout code already recorded by this library file.
#ifndef AFB_LOCAL_WAIT_NS
#define AFB_LOCAL_WAIT_NS 2000000000ull
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < AFB_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u) {
      if (status_peek() & kStatusAnyWaitTimeout) break;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now | 1ull;
      else if (now - t0 > AFB_LOCAL_WAIT_NS) break;
    }
  }
  status_set(code);
  return false;
}

// ----------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may start
// while its predecessor in the stream is still running: everything before griddep_wait() (barrier init, tensor
// memory allocation, descriptor prefetch, loads of data the predecessor does not produce, e.g. weights)
// overlaps the predecessor's tail; griddep_wait() returns once the predecessor has completed and its writes are
// visible.  griddep_launch() lets this kernel's own successor begin launching.  Both are no-ops for a kernel
// launched without the attribute.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// Thread-block clusters: distributed shared memory and the cluster barrier.  A kernel launched without a
// cluster dimension is a cluster of one, for which these degenerate to CTA-local operations.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_num_ctas() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Shared-window address of `local_addr` (a shared::cta address of this CTA) inside CTA `cta_rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ float4 ld_shared_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
// Every thread of every CTA of the cluster must execute both halves (warp-converged).
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// Flag-free cross-GPU hand-off of bf16 rows (Lamport-style): a slot holds the sentinel 0x8000 (bf16 -0.0) in
// every element until data lands; producers never send the sentinel, consumers poll the data and put the
// sentinel back.  Works at any store-tearing granularity of two bytes or more because every element is checked.
// ----------------------------------------------------------------------------------------------
constexpr uint32_t kLamportSentinelX2 = 0x80008000u;
__device__ __forceinline__ uint32_t lamport_clean_bf16x2(uint32_t w) {
  if ((w & 0xFFFFu) == 0x8000u) w &= 0xFFFF0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000FFFFu;
  return w;
}
// True if any 16-bit lane of w equals 0x8000 (zero-halfword test on w ^ 0x80008000).
__device__ __forceinline__ bool lamport_pending_x2(uint32_t w) {
  const uint32_t x = w ^ kLamportSentinelX2;
  return ((x - 0x00010001u) & ~x & 0x80008000u) != 0u;
}
__device__ __forceinline__ bool lamport_pending(const uint4& u) {
  return lamport_pending_x2(u.x) || lamport_pending_x2(u.y) || lamport_pending_x2(u.z) || lamport_pending_x2(u.w);
}
__device__ __forceinline__ void st_relaxed_sys_v4(void* p, const uint4& u) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 u;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
               : "l"(p)
               : "memory");
  return u;
}

// ----------------------------------------------------------------------------------------------
// Proxy fences
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  // Orders generic-proxy writes to shared memory before async-proxy reads (tcgen05.mma, TMA store).
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// TMA (tiled loads into this CTA's shared memory; never multicast)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ----------------------------------------------------------------------------------------------
// Whole-warp call.  Writes the TMEM base address of `ncols` columns (power of two, >= 32) to *dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: descriptors
// ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes and which was written with
// the 128-byte swizzle (TMA SWIZZLE_128B or the same XOR pattern applied by hand).  Groups of 8 rows are
// 1024 bytes apart.  The tile base must be 1024-byte aligned; a K step of 16 bf16 (32 bytes) inside the
// swizzle atom is taken by adding 32 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;                     // SWIZZLE_128B
  return d;
}

// MN-major tile, 128-byte swizzle: 64 contiguous 16-bit elements along MN per row of 128 bytes, rows run
// along K, groups of 8 K-rows are 1024 bytes apart (stride byte offset); successive 64-element MN panels
// are `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B, fp32 accumulate.
// a_mn / b_mn: 0 = K-major operand, 1 = MN-major operand.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn = 0, int b_mn = 0) {
  return (1u << 4)                               // D format fp32
         | (1u << 7)                             // A format bf16
         | (1u << 10)                            // B format bf16
         | (static_cast<uint32_t>(a_mn) << 15)   // A major
         | (static_cast<uint32_t>(b_mn) << 16)   // B major
         | (static_cast<uint32_t>(N >> 3) << 17) // N / 8
         | (static_cast<uint32_t>(M >> 4) << 24);  // M / 16
}

// Instruction descriptor for kind::f8f6f4 with e4m3 A/B, fp32 accumulate (K = 32 per instruction).
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int M, int N) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// ----------------------------------------------------------------------------------------------
// tcgen05: MMA issue / commit (single thread)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// A operand read from tensor memory (bf16 packed two per 32-bit column), B from shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_e4m3(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued by this thread so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: TMEM -> registers.  32x32b shape: thread i of the warp reads lane (base_lane + i); .xN reads N
// consecutive 32-bit columns.  A warp may only touch the 32 lanes of its own quarter (warp_id % 4).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// registers -> TMEM (same lane/column addressing as the load).
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// Small numeric helpers shared by kernels
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// GELU for bf16 outputs.  The erf form and the tanh form differ by < 5e-4 everywhere and the hardware tanh adds
// < 1e-3 * |x|, both well under half a bf16 ulp of the result wherever the result is not tiny (and the two forms
// agree to 1e-5 where it is), so the "exact" activation is evaluated with one MUFU op instead of an erf: the
// epilogue of the encoder FFN GEMM is special-function-unit bound otherwise.
__device__ __forceinline__ float gelu_erf(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  return 0.5f * x * (1.0f + tanh_approx(u));
}
__device__ __forceinline__ float gelu_tanh(float x) { return gelu_erf(x); }
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }
// x * sigmoid(1.702 x): the activation of the original CLIP checkpoints and of Qwen2-VL's vision blocks.
__device__ __forceinline__ float quick_gelu(float x) { return x / (1.0f + __expf(-1.702f * x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// e8m0 block-scale exponent byte -> float (2^(e-127)); e == 0 is the subnormal 2^-127.
__device__ __forceinline__ float e8m0_to_float(uint8_t e) {
  uint32_t bits = e ? (static_cast<uint32_t>(e) << 23) : 0x00400000u;
  return __uint_as_float(bits);
}

// Four packed e4m3 bytes -> four bf16 (two bf16x2 words: elements 0,1 and 2,3) without conversion instructions:
// the 7 exponent + mantissa bits dropped into bf16 bit positions 10..4 read as the same value times 2^-120
// (subnormals included), so one packed bf16 multiply by `scale2` = bf16x2(2^120 * s) finishes the job exactly
// for any power-of-two s.  kE4m3ToBf16Unit is the multiplier for s = 1.
constexpr uint32_t kE4m3ToBf16Unit = 0x7B807B80u;  // bf16 2^120 in both lanes (exponent field 247)
__device__ __forceinline__ void e4m3x4_to_bf16x4(uint32_t w, uint32_t scale2, uint32_t& lo01, uint32_t& hi23) {
  const uint32_t lo = __byte_perm(w, 0u, 0x1404);  // bytes 0,1 -> high byte of each 16-bit lane
  const uint32_t hi = __byte_perm(w, 0u, 0x3424);  // bytes 2,3
  const uint32_t blo = ((lo >> 4) & 0x07F007F0u) | (lo & 0x80008000u);
  const uint32_t bhi = ((hi >> 4) & 0x07F007F0u) | (hi & 0x80008000u);
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(lo01) : "r"(blo), "r"(scale2));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(hi23) : "r"(bhi), "r"(scale2));
}

// Two packed e4m3 bytes -> two floats.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}

}  // namespace afb
