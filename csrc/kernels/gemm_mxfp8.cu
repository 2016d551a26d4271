// Block-scaled fp8 x fp8 GEMM on the native MX path of the 5th-generation tensor cores:
//   out[t, n] = sum_k  (X8[t,k] * 2^(SX[t,k/32]-127))  *  (W8[n,k] * 2^(SW[n,k/32]-127))
// issued as tcgen05.mma.kind::mxf8f6f4.block_scale (e4m3 operands, one e8m0 scale per 32 K elements, applied by
// the tensor core itself from scale factors held in tensor memory).  Nothing but TMA and the tensor core touches
// the weights, so a decode step streams them at memory speed with no CUDA-core work in the loop.
//
// Activations are bf16 in memory between layers; the producer kernel (RMSNorm / activation quantiser below)
// emits them as MX fp8 in one or two terms: x ~= hi, or x ~= hi + lo where lo is the MX-fp8 quantisation of the
// residual x - hi.  Two terms carry about 7 mantissa bits, i.e. bf16-class accuracy, at the cost of a second
// (free at decode) MMA pass over the same weight tile.
//
// This kernel is the skinny-M (decode, speculative verify) linear layer of the decoder; large-M prefill uses
// the W8A16 kernel.  Quantised-matmul counterpart of the reference's Metal mul_mv / mul_mm MXFP4 / NVFP4 kernels
// (zig/pkg/inference/src/backends/metal_kernels.m:3491-3529) and its scalar CUDA Q8_0 / Q4_K linears
// (zig/pkg/inference/src/ops/cuda/artifacts/inference_cuda_kernels.cu:873-1553).
//
// Tile: weights fill the 128 UMMA-M lanes, tokens are UMMA-N (BT = 16..128).  A stage is 128 K elements:
// 128x128 B of weights + BT x 128 B of activations per term, 128-byte swizzle, plus 512-byte scale-factor atoms
// that are copied shared -> tensor memory with tcgen05.cp (32x128b.warpx4) right before the four K=32 MMAs that
// use them (scale-factor byte selected per MMA through the instruction descriptor).
//   warp 0      TMA producer      warp 1   tcgen05.cp + tcgen05.mma issue      warps 2..5  epilogue
//
// Scale-factor atom (512 B, covers 128 rows x 4 K-blocks): byte (r % 32) * 16 + (r / 32) * 4 + kblock.
#include "../common/mxquant.cuh"
#include "../common/ptx.cuh"
#include "../common/tmap.cuh"

namespace afb {

// Kept out of line so the unrolled epilogue does not evaluate every activation for every element.
__device__ __noinline__ float act_one_mx(float x, int act) {
  switch (act) {
    case 1: return gelu_erf(x);
    case 2: return gelu_tanh(x);
    case 3: return fmaxf(x, 0.0f);
    case 4: return silu(x);
    default: return x;
  }
}

struct MxParams {
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const uint8_t* sfw;   // [n_tiles, k_chunks, 512]
  const uint8_t* sfx0;  // [t_tiles, k_chunks, 512]
  const uint8_t* sfx1;  // second term or null
  int M, N, K;
  int ldc, ldr;
  int act;
  int mode;  // 0 bf16 out, 1 fp32 partials, 2 swiglu, 3 push partial tiles to owner ranks, 4 reduce + broadcast
  int chunks_per_split;
  int k_chunks;
  // ---- tensor-parallel fused collectives (unused when world == 0) ----
  // mode 3 (GEMM -> reduce-scatter): the epilogue pushes its fp32 partial tile straight into the symmetric
  // buffer of the rank that owns each token (plain peer stores over NVLink), laid out on the owner as
  // [world * slices][tokens_per_rank][ldc], then bumps this rank's arrival counter on every owner.
  float* peer_parts[8];
  int* peer_part_flags[8];
  int world, my_rank, tokens_per_rank, slices;
  // all-gather -> GEMM: the activation rows are pushed into this rank's X buffers by every rank's producer
  // kernel; the TMA producer streams weight tiles at once and only waits for `x_expected` arrivals before its
  // first activation load.
  int* x_ready;
  int x_expected;
  int* x_consumed;
  // mode 4 (GEMM -> one-shot all-reduce): the split-K CTAs of a tile form a thread-block cluster (1, 1, splits).
  // Each stages its fp32 slice in its own shared memory; after a cluster barrier every CTA sums one share of the
  // tile's rows over all slices (distributed shared memory, slice order), rounds to bf16 and stores the rows into
  // slot `my_rank` of every rank's [world][M][ldc] bf16 buffer (peer_parts reinterpreted).  There is no flag and no
  // fence: the slots hold a sentinel (bf16 -0.0, which the producer never sends: a computed -0.0 goes out as +0.0)
  // until the data lands, and the consumer polls the data itself and restores the sentinel after reading
  // (Lamport-style).  The consumer sums the world slots in rank order, so every rank computes bit-identical sums.
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait on a counter that other GPUs increment.  Returns false (status recorded) on expiry.
__device__ __forceinline__ bool wait_counter_sys(const int* p, int expected) {
  PeerDeadline dl;
  for (uint32_t it = 0; it < AFB_SPIN_LIMIT; ++it) {
    if (ld_acquire_sys(p) >= expected) return true;
    if (dl.expired()) break;
    __nanosleep(20);
  }
  status_set(kStatusPeerFlagTimeout);
  return false;
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Shared-memory descriptor of a 32-row x 16-byte scale-factor atom for tcgen05.cp: no swizzle, 8-row groups
// 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Instruction descriptor, kind::mxf8f6f4 block-scaled, e4m3 x e4m3, ue8m0 scales, K = 32.
__device__ __forceinline__ uint32_t idesc_mx(int M, int N, int a_sf, int b_sf) {
  return (static_cast<uint32_t>(b_sf) << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (1u << 23) | (static_cast<uint32_t>(M >> 4) << 24) | (static_cast<uint32_t>(a_sf) << 29);
}

__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

template <int BT, int STAGES, int TERMS>
struct MxSmem {
  static constexpr int kWBytes = 128 * 128;
  static constexpr int kXBytes = BT * 128;
  static constexpr int kXStage = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kSfBytes = 512;
  static constexpr int kStage = kWBytes + TERMS * kXStage + 1024 + TERMS * 1024;  // SF atoms padded to 1 KiB each
  static constexpr int kBarOff = STAGES * kStage;
  static constexpr int kTotal = kBarOff + (2 * STAGES + 1) * 8 + 16 + 1024;
  static constexpr int kTxBytes = kWBytes + TERMS * kXBytes + (1 + TERMS) * kSfBytes;
};

template <int BT, int STAGES, int TERMS>
__global__ void __launch_bounds__(192, (MxSmem<BT, STAGES, TERMS>::kTotal <= 110 * 1024 ? 2 : 1))
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x0,
                  const __grid_constant__ CUtensorMap tma_x1, MxParams p) {
  using L = MxSmem<BT, STAGES, TERMS>;
  constexpr int D_COLS = BT < 32 ? 32 : BT;
  constexpr int TMEM_COLS = D_COLS <= 32 ? 64 : (D_COLS <= 96 ? 128 : 256);  // D + 12 scale-factor columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, t_tile = blockIdx.y;
  const int n0 = n_tile * 128, t0 = t_tile * BT;
  const int c_begin = blockIdx.z * p.chunks_per_split;
  const int c_end = min(p.k_chunks, c_begin + p.chunks_per_split);
  const int num_c = c_end - c_begin;
  // Scale-factor atoms of the token tile: the atom covers 128 rows, so BT < 128 tiles share an atom.
  const int sfx_tile = t0 / 128;
  const int sfx_row0 = t0 % 128;  // first row of this tile inside the atom

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_w);
    tma_prefetch_desc(&tma_x0);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Dependents may start launching only now that this CTA HOLDS its tensor memory.  The dependent grid begins
  // once every CTA of this grid has passed this point (or exited), so no CTA of this grid can ever be left
  // waiting in tcgen05.alloc (an unbounded hardware wait) for columns held by dependents that are themselves
  // parked in griddepcontrol.wait until this grid completes.
  griddep_launch();

  if (warp == 0) {
    if (lane == 0) {
      auto load_w = [&](int i, int s) {
        uint8_t* st = smem + s * L::kStage;
        const int c = c_begin + i;
        mbar_expect_tx(&full[s], L::kTxBytes);
        tma_load_2d(st, &tma_w, &full[s], c * 128, n0);
        bulk_load(st + L::kWBytes + TERMS * L::kXStage, p.sfw + (static_cast<size_t>(n_tile) * p.k_chunks + c) * 512,
                  512, &full[s]);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* st = smem + s * L::kStage;
        const int c = c_begin + i;
        tma_load_2d(st + L::kWBytes, &tma_x0, &full[s], c * 128, t0);
        if (TERMS == 2) tma_load_2d(st + L::kWBytes + L::kXStage, &tma_x1, &full[s], c * 128, t0);
        uint8_t* sf = st + L::kWBytes + TERMS * L::kXStage;
        bulk_load(sf + 1024, p.sfx0 + (static_cast<size_t>(sfx_tile) * p.k_chunks + c) * 512, 512, &full[s]);
        if (TERMS == 2)
          bulk_load(sf + 2048, p.sfx1 + (static_cast<size_t>(sfx_tile) * p.k_chunks + c) * 512, 512, &full[s]);
      };
      bool alive = true;
      // Weight tiles depend neither on the previous kernel nor on the other ranks: fill the ring with them
      // first, then wait for the predecessor grid (and, tensor-parallel, for the gathered activation rows), then
      // complete those stages with the activation tiles.
      const int pre = min(num_c, STAGES);
      for (int i = 0; i < pre; ++i) load_w(i, i);
      griddep_wait();
      if (p.x_ready) {
        alive = wait_counter_sys(p.x_ready, p.x_expected);
        asm volatile("fence.proxy.async.global;" ::: "memory");
        const int ctas = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(p.x_consumed, 1) == ctas - 1) {
          // Every CTA of this GEMM is past its wait: re-arm the counters for the next use.
          *p.x_consumed = 0;
          atomicExch(p.x_ready, 0);
        }
      }
      for (int i = 0; i < pre; ++i) load_x(i, i);
      const int first = pre;
      for (int i = first; i < num_c && alive; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, kStatusEmptyWaitTimeout)) break;
        load_w(i, s);
        load_x(i, s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t t_sfa = tmem_base + D_COLS;
      const uint32_t t_sfb0 = t_sfa + 4;
      const uint32_t t_sfb1 = t_sfa + 8;
      // Token rows sfx_row0 .. +BT of the atom: row r lives in column r / 32 of the 4-column scale block, so a
      // tile that starts at row 32, 64 or 96 starts that many columns in.  (BT < 32 tiles start on a multiple
      // of BT inside a 32-row group; those use the lane offset implicitly because the MMA reads scale lanes
      // 0..N-1 -- such tiles are only launched with sfx_row0 % 32 == 0.)
      const uint32_t sfb_col = static_cast<uint32_t>(sfx_row0 / 32);
      for (int i = 0; i < num_c; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, kStatusTmaWaitTimeout)) break;
        tcgen05_fence_after();
        uint8_t* st = smem + s * L::kStage;
        uint8_t* sf = st + L::kWBytes + TERMS * L::kXStage;
        tmem_cp_32x128b_warpx4(t_sfa, sf_desc(smem_u32(sf)));
        tmem_cp_32x128b_warpx4(t_sfb0, sf_desc(smem_u32(sf + 1024)));
        if (TERMS == 2) tmem_cp_32x128b_warpx4(t_sfb1, sf_desc(smem_u32(sf + 2048)));
        const uint64_t adesc = umma_desc_k_sw128(smem_u32(st));
        const uint64_t b0desc = umma_desc_k_sw128(smem_u32(st + L::kWBytes));
        const uint64_t b1desc = umma_desc_k_sw128(smem_u32(st + L::kWBytes + L::kXStage));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t id = idesc_mx(128, BT < 16 ? 16 : BT, k, k);
          umma_mx(tmem_base, adesc + 2 * k, b0desc + 2 * k, id, t_sfa, t_sfb0 + sfb_col, (i | k) != 0);
          if (TERMS == 2) umma_mx(tmem_base, adesc + 2 * k, b1desc + 2 * k, id, t_sfa, t_sfb1 + sfb_col, 1);
        }
        umma_commit(&empty[s]);
      }
      umma_commit(tmem_full);
    }
  } else {
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    griddep_wait();
    const bool ok = mbar_wait(tmem_full, 0, kStatusMmaWaitTimeout);
    tcgen05_fence_after();
    if (ok && num_c > 0) {
      const float bias = (p.bias && p.mode != 1 && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
      constexpr int CH = BT < 32 ? 16 : 32;
#pragma unroll 1
      for (int c = 0; c < BT; c += CH) {
        float v[CH];
        if constexpr (CH == 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
        if (p.mode == 3) {
          if (n < p.N) {
            const float inv_tpr = 1.0f / static_cast<float>(p.tokens_per_rank);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int t = t0 + c + j;
              if (t < p.M) {
                const int owner = static_cast<int>((static_cast<float>(t) + 0.5f) * inv_tpr);
                const int row = t - owner * p.tokens_per_rank;
                float* op = p.peer_parts[owner] +
                            (static_cast<size_t>(p.my_rank * p.slices + blockIdx.z) * p.tokens_per_rank + row) * p.ldc;
                op[n] = v[j];
              }
            }
          }
        } else if (p.mode == 4) {
          // Stage the fp32 slice [BT][128] in the (now idle) pipeline stages for the cluster-wide reduction.
          float* stile = reinterpret_cast<float*>(smem);
#pragma unroll
          for (int j = 0; j < CH; ++j) stile[(c + j) * 128 + q * 32 + lane] = v[j];
        } else if (p.mode == 1) {
          float* op = reinterpret_cast<float*>(p.out) + static_cast<size_t>(blockIdx.z) * p.M * p.ldc;
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int t = t0 + c + j;
              if (t < p.M) op[static_cast<size_t>(t) * p.ldc + n] = v[j];
            }
          }
        } else if (p.mode == 2) {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const float mine = v[j] + bias;
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const int t = t0 + c + j;
            if (((lane ^ j) & 1) == 0 && t < p.M && n < p.N) {
              const float g = (lane & 1) ? other : mine;
              const float u = (lane & 1) ? mine : other;
              op[static_cast<size_t>(t) * p.ldc + (n >> 1)] = __float2bfloat16(silu(g) * u);
            }
          }
        } else {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out);
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int t = t0 + c + j;
              if (t < p.M) {
                float x = v[j] + bias;
                if (p.act) x = act_one_mx(x, p.act);
                if (p.residual) x += __bfloat162float(p.residual[static_cast<size_t>(t) * p.ldr + n]);
                op[static_cast<size_t>(t) * p.ldc + n] = __float2bfloat16(x);
              }
            }
          }
        }
      }
    }
    if (p.mode == 3) {
      // Publish: the four epilogue warps meet, one thread bumps this rank's arrival counter on every owner.
      // The barrier orders every epilogue thread's peer stores before thread 64's release at system scope
      // (release is cumulative over what the thread has observed), so one releasing atomic per owner suffices.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        for (int o = 0; o < p.world; ++o)
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(p.peer_part_flags[o] + p.my_rank) : "memory");
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (p.mode == 4) {
    // All slices of the tile are staged: cluster barrier, then this CTA reduces and publishes its share of rows.
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp >= 2) {
      const int S = static_cast<int>(gridDim.z);  // == cluster size; cluster rank == blockIdx.z
      const int et = threadIdx.x - 64;
      const int cg = et & 15, tr = et >> 4;  // 16 column groups of 8, 8 token rows per pass
      const int nn = n0 + cg * 8;
      const int valid = min(BT, p.M - t0);
      const int rows_per = (valid + S - 1) / S;
      const int r_lo = static_cast<int>(blockIdx.z) * rows_per;
      const int r_hi = min(valid, r_lo + rows_per);
      const uint32_t stile = smem_u32(smem);
      if (nn < p.N && num_c > 0) {
        for (int r = r_lo + tr; r < r_hi; r += 8) {
          const uint32_t off = static_cast<uint32_t>(r * 128 + cg * 8) * 4;
          float4 lo[8], hi[8];
#pragma unroll
          for (int z = 0; z < 8; ++z) {
            if (z < S) {
              const uint32_t ra = cluster_map_shared(stile + off, static_cast<uint32_t>(z));
              lo[z] = ld_shared_cluster_f4(ra);
              hi[z] = ld_shared_cluster_f4(ra + 16);
            }
          }
          float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int z = 0; z < 8; ++z) {
            if (z < S) {
              a[0] += lo[z].x; a[1] += lo[z].y; a[2] += lo[z].z; a[3] += lo[z].w;
              a[4] += hi[z].x; a[5] += hi[z].y; a[6] += hi[z].z; a[7] += hi[z].w;
            }
          }
          uint4 u;
          u.x = lamport_clean_bf16x2(pack_bf16x2(a[0], a[1])); u.y = lamport_clean_bf16x2(pack_bf16x2(a[2], a[3]));
          u.z = lamport_clean_bf16x2(pack_bf16x2(a[4], a[5])); u.w = lamport_clean_bf16x2(pack_bf16x2(a[6], a[7]));
          const size_t goff = (static_cast<size_t>(p.my_rank) * p.M + t0 + r) * p.ldc + nn;
          for (int o = 0; o < p.world; ++o)
            st_relaxed_sys_v4(reinterpret_cast<__nv_bfloat16*>(p.peer_parts[o]) + goff, u);
        }
      }
    }
    // No CTA may exit (and give up its shared memory) while a peer still reads its slice.
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BT, int STAGES, int TERMS>
int launch_mx(const void* W, const void* X0, const void* X1, MxParams p, int splits, cudaStream_t stream) {
  using L = MxSmem<BT, STAGES, TERMS>;
  CUtensorMap tw, tx0, tx1;
  if (make_tmap_2d(&tw, W, 1, p.N, p.K, static_cast<uint64_t>(p.K), 128, 128, 3)) return -1;
  if (make_tmap_2d(&tx0, X0, 1, p.M, p.K, static_cast<uint64_t>(p.K), BT, 128, 3)) return -1;
  if (make_tmap_2d(&tx1, TERMS == 2 ? X1 : X0, 1, p.M, p.K, static_cast<uint64_t>(p.K), BT, 128, 3)) return -1;
  {
    constexpr int D_COLS = BT < 32 ? 32 : BT;
    constexpr int TMEM_COLS = D_COLS <= 32 ? 64 : (D_COLS <= 96 ? 128 : 256);  // as in the kernel
    // Any mix of tcgen05 CTAs that shared memory lets an SM hold must also fit its 512 TMEM columns: every
    // kernel's share of tensor memory is at most its share of shared memory.
    static_assert(static_cast<long>(TMEM_COLS) * 227 * 1024 <= 512L * L::kTotal,
                  "tensor-memory share of a CTA exceeds its shared-memory share");
    AFB_CONFIGURE_KERNEL((gemm_mxfp8_kernel<BT, STAGES, TERMS>), L::kTotal, 192, TMEM_COLS);
  }
  dim3 grid((p.N + 127) / 128, (p.M + BT - 1) / BT, splits);
  if (p.mode == 4 && splits > 1) {
    AFB_CHECK_CUDA(launch_pdl_cluster(gemm_mxfp8_kernel<BT, STAGES, TERMS>, grid, dim3(192), dim3(1, 1, splits),
                                      L::kTotal, stream, tw, tx0, tx1, p));
    return 0;
  }
  AFB_CHECK_CUDA(launch_pdl(gemm_mxfp8_kernel<BT, STAGES, TERMS>, grid, dim3(192), L::kTotal, stream, tw, tx0, tx1, p));
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// Activation quantiser: bf16 [T, K] -> MX fp8 terms (e4m3 bytes [T, K]) + scale-factor atoms.
// One warp per (token, 128-wide K chunk ... ) : each lane owns 4 consecutive elements, 8 lanes share a 32-block.
// ---------------------------------------------------------------------------------------------------------
// Threads past K / 4 do not exist: the block has exactly K / 4 threads (K a multiple of 128, so whole warps) or
// 1024, and the loop bound is uniform per lane octet.
__global__ void quantize_mx_kernel(const __nv_bfloat16* x, long ldx, uint8_t* q0, uint8_t* q1, uint8_t* sf0,
                                   uint8_t* sf1, int T, int K) {
  const int t = blockIdx.x;
  griddep_launch();
  griddep_wait();
  for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t) * ldx + i);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    const float v[4] = {a.x, a.y, b.x, b.y};
    mx_quantize4_store(v, t, i, K, q0, q1, sf0, sf1, true);
  }
}

// SwiGLU over the fp32 split-K partial slices of an interleaved gate/up GEMM (column 2c = gate, 2c + 1 = up of
// output c), then MX quantisation: the consumer of a split gate/up GEMM and the producer of the down GEMM's
// activations in one pass.  parts: [S][T][ldp] fp32; bias (optional) bf16 [2F] in the same interleaved order.
__global__ void swiglu_quantize_mx_kernel(const float* parts, int S, long slice_stride, long ldp,
                                          const __nv_bfloat16* bias, uint8_t* q0, uint8_t* q1, uint8_t* sf0,
                                          uint8_t* sf1, __nv_bfloat16* y, long ldy, int T, int F) {
  const int t = blockIdx.x;
  griddep_launch();
  griddep_wait();
  for (int i = threadIdx.x * 4; i < F; i += blockDim.x * 4) {
    float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const float* src = parts + static_cast<size_t>(t) * ldp + 2 * i;
    for (int s = 0; s < S; ++s) {
      const float4 lo = *reinterpret_cast<const float4*>(src + s * slice_stride);
      const float4 hi = *reinterpret_cast<const float4*>(src + s * slice_stride + 4);
      a[0] += lo.x; a[1] += lo.y; a[2] += lo.z; a[3] += lo.w;
      a[4] += hi.x; a[5] += hi.y; a[6] += hi.z; a[7] += hi.w;
    }
    if (bias) {
#pragma unroll
      for (int c = 0; c < 8; ++c) a[c] += __bfloat162float(bias[2 * i + c]);
    }
    float v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = silu(a[2 * c]) * a[2 * c + 1];
    if (y) {
      uint2 o;
      o.x = pack_bf16x2(v[0], v[1]);
      o.y = pack_bf16x2(v[2], v[3]);
      *reinterpret_cast<uint2*>(y + static_cast<size_t>(t) * ldy + i) = o;
    }
    if (q0) mx_quantize4_store(v, t, i, F, q0, q1, sf0, sf1, true);
  }
}

}  // namespace afb

extern "C" {

// X8 terms [M, K] e4m3 with scale atoms sfx*; W8 [N, K] e4m3 with scale atoms sfw.  terms = 1 or 2.
// Modes as afb_gemm_w8a16.  K must be a multiple of 128.
int afb_gemm_mxfp8_tp(const void* X0, const void* X1, const void* sfx0, const void* sfx1, const void* W8,
                      const void* sfw, void* out, const void* bias, const void* residual, int M, int N, int K, int ldc,
                      int ldr, int act, int mode, int split_k, int terms, void* const* peer_parts,
                      void* const* peer_part_flags, int world, int my_rank, int tokens_per_rank, int slices,
                      int* x_ready, int x_expected, int* x_consumed, cudaStream_t stream);
int afb_gemm_mxfp8_bcast(const void* X0, const void* X1, const void* sfx0, const void* sfx1, const void* W8,
                         const void* sfw, int M, int N, int K, int ldc, int split_k, int terms,
                         void* const* peer_bufs, int world, int my_rank, cudaStream_t stream);

int afb_gemm_mxfp8(const void* X0, const void* X1, const void* sfx0, const void* sfx1, const void* W8, const void* sfw,
                   void* out, const void* bias, const void* residual, int M, int N, int K, int ldc, int ldr, int act,
                   int mode, int split_k, int terms, cudaStream_t stream) {
  return afb_gemm_mxfp8_tp(X0, X1, sfx0, sfx1, W8, sfw, out, bias, residual, M, N, K, ldc, ldr, act, mode, split_k,
                           terms, nullptr, nullptr, 0, 0, 0, 0, nullptr, 0, nullptr, stream);
}

// Tensor-parallel form.  mode 3 pushes fp32 partial tiles to the owners' symmetric buffers (peer_parts[o],
// laid out [world * slices][tokens_per_rank][ldc]) and signals peer_part_flags[o][my_rank]; x_ready != null makes
// the producer wait for x_expected arrivals before touching the activation buffers.
int afb_gemm_mxfp8_tp(const void* X0, const void* X1, const void* sfx0, const void* sfx1, const void* W8,
                      const void* sfw, void* out, const void* bias, const void* residual, int M, int N, int K, int ldc,
                      int ldr, int act, int mode, int split_k, int terms, void* const* peer_parts,
                      void* const* peer_part_flags, int world, int my_rank, int tokens_per_rank, int slices,
                      int* x_ready, int x_expected, int* x_consumed, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 128 || (N & 15) || M > 128 * 1024) {
    set_last_error("afb_gemm_mxfp8: K must be a multiple of 128 and N of 16 (K=%d N=%d)", K, N);
    return -1;
  }
  const int k_chunks = K / 128;
  if (split_k < 1) split_k = 1;
  if (split_k > k_chunks) split_k = k_chunks;
  int per = (k_chunks + split_k - 1) / split_k;
  split_k = (k_chunks + per - 1) / per;
  if (mode != 1 && mode != 3 && split_k != 1) {
    set_last_error("afb_gemm_mxfp8: split_k > 1 needs mode 1 or 3 (fp32 partials)");
    return -1;
  }
  if (mode == 3 && (world < 1 || world > 8 || split_k > slices || tokens_per_rank < 1)) {
    set_last_error("afb_gemm_mxfp8: mode 3 needs 1..8 ranks and split_k <= slices");
    return -1;
  }
  MxParams p = {};
  p.out = out;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.sfw = reinterpret_cast<const uint8_t*>(sfw);
  p.sfx0 = reinterpret_cast<const uint8_t*>(sfx0);
  p.sfx1 = reinterpret_cast<const uint8_t*>(sfx1);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr; p.act = act; p.mode = mode;
  p.chunks_per_split = per; p.k_chunks = k_chunks;
  p.world = mode == 3 ? world : 0; p.my_rank = my_rank; p.tokens_per_rank = tokens_per_rank; p.slices = slices;
  for (int o = 0; o < 8; ++o) {
    p.peer_parts[o] = (mode == 3 && o < world) ? reinterpret_cast<float*>(peer_parts[o]) : nullptr;
    p.peer_part_flags[o] = (mode == 3 && o < world) ? reinterpret_cast<int*>(peer_part_flags[o]) : nullptr;
  }
  p.x_ready = x_ready; p.x_expected = x_expected; p.x_consumed = x_consumed;
  if (terms == 2) {
    if (M <= 32) return launch_mx<32, 4, 2>(W8, X0, X1, p, split_k, stream);
    if (M <= 64) return launch_mx<64, 3, 2>(W8, X0, X1, p, split_k, stream);
    return launch_mx<128, 4, 2>(W8, X0, X1, p, split_k, stream);
  }
  if (M <= 32) return launch_mx<32, 5, 1>(W8, X0, X1, p, split_k, stream);
  if (M <= 64) return launch_mx<64, 4, 1>(W8, X0, X1, p, split_k, stream);
  return launch_mx<128, 5, 1>(W8, X0, X1, p, split_k, stream);
}

// Row-parallel GEMM whose reduced bf16 tile is broadcast to every rank (one-shot all-reduce; mode 4 above).
// peer_bufs[o]: rank o's bf16 [world][M][ldc] slot buffer, holding the sentinel 0x8000 wherever no data is
// pending (the consuming norm kernel restores it).  split_k <= 8 (the portable cluster size).
int afb_gemm_mxfp8_bcast(const void* X0, const void* X1, const void* sfx0, const void* sfx1, const void* W8,
                         const void* sfw, int M, int N, int K, int ldc, int split_k, int terms,
                         void* const* peer_bufs, int world, int my_rank, cudaStream_t stream) {
  using namespace afb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 128 || (N & 15) || (ldc & 7) || M > 128 || world < 1 || world > 8) {
    set_last_error("afb_gemm_mxfp8_bcast: needs K %% 128 == 0, N %% 16 == 0, ldc %% 8 == 0, M <= 128, 1..8 ranks");
    return -1;
  }
  const int k_chunks = K / 128;
  if (split_k < 1) split_k = 1;
  if (split_k > k_chunks) split_k = k_chunks;
  const int per = (k_chunks + split_k - 1) / split_k;
  split_k = (k_chunks + per - 1) / per;
  if (split_k > 8) {
    set_last_error("afb_gemm_mxfp8_bcast: at most 8 K splits (one thread-block cluster per tile)");
    return -1;
  }
  MxParams p = {};
  p.sfw = reinterpret_cast<const uint8_t*>(sfw);
  p.sfx0 = reinterpret_cast<const uint8_t*>(sfx0);
  p.sfx1 = reinterpret_cast<const uint8_t*>(sfx1);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.mode = 4;
  p.chunks_per_split = per; p.k_chunks = k_chunks;
  p.world = world; p.my_rank = my_rank;
  for (int o = 0; o < world; ++o) p.peer_parts[o] = reinterpret_cast<float*>(peer_bufs[o]);
  if (terms == 2) {
    if (M <= 32) return launch_mx<32, 4, 2>(W8, X0, X1, p, split_k, stream);
    if (M <= 64) return launch_mx<64, 3, 2>(W8, X0, X1, p, split_k, stream);
    return launch_mx<128, 4, 2>(W8, X0, X1, p, split_k, stream);
  }
  if (M <= 32) return launch_mx<32, 5, 1>(W8, X0, X1, p, split_k, stream);
  if (M <= 64) return launch_mx<64, 4, 1>(W8, X0, X1, p, split_k, stream);
  return launch_mx<128, 5, 1>(W8, X0, X1, p, split_k, stream);
}

int afb_mx_effective_splits(int K, int split_k) {
  const int k_chunks = K / 128;
  if (split_k < 1) split_k = 1;
  if (split_k > k_chunks) split_k = k_chunks;
  int per = (k_chunks + split_k - 1) / split_k;
  return (k_chunks + per - 1) / per;
}

// bf16 [T, K] (row pitch ldx) -> e4m3 terms + scale atoms ([ceil(T/128), K/128, 512] bytes each).
int afb_quantize_mx(const void* x, long ldx, void* q0, void* q1, void* sf0, void* sf1, int T, int K,
                    cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (K % 128 || (ldx & 3)) {
    set_last_error("afb_quantize_mx: K must be a multiple of 128 (got %d)", K);
    return -1;
  }
  int threads = K / 4;
  if (threads > 1024) threads = 1024;
  AFB_CHECK_CUDA(launch_pdl(quantize_mx_kernel, dim3(T), dim3(threads), 0, stream,
                            reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(q0),
                            reinterpret_cast<uint8_t*>(q1), reinterpret_cast<uint8_t*>(sf0),
                            reinterpret_cast<uint8_t*>(sf1), T, K));
  return 0;
}

// fp32 partial slices [S, T, 2F] of an interleaved gate/up GEMM -> SwiGLU -> MX fp8 terms [T, F] (+ scale atoms)
// and / or bf16 y [T, F].  F must be a multiple of 128; ldp a multiple of 4.
int afb_swiglu_quantize_mx(const float* parts, int S, long slice_stride, long ldp, const void* bias, void* q0,
                           void* q1, void* sf0, void* sf1, void* y, long ldy, int T, int F, cudaStream_t stream) {
  using namespace afb;
  if (T <= 0) return 0;
  if (F % 128 || (ldp & 3) || (slice_stride & 3) || (ldy & 3) || S < 1) {
    set_last_error("afb_swiglu_quantize_mx: F must be a multiple of 128 and pitches of 4 (F=%d)", F);
    return -1;
  }
  int threads = F / 4;
  if (threads > 1024) threads = 1024;
  AFB_CHECK_CUDA(launch_pdl(swiglu_quantize_mx_kernel, dim3(T), dim3(threads), 0, stream, parts, S, slice_stride, ldp,
                            reinterpret_cast<const __nv_bfloat16*>(bias), reinterpret_cast<uint8_t*>(q0),
                            reinterpret_cast<uint8_t*>(q1), reinterpret_cast<uint8_t*>(sf0),
                            reinterpret_cast<uint8_t*>(sf1), reinterpret_cast<__nv_bfloat16*>(y), ldy, T, F));
  return 0;
}

}  // extern "C"
