// fp16 strided/batched GEMM on the 5th-generation tensor cores:
//   out[b,y,x] = store(sum_k lhs[b,y,k] * rhs[b,k,x])
// replacing matmul_f16_fast / matmul_f16 (adrastea_kernels/cpp/matmul.cu:236-416,
// 493-513) and the WMMA kernels (matmul_nt_wmma_128x64x64.cu:8-78,
// matmul_nt_wmma_16x128x256.cu:8-68) for views TMA can describe.
//
// Tiles of 128 x BN outputs.  Warps are specialised:
//   warp 0    producer: one thread issues TMA loads of the A (128 x 64) and B (BN x 64)
//             k-blocks into a ring of 128-byte-swizzled shared-memory stages
//   warp 1    owns tensor memory (alloc/dealloc); one thread issues tcgen05.mma
//             (M = 128, N = BN, K = 16 per instruction, fp32 accumulators in TMEM) and
//             frees each stage with tcgen05.commit
//   warps 2.. epilogue: tcgen05.ld the accumulator (warp w reads TMEM lanes
//             32*(w%4)..+31 = tile rows), apply the reference's fused store op, mask
//             and scale, write fp16 to the (arbitrarily strided) output; eight warps in
//             the persistent kernel (two per lane quarter, alternating 32-column chunks),
//             four in the split-k kernel
// Two kernels share these roles:
//   gemm_f16_tc_kernel         persistent: one CTA per SM walks a list of tiles; two
//                              accumulator buffers in TMEM let the epilogue of one tile
//                              overlap the MMAs of the next
//   gemm_f16_tc_splitk_kernel  for grids that would leave most SMs idle (skinny m, prefill
//                              of a few hundred rows): a cluster of S CTAs splits k for one
//                              tile, the fp32 partial tiles are exchanged through distributed
//                              shared memory and added in rank order (deterministic, no
//                              scratch memory in HBM)
// Rows and k beyond the operands' extents are zero-filled by TMA, so m, n and k need no
// divisibility; only the 16-byte alignment rules of TMA apply (gemm_f16_tc_supports).
// Every mbarrier wait is bounded: a wait that runs out sets the context's status word,
// the kernel still frees its tensor memory and returns.
#include <algorithm>
#include <cmath>

#include "tcgen05.cuh"

namespace adr {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // fp16 elements: one 128-byte swizzle row
constexpr int TC_THREADS = 192;   // split-k kernel: producer, MMA, four epilogue warps
constexpr int TCP_THREADS = 320;  // persistent kernel: producer, MMA, eight epilogue warps
constexpr size_t SMEM_BUDGET = 200 * 1024;

template <int BN>
struct TcCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (int)((SMEM_BUDGET - 2048) / STAGE_BYTES) > 8
                                    ? 8
                                    : (int)((SMEM_BUDGET - 2048) / STAGE_BYTES);
  static constexpr size_t SMEM = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulator buffers
  // split-k: the fp32 partial tile, row-major with rows padded by 4 floats (row pitch = 16
  // bytes mod 128) so that the 16-byte row-wise writes of 8 lanes hit distinct bank groups
  // and the remote reads of a warp are 512 contiguous bytes
  static constexpr int PART_LD = BN + 4;
  static constexpr size_t PART_BYTES = (size_t)BM * PART_LD * 4;
  static_assert(PART_BYTES <= (size_t)STAGES * STAGE_BYTES, "partial tile must fit in the ring");
};

struct TcParams {
  __half* out;
  const __half* bias;
  int batches, m, k, n;
  int s_ox, s_oy, s_oz;
  int a_bcast, b_bcast;  // operand is shared by all batches (z-stride 0)
  float beta, scale;
  uint32_t store, load, mask;
  unsigned int* status;
};

__device__ __forceinline__ __half half_lo(uint32_t w) { return __ushort_as_half((unsigned short)(w & 0xFFFFu)); }
__device__ __forceinline__ __half half_hi(uint32_t w) { return __ushort_as_half((unsigned short)(w >> 16)); }

// The epilogue of one accumulator tile for one warp: the warp's 32 TMEM lanes are 32 tile
// rows (one per thread), and it walks the 32-column chunks chunk0, chunk0 + 2, ...  The
// loads of the old output and of the bias are in flight while tcgen05.ld completes.
// QuickGelu uses the fast exponential and reciprocal (the tensor-core path is held to a
// tolerance, not to the bits of the sequential reference sum).
template <int STORE>
__device__ __forceinline__ __half epilogue_op(const TcParams& p, float a, __half old, float bias,
                                              __half hscale) {
  if constexpr (STORE == ADR_STORE_QUICK_GELU_BIAS) {
    const float t = __half2float(__float2half_rn(a)) + bias;
    return __float2half_rn(__fdividef(t, 1.0f + __expf(-1.702f * t)));
  } else {
    return store_apply<STORE>(a, old, bias, p.beta, hscale);
  }
}

// `bar` (optional): the barrier that says the accumulator is complete.  It is awaited here,
// after the old outputs of the warp's first chunk have been requested (later chunks request
// theirs under their tensor-memory load; requesting them a chunk ahead into a second register
// set spilled and measured slower; the bias, 64 bytes per chunk, is requested a chunk ahead).  Returns false if the wait ran out.
template <int STORE, int BN, bool BIAS_AHEAD = false>
__device__ __forceinline__ bool epilogue_tile(const TcParams& p, uint32_t tmem_acc, __half* orow,
                                              int y, int n0, int chunk0, float pre, __half hscale,
                                              uint64_t* bar = nullptr, unsigned parity = 0) {
  const bool causal = p.mask == ADR_MASK_CAUSAL;
  const bool row_ok = y < p.m;
  // tcgen05.ld and its wait are warp-collective: every branch that contains one must be
  // uniform across the warp, so the vector path is taken only when all live rows allow it
  const bool lane_vec = p.s_ox == 1 && (reinterpret_cast<uintptr_t>(orow) & 15u) == 0 &&
                        (!store_uses_bias(STORE) || (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0);
  const bool row_vec = __all_sync(0xffffffffu, lane_vec || !row_ok);
  const __half ninf = __ushort_as_half((unsigned short)0xFC00);
  constexpr int NCH = (BN / 32 + 1) / 2;  // chunks per warp (chunk0, chunk0 + 2, ...)
  uint4 oldw[4], biasw[2][4];
  auto prefetch_bias = [&](int c, uint4 (&bsv)[4]) {
    const int x0 = n0 + c * 32;
    if (c < BN / 32 && row_vec && x0 + 32 <= p.n && row_ok) {
#pragma unroll
      for (int q = 0; q < 4; ++q) bsv[q] = reinterpret_cast<const uint4*>(p.bias + x0)[q];
    }
  };
  // (BIAS_AHEAD: the bias of the next chunk is requested a chunk ahead into a second register
  // set; only in the kernel compiled for one store operation, where the registers are there)
  if (store_uses_bias(STORE)) prefetch_bias(chunk0, biasw[0]);
  auto prefetch = [&](int c, uint4 (&o)[4]) {
    const int x0 = n0 + c * 32;
    if (c < BN / 32 && row_vec && x0 + 32 <= p.n && row_ok) {
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q] = reinterpret_cast<const uint4*>(orow + x0)[q];
    }
  };
  if (store_reads_out(STORE)) prefetch(chunk0, oldw);
  if (bar) {
    if (!mbar_wait(bar, parity)) return false;
    tc_fence_after_sync();
  }
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = chunk0 + 2 * i;
    if (c >= BN / 32) break;
    const int x0 = n0 + c * 32;
    if (x0 >= p.n) break;  // uniform across the warp
    uint32_t acc[32];
    __syncwarp();
    tmem_ld_32x32(tmem_acc + (uint32_t)(c * 32), acc);
    if (i > 0 && store_reads_out(STORE)) prefetch(c, oldw);
    if (BIAS_AHEAD) {
      if (i + 1 < NCH) prefetch_bias(c + 2, biasw[(i + 1) & 1]);
    } else if (i > 0 && store_uses_bias(STORE)) {
      prefetch_bias(c, biasw[0]);
    }
    if (row_vec && x0 + 32 <= p.n) {
      __syncwarp();
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (!row_ok) break;
        const uint4 oq = oldw[q], bq = biasw[BIAS_AHEAD ? (i & 1) : 0][q];
        const uint32_t ow[4] = {oq.x, oq.y, oq.z, oq.w};
        const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
        uint32_t rw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = q * 8 + e * 2;
          const float a0 = __uint_as_float(acc[j]) * pre, a1 = __uint_as_float(acc[j + 1]) * pre;
          const float b0 = store_uses_bias(STORE) ? __half2float(half_lo(bw[e])) : 0.0f;
          const float b1 = store_uses_bias(STORE) ? __half2float(half_hi(bw[e])) : 0.0f;
          const __half o0 = store_reads_out(STORE) ? half_lo(ow[e]) : __float2half_rn(0.0f);
          const __half o1 = store_reads_out(STORE) ? half_hi(ow[e]) : __float2half_rn(0.0f);
          __half r0 = epilogue_op<STORE>(p, a0, o0, b0, hscale);
          __half r1 = epilogue_op<STORE>(p, a1, o1, b1, hscale);
          if (causal && x0 + j > y) r0 = ninf;
          if (causal && x0 + j + 1 > y) r1 = ninf;
          rw[e] = (uint32_t)__half_as_ushort(r0) | ((uint32_t)__half_as_ushort(r1) << 16);
        }
        reinterpret_cast<uint4*>(orow + x0)[q] = make_uint4(rw[0], rw[1], rw[2], rw[3]);
      }
    } else {
      // strided, unaligned or ragged rows: one element at a time
      __syncwarp();
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int x = x0 + j;
        if (row_ok && x < p.n) {
          __half* dst = orow + (int64_t)x * p.s_ox;
          const float bias = store_uses_bias(STORE) ? __half2float(p.bias[x]) : 0.0f;
          const __half old = store_reads_out(STORE) ? *dst : __float2half_rn(0.0f);
          __half r = epilogue_op<STORE>(p, __uint_as_float(acc[j]) * pre, old, bias, hscale);
          if (causal && x > y) r = ninf;
          *dst = r;
        }
      }
    }
  }
  return true;
}

template <int BN>
__device__ __forceinline__ bool epilogue_tile_rt(const TcParams& p, uint32_t tmem_acc, __half* orow,
                                                 int y, int n0, int chunk0, float pre,
                                                 __half hscale, uint64_t* bar = nullptr,
                                                 unsigned parity = 0) {
  switch (p.store) {
    case ADR_STORE_SCALE: return epilogue_tile<ADR_STORE_SCALE, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    case ADR_STORE_ADD: return epilogue_tile<ADR_STORE_ADD, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    case ADR_STORE_BETA_BIAS: return epilogue_tile<ADR_STORE_BETA_BIAS, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    case ADR_STORE_BETA_GELU_BIAS: return epilogue_tile<ADR_STORE_BETA_GELU_BIAS, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    case ADR_STORE_QUICK_GELU_BIAS: return epilogue_tile<ADR_STORE_QUICK_GELU_BIAS, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    case STORE_NT_BETA: return epilogue_tile<STORE_NT_BETA, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
    default: return epilogue_tile<ADR_STORE_IDENTITY, BN>(p, tmem_acc, orow, y, n0, chunk0, pre, hscale, bar, parity);
  }
}

// Issues the four K=16 MMAs of one 64-wide k-block held in stage memory at `sa`.
// B_MN: the B stage holds an N-contiguous operand as BN/64 chunks of [64 k][64 n] (8 KB each).
template <int BN, bool B_MN>
__device__ __forceinline__ void mma_k_block(uint32_t tmem_d, uint32_t sa, bool first) {
  constexpr uint32_t idesc = umma_idesc_f16(BN, B_MN);
  const uint64_t adesc = umma_desc_k_sw128(sa);
  const uint64_t bdesc = B_MN ? umma_desc_mn_sw128(sa + TcCfg<BN>::A_BYTES, 8192)
                              : umma_desc_k_sw128(sa + TcCfg<BN>::A_BYTES);
  // per K=16 step: a k-major tile moves 32 bytes along its swizzled rows (+2 in the address
  // field), an n-major tile moves 16 k-rows of 128 bytes (+128)
  constexpr uint64_t b_step = B_MN ? 128 : 2;
#pragma unroll
  for (int kk = 0; kk < BK / 16; ++kk) {
    umma_f16(tmem_d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)kk * b_step, idesc,
             (!first || kk > 0) ? 1u : 0u);
  }
}

// One k-block of B into stage memory at `sb`.
template <int BN, bool B_MN>
__device__ __forceinline__ void load_b_block(uint8_t* sb, const CUtensorMap* map_b, int kb, int n0,
                                             int bz, uint64_t* bar) {
  if (B_MN) {
#pragma unroll
    for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * 8192, map_b, n0 + c * 64, kb * BK, bz, bar);
  } else {
    tma_load_3d(sb, map_b, kb * BK, n0, bz, bar);
  }
}

// Persistent tile scheduler: CTA c works on tiles c, c + gridDim.x, ...  Tiles are numbered
// batch-major, then in groups of GROUP_M row tiles swept along n, so that the tiles in
// flight at one time share A and B panels in L2.
struct TileCoord {
  int m0, n0, b;
};
constexpr int GROUP_M = 8;
__device__ __forceinline__ TileCoord tile_coord(int t, int mt, int nt, int bn) {
  const int per_batch = mt * nt;
  const int b = t / per_batch;
  const int r = t - b * per_batch;
  const int group = r / (GROUP_M * nt);
  const int first_m = group * GROUP_M;
  const int gsz = min(GROUP_M, mt - first_m);
  const int local = r - group * GROUP_M * nt;
  return {(first_m + local % gsz) * BM, (local / gsz) * bn, b};
}

// ONLY_STORE >= 0: the kernel compiled for that one store operation (its epilogue then has the
// registers to request the bias a chunk ahead); -1: the store operation is chosen at run time.
template <int BN, bool B_MN, int ONLY_STORE = -1>
__global__ void __launch_bounds__(TCP_THREADS, 1)
    gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_b, TcParams p) {
  using Cfg = TcCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* acc_full = empty_bar + Cfg::STAGES;  // [2]: accumulator buffer complete
  uint64_t* acc_empty = acc_full + 2;            // [2]: accumulator buffer drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.k + BK - 1) / BK;
  const int mt = (p.m + BM - 1) / BM, nt = (p.n + BN - 1) / BN;
  const int total_tiles = mt * nt * p.batches;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // ---------------- producer: TMA loads, one ring across all of this CTA's tiles ----------
    if (lane == 0) {
      int it = 0;  // k-blocks issued so far
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, mt, nt, BN);
        const int az = p.a_bcast ? 0 : tc.b, bz = p.b_bcast ? 0 : tc.b;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], phase ^ 1u)) { ok = false; break; }
          uint8_t* sa = stages + (size_t)s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          tma_load_3d(sa, &map_a, kb * BK, tc.m0, az, &full_bar[s]);
          load_b_block<BN, B_MN>(sa + Cfg::A_BYTES, &map_b, kb, tc.n0, bz, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: alternate between two accumulator buffers in TMEM ----------
    if (lane == 0) {
      int it = 0, local = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const int buf = local & 1;
        const unsigned use = (unsigned)(local >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], use ^ 1u)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], phase)) { ok = false; break; }
          tc_fence_after_sync();
          mma_k_block<BN, B_MN>(tmem_d, smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES), kb == 0);
          umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);  // the accumulator is complete once every MMA is done
      }
    }
  } else {
    // ---------------- epilogue: drains one buffer while the other is being filled ----------
    // Warps 2-5 take the even 32-column chunks of the tile, warps 6-9 the odd ones.
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id % 4) ..
    const int chunk0 = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const __half hscale = __float2half_rn(p.scale);
    // a load-side scale multiplies both operands (matmul.cu:62): s^2 on the product
    const float hs = __half2float(hscale);
    const float pre = p.load == ADR_LOAD_SCALE ? hs * hs : 1.0f;
    int local = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
      const TileCoord tc = tile_coord(t, mt, nt, BN);
      const int buf = local & 1;
      const unsigned use = (unsigned)(local >> 1) & 1u;
      const int y = tc.m0 + row;
      __half* orow = p.out + (int64_t)tc.b * p.s_oz + (int64_t)y * p.s_oy;
      // (the accumulator's barrier is awaited inside, behind the first loads of old outputs)
      const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
      bool done;
      if constexpr (ONLY_STORE >= 0)
        done = epilogue_tile<ONLY_STORE, BN, true>(p, tacc, orow, y, tc.n0, chunk0, pre, hscale, &acc_full[buf], use);
      else
        done = epilogue_tile_rt<BN>(p, tacc, orow, y, tc.n0, chunk0, pre, hscale, &acc_full[buf], use);
      if (!done) {
        ok = false;
        break;
      }
      // this warp's reads of the buffer are complete: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  if (!ok) atomicOr(p.status, 2u);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Split-k: grid (S, n tiles, m tiles * batches), cluster (S, 1, 1).  CTA `rank` of a cluster
// accumulates k-blocks [rank*num_kb/S, (rank+1)*num_kb/S) of its tile.
template <int BN, bool B_MN>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_f16_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a,
                              const __grid_constant__ CUtensorMap map_b, TcParams p, int S) {
  using Cfg = TcCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* acc_full = empty_bar + Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = blockIdx.x;
  const int mt = (p.m + BM - 1) / BM;
  const int n0 = blockIdx.y * BN, m0 = (blockIdx.z % mt) * BM, b = blockIdx.z / mt;
  const int num_kb = (p.k + BK - 1) / BK;
  const int kb0 = (int)((long long)rank * num_kb / S);
  const int kb1 = (int)((long long)(rank + 1) * num_kb / S);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      const int az = p.a_bcast ? 0 : b, bz = p.b_bcast ? 0 : b;
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0;
        const int s = it % Cfg::STAGES;
        const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) { ok = false; break; }
        uint8_t* sa = stages + (size_t)s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
        tma_load_3d(sa, &map_a, kb * BK, m0, az, &full_bar[s]);
        load_b_block<BN, B_MN>(sa + Cfg::A_BYTES, &map_b, kb, n0, bz, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = kb0; kb < kb1; ++kb) {
        const int it = kb - kb0;
        const int s = it % Cfg::STAGES;
        const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) { ok = false; break; }
        tc_fence_after_sync();
        mma_k_block<BN, B_MN>(tmem_base, smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES), kb == kb0);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_full);
    }
  }
  // ---- every warp: wait until the accumulator is complete (so the ring is idle too) ----
  ok = mbar_wait(acc_full, 0) && ok;
  tc_fence_after_sync();
  __syncthreads();  // producer and MMA threads are past their loops: the ring can be reused
  float* part = reinterpret_cast<float*>(stages);  // [BM][PART_LD], row-major, padded
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t acc[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), acc);
      tmem_ld_wait();
      float4* dst = reinterpret_cast<float4*>(part + (size_t)row * Cfg::PART_LD + c * 32);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        dst[q] = make_float4(__uint_as_float(acc[4 * q]), __uint_as_float(acc[4 * q + 1]),
                             __uint_as_float(acc[4 * q + 2]), __uint_as_float(acc[4 * q + 3]));
    }
  }
  if (!ok) atomicOr(p.status, 4u);
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

  // ---- rank r finishes rows [r*128/S, (r+1)*128/S): sum the S partial tiles in rank order.
  // A thread takes four consecutive columns; a warp reads 512 contiguous bytes per peer.
  {
    const int rpr = BM / S;
    const uint32_t pbase = smem_u32(part);
    const __half hscale = __float2half_rn(p.scale);
    const float hs = __half2float(hscale);
    const float pre = p.load == ADR_LOAD_SCALE ? hs * hs : 1.0f;
    const bool causal = p.mask == ADR_MASK_CAUSAL;
    const int store = (int)p.store;
    const bool rd_out = store_reads_out(store), use_bias = store_uses_bias(store);
    __half* obase = p.out + (int64_t)b * p.s_oz;
    for (int e = threadIdx.x; e < rpr * (BN / 4); e += TC_THREADS) {
      const int col = (e % (BN / 4)) * 4, row = rank * rpr + e / (BN / 4);
      const int x0 = n0 + col, y = m0 + row;
      if (x0 >= p.n || y >= p.m) continue;
      // all S remote reads are issued before the first is used, then added in rank order
      float4 pv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        pv[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < S) {
          uint32_t remote;
          asm("mapa.shared::cluster.u32 %0, %1, %2;"
              : "=r"(remote)
              : "r"(pbase + (uint32_t)(row * Cfg::PART_LD + col) * 4u), "r"(r));
          asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(pv[r].x), "=f"(pv[r].y), "=f"(pv[r].z), "=f"(pv[r].w)
                       : "r"(remote));
        }
      }
      float v[4] = {pv[0].x, pv[0].y, pv[0].z, pv[0].w};
#pragma unroll
      for (int r = 1; r < 8; ++r)
        if (r < S) {
          v[0] += pv[r].x;
          v[1] += pv[r].y;
          v[2] += pv[r].z;
          v[3] += pv[r].w;
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int x = x0 + j;
        if (x >= p.n) break;
        __half* dst = obase + (int64_t)y * p.s_oy + (int64_t)x * p.s_ox;
        __half res;
        if (causal && x > y) {
          res = __ushort_as_half((unsigned short)0xFC00);
        } else {
          const __half old = rd_out ? *dst : __float2half_rn(0.0f);
          const float bias = use_bias ? __half2float(p.bias[x]) : 0.0f;
          res = store_apply_rt(store, v[j] * pre, old, bias, p.beta, hscale);
        }
        *dst = res;
      }
    }
  }
  // every CTA stays resident until its peers have read its partial tile
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// The same tensor-core tile for views the copy engine cannot describe (a row pitch that is
// not a multiple of 16 bytes, an unaligned base, neither operand dimension contiguous): the
// [heads, 257, 257] score and probability tensors of a 257-token encoder have a 514-byte
// pitch (adrastea_models/src/clip.rs:374-388).  Eight loader warps read the operands with
// ordinary 2-byte loads, any strides, and write them into the 128-byte-swizzled stage
// layout themselves (zeros outside the extents), fence.proxy.async, arrive; the MMA warp and
// the eight epilogue warps are those of the persistent kernel.  One CTA per 128 x BN tile.
// B_MN: rhs rows are n-contiguous ([K,N] storage): lanes run along n and the stage holds
// chunks of [64 k][64 n], described to the tensor core as an N-major operand.
// ---------------------------------------------------------------------------------------
constexpr int GATHER_LOAD_WARPS = 8;
constexpr int GATHER_THREADS = (2 + 8 + GATHER_LOAD_WARPS) * 32;
constexpr int GATHER_STAGES = 3;

struct GatherParams {
  const __half* lhs;
  const __half* rhs;
  int s_lx, s_ly, s_lz, s_rx, s_ry, s_rz;
};

template <int BN, bool B_MN>
__global__ void __launch_bounds__(GATHER_THREADS, 1)
    gemm_f16_tc_gather_kernel(GatherParams g, TcParams p) {
  using Cfg = TcCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)GATHER_STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + GATHER_STAGES;
  uint64_t* acc_full = empty_bar + GATHER_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.k + BK - 1) / BK;
  const int n0 = blockIdx.x * BN;
  const int mt = (p.m + BM - 1) / BM;
  const int m0 = (blockIdx.y % mt) * BM, b = blockIdx.y / mt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GATHER_STAGES; ++s) {
      mbar_init(&full_bar[s], GATHER_LOAD_WARPS);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, BN < 32 ? 32 : BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % GATHER_STAGES;
        if (!mbar_wait(&full_bar[s], (unsigned)(kb / GATHER_STAGES) & 1u)) { ok = false; break; }
        tc_fence_after_sync();
        mma_k_block<BN, B_MN>(tmem_base, smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES), kb == 0);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_full);
    }
  } else if (warp >= 2 && warp < 10) {
    const int quarter = warp & 3;
    const int chunk0 = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const __half hscale = __float2half_rn(p.scale);
    const float hs = __half2float(hscale);
    const float pre = p.load == ADR_LOAD_SCALE ? hs * hs : 1.0f;
    if (!mbar_wait(acc_full, 0)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    if (ok) {
      const int y = m0 + row;
      __half* orow = p.out + (int64_t)b * p.s_oz + (int64_t)y * p.s_oy;
      epilogue_tile_rt<BN>(p, tmem_base + ((uint32_t)(quarter * 32) << 16), orow, y, n0, chunk0, pre,
                           hscale);
    }
  } else if (warp >= 10) {
    // ---------------- loaders ----------------
    const int lt = threadIdx.x - 10 * 32;  // 0 .. 255
    constexpr int LT = GATHER_LOAD_WARPS * 32;
    const __half* abase = g.lhs + (p.a_bcast ? 0 : (int64_t)b * g.s_lz);
    const __half* bbase = g.rhs + (p.b_bcast ? 0 : (int64_t)b * g.s_rz);
    const unsigned short zero = 0;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % GATHER_STAGES;
      if (!mbar_wait(&empty_bar[s], ((unsigned)(kb / GATHER_STAGES) & 1u) ^ 1u)) { ok = false; break; }
      uint8_t* sa = stages + (size_t)s * Cfg::STAGE_BYTES;
      uint8_t* sb = sa + Cfg::A_BYTES;
      const int k0 = kb * BK;
      // A: [128 rows][64 k], lanes along k
#pragma unroll 4
      for (int idx = lt; idx < BM * BK; idx += LT) {
        const int r = idx >> 6, kk = idx & 63;
        const int y = m0 + r, k = k0 + kk;
        unsigned short v = zero;
        if (y < p.m && k < p.k)
          v = __half_as_ushort(abase[(int64_t)y * g.s_ly + (int64_t)k * g.s_lx]);
        *reinterpret_cast<unsigned short*>(sa + r * 128 + ((((kk >> 3) ^ (r & 7))) << 4) + (kk & 7) * 2) = v;
      }
      if (B_MN) {
        // B: chunks of [64 k][64 n], lanes along n
#pragma unroll 4
        for (int idx = lt; idx < BN * BK; idx += LT) {
          const int kk = idx / BN, nn = idx % BN;
          const int x = n0 + nn, k = k0 + kk;
          unsigned short v = zero;
          if (x < p.n && k < p.k)
            v = __half_as_ushort(bbase[(int64_t)k * g.s_ry + (int64_t)x * g.s_rx]);
          const int c = nn >> 6, ni = nn & 63;
          *reinterpret_cast<unsigned short*>(sb + c * 8192 + kk * 128 + ((((ni >> 3) ^ (kk & 7))) << 4) +
                                             (ni & 7) * 2) = v;
        }
      } else {
        // B: [BN rows of n][64 k], lanes along k
#pragma unroll 4
        for (int idx = lt; idx < BN * BK; idx += LT) {
          const int r = idx >> 6, kk = idx & 63;
          const int x = n0 + r, k = k0 + kk;
          unsigned short v = zero;
          if (x < p.n && k < p.k)
            v = __half_as_ushort(bbase[(int64_t)k * g.s_ry + (int64_t)x * g.s_rx]);
          *reinterpret_cast<unsigned short*>(sb + r * 128 + ((((kk >> 3) ^ (r & 7))) << 4) + (kk & 7) * 2) = v;
        }
      }
      // make the generic-proxy writes visible to the tensor core's async-proxy reads
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[s]);
    }
  }
  if (!ok) atomicOr(p.status, 2u);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
  }
}

template <int BN, bool B_MN>
int launch_gather(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  using Cfg = TcCfg<BN>;
  auto kfn = gemm_f16_tc_gather_kernel<BN, B_MN>;
  constexpr size_t smem = 1024 + (size_t)GATHER_STAGES * Cfg::STAGE_BYTES + 256;
  int rc = opt_in_smem(ctx, kfn, smem);
  if (rc != ADR_OK) return rc;
  const bool a_bcast = a.batches > 1 && a.s_lz == 0;
  const bool b_bcast = a.batches > 1 && a.s_rz == 0;
  TcParams p{a.out, a.bias, a.batches, a.m, a.k, a.n, a.s_ox, a.s_oy, a.s_oz,
             a_bcast ? 1 : 0, b_bcast ? 1 : 0, a.beta, a.scale, a.store, a.load, a.mask,
             ctx->d_status};
  GatherParams g{a.lhs, a.rhs, a.s_lx, a.s_ly, a.s_lz, a.s_rx, a.s_ry, a.s_rz};
  const long long nt = (a.n + BN - 1) / BN, mt = (a.m + BM - 1) / BM;
  if (mt * a.batches > 65535) return ADR_ERR_SHAPE;
  kfn<<<dim3((unsigned)nt, (unsigned)(mt * a.batches)), GATHER_THREADS, smem, stream>>>(g, p);
  return after_launch(ctx);
}

template <int BN, bool B_MN>
int make_maps(adr_ctx* ctx, const MatmulArgs& a, CUtensorMap* map_a, CUtensorMap* map_b,
              TcParams* p) {
  const bool a_bcast = a.batches > 1 && a.s_lz == 0;
  const bool b_bcast = a.batches > 1 && a.s_rz == 0;
  {
    const uint64_t za = a_bcast || a.batches == 1 ? 1 : (uint64_t)a.batches;
    const uint64_t dims[3] = {(uint64_t)a.k, (uint64_t)a.m, za};
    const uint64_t zs = za == 1 ? (uint64_t)a.s_ly * 2 * (uint64_t)a.m : (uint64_t)a.s_lz * 2;
    const uint64_t strides[2] = {(uint64_t)a.s_ly * 2, zs};
    const uint32_t box[3] = {BK, BM, 1};
    int rc = tma_get(ctx, map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a.lhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  {
    const uint64_t zb = b_bcast || a.batches == 1 ? 1 : (uint64_t)a.batches;
    // k-major B: (k, n, batch) with rows of n; n-major B: (n, k, batch) with rows of k
    const uint64_t inner = B_MN ? (uint64_t)a.n : (uint64_t)a.k;
    const uint64_t outer = B_MN ? (uint64_t)a.k : (uint64_t)a.n;
    const uint64_t pitch = (uint64_t)(B_MN ? a.s_ry : a.s_rx) * 2;
    const uint64_t dims[3] = {inner, outer, zb};
    const uint64_t zs = zb == 1 ? pitch * outer : (uint64_t)a.s_rz * 2;
    const uint64_t strides[2] = {pitch, zs};
    const uint32_t box[3] = {BK, B_MN ? 64u : (uint32_t)BN, 1};
    int rc = tma_get(ctx, map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  *p = TcParams{a.out, a.bias, a.batches, a.m, a.k, a.n, a.s_ox, a.s_oy, a.s_oz,
                a_bcast ? 1 : 0, b_bcast ? 1 : 0, a.beta, a.scale, a.store, a.load, a.mask,
                ctx->d_status};
  return ADR_OK;
}

template <int BN, bool B_MN>
int launch_tc(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a, int S) {
  using Cfg = TcCfg<BN>;
  CUtensorMap map_a, map_b;
  TcParams p;
  int rc = make_maps<BN, B_MN>(ctx, a, &map_a, &map_b, &p);
  if (rc != ADR_OK) return rc;
  const int nt = (a.n + BN - 1) / BN, mt = (a.m + BM - 1) / BM;
  if (S <= 1) {
    const long long tiles = (long long)nt * mt * a.batches;
    const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const unsigned grid = (unsigned)std::min<long long>(tiles, sms);
    // The encoder's products with k = 1024 (bias, or bias + QuickGelu, on 256-wide tiles): their
    // epilogue, not their MMAs, sets the pace, and a kernel compiled for the one store operation
    // runs it 5-25 % faster than the one that chooses at run time (registers).
    if constexpr (BN == 256 && !B_MN) {
      if (p.store == ADR_STORE_QUICK_GELU_BIAS || p.store == ADR_STORE_BETA_BIAS) {
        auto kfn = p.store == ADR_STORE_QUICK_GELU_BIAS
                       ? gemm_f16_tc_kernel<BN, B_MN, (int)ADR_STORE_QUICK_GELU_BIAS>
                       : gemm_f16_tc_kernel<BN, B_MN, (int)ADR_STORE_BETA_BIAS>;
        rc = opt_in_smem(ctx, kfn, Cfg::SMEM);
        if (rc != ADR_OK) return rc;
        kfn<<<grid, TCP_THREADS, Cfg::SMEM, stream>>>(map_a, map_b, p);
        return after_launch(ctx);
      }
    }
    auto kfn = gemm_f16_tc_kernel<BN, B_MN>;
    rc = opt_in_smem(ctx, kfn, Cfg::SMEM);
    if (rc != ADR_OK) return rc;
    kfn<<<grid, TCP_THREADS, Cfg::SMEM, stream>>>(map_a, map_b, p);
    return after_launch(ctx);
  }
  auto kfn = gemm_f16_tc_splitk_kernel<BN, B_MN>;
  rc = opt_in_smem(ctx, kfn, Cfg::SMEM);
  if (rc != ADR_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, nt, mt * a.batches);
  cfg.blockDim = dim3(TC_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, map_a, map_b, p, S);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  return after_launch(ctx);
}

struct TcPlan {
  int bn, S;
};

// Picks the N-tile and the k-split.  Measured tensor-pipe efficiency by tile width (one CTA
// per tile, operands from shared memory): 256 -> 1.0, 128 -> 0.76 (shared-memory bandwidth
// bound), 64 -> 0.43, 32 -> 0.22.  The score is that efficiency times the SM utilisation of
// the schedule; a k-split costs a reduction through distributed shared memory.
TcPlan pick_plan(const adr_ctx* ctx, const MatmulArgs& a) {
  const double sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const double mt = (a.m + BM - 1) / BM;
  const int num_kb = (a.k + BK - 1) / BK;
  TcPlan best{64, 1};
  double best_score = -1.0;
  const bool b_mn = a.s_ry != 1;  // n-contiguous B needs 64-column chunks
  for (int bn : {256, 128, 64, 32}) {
    if (b_mn && bn < 64) continue;
    if (ctx->tune_tc_bn && bn != ctx->tune_tc_bn) continue;
    if (!ctx->tune_tc_bn && bn > 32 && a.n <= bn / 2) continue;  // do not pad n beyond the next tile size
    const double tiles = mt * ((a.n + bn - 1) / bn) * a.batches;
    const double eff = bn == 256 ? 1.0 : bn == 128 ? 0.76 : bn == 64 ? 0.43 : 0.22;
    for (int S : {1, 2, 4, 8}) {
      if (ctx->tune_tc_split && S != ctx->tune_tc_split) continue;
      if (S > 1 && (num_kb < 2 * S || mt * a.batches > 65535)) continue;
      const double ctas = tiles * S;
      double util;
      if (S == 1) {
        const double waves = tiles / sms;
        util = waves / std::ceil(waves);
      } else {
        if (ctas > sms && !ctx->tune_tc_split) continue;  // a split only pays on an under-filled grid
        util = std::min(1.0, ctas / sms);
      }
      // measured: the exchange of partial tiles costs about 40 % at these sizes
      const double score = util * eff * (S == 1 ? 1.0 : S == 8 ? 0.4 : 0.6);
      if (score > best_score) {
        best_score = score;
        best = {bn, S};
      }
    }
  }
  return best;
}

}  // namespace

bool gemm_f16_tc_supports(const adr_ctx* ctx, const MatmulArgs& a) {
  if (!ctx->encode_tiled_fn) return false;
  if (a.s_lx != 1 || a.s_ly % 8 != 0) return false;  // lhs k-contiguous, 16-byte row pitch
  // rhs either k-contiguous ([N,K] storage passed permuted) or n-contiguous ([K,N] storage)
  const bool b_k = a.s_ry == 1 && a.s_rx % 8 == 0;
  const bool b_n = a.s_rx == 1 && a.s_ry % 8 == 0 && a.s_ry != 1;
  if (!b_k && !b_n) return false;
  if (a.batches > 1 && (a.s_lz % 8 != 0 || a.s_rz % 8 != 0)) return false;
  if ((reinterpret_cast<uintptr_t>(a.lhs) & 15u) || (reinterpret_cast<uintptr_t>(a.rhs) & 15u))
    return false;
  if (a.batches > 65535 || (a.m + BM - 1) / BM > 65535) return false;
  return true;
}

int launch_gemm_f16_tc(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  const TcPlan pl = pick_plan(ctx, a);
  if (a.s_ry != 1) {
    switch (pl.bn) {
      case 256: return launch_tc<256, true>(ctx, stream, a, pl.S);
      case 128: return launch_tc<128, true>(ctx, stream, a, pl.S);
      default: return launch_tc<64, true>(ctx, stream, a, pl.S);
    }
  }
  switch (pl.bn) {
    case 256: return launch_tc<256, false>(ctx, stream, a, pl.S);
    case 128: return launch_tc<128, false>(ctx, stream, a, pl.S);
    case 64: return launch_tc<64, false>(ctx, stream, a, pl.S);
    default: return launch_tc<32, false>(ctx, stream, a, pl.S);
  }
}

// Tensor-core tiles behind a gathering loader: any strides, any alignment.
int launch_gemm_f16_gather(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  // lanes of a loader warp run along the contiguous dimension of rhs
  const bool b_mn = a.s_rx == 1 && a.s_ry != 1;
  if (a.n > 64) return b_mn ? launch_gather<128, true>(ctx, stream, a) : launch_gather<128, false>(ctx, stream, a);
  return b_mn ? launch_gather<64, true>(ctx, stream, a) : launch_gather<64, false>(ctx, stream, a);
}

int init_gemm_f16_tc(adr_ctx*) { return ADR_OK; }
void destroy_gemm_f16_tc(adr_ctx*) {}

}  // namespace adr
