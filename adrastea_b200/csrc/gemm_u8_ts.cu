// u8-weight dequantising GEMM for prefill (m > 32), weights through TENSOR MEMORY:
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// replacing matmul_nt_wmma_16x128x256_fp16u8 (adrastea_kernels/cpp/
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83) beyond the decode shapes, with that kernel's
// arithmetic: every weight is dequantised to fp16((q - zero) * scale), bit-exact, before the
// product; products accumulate in fp32.
//
// The product is transposed: the 128 WEIGHT rows of a tile are the M side of tcgen05.mma and up
// to 256 TOKENS its N side, so a weight is dequantised once per 256 tokens and the tensor core
// runs its widest instruction.
//   * producer warp: per 64-wide k-step one TMA box of the weights (128 rows x 64 bytes of u8)
//     and one of the activations (BT tokens x 64 fp16, 128-byte swizzle, K-major) into a ring;
//   * sixteen converter warps (warp w: TMEM lane quarter w % 4, k-steps with index % 4 ==
//     w / 4): thread = weight row; 16 bytes -> 16 fp16 in registers (u8_common.cuh) ->
//     tcgen05.st into one of eight A buffers in tensor memory.  The dequantised weights never
//     touch shared memory.  (Converting a k-step takes a warp about half a microsecond, the
//     tensor core needs a quarter: four phases keep it fed);
//   * one thread issues tcgen05.mma (A from tensor memory, B = activations from shared memory,
//     M = 128, N = BT, K = 16) into one accumulator of BT columns (one issuer: the order of
//     MMAs into one accumulator is only defined within a thread);
//   * after the last k-step the converter warps turn into the epilogue: tcgen05.ld, a
//     transposition of 32 rows x 8 tokens (fp32) through a small shared-memory tile so that
//     old outputs are read and new ones written as 16-byte vectors, fp16(acc + beta * old).
// Persistent CTAs walk the tiles with the token blocks of one weight block next to each
// other, so that a weight block is read from HBM once and then from L2.
// Needs p % 64 == 0 and block_size % 64 == 0 (one scale group per k-step); other shapes take
// the kernel that stages the dequantised operand in shared memory (gemm_u8_tc.cu).
#include <algorithm>
#include <map>
#include <mutex>
#include <utility>

#include "tcgen05.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int TS_BK = 64;            // k per step
constexpr int TS_ROWS = 128;         // weight rows per tile
constexpr int TS_NA = 8;             // A buffers in tensor memory (32 columns each)
constexpr int TS_PHASES = 4;         // converter phases (k-step index % 4)
constexpr int TS_CONV_WARPS = 4 * TS_PHASES;
constexpr int TS_W_PRODUCER = 16, TS_W_MMA = 17;
constexpr int TS_THREADS = 18 * 32;
constexpr int TS_EPI_TOK = 8;        // tokens per transposition pass
constexpr int TS_EPI_LD = 36;        // floats between token rows of the tile (16 bytes more than 32:
                                     // the eight token rows then start in different bank groups)
constexpr int TS_EPI_BYTES = TS_EPI_TOK * TS_EPI_LD * 4;  // per converter warp

template <int BT>
struct TsCfg {
  static constexpr int W_BYTES = TS_ROWS * TS_BK;      // u8
  static constexpr int X_BYTES = BT * TS_BK * 2;       // fp16
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int STAGES = (204 * 1024) / STAGE_BYTES > 8 ? 8 : (204 * 1024) / STAGE_BYTES;
  static constexpr size_t EPI_BYTES = (size_t)TS_CONV_WARPS * TS_EPI_BYTES;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 512;
  static constexpr uint32_t A_COL0 = BT;
  static constexpr uint32_t TMEM_COLS = BT + TS_NA * 32 <= 256 ? 256 : 512;
};

struct TsParams {
  __half* out;
  const __half* scales;
  const __half* zeros;
  int m, p, n, block_size;
  float beta;
  unsigned int* status;
  int tile0, tile1;  // this launch covers tiles [tile0, tile1)
};

__device__ __forceinline__ void ts_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void ts_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
template <bool ACCUMULATE>
__device__ __forceinline__ void ts_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
  if (ACCUMULATE)
    asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 1;" ::"r"(tmem_d), "r"(tmem_a),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
  else
    asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 0;" ::"r"(tmem_d), "r"(tmem_a),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
}

template <int BT, bool SPLIT>
__global__ void __launch_bounds__(TS_THREADS, 1)
    gemm_u8_ts_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      TsParams p) {
  using Cfg = TsCfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;  // per stage: activations (1024-aligned), then weights
  uint8_t* epi = smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES;  // [warp][16 tokens][32 rows] fp16
  uint64_t* full = reinterpret_cast<uint64_t*>(epi + Cfg::EPI_BYTES);
  uint64_t* empty = full + Cfg::STAGES;      // the weights of the stage are in registers
  uint64_t* a_ready = empty + Cfg::STAGES;   // [TS_NA]
  uint64_t* a_free = a_ready + TS_NA;        // [TS_NA] the MMAs of k-step (index % TS_NA) are done
  uint64_t* acc_full = a_free + TS_NA;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = p.p / TS_BK;
  // SPLIT: grid (S, tiles), cluster (S, 1, 1): CTA `rank` of a cluster accumulates k-steps
  // [rank * num_kb / S, (rank + 1) * num_kb / S) of the cluster's one tile, and the partial
  // accumulators are summed through distributed shared memory before the single rounding.
  const int S = SPLIT ? (int)gridDim.x : 1, rank = SPLIT ? (int)blockIdx.x : 0;
  const int kb_begin = SPLIT ? (int)((long long)rank * num_kb / S) : 0;
  const int kb_end = SPLIT ? (int)((long long)(rank + 1) * num_kb / S) : num_kb;
  const int tile_first = p.tile0 + (SPLIT ? (int)blockIdx.y : (int)blockIdx.x);
  const int tile_stride = SPLIT ? (1 << 30) : (int)gridDim.x;
  const int nb = (p.n + TS_ROWS - 1) / TS_ROWS, tt = (p.m + BT - 1) / BT;
  const int total_tiles = min(nb * tt, p.tile1);
  const int groups = p.p / p.block_size;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);  // the four converter warps of the step's phase
    }
    for (int i = 0; i < TS_NA; ++i) {
      mbar_init(&a_ready[i], 4);
      mbar_init(&a_free[i], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, TS_CONV_WARPS);
    mbar_fence_init();
  }
  if (warp == TS_W_MMA) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  // tiles: the token blocks of one weight block follow one another
  auto tile_n0 = [&](int t) { return (t / tt) * TS_ROWS; };
  auto tile_t0 = [&](int t) { return (t % tt) * BT; };

  if (warp == TS_W_PRODUCER) {
    if (lane == 0) {
      int it = 0;
      for (int t = tile_first; t < total_tiles && ok; t += tile_stride) {
        const int n0 = tile_n0(t), t0 = tile_t0(t);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          if (!mbar_wait(&empty[s], ((unsigned)(it / Cfg::STAGES) & 1u) ^ 1u)) { ok = false; break; }
          // ... and its activations read by the MMAs of the k-step that used the stage (one
          // commit per k-step serves the converters' buffer and the stage)
          if (it >= Cfg::STAGES) {
            const int j = it - Cfg::STAGES;
            if (!mbar_wait(&a_free[j & (TS_NA - 1)], (unsigned)(j / TS_NA) & 1u)) { ok = false; break; }
          }
          uint8_t* st = stages + (size_t)s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          tma_load_2d(st, &map_x, kb * TS_BK, t0, &full[s]);
          tma_load_2d(st + Cfg::X_BYTES, &map_w, kb * TS_BK, n0, &full[s]);
        }
      }
      if (!ok) atomicOr(p.status, 8u);
    }
  } else if (warp == TS_W_MMA) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BT, false);
      int it = 0, local = 0;
      for (int t = tile_first; t < total_tiles && ok; t += tile_stride, ++local) {
        // the single accumulator is free once the epilogue of the previous tile has read it
        if (!mbar_wait(acc_empty, ((unsigned)local & 1u) ^ 1u)) { ok = false; break; }
        // several k-steps per round: the waits and the bookkeeping of this single thread are
        // the tensor core's idle time, so they are paid once per round.  A round must leave the
        // ring room to load and convert the next one while it runs: two k-steps with five
        // stages, four with eight.
        constexpr int ROUND = Cfg::STAGES >= 8 ? 4 : 2;
        for (int kb = kb_begin; kb < kb_end && ok; kb += ROUND) {
          const int steps = min(ROUND, kb_end - kb);
          // (the converters waited for a stage's copies before they converted, so the
          // activations of the stage have landed too)
          for (int u = 0; u < steps; ++u) {
            const int ab = (it + u) & (TS_NA - 1);
            if (!mbar_wait(&a_ready[ab], (unsigned)((it + u) / TS_NA) & 1u)) ok = false;
          }
          if (!ok) break;
          tc_fence_after_sync();
          for (int u = 0; u < steps; ++u, ++it) {
            const int s = it % Cfg::STAGES, ab = it & (TS_NA - 1);
            const uint64_t xdesc = umma_desc_k_sw128(smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES));
            const uint32_t a_addr = tmem_base + Cfg::A_COL0 + (uint32_t)(ab * 32);
            if (kb + u == kb_begin) ts_mma<false>(tmem_base, a_addr, xdesc, idesc);
            else ts_mma<true>(tmem_base, a_addr, xdesc, idesc);
            ts_mma<true>(tmem_base, a_addr + 8, xdesc + 2, idesc);
            ts_mma<true>(tmem_base, a_addr + 16, xdesc + 4, idesc);
            ts_mma<true>(tmem_base, a_addr + 24, xdesc + 6, idesc);
            umma_commit(&a_free[ab]);
          }
        }
        umma_commit(acc_full);
      }
      if (!ok) atomicOr(p.status, 8u);
    }
  } else {
    // ---------------- converters, then epilogue ----------------
    const int quarter = warp & 3, phase = warp >> 2;
    const int row = quarter * 32 + lane;  // weight row of the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // the weight tile is stored with the 64-byte swizzle (16-byte piece ^ bits 7-8 of the
    // address), so that the eight rows a quarter-warp reads at once lie in different banks
    const int wswz = (row >> 1) & 3;
    const bool has_zero = p.zeros != nullptr;
    int it = 0, local = 0;
    for (int t = tile_first; t < total_tiles; t += tile_stride, ++local) {
      const int n0 = tile_n0(t), t0 = tile_t0(t);
      const int n_row = n0 + row;
      const size_t srow = (size_t)min(n_row, p.n - 1) * groups;
      // Scales (and zero points) are requested TWO of this warp's k-steps ahead, into two
      // register pairs used in turn (the loop body is written out twice, so that no register
      // move waits for a load in flight): the 2-byte loads, one row per lane, take longer than
      // a k-step's conversion, and requested one step ahead they were what every warp waited
      // for.
      const int kb_mine = (phase - (it & (TS_PHASES - 1)) + TS_PHASES) & (TS_PHASES - 1);
      const int it0 = it;
      auto fetch = [&](int kq, __half& sc, __half& zp) {
        if (kq < kb_end) {
          const int g = (kq * TS_BK) / p.block_size;
          sc = p.scales[srow + g];
          if (has_zero) zp = p.zeros[srow + g];
        }
      };
      __half sc_a = __float2half(0.f), zp_a = sc_a, sc_b = sc_a, zp_b = sc_a;
      fetch(kb_begin + kb_mine, sc_a, zp_a);
      fetch(kb_begin + kb_mine + TS_PHASES, sc_b, zp_b);
      auto convert_step = [&](int kb, __half& sc, __half& zp) {
        const int itk = it0 + (kb - kb_begin);
        const int s = itk % Cfg::STAGES, ab = itk & (TS_NA - 1);
        const ScalePair sp = make_scale(sc, has_zero, zp);
        fetch(kb + 2 * TS_PHASES, sc, zp);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (unsigned)(itk / Cfg::STAGES) & 1u));
        uint4 w[4];
        if (ok) {
          const uint8_t* wrow = stages + (size_t)s * Cfg::STAGE_BYTES + Cfg::X_BYTES + row * TS_BK;
#pragma unroll
          for (int c = 0; c < 4; ++c) w[c] = *reinterpret_cast<const uint4*>(wrow + ((c ^ wswz) * 16));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // the weights of the stage are in registers
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&a_free[ab], ((unsigned)(itk / TS_NA) & 1u) ^ 1u));
        tc_fence_after_sync();
        if (ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
            uint32_t h[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __half2 lo, hi;
              dequant4(ww[j], sp, lo, hi);
              h[2 * j] = half2_as_u32(lo);
              h[2 * j + 1] = half2_as_u32(hi);
            }
            ts_st_x8(tmem_base + lane_base + Cfg::A_COL0 + (uint32_t)(ab * 32 + c * 8), h);
          }
        }
        ts_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_ready[ab]);
      };
      for (int kb = kb_begin + kb_mine; kb < kb_end; kb += 2 * TS_PHASES) {
        convert_step(kb, sc_a, zp_a);
        if (kb + TS_PHASES < kb_end) convert_step(kb + TS_PHASES, sc_b, zp_b);
      }
      it = it0 + (kb_end - kb_begin);
      if constexpr (SPLIT) {
        // The partial accumulator goes into this CTA's ring as [token][weight row] fp32 (the
        // ring is idle once the accumulator is complete: every stage has been read, and a
        // cluster has one tile); the sum over the cluster follows below, outside the roles.
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, (unsigned)local & 1u));
        tc_fence_after_sync();
        if (ok) {
          constexpr int QTS = BT / TS_PHASES;
          float* part = reinterpret_cast<float*>(stages);
#pragma unroll 1
          for (int c = 0; c < QTS / TS_EPI_TOK; ++c) {
            const int tl = phase * QTS + c * TS_EPI_TOK;
            if (t0 + tl >= p.m) break;  // uniform across the warp
            uint32_t acc[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]),
                           "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7])
                         : "r"(tmem_base + lane_base + (uint32_t)tl)
                         : "memory");
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < TS_EPI_TOK; ++j) part[(size_t)(tl + j) * TS_ROWS + row] = __uint_as_float(acc[j]);
          }
        }
        continue;
      }
      // ---- epilogue of the tile: this warp's lane quarter (32 weight rows), token quarter
      // `phase`.  Passes of 8 tokens: the thread (= weight row) writes its 8 fp32 results into
      // the warp's [8 tokens][32 rows] tile, then every lane takes one piece (8 consecutive rows
      // of one token): old outputs read and new ones written as 16-byte vectors.
      constexpr int QT = BT / TS_PHASES;  // tokens per warp
      constexpr int PASSES = QT / TS_EPI_TOK;
      const int nq0 = n0 + quarter * 32;  // first output column of this warp
      const bool vec = (p.n % 8 == 0) && nq0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
      const int tk = lane >> 2, seg = lane & 3;  // this lane's piece of a pass
      // The old outputs of all this warp's pieces are requested before the accumulator is
      // awaited: their latency (DRAM, the first time a buffer is touched) then overlaps the
      // last MMAs of the tile instead of being paid once per pass.
      uint4 oldv[PASSES];
      if (ok && vec) {
#pragma unroll
        for (int c = 0; c < PASSES; ++c) {
          const int tok = t0 + phase * QT + c * TS_EPI_TOK + tk;
          oldv[c] = make_uint4(0, 0, 0, 0);
          if (tok < p.m) oldv[c] = *reinterpret_cast<const uint4*>(p.out + (size_t)tok * p.n + nq0 + seg * 8);
        }
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, (unsigned)local & 1u));
      tc_fence_after_sync();
      if (ok) {
        float* tile = reinterpret_cast<float*>(epi + (size_t)warp * TS_EPI_BYTES);
        if (vec) {
#pragma unroll
          for (int c = 0; c < PASSES; ++c) {
            const int tok0 = t0 + phase * QT + c * TS_EPI_TOK;
            if (tok0 >= p.m) break;  // uniform across the warp
            uint32_t acc[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]),
                           "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7])
                         : "r"(tmem_base + lane_base + (uint32_t)(phase * QT + c * TS_EPI_TOK))
                         : "memory");
            __half* optr = p.out + (size_t)(tok0 + tk) * p.n + nq0 + seg * 8;
            const bool live = tok0 + tk < p.m;
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < TS_EPI_TOK; ++j) tile[j * TS_EPI_LD + lane] = __uint_as_float(acc[j]);
            __syncwarp();
            if (live) {
              const float4 a0 = *reinterpret_cast<const float4*>(tile + tk * TS_EPI_LD + seg * 8);
              const float4 a1 = *reinterpret_cast<const float4*>(tile + tk * TS_EPI_LD + seg * 8 + 4);
              const __half2* o2 = reinterpret_cast<const __half2*>(&oldv[c]);
              const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
              uint4 res;
              __half2* r2 = reinterpret_cast<__half2*>(&res);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 ov = __half22float2(o2[e]);
                r2[e] = __floats2half2_rn(fmaf(p.beta, ov.x, av[2 * e]), fmaf(p.beta, ov.y, av[2 * e + 1]));
              }
              *reinterpret_cast<uint4*>(optr) = res;
            }
            __syncwarp();
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < PASSES; ++c) {
            const int tok0 = t0 + phase * QT + c * TS_EPI_TOK;
            if (tok0 >= p.m) break;  // uniform across the warp
            uint32_t acc[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(acc[0]), "=r"(acc[1]), "=r"(acc[2]), "=r"(acc[3]), "=r"(acc[4]),
                           "=r"(acc[5]), "=r"(acc[6]), "=r"(acc[7])
                         : "r"(tmem_base + lane_base + (uint32_t)(phase * QT + c * TS_EPI_TOK))
                         : "memory");
            const bool row_ok = n_row < p.n;
            unsigned short old[TS_EPI_TOK];
#pragma unroll
            for (int j = 0; j < TS_EPI_TOK; ++j) {
              const int tok = tok0 + j;
              old[j] = (row_ok && tok < p.m)
                           ? reinterpret_cast<const unsigned short*>(p.out)[(size_t)tok * p.n + n_row]
                           : (unsigned short)0;
            }
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < TS_EPI_TOK; ++j) {
              const int tok = tok0 + j;
              if (row_ok && tok < p.m)
                p.out[(size_t)tok * p.n + n_row] = __float2half_rn(
                    fmaf(p.beta, __half2float(__ushort_as_half(old[j])), __uint_as_float(acc[j])));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
    if (!ok && lane == 0) atomicOr(p.status, 8u);
  }
  if constexpr (SPLIT) {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // rank r finishes tokens [r * BT / S, (r + 1) * BT / S) of the tile: the S partial tiles are
    // read through distributed shared memory (all requested before the first is used), summed
    // in rank order, and rounded once: fp16(sum + beta * old).
    const int tpr = (BT + S - 1) / S;
    const int n0 = tile_n0(tile_first), t0 = tile_t0(tile_first);
    const uint32_t pbase = smem_u32(stages);
    const bool vec4 = (p.n % 4 == 0) && (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0;
    for (int e = threadIdx.x; e < tpr * (TS_ROWS / 4); e += TS_THREADS) {
      const int tl = rank * tpr + e / (TS_ROWS / 4), r4 = (e % (TS_ROWS / 4)) * 4;
      const int tok = t0 + tl, nr = n0 + r4;
      if (tl >= BT || tok >= p.m || nr >= p.n) continue;
      float4 pv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        pv[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < S) {
          uint32_t remote;
          asm("mapa.shared::cluster.u32 %0, %1, %2;"
              : "=r"(remote)
              : "r"(pbase + (uint32_t)(tl * TS_ROWS + r4) * 4u), "r"(r));
          asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(pv[r].x), "=f"(pv[r].y), "=f"(pv[r].z), "=f"(pv[r].w)
                       : "r"(remote));
        }
      }
      float v[4] = {pv[0].x, pv[0].y, pv[0].z, pv[0].w};
#pragma unroll
      for (int r = 1; r < 4; ++r)
        if (r < S) {
          v[0] += pv[r].x;
          v[1] += pv[r].y;
          v[2] += pv[r].z;
          v[3] += pv[r].w;
        }
      __half* optr = p.out + (size_t)tok * p.n + nr;
      if (vec4 && nr + 4 <= p.n) {
        const uint2 oldv = *reinterpret_cast<const uint2*>(optr);
        const __half2* o2 = reinterpret_cast<const __half2*>(&oldv);
        uint2 res;
        __half2* r2 = reinterpret_cast<__half2*>(&res);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 ov = __half22float2(o2[h]);
          r2[h] = __floats2half2_rn(fmaf(p.beta, ov.x, v[2 * h]), fmaf(p.beta, ov.y, v[2 * h + 1]));
        }
        *reinterpret_cast<uint2*>(optr) = res;
      } else {
        for (int j = 0; j < 4 && nr + j < p.n; ++j)
          optr[j] = __float2half_rn(fmaf(p.beta, __half2float(optr[j]), v[j]));
      }
    }
    // every CTA stays resident until its peers have read its partial tile
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == TS_W_MMA) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// Clusters of `split` CTAs of the split kernel that the GPU holds at the same time (a cluster
// needs its CTAs on one GPC, so fewer than SMs / split), asked once per configuration.
template <int BT>
int ts_clusters_resident(adr_ctx* ctx, int split) {
  using Cfg = TsCfg<BT>;
  static std::mutex mu;
  static std::map<std::pair<int, int>, int> known;
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_pair(ctx->device, split);
  auto it = known.find(key);
  if (it == known.end()) {
    auto kfn = gemm_u8_ts_kernel<BT, true>;
    int nc = 0;
    if (opt_in_smem(ctx, kfn, Cfg::SMEM) == ADR_OK) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)split, 64, 1);
      cfg.blockDim = dim3(TS_THREADS, 1, 1);
      cfg.dynamicSmemBytes = Cfg::SMEM;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)split;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&nc, kfn, &cfg) != cudaSuccess) {
        cudaGetLastError();
        nc = 0;
      }
    }
    if (nc < 1) nc = 0;  // the runtime names no such cluster: this size is not used
    it = known.emplace(key, nc).first;
  }
  return it->second;
}

template <int BT>
int launch_u8_ts_t(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, int split, long long tile0 = 0,
                   long long tile1 = -1) {
  using Cfg = TsCfg<BT>;
  CUtensorMap map_w, map_x;
  {
    const uint64_t dims[2] = {(uint64_t)a.p, (uint64_t)a.n};
    const uint64_t strides[1] = {(uint64_t)a.p};
    const uint32_t box[2] = {TS_BK, TS_ROWS};
    int rc = tma_get(ctx, &map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != ADR_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a.p, (uint64_t)a.m};
    const uint64_t strides[1] = {(uint64_t)a.p * 2};
    const uint32_t box[2] = {TS_BK, (uint32_t)BT};
    int rc = tma_get(ctx, &map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.lhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  const long long all_tiles = (long long)((a.n + TS_ROWS - 1) / TS_ROWS) * ((a.m + BT - 1) / BT);
  if (tile1 < 0) tile1 = all_tiles;
  const long long tiles = tile1 - tile0;
  if (tiles <= 0) return ADR_OK;
  TsParams p{a.out, a.scales, a.zeros, a.m, a.p, a.n, a.block_size, a.beta, ctx->d_status, (int)tile0, (int)tile1};
  const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  if (split > 1) {
    auto kfn = gemm_u8_ts_kernel<BT, true>;
    if (int rc = opt_in_smem(ctx, kfn, Cfg::SMEM); rc != ADR_OK) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)split, (unsigned)tiles, 1);
    cfg.blockDim = dim3(TS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, map_w, map_x, p);
    if (e != cudaSuccess) {
      ctx->last_cuda_error = (int)e;
      return ADR_ERR_CUDA;
    }
    return after_launch(ctx);
  }
  auto kfn = gemm_u8_ts_kernel<BT, false>;
  if (int rc = opt_in_smem(ctx, kfn, Cfg::SMEM); rc != ADR_OK) return rc;
  const unsigned grid = (unsigned)std::min<long long>(tiles, sms);
  kfn<<<grid, TS_THREADS, Cfg::SMEM, stream>>>(map_w, map_x, p);
  return after_launch(ctx);
}

}  // namespace

bool u8_ts_supports(const adr_ctx* ctx, const U8Args& a) {
  if (!ctx->encode_tiled_fn) return false;
  if (a.p % TS_BK != 0 || a.block_size % TS_BK != 0 || a.p % a.block_size != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.lhs) & 15u) || (reinterpret_cast<uintptr_t>(a.rhs) & 15u))
    return false;
  return true;
}

int launch_u8_ts(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  if (!u8_ts_supports(ctx, a)) return ADR_ERR_SHAPE;
  // Tiles run in waves of one per SM, and a tile of 128 tokens takes about 0.8 of the time of
  // one of 256 (measured at k = 4096 and 11008: the k-step rate is set by the tensor core at
  // 256 tokens and by the hand-overs of the ring at 128), so 128 is chosen only where it saves
  // waves: 384 tokens x [12288, 4096] run as two waves of the shorter tiles.
  const int forced = ctx->tune_ts_bt.load();
  const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const long long nb = (a.n + TS_ROWS - 1) / TS_ROWS;
  const int num_kb = a.p / TS_BK;
  auto tiles_of = [&](int bt) { return nb * ((a.m + bt - 1) / bt); };
  auto cost = [&](int bt) { return ((tiles_of(bt) + sms - 1) / sms) * (bt == 128 ? 16 : 20); };
  int bt = a.m <= 128 ? 128 : (cost(128) < cost(256) ? 128 : 256);
  if (forced == 128 || forced == 256) bt = forced;
  // Too few tiles for the GPU: a cluster of two or four CTAs shares a tile's k-steps (at least
  // eight each).  With 256-token tiles where the tokens allow: a cluster then moves the
  // activations once per 256 tokens.
  int split = 1;
  const int want = ctx->tune_ts_split.load();
  auto resident = [&](int tile_tokens, int sp) {
    return (long long)(tile_tokens == 128 ? ts_clusters_resident<128>(ctx, sp) : ts_clusters_resident<256>(ctx, sp));
  };
  if (want != 1) {
    if (a.m > 128 && forced != 128 && tiles_of(256) <= resident(256, 2)) bt = 256;
    for (int sp = 4; sp >= 2; --sp)
      if (tiles_of(bt) <= resident(bt, sp) && num_kb / sp >= 8 && (want == 0 || want == sp)) {
        split = sp;
        break;
      }
  }
  if (bt == 128) return launch_u8_ts_t<128>(ctx, stream, a, split);
  // More than one wave of 256-token tiles with a small last wave: the full waves run as the
  // persistent kernel, the rest as a second launch with every tile on a cluster, which ends
  // in a fraction of a tile's time (192 tiles on 148 SMs: 148, then 44 on clusters of three).
  if (split == 1 && want != 1) {
    const long long t = tiles_of(256), full = t / sms * sms, rem = t - full;
    if (full > 0 && rem > 0) {
      int sp = 0;
      for (int c = 4; c >= 2; --c)
        if (rem <= resident(256, c) && num_kb / c >= 8 && (want == 0 || want == c)) {
          sp = c;
          break;
        }
      if (sp) {
        if (int rc = launch_u8_ts_t<256>(ctx, stream, a, 1, 0, full); rc != ADR_OK) return rc;
        return launch_u8_ts_t<256>(ctx, stream, a, sp, full, t);
      }
    }
  }
  return launch_u8_ts_t<256>(ctx, stream, a, split);
}

}  // namespace adr
