// u8-weight dequantising GEMM on the 5th-generation tensor cores, for m > 16 (prefill):
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// replacing matmul_nt_wmma_16x128x256_fp16u8 (adrastea_kernels/cpp/
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83) and matmul_nt_fp16u8 (matmul_nt_fp16u8.cu:4-24)
// beyond the decode shapes.
//
// Same skeleton as the fp16 tensor-core GEMM (persistent CTAs, 128 x BN tiles, TMA producer
// warp, one MMA-issuing thread, accumulators double-buffered in TMEM, four epilogue warps),
// plus eight dequantising warps between the copy engine and the tensor core:
//   TMA   lhs k-block (128 x 64 fp16, 128-byte swizzle)   -> stage.A
//         weight k-block (BN rows x 64 bytes of u8)        -> stage.Q
//   warps 6-13: read Q 16 bytes at a time, dequantise in registers (u8_common.cuh, bit-exact
//         fp16((q - zero) * scale)), write the fp16 operand into stage.B in the 128-byte
//         swizzled K-major layout tcgen05.mma expects, fence.proxy.async, arrive
//   MMA   waits for the dequantised stage, issues tcgen05.mma, commits the stage free
// The weights cross HBM and L2 as bytes and become fp16 only inside the SM.
#include <algorithm>

#include "tcgen05.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int DQ_WARPS = 8;
constexpr int U8TC_THREADS = (2 + 4 + DQ_WARPS) * 32;

template <int BN>
struct U8Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int Q_BYTES = BN * BK;      // u8
  static constexpr int B_BYTES = BN * BK * 2;  // fp16, written by the dequantising warps
  static constexpr int STAGE_BYTES = A_BYTES + Q_BYTES + B_BYTES;
  static constexpr int STAGES = (int)((198 * 1024) / STAGE_BYTES);
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * BN;
};

struct U8TcParams {
  __half* out;
  const __half* scales;
  const __half* zeros;
  int m, p, n, block_size;
  float beta;
  unsigned int* status;
};

template <int BN, bool HAS_ZERO>
__global__ void __launch_bounds__(U8TC_THREADS, 1)
    gemm_u8_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                      const __grid_constant__ CUtensorMap map_q, U8TcParams p) {
  using Cfg = U8Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* b_full = q_full + Cfg::STAGES;   // dequantised operand ready (DQ_WARPS arrivals)
  uint64_t* empty_bar = b_full + Cfg::STAGES;
  uint64_t* acc_full = empty_bar + Cfg::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.p + BK - 1) / BK;
  const int mt = (p.m + BM - 1) / BM, nt = (p.n + BN - 1) / BN;
  const int total_tiles = mt * nt;
  const int groups = p.p / p.block_size;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_q);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&b_full[s], DQ_WARPS);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  // tiles: m fastest, so that the CTAs running together share weight rows in L2
  auto tile_m0 = [&](int t) { return (t % mt) * BM; };
  auto tile_n0 = [&](int t) { return (t / mt) * BN; };

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      int it = 0;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = tile_m0(t), n0 = tile_n0(t);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], phase ^ 1u)) { ok = false; break; }
          uint8_t* sa = stages + (size_t)s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&q_full[s], Cfg::A_BYTES + Cfg::Q_BYTES);
          tma_load_2d(sa, &map_a, kb * BK, m0, &q_full[s]);
          tma_load_2d(sa + Cfg::A_BYTES, &map_q, kb * BK, n0, &q_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BN, false);
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
          if (!mbar_wait(&b_full[s], phase)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::A_BYTES + Cfg::Q_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_f16(tmem_d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                     (kb > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&acc_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ---------------- epilogue: out = fp16(acc + beta * out) ----------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int local = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
      const int m0 = tile_m0(t), n0 = tile_n0(t);
      const int buf = local & 1;
      const unsigned use = (unsigned)(local >> 1) & 1u;
      if (!mbar_wait(&acc_full[buf], use)) { ok = false; break; }
      tc_fence_after_sync();
      const int y = m0 + row;
      __half* orow = p.out + (size_t)y * p.n;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int x0 = n0 + c * 32;
        if (x0 >= p.n) break;
        uint32_t acc[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32),
                      acc);
        tmem_ld_wait();
        if (y < p.m) {
          const bool vec = x0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(orow + x0) & 15u) == 0;
          __align__(16) __half v[32];
          if (vec) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(&v[q * 8]) = reinterpret_cast<const uint4*>(orow + x0)[q];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = x0 + j < p.n ? orow[x0 + j] : __float2half_rn(0.f);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float2half_rn(fmaf(p.beta, __half2float(v[j]), __uint_as_float(acc[j])));
          if (vec) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              reinterpret_cast<uint4*>(orow + x0)[q] = *reinterpret_cast<const uint4*>(&v[q * 8]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (x0 + j < p.n) orow[x0 + j] = v[j];
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  } else {
    // ---------------- dequantising warps ----------------
    // The stage holds BN rows x 64 bytes; four consecutive lanes take the four 16-byte pieces
    // of one row, so a quarter warp reads 128 contiguous bytes.  Piece q of row r becomes the
    // fp16 16-byte chunks 2q and 2q+1 of the 128-byte operand row, stored at chunk ^ (r & 7).
    const int dtid = threadIdx.x - 6 * 32;         // 0 .. DQ_WARPS*32-1
    constexpr int DQ_THREADS = DQ_WARPS * 32;
    constexpr int PIECES = BN * 4 / DQ_THREADS;     // per thread per k-block
    int it = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int n0 = tile_n0(t);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % Cfg::STAGES;
        const unsigned phase = (unsigned)(it / Cfg::STAGES) & 1u;
        // scales of this thread's pieces, requested before the wait so their latency overlaps it
        __half sc[PIECES], zp[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
          const int piece = dtid + i * DQ_THREADS;
          const int r = piece >> 2, q = piece & 3;
          const int row = min(n0 + r, p.n - 1);
          const int grp = min((kb * BK + q * 16) / p.block_size, groups - 1);
          sc[i] = p.scales[(size_t)row * groups + grp];
          if (HAS_ZERO) zp[i] = p.zeros[(size_t)row * groups + grp];
        }
        if (!mbar_wait(&q_full[s], phase)) { ok = false; break; }
        const uint8_t* sq = stages + (size_t)s * Cfg::STAGE_BYTES + Cfg::A_BYTES;
        uint8_t* sb = stages + (size_t)s * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::Q_BYTES;
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
          const int piece = dtid + i * DQ_THREADS;
          const int r = piece >> 2, q = piece & 3;
          const uint4 w = *reinterpret_cast<const uint4*>(sq + piece * 16);
          const ScalePair sp = make_scale(sc[i], HAS_ZERO, HAS_ZERO ? zp[i] : __half());
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
          uint32_t h[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __half2 lo, hi;
            dequant4(ww[j], sp, lo, hi);
            h[2 * j] = half2_as_u32(lo);
            h[2 * j + 1] = half2_as_u32(hi);
          }
          uint8_t* rowp = sb + r * 128;
          *reinterpret_cast<uint4*>(rowp + (((2 * q) ^ (r & 7)) * 16)) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(rowp + (((2 * q + 1) ^ (r & 7)) * 16)) = make_uint4(h[4], h[5], h[6], h[7]);
        }
        // make the generic-proxy writes visible to the tensor core's async-proxy reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[s]);
      }
    }
  }
  if (!ok) atomicOr(p.status, 8u);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool Z>
int launch_u8_tc_t(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  using Cfg = U8Cfg<BN>;
  auto kfn = gemm_u8_tc_kernel<BN, Z>;
  if (int rc = opt_in_smem(ctx, kfn, Cfg::SMEM); rc != ADR_OK) return rc;
  CUtensorMap map_a, map_q;
  {
    const uint64_t dims[2] = {(uint64_t)a.p, (uint64_t)a.m};
    const uint64_t strides[1] = {(uint64_t)a.p * 2};
    const uint32_t box[2] = {BK, BM};
    int rc = tma_get(ctx, &map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.lhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a.p, (uint64_t)a.n};
    const uint64_t strides[1] = {(uint64_t)a.p};
    const uint32_t box[2] = {BK, (uint32_t)BN};
    int rc = tma_get(ctx, &map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != ADR_OK) return rc;
  }
  U8TcParams p{a.out, a.scales, a.zeros, a.m, a.p, a.n, a.block_size, a.beta, ctx->d_status};
  const long long tiles = (long long)((a.n + BN - 1) / BN) * ((a.m + BM - 1) / BM);
  const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const unsigned grid = (unsigned)std::min<long long>(tiles, sms);
  kfn<<<grid, U8TC_THREADS, Cfg::SMEM, stream>>>(map_a, map_q, p);
  return after_launch(ctx);
}

}  // namespace

bool u8_tc_supports(const adr_ctx* ctx, const U8Args& a) {
  if (!ctx->encode_tiled_fn) return false;
  if (a.p % 16 != 0 || a.block_size % 16 != 0 || a.p % a.block_size != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.lhs) & 15u) || (reinterpret_cast<uintptr_t>(a.rhs) & 15u))
    return false;
  return true;
}

int launch_u8_tc(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  if (!u8_tc_supports(ctx, a)) return ADR_ERR_SHAPE;
  // 128 x 256 tiles when they fill the machine, 128 x 128 otherwise
  const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const long long mt = (a.m + BM - 1) / BM;
  const bool wide = mt * ((a.n + 255) / 256) >= sms || a.n >= 8192;
  const bool z = a.zeros != nullptr;
  if (wide) return z ? launch_u8_tc_t<256, true>(ctx, stream, a) : launch_u8_tc_t<256, false>(ctx, stream, a);
  return z ? launch_u8_tc_t<128, true>(ctx, stream, a) : launch_u8_tc_t<128, false>(ctx, stream, a);
}

}  // namespace adr
