// fp16 strided/batched GEMM on the 5th-generation tensor cores:
//   out[b,y,x] = store(sum_k lhs[b,y,k] * rhs[b,k,x])
// replacing matmul_f16_fast / matmul_f16 (adrastea_kernels/cpp/matmul.cu:236-416,
// 493-513) and the WMMA kernels (matmul_nt_wmma_128x64x64.cu:8-78,
// matmul_nt_wmma_16x128x256.cu:8-68) for views TMA can describe.
//
// One CTA computes one 128 x BN output tile.  Six warps, specialised:
//   warp 0    producer: one thread issues TMA loads of the A (128 x 64) and B (BN x 64)
//             k-blocks into a ring of 128-byte-swizzled shared-memory stages
//   warp 1    owns tensor memory (alloc/dealloc); one thread issues tcgen05.mma
//             (M = 128, N = BN, K = 16 per instruction, fp32 accumulators in TMEM) and
//             frees each stage with tcgen05.commit
//   warps 2-5 epilogue: tcgen05.ld the accumulator (warp w reads TMEM lanes
//             32*(w%4)..+31 = tile rows), apply the reference's fused store op, mask
//             and scale, write fp16 to the (arbitrarily strided) output
// Rows and k beyond the operands' extents are zero-filled by TMA, so m, n and k need no
// divisibility; only the 16-byte alignment rules of TMA apply (gemm_f16_tc_supports).
// Every mbarrier wait is bounded: a wait that runs out sets the context's status word,
// the kernel still frees its tensor memory and returns.
#include <algorithm>

#include "tcgen05.cuh"

namespace adr {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // fp16 elements: one 128-byte swizzle row
constexpr int TC_THREADS = 192;
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
  static constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
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

// One 32-column chunk of one accumulator row: apply the fused op and store.
template <int STORE>
__device__ __forceinline__ void store_chunk(const TcParams& p, const uint32_t (&acc)[32],
                                            __half* orow, int y, int x0, float pre, __half hscale) {
  const bool causal = p.mask == ADR_MASK_CAUSAL;
  const bool vec = p.s_ox == 1 && x0 + 32 <= p.n &&
                   (reinterpret_cast<uintptr_t>(orow + x0) & 15u) == 0;
  __align__(16) __half oldv[32];
  if (store_reads_out(STORE)) {
    if (vec) {
      const uint4* src = reinterpret_cast<const uint4*>(orow + x0);
#pragma unroll
      for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(&oldv[q * 8]) = src[q];
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        oldv[j] = (x0 + j < p.n) ? orow[(int64_t)(x0 + j) * p.s_ox] : __float2half_rn(0.0f);
    }
  }
  __align__(16) __half res[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int x = x0 + j;
    float bias = 0.0f;
    if (store_uses_bias(STORE)) bias = (x < p.n) ? __half2float(p.bias[x]) : 0.0f;
    const __half old = store_reads_out(STORE) ? oldv[j] : __float2half_rn(0.0f);
    __half r = store_apply<STORE>(__uint_as_float(acc[j]) * pre, old, bias, p.beta, hscale);
    if (causal && x > y) r = __ushort_as_half((unsigned short)0xFC00);  // -inf
    res[j] = r;
  }
  if (vec) {
    uint4* dst = reinterpret_cast<uint4*>(orow + x0);
#pragma unroll
    for (int q = 0; q < 4; ++q) dst[q] = *reinterpret_cast<const uint4*>(&res[q * 8]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (x0 + j < p.n) orow[(int64_t)(x0 + j) * p.s_ox] = res[j];
  }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_b, TcParams p) {
  using Cfg = TcCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* acc_bar = empty_bar + Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM, b = blockIdx.z;
  const int num_kb = (p.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const int az = p.a_bcast ? 0 : b, bz = p.b_bcast ? 0 : b;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::STAGES;
        const unsigned phase = (unsigned)(kb / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], phase ^ 1u)) { ok = false; break; }
        uint8_t* sa = stages + (size_t)s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
        tma_load_3d(sa, &map_a, kb * BK, m0, az, &full_bar[s]);
        tma_load_3d(sa + Cfg::A_BYTES, &map_b, kb * BK, n0, bz, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BN, false);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % Cfg::STAGES;
        const unsigned phase = (unsigned)(kb / Cfg::STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], phase)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(stages + (size_t)s * Cfg::STAGE_BYTES);
        const uint64_t adesc = umma_desc_k_sw128(sa);
        const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::A_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          // 16 fp16 = 32 bytes further along the swizzled row: +2 in the address field
          umma_f16(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                   (kb > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
      }
      umma_commit(acc_bar);  // the accumulator is complete once every MMA is done
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp id % 4) ..
    const int row = quarter * 32 + lane;
    const int y = m0 + row;
    ok = mbar_wait(acc_bar, 0);
    tc_fence_after_sync();
    const __half hscale = __float2half_rn(p.scale);
    // a load-side scale multiplies both operands (matmul.cu:62): s^2 on the product
    const float hs = __half2float(hscale);
    const float pre = p.load == ADR_LOAD_SCALE ? hs * hs : 1.0f;
    __half* orow = p.out + (int64_t)b * p.s_oz + (int64_t)y * p.s_oy;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      const int x0 = n0 + c * 32;
      if (x0 >= p.n) break;  // uniform across the warp
      uint32_t acc[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), acc);
      tmem_ld_wait();
      if (y < p.m && ok) {
        switch (p.store) {
          case ADR_STORE_SCALE: store_chunk<ADR_STORE_SCALE>(p, acc, orow, y, x0, pre, hscale); break;
          case ADR_STORE_ADD: store_chunk<ADR_STORE_ADD>(p, acc, orow, y, x0, pre, hscale); break;
          case ADR_STORE_BETA_BIAS: store_chunk<ADR_STORE_BETA_BIAS>(p, acc, orow, y, x0, pre, hscale); break;
          case ADR_STORE_BETA_GELU_BIAS: store_chunk<ADR_STORE_BETA_GELU_BIAS>(p, acc, orow, y, x0, pre, hscale); break;
          case ADR_STORE_QUICK_GELU_BIAS: store_chunk<ADR_STORE_QUICK_GELU_BIAS>(p, acc, orow, y, x0, pre, hscale); break;
          case STORE_NT_BETA: store_chunk<STORE_NT_BETA>(p, acc, orow, y, x0, pre, hscale); break;
          default: store_chunk<ADR_STORE_IDENTITY>(p, acc, orow, y, x0, pre, hscale); break;
        }
      }
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

template <int BN>
int launch_tc(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  using Cfg = TcCfg<BN>;
  auto kfn = gemm_f16_tc_kernel<BN>;
  static bool configured[64] = {};
  const int dev = ctx->device & 63;
  if (!configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
    if (e != cudaSuccess) {
      ctx->last_cuda_error = (int)e;
      return ADR_ERR_CUDA;
    }
    configured[dev] = true;
  }
  const bool a_bcast = a.batches > 1 && a.s_lz == 0;
  const bool b_bcast = a.batches > 1 && a.s_rz == 0;
  CUtensorMap map_a, map_b;
  {
    const uint64_t za = a_bcast || a.batches == 1 ? 1 : (uint64_t)a.batches;
    const uint64_t dims[3] = {(uint64_t)a.k, (uint64_t)a.m, za};
    const uint64_t zs = za == 1 ? (uint64_t)a.s_ly * 2 * (uint64_t)a.m : (uint64_t)a.s_lz * 2;
    const uint64_t strides[2] = {(uint64_t)a.s_ly * 2, zs};
    const uint32_t box[3] = {BK, BM, 1};
    int rc = tma_get(ctx, &map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a.lhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  {
    const uint64_t zb = b_bcast || a.batches == 1 ? 1 : (uint64_t)a.batches;
    const uint64_t dims[3] = {(uint64_t)a.k, (uint64_t)a.n, zb};
    const uint64_t zs = zb == 1 ? (uint64_t)a.s_rx * 2 * (uint64_t)a.n : (uint64_t)a.s_rz * 2;
    const uint64_t strides[2] = {(uint64_t)a.s_rx * 2, zs};
    const uint32_t box[3] = {BK, (uint32_t)BN, 1};
    int rc = tma_get(ctx, &map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  TcParams p{a.out, a.bias, a.batches, a.m, a.k, a.n, a.s_ox, a.s_oy, a.s_oz,
             a_bcast ? 1 : 0, b_bcast ? 1 : 0, a.beta, a.scale, a.store, a.load, a.mask,
             ctx->d_status};
  dim3 grid((a.n + BN - 1) / BN, (a.m + BM - 1) / BM, a.batches);
  kfn<<<grid, TC_THREADS, Cfg::SMEM, stream>>>(map_a, map_b, p);
  return after_launch(ctx);
}

int pick_bn(const adr_ctx* ctx, const MatmulArgs& a) {
  if (ctx->tune_tc_bn == 32 || ctx->tune_tc_bn == 64 || ctx->tune_tc_bn == 128 ||
      ctx->tune_tc_bn == 256)
    return ctx->tune_tc_bn;
  const long long sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const long long mt = (a.m + BM - 1) / BM;
  for (int bn : {256, 128, 64, 32}) {
    if (bn > 32 && a.n <= bn / 2) continue;  // do not pad n beyond the next tile size
    const long long ctas = mt * ((a.n + bn - 1) / bn) * a.batches;
    if (ctas >= sms || bn == 32) return bn;
  }
  return 32;
}

}  // namespace

bool gemm_f16_tc_supports(const adr_ctx* ctx, const MatmulArgs& a) {
  if (!ctx->encode_tiled_fn) return false;
  if (a.s_lx != 1 || a.s_ry != 1) return false;             // both operands k-contiguous
  if (a.s_ly % 8 != 0 || a.s_rx % 8 != 0) return false;     // 16-byte row pitches
  if (a.batches > 1 && (a.s_lz % 8 != 0 || a.s_rz % 8 != 0)) return false;
  if ((reinterpret_cast<uintptr_t>(a.lhs) & 15u) || (reinterpret_cast<uintptr_t>(a.rhs) & 15u))
    return false;
  if (a.batches > 65535 || (a.m + BM - 1) / BM > 65535) return false;
  return true;
}

int launch_gemm_f16_tc(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  switch (pick_bn(ctx, a)) {
    case 256: return launch_tc<256>(ctx, stream, a);
    case 128: return launch_tc<128>(ctx, stream, a);
    case 64: return launch_tc<64>(ctx, stream, a);
    default: return launch_tc<32>(ctx, stream, a);
  }
}

int init_gemm_f16_tc(adr_ctx*) { return ADR_OK; }
void destroy_gemm_f16_tc(adr_ctx*) {}

}  // namespace adr
