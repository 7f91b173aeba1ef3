// u8-weight dequantising GEMV/GEMM for decode shapes:
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// replacing adrastea_kernels/cpp/matmul_nt_fp16u8.cu:4-24 and
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83 for small m.
//
// These shapes are HBM-bound: the weight matrix is read exactly once with
// 128-bit loads that bypass L1, dequantised in registers (u8_common.cuh) and
// never staged through shared memory.  Three kernels:
//   u8_gemv_kernel  m <= 4   fp32 FMA on CUDA cores, warp-shuffle reduction
//   u8_mma_kernel   m <= 16  the dequantised fp16 weights feed
//                            mma.sync.m16n8k16 straight from registers
//                            (weights are the 16-row operand, the tokens the
//                            8-column operand), split-k across the warps of a
//                            CTA, reduced through shared memory
//   u8_simt_kernel  any m    plain restatement, used as a cross-check
#include "u8_common.cuh"

namespace adr {

namespace {

// ---------------------------------------------------------------------------
// Plain restatement: one CTA per output column, 8 rows of lhs per CTA.
// ---------------------------------------------------------------------------
template <bool HAS_ZERO>
__global__ void __launch_bounds__(128) u8_simt_kernel(U8Args a) {
  const int c = blockIdx.x;
  const int r0 = blockIdx.y * 8;
  const int groups = a.p / a.block_size;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int k = threadIdx.x; k < a.p; k += blockDim.x) {
    int g = k / a.block_size;
    float s = __half2float(a.scales[(size_t)c * groups + g]);
    float z = HAS_ZERO ? __half2float(a.zeros[(size_t)c * groups + g]) : 127.5f;
    float w = __half2float(dequant_one_f32(a.rhs[(size_t)c * a.p + k], s, z));
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (r0 + i < a.m) acc[i] = fmaf(__half2float(a.lhs[(size_t)(r0 + i) * a.p + k]), w, acc[i]);
  }
  __shared__ float red[4][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5][i] = v;
  }
  __syncthreads();
  if (threadIdx.x < 8 && r0 + threadIdx.x < a.m) {
    int i = threadIdx.x;
    float v = red[0][i] + red[1][i] + red[2][i] + red[3][i];
    __half* dst = a.out + (size_t)(r0 + i) * a.n + c;
    *dst = __float2half_rn(fmaf(a.beta, __half2float(*dst), v));
  }
}

// ---------------------------------------------------------------------------
// m <= 4: each warp owns ROWS weight rows over the whole of p.  A lane covers
// 16 consecutive k of every 512-byte step, so a warp reads 512 contiguous
// bytes per row per step.
// ---------------------------------------------------------------------------
template <int M, int ROWS, bool HAS_ZERO>
__global__ void __launch_bounds__(256) u8_gemv_kernel(U8Args a) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.x * 8 + warp) * ROWS;
  if (n0 >= a.n) return;
  const int groups = a.p / a.block_size;

  float acc[ROWS][M];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int i = 0; i < M; ++i) acc[r][i] = 0.0f;

  const uint8_t* wrow[ROWS];
  const __half* srow[ROWS];
  const __half* zrow[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    int n = min(n0 + r, a.n - 1);  // tail rows re-read the last row, never stored
    wrow[r] = a.rhs + (size_t)n * a.p;
    srow[r] = a.scales + (size_t)n * groups;
    zrow[r] = HAS_ZERO ? a.zeros + (size_t)n * groups : nullptr;
  }

  for (int k = lane * 16; k < a.p; k += 512) {
    uint4 wq[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) wq[r] = ldg_nc_16(wrow[r] + k);
    const int g = k / a.block_size;
    // activations for these 16 k: M rows of 16 halves, widened once
    float xf[M][16];
#pragma unroll
    for (int i = 0; i < M; ++i) {
      uint4 x0 = __ldg(reinterpret_cast<const uint4*>(a.lhs + (size_t)i * a.p + k));
      uint4 x1 = __ldg(reinterpret_cast<const uint4*>(a.lhs + (size_t)i * a.p + k + 8));
      const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 f = __half22float2(u32_as_half2(xw[j]));
        xf[i][2 * j] = f.x;
        xf[i][2 * j + 1] = f.y;
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      ScalePair sp = make_scale(srow[r][g], HAS_ZERO, HAS_ZERO ? zrow[r][g] : __half());
      const uint32_t ww[4] = {wq[r].x, wq[r].y, wq[r].z, wq[r].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 lo, hi;
        dequant4(ww[j], sp, lo, hi);
        float2 f0 = __half22float2(lo), f1 = __half22float2(hi);
#pragma unroll
        for (int i = 0; i < M; ++i) {
          acc[r][i] = fmaf(xf[i][4 * j + 0], f0.x, acc[r][i]);
          acc[r][i] = fmaf(xf[i][4 * j + 1], f0.y, acc[r][i]);
          acc[r][i] = fmaf(xf[i][4 * j + 2], f1.x, acc[r][i]);
          acc[r][i] = fmaf(xf[i][4 * j + 3], f1.y, acc[r][i]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int i = 0; i < M; ++i) {
      float v = acc[r][i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][i] = v;
    }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (n0 + r >= a.n) continue;
#pragma unroll
      for (int i = 0; i < M; ++i) {
        __half* dst = a.out + (size_t)i * a.n + n0 + r;
        *dst = __float2half_rn(fmaf(a.beta, __half2float(*dst), acc[r][i]));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// m <= 16: tensor-core form fed from registers.
//
// A CTA owns 16 weight rows (the "M" side of mma.m16n8k16) and all of p; its
// WARPS warps interleave over 64-byte k-chunks.  Lane (g = lane/4, t = lane%4)
// loads 16 bytes of row g and of row g+8 at chunk offset 16*t.  The four
// 32-bit words of that load become the A fragments of four MMAs; since any
// permutation of k is allowed as long as both operands use it, word j of the
// lane supplies k-slots (2t,2t+1) from bytes (4j,4j+1) and k-slots
// (2t+8,2t+9) from bytes (4j+2,4j+3), and the B fragment takes the tokens'
// activations at the same k.  Nothing goes through shared memory except the
// final cross-warp reduction.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int WARPS, int U, bool HAS_ZERO>
__global__ void __launch_bounds__(WARPS * 32) u8_mma_kernel(U8Args a) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int groups = a.p / a.block_size;
  const int nchunks = a.p / 64;  // p % 64 == 0 is checked by the launcher

  const int ra = min(n0 + g, a.n - 1);
  const int rb = min(n0 + g + 8, a.n - 1);
  const uint8_t* wa = a.rhs + (size_t)ra * a.p + t * 16;
  const uint8_t* wb = a.rhs + (size_t)rb * a.p + t * 16;
  const __half* sa = a.scales + (size_t)ra * groups;
  const __half* sb = a.scales + (size_t)rb * groups;
  const __half* za = HAS_ZERO ? a.zeros + (size_t)ra * groups : nullptr;
  const __half* zb = HAS_ZERO ? a.zeros + (size_t)rb * groups : nullptr;

  // activations of token g (and g+8): 16 halves at chunk offset 16*t
  const __half* x0 = a.lhs + (size_t)min(g, a.m - 1) * a.p + t * 16;
  const __half* x1 = a.lhs + (size_t)min(g + 8, a.m - 1) * a.p + t * 16;
  const bool x0_ok = g < a.m;
  const bool x1_ok = MT > 1 && (g + 8) < a.m;

  float d[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) d[i][j] = 0.0f;

  for (int c0 = warp; c0 < nchunks; c0 += WARPS * U) {
    uint4 qa[U], qb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int c = c0 + u * WARPS;
      if (c < nchunks) {
        qa[u] = ldg_nc_16(wa + (size_t)c * 64);
        qb[u] = ldg_nc_16(wb + (size_t)c * 64);
      } else {
        qa[u] = make_uint4(0, 0, 0, 0);
        qb[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int c = c0 + u * WARPS;
      if (c >= nchunks) break;
      const int grp = (c * 64 + t * 16) / a.block_size;
      ScalePair spa = make_scale(sa[grp], HAS_ZERO, HAS_ZERO ? za[grp] : __half());
      ScalePair spb = make_scale(sb[grp], HAS_ZERO, HAS_ZERO ? zb[grp] : __half());
      uint32_t xw0[8], xw1[8];
      {
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        if (x0_ok) {
          v0 = __ldg(reinterpret_cast<const uint4*>(x0 + (size_t)c * 64));
          v1 = __ldg(reinterpret_cast<const uint4*>(x0 + (size_t)c * 64 + 8));
        }
        xw0[0] = v0.x; xw0[1] = v0.y; xw0[2] = v0.z; xw0[3] = v0.w;
        xw0[4] = v1.x; xw0[5] = v1.y; xw0[6] = v1.z; xw0[7] = v1.w;
      }
      if (MT > 1) {
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        if (x1_ok) {
          v0 = __ldg(reinterpret_cast<const uint4*>(x1 + (size_t)c * 64));
          v1 = __ldg(reinterpret_cast<const uint4*>(x1 + (size_t)c * 64 + 8));
        }
        xw1[0] = v0.x; xw1[1] = v0.y; xw1[2] = v0.z; xw1[3] = v0.w;
        xw1[4] = v1.x; xw1[5] = v1.y; xw1[6] = v1.z; xw1[7] = v1.w;
      }
      const uint32_t wwa[4] = {qa[u].x, qa[u].y, qa[u].z, qa[u].w};
      const uint32_t wwb[4] = {qb[u].x, qb[u].y, qb[u].z, qb[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 a_lo, a_hi, b_lo, b_hi;
        dequant4(wwa[j], spa, a_lo, a_hi);
        dequant4(wwb[j], spb, b_lo, b_hi);
        uint32_t A0 = half2_as_u32(a_lo), A2 = half2_as_u32(a_hi);
        uint32_t A1 = half2_as_u32(b_lo), A3 = half2_as_u32(b_hi);
        mma_16816(d[0], A0, A1, A2, A3, xw0[2 * j], xw0[2 * j + 1]);
        if (MT > 1) mma_16816(d[MT - 1], A0, A1, A2, A3, xw1[2 * j], xw1[2 * j + 1]);
      }
    }
  }

  // cross-warp reduction: red[warp][row 0..15][token 0..8*MT-1]
  __shared__ float red[WARPS][16][8 * MT + 1];
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    red[warp][g][i * 8 + 2 * t] = d[i][0];
    red[warp][g][i * 8 + 2 * t + 1] = d[i][1];
    red[warp][g + 8][i * 8 + 2 * t] = d[i][2];
    red[warp][g + 8][i * 8 + 2 * t + 1] = d[i][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * a.m; e += WARPS * 32) {
    int row = e & 15, tok = e >> 4;
    if (n0 + row >= a.n) continue;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][row][tok];
    __half* dst = a.out + (size_t)tok * a.n + n0 + row;
    *dst = __float2half_rn(fmaf(a.beta, __half2float(*dst), v));
  }
}

template <int M, bool Z>
int launch_gemv_m(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  constexpr int ROWS = 2;
  int warps_needed = (a.n + ROWS - 1) / ROWS;
  int grid = (warps_needed + 7) / 8;
  u8_gemv_kernel<M, ROWS, Z><<<grid, 256, 0, stream>>>(a);
  return after_launch(ctx);
}

}  // namespace

int launch_u8_simt(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  dim3 grid(a.n, (a.m + 7) / 8);
  if (grid.y > 65535u) return ADR_ERR_SHAPE;
  if (a.zeros) u8_simt_kernel<true><<<grid, 128, 0, stream>>>(a);
  else u8_simt_kernel<false><<<grid, 128, 0, stream>>>(a);
  return after_launch(ctx);
}

int launch_u8_gemv(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  if (a.m < 1 || a.m > 4 || a.p % 16 != 0 || a.block_size % 16 != 0) return ADR_ERR_SHAPE;
  const bool z = a.zeros != nullptr;
  switch (a.m) {
    case 1: return z ? launch_gemv_m<1, true>(ctx, stream, a) : launch_gemv_m<1, false>(ctx, stream, a);
    case 2: return z ? launch_gemv_m<2, true>(ctx, stream, a) : launch_gemv_m<2, false>(ctx, stream, a);
    case 3: return z ? launch_gemv_m<3, true>(ctx, stream, a) : launch_gemv_m<3, false>(ctx, stream, a);
    default: return z ? launch_gemv_m<4, true>(ctx, stream, a) : launch_gemv_m<4, false>(ctx, stream, a);
  }
}

int launch_u8_mma(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  if (a.m < 1 || a.m > 16 || a.p % 64 != 0 || a.block_size % 16 != 0) return ADR_ERR_SHAPE;
  constexpr int WARPS = 8, U = 4;
  const int grid = (a.n + 15) / 16;
  const bool z = a.zeros != nullptr;
  if (a.m <= 8) {
    if (z) u8_mma_kernel<1, WARPS, U, true><<<grid, WARPS * 32, 0, stream>>>(a);
    else u8_mma_kernel<1, WARPS, U, false><<<grid, WARPS * 32, 0, stream>>>(a);
  } else {
    if (z) u8_mma_kernel<2, WARPS, U, true><<<grid, WARPS * 32, 0, stream>>>(a);
    else u8_mma_kernel<2, WARPS, U, false><<<grid, WARPS * 32, 0, stream>>>(a);
  }
  return after_launch(ctx);
}

int init_u8_kernels(adr_ctx*) { return ADR_OK; }

}  // namespace adr
