// fp16 strided/batched GEMM on CUDA cores, any strides, every fused op.
//
// This is the kernel behind adr_matmul_f16_slow and the fallback of
// adr_matmul_f16 for views the tensor-core kernel cannot take.  It keeps the
// reference's arithmetic exactly (adrastea_kernels/cpp/matmul.cu:214-218,
// 370-376): each product is an fp16 multiply (rounded to fp16), widened to
// fp32 and added sequentially in k order, so its output is bit-identical to
// the reference kernels' for the ops without transcendental functions.
#include "common.cuh"

namespace adr {

namespace {

constexpr int BM = 64, BN = 64, BK = 32;
constexpr int PAD = 2;

__global__ void __launch_bounds__(256) gemm_f16_simt_kernel(MatmulArgs a) {
  __shared__ __half As[BK][BM + PAD];
  __shared__ __half Bs[BK][BN + PAD];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int bx = blockIdx.x, by = blockIdx.y, b = blockIdx.z;
  const int m0 = by * BM, n0 = bx * BN;

  const __half* lhs = a.lhs + (int64_t)b * a.s_lz;
  const __half* rhs = a.rhs + (int64_t)b * a.s_rz;
  __half* out = a.out + (int64_t)b * a.s_oz;

  const __half hscale = __float2half_rn(a.scale);
  const bool load_scale = a.load == ADR_LOAD_SCALE;
  // Pick the thread->element mapping that walks the contiguous dimension.
  const bool a_k_fast = a.s_lx == 1 || a.s_ly != 1;
  const bool b_n_fast = a.s_rx == 1 || a.s_ry != 1;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < a.k; k0 += BK) {
    // ---- fill A tile: As[kk][r] = load(lhs[(m0+r), (k0+kk)]) ----
#pragma unroll
    for (int it = 0; it < (BM * BK) / 256; ++it) {
      int e = tid + it * 256;
      int kk, r;
      if (a_k_fast) { kk = e % BK; r = e / BK; } else { r = e % BM; kk = e / BM; }
      __half v = __float2half_rn(0.0f);
      if (m0 + r < a.m && k0 + kk < a.k) {
        v = lhs[(int64_t)(m0 + r) * a.s_ly + (int64_t)(k0 + kk) * a.s_lx];
        if (load_scale) v = __hmul(v, hscale);
      }
      As[kk][r] = v;
    }
    // ---- fill B tile: Bs[kk][c] = load(rhs[(k0+kk), (n0+c)]) ----
#pragma unroll
    for (int it = 0; it < (BN * BK) / 256; ++it) {
      int e = tid + it * 256;
      int kk, c;
      if (b_n_fast) { c = e % BN; kk = e / BN; } else { kk = e % BK; c = e / BK; }
      __half v = __float2half_rn(0.0f);
      if (n0 + c < a.n && k0 + kk < a.k) {
        v = rhs[(int64_t)(k0 + kk) * a.s_ry + (int64_t)(n0 + c) * a.s_rx];
        if (load_scale) v = __hmul(v, hscale);
      }
      Bs[kk][c] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      __half av[4];
      __half2 bv[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
      bv[0] = *reinterpret_cast<const __half2*>(&Bs[kk][tx * 4]);
      bv[1] = *reinterpret_cast<const __half2*>(&Bs[kk][tx * 4 + 2]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2 ai = __half2half2(av[i]);
        float2 p0 = __half22float2(__hmul2(ai, bv[0]));
        float2 p1 = __half22float2(__hmul2(ai, bv[1]));
        acc[i][0] += p0.x;
        acc[i][1] += p0.y;
        acc[i][2] += p1.x;
        acc[i][3] += p1.y;
      }
    }
    __syncthreads();
  }

  const int store = (int)a.store;
  const bool causal = a.mask == ADR_MASK_CAUSAL;
  const bool rd_out = store_reads_out(store);
  const bool use_bias = store_uses_bias(store);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int y = m0 + ty * 4 + i;
    if (y >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int x = n0 + tx * 4 + j;
      if (x >= a.n) continue;
      __half* dst = out + (int64_t)y * a.s_oy + (int64_t)x * a.s_ox;
      if (causal && x > y) {
        *dst = __ushort_as_half((unsigned short)0xFC00);  // -inf
        continue;
      }
      __half old = rd_out ? *dst : __float2half_rn(0.0f);
      float bias = use_bias ? __half2float(a.bias[x]) : 0.0f;
      *dst = store_apply_rt(store, acc[i][j], old, bias, a.beta, hscale);
    }
  }
}

}  // namespace

int launch_gemm_f16_simt(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a) {
  dim3 grid((a.n + BN - 1) / BN, (a.m + BM - 1) / BM, a.batches);
  if (grid.y > 65535u || grid.z > 65535u) return ADR_ERR_SHAPE;
  gemm_f16_simt_kernel<<<grid, 256, 0, stream>>>(a);
  return after_launch(ctx);
}

}  // namespace adr
