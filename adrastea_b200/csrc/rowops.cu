// The kernels either side of the matmuls in a decoder layer: row normalisation, rotary
// position encoding, row softmax, the SiluMul/Add elementwise pair, and two fused forms for
// decoding against a key/value cache.
//
// rms_norm, rotary, softmax_rows and elementwise_binary_2d_f16 restate the reference's
// kernels (adrastea_kernels/cpp/normalize.cu:7-58, 150-220; rotary.cu:4-29;
// elementwise.cu:16-33, 118-160) with the same thread-to-element mapping and the same
// order of floating-point operations, so that the results carry the same bits as those
// kernels compiled for this GPU:
//   * the row reductions sum elements tid, tid + 256, ... per thread in that order, then
//     combine lanes with an xor butterfly (16, 8, 4, 2, 1) and the eight warp sums with a
//     second butterfly (4, 2, 1);
//   * rotary computes (pos + row) / powf(theta, c / head_dim) and rotates with cosf/sinf.
// The loads are hoisted ahead of the dependent adds (order of additions unchanged).
//
// decode_rope_append and decode_attention have no counterpart: the reference re-runs the
// whole prefix for every token (adrastea_models/src/llama.rs:426-427) and keeps no cache.
// They apply the same formulas (rotary above; scores = fp16(q.k) *h fp16(scale), softmax in
// fp32 over fp16 scores, fp16 probabilities, fp32 sum of p.v) to one new token per sequence,
// with the position read from device memory so that a captured step can be replayed.
//
// Every kernel can be launched with programmatic stream serialisation (tunable "pdl"): it
// lets its successor start at once and itself waits for its predecessor before touching
// memory.
#include <algorithm>

#include "common.cuh"

namespace adr {

namespace {

constexpr int ROW_THREADS = 256;  // 8 warps per row, as the reference launches them

template <bool PDL>
__device__ __forceinline__ void pdl_enter() {
  if (PDL) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
}

// Sum over the block in the reference's order; every thread returns the same bits.
__device__ __forceinline__ float block_sum_256(float v, float* s_warp) {
  const int tid = threadIdx.x, warp = tid >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((tid & 31) == 0) s_warp[warp] = v;
  __syncthreads();
  float t = (tid & 31) < 8 ? s_warp[tid & 31] : 0.0f;
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
  // lanes 0..7 of every warp now hold the block sum
  t = __shfl_sync(0xffffffffu, t, 0);
  __syncthreads();  // s_warp may be reused
  return t;
}
__device__ __forceinline__ float block_max_256(float v, float* s_warp) {
  const int tid = threadIdx.x, warp = tid >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  if ((tid & 31) == 0) s_warp[warp] = v;
  __syncthreads();
  float t = (tid & 31) < 8 ? s_warp[tid & 31] : -INFINITY;
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
  t = __shfl_sync(0xffffffffu, t, 0);
  __syncthreads();
  return t;
}

// ---------------------------------------------------------------------------------------
// rms_norm (normalize.cu:7-58): out[r,i] = w[i] *h fp16(in[r,i] * rsqrt(mean(in^2) + eps))
// ---------------------------------------------------------------------------------------
template <bool PDL>
__global__ void __launch_bounds__(ROW_THREADS)
    rms_norm_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                    const __half* __restrict__ w, int lx, int s_ox, int s_oy, int s_ix, int s_iy,
                    float eps) {
  __shared__ float s_warp[8];
  pdl_enter<PDL>();
  const int tid = threadIdx.x;
  const __half* irow = in + (int64_t)blockIdx.x * s_iy;
  __half* orow = out + (int64_t)blockIdx.x * s_oy;
  float sum = 0.0f;
  int i = tid;
  for (; i + 3 * ROW_THREADS < lx; i += 4 * ROW_THREADS) {
    const float v0 = __half2float(irow[(int64_t)i * s_ix]);
    const float v1 = __half2float(irow[(int64_t)(i + ROW_THREADS) * s_ix]);
    const float v2 = __half2float(irow[(int64_t)(i + 2 * ROW_THREADS) * s_ix]);
    const float v3 = __half2float(irow[(int64_t)(i + 3 * ROW_THREADS) * s_ix]);
    sum += v0 * v0;
    sum += v1 * v1;
    sum += v2 * v2;
    sum += v3 * v3;
  }
  for (; i < lx; i += ROW_THREADS) {
    const float v = __half2float(irow[(int64_t)i * s_ix]);
    sum += v * v;
  }
  const float total = block_sum_256(sum, s_warp);
  const float rms_inv = rsqrtf((total / lx) + eps);
  for (i = tid; i < lx; i += ROW_THREADS) {
    const float v = __half2float(irow[(int64_t)i * s_ix]);
    orow[(int64_t)i * s_ox] = __hmul(w[i], __float2half(v * rms_inv));
  }
}

// rms_norm on R rows per CTA at once, thread for thread the arithmetic above (contiguous rows of
// at most 4096 elements, many rows: a prefill's 8192 x 4096 activations took 41 us with one row
// per CTA).  See layer_norm_rows_kernel below for the reasoning.
template <bool PDL, int R>
__global__ void __launch_bounds__(ROW_THREADS)
    rms_norm_rows_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                         const __half* __restrict__ w, int lx, int ly, int s_oy, int s_iy, float eps) {
  __shared__ float s_warp[R][8];
  pdl_enter<PDL>();
  constexpr int KEEP = 16;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = blockIdx.x * R;
  float v[R][KEEP];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const __half* irow = in + (int64_t)min(row0 + r, ly - 1) * s_iy;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      v[r][j] = i < lx ? __half2float(irow[i]) : 0.0f;
    }
  }
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      if (tid + j * ROW_THREADS < lx) sum += v[r][j] * v[r][j];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) s_warp[r][warp] = sum;
    acc[r] = sum;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float t = lane < 8 ? s_warp[r][lane] : 0.0f;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    acc[r] = __shfl_sync(0xffffffffu, t, 0);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (row0 + r >= ly) break;
    const float rms_inv = rsqrtf((acc[r] / lx) + eps);
    __half* orow = out + (int64_t)(row0 + r) * s_oy;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      if (i < lx) orow[i] = __hmul(w[i], __float2half(v[r][j] * rms_inv));
    }
  }
}

// ---------------------------------------------------------------------------------------
// layer_norm (normalize.cu:60-145): out[r,i] = fp16((in[r,i] - mean) / sqrt(var + eps) * w[i] + b[i])
// with mean and the (biased) variance in fp32, each summed in the reference's order: thread t
// adds elements t, t + 256, ..., then the butterflies of block_sum_256.  A thread keeps its
// elements in registers over the three passes when the row has at most 16 of them per thread.
// ---------------------------------------------------------------------------------------
template <bool PDL>
__global__ void __launch_bounds__(ROW_THREADS)
    layer_norm_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                      const __half* __restrict__ w, const __half* __restrict__ b, int lx, int s_ox,
                      int s_oy, int s_ix, int s_iy, float eps) {
  __shared__ float s_warp[8];
  pdl_enter<PDL>();
  constexpr int KEEP = 16;
  const int tid = threadIdx.x;
  const __half* irow = in + (int64_t)blockIdx.x * s_iy;
  __half* orow = out + (int64_t)blockIdx.x * s_oy;
  const bool cached = lx <= KEEP * ROW_THREADS;
  float v[KEEP];
  float sum = 0.0f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      v[j] = i < lx ? __half2float(irow[(int64_t)i * s_ix]) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      if (tid + j * ROW_THREADS < lx) sum += v[j];
  } else {
    for (int i = tid; i < lx; i += ROW_THREADS) sum += __half2float(irow[(int64_t)i * s_ix]);
  }
  const float mean = block_sum_256(sum, s_warp) / lx;
  float dev2 = 0.0f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      if (tid + j * ROW_THREADS < lx) dev2 += (v[j] - mean) * (v[j] - mean);
  } else {
    for (int i = tid; i < lx; i += ROW_THREADS) {
      const float x = __half2float(irow[(int64_t)i * s_ix]);
      dev2 += (x - mean) * (x - mean);
    }
  }
  const float stddev = sqrtf(block_sum_256(dev2, s_warp) / lx + eps);
  if (cached) {
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      if (i < lx)
        orow[(int64_t)i * s_ox] =
            __float2half((v[j] - mean) / stddev * __half2float(w[i]) + __half2float(b[i]));
    }
  } else {
    for (int i = tid; i < lx; i += ROW_THREADS)
      orow[(int64_t)i * s_ox] = __float2half((__half2float(irow[(int64_t)i * s_ix]) - mean) / stddev *
                                                 __half2float(w[i]) +
                                             __half2float(b[i]));
  }
}

// The same arithmetic, thread for thread, on R rows per CTA at once (contiguous rows of at most
// 1024 elements, many rows): with one 2 KB row per CTA the kernel ran at a tenth of the HBM rate
// (16448 rows of 1024: 92 us), bound by the latency of a row's load -> two block sums -> store
// chain with 8 bytes per thread in flight.  R rows put R x 8 bytes per thread in flight and share
// the two barriers of each block sum; weights and bias are read once per R rows.
template <bool PDL, int R>
__global__ void __launch_bounds__(ROW_THREADS)
    layer_norm_rows_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                           const __half* __restrict__ w, const __half* __restrict__ b, int lx, int ly,
                           int s_oy, int s_iy, float eps) {
  __shared__ float s_warp[R][8];
  pdl_enter<PDL>();
  constexpr int KEEP = 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = blockIdx.x * R;
  float v[R][KEEP];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const __half* irow = in + (int64_t)min(row0 + r, ly - 1) * s_iy;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      v[r][j] = i < lx ? __half2float(irow[i]) : 0.0f;
    }
  }
  // block sums of R values in block_sum_256's order
  auto block_sums = [&](float (&x)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) x[r] += __shfl_xor_sync(0xffffffffu, x[r], off);
      if (lane == 0) s_warp[r][warp] = x[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float t = lane < 8 ? s_warp[r][lane] : 0.0f;
#pragma unroll
      for (int off = 4; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
      x[r] = __shfl_sync(0xffffffffu, t, 0);
    }
    __syncthreads();
  };
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    acc[r] = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      if (tid + j * ROW_THREADS < lx) acc[r] += v[r][j];
  }
  block_sums(acc);
  float mean[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    mean[r] = acc[r] / lx;
    acc[r] = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      if (tid + j * ROW_THREADS < lx) acc[r] += (v[r][j] - mean[r]) * (v[r][j] - mean[r]);
  }
  block_sums(acc);
  float wf[KEEP], bf[KEEP];
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = tid + j * ROW_THREADS;
    wf[j] = i < lx ? __half2float(w[i]) : 0.0f;
    bf[j] = i < lx ? __half2float(b[i]) : 0.0f;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (row0 + r >= ly) break;
    const float stddev = sqrtf(acc[r] / lx + eps);
    __half* orow = out + (int64_t)(row0 + r) * s_oy;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = tid + j * ROW_THREADS;
      if (i < lx) orow[i] = __float2half((v[r][j] - mean[r]) / stddev * wf[j] + bf[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// softmax_rows (normalize.cu:150-220), rows of `w` elements `pitch` apart
// ---------------------------------------------------------------------------------------
template <bool PDL>
__global__ void __launch_bounds__(ROW_THREADS)
    softmax_rows_kernel(__half* __restrict__ out, const __half* __restrict__ in, int h, int w,
                        int pitch, float temp) {
  __shared__ float s_warp[8];
  pdl_enter<PDL>();
  const int tid = threadIdx.x;
  const int64_t row_idx = ((int64_t)blockIdx.y * h + blockIdx.x) * pitch;
  const __half* irow = in + row_idx;
  __half* orow = out + row_idx;
  float mx = -INFINITY;
  for (int i = tid; i < w; i += ROW_THREADS) mx = fmaxf(mx, __half2float(irow[i]) / temp);
  mx = block_max_256(mx, s_warp);
  float sum = 0.0f;
  for (int i = tid; i < w; i += ROW_THREADS) sum += expf(__half2float(irow[i]) / temp - mx);
  sum = block_sum_256(sum, s_warp);
  for (int i = tid; i < w; i += ROW_THREADS)
    orow[i] = __float2half(expf(__half2float(irow[i]) / temp - mx) / sum);
}

// ---------------------------------------------------------------------------------------
// Rotary position embedding (the arithmetic of rotary.cu:4-29): each head is a row of
// interleaved 2-vectors (even column, odd column); 2-vector j of a head at position t is
// turned by t / theta^(2j / head_dim).  The turn is computed once per 2-vector as a
// (cos, sin) pair and applied as a 2x2 rotation; the decode-time kernel below applies the
// same pair to the query and to the key.
// ---------------------------------------------------------------------------------------
// One thread per 2-vector; blockIdx.y / threadIdx.y walk the rows (positions pos_offset + row).
template <bool PDL>
__global__ void __launch_bounds__(256)
    rope_rows_kernel(__half* out, const __half* in, int lx, int ly, int s_ox, int s_oy, int s_ix,
                     int s_iy, int n_heads, int pos_offset, float theta) {
  pdl_enter<PDL>();
  const int row = blockIdx.y * blockDim.y + threadIdx.y;
  const int col = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (row >= ly || col >= lx) return;
  const int head_dim = lx / n_heads;
  const __half* src = in + (int64_t)row * s_iy + (int64_t)col * s_ix;
  __half* dst = out + (int64_t)row * s_oy + (int64_t)col * s_ox;
  const __half2 turned =
      rope_apply(src[0], src[s_ix], rope_turn(pos_offset + row, col % head_dim, head_dim, theta));
  dst[0] = __low2half(turned);
  dst[s_ox] = __high2half(turned);
}

// The same rotation with the turn computed once per (row, pair of a head) and applied to every
// fourth head by the same thread: cos, sin and powf depend on the position and on the pair's
// index within its head only, and they are most of the kernel's instructions (q and k of a
// 512-token LLaMA-7B prefill, 64 heads: 21 -> 6 us).  Contiguous columns, 4-byte aligned rows.
template <bool PDL>
__global__ void __launch_bounds__(256)
    rope_rows_heads_kernel(__half* out, const __half* in, int head_dim, int ly, int s_oy, int s_iy,
                           int n_heads, int pos_offset, float theta) {
  pdl_enter<PDL>();
  const int row = blockIdx.y;
  const int pair = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= ly || 2 * pair >= head_dim) return;
  const Turn w = rope_turn(pos_offset + row, 2 * pair, head_dim, theta);
  const __half* src = in + (int64_t)row * s_iy + 2 * pair;
  __half* dst = out + (int64_t)row * s_oy + 2 * pair;
  for (int h = threadIdx.y; h < n_heads; h += blockDim.y) {
    const __half2 v = *reinterpret_cast<const __half2*>(src + (int64_t)h * head_dim);
    *reinterpret_cast<__half2*>(dst + (int64_t)h * head_dim) = rope_apply(__low2half(v), __high2half(v), w);
  }
}

// ---------------------------------------------------------------------------------------
// elementwise_binary_2d_f16 (elementwise.cu:16-33): Add = left +h right,
// SiluMul = fp16(float(left) / (1 + expf(-left)) * float(right))
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ __half binary_op(int op, __half l, __half r) {
  if (op == ADR_BINARY_ADD) return __hadd(l, r);
  return __float2half(__half2float(l) / (1.0f + expf(__half2float(__hneg(l)))) * __half2float(r));
}

template <bool PDL>
__global__ void __launch_bounds__(256)
    binary_2d_kernel(__half* out, const __half* left, const __half* right, int rows, int cols,
                     int s_o, int s_l, int s_r, int op) {
  pdl_enter<PDL>();
  const int r = blockIdx.y;
  // eight columns per thread when the row segments are 16-byte aligned
  const bool vec = (cols % 8 == 0) && (s_o % 8 == 0) && (s_l % 8 == 0) && (s_r % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(left) |
                     reinterpret_cast<uintptr_t>(right)) & 15u) == 0;
  const __half* lrow = left + (int64_t)r * s_l;
  const __half* rrow = right + (int64_t)r * s_r;
  __half* orow = out + (int64_t)r * s_o;
  if (vec) {
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8; c < cols;
         c += gridDim.x * blockDim.x * 8) {
      uint4 lv = *reinterpret_cast<const uint4*>(lrow + c);
      uint4 rv = *reinterpret_cast<const uint4*>(rrow + c);
      const __half* lh = reinterpret_cast<const __half*>(&lv);
      const __half* rh = reinterpret_cast<const __half*>(&rv);
      __align__(16) __half res[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) res[j] = binary_op(op, lh[j], rh[j]);
      *reinterpret_cast<uint4*>(orow + c) = *reinterpret_cast<const uint4*>(res);
    }
  } else {
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x)
      orow[c] = binary_op(op, lrow[c], rrow[c]);
  }
}

// ---------------------------------------------------------------------------------------
// Decoding against a key/value cache.  Cache layout: [B, S, n_heads * head_dim] fp16 (one
// row per position, heads side by side), the layout the reference's [S, H*hd] key/value
// tensors have for one sequence (llama.rs:530-537).
// ---------------------------------------------------------------------------------------

// One new token per sequence: q rotated in place, k rotated into the cache row of its
// position, v copied there.  grid (pairs / 256, B).
template <bool PDL>
__global__ void __launch_bounds__(256)
    decode_rope_append_kernel(__half* q, const __half* k, const __half* v, __half* k_cache,
                              __half* v_cache, int width, int n_heads, int S, int s_q, int s_k,
                              int s_v, const int* pos_dev, float theta) {
  pdl_enter<PDL>();
  const int b = blockIdx.y;
  const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= width) return;
  const int pos = *pos_dev;
  if (pos < 0 || pos >= S) return;  // the caller's position is outside the cache: write nothing
  const int head_dim = width / n_heads;
  const Turn w = rope_turn(pos, c % head_dim, head_dim, theta);
  __half* qrow = q + (int64_t)b * s_q;
  const __half* krow = k + (int64_t)b * s_k;
  const __half* vrow = v + (int64_t)b * s_v;
  const int64_t crow = ((int64_t)b * S + pos) * width;
  const __half2 qt = rope_apply(qrow[c], qrow[c + 1], w);
  qrow[c] = __low2half(qt);
  qrow[c + 1] = __high2half(qt);
  const __half2 kt = rope_apply(krow[c], krow[c + 1], w);
  k_cache[crow + c] = __low2half(kt);
  k_cache[crow + c + 1] = __high2half(kt);
  *reinterpret_cast<__half2*>(&v_cache[crow + c]) = *reinterpret_cast<const __half2*>(&vrow[c]);
}

constexpr int ATT_THREADS = 512;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_MAX_HD = 256;  // two 128-wide chunks per lane

__device__ __forceinline__ float4 ld_half4(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&u.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// One (head, sequence) per block: scores over positions 0..pos, softmax, probabilities . v.
// The rounding points are those of the reference's chain of kernels: fp16(q.k) *h
// fp16(scale) (matmul.cu Scale store), softmax in fp32 (normalize.cu:150-220) rounded to
// fp16 probabilities, fp32 sum of p.v rounded to fp16.
template <bool PDL>
__global__ void __launch_bounds__(ATT_THREADS)
    decode_attention_kernel(__half* out, const __half* q, const __half* k_cache,
                            const __half* v_cache, int n_heads, int head_dim, int S, int s_q,
                            int s_o, const int* pos_dev, float scale) {
  extern __shared__ float att_smem[];
  float* sc = att_smem;                         // [S] scores, then probabilities
  float* red = att_smem + S;                    // [ATT_WARPS][head_dim] partial outputs
  __shared__ float s_warp[ATT_WARPS];
  __shared__ float s_bcast;
  pdl_enter<PDL>();
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int width = n_heads * head_dim;
  int T = *pos_dev + 1;
  T = T < 0 ? 0 : (T > S ? S : T);
  const __half* qh = q + (int64_t)b * s_q + (int64_t)h * head_dim;
  const __half* kb = k_cache + (int64_t)b * S * width + (int64_t)h * head_dim;
  const __half* vb = v_cache + (int64_t)b * S * width + (int64_t)h * head_dim;
  const int nchunk = (head_dim + 127) / 128;  // 1 or 2
  const __half hscale = __float2half_rn(scale);

  float4 qv[2];
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    const int j = ch * 128 + lane * 4;
    qv[ch] = (ch < nchunk && j < head_dim) ? ld_half4(qh + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // ---- scores: a warp takes positions warp, warp + 16, ...; four positions in flight
  for (int t0 = warp; t0 < T; t0 += 4 * ATT_WARPS) {
    float d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = t0 + u * ATT_WARPS;
      d[u] = 0.0f;
      if (t < T) {
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const int j = ch * 128 + lane * 4;
          if (ch < nchunk && j < head_dim) {
            const float4 kv = ld_half4(kb + (int64_t)t * width + j);
            d[u] += qv[ch].x * kv.x + qv[ch].y * kv.y + qv[ch].z * kv.z + qv[ch].w * kv.w;
          }
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int u = 0; u < 4; ++u) d[u] += __shfl_xor_sync(0xffffffffu, d[u], off);
    }
    if (lane == 0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int t = t0 + u * ATT_WARPS;
        if (t < T) sc[t] = __half2float(__hmul(__float2half_rn(d[u]), hscale));
      }
    }
  }
  __syncthreads();
  // ---- softmax over sc[0..T)
  float mx = -INFINITY;
  for (int t = tid; t < T; t += ATT_THREADS) mx = fmaxf(mx, sc[t]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (lane == 0) s_warp[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = s_warp[0];
    for (int w = 1; w < ATT_WARPS; ++w) m = fmaxf(m, s_warp[w]);
    s_bcast = m;
  }
  __syncthreads();
  mx = s_bcast;
  float sum = 0.0f;
  for (int t = tid; t < T; t += ATT_THREADS) sum += expf(sc[t] - mx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  __syncthreads();  // s_bcast and s_warp have been read
  if (lane == 0) s_warp[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float s = 0.0f;
    for (int w = 0; w < ATT_WARPS; ++w) s += s_warp[w];
    s_bcast = s;
  }
  __syncthreads();
  sum = s_bcast;
  for (int t = tid; t < T; t += ATT_THREADS)
    sc[t] = __half2float(__float2half_rn(expf(sc[t] - mx) / sum));
  __syncthreads();
  // ---- probabilities . v: a warp takes positions warp, warp + 16, ...; a lane four columns
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int t0 = warp; t0 < T; t0 += 4 * ATT_WARPS) {
    float4 vv[4][2];
    float p[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = t0 + u * ATT_WARPS;
      p[u] = t < T ? sc[t] : 0.0f;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int j = ch * 128 + lane * 4;
        vv[u][ch] = (t < T && ch < nchunk && j < head_dim) ? ld_half4(vb + (int64_t)t * width + j)
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        acc[ch].x += p[u] * vv[u][ch].x;
        acc[ch].y += p[u] * vv[u][ch].y;
        acc[ch].z += p[u] * vv[u][ch].z;
        acc[ch].w += p[u] * vv[u][ch].w;
      }
    }
  }
#pragma unroll
  for (int ch = 0; ch < 2; ++ch) {
    const int j = ch * 128 + lane * 4;
    if (ch < nchunk && j < head_dim)
      *reinterpret_cast<float4*>(&red[warp * head_dim + j]) = acc[ch];
  }
  __syncthreads();
  __half* orow = out + (int64_t)b * s_o + (int64_t)h * head_dim;
  for (int j = tid; j < head_dim; j += ATT_THREADS) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) s += red[w * head_dim + j];
    orow[j] = __float2half_rn(s);
  }
}

// The same computation for head_dim 64, 128 or 256, built for bandwidth: 16-byte loads (a
// group of head_dim/8 lanes per position, so a warp reads 32/(head_dim/8) positions at a
// time, four such steps in flight), and a thread-block cluster of CS CTAs per (head,
// sequence) that splits the positions when there are few (head, sequence) pairs.  The CTAs
// of a cluster exchange their maxima, their sums of exponentials and their partial outputs
// through distributed shared memory; rank 0 adds the partial outputs in rank order, so the
// result does not depend on timing.  Rounding points as above.
constexpr int ATT2_THREADS = 256;
constexpr int ATT2_WARPS = ATT2_THREADS / 32;

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, unsigned rank) {
  uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(local)), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(h[i]);
    f[2 * i + 1] = __high2float(h[i]);
  }
}

template <int HD, int CS, bool PDL>
__global__ void __launch_bounds__(ATT2_THREADS, 3)
    decode_attention_wide_kernel(__half* out, const __half* q, const __half* k_cache,
                                 const __half* v_cache, int n_heads, int S, int chunk_cap, int s_q,
                                 int s_o, const int* pos_dev, float scale) {
  constexpr int LPT = HD / 8;    // lanes per position
  constexpr int TPW = 32 / LPT;  // positions per warp step
  constexpr int U = 8;           // steps in flight
  extern __shared__ float att_smem[];
  float* sc = att_smem;                // [chunk_cap] scores, then probabilities, of this CTA's positions
  float* red = att_smem + chunk_cap;   // [ATT2_WARPS][HD] partial outputs of the warps
  __shared__ float s_warp[ATT2_WARPS];
  __shared__ float s_stat[2];          // this CTA's maximum and sum of exponentials
  __shared__ float s_part[HD];         // this CTA's partial output
  pdl_enter<PDL>();
  const int h = blockIdx.x / CS, rank = blockIdx.x % CS, b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sg = lane / LPT, li = lane % LPT;
  const int width = n_heads * HD;
  int T = *pos_dev + 1;
  T = T < 0 ? 0 : (T > S ? S : T);
  // positions of this CTA: a contiguous chunk
  const int per = (T + CS - 1) / CS;
  const int t_lo = min(T, rank * per), t_hi = min(T, t_lo + per);
  const int nloc = t_hi - t_lo;
  const __half* kb = k_cache + (int64_t)b * S * width + (int64_t)h * HD + li * 8;
  const __half* vb = v_cache + (int64_t)b * S * width + (int64_t)h * HD + li * 8;
  const __half hscale = __float2half_rn(scale);
  float qf[8];
  unpack8(*reinterpret_cast<const uint4*>(q + (int64_t)b * s_q + (int64_t)h * HD + li * 8), qf);

  // ---- scores
  // (the loop bound is the same for all lanes of a warp: the shuffles inside need every lane)
  for (int ib = warp * TPW; ib < nloc; ib += U * ATT2_WARPS * TPW) {
    const int i0 = ib + sg;
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * ATT2_WARPS * TPW;
      kv[u] = i < nloc ? *reinterpret_cast<const uint4*>(kb + (int64_t)(t_lo + i) * width)
                       : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8];
      unpack8(kv[u], kf);
      float d = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) d += qf[j] * kf[j];
#pragma unroll
      for (int off = LPT / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
      const int i = i0 + u * ATT2_WARPS * TPW;
      if (li == 0 && i < nloc) sc[i] = __half2float(__hmul(__float2half_rn(d), hscale));
    }
  }
  __syncthreads();
  // ---- maximum over all positions
  float mx = -INFINITY;
  for (int i = tid; i < nloc; i += ATT2_THREADS) mx = fmaxf(mx, sc[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (lane == 0) s_warp[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = s_warp[0];
    for (int w = 1; w < ATT2_WARPS; ++w) m = fmaxf(m, s_warp[w]);
    s_stat[0] = m;
  }
  if (CS > 1) cluster_sync_all(); else __syncthreads();
  mx = s_stat[0];
  if (CS > 1) {
    mx = -INFINITY;
    for (int r = 0; r < CS; ++r) mx = fmaxf(mx, ld_cluster_f32(&s_stat[0], r));
  }
  // ---- sum of exponentials
  float sum = 0.0f;
  for (int i = tid; i < nloc; i += ATT2_THREADS) sum += expf(sc[i] - mx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane == 0) s_warp[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float t = 0.0f;
    for (int w = 0; w < ATT2_WARPS; ++w) t += s_warp[w];
    s_stat[1] = t;
  }
  if (CS > 1) cluster_sync_all(); else __syncthreads();
  sum = s_stat[1];
  if (CS > 1) {
    sum = 0.0f;
    for (int r = 0; r < CS; ++r) sum += ld_cluster_f32(&s_stat[1], r);
  }
  for (int i = tid; i < nloc; i += ATT2_THREADS)
    sc[i] = __half2float(__float2half_rn(expf(sc[i] - mx) / sum));
  __syncthreads();
  // ---- probabilities . v
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  for (int ib = warp * TPW; ib < nloc; ib += U * ATT2_WARPS * TPW) {
    const int i0 = ib + sg;
    uint4 vv[U];
    float pr[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * ATT2_WARPS * TPW;
      vv[u] = i < nloc ? *reinterpret_cast<const uint4*>(vb + (int64_t)(t_lo + i) * width)
                       : make_uint4(0, 0, 0, 0);
      pr[u] = i < nloc ? sc[i] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float vf[8];
      unpack8(vv[u], vf);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += pr[u] * vf[j];
    }
  }
  // the position groups of a warp, then the warps, then the CTAs of the cluster
#pragma unroll
  for (int off = LPT; off < 32; off <<= 1)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  if (sg == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) red[warp * HD + li * 8 + j] = acc[j];
  }
  __syncthreads();
  for (int j = tid; j < HD; j += ATT2_THREADS) {
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT2_WARPS; ++w) t += red[w * HD + j];
    s_part[j] = t;
  }
  if (CS > 1) cluster_sync_all(); else __syncthreads();
  if (rank == 0) {
    __half* orow = out + (int64_t)b * s_o + (int64_t)h * HD;
    for (int j = tid; j < HD; j += ATT2_THREADS) {
      float t = s_part[j];
      if (CS > 1)
        for (int r = 1; r < CS; ++r) t += ld_cluster_f32(&s_part[j], r);
      orow[j] = __float2half_rn(t);
    }
  }
  if (CS > 1) cluster_sync_all();  // peers stay resident until rank 0 has read their partial outputs
}

template <int HD, int CS>
int launch_attention_wide(adr_ctx* ctx, cudaStream_t stream, __half* out, const __half* q,
                          const __half* k_cache, const __half* v_cache, int batch, int n_heads,
                          int S, int s_q, int s_o, const int* pos_dev, float scale) {
  const int chunk_cap = ((S + CS - 1) / CS + 7) & ~7;
  const size_t smem = ((size_t)chunk_cap + (size_t)ATT2_WARPS * HD) * sizeof(float);
  if (smem > 48 * 1024) return ADR_ERR_SHAPE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_heads * CS, batch, 1);
  cfg.blockDim = dim3(ATT2_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (CS > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = CS;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (ctx->tune_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = ctx->tune_pdl
      ? cudaLaunchKernelEx(&cfg, decode_attention_wide_kernel<HD, CS, true>, out, q, k_cache, v_cache,
                           n_heads, S, chunk_cap, s_q, s_o, pos_dev, scale)
      : cudaLaunchKernelEx(&cfg, decode_attention_wide_kernel<HD, CS, false>, out, q, k_cache, v_cache,
                           n_heads, S, chunk_cap, s_q, s_o, pos_dev, scale);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  if ((long long)n_heads * CS * batch >= (ctx->sm_count > 0 ? ctx->sm_count : 148))
    note_filling_launch(ctx, stream, 4);  // (see launch_row)
  return after_launch(ctx);
}

template <int HD>
int launch_attention_wide_hd(adr_ctx* ctx, cudaStream_t stream, __half* out, const __half* q,
                             const __half* k_cache, const __half* v_cache, int batch, int n_heads,
                             int S, int s_q, int s_o, const int* pos_dev, float scale) {
  // enough CTAs to fill the machine: split the positions when (head, sequence) pairs are few
  const int pairs = batch * n_heads;
  const int cs = pairs >= 256 ? 1 : pairs >= 128 ? 2 : pairs >= 64 ? 4 : 8;
  switch (cs) {
    case 1: return launch_attention_wide<HD, 1>(ctx, stream, out, q, k_cache, v_cache, batch, n_heads, S, s_q, s_o, pos_dev, scale);
    case 2: return launch_attention_wide<HD, 2>(ctx, stream, out, q, k_cache, v_cache, batch, n_heads, S, s_q, s_o, pos_dev, scale);
    case 4: return launch_attention_wide<HD, 4>(ctx, stream, out, q, k_cache, v_cache, batch, n_heads, S, s_q, s_o, pos_dev, scale);
    default: return launch_attention_wide<HD, 8>(ctx, stream, out, q, k_cache, v_cache, batch, n_heads, S, s_q, s_o, pos_dev, scale);
  }
}

// ---------------------------------------------------------------------------------------
// launch helper: plain launch, or one with programmatic stream serialisation
// ---------------------------------------------------------------------------------------
template <typename... KArgs, typename... Args>
int launch_row(adr_ctx* ctx, cudaStream_t stream, void (*plain)(KArgs...), void (*pdl)(KArgs...),
               dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->tune_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, ctx->tune_pdl ? pdl : plain, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  // a row kernel with at least one CTA per SM (decode attention over many heads) fills the GPU
  // like a large product does: the decode kernel's half-SM form must not start as it drains
  if ((long long)grid.x * grid.y * grid.z >= (ctx->sm_count > 0 ? ctx->sm_count : 148))
    note_filling_launch(ctx, stream, 4);
  else
    ctx->small_before = 1;
  return after_launch(ctx);
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

}  // namespace adr

using namespace adr;

extern "C" {

int adr_rms_norm(adr_ctx* ctx, adr_stream stream, void* out, const void* in, const void* weights,
                 int length_x, int length_y, int stride_ox, int stride_oy, int stride_ix,
                 int stride_iy, float eps) {
  if (!ctx || !out || !in || !weights) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (length_x <= 0 || length_y <= 0) return ADR_ERR_INVALID;
  if (stride_ox < 0 || stride_oy < 0 || stride_ix < 0 || stride_iy < 0) return ADR_ERR_INVALID;
  constexpr int RMS_ROWS = 2;
  if (stride_ox == 1 && stride_ix == 1 && length_x <= 16 * ROW_THREADS && length_y >= 1024)
    return launch_row(ctx, (cudaStream_t)stream, rms_norm_rows_kernel<false, RMS_ROWS>,
                      rms_norm_rows_kernel<true, RMS_ROWS>, dim3((length_y + RMS_ROWS - 1) / RMS_ROWS),
                      dim3(ROW_THREADS), 0, (__half*)out, (const __half*)in, (const __half*)weights,
                      length_x, length_y, stride_oy, stride_iy, eps);
  return launch_row(ctx, (cudaStream_t)stream, rms_norm_kernel<false>, rms_norm_kernel<true>,
                    dim3(length_y), dim3(ROW_THREADS), 0, (__half*)out, (const __half*)in,
                    (const __half*)weights, length_x, stride_ox, stride_oy, stride_ix, stride_iy, eps);
}

int adr_layer_norm(adr_ctx* ctx, adr_stream stream, void* out, const void* in, const void* weights,
                   const void* bias, int length_x, int length_y, int stride_ox, int stride_oy,
                   int stride_ix, int stride_iy, float eps) {
  if (!ctx || !out || !in || !weights || !bias) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (length_x <= 0 || length_y <= 0) return ADR_ERR_INVALID;
  if (stride_ox < 0 || stride_oy < 0 || stride_ix < 0 || stride_iy < 0) return ADR_ERR_INVALID;
  constexpr int LN_ROWS = 4;
  if (stride_ox == 1 && stride_ix == 1 && length_x <= 4 * ROW_THREADS && length_y >= 1024)
    return launch_row(ctx, (cudaStream_t)stream, layer_norm_rows_kernel<false, LN_ROWS>,
                      layer_norm_rows_kernel<true, LN_ROWS>, dim3((length_y + LN_ROWS - 1) / LN_ROWS),
                      dim3(ROW_THREADS), 0, (__half*)out, (const __half*)in, (const __half*)weights,
                      (const __half*)bias, length_x, length_y, stride_oy, stride_iy, eps);
  return launch_row(ctx, (cudaStream_t)stream, layer_norm_kernel<false>, layer_norm_kernel<true>,
                    dim3(length_y), dim3(ROW_THREADS), 0, (__half*)out, (const __half*)in,
                    (const __half*)weights, (const __half*)bias, length_x, stride_ox, stride_oy,
                    stride_ix, stride_iy, eps);
}

int adr_softmax_rows(adr_ctx* ctx, adr_stream stream, void* out, const void* in, int heads, int h,
                     int w, int pitch, float temperature) {
  if (!ctx || !out || !in) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (heads <= 0 || h <= 0 || w <= 0 || pitch < w) return ADR_ERR_INVALID;
  if (heads > 65535) return ADR_ERR_SHAPE;
  if (!(temperature > 0.0f)) return ADR_ERR_INVALID;
  return launch_row(ctx, (cudaStream_t)stream, softmax_rows_kernel<false>, softmax_rows_kernel<true>,
                    dim3(h, heads), dim3(ROW_THREADS), 0, (__half*)out, (const __half*)in, h, w,
                    pitch, temperature);
}

int adr_rotary(adr_ctx* ctx, adr_stream stream, void* out, const void* in, int length_x,
               int length_y, int stride_ox, int stride_oy, int stride_ix, int stride_iy, int n_heads,
               int pos_offset, float theta) {
  if (!ctx || !out || !in) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (length_x <= 0 || length_y <= 0 || n_heads <= 0) return ADR_ERR_INVALID;
  if (length_x % n_heads != 0 || (length_x / n_heads) % 2 != 0) return ADR_ERR_SHAPE;
  if (stride_ox < 0 || stride_oy < 0 || stride_ix < 0 || stride_iy < 0) return ADR_ERR_INVALID;
  const int head_dim = length_x / n_heads;
  if (stride_ox == 1 && stride_ix == 1 && n_heads >= 4 && length_y <= 65535 && stride_oy % 2 == 0 &&
      stride_iy % 2 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 3u) == 0) {
    const dim3 hblock(64, 4);
    const dim3 hgrid((head_dim / 2 + 63) / 64, length_y);
    return launch_row(ctx, (cudaStream_t)stream, rope_rows_heads_kernel<false>, rope_rows_heads_kernel<true>,
                      hgrid, hblock, 0, (__half*)out, (const __half*)in, head_dim, length_y, stride_oy,
                      stride_iy, n_heads, pos_offset, theta);
  }
  const dim3 block(64, 4);
  const dim3 grid((length_x / 2 + 63) / 64, (length_y + 3) / 4);
  if (grid.y > 65535) return ADR_ERR_SHAPE;
  return launch_row(ctx, (cudaStream_t)stream, rope_rows_kernel<false>, rope_rows_kernel<true>, grid,
                    block, 0, (__half*)out, (const __half*)in, length_x, length_y, stride_ox,
                    stride_oy, stride_ix, stride_iy, n_heads, pos_offset, theta);
}

int adr_elementwise_binary_2d_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* left,
                                  const void* right, int rows, int cols, int stride_o, int stride_l,
                                  int stride_r, uint32_t op) {
  if (!ctx || !out || !left || !right) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (rows <= 0 || cols <= 0) return ADR_ERR_INVALID;
  if (op != ADR_BINARY_ADD && op != ADR_BINARY_SILU_MUL) return ADR_ERR_UNSUPPORTED;
  if (stride_o < cols || stride_l < cols || stride_r < cols) return ADR_ERR_INVALID;
  if (rows > 65535) return ADR_ERR_SHAPE;
  const int per_block = 256 * 8;
  const dim3 grid(std::min((cols + per_block - 1) / per_block, 1024), rows);
  return launch_row(ctx, (cudaStream_t)stream, binary_2d_kernel<false>, binary_2d_kernel<true>,
                    grid, dim3(256), 0, (__half*)out, (const __half*)left, (const __half*)right,
                    rows, cols, stride_o, stride_l, stride_r, (int)op);
}

int adr_decode_rope_append(adr_ctx* ctx, adr_stream stream, void* q, const void* k, const void* v,
                           void* k_cache, void* v_cache, int batch, int n_heads, int head_dim,
                           int max_seq, int stride_q, int stride_k, int stride_v,
                           const int32_t* pos_dev, float theta) {
  if (!ctx || !q || !k || !v || !k_cache || !v_cache || !pos_dev) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (batch <= 0 || n_heads <= 0 || head_dim <= 0 || max_seq <= 0) return ADR_ERR_INVALID;
  if (head_dim % 2 != 0 || batch > 65535) return ADR_ERR_SHAPE;
  const int width = n_heads * head_dim;
  if (stride_q < width || stride_k < width || stride_v < width) return ADR_ERR_INVALID;
  if (stride_v % 2 != 0 || (reinterpret_cast<uintptr_t>(v) & 3u) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 3u))
    return ADR_ERR_SHAPE;
  return launch_row(ctx, (cudaStream_t)stream, decode_rope_append_kernel<false>,
                    decode_rope_append_kernel<true>, dim3((width / 2 + 255) / 256, batch), dim3(256),
                    0, (__half*)q, (const __half*)k, (const __half*)v, (__half*)k_cache,
                    (__half*)v_cache, width, n_heads, max_seq, stride_q, stride_k, stride_v,
                    (const int*)pos_dev, theta);
}

int adr_decode_attention(adr_ctx* ctx, adr_stream stream, void* out, const void* q,
                         const void* k_cache, const void* v_cache, int batch, int n_heads,
                         int head_dim, int max_seq, int stride_q, int stride_o,
                         const int32_t* pos_dev, float scale) {
  if (!ctx || !out || !q || !k_cache || !v_cache || !pos_dev) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (batch <= 0 || n_heads <= 0 || head_dim <= 0 || max_seq <= 0) return ADR_ERR_INVALID;
  if (head_dim % 8 != 0 || head_dim > ATT_MAX_HD || max_seq % 8 != 0 || batch > 65535)
    return ADR_ERR_SHAPE;
  if (stride_q % 4 != 0 || !al16(q) || !al16(k_cache) || !al16(v_cache)) return ADR_ERR_SHAPE;
  if (stride_q % 8 == 0 && n_heads * head_dim % 8 == 0 && n_heads <= 8191) {
    // the bandwidth-oriented form for the usual head sizes; its own limit on max_seq falls
    // through to the general kernel
    int rc = ADR_ERR_SHAPE;
    if (head_dim == 64)
      rc = launch_attention_wide_hd<64>(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, batch, n_heads, max_seq, stride_q, stride_o, (const int*)pos_dev, scale);
    else if (head_dim == 128)
      rc = launch_attention_wide_hd<128>(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, batch, n_heads, max_seq, stride_q, stride_o, (const int*)pos_dev, scale);
    else if (head_dim == 256)
      rc = launch_attention_wide_hd<256>(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, batch, n_heads, max_seq, stride_q, stride_o, (const int*)pos_dev, scale);
    if (rc != ADR_ERR_SHAPE) return rc;
  }
  const size_t smem = ((size_t)max_seq + (size_t)ATT_WARPS * head_dim) * sizeof(float);
  if (smem > 48 * 1024) return ADR_ERR_SHAPE;
  return launch_row(ctx, (cudaStream_t)stream, decode_attention_kernel<false>,
                    decode_attention_kernel<true>, dim3(n_heads, batch), dim3(ATT_THREADS), smem,
                    (__half*)out, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache,
                    n_heads, head_dim, max_seq, stride_q, stride_o, (const int*)pos_dev, scale);
}

}  // extern "C"
