// absmax-u8 quantiser and dequantiser, replacing
// adrastea_kernels/cpp/quantize.cu:3-56 (quantize_absmax_uint8,
// dequantize_absmax_uint8) for contiguous [rows, k] operands.
#include "u8_common.cuh"

namespace adr {

namespace {

// One thread per 16 weights; the same dequant4 the matmul kernels use, so a
// bit-exact check of this kernel's output checks their weight path too.
template <bool HAS_ZERO>
__global__ void __launch_bounds__(256) dequantize_u8_kernel(__half* out, const __half* scales,
                                                            const __half* zeros, const uint8_t* q,
                                                            int rows, int k, int block_size) {
  const int per_row = k / 16;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * per_row) return;
  const int r = (int)(idx / per_row);
  const int kk = (int)(idx % per_row) * 16;
  const int groups = k / block_size;
  const int g = kk / block_size;
  ScalePair sp = make_scale(scales[(size_t)r * groups + g], HAS_ZERO,
                            HAS_ZERO ? zeros[(size_t)r * groups + g] : __half());
  uint4 w = ldg_nc_16(q + (size_t)r * k + kk);
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 lo, hi;
    dequant4(ww[j], sp, lo, hi);
    o[2 * j] = half2_as_u32(lo);
    o[2 * j + 1] = half2_as_u32(hi);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * k + kk);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// embed_uint8 (adrastea_kernels/cpp/embed_uint8.cu:3-19): out[t, :] = the dequantised row
// in_ids[t] of the table (implicit zero point 127.5).  One thread per 16 values, as above.
__global__ void __launch_bounds__(256) embed_u8_kernel(int n_dim, int n_ids, const short* in_ids,
                                                       __half* out, const uint8_t* table,
                                                       const __half* scales, int block_size) {
  const int per_row = n_dim / 16;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)n_ids * per_row) return;
  const int t = (int)(idx / per_row);
  const int kk = (int)(idx % per_row) * 16;
  const int groups = n_dim / block_size;
  const int64_t id = in_ids[t];
  ScalePair sp = make_scale(scales[id * groups + kk / block_size], false, __half());
  uint4 w = ldg_nc_16(table + id * n_dim + kk);
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 lo, hi;
    dequant4(ww[j], sp, lo, hi);
    o[2 * j] = half2_as_u32(lo);
    o[2 * j + 1] = half2_as_u32(hi);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * n_dim + kk);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// One warp per (row, group): absmax by shuffles, then the scale in fp16 and
// the codes  u8(round(127.5 + x / float(scale)))  (quantize.cu:33, 42).
__global__ void __launch_bounds__(256) quantize_u8_kernel(uint8_t* q, __half* scales,
                                                          const __half* in, int rows, int k,
                                                          int block_size) {
  const int groups = k / block_size;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)rows * groups) return;
  const int r = (int)(wid / groups), g = (int)(wid % groups);
  const __half* src = in + (size_t)r * k + (size_t)g * block_size;
  float absmax = 0.0f;
  for (int i = lane; i < block_size; i += 32) absmax = fmaxf(absmax, fabsf(__half2float(src[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
  const __half s = __float2half_rn(absmax / 127.5f);
  if (lane == 0) scales[(size_t)r * groups + g] = s;
  const float sf = __half2float(s);
  uint8_t* dst = q + (size_t)r * k + (size_t)g * block_size;
  for (int i = lane; i < block_size; i += 32)
    dst[i] = static_cast<uint8_t>(roundf(127.5f + __half2float(src[i]) / sf));
}

}  // namespace

int launch_dequantize_u8(adr_ctx* ctx, cudaStream_t stream, __half* out, const __half* scales,
                         const __half* zeros, const uint8_t* q, int rows, int k, int block_size) {
  int64_t threads = (int64_t)rows * (k / 16);
  int64_t grid = (threads + 255) / 256;
  if (grid > 0x7fffffffLL) return ADR_ERR_SHAPE;
  if (zeros)
    dequantize_u8_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(out, scales, zeros, q, rows, k, block_size);
  else
    dequantize_u8_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(out, scales, zeros, q, rows, k, block_size);
  return after_launch(ctx);
}

int launch_quantize_u8(adr_ctx* ctx, cudaStream_t stream, uint8_t* q, __half* scales,
                       const __half* in, int rows, int k, int block_size) {
  int64_t warps = (int64_t)rows * (k / block_size);
  int64_t grid = (warps * 32 + 255) / 256;
  if (grid > 0x7fffffffLL) return ADR_ERR_SHAPE;
  quantize_u8_kernel<<<(unsigned)grid, 256, 0, stream>>>(q, scales, in, rows, k, block_size);
  return after_launch(ctx);
}

int launch_embed_u8(adr_ctx* ctx, cudaStream_t stream, int n_dim, int n_ids, const short* in_ids,
                    __half* out, const uint8_t* table, const __half* scales, int block_size) {
  int64_t threads = (int64_t)n_ids * (n_dim / 16);
  int64_t grid = (threads + 255) / 256;
  if (grid > 0x7fffffffLL) return ADR_ERR_SHAPE;
  embed_u8_kernel<<<(unsigned)grid, 256, 0, stream>>>(n_dim, n_ids, in_ids, out, table, scales, block_size);
  return after_launch(ctx);
}

}  // namespace adr
