// C ABI of adrastea_b200: argument checks, kernel selection, tracing.
// The host-side logic mirrors GpuKernels::matmul_f16 of the reference
// (adrastea_models/src/kernels.rs:821-890), which validates shapes, lowers
// the options and launches; here the lowering has already happened on the
// caller's side and the 22 kernel parameters arrive as they are.
#include <cstdio>
#include <cstring>
#include <new>

#include "tma.cuh"

namespace adr {

bool TraceKey::operator==(const TraceKey& o) const {
  return m == o.m && k == o.k && n == o.n && batches == o.batches &&
         memcmp(strides, o.strides, sizeof(strides)) == 0 && store == o.store && load == o.load &&
         mask == o.mask && kernel == o.kernel;
}

namespace {

void trace_record(adr_ctx* ctx, const MatmulArgs& a, int kernel) {
  if (!ctx->trace_on) return;
  TraceKey key{a.m, a.k, a.n, a.batches,
               {a.s_ox, a.s_oy, a.s_oz, a.s_lx, a.s_ly, a.s_lz, a.s_rx, a.s_ry, a.s_rz},
               a.store, a.load, a.mask, kernel};
  std::lock_guard<std::mutex> lock(ctx->mu);
  for (const auto& t : ctx->trace)
    if (t == key) return;
  ctx->trace.push_back(key);
}

int check_matmul_args(const adr_ctx* ctx, const MatmulArgs& a) {
  if (!ctx || !a.out || !a.lhs || !a.rhs) return ADR_ERR_INVALID;
  if (a.batches <= 0 || a.m <= 0 || a.k <= 0 || a.n <= 0) return ADR_ERR_INVALID;
  if (a.store == ADR_STORE_GELU_BIAS) return ADR_ERR_UNSUPPORTED;
  if (a.store > ADR_STORE_QUICK_GELU_BIAS || a.load > ADR_LOAD_SCALE || a.mask > ADR_MASK_CAUSAL)
    return ADR_ERR_INVALID;
  if (store_uses_bias((int)a.store) && !a.bias) return ADR_ERR_INVALID;
  if (a.s_ox < 0 || a.s_oy < 0 || a.s_oz < 0 || a.s_lx < 0 || a.s_ly < 0 || a.s_lz < 0 ||
      a.s_rx < 0 || a.s_ry < 0 || a.s_rz < 0)
    return ADR_ERR_INVALID;
  return ADR_OK;
}

int run_matmul(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a, bool slow,
               bool checked = false) {
  int rc = checked ? ADR_OK : check_matmul_args(ctx, a);
  if (rc != ADR_OK) return rc;
  DeviceGuard guard(ctx);
  int kernel = ctx->forced_kernel;
  if (slow) kernel = ADR_KERNEL_F16_SIMT;
  if (kernel == ADR_KERNEL_AUTO)
    kernel = gemm_f16_tc_supports(ctx, a) ? ADR_KERNEL_F16_TC : ADR_KERNEL_F16_TC_GATHER;
  if (kernel == ADR_KERNEL_F16_TC) {
    if (!gemm_f16_tc_supports(ctx, a)) return ADR_ERR_SHAPE;
    rc = launch_gemm_f16_tc(ctx, stream, a);
    if (rc == ADR_ERR_SHAPE && ctx->forced_kernel == ADR_KERNEL_AUTO) {
      // the view passed the static checks but the tensor map could not be encoded
      kernel = ADR_KERNEL_F16_TC_GATHER;
      rc = launch_gemm_f16_gather(ctx, stream, a);
    }
  } else if (kernel == ADR_KERNEL_F16_TC_GATHER) {
    rc = launch_gemm_f16_gather(ctx, stream, a);
  } else if (kernel == ADR_KERNEL_F16_SIMT) {
    rc = launch_gemm_f16_simt(ctx, stream, a);
  } else {
    return ADR_ERR_INVALID;
  }
  if (rc == ADR_OK) {
    ctx->last_kernel = kernel;
    trace_record(ctx, a, kernel);
  }
  return rc;
}

constexpr size_t kStatusBytes = 64;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace adr

using namespace adr;

extern "C" {

int adr_init(int device, adr_ctx** out_ctx) {
  if (!out_ctx) return ADR_ERR_INVALID;
  *out_ctx = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    return ADR_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return ADR_ERR_CUDA;
  if (prop.major != 10) return ADR_ERR_UNSUPPORTED;  // sm_100a code only
  adr_ctx* ctx = new (std::nothrow) adr_ctx();
  if (!ctx) return ADR_ERR_INVALID;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  int rc = ADR_OK;
  if (cudaMalloc(&ctx->d_status, kStatusBytes) != cudaSuccess ||
      cudaMemset(ctx->d_status, 0, kStatusBytes) != cudaSuccess) {
    rc = ADR_ERR_CUDA;
  }
  if (rc == ADR_OK) rc = tma_init(ctx);
  if (rc == ADR_OK) rc = init_gemm_f16_tc(ctx);
  if (rc == ADR_OK) rc = init_u8_kernels(ctx);
  cudaSetDevice(prev);
  if (rc != ADR_OK) {
    adr_destroy(ctx);
    return rc;
  }
  *out_ctx = ctx;
  return ADR_OK;
}

void adr_destroy(adr_ctx* ctx) {
  if (!ctx) return;
  DeviceGuard guard(ctx);
  destroy_gemm_f16_tc(ctx);
  tma_destroy(ctx);
  if (ctx->d_status) cudaFree(ctx->d_status);
  delete ctx;
}

const char* adr_strerror(int code) {
  switch (code) {
    case ADR_OK: return "ok";
    case ADR_ERR_INVALID: return "invalid argument";
    case ADR_ERR_SHAPE: return "shape, divisibility or alignment rule violated";
    case ADR_ERR_UNSUPPORTED: return "unsupported operation or device";
    case ADR_ERR_CUDA: return "CUDA call failed";
    case ADR_ERR_DEVICE: return "a kernel's bounded wait ran out";
    case ADR_ERR_NCCL: return "NCCL call failed";
    case ADR_ERR_TOO_LARGE: return "operands exceed the entry point's built-in scratch buffer";
    default: return "unknown error";
  }
}

int adr_last_cuda_error(const adr_ctx* ctx) { return ctx ? ctx->last_cuda_error.load() : 0; }

int adr_force_kernel(adr_ctx* ctx, int kernel) {
  if (!ctx || kernel < ADR_KERNEL_AUTO || kernel > ADR_KERNEL_U8_KSPLIT) return ADR_ERR_INVALID;
  ctx->forced_kernel = kernel;
  return ADR_OK;
}

int adr_set_tunable(adr_ctx* ctx, const char* name, int value) {
  if (!ctx || !name || value < 0) return ADR_ERR_INVALID;
  if (!strcmp(name, "u8_split")) ctx->tune_u8_split = value;
  else if (!strcmp(name, "u8_rows")) ctx->tune_u8_rows = value;
  else if (!strcmp(name, "tc_bn")) ctx->tune_tc_bn = value;
  else if (!strcmp(name, "tc_split")) ctx->tune_tc_split = value;
  else if (!strcmp(name, "pdl")) ctx->tune_pdl = value;
  else if (!strcmp(name, "u8_exact")) ctx->tune_u8_exact = value;
  else if (!strcmp(name, "wait_ms")) ctx->tune_wait_ms = value;
  else if (!strcmp(name, "pdl_guard")) ctx->tune_pdl_guard = value;
  else if (!strcmp(name, "ks_clusters")) ctx->tune_ks_clusters = value;
  else if (!strcmp(name, "ks_stages")) ctx->tune_ks_stages = value;
  else if (!strcmp(name, "ks_off")) ctx->tune_ks_off = value;
  else if (!strcmp(name, "ks_pdl")) ctx->tune_ks_pdl = value;
  else if (!strcmp(name, "ks_slack")) ctx->tune_ks_slack = value;
  else if (!strcmp(name, "u8_cps_m")) ctx->tune_u8_cps_m = value;
  else if (!strcmp(name, "u8_cps_x4")) ctx->tune_u8_cps_x4 = value;
  else if (!strcmp(name, "ts_bt")) ctx->tune_ts_bt = value;
  else if (!strcmp(name, "ts_split")) ctx->tune_ts_split = value;
  else return ADR_ERR_INVALID;
  return ADR_OK;
}

int adr_device_status(adr_ctx* ctx) {
  if (!ctx) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  unsigned int flag = 0;
  ADR_CUDA_CHECK(ctx, cudaDeviceSynchronize());
  ADR_CUDA_CHECK(ctx, cudaMemcpy(&flag, ctx->d_status, sizeof(flag), cudaMemcpyDeviceToHost));
  if (flag) {
    ADR_CUDA_CHECK(ctx, cudaMemset(ctx->d_status, 0, sizeof(flag)));
    return ADR_ERR_DEVICE;
  }
  return ADR_OK;
}

int adr_last_kernel(const adr_ctx* ctx) { return ctx ? ctx->last_kernel.load() : 0; }
uint64_t adr_launch_count(const adr_ctx* ctx) { return ctx ? ctx->launches.load() : 0; }

int adr_matmul_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs, const void* rhs,
                   int batches, int m, int k, int n, int stride_ox, int stride_oy, int stride_oz,
                   int stride_lx, int stride_ly, int stride_lz, int stride_rx, int stride_ry,
                   int stride_rz, const void* bias, float beta, float scale, uint32_t store_op,
                   uint32_t load_op, uint32_t mask_op) {
  MatmulArgs a{(__half*)out, (const __half*)lhs, (const __half*)rhs, batches, m, k, n,
               stride_ox, stride_oy, stride_oz, stride_lx, stride_ly, stride_lz,
               stride_rx, stride_ry, stride_rz, (const __half*)bias, beta, scale,
               store_op, load_op, mask_op};
  return run_matmul(ctx, (cudaStream_t)stream, a, false);
}

int adr_matmul_f16_b2(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs, const void* rhs,
                      int batches_outer, int batches, int m, int k, int n, int stride_ox,
                      int stride_oy, int stride_oz, int stride_ow, int stride_lx, int stride_ly,
                      int stride_lz, int stride_lw, int stride_rx, int stride_ry, int stride_rz,
                      int stride_rw, const void* bias, float beta, float scale, uint32_t store_op,
                      uint32_t load_op, uint32_t mask_op) {
  if (batches_outer <= 0 || batches <= 0) return ADR_ERR_INVALID;
  if (stride_ow < 0 || stride_lw < 0 || stride_rw < 0) return ADR_ERR_INVALID;
  // The two batch dimensions of an operand fold into one when its outer stride is `batches`
  // inner strides (or both are 0: broadcast); if that holds for all three, one launch does it.
  auto folds = [&](int sz, int sw) { return (long long)sw == (long long)sz * batches; };
  const long long total = (long long)batches_outer * batches;
  if (batches_outer == 1 ||
      (total <= 0x7fffffff && folds(stride_oz, stride_ow) && folds(stride_lz, stride_lw) &&
       folds(stride_rz, stride_rw)))
    return adr_matmul_f16(ctx, stream, out, lhs, rhs, (int)total, m, k, n, stride_ox, stride_oy,
                          stride_oz, stride_lx, stride_ly, stride_lz, stride_rx, stride_ry,
                          stride_rz, bias, beta, scale, store_op, load_op, mask_op);
  if (!out || !lhs || !rhs) return ADR_ERR_INVALID;
  // otherwise one launch per outer index, each over the inner batch
  for (int w = 0; w < batches_outer; ++w) {
    const int rc = adr_matmul_f16(
        ctx, stream, static_cast<__half*>(out) + (size_t)w * stride_ow,
        static_cast<const __half*>(lhs) + (size_t)w * stride_lw,
        static_cast<const __half*>(rhs) + (size_t)w * stride_rw, batches, m, k, n, stride_ox,
        stride_oy, stride_oz, stride_lx, stride_ly, stride_lz, stride_rx, stride_ry, stride_rz, bias,
        beta, scale, store_op, load_op, mask_op);
    if (rc != ADR_OK) return rc;
  }
  return ADR_OK;
}

int adr_matmul_f16_slow(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                        const void* rhs, int batches, int m, int k, int n, int stride_ox,
                        int stride_oy, int stride_oz, int stride_lx, int stride_ly, int stride_lz,
                        int stride_rx, int stride_ry, int stride_rz, const void* bias, float beta,
                        float scale, uint32_t store_op, uint32_t load_op, uint32_t mask_op) {
  MatmulArgs a{(__half*)out, (const __half*)lhs, (const __half*)rhs, batches, m, k, n,
               stride_ox, stride_oy, stride_oz, stride_lx, stride_ly, stride_lz,
               stride_rx, stride_ry, stride_rz, (const __half*)bias, beta, scale,
               store_op, load_op, mask_op};
  return run_matmul(ctx, (cudaStream_t)stream, a, true);
}

int adr_matmul_f16_raw(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                       const void* rhs, int batches, int m, int k, int n, int stride_ox,
                       int stride_oy, int stride_oz, int stride_lx, int stride_ly, int stride_lz,
                       int stride_rx, int stride_ry, int stride_rz) {
  return adr_matmul_f16(ctx, stream, out, lhs, rhs, batches, m, k, n, stride_ox, stride_oy,
                        stride_oz, stride_lx, stride_ly, stride_lz, stride_rx, stride_ry,
                        stride_rz, nullptr, 0.0f, 1.0f, ADR_STORE_IDENTITY, ADR_LOAD_IDENTITY,
                        ADR_MASK_NONE);
}

int adr_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                         const uint8_t* rhs, const void* scales, const void* zeros, int m, int p,
                         int n, int block_size, float beta) {
  if (!ctx || !out || !lhs || !rhs || !scales) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (m <= 0 || p <= 0 || n <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (p % block_size != 0 || block_size % 16 != 0 || p % 16 != 0) return ADR_ERR_SHAPE;
  if (!aligned16(lhs) || !aligned16(rhs)) return ADR_ERR_SHAPE;
  U8Args a{(__half*)out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, n, block_size, beta};
  cudaStream_t st = (cudaStream_t)stream;
  U8Args a16 = a;  // the streaming kernel takes 16 tokens per pass
  if (a16.m > 16) a16.m = 16;
  int kernel = ctx->forced_kernel;
  if (kernel == ADR_KERNEL_AUTO) {
    // up to 32 tokens two passes of the streaming kernel beat one tensor-core launch
    if (m > 32 && u8_ts_supports(ctx, a)) kernel = ADR_KERNEL_U8_TS;
    else if (m > 32 && u8_tc_supports(ctx, a)) kernel = ADR_KERNEL_U8_TC;
    else if (p % 64 != 0) kernel = m <= 4 ? ADR_KERNEL_U8_GEMV : ADR_KERNEL_U8_SIMT;
    else if (!ctx->tune_u8_exact && !ctx->tune_u8_split && !ctx->tune_u8_rows && !ctx->tune_ks_off &&
             (p <= 8192 ? (a16.m >= 5 || (a16.m >= 4 && p == 8192))
                        : (a16.m >= 7 || (a16.m >= 4 && p >= 16384))) &&
             u8_ksplit_supports(ctx, a16))
      kernel = ADR_KERNEL_U8_KSPLIT;  // measured: from these token counts on the cluster split wins
    else if (!ctx->tune_u8_exact && !ctx->tune_u8_split && !ctx->tune_u8_rows &&
             u8_ring_supports(ctx, a16))
      kernel = ADR_KERNEL_U8_RING;
    else if (u8_stream_supports(ctx, a16)) kernel = ADR_KERNEL_U8_STREAM;
    else kernel = ADR_KERNEL_U8_MMA;
  }
  int rc;
  switch (kernel) {
    case ADR_KERNEL_U8_GEMV: rc = launch_u8_gemv(ctx, st, a); break;
    case ADR_KERNEL_U8_SIMT: rc = launch_u8_simt(ctx, st, a); break;
    case ADR_KERNEL_U8_STREAM: {
      rc = ADR_OK;
      for (int r0 = 0; r0 < m && rc == ADR_OK; r0 += 16) {  // one pass per 16 tokens
        U8Args c = a;
        c.m = (m - r0 < 16) ? m - r0 : 16;
        c.lhs = a.lhs + (size_t)r0 * p;
        c.out = a.out + (size_t)r0 * n;
        rc = launch_u8_stream(ctx, st, c);
      }
      break;
    }
    case ADR_KERNEL_U8_RING: {
      rc = ADR_OK;
      for (int r0 = 0; r0 < m && rc == ADR_OK; r0 += 16) {  // one pass per 16 tokens
        U8Args c = a;
        c.m = (m - r0 < 16) ? m - r0 : 16;
        c.lhs = a.lhs + (size_t)r0 * p;
        c.out = a.out + (size_t)r0 * n;
        rc = launch_u8_ring(ctx, st, c);
      }
      break;
    }
    case ADR_KERNEL_U8_KSPLIT: {
      rc = ADR_OK;
      for (int r0 = 0; r0 < m && rc == ADR_OK; r0 += 16) {  // one pass per 16 tokens
        U8Args c = a;
        c.m = (m - r0 < 16) ? m - r0 : 16;
        c.lhs = a.lhs + (size_t)r0 * p;
        c.out = a.out + (size_t)r0 * n;
        rc = launch_u8_ksplit(ctx, st, c);
      }
      break;
    }
    case ADR_KERNEL_U8_TC: rc = launch_u8_tc(ctx, st, a); break;
    case ADR_KERNEL_U8_TS: rc = launch_u8_ts(ctx, st, a); break;
    case ADR_KERNEL_U8_MMA: {
      if (p % 64 != 0) return ADR_ERR_SHAPE;
      rc = ADR_OK;
      // m > 16: one pass over the weights per 16 tokens.
      for (int r0 = 0; r0 < m && rc == ADR_OK; r0 += 16) {
        U8Args c = a;
        c.m = (m - r0 < 16) ? m - r0 : 16;
        c.lhs = a.lhs + (size_t)r0 * p;
        c.out = a.out + (size_t)r0 * n;
        rc = launch_u8_mma(ctx, st, c);
      }
      break;
    }
    default: return ADR_ERR_INVALID;
  }
  if (rc == ADR_OK) ctx->last_kernel = kernel;
  return rc;
}

int adr_matmul_nt_fp16u8_grouped(adr_ctx* ctx, adr_stream stream, int count, void* const* outs,
                                 const void* lhs, const uint8_t* const* rhss,
                                 const void* const* scaless, const void* const* zeross, int m,
                                 int p, const int* ns, int block_size, float beta) {
  if (!ctx || !outs || !lhs || !rhss || !scaless || !ns || count < 1) return ADR_ERR_INVALID;
  for (int i = 0; i < count; ++i)
    if (!outs[i] || !rhss[i] || !scaless[i] || ns[i] <= 0) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  cudaStream_t st = (cudaStream_t)stream;
  // Up to four matrices per launch of the persistent decode kernel when it takes them (m <= 16,
  // activations resident); otherwise, and for what is left, one call per matrix.
  int i = 0;
  if (ctx->forced_kernel == ADR_KERNEL_AUTO || ctx->forced_kernel == ADR_KERNEL_U8_RING) {
    while (count - i >= 2 && m <= 16) {
      RingGroup g = {};
      g.count = count - i < 4 ? count - i : 4;
      for (int j = 0; j < g.count; ++j) {
        g.rhs[j] = rhss[i + j];
        g.scales[j] = (const __half*)scaless[i + j];
        g.zeros[j] = zeross ? (const __half*)zeross[i + j] : nullptr;
        g.out[j] = (__half*)outs[i + j];
        g.n[j] = ns[i + j];
      }
      U8Args common{nullptr, (const __half*)lhs, nullptr, nullptr, nullptr, m, p, 0, block_size, beta};
      const int rc = launch_u8_ring_grouped(ctx, st, common, g);
      if (rc == ADR_ERR_SHAPE) break;  // not a shape for the grouped form: separate calls below
      if (rc != ADR_OK) return rc;
      ctx->last_kernel = ADR_KERNEL_U8_RING;
      i += g.count;
    }
  }
  for (; i < count; ++i) {
    const int rc = adr_matmul_nt_fp16u8(ctx, stream, outs[i], lhs, rhss[i], scaless[i],
                                        zeross ? zeross[i] : nullptr, m, p, ns[i], block_size, beta);
    if (rc != ADR_OK) return rc;
  }
  return ADR_OK;
}

int adr_silu_mul_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                  const uint8_t* rhs_gate, const void* scales_gate,
                                  const void* zeros_gate, const uint8_t* rhs_up,
                                  const void* scales_up, const void* zeros_up, int m, int p, int n,
                                  int block_size) {
  if (!ctx || !out || !lhs || !rhs_gate || !scales_gate || !rhs_up || !scales_up) return ADR_ERR_INVALID;
  if (m <= 0 || p <= 0 || n <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if ((zeros_gate != nullptr) != (zeros_up != nullptr)) return ADR_ERR_INVALID;
  if (m > 16) return ADR_ERR_SHAPE;
  DeviceGuard guard(ctx);
  RingGroup g = {};
  g.count = 2;
  g.pair = 1;
  g.rhs[0] = rhs_gate, g.rhs[1] = rhs_up;
  g.scales[0] = (const __half*)scales_gate, g.scales[1] = (const __half*)scales_up;
  g.zeros[0] = (const __half*)zeros_gate, g.zeros[1] = (const __half*)zeros_up;
  g.out[0] = g.out[1] = (__half*)out;
  g.n[0] = g.n[1] = n;
  U8Args common{nullptr, (const __half*)lhs, nullptr, nullptr, nullptr, m, p, 0, block_size, 0.0f};
  const int rc = launch_u8_ring_grouped(ctx, (cudaStream_t)stream, common, g);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_U8_RING;
  return rc;
}

int adr_matmul_nt_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                      const void* rhs, int m, int p, int n, float beta) {
  // out[m,n] = lhs[m,p] . rhs[n,p]^T + beta*out  ==  matmul_f16 with NT strides and
  // a BETA store without bias; expressed through the strided entry point.
  if (!ctx || !out || !lhs || !rhs) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (m <= 0 || p <= 0 || n <= 0) return ADR_ERR_INVALID;
  // The reference always reads `out` (beta * old even when beta == 0), so stale NaN/Inf in
  // `out` propagates there; the same holds here.
  MatmulArgs a{(__half*)out, (const __half*)lhs, (const __half*)rhs, 1, m, p, n,
               1, n, 0, 1, p, 0, p, 1, 0, nullptr, beta, 1.0f,
               (uint32_t)STORE_NT_BETA, ADR_LOAD_IDENTITY, ADR_MASK_NONE};
  return run_matmul(ctx, (cudaStream_t)stream, a, false, true);
}

int adr_rms_norm_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                  const void* norm_weights, float eps, const uint8_t* rhs,
                                  const void* scales, const void* zeros, int m, int p, int n,
                                  int block_size, float beta) {
  if (!ctx || !out || !lhs || !norm_weights || !rhs || !scales) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (m <= 0 || p <= 0 || n <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (m > 16 || p % block_size != 0) return ADR_ERR_SHAPE;
  if (!aligned16(lhs) || !aligned16(rhs) || !aligned16(norm_weights)) return ADR_ERR_SHAPE;
  U8Args a{(__half*)out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, n, block_size, beta};
  a.norm_w = (const __half*)norm_weights;
  a.norm_eps = eps;
  if (!u8_ring_supports(ctx, a)) return ADR_ERR_SHAPE;
  int rc = launch_u8_ring(ctx, (cudaStream_t)stream, a);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_U8_RING;
  return rc;
}

int adr_qkv_rope_append_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* q_out,
                                         int stride_q, const void* lhs, const void* norm_weights,
                                         float eps, const uint8_t* rhs, const void* scales,
                                         const void* zeros, int m, int p, int width, int n_heads,
                                         int block_size, void* k_cache, void* v_cache, int max_seq,
                                         const int32_t* pos_dev, float theta) {
  if (!ctx || !q_out || !lhs || !rhs || !scales || !k_cache || !v_cache || !pos_dev) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (m <= 0 || p <= 0 || width <= 0 || n_heads <= 0 || block_size <= 0 || max_seq <= 0)
    return ADR_ERR_INVALID;
  if (m > 16 || p % block_size != 0) return ADR_ERR_SHAPE;
  // units of 16 columns must lie inside one of the q, k, v sections; heads hold whole pairs
  if (width % 16 != 0 || width % n_heads != 0 || (width / n_heads) % 2 != 0 || stride_q < width)
    return ADR_ERR_SHAPE;
  if (!aligned16(lhs) || !aligned16(rhs) || (norm_weights && !aligned16(norm_weights))) return ADR_ERR_SHAPE;
  U8Args a{(__half*)q_out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, 3 * width, block_size, 0.0f};
  a.norm_w = (const __half*)norm_weights;
  a.norm_eps = eps;
  if (!u8_ring_supports(ctx, a)) return ADR_ERR_SHAPE;
  RingRope rope{(__half*)k_cache, (__half*)v_cache, width, n_heads, max_seq, stride_q,
                (const int*)pos_dev, theta};
  int rc = launch_u8_ring(ctx, (cudaStream_t)stream, a, nullptr, &rope);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_U8_RING;
  return rc;
}

int adr_matmul_nt_fp16u8_allreduce(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                   const uint8_t* rhs, const void* scales, const void* zeros, int m,
                                   int p, int n, int block_size, int residual,
                                   void* const* inboxes, void* const* flags, void* epochs,
                                   int max_ctas, int rank, int world) {
  if (!ctx || !out || !lhs || !rhs || !scales || !inboxes || !flags || !epochs) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (m <= 0 || p <= 0 || n <= 0 || block_size <= 0 || max_ctas <= 0) return ADR_ERR_INVALID;
  if (world < 2 || world > 8 || rank < 0 || rank >= world) return ADR_ERR_INVALID;
  if (m > 16 || p % block_size != 0) return ADR_ERR_SHAPE;
  if (!aligned16(lhs) || !aligned16(rhs)) return ADR_ERR_SHAPE;
  U8Args a{(__half*)out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, n, block_size, 0.0f};
  if (!u8_ring_supports(ctx, a)) return ADR_ERR_SHAPE;
  RingArFuse ar = {};
  for (int r = 0; r < world; ++r) {
    if (!inboxes[r] || !flags[r]) return ADR_ERR_INVALID;
    ar.inbox[r] = static_cast<__half*>(inboxes[r]);
    ar.flags[r] = static_cast<unsigned int*>(flags[r]);
  }
  ar.epochs = static_cast<unsigned int*>(epochs);
  ar.rank = rank;
  ar.world = world;
  ar.residual = residual ? 1 : 0;
  ar.max_ctas = max_ctas;
  int rc = launch_u8_ring(ctx, (cudaStream_t)stream, a, &ar);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_U8_RING;
  return rc;
}

int adr_dequantize_absmax_uint8(adr_ctx* ctx, adr_stream stream, void* out, const void* scales,
                                const void* zeros, const uint8_t* q, int rows, int k,
                                int block_size) {
  if (!ctx || !out || !scales || !q) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (rows <= 0 || k <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (k % block_size != 0 || block_size % 16 != 0) return ADR_ERR_SHAPE;
  if (!aligned16(out) || !aligned16(q)) return ADR_ERR_SHAPE;
  return launch_dequantize_u8(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)scales,
                              (const __half*)zeros, q, rows, k, block_size);
}

int adr_quantize_absmax_uint8(adr_ctx* ctx, adr_stream stream, uint8_t* q, void* scales,
                              const void* in, int rows, int k, int block_size) {
  if (!ctx || !q || !scales || !in) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (rows <= 0 || k <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (k % block_size != 0) return ADR_ERR_SHAPE;
  return launch_quantize_u8(ctx, (cudaStream_t)stream, q, (__half*)scales, (const __half*)in, rows,
                            k, block_size);
}

int adr_embed_uint8(adr_ctx* ctx, adr_stream stream, int n_dim, int n_ids, const int16_t* in_ids,
                    void* out_embeddings, const uint8_t* embeddings_table, const void* scales,
                    int block_size) {
  if (!ctx || !in_ids || !out_embeddings || !embeddings_table || !scales) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (n_dim <= 0 || n_ids <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (n_dim % block_size != 0 || block_size % 16 != 0) return ADR_ERR_SHAPE;
  if (!aligned16(out_embeddings) || !aligned16(embeddings_table)) return ADR_ERR_SHAPE;
  return launch_embed_u8(ctx, (cudaStream_t)stream, n_dim, n_ids, (const short*)in_ids,
                         (__half*)out_embeddings, embeddings_table, (const __half*)scales, block_size);
}

int adr_trace_enable(adr_ctx* ctx, int on) {
  if (!ctx) return ADR_ERR_INVALID;
  ctx->trace_on = on != 0;
  return ADR_OK;
}

void adr_trace_clear(adr_ctx* ctx) {
  if (!ctx) return;
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->trace.clear();
}

size_t adr_trace_dump(adr_ctx* ctx, char* buf, size_t cap) {
  if (!ctx) return 0;
  std::string s;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    char line[512];
    for (const auto& t : ctx->trace) {
      snprintf(line, sizeof(line),
               "{\"m\":%d,\"k\":%d,\"n\":%d,\"batches\":%d,\"out_strides\":[%d,%d,%d],"
               "\"lhs_strides\":[%d,%d,%d],\"rhs_strides\":[%d,%d,%d],\"store\":%u,\"load\":%u,"
               "\"mask\":%u,\"kernel\":%d}\n",
               t.m, t.k, t.n, t.batches, t.strides[0], t.strides[1], t.strides[2], t.strides[3],
               t.strides[4], t.strides[5], t.strides[6], t.strides[7], t.strides[8], t.store,
               t.load, t.mask, t.kernel);
      s += line;
    }
  }
  if (buf && cap > 0) {
    size_t ncopy = s.size() < cap - 1 ? s.size() : cap - 1;
    memcpy(buf, s.data(), ncopy);
    buf[ncopy] = '\0';
  }
  return s.size() + 1;
}

}  // extern "C"
