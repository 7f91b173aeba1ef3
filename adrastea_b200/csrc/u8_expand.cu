// u8-weight GEMM for many rows (long prefills) by expansion: panels of weight rows are
// dequantised to fp16 into a scratch buffer (the fp16-rounded weights of
// adrastea_kernels/cpp/matmul_nt_wmma_16x128x256_fp16u8.cu:5-7, bit-exact) and multiplied by the
// fp16 tensor-core GEMM.  From a few thousand rows on, the fp16 GEMM's higher rate outweighs the
// extra pass over the weights; a panel is sized to stay in L2 between the two kernels, so the
// expansion costs no HBM traffic beyond reading the u8 weights once.
//   out[m,n] = lhs[m,p] . deq(rhs[n,p])^T + beta * out
#include "tma.cuh"

#include <mutex>

namespace adr {

namespace {

constexpr int EXPAND_MIN_ROWS = 3072;           // fewer rows: the dequantising GEMM is as fast
constexpr size_t EXPAND_PANEL_BYTES = 32u << 20;  // of fp16 weights per panel (L2 holds 126 MB)

// One call of the expansion path over `scratch` (fp16, at least 128 * p elements).
int expand_matmul(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, __half* scratch,
                  size_t scratch_elems) {
  size_t rows_fit = scratch_elems / (size_t)a.p;
  rows_fit = std::min(rows_fit, EXPAND_PANEL_BYTES / 2 / (size_t)a.p);
  if (rows_fit >= 256) rows_fit &= ~(size_t)255;  // whole tiles of the fp16 GEMM
  else if (rows_fit >= 128) rows_fit = 128;
  else return ADR_ERR_SHAPE;
  const int groups = a.p / a.block_size;
  for (int n0 = 0; n0 < a.n; n0 += (int)rows_fit) {
    const int rows = std::min((int)rows_fit, a.n - n0);
    int rc = launch_dequantize_u8(ctx, stream, scratch, a.scales + (size_t)n0 * groups,
                                  a.zeros ? a.zeros + (size_t)n0 * groups : nullptr,
                                  a.rhs + (size_t)n0 * a.p, rows, a.p, a.block_size);
    if (rc != ADR_OK) return rc;
    // out[:, n0 : n0 + rows] = lhs . panel^T + beta * out (the panel is [rows, p], k-contiguous)
    MatmulArgs g{a.out + n0, a.lhs, scratch, 1, a.m, a.p, rows,
                 1, a.n, 0, 1, a.p, 0, a.p, 1, 0, nullptr, a.beta, 1.0f,
                 (uint32_t)STORE_NT_BETA, ADR_LOAD_IDENTITY, ADR_MASK_NONE};
    if (!gemm_f16_tc_supports(ctx, g)) return ADR_ERR_SHAPE;
    rc = launch_gemm_f16_tc(ctx, stream, g);
    if (rc != ADR_OK) return rc;
  }
  return ADR_OK;
}

int check_u8(const adr_ctx* ctx, const void* out, const void* lhs, const void* rhs, const void* scales,
             int m, int p, int n, int block_size) {
  if (!ctx || !out || !lhs || !rhs || !scales) return ADR_ERR_INVALID;
  if (m <= 0 || p <= 0 || n <= 0 || block_size <= 0) return ADR_ERR_INVALID;
  if (p % block_size != 0 || block_size % 16 != 0 || p % 16 != 0) return ADR_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(lhs) & 15u) || (reinterpret_cast<uintptr_t>(rhs) & 15u))
    return ADR_ERR_SHAPE;
  return ADR_OK;
}

// Scratch for the entry point that may not allocate: one array per device, part of the loaded
// module, so it exists without any allocation call.  16 MiB holds 128 weight rows (the smallest
// panel) of up to 65536 columns as fp16.
constexpr size_t BUILTIN_SCRATCH_BYTES = 16u << 20;
constexpr int BUILTIN_MAX_P = (int)(BUILTIN_SCRATCH_BYTES / 2 / 128);
static __device__ __align__(256) unsigned char g_builtin_scratch[BUILTIN_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_builtin_mu;
void* g_builtin_ptr[MAX_DEVICES] = {};

// The array's device address, looked up once per device (the current device is the context's).
int builtin_scratch(adr_ctx* ctx, __half** ptr) {
  if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return ADR_ERR_INVALID;
  std::lock_guard<std::mutex> lock(g_builtin_mu);
  if (!g_builtin_ptr[ctx->device]) {
    void* a = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&a, g_builtin_scratch);
    if (e != cudaSuccess || !a) {
      ctx->last_cuda_error = (int)e;
      return ADR_ERR_CUDA;
    }
    g_builtin_ptr[ctx->device] = a;
  }
  *ptr = static_cast<__half*>(g_builtin_ptr[ctx->device]);
  return ADR_OK;
}

}  // namespace

}  // namespace adr

using namespace adr;

extern "C" int adr_matmul_nt_fp16u8_ws(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                       const uint8_t* rhs, const void* scales, const void* zeros,
                                       int m, int p, int n, int block_size, float beta,
                                       void* workspace, size_t workspace_bytes) {
  int rc = check_u8(ctx, out, lhs, rhs, scales, m, p, n, block_size);
  if (rc != ADR_OK) return rc;
  // few rows, no usable scratch, or a view the fp16 GEMM's copy engine cannot describe: the
  // entry point without scratch does the same product
  const bool usable = workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0 &&
                      workspace_bytes / 2 / (size_t)p >= 128 && p % 8 == 0 && n % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  if (m < EXPAND_MIN_ROWS || !usable || ctx->forced_kernel != ADR_KERNEL_AUTO)
    return adr_matmul_nt_fp16u8(ctx, stream, out, lhs, rhs, scales, zeros, m, p, n, block_size, beta);
  DeviceGuard guard(ctx);
  U8Args a{(__half*)out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, n, block_size, beta};
  rc = expand_matmul(ctx, (cudaStream_t)stream, a, (__half*)workspace, workspace_bytes / 2);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_F16_TC;
  return rc;
}

extern "C" int adr_matmul_nt_fp16u8_noalloc(adr_ctx* ctx, adr_stream stream, void* out,
                                            const void* lhs, const uint8_t* rhs, const void* scales,
                                            const void* zeros, int m, int p, int n, int block_size,
                                            float beta) {
  int rc = check_u8(ctx, out, lhs, rhs, scales, m, p, n, block_size);
  if (rc != ADR_OK) return rc;
  if (p > BUILTIN_MAX_P) return ADR_ERR_TOO_LARGE;  // 128 rows of p columns exceed the array
  if (p % 8 != 0 || n % 8 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) return ADR_ERR_SHAPE;
  DeviceGuard guard(ctx);
  __half* scratch = nullptr;
  rc = builtin_scratch(ctx, &scratch);
  if (rc != ADR_OK) return rc;
  U8Args a{(__half*)out, (const __half*)lhs, rhs, (const __half*)scales, (const __half*)zeros,
           m, p, n, block_size, beta};
  rc = expand_matmul(ctx, (cudaStream_t)stream, a, scratch, BUILTIN_SCRATCH_BYTES / 2);
  if (rc == ADR_OK) ctx->last_kernel = ADR_KERNEL_F16_TC;
  return rc;
}
