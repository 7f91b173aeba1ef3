// Shared declarations of the adrastea_b200 CUDA library: context, error
// plumbing, the fused store/load/mask arithmetic of the fp16 matmul path.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/adrastea_b200.h"

namespace adr {

// ---------------------------------------------------------------------------
// Arguments of one fp16 matmul call, in the reference's parameter order
// (adrastea_kernels/cpp/matmul.cu:186-190, 493-499).
// ---------------------------------------------------------------------------
struct MatmulArgs {
  __half* out;
  const __half* lhs;
  const __half* rhs;
  int batches, m, k, n;
  int s_ox, s_oy, s_oz;
  int s_lx, s_ly, s_lz;
  int s_rx, s_ry, s_rz;
  const __half* bias;
  float beta, scale;
  uint32_t store, load, mask;
};

struct TraceKey {
  int m, k, n, batches;
  int strides[9];
  uint32_t store, load, mask;
  int kernel;
  bool operator==(const TraceKey& o) const;
};

}  // namespace adr

// One context per device.  It may be shared by several host threads the way the reference
// shares its kernel object behind an Arc (adrastea_models/src/llama.rs:402): the counters and
// knobs are atomics, the trace, the tensor-map cache and the record of configured kernels
// are guarded by `mu`.  Launches from different threads on the same stream are ordered by
// the caller, as with any CUDA stream.
struct adr_ctx {
  int device = 0;
  int sm_count = 0;
  std::atomic<int> last_cuda_error{0};
  std::atomic<int> forced_kernel{ADR_KERNEL_AUTO};
  std::atomic<int> last_kernel{0};
  std::atomic<uint64_t> launches{0};
  std::atomic<bool> trace_on{false};
  std::mutex mu;
  std::vector<adr::TraceKey> trace;
  // kernels whose dynamic shared memory limit has been raised on this context's device
  std::unordered_map<const void*, size_t> smem_opt_in;
  // Device word written by kernels whose bounded waits ran out (0 = fine).
  unsigned int* d_status = nullptr;
  // Cache of TMA descriptors, keyed by (pointer, dims, strides, box).
  void* tma_cache = nullptr;
  void* encode_tiled_fn = nullptr;  // cuTensorMapEncodeTiled, resolved at init
  // tuning knobs (adr_set_tunable); 0 = let the planner choose
  std::atomic<int> tune_u8_split{0};
  std::atomic<int> tune_u8_rows{0};
  std::atomic<int> tune_u8_exact{0};  // 1: fp16-rounded dequantisation in the streaming kernel
  std::atomic<int> tune_tc_bn{0};
  std::atomic<int> tune_tc_split{0};
  std::atomic<int> tune_pdl{0};      // programmatic dependent launch of the decode and row kernels
  std::atomic<int> tune_wait_ms{0};  // limit of the peer waits in milliseconds (0: about a second)
  std::atomic<int> tune_u8_cps_m{2}, tune_u8_cps_x4{16};
  std::atomic<int> tune_ks_clusters{0}, tune_ks_stages{0}, tune_ks_off{0}, tune_ks_slack{1};  // cluster k-split kernel: clusters in the grid, ring stages
  std::atomic<int> tune_pdl_guard{15};
  std::atomic<int> tune_ts_split{0};  // k-split of the tensor-memory prefill kernel (1 = never, 2/4)
  std::atomic<int> tune_ts_bt{0};  // tokens per tile of the tensor-memory prefill kernel (128/256)
  std::atomic<int> tune_ks_pdl{1};  // the cluster k-split kernel may start early under "pdl"  // which SM-filling launches end a chain of early starts (bit 0: two CTAs per SM, bit 1: one large CTA)
  // the last launch whose CTAs left no room beside them on an SM: its number and its stream
  std::atomic<int> small_before{0};  // the last launch through this context was a small row kernel
  std::atomic<int> fill_flag{0};
  std::atomic<unsigned long long> fill_launch{0};
  std::atomic<uintptr_t> fill_stream{0};
};

namespace adr {

#define ADR_CUDA_CHECK(ctx, expr)                      \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) {                           \
      (ctx)->last_cuda_error = (int)_e;                \
      return ADR_ERR_CUDA;                             \
    }                                                  \
  } while (0)

// Makes the context's device current for the duration of an entry point and restores the
// caller's device afterwards (a process that drives several GPUs may call with another
// device current).
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(const adr_ctx* ctx) {
    if (ctx && cudaGetDevice(&prev) == cudaSuccess && prev != ctx->device)
      switched = cudaSetDevice(ctx->device) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};

// Raises a kernel's dynamic shared memory limit once per context (the attribute is per
// device; the context's device is current inside every entry point).
template <typename K>
int opt_in_smem(adr_ctx* ctx, K kfn, size_t bytes) {
  const void* key = reinterpret_cast<const void*>(kfn);
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->smem_opt_in.find(key);
  if (it != ctx->smem_opt_in.end() && it->second >= bytes) return ADR_OK;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  ctx->smem_opt_in[key] = bytes;
  return ADR_OK;
}

// Bound of a wait on a peer GPU in clock cycles (about 2 per nanosecond).
// Bookkeeping for chains of early starts (programmatic dependent launch).  A launch whose CTAs
// fill whole SMs leaves a mark on its stream; the persistent decode kernel's half-SM form reads
// it (it must not start as those SMs drain, see u8_ring.cu) and clears it once a launch with a
// full dependency has let the GPU run empty.  Small kernels in between do not clear it: they
// start early themselves and pass the early start on.
inline void note_filling_launch(adr_ctx* ctx, cudaStream_t stream, int kind_bit) {
  if (ctx->tune_pdl.load() && (ctx->tune_pdl_guard.load() & kind_bit)) {
    ctx->fill_stream = reinterpret_cast<uintptr_t>(stream);
    ctx->fill_flag = 1;
    ctx->fill_launch = ctx->launches.load() + 1;  // the number this launch is about to get
  }
}
inline bool behind_filling_launch(const adr_ctx* ctx, cudaStream_t stream) {
  if (ctx->fill_flag.load() == 0 || ctx->fill_stream.load() != reinterpret_cast<uintptr_t>(stream))
    return false;
  // bit 3 of the guard: the mark survives small kernels launched in between; without it only
  // the launch directly behind the filling one is held back
  return (ctx->tune_pdl_guard.load() & 8) != 0 || ctx->fill_launch.load() == ctx->launches.load();
}

inline long long peer_wait_cycles(const adr_ctx* ctx) {
  const int ms = ctx->tune_wait_ms;
  return ms > 0 ? (long long)ms * 2000000LL : 2000000000LL;
}

// Records a launch error, if any, and counts the launch.
inline int after_launch(adr_ctx* ctx, int nlaunches = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  ctx->launches += (uint64_t)nlaunches;
  return ADR_OK;
}

// ---------------------------------------------------------------------------
// Device arithmetic of the fused ops (matmul.cu:45-184, 444-491).
// Every store functor of the reference first converts the fp32 accumulator to
// __half; SCALE and ADD then compute in fp16, the bias/gelu/beta forms in
// fp32 with `inner + beta * old` contracted to one fma.
// ---------------------------------------------------------------------------
// The rotation of rotary.cu:4-29 for one (even, odd) pair: shared by the row kernel, the
// decode-time append kernel and the decode product's fused epilogue, so that they agree to the bit.
struct Turn {
  float c, s;
};
__device__ __forceinline__ Turn rope_turn(int position, int col_in_head, int head_dim, float theta) {
  const float phase = position / powf(theta, float(col_in_head) / head_dim);
  Turn w;
  w.c = cosf(phase);
  w.s = sinf(phase);
  return w;
}
__device__ __forceinline__ __half2 rope_apply(__half even, __half odd, Turn w) {
  const float x = __half2float(even), y = __half2float(odd);
  // The contraction is written out, so that every caller gets the same bits whatever code
  // surrounds the call: what the compiler makes of `x * c - y * s` (second product rounded, the
  // first fused into the difference) and of `x * s + y * c` (FIRST product rounded, the second
  // fused into the sum) in the reference kernel.  Checked against that kernel run live on
  // 327680 elements; the other form of the sum differs in about one element in twenty thousand.
  return __halves2half2(__float2half(__fmaf_rn(x, w.c, -__fmul_rn(y, w.s))),
                        __float2half(__fmaf_rn(y, w.c, __fmul_rn(x, w.s))));
}

__device__ __forceinline__ float gelu_tanh(float t) {
  return 0.5f * t * (1.0f + tanhf(0.7978845608028654f * (t + 0.044715f * t * t * t)));
}
__device__ __forceinline__ float quick_gelu(float t) {
  return t * (1.0f / (1.0f + expf(-1.702f * t)));
}

// Internal store op of adr_matmul_nt_f16: fp16(acc + beta * old) without the
// intermediate fp16 rounding of acc (matmul_nt_wmma_128x64x64.cu:71-76).
constexpr int STORE_NT_BETA = 16;

template <int STORE>
__device__ __forceinline__ __half store_apply(float acc, __half old, float bias, float beta,
                                              __half hscale) {
  __half hs = __float2half_rn(acc);
  if constexpr (STORE == STORE_NT_BETA) {
    return __float2half_rn(fmaf(beta, __half2float(old), acc));
  } else if constexpr (STORE == ADR_STORE_IDENTITY) {
    return hs;
  } else if constexpr (STORE == ADR_STORE_SCALE) {
    return __hmul(hs, hscale);
  } else if constexpr (STORE == ADR_STORE_ADD) {
    return __hadd(hs, old);
  } else if constexpr (STORE == ADR_STORE_BETA_BIAS) {
    float t = __half2float(hs) + bias;
    return __float2half_rn(fmaf(beta, __half2float(old), t));
  } else if constexpr (STORE == ADR_STORE_BETA_GELU_BIAS) {
    float t = gelu_tanh(__half2float(hs) + bias);
    return __float2half_rn(fmaf(beta, __half2float(old), t));
  } else {  // QUICK_GELU_BIAS
    return __float2half_rn(quick_gelu(__half2float(hs) + bias));
  }
}

constexpr __host__ __device__ bool store_reads_out(int store) {
  return store == ADR_STORE_ADD || store == ADR_STORE_BETA_BIAS ||
         store == ADR_STORE_BETA_GELU_BIAS || store == STORE_NT_BETA;
}
constexpr __host__ __device__ bool store_uses_bias(int store) {
  return store == ADR_STORE_BETA_BIAS || store == ADR_STORE_BETA_GELU_BIAS ||
         store == ADR_STORE_QUICK_GELU_BIAS;
}

// Runtime-dispatched form used by kernels that are not specialised per op.
__device__ __forceinline__ __half store_apply_rt(int store, float acc, __half old, float bias,
                                                 float beta, __half hscale) {
  switch (store) {
    case STORE_NT_BETA: return store_apply<STORE_NT_BETA>(acc, old, bias, beta, hscale);
    case ADR_STORE_SCALE: return store_apply<ADR_STORE_SCALE>(acc, old, bias, beta, hscale);
    case ADR_STORE_ADD: return store_apply<ADR_STORE_ADD>(acc, old, bias, beta, hscale);
    case ADR_STORE_BETA_BIAS: return store_apply<ADR_STORE_BETA_BIAS>(acc, old, bias, beta, hscale);
    case ADR_STORE_BETA_GELU_BIAS:
      return store_apply<ADR_STORE_BETA_GELU_BIAS>(acc, old, bias, beta, hscale);
    case ADR_STORE_QUICK_GELU_BIAS:
      return store_apply<ADR_STORE_QUICK_GELU_BIAS>(acc, old, bias, beta, hscale);
    default: return store_apply<ADR_STORE_IDENTITY>(acc, old, bias, beta, hscale);
  }
}

// ---------------------------------------------------------------------------
// u8 absmax dequantisation, bit-exact with
//   fp16((float(q) - zero) * float(scale))
// (matmul_nt_wmma_16x128x256_fp16u8.cu:5-7, quantize.cu:53-54).
// ---------------------------------------------------------------------------
__device__ __forceinline__ __half dequant_one_f32(uint32_t q, float scale, float zero) {
  return __float2half_rn(((float)q - zero) * scale);
}

// Kernel launchers implemented in the .cu files.
int launch_gemm_f16_simt(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a);
int launch_gemm_f16_tc(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a);
bool gemm_f16_tc_supports(const adr_ctx* ctx, const MatmulArgs& a);
int launch_gemm_f16_gather(adr_ctx* ctx, cudaStream_t stream, const MatmulArgs& a);
int init_gemm_f16_tc(adr_ctx* ctx);
void destroy_gemm_f16_tc(adr_ctx* ctx);

struct U8Args {
  __half* out;
  const __half* lhs;
  const uint8_t* rhs;
  const __half* scales;
  const __half* zeros;
  int m, p, n, block_size;
  float beta;
  // optional: rms_norm of the rows of lhs before the product (u8 ring kernel only)
  const __half* norm_w = nullptr;
  float norm_eps = 0.0f;
};
int launch_u8_simt(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
int launch_u8_gemv(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
int launch_u8_mma(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
int launch_u8_stream(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
bool u8_stream_supports(const adr_ctx* ctx, const U8Args& a);
// Optional fusion of a tensor-parallel all-reduce into the ring kernel (u8_ring.cu): inbox[r] and
// flags[r] are rank r's symmetric allocations as addressable from this GPU.
struct RingArFuse {
  __half* inbox[8];
  unsigned int* flags[8];
  unsigned int* epochs;
  int rank, world, residual, max_ctas;
};
// Optional epilogue of the ring kernel for a fused q/k/v projection at decode time: rotary
// embedding of q and k, k and v appended to the cache at position *pos.
struct RingRope {
  __half* k_cache;
  __half* v_cache;
  int width, n_heads, max_seq, q_pitch;
  const int* pos;
  float theta;
};
int launch_u8_ring(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const RingArFuse* ar = nullptr,
                   const RingRope* rope = nullptr);
// up to four weight matrices multiplied by the same activations in one launch
struct RingGroup {
  int count;
  const uint8_t* rhs[4];
  const __half* scales[4];
  const __half* zeros[4];
  __half* out[4];
  int n[4];
  int pair = 0;  // 1: two matrices of equal n (gate, up); out[0] receives SiluMul(gate, up), out[1] is unused
};
int launch_u8_ring_grouped(adr_ctx* ctx, cudaStream_t stream, const U8Args& common, const RingGroup& grp);
bool u8_ring_supports(const adr_ctx* ctx, const U8Args& a);
int launch_u8_ksplit(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
bool u8_ksplit_supports(const adr_ctx* ctx, const U8Args& a);
int launch_u8_tc(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
int launch_u8_ts(adr_ctx* ctx, cudaStream_t stream, const U8Args& a);
bool u8_ts_supports(const adr_ctx* ctx, const U8Args& a);
bool u8_tc_supports(const adr_ctx* ctx, const U8Args& a);
int init_u8_kernels(adr_ctx* ctx);

int launch_dequantize_u8(adr_ctx* ctx, cudaStream_t stream, __half* out, const __half* scales,
                         const __half* zeros, const uint8_t* q, int rows, int k, int block_size);
int launch_embed_u8(adr_ctx* ctx, cudaStream_t stream, int n_dim, int n_ids, const short* in_ids,
                    __half* out, const uint8_t* table, const __half* scales, int block_size);
int launch_quantize_u8(adr_ctx* ctx, cudaStream_t stream, uint8_t* q, __half* scales,
                       const __half* in, int rows, int k, int block_size);

}  // namespace adr
