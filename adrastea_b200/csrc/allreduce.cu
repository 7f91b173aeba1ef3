// One-shot all-reduce (sum) of an fp16 vector over peer memory, for the row-split products of
// tensor-parallel decoding (partial [tokens, hidden] per rank, 256 KB at 16 x 8192): every GPU
// reads all partial vectors straight from its peers' memory over NVLink and adds them in rank
// order, so all ranks get the same bits.  No counterpart in the reference (which has no
// multi-GPU path, adrastea_models/src/llama.rs:28-29); it replaces a latency-bound NCCL call
// and, unlike one, can sit inside a captured CUDA graph next to the GEMV kernels.
//
// Protocol.  Rank r's partial vector lies in its own copy of a symmetric buffer, written by the
// kernel that precedes this one on r's stream.  Block b of this kernel on rank r
//   1. stores its epoch number into slot [b][r] of every peer's flag array (release, system scope);
//   2. waits until slots [b][0..world) of its own flag array hold that epoch (acquire, system
//      scope; the wait is bounded: after about a second it sets the context's status word and
//      goes on, so a dead peer costs a wrong result, never a hung GPU);
//   3. adds slice b of all world vectors (16-byte loads from peer memory) and writes slice b of
//      the output (optionally plus the old output: the residual).
// A peer signals only after its preceding kernel has completed, so its whole vector is in place.
// There is no second barrier: callers alternate between two symmetric buffers, and a rank can
// overwrite a buffer only two all-reduces later, by which time every peer has passed step 2 of
// the all-reduce in between and therefore finished reading.  Epochs are per-block counters in
// device memory, advanced by the kernel itself, so a captured graph can be replayed.
// Plain peer loads and stores only: no multicast, no multimem.
#include "common.cuh"

namespace adr {

namespace {

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_THREADS = 256;

struct ArParams {
  const __half* bufs[AR_MAX_WORLD];   // the partial vector of every rank (peer pointers)
  unsigned int* flags[AR_MAX_WORLD];  // the flag array of every rank: [blocks][world]
  unsigned int* epochs;               // this rank's per-block epoch counters
  __half* out;
  int rank, world, residual;
  long long count;                    // elements, a multiple of 8
  long long wait_cycles;              // bound of the wait for the peers' flags
  unsigned int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool PDL>
__global__ void __launch_bounds__(AR_THREADS) allreduce_oneshot_kernel(ArParams p) {
  if (PDL) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  __shared__ unsigned int s_epoch;
  const int tid = threadIdx.x, b = blockIdx.x;
  if (tid == 0) {
    const unsigned int e = p.epochs[b] + 1u;
    p.epochs[b] = e;
    s_epoch = e;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  if (tid < p.world) {
    st_release_sys(p.flags[tid] + (size_t)b * p.world + p.rank, epoch);
    const unsigned int* mine = p.flags[p.rank] + (size_t)b * p.world + tid;
    const long long t0 = clock64();
    // (epoch - seen) as a signed difference: correct across wrap-around
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > p.wait_cycles) {
        atomicOr(p.status, 128u);
        break;
      }
    }
  }
  __syncthreads();
  const long long nvec = p.count / 8;
  const long long per = (nvec + gridDim.x - 1) / gridDim.x;
  const long long lo = (long long)b * per, hi = min(nvec, lo + per);
  for (long long i = lo + tid; i < hi; i += AR_THREADS) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    uint4 v[AR_MAX_WORLD];
#pragma unroll
    for (int r = 0; r < AR_MAX_WORLD; ++r)
      if (r < p.world) v[r] = __ldcg(reinterpret_cast<const uint4*>(p.bufs[r]) + i);
#pragma unroll
    for (int r = 0; r < AR_MAX_WORLD; ++r)
      if (r < p.world) {
        const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += __low2float(h[j]);
          acc[2 * j + 1] += __high2float(h[j]);
        }
      }
    uint4* dst = reinterpret_cast<uint4*>(p.out) + i;
    if (p.residual) {
      const uint4 o = *dst;
      const __half2* h = reinterpret_cast<const __half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __low2float(h[j]);
        acc[2 * j + 1] += __high2float(h[j]);
      }
    }
    uint4 res;
    __half2* rh = reinterpret_cast<__half2*>(&res);
#pragma unroll
    for (int j = 0; j < 4; ++j) rh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
    *dst = res;
  }
}

}  // namespace

}  // namespace adr

using namespace adr;

extern "C" int adr_allreduce_oneshot(adr_ctx* ctx, adr_stream stream, void* out,
                                     const void* const* bufs, void* const* flags, void* epochs,
                                     int blocks, int rank, int world, long long count,
                                     int residual) {
  if (!ctx || !out || !bufs || !flags || !epochs) return ADR_ERR_INVALID;
  DeviceGuard guard(ctx);
  if (world < 2 || world > AR_MAX_WORLD || rank < 0 || rank >= world) return ADR_ERR_INVALID;
  if (count <= 0 || blocks < 1 || blocks > 1024) return ADR_ERR_INVALID;
  if (count % 8 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) return ADR_ERR_SHAPE;
  ArParams p = {};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r] || !flags[r] || (reinterpret_cast<uintptr_t>(bufs[r]) & 15u)) return ADR_ERR_INVALID;
    p.bufs[r] = static_cast<const __half*>(bufs[r]);
    p.flags[r] = static_cast<unsigned int*>(flags[r]);
  }
  p.epochs = static_cast<unsigned int*>(epochs);
  p.out = static_cast<__half*>(out);
  p.rank = rank;
  p.world = world;
  p.residual = residual ? 1 : 0;
  p.count = count;
  p.status = ctx->d_status;
  p.wait_cycles = peer_wait_cycles(ctx);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, 1, 1);
  cfg.blockDim = dim3(AR_THREADS, 1, 1);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->tune_pdl ? 1 : 0;
  cudaError_t e = ctx->tune_pdl ? cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<true>, p)
                                : cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel<false>, p);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  ctx->small_before = 1;  // a small kernel that holds its CTA slots while it waits for the peers
  return after_launch(ctx);
}
