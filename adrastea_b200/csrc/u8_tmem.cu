// u8-weight decode GEMV/GEMM on the 5th-generation tensor cores (m <= 16, block_size 64 or 128):
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// (replaces adrastea_kernels/cpp/matmul_nt_fp16u8.cu:4-24 and
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83 for decode shapes).
//
// The product is laid out with the WEIGHTS as the 128-row operand of tcgen05.mma and the tokens
// as its 16-column operand, so the cost per weight byte does not depend on the number of tokens:
//   * a stage is 128 k-bytes of up to 128 weight rows (four TMA boxes of 32 rows x 128 bytes,
//     128-byte swizzle) in a ring of shared-memory stages, filled by a producer warp;
//   * the consumer warps turn each byte into the fp16 value 1024 + q with one PRMT per pair
//     (exact: the byte is put under the exponent of 1024) and write the result straight into
//     TENSOR MEMORY with tcgen05.st: thread = weight row = TMEM lane, 8 columns per 16 bytes.
//     The weights never exist as fp16 in shared memory;
//   * one thread issues tcgen05.mma with the A operand read from tensor memory and the tokens
//     (resident in shared memory as 128-byte-swizzled K-major tiles, loaded once by TMA) as B;
//     every scale group gets an accumulator of its own (128 lanes x 16 fp32 columns);
//   * the consumer warps read a finished group back (tcgen05.ld) and apply scale and zero point
//     in fp32:  sum_k (q_k - z) s x_k = s * (sum_k (1024 + q_k) x_k - (1024 + z) sum_k x_k),
//     the arithmetic of matmul_nt_fp16u8.cu:13-23 (weights not rounded to fp16);
//   * k is split over a thread-block cluster of S CTAs (each CTA keeps only its slice of the
//     activations); the partial sums are exchanged through distributed shared memory and added
//     in rank order, so the result is deterministic and no scratch memory in HBM is needed.
// A cluster walks a contiguous range of 32-row strips in chunks of up to four; the ranges are
// equal to within one strip.  Under programmatic dependent launch the producer fills the ring
// before griddepcontrol.wait (weights, scales and zero points are by contract not written by
// the previous kernel); activations and output are touched only after it.  Every wait is
// bounded; a wait that runs out sets the status word and the CTA drains its copies, frees its
// tensor memory and returns.
#include <algorithm>

#include "tcgen05.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int TM_STAGE_BYTES = 128 * 128;  // 128 rows x 128 k-bytes
constexpr int TM_STRIP_BYTES = 32 * 128;
constexpr int TM_MAX_STAGES = 12;
constexpr int TM_NA = 2;        // A buffers in tensor memory (64 columns each); a power of two
constexpr int TM_ND = 8;        // group accumulators in tensor memory (16 columns each); a power of two
constexpr int TM_TOK = 16;      // token columns of the MMA
constexpr uint32_t TM_COLS = 256;  // TM_NA * 64 + TM_ND * 16
constexpr int TM_XTILE_BYTES = TM_TOK * 128;  // 16 tokens x 64 k fp16

struct TmemParams {
  U8Args a;
  int S;          // cluster size = k-split
  int per;        // strips per cluster
  int strips;     // ceil(n / 32)
  int NS;         // ring slots
  int T;          // k-tiles per ring slot (one TMA box covers T * 128 contiguous bytes of a row)
  int gps;        // scale groups per 128-k stage (1 or 2)
  int max_tiles;  // k-tiles of the longest slice
  unsigned int* status;
};

// ---- PTX wrappers that the other kernels do not need ----------------------------------
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: the A operand is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the accumulate flag known at compile time (no predicate to set up).
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_f16_ts_c(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                              uint32_t idesc) {
  if (ACCUMULATE)
    asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 1;" ::"r"(tmem_d), "r"(tmem_a),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
  else
    asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 0;" ::"r"(tmem_d), "r"(tmem_a),
                 "l"(bdesc), "r"(idesc)
                 : "memory");
}
__device__ __forceinline__ void named_bar(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, unsigned parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__device__ __forceinline__ void tmem_ld_x16t(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// Warp roles.  Every role runs at its own pace on its own stage of the pipeline, coupled to
// the others only through mbarriers:
//   warps 0-3   converters, one per TMEM lane quarter: bytes -> 1024 + q -> tensor memory
//               (A buffer q % 2 for stage q)
//   warps 4-7   drainers, one per lane quarter: read a finished group accumulator, apply
//               scale and zero point, keep the 16 token sums of their row in registers; at the
//               end of a chunk push them into the shared memory of the CTA that owns the row
//               (k-split: CTA r of the cluster owns rows [r * 128 / S, (r + 1) * 128 / S) of
//               every chunk) and go on with the next chunk at once
//   warp 8      finisher: adds the S partial sums of this CTA's rows in rank order, applies
//               beta * old and writes the outputs, off the critical path
//   warp 9      producer (TMA)
//   warps 10-11 MMA issue, k-tiles of even and of odd index (issuing an MMA costs the thread
//               tens of nanoseconds; two threads alternate so that one waits for its operands
//               while the other issues); warp 10 also allocates the tensor memory
constexpr int TM_CONV_WARPS = 4;
constexpr int TM_DRAIN_WARPS = 4;
constexpr int TM_W_FINISH = 8, TM_W_PRODUCER = 9, TM_W_MMA = 10;  // and TM_W_MMA + 1
constexpr int TM_THREADS = 12 * 32;
constexpr int TM_SCALE_AHEAD = 8;  // scale groups requested ahead of their use

template <bool PDL>
__global__ void __launch_bounds__(TM_THREADS, PDL ? 2 : 1)
    u8_tmem_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap wmap_strip,
                   const __grid_constant__ CUtensorMap xmap, TmemParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const U8Args& a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t S = (uint32_t)p.S;
  const uint32_t rank = S > 1 ? cluster_rank() : 0u;
  const int cluster_id = (int)(blockIdx.x / S);
  const int rpr = 128 / (int)S;  // rows of a chunk owned by each CTA of the cluster

  // ---- this CTA's slice of k and this cluster's range of strips ----
  const int ntiles = a.p / 128;
  const int tb = (int)((long long)rank * ntiles / S);
  const int te = (int)((long long)(rank + 1) * ntiles / S);
  const int nt = te - tb;  // stages per chunk
  const int strip_lo = cluster_id * p.per;
  const int strip_hi = min(p.strips, strip_lo + p.per);
  const int my_strips = max(0, strip_hi - strip_lo);
  const int nchunks = (my_strips + 3) / 4;
  const int total_stages = nchunks * nt;
  const int groups = a.p / a.block_size;

  // ---- shared memory ----
  uint8_t* ring = smem_raw;
  const int slot_bytes = p.T * TM_STAGE_BYTES;  // [4 strips][T tiles][32 rows][128 bytes]
  const int spc = (nt + p.T - 1) / p.T;         // ring slots per chunk
  const int total_slots = nchunks * spc;
  uint8_t* Xsm = ring + (size_t)p.NS * slot_bytes;                           // [2 * max_tiles][16][128 B]
  // partial sums pushed by the cluster: [2 buffers][S sources][m tokens][rpr rows]
  float* partial = reinterpret_cast<float*>(Xsm + (size_t)2 * p.max_tiles * TM_XTILE_BYTES);
  float* xs64 = partial + (size_t)2 * a.m * 128;                             // [2 * max_tiles][16]
  uint64_t* full = reinterpret_cast<uint64_t*>(xs64 + (size_t)2 * p.max_tiles * TM_TOK);
  uint64_t* empty = full + TM_MAX_STAGES;
  uint64_t* a_ready = empty + TM_MAX_STAGES;
  uint64_t* a_free = a_ready + TM_NA;
  uint64_t* d_ready = a_free + TM_NA;
  uint64_t* d_free = d_ready + TM_ND;
  uint64_t* red_ready = d_free + TM_ND;  // [2] partial sums of a chunk have arrived
  uint64_t* red_free = red_ready + 2;    // [2] every owner has consumed the buffer
  uint64_t* xfull = red_free + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const bool aligned = (smem_u32(smem_raw) & 1023u) == 0;  // same for every CTA of the launch
  if (tid == 0) {
    tma_prefetch_desc(&wmap);
    tma_prefetch_desc(&wmap_strip);
    tma_prefetch_desc(&xmap);
    for (int s = 0; s < p.NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], TM_CONV_WARPS);
    }
    for (int i = 0; i < TM_NA; ++i) {
      mbar_init(&a_ready[i], TM_CONV_WARPS);
      mbar_init(&a_free[i], 1);
    }
    for (int i = 0; i < TM_ND; ++i) {
      mbar_init(&d_ready[i], 1);
      mbar_init(&d_free[i], TM_DRAIN_WARPS);
    }
    // an owner hears from every drainer warp of the cluster that holds some of its rows
    const unsigned pushers = S <= 4 ? 4u : S;
    mbar_init(&red_ready[0], pushers);
    mbar_init(&red_ready[1], pushers);
    mbar_init(&red_free[0], S);
    mbar_init(&red_free[1], S);
    mbar_init(xfull, 1);
    *abort_flag = aligned ? 0 : 1;
    mbar_fence_init();
    if (!aligned) atomicOr(p.status, 16u);
  }
  if (warp == TM_W_MMA) tmem_alloc(tmem_slot, TM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (S > 1) {
    // the peers' barriers exist before anyone can arrive on them
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (PDL) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == TM_W_PRODUCER) {
    // ------------------------------- producer -------------------------------
    if (lane == 0 && aligned) {
      bool ok = true;
      int q = 0;
      int s = 0;
      unsigned par = 0;
      // One ring slot: T k-tiles of up to four strips.  A full chunk is ONE 3-D box (128 bytes
      // x 128 rows x T tiles); the last chunk of a range may hold fewer strips and is loaded
      // strip by strip (128 bytes x 32 rows x T tiles each).  Issuing a copy costs this thread
      // tens of nanoseconds, so the number of copies matters.
      auto issue = [&](int ci, int ks) {
        const int strip0 = strip_lo + 4 * ci;
        const int ns = min(4, strip_hi - strip0);
        uint8_t* slot = ring + (size_t)s * slot_bytes;
        mbar_expect_tx(&full[s], (unsigned)(ns * p.T * TM_STRIP_BYTES));
        if (ns == 4 && p.T == 1) {
          tma_load_3d(slot, &wmap, 0, strip0 * 32, tb + ks, &full[s]);
        } else {
          for (int j = 0; j < ns; ++j)
            tma_load_3d(slot + (size_t)j * p.T * TM_STRIP_BYTES, &wmap_strip, 0, (strip0 + j) * 32,
                        tb + ks * p.T, &full[s]);
        }
        if (++s == p.NS) s = 0, par ^= 1u;
      };
      int ci = 0, ks = 0;
      auto advance = [&]() {
        if (++ks == spc) ks = 0, ++ci;
      };
      // fill the ring before waiting for the previous kernel: these loads touch only weights
      for (; q < total_slots && q < p.NS; ++q) {
        issue(ci, ks);
        advance();
      }
      if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
      // this CTA's slice of the activations: 2 * nt tiles of [16 tokens][64 k] (rows >= m are
      // filled with zeros by the copy engine)
      if (my_strips > 0) {
        // one box: 64 k x 16 tokens x all 64-wide tiles of the longest slice (a shorter slice
        // reads one or two tiles beyond its own, which nobody uses)
        mbar_expect_tx(xfull, (unsigned)(2 * p.max_tiles * TM_XTILE_BYTES));
        tma_load_3d(Xsm, &xmap, 0, 0, 2 * tb, xfull);
      } else {
        mbar_arrive(xfull);
      }
      for (; q < total_slots; ++q) {
        if (!mbar_wait(&empty[s], par ^ 1u) || *abort_flag) { ok = false; break; }
        issue(ci, ks);
        advance();
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.status, 32u);
      }
      // drain: every issued copy has landed before the CTA may exit
      const int issued = q;
      for (int qq = max(0, issued - p.NS); qq < issued; ++qq)
        if (!mbar_wait(&full[qq % p.NS], (unsigned)(qq / p.NS) & 1u)) atomicOr(p.status, 64u);
      if (!mbar_wait(xfull, 0)) atomicOr(p.status, 64u);
    }
  } else if (warp >= TM_W_MMA) {
    // ------------------------------- MMA issue -------------------------------
    const int mma_phase = warp - TM_W_MMA;  // this warp issues the k-tiles with q % 2 == mma_phase
    if (lane == 0 && aligned && total_stages > 0) {
      constexpr uint32_t idesc = umma_idesc_f16(TM_TOK, false);
      bool ok = mbar_wait(xfull, 0) && !*abort_flag;
      // One thread issues everything, so the loop is kept free of divisions and of address
      // arithmetic that can be folded: per k-tile one descriptor base, per MMA constant offsets.
      const uint64_t xdesc0 = umma_desc_k_sw128(smem_u32(Xsm));
      const bool two_groups = p.gps == 2;
      int q = 0;    // k-tiles issued so far
      int gi = 0;   // scale groups issued so far
      for (int ci = 0; ci < nchunks && ok; ++ci) {
        for (int kt = 0; kt < nt && ok; ++kt, ++q, gi += two_groups ? 2 : 1) {
          if ((q & 1) != mma_phase) continue;
          const int ab = q & (TM_NA - 1);
          if (!mbar_wait(&a_ready[ab], (unsigned)(q / TM_NA) & 1u) || *abort_flag) { ok = false; break; }
          const int acc0 = gi & (TM_ND - 1), acc1 = (gi + 1) & (TM_ND - 1);
          if (!mbar_wait(&d_free[acc0], ((unsigned)(gi / TM_ND) & 1u) ^ 1u)) ok = false;
          if (two_groups && !mbar_wait(&d_free[acc1], ((unsigned)((gi + 1) / TM_ND) & 1u) ^ 1u)) ok = false;
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = tmem_base + (uint32_t)(ab * 64);
          const uint32_t d0 = tmem_base + (uint32_t)(TM_NA * 64 + acc0 * TM_TOK);
          const uint32_t d1 = two_groups ? tmem_base + (uint32_t)(TM_NA * 64 + acc1 * TM_TOK) : d0;
          // B: tiles 2 * kt and 2 * kt + 1 of the resident activations (2 KB = 128 sixteen-byte
          // units apart), 32 bytes (2 units) further per k16 step
          const uint64_t xdesc = xdesc0 + (uint64_t)(2 * kt) * (TM_XTILE_BYTES >> 4);
          constexpr uint64_t T1 = TM_XTILE_BYTES >> 4;  // the second 64-wide tile of the k-tile
          umma_f16_ts_c<false>(d0, a_addr, xdesc, idesc);
          umma_f16_ts_c<true>(d0, a_addr + 8, xdesc + 2, idesc);
          umma_f16_ts_c<true>(d0, a_addr + 16, xdesc + 4, idesc);
          umma_f16_ts_c<true>(d0, a_addr + 24, xdesc + 6, idesc);
          if (two_groups) umma_f16_ts_c<false>(d1, a_addr + 32, xdesc + T1, idesc);
          else umma_f16_ts_c<true>(d1, a_addr + 32, xdesc + T1, idesc);
          umma_f16_ts_c<true>(d1, a_addr + 40, xdesc + T1 + 2, idesc);
          umma_f16_ts_c<true>(d1, a_addr + 48, xdesc + T1 + 4, idesc);
          umma_f16_ts_c<true>(d1, a_addr + 56, xdesc + T1 + 6, idesc);
          umma_commit(&a_free[ab]);
          umma_commit(&d_ready[acc0]);
          if (two_groups) umma_commit(&d_ready[acc1]);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicOr(p.status, 8u);
      }
    }
  } else if (warp < TM_CONV_WARPS) {
    // ------------------------------- converters -------------------------------
    const int quarter = warp;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = aligned;
    int q = 0;   // k-tiles converted so far (A buffer q % 2)
    int sq = 0;  // ring slots consumed so far
    for (int ci = 0; ci < nchunks; ++ci) {
      const int ns = min(4, strip_hi - (strip_lo + 4 * ci));
      const bool have_rows = quarter < ns;
      for (int ks = 0; ks < spc; ++ks, ++sq) {
        const int slot = sq % p.NS;
        const int tcount = min(p.T, nt - ks * p.T);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[slot], (unsigned)(sq / p.NS) & 1u) && !*abort_flag);
        for (int t = 0; t < tcount; ++t, ++q) {
          const int ab = q % TM_NA;
          uint4 w[8];
          if (ok && have_rows) {
            const uint8_t* wrow = ring + (size_t)slot * slot_bytes +
                                  (size_t)(quarter * p.T + t) * TM_STRIP_BYTES + lane * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)  // logical 16-byte chunk c of this thread's row
              w[c] = *reinterpret_cast<const uint4*>(wrow + ((c ^ (lane & 7)) * 16));
          }
          if (t == tcount - 1) {
            // the slot is in registers: hand it back before waiting for the A buffer
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
          }
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&a_free[ab], ((unsigned)(q / TM_NA) & 1u) ^ 1u));
          tc_fence_after_sync();
          if (ok && have_rows) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
              uint32_t h[8];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                h[2 * j] = prmt(ww[j], 0x64646464u, 0x4140u);      // (1024 + q) for bytes 0, 1
                h[2 * j + 1] = prmt(ww[j], 0x64646464u, 0x4342u);  // bytes 2, 3
              }
              tmem_st_x8(tmem_base + lane_base + (uint32_t)(ab * 64 + c * 8), h);
            }
          }
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_ready[ab]);  // also on failure, so that nobody waits for this warp
        }
      }
    }
    if (!ok && lane == 0) atomicOr(p.status, 1u);
  } else if (warp < TM_CONV_WARPS + TM_DRAIN_WARPS) {
    // ------------------------------- drainers -------------------------------
    const int quarter = warp & 3;
    const int dt = tid - TM_CONV_WARPS * 32;  // 0 .. 127
    const int row = quarter * 32 + lane;      // row of the chunk = TMEM lane
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const bool wide = a.m > 8;                // tokens 8..15 exist
    const int gshift = p.gps == 2 ? 1 : 0;
    const unsigned short* sc16 = reinterpret_cast<const unsigned short*>(a.scales);
    const unsigned short* zp16 = reinterpret_cast<const unsigned short*>(a.zeros);
    const int G = nt * p.gps;                 // scale groups of a chunk in this CTA's slice
    const int total_groups = nchunks * G;
    bool ok = aligned;

    // (chunk, group) of the scale that is requested next: TM_SCALE_AHEAD groups ahead of the
    // one being drained, across chunk boundaries
    int pf_ci = 0, pf_gl = 0;
    auto scale_index = [&](int ci, int gl, bool& valid) -> size_t {
      const int strip0 = strip_lo + 4 * ci;
      const int nrow = strip0 * 32 + row;
      valid = ci < nchunks && quarter < min(4, strip_hi - strip0) && nrow < a.n;
      return (size_t)min(nrow, a.n - 1) * groups + (size_t)tb * p.gps + gl;
    };
    unsigned short sreg[TM_SCALE_AHEAD], zreg[TM_SCALE_AHEAD];
#pragma unroll
    for (int j = 0; j < TM_SCALE_AHEAD; ++j) {
      bool valid;
      const size_t gi = scale_index(pf_ci, pf_gl, valid);
      sreg[j] = 0, zreg[j] = 0;
      if (valid) {
        sreg[j] = __ldg(sc16 + gi);
        if (zp16 != nullptr) zreg[j] = __ldg(zp16 + gi);
      }
      if (++pf_gl == G) pf_gl = 0, ++pf_ci;
    }

    if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
    // the activation sums per 64-wide tile and token (the 16-byte pieces of a row are visited
    // in an order rotated by the token, so that the lanes of a warp read different banks)
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(xfull, 0) && !*abort_flag);
    if (ok) {
      for (int idx = dt; idx < 2 * nt * TM_TOK; idx += TM_DRAIN_WARPS * 32) {
        const int tile = idx >> 4, tok = idx & 15;
        const uint8_t* xr = Xsm + (size_t)tile * TM_XTILE_BYTES + tok * 128;
        float sum = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 u = *reinterpret_cast<const uint4*>(xr + ((c + tok) & 7) * 16);
          const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            sum += f.x;
            sum += f.y;
          }
        }
        xs64[tile * TM_TOK + tok] = sum;
      }
    }
    named_bar(1, TM_DRAIN_WARPS * 32);

    float d[TM_TOK];
#pragma unroll
    for (int t = 0; t < TM_TOK; ++t) d[t] = 0.0f;
    int ci = 0, gl = 0;  // chunk and group within the chunk of the group being drained
    for (int gs0 = 0; gs0 < total_groups; gs0 += TM_SCALE_AHEAD) {
#pragma unroll
      for (int j = 0; j < TM_SCALE_AHEAD; ++j) {
        const int gs = gs0 + j;
        if (gs >= total_groups) break;
        const int ns = min(4, strip_hi - (strip_lo + 4 * ci));
        const bool have_rows = quarter < ns;
        const int acc = gs % TM_ND;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&d_ready[acc], (unsigned)(gs / TM_ND) & 1u) && !*abort_flag);
        tc_fence_after_sync();
        if (ok && have_rows) {
          const int kt = gl >> gshift, e = gl & (p.gps - 1);
          const float sc = __half2float(__ushort_as_half(sreg[j]));
          const float cz = zp16 != nullptr ? 1024.0f + __half2float(__ushort_as_half(zreg[j])) : 1151.5f;
          const uint32_t d_addr = tmem_base + lane_base + (uint32_t)(TM_NA * 64 + acc * TM_TOK);
          const float* x0 = xs64 + (size_t)(2 * kt + (p.gps == 2 ? e : 0)) * TM_TOK;
          if (wide) {
            uint32_t v[16];
            tmem_ld_x16t(d_addr, v);
            float xs[16];
#pragma unroll
            for (int t = 0; t < 16; t += 4) {
              const float4 f = *reinterpret_cast<const float4*>(x0 + t);
              xs[t] = f.x, xs[t + 1] = f.y, xs[t + 2] = f.z, xs[t + 3] = f.w;
            }
            if (p.gps == 1) {
#pragma unroll
              for (int t = 0; t < 16; t += 4) {
                const float4 f = *reinterpret_cast<const float4*>(x0 + TM_TOK + t);
                xs[t] += f.x, xs[t + 1] += f.y, xs[t + 2] += f.z, xs[t + 3] += f.w;
              }
            }
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 16; ++t) d[t] = fmaf(sc, fmaf(-cz, xs[t], __uint_as_float(v[t])), d[t]);
          } else {
            uint32_t v[8];
            tmem_ld_x8(d_addr, v);
            float xs[8];
#pragma unroll
            for (int t = 0; t < 8; t += 4) {
              const float4 f = *reinterpret_cast<const float4*>(x0 + t);
              xs[t] = f.x, xs[t + 1] = f.y, xs[t + 2] = f.z, xs[t + 3] = f.w;
            }
            if (p.gps == 1) {
#pragma unroll
              for (int t = 0; t < 8; t += 4) {
                const float4 f = *reinterpret_cast<const float4*>(x0 + TM_TOK + t);
                xs[t] += f.x, xs[t + 1] += f.y, xs[t + 2] += f.z, xs[t + 3] += f.w;
              }
            }
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 8; ++t) d[t] = fmaf(sc, fmaf(-cz, xs[t], __uint_as_float(v[t])), d[t]);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&d_free[acc]);  // also on failure, so that the MMA warp can finish
        {  // request the scale TM_SCALE_AHEAD groups ahead into the register just used
          bool valid;
          const size_t gi = scale_index(pf_ci, pf_gl, valid);
          if (valid) {
            sreg[j] = __ldg(sc16 + gi);
            if (zp16 != nullptr) zreg[j] = __ldg(zp16 + gi);
          }
          if (++pf_gl == G) pf_gl = 0, ++pf_ci;
        }
        if (++gl == G) {
          // ---- end of the chunk: push this row's sums to the CTA that owns the row ----
          const int buf = ci & 1;
          // the owners have consumed what this buffer held two chunks ago
          if (!__all_sync(0xffffffffu, mbar_wait_cluster(&red_free[buf], ((unsigned)(ci >> 1) & 1u) ^ 1u))) {
            ok = false;
            if (lane == 0) atomicOr(p.status, 4u);
          }
          const uint32_t owner = (uint32_t)(row / rpr);
          const uint32_t slot_addr =
              smem_u32(partial + ((size_t)(buf * (int)S + (int)rank) * a.m) * rpr + (row % rpr));
          const uint32_t dst = map_to_rank(slot_addr, owner);
          if (have_rows) {
#pragma unroll
            for (int t = 0; t < TM_TOK; ++t)
              if (t < a.m) st_cluster_f32(dst + (uint32_t)(t * rpr) * 4u, ok ? d[t] : 0.0f);
          }
          // the lanes' stores are ordered before the release by the warp barrier
          __syncwarp();
          if (lane == 0 || (S == 8 && lane == 16))
            mbar_arrive_remote(map_to_rank(smem_u32(&red_ready[buf]), owner));
#pragma unroll
          for (int t = 0; t < TM_TOK; ++t) d[t] = 0.0f;
          gl = 0;
          ++ci;
        }
      }
    }
    if (!ok && lane == 0) atomicOr(p.status, 2u);
  } else if (warp == TM_W_FINISH) {
    // ------------------------------- finisher -------------------------------
    // rows [rank * rpr, (rank + 1) * rpr) of every chunk: sum of the S pushed partial sums in
    // rank order, beta * old, store.  Output e of the chunk = token e / rpr, row e % rpr.
    bool ok = aligned;
    if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int ci = 0; ci < nchunks; ++ci) {
      const int buf = ci & 1;
      const int strip0 = strip_lo + 4 * ci;
      const int ns = min(4, strip_hi - strip0);
      const int nr0 = strip0 * 32 + (int)rank * rpr;  // first row of this CTA's share
      const int outs = rpr * a.m;
      const float* pb = partial + (size_t)buf * S * a.m * rpr;
      const int rshift = 31 - __clz(rpr);  // rpr is a power of two
      constexpr int FB = 16;               // outputs per lane and round: their loads are in flight together
      bool arrived = false;
      for (int e0 = 0; e0 < outs; e0 += 32 * FB) {
        float old[FB];
#pragma unroll
        for (int u = 0; u < FB; ++u) {
          const int e = e0 + u * 32 + lane;
          const int r_in = e & (rpr - 1), tok = e >> rshift;
          const bool live = e < outs && (int)rank * rpr + r_in < ns * 32 && nr0 + r_in < a.n;
          old[u] = live ? __half2float(a.out[(size_t)tok * a.n + nr0 + r_in]) : 0.0f;
        }
        // the old values of the first round are requested before the partial sums are awaited
        if (!arrived) {
          if (!__all_sync(0xffffffffu, mbar_wait_cluster(&red_ready[buf], (unsigned)(ci >> 1) & 1u))) {
            ok = false;
            if (lane == 0) atomicOr(p.status, 4u);
          }
          arrived = true;
        }
#pragma unroll
        for (int u = 0; u < FB; ++u) {
          const int e = e0 + u * 32 + lane;
          const int r_in = e & (rpr - 1), tok = e >> rshift;
          const bool live = e < outs && (int)rank * rpr + r_in < ns * 32 && nr0 + r_in < a.n;
          if (live && ok) {
            float v = 0.0f;
            for (uint32_t r = 0; r < S; ++r) v += pb[(size_t)(r * a.m + tok) * rpr + r_in];
            a.out[(size_t)tok * a.n + nr0 + r_in] = __float2half_rn(fmaf(a.beta, old[u], v));
          }
        }
      }
      // The buffer may be pushed into again: tell every CTA of the cluster - unless nobody will
      // (the last two chunks): a CTA that has finished must not be signalled any more.
      __syncwarp();
      if (lane == 0 && ci + 2 < nchunks)
        for (uint32_t r = 0; r < S; ++r) mbar_arrive_remote(map_to_rank(smem_u32(&red_free[buf]), r));
    }
  }

  // No cluster barrier at the end: a CTA's finisher returns only after every peer's partial
  // sums for its rows have arrived, and nothing else is ever written into its shared memory
  // (the buffer-free signals above stop two chunks before the end).
  tc_fence_before_sync();
  __syncthreads();
  if (warp == TM_W_MMA) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TM_COLS);
  }
}

struct TmemPlan {
  int S, per, strips, clusters, NS, T, gps, max_tiles;
  size_t smem;
};

}  // namespace

// Number of clusters of S CTAs that can be resident at once, asked of the runtime once per
// context and cluster size (0: such a launch is not possible).
static int max_clusters(adr_ctx* ctx, int S, size_t smem, bool pdl);

namespace {

bool plan_tmem(adr_ctx* ctx, const U8Args& a, bool pdl, TmemPlan& pl) {
  if (a.m < 1 || a.m > TM_TOK || a.p % 128 != 0 || a.n < 1) return false;
  if (a.block_size != 64 && a.block_size != 128) return false;
  if (a.norm_w != nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(a.rhs) & 15u) || (reinterpret_cast<uintptr_t>(a.lhs) & 15u) ||
      (a.p % 16) != 0)
    return false;
  if (!ctx->encode_tiled_fn) return false;
  const int ntiles = a.p / 128;
  const int strips = (a.n + 31) / 32;
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  // Shared memory per CTA: half an SM's worth under programmatic dependent launch, so that
  // the first CTAs of the next launch fit beside this one and prefetch; all of it otherwise.
  const size_t budget = pdl ? 113 * 1024 : 224 * 1024;
  for (int S : {4, 2, 1, 8}) {
    if (S > ntiles) continue;
    const int max_tiles = (ntiles + S - 1) / S;
    if (2 * max_tiles > 256) continue;  // one copy brings the whole activation slice
    const size_t fixed = (size_t)2 * max_tiles * TM_XTILE_BYTES + (size_t)2 * a.m * 128 * 4 +
                         (size_t)2 * max_tiles * TM_TOK * 4 + 512;
    // k-tiles per ring slot: a copy then takes T * 128 contiguous bytes of every row
    const int want_t = ctx->tune_u8_tiles;
    int T = want_t > 0 ? want_t : 1;
    T = std::max(1, std::min(T, max_tiles));
    const size_t slot_bytes = (size_t)T * TM_STAGE_BYTES;
    if (fixed + 2 * slot_bytes > 224 * 1024) continue;
    size_t room = budget > fixed ? budget - fixed : 0;
    int ns = (int)(room / slot_bytes);
    if (ns < 2) ns = (int)((224 * 1024 - fixed) / slot_bytes);  // one CTA per SM
    ns = std::min(ns, TM_MAX_STAGES);
    if (ns < 2) continue;
    const size_t smem = fixed + (size_t)ns * slot_bytes;
    int maxc = S == 1 ? sms : max_clusters(ctx, S, smem, pdl);
    if (maxc <= 0) continue;
    maxc = std::min(maxc, sms / S);
    const int per = (strips + maxc - 1) / maxc;
    pl.S = S;
    pl.per = per;
    pl.strips = strips;
    pl.clusters = (strips + per - 1) / per;
    pl.NS = ns;
    pl.T = T;
    pl.gps = 128 / a.block_size;
    pl.max_tiles = max_tiles;
    pl.smem = smem;
    return true;
  }
  return false;
}

template <bool PDL>
int launch_tmem_p(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const TmemPlan& pl) {
  auto kfn = u8_tmem_kernel<PDL>;
  if (int rc = opt_in_smem(ctx, kfn, 226 * 1024); rc != ADR_OK) return rc;
  CUtensorMap wmap, wmap_strip, xmap;
  {
    // weights as (k within tile, row, k-tile): a box of 128 x R x T lands as T tiles of
    // [R rows][128 bytes], each row swizzled by its own index; R = 128 for a whole chunk,
    // 32 for one strip
    const uint64_t dims[3] = {128u, (uint64_t)a.n, (uint64_t)(a.p / 128)};
    const uint64_t strides[2] = {(uint64_t)a.p, 128u};
    const uint32_t box[3] = {128u, 128u, 1u};
    int rc = tma_get(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
    const uint32_t sbox[3] = {128u, 32u, (uint32_t)pl.T};
    rc = tma_get(ctx, &wmap_strip, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.rhs, dims, strides, sbox,
                 CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  {
    // activations as (k within a 64-wide tile, token, tile): one box brings a CTA's whole slice
    const uint64_t dims[3] = {64u, (uint64_t)a.m, (uint64_t)(a.p / 64)};
    const uint64_t strides[2] = {(uint64_t)a.p * 2, 128u};
    const uint32_t box[3] = {64u, (uint32_t)TM_TOK, (uint32_t)(2 * pl.max_tiles)};
    int rc = tma_get(ctx, &xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a.lhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  TmemParams p;
  p.a = a;
  p.S = pl.S;
  p.per = pl.per;
  p.strips = pl.strips;
  p.NS = pl.NS;
  p.T = pl.T;
  p.gps = pl.gps;
  p.max_tiles = pl.max_tiles;
  p.status = ctx->d_status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.clusters * pl.S, 1, 1);
  cfg.blockDim = dim3(TM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pl.S > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = pl.S;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (PDL) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, wmap, wmap_strip, xmap, p);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  return after_launch(ctx);
}

}  // namespace

static int max_clusters(adr_ctx* ctx, int S, size_t smem, bool pdl) {
  const uint64_t key = ((uint64_t)(pdl ? 1 : 0) << 40) | ((uint64_t)S << 32) | (uint64_t)smem;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->cluster_capacity.find(key);
    if (it != ctx->cluster_capacity.end()) return it->second;
  }
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S * 64, 1, 1);
  cfg.blockDim = dim3(TM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (pdl) {
    auto kfn = u8_tmem_kernel<true>;
    if (opt_in_smem(ctx, kfn, 226 * 1024) != ADR_OK) return 0;
    e = cudaOccupancyMaxActiveClusters(&n, kfn, &cfg);
  } else {
    auto kfn = u8_tmem_kernel<false>;
    if (opt_in_smem(ctx, kfn, 226 * 1024) != ADR_OK) return 0;
    e = cudaOccupancyMaxActiveClusters(&n, kfn, &cfg);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->cluster_capacity[key] = n;
  return n;
}

bool u8_tmem_supports(adr_ctx* ctx, const U8Args& a) {
  TmemPlan pl;
  return plan_tmem(ctx, a, ctx->tune_pdl != 0, pl);
}

int launch_u8_tmem(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  TmemPlan pl;
  const bool pdl = ctx->tune_pdl != 0;
  if (!plan_tmem(ctx, a, pdl, pl)) return ADR_ERR_SHAPE;
  return pdl ? launch_tmem_p<true>(ctx, stream, a, pl) : launch_tmem_p<false>(ctx, stream, a, pl);
}

}  // namespace adr
