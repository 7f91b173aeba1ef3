// u8-weight decode GEMV/GEMM, k split over a thread-block cluster (m <= 16, block_size 64 or
// 128, p a multiple of 128 from 2048 on; a cluster of S <= 8 CTAs covers 1024 * S of k, a longer k
// goes out as several launches over consecutive k ranges):
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// (replaces adrastea_kernels/cpp/matmul_nt_fp16u8.cu:4-24 for decode shapes; same arithmetic as
// the persistent ring kernel: one PRMT per weight pair makes 1024 + q, mma.sync.m16n8k16 sums
// (1024 + q) x, scale and zero point are applied in fp32 once per scale group.)
//
// What the split buys.  CTA r of a cluster owns the k range [1024 r, 1024 r + 1024) for the whole
// launch, and consumer warp w of it the 128-wide tile w of that range.  So
//   * a warp's activations never change: it loads its 128 k x m tokens once, straight into the
//     registers of the MMA's B operand (32 registers at 16 tokens), together with their sums.
//     No activations in shared memory: nothing to load per launch and per CTA but 2-4 KB a warp,
//     no fragment loads in the main loop, and room for two CTAs per SM at any token count;
//   * a unit of work (16 weight rows x this CTA's 1024 k, one ring stage) is a quarter or an
//     eighth of the ring kernel's, so that n / 16 units spread evenly over the SMs.
// The price is a reduction over the cluster.  Per unit, the eight consumer warps leave their
// partial sums in shared memory and go on; a ninth warp adds them up and pushes the 16 x tokens
// partial result into the inbox of the unit's owner (CTA unit % S of the cluster) through
// distributed shared memory; for the units its CTA owns it also adds the S pushed results in
// rank order, adds beta * old and writes the outputs.  Inbox slots are handed back to the pushers by
// remote mbarrier arrivals.  All waits are bounded: one that runs out sets the status word and
// makes the CTA skip its remaining waits, so the kernel always ends.
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

#include "tma.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int KS_TILE_BYTES = 16 * 128;               // 16 rows x 128 k
constexpr int KS_W_BYTES = 8 * KS_TILE_BYTES;         // 16 KB: eight tiles, one per consumer warp
constexpr int KS_STAGE_BYTES = KS_W_BYTES + 1024;     // + scales and zero points
constexpr int KS_MAX_STAGES = 6;
constexpr int KS_NR = 2;                              // partial-sum buffers in rotation
constexpr int KS_INB = 2;                             // inbox slots per owner
constexpr int KS_MAX_S = 8;
constexpr int KS_THREADS = 10 * 32;                   // producer, eight consumers, reducer
constexpr int KS_RLD = 20;                            // floats per token in a partial-sum buffer (16 rows + padding)

__device__ __forceinline__ void ks_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ks_mma_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void ks_cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ks_cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ks_cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ks_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void ks_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of this CTA's `local` address in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// Sixteen bytes into another CTA's shared memory, counted (as 16 transaction bytes) on an
// mbarrier of that CTA when they have landed: the sender neither waits nor fences.
__device__ __forceinline__ void st_async_f32x4(uint32_t addr, float a, float b, float c, float d,
                                               uint32_t remote_bar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::
          "r"(addr),
      "f"(a), "f"(b), "f"(c), "f"(d), "r"(remote_bar)
      : "memory");
}
// One arrival on an mbarrier of another CTA of the cluster, without ordering anything: for a
// signal whose only precondition the sender has
// already made sure of by other means.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar)
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
// The same test without any waiting (try_wait may suspend the thread for a while before it
// answers "not yet").
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, unsigned parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait on a barrier that other CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity, long long limit) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > limit) return false;
  }
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}

struct KsParams {
  U8Args a;
  int NS;        // stages in the ring
  int gps;       // scale groups per stage (1024 / block_size)
  int bs_shift;  // log2(block_size)
  int units;     // ceil(n / 16)
  int S;         // CTAs per cluster = k slices
  int Q;         // clusters in the grid
  int t0;        // first 128-wide k tile of this launch (a long k goes out as several launches)
  float beta;    // of this launch: the caller's for the first k range, 1 for the ranges after it
  long long wait_cycles;
  unsigned int* status;
};

// MT: 8-token column blocks (1 or 2).
template <int MT, bool HAS_ZERO, bool PDL>
__global__ void __launch_bounds__(KS_THREADS, 2)
    u8_ksplit_kernel(const __grid_constant__ CUtensorMap wmap, KsParams p) {
  constexpr int TOK = 8 * MT;
  constexpr int OPL = 16 * TOK / 32;  // outputs per lane of a summing or finishing warp
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const U8Args& a = p.a;
  const int S = p.S;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // same for every CTA of the launch
    if (threadIdx.x == 0) atomicOr(p.status, 16u);
    return;
  }
  uint8_t* ring = smem_raw;
  float* red = reinterpret_cast<float*>(ring + (size_t)p.NS * KS_STAGE_BYTES);  // [KS_NR][8][TOK][KS_RLD]
  float* inbox = red + (size_t)KS_NR * 8 * TOK * KS_RLD;                          // [KS_INB][S][16 * TOK]
  uint64_t* full = reinterpret_cast<uint64_t*>(inbox + (size_t)KS_INB * S * 16 * TOK);
  uint64_t* empty = full + KS_MAX_STAGES;
  uint64_t* inbox_full = empty + KS_MAX_STAGES;         // [KS_INB]: S partial results (as bytes) per use
  uint64_t* credit = inbox_full + KS_INB;               // [KS_MAX_S][KS_INB]: owner o took my push
  uint64_t* red_free = credit + KS_MAX_S * KS_INB;      // [KS_NR]: the reducer has read the buffer
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red_free + KS_NR);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = (int)cluster_rank();
  const int q = (int)blockIdx.x / S;  // this cluster
  const int groups = a.p >> p.bs_shift;
  // units of this cluster: q, q + Q, ...; unit number j of the cluster is finished by CTA j % S
  const int J = q < p.units ? (p.units - q + p.Q - 1) / p.Q : 0;

  if (tid == 0) {
    tma_prefetch_desc(&wmap);
    for (int s = 0; s < p.NS; ++s) {
      mbar_init(&full[s], 33);  // expect_tx arrival + one cp.async arrival per producer lane
      mbar_init(&empty[s], 8);  // the eight consumer warps
    }
    for (int i = 0; i < KS_INB; ++i) {
      // one arrival per use, by this CTA's reducer, which also states the bytes to expect: S
      // partial results.  The first use of every slot is announced here.
      mbar_init(&inbox_full[i], 1);
      if (rank + i * S < J) mbar_expect_tx(&inbox_full[i], (unsigned)(S * 16 * TOK * 4));
    }
    for (int i = 0; i < KS_MAX_S * KS_INB; ++i) mbar_init(&credit[i], 1);
    for (int i = 0; i < KS_NR; ++i) mbar_init(&red_free[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (PDL) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // no CTA may push into, or arrive on barriers of, a CTA that has not set them up yet
  cluster_sync_all();

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    // Weights, scales and zero points only: by contract not written by the kernel before, so
    // nothing here waits for it.
    bool ok = true;
    // (a slice that reaches past the end of k copies its scales in 4-byte pieces, each checked)
    const int tiles_total = a.p / 128;
    const int tile0 = p.t0 + rank * 8;  // this CTA's first tile
    const bool whole = tile0 + 8 <= tiles_total;
    const bool wide = whole && (groups % 8) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 15u) == 0 &&
                      (!HAS_ZERO || (reinterpret_cast<uintptr_t>(a.zeros) & 15u) == 0);
    const int per = wide ? 8 : 2;          // halves per copy
    const int per_row = p.gps / per;       // copies per row
    const int copies = 16 * per_row;       // per stage and table (16..128)
    int c_row[4], c_col[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = lane + 32 * u;
      c_row[u] = c < copies ? c / per_row : -1;
      c_col[u] = c < copies ? (c % per_row) * per : 0;
    }
    const int g0 = (tile0 * 128) >> p.bs_shift;
    int s = 0;
    unsigned par = 0;
    for (int j = 0; j < J && ok; ++j) {
      if (j >= p.NS && (!mbar_wait(&empty[s], par ^ 1u) || *abort_flag)) {
        ok = false;
        break;
      }
      const int n0 = (q + j * p.Q) * 16;
      uint8_t* stage = ring + (size_t)s * KS_STAGE_BYTES;
      if (lane == 0) {
        mbar_expect_tx(&full[s], (unsigned)KS_W_BYTES);
        tma_load_3d(stage, &wmap, 0, n0, tile0, &full[s]);  // tiles past the end of k arrive as zeros
      }
      __half* stab = reinterpret_cast<__half*>(stage + KS_W_BYTES);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (c_row[u] >= 0 && g0 + c_col[u] < groups) {
          const size_t src = (size_t)min(n0 + c_row[u], a.n - 1) * groups + g0 + c_col[u];
          __half* dst = stab + c_row[u] * p.gps + c_col[u];
          if (wide) {
            ks_cp_async_16(dst, a.scales + src);
            if (HAS_ZERO) ks_cp_async_16(dst + 16 * p.gps, a.zeros + src);
          } else {
            ks_cp_async_4(dst, a.scales + src);
            if (HAS_ZERO) ks_cp_async_4(dst + 16 * p.gps, a.zeros + src);
          }
        }
      }
      ks_cp_async_arrive(&full[s]);
      if (++s == p.NS) s = 0, par ^= 1u;
    }
    if (!ok) {
      *abort_flag = 1;
      if (lane == 0) atomicOr(p.status, 32u);
    }
    // drain: every issued stage has landed before the CTA may exit
    const int issued = ok ? J : 0;
    for (int jj = max(0, issued - p.NS); jj < issued; ++jj)
      if (!mbar_wait(&full[jj % p.NS], (unsigned)(jj / p.NS) & 1u) && lane == 0) atomicOr(p.status, 64u);
  } else if (warp <= 8) {
    // ------------------------------- consumers -------------------------------
    const int cw = warp - 1;  // the tile of every stage that this warp takes
    const int g = lane >> 2, t = lane & 3;
    const int pg = (g >> 1) + 4 * (g & 1);  // tile row read by MMA row g (conflict-free under the swizzle)
    const bool per_piece = p.bs_shift < 7;
    bool ok = true;
    if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- this warp's activations, for the whole launch: tokens g (and g + 8) of the 128 k of
    // its tile, 32 bytes per 64-wide piece, in the order the weight bytes are consumed in
    // (a tile past the end of k: zero activations, and its stages are not computed at all: the
    // scales were not copied for it)
    const bool tile_ok = p.t0 + rank * 8 + cw < a.p / 128;
    uint32_t xw[MT][2][8];
    {
      const size_t koff = (size_t)(p.t0 + rank * 8 + cw) * 256 + (size_t)t * 32;  // bytes into a row
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int tok = i * 8 + g;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
          if (tok < a.m && tile_ok) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.lhs) + (size_t)tok * a.p * 2 + koff + h * 128;
            v0 = *reinterpret_cast<const uint4*>(src);
            v1 = *reinterpret_cast<const uint4*>(src + 16);
          }
          xw[i][h][0] = v0.x, xw[i][h][1] = v0.y, xw[i][h][2] = v0.z, xw[i][h][3] = v0.w;
          xw[i][h][4] = v1.x, xw[i][h][5] = v1.y, xw[i][h][6] = v1.z, xw[i][h][7] = v1.w;
        }
      }
    }
    // their sums per 64-wide piece and token, by MMAs with an all-ones weight operand: the
    // accumulator then holds sum_k x[k][token] in every row, in the layout of the products
    float xs[2][MT][4];
    {
      constexpr uint32_t ONES = 0x3C003C00u;  // (1.0, 1.0)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            if (w == 0) ks_mma_z(xs[h][i], ONES, ONES, ONES, ONES, xw[i][h][0], xw[i][h][1]);
            else ks_mma(xs[h][i], ONES, ONES, ONES, ONES, xw[i][h][2 * w], xw[i][h][2 * w + 1]);
          }
    }

    int s = 0;
    unsigned par = 0;
    for (int j = 0; j < J; ++j) {
      float d[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) d[i][e] = 0.0f;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[s], par) && !*abort_flag);
      if (ok && tile_ok) {
        const uint8_t* stage = ring + (size_t)s * KS_STAGE_BYTES;
        const uint8_t* trow = stage + cw * KS_TILE_BYTES + pg * 128;
        const __half* stab = reinterpret_cast<const __half*>(stage + KS_W_BYTES);
        // two accumulator chains per token block (the parity of the k16 step)
        float acc[2][MT][4];
        auto compute_piece = [&](const uint8_t* wrow, auto piece_tag, auto fresh_tag) {
          constexpr int H = decltype(piece_tag)::value;
          constexpr bool FRESH = decltype(fresh_tag)::value;  // the chains start at zero
          const uint4 qa = *reinterpret_cast<const uint4*>(wrow);
          const uint4 qb = *reinterpret_cast<const uint4*>(wrow + 8 * 128);
          const uint32_t wwa[4] = {qa.x, qa.y, qa.z, qa.w};
          const uint32_t wwb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const uint32_t A0 = prmt(wwa[w], 0x64646464u, 0x4140u), A2 = prmt(wwa[w], 0x64646464u, 0x4342u);
            const uint32_t A1 = prmt(wwb[w], 0x64646464u, 0x4140u), A3 = prmt(wwb[w], 0x64646464u, 0x4342u);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              const uint32_t b0 = xw[i][H][2 * w], b1 = xw[i][H][2 * w + 1];
              if (FRESH && w < 2) ks_mma_z(acc[w & 1][i], A0, A1, A2, A3, b0, b1);
              else ks_mma(acc[w & 1][i], A0, A1, A2, A3, b0, b1);
            }
          }
        };
        // d += s * ((acc0 + acc1) - (1024 + z) * sum x) for scale group `gi` of the stage, whose
        // activation sums are those of pieces h0..h1
        auto correct = [&](int gi, int h0, int h1) {
          const float sa = __half2float(stab[pg * p.gps + gi]);
          const float sb = __half2float(stab[(pg + 8) * p.gps + gi]);
          float ca = 1151.5f, cb = 1151.5f;
          if (HAS_ZERO) {
            ca = 1024.0f + __half2float(stab[16 * p.gps + pg * p.gps + gi]);
            cb = 1024.0f + __half2float(stab[16 * p.gps + (pg + 8) * p.gps + gi]);
          }
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            float2 xv = make_float2(xs[h0][i][0], xs[h0][i][1]);
            if (h0 != h1) xv.x += xs[h1][i][0], xv.y += xs[h1][i][1];
            d[i][0] = fmaf(sa, fmaf(-ca, xv.x, acc[0][i][0] + acc[1][i][0]), d[i][0]);
            d[i][1] = fmaf(sa, fmaf(-ca, xv.y, acc[0][i][1] + acc[1][i][1]), d[i][1]);
            d[i][2] = fmaf(sb, fmaf(-cb, xv.x, acc[0][i][2] + acc[1][i][2]), d[i][2]);
            d[i][3] = fmaf(sb, fmaf(-cb, xv.y, acc[0][i][3] + acc[1][i][3]), d[i][3]);
          }
        };
        // piece h: the 16 bytes at logical offset (t + 4h) * 16 of the 128-byte row
        using T = std::true_type;
        using F = std::false_type;
        compute_piece(trow + ((t ^ pg) * 16), std::integral_constant<int, 0>{}, T{});
        if (per_piece) {
          correct(2 * cw, 0, 0);  // (group indices are relative to the stage)
          compute_piece(trow + (((t + 4) ^ pg) * 16), std::integral_constant<int, 1>{}, T{});
          correct(2 * cw + 1, 1, 1);
        } else {
          compute_piece(trow + (((t + 4) ^ pg) * 16), std::integral_constant<int, 1>{}, F{});
          correct(cw, 0, 1);
        }
      }
      // the stage is read: it may be refilled (also on failure, so that the producer can finish)
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      // ---- the partial sums go into buffer j % KS_NR, once the reducer has read what unit
      // j - KS_NR left there: [token][row] with rows padded to 20 floats (conflict-free stores,
      // 16-byte loads for the reducing warp); then the warp moves on
      const int b = j % KS_NR;
      if (j >= KS_NR && ok)
        ok = __all_sync(0xffffffffu, mbar_wait(&red_free[b], (unsigned)(j / KS_NR - 1) & 1u) && !*abort_flag);
      float* rw = red + ((size_t)b * 8 + cw) * TOK * KS_RLD;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        rw[(i * 8 + 2 * t) * KS_RLD + pg] = d[i][0];
        rw[(i * 8 + 2 * t + 1) * KS_RLD + pg] = d[i][1];
        rw[(i * 8 + 2 * t) * KS_RLD + pg + 8] = d[i][2];
        rw[(i * 8 + 2 * t + 1) * KS_RLD + pg + 8] = d[i][3];
      }
      __threadfence_block();  // the partial sums are visible before the arrival is counted
      __syncwarp();
      ks_bar_arrive(1 + b, 9 * 32);
      if (++s == p.NS) s = 0, par ^= 1u;
    }
    if (!ok && lane == 0) atomicOr(p.status, 1u);
  } else {
    // ------------------------------- reducer -------------------------------
    // Per unit: add the eight warps' partial sums and push the result to the unit's owner.  For
    // the units this CTA owns (j = rank, rank + S, ...): add the S pushed results in rank order,
    // add beta * old, write 16 columns for every token; done as soon as a unit's pushes are all
    // in, without holding up the units after it.
    if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
    bool ok = true;
    const bool vec = (a.n % 8) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
    // lane's outputs of a unit: token tok, rows row0 .. row0 + OPL - 1
    const int o0 = lane * OPL, row0 = o0 & 15, tok = o0 >> 4;
    const bool tok_ok = tok < a.m;
    unsigned short old[OPL];
    auto load_old = [&](int j) {  // requested one unit ahead, so that the finishing does not wait for it
#pragma unroll
      for (int e = 0; e < OPL; ++e) old[e] = 0;
      if (j >= J || !tok_ok) return;
      const int n0 = (q + j * p.Q) * 16;
      const __half* optr = a.out + (size_t)tok * a.n + n0 + row0;
      if (vec && n0 + 16 <= a.n) {
        if (OPL == 8) {
          const uint4 u = *reinterpret_cast<const uint4*>(optr);
          const unsigned short* h = reinterpret_cast<const unsigned short*>(&u);
#pragma unroll
          for (int e = 0; e < OPL; ++e) old[e] = h[e];
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(optr);
          const unsigned short* h = reinterpret_cast<const unsigned short*>(&u);
#pragma unroll
          for (int e = 0; e < OPL; ++e) old[e] = h[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < OPL; ++e)
          if (n0 + row0 + e < a.n) old[e] = reinterpret_cast<const unsigned short*>(optr)[e];
      }
    };
    // Finishes owned unit j if its pushes are in (or waits for them when `blocking`).
    auto finish = [&](int j, bool blocking) -> bool {
      const int k = j / S, slot = k % KS_INB, use = k / KS_INB;
      if (*abort_flag) ok = false;  // another warp gave up: no more waits, no more stores
      if (ok) {
        if (!blocking) {
          if (!__all_sync(0xffffffffu, mbar_test_cluster(&inbox_full[slot], (unsigned)use & 1u)))
            return false;
        } else if (!__all_sync(0xffffffffu,
                               mbar_wait_cluster(&inbox_full[slot], (unsigned)use & 1u, p.wait_cycles))) {
          ok = false;
          *abort_flag = 1;
          if (lane == 0) atomicOr(p.status, 2048u);
        }
      }
      float v[OPL];
#pragma unroll
      for (int e = 0; e < OPL; ++e) v[e] = 0.0f;
      for (int r = 0; r < S; ++r) {
        const float* src = inbox + ((size_t)slot * S + r) * 16 * TOK + lane * OPL;
#pragma unroll
        for (int e = 0; e < OPL; e += 4) {
          const float4 f = *reinterpret_cast<const float4*>(src + e);
          v[e] += f.x, v[e + 1] += f.y, v[e + 2] += f.z, v[e + 3] += f.w;
        }
      }
      // If the slot has another use: announce it, then tell every CTA of the cluster that it may
      // push again (every such arrival is waited for by its receiver before that push, so none
      // can reach a CTA that has already left).  The arrival carries no fence (a release at
      // cluster scope here cost 6-9 % of the whole launch); what it must follow is only this
      // warp's own reads of the slot, and it does: its address is made to depend on the sums of
      // everything read, so it cannot issue before those loads have returned their data.
      __syncwarp();
      if (j + S * KS_INB < J) {
        if (lane == 0) mbar_expect_tx(&inbox_full[slot], (unsigned)(S * 16 * TOK * 4));
        __syncwarp();
        float all = 0.0f;
#pragma unroll
        for (int e = 0; e < OPL; ++e) all += v[e];
        all += __shfl_xor_sync(0xffffffffu, all, 16);
        all += __shfl_xor_sync(0xffffffffu, all, 8);
        all += __shfl_xor_sync(0xffffffffu, all, 4);
        all += __shfl_xor_sync(0xffffffffu, all, 2);
        all += __shfl_xor_sync(0xffffffffu, all, 1);
        uint32_t nothing;
        asm volatile("and.b32 %0, %1, 0;" : "=r"(nothing) : "r"(__float_as_uint(all)));
        if (lane < S)
          mbar_arrive_cluster_relaxed(
              map_to_rank(smem_u32(&credit[rank * KS_INB + slot]), (uint32_t)lane) + nothing);
      }
      const int n0 = (q + j * p.Q) * 16;
      __half* optr = a.out + (size_t)tok * a.n + n0 + row0;
      if (tok_ok && ok) {
        unsigned short res[OPL];
#pragma unroll
        for (int e = 0; e < OPL; ++e)
          res[e] = __half_as_ushort(
              __float2half_rn(fmaf(p.beta, __half2float(__ushort_as_half(old[e])), v[e])));
        if (vec && n0 + 16 <= a.n) {
          if (OPL == 8) *reinterpret_cast<uint4*>(optr) = *reinterpret_cast<const uint4*>(res);
          else *reinterpret_cast<uint2*>(optr) = *reinterpret_cast<const uint2*>(res);
        } else {
#pragma unroll
          for (int e = 0; e < OPL; ++e)
            if (n0 + row0 + e < a.n) reinterpret_cast<unsigned short*>(optr)[e] = res[e];
        }
      }
      load_old(j + S);
      return true;
    };
    int fin_j = rank;  // the next owned unit to finish
    load_old(fin_j);
    for (int j = 0; j < J; ++j) {
      const int b = j % KS_NR;
      ks_bar_sync(1 + b, 9 * 32);
      float v[OPL];
#pragma unroll
      for (int e = 0; e < OPL; ++e) v[e] = 0.0f;
      const float* rb = red + (size_t)b * 8 * TOK * KS_RLD + tok * KS_RLD + row0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
#pragma unroll
        for (int e = 0; e < OPL; e += 4) {
          const float4 f = *reinterpret_cast<const float4*>(rb + (size_t)w * TOK * KS_RLD + e);
          v[e] += f.x, v[e + 1] += f.y, v[e + 2] += f.z, v[e + 3] += f.w;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_free[b]);  // the buffer is read: unit j + KS_NR may use it
      const int owner = j % S, k = j / S, slot = k % KS_INB, use = k / KS_INB;
      // Own units that the cluster may be waiting for (their slots are due for reuse) first:
      // every owner does this before it waits for a slot itself, so the oldest unfinished unit
      // of the cluster always gets finished and nobody waits in a circle.
      while (fin_j <= j - S * KS_INB) {
        finish(fin_j, true);
        fin_j += S;
      }
      // the owner has taken what was pushed into this slot KS_INB of its units ago
      if (*abort_flag) ok = false;
      if (use > 0 && ok) {
        if (!__all_sync(0xffffffffu,
                        mbar_wait_cluster(&credit[owner * KS_INB + slot], (unsigned)(use - 1) & 1u, p.wait_cycles))) {
          ok = false;
          *abort_flag = 1;
          if (lane == 0) atomicOr(p.status, 1024u);
        }
      }
      const uint32_t dst = map_to_rank(
          smem_u32(inbox + ((size_t)slot * S + rank) * 16 * TOK + lane * OPL), (uint32_t)owner);
      const uint32_t dbar = map_to_rank(smem_u32(&inbox_full[slot]), (uint32_t)owner);
#pragma unroll
      for (int e = 0; e < OPL; e += 4) st_async_f32x4(dst + e * 4, v[e], v[e + 1], v[e + 2], v[e + 3], dbar);
      // owned units whose pushes happen to be complete
      while (fin_j <= j && finish(fin_j, false)) fin_j += S;
    }
    for (; fin_j < J; fin_j += S) finish(fin_j, true);
    if (!ok && lane == 0) atomicOr(p.status, 1u);
  }
  // A CTA may leave when its own work is done: everything pushed into it has been waited for
  // by its reducer, and what it pushed is waited for by the receiver before that one leaves.
}

struct KsPlan {
  int S, Q, NS;
  size_t smem;
};

// Plan for the k range of `kc` elements (at most 8192) of a product; the range may end inside
// a CTA's slice.
bool plan_ksplit(const adr_ctx* ctx, const U8Args& a, int kc, KsPlan& pl) {
  if (a.m < 1 || a.m > 16 || a.n < 16) return false;
  if (a.block_size != 64 && a.block_size != 128) return false;
  if (a.p % 128 != 0 || a.p < 2048 || ((a.p / a.block_size) & 1)) return false;  // 4-byte scale copies
  if (kc < 128 || kc > 1024 * KS_MAX_S) return false;
  if (a.norm_w != nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(a.rhs) & 15u) || (reinterpret_cast<uintptr_t>(a.lhs) & 15u) ||
      (reinterpret_cast<uintptr_t>(a.scales) & 3u) ||
      (a.zeros && (reinterpret_cast<uintptr_t>(a.zeros) & 3u)))
    return false;
  if (!ctx->encode_tiled_fn) return false;
  const int tok = a.m > 8 ? 16 : 8;
  pl.S = (kc + 1023) / 1024;
  pl.Q = 0;  // chosen by the launcher, which knows how many clusters the GPU holds at once
  const size_t half = 113 * 1024;
  const size_t per_stage = KS_STAGE_BYTES;
  const size_t fixed = (size_t)KS_NR * 8 * tok * KS_RLD * 4 + (size_t)KS_INB * pl.S * 16 * tok * 4 +
                       (2 * KS_MAX_STAGES + KS_INB + KS_MAX_S * KS_INB + KS_NR + 1) * 8;
  int ns = fixed < half ? (int)((half - fixed) / per_stage) : 0;
  ns = std::min(ns, KS_MAX_STAGES);
  const int tune_ns = ctx->tune_ks_stages.load();
  if (tune_ns > 0) ns = std::min(tune_ns, KS_MAX_STAGES);
  if (ns < 2) return false;
  pl.NS = ns;
  pl.smem = (size_t)ns * per_stage + fixed;
  return pl.smem <= 226 * 1024;
}

template <int MT, bool Z, bool PDL>
int launch_ksplit_t(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const KsPlan& pl, int t0,
                    float beta) {
  auto kfn = u8_ksplit_kernel<MT, Z, PDL>;
  if (int rc0 = opt_in_smem(ctx, kfn, 226 * 1024); rc0 != ADR_OK) return rc0;
  // weights as (k within tile, row, k-tile): a box of 128 x 16 x 8 lands as eight tiles of
  // [16 rows][128 bytes], each swizzled by its own row index
  CUtensorMap wmap;
  const uint64_t dims[3] = {128u, (uint64_t)a.n, (uint64_t)(a.p / 128)};
  const uint64_t strides[2] = {(uint64_t)a.p, 128u};
  const uint32_t box[3] = {128u, 16u, 8u};
  int rc = tma_get(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.rhs, dims, strides, box,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != ADR_OK) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(KS_THREADS, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // As many clusters as the GPU holds at the same time (a cluster needs its S CTAs on one GPC, so
  // this is less than SMs x 2 / S: 71 clusters of 4, 33 of 8 on a B200), asked once per
  // configuration, less one: measured, a grid of exactly the number the runtime names runs a
  // third longer with clusters of 8 (32 are fine, 33 are not), and a grid of more than fit runs
  // in two waves.  The units are then spread evenly over as few rounds as that allows.
  int qmax = ctx->tune_ks_clusters.load();
  if (qmax <= 0) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, size_t>, int> known;
    const auto key = std::make_tuple((const void*)kfn, ctx->device, pl.S, pl.smem);
    std::lock_guard<std::mutex> lock(mu);
    auto it = known.find(key);
    if (it == known.end()) {
      int nc = 0;
      cfg.gridDim = dim3(pl.S * 64, 1, 1);
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&nc, kfn, &cfg) != cudaSuccess || nc < 1) {
        cudaGetLastError();
        nc = std::max(1, (ctx->sm_count > 0 ? ctx->sm_count : 148) / pl.S);
      }
      it = known.emplace(key, std::max(1, nc - 1)).first;
    }
    qmax = it->second;
    // Behind a small kernel of this library that started early (a norm, an elementwise op, the
    // all-reduce) some of its CTAs still hold a slot each when this launch's clusters are
    // placed, and a cluster that finds no room runs as a second wave.  Leave room for about
    // sixteen such CTAs then (tunable "ks_slack", default on; measured in a LLaMA-7B decode
    // step: 4.37 -> 3.99 ms at batch 16, 3.14 -> 2.70 ms at batch 5; in chains of products
    // alone the full grid is 10 % quicker on some shapes, so it stays there).  Capping the kernel at 88
    // registers so that such a CTA fits beside two of this kernel's was tried instead: 7-10 %
    // slower in chains of products, and no cure.
    if (PDL && ctx->tune_ks_slack.load() != 0 && ctx->small_before.load() != 0)
      qmax = std::max(1, qmax - (16 + pl.S - 1) / pl.S);
  }
  ctx->small_before = 0;
  const int units = (a.n + 15) / 16;
  const int rounds = (units + qmax - 1) / qmax;
  const int Q = (units + rounds - 1) / rounds;
  KsParams p;
  p.a = a;
  p.NS = pl.NS;
  p.gps = 1024 / a.block_size;
  p.bs_shift = a.block_size == 64 ? 6 : 7;
  p.units = (a.n + 15) / 16;
  p.S = pl.S;
  p.t0 = t0;
  p.beta = beta;
  p.Q = Q;
  p.wait_cycles = peer_wait_cycles(ctx);
  p.status = ctx->d_status;
  cfg.gridDim = dim3(Q * pl.S, 1, 1);
  cfg.numAttrs = (PDL && ctx->tune_ks_pdl.load()) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, wmap, p);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  note_filling_launch(ctx, stream, 1);  // two CTAs per SM: a half-SM launch must not start as they drain
  return after_launch(ctx);
}

}  // namespace

// A cluster covers at most 8192 of k, so a longer k goes out as several launches over
// consecutive k ranges, the later ones adding to what the earlier ones wrote (beta = 1; the
// output passes through fp16 between them).  The ranges are cut evenly in units of 1024.
namespace {
int ksplit_ranges(int p) { return (p + 1024 * KS_MAX_S - 1) / (1024 * KS_MAX_S); }
int ksplit_range_len(int p) {
  const int slices = (p + 1023) / 1024, r = ksplit_ranges(p);
  return ((slices + r - 1) / r) * 1024;
}
}  // namespace

bool u8_ksplit_supports(const adr_ctx* ctx, const U8Args& a) {
  if (a.p < 2048) return false;
  KsPlan pl;
  const int len = ksplit_range_len(a.p);
  for (int k0 = 0; k0 < a.p; k0 += len)
    if (!plan_ksplit(ctx, a, std::min(len, a.p - k0), pl)) return false;
  return true;
}

int launch_u8_ksplit(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  if (!u8_ksplit_supports(ctx, a)) return ADR_ERR_SHAPE;
  const bool z = a.zeros != nullptr, two = a.m > 8, pdl = ctx->tune_pdl != 0;
  const int len = ksplit_range_len(a.p);
  for (int k0 = 0; k0 < a.p; k0 += len) {
    KsPlan pl;
    if (!plan_ksplit(ctx, a, std::min(len, a.p - k0), pl)) return ADR_ERR_SHAPE;
    const int t0 = k0 / 128;
    const float beta = k0 == 0 ? a.beta : 1.0f;
    int rc;
    if (two)
      rc = z ? (pdl ? launch_ksplit_t<2, true, true>(ctx, stream, a, pl, t0, beta)
                    : launch_ksplit_t<2, true, false>(ctx, stream, a, pl, t0, beta))
             : (pdl ? launch_ksplit_t<2, false, true>(ctx, stream, a, pl, t0, beta)
                    : launch_ksplit_t<2, false, false>(ctx, stream, a, pl, t0, beta));
    else
      rc = z ? (pdl ? launch_ksplit_t<1, true, true>(ctx, stream, a, pl, t0, beta)
                    : launch_ksplit_t<1, true, false>(ctx, stream, a, pl, t0, beta))
             : (pdl ? launch_ksplit_t<1, false, true>(ctx, stream, a, pl, t0, beta)
                    : launch_ksplit_t<1, false, false>(ctx, stream, a, pl, t0, beta));
    if (rc != ADR_OK) return rc;
  }
  return ADR_OK;
}

}  // namespace adr
