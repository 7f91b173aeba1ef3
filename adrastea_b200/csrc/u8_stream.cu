// u8-weight decode GEMV/GEMM, streaming form (m <= 16):
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// (replaces adrastea_kernels/cpp/matmul_nt_fp16u8.cu:4-24 and
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83 for decode shapes).
//
// The shape is HBM-bound and small (17-45 MB of weights, 2.6-7 us at the HBM
// roof), so the kernel is built to have every byte it will read in flight
// from its first instructions:
//   * a CTA owns R weight rows (16, 32 or 64) and one k-slice of them.  With
//     S = 1 the slice is all of k.  With S > 1 a thread-block cluster of S CTAs
//     covers k for those rows (split-k without scratch memory: the partial sums
//     are exchanged through distributed shared memory and added in rank order,
//     so the result is deterministic);
//   * at start one thread requests the whole slice as TMA tiles of R rows x
//     128 bytes (128-byte swizzle), one mbarrier per tile, and the matching
//     activation slice with one bulk copy per token, so compute starts when
//     the first tile lands;
//   * eight warps consume: the dequantised fp16 weights (u8_common.cuh,
//     bit-exact) feed mma.sync.m16n8k16 from registers with the weights as
//     the 16-row operand and the tokens as the 8-column operand; the shared
//     loads of the next 16-byte piece are issued before the current piece is
//     computed;
//   * MMA row g of a 16-row set reads tile row (g>>1) + 4*(g&1): with the
//     128-byte swizzle the two rows a quarter warp touches then fall in
//     different 64-byte halves, so every 128-bit shared load is conflict-free;
//     activation rows are padded to an odd number of 16-byte units.
#include <algorithm>
#include <cmath>
#include <type_traits>

#include "tma.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int MAX_TILES = 96;  // 128-byte tiles per k-slice (12 KB of k)

// Not volatile: the compiler may move it among the surrounding arithmetic.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with a zero accumulator on input (starts a chain without clearing registers).
__device__ __forceinline__ void mma_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

template <int MT, bool HAS_ZERO>
struct Piece {  // 16 bytes of two weight rows and their scale-table entries; fetched one ahead
  uint4 qa, qb;
  uint2 sa, sb;
  int xoff;
};

// MT: 8-token column blocks (1: m <= 8, 2: m <= 16).  R: weight rows per CTA.  NW: warps per CTA.
// DEFER: the scale and the zero point are applied to fp32 partial sums, once per scale group
// (or per 128-byte tile when a group is longer), instead of to every weight:
//   sum_k (q_k - z) s x_k = s * (sum_k (1024 + q_k) x_k  -  (1024 + z) * sum_k x_k)
// The operand 1024 + q_k is the byte under the fp16 exponent 0x64, one PRMT per pair and
// exact; sum_k x_k comes from a second MMA whose weight operand is all ones, which lands it
// in the accumulator layout the correction needs.  The products are exact in fp32 and the
// weights are not rounded to fp16 first, which is the arithmetic of matmul_nt_fp16u8.cu:13-23
// rather than that of the WMMA kernel; the dequantise-multiply work per weight pair drops from
// three instructions to one.  Needs block_size >= 64 (a 64-wide piece must lie in one group).
template <int MT, int R, int NW, bool HAS_ZERO, bool PDL, bool DEFER>
__global__ void __launch_bounds__(NW * 32, MT == 1 ? 3 : 2)
    u8_stream_kernel(const __grid_constant__ CUtensorMap wmap, U8Args a, int S, int XS, int NG,
                     int bs_shift, unsigned int* status) {
  constexpr int RS = R / 16;  // 16-row sets
  constexpr int NT = NW * 32;  // threads per CTA
  constexpr int KP = NW / RS;  // k-phases: warps sharing a row set interleave over tiles
  constexpr int TOK = 8 * MT;
  constexpr int TILE_BYTES = R * 128;

  // Shared memory, tightly packed so that three CTAs fit an SM at k = 4096, m = 1 (which
  // leaves room for the next launch's CTAs under programmatic dependent launch):
  //   [tiles: nt * R * 128] [activations: m * XS] [scale table] [mbarriers: nt + 1]
  // The swizzled tiles need a 1024-byte aligned base.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* Wsm = smem_raw;
  if ((smem_u32(Wsm) & 1023u) != 0) {  // same for every CTA of the launch
    if (threadIdx.x == 0) atomicOr(status, 16u);
    return;
  }

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int pg = (g >> 1) + 4 * (g & 1);  // tile row read by MMA row g
  const int rs = warp % RS, kp = warp / RS;
  const int rank = blockIdx.x;  // position in the cluster == k-slice index
  const int n0 = blockIdx.y * R;
  const int groups = a.p >> bs_shift;

  const int ntiles = a.p / 128;
  const int tb = (int)((long long)rank * ntiles / S);
  const int te = (int)((long long)(rank + 1) * ntiles / S);
  const int nt = te - tb;
  const int k0 = tb * 128;
  uint8_t* Xsm = Wsm + (size_t)nt * TILE_BYTES;

  // Request order matters: everything this CTA reads is requested at once, and requests are
  // served roughly in issue order, so the small operands that gate the first MMA (scales,
  // zero points, activations) go out before the weight tiles.
  // Scale table in shared memory, one 8-byte entry per (row, group - g_lo):
  //   (s, s) as packed halves, plus (z, z) when zero points are given.
  // (DEFER: the scale as a float, plus 1024 + zero point when zero points are given)
  using Entry = std::conditional_t<DEFER, std::conditional_t<HAS_ZERO, float2, float>,
                                   std::conditional_t<HAS_ZERO, uint2, uint32_t>>;
  Entry* Ssm = reinterpret_cast<Entry*>(Xsm + (size_t)a.m * XS);
  // mbarriers behind the table: [0, nt) one per tile, [nt] the activations
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ssm + (size_t)R * NG);
  uint64_t* xbar = bars + nt;
  const int g_lo = k0 >> bs_shift;
  const int ng = ((k0 + nt * 128 - 1) >> bs_shift) - g_lo + 1;
  constexpr int EARLY = 4;  // table entries per thread fetched into registers first
  __half es[EARLY], ez[EARLY];
#pragma unroll
  for (int u = 0; u < EARLY; ++u) {
    const int e = tid + u * NT;
    if (e < R * ng) {
      const int row = e / ng, gi = e - row * ng;
      const size_t src = (size_t)min(n0 + row, a.n - 1) * groups + g_lo + gi;
      es[u] = a.scales[src];
      if (HAS_ZERO) ez[u] = a.zeros[src];
    }
  }
  // Warp 0 sets up the barriers and issues the copies; the other warps meet the barriers
  // only after the __syncthreads below.  Under programmatic dependent launch this kernel
  // may start while the previous kernel of the stream is still running: the weight matrix,
  // its scales and zero points are by contract not written by that kernel and are requested
  // at once; the activations and the output are touched only after griddepcontrol.wait.
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&wmap);
      for (int i = 0; i < nt; ++i) mbar_init(&bars[i], 1);
      mbar_init(xbar, 1);
      mbar_fence_init();
      mbar_expect_tx(&xbar[0], (unsigned)(a.m * nt * 256));
    }
    __syncwarp();
    if (!PDL && lane < a.m)
      bulk_g2s(Xsm + (size_t)lane * XS, a.lhs + (size_t)lane * a.p + k0, (unsigned)(nt * 256),
               &xbar[0]);
    if (lane == 0) {
      for (int i = 0; i < nt; ++i) {
        mbar_expect_tx(&bars[i], TILE_BYTES);
        tma_load_2d(Wsm + (size_t)i * TILE_BYTES, &wmap, k0 + i * 128, n0, &bars[i]);
      }
    }
  }
  if (PDL) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp == 0 && lane < a.m)
      bulk_g2s(Xsm + (size_t)lane * XS, a.lhs + (size_t)lane * a.p + k0, (unsigned)(nt * 256),
               &xbar[0]);
  }
  // The packed-half dequantisation is exact for a scale whose half is exact (biased
  // exponent >= 2, finite) and only without zero points; one scale outside that range
  // sends the whole CTA down the general path.
  auto table_entry = [&](__half s, __half z, bool& fast) {
    if constexpr (DEFER) {
      if constexpr (HAS_ZERO) {
        return make_float2(__half2float(s), 1024.0f + __half2float(z));
      } else {
        return __half2float(s);
      }
    } else {
      const unsigned short bits = __half_as_ushort(s) & 0x7FFFu;
      fast = fast && !HAS_ZERO && bits >= 0x0800u && bits < 0x7C00u;
      const __half2 s2 = __half2half2(s);
      if constexpr (HAS_ZERO) {
        return make_uint2(half2_as_u32(s2), half2_as_u32(__half2half2(z)));
      } else {
        return half2_as_u32(s2);
      }
    }
  };
  bool fast = true;
#pragma unroll
  for (int u = 0; u < EARLY; ++u) {
    const int e = tid + u * NT;
    if (e < R * ng) {
      const int row = e / ng, gi = e - row * ng;
      Ssm[row * NG + gi] = table_entry(es[u], HAS_ZERO ? ez[u] : __half(), fast);
    }
  }
  for (int e = tid + EARLY * NT; e < R * ng; e += NT) {
    const int row = e / ng, gi = e - row * ng;
    const size_t src = (size_t)min(n0 + row, a.n - 1) * groups + g_lo + gi;
    Ssm[row * NG + gi] = table_entry(a.scales[src], HAS_ZERO ? a.zeros[src] : __half(), fast);
  }
  const bool all_fast = __syncthreads_and(fast) != 0;

  // two accumulator sets for one token block, used alternately, halve the MMA dependency chain
  float d[MT][4], d2[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) d2[j] = 0.0f;
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) d[i][j] = 0.0f;

  const uint8_t* xa = Xsm + (size_t)g * XS;
  const uint8_t* xb = Xsm + (size_t)(g + 8) * XS;
  const bool x0_ok = g < a.m;
  const bool x1_ok = MT > 1 && (g + 8) < a.m;
  const int row_a = rs * 16 + pg;  // tile row of MMA row g; row g+8 is 8 rows further
  const uint8_t* w_a = Wsm + row_a * 128;
  const Entry* s_a = Ssm + (size_t)row_a * NG - g_lo;
  const Entry* s_b = s_a + (size_t)8 * NG;
  // a table entry as (packed scale, packed scale/2 or packed zero point)
  auto expand = [&](Entry e) {
    if constexpr (DEFER) {
      return make_uint2(0u, 0u);  // scales are read at the correction step instead
    } else if constexpr (HAS_ZERO) {
      return e;
    } else {
      return make_uint2(e, half2_as_u32(__hmul2(u32_as_half2(e), __float2half2_rn(0.5f))));
    }
  };
  const int kbase = k0 + t * 16;

  using P = Piece<MT, HAS_ZERO>;
  // Piece h (0/1) of tile ti: the 16 bytes at logical offset (t + 4h) * 16 of the 128-byte
  // row, found at ((t + 4h) ^ row) * 16 under the swizzle.
  auto load_piece = [&](int ti, int h, P& pc) {
    const int j = t + 4 * h;
    const uint8_t* tile = w_a + (size_t)ti * TILE_BYTES + ((j ^ pg) * 16);
    pc.qa = *reinterpret_cast<const uint4*>(tile);
    pc.qb = *reinterpret_cast<const uint4*>(tile + 8 * 128);
    pc.xoff = ti * 256 + j * 32;
    if constexpr (!DEFER) {
      const int grp = (kbase + ti * 128 + h * 64) >> bs_shift;
      pc.sa = expand(s_a[grp]);
      pc.sb = expand(s_b[grp]);
    }
  };
  auto compute_piece = [&](const P& pc, auto fast_tag) {
    constexpr bool FAST = decltype(fast_tag)::value;
    const uint32_t wwa[4] = {pc.qa.x, pc.qa.y, pc.qa.z, pc.qa.w};
    const uint32_t wwb[4] = {pc.qb.x, pc.qb.y, pc.qb.z, pc.qb.w};
    // the activations are read here; their latency hides behind the dequantisation
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    const uint4 v0 = x0_ok ? *reinterpret_cast<const uint4*>(xa + pc.xoff) : zero4;
    const uint4 v1 = x0_ok ? *reinterpret_cast<const uint4*>(xa + pc.xoff + 16) : zero4;
    uint4 v2 = zero4, v3 = zero4;
    if (MT > 1 && x1_ok) {
      v2 = *reinterpret_cast<const uint4*>(xb + pc.xoff);
      v3 = *reinterpret_cast<const uint4*>(xb + pc.xoff + 16);
    }
    const uint32_t xw0[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    const uint32_t xw1[8] = {v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w};
    ScalePair spa, spb;
    if (!FAST) {
      spa = make_scale(__low2half(u32_as_half2(pc.sa.x)), HAS_ZERO, __low2half(u32_as_half2(pc.sa.y)));
      spb = make_scale(__low2half(u32_as_half2(pc.sb.x)), HAS_ZERO, __low2half(u32_as_half2(pc.sb.y)));
    }
    const __half2 k1152 = u32_as_half2(0x64806480u);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      __half2 a_lo, a_hi, b_lo, b_hi;
      if (FAST) {
        // (0x6400 | q) - 1152 = q - 128 exactly; fma(q - 128, s, s/2) rounds (q - 127.5) s once
        a_lo = __hfma2(__hsub2(u32_as_half2(prmt(wwa[w], 0x64646464u, 0x4140u)), k1152),
                       u32_as_half2(pc.sa.x), u32_as_half2(pc.sa.y));
        a_hi = __hfma2(__hsub2(u32_as_half2(prmt(wwa[w], 0x64646464u, 0x4342u)), k1152),
                       u32_as_half2(pc.sa.x), u32_as_half2(pc.sa.y));
        b_lo = __hfma2(__hsub2(u32_as_half2(prmt(wwb[w], 0x64646464u, 0x4140u)), k1152),
                       u32_as_half2(pc.sb.x), u32_as_half2(pc.sb.y));
        b_hi = __hfma2(__hsub2(u32_as_half2(prmt(wwb[w], 0x64646464u, 0x4342u)), k1152),
                       u32_as_half2(pc.sb.x), u32_as_half2(pc.sb.y));
      } else {
        dequant4(wwa[w], spa, a_lo, a_hi);
        dequant4(wwb[w], spb, b_lo, b_hi);
      }
      const uint32_t A0 = half2_as_u32(a_lo), A2 = half2_as_u32(a_hi);
      const uint32_t A1 = half2_as_u32(b_lo), A3 = half2_as_u32(b_hi);
      mma_16816((w & 1) ? d2 : d[0], A0, A1, A2, A3, xw0[2 * w], xw0[2 * w + 1]);
      if (MT > 1) mma_16816(d[MT - 1], A0, A1, A2, A3, xw1[2 * w], xw1[2 * w + 1]);
    }
  };

  // ---- deferred-scale form: per-group accumulators, corrected and scaled in fp32 ----
  float acc0[MT][4], acc1[MT][4], xs[MT][4];
  auto compute_piece_defer = [&](const P& pc, auto first_tag) {
    constexpr bool FIRST = decltype(first_tag)::value;
    const uint32_t wwa[4] = {pc.qa.x, pc.qa.y, pc.qa.z, pc.qa.w};
    const uint32_t wwb[4] = {pc.qb.x, pc.qb.y, pc.qb.z, pc.qb.w};
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    const uint4 v0 = x0_ok ? *reinterpret_cast<const uint4*>(xa + pc.xoff) : zero4;
    const uint4 v1 = x0_ok ? *reinterpret_cast<const uint4*>(xa + pc.xoff + 16) : zero4;
    uint4 v2 = zero4, v3 = zero4;
    if (MT > 1 && x1_ok) {
      v2 = *reinterpret_cast<const uint4*>(xb + pc.xoff);
      v3 = *reinterpret_cast<const uint4*>(xb + pc.xoff + 16);
    }
    const uint32_t xw[2][8] = {{v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w},
                               {v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w}};
    constexpr uint32_t ONES = 0x3C003C00u;  // (1.0, 1.0)
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      // byte pairs (0,1) and (2,3) of each word under the exponent of 1024: 1024 + q, exact
      const uint32_t A0 = prmt(wwa[w], 0x64646464u, 0x4140u), A2 = prmt(wwa[w], 0x64646464u, 0x4342u);
      const uint32_t A1 = prmt(wwb[w], 0x64646464u, 0x4140u), A3 = prmt(wwb[w], 0x64646464u, 0x4342u);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const uint32_t b0 = xw[i][2 * w], b1 = xw[i][2 * w + 1];
        if (FIRST && w < 2) mma_16816_z((w & 1) ? acc1[i] : acc0[i], A0, A1, A2, A3, b0, b1);
        else mma_16816((w & 1) ? acc1[i] : acc0[i], A0, A1, A2, A3, b0, b1);
        if (FIRST && w == 0) mma_16816_z(xs[i], ONES, ONES, ONES, ONES, b0, b1);
        else mma_16816(xs[i], ONES, ONES, ONES, ONES, b0, b1);
      }
    }
  };
  // d += s * ((acc0 + acc1) - (1024 + z) * sum x) for the group `grp` just accumulated
  auto correct = [&](int grp) {
    float sa, sb, ca, cb;
    if constexpr (DEFER && HAS_ZERO) {
      const float2 ea = s_a[grp], eb = s_b[grp];
      sa = ea.x, ca = ea.y, sb = eb.x, cb = eb.y;
    } else if constexpr (DEFER) {
      sa = s_a[grp], sb = s_b[grp], ca = 1151.5f, cb = 1151.5f;
    } else {
      sa = sb = ca = cb = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      d[i][0] = fmaf(sa, fmaf(-ca, xs[i][0], acc0[i][0] + acc1[i][0]), d[i][0]);
      d[i][1] = fmaf(sa, fmaf(-ca, xs[i][1], acc0[i][1] + acc1[i][1]), d[i][1]);
      d[i][2] = fmaf(sb, fmaf(-cb, xs[i][2], acc0[i][2] + acc1[i][2]), d[i][2]);
      d[i][3] = fmaf(sb, fmaf(-cb, xs[i][3], acc0[i][3] + acc1[i][3]), d[i][3]);
    }
  };

  bool ok = mbar_wait(&xbar[0], 0);
  auto run_tiles = [&](auto fast_tag) {
    P cur, nxt;
    int ti = kp;
    if (ti < nt) {
      ok = mbar_wait(&bars[ti], 0) && ok;
      load_piece(ti, 0, cur);
    }
#pragma unroll 1
    while (ti < nt) {
      load_piece(ti, 1, nxt);  // same tile: already here
      compute_piece(cur, fast_tag);
      const int tn = ti + KP;
      bool pre = false;
      if (tn < nt && mbar_try_wait(&bars[tn], 0)) {  // next tile landed: fetch ahead
        load_piece(tn, 0, cur);
        pre = true;
      }
      compute_piece(nxt, fast_tag);
      if (tn < nt && !pre) {
        ok = mbar_wait(&bars[tn], 0) && ok;
        load_piece(tn, 0, cur);
      }
      ti = tn;
    }
  };
  auto run_tiles_defer = [&]() {
    P cur, nxt;
    int ti = kp;
    const bool per_piece = bs_shift < 7;  // 64-wide groups: correct after every piece
    if (ti < nt) {
      ok = mbar_wait(&bars[ti], 0) && ok;
      load_piece(ti, 0, cur);
    }
#pragma unroll 1
    while (ti < nt) {
      load_piece(ti, 1, nxt);
      compute_piece_defer(cur, std::true_type{});
      const int grp0 = (k0 + ti * 128) >> bs_shift;
      if (per_piece) correct(grp0);
      const int tn = ti + KP;
      bool pre = false;
      if (tn < nt && mbar_try_wait(&bars[tn], 0)) {
        load_piece(tn, 0, cur);
        pre = true;
      }
      if (per_piece) {
        compute_piece_defer(nxt, std::true_type{});
        correct(grp0 + 1);
      } else {
        compute_piece_defer(nxt, std::false_type{});
        correct(grp0);
      }
      if (tn < nt && !pre) {
        ok = mbar_wait(&bars[tn], 0) && ok;
        load_piece(tn, 0, cur);
      }
      ti = tn;
    }
  };
  if constexpr (DEFER) {
    run_tiles_defer();
  } else {
    if (all_fast) run_tiles(std::true_type{});
    else run_tiles(std::false_type{});
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) d[0][j] += d2[j];
  // every warp sees every copy land before shared memory is reused below
  for (int i = 0; i < nt; ++i) ok = mbar_wait(&bars[i], 0) && ok;
  if (!ok && lane == 0) atomicOr(status, 1u);
  __syncthreads();

  // ---- reduce the KP k-phases of each row set; the staging area is free now ----
  float* red = reinterpret_cast<float*>(Wsm);  // [NW warps][16][TOK + 1]
  float* partial = red + NW * 16 * (TOK + 1);  // [R][TOK]
  {
    float* rw = red + (size_t)warp * 16 * (TOK + 1);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      rw[pg * (TOK + 1) + i * 8 + 2 * t] = d[i][0];
      rw[pg * (TOK + 1) + i * 8 + 2 * t + 1] = d[i][1];
      rw[(pg + 8) * (TOK + 1) + i * 8 + 2 * t] = d[i][2];
      rw[(pg + 8) * (TOK + 1) + i * 8 + 2 * t + 1] = d[i][3];
    }
  }
  __syncthreads();
  if (S == 1) {
    // no k-split: finish here
    for (int e = tid; e < R * a.m; e += NT) {
      const int row = e % R, tok = e / R;
      if (n0 + row >= a.n) continue;
      const int set = row >> 4, r16 = row & 15;
      float v = 0.0f;
#pragma unroll
      for (int ph = 0; ph < KP; ++ph)
        v += red[(size_t)(ph * RS + set) * 16 * (TOK + 1) + r16 * (TOK + 1) + tok];
      __half* dst = a.out + (size_t)tok * a.n + n0 + row;
      *dst = __float2half_rn(fmaf(a.beta, __half2float(*dst), v));
    }
    return;
  }
  for (int e = tid; e < R * TOK; e += NT) {
    const int row = e % R, tok = e / R;
    const int set = row >> 4, r16 = row & 15;
    float v = 0.0f;
#pragma unroll
    for (int ph = 0; ph < KP; ++ph)
      v += red[(size_t)(ph * RS + set) * 16 * (TOK + 1) + r16 * (TOK + 1) + tok];
    partial[row * TOK + tok] = v;
  }

  // ---- reduce the k-slices across the cluster.  Every CTA finishes R/S of the rows: it
  // reads the S partial sums of those rows through distributed shared memory and adds
  // them in rank order (the same order whoever does it, so the result is deterministic).
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  {
    const int rpr = R / S;  // rows finished by each rank
    const uint32_t paddr = smem_u32(partial);
    for (int e = tid; e < rpr * a.m; e += NT) {
      const int row = rank * rpr + e % rpr, tok = e / rpr;
      if (n0 + row >= a.n) continue;
      __half* dst = a.out + (size_t)tok * a.n + n0 + row;
      const float old = __half2float(*dst);
      float pv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        pv[r] = 0.0f;
        if (r < S) {
          uint32_t remote;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                       : "=r"(remote)
                       : "r"(paddr + (uint32_t)(row * TOK + tok) * 4u), "r"(r));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[r]) : "r"(remote) : "memory");
        }
      }
      float v = pv[0];
#pragma unroll
      for (int r = 1; r < 8; ++r)
        if (r < S) v += pv[r];
      *dst = __float2half_rn(fmaf(a.beta, old, v));
    }
  }
  // every CTA stays resident until its peers have read its partial sums
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct StreamPlan {
  int S, R, NW, XS, NG, shift;
  size_t smem;
};

// Picks the rows per CTA and the cluster size (k-split) by a small cost model: all CTAs
// resident at once if possible, no cluster if possible, little activation re-reading.
bool plan_stream(const adr_ctx* ctx, const U8Args& a, int force_split, int force_rows,
                 StreamPlan& pl) {
  if (a.m < 1 || a.m > 16 || a.p % 128 != 0 || a.block_size < 16 ||
      (a.block_size & (a.block_size - 1)) != 0)
    return false;
  const int ntiles = a.p / 128;
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  int shift = 0;
  while ((1 << shift) < a.block_size) ++shift;
  bool found = false;
  double best = 1e30;
  for (int R : {16, 32, 64}) {
    if (force_rows && R != force_rows) continue;
    for (int S : {1, 2, 4, 8}) {
      if (force_split && S != force_split) continue;
      if (S > ntiles || R % S != 0) continue;
      const int maxt = (ntiles + S - 1) / S;
      if (maxt > MAX_TILES) continue;
      const int xs = 2 * maxt * 128 + 16;
      const int ngmax = (maxt * 128) / a.block_size + 2;  // groups a slice can touch
      const size_t tables = (size_t)R * ngmax * (a.zeros ? 8 : 4) + (size_t)(maxt + 1) * 8;
      // the reduction buffers reuse the staging area once the copies are consumed
      const int nw = 8;
      const size_t alias = (size_t)(nw * 16 * 17 + R * 16) * 4;
      const size_t smem = std::max((size_t)maxt * R * 128 + (size_t)a.m * xs + tables, alias);
      if (smem > 200 * 1024) continue;
      const double ctas = (double)((a.n + R - 1) / R) * S;
      const int per_sm = (int)std::min<size_t>(8, (227 * 1024) / (smem + 1024));
      const double waves = ctas / ((double)sms * per_sm);
      double cost = waves <= 1.0 ? 1.0 : waves;
      if (ctas < sms) cost += (sms - ctas) / sms;
      if (S > 1) cost += 0.25 + 0.05 * std::log2((double)S);
      cost += 0.5 * (2.0 * a.m / R);  // activation bytes re-read per weight byte
      if (cost < best) {
        best = cost;
        found = true;
        pl = {S, R, nw, xs, ngmax, shift, smem};
      }
    }
  }
  return found;
}

template <int MT, int R, bool Z, bool PDL, bool DEFER>
int launch_stream_p(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const StreamPlan& pl) {
  constexpr int NW = 8;
  auto kfn = u8_stream_kernel<MT, R, NW, Z, PDL, DEFER>;
  cudaError_t e;
  if (int rc0 = opt_in_smem(ctx, kfn, 200 * 1024); rc0 != ADR_OK) return rc0;
  CUtensorMap wmap;
  const uint64_t dims[2] = {(uint64_t)a.p, (uint64_t)a.n};
  const uint64_t strides[1] = {(uint64_t)a.p};
  const uint32_t box[2] = {128u, (uint32_t)R};
  int rc = tma_get(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.rhs, dims, strides, box,
                   CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != ADR_OK) return rc;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.S, (a.n + R - 1) / R, 1);
  cfg.blockDim = dim3(NW * 32, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  // the cluster attribute is dropped for S == 1, the serialization one without PDL
  cudaLaunchAttribute* first = pl.S > 1 ? &attr[0] : &attr[1];
  cfg.attrs = first;
  cfg.numAttrs = (pl.S > 1 ? 1 : 0) + (PDL ? 1 : 0);
  if (pl.S > 1 && !PDL) cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kfn, wmap, a, pl.S, pl.XS, pl.NG, pl.shift, ctx->d_status);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  return after_launch(ctx);
}

template <int MT, int R, bool Z>
int launch_stream_t(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const StreamPlan& pl) {
  // deferred scaling unless the caller asked for the fp16-rounded dequantisation of the WMMA
  // kernel (tunable "u8_exact") or the groups are shorter than a 64-wide piece
  const bool defer = !ctx->tune_u8_exact && a.block_size >= 64;
  if (defer)
    return ctx->tune_pdl ? launch_stream_p<MT, R, Z, true, true>(ctx, stream, a, pl)
                         : launch_stream_p<MT, R, Z, false, true>(ctx, stream, a, pl);
  return ctx->tune_pdl ? launch_stream_p<MT, R, Z, true, false>(ctx, stream, a, pl)
                       : launch_stream_p<MT, R, Z, false, false>(ctx, stream, a, pl);
}

}  // namespace

bool u8_stream_supports(const adr_ctx* ctx, const U8Args& a) {
  StreamPlan pl;
  return plan_stream(ctx, a, ctx->tune_u8_split, ctx->tune_u8_rows, pl);
}

int launch_u8_stream(adr_ctx* ctx, cudaStream_t stream, const U8Args& a) {
  StreamPlan pl;
  if (!plan_stream(ctx, a, ctx->tune_u8_split, ctx->tune_u8_rows, pl)) return ADR_ERR_SHAPE;
  if ((a.n + pl.R - 1) / pl.R > 65535) return ADR_ERR_SHAPE;
  const bool z = a.zeros != nullptr;
  const bool two = a.m > 8;
#define ADR_STREAM_CASE(RR)                                                                   \
  if (pl.R == RR) {                                                                           \
    if (two)                                                                                  \
      return z ? launch_stream_t<2, RR, true>(ctx, stream, a, pl)                             \
               : launch_stream_t<2, RR, false>(ctx, stream, a, pl);                           \
    return z ? launch_stream_t<1, RR, true>(ctx, stream, a, pl)                               \
             : launch_stream_t<1, RR, false>(ctx, stream, a, pl);                             \
  }
  ADR_STREAM_CASE(16)
  ADR_STREAM_CASE(32)
  ADR_STREAM_CASE(64)
#undef ADR_STREAM_CASE
  return ADR_ERR_SHAPE;
}

}  // namespace adr
