// Fused attention for prefill and for the CLIP encoder: one kernel for the reference's chain
//   scores = matmul_f16(q, k^T) with store Scale (and the causal mask)      llama.rs:538-547
//   probs  = softmax_rows(scores)                                           normalize.cu:150-220
//   out    = matmul_f16(probs, v) into a strided [tokens, heads, head_dim] view   llama.rs:548-554,
// (adrastea_models/src/clip.rs:374-388 is the same chain without the mask).  The [heads, S, S]
// score tensor never exists in memory: a CTA takes 128 query rows of one head and walks the keys
// in blocks of 128;
//   * S = Q K^T by tcgen05.mma into tensor memory (Q, K as 128-byte-swizzled K-major tiles
//     loaded by TMA with the caller's strides);
//   * four softmax warps, one thread per query row (TMEM lane): tcgen05.ld the row, round the
//     score to fp16 and multiply by fp16(scale) in fp16 (the reference's Scale store op), mask,
//     running maximum and sum in fp32, P = exp(score - max) rounded to fp16 (the reference
//     rounds its probabilities to fp16 too) written back over S in tensor memory;
//   * O_j = P V_j by tcgen05.mma with P read from tensor memory and V as an N-major operand
//     (V is [keys, head_dim] row-major, exactly as it lies in memory);
//   * the softmax warps keep the output row in registers: O = (O + O_j) * exp(max_old - max_new),
//     divide by the sum at the end and store fp16.
// Difference from the three-kernel chain: the probabilities are normalised after the PV
// product instead of before it (one rounding of p / sum per element is replaced by one rounding
// of exp(x - max)); the result stays within the 1e-2 tolerance of this path.
// head_dim 64 or 128; any sequence lengths; two batch dimensions (heads inside images).
#include <algorithm>
#include <cmath>

#include "tcgen05.cuh"

namespace adr {

namespace {

constexpr int AT_BM = 128;  // query rows per CTA
constexpr int AT_BN = 128;  // keys per block
constexpr int AT_THREADS = 192;  // producer, MMA, four softmax warps

template <int HD>
struct AtCfg {
  static constexpr int CH = HD / 64;                     // 64-wide chunks of the head dimension
  static constexpr int TILE_BYTES = AT_BM * HD * 2;      // Q, one K block, one V block
  static constexpr int SBUF = HD == 64 ? 1 : 2;          // score buffers in tensor memory
  static constexpr uint32_t TMEM_COLS = HD == 64 ? 256 : 512;  // SBUF * 128 + 2 * HD
  static constexpr uint32_t O_COL0 = SBUF * 128;
  static constexpr size_t SMEM = 1024 + (size_t)TILE_BYTES * 5 + 512;
};

struct AtParams {
  __half* out;
  int s_q, s_k;
  long long so_row, so_bi, so_bo;  // output strides in elements
  float scale;
  int causal;
  unsigned int* status;
};

__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x8b(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait_b() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_f16_ts_b(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Barriers: q_full; per K/V ring slot k_full, v_full, kv_empty; per score buffer s_ready,
// p_ready, sp_free; per output buffer o_ready, o_free.
template <int HD>
__global__ void __launch_bounds__(AT_THREADS, HD == 64 ? 2 : 1)
    attention_f16_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, AtParams p) {
  using Cfg = AtCfg<HD>;
  constexpr int SBUF = Cfg::SBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = q_sm + Cfg::TILE_BYTES;       // [2][TILE]
  uint8_t* v_sm = k_sm + 2 * Cfg::TILE_BYTES;   // [2][TILE]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + 2 * Cfg::TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* v_full = bars + 3;     // [2]
  uint64_t* kv_empty = bars + 5;   // [2]
  uint64_t* s_ready = bars + 7;    // [2]
  uint64_t* p_ready = bars + 9;    // [2]
  uint64_t* sp_free = bars + 11;   // [2]
  uint64_t* o_ready = bars + 13;   // [2]
  uint64_t* o_free = bars + 15;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * AT_BM;
  const int bi = blockIdx.y, bo = blockIdx.z;
  // keys this block of queries can see
  const int kend = p.causal ? min(p.s_k, q0 + AT_BM) : p.s_k;
  const int nb = (kend + AT_BN - 1) / AT_BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_ready[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&sp_free[i], 1);
      mbar_init(&o_ready[i], 1);
      mbar_init(&o_free[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // keys of block j, rounded up to the MMA's granularity of 16
  auto block_n = [&](int j) { return min(AT_BN, ((kend - j * AT_BN) + 15) & ~15); };

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
      for (int c = 0; c < Cfg::CH; ++c)
        tma_load_4d(q_sm + c * (AT_BM * 128), &map_q, c * 64, q0, bi, bo, q_full);
      for (int j = 0; j < nb && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((unsigned)(j >> 1) & 1u) ^ 1u)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], Cfg::TILE_BYTES);
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_4d(k_sm + s * Cfg::TILE_BYTES + c * (AT_BN * 128), &map_k, c * 64, j * AT_BN, bi, bo,
                      &k_full[s]);
        mbar_expect_tx(&v_full[s], Cfg::TILE_BYTES);
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_4d(v_sm + s * Cfg::TILE_BYTES + c * (AT_BN * 128), &map_v, c * 64, j * AT_BN, bi, bo,
                      &v_full[s]);
        issued = j + 1;
      }
      // every issued copy has landed before the CTA may exit (also when somebody gave up)
      if (!mbar_wait(q_full, 0)) ok = false;
      for (int j = max(0, issued - 2); j < issued; ++j) {
        if (!mbar_wait(&k_full[j & 1], (unsigned)(j >> 1) & 1u)) ok = false;
        if (!mbar_wait(&v_full[j & 1], (unsigned)(j >> 1) & 1u)) ok = false;
      }
      if (!ok) atomicOr(p.status, 512u);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issue -------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0);
      const uint32_t qa = smem_u32(q_sm);
      auto issue_qk = [&](int j) {
        const int s = j & 1, sb = j % SBUF;
        const int use = j / SBUF;
        if (!mbar_wait(&k_full[s], (unsigned)(j >> 1) & 1u)) { ok = false; return; }
        if (!mbar_wait(&sp_free[sb], ((unsigned)use & 1u) ^ 1u)) { ok = false; return; }
        tc_fence_after_sync();
        const uint32_t idesc = umma_idesc_f16(block_n(j), false);
        const uint32_t ka = smem_u32(k_sm + s * Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + (uint32_t)(sb * 128), umma_desc_k_sw128(qa + c * (AT_BM * 128)) + (uint64_t)(kk * 2),
                     umma_desc_k_sw128(ka + c * (AT_BN * 128)) + (uint64_t)(kk * 2), idesc,
                     (c > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&s_ready[sb]);
      };
      auto issue_pv = [&](int j) {
        const int s = j & 1, sb = j % SBUF, ob = j & 1;
        if (!mbar_wait(&p_ready[sb], (unsigned)(j / SBUF) & 1u)) { ok = false; return; }
        if (!mbar_wait(&v_full[s], (unsigned)(j >> 1) & 1u)) { ok = false; return; }
        if (!mbar_wait(&o_free[ob], ((unsigned)(j >> 1) & 1u) ^ 1u)) { ok = false; return; }
        tc_fence_after_sync();
        constexpr uint32_t idesc = umma_idesc_f16(HD, true);
        const uint64_t vdesc = umma_desc_mn_sw128(smem_u32(v_sm + s * Cfg::TILE_BYTES), AT_BN * 128);
        const int steps = block_n(j) / 16;
        for (int ks = 0; ks < steps; ++ks)
          umma_f16_ts_b(tmem_base + Cfg::O_COL0 + (uint32_t)(ob * HD), tmem_base + (uint32_t)(sb * 128 + ks * 8),
                        vdesc + (uint64_t)ks * 128, idesc, ks > 0 ? 1u : 0u);
        umma_commit(&o_ready[ob]);
        umma_commit(&kv_empty[s]);
        umma_commit(&sp_free[sb]);
      };
      if (ok && nb > 0) issue_qk(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (SBUF == 2 && j + 1 < nb) issue_qk(j + 1);
        if (!ok) break;
        issue_pv(j);
        if (SBUF == 1 && j + 1 < nb && ok) issue_qk(j + 1);
      }
      if (!ok) atomicOr(p.status, 1024u);
    }
  } else {
    // ------------------------------- softmax + output -------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // row of the query block = TMEM lane
    const int qrow = q0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const __half hscale = __float2half_rn(p.scale);
    constexpr float LOG2E = 1.4426950408889634f;
    const int klimit = p.causal ? min(p.s_k, qrow + 1) : p.s_k;  // keys < klimit are visible
    float m_run = -INFINITY, l_run = 0.0f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.0f;
    bool ok = true;

    // adds O_j (finished by the tensor core) to the running output, then rescales
    auto drain = [&](int j, float alpha) {
      const int ob = j & 1;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_ready[ob], (unsigned)(j >> 1) & 1u));
      tc_fence_after_sync();
      if (ok) {
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) {
          uint32_t v[16];
          tmem_ld_x16(tmem_base + lane_base + Cfg::O_COL0 + (uint32_t)(ob * HD + c * 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[c * 16 + i] = (o[c * 16 + i] + __uint_as_float(v[i])) * alpha;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_free[ob]);
    };

    for (int j = 0; j < nb; ++j) {
      const int sb = j % SBUF;
      const int ncols = block_n(j);
      const int key0 = j * AT_BN;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_ready[sb], (unsigned)(j / SBUF) & 1u));
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + lane_base + (uint32_t)(sb * 128);
      float alpha = 1.0f;
      if (ok) {
        // pass 1: the row maximum of fp16(score) * fp16(scale) over the visible keys
        float mloc = -INFINITY;
        for (int c = 0; c < ncols / 16; ++c) {
          uint32_t v[16];
          tmem_ld_x16(s_addr + (uint32_t)(c * 16), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float s = __half2float(__hmul(__float2half_rn(__uint_as_float(v[i])), hscale));
            if (key0 + c * 16 + i < klimit) mloc = fmaxf(mloc, s);
          }
        }
        const float m_new = fmaxf(m_run, mloc);
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        alpha = m_run == -INFINITY ? 0.0f : fast_exp2((m_run - m_use) * LOG2E);
        // pass 2: P = exp(score - max) as fp16, written over the scores (two P columns per
        // 32-bit cell, always behind the columns still to be read)
        float rowsum = 0.0f;
        const float mo = m_use * LOG2E;
        for (int c = 0; c < ncols / 16; ++c) {
          uint32_t v[16];
          tmem_ld_x16(s_addr + (uint32_t)(c * 16), v);
          tmem_ld_wait();
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float s0 = __half2float(__hmul(__float2half_rn(__uint_as_float(v[i])), hscale));
            const float s1 = __half2float(__hmul(__float2half_rn(__uint_as_float(v[i + 1])), hscale));
            const float p0 = key0 + c * 16 + i < klimit ? fast_exp2(fmaf(s0, LOG2E, -mo)) : 0.0f;
            const float p1 = key0 + c * 16 + i + 1 < klimit ? fast_exp2(fmaf(s1, LOG2E, -mo)) : 0.0f;
            const __half2 h = __floats2half2_rn(p0, p1);
            const float2 hf = __half22float2(h);
            rowsum += hf.x + hf.y;
            pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
          }
          tmem_st_x8b(s_addr + (uint32_t)(c * 8), pk);
        }
        l_run = l_run * alpha + rowsum;
        m_run = m_new;
      }
      tmem_st_wait_b();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[sb]);
      // O_{j-1} was computed against the previous maximum: add it, then move everything to
      // the new maximum
      if (j > 0) drain(j - 1, alpha);
      else {
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] *= alpha;  // zeros; keeps the two paths alike
      }
    }
    if (nb > 0) drain(nb - 1, 1.0f);
    if (ok && qrow < p.s_q) {
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      __half* dst = p.out + (long long)bo * p.so_bo + (long long)bi * p.so_bi + (long long)qrow * p.so_row;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        uint4 w;
        __half2* h = reinterpret_cast<__half2*>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(dst + c * 8) = w;
      }
    }
    if (!ok && lane == 0) atomicOr(p.status, 2048u);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// The last few query rows of a problem whose length is just over a multiple of the query
// tile (257 = 2 x 128 + 1 in a ViT-L/14 encoder: a third tile would hold one row and cost a
// whole tile's MMAs).  One CTA per (row, problem), plain loads, the arithmetic of the tile
// kernel: s = fp16(fp16(q . k) x fp16(scale)), p = fp16(exp(s - max)), out = fp16(sum p v / sum p).
// ---------------------------------------------------------------------------------------
constexpr int AR_THREADS = 128;
constexpr int AR_MAX_KEYS = 8192;   // scores of a row in shared memory
constexpr int AR_MAX_ROWS = 2;      // more rows than this take a tile (measured: a row costs 9-26 us
                                    // over 1024 problems of 257 keys, a third tile 44 us)

struct ArParams {
  __half* out;
  const __half* q;
  const __half* k;
  const __half* v;
  int row0, s_k;
  long long sq[3], sk[3], sv[3], so[3];  // row, inner batch, outer batch (elements)
  float scale;
  int causal;
};

template <int HD>
__global__ void __launch_bounds__(AR_THREADS) attention_rows_kernel(ArParams p) {
  // A key or value row (HD fp16) is read by HD / 8 neighbouring lanes, 16 bytes each, and
  // AR_THREADS / (HD / 8) rows per pass; eight passes' loads are issued before the first is
  // used: the rows of one problem lie a whole token apart (hundreds of KB in token-major
  // storage), so the kernel is as fast as it keeps loads in flight.
  constexpr int LPR = HD / 8;            // lanes per row
  constexpr int RPP = AR_THREADS / LPR;  // rows per pass
  constexpr int U = 8;                   // passes in flight
  extern __shared__ float ar_scores[];          // [s_k] scores, then probabilities
  __shared__ float red[AR_THREADS / 32];
  __shared__ float part[RPP * HD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rslot = tid / LPR, piece = tid % LPR;
  const int row = p.row0 + blockIdx.x, bi = blockIdx.y, bo = blockIdx.z;
  const __half* q = p.q + bo * p.sq[2] + bi * p.sq[1] + (long long)row * p.sq[0];
  const __half* kb = p.k + bo * p.sk[2] + bi * p.sk[1] + piece * 8;
  const __half* vb = p.v + bo * p.sv[2] + bi * p.sv[1] + piece * 8;
  const int klimit = p.causal ? min(p.s_k, row + 1) : p.s_k;
  float qf[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(q + piece * 8);
    const __half2* q2 = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(q2[i]);
      qf[2 * i] = f.x;
      qf[2 * i + 1] = f.y;
    }
  }
  const __half hscale = __float2half_rn(p.scale);
  constexpr float LOG2E = 1.4426950408889634f;
  float mloc = -INFINITY;
  for (int j0 = 0; j0 < klimit; j0 += RPP * U) {
    uint4 kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * RPP + rslot;
      kv[u] = j < klimit ? *reinterpret_cast<const uint4*>(kb + (long long)j * p.sk[0]) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * RPP + rslot;
      const __half2* k2 = reinterpret_cast<const __half2*>(&kv[u]);
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(k2[i]);
        acc = fmaf(qf[2 * i], f.x, acc);
        acc = fmaf(qf[2 * i + 1], f.y, acc);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (j < klimit) {
        const float sc = __half2float(__hmul(__float2half_rn(acc), hscale));
        if (piece == 0) ar_scores[j] = sc;
        mloc = fmaxf(mloc, sc);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
  if (lane == 0) red[warp] = mloc;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int w = 1; w < AR_THREADS / 32; ++w) m = fmaxf(m, red[w]);
  const float mo = (m == -INFINITY ? 0.0f : m) * LOG2E;
  __syncthreads();
  float lsum = 0.0f;
  for (int j = tid; j < klimit; j += AR_THREADS) {
    const float pr = __half2float(__float2half_rn(fast_exp2(fmaf(ar_scores[j], LOG2E, -mo))));
    ar_scores[j] = pr;
    lsum += pr;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  if (lane == 0) red[warp] = lsum;
  __syncthreads();
  float l = 0.0f;
#pragma unroll
  for (int w = 0; w < AR_THREADS / 32; ++w) l += red[w];
  // output: this thread's eight columns over the rows of its slot, then the slots are added
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int j0 = 0; j0 < klimit; j0 += RPP * U) {
    uint4 vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * RPP + rslot;
      vv[u] = j < klimit ? *reinterpret_cast<const uint4*>(vb + (long long)j * p.sv[0]) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + u * RPP + rslot;
      const float pr = j < klimit ? ar_scores[j] : 0.0f;
      const __half2* v2 = reinterpret_cast<const __half2*>(&vv[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(v2[i]);
        acc[2 * i] = fmaf(pr, f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(pr, f.y, acc[2 * i + 1]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[rslot * HD + piece * 8 + i] = acc[i];
  __syncthreads();
  if (tid < HD) {
    float o = 0.0f;
#pragma unroll
    for (int sl = 0; sl < RPP; ++sl) o += part[sl * HD + tid];
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    p.out[bo * p.so[2] + bi * p.so[1] + (long long)row * p.so[0] + tid] = __float2half_rn(o * inv);
  }
}

template <int HD>
int launch_attention(adr_ctx* ctx, cudaStream_t stream, __half* out, const __half* q, const __half* k,
                     const __half* v, int b_outer, int b_inner, int s_q, int s_k,
                     const long long* sq, const long long* sk, const long long* sv, const long long* so,
                     float scale, int causal) {
  using Cfg = AtCfg<HD>;
  auto kfn = attention_f16_kernel<HD>;
  if (int rc = opt_in_smem(ctx, kfn, Cfg::SMEM); rc != ADR_OK) return rc;
  CUtensorMap maps[3];
  const __half* ptr[3] = {q, k, v};
  const long long* st[3] = {sq, sk, sv};
  const int rows[3] = {s_q, s_k, s_k};
  for (int i = 0; i < 3; ++i) {
    // a broadcast batch dimension (stride 0) is described with extent 1: the copy engine
    // wants positive strides
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)rows[i], (uint64_t)b_inner, (uint64_t)b_outer};
    uint64_t strides[3] = {(uint64_t)st[i][0] * 2, (uint64_t)st[i][1] * 2, (uint64_t)st[i][2] * 2};
    if (b_inner == 1 || strides[1] == 0) strides[1] = strides[0] * (uint64_t)rows[i];
    if (b_outer == 1 || strides[2] == 0) strides[2] = strides[1] * (uint64_t)b_inner;
    const uint32_t box[4] = {64u, (uint32_t)AT_BM, 1u, 1u};
    int rc = tma_get(ctx, &maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, ptr[i], dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
  }
  // rows past the last full query tile, when they are few, go to the row kernel
  int tail = s_q % AT_BM;
  if (s_q < AT_BM || tail > AR_MAX_ROWS || s_k > AR_MAX_KEYS) tail = 0;
  s_q -= tail;
  AtParams p;
  p.out = out;
  p.s_q = s_q;
  p.s_k = s_k;
  p.so_row = so[0];
  p.so_bi = so[1];
  p.so_bo = so[2];
  p.scale = scale;
  p.causal = causal;
  p.status = ctx->d_status;
  const dim3 grid((s_q + AT_BM - 1) / AT_BM, b_inner, b_outer);
  kfn<<<grid, AT_THREADS, Cfg::SMEM, stream>>>(maps[0], maps[1], maps[2], p);
  if (int rc = after_launch(ctx); rc != ADR_OK) return rc;
  // the tail rows afterwards: their keys and values are then still in L2
  if (tail > 0) {
    ArParams r;
    r.out = out;
    r.q = q;
    r.k = k;
    r.v = v;
    r.row0 = s_q;
    r.s_k = s_k;
    for (int d = 0; d < 3; ++d) {
      r.sq[d] = sq[d];
      r.sk[d] = sk[d];
      r.sv[d] = sv[d];
      r.so[d] = so[d];
    }
    r.scale = scale;
    r.causal = causal;
    attention_rows_kernel<HD><<<dim3(tail, b_inner, b_outer), AR_THREADS, (size_t)s_k * sizeof(float), stream>>>(r);
    return after_launch(ctx);
  }
  return ADR_OK;
}

}  // namespace

}  // namespace adr

using namespace adr;

extern "C" int adr_attention_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* q, const void* k,
                                 const void* v, int batches_outer, int batches_inner, int s_q, int s_k,
                                 int head_dim, const long long* strides_q, const long long* strides_k,
                                 const long long* strides_v, const long long* strides_o, float scale,
                                 uint32_t mask_op) {
  if (!ctx || !out || !q || !k || !v || !strides_q || !strides_k || !strides_v || !strides_o)
    return ADR_ERR_INVALID;
  if (batches_outer <= 0 || batches_inner <= 0 || s_q <= 0 || s_k <= 0) return ADR_ERR_INVALID;
  if (mask_op > ADR_MASK_CAUSAL) return ADR_ERR_INVALID;
  if (head_dim != 64 && head_dim != 128) return ADR_ERR_SHAPE;
  if (batches_inner > 65535 || batches_outer > 65535) return ADR_ERR_SHAPE;
  if (!ctx->encode_tiled_fn) return ADR_ERR_UNSUPPORTED;
  const void* ptrs[4] = {q, k, v, out};
  const long long* st[4] = {strides_q, strides_k, strides_v, strides_o};
  for (int i = 0; i < 4; ++i) {
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15u) return ADR_ERR_SHAPE;
    for (int d = 0; d < 3; ++d)
      if (st[i][d] < 0 || (st[i][d] % 8) != 0) return ADR_ERR_SHAPE;  // 16-byte rows for the copy engine
    if (st[i][0] < head_dim) return ADR_ERR_SHAPE;
  }
  DeviceGuard guard(ctx);
  int rc;
  if (head_dim == 64)
    rc = launch_attention<64>(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)q, (const __half*)k,
                              (const __half*)v, batches_outer, batches_inner, s_q, s_k, strides_q,
                              strides_k, strides_v, strides_o, scale, mask_op == ADR_MASK_CAUSAL);
  else
    rc = launch_attention<128>(ctx, (cudaStream_t)stream, (__half*)out, (const __half*)q, (const __half*)k,
                               (const __half*)v, batches_outer, batches_inner, s_q, s_k, strides_q,
                               strides_k, strides_v, strides_o, scale, mask_op == ADR_MASK_CAUSAL);
  return rc;
}
