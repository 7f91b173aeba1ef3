// u8-weight decode GEMV/GEMM, persistent ring form (m <= 16, block_size 64 or 128):
//   out[m,n] = lhs[m,p] . deq(Q[n,p])^T + beta * out
// (replaces adrastea_kernels/cpp/matmul_nt_fp16u8.cu:4-24 and
// matmul_nt_wmma_16x128x256_fp16u8.cu:12-83 for decode shapes).
//
// One CTA per SM walks a list of units (16 weight rows x all of k) and streams them through
// a ring of shared-memory stages, so that the memory pipe is kept full by a bounded amount of
// data in flight and a CTA's lifetime does not depend on the whole matrix having landed:
//   * a stage is eight 128-byte-wide tiles of the unit's 16 rows (16 KB, one 3-D TMA load,
//     128-byte swizzle) plus the scales (and zero points) of those 16 rows x 1024 k, which
//     the producer warp copies with 4-byte cp.async tied to the stage's mbarrier;
//   * warp 0 produces (waits for a free stage, issues the loads); the consumer warps work in
//     groups of eight, a group per stage, a warp per tile: one PRMT per weight pair puts
//     the byte under the fp16 exponent of 1024 (1024 + q, exact), mma.sync.m16n8k16 sums
//     (1024 + q) x; sum x per scale group comes from one pass of MMAs with an all-ones
//     operand at the start of the launch; the scale and the zero point are applied in fp32
//     once per scale group:
//        sum_k (q_k - z) s x_k = s * (sum_k (1024 + q_k) x_k - (1024 + z) sum_k x_k)
//     which is the arithmetic of matmul_nt_fp16u8.cu:13-23 (weights not rounded to fp16);
//   * at the end of a unit the consumer warps add their partial sums through shared memory
//     in a fixed order and write 16 output columns for every token;
//   * the activations stay in shared memory for the whole launch when they fit beside a ring of
//     at least four stages; otherwise every stage carries its own slice of them.
// Under programmatic dependent launch the producer starts filling the ring while the
// previous kernel of the stream is still running (weights, scales and zero points are by
// contract not written by it); activations and output are touched only after
// griddepcontrol.wait.  The CTA is sized to leave room for such a successor on the SM when
// the activations are small.  Every wait is bounded; a wait that runs out sets the status
// word and the kernel drains its copies and returns.
#include <algorithm>
#include <cstdlib>

#include "tma.cuh"
#include "u8_common.cuh"

namespace adr {

namespace {

constexpr int RING_TILES = 8;                       // tiles per stage = warps per consumer group
constexpr int RING_TILE_BYTES = 16 * 128;           // 16 rows x 128 k
constexpr int RING_W_BYTES = RING_TILES * RING_TILE_BYTES;  // 16 KB
constexpr int RING_STAGE_BYTES = RING_W_BYTES + 1024;       // + scales/zeros, keeps 1 KB alignment
constexpr int RING_MAX_STAGES = 12;

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// The mbarrier receives one (pre-counted) arrival when all earlier cp.async of this thread
// have landed.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
constexpr int RING_RED_BUFS = 4;  // partial-sum buffers (and named barriers) in rotation

constexpr int RING_MAX_PROBLEMS = 4;
// The grouped form: several weight matrices (same k, block size and activations; q/k/v or
// gate/up of a decoder layer) walked by one launch.  Units are numbered across the problems.
struct RingProblem {
  const __half* scales;
  const __half* zeros;
  __half* out;
  int n;      // rows of this matrix
  int unit0;  // number of the first unit of this matrix
};
struct RingMaps {
  CUtensorMap m[RING_MAX_PROBLEMS];
};

struct RingParams {
  U8Args a;
  int nprob;  // grouped form: number of problems (a.rhs/scales/zeros/out/n are then unused)
  // Paired form (two problems of equal n: the gate and up projections): a CTA takes the gate unit
  // and the up unit of the same 16 rows one after the other and writes SiluMul(gate, up), each
  // rounded to fp16 first as the separate kernels would (elementwise.cu:28-33), to prob[0].out.
  // `units` then counts pairs.
  int pair;
  int wide_ok;  // grouped form: every scale (and zero point) matrix allows 16-byte copies
  RingProblem prob[RING_MAX_PROBLEMS];
  int NS;        // stages in the ring
  int XS;        // bytes between activation rows in shared memory
  int gps;       // scale groups per stage (1024 / block_size)
  int bs_shift;  // log2(block_size)
  int units;     // ceil(n / 16)
  int spu;       // stages per unit
  int xsum_entries;  // k-units of the activation-sum table
  int stage_bytes;   // distance between ring stages
  int xss;           // XR: bytes between activation rows inside a stage
  int rbufs;         // partial-sum buffers in rotation (2 or 4)
  unsigned int* status;
  // fused all-reduce (ar_world > 1): the unit results are pushed to every rank's inbox
  // [world][m][n] fp16 (slot = pushing rank) and summed after a flag exchange per CTA
  __half* ar_inbox[8];         // inbox of rank p, addressable from this GPU
  unsigned int* ar_flags[8];   // flag array of rank p: [ctas][world]
  unsigned int* ar_epochs;     // this rank's per-CTA epoch counters
  int ar_rank, ar_world, ar_residual;
  long long ar_wait_cycles;    // bound of the wait for the peers' flags
  // fused rms_norm of the activations (norm_w != nullptr; resident activations only)
  const __half* norm_w;
  float norm_eps;
  // fused rotary embedding + KV-cache append (the product is a fused q/k/v projection of 3 x
  // rope_width columns): q is rotated and written to out with row pitch rope_q_pitch, k is rotated
  // into k_cache[token][*rope_pos], v copied into v_cache[token][*rope_pos]
  int rope_width, rope_heads, rope_max_seq, rope_q_pitch;
  const int* rope_pos;
  float rope_theta;
  __half* rope_k_cache;
  __half* rope_v_cache;
};

// MT: 8-token column blocks.  NCW: consumer warps (a multiple of 8).
// XR: the activations do not fit beside the ring (m x k x 2 bytes: 262 KB at m = 16, k = 8192),
// so every stage carries its own 1024-wide slice of them (m bulk copies next to the weight box);
// the activation sums are then taken per tile by an extra MMA with an all-ones weight operand, and
// nothing is loaded before griddepcontrol.wait.
// FUSE: compiles in the optional rms_norm of the activations and the fused all-reduce; the plain
// product uses the instantiation without them (they cost registers and 6 % of its speed).
// The problem that unit `gu` belongs to (grouped form).
__device__ __forceinline__ int ring_locate(const RingParams& p, int gu) {
  int i = 0;
#pragma unroll
  for (int j = 1; j < RING_MAX_PROBLEMS; ++j)
    if (j < p.nprob && gu >= p.prob[j].unit0) i = j;
  return i;
}

template <int MT, int NCW, bool HAS_ZERO, bool PDL, bool XR, bool FUSE, bool SUMS_IN_LOOP, bool GROUPED>
__global__ void __launch_bounds__((NCW + 1) * 32, (NCW == 8 && MT == 1) ? 2 : 1)
    u8_ring_kernel(const __grid_constant__ RingMaps maps, RingParams p) {
  static_assert(!GROUPED || (!XR && !FUSE), "the grouped form keeps the activations resident and fuses nothing");
  constexpr int TOK = 8 * MT;
  constexpr int NG = NCW / 8;  // consumer groups
  constexpr int RED_LD = TOK + 1;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const U8Args& a = p.a;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // same for every CTA of the launch
    if (threadIdx.x == 0) atomicOr(p.status, 16u);
    return;
  }
  uint8_t* ring = smem_raw;
  uint8_t* Xsm = ring + (size_t)p.NS * p.stage_bytes;
  float* red = reinterpret_cast<float*>(Xsm + (XR ? 0 : (size_t)a.m * p.XS));  // [RBUFS][NCW][16][RED_LD]
  // sum of the activations over every scale-group unit (a tile, or a 64-wide piece when
  // block_size is 64), per token: [units of k][TOK]
  const int RBUFS = p.rbufs;  // four in rotation, or two (the all-sync form, or to save room)
  float* xsum = red + RBUFS * NCW * 16 * RED_LD;
  uint64_t* full = reinterpret_cast<uint64_t*>(xsum + (XR ? 0 : (size_t)p.xsum_entries * TOK));
  uint64_t* empty = full + RING_MAX_STAGES;
  uint64_t* xbar = empty + RING_MAX_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(xbar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ntiles = a.p / 128;
  const int groups = a.p >> p.bs_shift;
  // units of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const bool paired = GROUPED && p.pair != 0;
  const int my_units = ((p.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * (paired ? 2 : 1);
  // paired form: the gate results of a pair, as fp16, for the warp that finishes the pair
  unsigned short* pairbuf = reinterpret_cast<unsigned short*>(xbar + 2);  // [2][16 * TOK]
  const int total_stages = my_units * p.spu;

  if (tid == 0) {
    tma_prefetch_desc(&maps.m[0]);
    for (int s = 0; s < p.NS; ++s) {
      mbar_init(&full[s], 33);  // expect_tx arrival + one cp.async arrival per producer lane
      mbar_init(&empty[s], 8);  // the eight warps of the group that consumed the stage
    }
    mbar_init(xbar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (PDL) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    bool ok = true;
    // scales of a stage: 16 rows x gps halves, copied in 16-byte pieces when every row of the
    // scale matrix starts on a 16-byte boundary, else in 4-byte pieces.  A lane's share of the
    // copies (row, position in the row) is the same for every stage and is worked out once.
    const bool wide = GROUPED ? (groups % 8) == 0 && p.wide_ok != 0
                              : (groups % 8) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 15u) == 0 &&
                                    (!HAS_ZERO || (reinterpret_cast<uintptr_t>(a.zeros) & 15u) == 0);
    const int per = wide ? 8 : 2;          // halves per copy
    const int per_row = p.gps / per;       // copies per row
    const int copies = 16 * per_row;       // per stage and table (16..128)
    int c_row[4], c_col[4];                // this lane's copies: row, first group within the stage
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = lane + 32 * u;
      c_row[u] = c < copies ? c / per_row : -1;
      c_col[u] = c < copies ? (c % per_row) * per : 0;
    }
    // stage counters, advanced without divisions: ring slot s, k-position st within the unit,
    // first row n0 of the unit (grouped form: unit number gu, from which the matrix and the row)
    int s = 0, st = 0, n0 = (int)blockIdx.x * 16, gu = (int)blockIdx.x, uq = 0;
    unsigned par = 0;  // parity of the current pass over the ring
    auto issue = [&]() {
      const CUtensorMap* wm = &maps.m[0];
      const __half* scales = a.scales;
      const __half* zeros = a.zeros;
      int rows = a.n;
      if constexpr (GROUPED) {
        const int pi = paired ? (uq & 1) : ring_locate(p, gu);
        wm = &maps.m[pi];
        scales = p.prob[pi].scales;
        zeros = p.prob[pi].zeros;
        rows = p.prob[pi].n;
        n0 = paired ? gu * 16 : (gu - p.prob[pi].unit0) * 16;
      }
      uint8_t* stage = ring + (size_t)s * p.stage_bytes;
      // XR: this stage's slice of every activation row (the last stage of a unit may be short)
      const int xbytes = XR ? min(2048, (a.p - st * 1024) * 2) : 0;
      if (lane == 0) {
        mbar_expect_tx(&full[s], (unsigned)(RING_W_BYTES + a.m * xbytes));
        tma_load_3d(stage, wm, 0, n0, st * RING_TILES, &full[s]);
      }
      if (XR) {
        __syncwarp();  // the transaction count is posted before any of the copies can complete
        if (lane < a.m)
          bulk_g2s(stage + RING_STAGE_BYTES + (size_t)lane * p.xss,
                   a.lhs + (size_t)lane * a.p + (size_t)st * 1024, (unsigned)xbytes, &full[s]);
      }
      __half* stab = reinterpret_cast<__half*>(stage + RING_W_BYTES);
      const int g0 = st * p.gps;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (c_row[u] >= 0 && g0 + c_col[u] < groups) {
          const size_t src = (size_t)min(n0 + c_row[u], rows - 1) * groups + g0 + c_col[u];
          __half* dst = stab + c_row[u] * p.gps + c_col[u];
          if (wide) {
            cp_async_16(dst, scales + src);
            if (HAS_ZERO) cp_async_16(dst + 16 * p.gps, zeros + src);
          } else {
            cp_async_4(dst, scales + src);
            if (HAS_ZERO) cp_async_4(dst + 16 * p.gps, zeros + src);
          }
        }
      }
      cp_async_arrive(&full[s]);
      if (++s == p.NS) s = 0, par ^= 1u;
      if (++st == p.spu) {
        st = 0, n0 += (int)gridDim.x * 16;
        ++uq;
        if (!paired || !(uq & 1)) gu += (int)gridDim.x;  // paired: the same rows twice (gate, up)
      }
    };
    int q = 0;
    if (XR) {
      // the stages carry activations: nothing may be requested before the previous kernel is done
      if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (; q < total_stages && q < p.NS; ++q) issue();
      if (lane == 0) mbar_arrive(xbar);  // unused in this mode; completed for the drain below
    } else {
      // fill the ring before waiting for the previous kernel: these loads touch only weights
      for (; q < total_stages && q < p.NS; ++q) issue();
      // (Asking here for the next stages to be brought into L2 while the ring is full was tried
      // and lost 1-7 %: the requests compete with the launch before, which is still streaming.
      // So was, on the consumer side, taking the next stage's weight bytes into registers while
      // the current stage's MMAs run: 10-20 % slower.)
      if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
      if (lane == 0) mbar_expect_tx(xbar, (unsigned)(a.m * a.p * 2));
      __syncwarp();
      if (lane < a.m)
        bulk_g2s(Xsm + (size_t)lane * p.XS, a.lhs + (size_t)lane * a.p, (unsigned)(a.p * 2), xbar);
    }
    for (; q < total_stages && ok; ++q) {
      // slot s was last filled one pass ago: wait until its consumers have released that use
      if (!mbar_wait(&empty[s], par ^ 1u) || *abort_flag) { ok = false; break; }
      issue();
    }
    if (!ok) {
      *abort_flag = 1;
      if (lane == 0) atomicOr(p.status, 32u);
    }
    // drain: every issued stage has landed before the CTA may exit
    const int issued = q;
    for (int qq = max(0, issued - p.NS); qq < issued; ++qq)
      if (!mbar_wait(&full[qq % p.NS], (unsigned)(qq / p.NS) & 1u) && lane == 0) atomicOr(p.status, 64u);
    if (!mbar_wait(xbar, 0) && lane == 0) atomicOr(p.status, 64u);
  } else {
    // ------------------------------- consumers -------------------------------
    const int cw = warp - 1;
    const int grp = cw >> 3, tile = cw & 7;
    const int g = lane >> 2, t = lane & 3;
    const int pg = (g >> 1) + 4 * (g & 1);  // tile row read by MMA row g (conflict-free under the swizzle)
    // activation rows g and g + 8 (XR: re-pointed at every stage's own slice)
    const uint8_t* xa = Xsm + (size_t)g * p.XS;
    const uint8_t* xb = Xsm + (size_t)(g + 8) * p.XS;
    const bool x0_ok = g < a.m;
    const bool x1_ok = MT > 1 && (g + 8) < a.m;
    const bool per_piece = p.bs_shift < 7;
    bool ok = true;
    if (PDL) asm volatile("griddepcontrol.wait;" ::: "memory");
    ok = __all_sync(0xffffffffu, mbar_wait(xbar, 0));  // the same verdict in every lane

    // ---- optional rms_norm of the activation rows, in place in shared memory, with the bits of
    // the reference kernel (normalize.cu:7-58; rowops.cu): that kernel's thread tid sums elements
    // tid, tid + 256, ...; here one warp takes a row and lane l keeps the eight partial sums of
    // "threads" 8l .. 8l+7 (it reads elements 8(l + 32j) .. +7, i.e. 8l + e + 256j, in the same
    // order), then replays the reference's xor butterfly: offsets 16 and 8 cross lanes (l^2,
    // l^1), offsets 4, 2, 1 stay inside a lane, and the eight warp sums sit in lanes 0, 4, .., 28.
    if constexpr (!XR && FUSE) {
      if (p.norm_w != nullptr) {
        for (int r = cw; r < a.m && ok; r += NCW) {
          uint8_t* xrow = Xsm + (size_t)r * p.XS;
          float part[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) part[e] = 0.0f;
          for (int c = lane; c * 8 < a.p; c += 32) {
            const uint4 u = *reinterpret_cast<const uint4*>(xrow + (size_t)c * 16);
            const __half* hv = reinterpret_cast<const __half*>(&u);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float v = __half2float(hv[e]);
              part[e] += v * v;
            }
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) part[e] += __shfl_xor_sync(0xffffffffu, part[e], 2);
#pragma unroll
          for (int e = 0; e < 8; ++e) part[e] += __shfl_xor_sync(0xffffffffu, part[e], 1);
          float q4[4], q2[2];
#pragma unroll
          for (int e = 0; e < 4; ++e) q4[e] = part[e] + part[e + 4];
          q2[0] = q4[0] + q4[2];
          q2[1] = q4[1] + q4[3];
          const float wsum = q2[0] + q2[1];  // the sum of "warp" lane / 4
          float W[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) W[q] = __shfl_sync(0xffffffffu, wsum, 4 * q);
          const float total = ((W[0] + W[4]) + (W[2] + W[6])) + ((W[1] + W[5]) + (W[3] + W[7]));
          const float rms_inv = rsqrtf((total / a.p) + p.norm_eps);
          for (int c = lane; c * 8 < a.p; c += 32) {
            uint4 u = *reinterpret_cast<const uint4*>(xrow + (size_t)c * 16);
            const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + (size_t)c * 8);
            __half* hv = reinterpret_cast<__half*>(&u);
            const __half* hw = reinterpret_cast<const __half*>(&wv);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              hv[e] = __hmul(hw[e], __float2half(__half2float(hv[e]) * rms_inv));
            *reinterpret_cast<uint4*>(xrow + (size_t)c * 16) = u;
          }
        }
        named_bar_sync(13, NCW * 32);
      }
    }

    // four accumulator chains per token block (piece x parity of the k16 step): two dependent
    // MMAs each, so that the tensor pipe's latency is overlapped within one warp
    float acc[2][2][MT][4];
    // Sums of the activations over each 64-wide piece, by an MMA with an all-ones weight operand
    // next to every weight MMA, when they are not taken from the table made once per launch.
    // The table costs less arithmetic, but making it stands between the arrival of the
    // activations and the first stage; which way wins depends on the token count (see the
    // launcher).
    constexpr bool XS_INLINE = XR || SUMS_IN_LOOP;
    float xs[2][MT][4];
    auto compute_piece = [&](const uint8_t* wrow, int xoff, auto piece_tag) {
      constexpr int H = decltype(piece_tag)::value;
      const uint4 qa = *reinterpret_cast<const uint4*>(wrow);
      const uint4 qb = *reinterpret_cast<const uint4*>(wrow + 8 * 128);
      const uint32_t wwa[4] = {qa.x, qa.y, qa.z, qa.w};
      const uint32_t wwb[4] = {qb.x, qb.y, qb.z, qb.w};
      const uint4 zero4 = make_uint4(0, 0, 0, 0);
      const uint4 v0 = x0_ok ? *reinterpret_cast<const uint4*>(xa + xoff) : zero4;
      const uint4 v1 = x0_ok ? *reinterpret_cast<const uint4*>(xa + xoff + 16) : zero4;
      uint4 v2 = zero4, v3 = zero4;
      if (MT > 1 && x1_ok) {
        v2 = *reinterpret_cast<const uint4*>(xb + xoff);
        v3 = *reinterpret_cast<const uint4*>(xb + xoff + 16);
      }
      const uint32_t xw[2][8] = {{v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w},
                                 {v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w}};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t A0 = prmt(wwa[w], 0x64646464u, 0x4140u), A2 = prmt(wwa[w], 0x64646464u, 0x4342u);
        const uint32_t A1 = prmt(wwb[w], 0x64646464u, 0x4140u), A3 = prmt(wwb[w], 0x64646464u, 0x4342u);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          const uint32_t b0 = xw[i][2 * w], b1 = xw[i][2 * w + 1];
          if (w < 2) mma_16816_z(acc[H][w & 1][i], A0, A1, A2, A3, b0, b1);
          else mma_16816(acc[H][w & 1][i], A0, A1, A2, A3, b0, b1);
          if constexpr (XS_INLINE) {
            constexpr uint32_t ONES = 0x3C003C00u;  // (1.0, 1.0)
            if (w == 0) mma_16816_z(xs[H][i], ONES, ONES, ONES, ONES, b0, b1);
            else mma_16816(xs[H][i], ONES, ONES, ONES, ONES, b0, b1);
          }
        }
      }
    };
    // ---- the activation sums, once per launch: an MMA with an all-ones weight operand leaves
    // sum_k x[k][token] in the accumulator layout; warp cw takes tiles cw, cw + NCW, ...
    if constexpr (!XS_INLINE) {
      constexpr uint32_t ONES = 0x3C003C00u;  // (1.0, 1.0)
      if (MT == 1 && a.m <= 4) {
        // few tokens: plain sums are quicker than the chain of MMAs.  Eight lanes share one
        // (token, scale-group unit) pair; the columns of the absent tokens are zeroed.
        const int ctid = tid - 32, sub = ctid & 7;
        const int entries = p.xsum_entries;
        for (int idx = ctid; idx < entries * TOK; idx += NCW * 32)
          if ((idx & (TOK - 1)) >= a.m) xsum[idx] = 0.0f;
        const int halves = per_piece ? 8 : 16;  // elements per lane
        const int pairs = entries * a.m;
        // (the trip count is the same for all lanes of a warp: the shuffles below need them all)
        for (int base = (ctid >> 5) * 4; base < pairs && ok; base += NCW * 4) {
          const int pr = base + ((ctid >> 3) & 3);
          const bool live = pr < pairs;
          const int r = live ? pr % a.m : 0, e = live ? pr / a.m : 0;
          const uint8_t* xr = Xsm + (size_t)r * p.XS + (size_t)(e * 8 + sub) * halves * 2;
          float sum = 0.0f;
          for (int c = 0; c < (live ? halves / 8 : 0); ++c) {
            const uint4 u = *reinterpret_cast<const uint4*>(xr + c * 16);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(h[j]);
              sum += f.x;
              sum += f.y;
            }
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          if (sub == 0 && live) xsum[(size_t)e * TOK + r] = sum;
        }
      } else
      for (int kt = cw; kt < ntiles && ok; kt += NCW) {
        float xs[2][MT][4];  // one chain per 64-wide piece
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int xoff = kt * 256 + (t + 4 * h) * 32;
          const uint4 zero4 = make_uint4(0, 0, 0, 0);
          const uint4 v0 = x0_ok ? *reinterpret_cast<const uint4*>(xa + xoff) : zero4;
          const uint4 v1 = x0_ok ? *reinterpret_cast<const uint4*>(xa + xoff + 16) : zero4;
          uint4 v2 = zero4, v3 = zero4;
          if (MT > 1 && x1_ok) {
            v2 = *reinterpret_cast<const uint4*>(xb + xoff);
            v3 = *reinterpret_cast<const uint4*>(xb + xoff + 16);
          }
          const uint32_t xw[2][8] = {{v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w},
                                     {v2.x, v2.y, v2.z, v2.w, v3.x, v3.y, v3.z, v3.w}};
#pragma unroll
          for (int w = 0; w < 4; ++w)
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              if (w == 0) mma_16816_z(xs[h][i], ONES, ONES, ONES, ONES, xw[i][0], xw[i][1]);
              else mma_16816(xs[h][i], ONES, ONES, ONES, ONES, xw[i][2 * w], xw[i][2 * w + 1]);
            }
        }
        if (g == 0) {
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if (per_piece) {
              *reinterpret_cast<float2*>(xsum + (size_t)(2 * kt) * TOK + i * 8 + 2 * t) =
                  make_float2(xs[0][i][0], xs[0][i][1]);
              *reinterpret_cast<float2*>(xsum + (size_t)(2 * kt + 1) * TOK + i * 8 + 2 * t) =
                  make_float2(xs[1][i][0], xs[1][i][1]);
            } else {
              *reinterpret_cast<float2*>(xsum + (size_t)kt * TOK + i * 8 + 2 * t) =
                  make_float2(xs[0][i][0] + xs[1][i][0], xs[0][i][1] + xs[1][i][1]);
            }
          }
        }
      }
      named_bar_sync(15, NCW * 32);
    }

    int cs = 0;          // ring slot of the next stage
    unsigned cpar = 0;   // parity of the current pass over the ring
    int cgrp = 0;        // consumer group whose turn it is
    for (int ui = 0; ui < my_units; ++ui) {
      int n0 = ((int)blockIdx.x + ui * (int)gridDim.x) * 16;
      __half* out = a.out;
      int rows = a.n;
      if constexpr (GROUPED) {
        if (paired) {
          n0 = ((int)blockIdx.x + (ui >> 1) * (int)gridDim.x) * 16;
          out = p.prob[0].out;
          rows = p.prob[0].n;
        } else {
          const int gu = (int)blockIdx.x + ui * (int)gridDim.x, pi = ring_locate(p, gu);
          n0 = (gu - p.prob[pi].unit0) * 16;
          out = p.prob[pi].out;
          rows = p.prob[pi].n;
        }
      }
      float d[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) d[i][j] = 0.0f;
      // m <= 8: one warp per unit, in rotation, adds the partial sums and writes the unit's
      // 16 x m outputs; lane l takes outputs l, l + 32, ... (output e = token * 16 + row).
      // m > 8: every consumer thread takes one output.  Either way the old output values are
      // requested now, so that their latency is hidden behind the unit's stages.
      // (the rotation relies on every stage being released by all consumer warps, i.e. one group)
      constexpr bool ROTATE = MT == 1 && NG == 1;
      const bool summer = ROTATE ? (ui % NCW) == cw : true;
      constexpr int OPL = ROTATE ? 16 * TOK / 32 : 1;  // outputs per summing thread
      // (kept as loaded: a conversion here would make the warp wait for the loads at once,
      // and with it the seven warps that share its ring stages)
      unsigned short old[OPL];
      const bool fused_ar = FUSE && p.ar_world > 1;
      if (summer && !fused_ar) {
#pragma unroll
        for (int j = 0; j < OPL; ++j) {
          const int e = ROTATE ? lane + 32 * j : tid - 32, row = e & 15, tok = e >> 4;
          old[j] = (tok < a.m && n0 + row < rows && !paired && !(FUSE && p.rope_width > 0))
                       ? reinterpret_cast<const unsigned short*>(out)[(size_t)tok * rows + n0 + row]
                       : (unsigned short)0;
        }
      }
      for (int st = 0; st < p.spu; ++st) {
        const int s = cs;
        const unsigned par = cpar;
        const bool mine = NG == 1 || cgrp == grp;
        if (++cs == p.NS) cs = 0, cpar ^= 1u;
        if (NG > 1 && ++cgrp == NG) cgrp = 0;
        if (!mine) continue;  // another group's stage
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[s], par) && !*abort_flag);
        const int kt = st * RING_TILES + tile;
        if (ok && kt < ntiles) {
          const uint8_t* stage = ring + (size_t)s * p.stage_bytes;
          const uint8_t* trow = stage + tile * RING_TILE_BYTES + pg * 128;
          if constexpr (XR) {
            xa = stage + RING_STAGE_BYTES + (size_t)g * p.xss;
            xb = stage + RING_STAGE_BYTES + (size_t)(g + 8) * p.xss;
          }
          const __half* stab = reinterpret_cast<const __half*>(stage + RING_W_BYTES);
          // d += s * ((acc0 + acc1) - (1024 + z) * sum x) for scale group `gi` of the stage,
          // whose activation sums are entry `xe` of the table
          auto correct = [&](int gi, int xe, int h0, int h1) {  // pieces h0..h1 were accumulated
            const float sa = __half2float(stab[pg * p.gps + gi]);
            const float sb = __half2float(stab[(pg + 8) * p.gps + gi]);
            float ca = 1151.5f, cb = 1151.5f;
            if (HAS_ZERO) {
              ca = 1024.0f + __half2float(stab[16 * p.gps + pg * p.gps + gi]);
              cb = 1024.0f + __half2float(stab[16 * p.gps + (pg + 8) * p.gps + gi]);
            }
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              float2 xv;
              if constexpr (XS_INLINE) {
                xv = make_float2(xs[h0][i][0], xs[h0][i][1]);
                if (h0 != h1) xv.x += xs[h1][i][0], xv.y += xs[h1][i][1];
              } else {
                xv = *reinterpret_cast<const float2*>(xsum + (size_t)xe * TOK + i * 8 + 2 * t);
              }
              float sum[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                sum[j] = acc[0][0][i][j] + acc[0][1][i][j];
                if (h0 == 1) sum[j] = acc[1][0][i][j] + acc[1][1][i][j];
                else if (h1 == 1) sum[j] += acc[1][0][i][j] + acc[1][1][i][j];
              }
              d[i][0] = fmaf(sa, fmaf(-ca, xv.x, sum[0]), d[i][0]);
              d[i][1] = fmaf(sa, fmaf(-ca, xv.y, sum[1]), d[i][1]);
              d[i][2] = fmaf(sb, fmaf(-cb, xv.x, sum[2]), d[i][2]);
              d[i][3] = fmaf(sb, fmaf(-cb, xv.y, sum[3]), d[i][3]);
            }
          };
          // piece h: the 16 bytes at logical offset (t + 4h) * 16 of the 128-byte row
          const int xoff = (XR ? tile : kt) * 256 + t * 32;
          compute_piece(trow + ((t ^ pg) * 16), xoff, std::integral_constant<int, 0>{});
          compute_piece(trow + (((t + 4) ^ pg) * 16), xoff + 128, std::integral_constant<int, 1>{});
          if (per_piece) {
            correct(2 * tile, 2 * kt, 0, 0);
            correct(2 * tile + 1, 2 * kt + 1, 1, 1);
          } else {
            correct(tile, kt, 0, 1);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // also on failure, so that the producer can finish
      }
      // ---- add the partial sums of all consumer warps in warp order, write 16 columns ----
      // The other warps only announce their partial sums and go on to the next unit.  Buffer
      // and barrier `ui % RING_RED_BUFS` are reused four units later; a warp cannot be that
      // far ahead of the summing warp, because the ring (at most 4 * spu - 1 stages, see
      // plan_ring) refills a stage only after all eight warps have released it.
      const int rbuf = ui & (RBUFS - 1);
      float* rb = red + (size_t)rbuf * NCW * 16 * RED_LD;
      {
        float* rw = rb + (size_t)cw * 16 * RED_LD;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          rw[pg * RED_LD + i * 8 + 2 * t] = d[i][0];
          rw[pg * RED_LD + i * 8 + 2 * t + 1] = d[i][1];
          rw[(pg + 8) * RED_LD + i * 8 + 2 * t] = d[i][2];
          rw[(pg + 8) * RED_LD + i * 8 + 2 * t + 1] = d[i][3];
        }
      }
      if (!summer) {
        __threadfence_block();  // the partial sums are visible before the arrival is counted
        __syncwarp();
        named_bar_arrive(1 + rbuf, NCW * 32);
      } else {
        named_bar_sync(1 + rbuf, NCW * 32);
        if (FUSE && p.rope_width > 0) {
          // ---- rotary embedding + cache append on the way out (decode_rope_append's arithmetic on
          // the fp16-rounded products).  Columns come in (even, odd) pairs held by neighbouring
          // lanes; a unit of 16 columns lies inside one of the q, k, v sections.
          const int pos = *p.rope_pos;
          const int sect = n0 / p.rope_width, c0 = n0 - sect * p.rope_width;
          const int head_dim = p.rope_width / p.rope_heads;
#pragma unroll
          for (int j = 0; j < OPL; ++j) {
            const int e = ROTATE ? lane + 32 * j : tid - 32, row = e & 15, tok = e >> 4;
            float v = 0.0f;
            if (tok < a.m) {
#pragma unroll
              for (int w = 0; w < NCW; ++w) v += rb[(size_t)w * 16 * RED_LD + row * RED_LD + tok];
            }
            const __half mine = __float2half_rn(v);
            const __half other = __ushort_as_half(
                (unsigned short)__shfl_xor_sync(0xffffffffu, (unsigned int)__half_as_ushort(mine), 1));
            if (tok < a.m && pos >= 0 && pos < p.rope_max_seq) {
              const int col = c0 + row;
              __half res = mine;
              if (sect < 2) {
                const __half2 turned = (row & 1) ? rope_apply(other, mine, rope_turn(pos, (col - 1) % head_dim, head_dim, p.rope_theta))
                                                 : rope_apply(mine, other, rope_turn(pos, col % head_dim, head_dim, p.rope_theta));
                res = (row & 1) ? __high2half(turned) : __low2half(turned);
              }
              if (sect == 0) out[(size_t)tok * p.rope_q_pitch + col] = res;
              else if (sect == 1) p.rope_k_cache[((size_t)tok * p.rope_max_seq + pos) * p.rope_width + col] = res;
              else p.rope_v_cache[((size_t)tok * p.rope_max_seq + pos) * p.rope_width + col] = res;
            }
          }
        } else
#pragma unroll
        for (int j = 0; j < OPL; ++j) {
          const int e = ROTATE ? lane + 32 * j : tid - 32, row = e & 15, tok = e >> 4;
          if (tok < a.m && n0 + row < rows) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < NCW; ++w) v += rb[(size_t)w * 16 * RED_LD + row * RED_LD + tok];
            if (GROUPED && paired) {
              // gate unit: keep fp16(gate) for the warp that finishes the up unit (it cannot get
              // there before this warp has announced its partial sums of the up unit, which it
              // does after these stores); up unit: SiluMul with the arithmetic of the
              // elementwise kernel
              unsigned short* pb = pairbuf + ((ui >> 1) & 1) * 16 * TOK;
              if (!(ui & 1)) {
                pb[e] = __half_as_ushort(__float2half_rn(v));
              } else {
                const float gf = __half2float(__ushort_as_half(pb[e]));
                const float uf = __half2float(__float2half_rn(v));
                out[(size_t)tok * rows + n0 + row] = __float2half(gf / (1.0f + expf(-gf)) * uf);
              }
            } else if (!fused_ar) {
              out[(size_t)tok * rows + n0 + row] =
                  __float2half_rn(fmaf(a.beta, __half2float(__ushort_as_half(old[j])), v));
            } else {
              // this rank's partial result goes into slot ar_rank of every rank's inbox (peer
              // stores; 16 lanes cover 32 contiguous bytes of one token's row)
              const __half hv = __float2half_rn(v);
              const size_t off = ((size_t)p.ar_rank * a.m + tok) * a.n + n0 + row;
              for (int r = 0; r < p.ar_world; ++r) p.ar_inbox[r][off] = hv;
            }
          }
        }
      }
    }
    if (FUSE && p.ar_world > 1) {
      // ---- fused all-reduce.  CTA c of every rank works on the same units, so it needs only
      // the partial results pushed by CTA c of the peers: make this CTA's pushes visible, tell
      // CTA c of every peer, wait (bounded) for theirs, then add the world slots of this rank's
      // own inbox in rank order (plus the residual) for the units of this CTA.
      // (the word after the abort flag in the barrier area: no static shared memory, which
      // would push the dynamic area past half an SM)
      volatile unsigned int* s_ar_epoch = reinterpret_cast<volatile unsigned int*>(abort_flag + 1);
      __threadfence_system();
      if (tid == 32) {
        const unsigned int e = p.ar_epochs[blockIdx.x] + 1u;
        p.ar_epochs[blockIdx.x] = e;
        *s_ar_epoch = e;
      }
      named_bar_sync(14, NCW * 32);
      const unsigned int epoch = *s_ar_epoch;
      const int pe = tid - 32;
      if (pe < p.ar_world) {
        st_release_sys_u32(p.ar_flags[pe] + (size_t)blockIdx.x * p.ar_world + p.ar_rank, epoch);
        const unsigned int* mine = p.ar_flags[p.ar_rank] + (size_t)blockIdx.x * p.ar_world + pe;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys_u32(mine) - epoch) < 0) {
          if (clock64() - t0 > p.ar_wait_cycles) {
            atomicOr(p.status, 256u);
            break;
          }
        }
        __threadfence_system();
      }
      named_bar_sync(14, NCW * 32);
      const __half* box = p.ar_inbox[p.ar_rank];
      const size_t slot = (size_t)a.m * a.n;
      for (int ui = 0; ui < my_units; ++ui) {
        const int n0 = ((int)blockIdx.x + ui * (int)gridDim.x) * 16;
        for (int e = pe; e < 16 * a.m; e += NCW * 32) {
          const int row = e & 15, tok = e >> 4;
          if (n0 + row < a.n) {
            const size_t off = (size_t)tok * a.n + n0 + row;
            float v = p.ar_residual ? __half2float(a.out[off]) : 0.0f;
            for (int r = 0; r < p.ar_world; ++r)
              v += __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(box + r * slot + off))));
            a.out[off] = __float2half_rn(v);
          }
        }
      }
    }
    if (!ok && lane == 0) atomicOr(p.status, 1u);
  }
}

struct RingPlan {
  int NS, XS, gps, shift, ncw, xsum_entries, cps, xr, stage_bytes, xss, rbufs;
  size_t smem;
};

// `extra`: bytes of shared memory the launch needs beyond the usual areas (paired form).
bool plan_ring(const adr_ctx* ctx, const U8Args& a, RingPlan& pl, size_t extra = 0) {
  if (a.m < 1 || a.m > 16 || a.p % 128 != 0 || a.n < 16) return false;
  if (a.block_size != 64 && a.block_size != 128) return false;
  if (a.p % a.block_size != 0 || ((a.p / a.block_size) & 1)) return false;  // 4-byte scale copies
  if (a.p > 65536) return false;  // one bulk copy per activation row
  if ((reinterpret_cast<uintptr_t>(a.rhs) & 15u) || (reinterpret_cast<uintptr_t>(a.lhs) & 15u) ||
      (reinterpret_cast<uintptr_t>(a.scales) & 3u) ||
      (a.zeros && (reinterpret_cast<uintptr_t>(a.zeros) & 3u)))
    return false;
  if (!ctx->encode_tiled_fn) return false;
  const int tok = a.m > 8 ? 16 : 8;
  pl.ncw = 8;  // two CTAs (this launch and an early successor) fit an SM's registers
  pl.XS = a.p * 2 + 16;
  pl.gps = 1024 / a.block_size;
  pl.shift = a.block_size == 64 ? 6 : 7;
  pl.xsum_entries = (a.p / 128) * (a.block_size == 64 ? 2 : 1);
  auto fixed_for = [&](int rbufs) {
    return (size_t)a.m * pl.XS + (size_t)rbufs * pl.ncw * 16 * (tok + 1) * 4 +
           (size_t)pl.xsum_entries * tok * 4 + (2 * RING_MAX_STAGES + 2) * 8 + extra;
  };
  pl.rbufs = a.m > 8 ? 2 : RING_RED_BUFS;
  size_t fixed = fixed_for(pl.rbufs);
  const int spu = (a.p / 128 + RING_TILES - 1) / RING_TILES;
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const int units = (a.n + 15) / 16;
  const size_t half = 113 * 1024, all = 224 * 1024;
  // Shared memory per CTA.  Half an SM's worth lets a second CTA run beside this one: a
  // second CTA of this launch when there are one or two tokens and at least four units per
  // CTA (sixteen consumer warps per SM hide the latency of the arithmetic better than eight),
  // else the first CTAs of the next launch, started early under programmatic dependent
  // launch.  When half an SM leaves fewer than five stages, one CTA takes all of it.
  int ns_half = fixed < half ? (int)((half - fixed) / RING_STAGE_BYTES) : 0;
  int half_min = 5;
  if (a.m > 2 && a.m <= 8 && ns_half < 5) {
    // A few tokens more and the activations crowd the ring out of half an SM.  Two partial-sum
    // buffers instead of four win a stage back, and four stages beside an early successor
    // measured better than ten without one.
    const size_t f2 = fixed_for(2);
    const int nh2 = f2 < half ? (int)((half - f2) / RING_STAGE_BYTES) : 0;
    if (nh2 >= 4 && nh2 <= 2 * spu - 1) {
      pl.rbufs = 2;
      fixed = f2;
      ns_half = nh2;
      half_min = 4;
    }
  }
  int ns;
  pl.cps = 1;
  const int cps_m = ctx->tune_u8_cps_m.load(), cps_x4 = ctx->tune_u8_cps_x4.load();
  if (a.m <= cps_m && units * 4 >= cps_x4 * sms && ns_half >= 4) {
    pl.cps = 2;
    ns = ns_half;
  } else if (ns_half >= half_min) {
    ns = ns_half;
  } else {
    ns = fixed < all ? (int)((all - fixed) / RING_STAGE_BYTES) : 0;
  }
  ns = std::min(ns, RING_MAX_STAGES);
  if (a.m <= 8) ns = std::min(ns, pl.rbufs * spu - 1);  // keeps the rotation of partial-sum buffers safe
  pl.xr = 0;
  pl.stage_bytes = RING_STAGE_BYTES;
  pl.xss = 0;
  if (a.norm_w != nullptr) {
    // the fused rms_norm rewrites resident activations: no streamed-activation form, 16-byte rows
    if (ns < 3 || a.p % 8 != 0 || (reinterpret_cast<uintptr_t>(a.norm_w) & 15u)) return false;
  } else if (ns < 4) {
    // The activations leave too little room for a ring (or none): stream them through the ring
    // with the weights instead, 1024 k per stage and token (rows padded by 16 bytes so that the
    // fragment loads of different tokens fall in different banks).
    const int xss = 2048 + 16;
    const int stage = (RING_STAGE_BYTES + a.m * xss + 1023) & ~1023;
    const int rb_xr = a.m > 8 ? 2 : RING_RED_BUFS;
    const size_t fixed_xr = (size_t)rb_xr * pl.ncw * 16 * (tok + 1) * 4 +
                            (2 * RING_MAX_STAGES + 2) * 8;
    int ns_xr = (int)((all - fixed_xr) / stage);
    ns_xr = std::min(ns_xr, RING_MAX_STAGES);
    if (a.m <= 8) ns_xr = std::min(ns_xr, RING_RED_BUFS * spu - 1);
    if (ns_xr >= 3 && ns_xr > ns) {
      pl.rbufs = rb_xr;
      pl.xr = 1;
      pl.cps = 1;
      pl.stage_bytes = stage;
      pl.xss = xss;
      pl.NS = ns_xr;
      pl.smem = (size_t)ns_xr * stage + fixed_xr;
      return true;
    }
  }
  if (ns < 3) return false;
  pl.NS = ns;
  pl.smem = (size_t)ns * RING_STAGE_BYTES + fixed;
  return true;
}

// `grp` (grouped form): the matrices of the launch; `a` then carries the common arguments and
// n = 16 x the total number of units.
template <int MT, bool Z, bool PDL, int NCW, bool XR, bool FUSE, bool XSI, bool G = false>
int launch_ring_f(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const RingPlan& pl,
                  const RingArFuse* ar, const RingGroup* grp = nullptr, const RingRope* rope = nullptr) {
  auto kfn = u8_ring_kernel<MT, NCW, Z, PDL, XR, FUSE, XSI, G>;
  cudaError_t e;
  if (int rc0 = opt_in_smem(ctx, kfn, 226 * 1024); rc0 != ADR_OK) return rc0;
  // weights as (k within tile, row, k-tile): a box of 128 x 16 x 8 lands as eight tiles of
  // [16 rows][128 bytes], each swizzled by its own row index
  RingMaps maps;
  RingParams p;
  p.nprob = 1;
  p.wide_ok = 1;
  p.pair = 0;
  const uint64_t strides[2] = {(uint64_t)a.p, 128u};
  const uint32_t box[3] = {128u, 16u, (uint32_t)RING_TILES};
  int units_total = (a.n + 15) / 16;
  if (G) {
    units_total = 0;
    p.nprob = grp->count;
    for (int i = 0; i < grp->count; ++i) {
      const uint64_t dims[3] = {128u, (uint64_t)grp->n[i], (uint64_t)(a.p / 128)};
      int rc = tma_get(ctx, &maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, grp->rhs[i], dims, strides,
                       box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != ADR_OK) return rc;
      p.prob[i] = RingProblem{grp->scales[i], Z ? grp->zeros[i] : nullptr, grp->out[i], grp->n[i],
                              units_total};
      units_total += (grp->n[i] + 15) / 16;
      if ((reinterpret_cast<uintptr_t>(grp->scales[i]) & 15u) ||
          (Z && (reinterpret_cast<uintptr_t>(grp->zeros[i]) & 15u)))
        p.wide_ok = 0;
    }
    for (int i = grp->count; i < RING_MAX_PROBLEMS; ++i) {
      maps.m[i] = maps.m[0];
      p.prob[i] = p.prob[0];
    }
    if (grp->pair) {
      p.pair = 1;
      units_total = (grp->n[0] + 15) / 16;  // pairs
    }
  } else {
    const uint64_t dims[3] = {128u, (uint64_t)a.n, (uint64_t)(a.p / 128)};
    int rc = tma_get(ctx, &maps.m[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.rhs, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != ADR_OK) return rc;
    for (int i = 1; i < RING_MAX_PROBLEMS; ++i) maps.m[i] = maps.m[0];
    for (int i = 0; i < RING_MAX_PROBLEMS; ++i)
      p.prob[i] = RingProblem{a.scales, a.zeros, a.out, a.n, 0};
  }
  p.a = a;
  p.NS = pl.NS;
  p.XS = pl.XS;
  p.gps = pl.gps;
  p.bs_shift = pl.shift;
  p.units = units_total;
  p.spu = (a.p / 128 + RING_TILES - 1) / RING_TILES;
  p.xsum_entries = pl.xsum_entries;
  p.stage_bytes = pl.stage_bytes;
  p.xss = pl.xss;
  p.rbufs = pl.rbufs;
  p.status = ctx->d_status;
  p.norm_w = a.norm_w;
  p.norm_eps = a.norm_eps;
  p.rope_width = 0;
  if (rope) {
    p.rope_width = rope->width;
    p.rope_heads = rope->n_heads;
    p.rope_max_seq = rope->max_seq;
    p.rope_q_pitch = rope->q_pitch;
    p.rope_pos = rope->pos;
    p.rope_theta = rope->theta;
    p.rope_k_cache = rope->k_cache;
    p.rope_v_cache = rope->v_cache;
  }
  p.ar_world = 0;
  p.ar_wait_cycles = peer_wait_cycles(ctx);
  if (ar) {
    for (int r = 0; r < ar->world; ++r) {
      p.ar_inbox[r] = ar->inbox[r];
      p.ar_flags[r] = ar->flags[r];
    }
    p.ar_epochs = ar->epochs;
    p.ar_rank = ar->rank;
    p.ar_world = ar->world;
    p.ar_residual = ar->residual;
  }
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  cudaLaunchConfig_t cfg = {};
  const int grid = std::min(p.units, sms * pl.cps);
  if (ar && grid > ar->max_ctas) return ADR_ERR_SHAPE;  // the flag arrays do not cover this grid
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3((NCW + 1) * 32, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // CTAs of half an SM's size rely on landing one per SM, each beside a CTA of the launch
  // before.  Behind a launch that filled whole SMs (two CTAs each, or one large CTA) they would
  // start as those SMs drain, two to an SM on the first half of the SMs to finish, and every
  // later launch of the chain would inherit that placement: each one running on half the SMs,
  // a quarter slower.  So the first such launch behind a filling launch gives up its early
  // start and begins on an empty GPU, which spreads its CTAs one per SM again.
  // (Other kernels of this library that fill the SMs — the cluster k-split kernel, decode
  // attention over many heads — leave the same mark; small kernels in between pass it on.)
  const int fill_kind = pl.cps == 2 ? 1 : (pl.smem > 114 * 1024 ? 2 : 0);
  bool early = PDL;
  if (PDL && fill_kind == 0 && behind_filling_launch(ctx, stream)) early = false;
  if (PDL && !early) ctx->fill_flag = 0;  // this launch waits for everything before it: the GPU runs empty
  cfg.numAttrs = early ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kfn, maps, p);
  if (e != cudaSuccess) {
    ctx->last_cuda_error = (int)e;
    return ADR_ERR_CUDA;
  }
  if (fill_kind) note_filling_launch(ctx, stream, fill_kind);
  ctx->small_before = 0;
  return after_launch(ctx);
}

template <int MT, bool Z, bool PDL, int NCW, bool XR>
int launch_ring_p(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const RingPlan& pl,
                  const RingArFuse* ar, const RingRope* rope) {
  // Two to eight tokens: the activation sums ride along in the main loop (measured 3-9 %
  // quicker than making the table first); one token, or more than eight, make the table (3 %
  // quicker: the loop is the bottleneck there).
  if constexpr (MT == 1 && !XR) {
    if (a.m >= 2) {
      if (ar != nullptr || a.norm_w != nullptr || rope != nullptr)
        return launch_ring_f<MT, Z, PDL, NCW, XR, true, true>(ctx, stream, a, pl, ar, nullptr, rope);
      return launch_ring_f<MT, Z, PDL, NCW, XR, false, true>(ctx, stream, a, pl, ar);
    }
  }
  if (ar != nullptr || a.norm_w != nullptr || rope != nullptr)
    return launch_ring_f<MT, Z, PDL, NCW, XR, true, false>(ctx, stream, a, pl, ar, nullptr, rope);
  return launch_ring_f<MT, Z, PDL, NCW, XR, false, false>(ctx, stream, a, pl, ar);
}

}  // namespace

// Several matrices with the same activations in one launch; ADR_ERR_SHAPE when the ring kernel
// does not take them with the activations resident (the caller then makes separate calls).
int launch_u8_ring_grouped(adr_ctx* ctx, cudaStream_t stream, const U8Args& common,
                           const RingGroup& grp) {
  if (grp.count < 1 || grp.count > RING_MAX_PROBLEMS) return ADR_ERR_INVALID;
  int units = 0;
  bool z = grp.zeros[0] != nullptr;
  for (int i = 0; i < grp.count; ++i) {
    if (!grp.rhs[i] || !grp.scales[i] || !grp.out[i] || grp.n[i] < 16) return ADR_ERR_SHAPE;
    if ((grp.zeros[i] != nullptr) != z) return ADR_ERR_INVALID;  // all with zero points, or none
    if ((reinterpret_cast<uintptr_t>(grp.rhs[i]) & 15u) || (reinterpret_cast<uintptr_t>(grp.scales[i]) & 3u) ||
        (z && (reinterpret_cast<uintptr_t>(grp.zeros[i]) & 3u)))
      return ADR_ERR_SHAPE;
    units += (grp.n[i] + 15) / 16;
  }
  U8Args a = common;
  a.rhs = grp.rhs[0];
  a.scales = grp.scales[0];
  a.zeros = grp.zeros[0];
  a.out = grp.out[0];
  a.n = units * 16;
  a.norm_w = nullptr;
  if (grp.pair && (grp.count != 2 || grp.n[0] != grp.n[1] || common.beta != 0.0f)) return ADR_ERR_INVALID;
  RingPlan pl;
  if (!plan_ring(ctx, a, pl, grp.pair ? 2 * 16 * 16 * 2 + 16 : 0) || pl.xr) return ADR_ERR_SHAPE;
  const bool two = a.m > 8, pdl = ctx->tune_pdl != 0, xsi = !two && a.m >= 2;
#define ADR_RING_G(MT, Z, XSI)                                                                        \
  return pdl ? launch_ring_f<MT, Z, true, 8, false, false, XSI, true>(ctx, stream, a, pl, nullptr, &grp) \
             : launch_ring_f<MT, Z, false, 8, false, false, XSI, true>(ctx, stream, a, pl, nullptr, &grp)
  if (two) {
    if (z) { ADR_RING_G(2, true, false); }
    ADR_RING_G(2, false, false);
  }
  if (xsi) {
    if (z) { ADR_RING_G(1, true, true); }
    ADR_RING_G(1, false, true);
  }
  if (z) { ADR_RING_G(1, true, false); }
  ADR_RING_G(1, false, false);
#undef ADR_RING_G
}

bool u8_ring_supports(const adr_ctx* ctx, const U8Args& a) {
  RingPlan pl;
  return plan_ring(ctx, a, pl);
}

int launch_u8_ring(adr_ctx* ctx, cudaStream_t stream, const U8Args& a, const RingArFuse* ar,
                   const RingRope* rope) {
  RingPlan pl;
  if (!plan_ring(ctx, a, pl)) return ADR_ERR_SHAPE;
  if (rope && (pl.xr || a.beta != 0.0f)) return ADR_ERR_SHAPE;
  const bool z = a.zeros != nullptr, two = a.m > 8, pdl = ctx->tune_pdl != 0;
#define ADR_RING_CASE(MT, Z)                                                       \
  if (pl.xr)                                                                       \
    return pdl ? launch_ring_p<MT, Z, true, 8, true>(ctx, stream, a, pl, ar, rope)       \
               : launch_ring_p<MT, Z, false, 8, true>(ctx, stream, a, pl, ar, rope);     \
  return pdl ? launch_ring_p<MT, Z, true, 8, false>(ctx, stream, a, pl, ar, rope)        \
             : launch_ring_p<MT, Z, false, 8, false>(ctx, stream, a, pl, ar, rope)
  if (two) {
    if (z) { ADR_RING_CASE(2, true); }
    ADR_RING_CASE(2, false);
  }
  if (z) { ADR_RING_CASE(1, true); }
  ADR_RING_CASE(1, false);
#undef ADR_RING_CASE
}

}  // namespace adr
