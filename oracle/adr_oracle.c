/*
 * CPU oracle for the adrastea matmul hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's device
 * kernels so that the CUDA library can be checked against it.  Nothing in the
 * product path links, loads or calls it; only the test-suite, the smoke check
 * and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: the restatements of the device kernels are pinned against
 * the reference's own kernels (compiled unmodified from the reference tree by
 * oracle/Makefile and executed on a B200) through the fixtures under
 * tests/golden/.  orc_sgemm restates the call convention of the reference's
 * only host matmul (crate matrixmultiply 0.3.7, feature "threading", called
 * at adrastea_core/src/mel.rs:140-158); that crate is not vendored in the
 * reference tree and no reference test pins its output: PARITY UNPINNED for
 * orc_sgemm, which is therefore used only as a timed CPU baseline.
 *
 * Each function cites the reference lines it follows (paths are relative to
 * the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_OK 0
#define ORC_ERR_UNSUPPORTED 3

/* ------------------------------------------------------------------------ */
/* fp16 helpers.  _Float16 conversions in gcc are correctly rounded          */
/* (round-to-nearest-even, subnormals kept), from float and from double.     */
/* ------------------------------------------------------------------------ */
typedef uint16_t h16;

static inline float h2f(h16 h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline h16 f2h(float f) {
  _Float16 v = (_Float16)f;
  h16 h;
  memcpy(&h, &v, 2);
  return h;
}
static inline h16 d2h(double d) {
  _Float16 v = (_Float16)d;
  h16 h;
  memcpy(&h, &v, 2);
  return h;
}
/* __half * __half: the exact product of two fp16 values fits in fp32
 * (22 significant bits), so one rounding to fp16 gives the device result. */
static inline h16 hmul(h16 a, h16 b) { return f2h(h2f(a) * h2f(b)); }
/* __half + __half: the exact sum fits in a double. */
static inline h16 hadd(h16 a, h16 b) { return d2h((double)h2f(a) + (double)h2f(b)); }

h16 orc_f32_to_f16(float f) { return f2h(f); }
float orc_f16_to_f32(h16 h) { return h2f(h); }
h16 orc_f64_to_f16(double d) { return d2h(d); }
h16 orc_hmul(h16 a, h16 b) { return hmul(a, b); }
h16 orc_hadd(h16 a, h16 b) { return hadd(a, b); }

/* Enum values of adrastea_kernels/cpp/matmul.cu:26-36 (mirrored by
 * adrastea_models/src/kernels.rs:80-139). */
enum { LOAD_IDENTITY = 0, LOAD_SCALE = 1 };
enum {
  STORE_IDENTITY = 0,
  STORE_GELU_BIAS = 1,
  STORE_BETA_GELU_BIAS = 2,
  STORE_BETA_BIAS = 3,
  STORE_SCALE = 4,
  STORE_ADD = 5,
  STORE_QUICK_GELU_BIAS = 6
};
enum { MASK_NONE = 0, MASK_CAUSAL = 1 };

static inline float gelu_tanh(float t) {
  /* matmul.cu:119-121 */
  return 0.5f * t * (1.0f + tanhf(0.7978845608028654f * (t + 0.044715f * t * t * t)));
}
static inline float quick_gelu(float t) {
  /* matmul.cu:127-129, 143-144 */
  return t * (1.0f / (1.0f + expf(-1.702f * t)));
}

/*
 * The store functors of matmul.cu:45-176 as dispatched by matmul.cu:444-491.
 * `sum` is the fp32 accumulator; every functor chain starts by converting it
 * to __half (the functors take `__half const& value`).  `old` is the value
 * already at the output location.  beta*old + inner is evaluated with one
 * rounding (fmaf) as nvcc contracts it; the fixtures from the reference
 * kernels confirm that choice.
 */
static inline h16 store_apply(int store, float sum, h16 old, h16 bias, float beta, float scale) {
  h16 hs = f2h(sum);
  switch (store) {
    case STORE_IDENTITY:
      return hs;
    case STORE_SCALE: /* Scale<half>: half * half(scale), matmul.cu:63-73 */
      return hmul(hs, f2h(scale));
    case STORE_ADD: /* Add<half,half>: half + half, matmul.cu:163-176 */
      return hadd(hs, old);
    case STORE_BETA_BIAS: {
      float t = h2f(hs) + h2f(bias);
      return f2h(fmaf(beta, h2f(old), t));
    }
    case STORE_BETA_GELU_BIAS: {
      float t = gelu_tanh(h2f(hs) + h2f(bias));
      return f2h(fmaf(beta, h2f(old), t));
    }
    case STORE_QUICK_GELU_BIAS: {
      return f2h(quick_gelu(h2f(hs) + h2f(bias)));
    }
    default:
      return 0;
  }
}

static int store_supported(int store) {
  /* GELU_BIAS has an enum value but no device case: the reference traps
   * (matmul.cu:489-490).  The oracle reports it as unsupported. */
  return store == STORE_IDENTITY || store == STORE_BETA_GELU_BIAS || store == STORE_BETA_BIAS ||
         store == STORE_SCALE || store == STORE_ADD || store == STORE_QUICK_GELU_BIAS;
}

/*
 * Reference-faithful restatement of matmul_f16 / matmul_f16_fast
 * (matmul.cu:195-222 and 236-416; both sum the same fp16-rounded products
 * in the same sequential k order, so they agree bit for bit).
 * Parameter order is that of MATMUL_COMMON_PARAMS + the six trailing
 * arguments (matmul.cu:186-190, 493-499).  Strides are in elements.
 * mode 0: products rounded to fp16, fp32 sequential sum (the reference).
 * mode 1: exact products summed in double (the "ideal" tensor-core result),
 *         same epilogue.
 */
static int matmul_f16_impl(int mode, h16* output, const h16* lhs, const h16* rhs, int batches,
                           int m, int k, int n, int stride_ox, int stride_oy, int stride_oz,
                           int stride_lx, int stride_ly, int stride_lz, int stride_rx,
                           int stride_ry, int stride_rz, const h16* bias, float beta, float scale,
                           unsigned store, unsigned load, unsigned mask) {
  if (!store_supported((int)store) || load > LOAD_SCALE || mask > MASK_CAUSAL)
    return ORC_ERR_UNSUPPORTED;
  const h16 hscale = f2h(scale);
  const int need_bias = (store == STORE_BETA_GELU_BIAS || store == STORE_BETA_BIAS ||
                         store == STORE_QUICK_GELU_BIAS);
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batches; ++b) {
    for (int y = 0; y < m; ++y) {
      h16* o = output + (ptrdiff_t)b * stride_oz;
      const h16* l = lhs + (ptrdiff_t)b * stride_lz;
      const h16* r = rhs + (ptrdiff_t)b * stride_rz;
      for (int x = 0; x < n; ++x) {
        h16* dst = o + (ptrdiff_t)y * stride_oy + (ptrdiff_t)x * stride_ox;
        if (mask == MASK_CAUSAL && x > y) { /* matmul.cu:182-184, 210-213 */
          *dst = 0xFC00;                    /* -inf */
          continue;
        }
        float sum;
        if (mode == 0) {
          float s = 0.0f;
          for (int i = 0; i < k; ++i) {
            h16 a = l[(ptrdiff_t)y * stride_ly + (ptrdiff_t)i * stride_lx];
            h16 w = r[(ptrdiff_t)i * stride_ry + (ptrdiff_t)x * stride_rx];
            if (load == LOAD_SCALE) { /* Scale<half> on both operands, matmul.cu:62 */
              a = hmul(a, hscale);
              w = hmul(w, hscale);
            }
            s += h2f(hmul(a, w)); /* matmul.cu:216-217 */
          }
          sum = s;
        } else {
          double s = 0.0;
          for (int i = 0; i < k; ++i) {
            h16 a = l[(ptrdiff_t)y * stride_ly + (ptrdiff_t)i * stride_lx];
            h16 w = r[(ptrdiff_t)i * stride_ry + (ptrdiff_t)x * stride_rx];
            if (load == LOAD_SCALE) {
              a = hmul(a, hscale);
              w = hmul(w, hscale);
            }
            s += (double)h2f(a) * (double)h2f(w);
          }
          sum = (float)s;
        }
        *dst = store_apply((int)store, sum, *dst, need_bias ? bias[x] : 0, beta, scale);
      }
    }
  }
  return ORC_OK;
}

int orc_matmul_f16_ref(h16* output, const h16* lhs, const h16* rhs, int batches, int m, int k,
                       int n, int stride_ox, int stride_oy, int stride_oz, int stride_lx,
                       int stride_ly, int stride_lz, int stride_rx, int stride_ry, int stride_rz,
                       const h16* bias, float beta, float scale, unsigned store, unsigned load,
                       unsigned mask) {
  return matmul_f16_impl(0, output, lhs, rhs, batches, m, k, n, stride_ox, stride_oy, stride_oz,
                         stride_lx, stride_ly, stride_lz, stride_rx, stride_ry, stride_rz, bias,
                         beta, scale, store, load, mask);
}

int orc_matmul_f16_ideal(h16* output, const h16* lhs, const h16* rhs, int batches, int m, int k,
                         int n, int stride_ox, int stride_oy, int stride_oz, int stride_lx,
                         int stride_ly, int stride_lz, int stride_rx, int stride_ry, int stride_rz,
                         const h16* bias, float beta, float scale, unsigned store, unsigned load,
                         unsigned mask) {
  return matmul_f16_impl(1, output, lhs, rhs, batches, m, k, n, stride_ox, stride_oy, stride_oz,
                         stride_lx, stride_ly, stride_lz, stride_rx, stride_ry, stride_rz, bias,
                         beta, scale, store, load, mask);
}

/* ------------------------------------------------------------------------ */
/* u8 absmax layout (quantize.cu:3-56): Q[rows,k] u8 row-major,             */
/* S[rows,k/bs] fp16 row-major, implicit zero point 127.5.                   */
/* ------------------------------------------------------------------------ */

/*
 * dequantize_absmax_one (matmul_nt_wmma_16x128x256_fp16u8.cu:5-7) and
 * dequantize_absmax_uint8 (quantize.cu:46-56): fp16((float(q) - 127.5f) *
 * float(s)).  With `zeros` given (an extension that the reference does not
 * have) the constant 127.5f is replaced by float(zeros[row, group]).
 */
static inline h16 dequant_one(uint8_t q, h16 s, float zero) {
  return f2h(((float)q - zero) * h2f(s));
}

void orc_dequantize_absmax_uint8(h16* out, const h16* scales, const h16* zeros, const uint8_t* q,
                                 int rows, int k, int block_size) {
  const int groups = k / block_size;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    for (int i = 0; i < k; ++i) {
      int g = i / block_size;
      float z = zeros ? h2f(zeros[(size_t)r * groups + g]) : 127.5f;
      out[(size_t)r * k + i] = dequant_one(q[(size_t)r * k + i], scales[(size_t)r * groups + g], z);
    }
  }
}

/*
 * quantize_absmax_uint8 (quantize.cu:3-44): per (row, group):
 *   s = fp16(max|x| / 127.5f);  q = uint8(round(127.5f + float(x) / float(s))).
 * round() is half-away-from-zero; the float->uint8 conversion of the device
 * truncates toward zero and saturates, NaN (an all-zero group: 0/0) gives 0.
 */
void orc_quantize_absmax_uint8(uint8_t* q, h16* scales, const h16* in, int rows, int k,
                               int block_size) {
  const int groups = k / block_size;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    for (int g = 0; g < groups; ++g) {
      float absmax = 0.0f;
      for (int i = g * block_size; i < (g + 1) * block_size; ++i)
        absmax = fmaxf(absmax, fabsf(h2f(in[(size_t)r * k + i])));
      h16 s = f2h(absmax / 127.5f);
      scales[(size_t)r * groups + g] = s;
      float sf = h2f(s);
      for (int i = g * block_size; i < (g + 1) * block_size; ++i) {
        float v = roundf(127.5f + h2f(in[(size_t)r * k + i]) / sf);
        uint8_t o;
        if (!(v == v)) o = 0;
        else if (v <= 0.0f) o = 0;
        else if (v >= 255.0f) o = 255;
        else o = (uint8_t)v;
        q[(size_t)r * k + i] = o;
      }
    }
  }
}

/*
 * matmul_nt_fp16u8 (matmul_nt_fp16u8.cu:4-24), faithful form.  The literal
 * 127.5 there is a double, so each term float(l) * (float(q) - 127.5) *
 * float(s) is evaluated in double and added to a float accumulator
 * (sum = float(double(sum) + term)), sequentially over i.  Output is
 * float sum + beta * float(old), stored as fp16.
 */
void orc_matmul_nt_fp16u8_ref(h16* output, const h16* lhs, const uint8_t* rhs, const h16* scales,
                              int m, int p, int n, int block_size, float beta) {
  const int block_count = p / block_size;
#pragma omp parallel for collapse(2) schedule(static)
  for (int r = 0; r < m; ++r) {
    for (int c = 0; c < n; ++c) {
      float sum = 0.0f;
      for (int i = 0; i < p; ++i) {
        double term = (double)h2f(lhs[(size_t)r * p + i]) *
                      ((double)(float)rhs[(size_t)c * p + i] - 127.5) *
                      (double)h2f(scales[(size_t)c * block_count + i / block_size]);
        sum = (float)((double)sum + term);
      }
      h16* dst = output + (size_t)r * n + c;
      *dst = f2h(fmaf(beta, h2f(*dst), sum));
    }
  }
}

/*
 * Ideal form of the dequantising GEMM, which is what
 * matmul_nt_wmma_16x128x256_fp16u8.cu:12-83 computes on tensor cores: the
 * weight is first rounded to fp16 by dequantize_absmax_one, the products
 * fp16 x fp16 are exact and are accumulated (here in double), and the result
 * is acc + beta * float(old), stored as fp16 (:74-77).  `zeros` NULL means the
 * reference's constant 127.5.
 */
void orc_matmul_nt_fp16u8_ideal(h16* output, const h16* lhs, const uint8_t* rhs, const h16* scales,
                                const h16* zeros, int m, int p, int n, int block_size, float beta) {
  const int block_count = p / block_size;
#pragma omp parallel for collapse(2) schedule(static)
  for (int r = 0; r < m; ++r) {
    for (int c = 0; c < n; ++c) {
      double sum = 0.0;
      for (int i = 0; i < p; ++i) {
        int g = i / block_size;
        float z = zeros ? h2f(zeros[(size_t)c * block_count + g]) : 127.5f;
        h16 w = dequant_one(rhs[(size_t)c * p + i], scales[(size_t)c * block_count + g], z);
        sum += (double)h2f(lhs[(size_t)r * p + i]) * (double)h2f(w);
      }
      h16* dst = output + (size_t)r * n + c;
      *dst = f2h(fmaf(beta, h2f(*dst), (float)sum));
    }
  }
}

/*
 * matmul_nt_wmma_128x64x64 / matmul_nt_wmma_16x128x256
 * (matmul_nt_wmma_128x64x64.cu:8-78, matmul_nt_wmma_16x128x256.cu:8-68):
 * out[m,n] = lhs[m,p] . rhs[n,p]^T + beta * out, contiguous operands, exact
 * products, fp32-class accumulation (double here), fp16 store.
 */
void orc_matmul_nt_f16_ideal(h16* output, const h16* lhs, const h16* rhs, int m, int p, int n,
                             float beta) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int r = 0; r < m; ++r) {
    for (int c = 0; c < n; ++c) {
      double sum = 0.0;
      for (int i = 0; i < p; ++i)
        sum += (double)h2f(lhs[(size_t)r * p + i]) * (double)h2f(rhs[(size_t)c * p + i]);
      h16* dst = output + (size_t)r * n + c;
      *dst = f2h(fmaf(beta, h2f(*dst), (float)sum));
    }
  }
}

/*
 * error_stats (error_stats.cu:13-75): [mean squared error, max |d|, mean |d|]
 * between two fp16 arrays, in fp32-class arithmetic (double here).
 */
void orc_error_stats_f16(float out[3], const h16* a, const h16* b, size_t count) {
  double mse = 0, mae = 0, mx = 0;
  for (size_t i = 0; i < count; ++i) {
    double d = fabs((double)h2f(a[i]) - (double)h2f(b[i]));
    mse += d * d;
    mae += d;
    if (d > mx) mx = d;
  }
  out[0] = (float)(mse / (double)count);
  out[1] = (float)mx;
  out[2] = (float)(mae / (double)count);
}

/* ------------------------------------------------------------------------ */
/* Host f32 GEMM, call convention of matrixmultiply::sgemm as used at        */
/* adrastea_core/src/mel.rs:140-158:  C = alpha * A . B + beta * C with      */
/* A[m,k] (row stride rsa, col stride csa), B[k,n] (rsb, csb), C[m,n]        */
/* (rsc, csc), strides in elements.  Threaded over row blocks of C.          */
/* PARITY UNPINNED (see the header); used as the timed CPU baseline.         */
/* ------------------------------------------------------------------------ */
#define SG_MB 64
#define SG_KB 256

void orc_sgemm(int m, int k, int n, float alpha, const float* a, ptrdiff_t rsa, ptrdiff_t csa,
               const float* b, ptrdiff_t rsb, ptrdiff_t csb, float beta, float* c, ptrdiff_t rsc,
               ptrdiff_t csc) {
  if (m <= 0 || n <= 0) return;
  /* Fast path 1: B row-major (csb == 1), C row-major: axpy form, vectorises along n. */
  if (csb == 1 && csc == 1) {
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    /* split n across threads when m is small so that every core streams B */
    int split_n = (m < nthreads * 4);
    if (split_n) {
      int chunks = nthreads;
      int per = ((n + chunks - 1) / chunks + 15) & ~15;
#pragma omp parallel for schedule(static)
      for (int t = 0; t < chunks; ++t) {
        int j0 = t * per, j1 = j0 + per > n ? n : j0 + per;
        if (j0 >= j1) continue;
        for (int i = 0; i < m; ++i) {
          float* ci = c + i * rsc;
          if (beta == 0.0f) for (int j = j0; j < j1; ++j) ci[j] = 0.0f;
          else for (int j = j0; j < j1; ++j) ci[j] *= beta;
        }
        for (int k0 = 0; k0 < k; k0 += SG_KB) {
          int k1 = k0 + SG_KB > k ? k : k0 + SG_KB;
          for (int i = 0; i < m; ++i) {
            float* ci = c + i * rsc;
            for (int kk = k0; kk < k1; ++kk) {
              float av = alpha * a[i * rsa + kk * csa];
              const float* bk = b + kk * rsb;
#pragma omp simd
              for (int j = j0; j < j1; ++j) ci[j] += av * bk[j];
            }
          }
        }
      }
      return;
    }
#pragma omp parallel for schedule(dynamic)
    for (int i0 = 0; i0 < m; i0 += 4) {
      int i1 = i0 + 4 > m ? m : i0 + 4;
      for (int i = i0; i < i1; ++i) {
        float* ci = c + i * rsc;
        if (beta == 0.0f) for (int j = 0; j < n; ++j) ci[j] = 0.0f;
        else for (int j = 0; j < n; ++j) ci[j] *= beta;
      }
      for (int k0 = 0; k0 < k; k0 += SG_KB) {
        int k1 = k0 + SG_KB > k ? k : k0 + SG_KB;
        for (int i = i0; i < i1; ++i) {
          float* ci = c + i * rsc;
          for (int kk = k0; kk < k1; ++kk) {
            float av = alpha * a[i * rsa + kk * csa];
            const float* bk = b + kk * rsb;
#pragma omp simd
            for (int j = 0; j < n; ++j) ci[j] += av * bk[j];
          }
        }
      }
    }
    return;
  }
  /* Fast path 2: A and B both contiguous along k (the "NT" weight layout):
   * dot-product form, vectorises along k. */
  if (csa == 1 && rsb == 1) {
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; ++j) {
      const float* bj = b + j * csb;
      for (int i = 0; i < m; ++i) {
        const float* ai = a + i * rsa;
        float s = 0.0f;
#pragma omp simd reduction(+ : s)
        for (int kk = 0; kk < k; ++kk) s += ai[kk] * bj[kk];
        float* dst = c + i * rsc + j * csc;
        *dst = (beta == 0.0f) ? alpha * s : alpha * s + beta * *dst;
      }
    }
    return;
  }
  /* Generic strides. */
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) {
      float s = 0.0f;
      for (int kk = 0; kk < k; ++kk) s += a[i * rsa + kk * csa] * b[kk * rsb + j * csb];
      float* dst = c + i * rsc + j * csc;
      *dst = (beta == 0.0f) ? alpha * s : alpha * s + beta * *dst;
    }
  }
}

/* Widen helpers used by the CPU baseline (inputs are the same seeded fp16 /
 * u8 data the GPU sees, widened to f32 as the host path would hold them). */
void orc_widen_f16(float* out, const h16* in, size_t count) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < count; ++i) out[i] = h2f(in[i]);
}

void orc_dequantize_to_f32(float* out, const h16* scales, const h16* zeros, const uint8_t* q,
                           int rows, int k, int block_size) {
  const int groups = k / block_size;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
    for (int i = 0; i < k; ++i) {
      int g = i / block_size;
      float z = zeros ? h2f(zeros[(size_t)r * groups + g]) : 127.5f;
      out[(size_t)r * k + i] =
          h2f(dequant_one(q[(size_t)r * k + i], scales[(size_t)r * groups + g], z));
    }
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Overrides the thread count taken from the environment (launchers such as torchrun export
 * OMP_NUM_THREADS=1 to every rank); returns the count now in force. */
int orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* The kernels either side of the matmuls (row ops).  The reductions follow  */
/* the reference's order: thread `tid` of 256 sums elements tid, tid+256, .. */
/* in that order, lanes combine by an xor butterfly (16, 8, 4, 2, 1), the    */
/* eight warp results by a second butterfly (4, 2, 1).  Where the device     */
/* uses approximate intrinsics (rsqrt, expf, powf, sinf, cosf) this file     */
/* uses libm, so agreement with a GPU is to a unit in the last place of the  */
/* fp16 result, not to the bit.                                              */
/* ------------------------------------------------------------------------ */
static float butterfly_256(float part[256], int is_max) {
  float warp[8];
  for (int w = 0; w < 8; ++w) {
    float v[32];
    for (int l = 0; l < 32; ++l) v[l] = part[w * 32 + l];
    for (int off = 16; off > 0; off >>= 1) {
      float nv[32];
      for (int l = 0; l < 32; ++l)
        nv[l] = is_max ? fmaxf(v[l], v[l ^ off]) : v[l] + v[l ^ off];
      memcpy(v, nv, sizeof v);
    }
    warp[w] = v[0];
  }
  for (int off = 4; off > 0; off >>= 1) {
    float nv[8];
    for (int l = 0; l < 8; ++l)
      nv[l] = is_max ? fmaxf(warp[l], warp[l ^ off]) : warp[l] + warp[l ^ off];
    memcpy(warp, nv, sizeof warp);
  }
  return warp[0];
}

/* normalize.cu:7-58 (output columns addressed with stride_ox; see the header of the
 * library for the one difference from normalize.cu:56) */
void orc_rms_norm(h16* out, const h16* in, const h16* w, int lx, int ly, int s_ox, int s_oy,
                  int s_ix, int s_iy, float eps) {
  for (int r = 0; r < ly; ++r) {
    const h16* irow = in + (ptrdiff_t)r * s_iy;
    h16* orow = out + (ptrdiff_t)r * s_oy;
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float s = 0.0f;
      for (int i = t; i < lx; i += 256) {
        float v = h2f(irow[(ptrdiff_t)i * s_ix]);
        s = fmaf(v, v, s); /* nvcc contracts sum += v * v */
      }
      part[t] = s;
    }
    float total = butterfly_256(part, 0);
    float rms_inv = 1.0f / sqrtf((total / (float)lx) + eps);
    for (int i = 0; i < lx; ++i) {
      float v = h2f(irow[(ptrdiff_t)i * s_ix]);
      orow[(ptrdiff_t)i * s_ox] = hmul(w[i], f2h(v * rms_inv));
    }
  }
}

/* normalize.cu:60-145: two reductions in the kernel's order (thread t sums elements t, t + 256,
 * ...; `sum += (v - mean) * (v - mean)` and `q * w + b` are contracted to fma by nvcc), output
 * columns addressed with stride_ox. */
void orc_layer_norm(h16* out, const h16* in, const h16* w, const h16* b, int lx, int ly, int s_ox,
                    int s_oy, int s_ix, int s_iy, float eps) {
  for (int r = 0; r < ly; ++r) {
    const h16* irow = in + (ptrdiff_t)r * s_iy;
    h16* orow = out + (ptrdiff_t)r * s_oy;
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float s = 0.0f;
      for (int i = t; i < lx; i += 256) s += h2f(irow[(ptrdiff_t)i * s_ix]);
      part[t] = s;
    }
    float mean = butterfly_256(part, 0) / (float)lx;
    for (int t = 0; t < 256; ++t) {
      float s = 0.0f;
      for (int i = t; i < lx; i += 256) {
        float d = h2f(irow[(ptrdiff_t)i * s_ix]) - mean;
        s = fmaf(d, d, s);
      }
      part[t] = s;
    }
    float stddev = sqrtf(butterfly_256(part, 0) / (float)lx + eps);
    for (int i = 0; i < lx; ++i) {
      float q = (h2f(irow[(ptrdiff_t)i * s_ix]) - mean) / stddev;
      orow[(ptrdiff_t)i * s_ox] = f2h(fmaf(q, h2f(w[i]), h2f(b[i])));
    }
  }
}

/* normalize.cu:150-220, rows `pitch` elements apart (pitch == w in the reference) */
void orc_softmax_rows(h16* out, const h16* in, int heads, int h, int w, int pitch, float temp) {
  for (int hd = 0; hd < heads; ++hd)
    for (int r = 0; r < h; ++r) {
      const h16* irow = in + ((ptrdiff_t)hd * h + r) * pitch;
      h16* orow = out + ((ptrdiff_t)hd * h + r) * pitch;
      float part[256];
      for (int t = 0; t < 256; ++t) {
        float m = -INFINITY;
        for (int i = t; i < w; i += 256) m = fmaxf(m, h2f(irow[i]) / temp);
        part[t] = m;
      }
      float mx = butterfly_256(part, 1);
      for (int t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (int i = t; i < w; i += 256) s += expf(h2f(irow[i]) / temp - mx);
        part[t] = s;
      }
      float sum = butterfly_256(part, 0);
      for (int i = 0; i < w; ++i) orow[i] = f2h(expf(h2f(irow[i]) / temp - mx) / sum);
    }
}

/* rotary.cu:4-29; `same_pos` != 0 takes the angle at pos_offset for every row (the
 * decode form, one new token per sequence) instead of pos_offset + row */
void orc_rotary(h16* out, const h16* in, int lx, int ly, int s_ox, int s_oy, int s_ix, int s_iy,
                int n_heads, int pos_offset, float theta, int same_pos) {
  int head_dim = lx / n_heads;
  for (int r = 0; r < ly; ++r)
    for (int c = 0; c < lx; c += 2) {
      int head_c = c % head_dim;
      int pos = same_pos ? pos_offset : pos_offset + r;
      float angle = (float)pos / powf(theta, (float)head_c / (float)head_dim);
      float re = h2f(in[(ptrdiff_t)r * s_iy + (ptrdiff_t)c * s_ix]);
      float im = h2f(in[(ptrdiff_t)r * s_iy + (ptrdiff_t)(c + 1) * s_ix]);
      float a_cos = cosf(angle), a_sin = sinf(angle);
      /* nvcc contracts one product of each line into an fma; which one cannot be told from
       * the source, one more reason why agreement with the GPU is to one unit, not the bit */
      out[(ptrdiff_t)r * s_oy + (ptrdiff_t)c * s_ox] = f2h(fmaf(re, a_cos, -(im * a_sin)));
      out[(ptrdiff_t)r * s_oy + (ptrdiff_t)(c + 1) * s_ox] = f2h(fmaf(re, a_sin, im * a_cos));
    }
}

/* elementwise.cu:16-33: op 1 = Add (left +h right), 2 = SiluMul */
int orc_elementwise_binary_2d_f16(h16* out, const h16* left, const h16* right, int rows, int cols,
                                  int s_o, int s_l, int s_r, int op) {
  if (op != 1 && op != 2) return ORC_ERR_UNSUPPORTED;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      h16 l = left[(ptrdiff_t)r * s_l + c], rr = right[(ptrdiff_t)r * s_r + c];
      if (op == 1) {
        out[(ptrdiff_t)r * s_o + c] = hadd(l, rr);
      } else {
        float lf = h2f(l);
        out[(ptrdiff_t)r * s_o + c] = f2h(lf / (1.0f + expf(-lf)) * h2f(rr));
      }
    }
  return ORC_OK;
}

/* One new token per sequence against caches [batch, max_seq, n_heads*head_dim]: the chain
 * matmul(Scale) -> softmax_rows -> matmul of llama.rs:538-554 over positions 0..pos, with
 * exact products and wide accumulation in the two contractions. */
void orc_decode_attention(h16* out, const h16* q, const h16* k_cache, const h16* v_cache, int batch,
                          int n_heads, int head_dim, int max_seq, int s_q, int s_o, int pos,
                          float scale) {
  int width = n_heads * head_dim;
  int T = pos + 1 < max_seq ? pos + 1 : max_seq;
  h16 hscale = f2h(scale);
  float* sc = (float*)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1));
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < n_heads; ++h) {
      const h16* qh = q + (ptrdiff_t)b * s_q + (ptrdiff_t)h * head_dim;
      const h16* kb = k_cache + (ptrdiff_t)b * max_seq * width + (ptrdiff_t)h * head_dim;
      const h16* vb = v_cache + (ptrdiff_t)b * max_seq * width + (ptrdiff_t)h * head_dim;
      float mx = -INFINITY;
      for (int t = 0; t < T; ++t) {
        double d = 0.0;
        for (int j = 0; j < head_dim; ++j)
          d += (double)h2f(qh[j]) * (double)h2f(kb[(ptrdiff_t)t * width + j]);
        sc[t] = h2f(hmul(d2h(d), hscale));
        mx = fmaxf(mx, sc[t]);
      }
      double sum = 0.0;
      for (int t = 0; t < T; ++t) sum += (double)expf(sc[t] - mx);
      for (int t = 0; t < T; ++t) sc[t] = h2f(f2h(expf(sc[t] - mx) / (float)sum));
      for (int j = 0; j < head_dim; ++j) {
        double a = 0.0;
        for (int t = 0; t < T; ++t) a += (double)sc[t] * (double)h2f(vb[(ptrdiff_t)t * width + j]);
        out[(ptrdiff_t)b * s_o + (ptrdiff_t)h * head_dim + j] = d2h(a);
      }
    }
  free(sc);
}

/* embed_uint8.cu:3-19 */
void orc_embed_uint8(int n_dim, int n_ids, const int16_t* in_ids, h16* out, const uint8_t* table,
                     const h16* scales, int block_size) {
  int block_count = n_dim / block_size;
  for (int t = 0; t < n_ids; ++t) {
    ptrdiff_t id = in_ids[t];
    for (int i = 0; i < n_dim; ++i)
      out[(ptrdiff_t)t * n_dim + i] =
          f2h(((float)table[id * n_dim + i] - 127.5f) * h2f(scales[id * block_count + i / block_size]));
  }
}
