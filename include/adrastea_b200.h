/*
 * adrastea_b200 — C ABI of the B200-native matmul path.
 *
 * Every entry point is what an FFI binding for the reference's kernel-call
 * interface would bind for this path.  Reference citations are relative to
 * the reference project root (eiz/adrastea).
 *
 * Conventions (identical to the reference's):
 *   - all tensor pointers are device pointers owned by the caller; the
 *     library allocates nothing on the per-call path;
 *   - dimensions and strides are in ELEMENTS, `int`; x = last dimension,
 *     y = second-last, z = third-last; a z-stride of 0 broadcasts that
 *     operand over the batch (adrastea_models/src/kernels.rs:864-887);
 *   - calls are asynchronous: work is enqueued on `stream` (0 = the legacy
 *     default stream, which is what the reference always uses,
 *     kernels.rs:862);
 *   - the return value is 0 on success or an ADR_ERR_* code; nothing aborts
 *     or traps.  Where the reference panics (shape asserts,
 *     kernels.rs:825-827) or traps on the device (unknown op,
 *     adrastea_kernels/cpp/matmul.cu:428-429, 489-490) this library returns
 *     an error code before launching anything.
 *
 * `void*` stands for `__half*` so that the header needs no CUDA includes.
 */
#ifndef ADRASTEA_B200_H_
#define ADRASTEA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct adr_ctx adr_ctx;
typedef void* adr_stream; /* cudaStream_t */

enum {
  ADR_OK = 0,
  ADR_ERR_INVALID = 1,     /* null pointer, non-positive size, bad enum value */
  ADR_ERR_SHAPE = 2,       /* shape / divisibility / alignment rule violated  */
  ADR_ERR_UNSUPPORTED = 3, /* op the reference has no device code for         */
  ADR_ERR_CUDA = 4,        /* a CUDA call failed; see adr_last_cuda_error     */
  ADR_ERR_DEVICE = 5,      /* a kernel reported a bounded wait that ran out   */
  ADR_ERR_NCCL = 6,
  ADR_ERR_TOO_LARGE = 7    /* operands exceed a fixed built-in buffer (see the entry point) */
};

/* matmul.cu:26-36, kernels.rs:80-139 */
/* ADR_LOAD_SCALE: the reference multiplies both operands by fp16(scale) in fp16 before the
 * product (matmul.cu:45-60).  The CUDA-core kernel does the same, bit for bit; the tensor-core
 * kernel multiplies the fp32 accumulator by fp16(scale)^2 instead: within the 1e-2 tolerance
 * of this path, not bit-equal. */
enum { ADR_LOAD_IDENTITY = 0, ADR_LOAD_SCALE = 1 };
enum {
  ADR_STORE_IDENTITY = 0,
  ADR_STORE_GELU_BIAS = 1, /* enum value without device code in the reference: rejected */
  ADR_STORE_BETA_GELU_BIAS = 2,
  ADR_STORE_BETA_BIAS = 3,
  ADR_STORE_SCALE = 4,
  ADR_STORE_ADD = 5,
  ADR_STORE_QUICK_GELU_BIAS = 6
};
enum { ADR_MASK_NONE = 0, ADR_MASK_CAUSAL = 1 };
/* enum BinaryOp, elementwise.cu:16-19 */
enum { ADR_BINARY_ADD = 1, ADR_BINARY_SILU_MUL = 2 };

/* Kernel families the dispatcher can pick; see adr_force_kernel / adr_last_kernel. */
enum {
  ADR_KERNEL_AUTO = 0,
  ADR_KERNEL_F16_SIMT = 1,    /* any strides, any op; CUDA cores                    */
  ADR_KERNEL_F16_TC = 2,      /* TMA + tcgen05.mma, accumulators in TMEM             */
  ADR_KERNEL_U8_GEMV = 3,     /* m <= 4: 128-bit weight loads, fp32 FMA, shuffles    */
  ADR_KERNEL_U8_MMA = 4,      /* m <= 16: 128-bit weight loads, register-fed MMA     */
  ADR_KERNEL_U8_TC = 5,       /* m > 16: dequantise into shared memory, tcgen05.mma  */
  ADR_KERNEL_U8_SIMT = 6,     /* any m; thread-per-output restatement (slow)         */
  ADR_KERNEL_U8_STREAM = 7,   /* m <= 16: bulk-copy staged, cluster split-k, register-fed MMA */
  ADR_KERNEL_U8_RING = 8,     /* m <= 16, block 64/128: persistent CTAs, TMA ring, scale applied per group */
  ADR_KERNEL_F16_TC_GATHER = 9, /* tcgen05.mma behind loader warps that gather operands of any stride
                                   or alignment into the swizzled stage layout (views TMA cannot describe) */
  ADR_KERNEL_U8_TS = 10,      /* m > 32, p % 64 == 0, block % 64 == 0: weights dequantised into tensor
                                 memory (A operand), 256 tokens per tcgen05.mma */
  ADR_KERNEL_U8_KSPLIT = 11   /* m <= 16, p = 1024 * (2..8), block 64/128: k split over a thread-block
                                 cluster, activations in registers, partial sums through
                                 distributed shared memory */
};

/*
 * Replaces GpuKernels::new(capability) (kernels.rs:458-502): binds to `device`
 * (a CUDA ordinal), checks that it is an sm_100 part, sets the opt-in shared
 * memory sizes of the kernels.  The context is thread-compatible.
 */
int adr_init(int device, adr_ctx** out_ctx);
void adr_destroy(adr_ctx* ctx);
const char* adr_strerror(int code);
/* cudaError_t of the last failing CUDA call seen by this context (0 if none). */
int adr_last_cuda_error(const adr_ctx* ctx);
/* Pin the kernel family used by the next calls (ADR_KERNEL_AUTO restores dispatch).
 * A call whose shape the pinned kernel cannot take returns ADR_ERR_SHAPE. */
int adr_force_kernel(adr_ctx* ctx, int kernel);
/* Tuning knobs for A/B runs; value 0 restores the planner's own choice.
 *   "u8_split": cluster size (k-split) of the streaming u8 kernel, 1/2/4/8
 *   "u8_rows":  weight rows per CTA of the streaming u8 kernel, 32/64
 *   "tc_bn":    N-tile of the tensor-core fp16 kernel, 32/64/128/256
 *   "tc_split": cluster size (k-split) of the tensor-core fp16 kernel, 1/2/4/8
 *   "pdl":      1 = launch the u8 streaming kernel with programmatic dependent launch: it
 *               may then start, and prefetch its weight matrix, scales and zero points,
 *               while the previous kernel of the stream is still running.  The caller
 *               promises that those three buffers are not written by work enqueued just
 *               before on the same stream.  Activations and output are only touched after
 *               the previous kernel has completed.  The row-op kernels honour it too.
 *               Default 0.
 *   "pdl_guard": with "pdl" on, which launches of the persistent decode kernel end a chain of
 *               early starts (the launch behind them begins on an empty GPU): bit 0 = launches
 *               with two CTAs per SM (the cluster k-split kernel included), bit 1 = launches
 *               whose CTAs take a whole SM, bit 2 = row kernels with at least one CTA per SM
 *               (decode attention over many heads), bit 3 = the mark survives small kernels
 *               launched in between (they start early themselves and pass the early start
 *               on).  Default 15; 0 shows what the guard is worth (CTAs then land two to an SM
 *               on half the SMs).  Measured in a LLaMA-7B decode step: 15 against 3 is 9 %
 *               faster at batch 4 and 1 % slower at batch 1.
 *   "ts_bt":    tokens per tile of the tensor-memory prefill kernel, 128/256 (0 = the
 *               launcher's choice: 128 only where it does not add a wave of tiles).
 *   "ts_split": k-split of the tensor-memory prefill kernel over a cluster of 2 or 4 CTAs when a
 *               problem has too few tiles for the GPU (0 = the launcher's choice, 1 = never).
 *   "ks_pdl":   0 = the cluster k-split kernel never starts early under "pdl" (default 1).
 *   "ks_off":   1 = the dispatcher never picks the cluster k-split kernel (A/B runs).
 *   "ks_slack": 1 (default) = behind a small kernel of this library the cluster k-split kernel
 *               leaves about sixteen CTA slots of its grid unused, so that none of its clusters
 *               is pushed into a second wave by CTAs that started early and are still waiting.
 *   "ks_clusters", "ks_stages": clusters in the grid / ring stages of the cluster k-split
 *               decode kernel (0 = the planner's choice).
 *   "wait_ms":  bound, in milliseconds, of the waits on a peer GPU in adr_allreduce_oneshot and
 *               adr_matmul_nt_fp16u8_allreduce (0 = about a second).
 *   "u8_exact": 1 = the streaming u8 kernel rounds every dequantised weight to fp16 before
 *               the product, the arithmetic of matmul_nt_wmma_16x128x256_fp16u8.cu:5-7.
 *               Default 0: weights are not rounded and scale and zero point are applied to
 *               fp32 partial sums per scale group, the arithmetic of
 *               matmul_nt_fp16u8.cu:13-23 (used when block_size >= 64). */
int adr_set_tunable(adr_ctx* ctx, const char* name, int value);
/* Synchronises the device and returns ADR_ERR_DEVICE if any kernel launched through this
 * context gave up on a bounded wait (the flag is then cleared), ADR_OK otherwise. */
int adr_device_status(adr_ctx* ctx);
/* Kernel family chosen by the most recent successful matmul call. */
int adr_last_kernel(const adr_ctx* ctx);
/* Number of kernel launches issued through this context so far. */
uint64_t adr_launch_count(const adr_ctx* ctx);

/*
 * Replaces CommonKernels::matmul_f16 -> GpuKernels::matmul_f16 -> kernel
 * matmul_f16_fast (kernels.rs:210-213, 821-890; matmul.cu:504-513).
 * The 22 arguments after `stream` are, in order, exactly the kernel
 * parameters the reference marshals (matmul.cu:186-190, 493-499):
 *   out[b,y,x] = store(sum_k load(lhs[b,y,k]) * load(rhs[b,k,x]))
 * with the causal mask writing -inf where x > y.
 * `out` is read in place by ADD, BETA_BIAS and BETA_GELU_BIAS.
 */
int adr_matmul_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs, const void* rhs,
                   int batches, int m, int k, int n, int stride_ox, int stride_oy, int stride_oz,
                   int stride_lx, int stride_ly, int stride_lz, int stride_rx, int stride_ry,
                   int stride_rz, const void* bias, float beta, float scale, uint32_t store_op,
                   uint32_t load_op, uint32_t mask_op);

/*
 * adr_matmul_f16 with a second, outer batch dimension `w` (4th-last; its element strides follow
 * each operand's z stride), for operands that are rank-4 views such as the [B, H, S, hd] views of
 * [B, S, H*hd] storage that a batched attention block multiplies (clip.rs:374-388 at batch > 1).
 * No counterpart in the reference, whose launch takes its batch count from out.size(-3) only
 * (kernels.rs:858, 868-880).  When the two batch dimensions of every operand fold into one
 * (outer stride == batches * z stride, or both 0) this is one launch over batches_outer * batches;
 * otherwise it is one launch per outer index.  The bias is shared by all batches.
 */
int adr_matmul_f16_b2(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs, const void* rhs,
                      int batches_outer, int batches, int m, int k, int n, int stride_ox,
                      int stride_oy, int stride_oz, int stride_ow, int stride_lx, int stride_ly,
                      int stride_lz, int stride_lw, int stride_rx, int stride_ry, int stride_rz,
                      int stride_rw, const void* bias, float beta, float scale, uint32_t store_op,
                      uint32_t load_op, uint32_t mask_op);

/*
 * Replaces CommonKernels::matmul_f16_slow -> kernel matmul_f16
 * (kernels.rs:206-209, 753-819; matmul.cu:493-502).  Same contract; always
 * takes the CUDA-core kernel that accepts any strides.
 */
int adr_matmul_f16_slow(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                        const void* rhs, int batches, int m, int k, int n, int stride_ox,
                        int stride_oy, int stride_oz, int stride_lx, int stride_ly, int stride_lz,
                        int stride_rx, int stride_ry, int stride_rz, const void* bias, float beta,
                        float scale, uint32_t store_op, uint32_t load_op, uint32_t mask_op);

/*
 * Replaces kernel matmul_f16_raw (matmul.cu:515-517): identity ops, no mask.
 */
int adr_matmul_f16_raw(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                       const void* rhs, int batches, int m, int k, int n, int stride_ox,
                       int stride_oy, int stride_oz, int stride_lx, int stride_ly, int stride_lz,
                       int stride_rx, int stride_ry, int stride_rz);

/*
 * Replaces kernels matmul_nt_fp16u8 (matmul_nt_fp16u8.cu:4-24) and
 * matmul_nt_wmma_16x128x256_fp16u8 (matmul_nt_wmma_16x128x256_fp16u8.cu:12-83),
 * same parameter list:  out[m,n] = lhs[m,p] . deq(rhs[n,p])^T + beta * out.
 * rhs is u8 [n,p] row-major, scales fp16 [n, p/block_size] row-major.
 * The reference defines the product twice, and so does this entry point:
 *   - decode shapes (m <= 16 per pass; the default kernels) follow matmul_nt_fp16u8.cu:13-23:
 *     the dequantised weight (float(q) - zero) * float(scale) is NOT rounded to fp16; the kernels
 *     sum (1024 + q) * x exactly per scale group in fp32 and apply scale and zero point to the
 *     group sums.  Against that kernel the outputs differ only by fp32 summation order.
 *   - the prefill kernel (m > 32), and the decode kernels when the tunable "u8_exact" is 1, follow
 *     matmul_nt_wmma_16x128x256_fp16u8.cu:5-7: deq(q) = fp16((float(q) - zero) * float(scale)),
 *     bit-exact, products accumulated in fp32.
 * The two forms differ by the fp16 rounding of the weights (about 1e-3 relative on an output).
 * `zeros` NULL: zero = 127.5 (the reference's layout).  `zeros` non-NULL
 * (fp16 [n, p/block_size]; an extension without counterpart in the
 * reference): zero = float(zeros[n, group]).
 * Requires p % block_size == 0, block_size % 16 == 0 and p % 16 == 0; any m, n.
 * Like the reference kernels, `out` is always read (beta * old even when beta == 0), so a
 * NaN or Inf left in an uninitialised `out` propagates: pass a defined buffer.
 */
int adr_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                         const uint8_t* rhs, const void* scales, const void* zeros, int m, int p,
                         int n, int block_size, float beta);

/*
 * The same product as adr_matmul_nt_fp16u8 for callers with scratch memory to lend (no
 * counterpart in the reference, whose kernels take none): from a few thousand rows on, panels
 * of weight rows are dequantised to fp16 (the bit-exact fp16-rounded weights of
 * matmul_nt_wmma_16x128x256_fp16u8.cu:5-7) into `workspace` and multiplied by the fp16
 * tensor-core GEMM, which at that size outruns the dequantising GEMM by about a third.
 * `workspace` is device memory of `workspace_bytes` bytes, 16-byte aligned, at least 256 * p
 * bytes (128 weight rows as fp16); 32 MiB or more lets every panel be as large as the kernel
 * wants.  Its contents are scratch: undefined before and after the call.  With fewer rows, or a
 * NULL or too small workspace, the call is adr_matmul_nt_fp16u8.
 */
int adr_matmul_nt_fp16u8_ws(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                            const uint8_t* rhs, const void* scales, const void* zeros, int m, int p,
                            int n, int block_size, float beta, void* workspace,
                            size_t workspace_bytes);

/*
 * adr_matmul_nt_fp16u8_ws without a workspace argument and without any allocation: the weight
 * panels are expanded into a 16 MiB array that is part of the library itself (one per device
 * and process).  No counterpart in the reference.  It is for callers that have no device
 * memory of their own to lend and may not ask for any at this point: every byte of the device
 * belongs to another allocator, or the call sits in a loop where cudaMalloc and cudaFree
 * (which synchronise the whole device) are not acceptable.  The call issues no allocating or
 * freeing CUDA call.  It always takes the expansion path (dequantise a panel of weight rows,
 * fp16 tensor-core GEMM), whatever m is, so it pays off from a few thousand rows on.
 *   - p <= 65536 (128 weight rows of p fp16 columns must fit the array), else
 *     ADR_ERR_TOO_LARGE, and nothing is launched.  p % 8 == 0, n % 8 == 0 and `out`, `lhs`,
 *     `rhs` 16-byte aligned, else ADR_ERR_SHAPE.  A panel is 16 MiB / (2 p) weight rows, so
 *     long rows mean many small GEMMs: with 32 MiB to lend, adr_matmul_nt_fp16u8_ws is faster.
 *   - The first call on a device looks up the array's address (cudaGetSymbolAddress): make
 *     that first call before any stream capture begins.
 *   - The array is shared by all calls on the device.  It keeps the last call's panels, and
 *     two calls in flight at the same time (other streams, other threads) overwrite each
 *     other's panels: keep the calls on one stream or order them with events.
 */
int adr_matmul_nt_fp16u8_noalloc(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                 const uint8_t* rhs, const void* scales, const void* zeros,
                                 int m, int p, int n, int block_size, float beta);

/*
 * `count` u8 products over the SAME activations, out_i[m, n_i] = lhs[m, p] . deq(rhs_i[n_i, p])^T +
 * beta * out_i, for callers that keep q/k/v or gate/up as separate matrices the way the reference
 * does (llama.rs:503-527, 565-577).  No counterpart in the reference, which launches them one by
 * one.  For decode shapes (m <= 16, activations that fit the kernel's shared memory, block 64/128,
 * p % 128 == 0) up to four matrices go out as ONE launch of the persistent decode kernel, whose
 * CTAs walk the rows of all of them: one launch-to-launch gap and one load of the activations
 * instead of one per matrix.  Results are bit-identical to separate adr_matmul_nt_fp16u8 calls
 * with the persistent kernel.  Shapes that kernel does not take are served by separate calls.
 * `zeross` is NULL, or an array without NULL entries.  All matrices share p, block_size and beta.
 */
int adr_matmul_nt_fp16u8_grouped(adr_ctx* ctx, adr_stream stream, int count, void* const* outs,
                                 const void* lhs, const uint8_t* const* rhss,
                                 const void* const* scaless, const void* const* zeross, int m,
                                 int p, const int* ns, int block_size, float beta);

/*
 * out[m, n] = SiluMul(lhs . deq(rhs_gate)^T, lhs . deq(rhs_up)^T): the gate and up products of a
 * feed-forward block (llama.rs:565-577) and the elementwise kernel that follows them
 * (elementwise.cu:28-33) as ONE launch of the persistent decode kernel.  A CTA takes the gate unit
 * and the up unit of the same 16 rows one after the other; both results are rounded to fp16 as
 * the separate kernels would before fp16(g / (1 + expf(-g)) * u) is written, so the bits equal
 * two adr_matmul_nt_fp16u8 calls (persistent kernel) followed by adr_elementwise_binary_2d_f16
 * (SiluMul).  Decode shapes only (m <= 16, activations resident, block 64/128, p % 128 == 0), else
 * ADR_ERR_SHAPE: make the three calls.  The two matrices may be halves of one [2n, p] matrix.
 */
int adr_silu_mul_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                  const uint8_t* rhs_gate, const void* scales_gate,
                                  const void* zeros_gate, const uint8_t* rhs_up,
                                  const void* scales_up, const void* zeros_up, int m, int p, int n,
                                  int block_size);

/*
 * The fused q/k/v projection of a decode step together with what follows it: rhs is [3 * width, p]
 * (q rows, then k rows, then v rows); q is rotated (adr_rotary's formula at position *pos_dev) and
 * written to q_out[m, width] with row pitch stride_q, k is rotated into k_cache[token, pos, :],
 * v is copied into v_cache[token, pos, :] (caches [m or more, max_seq, width] fp16).  With
 * norm_weights non-NULL the rows of lhs are rms-normalised first (adr_rms_norm's bits).  One
 * launch of the persistent decode kernel instead of adr_(rms_norm +) matmul_nt_fp16u8 +
 * adr_decode_rope_append, same bits.  No counterpart in the reference (no KV cache there).
 * Decode shapes only (m <= 16, activations resident, block 64/128, p % 128 == 0, width % 16 == 0),
 * else ADR_ERR_SHAPE: make the separate calls.  A position outside [0, max_seq) writes nothing.
 */
int adr_qkv_rope_append_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* q_out,
                                         int stride_q, const void* lhs, const void* norm_weights,
                                         float eps, const uint8_t* rhs, const void* scales,
                                         const void* zeros, int m, int p, int width, int n_heads,
                                         int block_size, void* k_cache, void* v_cache, int max_seq,
                                         const int32_t* pos_dev, float theta);

/*
 * Replaces kernels matmul_nt_wmma_128x64x64 (matmul_nt_wmma_128x64x64.cu:8-78)
 * and matmul_nt_wmma_16x128x256 (matmul_nt_wmma_16x128x256.cu:8-68), same
 * parameter list:  out[m,n] = lhs[m,p] . rhs[n,p]^T + beta * out, contiguous
 * row-major operands.  The reference's divisibility rules are not required.
 */
int adr_matmul_nt_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                      const void* rhs, int m, int p, int n, float beta);

/*
 * Replaces kernel dequantize_absmax_uint8 (quantize.cu:46-56):
 * out[r,i] = fp16((float(q[r,i]) - zero) * float(scales[r, i / block_size])),
 * contiguous [rows,k] operands; `zeros` as in adr_matmul_nt_fp16u8.
 */
int adr_dequantize_absmax_uint8(adr_ctx* ctx, adr_stream stream, void* out, const void* scales,
                                const void* zeros, const uint8_t* q, int rows, int k,
                                int block_size);

/*
 * Replaces kernel quantize_absmax_uint8 (quantize.cu:3-44): per (row, group)
 * scale = fp16(max|x| / 127.5), q = u8(round(127.5 + x / scale)).
 */
int adr_quantize_absmax_uint8(adr_ctx* ctx, adr_stream stream, uint8_t* q, void* scales,
                              const void* in, int rows, int k, int block_size);

/*
 * Replaces kernel embed_uint8 (embed_uint8.cu:3-19; parameters in its order):
 * out_embeddings[t, i] = fp16((float(table[in_ids[t], i]) - 127.5) *
 *                             float(scales[in_ids[t], i / block_size])),
 * token ids are 16-bit as in the reference kernel; contiguous operands.
 */
int adr_embed_uint8(adr_ctx* ctx, adr_stream stream, int n_dim, int n_ids, const int16_t* in_ids,
                    void* out_embeddings, const uint8_t* embeddings_table, const void* scales,
                    int block_size);

/* ------------------------------------------------------------------------
 * The kernels either side of the matmuls in a decoder layer.  The first four
 * restate reference kernels with the same order of floating-point operations
 * (the bits of those kernels compiled for this GPU); parameters are in the
 * reference kernels' order, strides in elements.
 * ------------------------------------------------------------------------ */

/*
 * Replaces kernel rms_norm (normalize.cu:7-58; host side kernels.rs:680-706):
 * out[r,i] = weights[i] *h fp16(in[r,i] * rsqrt(sum_i in[r,i]^2 / length_x + eps)).
 * One difference: the reference addresses the output columns with stride_ix
 * (normalize.cu:56); here stride_ox is used (identical whenever the two are
 * equal, as at every call site of the reference).
 */
int adr_rms_norm(adr_ctx* ctx, adr_stream stream, void* out, const void* in, const void* weights,
                 int length_x, int length_y, int stride_ox, int stride_oy, int stride_ix,
                 int stride_iy, float eps);

/*
 * Replaces kernel layer_norm (normalize.cu:60-145; host side kernels.rs:652-678):
 * out[r,i] = fp16((in[r,i] - mean_r) / sqrt(var_r + eps) * weights[i] + bias[i]), mean and the
 * biased variance of row r in fp32, summed in the reference kernel's order.  Like adr_rms_norm
 * the output columns are addressed with stride_ox where the reference uses stride_ix.
 */
int adr_layer_norm(adr_ctx* ctx, adr_stream stream, void* out, const void* in, const void* weights,
                   const void* bias, int length_x, int length_y, int stride_ox, int stride_oy,
                   int stride_ix, int stride_iy, float eps);

/*
 * Replaces kernel softmax_rows (normalize.cu:150-220; kernels.rs:892-915):
 * `heads` matrices of h rows, softmax over the first w elements of every row,
 * out = fp16(expf(x/temperature - max) / sum).  `pitch` is the distance between
 * rows in elements; the reference kernel is the case pitch == w.  In place
 * (out == in) is allowed.
 */
int adr_softmax_rows(adr_ctx* ctx, adr_stream stream, void* out, const void* in, int heads, int h,
                     int w, int pitch, float temperature);

/*
 * Replaces kernel rotary (rotary.cu:4-29; kernels.rs:722-751): the pairs
 * (c, c+1) of every head of row r are rotated by the angle
 * (pos_offset + r) / powf(theta, (c % head_dim) / head_dim), head_dim =
 * length_x / n_heads.  In place (out == in) is allowed.
 */
int adr_rotary(adr_ctx* ctx, adr_stream stream, void* out, const void* in, int length_x,
               int length_y, int stride_ox, int stride_oy, int stride_ix, int stride_iy, int n_heads,
               int pos_offset, float theta);

/*
 * Replaces kernel elementwise_binary_2d_f16 (elementwise.cu:16-33, 118-160;
 * kernels.rs:633-650) for rows of contiguous columns `stride_*` elements apart:
 * ADR_BINARY_ADD: left +h right; ADR_BINARY_SILU_MUL:
 * fp16(float(left) / (1 + expf(-left)) * float(right)).  out may be left.
 */
int adr_elementwise_binary_2d_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* left,
                                  const void* right, int rows, int cols, int stride_o, int stride_l,
                                  int stride_r, uint32_t op);

/*
 * No counterpart in the reference, which keeps no key/value cache and re-runs
 * the whole prefix for every token (llama.rs:426-427).  Caches are
 * [batch, max_seq, n_heads*head_dim] fp16; *pos_dev (device memory, so that a
 * captured step can be replayed) is the position of the new token.
 *
 * adr_decode_rope_append: q[b,:] rotated in place, k[b,:] rotated into
 * k_cache[b, pos, :], v[b,:] copied into v_cache[b, pos, :] (formula of
 * adr_rotary with the angle taken at `pos` for every row).  A position outside
 * [0, max_seq) writes nothing.
 *
 * adr_decode_attention: for every (sequence, head), over positions 0..pos:
 * score = fp16(q.k) *h fp16(scale), softmax in fp32, probabilities rounded to
 * fp16, out = fp16(sum_t p_t * v_t) - the rounding points of the reference's
 * matmul(Scale) -> softmax_rows -> matmul chain (llama.rs:538-554).
 * head_dim % 8 == 0, head_dim <= 256, max_seq % 8 == 0.
 */
int adr_decode_rope_append(adr_ctx* ctx, adr_stream stream, void* q, const void* k, const void* v,
                           void* k_cache, void* v_cache, int batch, int n_heads, int head_dim,
                           int max_seq, int stride_q, int stride_k, int stride_v,
                           const int32_t* pos_dev, float theta);
int adr_decode_attention(adr_ctx* ctx, adr_stream stream, void* out, const void* q,
                         const void* k_cache, const void* v_cache, int batch, int n_heads,
                         int head_dim, int max_seq, int stride_q, int stride_o,
                         const int32_t* pos_dev, float scale);

/*
 * Replaces, in ONE launch, the reference's attention chain
 *   matmul_f16(scores, q, k^T, store Scale(scale)[, mask Causal])   llama.rs:538-547, clip.rs:374-380
 *   softmax_rows_inplace(scores)                                    llama.rs:548; normalize.cu:150-220
 *   matmul_f16(out, scores, v)                                      llama.rs:549-554, clip.rs:381-388
 * for batches_outer x batches_inner independent (query, key, value) matrices (heads inside
 * sequences or images): q is [s_q, head_dim], k and v are [s_k, head_dim], out is
 * [s_q, head_dim], each addressed as base + outer * strides[2] + inner * strides[1] +
 * row * strides[0] + column (strides in elements, innermost stride 1; a stride of 0 broadcasts).
 * Rounding points of the chain that are kept: score = fp16(q.k) *h fp16(scale) (the Scale store
 * op), softmax statistics in fp32, probabilities rounded to fp16 before the product with v,
 * output fp16.  One difference: the probabilities are exp(score - max) and the division by
 * their sum happens after the product with v (within the 1e-2 tolerance of this path, not
 * bit-equal to the chain).  Mask Causal hides key x from query y when x > y, as matmul.cu does.
 * The score matrix is never written to memory.
 * head_dim 64 or 128; pointers 16-byte aligned; every stride a multiple of 8 elements; else
 * ADR_ERR_SHAPE (make the three calls).
 */
int adr_attention_f16(adr_ctx* ctx, adr_stream stream, void* out, const void* q, const void* k,
                      const void* v, int batches_outer, int batches_inner, int s_q, int s_k,
                      int head_dim, const long long* strides_q, const long long* strides_k,
                      const long long* strides_v, const long long* strides_o, float scale,
                      uint32_t mask_op);

/*
 * No counterpart in the reference (it has no multi-GPU path, llama.rs:28-29): one-shot
 * all-reduce (sum) of an fp16 vector over peer memory, for the row-split products of
 * tensor-parallel decoding.  bufs[r] is rank r's partial vector and flags[r] rank r's flag array
 * (`blocks` * world 32-bit words, zero before the first call), all addressable from this GPU
 * (peer-mapped symmetric allocations); `epochs` is `blocks` 32-bit words of this rank's own
 * memory, zero before the first call.  out[i] = fp16(sum_r bufs[r][i] (+ out[i] if residual)),
 * summed in rank order in fp32, so every rank gets the same bits.  Every rank must make the same
 * sequence of calls with the same `blocks`, and consecutive calls must alternate between two
 * buffers (a buffer may be rewritten only after the NEXT all-reduce has been enqueued behind this
 * one).  The wait for the peers is bounded (about a second), after which the status word is set
 * (adr_device_status) and the call completes with a wrong result rather than hanging.
 * count % 8 == 0, world <= 8.
 */
int adr_allreduce_oneshot(adr_ctx* ctx, adr_stream stream, void* out, const void* const* bufs,
                          void* const* flags, void* epochs, int blocks, int rank, int world,
                          long long count, int residual);

/*
 * No counterpart in the reference (its layers launch rms_norm and the matmul separately,
 * llama.rs:497-508): out = rms_norm(lhs, norm_weights, eps) . deq(rhs)^T + beta * out for decode
 * shapes, with the bits of adr_rms_norm followed by adr_matmul_nt_fp16u8.  The decode kernel
 * normalises the activation rows it has just copied into shared memory (every CTA does so for
 * itself), which saves a kernel launch per norm.  lhs is contiguous [m, p]; m <= 16 and a shape the
 * persistent decode kernel takes with the activations resident (else ADR_ERR_SHAPE: make the two
 * calls).
 */
int adr_rms_norm_matmul_nt_fp16u8(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                  const void* norm_weights, float eps, const uint8_t* rhs,
                                  const void* scales, const void* zeros, int m, int p, int n,
                                  int block_size, float beta);

/*
 * No counterpart in the reference: the row-split product of tensor-parallel decoding with its
 * all-reduce in the same kernel.  Each rank holds a [n, p] slice (p = K / world) of the weight and
 * the matching slice of the activations; out[m, n] = sum over ranks of lhs_r . deq(rhs_r)^T (+ the
 * old out if residual), the same bits on every rank.  The decode kernel pushes the result of every
 * 16-column unit, as fp16, into slot `rank` of every rank's inbox ([world][m][n] fp16, peer-mapped:
 * inboxes[r] is rank r's inbox as addressable from this GPU), then CTA c exchanges one flag with
 * CTA c of every peer (flags[r]: rank r's array of max_ctas * world 32-bit words, zero before the
 * first call; epochs: max_ctas words of this rank's own memory, zero before the first call; the
 * wait is bounded, see adr_allreduce_oneshot) and adds the world slots of its own inbox in rank
 * order.  Consecutive calls must alternate between two inboxes.  Every rank must make the same
 * calls with the same shapes.  m <= 16 and a shape the persistent decode kernel takes
 * (block_size 64 or 128, p % 128 == 0), else ADR_ERR_SHAPE: fall back to adr_matmul_nt_fp16u8 +
 * adr_allreduce_oneshot.
 */
int adr_matmul_nt_fp16u8_allreduce(adr_ctx* ctx, adr_stream stream, void* out, const void* lhs,
                                   const uint8_t* rhs, const void* scales, const void* zeros, int m,
                                   int p, int n, int block_size, int residual,
                                   void* const* inboxes, void* const* flags, void* epochs,
                                   int max_ctas, int rank, int world);

/*
 * Replaces MatmulTracer (kernels.rs:231-248, 306-333).  When enabled, every
 * matmul call records (m, k, n, batches, strides, ops, kernel family) once per
 * distinct combination.  adr_trace_dump writes one JSON object per line into
 * `buf` (at most `cap` bytes, NUL terminated) and returns the number of bytes
 * the full dump needs.
 */
int adr_trace_enable(adr_ctx* ctx, int on);
void adr_trace_clear(adr_ctx* ctx);
size_t adr_trace_dump(adr_ctx* ctx, char* buf, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* ADRASTEA_B200_H_ */
