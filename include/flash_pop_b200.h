/*
 * flash_pop_b200 — C ABI of the B200 (sm_100a) retention / POP-retention kernels.
 *
 * This is the whole boundary between a host framework and the CUDA code: plain pointers,
 * sizes and a cudaStream_t.  No entry point allocates, frees or keeps device memory, none
 * synchronises the host, all are stream-ordered and re-entrant (the only state the library keeps is
 * per-thread caches of encoded tensor maps and per-device "kernel configured" flags).  Every entry
 * point returns an fpb_status (0 = ok); nothing aborts or traps.
 *
 * Tensor conventions (the reference's own, flash_pop/fused_retention/fused_chunk_fwd.py:96-101):
 *   q, k          (B, T, H, dk)      element strides (stride_b, stride_t, stride_h), inner stride 1
 *   v, o, dO      (B, T, H, dv)
 *   states        (B, H, dk, dv)     inner (dk, dv) block contiguous, strides (stride_b, stride_h)
 *   block_states  (B, N, H, dk, dv)  contiguous, N = T / block_size
 * The operator scales k by 1/sqrt(dk) itself (flash_pop/fused_retention/reference.py:57).
 * head_decays is a HOST array of H doubles, gamma_h in [0, 1]  (the reference passes a Python
 * tuple of floats: flash_pop/fused_retention/__init__.py:13,20).
 * Limits: H <= 256, dk, dv <= 256, and at most 65535 sequences per call (B, or B * M for the suffix entry points):
 * the batch is a grid dimension.  Larger batches return FPB_ERR_TOO_LARGE; split them.
 */
#ifndef FLASH_POP_B200_H_
#define FLASH_POP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* fpb_stream_t; /* == cudaStream_t */

typedef enum fpb_status {
  FPB_OK = 0,
  FPB_ERR_NULL_POINTER = 1,
  FPB_ERR_BAD_SHAPE = 2,       /* negative size, dk/dv not supported by any kernel, H too large */
  FPB_ERR_BAD_DTYPE = 3,
  FPB_ERR_BAD_STRIDE = 4,      /* overlapping or negative strides */
  FPB_ERR_BAD_DECAY = 5,       /* decay outside [0, 1] or not finite */
  FPB_ERR_BAD_BLOCK_SIZE = 6,
  FPB_ERR_NO_DEVICE_CODE = 7,  /* current device is not sm_100 */
  FPB_ERR_LAUNCH = 8,          /* cudaGetLastError() after a launch, see fpb_last_cuda_error */
  FPB_ERR_DEVICE_TIMEOUT = 9,  /* a bounded in-kernel wait gave up (reported by fpb_device_status) */
  FPB_ERR_TENSOR_MAP = 10,     /* cuTensorMapEncodeTiled refused the tensor */
  FPB_ERR_TOO_LARGE = 11,      /* size beyond a fixed limit of this entry point */
  FPB_ERR_BAD_WORKSPACE = 12   /* workspace pointer misaligned or size negative */
} fpb_status;

typedef enum fpb_dtype { FPB_BF16 = 0, FPB_F32 = 1 } fpb_dtype;

/* which implementation a call took (fpb_last_path) */
typedef enum fpb_path { FPB_PATH_NONE = 0, FPB_PATH_SIMT = 1, FPB_PATH_TCGEN05 = 2 } fpb_path;

enum {
  FPB_FLAG_FORCE_SIMT = 1,  /* take the CUDA-core fp32-math kernels even where the tensor-core ones apply */
  /* backward entry points only: leave out a part nobody needs (its output tensors may then have data == NULL) */
  FPB_FLAG_SKIP_DQ = 2,     /* no dQ: skips the forward walk that recomputes the states */
  FPB_FLAG_SKIP_DKDV = 4,   /* no dK, dV, dS_0 (nor suffix state gradients): skips the reverse walk */
  /* Every state tensor of the call (s0, s_out, d_s_out, d_s0, block_states, d_block_states) is fp32 although the
   * activations are bf16: a state carried from one call to the next (a long sequence fed in pieces,
   * flash_pop/retnet.py:548-558) is then not re-rounded to bf16 at every hand-off.  Implied for fp32 activations. */
  FPB_FLAG_STATE_F32 = 8
};

/* A (B, T, H, d) activation. */
typedef struct fpb_seq {
  void* data;
  int64_t stride_b, stride_t, stride_h;
} fpb_seq;

/* A (B, H, dk, dv) state; data == NULL means "all zeros" for inputs, "not wanted" for outputs. */
typedef struct fpb_state {
  void* data;
  int64_t stride_b, stride_h;
} fpb_state;

typedef struct fpb_dims {
  int32_t dtype;        /* fpb_dtype of every tensor of the call */
  int32_t B, T, H, dk, dv;
  int32_t block_size;   /* POP entry points only: tokens per block (> 0) */
  int32_t flags;
  const double* head_decays; /* host, H entries */
  /* Optional device scratch memory (16-byte aligned), used only during the call.  A walk is one CTA per (batch, head,
   * state tile); a call with few of them leaves most SMs idle.  Given scratch memory, such a call cuts every sequence
   * into T-segments that run concurrently (local end states -> a scan over them -> the walk per segment).  NULL / 0:
   * sequences are walked whole.  fpb_workspace_bytes says how much a shape can use; less means fewer segments. */
  void* workspace;
  int64_t workspace_bytes;
} fpb_dims;

/* Scratch bytes that let a call of this shape (dtype, B, T, H, dk, dv) split its walks as far as the current device
 * makes worthwhile; 0 when the launch fills the device anyway.  No counterpart in the reference, whose grid is fixed
 * by the shape (flash_pop/fused_retention/fused_chunk_fwd.py:119). */
int64_t fpb_workspace_bytes(const fpb_dims* dims);

/*
 * Forward of fused chunked retention.
 *   o = (Q K^T/sqrt(dk) . D) V + zeta . (Q S_0),   s_out = gamma^T S_0 + sum_j gamma^(T-1-j) k_j^T v_j / sqrt(dk)
 * Replaces FusedChunkRetention.forward + the fused_chunk_retention_fwd kernel
 * (flash_pop/fused_retention/__init__.py:12-31, fused_chunk_fwd.py:95-187).
 */
int fpb_retention_fwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                      const fpb_state* s0, const fpb_seq* o, const fpb_state* s_out, fpb_stream_t stream);

/*
 * Host <-> device copy of a (batch rows, head group) slice of a contiguous (B, T, H, d) tensor: `rows` runs of
 * `width_bytes` bytes, `src_pitch` / `dst_pitch` bytes apart (one run per (row, token): the heads of the group), queued
 * on `stream` as ONE two-dimensional copy (cudaMemcpy2DAsync, direction from the pointers).  It lets
 * flash_pop_b200.host_io pipeline its slices by heads as well as by rows - a strided slice copied tensor-wise by the
 * framework goes through at a quarter of the link rate.  No counterpart in the reference, which keeps its tensors on
 * the device.  Host memory should be pinned; widths and pitches in bytes, width <= both pitches.
 */
int fpb_copy_rows_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes, int64_t rows,
                        fpb_stream_t stream);

/*
 * fpb_retention_fwd for callers that cannot allocate device memory.  This entry point has no counterpart in the
 * reference.  Who needs it: a host that hands the whole GPU to one arena at start-up (an inference server, a process
 * held to a fixed memory budget) has nothing left for a later cudaMalloc to take, and a plugin running on such a
 * host's hot path may be forbidden to allocate at all - an allocation can fail there, and cudaMalloc also makes the
 * whole device wait.  Such a caller still wants an under-filled call (few batch rows x heads) cut into T-segments,
 * which needs scratch memory; here the scratch is an array built into the library image,
 * FPB_STATIC_SCRATCH_BYTES of device memory per GPU that loads the library, held until the process exits.
 *   - Inputs and outputs are the caller's as in fpb_retention_fwd; dims->workspace must be NULL.
 *   - The call itself allocates nothing and frees nothing (no cudaMalloc / cudaFree, no allocating library routine).
 *   - A shape whose split would use more scratch than the array holds (fpb_workspace_bytes(dims) >
 *     FPB_STATIC_SCRATCH_BYTES) is refused with FPB_ERR_TOO_LARGE; shapes that fill the GPU unsplit use no scratch.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) and keeps it; make that
 *     first call outside any stream capture.
 *   - All calls on a device share the one array.  It keeps whatever the last call left; nothing in it has to start at
 *     zero, since every slot a call reads it has written first.  Two calls that overlap on the GPU (different streams,
 *     or the same stream from two threads without ordering) race on it: order them.
 */
#define FPB_STATIC_SCRATCH_BYTES (16u << 20)
int fpb_retention_fwd_static(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                             const fpb_state* s0, const fpb_seq* o, const fpb_state* s_out, fpb_stream_t stream);

/*
 * Backward of fused chunked retention: given dO and the gradient d_s_out of the returned state,
 * writes dQ, dK, dV and (if wanted) dS_0.
 * Replaces FusedChunkRetention.backward + fused_retention_bwd_dk_dv_ds + fused_retention_bwd_dq
 * (flash_pop/fused_retention/__init__.py:33-47, fused_chunk_bwd.py:218-346,349-449).
 */
int fpb_retention_bwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                      const fpb_state* s0, const fpb_seq* d_o, const fpb_state* d_s_out,
                      const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                      fpb_stream_t stream);

/*
 * Forward of POP retention: retention outputs plus the state after every full block of
 * dims->block_size tokens, block_states (B, N, H, dk, dv) contiguous with N = T / block_size.
 * No final state is produced.
 * Replaces FlashPOPRetention.forward + fused_pop_retention_fwd
 * (flash_pop/pop_retention/__init__.py:13-31, pop_fwd.py:7-140).
 */
int fpb_pop_retention_fwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                          const fpb_state* s0, const fpb_seq* o, void* block_states, fpb_stream_t stream);

/*
 * Backward of POP retention: d_block_states (B, N, H, dk, dv) is added to the carried state
 * gradient where each block ends.
 * Replaces FlashPOPRetention.backward + pop_retention_bwd_dk_dv_ds + fused_retention_bwd_dq
 * (flash_pop/pop_retention/__init__.py:33-50, pop_bwd.py:9-165).
 */
int fpb_pop_retention_bwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                          const fpb_state* s0, const fpb_seq* d_o, const void* d_block_states,
                          const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                          fpb_stream_t stream);

/*
 * POP prediction-token suffixes, forward and backward.  Tensors are (B*M, P, H, d): M suffixes
 * of P tokens per batch row, flattened into the batch as the reference does.  Suffix m of row b
 * starts from the state at the START of block m — s0[b] for m == 0, block_states[b, m-1]
 * otherwise — read in place; its own end state is dropped, so the stream state is never written.
 * dims->B is the number of stream rows B, dims->T the suffix length P, dims->block_size is unused.
 * The backward writes d_s0 (B,H,dk,dv) and d_block_states (B, N, H, dk, dv), N >= M-1 (blocks
 * with no suffix get zero).
 * Replaces POPDecoderLayer._suffixes_forward's torch.cat + second operator call
 * (flash_pop/pop_retnet.py:152-171).
 */
int fpb_pop_suffix_fwd(const fpb_dims* dims, int32_t M, int32_t N, const fpb_seq* q, const fpb_seq* k,
                       const fpb_seq* v, const fpb_state* s0, const void* block_states, const fpb_seq* o,
                       fpb_stream_t stream);
int fpb_pop_suffix_bwd(const fpb_dims* dims, int32_t M, int32_t N, const fpb_seq* q, const fpb_seq* k,
                       const fpb_seq* v, const fpb_state* s0, const void* block_states, const fpb_seq* d_o,
                       const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                       void* d_block_states, fpb_stream_t stream);

/*
 * One recurrent decoding step for B rows of one token each:
 *   s_out = gamma s_prev + k^T v / sqrt(dk),   o = q s_out
 * q, k are (B, 1, H, dk) and v, o (B, 1, H, dv): dims->T must be 1 and stride_t is not read.  The states have
 * their own element type `state_dtype` (an fp32 state under bf16 activations is not re-rounded every token);
 * s_prev->data == NULL means a zero state, s_out may be the same memory as s_prev (update in place) and
 * s_out->data == NULL drops the new state.  Arithmetic is fp32.
 * Replaces retention_recurrent (flash_pop/retnet.py:79-101) as MultiScaleRetention.forward_recurrent calls it
 * (flash_pop/retnet.py:325-366).
 */
int fpb_retention_step(const fpb_dims* dims, int32_t state_dtype, const fpb_seq* q, const fpb_seq* k,
                       const fpb_seq* v, const fpb_state* s_prev, const fpb_seq* o, const fpb_state* s_out,
                       fpb_stream_t stream);

/*
 * The two elementwise passes of a retention layer either side of the operator, each as one streaming kernel
 * (fp32 arithmetic).  They replace PyTorch expressions of the reference rather than kernels of its own.
 *
 * fpb_rotary: rotates the channel pairs (2i, 2i+1) of q and k (B, T, H, d), d a multiple of 8, by the unit phasors
 * phasors[b, t, i] = (cos, sin) — a device array of (rows, T, d/2, 2) floats, `phasor_stride_b` floats-pairs between
 * batch rows or 0 when all rows share one table — and writes them as `out_dtype`.  conjugate != 0 rotates by the
 * negative angle (the backward pass).  k_in / k_out may be NULL to rotate one tensor.  Tensors and strides must be
 * 16-byte aligned.  Replaces XPos.__call__ / _theta_shift (flash_pop/xpos_emb.py:32-40,120-126) and the cast that
 * follows it (flash_pop/retnet.py:268-290).
 *
 * fpb_groupnorm_gate_fwd: y = GroupNorm_head(o) * gate, GroupNorm over the dv channels of each (row, token, head)
 * with biased variance, eps inside the square root and no affine parameters; gate = z * sigmoid(z) when swish != 0,
 * else z itself (the caller applied another activation).  dv even, at most 256.  Replaces the GroupNorm, casts,
 * activation and product of MultiScaleRetention (flash_pop/retnet.py:294-309).
 * fpb_groupnorm_gate_bwd: from d_y writes d_o and d_z.
 */
int fpb_rotary(int32_t B, int32_t T, int32_t H, int32_t d, int32_t in_dtype, int32_t out_dtype, int32_t conjugate,
               const float* phasors, int64_t phasor_stride_b, const fpb_seq* q_in, const fpb_seq* k_in,
               const fpb_seq* q_out, const fpb_seq* k_out, fpb_stream_t stream);
int fpb_groupnorm_gate_fwd(int32_t B, int32_t T, int32_t H, int32_t dv, int32_t dtype, float eps, int32_t swish,
                           const fpb_seq* o, const fpb_seq* z, const fpb_seq* y, fpb_stream_t stream);
int fpb_groupnorm_gate_bwd(int32_t B, int32_t T, int32_t H, int32_t dv, int32_t dtype, float eps, int32_t swish,
                           const fpb_seq* o, const fpb_seq* z, const fpb_seq* d_y, const fpb_seq* d_o,
                           const fpb_seq* d_z, fpb_stream_t stream);

/*
 * LayerNorm over the last dimension with fp32 arithmetic on bf16 (or fp32) rows, in one pass each way.
 *   y = (x - mean) / sqrt(var + eps) * weight + bias      (biased variance; weight / bias fp32, either may be NULL)
 * x, y: `rows` rows of d elements, `*_stride` elements apart, 16-byte aligned; d a multiple of 8 (bf16) / 4 (fp32)
 * and at most 1024 (bf16) / 512 (fp32).  The backward recomputes the statistics from x, writes d_x (x's strides)
 * and overwrites d_weight / d_bias (fp32, d entries each, either may be NULL) with the sums over all rows; the
 * sums are accumulated with atomic adds, so their last bits depend on the order.
 * Replaces the cast - nn.LayerNorm(fp32) - cast sequence around the layers' norms (flash_pop/retnet.py:474-486).
 */
int fpb_layernorm_fwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride,
                      const float* weight, const float* bias, void* y, int64_t y_stride, fpb_stream_t stream);
int fpb_layernorm_bwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride,
                      const float* weight, const void* d_y, int64_t dy_stride, void* d_x, float* d_weight,
                      float* d_bias, fpb_stream_t stream);

/*
 * Adaptive LayerNorm modulation and gated residual of the diffusion RetNet layers, one streaming kernel each way.
 *   fpb_adaln_fwd:          y = LayerNorm(x) * (1 + scale) + shift     (no affine parameters, biased variance, fp32 arithmetic)
 *   fpb_gate_residual_fwd:  out = x + gate * branch
 * x, y, branch, out: `rows` rows of d elements as for fpb_layernorm_*.  shift / scale / gate are rows of the modulation
 * MLP's output read in place: row m (elements `mod_stride` apart, 16-byte aligned, the activations' type) serves the
 * rows_per_mod consecutive rows m * rows_per_mod ... of x - all tokens of a batch row, the tokens of a frame, or one.
 * The backward entry points overwrite the fp32 gradients d_shift / d_scale / d_gate, (ceil(rows / rows_per_mod), d)
 * contiguous, with sums over the rows that share a modulation row (atomic adds: last bits depend on the order);
 * fpb_adaln_bwd writes d_x with x's row stride, fpb_gate_residual_bwd writes d_branch with branch's (d_x of the
 * residual is d_out itself).
 * Replace modulate / AdaLayerNorm / AdaLayerNormZero (flash_pop/modules/adaln.py:13-15,90-99,154-166) and the gated
 * residuals of DiffusionRetNetDecoderLayer (flash_pop/diffusion_retnet.py:133-146).
 */
int fpb_adaln_fwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride, const void* shift,
                  const void* scale, int64_t mod_stride, int64_t rows_per_mod, void* y, int64_t y_stride, fpb_stream_t stream);
int fpb_adaln_bwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride, const void* scale,
                  int64_t mod_stride, int64_t rows_per_mod, const void* d_y, int64_t dy_stride, void* d_x, float* d_shift,
                  float* d_scale, fpb_stream_t stream);
int fpb_gate_residual_fwd(int64_t rows, int32_t d, int32_t dtype, const void* x, int64_t x_stride, const void* branch,
                          int64_t branch_stride, const void* gate, int64_t mod_stride, int64_t rows_per_mod, void* out,
                          int64_t out_stride, fpb_stream_t stream);
int fpb_gate_residual_bwd(int64_t rows, int32_t d, int32_t dtype, const void* branch, int64_t branch_stride, const void* gate,
                          int64_t mod_stride, int64_t rows_per_mod, const void* d_out, int64_t dout_stride, void* d_branch,
                          float* d_gate, fpb_stream_t stream);

/*
 * Softmax cross entropy of `rows` rows of V logits (bf16 or fp32, `row_stride` elements apart, 16-byte aligned rows)
 * against int64 targets, fp32 arithmetic, for the language-model head of the full-stack training workload (the
 * reference has no loss of its own; this replaces the cast-to-fp32 + log_softmax + nll_loss passes of PyTorch).
 * The forward writes per row loss[r] = logsumexp(x_r) - x_r[target] and lse[r] (kept for the backward); a target
 * outside [0, V) (PyTorch's ignore_index = -100 among them) gives loss 0 and a zero gradient row; such rows still count
 * in row_weight = 1 / rows, i.e. the mean is over ALL rows.  The backward writes
 *   d_logits[r, j] = (exp(x[r, j] - lse[r]) - [j == target_r]) * scale[0] * row_weight
 * in the logits' type (`scale`: device pointer to the upstream gradient of the reduced loss; row_weight = 1 / rows
 * for a mean over all rows).  d_logits may be the logits buffer itself (each element is read before it is written).
 */
int fpb_cross_entropy_fwd(int64_t rows, int32_t V, int32_t dtype, const void* logits, int64_t row_stride,
                          const int64_t* targets, float* loss, float* lse, fpb_stream_t stream);
int fpb_cross_entropy_bwd(int64_t rows, int32_t V, int32_t dtype, const void* logits, int64_t row_stride,
                          const int64_t* targets, const float* lse, const float* scale, float row_weight,
                          void* d_logits, int64_t d_stride, fpb_stream_t stream);

/* Text for a status code. */
const char* fpb_strerror(int status);
/* Library version, major*10000 + minor*100 + patch. */
int fpb_version(void);
/* Which implementation the last successful retention / POP / decoding-step call on this host thread launched (fpb_path). */
int fpb_last_path(void);
/* The cudaError_t behind the last FPB_ERR_LAUNCH on this host thread. */
int fpb_last_cuda_error(void);
/* How many kernels this library has launched so far in this process. */
int64_t fpb_launch_count(void);
/*
 * Synchronises `stream`, then reads and clears the device status word that the kernels set when
 * one of their bounded waits (mbarrier / tensor-memory allocation) gave up.  Returns FPB_OK or
 * FPB_ERR_DEVICE_TIMEOUT; *detail (optional) receives the raw word (role and barrier that gave up).
 */
int fpb_device_status(fpb_stream_t stream, int32_t* detail);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_POP_B200_H_ */
