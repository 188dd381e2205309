// Shared declarations of the flash_pop_b200 CUDA sources: launch parameter blocks, the device
// status word, and the internal launcher interface between api.cu and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/flash_pop_b200.h"

#define FPB_MAX_HEADS 256

namespace fpb {

// One (B,T,H,d) tensor as the kernels see it.
struct SeqView {
  void* data;
  int64_t sb, st, sh;
};

// One (B,H,dk,dv) state, or a slice of a (B,N,H,dk,dv) block-state tensor.
struct StateView {
  void* data;
  int64_t sb, sh;
};

// Where a walk starts (or a reverse walk ends) when the batch is a flattened (row, suffix) pair:
// suffix m of row r uses first[r] for m == 0 and blocks[r, m-1] otherwise.
struct SuffixStates {
  int32_t M;           // suffixes per row; 0 = not a suffix call
  int32_t N;           // blocks per row in `blocks`
  void* blocks;        // (B, N, H, dk, dv) contiguous
};

// Parameters of the CUDA-core "walk" kernel (walk_generic.cu).
struct WalkParams {
  SeqView u, w, r, out;
  StateView x0, x_out;
  SuffixStates sfx;
  void* block_out;         // forward: states after full blocks (B, NB, H, dk, dv)
  const void* block_in;    // reverse: gradients of those states
  int64_t x_stride_red, x_stride_own;   // element strides inside one (dk, dv) state
  int32_t n_own, n_red, T, H, dk, dv;
  int32_t dir;             // +1 walks t = 0..T-1, -1 walks t = T-1..0
  int32_t block_size, n_blocks;
  float scale_u, scale_w, scale_r, scale_out;
  float gamma[FPB_MAX_HEADS];
};

// `state_f32`: the states (x0, x_out, block states, suffix start states) are fp32 whatever the activations are
int launch_walk(const WalkParams& p, int dtype, bool state_f32, int B, cudaStream_t stream);

// One recurrent decoding step (retention_step.cu); `dtype` is that of q, k, v, o, `state_dtype` that of the states.
int launch_retention_step(int dtype, int state_dtype, int B, int H, int dk, int dv, const float* gamma, SeqView q,
                          SeqView k, SeqView v, SeqView o, StateView s_prev, StateView s_out, cudaStream_t stream);

// Fused elementwise passes around the operator (layer_fused.cu).
int launch_rotary(int in_dtype, int out_dtype, int B, int T, int H, int d, bool conjugate, const float* phasors,
                  int64_t phasor_stride_b, const SeqView in[2], const SeqView out[2], int n_tensors, cudaStream_t stream);
// `wide`: every tensor allows accesses of four elements (dv % 4 == 0, pointers and strides aligned for them);
// `packed`: every tensor allows 16-byte accesses
int launch_gn_gate(int dtype, bool backward, bool wide, bool packed, int B, int T, int H, int dv, float eps, bool swish, SeqView o,
                   SeqView z, SeqView y, SeqView dy, SeqView d_o, SeqView d_z, cudaStream_t stream);

int launch_layernorm(int dtype, bool backward, int64_t rows, int d, float eps, const void* x, int64_t x_stride,
                     const float* w, const float* b, void* y, int64_t y_stride, const void* dy, void* dx, float* dw,
                     float* db, cudaStream_t stream);

// Adaptive LayerNorm modulation and gated residual with row-broadcast operands (adaln_fused.cu).
int launch_adaln(int dtype, bool backward, int64_t rows, int d, float eps, const void* x, int64_t x_stride, const void* shift,
                 const void* scale, int64_t mod_stride, int64_t rows_per_mod, void* y, int64_t y_stride, const void* dy,
                 int64_t dy_stride, void* dx, float* d_shift, float* d_scale, cudaStream_t stream);
int launch_gate_residual(int dtype, bool backward, int64_t rows, int d, const void* x_or_dout, int64_t x_stride, const void* branch,
                         int64_t branch_stride, const void* gate, int64_t mod_stride, int64_t rows_per_mod, void* out,
                         int64_t out_stride, void* d_branch, float* d_gate, cudaStream_t stream);

// Softmax cross entropy of (rows x V) logits against int64 targets (loss_fused.cu).
int launch_xent_fwd(int dtype, int64_t rows, int V, const void* logits, int64_t row_stride, const int64_t* targets, float* loss,
                    float* lse, cudaStream_t stream);
int launch_xent_bwd(int dtype, int64_t rows, int V, const void* logits, int64_t row_stride, const int64_t* targets, const float* lse,
                    const float* scale, float row_weight, void* d_logits, int64_t d_stride, cudaStream_t stream);

// Per-launch knobs of the tcgen05 kernels.  A release build always passes the defaults; the diagnostics build
// (-DFPB_DIAGNOSTICS) exports setters so that tests can shorten the wait limit or compare schedules.
struct WalkTuning {
  long long wait_cycles;    // limit of every bounded wait inside a kernel, in clock64() ticks
  int32_t idle_ns;          // suspend hint (ns) of a polling loop that found nothing to do
  int32_t sc_early;         // walks whose scores do not read the scaled tile issue them as soon as the tiles landed
  int32_t withhold_chunk;   // diagnostics only: the producer never loads this chunk of any sequence (-1 = none)
  int32_t ablate;           // diagnostics only: bit mask of work to leave out (results are then wrong; timing experiments)
};
const WalkTuning& walk_tuning();

// Cutting each sequence of an under-filled launch into `n` T-segments of `seg_len` tokens (see segment_scan.cu).
struct Segments {
  int32_t n, seg_len;       // n == 1: the sequences are walked whole
};
// `units` CTAs the launch would have unsplit, `ctas_per_sm` of them resident per SM; `align` = token count every
// segment start must be a multiple of; state_floats = dk * dv; scratch holds B*H*n*state_floats floats.
Segments choose_segments(long long units, int ctas_per_sm, int T, int align, long long batch_heads, long long state_floats,
                         long long scratch_bytes, int B);
// Start values of the segments from the local end values of all but the piece reached last: in place over `seg`
// (B, H, n, dk, dv) fp32.
//   forward : A_0 = start, A_{s+1} = gamma^len_s A_s + E_s ; seg[s] <- A_s
//   reverse : A_{n-1} = start, A_{s-1} = gamma^len_s A_s + E_s ; seg[s] <- A_s
int launch_segment_combine(float* seg, Segments sg, int B, int T, int H, int dk, int dv, const float* gamma, bool reverse,
                           StateView start, bool state_f32, cudaStream_t stream);

// Device status word shared by all kernels: 0 = fine; otherwise (role << 8 | barrier id) of the
// first bounded wait that gave up.
int32_t* device_status_ptr();

}  // namespace fpb
