// Interface between api.cu and the tcgen05 (5th-generation tensor core) kernel files.
#pragma once

#include "fpb_common.cuh"

namespace fpb {

// Returned by a launcher when the call's shape, dtype or alignment is outside what the tcgen05
// kernels take; the caller then uses the CUDA-core kernels.
constexpr int FPB_UMMA_NOT_APPLICABLE = -1;

struct UmmaFwdArgs {
  SeqView q, k, v, o;
  StateView s0, s_out;
  void* block_states;
  SuffixStates sfx;
  const float* gamma;   // host, H entries
  int B, T, H, dk, dv, dtype, block_size, n_blocks;
  bool state_f32;       // states (s0, s_out, block states) are fp32 although the activations are bf16
  float* scratch; int64_t scratch_bytes;   // caller's fp32 scratch memory for T-segments, or null
};

struct UmmaBwdArgs {
  SeqView q, k, v, dO, dQ, dK, dV;
  StateView s0, d_s_out, d_s0;
  const void* d_block_states;
  SuffixStates sfx_in, sfx_grad;
  const float* gamma;
  int B, T, H, dk, dv, dtype, block_size, n_blocks;
  bool skip_dq, skip_dkdv;
  bool state_f32;
  float* scratch; int64_t scratch_bytes;
};

// *n_launched receives the number of kernels launched (a T-segmented pass is three)
int launch_umma_fwd(const UmmaFwdArgs& a, cudaStream_t stream, int* n_launched);
int launch_umma_bwd(const UmmaBwdArgs& a, cudaStream_t stream, int* n_launched);
// dK, dV, dS_0 in one reverse walk (retention_bwd_fused_sm100.cu); adds its launches to *n_launched
int launch_bwd_fused(const UmmaBwdArgs& a, cudaStream_t stream, int* n_launched);
// local end values of the T-segments of a (reverse) walk over (k, v), into `scratch` (retention_scan_sm100.cu)
int launch_segment_states(SeqView k, SeqView v, bool rev, const void* block_grads, const float* gamma, int B, int T, int H, int dk,
                          int dv, int block_size, int n_blocks, bool state_f32, Segments sg, float* scratch, cudaStream_t stream);
bool segments_enabled();
// dv = 256: the gradient walks cut dv into 128-wide tiles whose partial results TMA adds to a zeroed output
bool col_split_enabled();
// zeros over the (B, T, H, d) bf16 elements of a strided view (d a multiple of 8, 16-byte aligned rows)
void launch_zero_seq(const SeqView& v, int B, int T, int H, int d, cudaStream_t stream);
// How many consecutive suffixes of a row one CTA walks as one sequence: the largest divisor of M (up to a limit)
// that leaves enough CTAs to fill the GPU a few times over; `units` = CTAs per suffix index (rows x heads x tiles).
int choose_suffix_group(int M, long long units);
// diagnostics: device buffer for per-chunk time stamps, or null
long long* debug_trace_ptr();

}  // namespace fpb
