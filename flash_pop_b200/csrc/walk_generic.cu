// CUDA-core retention kernels with fp32 arithmetic: the path for fp32 tensors and for head
// dimensions / decays the tensor-core kernels do not take.
//
// All four passes of the operator are the same rank-1 recurrence on a (dk, dv) state X, walked
// token by token (the reference's recurrent form, flash_pop/retnet.py:79-101, and its transpose
// for the gradients):
//
//        X <- pre * X (+ injected block gradient) + w (x) u ;   out[own] = sum_red r[red] * X[red][own] ;   X <- post * X
//
//   pass            own  red   u        w     r        walk      (pre, post)
//   outputs o       dv   dk    v        k/√dk q        forward   (gamma, 1)
//   dQ              dk   dv    k/√dk    v     dO       forward   (gamma, 1)
//   dV (+ dS_0)     dv   dk    dO       q     k/√dk    reverse   (1, gamma)
//   dK              dk   dv    q        dO    v (/√dk) reverse   (1, gamma)
//
// A CTA owns OWN_TILE indices of the "own" dimension for one (batch, head); KS adjacent lanes share
// one own index and split the "red" dimension between them, NPT contiguous elements each, kept in
// registers for the whole sequence.  Tokens are staged through shared memory TT at a time.
#include "fpb_common.cuh"

namespace fpb {
namespace {

constexpr int KS = 4;          // lanes per own index
constexpr int OWN_TILE = 32;   // own indices per CTA
constexpr int TT = 16;         // tokens per shared-memory tile
constexpr int WALK_THREADS = KS * OWN_TILE;

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// red index -> padded shared-memory column: 4 floats of padding per lane slice keeps the KS lanes
// of one own index on different banks while preserving 16-byte alignment.
template <int NPT> __device__ __forceinline__ int pad_red(int red) { return red + (red / NPT) * 4; }

// T: element type of the activations, TS: element type of the states
template <typename T, typename TS, int NPT>
__global__ void __launch_bounds__(WALK_THREADS) walk_kernel(const __grid_constant__ WalkParams p) {
  constexpr int RED_PAD = KS * NPT + KS * 4;
  __shared__ __align__(16) float s_w[TT][RED_PAD];
  __shared__ __align__(16) float s_r[TT][RED_PAD];
  __shared__ float s_u[TT][OWN_TILE];
  __shared__ float s_o[TT][OWN_TILE];

  const int tid = threadIdx.x;
  const int own_l = tid / KS;
  const int part = tid % KS;
  const int own = blockIdx.x * OWN_TILE + own_l;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int red0 = part * NPT;
  const bool own_ok = own < p.n_own;
  const float gamma = p.gamma[h];
  const float pre = p.dir > 0 ? gamma : 1.0f;
  const float post = p.dir > 0 ? 1.0f : gamma;

  // where this (batch, head)'s start state lives
  const TS* x0 = nullptr;
  TS* x_end = nullptr;
  if (p.sfx.M > 0) {
    const int row = b / p.sfx.M, m = b % p.sfx.M;
    const int64_t state_elems = (int64_t)p.dk * p.dv;
    if (m == 0) {
      if (p.x0.data) x0 = (const TS*)p.x0.data + row * p.x0.sb + h * p.x0.sh;
      if (p.x_out.data) x_end = (TS*)p.x_out.data + row * p.x_out.sb + h * p.x_out.sh;
    } else if (p.sfx.blocks) {   // null in the reverse pass that does not own the state gradient
      TS* blk = (TS*)p.sfx.blocks + (((int64_t)row * p.sfx.N + (m - 1)) * p.H + h) * state_elems;
      if (p.dir > 0) x0 = blk; else x_end = blk;
    }
    if (p.dir < 0) x0 = nullptr;   // suffix end states are dropped: their gradient is zero
  } else {
    if (p.x0.data) x0 = (const TS*)p.x0.data + b * p.x0.sb + h * p.x0.sh;
    if (p.x_out.data) x_end = (TS*)p.x_out.data + b * p.x_out.sb + h * p.x_out.sh;
  }

  float X[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int red = red0 + i;
    X[i] = (x0 && own_ok && red < p.n_red) ? to_f<TS>(x0[red * p.x_stride_red + own * p.x_stride_own]) : 0.0f;
  }

  const T* gu = (const T*)p.u.data + b * p.u.sb + h * p.u.sh;
  const T* gw = (const T*)p.w.data + b * p.w.sb + h * p.w.sh;
  const T* gr = (const T*)p.r.data + b * p.r.sb + h * p.r.sh;
  T* go = (T*)p.out.data + b * p.out.sb + h * p.out.sh;
  const int64_t state_elems = (int64_t)p.dk * p.dv;

  const int n_tiles = (p.T + TT - 1) / TT;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int t_lo = (p.dir > 0 ? tile : n_tiles - 1 - tile) * TT;
    const int t_n = min(TT, p.T - t_lo);
    // stage the tile
    for (int i = tid; i < t_n * p.n_red; i += WALK_THREADS) {
      const int tt = i / p.n_red, red = i % p.n_red;
      const int64_t t = t_lo + tt;
      s_w[tt][pad_red<NPT>(red)] = to_f<T>(gw[t * p.w.st + red]) * p.scale_w;
      s_r[tt][pad_red<NPT>(red)] = to_f<T>(gr[t * p.r.st + red]) * p.scale_r;
    }
    for (int i = tid; i < t_n * OWN_TILE; i += WALK_THREADS) {
      const int tt = i / OWN_TILE, c = i % OWN_TILE;
      const int o_idx = blockIdx.x * OWN_TILE + c;
      s_u[tt][c] = o_idx < p.n_own ? to_f<T>(gu[(int64_t)(t_lo + tt) * p.u.st + o_idx]) * p.scale_u : 0.0f;
    }
    __syncthreads();

    for (int step = 0; step < t_n; ++step) {
      const int tt = p.dir > 0 ? step : t_n - 1 - step;
      const int t = t_lo + tt;
      const bool block_end = p.block_size > 0 && (t + 1) % p.block_size == 0 &&
                             (t + 1) / p.block_size - 1 < p.n_blocks;
      if (p.dir < 0 && block_end && p.block_in && own_ok) {
        const TS* g = (const TS*)p.block_in +
                     (((int64_t)b * p.n_blocks + ((t + 1) / p.block_size - 1)) * p.H + h) * state_elems;
#pragma unroll
        for (int i = 0; i < NPT; ++i)
          if (red0 + i < p.n_red) X[i] += to_f<TS>(g[(red0 + i) * p.x_stride_red + own * p.x_stride_own]);
      }
      const float u = s_u[tt][own_l];
      const float* w = &s_w[tt][pad_red<NPT>(red0)];
      const float* r = &s_r[tt][pad_red<NPT>(red0)];
      float acc = 0.0f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        if (red0 + i < p.n_red) {
          X[i] = fmaf(pre, X[i], w[i] * u);
          acc = fmaf(r[i], X[i], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (part == 0) s_o[tt][own_l] = acc * p.scale_out;
      if (p.dir > 0 && block_end && p.block_out && own_ok) {
        TS* g = (TS*)p.block_out +
               (((int64_t)b * p.n_blocks + ((t + 1) / p.block_size - 1)) * p.H + h) * state_elems;
#pragma unroll
        for (int i = 0; i < NPT; ++i)
          if (red0 + i < p.n_red) g[(red0 + i) * p.x_stride_red + own * p.x_stride_own] = from_f<TS>(X[i]);
      }
#pragma unroll
      for (int i = 0; i < NPT; ++i) X[i] *= post;
    }
    __syncthreads();
    for (int i = tid; i < t_n * OWN_TILE; i += WALK_THREADS) {
      const int tt = i / OWN_TILE, c = i % OWN_TILE;
      const int o_idx = blockIdx.x * OWN_TILE + c;
      if (o_idx < p.n_own) go[(int64_t)(t_lo + tt) * p.out.st + o_idx] = from_f<T>(s_o[tt][c]);
    }
    __syncthreads();
  }

  if (x_end && own_ok) {
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      if (red0 + i < p.n_red) x_end[(red0 + i) * p.x_stride_red + own * p.x_stride_own] = from_f<TS>(X[i]);
  }
}

template <typename T, typename TS>
int launch_t(const WalkParams& p, int B, cudaStream_t stream) {
  // the batch goes into grid.z: launch_walk refuses more than 65535 rows
  const dim3 grid((p.n_own + OWN_TILE - 1) / OWN_TILE, p.H, B);
  if (p.n_red <= 64) walk_kernel<T, TS, 16><<<grid, WALK_THREADS, 0, stream>>>(p);
  else if (p.n_red <= 128) walk_kernel<T, TS, 32><<<grid, WALK_THREADS, 0, stream>>>(p);
  else if (p.n_red <= 256) walk_kernel<T, TS, 64><<<grid, WALK_THREADS, 0, stream>>>(p);
  else return FPB_ERR_BAD_SHAPE;
  return FPB_OK;
}

}  // namespace

int launch_walk(const WalkParams& p, int dtype, bool state_f32, int B, cudaStream_t stream) {
  if (B > 65535) return FPB_ERR_TOO_LARGE;
  if (dtype == FPB_F32) return launch_t<float, float>(p, B, stream);
  if (dtype == FPB_BF16) return state_f32 ? launch_t<__nv_bfloat16, float>(p, B, stream) : launch_t<__nv_bfloat16, __nv_bfloat16>(p, B, stream);
  return FPB_ERR_BAD_DTYPE;
}

}  // namespace fpb
