// Adaptive LayerNorm modulation and gated residual of the diffusion RetNet layers, each as one streaming kernel
// (fp32 arithmetic on bf16 or fp32 rows).  The reference computes them as separate PyTorch passes over (B, T, D):
//   modulate:  y = LayerNorm(x) * (1 + scale) + shift          (flash_pop/modules/adaln.py:13-15,90-99,154-166)
//   residual:  out = x + gate * branch                          (flash_pop/diffusion_retnet.py:133-146)
// where shift / scale / gate come from a small MLP on the conditioning and are shared by `rows_per_mod` consecutive
// rows of x: all T tokens of a batch row (conditioning (B, D)), the tokens of one frame ((B, T', D)), or one token.
// They are read as rows of the MLP's output in place - a (rows / rows_per_mod, n * D) matrix viewed with a row stride -
// and never expanded to (B, T, D).
//
// A warp owns a contiguous range of rows, 16 bytes per lane and pass (as layernorm_kernel in layer_fused.cu).  In the
// backward passes the gradients of shift, scale and gate are sums over the rows that share a modulation row: the warp
// keeps them in registers while its rows stay on one modulation row and adds them to the fp32 outputs (atomically:
// several warps may share a modulation row) when that changes.
#include <type_traits>

#include "fpb_common.cuh"

namespace fpb {
namespace {

template <typename T, int V> __device__ __forceinline__ void ld16(const T* ptr, float (&f)[V]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(ptr);
  if constexpr (sizeof(T) == 2) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
  } else {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
}
template <typename T, int V> __device__ __forceinline__ void st16(T* ptr, const float (&f)[V]) {
  uint4 raw;
  if constexpr (sizeof(T) == 2) {
    __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = __float22bfloat162_rn(make_float2(f[2 * i], f[2 * i + 1]));
  } else {
    raw = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  *reinterpret_cast<uint4*>(ptr) = raw;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct ModParams {
  const void* x; const void* other;      // other: dy (modulate backward), branch (residual)
  void* y; void* d_in;                   // y: forward output; d_in: dx (modulate backward) / d_branch (residual backward)
  const void* shift; const void* scale;  // modulate; `scale` is the gate of the residual
  float* g_a; float* g_b;                // backward: fp32 (mod_rows, d) sums: d_shift, d_scale | d_gate, unused
  int64_t rows, x_stride, other_stride, y_stride, mod_stride, rows_per_mod;
  int32_t d;
  float eps;
};

// rows [lo, hi) of this warp: the rows are dealt out in contiguous ranges so that a warp stays on one modulation row
__device__ __forceinline__ void my_rows(const ModParams& p, int64_t& lo, int64_t& hi) {
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t per = (p.rows + warps - 1) / warps;
  lo = w * per;
  hi = lo + per < p.rows ? lo + per : p.rows;
}

// MODE 0: y = norm(x) (1 + scale) + shift      MODE 1: its backward (dx, d_shift, d_scale)
template <typename T, int NPASS, int MODE>
__global__ void __launch_bounds__(128) adaln_kernel(const __grid_constant__ ModParams p) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const float inv_n = 1.0f / (float)p.d;
  int64_t lo, hi;
  my_rows(p, lo, hi);
  float ga[MODE ? NPASS : 1][V], gb[MODE ? NPASS : 1][V];     // running d_shift, d_scale of the current modulation row
  int64_t cur = -1;
  auto flush = [&]() {
    if constexpr (MODE == 1) {
      if (cur < 0) return;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            atomicAdd(p.g_a + cur * p.d + c + e, ga[i][e]);
            atomicAdd(p.g_b + cur * p.d + c + e, gb[i][e]);
            ga[i][e] = gb[i][e] = 0.0f;
          }
        }
      }
    }
  };
  if constexpr (MODE == 1) {
#pragma unroll
    for (int i = 0; i < NPASS; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) ga[i][e] = gb[i][e] = 0.0f;
  }
  for (int64_t row = lo; row < hi; ++row) {
    const int64_t m = row / p.rows_per_mod;
    if (MODE == 1 && m != cur) { flush(); cur = m; }
    const T* x = (const T*)p.x + row * p.x_stride;
    float xv[NPASS][V];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      const int c = V * (lane + 32 * i);
      if (c < p.d) {
        ld16<T, V>(x + c, xv[i]);
#pragma unroll
        for (int e = 0; e < V; ++e) sum += xv[i][e];
      }
    }
    const float mean = wsum(sum) * inv_n;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      if (V * (lane + 32 * i) < p.d) {
#pragma unroll
        for (int e = 0; e < V; ++e) { xv[i][e] -= mean; sq += xv[i][e] * xv[i][e]; }
      }
    }
    const float rstd = rsqrtf(wsum(sq) * inv_n + p.eps);
    const T* sc = (const T*)p.scale + m * p.mod_stride;
    if constexpr (MODE == 0) {
      const T* sh = (const T*)p.shift + m * p.mod_stride;
      T* y = (T*)p.y + row * p.y_stride;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
          float a[V], b[V], res[V];
          ld16<T, V>(sc + c, a);
          ld16<T, V>(sh + c, b);
#pragma unroll
          for (int e = 0; e < V; ++e) res[e] = xv[i][e] * rstd * (1.0f + a[e]) + b[e];
          st16<T, V>(y + c, res);
        }
      }
    } else {
      // n = (x - mean) rstd, y = n (1 + scale) + shift:  dn = dy (1 + scale);  dx = rstd (dn - mean(dn) - n mean(dn n));
      // d_shift += dy;  d_scale += dy n
      const T* dy = (const T*)p.other + row * p.other_stride;
      float dn[NPASS][V];
      float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
          float a[V], g[V];
          ld16<T, V>(sc + c, a);
          ld16<T, V>(dy + c, g);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float n = xv[i][e] * rstd;
            ga[i][e] += g[e];
            gb[i][e] += g[e] * n;
            xv[i][e] = n;
            dn[i][e] = g[e] * (1.0f + a[e]);
            s1 += dn[i][e];
            s2 += dn[i][e] * n;
          }
        }
      }
      const float m1 = wsum(s1) * inv_n, m2 = wsum(s2) * inv_n;
      T* dx = (T*)p.d_in + row * p.x_stride;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
          float res[V];
#pragma unroll
          for (int e = 0; e < V; ++e) res[e] = rstd * (dn[i][e] - m1 - xv[i][e] * m2);
          st16<T, V>(dx + c, res);
        }
      }
    }
  }
  flush();
}

// MODE 0: out = x + gate * branch      MODE 1: d_branch = d_out * gate, d_gate += d_out * branch   (d_x = d_out itself)
template <typename T, int NPASS, int MODE>
__global__ void __launch_bounds__(256) gate_residual_kernel(const __grid_constant__ ModParams p) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  int64_t lo, hi;
  my_rows(p, lo, hi);
  float gg[MODE ? NPASS : 1][V];
  int64_t cur = -1;
  auto flush = [&]() {
    if constexpr (MODE == 1) {
      if (cur < 0) return;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
#pragma unroll
          for (int e = 0; e < V; ++e) { atomicAdd(p.g_a + cur * p.d + c + e, gg[i][e]); gg[i][e] = 0.0f; }
        }
      }
    }
  };
  if constexpr (MODE == 1) {
#pragma unroll
    for (int i = 0; i < NPASS; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) gg[i][e] = 0.0f;
  }
  for (int64_t row = lo; row < hi; ++row) {
    const int64_t m = row / p.rows_per_mod;
    if (MODE == 1 && m != cur) { flush(); cur = m; }
    const T* gate = (const T*)p.scale + m * p.mod_stride;
    const T* br = (const T*)p.other + row * p.other_stride;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      const int c = V * (lane + 32 * i);
      if (c < p.d) {
        float g[V], b[V], a[V], res[V];
        ld16<T, V>(gate + c, g);
        ld16<T, V>(br + c, b);
        ld16<T, V>((const T*)p.x + row * p.x_stride + c, a);       // x (forward) or d_out (backward)
        if constexpr (MODE == 0) {
#pragma unroll
          for (int e = 0; e < V; ++e) res[e] = a[e] + g[e] * b[e];
          st16<T, V>((T*)p.y + row * p.y_stride + c, res);
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e) { res[e] = a[e] * g[e]; gg[i][e] += a[e] * b[e]; }
          st16<T, V>((T*)p.d_in + row * p.other_stride + c, res);
        }
      }
    }
  }
  flush();
}

int blocks_for(int64_t rows, int warps_per_block, int ctas_per_sm) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (rows + warps_per_block - 1) / warps_per_block;
  const int64_t cap = (int64_t)sms * ctas_per_sm;                // one resident wave; every warp walks a range of rows
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename F>
void by_shape(int dtype, int d, F&& go) {
  const int V = dtype == FPB_F32 ? 4 : 8;
  const int npass = (d + 32 * V - 1) / (32 * V);
  auto passes = [&](auto tag) {
    if (npass == 1) go(tag, std::integral_constant<int, 1>{});
    else if (npass == 2) go(tag, std::integral_constant<int, 2>{});
    else go(tag, std::integral_constant<int, 4>{});
  };
  if (dtype == FPB_BF16) passes(__nv_bfloat16{}); else passes(float{});
}

}  // namespace

int launch_adaln(int dtype, bool backward, int64_t rows, int d, float eps, const void* x, int64_t x_stride, const void* shift,
                 const void* scale, int64_t mod_stride, int64_t rows_per_mod, void* y, int64_t y_stride, const void* dy,
                 int64_t dy_stride, void* dx, float* d_shift, float* d_scale, cudaStream_t stream) {
  ModParams p{};
  p.x = x; p.other = dy; p.y = y; p.d_in = dx; p.shift = shift; p.scale = scale; p.g_a = d_shift; p.g_b = d_scale;
  p.rows = rows; p.x_stride = x_stride; p.other_stride = dy_stride; p.y_stride = y_stride; p.mod_stride = mod_stride;
  p.rows_per_mod = rows_per_mod; p.d = d; p.eps = eps;
  by_shape(dtype, d, [&](auto tag, auto passes) {
    using T = decltype(tag);
    constexpr int NP = decltype(passes)::value;
    if (backward) adaln_kernel<T, NP, 1><<<blocks_for(rows, 4, 4), 128, 0, stream>>>(p);
    else adaln_kernel<T, NP, 0><<<blocks_for(rows, 4, 8), 128, 0, stream>>>(p);
  });
  return FPB_OK;
}

int launch_gate_residual(int dtype, bool backward, int64_t rows, int d, const void* x_or_dout, int64_t x_stride, const void* branch,
                         int64_t branch_stride, const void* gate, int64_t mod_stride, int64_t rows_per_mod, void* out,
                         int64_t out_stride, void* d_branch, float* d_gate, cudaStream_t stream) {
  ModParams p{};
  p.x = x_or_dout; p.other = branch; p.y = out; p.d_in = d_branch; p.scale = gate; p.g_a = d_gate;
  p.rows = rows; p.x_stride = x_stride; p.other_stride = branch_stride; p.y_stride = out_stride; p.mod_stride = mod_stride;
  p.rows_per_mod = rows_per_mod; p.d = d;
  by_shape(dtype, d, [&](auto tag, auto passes) {
    using T = decltype(tag);
    constexpr int NP = decltype(passes)::value;
    if (backward) gate_residual_kernel<T, NP, 1><<<blocks_for(rows, 8, 4), 256, 0, stream>>>(p);
    else gate_residual_kernel<T, NP, 0><<<blocks_for(rows, 8, 4), 256, 0, stream>>>(p);
  });
  return FPB_OK;
}

}  // namespace fpb
