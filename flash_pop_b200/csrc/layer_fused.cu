// Elementwise passes either side of the retention operator in a retention layer, each fused into
// one streaming kernel (fp32 arithmetic, bf16 or fp32 tensors):
//   * rotary_kernel: the position rotation of queries and keys (flash_pop/xpos_emb.py:32-40,120-126)
//     from a table of unit phasors, both tensors in one launch; the conjugate rotation is its backward.
//   * gn_gate_fwd / gn_gate_bwd: GroupNorm over each head of each token, without affine parameters,
//     times the (optionally swish-activated) gate (flash_pop/retnet.py:294-309), and its backward.
// All three are HBM-bound: every element is read once and written once.
#include <type_traits>

#include "fpb_common.cuh"

namespace fpb {
namespace {

template <typename T> __device__ __forceinline__ float2 load2(const T* p);
template <> __device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void store2(T* p, float2 v);
template <> __device__ __forceinline__ void store2<float>(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
}

// ---- rotary ---------------------------------------------------------------------------------------
struct RotaryParams {
  SeqView in[2], out[2];
  const float2* phasors;       // (rows, T, d/2) of (cos, sin)
  int64_t ph_sb;               // phasor row stride in float2 units; 0 when every batch row shares one table
  int32_t B, T, H, d;
  float sign;                  // +1 rotates by the angle, -1 by its negative (the backward)
};

// One thread rotates four channel pairs (eight consecutive channels) of one (row, token, head).  A CTA takes whole
// tokens: when a token's H*d/8 units fit its 256 threads, each thread keeps one (head, channel group) for the whole
// launch and only the token changes from one pass to the next, so that the index arithmetic stays out of the loop.
template <typename TIN, typename TOUT>
__device__ __forceinline__ void rotate_unit(const RotaryParams& p, const SeqView& in, const SeqView& out, uint32_t b,
                                            uint32_t t, uint32_t h, uint32_t c) {
  const TIN* src = (const TIN*)in.data + b * in.sb + t * in.st + h * in.sh + c * 8;
  TOUT* dst = (TOUT*)out.data + b * out.sb + t * out.st + h * out.sh + c * 8;
  const float2* ph = p.phasors + b * p.ph_sb + (int64_t)t * (p.d / 2) + c * 4;
  float2 x[4];
  if constexpr (sizeof(TIN) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __bfloat1622float2(e[i]);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(src), b4 = *reinterpret_cast<const float4*>(src + 4);
    x[0] = make_float2(a.x, a.y); x[1] = make_float2(a.z, a.w); x[2] = make_float2(b4.x, b4.y); x[3] = make_float2(b4.z, b4.w);
  }
  const float4 w01 = __ldg(reinterpret_cast<const float4*>(ph)), w23 = __ldg(reinterpret_cast<const float4*>(ph + 2));
  const float2 w[4] = {make_float2(w01.x, w01.y), make_float2(w01.z, w01.w), make_float2(w23.x, w23.y), make_float2(w23.z, w23.w)};
  float2 y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float s = p.sign * w[i].y;
    y[i].x = x[i].x * w[i].x - x[i].y * s;
    y[i].y = x[i].x * s + x[i].y * w[i].x;
  }
  if constexpr (sizeof(TOUT) == 2) {
    uint4 raw;
    __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = __float22bfloat162_rn(y[i]);
    *reinterpret_cast<uint4*>(dst) = raw;
  } else {
    *reinterpret_cast<float4*>(dst) = make_float4(y[0].x, y[0].y, y[1].x, y[1].y);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(y[2].x, y[2].y, y[3].x, y[3].y);
  }
}

template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(256) rotary_kernel(const __grid_constant__ RotaryParams p) {
  const SeqView in = p.in[blockIdx.y], out = p.out[blockIdx.y];
  const uint32_t per_head = p.d / 8, upt = p.H * per_head;          // units per token
  const uint32_t tokens = (uint32_t)p.B * p.T;
  if (upt <= 256) {
    const uint32_t tpb = 256 / upt;                                  // tokens a CTA takes per pass
    const uint32_t lt = threadIdx.x / upt, i = threadIdx.x % upt, h = i / per_head, c = i % per_head;
    if (lt >= tpb) return;
    for (uint32_t tok = blockIdx.x * tpb + lt; tok < tokens; tok += gridDim.x * tpb)
      rotate_unit<TIN, TOUT>(p, in, out, tok / p.T, tok % p.T, h, c);
  } else {
    for (uint32_t tok = blockIdx.x; tok < tokens; tok += gridDim.x)
      for (uint32_t i = threadIdx.x; i < upt; i += 256)
        rotate_unit<TIN, TOUT>(p, in, out, tok / p.T, tok % p.T, i / per_head, i % per_head);
  }
}

// ---- GroupNorm x gate -----------------------------------------------------------------------------
struct GateParams {
  SeqView o, z, y;             // forward: retention output, gate pre-activation (or gate), result
  SeqView dy, d_o, d_z;        // backward
  int64_t groups;              // B*T*H
  int32_t T, H, dv;
  float eps;
  int32_t swish;               // 1: gate = z * sigmoid(z); 0: gate = z
};

template <typename T, int V> __device__ __forceinline__ void load_vec(const T* p, float (&f)[V]) {
  if constexpr (sizeof(T) == 2 && V == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else if constexpr (sizeof(T) == 4 && V == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  } else {
    const float2 a = load2<T>(p);
    f[0] = a.x; f[1] = a.y;
  }
}
template <typename T, int V> __device__ __forceinline__ void store_vec(T* p, const float (&f)[V]) {
  if constexpr (sizeof(T) == 2 && V == 4) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __float22bfloat162_rn(make_float2(f[0], f[1]));
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __float22bfloat162_rn(make_float2(f[2], f[3]));
    *reinterpret_cast<uint2*>(p) = raw;
  } else if constexpr (sizeof(T) == 4 && V == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    store2<T>(p, make_float2(f[0], f[1]));
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int64_t seq_offset(const SeqView& s, uint32_t b, uint32_t t, uint32_t h) {
  return b * s.sb + t * s.st + h * s.sh;
}

// One warp per (row, token, head), G of them in flight per warp so that their loads and reductions overlap:
// lane l owns channels [V*l, V*l + V) of each of the NPASS 32*V-channel passes over a head.
template <typename T, int V, int NPASS, bool BWD>
__global__ void __launch_bounds__(256) gn_gate_kernel(const __grid_constant__ GateParams p) {
  constexpr int G = 1;   // more heads in flight per warp cost registers and measured slower here
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  const uint32_t groups = (uint32_t)p.groups;
  const float inv_n = 1.0f / (float)p.dv;
  for (uint32_t g0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G; g0 < groups; g0 += warps * G) {
    float xo[G][NPASS][V], xz[G][NPASS][V], xd[G][NPASS][V];
    uint32_t hb[G], ht[G], hh[G];
    float sum[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const uint32_t g = g0 + j < groups ? g0 + j : groups - 1;   // a warp past the end repeats the last group
      hh[j] = g % p.H; const uint32_t r = g / p.H; hb[j] = r / p.T; ht[j] = r % p.T;
      const T* o = (const T*)p.o.data + seq_offset(p.o, hb[j], ht[j], hh[j]);
      const T* z = (const T*)p.z.data + seq_offset(p.z, hb[j], ht[j], hh[j]);
      sum[j] = 0.0f;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.dv) {
          load_vec<T, V>(o + c, xo[j][i]);
          load_vec<T, V>(z + c, xz[j][i]);
          if constexpr (BWD) load_vec<T, V>((const T*)p.dy.data + seq_offset(p.dy, hb[j], ht[j], hh[j]) + c, xd[j][i]);
#pragma unroll
          for (int e = 0; e < V; ++e) sum[j] += xo[j][i][e];
        }
      }
    }
    float rstd[G];
#pragma unroll
    for (int j = 0; j < G; ++j) sum[j] = warp_sum(sum[j]) * inv_n;          // mean
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float sq = 0.0f;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        if (V * (lane + 32 * i) < p.dv) {
#pragma unroll
          for (int e = 0; e < V; ++e) { xo[j][i][e] -= sum[j]; sq += xo[j][i][e] * xo[j][i][e]; }
        }
      }
      rstd[j] = sq;
    }
#pragma unroll
    for (int j = 0; j < G; ++j) rstd[j] = rsqrtf(warp_sum(rstd[j]) * inv_n + p.eps);

    if constexpr (!BWD) {
#pragma unroll
      for (int j = 0; j < G; ++j) {
        if (g0 + j >= groups) break;
        T* y = (T*)p.y.data + seq_offset(p.y, hb[j], ht[j], hh[j]);
#pragma unroll
        for (int i = 0; i < NPASS; ++i) {
          const int c = V * (lane + 32 * i);
          if (c < p.dv) {
            float res[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {
              const float gate = p.swish ? __fdividef(xz[j][i][e], 1.0f + __expf(-xz[j][i][e])) : xz[j][i][e];
              res[e] = xo[j][i][e] * rstd[j] * gate;
            }
            store_vec<T, V>(y + c, res);
          }
        }
      }
    } else {
      // y = n * gate(z), n = (o - mean) rstd:  dz = dy n gate'(z);  dn = dy gate;  do = rstd (dn - mean(dn) - n mean(dn n))
      // xd is overwritten with dn, xo with n.
      float s1[G], s2[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        s1[j] = s2[j] = 0.0f;
        const bool real = g0 + j < groups;
        T* d_z = (T*)p.d_z.data + seq_offset(p.d_z, hb[j], ht[j], hh[j]);
#pragma unroll
        for (int i = 0; i < NPASS; ++i) {
          const int c = V * (lane + 32 * i);
          if (c < p.dv) {
            float dz[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {
              const float n = xo[j][i][e] * rstd[j], zz = xz[j][i][e];
              float gate = zz, slope = 1.0f;
              if (p.swish) {
                const float sg = __fdividef(1.0f, 1.0f + __expf(-zz));
                gate = zz * sg;
                slope = sg * (1.0f + zz * (1.0f - sg));
              }
              dz[e] = xd[j][i][e] * n * slope;
              const float dn = xd[j][i][e] * gate;
              xo[j][i][e] = n; xd[j][i][e] = dn;
              s1[j] += dn;
              s2[j] += dn * n;
            }
            if (real) store_vec<T, V>(d_z + c, dz);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < G; ++j) { s1[j] = warp_sum(s1[j]) * inv_n; s2[j] = warp_sum(s2[j]) * inv_n; }
#pragma unroll
      for (int j = 0; j < G; ++j) {
        if (g0 + j >= groups) break;
        T* d_o = (T*)p.d_o.data + seq_offset(p.d_o, hb[j], ht[j], hh[j]);
#pragma unroll
        for (int i = 0; i < NPASS; ++i) {
          const int c = V * (lane + 32 * i);
          if (c < p.dv) {
            float res[V];
#pragma unroll
            for (int e = 0; e < V; ++e) res[e] = rstd[j] * (xd[j][i][e] - s1[j] - xo[j][i][e] * s2[j]);
            store_vec<T, V>(d_o + c, res);
          }
        }
      }
    }
  }
}

// The same computation for heads of 128, 256 or 512 bytes: LPG lanes share a head, 16 bytes each, so a warp holds
// 32/LPG heads per pass and G passes in flight — every access is 16 bytes wide and a warp has 1-2 KB per tensor
// outstanding, which is what it takes to keep HBM busy from a kernel this short.
template <typename T, int LPG, bool BWD>
__global__ void __launch_bounds__(256) gn_gate_packed_kernel(const __grid_constant__ GateParams p) {
  constexpr int V = 16 / sizeof(T), GPW = 32 / LPG, G = 2;
  const int lane = threadIdx.x & 31, sub = lane / LPG, c = (lane % LPG) * V;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  const uint32_t groups = (uint32_t)p.groups;
  const float inv_n = 1.0f / (float)p.dv;
  auto sub_sum = [](float v) {
#pragma unroll
    for (int o = LPG / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  };
  auto load16 = [](const T* ptr, float (&f)[V]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(ptr);
    if constexpr (sizeof(T) == 2) {
      const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
    } else {
      f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
  };
  auto store16 = [](T* ptr, const float (&f)[V]) {
    uint4 raw;
    if constexpr (sizeof(T) == 2) {
      __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) e[i] = __float22bfloat162_rn(make_float2(f[2 * i], f[2 * i + 1]));
    } else {
      raw = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    *reinterpret_cast<uint4*>(ptr) = raw;
  };
  for (uint32_t g0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (GPW * G); g0 < groups; g0 += warps * (GPW * G)) {
    float xo[G][V], xz[G][V], xd[G][V], mean[G], rstd[G];
    int64_t off_o[G], off_z[G];
    uint32_t hb[G], ht[G], hh[G];
    bool real[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const uint32_t want = g0 + j * GPW + sub;
      real[j] = want < groups;
      const uint32_t g = real[j] ? want : groups - 1;             // lanes past the end repeat the last head
      hh[j] = g % p.H; const uint32_t r = g / p.H; hb[j] = r / p.T; ht[j] = r % p.T;
      off_o[j] = seq_offset(p.o, hb[j], ht[j], hh[j]) + c;
      off_z[j] = seq_offset(p.z, hb[j], ht[j], hh[j]) + c;
      load16((const T*)p.o.data + off_o[j], xo[j]);
      load16((const T*)p.z.data + off_z[j], xz[j]);
      if constexpr (BWD) load16((const T*)p.dy.data + seq_offset(p.dy, hb[j], ht[j], hh[j]) + c, xd[j]);
    }
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float s = 0.0f;
#pragma unroll
      for (int e = 0; e < V; ++e) s += xo[j][e];
      mean[j] = s;
    }
#pragma unroll
    for (int j = 0; j < G; ++j) mean[j] = sub_sum(mean[j]) * inv_n;
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float sq = 0.0f;
#pragma unroll
      for (int e = 0; e < V; ++e) { xo[j][e] -= mean[j]; sq += xo[j][e] * xo[j][e]; }
      rstd[j] = sq;
    }
#pragma unroll
    for (int j = 0; j < G; ++j) rstd[j] = rsqrtf(sub_sum(rstd[j]) * inv_n + p.eps);

    if constexpr (!BWD) {
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float res[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float gate = p.swish ? __fdividef(xz[j][e], 1.0f + __expf(-xz[j][e])) : xz[j][e];
          res[e] = xo[j][e] * rstd[j] * gate;
        }
        if (real[j]) store16((T*)p.y.data + seq_offset(p.y, hb[j], ht[j], hh[j]) + c, res);
      }
    } else {
      float s1[G], s2[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        s1[j] = s2[j] = 0.0f;
        float dz[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const float n = xo[j][e] * rstd[j], zz = xz[j][e];
          float gate = zz, slope = 1.0f;
          if (p.swish) {
            const float sg = __fdividef(1.0f, 1.0f + __expf(-zz));
            gate = zz * sg;
            slope = sg * (1.0f + zz * (1.0f - sg));
          }
          dz[e] = xd[j][e] * n * slope;
          const float dn = xd[j][e] * gate;
          xo[j][e] = n; xd[j][e] = dn;
          s1[j] += dn;
          s2[j] += dn * n;
        }
        if (real[j]) store16((T*)p.d_z.data + seq_offset(p.d_z, hb[j], ht[j], hh[j]) + c, dz);
      }
#pragma unroll
      for (int j = 0; j < G; ++j) { s1[j] = sub_sum(s1[j]) * inv_n; s2[j] = sub_sum(s2[j]) * inv_n; }
#pragma unroll
      for (int j = 0; j < G; ++j) {
        float res[V];
#pragma unroll
        for (int e = 0; e < V; ++e) res[e] = rstd[j] * (xd[j][e] - s1[j] - xo[j][e] * s2[j]);
        if (real[j]) store16((T*)p.d_o.data + seq_offset(p.d_o, hb[j], ht[j], hh[j]) + c, res);
      }
    }
  }
}

// ---- LayerNorm with fp32 arithmetic on bf16 (or fp32) rows -----------------------------------------
// The reference's layers run their LayerNorms in fp32 on bf16 activations by casting around them
// (flash_pop/retnet.py:474-486): three passes forward, and a backward whose weight/bias gradient is a
// separate column reduction.  Here a warp owns a row at a time, 16 bytes per lane and pass, statistics
// in registers; the backward keeps its lanes' weight and bias gradient sums in registers over all the
// rows the warp walks and adds them to the output once at the end.
struct NormParams {
  const void* x; const void* dy; void* y; void* dx;
  const float* w; const float* b;
  float* dw; float* db;
  int64_t rows, x_stride, y_stride;      // row strides in elements (dy and dx share y_stride / x_stride)
  int32_t d;
  float eps;
};

template <typename T, int V> __device__ __forceinline__ void load16v(const T* ptr, float (&f)[V]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(ptr);
  if constexpr (sizeof(T) == 2) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
  } else {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
}
template <typename T, int V> __device__ __forceinline__ void store16v(T* ptr, const float (&f)[V]) {
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

// V consecutive fp32 parameters starting at channel c (16-byte loads), or `fill` when there is no such parameter
template <int V> __device__ __forceinline__ void load_params(const float* base, int c, float fill, float (&f)[V]) {
  if (base) {
#pragma unroll
    for (int i = 0; i < V / 4; ++i) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(base + c) + i);
      f[4 * i] = a.x; f[4 * i + 1] = a.y; f[4 * i + 2] = a.z; f[4 * i + 3] = a.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) f[i] = fill;
  }
}

template <typename T, int NPASS>
__global__ void __launch_bounds__(256) layernorm_kernel(const __grid_constant__ NormParams p) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float inv_n = 1.0f / (float)p.d;
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows; row += warps) {
    const T* x = (const T*)p.x + row * p.x_stride;
    float xv[NPASS][V];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      const int c = V * (lane + 32 * i);
      if (c < p.d) {
        load16v<T, V>(x + c, xv[i]);
#pragma unroll
        for (int e = 0; e < V; ++e) sum += xv[i][e];
      }
    }
    const float mean = warp_sum(sum) * inv_n;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      if (V * (lane + 32 * i) < p.d) {
#pragma unroll
        for (int e = 0; e < V; ++e) { xv[i][e] -= mean; sq += xv[i][e] * xv[i][e]; }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_n + p.eps);
    T* y = (T*)p.y + row * p.y_stride;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      const int c = V * (lane + 32 * i);
      if (c < p.d) {
        float res[V], w[V], b[V];
        load_params<V>(p.w, c, 1.0f, w);
        load_params<V>(p.b, c, 0.0f, b);
#pragma unroll
        for (int e = 0; e < V; ++e) res[e] = xv[i][e] * rstd * w[e] + b[e];
        store16v<T, V>(y + c, res);
      }
    }
  }
}

// Sums of N values over the CTA (every thread gets them): a shuffle reduction per warp, then the warps' partial sums
// through `buf` ([warps][N]).  The caller rotates three buffers, so a buffer is rewritten two barriers after its last read.
template <int N> __device__ __forceinline__ void cta_sums(float (&v)[N], float* buf, int warp, int lane, int n_warps) {
#pragma unroll
  for (int k = 0; k < N; ++k) v[k] = warp_sum(v[k]);
  if (n_warps == 1) return;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < N; ++k) buf[warp * N + k] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < N; ++k) {
    float acc = 0.0f;
    for (int w = 0; w < n_warps; ++w) acc += buf[w * N + k];
    v[k] = acc;
  }
}

// 16 raw bytes -> V floats
template <typename T, int V> __device__ __forceinline__ void unpack16v(const uint4& raw, float (&f)[V]) {
  if constexpr (sizeof(T) == 2) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
  } else {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// LayerNorm backward with the whole CTA across a row: thread t owns channels [V t, V t + V) of every row the CTA walks
// (ceil(d / V) threads rounded up to whole warps, at most 128), R rows per step.  A thread's share of the weight and
// bias gradients is then 2 V registers - with one warp per row it was 2 d / 32, which left a quarter of the warps
// resident.  What bounds the pass is the number of bytes in flight, so every thread keeps a ring of LN_DEPTH steps of
// its own 16-byte pieces of x and dy in shared memory, filled by asynchronous copies that it alone waits for and reads
// (no barrier belongs to the ring), while the three CTA-wide reductions of a step (mean; variance; the two sums of the
// input gradient) run.  The gradient sums go out as 16-byte atomic adds at the end (atomic adds into one 32-byte
// sector serialise at a few nanoseconds each, so their number matters: one wave of CTAs, four floats per add).
//   n = (x - mean) rstd, y = n w + b:  dn = dy w;  dx = rstd (dn - mean(dn) - n mean(dn n));  dw += dy n;  db += dy
constexpr int LN_DEPTH = 4;
template <typename T, int R>
__global__ void __launch_bounds__(128) layernorm_bwd_kernel(const __grid_constant__ NormParams p) {
  constexpr int V = 16 / sizeof(T);
  extern __shared__ __align__(16) uint4 ln_ring[];          // [LN_DEPTH][2 R][blockDim.x]
  __shared__ float red[3][4 * 2 * R];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int c = V * threadIdx.x;
  const bool active = c < p.d;
  const float inv_n = 1.0f / (float)p.d;
  float gw[V], gb[V], w[V];
#pragma unroll
  for (int e = 0; e < V; ++e) gw[e] = gb[e] = 0.0f;
  load_params<V>(active ? p.w : nullptr, c, 1.0f, w);
  auto slot = [&](int step, int j) { return ln_ring + ((step % LN_DEPTH) * 2 * R + j) * blockDim.x + threadIdx.x; };
  auto fetch = [&](int step, int64_t base) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (active && base + r < p.rows) {
        cp_async_16(slot(step, 2 * r), (const T*)p.x + (base + r) * p.x_stride + c);
        cp_async_16(slot(step, 2 * r + 1), (const T*)p.dy + (base + r) * p.y_stride + c);
      }
    }
    cp_async_commit();
  };
  const int64_t stride = (int64_t)gridDim.x * R, base0 = (int64_t)blockIdx.x * R;
#pragma unroll
  for (int k = 0; k < LN_DEPTH - 1; ++k) fetch(k, base0 + k * stride);
  int step = 0;
  for (int64_t base = base0; base < p.rows; base += stride, ++step) {
    fetch(step + LN_DEPTH - 1, base + (LN_DEPTH - 1) * stride);
    cp_async_wait<LN_DEPTH - 1>();                          // this step's pieces have landed
    float xv[R][V], dv[R][V];
    float a[R], s[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      uint4 rx = make_uint4(0u, 0u, 0u, 0u), ry = rx;
      if (active && base + r < p.rows) { rx = *slot(step, 2 * r); ry = *slot(step, 2 * r + 1); }
      unpack16v<T, V>(rx, xv[r]);
      unpack16v<T, V>(ry, dv[r]);
      a[r] = 0.0f;
#pragma unroll
      for (int e = 0; e < V; ++e) a[r] += xv[r][e];
    }
    cta_sums<R>(a, red[0], warp, lane, n_warps);
    float mean[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      mean[r] = a[r] * inv_n;
      a[r] = 0.0f;
      if (active) {
#pragma unroll
        for (int e = 0; e < V; ++e) { xv[r][e] -= mean[r]; a[r] += xv[r][e] * xv[r][e]; }
      }
    }
    cta_sums<R>(a, red[1], warp, lane, n_warps);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float rstd = rsqrtf(a[r] * inv_n + p.eps);
      a[r] = rstd;
      s[2 * r] = s[2 * r + 1] = 0.0f;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float n = xv[r][e] * rstd, g = dv[r][e];
        gw[e] += g * n;
        gb[e] += g;
        const float dn = g * w[e];
        xv[r][e] = n; dv[r][e] = dn;
        s[2 * r] += dn;
        s[2 * r + 1] += dn * n;
      }
    }
    cta_sums<2 * R>(s, red[2], warp, lane, n_warps);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (active && base + r < p.rows) {
        const float m1 = s[2 * r] * inv_n, m2 = s[2 * r + 1] * inv_n;
        float res[V];
#pragma unroll
        for (int e = 0; e < V; ++e) res[e] = a[r] * (dv[r][e] - m1 - xv[r][e] * m2);
        store16v<T, V>((T*)p.dx + (base + r) * p.x_stride + c, res);
      }
    }
  }
  cp_async_wait<0>();
  if (active) {
    auto add_out = [&](float* dst, const float (&g)[V]) {
      if (!dst) return;
      if (((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int e = 0; e < V; e += 4) atomicAdd(reinterpret_cast<float4*>(dst + c + e), make_float4(g[e], g[e + 1], g[e + 2], g[e + 3]));
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) atomicAdd(dst + c + e, g[e]);
      }
    };
    add_out(p.dw, gw);
    add_out(p.db, gb);
  }
}

// LayerNorm backward, one warp per row (rows of at most 2 passes of 32 lanes x 16 bytes: the weight / bias gradient sums
// are then at most 32 registers of a lane).  The CTA's sums meet in shared memory and go out as 16-byte atomic adds.
template <typename T, int NPASS>
__global__ void __launch_bounds__(128) layernorm_bwd_warp_kernel(const __grid_constant__ NormParams p) {
  constexpr int V = 16 / sizeof(T);
  extern __shared__ float sh_grad[];             // backward: d floats of weight gradient, d of bias gradient
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float inv_n = 1.0f / (float)p.d;
  float gw[NPASS][V], gb[NPASS][V];
  {
#pragma unroll
    for (int i = 0; i < NPASS; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) gw[i][e] = gb[i][e] = 0.0f;
    for (int i = threadIdx.x; i < 2 * p.d; i += blockDim.x) sh_grad[i] = 0.0f;
    __syncthreads();
  }
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows; row += warps) {
    const T* x = (const T*)p.x + row * p.x_stride;
    float xv[NPASS][V], dv[NPASS][V];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      const int c = V * (lane + 32 * i);
      if (c < p.d) {
        load16v<T, V>(x + c, xv[i]);
        load16v<T, V>((const T*)p.dy + row * p.y_stride + c, dv[i]);
#pragma unroll
        for (int e = 0; e < V; ++e) sum += xv[i][e];
      }
    }
    const float mean = warp_sum(sum) * inv_n;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < NPASS; ++i) {
      if (V * (lane + 32 * i) < p.d) {
#pragma unroll
        for (int e = 0; e < V; ++e) { xv[i][e] -= mean; sq += xv[i][e] * xv[i][e]; }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_n + p.eps);
    {
      // n = (x - mean) rstd, y = n w + b:  dn = dy w;  dx = rstd (dn - mean(dn) - n mean(dn n));  dw += dy n;  db += dy
      float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
          float w[V];
          load_params<V>(p.w, c, 1.0f, w);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float n = xv[i][e] * rstd, g = dv[i][e];
            gw[i][e] += g * n;
            gb[i][e] += g;
            const float dn = g * w[e];
            xv[i][e] = n; dv[i][e] = dn;
            s1 += dn;
            s2 += dn * n;
          }
        }
      }
      const float m1 = warp_sum(s1) * inv_n, m2 = warp_sum(s2) * inv_n;
      T* dx = (T*)p.dx + row * p.x_stride;
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
          float res[V];
#pragma unroll
          for (int e = 0; e < V; ++e) res[e] = rstd * (dv[i][e] - m1 - xv[i][e] * m2);
          store16v<T, V>(dx + c, res);
        }
      }
    }
  }
  {
    if (p.dw || p.db) {
#pragma unroll
      for (int i = 0; i < NPASS; ++i) {
        const int c = V * (lane + 32 * i);
        if (c < p.d) {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            atomicAdd(&sh_grad[c + e], gw[i][e]);
            atomicAdd(&sh_grad[p.d + c + e], gb[i][e]);
          }
        }
      }
      __syncthreads();
      auto add_out = [&](float* dst, const float* src) {
        if (!dst) return;
        if (((uintptr_t)dst & 15) == 0 && p.d % 4 == 0) {
          for (int i = 4 * threadIdx.x; i < p.d; i += 4 * blockDim.x)
            atomicAdd(reinterpret_cast<float4*>(dst + i), make_float4(src[i], src[i + 1], src[i + 2], src[i + 3]));
        } else {
          for (int i = threadIdx.x; i < p.d; i += blockDim.x) atomicAdd(dst + i, src[i]);
        }
      };
      add_out(p.dw, sh_grad);
      add_out(p.db, sh_grad + p.d);
    }
  }
}

int grid_for(int64_t work_items, int per_block) {
  const int64_t blocks = (work_items + per_block - 1) / per_block;
  const int64_t cap = 148 * 16;              // a few waves of the 148 SMs; the kernels loop over the rest
  return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace

int launch_rotary(int in_dtype, int out_dtype, int B, int T, int H, int d, bool conjugate, const float* phasors,
                  int64_t phasor_stride_b, const SeqView in[2], const SeqView out[2], int n_tensors, cudaStream_t stream) {
  RotaryParams p;
  for (int i = 0; i < 2; ++i) { p.in[i] = in[i < n_tensors ? i : 0]; p.out[i] = out[i < n_tensors ? i : 0]; }
  p.phasors = reinterpret_cast<const float2*>(phasors);
  p.ph_sb = phasor_stride_b; p.B = B; p.T = T; p.H = H; p.d = d; p.sign = conjugate ? -1.0f : 1.0f;
  const int64_t upt = (int64_t)H * (d / 8);
  const dim3 grid(grid_for((int64_t)B * T, upt <= 256 ? (int)(256 / upt) : 1), n_tensors);
  if (in_dtype == FPB_BF16 && out_dtype == FPB_BF16) rotary_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else if (in_dtype == FPB_BF16) rotary_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(p);
  else if (out_dtype == FPB_BF16) rotary_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else rotary_kernel<float, float><<<grid, 256, 0, stream>>>(p);
  return FPB_OK;
}

// d <= 4 passes of 32 lanes x 16 bytes (1024 bf16 / 512 fp32 channels); the caller has checked it
int launch_layernorm(int dtype, bool backward, int64_t rows, int d, float eps, const void* x, int64_t x_stride,
                     const float* w, const float* b, void* y, int64_t y_stride, const void* dy, void* dx, float* dw,
                     float* db, cudaStream_t stream) {
  NormParams p;
  p.x = x; p.dy = dy; p.y = y; p.dx = dx; p.w = w; p.b = b; p.dw = dw; p.db = db;
  p.rows = rows; p.x_stride = x_stride; p.y_stride = y_stride; p.d = d; p.eps = eps;
  const int V = dtype == FPB_F32 ? 4 : 8;
  const int npass = (d + 32 * V - 1) / (32 * V);
  if (backward) {
    // one wave of resident CTAs, each walking its share of the rows: a second, partial wave would cost as much as a
    // full one, and every CTA ends with atomic adds into the 2 d gradient sums
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    auto launch = [&](auto kernel, int threads, size_t smem, int64_t blocks) {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
      const int64_t cap = (int64_t)per_sm * sms;
      kernel<<<(int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap)), threads, smem, stream>>>(p);
    };
    auto go = [&](auto tag) {
      using T = decltype(tag);
      if (npass <= 2) {         // narrow rows: a warp per row (measured faster up to 512 bf16 / 256 fp32 channels)
        const size_t smem = 2 * (size_t)d * sizeof(float);
        if (npass == 1) launch(layernorm_bwd_warp_kernel<T, 1>, 128, smem, (rows + 3) / 4);
        else launch(layernorm_bwd_warp_kernel<T, 2>, 128, smem, (rows + 3) / 4);
      } else {                  // wide rows: the CTA across a row, two rows per step
        constexpr int R = 2;
        const int threads = ((d + V - 1) / V + 31) / 32 * 32;
        launch(layernorm_bwd_kernel<T, R>, threads, (size_t)LN_DEPTH * 2 * R * threads * 16, (rows + R - 1) / R);
      }
    };
    if (dtype == FPB_BF16) go(__nv_bfloat16{}); else go(float{});
    return FPB_OK;
  }
  const int64_t blocks = (rows + 7) / 8;
  auto go = [&](auto tag, auto passes) {
    using T = decltype(tag);
    constexpr int NP = decltype(passes)::value;
    const int64_t cap = 148 * 16;
    layernorm_kernel<T, NP><<<(int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap)), 256, 0, stream>>>(p);
  };
  auto by_passes = [&](auto tag) {
    if (npass == 1) go(tag, std::integral_constant<int, 1>{});
    else if (npass == 2) go(tag, std::integral_constant<int, 2>{});
    else go(tag, std::integral_constant<int, 4>{});
  };
  if (dtype == FPB_BF16) by_passes(__nv_bfloat16{}); else by_passes(float{});
  return FPB_OK;
}

int launch_gn_gate(int dtype, bool backward, bool wide, bool packed, int B, int T, int H, int dv, float eps, bool swish, SeqView o,
                   SeqView z, SeqView y, SeqView dy, SeqView d_o, SeqView d_z, cudaStream_t stream) {
  GateParams p;
  p.o = o; p.z = z; p.y = y; p.dy = dy; p.d_o = d_o; p.d_z = d_z;
  p.groups = (int64_t)B * T * H; p.T = T; p.H = H; p.dv = dv; p.eps = eps; p.swish = swish ? 1 : 0;
  const int head_bytes = dv * (dtype == FPB_F32 ? 4 : 2);
  if (packed && (head_bytes == 128 || head_bytes == 256 || head_bytes == 512)) {
    const int lpg = head_bytes / 16;
    const int grid = grid_for((p.groups + (32 / lpg) * 2 - 1) / ((32 / lpg) * 2), 8);
    auto run = [&](auto tag, auto lanes) {
      using T = decltype(tag);
      constexpr int L = decltype(lanes)::value;
      if (backward) gn_gate_packed_kernel<T, L, true><<<grid, 256, 0, stream>>>(p);
      else gn_gate_packed_kernel<T, L, false><<<grid, 256, 0, stream>>>(p);
    };
    auto by_lanes = [&](auto tag) {
      if (lpg == 8) run(tag, std::integral_constant<int, 8>{});
      else if (lpg == 16) run(tag, std::integral_constant<int, 16>{});
      else run(tag, std::integral_constant<int, 32>{});
    };
    if (dtype == FPB_BF16) by_lanes(__nv_bfloat16{}); else by_lanes(float{});
    return FPB_OK;
  }
  // passes of 32 lanes x V channels that cover a head; G groups per warp as in the kernel
  const int V = wide ? 4 : 2;
  const int npass = (dv + 32 * V - 1) / (32 * V);
  const int per_warp = 1;
  const int grid = grid_for((p.groups + per_warp - 1) / per_warp, 8);
  auto go = [&](auto tag, auto vec, auto passes) {
    using T = decltype(tag);
    constexpr int VV = decltype(vec)::value, NP = decltype(passes)::value;
    if (backward) gn_gate_kernel<T, VV, NP, true><<<grid, 256, 0, stream>>>(p);
    else gn_gate_kernel<T, VV, NP, false><<<grid, 256, 0, stream>>>(p);
  };
  auto by_passes = [&](auto tag, auto vec) {
    constexpr int VV = decltype(vec)::value;
    if (npass == 1) go(tag, vec, std::integral_constant<int, 1>{});
    else if (npass == 2) go(tag, vec, std::integral_constant<int, 2>{});
    else if constexpr (VV == 2) {
      if (npass == 3) go(tag, vec, std::integral_constant<int, 3>{}); else go(tag, vec, std::integral_constant<int, 4>{});
    }
  };
  if (dtype == FPB_BF16) {
    if (wide) by_passes(__nv_bfloat16{}, std::integral_constant<int, 4>{}); else by_passes(__nv_bfloat16{}, std::integral_constant<int, 2>{});
  } else {
    if (wide) by_passes(float{}, std::integral_constant<int, 4>{}); else by_passes(float{}, std::integral_constant<int, 2>{});
  }
  return FPB_OK;
}

}  // namespace fpb
