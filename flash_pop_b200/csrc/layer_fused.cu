// Elementwise passes either side of the retention operator in a retention layer, each fused into
// one streaming kernel (fp32 arithmetic, bf16 or fp32 tensors):
//   * rotary_kernel: the position rotation of queries and keys (flash_pop/xpos_emb.py:32-40,120-126)
//     from a table of unit phasors, both tensors in one launch; the conjugate rotation is its backward.
//   * gn_gate_fwd / gn_gate_bwd: GroupNorm over each head of each token, without affine parameters,
//     times the (optionally swish-activated) gate (flash_pop/retnet.py:294-309), and its backward.
// All three are HBM-bound: every element is read once and written once.
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

// One thread rotates four channel pairs (eight consecutive channels) of one (row, token, head).
template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(256) rotary_kernel(const __grid_constant__ RotaryParams p) {
  const int which = blockIdx.y;
  const int per_head = p.d / 8;
  const int64_t total = (int64_t)p.B * p.T * p.H * per_head;
  const SeqView in = p.in[which], out = p.out[which];
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(u % per_head);
    int64_t r = u / per_head;
    const int h = (int)(r % p.H); r /= p.H;
    const int t = (int)(r % p.T);
    const int b = (int)(r / p.T);
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
    const float4 w01 = *reinterpret_cast<const float4*>(ph), w23 = *reinterpret_cast<const float4*>(ph + 2);
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

constexpr int GN_MAX_PAIRS = 4;     // channel pairs per lane: dv <= 256

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int64_t group_offset(const SeqView& s, int64_t g, int T, int H) {
  const int h = (int)(g % H);
  const int64_t r = g / H;
  return (r / T) * s.sb + (r % T) * s.st + h * s.sh;
}

// One warp per (row, token, head): lane l owns channel pairs l, l+32, ... of the head.
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) gn_gate_kernel(const __grid_constant__ GateParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float inv_n = 1.0f / (float)p.dv;
  for (int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g < p.groups; g += warps) {
    const T* o = (const T*)p.o.data + group_offset(p.o, g, p.T, p.H);
    const T* z = (const T*)p.z.data + group_offset(p.z, g, p.T, p.H);
    float2 xo[GN_MAX_PAIRS], xz[GN_MAX_PAIRS], xd[GN_MAX_PAIRS];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < GN_MAX_PAIRS; ++i) {
      const int c = 2 * (lane + 32 * i);
      if (c < p.dv) {
        xo[i] = load2<T>(o + c);
        xz[i] = load2<T>(z + c);
        if constexpr (BWD) xd[i] = load2<T>((const T*)p.dy.data + group_offset(p.dy, g, p.T, p.H) + c);
        sum += xo[i].x + xo[i].y;
      }
    }
    const float mean = warp_sum(sum) * inv_n;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < GN_MAX_PAIRS; ++i) {
      if (2 * (lane + 32 * i) < p.dv) {
        xo[i].x -= mean; xo[i].y -= mean;
        sq += xo[i].x * xo[i].x + xo[i].y * xo[i].y;
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_n + p.eps);
    if constexpr (!BWD) {
      T* y = (T*)p.y.data + group_offset(p.y, g, p.T, p.H);
#pragma unroll
      for (int i = 0; i < GN_MAX_PAIRS; ++i) {
        const int c = 2 * (lane + 32 * i);
        if (c < p.dv) {
          float2 gate = xz[i];
          if (p.swish) { gate.x = gate.x / (1.0f + __expf(-gate.x)); gate.y = gate.y / (1.0f + __expf(-gate.y)); }
          store2<T>(y + c, make_float2(xo[i].x * rstd * gate.x, xo[i].y * rstd * gate.y));
        }
      }
    } else {
      // y = n * gate(z), n = (o - mean) rstd:  dz = dy n gate'(z);  dn = dy gate;  do = rstd (dn - mean(dn) - n mean(dn n))
      float2 dn[GN_MAX_PAIRS];
      float s1 = 0.0f, s2 = 0.0f;
      T* d_z = (T*)p.d_z.data + group_offset(p.d_z, g, p.T, p.H);
#pragma unroll
      for (int i = 0; i < GN_MAX_PAIRS; ++i) {
        const int c = 2 * (lane + 32 * i);
        if (c < p.dv) {
          xo[i].x *= rstd; xo[i].y *= rstd;                  // n
          float2 gate = xz[i], slope = make_float2(1.0f, 1.0f);
          if (p.swish) {
            const float sx = 1.0f / (1.0f + __expf(-xz[i].x)), sy = 1.0f / (1.0f + __expf(-xz[i].y));
            gate = make_float2(xz[i].x * sx, xz[i].y * sy);
            slope = make_float2(sx * (1.0f + xz[i].x * (1.0f - sx)), sy * (1.0f + xz[i].y * (1.0f - sy)));
          }
          store2<T>(d_z + c, make_float2(xd[i].x * xo[i].x * slope.x, xd[i].y * xo[i].y * slope.y));
          dn[i] = make_float2(xd[i].x * gate.x, xd[i].y * gate.y);
          s1 += dn[i].x + dn[i].y;
          s2 += dn[i].x * xo[i].x + dn[i].y * xo[i].y;
        }
      }
      const float m1 = warp_sum(s1) * inv_n, m2 = warp_sum(s2) * inv_n;
      T* d_o = (T*)p.d_o.data + group_offset(p.d_o, g, p.T, p.H);
#pragma unroll
      for (int i = 0; i < GN_MAX_PAIRS; ++i) {
        const int c = 2 * (lane + 32 * i);
        if (c < p.dv)
          store2<T>(d_o + c, make_float2(rstd * (dn[i].x - m1 - xo[i].x * m2), rstd * (dn[i].y - m1 - xo[i].y * m2)));
      }
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
  const dim3 grid(grid_for((int64_t)B * T * H * (d / 8), 256), n_tensors);
  if (in_dtype == FPB_BF16 && out_dtype == FPB_BF16) rotary_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else if (in_dtype == FPB_BF16) rotary_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(p);
  else if (out_dtype == FPB_BF16) rotary_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else rotary_kernel<float, float><<<grid, 256, 0, stream>>>(p);
  return FPB_OK;
}

int launch_gn_gate(int dtype, bool backward, int B, int T, int H, int dv, float eps, bool swish, SeqView o, SeqView z,
                   SeqView y, SeqView dy, SeqView d_o, SeqView d_z, cudaStream_t stream) {
  GateParams p;
  p.o = o; p.z = z; p.y = y; p.dy = dy; p.d_o = d_o; p.d_z = d_z;
  p.groups = (int64_t)B * T * H; p.T = T; p.H = H; p.dv = dv; p.eps = eps; p.swish = swish ? 1 : 0;
  const int grid = grid_for(p.groups, 8);
  if (dtype == FPB_BF16) {
    if (backward) gn_gate_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(p);
    else gn_gate_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(p);
  } else {
    if (backward) gn_gate_kernel<float, true><<<grid, 256, 0, stream>>>(p);
    else gn_gate_kernel<float, false><<<grid, 256, 0, stream>>>(p);
  }
  return FPB_OK;
}

}  // namespace fpb
