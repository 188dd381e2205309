// Softmax cross entropy over a vocabulary row, fp32 arithmetic on bf16 (or fp32) logits, for the language-model
// head of the full-stack training workload.  PyTorch's path casts the (tokens x vocabulary) logits to fp32 and runs
// log-softmax, the loss and their backward as separate passes over that copy; here the forward reads each row once
// (online max / sum) and the backward reads it once more and writes the gradient in the logits' own type.
// One CTA per row; a 32000-entry bf16 row is 64 KB and stays in L2 between the two reads of the backward's owner.
#include "fpb_common.cuh"

namespace fpb {
namespace {

constexpr int XENT_THREADS = 256;

template <typename T> __device__ __forceinline__ float xe_to_f(T x);
template <> __device__ __forceinline__ float xe_to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float xe_to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

// V elements (16 bytes' worth) of a row as floats
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };
template <typename T> __device__ __forceinline__ void load16(const T* p, float (&f)[Vec16<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 2) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
  } else {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
}
template <typename T> __device__ __forceinline__ void store16(T* p, const float (&f)[Vec16<T>::N]) {
  uint4 raw;
  if constexpr (sizeof(T) == 2) {
    __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = __float22bfloat162_rn(make_float2(f[2 * i], f[2 * i + 1]));
  } else {
    raw = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  *reinterpret_cast<uint4*>(p) = raw;
}

// (running max, sum of exp(x - max)) pairs combine associatively
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  s = (m == -INFINITY ? 0.0f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.0f : s2 * __expf(m2 - mm));
  m = mm;
}

template <typename T>
__global__ void __launch_bounds__(XENT_THREADS) xent_fwd_kernel(const T* __restrict__ logits, int64_t row_stride, int V,
                                                               const int64_t* __restrict__ targets, float* __restrict__ loss,
                                                               float* __restrict__ lse) {
  constexpr int N = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const T* x = logits + row * row_stride;
  float m = -INFINITY, s = 0.0f;
  const int vec_end = (V / N) * N;
  for (int c = threadIdx.x * N; c < vec_end; c += XENT_THREADS * N) {
    float f[N];
    load16<T>(x + c, f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < N; ++i) lm = fmaxf(lm, f[i]);
    if (lm > m) { s *= __expf(m - lm); m = lm; }       // exp(-inf) = 0 covers the first vector
#pragma unroll
    for (int i = 0; i < N; ++i) s += __expf(f[i] - m);
  }
  for (int c = vec_end + threadIdx.x; c < V; c += XENT_THREADS) lse_merge(m, s, xe_to_f<T>(x[c]), 1.0f);
  // combine over the CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lse_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  __shared__ float sh_m[XENT_THREADS / 32], sh_s[XENT_THREADS / 32];
  if ((threadIdx.x & 31) == 0) { sh_m[threadIdx.x >> 5] = m; sh_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < XENT_THREADS / 32; ++w) lse_merge(m, s, sh_m[w], sh_s[w]);
    const float l = m + __logf(s);
    const int64_t t = targets[row];
    lse[row] = l;
    loss[row] = (t >= 0 && t < V) ? l - xe_to_f<T>(x[t]) : 0.0f;   // a target outside the vocabulary is ignored
  }
}

// d_logits[row, j] = (softmax_j - [j == target]) * scale[0] * row_weight, row_weight = 1 / rows for the mean loss
template <typename T>
// logits and d_logits may be the same buffer (each thread reads an element before it writes it): no __restrict__ on them
__global__ void __launch_bounds__(XENT_THREADS) xent_bwd_kernel(const T* logits, int64_t row_stride, int V,
                                                               const int64_t* __restrict__ targets, const float* __restrict__ lse,
                                                               const float* __restrict__ scale, float row_weight,
                                                               T* d_logits, int64_t d_stride) {
  constexpr int N = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const T* x = logits + row * row_stride;
  T* dx = d_logits + row * d_stride;
  const float l = lse[row];
  const int64_t t = targets[row];
  const bool live = t >= 0 && t < V;
  const float g = live ? scale[0] * row_weight : 0.0f;
  const int vec_end = (V / N) * N;
  for (int c = threadIdx.x * N; c < vec_end; c += XENT_THREADS * N) {
    float f[N];
    load16<T>(x + c, f);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = (__expf(f[i] - l) - ((int64_t)(c + i) == t ? 1.0f : 0.0f)) * g;
    store16<T>(dx + c, f);
  }
  for (int c = vec_end + threadIdx.x; c < V; c += XENT_THREADS) {
    const float v = (__expf(xe_to_f<T>(x[c]) - l) - ((int64_t)c == t ? 1.0f : 0.0f)) * g;
    if constexpr (sizeof(T) == 2) dx[c] = __float2bfloat16_rn(v); else dx[c] = v;
  }
}

}  // namespace

int launch_xent_fwd(int dtype, int64_t rows, int V, const void* logits, int64_t row_stride, const int64_t* targets, float* loss,
                    float* lse, cudaStream_t stream) {
  if (dtype == FPB_BF16)
    xent_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, XENT_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, row_stride, V, targets, loss, lse);
  else
    xent_fwd_kernel<float><<<(unsigned)rows, XENT_THREADS, 0, stream>>>((const float*)logits, row_stride, V, targets, loss, lse);
  return FPB_OK;
}

int launch_xent_bwd(int dtype, int64_t rows, int V, const void* logits, int64_t row_stride, const int64_t* targets, const float* lse,
                    const float* scale, float row_weight, void* d_logits, int64_t d_stride, cudaStream_t stream) {
  if (dtype == FPB_BF16)
    xent_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, XENT_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, row_stride, V, targets, lse,
                                                                             scale, row_weight, (__nv_bfloat16*)d_logits, d_stride);
  else
    xent_bwd_kernel<float><<<(unsigned)rows, XENT_THREADS, 0, stream>>>((const float*)logits, row_stride, V, targets, lse, scale,
                                                                     row_weight, (float*)d_logits, d_stride);
  return FPB_OK;
}

}  // namespace fpb
