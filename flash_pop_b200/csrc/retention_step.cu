// One recurrent decoding step of retention for every (row, head):
//     S' = gamma_h S + (k / sqrt(dk))^T v,     o = q S'
// (the reference's retention_recurrent, flash_pop/retnet.py:79-101).  The state is the only large
// operand — dk*dv elements read and written per (row, head) — so the kernel is a streaming pass
// over it: 16-byte loads and stores, fp32 arithmetic, the q-weighted column sums reduced through
// shared memory.  A CTA owns one (row, head) and a strip of state columns.
#include "fpb_common.cuh"

namespace fpb {
namespace {

constexpr int STEP_THREADS = 256;
constexpr int STEP_ROW_BYTES = 256;  // bytes of each state row that one CTA owns

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// A thread's VEC state elements of one row as they travel: one 16-byte word, or a single element.
template <typename TS, int VEC> struct RawOf { using type = uint4; };
template <typename TS> struct RawOf<TS, 1> { using type = TS; };

template <typename TS, int VEC> __device__ __forceinline__ void unpack(const typename RawOf<TS, VEC>::type& raw, float (&f)[VEC]) {
  const TS* e = reinterpret_cast<const TS*>(&raw);
#pragma unroll
  for (int i = 0; i < VEC; ++i) f[i] = to_f32<TS>(e[i]);
}
template <typename TS, int VEC> __device__ __forceinline__ typename RawOf<TS, VEC>::type pack(const float (&f)[VEC]) {
  typename RawOf<TS, VEC>::type raw;
  TS* e = reinterpret_cast<TS*>(&raw);
#pragma unroll
  for (int i = 0; i < VEC; ++i) e[i] = from_f32<TS>(f[i]);
  return raw;
}

struct StepParams {
  SeqView q, k, v, o;
  StateView s_prev, s_out;
  int32_t H, dk, dv;
  float gamma[FPB_MAX_HEADS];
};

// TS: state element type, TIO: activation element type, VEC: state elements per thread and row
// (16 bytes' worth when the state is aligned for it, else 1).
template <typename TS, typename TIO, int VEC>
__global__ void __launch_bounds__(STEP_THREADS) step_kernel(const __grid_constant__ StepParams p) {
  constexpr int STEP_COLS = STEP_ROW_BYTES / sizeof(TS);   // state columns per CTA
  constexpr int TX = STEP_COLS / VEC;            // threads across the column strip
  constexpr int TY = STEP_THREADS / TX;          // state rows per pass
  __shared__ float sh_q[256], sh_k[256];
  __shared__ float sh_acc[TY][STEP_COLS + 1];

  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  const int col = blockIdx.y * STEP_COLS + tx * VEC;
  const float gamma = p.gamma[h];
  const float rs = rsqrtf((float)p.dk);

  const TIO* q = (const TIO*)p.q.data + b * p.q.sb + h * p.q.sh;
  const TIO* k = (const TIO*)p.k.data + b * p.k.sb + h * p.k.sh;
  using Raw = typename RawOf<TS, VEC>::type;
  constexpr int UN = 4;                          // state rows a thread has in flight
  const bool live = col < p.dv;                  // dv is a multiple of VEC whenever VEC > 1
  const Raw* sp = live && p.s_prev.data
      ? reinterpret_cast<const Raw*>((const TS*)p.s_prev.data + b * p.s_prev.sb + h * p.s_prev.sh + col) : nullptr;
  Raw* so = live && p.s_out.data ? reinterpret_cast<Raw*>((TS*)p.s_out.data + b * p.s_out.sb + h * p.s_out.sh + col) : nullptr;
  const int64_t row_stride = p.dv / VEC;         // in Raw units
  float vv[VEC], acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) { vv[i] = 0.0f; acc[i] = 0.0f; }

  Raw raw[UN];
  auto fetch = [&](int r0) {                     // rows r0, r0 + TY, ... of this thread's columns
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int r = r0 + u * TY;
      if (sp && r < p.dk) raw[u] = sp[r * row_stride];
    }
  };
  auto update = [&](int r0) {
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int r = r0 + u * TY;
      if (live && r < p.dk) {
        float s[VEC];
        if (sp) {
          unpack<TS, VEC>(raw[u], s);
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) s[i] = 0.0f;
        }
        const float kr = sh_k[r], qr = sh_q[r];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          s[i] = fmaf(gamma, s[i], kr * vv[i]);
          acc[i] = fmaf(qr, s[i], acc[i]);
        }
        if (so) so[r * row_stride] = pack<TS, VEC>(s);
      }
    }
  };

  // the first state rows are requested before q, k, v are staged, so that the two latencies overlap
  fetch(ty);
  for (int i = threadIdx.x; i < p.dk; i += STEP_THREADS) {
    sh_q[i] = to_f32<TIO>(q[i]);
    sh_k[i] = to_f32<TIO>(k[i]) * rs;
  }
  if (live) {
    const TIO* v = (const TIO*)p.v.data + b * p.v.sb + h * p.v.sh + col;
#pragma unroll
    for (int i = 0; i < VEC; ++i) vv[i] = to_f32<TIO>(v[i]);
  }
  __syncthreads();
  update(ty);
  for (int r0 = ty + UN * TY; r0 < p.dk; r0 += UN * TY) {
    fetch(r0);
    update(r0);
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) sh_acc[ty][tx * VEC + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < STEP_COLS) {
    const int c = blockIdx.y * STEP_COLS + threadIdx.x;
    if (c < p.dv) {
      float sum = 0.0f;
#pragma unroll
      for (int y = 0; y < TY; ++y) sum += sh_acc[y][threadIdx.x];
      TIO* o = (TIO*)p.o.data + b * p.o.sb + h * p.o.sh;
      o[c] = from_f32<TIO>(sum);
    }
  }
}

template <typename TS, typename TIO>
void launch_typed(const StepParams& p, int B, bool wide, cudaStream_t stream) {
  constexpr int cols = STEP_ROW_BYTES / sizeof(TS);
  const dim3 grid(B * p.H, (p.dv + cols - 1) / cols);
  if (wide) step_kernel<TS, TIO, 16 / sizeof(TS)><<<grid, STEP_THREADS, 0, stream>>>(p);
  else step_kernel<TS, TIO, 1><<<grid, STEP_THREADS, 0, stream>>>(p);
}

bool aligned16(const StateView& s, int vec) {
  return !s.data || ((uintptr_t)s.data % 16 == 0 && s.sb % vec == 0 && s.sh % vec == 0);
}

}  // namespace

// Launches the decoding step; the caller has validated shapes and strides.
int launch_retention_step(int dtype, int state_dtype, int B, int H, int dk, int dv, const float* gamma, SeqView q,
                          SeqView k, SeqView v, SeqView o, StateView s_prev, StateView s_out, cudaStream_t stream) {
  StepParams p;
  p.q = q; p.k = k; p.v = v; p.o = o; p.s_prev = s_prev; p.s_out = s_out; p.H = H; p.dk = dk; p.dv = dv;
  for (int h = 0; h < H; ++h) p.gamma[h] = gamma[h];
  const size_t es = state_dtype == FPB_F32 ? 4 : 2;
  const int vec = (int)(16 / es);
  const bool wide = dv % vec == 0 && aligned16(s_prev, vec) && aligned16(s_out, vec);
  if (state_dtype == FPB_F32) {
    if (dtype == FPB_F32) launch_typed<float, float>(p, B, wide, stream);
    else launch_typed<float, __nv_bfloat16>(p, B, wide, stream);
  } else {
    if (dtype == FPB_F32) launch_typed<__nv_bfloat16, float>(p, B, wide, stream);
    else launch_typed<__nv_bfloat16, __nv_bfloat16>(p, B, wide, stream);
  }
  return FPB_OK;
}

}  // namespace fpb
