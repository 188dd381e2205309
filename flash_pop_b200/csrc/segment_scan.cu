// T-segments for under-filled launches of the retention walks.
//
// A walk is one CTA per (batch, head, state tile), strictly sequential over the T/64 chunks of its sequence, so a
// call with few sequences leaves most of the GPU idle (the reference's grid has the same shape:
// flash_pop/fused_retention/fused_chunk_fwd.py:119).  The retention recurrence is linear in the state,
//     S_end = gamma^len S_start + E,   E = the end value of the same piece walked from a zero state,
// so a sequence can be cut into n pieces that are walked concurrently:
//   1. every piece but the last computes its local end value E_s from a zero start (state-only instance of the scan
//      kernel: it reads the two operands of the increment and nothing else) into fp32 scratch memory (B, H, n, dk, dv);
//   2. this file's kernel scans the pieces of each (batch, head): A_0 = S_0, A_{s+1} = gamma^len_s A_s + E_s, and
//      writes A_s over E_s;
//   3. the walk proper runs one CTA per piece from A_s; the last piece ends in the call's end state.
// Reverse walks (the state gradient) are the mirror image: pieces are scanned from the last to the first.
// Everything is deterministic; results differ from the unsplit walk by fp32 rounding of the state only.
#include <atomic>
#include <cmath>

#include "fpb_common.cuh"

namespace fpb {
namespace {

struct CombineParams {
  float* seg;
  const void* start; int64_t start_sb, start_sh;
  int32_t n_seg, seg_len, T, H, reverse, state_f32;
  int64_t state_floats;
  float log2g[FPB_MAX_HEADS];
};

__device__ __forceinline__ float4 load4(const void* base, int64_t off, bool f32) {
  if (f32) return *reinterpret_cast<const float4*>((const float*)base + off);
  const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + off);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
// grid (ceil(dk*dv / 4 / 256), H, B); one thread carries four adjacent state elements through the n pieces
__global__ void __launch_bounds__(256) segment_combine_kernel(const __grid_constant__ CombineParams p) {
  const int64_t e = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (e >= p.state_floats) return;
  const int h = blockIdx.y, b = blockIdx.z;
  const float lg = p.log2g[h];
  float* seg = p.seg + ((int64_t)b * p.H + h) * p.n_seg * p.state_floats + e;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.start) a = load4(p.start, b * p.start_sb + h * p.start_sh + e, p.state_f32 != 0);
  // The local values do not depend on the running value, so the next one is fetched before the current slot is
  // overwritten: the n loads overlap instead of queueing behind one another's stores (the chain of n dependent
  // round trips made this scan the longest of a split call's three launches).
  auto slot_of = [&](int i) { return reinterpret_cast<float4*>(seg + (int64_t)(p.reverse ? p.n_seg - 1 - i : i) * p.state_floats); };
  float4 loc = p.n_seg > 1 ? *slot_of(0) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < p.n_seg; ++i) {
    const int s = p.reverse ? p.n_seg - 1 - i : i;
    float4* slot = slot_of(i);
    if (i == p.n_seg - 1) { *slot = a; break; }      // the piece reached last has no local value: the walk itself ends it
    const float4 next = i + 2 < p.n_seg ? *slot_of(i + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
    const int len = min(p.seg_len, p.T - s * p.seg_len);
    const float g = exp2f((float)len * lg);
    *slot = a;
    a.x = fmaf(g, a.x, loc.x); a.y = fmaf(g, a.y, loc.y); a.z = fmaf(g, a.z, loc.z); a.w = fmaf(g, a.w, loc.w);
    loc = next;
  }
}

int sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cache[dev].load(std::memory_order_acquire);
  if (!n) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_release);
  }
  return n;
}

}  // namespace

constexpr int kMinSegmentTokens = 512;   // a piece shorter than 8 chunks does not pay for its pipeline fill

Segments choose_segments(long long units, int ctas_per_sm, int T, int align, long long batch_heads, long long state_floats,
                         long long scratch_bytes, int B) {
  Segments none{1, 0};
  // Worth it only when the unsplit launch leaves at least half of the SMs without a CTA: with one CTA on (nearly) every
  // SM a second resident CTA adds little, and the first pass and the scan are not free (POP at B x H = 128, d = 64:
  // forward 0.189 ms whole, 0.204 ms in two pieces).
  const long long sms = sm_count();
  const long long slots = sms * ctas_per_sm;
  if (units <= 0 || units * 2 > sms || align <= 0) return none;
  const int min_len = ((kMinSegmentTokens + align - 1) / align) * align;
  long long n = slots / units;
  if (n > T / min_len) n = T / min_len;
  if (scratch_bytes > 0) {                                               // 0: the caller only asks how far a split would go
    const long long fit = scratch_bytes / (batch_heads * state_floats * 4);
    if (n > fit) n = fit;
  }
  if (B > 0 && n > 65535 / B) n = 65535 / B;                             // grid.z = batch x pieces
  if (n < 2) return none;
  const long long per = (T + n - 1) / n;
  const int seg_len = (int)((per + align - 1) / align) * align;
  const int count = (T + seg_len - 1) / seg_len;
  if (count < 2) return none;
  return Segments{count, seg_len};
}

int launch_segment_combine(float* seg, Segments sg, int B, int T, int H, int dk, int dv, const float* gamma, bool reverse,
                           StateView start, bool state_f32, cudaStream_t stream) {
  CombineParams p;
  p.seg = seg;
  p.start = start.data; p.start_sb = start.sb; p.start_sh = start.sh;
  p.n_seg = sg.n; p.seg_len = sg.seg_len; p.T = T; p.H = H; p.reverse = reverse ? 1 : 0; p.state_f32 = state_f32 ? 1 : 0;
  p.state_floats = (int64_t)dk * dv;
  for (int h = 0; h < H; ++h) p.log2g[h] = (float)std::log2((double)gamma[h]);
  const dim3 grid((unsigned)((p.state_floats / 4 + 255) / 256), H, B);
  segment_combine_kernel<<<grid, 256, 0, stream>>>(p);
  return FPB_OK;
}

}  // namespace fpb
