// Device helpers shared by the tcgen05 retention kernels: the chunk schedule, packing, the bounded-wait
// bookkeeping and the diagnostics stamps.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace fpb {
namespace scan {

using namespace ptx;
constexpr int C = 64;                 // chunk length in tokens

struct Chunk { int a, L; };
__device__ __forceinline__ bool next_chunk(Chunk& ck, int T, int bs) {
  const int a = ck.a + ck.L;
  if (a >= T) return false;
  int b = min(a + C, T);
  if (bs > 0) b = min(b, (a / bs + 1) * bs);
  ck.a = a; ck.L = b - a;
  return true;
}
// the same schedule walked from the end: ck.a is the start of the chunk processed before
__device__ __forceinline__ bool prev_chunk(Chunk& ck, int bs) {
  const int end = ck.a;
  if (end <= 0) return false;
  const int base = bs > 0 ? ((end - 1) / bs) * bs : 0;
  const int start = base + ((end - base - 1) / C) * C;
  ck.a = start; ck.L = end - start;
  return true;
}
template <int REV> __device__ __forceinline__ bool advance(Chunk& ck, int T, int bs) {
  return REV ? prev_chunk(ck, bs) : next_chunk(ck, T, bs);
}
__device__ __forceinline__ int chunk_count(int T, int bs) {
  if (bs <= 0) return (T + C - 1) / C;
  return (T / bs) * ((bs + C - 1) / C) + (T % bs + C - 1) / C;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

#define FPB_GIVE_UP(code)                                             \
  do {                                                                \
    atomicCAS(p.status, 0, (code));                                   \
    *abort_flag = 1;                                                  \
  } while (0)

// diagnostics build: stamp event `slot` (0..15) of chunk `c` for CTA (0,0,0) when a trace buffer is installed
#ifdef FPB_DIAGNOSTICS
#define FPB_TRACE(slot, c)                                                                              \
  do {                                                                                                  \
    if (p.trace && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && (c) < 64) p.trace[(c) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define FPB_TRACE(slot, c) do { } while (0)
#endif

// diagnostics build: "leave this piece of work out" switches for timing experiments (the hand-offs stay, the results
// are wrong).  1 tile rescaling, 2 state copy, 4 P', 8 epilogue, 16 state update, 32 one k-step per product, 64 proxy fences
#ifdef FPB_DIAGNOSTICS
#define FPB_ABL(bit) ((p.tune.ablate & (bit)) != 0)
#else
#define FPB_ABL(bit) false
#endif

// diagnostics build: cycles the MMA-issuing thread spends in barrier tests (0), commits (1), tcgen05.mma issue (2) and
// tcgen05 fences (3), with their counts in slots 4-7; written to row 63 of the trace buffer by CTA (0,0,0)
#ifdef FPB_DIAGNOSTICS
#define FPB_PROF_DECL() long long prof_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t_ = 0
#define FPB_PROF_BEGIN() (prof_t_ = clock64())
#define FPB_PROF_END(i) (prof_[i] += clock64() - prof_t_, ++prof_[(i) + 4])
#define FPB_PROF_STORE()                                                                       \
  do {                                                                                         \
    if (p.trace && leader && (blockIdx.x | blockIdx.y | blockIdx.z) == 0)                      \
      for (int i_ = 0; i_ < 8; ++i_) p.trace[63 * 16 + i_] = prof_[i_];                        \
  } while (0)
#else
#define FPB_PROF_DECL() do { } while (0)
#define FPB_PROF_BEGIN() do { } while (0)
#define FPB_PROF_END(i) do { } while (0)
#define FPB_PROF_STORE() do { } while (0)
#endif

// A polling loop that made no progress: true when it should give up (another thread did, or the CTA's wait limit,
// kept in shared memory right after the abort flag, has passed since the last progress).
struct Patience {
  long long t_last;
  int idle;
  __device__ __forceinline__ void progress() { idle = 0; }
  __device__ __forceinline__ bool exhausted(volatile int* abort_flag) {
    if (idle == 0) t_last = clock64();
    if ((++idle & 31) != 0) return false;
    return *abort_flag != 0 || clock64() - t_last > wait_limit(abort_flag);
  }
};


}  // namespace scan
}  // namespace fpb
