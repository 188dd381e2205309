// Host-side construction of TMA tensor maps for (B,T,H,d) bf16 activations.  The driver entry point
// cuTensorMapEncodeTiled is looked up at run time through the CUDA runtime, so the library does not
// link against libcuda and can be built on a machine without a GPU driver.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "fpb_common.cuh"

namespace fpb {

typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline tensor_map_encode_fn tensor_map_encoder() {
  static tensor_map_encode_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (tensor_map_encode_fn)p;
  }();
  return fn;
}

// True if TMA can address the tensor: 16-byte aligned base and strides.
inline bool tma_addressable(const SeqView& s, int elem_bytes) {
  const int64_t m = 16 / elem_bytes;
  return s.data && ((uintptr_t)s.data % 16 == 0) && s.st % m == 0 && s.sh % m == 0 && s.sb % m == 0;
}

// Map over a bf16 (B,T,H,d) tensor as dims (d, T, H, B); box = 64 elements (128 bytes, swizzled) x
// `box_rows` tokens of one head of one batch row.  Rows past T read as zero and are not written.
//
// Encoded maps are kept in a small per-thread cache keyed by everything the encoding depends on (pointer, extents,
// strides, box): a training step calls the operator with the same few tensors' shapes over and over (12 layers x 3
// launches x 4-6 maps), and a map stays valid for as long as the address does.  Per thread, so no lock is needed and
// the entry points stay re-entrant.
struct SeqMapKey {
  const void* data;
  int64_t st, sh, sb;
  int32_t B, T, H, d, box_rows;
  bool operator==(const SeqMapKey& o) const {
    return data == o.data && st == o.st && sh == o.sh && sb == o.sb && B == o.B && T == o.T && H == o.H && d == o.d && box_rows == o.box_rows;
  }
};
struct SeqMapSlot { SeqMapKey key; CUtensorMap map; bool used; };
constexpr int kSeqMapSlots = 256;

inline int make_seq_map(CUtensorMap* out, const SeqView& s, int B, int T, int H, int d, int box_rows) {
  // a dimension of extent 1 may come with any stride; give the encoder a harmless valid one
  const int64_t st = T > 1 ? s.st : (int64_t)d;
  const int64_t sh = H > 1 ? s.sh : (int64_t)d;
  const int64_t sb = B > 1 ? s.sb : (int64_t)d;
  const SeqMapKey key{s.data, st, sh, sb, B, T, H, d, box_rows};
  thread_local SeqMapSlot cache[kSeqMapSlots] = {};
  uint64_t hsh = (uint64_t)(uintptr_t)s.data * 0x9E3779B97F4A7C15ull;
  hsh ^= ((uint64_t)T * 0x100000001B3ull) ^ ((uint64_t)box_rows << 40) ^ ((uint64_t)d << 48) ^ ((uint64_t)st << 20) ^ (uint64_t)sb;
  SeqMapSlot& slot = cache[(hsh >> 24) % kSeqMapSlots];
  if (slot.used && slot.key == key) { *out = slot.map; return FPB_OK; }
  tensor_map_encode_fn enc = tensor_map_encoder();
  if (!enc) return FPB_ERR_TENSOR_MAP;
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, s.data, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return FPB_ERR_TENSOR_MAP;
  slot.key = key; slot.map = *out; slot.used = true;
  return FPB_OK;
}

}  // namespace fpb
