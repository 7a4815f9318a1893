// Tree-attention mask rows in the forms the reference's callers hand to the model forward.
//
//   bool rows            Tree.create_attention_mask / TreeMaskCache (specdecodes/models/utils/cpu_tree.py:263-286,
//                        specdecodes/models/draft_models/base.py:93-117): 1 = may attend
//   additive rows        invert_mask (specdecodes/models/utils/utils.py:4-6): (~m).to(dtype) * finfo(dtype).min,
//                        i.e. -0.0 where the row may attend (0 * a negative number) and finfo.min elsewhere
//
// A row is [prefix ones | tree columns | zeros up to `cols`]: the zeros are what the reference's preallocated
// [1, 1, rows, max_cache_len] buffers hold behind the columns in use (generators/classic_sd.py:33-55).
#pragma once

#include "common.cuh"

namespace subspec {

struct MaskFmt {
  int esz;       // bytes per element: 1, 2 or 4
  uint32_t on;   // element pattern of "may attend", replicated to 32 bits
  uint32_t off;  // element pattern of "masked", replicated to 32 bits
};

__host__ __device__ inline bool mask_kind_ok(int kind) { return kind >= SUBSPEC_MASK_BOOL && kind <= SUBSPEC_MASK_ADD_F16; }
__host__ __device__ inline int mask_elem_bytes(int kind) {
  return kind == SUBSPEC_MASK_BOOL ? 1 : (kind == SUBSPEC_MASK_ADD_F32 ? 4 : 2);
}

#ifdef __CUDACC__

__device__ __forceinline__ MaskFmt mask_fmt(int kind) {
  switch (kind) {
    case SUBSPEC_MASK_ADD_F32:
      return MaskFmt{4, 0x80000000u, 0xff7fffffu};  // -0.0f, -FLT_MAX
    case SUBSPEC_MASK_ADD_BF16:
      return MaskFmt{2, 0x80008000u, 0xff7fff7fu};  // -0.0, -3.3895e38
    case SUBSPEC_MASK_ADD_F16:
      return MaskFmt{2, 0x80008000u, 0xfbfffbffu};  // -0.0, -65504
    default:
      return MaskFmt{1, 0x01010101u, 0u};
  }
}

__device__ __forceinline__ void mask_store(uint8_t* row, int64_t c, const MaskFmt& f, bool on) {
  const uint32_t v = on ? f.on : f.off;
  if (f.esz == 1)
    row[c] = (uint8_t)v;
  else if (f.esz == 2)
    reinterpret_cast<uint16_t*>(row)[c] = (uint16_t)v;
  else
    reinterpret_cast<uint32_t*>(row)[c] = v;
}

// The whole CTA writes rows [0, rows) x columns [0, cols) of the matrix at `base` (row stride in elements):
// "may attend" in the first `prefix` columns, "masked" behind.  16-byte stores where the rows allow them.
// No barrier inside: the caller synchronises before it sets single elements on top.
__device__ inline void mask_fill_rows(uint8_t* base, int64_t row_stride, int rows, int64_t cols, int64_t prefix,
                                      const MaskFmt& f) {
  const int epv = 16 / f.esz;
  const bool vec = ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) && ((row_stride * f.esz) % 16 == 0);
  const int64_t nvec = vec ? cols / epv : 0;
  for (int64_t i = threadIdx.x; i < (int64_t)rows * nvec; i += blockDim.x) {
    const int64_t r = i / nvec, v = i - r * nvec;
    const int64_t c0 = v * epv;
    uint4* dst = reinterpret_cast<uint4*>(base + r * row_stride * f.esz) + v;
    if (c0 + epv <= prefix) {
      *dst = make_uint4(f.on, f.on, f.on, f.on);
    } else if (c0 >= prefix) {
      *dst = make_uint4(f.off, f.off, f.off, f.off);
    } else {  // the one vector of a row that holds the end of the prefix
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t word = 0;
        const int per = 4 / f.esz;
        for (int e = 0; e < per; ++e) {
          const int64_t c = c0 + (int64_t)j * per + e;
          const uint32_t pat = (c < prefix ? f.on : f.off) & (f.esz == 4 ? 0xffffffffu : (f.esz == 2 ? 0xffffu : 0xffu));
          word |= pat << (8 * f.esz * e);
        }
        w[j] = word;
      }
      *dst = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  const int64_t tail0 = nvec * epv, tail = cols - tail0;
  for (int64_t i = threadIdx.x; i < (int64_t)rows * tail; i += blockDim.x) {
    const int64_t r = i / tail, c = tail0 + (i - r * tail);
    mask_store(base + r * row_stride * f.esz, c, f, c < prefix);
  }
}

#endif  // __CUDACC__

}  // namespace subspec
