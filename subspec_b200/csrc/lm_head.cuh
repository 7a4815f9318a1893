// Interface between the lm_head GEMM with a statistics epilogue (lm_head_gemm.cu) and the verifier's tail that
// consumes those statistics (verify.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace subspec {

// What one N tile of a row of logits contributes: the fields of the verifier's row statistics.  With
// y = logit * k - c:  s = sum 2^y,  t2 = sum y * 2^y;  vmax / amax = the largest logit of the tile and the
// smallest token index that has it (INT_MAX: the tile had no column inside the vocabulary).
struct LmHeadStat {
  float c, s, t2, vmax;
  int amax;
};

constexpr int kLmTileN = 256;     // vocabulary columns per tile, at most
constexpr int kLmMinTileN = 192;  // ... and at least (the launcher picks a multiple of 16 in between)

struct LmHeadGemmArgs {
  int half;                 // operands and the logits' rounding: 0 bf16, 1 fp16
  const void* hidden;       // [rows, dim]
  int64_t hidden_stride;    // elements between rows
  const void* weight;       // [vocab, dim]
  int64_t weight_stride;
  int rows, vocab, dim;
  int soft;                 // 0: maxima only (greedy targets); 1: softmax sums as well
  float k;                  // log2(e) / temperature
  LmHeadStat* partial;      // [rows, ntiles], room for ntiles = ceil(vocab / kLmMinTileN)
  uint32_t* dev_status;
};

// Launches the GEMM and reports how many column tiles (records per row) it cut the vocabulary into;
// cudaErrorInvalidValue when the operands cannot be described to the copy engine (addresses and strides have
// to be multiples of 16 bytes).
cudaError_t launch_lm_head_stats(const LmHeadGemmArgs& args, cudaStream_t stream, int* ntiles);

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline tensor_map_encode_fn tensor_map_encoder() {
  static tensor_map_encode_fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<tensor_map_encode_fn>(f);
  }();
  return fn;
}

}  // namespace subspec
