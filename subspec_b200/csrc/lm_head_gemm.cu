// lm_head GEMM whose epilogue keeps the verifier's row statistics instead of the logits (sm_100a).
//
// The reference's target forward ends in `logits = lm_head(hidden)` and the verifier then reads those logits
// once per row (generators/classic_sd.py:100-116, verify/exact_tree_verify.py:23-28, lossy_tree_verify.py:84-100):
// a [rows, vocab] 16-bit tensor written and read again, 2 x 1.25 GB per wave of 64 trees of 64 nodes.  Here every
// element of the GEMM's accumulator tile is rounded to the model's dtype (bf16 or fp16: what the reference's
// lm_head returns) and goes into the row's maximum / first arg-max and, for the lossy gates, into sum 2^y and
// sum y 2^y; what leaves the kernel is one 20-byte record per (row, column tile).
//
// One persistent CTA per SM walks (row tile, column tile) pairs, the row tiles of one column tile next to each
// other so that CTAs running at the same time share weight tiles in L2.  A tile is 256 rows x 256 columns: two
// 128-row blocks (the MMA's M) share every weight tile, which halves the shared-memory traffic per flop
// against one block.  Roles: warp 8 issues the tensor copies (TMA, 128-byte swizzle) into a three-stage ring of
// (256 x 64 hidden, 256 x 64 weight) pairs; warp 9 issues tcgen05.mma (both operands in shared memory, K-major,
// accumulators in tensor memory: 2 x 256 columns, all there is); warps 0-7 are the epilogue, thread = row =
// tensor-memory lane: they first move the tile's row out of tensor memory, rounded and packed two to a
// register, hand the accumulators back, and do the arithmetic while the next tile's MMAs run.  All waits are
// bounded.
#include <limits.h>

#include "lm_head.cuh"
#include "tcgen05.cuh"

namespace subspec {
namespace {

constexpr int kBlockRows = 128;                    // MMA M
constexpr int kTileRows = 2 * kBlockRows;          // rows per tile
constexpr int kTileK = 64;                         // 128 bytes of bf16: one swizzle span
constexpr int kStages = 3;
constexpr int kABytes = kTileRows * kTileK * 2;    // 32 KB
constexpr int kBBytes = kLmTileN * kTileK * 2;     // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmem = kStages * kStageBytes + 1024;  // + room to align the ring to 1024 bytes
constexpr int kEpiWarps = 8, kLoadWarp = 8, kMmaWarp = 9, kThreads = 320;
constexpr uint32_t kCols = 512;                    // tensor-memory columns: two accumulators of 256
constexpr float kHeadroom = 64.f;                  // log2 units a chunk maximum may exceed the row's shift
constexpr uint32_t kPollLimit = 1u << 24;

__device__ __forceinline__ bool lm_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kPollLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Shared-memory matrix descriptor of a K-major operand in the 128-byte swizzle: 8-row atoms of 1024 bytes.
// [0,14) address >> 4, [16,30) leading byte offset >> 4 (unused here), [32,46) stride byte offset >> 4,
// [46,48) version 1, [61,64) layout 2.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16: D fp32 (bit 4), A and B bf16 (1 at [7,10) and [10,13)) or fp16 (0), both K-major,
// N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t make_idesc(int n, bool half) {
  const uint32_t fmt = half ? 0u : 1u;  // fp16 : bf16
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBlockRows >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Tensor copy (TMA), two coordinates (element of the row, row), global -> shared, completion counted in bytes
// on `bar`.  c0 is a multiple of 64 two-byte elements here, so the copy starts on a 16-byte boundary.
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

struct RingPos {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() {
    if (++s == kStages) {
      s = 0;
      ph ^= 1u;
    }
  }
};

// 16 fp32 accumulators -> 8 pairs of 16-bit floats: the logits as the reference sees them, rounded to the
// model's dtype (HALF: fp16, else bf16).
template <bool HALF>
__device__ __forceinline__ void round_pairs(const uint32_t (&r)[16], uint32_t* p) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (HALF)
      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p[j]) : "f"(__uint_as_float(r[2 * j + 1])), "f"(__uint_as_float(r[2 * j])));
    else
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p[j]) : "f"(__uint_as_float(r[2 * j + 1])), "f"(__uint_as_float(r[2 * j])));
  }
}

// Folds 32 consecutive columns of a row, held as 16 pairs of 16-bit floats, into the row's statistics.  `valid`
// columns of the chunk lie inside the tile and the vocabulary (>= 32 everywhere but at their ends).
template <bool SOFT, bool HALF>
__device__ __forceinline__ void fold_chunk(const uint32_t* p, int col0, int valid, float k, float& c, uint64_t& s2,
                                           uint64_t& t2, float& vmax, int& amax) {
  float x[32];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (HALF) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&p[j]));
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    } else {
      x[2 * j] = __uint_as_float(p[j] << 16);
      x[2 * j + 1] = __uint_as_float(p[j] & 0xffff0000u);
    }
  }
  if (valid < 32) {
    // columns past the vocabulary (the copy engine filled their weights with zeros): far below any logit, and
    // finite, so that their 2^y is an exact zero and y * 2^y is not a NaN
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = j < valid ? x[j] : -1e30f;
  }
  float m = x[0];
#pragma unroll
  for (int j = 1; j < 32; ++j) m = fmaxf(m, x[j]);
  if (m > vmax) {  // strictly: an equal maximum further right never replaces the first one
    int idx = 31;
#pragma unroll
    for (int j = 30; j >= 0; --j) idx = x[j] == m ? j : idx;
    vmax = m;
    amax = col0 + idx;
  }
  if (SOFT) {
    const float mk = m * k;
    if (!(mk <= c + kHeadroom)) {  // also the first chunk (c = -inf)
      if (c != -INFINITY) {
        const float d = c - mk, f = ex2f(d);
        float s_lo, s_hi, t_lo, t_hi;
        f2_unpack(s2, s_lo, s_hi);
        f2_unpack(t2, t_lo, t_hi);
        t2 = f2_pack(f * fmaf(d, s_lo, t_lo), f * fmaf(d, s_hi, t_hi));
        s2 = f2_pack(s_lo * f, s_hi * f);
      }
      c = mk;
    }
    const uint64_t k2 = f2_pack(k, k), nc2 = f2_pack(-c, -c);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint64_t y2 = f2_fma(f2_pack(x[2 * j], x[2 * j + 1]), k2, nc2);
      float y_lo, y_hi;
      f2_unpack(y2, y_lo, y_hi);
      const uint64_t e2 = f2_pack(ex2f(y_lo), ex2f(y_hi));
      s2 = f2_add(s2, e2);
      t2 = f2_fma(y2, e2, t2);
    }
  }
}

// FLEX: the column tile's width is a run-time value (a multiple of 16 up to 256) and a row block without rows
// is skipped -- the build for launches of one row tile (up to four requests' trees of 64 nodes); without it the
// width is 256 and both blocks always run.
template <bool SOFT, bool FLEX, bool HALF>
__global__ void __launch_bounds__(kThreads, 1)
    lm_head_stats_kernel(const LmHeadGemmArgs ga, const int ntiles, const int tile_n_arg,
                         const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kStages], empty[kStages], acc_ready, acc_free;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  volatile int* abort_flag = &s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_ready, 1);
    mbar_init(&acc_free, kEpiWarps);
    s_abort = 0;
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&s_tmem, kCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  const int tile_n = FLEX ? tile_n_arg : kLmTileN;
  const int mtiles = (ga.rows + kTileRows - 1) / kTileRows;
  const int total = mtiles * ntiles;
  const int nkb = (ga.dim + kTileK - 1) / kTileK;

  if (warp == kLoadWarp) {
    if (lane == 0) {
      RingPos pos;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int nt = tile / mtiles, mt = tile - nt * mtiles;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!lm_wait(&empty[pos.s], pos.ph ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          unsigned char* stage = ring + (size_t)pos.s * kStageBytes;
          mbar_expect_tx(&full[pos.s], (uint32_t)(kABytes + tile_n * kTileK * 2));
          tma_load_2d(stage, &map_a, kb * kTileK, mt * kTileRows, &full[pos.s]);
          tma_load_2d(stage + kABytes, &map_b, kb * kTileK, nt * tile_n, &full[pos.s]);
          pos.next();
          ++issued;
        }
      }
      if (!ok) {
        // copies still in flight land in this CTA's shared memory: see the last ones in before the CTA ends
        const int back = issued < kStages ? issued : kStages;
        for (int i = 0; i < back; ++i) {
          pos.s = pos.s == 0 ? kStages - 1 : pos.s - 1;
          if (pos.s == kStages - 1) pos.ph ^= 1u;
          mbar_wait_bounded(&full[pos.s], pos.ph);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      RingPos pos;
      bool ok = true;
      uint32_t it = 0;
      const uint32_t idesc = make_idesc(tile_n, HALF);
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++it) {
        const int mt = tile % mtiles;
        const int nblk = FLEX && ga.rows - mt * kTileRows <= kBlockRows ? 1 : 2;  // a second row block with rows in it?
        // the epilogue of the tile before has to be out of the accumulators
        if (!lm_wait(&acc_free, (it & 1u) ^ 1u, abort_flag)) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb) {
          if (!lm_wait(&full[pos.s], pos.ph, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + (size_t)pos.s * kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk) {
            const uint64_t bdesc = kmajor_desc(b_addr + kk * 32);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
              if (blk < nblk)
                mma_bf16_ss(tmem + (uint32_t)(blk * kLmTileN), kmajor_desc(a_addr + blk * (kABytes / 2) + kk * 32),
                            bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[pos.s]);  // the stage is free once these MMAs have read it
          pos.next();
        }
        if (ok) tc_commit(&acc_ready);
      }
    }
  } else {
    const int blk = warp >> 2, quarter = warp & 3;  // a warp reaches the 32 tensor-memory lanes of its quarter
    const uint32_t tbase = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(blk * kLmTileN);
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
      const int nt = tile / mtiles, mt = tile - nt * mtiles;
      if (!__all_sync(0xffffffffu, lm_wait(&acc_ready, it & 1u, abort_flag))) break;
      tc_fence_after();
      const int row = mt * kTileRows + blk * kBlockRows + quarter * 32 + lane;
      const int col0 = nt * tile_n;
      const int col_end = min(col0 + tile_n, ga.vocab);
      if (FLEX && mt * kTileRows + blk * kBlockRows >= ga.rows) {  // the block holds no row: nothing was computed for it
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_free);
        continue;
      }
      float c = -INFINITY, vmax = -INFINITY;
      int amax = INT_MAX;
      uint64_t s2 = 0, t2 = 0;
      // The whole row of the tile comes out of tensor memory first, as pairs of 16-bit floats (128 registers),
      // and the accumulators go back to the MMA warp: the arithmetic below runs under the next tile's MMAs.
      uint32_t p[kLmTileN / 2];
      {
        uint32_t ra[16], rb[16];
        tmem_ld16_async(tbase, ra);
#pragma unroll
        for (int sc = 0; sc < kLmTileN / 16; sc += 2) {
          // (columns past the tile's width hold an earlier tile's values: loaded, never looked at)
          tmem_wait_ld_dep(ra);
          tmem_ld16_async(tbase + (uint32_t)((sc + 1) * 16), rb);
          round_pairs<HALF>(ra, p + sc * 8);
          tmem_wait_ld_dep(rb);
          if (sc + 2 < kLmTileN / 16) tmem_ld16_async(tbase + (uint32_t)((sc + 2) * 16), ra);
          round_pairs<HALF>(rb, p + (sc + 1) * 8);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free);
#pragma unroll
      for (int ch = 0; ch < kLmTileN / 32; ++ch)
        if (col0 + ch * 32 < col_end)
          fold_chunk<SOFT, HALF>(p + ch * 16, col0 + ch * 32, col_end - (col0 + ch * 32), ga.k, c, s2, t2, vmax, amax);
      if (row < ga.rows) {
        float s_lo, s_hi, t_lo, t_hi;
        f2_unpack(s2, s_lo, s_hi);
        f2_unpack(t2, t_lo, t_hi);
        LmHeadStat st;
        st.c = c;
        st.s = s_lo + s_hi;
        st.t2 = t_lo + t_hi;
        st.vmax = vmax;
        st.amax = amax;
        ga.partial[(size_t)row * ntiles + nt] = st;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) {
    __syncwarp();  // lane 0 comes out of the issue loop, the others straight from the top: one warp again
    tmem_dealloc(tmem, kCols);
  }
  if (threadIdx.x == 0 && s_abort) flag(ga.dev_status, SUBSPEC_DEV_TIMEOUT);
}

bool encode_rows_map(CUtensorMap* m, const void* base, int64_t stride_elems, int rows, int dim, int box_rows, bool half) {
  const cuuint64_t dims[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)stride_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return tensor_map_encoder()(m, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_lm_head_stats(const LmHeadGemmArgs& ga, cudaStream_t stream, int* ntiles_out) {
  if (!tensor_map_encoder()) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(ga.hidden) & 15u) || (reinterpret_cast<uintptr_t>(ga.weight) & 15u) ||
      (ga.hidden_stride % 8) || (ga.weight_stride % 8) || ga.hidden_stride < ga.dim || ga.weight_stride < ga.dim)
    return cudaErrorInvalidValue;
  // Width of a column tile.  256 keeps the MMAs at their best.  With no more than one row tile (up to four
  // requests' trees) the call is a stream of the weights through HBM, the MMAs idle, and the number of rounds of
  // tiles the CTAs go through decides (594 tiles of 256 on 148 SMs are five rounds, 732 of 208 five shorter
  // ones): there, take the width with the smallest rounds x (width + fixed cost).  (With more rows narrower
  // tiles lost: 512 rows 447 us at 240 against 393 us at 256, though both need nine rounds.)
  const int64_t mtiles = (ga.rows + kTileRows - 1) / kTileRows;
  int tile_n = kLmTileN;
  double best = 1e30;
  for (int wdt = kLmTileN; wdt >= (ga.rows <= kTileRows ? kLmMinTileN : kLmTileN); wdt -= 16) {
    const int64_t tiles = mtiles * ((ga.vocab + wdt - 1) / wdt);
    const int64_t rounds = (tiles + kNumSMs - 1) / kNumSMs;
    const double cost = (double)rounds * (wdt + 12);
    if (cost < best * 0.97) {  // a narrower tile has to gain 3 % to be taken
      best = cost;
      tile_n = wdt;
    }
  }
  CUtensorMap map_a, map_b;
  const bool half = ga.half != 0;
  if (!encode_rows_map(&map_a, ga.hidden, ga.hidden_stride, ga.rows, ga.dim, kTileRows, half) ||
      !encode_rows_map(&map_b, ga.weight, ga.weight_stride, ga.vocab, ga.dim, tile_n, half))
    return cudaErrorInvalidValue;
  const int ntiles = (ga.vocab + tile_n - 1) / tile_n;
  const int64_t total = mtiles * ntiles;
  if (total > INT_MAX) return cudaErrorInvalidValue;  // the kernel counts tiles in 32 bits
  const int grid = (int)(total < kNumSMs ? total : kNumSMs);
  const bool flex = ga.rows <= kTileRows;
  using Kernel = void (*)(const LmHeadGemmArgs, const int, const int, const CUtensorMap, const CUtensorMap);
  static const Kernel kernels[8] = {
      lm_head_stats_kernel<false, false, false>, lm_head_stats_kernel<false, false, true>,
      lm_head_stats_kernel<false, true, false>,  lm_head_stats_kernel<false, true, true>,
      lm_head_stats_kernel<true, false, false>,  lm_head_stats_kernel<true, false, true>,
      lm_head_stats_kernel<true, true, false>,   lm_head_stats_kernel<true, true, true>};
  const Kernel kernel = kernels[(ga.soft ? 4 : 0) + (flex ? 2 : 0) + (half ? 1 : 0)];
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return e;
  kernel<<<grid, kThreads, kSmem, stream>>>(ga, ntiles, tile_n, map_a, map_b);
  *ntiles_out = ntiles;
  return cudaGetLastError();
}

}  // namespace subspec
