// W4A16 group-wise dequant GEMM for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
//   y[m, n] = sum_k x[m, k] * (q[n, k] - zero[n, k / 64]) * scale[n, k / 64]
//
// This is the arithmetic behind the reference's HQQ 4-bit draft linears
// (specdecodes/helpers/quantizers/hqq/__init__.py:17-119: HQQLinear(nbits=4, group_size=64, axis=1)
// patched to a GemLite A16W4 kernel; both third-party).  M is the number of draft tree tokens
// (16..256), so the weights are the large operand and the problem is swapped: the 128 rows of a
// weight tile are the MMA's M dimension, the tokens its N dimension, D[n, m] lives in TMEM.
//
// Data flow per CTA (one 128-row weight tile, a contiguous range of 64-wide K blocks):
//   warp 0, one thread : cp.async.bulk (TMA) of the packed block (4 KB of nibbles + 512 B of
//                        scale / -zero*scale) and of the pre-arranged fp16 activation block into a
//                        kStages-deep shared-memory ring, completion on mbarriers;
//   warps 4-7          : dequantise the nibbles to fp16 (lop3 magic-number trick, packed half2 FMA)
//                        straight into the 128-byte-swizzled K-major tile the tensor core reads;
//   warp 1, one thread : tcgen05.mma (kind::f16, 128 x Mpad x 16, fp32 accumulate in TMEM), four per
//                        K block, tcgen05.commit frees the stage;
//   warps 4-7          : epilogue, tcgen05.ld of the accumulator, bf16 store (or fp32 split-K partial
//                        + ticket: the last CTA of a tile adds the partials up).
// Every wait is bounded; a wait that runs out raises SUBSPEC_DEV_TIMEOUT and the CTA winds down
// (TMEM is released on every path).  No clusters, no multicast.
#include <limits.h>

#include "common.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

constexpr int kTileN = 128;      // weight rows per CTA = MMA M
constexpr int kBlockK = 64;      // K per stage = one quantisation group = one 128-byte swizzle row of fp16
constexpr int kRawBytes = kTileN * 32 + kTileN * 4;  // nibbles + (scale, -zero*scale) half2 per row
constexpr int kATileBytes = kTileN * 128;
constexpr int kDeqWarps = 16;        // warps 4..19 dequantise (four threads per weight row) and run the epilogue
constexpr int kThreads = 128 + 32 * kDeqWarps;
constexpr int kMaxM = 256;
constexpr int kMaxRing = 32;

struct GemmArgs {
  const unsigned char* wpk;  // packed weights: [N/128][K/64] blocks of kRawBytes
  const __half* xp;          // prepared activations: [K/64][Mpad][64] fp16, rows swizzled
  __nv_bfloat16* y;          // [M, N]
  float* partial;            // [tiles][splits][Mpad][128]
  int* ticket;               // [tiles]
  uint32_t* dev_status;
  int M, Mpad, N, K, kblocks, splits, ring_a, ring_b, ring_raw;
  int64_t y_stride;
};

#ifdef SUBSPEC_GEMM_PROFILE
__device__ long long g_prof[16];
#define PROF_T0 const long long prof_t0 = clock64()
#define PROF_ADD(slot) \
  if (blockIdx.x == 0 && blockIdx.y == 0) atomicAdd((unsigned long long*)&g_prof[slot], (unsigned long long)(clock64() - prof_t0))
#else
#define PROF_T0
#define PROF_ADD(slot)
#endif

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns; lane i of the warp reads TMEM lane (lane base + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row atoms
// 1024 bytes apart.  Bits: [0,14) address >> 4; [16,30) leading byte offset >> 4 (unused for
// swizzled K-major, 1); [32,46) stride byte offset >> 4 (1024 >> 4); [46,48) version = 1;
// [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16: D = fp32 (bit 4), A = B = fp16 (format 0), both K-major,
// N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int mma_m, int mma_n) {
  return (1u << 4) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}

// ---- kernels ----------------------------------------------------------------------------------
// HQQ-style tensors -> kernel blocks.  qweight [N, K/8] int32, nibble i of word j = q[n, 8 j + i];
// scale / zero [N, K/64] fp16.  In a block, row r owns 32 bytes: word j carries k = 8j..8j+7 with
// nibble s <-> k = 8j + 2s and nibble s + 4 <-> k = 8j + 2s + 1 (s = 0..3), so that
// (word >> 4s) & 0x000F000F yields two consecutive k as one half2.
__global__ void w4a16_pack_kernel(const uint32_t* __restrict__ qweight, const __half* __restrict__ scale,
                                  const __half* __restrict__ zero, unsigned char* __restrict__ out, int N, int K) {
  const int kblocks = K / kBlockK;
  const int64_t total = (int64_t)N * kblocks;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(idx / kblocks), kb = (int)(idx - (int64_t)n * kblocks);
    const int tile = n / kTileN, r = n - tile * kTileN;
    unsigned char* blk = out + ((size_t)tile * kblocks + kb) * kRawBytes;
    uint32_t* dstw = reinterpret_cast<uint32_t*>(blk + r * 32);
    for (int j = 0; j < 8; ++j) {
      const uint32_t w = qweight[(size_t)n * (K / 8) + kb * 8 + j];
      uint32_t o = 0;
      for (int s = 0; s < 4; ++s) {
        o |= ((w >> (4 * (2 * s))) & 0xFu) << (4 * s);
        o |= ((w >> (4 * (2 * s + 1))) & 0xFu) << (4 * (s + 4));
      }
      dstw[j] = o;
    }
    const float s = __half2float(scale[(size_t)n * kblocks + kb]);
    const float z = __half2float(zero[(size_t)n * kblocks + kb]);
    reinterpret_cast<__half2*>(blk + kTileN * 32)[r] = __halves2half2(__float2half_rn(s), __float2half_rn(-z * s));
  }
}

// x bf16 [M, K] -> fp16 blocks [K/64][Mpad][64], 16-byte chunk c of row r stored at chunk c ^ (r & 7)
// (the 128-byte swizzle the tensor core expects); rows >= M are zero.
__global__ void w4a16_prep_x_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_stride, __half* __restrict__ xp,
                                    int M, int Mpad, int K) {
  const int kblocks = K / kBlockK;
  const int64_t total = (int64_t)kblocks * Mpad * 8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx & 7);
    const int r = (int)((idx >> 3) % Mpad);
    const int kb = (int)(idx / ((int64_t)Mpad * 8));
    uint4 o = make_uint4(0, 0, 0, 0);
    if (r < M) {
      const __nv_bfloat16* src = x + (size_t)r * x_stride + (size_t)kb * kBlockK + c * 8;
      __half h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float f = fminf(fmaxf(__bfloat162float(src[i]), -65504.f), 65504.f);
        h[i] = __float2half_rn(f);
      }
      o = *reinterpret_cast<uint4*>(h);
    }
    uint4* dst = reinterpret_cast<uint4*>(xp + ((size_t)kb * Mpad + r) * kBlockK);
    dst[c ^ (r & 7)] = o;
  }
}

__global__ void __launch_bounds__(kThreads, 1) w4a16_gemm_kernel(const GemmArgs g) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // the swizzle atoms must sit on 1024-byte boundaries of the shared-memory address space
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t raw_full[kMaxRing], raw_empty[kMaxRing], b_full[kMaxRing], b_empty[kMaxRing],
      a_full[kMaxRing], a_empty[kMaxRing], acc_full;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;

  // Three rings with their own depths: packed weight blocks (deep: this is the HBM stream), activation
  // blocks (read by the tensor core) and dequantised fp16 tiles (written here, read by the tensor core).
  const int Ra = g.ring_a, Rb = g.ring_b, Rr = g.ring_raw;
  const int b_bytes = g.Mpad * 128;
  unsigned char* a_ring = smem;                                  // Ra x 16 KB, 1024-aligned
  unsigned char* b_ring = a_ring + (size_t)Ra * kATileBytes;     // Rb x Mpad*128 (a multiple of 2 KB)
  unsigned char* raw_ring = b_ring + (size_t)Rb * b_bytes;       // Rr x 4608 B
  const int tile = blockIdx.x, split = blockIdx.y;
  const int kb_per = (g.kblocks + g.splits - 1) / g.splits;
  const int kb0 = min(split * kb_per, g.kblocks), kb1 = min(kb0 + kb_per, g.kblocks);
  const int nkb = kb1 - kb0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t ncols = 32;
  while ((int)ncols < g.Mpad) ncols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxRing; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], kDeqWarps);
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
      mbar_init(&a_full[s], kDeqWarps);
      mbar_init(&a_empty[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init_fence();
    s_abort = 0;
    s_last = 0;
  }
  if (warp == 2) {
    tmem_alloc(&s_tmem, ncols);
    tmem_relinquish();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = s_tmem;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---- TMA producer, packed weights ----
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Rr;
        {
          PROF_T0;
          if (i >= Rr && !wait_or_abort(&raw_empty[s], (uint32_t)((i / Rr) - 1) & 1u, abort_flag)) break;
          PROF_ADD(0);
        }
        mbar_expect_tx(&raw_full[s], (uint32_t)kRawBytes);
        bulk_g2s(raw_ring + (size_t)s * kRawBytes, g.wpk + ((size_t)tile * g.kblocks + kb0 + i) * kRawBytes,
                 kRawBytes, &raw_full[s]);
      }
    }
    __syncwarp();  // the role lane rejoins its warp before the CTA-wide barrier below
  } else if (warp == 3) {
    // ---- TMA producer, activations ----
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Rb;
        if (i >= Rb && !wait_or_abort(&b_empty[s], (uint32_t)((i / Rb) - 1) & 1u, abort_flag)) break;
        mbar_expect_tx(&b_full[s], (uint32_t)b_bytes);
        bulk_g2s(b_ring + (size_t)s * b_bytes, g.xp + (size_t)(kb0 + i) * g.Mpad * kBlockK, (uint32_t)b_bytes,
                 &b_full[s]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kTileN, g.Mpad);
      for (int i = 0; i < nkb; ++i) {
        const int sa = i % Ra, sb = i % Rb;
        {
          PROF_T0;
          if (!wait_or_abort(&b_full[sb], (uint32_t)(i / Rb) & 1u, abort_flag)) break;
          PROF_ADD(1);
        }
        {
          PROF_T0;
          if (!wait_or_abort(&a_full[sa], (uint32_t)(i / Ra) & 1u, abort_flag)) break;
          PROF_ADD(2);
        }
        tc_fence_after();
        const uint64_t adesc = make_desc(smem_u32(a_ring + (size_t)sa * kATileBytes));
        const uint64_t bdesc = make_desc(smem_u32(b_ring + (size_t)sb * b_bytes));
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k)  // +32 bytes (2 x 16-byte units) per K = 16 step inside the swizzle row
          tc_mma_f16(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (i | k) ? 1u : 0u);
        tc_commit(&a_empty[sa]);
        tc_commit(&b_empty[sb]);
      }
      tc_commit(&acc_full);
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---- dequantise: threads r, r + 128, r + 256, r + 384 own the four quarters (16 weights each) of row r ----
    const int dt = threadIdx.x - 128;
    const int r = dt & (kTileN - 1), quarter = dt >> 7;
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    for (int i = 0; i < nkb; ++i) {
      const int sr = i % Rr, sa = i % Ra;
      {
        PROF_T0;
        if (!wait_or_abort(&raw_full[sr], (uint32_t)(i / Rr) & 1u, abort_flag)) break;
        if (threadIdx.x == 128) PROF_ADD(3);
      }
      {
        PROF_T0;
        if (i >= Ra && !wait_or_abort(&a_empty[sa], (uint32_t)((i / Ra) - 1) & 1u, abort_flag)) break;
        if (threadIdx.x == 128) PROF_ADD(4);
      }
      PROF_T0;
      const unsigned char* raw = raw_ring + (size_t)sr * kRawBytes;
      const uint2 q0 = reinterpret_cast<const uint2*>(raw + r * 32)[quarter];
      const __half2 sz = reinterpret_cast<const __half2*>(raw + kTileN * 32)[r];
      const __half2 s2 = __half2half2(__low2half(sz));
      const __half2 b2 = __half2half2(__high2half(sz));
      const uint32_t words[2] = {q0.x, q0.y};
      uint4* arow = reinterpret_cast<uint4*>(a_ring + (size_t)sa * kATileBytes + (r >> 3) * 1024 + (r & 7) * 128);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t o[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          // 0x6400 = 1024.0 in fp16: OR-ing a nibble into the mantissa gives 1024 + q exactly
          uint32_t v = ((words[j] >> (4 * t)) & 0x000F000Fu) | 0x64006400u;
          __half2 h = *reinterpret_cast<__half2*>(&v);
          h = __hfma2(__hsub2(h, k1024), s2, b2);  // (q * scale) + (-zero * scale)
          o[t] = *reinterpret_cast<uint32_t*>(&h);
        }
        arow[(2 * quarter + j) ^ (r & 7)] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) {     // one arrival per warp: 256 threads hitting one barrier word would serialise
        mbar_arrive(&a_full[sa]);
        mbar_arrive(&raw_empty[sr]);
      }
      if (threadIdx.x == 128) PROF_ADD(5);
    }
    // ---- epilogue ----
    PROF_T0;
    if (wait_or_abort(&acc_full, 0, abort_flag) && !*abort_flag) {
      if (threadIdx.x == 128) PROF_ADD(6);
      tc_fence_after();
      const int ew = warp & 3;  // TMEM lanes 32 ew .. 32 ew + 31 (a warp reaches the quarter given by its id mod 4)
      const int n = tile * kTileN + ew * 32 + lane;
      // each group of four warps takes every (kDeqWarps / 4)-th 16-column group
      for (int c0 = 16 * ((warp - 4) >> 2); c0 < g.Mpad; c0 += 16 * (kDeqWarps / 4)) {
        float v[16];
        tmem_ld16(tmem_d + ((uint32_t)(ew * 32) << 16) + (uint32_t)c0, v);
        if (g.splits == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < g.M) g.y[(size_t)(c0 + j) * g.y_stride + n] = __float2bfloat16_rn(v[j]);
        } else {
          float* part = g.partial + (((size_t)tile * g.splits + split) * g.Mpad + c0) * kTileN + ew * 32 + lane;
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(size_t)j * kTileN] = v[j];
        }
      }
      tc_fence_before();
    }
  }
  __syncthreads();
  if (s_abort && threadIdx.x == 0) flag(g.dev_status, SUBSPEC_DEV_TIMEOUT);

  // ---- split-K: the last CTA of the tile adds the partials ----
  if (g.splits > 1 && !s_abort) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(g.ticket + tile, 1) == g.splits - 1);
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int e = threadIdx.x; e < g.M * kTileN; e += kThreads) {
        const int m = e / kTileN, c = e - m * kTileN;
        float acc = 0.f;
        for (int sp = 0; sp < g.splits; ++sp)
          acc += __ldcg(g.partial + (((size_t)tile * g.splits + sp) * g.Mpad + m) * kTileN + c);
        g.y[(size_t)m * g.y_stride + tile * kTileN + c] = __float2bfloat16_rn(acc);
      }
      if (threadIdx.x == 0) g.ticket[tile] = 0;  // ready for the next call
    }
  }
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_d, ncols);
  }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct Plan {
  int Mpad, kblocks, tiles, splits, ring_a, ring_b, ring_raw;
  size_t xp_bytes, partial_bytes, ticket_bytes, smem_bytes;
};

bool make_plan(int M, int N, int K, Plan* p) {
  if (M < 1 || M > kMaxM || N < kTileN || N % kTileN || K < kBlockK || K % kBlockK) return false;
  p->Mpad = (M + 15) / 16 * 16;
  p->kblocks = K / kBlockK;
  p->tiles = N / kTileN;
  int splits = kNumSMs / p->tiles;
  if (splits < 1) splits = 1;
  if (splits > p->kblocks) splits = p->kblocks;
  if (splits > 64) splits = 64;
  // every split gets at least one K block
  const int per = (p->kblocks + splits - 1) / splits;
  splits = (p->kblocks + per - 1) / per;
  p->splits = splits;
  // shared-memory budget: dequantised tiles and activation blocks get 3-4 stages, the rest goes to packed blocks
  const int budget = 212 * 1024;
  const int b_bytes = p->Mpad * 128;
  p->ring_a = p->Mpad > 128 ? 4 : (p->Mpad > 32 ? 6 : 8);
  p->ring_b = p->Mpad > 128 ? 3 : (p->Mpad > 32 ? 8 : 12);
  // shrink the two tile rings until at least eight packed blocks fit beside them
  while (budget - p->ring_a * kATileBytes - p->ring_b * b_bytes < 8 * kRawBytes) {
    if (p->ring_b > 3)
      --p->ring_b;
    else if (p->ring_a > 2)
      --p->ring_a;
    else if (p->ring_b > 2)
      --p->ring_b;
    else
      return false;
  }
  int left = budget - p->ring_a * kATileBytes - p->ring_b * b_bytes;
  p->ring_raw = left / kRawBytes;
  if (p->ring_raw > kMaxRing) p->ring_raw = kMaxRing;
  p->smem_bytes = (size_t)p->ring_a * kATileBytes + (size_t)p->ring_b * b_bytes + (size_t)p->ring_raw * kRawBytes + 1024;
  p->xp_bytes = align_up((size_t)p->kblocks * p->Mpad * kBlockK * sizeof(__half), 256);
  p->partial_bytes = splits > 1 ? align_up((size_t)p->tiles * splits * p->Mpad * kTileN * sizeof(float), 256) : 0;
  p->ticket_bytes = align_up(sizeof(int) * (size_t)p->tiles, 256);
  return true;
}

}  // namespace
}  // namespace subspec

using namespace subspec;

#ifdef SUBSPEC_GEMM_PROFILE
extern "C" __attribute__((visibility("default"))) int subspec_debug_prof(long long* out, int reset) {
  if (reset) {
    long long z[16] = {};
    return (int)cudaMemcpyToSymbol(g_prof, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * 16);
}
#endif

extern "C" int subspec_w4a16_packed_bytes(int32_t n, int32_t k, size_t* bytes) {
  if (!bytes || n < kTileN || n % kTileN || k < kBlockK || k % kBlockK) return SUBSPEC_EUNSUPPORTED;
  *bytes = (size_t)(n / kTileN) * (k / kBlockK) * kRawBytes;
  return SUBSPEC_OK;
}

extern "C" int subspec_w4a16_pack(const void* qweight, const void* scale, const void* zero, void* packed, int32_t n,
                                  int32_t k, subspec_stream_t stream) {
  if (!qweight || !scale || !zero || !packed) return SUBSPEC_EINVAL;
  size_t bytes;
  const int rc = subspec_w4a16_packed_bytes(n, k, &bytes);
  if (rc) return rc;
  const int64_t total = (int64_t)n * (k / kBlockK);
  const int grid = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
  w4a16_pack_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const __half*>(scale),
      reinterpret_cast<const __half*>(zero), reinterpret_cast<unsigned char*>(packed), n, k);
  return cuda_check(cudaGetLastError());
}

extern "C" int subspec_w4a16_scratch_bytes(int32_t m, int32_t n, int32_t k, size_t* bytes) {
  Plan p;
  if (!bytes) return SUBSPEC_EINVAL;
  if (!make_plan(m, n, k, &p)) return SUBSPEC_EUNSUPPORTED;
  *bytes = p.xp_bytes + p.partial_bytes + p.ticket_bytes;
  return SUBSPEC_OK;
}

extern "C" int subspec_w4a16_gemm(const subspec_w4a16_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_w4a16_args)) return SUBSPEC_EINVAL;
  const subspec_w4a16_args& a = *args;
  if (!a.x || !a.packed || !a.y || !a.scratch) return SUBSPEC_EINVAL;
  Plan p;
  if (!make_plan(a.m, a.n, a.k, &p)) return SUBSPEC_EUNSUPPORTED;
  if (a.x_stride < a.k || a.y_stride < a.n) return SUBSPEC_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a.packed) & 15u) || (reinterpret_cast<uintptr_t>(a.scratch) & 255u))
    return SUBSPEC_ESCRATCH;
  if (a.scratch_bytes < p.xp_bytes + p.partial_bytes + p.ticket_bytes) return SUBSPEC_ESCRATCH;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* sp = reinterpret_cast<char*>(a.scratch);
  GemmArgs g;
  g.wpk = reinterpret_cast<const unsigned char*>(a.packed);
  g.xp = reinterpret_cast<const __half*>(sp);
  g.partial = reinterpret_cast<float*>(sp + p.xp_bytes);
  g.ticket = reinterpret_cast<int*>(sp + p.xp_bytes + p.partial_bytes);
  g.y = reinterpret_cast<__nv_bfloat16*>(a.y);
  g.dev_status = a.dev_status;
  g.M = a.m;
  g.Mpad = p.Mpad;
  g.N = a.n;
  g.K = a.k;
  g.kblocks = p.kblocks;
  g.splits = p.splits;
  g.ring_a = p.ring_a;
  g.ring_b = p.ring_b;
  g.ring_raw = p.ring_raw;
  g.y_stride = a.y_stride;
  int rc = cuda_check(cudaMemsetAsync(g.ticket, 0, p.ticket_bytes, st));
  if (rc) return rc;
  {
    const int64_t total = (int64_t)p.kblocks * p.Mpad * 8;
    const int grid = (int)((total + 255) / 256 > 2368 ? 2368 : (total + 255) / 256);
    w4a16_prep_x_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(a.x), a.x_stride,
                                              reinterpret_cast<__half*>(sp), a.m, p.Mpad, a.k);
    rc = cuda_check(cudaGetLastError());
    if (rc) return rc;
  }
  rc = cuda_check(cudaFuncSetAttribute(w4a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)p.smem_bytes));
  if (rc) return rc;
  w4a16_gemm_kernel<<<dim3(p.tiles, p.splits), kThreads, p.smem_bytes, st>>>(g);
  return cuda_check(cudaGetLastError());
}
