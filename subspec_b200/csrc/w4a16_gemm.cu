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
// Data flow per CTA (one 128-row weight tile, a contiguous range of 64-wide K blocks; 22 warps):
//   warp 0, one thread : cp.async.bulk (TMA) of the packed weights, one copy per chunk of four K blocks
//                        (4 x (4 KB of nibbles + 512 B of scale / -zero*scale)), into a shared-memory
//                        ring, completion on mbarriers;
//   warp 1, one thread : cp.async.bulk of the pre-arranged fp16 activation blocks, one copy per slot of
//                        up to four K blocks, into a ring of its own that looks as far ahead in K as
//                        the packed ring;
//   warps 6-21         : four groups of four warps, group q dequantises K blocks q, q + 4, ... (one
//                        thread per weight row: lop3 magic-number trick, packed half2 FMA) and stores
//                        the fp16 row with tcgen05.st into TENSOR MEMORY, where lane = weight row and
//                        a 32-bit column holds two consecutive k: the dequantised operand never
//                        touches shared memory.  Four K blocks are in flight at once, eight stages;
//   warps 2-5          : MMA issuers (1, 2 or 4 of them, as many as there are accumulators, each taking
//                        every n-th K block): tcgen05.mma kind::f16, 128 x Mpad x 16, A from tensor
//                        memory, B = activation block in shared memory (128-byte swizzle, K-major), fp32
//                        accumulate in TMEM, four per K block; one tcgen05.commit frees the stage.  The
//                        whole warp runs the loop and an elected lane issues, which keeps the
//                        descriptors in uniform registers;
//   warps 6-21         : epilogue, tcgen05.ld of the accumulators, sum, bf16 store (or fp32 split-K
//                        partial: through the shared memory of a thread-block cluster formed by the
//                        splits of a tile, or through global memory + ticket, the last CTA adding up).
// What bounds it at these token counts is neither HBM nor the tensor core's arithmetic but instruction
// issue: a warp gets one tcgen05.mma out every 100-200 cycles whatever its N, hence several issuing
// warps with accumulators of their own, and the role loops keep (stage, parity) counters instead of
// dividing by ring depths.
// Every mbarrier wait is bounded; a wait that runs out raises SUBSPEC_DEV_TIMEOUT and the CTA winds down
// (TMEM is released on every path, and the cluster barriers of the split-K tail are reached on every path).
// Clusters serve the split-K exchange only: every copy is a plain per-CTA bulk copy of this GPU's memory.
#include <limits.h>

#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace subspec {
namespace {

constexpr int kTileN = 128;      // weight rows per CTA = MMA M
constexpr int kBlockK = 64;      // K per stage = one quantisation group = one 128-byte swizzle row of fp16
constexpr int kRawBytes = kTileN * 32 + kTileN * 4;  // nibbles + (scale, -zero*scale) half2 per row
constexpr int kTmemCols = 512;        // the whole tensor memory of the SM (one CTA per SM)
constexpr int kAColBase = 256;        // accumulator in columns [0, 256), dequantised operand stages above
constexpr int kAStageCols = kBlockK / 2;  // one stage = 128 lanes x 32 columns of packed fp16 pairs
constexpr int kMaxStages = (kTmemCols - kAColBase) / kAStageCols;  // 8
constexpr int kDeqWarps = 16;        // the last sixteen warps dequantise and run the epilogue
constexpr int kDeqGroups = 4;        // groups of four warps (128 threads = 128 weight rows) taking K blocks in turn
constexpr int kIssuerWarp0 = 2;      // warps 2..5 issue MMAs (as many as the plan asks for); warp 0, 1: TMA producers
constexpr int kMaxIssuers = 4;
constexpr int kDeqWarp0 = kIssuerWarp0 + kMaxIssuers;
constexpr int kThreads = 32 * (kDeqWarp0 + kDeqWarps);
constexpr int kMaxM = 256;
constexpr int kEarlyChunks = 2;       // packed chunks requested before the prologue's barrier (the ring holds at least two)
constexpr int kMaxRing = 8;           // packed ring, in chunks of kDeqGroups K blocks (one TMA copy each)
constexpr int kChunkBytes = kDeqGroups * kRawBytes;

constexpr int kMaxGroup = SUBSPEC_W4A16_MAX_GROUP;

struct GemmArgs {
  const unsigned char* wpk;  // packed weights: [N/128][K/64] blocks of kRawBytes
  const __half* xp;          // prepared activations: [K/64][Mpad][64] fp16, rows swizzled
  __nv_bfloat16* y;          // [M, N]
  float* partial;            // [tiles][splits][Mpad][128]
  int* ticket;               // [tiles]
  uint32_t* dev_status;
  int M, Mpad, N, K, kblocks, splits, ring_raw, b_slots, b_blocks, b_shift, acc_n, acc_stride, issuers;
  int64_t y_stride;
  int cluster;  // the splits of a tile form a thread-block cluster (1, splits, 1): partial sums meet in shared memory
  // Grouped call: several weight matrices that share the activations are one launch over the concatenation of
  // their tiles.  Segment s owns tiles [seg_tile0[s], seg_tile0[s + 1]); wpk / y / y_stride above are segment 0's.
  int nseg;
  int seg_tile0[kMaxGroup];
  const unsigned char* seg_wpk[kMaxGroup];
  __nv_bfloat16* seg_y[kMaxGroup];
  int64_t seg_ystride[kMaxGroup];
};

// ---- thread-block cluster: barrier and loads from a peer CTA's shared memory ----------------
// Every thread of every CTA of the cluster executes arrive and wait the same number of times, on every
// path (also after an abort): the barrier has no time limit of its own.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t peer_smem(uint32_t own_addr, uint32_t rank) {
  uint32_t d;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(own_addr), "r"(rank));
  return d;
}
__device__ __forceinline__ float4 ld_peer_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
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
// (the 128-byte swizzle the tensor core expects); rows >= M are zero.  Also clears the split-K tickets.
__global__ void w4a16_prep_x_kernel(const __nv_bfloat16* x, int64_t x_stride, __half* __restrict__ xp,
                                    int M, int Mpad, int K, int* __restrict__ ticket, int tiles) {
  // The GEMM that follows in the stream is launched as a programmatic dependent: it may start now and run
  // its prologue and its weight stream beside this kernel; it waits for this grid's completion (and the
  // visibility of everything written here) before the first activation copy.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // This kernel is itself launched as a programmatic dependent of whatever precedes it in the stream, so
  // that its blocks are in place when that ends (after a GEMM of this library, which signals early, this
  // hides a launch latency of 2-3 us per call in back-to-back projections).  Nothing is written before the
  // predecessor has completed: it may be the previous GEMM, still reading this scratch.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (blockIdx.x == 0)  // split-K tickets of that GEMM
    for (int t = threadIdx.x; t < tiles; t += blockDim.x) ticket[t] = 0;
  const int kblocks = K / kBlockK;
  const int64_t total = (int64_t)kblocks * Mpad * 8;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (x_stride & 7) == 0;  // every row chunk 16-byte aligned
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx & 7);
    const int r = (int)((idx >> 3) % Mpad);
    const int kb = (int)(idx / ((int64_t)Mpad * 8));
    uint4 o = make_uint4(0, 0, 0, 0);
    if (r < M) {
      // read past L1: this grid is resident while its predecessor, which may have written x, still runs
      const unsigned short* src =
          reinterpret_cast<const unsigned short*>(x + (size_t)r * x_stride + (size_t)kb * kBlockK + c * 8);
      unsigned short e[8];
      if (vec) {  // one 16-byte load (eight 2-byte loads past L1 cost every projection 2-3 us)
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = (unsigned short)(w[i >> 1] >> (16 * (i & 1)));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = __ldcg(src + i);
      }
      __half h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float f = fminf(fmaxf(__uint_as_float((uint32_t)e[i] << 16), -65504.f), 65504.f);
        h[i] = __float2half_rn(f);
      }
      o = *reinterpret_cast<uint4*>(h);
    }
    uint4* dst = reinterpret_cast<uint4*>(xp + ((size_t)kb * Mpad + r) * kBlockK);
    dst[c ^ (r & 7)] = o;
  }
}

// Ring bookkeeping without divisions: the role loops are single-thread dependent chains, where one
// integer division by a run-time ring depth costs more than the rest of the iteration.
struct RingPos {
  int s, ph;  // stage, parity of the current pass over the ring
  __device__ __forceinline__ void advance(int by, int depth) {
    s += by;
    while (s >= depth) {
      s -= depth;
      ph ^= 1;
    }
  }
};

__global__ void __launch_bounds__(kThreads, 1) w4a16_gemm_kernel(const GemmArgs g) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  // the swizzle atoms must sit on 1024-byte boundaries of the shared-memory address space
  unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  // raw_*: ring of packed weight blocks (the HBM stream, deep).  full / empty: ring of the dequantised
  // 128 x 64 fp16 weight tiles in tensor memory (32 columns each).  b_*: ring of activation slots, one slot =
  // b_blocks consecutive Mpad x 64 fp16 blocks.  The activations have a ring of their own, as deep in K as
  // the packed one: the TMA unit serves an SM's requests in order, so an activation copy issued only when
  // its stage frees up would queue behind every packed block already requested.
  __shared__ __align__(8) uint64_t raw_full[kMaxRing], raw_empty[kMaxRing], full[kMaxStages], empty[kMaxStages],
      b_full[kMaxStages], b_empty[kMaxStages], acc_full;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;

  constexpr int R = kMaxStages;
  const int Rr = g.ring_raw, Rb = g.b_slots, bs = g.b_blocks;
  const int b_bytes = g.Mpad * 128;                             // one K block of activations (a multiple of 2 KB)
  const int slot_bytes = bs * b_bytes;
  unsigned char* b_ring = smem;                                 // Rb slots, 1024-aligned
  unsigned char* raw_ring = b_ring + (size_t)Rb * slot_bytes;   // Rr chunks of four packed blocks
  const int tile = blockIdx.x, split = blockIdx.y;
  // the weight matrix this tile belongs to (one in a plain call), and the tile's number inside it
  int ltile = tile;
  const unsigned char* wpk = g.wpk;
  __nv_bfloat16* yout = g.y;
  int64_t ystride = g.y_stride;
  for (int sgm = 1; sgm < g.nseg; ++sgm)
    if (tile >= g.seg_tile0[sgm]) {
      ltile = tile - g.seg_tile0[sgm];
      wpk = g.seg_wpk[sgm];
      yout = g.seg_y[sgm];
      ystride = g.seg_ystride[sgm];
    }
  const int kb_per = (g.kblocks + g.splits - 1) / g.splits;
  const int kb0 = min(split * kb_per, g.kblocks), kb1 = min(kb0 + kb_per, g.kblocks);
  const int nkb = kb1 - kb0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ncols = kTmemCols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Rr; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], kDeqWarps);
    }
    for (int s = 0; s < R; ++s) {
      mbar_init(&full[s], kDeqWarps / kDeqGroups);
      mbar_init(&empty[s], 1);
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], (uint32_t)g.issuers);
    }
    mbar_init(&acc_full, (uint32_t)g.issuers);
    mbar_init_fence();
    s_abort = 0;
    s_last = 0;
    // The packed-weight stream starts here, before the CTA has its tensor memory and has met at the barrier
    // below: the first chunks' trip from HBM (about a microsecond) runs beside the rest of the prologue.
    // Only kEarlyChunks of them: the copy unit serves an SM's requests in order, and the first activation
    // copy must not queue behind a whole ring of packed data.  This thread is also the producer of that
    // ring and carries on after the barrier.
    const unsigned char* src = wpk + ((size_t)ltile * g.kblocks + kb0) * kRawBytes;
    const int nchunks = (nkb + kDeqGroups - 1) / kDeqGroups;
    for (int c = 0; c < min(nchunks, kEarlyChunks); ++c) {
      const uint32_t bytes = (uint32_t)(min(kDeqGroups, nkb - c * kDeqGroups) * kRawBytes);
      mbar_expect_tx(&raw_full[c], bytes);
      bulk_g2s(raw_ring + (size_t)c * kChunkBytes, src + (size_t)c * kChunkBytes, bytes, &raw_full[c]);
    }
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
  // A kernel launched behind this one as a programmatic dependent may be scheduled from now on (it still
  // has to wait for this grid's completion before it touches anything this grid reads or writes).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---- TMA producer, packed weights: one copy per chunk of four K blocks (a single thread gets a
    // copy out every few hundred cycles at best, which 4.5 KB copies would turn into the bound) ----
    if (lane == 0) {
      // the first kEarlyChunks went out in the prologue
      RingPos p{0, 0};
      p.advance(kEarlyChunks, Rr);
      const int nchunks = (nkb + kDeqGroups - 1) / kDeqGroups;
      const unsigned char* src =
          wpk + ((size_t)ltile * g.kblocks + kb0) * kRawBytes + (size_t)kEarlyChunks * kChunkBytes;
      for (int c = kEarlyChunks; c < nchunks; ++c, src += kChunkBytes) {
        if (c >= Rr && !wait_or_abort(&raw_empty[p.s], (uint32_t)p.ph ^ 1u, abort_flag)) break;
        const uint32_t bytes = (uint32_t)(min(kDeqGroups, nkb - c * kDeqGroups) * kRawBytes);
        mbar_expect_tx(&raw_full[p.s], bytes);
        bulk_g2s(raw_ring + (size_t)p.s * kChunkBytes, src, bytes, &raw_full[p.s]);
        p.advance(1, Rr);
      }
    }
    __syncwarp();  // the role lane rejoins its warp before the CTA-wide barrier below
  } else if (warp == 1) {
    // ---- TMA producer, activations: one copy per slot of bs K blocks ----
    if (lane == 0) {
      RingPos p{0, 0}, pe{0, 0};
      const unsigned char* src = reinterpret_cast<const unsigned char*>(g.xp) + (size_t)kb0 * b_bytes;
      const int nslots = (nkb + bs - 1) / bs;
      // The activations (and the zeroed split-K tickets) come from the preparation kernel launched just
      // before this one: wait for it here, and nowhere else; all later uses hang off these copies.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int j = 0; j < nslots; ++j, src += slot_bytes) {
        if (j >= Rb) {
          if (bs == 1) {
            // one K block per slot: the slot is free when the block's tensor-memory stage is, so the issuing
            // warp's one commit per block serves both (this thread sees every phase of every empty[] in turn)
            if (!wait_or_abort(&empty[pe.s], (uint32_t)pe.ph, abort_flag)) break;
            pe.advance(1, R);
          } else if (!wait_or_abort(&b_empty[p.s], (uint32_t)p.ph ^ 1u, abort_flag)) {
            break;
          }
        }
        const uint32_t bytes = (uint32_t)(min(bs, nkb - j * bs) * b_bytes);
        mbar_expect_tx(&b_full[p.s], bytes);
        bulk_g2s(b_ring + (size_t)p.s * slot_bytes, src, bytes, &b_full[p.s]);
        p.advance(1, Rb);
      }
    }
    __syncwarp();
  }
  if (warp >= kIssuerWarp0 && warp < kIssuerWarp0 + g.issuers) {
    // ---- MMA issuers: with two of them, warp 1 takes the even K blocks, warp 2 the odd ones, each into its own
    // accumulators.  The WHOLE warp runs the loop and one elected lane issues: with warp-uniform control
    // flow the descriptors live in uniform registers, where the tensor-core instructions take them from;
    // under a per-lane branch every operand of every MMA first has to be moved there. ----
    const int me = warp - kIssuerWarp0;
    // The 256 accumulator columns hold acc_n accumulators of acc_stride columns, split evenly between the
    // issuers; an issuer's consecutive K steps rotate over its share, and the epilogue adds everything up
    // (above 128 tokens there is room for one accumulator, hence one issuer).
    const uint32_t idesc = make_idesc(kTileN, g.Mpad);
    const int share = g.acc_n / g.issuers;  // a power of two; at most four are used (one per K step)
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_d, 0);  // the same in every lane, and known to be
    const uint32_t acc0 = tmem_u + (uint32_t)(me * share * g.acc_stride);
    const uint64_t bdesc0 = make_desc(smem_u32(b_ring));
    const uint32_t b_step = (uint32_t)b_bytes >> 4, slot_step = (uint32_t)slot_bytes >> 4;
    RingPos p{0, 0}, pb{0, 0};
    p.advance(me, R);
    int slot_of = -1;  // activation slot (index along K) this warp has waited for
    for (int i = me; i < nkb; i += g.issuers) {
      const int j = i >> g.b_shift, within = i & (bs - 1);  // bs = 1 << b_shift
      bool ok = true;
      if (j != slot_of) {  // first block of this warp in the slot
        if (slot_of >= 0) pb.advance(1, Rb);
        slot_of = j;
        ok = wait_or_abort(&b_full[pb.s], (uint32_t)pb.ph, abort_flag);
      }
      ok = ok && wait_or_abort(&full[p.s], (uint32_t)p.ph, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      const uint32_t tmem_a = tmem_u + (uint32_t)(kAColBase + p.s * kAStageCols);
      const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)pb.s * slot_step + (uint32_t)within * b_step);
      const bool last_in_slot = ((i + g.issuers) >> g.b_shift) != j;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) {  // per K = 16 step: 8 columns of A, +32 bytes (2 x 16-byte units) of B
          tc_mma_f16_ta(acc0 + (uint32_t)((k & (share - 1)) * g.acc_stride), tmem_a + (uint32_t)(8 * k),
                        bdesc + (uint64_t)(2 * k), idesc, (i != me || k >= share) ? 1u : 0u);
        }
        tc_commit(&empty[p.s]);                     // frees the stage for the dequantising group
        if (last_in_slot && bs > 1) tc_commit(&b_empty[pb.s]);  // this warp's last block in the activation slot
      }
      __syncwarp();
      p.advance(g.issuers, R);
    }
    if (elect_one()) {
      if (me < nkb)
        tc_commit(&acc_full);
      else
        mbar_arrive(&acc_full);  // nothing issued by this warp
    }
    __syncwarp();
  } else if (warp >= kDeqWarp0) {
    // ---- dequantise: four groups of four warps; group q takes K blocks q, q + 4, ..., thread = weight row ----
    const int r = (warp & 3) * 32 + lane, grp = (warp - kDeqWarp0) >> 2;
    // a warp reaches the TMEM lanes 32 (warp % 4) .. + 31: the four warps of a group cover rows 0..127 in order
    const uint32_t tmem_row = tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)kAColBase;
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    const __half2 k16th = __half2half2(__ushort_as_half((unsigned short)0x2C00));   // 1 / 16
    const __half2 kneg64 = __half2half2(__ushort_as_half((unsigned short)0xD400));  // -64
    RingPos pr{0, 0}, pa{0, 0};
    pa.advance(grp, R);
    for (int i = grp; i < nkb; i += kDeqGroups) {
      if (!wait_or_abort(&raw_full[pr.s], (uint32_t)pr.ph, abort_flag)) break;
      if (i >= R && !wait_or_abort(&empty[pa.s], (uint32_t)pa.ph ^ 1u, abort_flag)) break;
      const unsigned char* raw = raw_ring + (size_t)pr.s * kChunkBytes + grp * kRawBytes;
      const uint4 q0 = reinterpret_cast<const uint4*>(raw + r * 32)[0];
      const uint4 q1 = reinterpret_cast<const uint4*>(raw + r * 32)[1];
      const __half2 sz = reinterpret_cast<const __half2*>(raw + kTileN * 32)[r];
      const __half2 s2 = __half2half2(__low2half(sz));
      const __half2 b2 = __half2half2(__high2half(sz));
      const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      tc_fence_after();  // the stage's previous reader (the tensor core) is done: ordered before the overwrite
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        uint32_t o[16];  // column c = (k = 2c, 2c + 1) of this thread's row
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          // 0x6400 = 1024.0 in fp16: a nibble OR-ed into mantissa bits 0-3 gives 1024 + q, into bits 4-7
          // 1024 + 16 q; (1024 + q) - 1024 and (1024 + 16 q) / 16 - 64 are both q exactly.  Two of the four
          // nibble pairs of a word are thus reached without a shift.
          const uint32_t w = words[4 * hlf + jj], w8 = w >> 8;
          uint32_t v[4] = {(w & 0x000F000Fu) | 0x64006400u, (w & 0x00F000F0u) | 0x64006400u,
                           (w8 & 0x000F000Fu) | 0x64006400u, (w8 & 0x00F000F0u) | 0x64006400u};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            __half2 h = *reinterpret_cast<__half2*>(&v[t]);
            h = (t & 1) ? __hfma2(h, k16th, kneg64) : __hsub2(h, k1024);
            h = __hfma2(h, s2, b2);  // (q * scale) + (-zero * scale)
            o[4 * jj + t] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        tmem_st16(tmem_row + (uint32_t)(pa.s * kAStageCols + 16 * hlf), o);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {     // one arrival per warp
        mbar_arrive(&full[pa.s]);
        mbar_arrive(&raw_empty[pr.s]);
      }
      pr.advance(1, Rr);
      pa.advance(kDeqGroups, R);
    }
    // ---- epilogue ----
    if (wait_or_abort(&acc_full, 0, abort_flag) && !*abort_flag) {
      tc_fence_after();
      const int ew = warp & 3;  // TMEM lanes 32 ew .. 32 ew + 31 (a warp reaches the quarter given by its id mod 4)
      const int n = ltile * kTileN + ew * 32 + lane;
      // each group of four warps takes every (kDeqWarps / 4)-th group of 16 tokens
      // accumulators that were written: an issuer's share has at most four members in use, and the second
      // issuer has work only from two K blocks on
      const int n_own = g.acc_n / g.issuers;
      const int share = min(n_own, 4);
      for (int c0 = 16 * ((warp - kDeqWarp0) >> 2); c0 < g.Mpad; c0 += 16 * (kDeqWarps / 4)) {
        const int col = c0;  // tokens c0 .. c0 + 15 sit in columns c0 .. c0 + 15 of every accumulator
        float v[16];
        tmem_ld16(tmem_d + ((uint32_t)(ew * 32) << 16) + (uint32_t)col, v);
        for (int is = 0; is < min(g.issuers, nkb); ++is) {
          // the issuer's other accumulators: two loads in flight where its share has that many left
          int a = (is == 0 ? 1 : 0);
          const uint32_t tis = tmem_d + ((uint32_t)(ew * 32) << 16) + (uint32_t)(col + is * n_own * g.acc_stride);
          for (; a + 1 < share; a += 2) {
            uint32_t w0[16], w1[16];
            tmem_ld16_async(tis + (uint32_t)(a * g.acc_stride), w0);
            tmem_ld16_async(tis + (uint32_t)((a + 1) * g.acc_stride), w1);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(w0[j]);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(w1[j]);
          }
          if (a < share) {
            float w[16];
            tmem_ld16(tis + (uint32_t)(a * g.acc_stride), w);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += w[j];
          }
        }
        if (g.splits == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < g.M) yout[(size_t)(c0 + j) * ystride + n] = __float2bfloat16_rn(v[j]);
        } else if (g.cluster) {
          // [Mpad][128] fp32 over the rings, which nothing uses any more: every MMA has completed
          float* part = reinterpret_cast<float*>(smem) + (size_t)c0 * kTileN + ew * 32 + lane;
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(size_t)j * kTileN] = v[j];
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

  // ---- split-K inside a cluster: every CTA adds its share of the outputs from all the splits' shared memory,
  // in split order (the same bits as the path through global memory below) ----
  if (g.cluster) {
    cluster_arrive();  // this CTA's partial sums are written (the CTA barrier above ordered them before this)
    cluster_wait();    // ... and so are everybody else's
    if (!s_abort) {
      const uint32_t own = smem_u32(smem);
      const int total = g.M * (kTileN / 4);
      for (int e = split * kThreads + threadIdx.x; e < total; e += g.splits * kThreads) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          v[u] = u < g.splits ? ld_peer_f4(peer_smem(own + (uint32_t)e * 16u, (uint32_t)u))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc.x += v[u].x;
          acc.y += v[u].y;
          acc.z += v[u].z;
          acc.w += v[u].w;
        }
        const int m = e / (kTileN / 4), c = (e - m * (kTileN / 4)) * 4;
        __nv_bfloat16* dst = yout + (size_t)m * ystride + ltile * kTileN + c;
        dst[0] = __float2bfloat16_rn(acc.x);
        dst[1] = __float2bfloat16_rn(acc.y);
        dst[2] = __float2bfloat16_rn(acc.z);
        dst[3] = __float2bfloat16_rn(acc.w);
      }
    }
    cluster_arrive();  // nobody leaves while a peer may still read its shared memory
    cluster_wait();
  }

  // ---- split-K through global memory: the last CTA of the tile adds the partials ----
  if (g.splits > 1 && !g.cluster && !s_abort) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(g.ticket + tile, 1) == g.splits - 1);
    __syncthreads();
    if (s_last) {
      __threadfence();
      // four columns per thread and step, the partials of up to eight splits in flight at once, added in
      // split order (the same bits on every call)
      const float4* part4 = reinterpret_cast<const float4*>(g.partial + (size_t)tile * g.splits * g.Mpad * kTileN);
      const size_t split_stride = (size_t)g.Mpad * (kTileN / 4);
      for (int e = threadIdx.x; e < g.M * (kTileN / 4); e += kThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp0 = 0; sp0 < g.splits; sp0 += 8) {
          float4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            v[u] = sp0 + u < g.splits ? __ldcg(part4 + (size_t)(sp0 + u) * split_stride + e)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            acc.x += v[u].x;
            acc.y += v[u].y;
            acc.z += v[u].z;
            acc.w += v[u].w;
          }
        }
        const int m = e / (kTileN / 4), c = (e - m * (kTileN / 4)) * 4;
        __nv_bfloat16* dst = yout + (size_t)m * ystride + ltile * kTileN + c;
        dst[0] = __float2bfloat16_rn(acc.x);
        dst[1] = __float2bfloat16_rn(acc.y);
        dst[2] = __float2bfloat16_rn(acc.z);
        dst[3] = __float2bfloat16_rn(acc.w);
      }
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
  int Mpad, kblocks, tiles, splits, ring_raw, b_slots, b_blocks, b_shift, acc_n, acc_stride, issuers;
  size_t xp_bytes, partial_bytes, ticket_bytes, smem_bytes;
};

bool make_plan(int M, int N, int K, Plan* p) {
  if (M < 1 || M > kMaxM || N < kTileN || N % kTileN || K < kBlockK || K % kBlockK) return false;
  p->Mpad = (M + 15) / 16 * 16;  // tokens padded to the MMA's N granule
  // accumulators in TMEM columns [0, 256): as many as fit, a power of two, each at least 32 columns wide
  p->acc_stride = 32;
  while (p->acc_stride < p->Mpad) p->acc_stride <<= 1;
  p->acc_n = 256 / p->acc_stride;
  p->issuers = p->acc_n < kMaxIssuers ? p->acc_n : kMaxIssuers;  // every issuing warp needs an accumulator of its own
  p->kblocks = K / kBlockK;
  p->tiles = N / kTileN;
  int splits = kNumSMs / p->tiles;
  if (splits < 1) splits = 1;
  if (splits > p->kblocks) splits = p->kblocks;
  if (splits > 8) splits = 8;  // the split-K tail reads the partials eight at a time: one round (28 splits: a tail of 3.8 us)
  // the last CTA of a tile reads splits x Mpad x 128 partial sums alone: keep that under 1 MB
  if (splits * p->Mpad > 2048) splits = 2048 / p->Mpad;
  // every split gets at least one K block
  const int per = (p->kblocks + splits - 1) / splits;
  splits = (p->kblocks + per - 1) / per;
  p->splits = splits;
  // Shared memory.  Activation slots: b_blocks K blocks each (a power of two, at least one per issuing
  // warp, at most 32 KB), up to eight slots in at most 128 KB.  Packed ring: the rest, in chunks of
  // kDeqGroups K blocks, not so deep that an activation copy queues behind more packed data than its own
  // look-ahead covers.  Every dequantising group takes one block of every chunk and every fourth stage of
  // the eight in tensor memory, and an issuing warp always frees the same stages, in order: each waiter
  // sees every phase of the barriers it polls, which is what keeps the parity waits sound.
  const int budget = 220 * 1024;
  const int b_bytes = p->Mpad * 128;
  p->b_blocks = 4;
  while (p->b_blocks > p->issuers && p->b_blocks * b_bytes > 32 * 1024) p->b_blocks >>= 1;
  p->b_shift = p->b_blocks == 4 ? 2 : (p->b_blocks == 2 ? 1 : 0);
  const int slot = p->b_blocks * b_bytes;
  p->b_slots = 128 * 1024 / slot;
  if (p->b_slots > kMaxStages) p->b_slots = kMaxStages;
  if (p->b_slots < 2) return false;
  const int ahead = p->b_slots * p->b_blocks;  // activation look-ahead in K blocks
  int raw = (budget - p->b_slots * slot) / kChunkBytes;  // packed ring, in chunks
  if (raw * kDeqGroups > 2 * ahead) raw = 2 * ahead / kDeqGroups;
  if (raw > kMaxRing) raw = kMaxRing;
  if (raw < 2) return false;
  p->ring_raw = raw;
  p->smem_bytes = (size_t)p->b_slots * slot + (size_t)raw * kChunkBytes + 1024;
  if (p->smem_bytes > (size_t)budget + 1024) return false;
  p->xp_bytes = align_up((size_t)p->kblocks * p->Mpad * kBlockK * sizeof(__half), 256);
  p->partial_bytes = splits > 1 ? align_up((size_t)p->tiles * splits * p->Mpad * kTileN * sizeof(float), 256) : 0;
  p->ticket_bytes = align_up(sizeof(int) * (size_t)p->tiles, 256);
  return true;
}

// How many clusters of (1, c, 1) CTAs of the GEMM kernel the device holds at once; 0 when it cannot say.
// Asked once per device and cluster size (the kernel's footprint is one CTA per SM whatever the plan).
int resident_clusters(int dev, int c, int smem_bytes) {
  static int cache[64][9];  // 0 = not asked yet, -1 = asked and failed, n + 1 otherwise
  if (dev < 0 || dev >= 64 || c < 2 || c > 8) return 0;
  if (cache[dev][c] == 0) {
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(1, (unsigned)c);
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = (unsigned)c;
    at[0].val.clusterDim.z = 1;
    q.attrs = at;
    q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, w4a16_gemm_kernel, &q) != cudaSuccess) {
      cudaGetLastError();  // not an error of the call being served
      cache[dev][c] = -1;
    } else {
      cache[dev][c] = n + 1;
    }
  }
  return cache[dev][c] > 0 ? cache[dev][c] - 1 : 0;
}

}  // namespace
}  // namespace subspec

using namespace subspec;

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

namespace {
// One launch over `nseg` weight matrices [n[i], k] that share the activations x [m, k].
int run_gemm(int m, int k, int nseg, const void* const* packed, const int32_t* n, void* const* y,
             const int64_t* y_stride, const void* x, int64_t x_stride, void* scratch, size_t scratch_bytes,
             uint32_t* dev_status, subspec_stream_t stream) {
  if (!x || !scratch || nseg < 1 || nseg > kMaxGroup) return SUBSPEC_EINVAL;
  int64_t n_total = 0;
  for (int i = 0; i < nseg; ++i) {
    if (!packed[i] || !y[i]) return SUBSPEC_EINVAL;
    if (n[i] < kTileN || n[i] % kTileN) return SUBSPEC_EUNSUPPORTED;
    if (y_stride[i] < n[i]) return SUBSPEC_EINVAL;
    if (reinterpret_cast<uintptr_t>(packed[i]) & 15u) return SUBSPEC_ESCRATCH;
    n_total += n[i];
  }
  if (n_total > (1 << 24)) return SUBSPEC_EUNSUPPORTED;
  Plan p;
  if (!make_plan(m, (int)n_total, k, &p)) return SUBSPEC_EUNSUPPORTED;
  if (x_stride < k) return SUBSPEC_EINVAL;
  if (reinterpret_cast<uintptr_t>(scratch) & 255u) return SUBSPEC_ESCRATCH;
  if (scratch_bytes < p.xp_bytes + p.partial_bytes + p.ticket_bytes) return SUBSPEC_ESCRATCH;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* sp = reinterpret_cast<char*>(scratch);
  GemmArgs g;
  g.wpk = reinterpret_cast<const unsigned char*>(packed[0]);
  g.xp = reinterpret_cast<const __half*>(sp);
  g.partial = reinterpret_cast<float*>(sp + p.xp_bytes);
  g.ticket = reinterpret_cast<int*>(sp + p.xp_bytes + p.partial_bytes);
  g.y = reinterpret_cast<__nv_bfloat16*>(y[0]);
  g.dev_status = dev_status;
  g.M = m;
  g.Mpad = p.Mpad;
  g.N = (int)n_total;
  g.K = k;
  g.kblocks = p.kblocks;
  g.splits = p.splits;
  g.b_slots = p.b_slots;
  g.b_blocks = p.b_blocks;
  g.b_shift = p.b_shift;
  g.ring_raw = p.ring_raw;
  g.acc_n = p.acc_n;
  g.acc_stride = p.acc_stride;
  g.issuers = p.issuers;
  g.y_stride = y_stride[0];
  g.nseg = nseg;
  {
    int t0 = 0;
    for (int i = 0; i < kMaxGroup; ++i) {
      g.seg_tile0[i] = t0;
      g.seg_wpk[i] = i < nseg ? reinterpret_cast<const unsigned char*>(packed[i]) : nullptr;
      g.seg_y[i] = i < nseg ? reinterpret_cast<__nv_bfloat16*>(y[i]) : nullptr;
      g.seg_ystride[i] = i < nseg ? y_stride[i] : 0;
      if (i < nseg) t0 += n[i] / kTileN;
    }
  }
  struct { const void* x; int64_t x_stride; int m, k; } a{x, x_stride, m, k};
  int rc;
  {
    const int64_t total = (int64_t)p.kblocks * p.Mpad * 8;
    const int grid = (int)((total + 255) / 256 > 2368 ? 2368 : (total + 255) / 256);
    cudaLaunchConfig_t pc = {};
    pc.gridDim = dim3(grid);
    pc.blockDim = dim3(256);
    pc.stream = st;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pa[0].val.programmaticStreamSerializationAllowed = 1;
    pc.attrs = pa;
    pc.numAttrs = 1;
    rc = cuda_check(cudaLaunchKernelEx(&pc, w4a16_prep_x_kernel, reinterpret_cast<const __nv_bfloat16*>(a.x),
                                       (int64_t)a.x_stride, reinterpret_cast<__half*>(sp), (int)a.m, (int)p.Mpad,
                                       (int)a.k, g.ticket, (int)p.tiles));
    if (rc) return rc;
  }
  rc = cuda_check(cudaFuncSetAttribute(w4a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)p.smem_bytes));
  if (rc) return rc;
  // programmatic dependent launch: the prologue and the packed-weight copies overlap the preparation kernel
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.tiles, p.splits);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  g.cluster = 0;
  if (p.splits > 1) {
    // Split-K inside a thread-block cluster (one cluster = the splits of a tile) when all the tiles' clusters
    // can be resident at once: the partial sums then meet in shared memory instead of making the trip through
    // global memory, a fence and a ticket.  Fewer splits fit more clusters of a GPC's SMs: take the largest
    // count that leaves no tile waiting for a second wave; none does -> the path through global memory.
    int dev = 0;
    cudaGetDevice(&dev);
    const int per_plan = (p.kblocks + p.splits - 1) / p.splits;
    for (int c = p.splits; c >= 2 && !g.cluster; --c) {
      const int per = (p.kblocks + c - 1) / c;
      if ((p.kblocks + per - 1) / per != c) continue;  // some split would be empty
      // what the shorter tail saves (1.5 - 2 us) is worth about six more K blocks per CTA (measured on the
      // 3584 x 18944 shape: 74 instead of 60 K blocks per CTA cost more than the tail gave back)
      if (per - per_plan > 6) break;
      if (resident_clusters(dev, c, (int)p.smem_bytes) >= p.tiles) {
        g.cluster = 1;
        g.splits = c;
      }
    }
    if (g.cluster) {
      cfg.gridDim = dim3(p.tiles, g.splits);
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = 1;
      attr[1].val.clusterDim.y = (unsigned)g.splits;
      attr[1].val.clusterDim.z = 1;
      cfg.numAttrs = 2;
    }
  }
  return cuda_check(cudaLaunchKernelEx(&cfg, w4a16_gemm_kernel, g));
}
}  // namespace

extern "C" int subspec_w4a16_gemm(const subspec_w4a16_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_w4a16_args)) return SUBSPEC_EINVAL;
  const subspec_w4a16_args& a = *args;
  if (!a.x || !a.packed || !a.y || !a.scratch) return SUBSPEC_EINVAL;
  const void* packed[1] = {a.packed};
  void* y[1] = {a.y};
  const int32_t n[1] = {a.n};
  const int64_t ys[1] = {a.y_stride};
  return run_gemm(a.m, a.k, 1, packed, n, y, ys, a.x, a.x_stride, a.scratch, a.scratch_bytes, a.dev_status, stream);
}

extern "C" int subspec_w4a16_gemm_grouped(const subspec_w4a16_group_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_w4a16_group_args)) return SUBSPEC_EINVAL;
  const subspec_w4a16_group_args& a = *args;
  if (a.count < 1 || a.count > SUBSPEC_W4A16_MAX_GROUP) return SUBSPEC_EINVAL;
  return run_gemm(a.m, a.k, a.count, a.packed, a.n, a.y, a.y_stride, a.x, a.x_stride, a.scratch, a.scratch_bytes,
                  a.dev_status, stream);
}
