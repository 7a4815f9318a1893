// Tree attention over the paged KV cache, and the append of the tree's own K / V rows to it.
//
// Reference: the FlashInfer path of the generators -- append_paged_kv_cache followed by
// BatchPrefillWithPagedKVCacheWrapper.run with a custom mask
// (specdecodes/models/utils/flashinfer/attention_wrapper.py:104-151, 234-253, 288-316;
//  specdecodes/models/utils/flashinfer/attention.py:26-102).  The tree's tokens are the queries; every one of
// them sees the whole committed prefix and, among the tree's rows, itself and its ancestors (the mask the tree
// finaliser writes: prefix ones | ancestor-or-self columns | zeros).
//
// One CTA = 128 query rows of one (request, KV head): the rows are (head of the GQA group, tree token) pairs,
// so the seven query heads that share a KV head share its K / V tiles.  K / V tiles of 64 cache rows are
// gathered page by page with 16-byte cp.async copies into padded shared-memory rows (double-buffered); each
// warp owns 16 query rows: S = Q K^T and O += P V run on the tensor cores (mma.sync m16n8k16, bf16 in, fp32
// out), the online softmax in registers in the log2 domain.  Tiles that lie wholly inside the prefix need no
// mask look-up.  This is the warp-level tensor path, not tcgen05: the kernel is a first, correct version of
// this row of the hot path, and its distance from the tcgen05 roofline is reported as measured.
#include <math.h>

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

constexpr int kD = 128;           // head dimension (the only one built)
constexpr int kTileKV = 64;       // cache rows per tile
constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kRowsPerCta = kAttnWarps * 16;
constexpr int kPad = 8;                     // bf16 elements of padding per shared-memory row (bank spread)
constexpr int kRowElems = kD + kPad;        // 136 elements = 272 bytes
constexpr int kTileBytes = kTileKV * kRowElems * 2;
constexpr size_t kAttnSmem = (size_t)kTileBytes * 2 /*K, V*/ * 2 /*stages*/;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
               "l"(gmem), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int kAhead = 3;  // fragment loads in flight ahead of the MMAs

struct AttnArgs {
  subspec_tree_attn_args a;
  int group;        // query heads per KV head
  float scale_log2; // sm_scale * log2(e)
  int page_shift;   // log2(page_len) when it is a power of two, else -1
  int box_rows;     // cache rows per tensor copy (0: the page length does not suit them)
};

__global__ void __launch_bounds__(kAttnThreads, 1) tree_attn_kernel(const AttnArgs ka) {
  extern __shared__ __align__(16) unsigned char smem[];
  const subspec_tree_attn_args& a = ka.a;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = ka.group, QL = a.q_len;
  int nq = a.n_q ? a.n_q[b] : QL;
  nq = min(max(nq, 0), QL);
  int kv_len = a.kv_len[b];
  const int cap = a.pages_per_seq * a.page_len;
  if (kv_len < 0 || kv_len > cap) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
    kv_len = min(max(kv_len, 0), cap);
  }
  int prefix = a.prefix_len ? a.prefix_len[b] : kv_len - nq;
  prefix = min(max(prefix, 0), kv_len);
  const int row_base = blockIdx.x * kRowsPerCta + warp * 16;
  if (blockIdx.x * kRowsPerCta >= G * QL) return;

  // this thread's two query rows: r0 = row_base + lane / 4 and r0 + 8; a row is (head of the group, tree token)
  const int rA = row_base + (lane >> 2), rB = rA + 8;
  const int gA = rA / QL, iA = rA - gA * QL, gB = rB / QL, iB = rB - gB * QL;
  const bool okA = gA < G && iA < nq, okB = gB < G && iB < nq;
  const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* qA = q + (size_t)b * a.q_batch_stride + (size_t)iA * a.q_token_stride +
                            (size_t)(kvh * G + gA) * a.q_head_stride;
  const __nv_bfloat16* qB = q + (size_t)b * a.q_batch_stride + (size_t)iB * a.q_token_stride +
                            (size_t)(kvh * G + gB) * a.q_head_stride;
  // Q fragments: 8 k-steps of 16 dims
  uint32_t qf[kD / 16][4];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    const int c = ks * 16 + (lane & 3) * 2;
    qf[ks][0] = okA ? *reinterpret_cast<const uint32_t*>(qA + c) : 0u;
    qf[ks][1] = okB ? *reinterpret_cast<const uint32_t*>(qB + c) : 0u;
    qf[ks][2] = okA ? *reinterpret_cast<const uint32_t*>(qA + c + 8) : 0u;
    qf[ks][3] = okB ? *reinterpret_cast<const uint32_t*>(qB + c + 8) : 0u;
  }
  const uint8_t* mA = a.mask + (size_t)b * a.mask_batch_stride + (size_t)iA * a.mask_row_stride;
  const uint8_t* mB = a.mask + (size_t)b * a.mask_batch_stride + (size_t)iB * a.mask_row_stride;

  float o[kD / 8][4];
#pragma unroll
  for (int nt = 0; nt < kD / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float mxA = -INFINITY, mxB = -INFINITY, lA = 0.f, lB = 0.f;

  // ---- the gather of one K / V tile: 64 cache rows x 256 bytes each for K and for V, 16 bytes per copy ----
  const size_t row_bytes = (size_t)a.num_kv_heads * kD * 2;             // one cache row, all KV heads
  const size_t kv_plane = (size_t)a.page_len * row_bytes;              // K (or V) of one page
  const unsigned char* pool = reinterpret_cast<const unsigned char*>(a.pool) +
                              (size_t)a.layer * a.num_pages * 2 * kv_plane + (size_t)kvh * kD * 2;
  const int* table = a.page_table + (size_t)b * a.pages_per_seq;
  auto load_tile = [&](int tile, int stage) {
    unsigned char* ks_ = smem + (size_t)stage * 2 * kTileBytes;
    unsigned char* vs_ = ks_ + kTileBytes;
    for (int c = threadIdx.x; c < kTileKV * 16; c += kAttnThreads) {  // 16 copies of 16 bytes per row
      const int r = c >> 4, part = c & 15;
      const int pos = tile * kTileKV + r;
      const unsigned char* src = pool;
      int bytes = 0;
      if (pos < kv_len) {
        int page = table[pos / a.page_len];
        if (page < 0 || page >= a.num_pages) {
          flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
          page = 0;
        } else {
          bytes = 16;
        }
        src = pool + (size_t)page * 2 * kv_plane + (size_t)(pos % a.page_len) * row_bytes + part * 16;
      }
      cp_async16(ks_ + (size_t)r * kRowElems * 2 + part * 16, src, bytes);            // rows past the end: zeros
      cp_async16(vs_ + (size_t)r * kRowElems * 2 + part * 16, src + kv_plane, bytes);
    }
    cp_async_commit();
  };

  const int ntiles = (kv_len + kTileKV - 1) / kTileKV;
  if (ntiles > 0) load_tile(0, 0);
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) {
      load_tile(t + 1, (t + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* Ks = reinterpret_cast<const __nv_bfloat16*>(smem + (size_t)(t & 1) * 2 * kTileBytes);
    const __nv_bfloat16* Vs = Ks + kTileKV * kRowElems;

    // ---- S = Q K^T for 64 cache rows: 8 n-tiles of 8 rows ----
    float s[kTileKV / 8][4];
#pragma unroll
    for (int nt = 0; nt < kTileKV / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    // k-steps outside, n-tiles inside: consecutive MMAs write different accumulators (eight in flight) instead
    // of queueing behind one another on the same one.  One x4 load = the K fragments of two k-steps: lanes
    // 0-7 / 8-15 / 16-23 / 24-31 address cache rows nt*8 + 0..7 at dims 32 j + 0 / 8 / 16 / 24.
    const __nv_bfloat16* kbase = Ks + (size_t)(lane & 7) * kRowElems + ((lane >> 3) << 3);
    // The fragment loads run kAhead iterations ahead of the MMAs that use them (both are volatile asm, which
    // the compiler keeps in program order): a load's latency is covered by the MMAs of the iterations between.
    {
      constexpr int kIters = (kD / 32) * (kTileKV / 8);
      uint32_t kf[kAhead + 1][4];
#pragma unroll
      for (int i = 0; i < kAhead; ++i)
        ldmatrix_x4(kf[i], kbase + (size_t)(i % (kTileKV / 8)) * 8 * kRowElems + (i / (kTileKV / 8)) * 32);
#pragma unroll
      for (int i = 0; i < kIters; ++i) {
        if (i + kAhead < kIters) {
          const int n = i + kAhead;
          ldmatrix_x4(kf[n % (kAhead + 1)], kbase + (size_t)(n % (kTileKV / 8)) * 8 * kRowElems + (n / (kTileKV / 8)) * 32);
        }
        const int j = i / (kTileKV / 8), nt = i % (kTileKV / 8);
        mma_bf16(s[nt], qf[2 * j], kf[i % (kAhead + 1)][0], kf[i % (kAhead + 1)][1]);
        mma_bf16(s[nt], qf[2 * j + 1], kf[i % (kAhead + 1)][2], kf[i % (kAhead + 1)][3]);
      }
    }
    // ---- scale, mask, online softmax ----
    const int t0 = t * kTileKV;
    const bool need_mask = t0 + kTileKV > prefix;  // tiles inside the prefix are visible to every row
    float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < kTileKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * ka.scale_log2;
        if (need_mask) {
          const int pos = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const uint8_t* mrow = (e & 2) ? mB : mA;
          const bool row_ok = (e & 2) ? okB : okA;
          const bool vis = pos < prefix || (pos < kv_len && row_ok && mrow[pos] != 0);
          v = vis ? v : -INFINITY;
        }
        s[nt][e] = v;
      }
      tmA = fmaxf(tmA, fmaxf(s[nt][0], s[nt][1]));
      tmB = fmaxf(tmB, fmaxf(s[nt][2], s[nt][3]));
    }
    tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
    tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
    tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
    tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
    const float nA = fmaxf(mxA, tmA), nB = fmaxf(mxB, tmB);
    const float uA = nA == -INFINITY ? 0.f : nA, uB = nB == -INFINITY ? 0.f : nB;  // a row with nothing visible yet
    const float alA = ex2f(mxA - uA), alB = ex2f(mxB - uB);
    mxA = nA;
    mxB = nB;
    float sumA = 0.f, sumB = 0.f;
#pragma unroll
    for (int nt = 0; nt < kTileKV / 8; ++nt) {
      s[nt][0] = ex2f(s[nt][0] - uA);
      s[nt][1] = ex2f(s[nt][1] - uA);
      s[nt][2] = ex2f(s[nt][2] - uB);
      s[nt][3] = ex2f(s[nt][3] - uB);
      sumA += s[nt][0] + s[nt][1];
      sumB += s[nt][2] + s[nt][3];
    }
    lA = lA * alA + sumA;  // per-thread partial sums: the quad is added up once, at the end
    lB = lB * alB + sumB;
#pragma unroll
    for (int nt = 0; nt < kD / 8; ++nt) {
      o[nt][0] *= alA;
      o[nt][1] *= alA;
      o[nt][2] *= alB;
      o[nt][3] *= alB;
    }
    // ---- O += P V: 4 k-steps of 16 cache rows; V row-major [row][dim] is read transposed ----
    // lanes 0-7 / 8-15 address cache rows ks*16 + 0..7 / 8..15 of dims [16 j, 16 j + 8), lanes 16-31 the same
    // rows of dims [16 j + 8, 16 j + 16): one x4 load feeds two n-tiles.  Loads run kAhead iterations ahead.
    {
      constexpr int kJ = kD / 16, kIters = (kTileKV / 16) * kJ;
      const __nv_bfloat16* vbase = Vs + (size_t)(lane & 15) * kRowElems + ((lane >> 4) << 3);
      uint32_t vf[kAhead + 1][4];
#pragma unroll
      for (int i = 0; i < kAhead; ++i) ldmatrix_x4_trans(vf[i], vbase + (size_t)(i / kJ) * 16 * kRowElems + (i % kJ) * 16);
      uint32_t pf[4];
#pragma unroll
      for (int i = 0; i < kIters; ++i) {
        if (i + kAhead < kIters) {
          const int n = i + kAhead;
          ldmatrix_x4_trans(vf[n % (kAhead + 1)], vbase + (size_t)(n / kJ) * 16 * kRowElems + (n % kJ) * 16);
        }
        const int ks = i / kJ, j = i % kJ;
        if (j == 0) {
          pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
          pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
          pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
          pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
        }
        mma_bf16(o[2 * j], pf, vf[i % (kAhead + 1)][0], vf[i % (kAhead + 1)][1]);
        mma_bf16(o[2 * j + 1], pf, vf[i % (kAhead + 1)][2], vf[i % (kAhead + 1)][3]);
      }
    }
    __syncthreads();  // the stage is free for the load after next
  }
  lA += __shfl_xor_sync(0xffffffffu, lA, 1);
  lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1);
  lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  const float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
  __nv_bfloat16* oA = out + (size_t)b * a.o_batch_stride + (size_t)iA * a.o_token_stride +
                      (size_t)(kvh * G + gA) * a.o_head_stride;
  __nv_bfloat16* oB = out + (size_t)b * a.o_batch_stride + (size_t)iB * a.o_token_stride +
                      (size_t)(kvh * G + gB) * a.o_head_stride;
#pragma unroll
  for (int nt = 0; nt < kD / 8; ++nt) {
    const int c = nt * 8 + (lane & 3) * 2;
    if (okA) *reinterpret_cast<uint32_t*>(oA + c) = pack_bf16(o[nt][0] * invA, o[nt][1] * invA);
    if (okB) *reinterpret_cast<uint32_t*>(oB + c) = pack_bf16(o[nt][2] * invB, o[nt][3] * invB);
  }
}

// ================================ the tcgen05 kernel ================================================
// One CTA = 256 query rows of one (request, KV head) -- two blocks of 128 rows that share every K / V tile --
// and tiles of 128 cache rows.
//
//   warps 0-7   softmax, four warps per row block: thread = query row = lane of tensor memory.  Per tile a
//               thread reads its row of S (tcgen05.ld), keeps the running maximum and sum, rescales its row of O
//               in tensor memory when the maximum of any row of the warp moved, and writes P = exp2(S c - m)
//               as packed bf16 over the first half of the S columns it has just read (tcgen05.st).
//   warp 8      one elected thread issues the MMAs.  S = Q K^T: A = the block's Q tile, B = the K tile, both
//               K-major in shared memory.  O += P V: A = P from tensor memory, B = the V tile, MN-major: V lies
//               [cache row][dim] as the cache has it, so K and V tiles share one shared-memory layout and the
//               gather never transposes.  Order per tile: PV(a), S(a, next tile), PV(b), S(b, next tile): while
//               one block's softmax runs, the tensor core works for the other.
//   warps 9-11  gather: 16-byte cp.async copies, row by row (cache rows through the page table), into the
//               128-byte-swizzled layout the tensor core reads: a tile = two blocks of 64 dims, a block = 128
//               rows of 128 bytes, 16-byte chunk c of row r stored at chunk c ^ (r & 7).  First the two Q
//               tiles, then K(0), V(0), K(1), V(1), ... through a ring of five 32 KB entries.
//
// Tensor memory (512 columns, one CTA per SM): S(a) | S(b) | O(a) | O(b), 128 columns each.
constexpr int kTcBlockRows = 128;                   // query rows per row block = MMA M
constexpr int kTcRows = 2 * kTcBlockRows;           // query rows per CTA
constexpr int kTcKeys = 128;                        // cache rows per tile
constexpr int kTcRing = 5;                          // ring entries: one K or V tile each
constexpr int kTcHalfBytes = kTcKeys * 128;         // 64 dims of 128 rows
constexpr int kTcTileBytes = 2 * kTcHalfBytes;      // one Q, K or V tile: 32 KB
constexpr size_t kTcSmem = (size_t)(2 + kTcRing) * kTcTileBytes + 1024;  // + room to align to the swizzle atom
constexpr int kTcSoftmaxWarps = 8;
constexpr int kTcIssuerWarp = 8;                    // warps 8, 9: one issuer per row block
constexpr int kTcLoadWarp0 = 10;
constexpr int kTcLoadWarps = 2;                     // twelve warps in all: three per scheduler, 168 registers each
constexpr int kTcLoadThreads = 32 * kTcLoadWarps;
constexpr int kTcLoadRows = kTcLoadThreads / 16;    // rows a gather pass covers (16 lanes per row)
constexpr int kTcThreads = 32 * (kTcLoadWarp0 + kTcLoadWarps);
constexpr int kTcInflight = 3;                      // ring entries a gather thread keeps in flight
constexpr uint32_t kColS = 0, kColO = 256, kTcCols = 512;

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row atoms of 1024 bytes: [0,14) address >> 4, [16,30)
// leading byte offset >> 4, [32,46) stride byte offset >> 4, [46,48) version 1, [61,64) layout 2.
// K-major operand (Q and K tiles: rows x dims): stride = 1024 between 8-row groups, leading unused.
// MN-major operand (the V tile: N = dims, K = cache rows): stride = 1024 between groups of 8 cache rows,
// leading = the distance between the two 64-dim halves.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t leading_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(leading_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16: D fp32 (bit 4), A and B bf16 (1 at [7,10) and [10,13)), bit 16 = B is
// MN-major, N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t tc_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The hand-overs between the roles of this kernel are short and on the critical path of every tile: poll the
// barrier (try_wait comes back as soon as the phase completes) instead of sleeping on a suspend-time hint,
// which was seen to cost about a microsecond per hand-over.  Bounded like every wait here.
constexpr uint32_t kTcPollLimit = 1u << 24;
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kTcPollLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Tensor copy (TMA), five coordinates, global -> shared, completion counted in bytes on `bar`.  The innermost
// coordinate times the element size must be a multiple of 16 bytes (here 0 or 64 bf16).
__device__ __forceinline__ void tma_load_5d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], "
      "[%7];" ::"r"(smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
      : "memory");
}

struct TcRingPos {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next() {
    if (++s == kTcRing) {
      s = 0;
      ph ^= 1u;
    }
  }
};

__global__ void __launch_bounds__(kTcThreads, 1)
    tree_attn_tc_kernel(const AttnArgs ka, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kTcRing], empty[kTcRing], s_ready[2], p_ready[2], o_done[2], q_ready;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const subspec_tree_attn_args& a = ka.a;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = ka.group, QL = a.q_len;
  const int row0 = (int)blockIdx.x * kTcRows;
  if (row0 >= G * QL) return;
  const int nblk = row0 + kTcBlockRows < G * QL ? 2 : 1;  // the second row block may be empty
  int nq = a.n_q ? a.n_q[b] : QL;
  nq = min(max(nq, 0), QL);
  int kv_len = a.kv_len[b];
  const int cap = a.pages_per_seq * a.page_len;
  if (kv_len < 0 || kv_len > cap) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
    kv_len = min(max(kv_len, 0), cap);
  }
  int prefix = a.prefix_len ? a.prefix_len[b] : kv_len - nq;
  prefix = min(max(prefix, 0), kv_len);
  const int ntiles = (kv_len + kTcKeys - 1) / kTcKeys;

  if (ntiles == 0) {  // nothing to attend to: zeros, as the sum of no terms
    if (threadIdx.x < kTcRows) {
      const int row = row0 + (int)threadIdx.x, rg = row / QL, ri = row - rg * QL;
      if (rg < G && ri < nq) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.o_batch_stride +
                           (size_t)ri * a.o_token_stride + (size_t)(kvh * G + rg) * a.o_head_stride;
        for (int c = 0; c < kD / 2; ++c) reinterpret_cast<uint32_t*>(o)[c] = 0u;
      }
    }
    return;
  }

  unsigned char* qtiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* ring = qtiles + 2 * kTcTileBytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcRing; ++s) {
      mbar_init(&full[s], kTcLoadThreads);
      mbar_init(&empty[s], (uint32_t)nblk);  // every row block's issuer lets go of the entry
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&s_ready[k], 1);
      mbar_init(&p_ready[k], kTcSoftmaxWarps / 2);
      mbar_init(&o_done[k], 1);
    }
    mbar_init(&q_ready, 32 * kTcSoftmaxWarps);
    mbar_init_fence();
    s_abort = 0;
  }
  if (warp == kTcIssuerWarp) {
    tmem_alloc(&s_tmem, kTcCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  volatile int* abort_flag = &s_abort;

  if (warp < kTcSoftmaxWarps) {
    // ================= softmax: thread = query row = tensor-memory lane =================
    {  // the two Q tiles, gathered by all the softmax threads (16 lanes per row, 16 rows per pass): rows that
       // do not exist are zeros
      const int chunk = (int)threadIdx.x & 15, sub = (int)threadIdx.x >> 4;
      const unsigned char* qbase = reinterpret_cast<const unsigned char*>(a.q) + chunk * 16;
#pragma unroll 4
      for (int pass = 0; pass < kTcRows / 16; ++pass) {
        const int rr = pass * 16 + sub;  // row of the CTA; its block = rr / 128
        const int qrow = row0 + rr, qg = qrow / QL, qi = qrow - qg * QL;
        const bool okr = qg < G && qi < nq;
        const unsigned char* src = okr ? qbase + 2 * ((size_t)b * a.q_batch_stride + (size_t)qi * a.q_token_stride +
                                                      (size_t)(kvh * G + qg) * a.q_head_stride)
                                       : qbase;
        unsigned char* d = qtiles + (size_t)(rr >> 7) * kTcTileBytes + (chunk >> 3) * kTcHalfBytes + (rr & 127) * 128 +
                           (((chunk & 7) ^ (rr & 7)) << 4);
        cp_async16(d, src, okr ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_async_smem();
      mbar_arrive(&q_ready);
    }
    const int blk = warp >> 2;
    const int row = row0 + (int)threadIdx.x, rg = row / QL, ri = row - rg * QL;
    const bool row_ok = rg < G && ri < nq;
    if (blk < nblk) {
      const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t s_addr = lane_base + kColS + (uint32_t)(blk * kTcKeys);
      const uint32_t o_addr = lane_base + kColO + (uint32_t)(blk * kD);
      const uint8_t* mrow = a.mask + (size_t)b * a.mask_batch_stride + (size_t)ri * a.mask_row_stride;
      const float c2 = ka.scale_log2;
      float m = -INFINITY, l = 0.f;  // running maximum (in the exponent's units) and sum of this row
      bool live = true;
      for (int t = 0; t < ntiles; ++t) {
        // S(t) complete; the MMAs run in order, so the block's O += P V of the tile before is complete too
        live = __all_sync(0xffffffffu, tc_wait(&s_ready[blk], (uint32_t)t & 1u, abort_flag));
        if (!live) break;
        tc_fence_after();
        const int t0 = t * kTcKeys;
        const bool need_mask = t0 + kTcKeys > prefix;  // tiles inside the prefix are visible to every row
        uint32_t vis[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t bits = 0;
            for (int j = 0; j < 32; ++j) {
              const int pos = t0 + 32 * c + j;
              const bool v = pos < prefix || (pos < kv_len && row_ok && mrow[pos] != 0);
              bits |= (v ? 1u : 0u) << j;
            }
            vis[c] = bits;
          }
        }
        // ---- pass 1: the row's maximum over the tile (four chains, not one) ----
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32_async(s_addr + 32 * c, r);
          tmem_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if ((vis[c] >> j) & 1u) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r[j]));
          }
        }
        const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        const float m_new = fmaxf(m, tmax * c2);           // c2 > 0: the maximum commutes with the scaling
        const float u = m_new == -INFINITY ? 0.f : m_new;  // a row with nothing visible yet
        const float alpha = ex2f(m - u);                   // 0 while m is -inf
        m = m_new;
        if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32_async(o_addr + 32 * c, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
            tmem_st32(o_addr + 32 * c, r);
          }
        }
        // ---- pass 2: P = exp2(S c2 - m) over the S columns already read, the row sum ----
        float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32_async(s_addr + 32 * c, r);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float p0 = ex2f(fmaf(__uint_as_float(r[2 * j]), c2, -u));
            float p1 = ex2f(fmaf(__uint_as_float(r[2 * j + 1]), c2, -u));
            if (need_mask) {
              p0 = ((vis[c] >> (2 * j)) & 1u) ? p0 : 0.f;
              p1 = ((vis[c] >> (2 * j + 1)) & 1u) ? p1 : 0.f;
            }
            sm[j & 3] += p0 + p1;
            pk[j] = pack_bf16(p0, p1);
          }
          tmem_st16(s_addr + 16 * c, pk);  // columns [16 c, 16 c + 16) <- keys [32 c, 32 c + 32): behind the reads
        }
        l = l * alpha + ((sm[0] + sm[1]) + (sm[2] + sm[3]));
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[blk]);
      }
      // ---- the result: O / l ----
      if (live) live = __all_sync(0xffffffffu, tc_wait(&o_done[blk], (uint32_t)(ntiles - 1) & 1u, abort_flag));
      if (live) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.o_batch_stride +
                                 (size_t)ri * a.o_token_stride + (size_t)(kvh * G + rg) * a.o_head_stride;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32_async(o_addr + 32 * c, r);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * j]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
              reinterpret_cast<uint4*>(out_row)[4 * c + j] = v;
            }
          }
        }
        tc_fence_before();
      }
    }
  } else if (warp < kTcLoadWarp0) {
    // ================= MMA issue, one warp per row block: the whole warp runs the loop, one elected lane
    // issues.  A thread gets a tcgen05.mma out every 150 cycles or so, more than the tensor core needs for a
    // 128 x 128 x 16 step: two issuing threads keep it busy where one does not. =================
    const int blk = warp - kTcIssuerWarp;
    if (blk < nblk) {
      constexpr uint32_t idesc_s = tc_idesc(kTcBlockRows, kTcKeys, false);
      constexpr uint32_t idesc_o = tc_idesc(kTcBlockRows, kD, true);
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
      const uint32_t tm_s = tm + kColS + (uint32_t)(blk * kTcKeys), tm_o = tm + kColO + (uint32_t)(blk * kD);
      const uint32_t q_u32 = smem_u32(qtiles) + (uint32_t)blk * kTcTileBytes, ring_u32 = smem_u32(ring);
      // S = Q K^T: 8 steps of 16 dims; a step moves 32 bytes inside a 64-dim half, 4 steps per half
      auto issue_s = [&](int kstage) {
        const uint32_t kaddr = ring_u32 + (uint32_t)kstage * kTcTileBytes;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          const uint32_t off = (uint32_t)((ks >> 2) * kTcHalfBytes + (ks & 3) * 32);
          tc_mma_f16_ss(tm_s, tc_desc(q_u32 + off, 16), tc_desc(kaddr + off, 16), idesc_s, ks > 0 ? 1u : 0u);
        }
      };
      // O += P V: 8 steps of 16 cache rows = 2048 bytes of the V tile each; P = the first 64 columns of S
      auto issue_pv = [&](int vstage, bool first) {
        const uint32_t vaddr = ring_u32 + (uint32_t)vstage * kTcTileBytes;
#pragma unroll
        for (int ks = 0; ks < kTcKeys / 16; ++ks)
          tc_mma_f16_ta(tm_o, tm_s + (uint32_t)(8 * ks), tc_desc(vaddr + (uint32_t)(ks * 2048), kTcHalfBytes), idesc_o,
                        (!first || ks > 0) ? 1u : 0u);
      };
      TcRingPos pos;  // ring entries in the order they are consumed: K(0), V(0), K(1), V(1), ...
      bool ok = __all_sync(0xffffffffu, tc_wait(&q_ready, 0, abort_flag));
      ok = ok && __all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag));
      if (ok) {
        tc_fence_after();
        if (elect_one()) {
          issue_s(pos.s);
          tc_commit(&s_ready[blk]);
          tc_commit(&empty[pos.s]);
        }
        __syncwarp();
        pos.next();
        for (int t = 0; t < ntiles; ++t) {
          // O += P V(t), then S of the next tile over the P just consumed: the MMAs of a thread run in order
          ok = __all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag)) &&
               __all_sync(0xffffffffu, tc_wait(&p_ready[blk], (uint32_t)t & 1u, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_pv(pos.s, t == 0);
            tc_commit(&o_done[blk]);
            tc_commit(&empty[pos.s]);
          }
          __syncwarp();
          pos.next();
          if (t + 1 < ntiles) {
            if (!__all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag))) break;
            tc_fence_after();
            if (elect_one()) {
              issue_s(pos.s);
              tc_commit(&s_ready[blk]);
              tc_commit(&empty[pos.s]);
            }
            __syncwarp();
            pos.next();
          }
        }
      }
    }
  } else {
    // ================= gather: 16 lanes per row (its 16 chunks of 16 bytes), 4 rows per pass =================
    const int p = (int)threadIdx.x - 32 * kTcLoadWarp0;
    const int chunk = p & 15, sub = p >> 4;
    const uint32_t dst_half = (uint32_t)((chunk >> 3) * kTcHalfBytes);
    const size_t row_bytes = (size_t)a.num_kv_heads * kD * 2;   // one cache row, all KV heads
    const size_t kv_plane = (size_t)a.page_len * row_bytes;     // K (or V) of one page
    const unsigned char* pool = reinterpret_cast<const unsigned char*>(a.pool) +
                                (size_t)a.layer * a.num_pages * 2 * kv_plane + (size_t)kvh * kD * 2 + chunk * 16;
    const int* table = a.page_table + (size_t)b * a.pages_per_seq;
    TcRingPos wr, done;
    int pending = 0;  // cp.async entries committed and not yet handed over
    const int nent = 2 * ntiles;
    for (int n = 0; n < nent; ++n) {
      if (n >= kTcRing && !tc_wait(&empty[wr.s], wr.ph ^ 1u, abort_flag)) break;
      const int t = n >> 1, t0 = t * kTcKeys;
      if (ka.box_rows > 0 && t0 + kTcKeys <= kv_len) {
        // A whole tile of whole pages: tensor copies (TMA) of box_rows cache rows x 64 dims each, which the copy
        // unit lays out in the swizzled form itself.  One thread announces the bytes, the others just arrive;
        // the first 2 * (128 / box_rows) threads issue one copy each.
        if (p == 0)
          mbar_expect_tx(&full[wr.s], (uint32_t)kTcTileBytes);
        else
          mbar_arrive(&full[wr.s]);
        const int j = p >> 1, half = p & 1;
        if (j * ka.box_rows < kTcKeys) {
          const int kpos = t0 + j * ka.box_rows;
          const int pi = ka.page_shift >= 0 ? kpos >> ka.page_shift : kpos / a.page_len;
          int page = table[pi];
          if (page < 0 || page >= a.num_pages) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
            page = a.num_pages;  // outside the tensor: the copy unit fills zeros and touches no memory
          }
          tma_load_5d(ring + (size_t)wr.s * kTcTileBytes + half * kTcHalfBytes + (size_t)j * ka.box_rows * 128, &tmap,
                      half * 64, kvh, kpos - pi * a.page_len, n & 1, page, &full[wr.s]);
        }
        wr.next();
        done = wr;
        continue;
      }
      // The last, partial tile (or a page length the tensor copies do not cover): 16-byte copies, row by row
      const size_t plane_off = (n & 1) ? kv_plane : 0;
      unsigned char* dst = ring + (size_t)wr.s * kTcTileBytes + dst_half;
#pragma unroll 4
      for (int pass = 0; pass < (kTcKeys + kTcLoadRows - 1) / kTcLoadRows; ++pass) {
        const int rr = pass * kTcLoadRows + sub;
        if (rr >= kTcKeys) break;
        const int kpos = t0 + rr;
        const unsigned char* src = pool;
        int bytes = 0;
        if (kpos < kv_len) {
          const int pi = ka.page_shift >= 0 ? kpos >> ka.page_shift : kpos / a.page_len;
          int page = table[pi];
          if (page < 0 || page >= a.num_pages) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
            page = 0;
          } else {
            bytes = 16;
          }
          src = pool + (size_t)page * 2 * kv_plane + plane_off + (size_t)(kpos - pi * a.page_len) * row_bytes;
        }
        cp_async16(dst + rr * 128 + (((chunk & 7) ^ (rr & 7)) << 4), src, bytes);  // rows past the end: zeros
      }
      cp_async_commit();
      wr.next();
      if (++pending == kTcInflight) {  // the oldest entry in flight has landed: hand it to the tensor core's proxy
        cp_async_wait<kTcInflight - 1>();
        fence_async_smem();
        mbar_arrive(&full[done.s]);
        done.next();
        --pending;
      }
    }
    cp_async_wait<0>();
    fence_async_smem();
    for (; pending > 0; --pending) {
      mbar_arrive(&full[done.s]);
      done.next();
    }
  }
  __syncthreads();
  if (s_abort && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_TIMEOUT);
  if (warp == kTcIssuerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTcCols);
  }
}

// The tree's own K / V rows into the cache: token i of request b goes to cache row kv_len[b] - n_q[b] + i.
__global__ void kv_append_kernel(const subspec_kv_append_args a) {
  const int b = blockIdx.y, i = blockIdx.x;
  int nq = a.n_q ? a.n_q[b] : a.q_len;
  nq = min(max(nq, 0), a.q_len);
  if (i >= nq) return;
  const int pos = a.kv_len[b] - nq + i;
  if (pos < 0 || pos >= a.pages_per_seq * a.page_len) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_INDEX);
    return;
  }
  const int page = a.page_table[(size_t)b * a.pages_per_seq + pos / a.page_len];
  if (page < 0 || page >= a.num_pages) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
    return;
  }
  const size_t row_elems = (size_t)a.num_kv_heads * a.head_dim;
  const size_t plane = (size_t)a.page_len * row_elems;
  uint4* dk = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.pool) +
                                       (((size_t)a.layer * a.num_pages + page) * 2) * plane +
                                       (size_t)(pos % a.page_len) * row_elems);
  uint4* dv = dk + plane / 8;
  const uint4* sk = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.k) +
                                                   (size_t)b * a.batch_stride + (size_t)i * a.token_stride);
  const uint4* sv = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.v) +
                                                   (size_t)b * a.batch_stride + (size_t)i * a.token_stride);
  for (int c = threadIdx.x; c < (int)(row_elems / 8); c += blockDim.x) {
    dk[c] = sk[c];
    dv[c] = sv[c];
  }
}

}  // namespace
}  // namespace subspec

using namespace subspec;

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tensor_map_encode_fn tensor_map_encoder() {
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

extern "C" int subspec_tree_attention_paged(const subspec_tree_attn_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_tree_attn_args)) return SUBSPEC_EINVAL;
  const subspec_tree_attn_args& a = *args;
  if (a.batch < 0 || a.q_len < 1 || a.num_q_heads < 1 || a.num_kv_heads < 1 || a.layers < 1 || a.layer < 0 ||
      a.layer >= a.layers || a.num_pages < 1 || a.page_len < 1 || a.pages_per_seq < 1)
    return SUBSPEC_EINVAL;
  if (a.head_dim != kD || a.num_q_heads % a.num_kv_heads) return SUBSPEC_EUNSUPPORTED;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.q || !a.out || !a.pool || !a.page_table || !a.kv_len || !a.mask) return SUBSPEC_EINVAL;
  if (!(a.sm_scale > 0.0)) return SUBSPEC_EINVAL;
  // 32-bit loads of query / output pairs, 16-byte copies of cache rows
  if ((reinterpret_cast<uintptr_t>(a.q) & 3u) || (reinterpret_cast<uintptr_t>(a.out) & 3u) ||
      (reinterpret_cast<uintptr_t>(a.pool) & 15u) || (a.q_token_stride & 1) || (a.q_head_stride & 1) ||
      (a.q_batch_stride & 1) || (a.o_token_stride & 1) || (a.o_head_stride & 1) || (a.o_batch_stride & 1))
    return SUBSPEC_EUNSUPPORTED;
  AttnArgs ka;
  ka.a = a;
  ka.group = a.num_q_heads / a.num_kv_heads;
  ka.scale_log2 = (float)(a.sm_scale * 1.4426950408889634);
  ka.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft)
    if ((1 << sft) == a.page_len) ka.page_shift = sft;
  const cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (getenv("SUBSPEC_ATTN_MMA_SYNC")) {
    int rc = cuda_check(
        cudaFuncSetAttribute(tree_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem));
    if (rc) return rc;
    const dim3 grid((unsigned)((ka.group * a.q_len + kRowsPerCta - 1) / kRowsPerCta), (unsigned)a.num_kv_heads,
                    (unsigned)a.batch);
    tree_attn_kernel<<<grid, kAttnThreads, kAttnSmem, st>>>(ka);
    return cuda_check(cudaGetLastError());
  }
  const int rc =
      cuda_check(cudaFuncSetAttribute(tree_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
  if (rc) return rc;
  const dim3 grid((unsigned)((ka.group * a.q_len + kTcRows - 1) / kTcRows), (unsigned)a.num_kv_heads, (unsigned)a.batch);
  // The tensor map of this layer's slab of the pool: [page][K / V][slot][KV head][dim], bf16.  A box is 64 dims of
  // box_rows consecutive slots of one page and one head; it exists when whole pages tile the 128 cache rows of a
  // tile (or a page holds whole tiles) and the swizzle atom of 8 rows divides a page.
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  ka.box_rows = 0;
  int box = 0;
  if (a.page_len % 8 == 0) {
    if (a.page_len <= kTcKeys && kTcKeys % a.page_len == 0)
      box = a.page_len;
    else if (a.page_len % kTcKeys == 0)
      box = kTcKeys;
  }
  if (box && tensor_map_encoder()) {
    const cuuint64_t row_bytes = (cuuint64_t)a.num_kv_heads * kD * 2, plane = (cuuint64_t)a.page_len * row_bytes;
    const cuuint64_t dims[5] = {(cuuint64_t)kD, (cuuint64_t)a.num_kv_heads, (cuuint64_t)a.page_len, 2, (cuuint64_t)a.num_pages};
    const cuuint64_t strides[4] = {(cuuint64_t)kD * 2, row_bytes, plane, 2 * plane};
    const cuuint32_t boxdim[5] = {64, 1, (cuuint32_t)box, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    void* base = const_cast<unsigned char*>(reinterpret_cast<const unsigned char*>(a.pool)) +
                 (size_t)a.layer * a.num_pages * 2 * plane;
    if (tensor_map_encoder()(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, boxdim, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
      ka.box_rows = box;
  }
  tree_attn_tc_kernel<<<grid, kTcThreads, kTcSmem, st>>>(ka, tmap);
  return cuda_check(cudaGetLastError());
}

extern "C" int subspec_kv_append_paged(const subspec_kv_append_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_kv_append_args)) return SUBSPEC_EINVAL;
  const subspec_kv_append_args& a = *args;
  if (a.batch < 0 || a.q_len < 1 || a.num_kv_heads < 1 || a.head_dim < 1 || a.layers < 1 || a.layer < 0 ||
      a.layer >= a.layers || a.num_pages < 1 || a.page_len < 1 || a.pages_per_seq < 1)
    return SUBSPEC_EINVAL;
  if (((size_t)a.num_kv_heads * a.head_dim) % 8 || (a.batch_stride % 8) || (a.token_stride % 8) ||
      (reinterpret_cast<uintptr_t>(a.pool) & 15u) || (reinterpret_cast<uintptr_t>(a.k) & 15u) ||
      (reinterpret_cast<uintptr_t>(a.v) & 15u))
    return SUBSPEC_EUNSUPPORTED;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.k || !a.v || !a.pool || !a.page_table || !a.kv_len) return SUBSPEC_EINVAL;
  kv_append_kernel<<<dim3((unsigned)a.q_len, (unsigned)a.batch), 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cuda_check(cudaGetLastError());
}
