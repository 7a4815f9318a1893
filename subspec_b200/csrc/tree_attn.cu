// Tree attention over the KV cache, and the append of the tree's own K / V rows to the paged cache.
//
// Reference: the FlashInfer path of the generators -- append_paged_kv_cache followed by
// BatchPrefillWithPagedKVCacheWrapper.run with a custom mask
// (specdecodes/models/utils/flashinfer/attention_wrapper.py:104-151, 234-253, 288-316;
//  specdecodes/models/utils/flashinfer/attention.py:26-102) -- and, on the default path, the model's
// scaled_dot_product_attention over the static caches (specdecodes/models/utils/cache_utils.py, TreeStaticCache)
// with the additive mask the generators splice into their static buffer (generators/classic_sd.py:57-89).  The
// tree's tokens are the queries; every one of them sees the whole committed prefix and, among the tree's rows,
// itself and its ancestors (the mask the tree finaliser writes: prefix ones | ancestor-or-self columns | zeros).
//
// The rows of the attention problem are (head of the GQA group, tree token) pairs, so the query heads that share
// a KV head share its K / V tiles.  The kernel runs on the tcgen05 tensor cores; its layout is described where
// it starts.
#include <math.h>

#include <type_traits>

#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

// Head dimensions 64 and 128 (kDim below); shared and tensor memory are laid out for 128 either way.

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
// two floats -> one 32-bit word of the cache's 16-bit type (kHalf: fp16, else bf16), low half first
template <bool kHalf>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if (kHalf) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// 2^x for a pair of exponents without the special-function unit: x = n + f with n = round(x), f in [-0.5, 0.5];
// 2^f by a cubic (relative error below 8e-5: a twenty-fifth of what rounding P to bf16 costs, a sixth for fp16),
// n added into the exponent field.  The magic constant 1.5 * 2^23 leaves n in the low mantissa bits of x + magic.
__device__ __forceinline__ void exp2_pair_fma(float x0, float x1, float& p0, float& p1) {
  const uint64_t xc = f2_pack(fmaxf(x0, -125.f), fmaxf(x1, -125.f));  // -inf (masked away later) and underflow
  const uint64_t magic = f2_pack(12582912.f, 12582912.f), nmagic = f2_pack(-12582912.f, -12582912.f);
  const uint64_t t2 = f2_add(xc, magic);
  const uint64_t n2 = f2_add(t2, nmagic);
  const uint64_t f2 = f2_fma(n2, f2_pack(-1.f, -1.f), xc);
  uint64_t q = f2_fma(f2_pack(0.0551716685f, 0.0551716685f), f2, f2_pack(0.242611125f, 0.242611125f));
  q = f2_fma(q, f2, f2_pack(0.693260968f, 0.693260968f));
  q = f2_fma(q, f2, f2_pack(0.999928057f, 0.999928057f));
  float q0, q1, t0, t1;
  f2_unpack(q, q0, q1);
  f2_unpack(t2, t0, t1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

struct AttnArgs {
  subspec_tree_attn_args a;
  int group;        // query heads per KV head
  float scale_log2; // sm_scale * log2(e)
  int page_shift;   // log2(page_len) when it is a power of two, else -1
  int box_rows;     // cache rows per tensor copy (0: the page length does not suit them)
  // where the rows lie: K (V) row `slot` of page `pg`, KV head h = k_base (v_base) + pg * page_stride +
  // slot * row_stride + h * head_stride bytes.  The paged pool and the [batch, heads, rows, dim] caches of the
  // Hugging Face path (a "page" = a batch entry, the page table the identity) differ in these numbers only.
  const unsigned char* k_base;
  const unsigned char* v_base;
  long long page_stride, row_stride, head_stride;
  int identity_table;
  int rows_before_heads;  // order of the two middle coordinates of the tensor maps (strides ascend in them)
  int mask_bytes;   // bytes per mask element: 1 (bool: non-zero = visible), 2 or 4 (additive: +-0 = visible)
  int splits;       // CTAs that share the cache rows of one (request, KV head, 256 query rows); 1: none
  float* part_o;    // splits > 1: [row][split][128] unnormalised outputs, row = (batch * q_heads + head) * q_len + token
  float* part_ml;   //             [row][split][2]   reference point (log2 units) and sum of the split
};

// One CTA = 256 query rows of one (request, KV head) -- two blocks of 128 rows that share every K / V tile --
// and tiles of 64 cache rows.
//
//   warps 0-7   softmax, four warps per row block: thread = query row = lane of tensor memory.  Per tile a
//               thread reads its row of S (tcgen05.ld) and writes P = exp2(S c - m) as packed 16-bit values
//               over the first half of the S columns it has just read, keeping the row sum; m, the reference
//               point of the row's exponents, moves (and the row of O in tensor memory is rescaled) only when
//               the row's maximum has run more than 2^8 ahead of it.
//   warps 8, 9  one MMA issuer per row block (an elected thread).  S = Q K^T: A = the block's Q tile, B = the K
//               tile, both K-major in shared memory.  O += P V: A = P from tensor memory, B = the V tile,
//               MN-major: V lies [cache row][dim] as the cache has it, so K and V tiles share one shared-memory
//               layout and the gather never transposes.  A block has two S buffers: S of tile t + 1 is computed
//               while the softmax works on tile t, and S of tile t + 2 goes over the P of tile t as soon as
//               O += P V of tile t has been issued (the MMAs of a thread run in order).
//   warps 10,11 gather, the two warps taking the ring entries in turn (a tensor copy costs its issuing warp
//               about 75 cycles whatever its size: one warp issuing them all was the bound of the kernel).
//               Whole tiles of whole pages come by tensor copies (TMA) of 64 dims x the page's rows, which
//               the copy unit lays out in the 128-byte-swizzled form the tensor core reads: a tile = two
//               halves of 64 dims, a half = 64 rows of 128 bytes, 16-byte chunk c of row r stored at chunk
//               c ^ (r & 7).  The last, partial tile (and page lengths the tensor copies do not suit) comes by
//               16-byte cp.async copies, row by row, into the same layout, rows past the end as zeros.  The
//               ring of ten 16 KB entries is filled in the order the issuers consume it:
//               K(0), K(1), V(0), K(2), V(1), K(3), ...
//
// Tensor memory (512 columns, one CTA per SM), per row block 256 columns: S0 | S1 (64 each) | O (128).
constexpr int kTcBlockRows = 128;                   // query rows per row block = MMA M
constexpr int kTcRows = 2 * kTcBlockRows;           // query rows per CTA
constexpr int kTcKeys = 64;                         // cache rows per tile
constexpr int kTcRing = 10;                         // ring entries: one K or V tile each
constexpr int kTcQHalfBytes = kTcBlockRows * 128;   // 64 dims of a Q tile's 128 rows
constexpr int kTcQTileBytes = 2 * kTcQHalfBytes;    // 32 KB
constexpr int kTcHalfBytes = kTcKeys * 128;         // 64 dims of a K / V tile's 64 rows
constexpr int kTcTileBytes = 2 * kTcHalfBytes;      // 16 KB
constexpr size_t kTcSmem = (size_t)2 * kTcQTileBytes + (size_t)kTcRing * kTcTileBytes + 1024;  // + alignment room
constexpr int kTcSoftmaxWarps = 8;
constexpr int kTcIssuerWarp = 8;                    // warps 8, 9: one issuer per row block
constexpr int kTcLoadWarp0 = 10;
constexpr int kTcLoadWarps = 2;                     // twelve warps in all: three per scheduler, 168 registers each
constexpr int kTcThreads = 32 * (kTcLoadWarp0 + kTcLoadWarps);
constexpr int kTcInflight = 3;                      // row-by-row entries a gather warp keeps in flight
constexpr uint32_t kColBlock = 256, kColO = 128, kTcCols = 512;
constexpr float kTcSumLimit = 256.f;                // a row sum up to here proves every P of the tile <= 2^8
constexpr float kTcRescaleAt = 8.f;                 // log2 units the maximum may run ahead of the exponents' reference

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
// Instruction descriptor, kind::f16: D fp32 (bit 4), A and B bf16 (1 at [7,10) and [10,13)) or fp16 (0), bit 16 = B is
// MN-major, N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t tc_idesc(int m, int n, bool b_mn_major, bool half) {
  return (1u << 4) | ((half ? 0u : 1u) << 7) | ((half ? 0u : 1u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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
// Tensor copy (TMA), four coordinates (dim, KV head, row of the page, page), global -> shared, completion
// counted in bytes on `bar`.  The innermost coordinate times the element size must be a multiple of 16 bytes
// (here 0 or 64 elements of 2 bytes).
__device__ __forceinline__ void tma_load_4d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// Which of 32 consecutive mask elements starting at `p` (element size `bytes`) say "visible": for byte masks a
// non-zero byte, for the additive kinds a zero of either sign.  `vec`: p's address is 16-byte aligned and all 32
// elements may be read.  Otherwise element by element, where `readable(j)`.
template <typename Readable>
__device__ __forceinline__ uint32_t mask_bits32(const unsigned char* p, int bytes, bool vec, Readable readable) {
  uint32_t bits = 0;
  if (bytes == 1) {
    uint8_t mb[32];
    if (vec) {
      const uint4 lo = *reinterpret_cast<const uint4*>(p), hi = *reinterpret_cast<const uint4*>(p + 16);
      const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int j = 0; j < 32; ++j) mb[j] = (uint8_t)(w[j >> 2] >> (8 * (j & 3)));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) mb[j] = readable(j) ? p[j] : (uint8_t)0;  // all the loads first: one trip to memory
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) bits |= (mb[j] != 0 ? 1u : 0u) << j;
  } else if (bytes == 2) {
    uint16_t mh[32];
    if (vec) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 v = reinterpret_cast<const uint4*>(p)[q];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) mh[8 * q + j] = (uint16_t)(w[j >> 1] >> (16 * (j & 1)));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) mh[j] = readable(j) ? reinterpret_cast<const uint16_t*>(p)[j] : (uint16_t)0xffff;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) bits |= ((mh[j] & 0x7fffu) == 0 ? 1u : 0u) << j;
  } else {
    uint32_t mw[32];
    if (vec) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint4 v = reinterpret_cast<const uint4*>(p)[q];
        mw[4 * q] = v.x, mw[4 * q + 1] = v.y, mw[4 * q + 2] = v.z, mw[4 * q + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) mw[j] = readable(j) ? reinterpret_cast<const uint32_t*>(p)[j] : 0xffffffffu;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) bits |= ((mw[j] & 0x7fffffffu) == 0 ? 1u : 0u) << j;
  }
  return bits;
}

// The hand-overs between the roles of this kernel are short and on the critical path: try_wait without a
// suspend-time hint (the waiting warp is parked by the hardware and comes back when the phase completes, so its
// polls do not fill the queue that the exponentials of the softmax warps pass through).  Bounded like every
// wait here.
constexpr uint32_t kTcPollLimit = 1u << 24;
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < kTcPollLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
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

template <bool kHalf, int kDim>
__global__ void __launch_bounds__(kTcThreads, 1)
    tree_attn_tc_kernel(const AttnArgs ka, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kTcRing], empty[kTcRing], s_ready[2][2], p_ready[2][2], o_done[2][2], q_ready;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const subspec_tree_attn_args& a = ka.a;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = ka.group, QL = a.q_len;
  // With splits > 1, `splits` consecutive CTAs take consecutive ranges of the cache rows for the same query rows
  // and leave unnormalised partial results, which a second kernel combines: a lone request has four KV heads'
  // worth of CTAs otherwise, each walking the whole cache.
  const int split = (int)blockIdx.x % ka.splits;
  const int row0 = ((int)blockIdx.x / ka.splits) * kTcRows;
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
  const int all_tiles = (kv_len + kTcKeys - 1) / kTcKeys;
  const int per_split = (all_tiles + ka.splits - 1) / ka.splits;
  const int tb = split * per_split;                              // this CTA's first tile
  const int ntiles = max(min(per_split, all_tiles - tb), 0);     // and how many it takes (t below counts from tb)

  if (ntiles == 0) {  // nothing to attend to: zeros, as the sum of no terms (a split: sum 0, which the merge skips)
    if (threadIdx.x < kTcRows) {
      const int row = row0 + (int)threadIdx.x, rg = row / QL, ri = row - rg * QL;
      if (rg < G && ri < nq) {
        if (ka.splits > 1) {
          float* ml = ka.part_ml + ((((size_t)b * a.num_q_heads + kvh * G + rg) * QL + ri) * ka.splits + split) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.o_batch_stride +
                             (size_t)ri * a.o_token_stride + (size_t)(kvh * G + rg) * a.o_head_stride;
          for (int c = 0; c < kDim / 2; ++c) reinterpret_cast<uint32_t*>(o)[c] = 0u;
        }
      }
    }
    return;
  }

  unsigned char* qtiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* ring = qtiles + 2 * kTcQTileBytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcRing; ++s) {
      mbar_init(&full[s], 1);  // the producing warp's one arrival (plus the bytes of its tensor copies)
      mbar_init(&empty[s], (uint32_t)nblk);  // every row block's issuer lets go of the entry
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&s_ready[k][0], 1);
      mbar_init(&s_ready[k][1], 1);
      mbar_init(&p_ready[k][0], kTcSoftmaxWarps / 2);
      mbar_init(&p_ready[k][1], kTcSoftmaxWarps / 2);
      mbar_init(&o_done[k][0], 1);
      mbar_init(&o_done[k][1], 1);
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
    {  // the two Q tiles: every softmax thread brings its own row (16 copies of 16 bytes; a row that does not
       // exist: zeros)
      const int rr = (int)threadIdx.x;  // row of the CTA; its block = rr / 128
      const int qrow = row0 + rr, qg = qrow / QL, qi = qrow - qg * QL;
      const bool okr = qg < G && qi < nq;
      const unsigned char* src = reinterpret_cast<const unsigned char*>(a.q);
      if (okr)
        src += 2 * ((size_t)b * a.q_batch_stride + (size_t)qi * a.q_token_stride + (size_t)(kvh * G + qg) * a.q_head_stride);
      unsigned char* d = qtiles + (size_t)(rr >> 7) * kTcQTileBytes + (rr & 127) * 128;
#pragma unroll
      for (int chunk = 0; chunk < kDim / 8; ++chunk)
        cp_async16(d + (chunk >> 3) * kTcQHalfBytes + (((chunk & 7) ^ (rr & 7)) << 4), src + chunk * 16, okr ? 16 : 0);
      cp_async_commit();
      cp_async_wait<0>();
      fence_async_smem();
      mbar_arrive(&q_ready);
    }
    const int blk = warp >> 2;
    const int row = row0 + (int)threadIdx.x, rg = row / QL, ri = row - rg * QL;
    const bool row_ok = rg < G && ri < nq;
    if (blk < nblk) {
      const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)blk * kColBlock;
      const uint32_t o_addr = lane_base + kColO;
      const unsigned char* mrow = a.mask + ((size_t)b * a.mask_batch_stride + (size_t)ri * a.mask_row_stride) * ka.mask_bytes;
      const float c2 = ka.scale_log2;
      float m = -INFINITY, l = 0.f;  // reference point of the exponents (in their units) and sum of this row
      bool live = true;
      for (int t = 0; t < ntiles; ++t) {
        const uint32_t s_addr = lane_base + (uint32_t)((t & 1) * kTcKeys);
        live = __all_sync(0xffffffffu, tc_wait(&s_ready[blk][t & 1], (uint32_t)(t >> 1) & 1u, abort_flag));
        if (!live) break;
        tc_fence_after();
        uint32_t ra[32], rb[32];
        tmem_ld32_async(s_addr, ra);
        tmem_ld32_async(s_addr + 32, rb);
        const int t0 = (tb + t) * kTcKeys;
        const bool need_mask = t0 + kTcKeys > prefix;  // tiles inside the prefix are visible to every row
        uint32_t vis[2] = {0xffffffffu, 0xffffffffu};
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            // sixteen bytes at a time where that stays inside the row's columns and is aligned
            const int p0 = t0 + 32 * c;
            const unsigned char* mp = mrow + (size_t)p0 * ka.mask_bytes;
            const bool vec = row_ok && p0 + 32 <= kv_len && ((reinterpret_cast<uintptr_t>(mp) & 15u) == 0);
            uint32_t bits = mask_bits32(mp, ka.mask_bytes, vec,
                                        [&](int j) { return p0 + j >= prefix && p0 + j < kv_len && row_ok; });
            if (p0 < prefix) bits |= prefix - p0 >= 32 ? 0xffffffffu : (1u << (prefix - p0)) - 1u;  // the prefix is seen
            if (p0 + 32 > kv_len) bits &= kv_len <= p0 ? 0u : (kv_len - p0 >= 32 ? 0xffffffffu : (1u << (kv_len - p0)) - 1u);
            if (!row_ok) bits = p0 >= prefix ? 0u : (prefix - p0 >= 32 ? 0xffffffffu : (1u << (prefix - p0)) - 1u);
            vis[c] = bits;
          }
        }
        tmem_wait_ld_dep(ra);
        tmem_wait_ld_dep(rb);
        // P = exp2(S c2 - u), u the reference point of the row's exponents.  (Two copies of the loop, with and
        // without the mask: inside the prefix no instruction is spent on it; scaling and sums two floats at a time.)
        uint64_t sm2[2];
        float u = m;
        auto exp_chunk = [&](auto masked, const uint32_t (&r)[32], uint32_t bits, int c) {
          const uint64_t c2p = f2_pack(c2, c2), nup = f2_pack(-u, -u);
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), c2p, nup), x0, x1);
            float p0, p1;
            if ((j & 3) == 3 || (j & 7) == 1) {
              exp2_pair_fma(x0, x1, p0, p1);  // three pairs in eight on the FMA pipe: the special-function unit's
                                               // queue is what the warps of this role stall on most
            } else {
              p0 = ex2f(x0);
              p1 = ex2f(x1);
            }
            if (decltype(masked)::value) {
              p0 = ((bits >> (2 * j)) & 1u) ? p0 : 0.f;
              p1 = ((bits >> (2 * j + 1)) & 1u) ? p1 : 0.f;
            }
            sm2[j & 1] = f2_add(sm2[j & 1], f2_pack(p0, p1));
            pk[j] = pack16<kHalf>(p0, p1);
          }
          tmem_st16(s_addr + 16 * c, pk);  // columns [16 c, 16 c + 16) <- keys [32 c, 32 c + 32)
        };
        auto row_sum = [&]() {
          float e0, e1, e2, e3;
          f2_unpack(sm2[0], e0, e1);
          f2_unpack(sm2[1], e2, e3);
          return (e0 + e1) + (e2 + e3);
        };
        // Most tiles move no reference point: try the tile against the old one first, without looking for its
        // maximum.  Every P is positive, so a row sum of at most 2^8 proves that no P went past 2^8 -- the same
        // bound the search for the maximum would have enforced -- and anything else (a larger sum, an overflow)
        // sends the warp down the careful path, which recomputes the tile from the registers it still holds.
        bool careful = t == 0 || need_mask || __any_sync(0xffffffffu, m == -INFINITY);
        float alpha = 1.f;
        if (!careful) {
          sm2[0] = sm2[1] = f2_pack(0.f, 0.f);
          exp_chunk(std::false_type{}, ra, 0u, 0);
          exp_chunk(std::false_type{}, rb, 0u, 1);
          const float ts = row_sum();
          careful = __any_sync(0xffffffffu, !(ts <= kTcSumLimit));
          if (!careful) l += ts;
        }
        if (careful) {
          // ---- the row's maximum over the tile (four chains, not one) ----
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (need_mask) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if ((vis[0] >> j) & 1u) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(ra[j]));
              if ((vis[1] >> j) & 1u) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(rb[j]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) mx[j & 3] = fmaxf(mx[j & 3], fmaxf(__uint_as_float(ra[j]), __uint_as_float(rb[j])));
          }
          const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c2;  // c2 > 0: max commutes with scaling
          // The reference point of the exponents moves only when the row's maximum has grown by more than 2^8
          // past it: between moves P reaches at most 256, which bf16 and the fp32 sums hold as well as 1, and
          // the rescaling of O (a pass over tensor memory) becomes rare instead of per tile.
          if (tmax > m + kTcRescaleAt || m == -INFINITY) {
            const float m_new = fmaxf(m, tmax);
            alpha = ex2f(m - (m_new == -INFINITY ? 0.f : m_new));  // 0 while m is -inf
            m = m_new;
          }
          u = m == -INFINITY ? 0.f : m;  // a row with nothing visible yet
          if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
            // O += P V of the tile before must have landed before O is rescaled.  The tiles complete on two
            // barriers in turn, so the phase asked for is unambiguous although most tiles never ask: of this
            // barrier's tiles all up to t - 3 are known complete (S of this tile was issued behind them) and
            // none after t - 1 can have been issued.
            live = __all_sync(0xffffffffu, tc_wait(&o_done[blk][(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1u, abort_flag));
            if (!live) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < kDim / 32; ++c) {
              uint32_t rc[32];
              tmem_ld32_async(o_addr + 32 * c, rc);
              tmem_wait_ld_dep(rc);
#pragma unroll
              for (int j = 0; j < 32; ++j) rc[j] = __float_as_uint(__uint_as_float(rc[j]) * alpha);
              tmem_st32(o_addr + 32 * c, rc);
            }
          }
          sm2[0] = sm2[1] = f2_pack(0.f, 0.f);
          if (need_mask) {
            exp_chunk(std::true_type{}, ra, vis[0], 0);
            exp_chunk(std::true_type{}, rb, vis[1], 1);
          } else {
            exp_chunk(std::false_type{}, ra, 0u, 0);
            exp_chunk(std::false_type{}, rb, 0u, 1);
          }
          l = l * alpha + row_sum();
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[blk][t & 1]);
      }
      // ---- the result: O / l ----
      if (live)
        live = __all_sync(0xffffffffu,
                          tc_wait(&o_done[blk][(ntiles - 1) & 1], (uint32_t)((ntiles - 1) >> 1) & 1u, abort_flag));
      if (live) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.o_batch_stride +
                                 (size_t)ri * a.o_token_stride + (size_t)(kvh * G + rg) * a.o_head_stride;
        const size_t prow = (((size_t)b * a.num_q_heads + kvh * G + rg) * QL + ri) * ka.splits + split;
        if (ka.splits > 1 && row_ok) {
          ka.part_ml[prow * 2] = m;
          ka.part_ml[prow * 2 + 1] = l;
        }
#pragma unroll
        for (int c = 0; c < kDim / 32; ++c) {
          uint32_t r[32];
          tmem_ld32_async(o_addr + 32 * c, r);
          tmem_wait_ld_dep(r);
          if (ka.splits > 1) {  // the unnormalised row, for the merge
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<uint4*>(ka.part_o + prow * kDim)[8 * c + j] =
                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
          } else if (row_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack16<kHalf>(__uint_as_float(r[8 * j]) * inv, __uint_as_float(r[8 * j + 1]) * inv);
              v.y = pack16<kHalf>(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv);
              v.z = pack16<kHalf>(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv);
              v.w = pack16<kHalf>(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv);
              reinterpret_cast<uint4*>(out_row)[4 * c + j] = v;
            }
          }
        }
        tc_fence_before();
      }
    }
  } else if (warp < kTcLoadWarp0) {
    // ================= MMA issue, one warp per row block: the whole warp runs the loop, one elected lane
    // issues (a thread gets a tcgen05.mma out every 50 cycles or so) =================
    const int blk = warp - kTcIssuerWarp;
    if (blk < nblk) {
      constexpr uint32_t idesc_s = tc_idesc(kTcBlockRows, kTcKeys, false, kHalf);
      constexpr uint32_t idesc_o = tc_idesc(kTcBlockRows, kDim, true, kHalf);
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0) + (uint32_t)blk * kColBlock;
      const uint32_t q_u32 = smem_u32(qtiles) + (uint32_t)blk * kTcQTileBytes, ring_u32 = smem_u32(ring);
      // S = Q K^T: 8 steps of 16 dims; a step moves 32 bytes inside a 64-dim half, 4 steps per half
      auto issue_s = [&](int kstage, int buf) {
        const uint32_t kaddr = ring_u32 + (uint32_t)kstage * kTcTileBytes;
#pragma unroll
        for (int ks = 0; ks < kDim / 16; ++ks)
          tc_mma_f16_ss(tm + (uint32_t)(buf * kTcKeys), tc_desc(q_u32 + (uint32_t)((ks >> 2) * kTcQHalfBytes + (ks & 3) * 32), 16),
                        tc_desc(kaddr + (uint32_t)((ks >> 2) * kTcHalfBytes + (ks & 3) * 32), 16), idesc_s, ks > 0 ? 1u : 0u);
      };
      // O += P V: 4 steps of 16 cache rows = 2048 bytes of the V tile each; P = the first 32 columns of S
      auto issue_pv = [&](int vstage, int buf, bool first) {
        const uint32_t vaddr = ring_u32 + (uint32_t)vstage * kTcTileBytes;
#pragma unroll
        for (int ks = 0; ks < kTcKeys / 16; ++ks)
          tc_mma_f16_ta(tm + kColO, tm + (uint32_t)(buf * kTcKeys + 8 * ks), tc_desc(vaddr + (uint32_t)(ks * 2048), kTcHalfBytes),
                        idesc_o, (!first || ks > 0) ? 1u : 0u);
      };
      TcRingPos pos;  // ring entries in the order they are consumed: K(0), K(1), V(0), K(2), V(1), ...
      bool ok = __all_sync(0xffffffffu, tc_wait(&q_ready, 0, abort_flag));
      for (int t = 0; t < min(ntiles, 2) && ok; ++t) {
        ok = __all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          issue_s(pos.s, t);
          tc_commit(&s_ready[blk][t]);
          tc_commit(&empty[pos.s]);
        }
        __syncwarp();
        pos.next();
      }
      for (int t = 0; t < ntiles && ok; ++t) {
        // O += P V(t), then S(t + 2) over the P just consumed: the MMAs of a thread run in order.  (The softmax
        // may be a tile ahead of this loop, hence two P barriers in turn, like the S and O ones.)
        ok = __all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag)) &&
             __all_sync(0xffffffffu, tc_wait(&p_ready[blk][t & 1], (uint32_t)(t >> 1) & 1u, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          issue_pv(pos.s, t & 1, t == 0);
          tc_commit(&o_done[blk][t & 1]);
          tc_commit(&empty[pos.s]);
        }
        __syncwarp();
        pos.next();
        if (t + 2 < ntiles) {
          ok = __all_sync(0xffffffffu, tc_wait(&full[pos.s], pos.ph, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_s(pos.s, t & 1);
            tc_commit(&s_ready[blk][t & 1]);
            tc_commit(&empty[pos.s]);
          }
          __syncwarp();
          pos.next();
        }
      }
    }
  } else {
    // ================= gather: the two warps take the ring entries in turn =================
    const int gw = warp - kTcLoadWarp0;
    const int chunk = lane & 15, sub = lane >> 4;  // row-by-row copies: 16 lanes per row, two rows per pass
    const uint32_t dst_half = (uint32_t)((chunk >> 3) * kTcHalfBytes);
    const unsigned char* kbase = ka.k_base + (size_t)kvh * ka.head_stride + chunk * 16;  // this lane's 16 bytes of a row
    const unsigned char* vbase = ka.v_base + (size_t)kvh * ka.head_stride + chunk * 16;
    const int* table = a.page_table + (size_t)b * a.pages_per_seq;
    TcRingPos wr;            // the entry about to be produced (by this warp or the other)
    TcRingPos q0, q1, q2;    // this warp's row-by-row entries committed and not yet handed over, oldest first
    int pending = 0;
    int n = 0;               // entries so far
    bool live = true;
    // The page a lane's tensor copy of tile t reads (lane l: page slot l / 2 of the tile, half l % 2), looked up
    // a tile ahead of its first use: the look-up is a trip to memory, and the copies of an entry must not wait
    // for one each.  -1: no copy by this lane for that tile.
    const int tj = lane >> 1, thalf = lane & 1;
    const bool tma_lane = ka.box_rows > 0 && tj * ka.box_rows < kTcKeys && thalf < kDim / 64;
    auto page_of = [&](int t) -> int {
      const int kpos = (tb + t) * kTcKeys + tj * ka.box_rows;
      if (!tma_lane || (tb + t + 1) * kTcKeys > kv_len) return -1;
      return ka.identity_table ? b : table[ka.page_shift >= 0 ? kpos >> ka.page_shift : kpos / a.page_len];
    };
    auto hand_over_oldest = [&]() {
      if (lane == 0) mbar_arrive(&full[q0.s]);
      q0 = q1;
      q1 = q2;
      --pending;
    };
    // one ring entry: the K (is_v = 0) or V (1) rows of tile t
    auto produce = [&](int is_v, int t, int page) {
      if (!live) return;
      const bool mine = (n & 1) == gw;
      if (mine && n >= kTcRing && !tc_wait(&empty[wr.s], wr.ph ^ 1u, abort_flag)) {
        live = false;
        return;
      }
      ++n;
      const TcRingPos at = wr;
      wr.next();
      if (!mine) return;
      const int t0 = (tb + t) * kTcKeys;
      if (ka.box_rows > 0 && t0 + kTcKeys <= kv_len) {
        // A whole tile of whole pages: lane 0 announces the bytes (the entry's one arrival); the first
        // 2 * (64 / box_rows) lanes issue one tensor copy each (a page's rows x 64 dims).
        if (lane == 0) mbar_expect_tx(&full[at.s], (uint32_t)(kDim / 64 * kTcHalfBytes));
        __syncwarp();
        if (tma_lane) {
          const int kpos = t0 + tj * ka.box_rows;
          const int pi = ka.page_shift >= 0 ? kpos >> ka.page_shift : kpos / a.page_len;
          if (page < 0 || page >= a.num_pages) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
            page = a.num_pages;  // outside the tensor: the copy unit fills zeros and touches no memory
          }
          const int slot = kpos - pi * a.page_len;
          tma_load_4d(ring + (size_t)at.s * kTcTileBytes + thalf * kTcHalfBytes + (size_t)tj * ka.box_rows * 128,
                      is_v ? &tmap_v : &tmap_k, thalf * 64, ka.rows_before_heads ? slot : kvh,
                      ka.rows_before_heads ? kvh : slot, page, &full[at.s]);
        }
        return;
      }
      // The last, partial tile (or a page length the tensor copies do not suit): 16-byte copies, row by row
      const unsigned char* base = is_v ? vbase : kbase;
      unsigned char* dst = ring + (size_t)at.s * kTcTileBytes + dst_half;
#pragma unroll 4
      for (int pass = 0; pass < kTcKeys / 2; ++pass) {
        const int rr = pass * 2 + sub;
        const int kpos = t0 + rr;
        const unsigned char* src = base;
        int bytes = 0;
        if (kpos < kv_len) {
          const int pi = ka.page_shift >= 0 ? kpos >> ka.page_shift : kpos / a.page_len;
          int pg = ka.identity_table ? b : table[pi];
          if (pg < 0 || pg >= a.num_pages) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
            pg = 0;
          } else {
            bytes = 16;
          }
          src = base + (size_t)pg * ka.page_stride + (size_t)(kpos - pi * a.page_len) * ka.row_stride;
        }
        if (chunk < kDim / 8)
          cp_async16(dst + rr * 128 + (((chunk & 7) ^ (rr & 7)) << 4), src, bytes);  // rows past the end: zeros
      }
      cp_async_commit();
      if (pending == 0)
        q0 = at;
      else if (pending == 1)
        q1 = at;
      else
        q2 = at;
      ++pending;
      // among tensor copies a row-by-row entry is handed over as soon as it has landed; among its like, when
      // kTcInflight of this warp's are in flight the oldest has landed
      if (ka.box_rows > 0) {
        cp_async_wait<0>();
        fence_async_smem();
        __syncwarp();
        hand_over_oldest();
      } else if (pending == kTcInflight) {
        cp_async_wait<kTcInflight - 1>();
        fence_async_smem();
        __syncwarp();
        hand_over_oldest();
      }
    };
    int pg0 = page_of(0), pg1 = page_of(1), pg2 = page_of(2);  // tiles t, t + 1, t + 2 of the loop below
    produce(0, 0, pg0);
    if (ntiles > 1) produce(0, 1, pg1);
    for (int t = 0; t < ntiles; ++t) {
      const int pg3 = page_of(t + 3);  // asked for now, used an iteration later
      produce(1, t, pg0);
      if (t + 2 < ntiles) produce(0, t + 2, pg2);
      pg0 = pg1;
      pg1 = pg2;
      pg2 = pg3;
    }
    cp_async_wait<0>();
    fence_async_smem();
    __syncwarp();
    while (pending > 0) hand_over_oldest();
  }
  __syncthreads();
  if (s_abort && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_TIMEOUT);
  if (warp == kTcIssuerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTcCols);
  }
}

// Split cache ranges: one warp per (request, query head, token) adds up the splits' unnormalised rows, each
// weighted by 2^(its reference point - the largest one), and divides by the likewise weighted sum of their sums.
template <bool kHalf, int kDim>
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnArgs ka) {
  const subspec_tree_attn_args& a = ka.a;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const long long rows = (long long)a.batch * a.num_q_heads * a.q_len;
  if (row >= rows) return;
  const int i = (int)(row % a.q_len), h = (int)((row / a.q_len) % a.num_q_heads), b = (int)(row / ((long long)a.q_len * a.num_q_heads));
  int nq = a.n_q ? a.n_q[b] : a.q_len;
  if (i >= min(max(nq, 0), a.q_len)) return;
  const float* ml = ka.part_ml + (size_t)row * ka.splits * 2;
  float mstar = -INFINITY;
  for (int s = 0; s < ka.splits; ++s)
    if (ml[2 * s + 1] > 0.f) mstar = fmaxf(mstar, ml[2 * s]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  for (int s = 0; s < ka.splits; ++s) {
    const float l = ml[2 * s + 1];
    if (!(l > 0.f)) continue;  // a split with nothing visible (or nothing at all) left no row behind
    const float w = ex2f(ml[2 * s] - mstar);
    const float4 o = lane < kDim / 4 ? reinterpret_cast<const float4*>(ka.part_o + ((size_t)row * ka.splits + s) * kDim)[lane]
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
    acc.x += w * o.x, acc.y += w * o.y, acc.z += w * o.z, acc.w += w * o.w;
    lsum += w * l;
  }
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.o_batch_stride +
                           (size_t)i * a.o_token_stride + (size_t)h * a.o_head_stride;
  if (lane < kDim / 4)
    reinterpret_cast<uint2*>(out_row)[lane] =
        make_uint2(pack16<kHalf>(acc.x * inv, acc.y * inv), pack16<kHalf>(acc.z * inv, acc.w * inv));
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
  if ((a.head_dim != 64 && a.head_dim != 128) || a.num_q_heads % a.num_kv_heads) return SUBSPEC_EUNSUPPORTED;
  const int hd = a.head_dim;
  if (a.dtype != 0 && a.dtype != SUBSPEC_BF16 && a.dtype != SUBSPEC_F16) return SUBSPEC_EINVAL;
  if (a.mask_kind != SUBSPEC_MASK_BOOL && a.mask_kind != SUBSPEC_MASK_ADD_F32 && a.mask_kind != SUBSPEC_MASK_ADD_BF16 &&
      a.mask_kind != SUBSPEC_MASK_ADD_F16)
    return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  const bool hf = a.v_cache != nullptr;  // key / value tensors of a static cache instead of the paged pool
  if (!a.q || !a.out || !a.pool || !a.kv_len || !a.mask || (!hf && !a.page_table)) return SUBSPEC_EINVAL;
  if (hf && (a.pages_per_seq != 1 || a.num_pages < a.batch || a.layer != 0 || a.kv_row_stride < hd ||
             a.kv_head_stride < 0 || a.kv_batch_stride < 0))
    return SUBSPEC_EINVAL;
  if (!(a.sm_scale > 0.0)) return SUBSPEC_EINVAL;
  AttnArgs ka;
  ka.a = a;
  ka.mask_bytes = a.mask_kind == SUBSPEC_MASK_BOOL ? 1 : (a.mask_kind == SUBSPEC_MASK_ADD_F32 ? 4 : 2);
  if (hf) {
    ka.k_base = reinterpret_cast<const unsigned char*>(a.pool);
    ka.v_base = reinterpret_cast<const unsigned char*>(a.v_cache);
    ka.page_stride = 2 * a.kv_batch_stride, ka.row_stride = 2 * a.kv_row_stride, ka.head_stride = 2 * a.kv_head_stride;
    ka.identity_table = a.page_table == nullptr;
  } else {
    const long long row_bytes = (long long)a.num_kv_heads * hd * 2, plane = (long long)a.page_len * row_bytes;
    ka.k_base = reinterpret_cast<const unsigned char*>(a.pool) + (size_t)a.layer * a.num_pages * 2 * plane;
    ka.v_base = ka.k_base + plane;
    ka.page_stride = 2 * plane, ka.row_stride = row_bytes, ka.head_stride = hd * 2;
    ka.identity_table = 0;
  }
  // 32-bit loads of query / output pairs, 16-byte copies of cache rows, mask elements at their own alignment
  if ((reinterpret_cast<uintptr_t>(a.q) & 3u) || (reinterpret_cast<uintptr_t>(a.out) & 3u) ||
      (reinterpret_cast<uintptr_t>(ka.k_base) & 15u) || (reinterpret_cast<uintptr_t>(ka.v_base) & 15u) ||
      (ka.page_stride & 15) || (ka.row_stride & 15) || (ka.head_stride & 15) || (a.q_token_stride & 1) ||
      (a.q_head_stride & 1) || (a.q_batch_stride & 1) || (a.o_token_stride & 1) || (a.o_head_stride & 1) ||
      (a.o_batch_stride & 1) || (reinterpret_cast<uintptr_t>(a.mask) & (uintptr_t)(ka.mask_bytes - 1)))
    return SUBSPEC_EUNSUPPORTED;
  ka.rows_before_heads = ka.row_stride < ka.head_stride;
  ka.splits = a.kv_splits > 1 ? a.kv_splits : 1;
  ka.part_o = nullptr, ka.part_ml = nullptr;
  if (ka.splits > 1) {
    if (!a.split_scratch || (reinterpret_cast<uintptr_t>(a.split_scratch) & 15u) || ka.splits > 1024) return SUBSPEC_EINVAL;
    if ((reinterpret_cast<uintptr_t>(a.out) & 7u) || (a.o_token_stride & 3) || (a.o_head_stride & 3) || (a.o_batch_stride & 3))
      return SUBSPEC_EUNSUPPORTED;  // the merge stores four outputs at a time
    const size_t rows = (size_t)a.batch * a.num_q_heads * a.q_len;
    ka.part_o = reinterpret_cast<float*>(a.split_scratch);
    ka.part_ml = ka.part_o + rows * ka.splits * hd;
  }
  ka.group = a.num_q_heads / a.num_kv_heads;
  ka.scale_log2 = (float)(a.sm_scale * 1.4426950408889634);
  ka.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft)
    if ((1 << sft) == a.page_len) ka.page_shift = sft;
  const cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool half = a.dtype == SUBSPEC_F16;
  auto kernel = hd == 128 ? (half ? tree_attn_tc_kernel<true, 128> : tree_attn_tc_kernel<false, 128>)
                          : (half ? tree_attn_tc_kernel<true, 64> : tree_attn_tc_kernel<false, 64>);
  const int rc = cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem));
  if (rc) return rc;
  const dim3 grid((unsigned)((ka.group * a.q_len + kTcRows - 1) / kTcRows * ka.splits), (unsigned)a.num_kv_heads,
                  (unsigned)a.batch);
  // Tensor maps of the K and of the V rows: [page][row of the page][KV head][dim] with the strides above.  A box
  // is 64 dims of box_rows consecutive rows of one page and one head; it exists when whole pages tile the 64
  // cache rows of a tile (or a page holds whole tiles) and the swizzle atom of 8 rows divides a page.
  CUtensorMap tmap_k, tmap_v;
  memset(&tmap_k, 0, sizeof(tmap_k));
  memset(&tmap_v, 0, sizeof(tmap_v));
  ka.box_rows = 0;
  int box = 0;
  if (a.page_len % 8 == 0) {
    if (a.page_len <= kTcKeys && kTcKeys % a.page_len == 0)
      box = a.page_len;
    else if (a.page_len % kTcKeys == 0)
      box = kTcKeys;
  }
  if (box && tensor_map_encoder() && ka.head_stride > 0 && ka.page_stride > 0) {
    const bool rbh = ka.rows_before_heads != 0;
    const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)(rbh ? a.page_len : a.num_kv_heads),
                                (cuuint64_t)(rbh ? a.num_kv_heads : a.page_len), (cuuint64_t)a.num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)(rbh ? ka.row_stride : ka.head_stride),
                                   (cuuint64_t)(rbh ? ka.head_stride : ka.row_stride), (cuuint64_t)ka.page_stride};
    const cuuint32_t boxdim[4] = {64, rbh ? (cuuint32_t)box : 1u, rbh ? 1u : (cuuint32_t)box, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    auto encode = [&](CUtensorMap* m, const unsigned char* base) {
      return tensor_map_encoder()(m, dt, 4, const_cast<unsigned char*>(base), dims, strides, boxdim, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    if (encode(&tmap_k, ka.k_base) && encode(&tmap_v, ka.v_base)) ka.box_rows = box;
  }
  kernel<<<grid, kTcThreads, kTcSmem, st>>>(ka, tmap_k, tmap_v);
  if (ka.splits > 1) {
    const long long rows = (long long)a.batch * a.num_q_heads * a.q_len;
    auto merge = hd == 128 ? (half ? attn_merge_kernel<true, 128> : attn_merge_kernel<false, 128>)
                           : (half ? attn_merge_kernel<true, 64> : attn_merge_kernel<false, 64>);
    merge<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(ka);
  }
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
