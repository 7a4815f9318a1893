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

#include "common.cuh"

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

struct AttnArgs {
  subspec_tree_attn_args a;
  int group;        // query heads per KV head
  float scale_log2; // sm_scale * log2(e)
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
    for (int nt = 0; nt < kTileKV / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      // one x4 load = the K fragments of two k-steps: lanes 0-7 / 8-15 / 16-23 / 24-31 address cache rows
      // nt*8 + 0..7 at dims 32 j + 0 / 8 / 16 / 24
      const __nv_bfloat16* krow = Ks + (size_t)(nt * 8 + (lane & 7)) * kRowElems + ((lane >> 3) << 3);
#pragma unroll
      for (int j = 0; j < kD / 32; ++j) {
        uint32_t kf[4];
        ldmatrix_x4(kf, krow + j * 32);
        mma_bf16(s[nt], qf[2 * j], kf[0], kf[1]);
        mma_bf16(s[nt], qf[2 * j + 1], kf[2], kf[3]);
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
#pragma unroll
    for (int ks = 0; ks < kTileKV / 16; ++ks) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
      // lanes 0-7 / 8-15 address cache rows ks*16 + 0..7 / 8..15 of dims [16 j, 16 j + 8), lanes 16-31 the same
      // rows of dims [16 j + 8, 16 j + 16): one x4 load feeds two n-tiles
      const __nv_bfloat16* vrow = Vs + (size_t)(ks * 16 + (lane & 15)) * kRowElems + ((lane >> 4) << 3);
#pragma unroll
      for (int j = 0; j < kD / 16; ++j) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vrow + j * 16);
        mma_bf16(o[2 * j], pf, vf[0], vf[1]);
        mma_bf16(o[2 * j + 1], pf, vf[2], vf[3]);
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
  int rc = cuda_check(
      cudaFuncSetAttribute(tree_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem));
  if (rc) return rc;
  const dim3 grid((unsigned)((ka.group * a.q_len + kRowsPerCta - 1) / kRowsPerCta), (unsigned)a.num_kv_heads,
                  (unsigned)a.batch);
  tree_attn_kernel<<<grid, kAttnThreads, kAttnSmem, reinterpret_cast<cudaStream_t>(stream)>>>(ka);
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
