// Accepted-path KV compaction for sm_100a: a TMA bulk-copy gather/scatter.
//
// After a verify step only the rows of the accepted path survive.  Row
// offset + beam[i] moves to offset + i for every layer and for K and V
// (reference: KvCachePool.reorder_cache_with_offset, cache_manager.py:119-213;
// TreeStaticCache.reorder_cache_with_offset, cache_utils.py:166-208).  The
// reference clones the whole pool twice per step; here only the kept rows move.
//
// One warp-sized CTA owns one (sequence, row group): a row group is one
// (layer, K|V) plane of the paged pool (rows of heads*head_dim elements) or one
// (tensor, head) plane of the HF layout (rows of head_dim elements).  Rows are
// staged through shared memory with cp.async.bulk (global -> shared, completion
// on an mbarrier) and written back with cp.async.bulk (shared -> global, bulk
// group).  Chunks of kChunk rows are processed in ascending order; because
// beam is strictly increasing with beam[i] >= i, a destination can only alias
// the source of an element at or before it, so "read the whole chunk, then write
// it" preserves the reference's gather-then-scatter result.
#include "common.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

constexpr int kChunk = 16;        // rows staged per round
constexpr int kMaxRowBytes = 4096;

// Address of logical row `pos` of sequence b in row group g.
struct PagedAddr {
  subspec_kv_paged_args a;
  size_t row_bytes;
  __device__ __forceinline__ char* row(int b, int g, int pos, bool* ok) const {
    const int layer = g >> 1, kv = g & 1;
    const int lp = pos / a.page_len, slot = pos - lp * a.page_len;
    int page = lp;
    if (a.page_table) {
      if (lp >= a.pages_per_seq) {
        *ok = false;
        return nullptr;
      }
      page = a.page_table[(size_t)b * a.pages_per_seq + lp];
    }
    if (page < 0 || page >= a.num_pages) {
      *ok = false;
      return nullptr;
    }
    const size_t idx = (((size_t)layer * a.num_pages + page) * 2 + kv) * a.page_len + slot;
    return reinterpret_cast<char*>(a.pool) + idx * row_bytes;
  }
  __device__ __forceinline__ int groups() const { return a.layers * 2; }
  __device__ __forceinline__ int limit() const {
    return (a.page_table ? a.pages_per_seq : a.num_pages) * a.page_len;
  }
};

struct HfAddr {
  subspec_kv_hf_args a;
  size_t row_bytes;
  __device__ __forceinline__ char* row(int b, int g, int pos, bool* ok) const {
    const int t = g / a.heads, h = g - t * a.heads;
    char* base = reinterpret_cast<char*>(a.layer_ptrs[t]);
    const size_t e = (size_t)b * a.batch_stride + (size_t)h * a.head_stride + (size_t)pos * a.token_stride;
    (void)ok;
    return base + e * a.elem_bytes;
  }
  __device__ __forceinline__ int groups() const { return a.num_tensors * a.heads; }
  __device__ __forceinline__ int limit() const { return a.tokens; }
};

template <typename Addr>
__global__ void __launch_bounds__(32) kv_compact_kernel(const Addr ad, const int32_t* offset, const int32_t* n_keep,
                                                        const int64_t* beam, int max_beam,
                                                        int n_stride, uint32_t* dev_status) {
  extern __shared__ __align__(128) unsigned char stage[];
  __shared__ __align__(8) uint64_t bar;

  const int groups = ad.groups();
  const int b = blockIdx.x / groups;
  const int g = blockIdx.x - b * groups;
  const int lane = threadIdx.x;
  if (lane == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  // Launched as a programmatic dependent of whatever precedes it in the stream: when that is the verify kernel
  // (which lets its dependents go early), this grid's CTAs are resident by the time it ends, and only from
  // here on do they look at what it wrote (counts, accepted-path indices).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // (read past L1, like everything else the grid before this one wrote: this grid is resident while that one
  // still runs, so nothing it writes may be treated as read-only data)
  int n = __ldcg(n_keep + (size_t)b * n_stride);
  if (n > max_beam) {
    flag(dev_status, SUBSPEC_DEV_BAD_INDEX);
    n = max_beam;
  }
  if (n <= 0) return;
  const int off = __ldcg(offset + b);
  const int limit = ad.limit();
  const uint32_t rb = (uint32_t)ad.row_bytes;

  fence_async_smem();
  __syncwarp();

  uint32_t phase = 0;
  for (int i0 = 0; i0 < n; i0 += kChunk) {
    const int i = i0 + lane;
    bool active = lane < kChunk && i < n;
    char* src = nullptr;
    char* dst = nullptr;
    if (active) {
      const int64_t bi = __ldcg(beam + (size_t)b * max_beam + i);
      const int64_t sp = (int64_t)off + bi;
      if (bi < i || sp >= limit || off < 0) {
        flag(dev_status, SUBSPEC_DEV_BAD_INDEX);
        active = false;
      } else if (bi == i) {
        active = false;  // the row already sits where it belongs
      } else {
        bool ok = true;
        src = ad.row(b, g, (int)sp, &ok);
        dst = ad.row(b, g, off + i, &ok);
        if (!ok) {
          flag(dev_status, SUBSPEC_DEV_BAD_PAGE);
          active = false;
        }
      }
    }
    const uint32_t mask = __ballot_sync(0xffffffffu, active);
    if (mask == 0) continue;
    // the previous round's stores must have finished reading the staging buffer
    bulk_wait_read0();
    __syncwarp();
    if (lane == 0) mbar_expect_tx(&bar, rb * (uint32_t)__popc(mask));
    __syncwarp();
    if (active) bulk_g2s(stage + (size_t)lane * rb, src, rb, &bar);
    const bool done = mbar_wait_bounded(&bar, phase);
    phase ^= 1u;
    if (!done) {
      flag(dev_status, SUBSPEC_DEV_TIMEOUT);
      return;
    }
    if (active) {
      bulk_s2g(dst, stage + (size_t)lane * rb, rb);
      bulk_commit();
    }
    __syncwarp();
  }
  bulk_wait0();
}

template <typename Addr>
cudaError_t launch_compact(const Addr& ad, unsigned grid, size_t smem, cudaStream_t st, const int32_t* offset,
                           const int32_t* n, const int64_t* beam, int max_beam, int n_stride, uint32_t* status) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kv_compact_kernel<Addr>, ad, offset, n, beam, max_beam, n_stride, status);
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_kv_compact_paged(const subspec_kv_paged_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_kv_paged_args)) return SUBSPEC_EINVAL;
  const subspec_kv_paged_args& a = *args;
  if (a.batch < 0 || a.layers < 1 || a.num_pages < 1 || a.page_len < 1 || a.heads < 1 || a.head_dim < 1)
    return SUBSPEC_EINVAL;
  if (a.elem_bytes != 2 && a.elem_bytes != 4) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.pool || !a.offset || !a.n || !a.beam || a.max_beam < 1) return SUBSPEC_EINVAL;
  if (a.page_table && a.pages_per_seq < 1) return SUBSPEC_EINVAL;
  const size_t row_bytes = (size_t)a.heads * a.head_dim * a.elem_bytes;
  if (row_bytes % 16 || row_bytes > kMaxRowBytes || (reinterpret_cast<uintptr_t>(a.pool) & 15u))
    return SUBSPEC_EUNSUPPORTED;
  const int64_t grid = (int64_t)a.batch * a.layers * 2;
  if (grid > 0x7fffffffLL) return SUBSPEC_EUNSUPPORTED;
  PagedAddr ad{a, row_bytes};
  const size_t smem = row_bytes * kChunk;
  if (smem > 48 * 1024) {
    int rc = cuda_check(cudaFuncSetAttribute(kv_compact_kernel<PagedAddr>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (rc) return rc;
  }
  return cuda_check(launch_compact(ad, (unsigned)grid, smem, reinterpret_cast<cudaStream_t>(stream), a.offset, a.n,
                                   a.beam, a.max_beam, a.n_stride > 0 ? a.n_stride : 1, a.dev_status));
}

extern "C" int subspec_kv_compact_hf(const subspec_kv_hf_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_kv_hf_args)) return SUBSPEC_EINVAL;
  const subspec_kv_hf_args& a = *args;
  if (a.batch < 0 || a.num_tensors < 1 || a.heads < 1 || a.tokens < 1 || a.head_dim < 1) return SUBSPEC_EINVAL;
  if (a.elem_bytes != 2 && a.elem_bytes != 4) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.layer_ptrs || !a.offset || !a.n || !a.beam || a.max_beam < 1) return SUBSPEC_EINVAL;
  const size_t row_bytes = (size_t)a.head_dim * a.elem_bytes;
  if (row_bytes % 16 || row_bytes > kMaxRowBytes) return SUBSPEC_EUNSUPPORTED;
  if ((a.batch_stride * a.elem_bytes) % 16 || (a.head_stride * a.elem_bytes) % 16 ||
      (a.token_stride * a.elem_bytes) % 16)
    return SUBSPEC_EUNSUPPORTED;
  const int64_t grid = (int64_t)a.batch * a.num_tensors * a.heads;
  if (grid > 0x7fffffffLL) return SUBSPEC_EUNSUPPORTED;
  HfAddr ad{a, row_bytes};
  const size_t smem = row_bytes * kChunk;
  return cuda_check(launch_compact(ad, (unsigned)grid, smem, reinterpret_cast<cudaStream_t>(stream), a.offset, a.n,
                                   a.beam, a.max_beam, a.n_stride > 0 ? a.n_stride : 1, a.dev_status));
}
