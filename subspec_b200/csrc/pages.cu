// Page bookkeeping of the paged KV cache for a batch of requests, on the device.
//
// The reference keeps it in Python objects and CPU tensors: a free-page mask (KvCachePool.allocate /
// deallocate, specdecodes/models/utils/flashinfer/cache_manager.py:66-80), per request a page list, a length
// and a last-page fill (RequestKvCache.increment / decrement / crop and the tail of reorder_cache_with_offset,
// :237-346), and per forward the flattened page-table tensors (getKvCacheBatchPosition, :350-414).  Every
// step of a generation loop goes through them, which ties the loop to the host.  Here the same state lives in
// device arrays and one single-CTA kernel per step brings it up to date:
//
//   1. kv_len[b] <- set_len[b] (after a reorder or crop), then += add_len[b] + add_all (increment)
//   2. pages a request no longer needs go back to the pool (its page list is cut from the end)
//   3. requests that need more pages get the lowest free ones, requests in batch order (the reference's
//      allocate() takes the first free pages; with all releases of the step done first, the assignment is the
//      one the reference makes when it serves the requests in order)
//   4. kv_last_page_len, and the tensors the attention plan takes: seq_indptr, kv_page_indptr,
//      kv_page_indices, batch_indices / positions of the tokens about to be appended
#include "common.cuh"

namespace subspec {
namespace {

constexpr int kPgThreads = 1024;
constexpr int kPgWarps = kPgThreads / 32;

// Exclusive scan of one int per thread over the CTA; returns the thread's prefix, *total gets the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* s_warp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  __syncthreads();  // s_warp may still be read from a previous scan
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane];
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += o;
    }
    s_warp[lane] = wi - w;  // exclusive over warps
    if (lane == 31) *total = wi;
  }
  __syncthreads();
  return s_warp[warp] + incl - v;
}

__global__ void __launch_bounds__(kPgThreads) pages_update_kernel(const subspec_pages_args a) {
  extern __shared__ int sm[];
  __shared__ int s_warp[kPgWarps];
  __shared__ int s_total, s_free_total;
  const int B = a.batch, P = a.pages_per_seq, page_len = a.page_len;
  const int words = (a.num_pages + 31) / 32;
  int* need_more = sm;            // [B] pages each request still lacks
  int* first_rank = need_more + B;  // [B] rank (among the free pages, ascending) of the first page it gets
  int* word_rank = first_rank + B;  // [words] free pages in the words before this one

  // ---- 1, 2: new lengths; surplus pages back to the pool ----
  for (int b = threadIdx.x; b < B; b += kPgThreads) {
    int len = a.set_len ? a.set_len[b] : a.kv_len[b];
    len += (a.add_len ? a.add_len[b] : 0) + a.add_all;
    if (len < 0) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
      len = 0;
    }
    int need = (len + page_len - 1) / page_len;
    if (need > P) {  // the request's page list has no room for that many pages
      flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
      need = P;
      len = P * page_len;
    }
    int have = a.n_pages[b];
    if (have < 0 || have > P) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
      have = min(max(have, 0), P);
    }
    for (int j = need; j < have; ++j) {
      const int pg = a.page_table[(size_t)b * P + j];
      if (pg >= 0 && pg < a.num_pages)
        atomicOr(a.free_mask + (pg >> 5), 1u << (pg & 31));
      else
        flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);
    }
    if (have > need) have = need;
    a.n_pages[b] = have;
    a.kv_len[b] = len;
    a.kv_last_page_len[b] = len == 0 ? 0 : (len - 1) % page_len + 1;
    need_more[b] = need - have;
  }
  __syncthreads();

  // ---- 3: the lowest free pages, requests in batch order ----
  // rank of every request's first new page = pages wanted by the requests before it
  {
    int carry = 0;
    for (int b0 = 0; b0 < B; b0 += kPgThreads) {
      const int b = b0 + threadIdx.x;
      const int v = b < B ? need_more[b] : 0;
      const int ex = block_exclusive_scan(v, s_warp, &s_total);
      if (b < B) first_rank[b] = carry + ex;
      carry += s_total;
    }
    if (threadIdx.x == 0) s_free_total = 0;
    __syncthreads();
    // free pages before every word of the mask
    int wcarry = 0;
    for (int w0 = 0; w0 < words; w0 += kPgThreads) {
      const int w = w0 + threadIdx.x;
      uint32_t bits = w < words ? a.free_mask[w] : 0u;
      if (w == words - 1 && (a.num_pages & 31)) bits &= (1u << (a.num_pages & 31)) - 1u;  // no pages past the pool
      const int ex = block_exclusive_scan(__popc(bits), s_warp, &s_total);
      if (w < words) word_rank[w] = wcarry + ex;
      wcarry += s_total;
    }
    const int free_total = wcarry, wanted = carry;
    if (wanted > free_total && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_PAGE);  // out of cache pages
    __syncthreads();
    // every wanted page: find the word that holds the free page of its rank, then the bit
    for (int b = threadIdx.x; b < B; b += kPgThreads) {
      const int want = need_more[b];
      int have = a.n_pages[b];
      for (int j = 0; j < want; ++j) {
        const int r = first_rank[b] + j;
        if (r >= free_total) break;
        int lo = 0, hi = words - 1;  // last word whose rank is <= r
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (word_rank[mid] <= r)
            lo = mid;
          else
            hi = mid - 1;
        }
        uint32_t bits = a.free_mask[lo];
        if (lo == words - 1 && (a.num_pages & 31)) bits &= (1u << (a.num_pages & 31)) - 1u;
        int skip = r - word_rank[lo];
        while (skip-- > 0) bits &= bits - 1u;  // drop the lowest set bits
        const int bit = __ffs(bits) - 1;
        a.page_table[(size_t)b * P + have++] = lo * 32 + bit;
      }
      a.n_pages[b] = have;
    }
    __syncthreads();
    // the pages handed out are the `min(wanted, free_total)` lowest free ones: clear them word by word
    const int given = min(wanted, free_total);
    for (int w = threadIdx.x; w < words; w += kPgThreads) {
      uint32_t bits = a.free_mask[w];
      uint32_t valid = bits;
      if (w == words - 1 && (a.num_pages & 31)) valid &= (1u << (a.num_pages & 31)) - 1u;
      int take = min(max(given - word_rank[w], 0), __popc(valid));
      while (take-- > 0) {
        const uint32_t low = valid & (0u - valid);
        valid ^= low;
        bits ^= low;
      }
      a.free_mask[w] = bits;
    }
  }
  __syncthreads();

  // ---- 4: what the attention plan takes ----
  if (a.kv_page_indptr) {
    int pcarry = 0, scarry = 0;
    for (int b0 = 0; b0 < B; b0 += kPgThreads) {
      const int b = b0 + threadIdx.x;
      const int np = b < B ? a.n_pages[b] : 0;
      int app = 0;
      if (b < B) app = a.mode == SUBSPEC_PAGES_PREFILL ? a.kv_len[b] : (a.mode == SUBSPEC_PAGES_DECODE ? 1 : a.tree_tokens);
      const int pex = block_exclusive_scan(np, s_warp, &s_total);
      const int ptot = s_total;
      const int sex = block_exclusive_scan(app, s_warp, &s_total);
      if (b < B) {
        a.kv_page_indptr[b] = pcarry + pex;
        if (a.seq_indptr) a.seq_indptr[b] = scarry + sex;
        if (a.kv_page_indices)
          for (int j = 0; j < np; ++j) a.kv_page_indices[pcarry + pex + j] = a.page_table[(size_t)b * P + j];
        if (a.batch_indices && a.positions) {
          const int at = a.kv_len[b] - app;  // where the request's appended tokens start
          for (int j = 0; j < app && scarry + sex + j < a.max_append; ++j) {
            a.batch_indices[scarry + sex + j] = b;
            a.positions[scarry + sex + j] = at + j;
          }
        }
      }
      pcarry += ptot;
      scarry += s_total;
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      a.kv_page_indptr[B] = pcarry;
      if (a.seq_indptr) a.seq_indptr[B] = scarry;
    }
  }
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_pages_update(const subspec_pages_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_pages_args)) return SUBSPEC_EINVAL;
  const subspec_pages_args& a = *args;
  if (a.batch < 0 || a.num_pages < 1 || a.page_len < 1 || a.pages_per_seq < 1) return SUBSPEC_EINVAL;
  if (a.mode != SUBSPEC_PAGES_PREFILL && a.mode != SUBSPEC_PAGES_DECODE && a.mode != SUBSPEC_PAGES_TREE)
    return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.free_mask || !a.page_table || !a.n_pages || !a.kv_len || !a.kv_last_page_len) return SUBSPEC_EINVAL;
  if ((a.batch_indices == nullptr) != (a.positions == nullptr)) return SUBSPEC_EINVAL;
  const size_t words = ((size_t)a.num_pages + 31) / 32;
  const size_t smem = sizeof(int) * (2 * (size_t)a.batch + words);
  if (smem > 200 * 1024) return SUBSPEC_EUNSUPPORTED;
  if (smem > 48 * 1024) {
    const int rc = cuda_check(
        cudaFuncSetAttribute(pages_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (rc) return rc;
  }
  pages_update_kernel<<<1, kPgThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cuda_check(cudaGetLastError());
}
