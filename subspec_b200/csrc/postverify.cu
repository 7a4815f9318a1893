// What the SubSpec-v2 loop does between one verification and the next, for a batch of sequences, on the device:
//
//   re-rooting      root_ind = tree.find_child_index(last_accepted_ind, bonus_token)
//                   (specdecodes/models/generators/subspec_sd_v2.py:231-236,
//                    specdecodes/models/utils/cpu_tree.py:232-236)
//   delayed reorder hidden_indices_cache = cat(hidden_indices_cache, hidden_indices) while the bonus token keeps
//                   hitting a child of the tree; the KV reorder runs only when it misses (or the sequence has
//                   finished), with all the indices gathered since, and seq_len grows by their number
//                   (subspec_sd_v2.py:223-229, 250-262)
//   prune_to_depth  keep the nodes with depth <= max_depth in their original order
//                   (cpu_tree.py:119-173; called from _post_verify, subspec_sd_v2.py:44-45)
//
// The reference does all of it in Python between device synchronisations; here one small kernel reads the
// verify kernel's outputs where they lie and leaves what the compaction kernel and the next verification need
// (rows to keep, their offset, the next root) in device arrays.
#include <limits.h>

#include "common.cuh"

namespace subspec {
namespace {

// One thread per sequence: everything here is a handful of integers.
__global__ void post_verify_kernel(const subspec_post_verify_args a) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= a.batch) return;
  const int N = a.max_nodes;
  const int skip = a.skip_nodes ? a.skip_nodes[b] : 0;
  const int n_nodes = min(max(a.n_nodes[b], 0), N);
  // (read past L1: this grid may be resident while the verify kernel that writes these still runs)
  int L = __ldcg(a.out_meta + (size_t)b * 4);
  if (L < 0 || L > a.max_out) {
    flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
    L = min(max(L, 0), a.max_out);
  }
  const int64_t* toks = a.out_tokens + (size_t)b * a.max_out;
  const int64_t* hid = a.out_hidden + (size_t)b * a.max_out;

  // ---- re-rooting: the child of the last context that carries the bonus token ----
  int next_root = -1;
  if (L > 0) {
    const int64_t ctx = __ldcg(hid + L - 1);
    const int64_t bonus = __ldcg(toks + L - 1);
    if (ctx < 0 || ctx >= n_nodes) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_INDEX);
    } else {
      const int* coff = a.child_off + (size_t)b * (N + 1);
      const int cb = min(max(coff[ctx], 0), n_nodes), ce = min(max(coff[ctx + 1], cb), n_nodes);
      for (int e = cb; e < ce; ++e) {  // first match in list order, like the reference's loop
        const int c = a.child_idx[(size_t)b * N + e];
        if (c < 0 || c >= n_nodes) {
          flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
          continue;
        }
        if ((int64_t)a.token_ids[(size_t)b * N + c] == bonus) {
          next_root = c + skip;
          break;
        }
      }
    }
  }
  a.next_root[b] = next_root;
  const int accepted = next_root >= 0 ? 1 : 0;
  if (a.accepted) a.accepted[b] = accepted;

  // ---- delayed reorder: gather this step's hidden indices (original tree numbering) ----
  int len = a.beam_len[b];
  if (len < 0 || len > a.beam_stride) {
    flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
    len = min(max(len, 0), a.beam_stride);
  }
  int64_t* cache = a.beam_cache + (size_t)b * a.beam_stride;
  for (int i = 0; i < L; ++i) {
    if (len >= a.beam_stride) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_INDEX);  // more accepted rows than the caller made room for
      break;
    }
    cache[len++] = __ldcg(hid + i) + skip;
  }
  const bool fin = a.finished && a.finished[b];
  const bool reorder = !accepted || fin;
  const int n = reorder ? len : 0;
  a.reorder_n[b] = n;
  if (a.kv_len) {
    const int at = a.kv_len[b];
    if (a.reorder_offset) a.reorder_offset[b] = at;
    a.kv_len[b] = at + n;
  }
  a.beam_len[b] = reorder ? 0 : len;
}

// ---- prune_to_depth: one CTA per sequence ------------------------------------------------------------
constexpr int kPruneThreads = 256;

__global__ void __launch_bounds__(kPruneThreads) prune_depth_kernel(const subspec_tree_prune_depth_args a) {
  extern __shared__ int sm[];
  const int b = blockIdx.x;
  const int S = a.tree_stride;
  int n = a.n_nodes[b];
  if (n < 0 || n > S) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
    n = min(max(n, 0), S);
  }
  const int maxd = a.max_depth[b];
  int* tok = sm;            // [n] copies of the old arrays: the compaction below is in place
  int* par = tok + S;
  int* dep = par + S;
  float* prb = reinterpret_cast<float*>(dep + S);
  int* newi = reinterpret_cast<int*>(prb + S);  // [n] new index of old node i, or -1
  __shared__ int s_warp[kPruneThreads / 32];
  __shared__ int s_total;
  const size_t tb = (size_t)b * S;
  for (int i = threadIdx.x; i < n; i += kPruneThreads) {
    tok[i] = a.tokens[tb + i];
    par[i] = a.parents[tb + i];
    dep[i] = a.depths[tb + i];
    prb[i] = a.probs ? a.probs[tb + i] : 0.f;
  }
  __syncthreads();
  // new indices: an exclusive scan of the keep flags, a chunk of kPruneThreads nodes at a time
  int base = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i0 = 0; i0 < n; i0 += kPruneThreads) {
    const int i = i0 + threadIdx.x;
    const int keep = (i < n && dep[i] <= maxd) ? 1 : 0;
    int incl = keep;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (threadIdx.x == kPruneThreads - 1) s_total = before + incl;
    if (i < n) newi[i] = keep ? base + before + incl - 1 : -1;
    __syncthreads();
    base += s_total;
    __syncthreads();
  }
  const int kept = base;
  for (int i = threadIdx.x; i < n; i += kPruneThreads) {
    const int r = newi[i];
    if (r < 0) continue;
    const int p = par[i];
    int np = -1;
    if (p >= 0) {
      if (p >= n) {
        flag(a.dev_status, SUBSPEC_DEV_BAD_PARENT);
      } else {
        np = newi[p];  // a kept node's parent is shallower, hence kept
      }
    }
    a.tokens[tb + r] = tok[i];
    a.parents[tb + r] = np;
    a.depths[tb + r] = dep[i];
    if (a.probs) a.probs[tb + r] = prb[i];
    a.keep_idx[tb + r] = i;
  }
  if (threadIdx.x == 0) a.n_out[b] = kept;
  if (a.child_off) {
    // The children lists (verify's layout), filtered in place: a kept node keeps its kept children in the order
    // its list had them, as the reference's re-link loop does (cpu_tree.py:157-161).
    int* off = a.child_off + (size_t)b * (S + 1);
    int* idx = a.child_idx + tb;
    int* ooff = newi + S;      // [S + 1] the old offsets
    int* oidx = ooff + S + 1;  // [S]     the old lists
    int* cnt = tok;            // reuse: kept children per new node (the tokens have been written out)
    __syncthreads();
    for (int i = threadIdx.x; i <= n; i += kPruneThreads) ooff[i] = min(max(off[i], 0), n);
    for (int e = threadIdx.x; e < n; e += kPruneThreads) oidx[e] = idx[e];
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kPruneThreads) {
      const int r = newi[i];
      if (r < 0) continue;
      int c = 0;
      for (int e = ooff[i]; e < ooff[i + 1]; ++e) {
        const int ch = oidx[e];
        c += (ch >= 0 && ch < n && newi[ch] >= 0) ? 1 : 0;
      }
      cnt[r] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int r = 0; r < kept; ++r) {
        const int c = cnt[r];
        cnt[r] = run;
        run += c;
      }
      s_total = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kPruneThreads) {
      const int r = newi[i];
      if (r < 0) continue;
      int w = cnt[r];
      off[r] = w;
      for (int e = ooff[i]; e < ooff[i + 1]; ++e) {
        const int ch = oidx[e];
        if (ch >= 0 && ch < n && newi[ch] >= 0) idx[w++] = newi[ch];
      }
    }
    for (int r = kept + threadIdx.x; r <= S; r += kPruneThreads) off[r] = s_total;
  }
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_post_verify(const subspec_post_verify_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_post_verify_args)) return SUBSPEC_EINVAL;
  const subspec_post_verify_args& a = *args;
  if (a.batch < 0 || a.max_nodes < 1 || a.max_out < 1 || a.beam_stride < 1) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.n_nodes || !a.token_ids || !a.child_off || !a.child_idx || !a.out_tokens || !a.out_hidden || !a.out_meta ||
      !a.next_root || !a.beam_cache || !a.beam_len || !a.reorder_n)
    return SUBSPEC_EINVAL;
  const int threads = 128;
  post_verify_kernel<<<(a.batch + threads - 1) / threads, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cuda_check(cudaGetLastError());
}

extern "C" int subspec_tree_prune_depth(const subspec_tree_prune_depth_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_tree_prune_depth_args)) return SUBSPEC_EINVAL;
  const subspec_tree_prune_depth_args& a = *args;
  if (a.batch < 0 || a.tree_stride < 1) return SUBSPEC_EINVAL;
  if (a.tree_stride > 4096) return SUBSPEC_EUNSUPPORTED;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.n_nodes || !a.max_depth || !a.tokens || !a.parents || !a.depths || !a.keep_idx || !a.n_out)
    return SUBSPEC_EINVAL;
  if ((a.child_off == nullptr) != (a.child_idx == nullptr)) return SUBSPEC_EINVAL;
  const size_t smem = sizeof(int) * ((a.child_off ? 7 : 5) * (size_t)a.tree_stride + 2);
  if (smem > 48 * 1024) {
    const int rc = cuda_check(
        cudaFuncSetAttribute(prune_depth_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (rc) return rc;
  }
  prune_depth_kernel<<<a.batch, kPruneThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cuda_check(cudaGetLastError());
}
