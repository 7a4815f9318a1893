// Draft-tree expansion for sm_100a: fused softmax + global top-k over leaves x vocab, and the
// tree finaliser (prune to the best n nodes, renumber, ancestor mask, position ids, children CSR).
//
// Reference semantics (specdecodes/models/draft_models/base.py:281-305, classic_sd.py:10-16):
//   probs  = softmax(logits / T)                       in the model dtype
//   score  = probs[l, v] * parent_probs[l]             in the model dtype
//   top-k over the flattened [leaves * vocab] scores, sorted descending;
//   parent = idx // vocab, token = idx % vocab.
// The reference materialises the scores (a full-size write and read) and runs a generic top-k
// over ~2M candidates per sequence.  Here each [vocab] row is streamed once: per row the k best
// logits (value desc, index asc) and the softmax denominator; the last CTA of a sequence turns the
// leaves * k survivors into scores with the reference's rounding (probability rounded to the
// dtype, product rounded to the dtype) and keeps the k best (score desc, flat index asc).  Scores
// are monotone in the logit within a row, so the survivors contain the true top-k values.
//
// Tree finaliser: Tree.add_nodes numbering (cpu_tree.py:87-117), prune_to_top_n (:175-215),
// create_attention_mask (:263-286), position ids = depth + offset (classic_sd.py:73-75).
#include <limits.h>
#include <math.h>

#include "common.cuh"
#include "mask.cuh"

namespace subspec {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;
constexpr int kMaxK = 32;
constexpr int kMaxRowSplits = 16;   // slices a row may be cut into when a launch has few rows
constexpr int kPrefetchAhead = 6;  // iterations (16 KB each) a row's L2 prefetch runs ahead of its loads
constexpr int kQueue = 256;  // per-warp candidate queue: one 16-byte vector per lane, 8 elements each

struct Cand {
  float v;
  int id;
};
__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
  return av > bv || (av == bv && ai < bi);
}

// A warp-wide list of the k best (value desc, index asc): lane i holds entry i.
struct WarpTopK {
  float v;
  int id;
  int k;
  __device__ __forceinline__ void init(int k_) {
    k = k_;
    v = -INFINITY;
    id = INT_MAX;
  }
  __device__ __forceinline__ float kth_value() const { return __shfl_sync(0xffffffffu, v, k - 1); }
  __device__ __forceinline__ float value_at(int j) const { return __shfl_sync(0xffffffffu, v, j); }
  // All lanes call with the same candidate.
  __device__ __forceinline__ void insert(float cv, int cid) {
    const int lane = threadIdx.x & 31;
    const uint32_t ahead = __ballot_sync(0xffffffffu, lane < k && better(v, id, cv, cid));
    const int pos = __popc(ahead);
    if (pos >= k) return;
    const float pv = __shfl_up_sync(0xffffffffu, v, 1);
    const int pi = __shfl_up_sync(0xffffffffu, id, 1);
    if (lane > pos) {
      v = pv;
      id = pi;
    } else if (lane == pos) {
      v = cv;
      id = cid;
    }
    if (lane >= k) {
      v = -INFINITY;
      id = INT_MAX;
    }
  }
};

// k-th largest (k = 1..32) of the 32 lane values: bitonic sort across the warp, descending.
__device__ __forceinline__ float warp_kth_largest(float v, int k) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const float o = __shfl_xor_sync(0xffffffffu, v, stride);
      const bool desc = (lane & size) == 0;       // direction of this bitonic block
      const bool lower = (lane & stride) == 0;    // this lane keeps the "first" element of the pair
      v = (desc == lower) ? fmaxf(v, o) : fminf(v, o);
    }
  }
  return __shfl_sync(0xffffffffu, v, k - 1);
}

// The k best (value descending, index ascending) of n candidates, by the whole CTA: every candidate counts
// the candidates that beat it and, if fewer than k do, is the result's entry of that rank.  n^2 compares
// spread over the CTA's threads, against one warp inserting the candidates one after the other, each insert
// a chain of dependent shuffles: 128 to 256 candidates took that warp 11 us, three times per step.
// get(i) returns candidate i (id INT_MAX = empty); out[0..k) in shared memory; ends with a CTA barrier.
template <typename Get>
__device__ __forceinline__ void cta_topk(int n, int k, Get&& get, Cand* out) {
  for (int i = threadIdx.x; i < k; i += blockDim.x) out[i] = Cand{-INFINITY, INT_MAX};
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const Cand me = get(i);
    if (me.id == INT_MAX) continue;
    int rank = 0;
#pragma unroll 8  // the loads of a group go out together: one after the other they are the whole cost
    for (int j = 0; j < n; ++j) {
      const Cand o = get(j);
      rank += (o.id != INT_MAX && better(o.v, o.id, me.v, me.id)) ? 1 : 0;
    }
    if (rank < k) out[rank] = me;
  }
  __syncthreads();
}

struct RowOut {  // per (sequence, leaf) row, in scratch
  float c, s;    // softmax shift (log2 domain) and denominator; unused for probabilities in
};

struct KArgs {
  subspec_expand_args a;
  int* ticket;     // [batch]
  RowOut* rowout;  // [batch * leaves]
  Cand* rowtop;    // [batch * leaves * k]
  float kT;        // scale inside 2^(x * kT - c): log2(e) / temperature, or log2(e) when the logits are pre-scaled
  float invT, T;   // 16-bit dtypes with temperature != 1: the reference rounds logits / T to the dtype first
  int prescale;
  int vec_ok;
  // few rows: every row is cut into `splits` slices, one CTA each; the slices' lists and softmax sums meet
  // in scratch behind a ticket per row, and the last slice to arrive carries on as the row's CTA
  int splits;
  int64_t dm_row_stride, dm_seq_stride;  // draft-side mask geometry in elements, defaults resolved
  int* rowticket;   // [batch * leaves]
  RowOut* partout;  // [batch * leaves * splits]
  Cand* parttop;    // [batch * leaves * splits * k]
};

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& q, float (&x)[4]) {
    x[0] = __uint_as_float(q.x);
    x[1] = __uint_as_float(q.y);
    x[2] = __uint_as_float(q.z);
    x[3] = __uint_as_float(q.w);
  }
  static __device__ __forceinline__ float vmax(const uint4& q) {
    return fmaxf(fmaxf(__uint_as_float(q.x), __uint_as_float(q.y)), fmaxf(__uint_as_float(q.z), __uint_as_float(q.w)));
  }
  static __device__ __forceinline__ float round_to(float x) { return x; }
  static __device__ __forceinline__ float load(const void* p, size_t i) { return reinterpret_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void store(void* p, size_t i, float x) { reinterpret_cast<float*>(p)[i] = x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& q, float (&x)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ float vmax(const uint4& q) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    const __nv_bfloat162 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(__low2float(m), __high2float(m));
  }
  static __device__ __forceinline__ float round_to(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ float load(const void* p, size_t i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ void store(void* p, size_t i, float x) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  }
};
template <>
struct Elem<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& q, float (&x)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float vmax(const uint4& q) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
    const __half2 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(__low2float(m), __high2float(m));
  }
  static __device__ __forceinline__ float round_to(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ float load(const void* p, size_t i) {
    return __half2float(reinterpret_cast<const __half*>(p)[i]);
  }
  static __device__ __forceinline__ void store(void* p, size_t i, float x) {
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
  }
};

// Softmax denominator with a movable shift, packed lanes (see verify.cu for the reasoning).
struct SoftAcc {
  uint64_t s2, k2, nc2;
  float c, k;
  __device__ __forceinline__ void init(float k_) {
    k = k_;
    k2 = f2_pack(k_, k_);
    c = -INFINITY;
    nc2 = f2_pack(INFINITY, INFINITY);
    s2 = f2_pack(0.f, 0.f);
  }
  __device__ __forceinline__ void ensure(float m) {  // m: a maximum met so far
    const float y = fmaf(m, k, -c);
    if (y > 64.f) {
      const float cn = m * k;
      if (c != -INFINITY) {
        const float f = ex2f(c - cn);
        float s0, s1;
        f2_unpack(s2, s0, s1);
        s2 = f2_pack(s0 * f, s1 * f);
      }
      c = cn;
      nc2 = f2_pack(-cn, -cn);
    }
  }
  __device__ __forceinline__ void add_pair(float x0, float x1) {
    float y0, y1;
    f2_unpack(f2_fma(f2_pack(x0, x1), k2, nc2), y0, y1);
    s2 = f2_add(s2, f2_pack(ex2f(y0), ex2f(y1)));
  }
  __device__ __forceinline__ void add_one(float x) {
    float s0, s1;
    f2_unpack(s2, s0, s1);
    s0 += ex2f(fmaf(fmaxf(x, -1.0e30f), k, -c));
    s2 = f2_pack(s0, s1);
  }
  __device__ __forceinline__ float sum() const {
    float s0, s1;
    f2_unpack(s2, s0, s1);
    return s0 + s1;
  }
};

__device__ __forceinline__ void combine_soft(float& c, float& s, float oc, float os) {
  const float cn = fmaxf(c, oc);
  float r = 0.f;
  if (c != -INFINITY) r += s * ex2f(c - cn);
  if (oc != -INFINITY) r += os * ex2f(oc - cn);
  c = cn;
  s = r;
}

// ---- per-row streaming kernel ----------------------------------------------------------------
template <typename T, int KIND>
__global__ void __launch_bounds__(kThreads, 4) expand_rows_kernel(const KArgs ka) {
  __shared__ Cand s_queue[kWarps][kQueue];
  __shared__ int s_qn[kWarps];
  __shared__ float s_pub[kWarps];  // each warp's j-th best value: min over warps bounds the k-th best of the row
  __shared__ Cand s_cand[kMaxK * kMaxK];  // the candidates of a merge across slices or across a sequence's rows
  __shared__ Cand s_best[kMaxK];
  __shared__ float s_c[kWarps], s_s[kWarps];
  __shared__ int s_flag;

  const subspec_expand_args& a = ka.a;
  const int L = a.leaves, V = a.vocab, k = a.k;
  const int S = ka.splits;
  const int row = blockIdx.x / S;
  const int split = blockIdx.x - row * S;
  const int b = row / L;
  const T* rowp = reinterpret_cast<const T*>(a.scores) + (size_t)b * a.seq_stride + (size_t)(row - b * L) * a.row_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int VN = Elem<T>::N;
  const int jpub = (k + kWarps - 1) / kWarps;  // kWarps * jpub >= k distinct elements

  WarpTopK top;
  top.init(k);
  SoftAcc soft;
  soft.init(ka.kT);
  if (lane == 0) {
    s_qn[warp] = 0;
    s_pub[warp] = -INFINITY;
  }
  __syncthreads();
  float thr = -INFINITY;

  const int nvec = ka.vec_ok ? V / VN : 0;
  // this CTA's slice of the row's vectors (the whole row when S == 1); the scalar tail goes with the last slice
  const int vec_per = (nvec + S - 1) / S;
  const int v0 = min(split * vec_per, nvec), v1 = min(v0 + vec_per, nvec);
  const uint4* vp = reinterpret_cast<const uint4*>(rowp);
  // One thread asks L2 for the row a few iterations ahead of the loads (bulk prefetch, no registers, no
  // barrier): a thread has its four loads in flight only while it waits for them, which alone leaves the
  // SM far short of the bytes in flight that its share of the HBM bandwidth needs.
  constexpr int kIterVecs = kThreads * kUnroll;  // 16 KB of the row per iteration
  auto prefetch_iter = [&](int it) {
    const int p0 = v0 + it * kIterVecs;
    if (p0 < v1) l2_prefetch(vp + p0, (uint32_t)(min(kIterVecs, v1 - p0) * 16));
  };
  if (threadIdx.x == 0)
    for (int it = 0; it < kPrefetchAhead; ++it) prefetch_iter(it);
  for (int i0 = v0; i0 < v1; i0 += kThreads * kUnroll) {
    if (threadIdx.x == 0) prefetch_iter((i0 - v0) / kIterVecs + kPrefetchAhead);
    // refresh the threshold: own k-th best, and the bound the other warps have published
    {
      float t = s_pub[0];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) t = fminf(t, s_pub[w]);
      thr = fmaxf(top.kth_value(), t);
    }
    uint4 q[kUnroll];
    float m[kUnroll];
    bool have[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const int i = i0 + threadIdx.x + j * kThreads;
      have[j] = i < v1;
      if (have[j]) {
        q[j] = ld_stream_u4(vp + i);
        m[j] = Elem<T>::vmax(q[j]);
      } else {
        q[j] = make_uint4(0, 0, 0, 0);
        m[j] = -INFINITY;
      }
    }
    const float gm = fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
    if (i0 == v0) {
      // First group: the k-th largest of the 32 lane maxima is k distinct elements' worth of evidence that the
      // warp's k-th best is at least that, which keeps the first round of candidates to a few dozen.
      thr = fmaxf(thr, warp_kth_largest(gm, k));
    }
    if (KIND == SUBSPEC_IN_LOGITS) {
      // With pre-scaling the sums run over round(x / T); the multiply by 1 / T used here can differ from the
      // division by one fp32 ulp before rounding, which the k survivors (recomputed exactly below) never see.
      soft.ensure(ka.prescale ? Elem<T>::round_to(gm * ka.invT) : gm);
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        if (!have[j]) continue;
        float x[VN];
        Elem<T>::unpack(q[j], x);
        if (ka.prescale) {
#pragma unroll
          for (int e = 0; e < VN; ++e) x[e] = Elem<T>::round_to(x[e] * ka.invT);
        }
#pragma unroll
        for (int e = 0; e < VN; e += 2) soft.add_pair(x[e], x[e + 1]);
      }
    }
    // candidates: rare after the first groups
    if (__ballot_sync(0xffffffffu, gm >= thr)) {
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        if (!__ballot_sync(0xffffffffu, m[j] >= thr)) continue;
        if (m[j] >= thr) {
          float x[VN];
          Elem<T>::unpack(q[j], x);
          const int base = (i0 + threadIdx.x + j * kThreads) * VN;
#pragma unroll
          for (int e = 0; e < VN; ++e)
            if (x[e] >= thr) {
              const int p = atomicAdd(&s_qn[warp], 1);
              s_queue[warp][p] = Cand{x[e], base + e};
            }
        }
        __syncwarp();
        const int qn = s_qn[warp];
        for (int i = 0; i < qn; ++i) {
          const Cand cnd = s_queue[warp][i];
          top.insert(cnd.v, cnd.id);
        }
        const float pub = top.value_at(jpub - 1);
        thr = fmaxf(thr, top.kth_value());
        __syncwarp();
        if (lane == 0) {
          s_qn[warp] = 0;
          s_pub[warp] = pub;
        }
        __syncwarp();
      }
    }
  }
  // scalar tail (and whole unaligned rows): lane by lane through the same queue
  for (int i0 = (split == S - 1 ? nvec * VN : V); i0 < V; i0 += kThreads) {
    const int i = i0 + threadIdx.x;
    float x = -INFINITY;
    if (i < V) x = to_f32<T>(rowp[i]);
    if (KIND == SUBSPEC_IN_LOGITS && i < V) {
      const float xs = ka.prescale ? Elem<T>::round_to(x * ka.invT) : x;
      soft.ensure(fmaxf(xs, -1.0e30f));
      soft.add_one(xs);
    }
    thr = fmaxf(thr, top.kth_value());
    if (__ballot_sync(0xffffffffu, i < V && x >= thr)) {
      if (i < V && x >= thr) {
        const int p = atomicAdd(&s_qn[warp], 1);
        s_queue[warp][p] = Cand{x, i};
      }
      __syncwarp();
      const int qn = s_qn[warp];
      for (int t = 0; t < qn; ++t) {
        const Cand cnd = s_queue[warp][t];
        top.insert(cnd.v, cnd.id);
      }
      __syncwarp();
      if (lane == 0) s_qn[warp] = 0;
      __syncwarp();
    }
  }

  // ---- merge the warps' lists and softmax sums ----
  if (lane < k) s_cand[warp * k + lane] = Cand{top.v, top.id};  // the warps' lists, back to back
  {
    float c = soft.c, s = soft.sum();
    if (KIND != SUBSPEC_IN_LOGITS) {
      c = 0.f;
      s = 1.f;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float oc = __shfl_xor_sync(0xffffffffu, c, off);
      const float os = __shfl_xor_sync(0xffffffffu, s, off);
      combine_soft(c, s, oc, os);
    }
    if (lane == 0) {
      s_c[warp] = c;
      s_s[warp] = s;
    }
  }
  __syncthreads();
  // ---- the k best of the warps' lists: every candidate counts who beats it (see cta_topk) ----
  cta_topk(
      kWarps * k, k, [&](int i) { return s_cand[i]; }, s_best);
  Cand* top_dst = S > 1 ? ka.parttop + ((size_t)row * S + split) * k : ka.rowtop + (size_t)row * k;
  RowOut* out_dst = S > 1 ? ka.partout + (size_t)row * S + split : ka.rowout + row;
  if (threadIdx.x < k) top_dst[threadIdx.x] = s_best[threadIdx.x];
  if (threadIdx.x == 0) {
    float c = s_c[0], sm = s_s[0];
    for (int w = 1; w < kWarps; ++w) combine_soft(c, sm, s_c[w], s_s[w]);
    if (KIND != SUBSPEC_IN_LOGITS) {
      c = 0.f;
      sm = 1.f;
    }
    *out_dst = RowOut{c, sm};
  }
  if (S > 1) {
    // ---- the row's slices meet: the last one to arrive folds all S lists and sums into the row's ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_flag = (atomicAdd(ka.rowticket + row, 1) == S - 1);
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
    const int total = S * k;  // <= kMaxRowSplits * kMaxK
    const volatile Cand* src = ka.parttop + (size_t)row * S * k;
    for (int t = threadIdx.x; t < total; t += kThreads) s_cand[t] = Cand{src[t].v, src[t].id};
    __syncthreads();
    cta_topk(
        total, k, [&](int i) { return s_cand[i]; }, s_best);
    if (threadIdx.x < k) ka.rowtop[(size_t)row * k + threadIdx.x] = s_best[threadIdx.x];
    if (threadIdx.x == 0) {
      const volatile RowOut* po = ka.partout + (size_t)row * S;
      float c = po[0].c, sm = po[0].s;
      for (int i = 1; i < S; ++i) combine_soft(c, sm, po[i].c, po[i].s);
      ka.rowout[row] = RowOut{c, sm};
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_flag = (atomicAdd(ka.ticket + b, 1) == L - 1);
  __syncthreads();
  if (!s_flag) return;
  __threadfence();

  // ---- the last CTA of the sequence: scores with the reference's rounding, global top-k ----
  {
    const int total = L * k;  // <= kMaxK * kMaxK
    for (int t = threadIdx.x; t < total; t += kThreads) {
      const int l = t / k;
      const volatile Cand* src = ka.rowtop + ((size_t)b * L + l) * k + (t - l * k);
      const float xv = src->v;
      const int xi = src->id;
      Cand out{-INFINITY, INT_MAX};
      if (xi != INT_MAX) {
        const volatile RowOut* ro = ka.rowout + (size_t)b * L + l;
        float p = xv;
        if (KIND == SUBSPEC_IN_LOGITS) {
          // The survivors' probabilities in double precision: a 16-bit dtype rounds them next, and an error of
          // 1e-6 in fp32 arithmetic on an exponent near 20 would land on the other side of a rounding boundary
          // a few times per thousand values; what is left is the error of the fp32 denominator (~1e-7).
          const float xs = ka.prescale ? Elem<T>::round_to(__fdiv_rn(xv, ka.T)) : xv;
          p = (float)(exp2((double)xs * (double)ka.kT - (double)ro->c) / (double)ro->s);
        }
        p = Elem<T>::round_to(p);
        const float pp = a.parent_probs ? Elem<T>::load(a.parent_probs, (size_t)b * L + l) : 1.f;
        out = Cand{Elem<T>::round_to(p * pp), l * V + xi};
      }
      s_cand[t] = out;
    }
    __syncthreads();
    cta_topk(
        total, k, [&](int i) { return s_cand[i]; }, s_best);
    if (threadIdx.x < k) {
      const int lane_k = threadIdx.x;
      const Cand best = s_best[lane_k];
      const size_t o = (size_t)b * k + lane_k;
      const int l = best.id == INT_MAX ? 0 : best.id / V;
      const int tok = best.id == INT_MAX ? 0 : best.id - l * V;
      a.out_tokens[o] = tok;
      a.out_parents[o] = l;
      Elem<T>::store(a.out_probs, o, best.v);
      if (a.tree_tokens) {  // Tree.add_nodes numbering: level d occupies 1 + d k ... d k + k
        const size_t node = (size_t)b * a.tree_stride + 1 + (size_t)a.level * k + lane_k;
        a.tree_tokens[node] = tok;
        a.tree_parents[node] = a.level == 0 ? 0 : 1 + (a.level - 1) * k + l;
        a.tree_probs[node] = best.v;
        a.tree_depths[node] = a.level + 1;
      }
    }
    if (a.draft_mask) {
      // ---- the new level's draft-side mask rows and position ids (TreeMaskCache, base.py:93-117) ----
      const MaskFmt mf = mask_fmt(a.draft_mask_kind);
      const int64_t prefix = a.prefix_len ? (int64_t)a.prefix_len[b] : 0;
      const int64_t rs = ka.dm_row_stride;
      uint8_t* mbase = reinterpret_cast<uint8_t*>(a.draft_mask) + (size_t)b * ka.dm_seq_stride * mf.esz;
      const bool ok = prefix >= 0 && prefix + (int64_t)(a.level + 1) * k <= a.draft_mask_cols;
      if (!ok && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_INDEX);
      if (ok) mask_fill_rows(mbase, rs, k, a.draft_mask_cols, prefix, mf);
      __syncthreads();
      if (threadIdx.x < k) {
        const int i = threadIdx.x;
        if (a.draft_position_ids) a.draft_position_ids[(size_t)b * k + i] = prefix + a.level;
        if (ok) {
          uint8_t* mrow = mbase + (size_t)i * rs * mf.esz;
          const Cand best = s_best[i];
          const int l = best.id == INT_MAX ? 0 : best.id / V;
          int node = 1 + a.level * k + i;
          mask_store(mrow, prefix + node - 1, mf, true);
          node = a.level == 0 ? 0 : 1 + (a.level - 1) * k + l;  // this level's parents are not read back
          const int32_t* tp = a.tree_parents + (size_t)b * a.tree_stride;
          for (int hop = 0; hop < a.level && node > 0; ++hop) {  // one ancestor per earlier level, then the root
            mask_store(mrow, prefix + node - 1, mf, true);
            const int up = tp[node];
            node = (up >= 0 && up < node) ? up : 0;
          }
        }
      }
    }
  }
}

// ---- tree finaliser ------------------------------------------------------------------------------
struct FinArgs {
  subspec_tree_finalize_args a;
  int64_t cols, row_stride, seq_stride;  // mask geometry in elements, defaults resolved on the host
};

__global__ void __launch_bounds__(256) tree_finalize_kernel(const FinArgs fa) {
  extern __shared__ int sm[];
  const subspec_tree_finalize_args& a = fa.a;
  const int b = blockIdx.x;
  const int n = a.n_nodes, keep = min(a.keep, a.n_nodes);
  const bool identity = a.n_nodes <= a.keep;  // nothing to prune: the reference leaves the tree alone (cpu_tree.py:176-177)
  int* rank = sm;            // [n] rank of old node i (0 = best)
  int* old_of = rank + n;    // [keep]
  int* par = old_of + keep;  // [n] parents, old numbering (a copy: the loops below read them many times)
  int* coff = par + n;       // [keep + 1] children CSR offsets, new numbering
  const size_t tb = (size_t)b * a.tree_stride;
  const float* prob = a.tree_probs + tb;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int p = i == 0 ? -1 : a.tree_parents[tb + i];
    if (i > 0 && (p < 0 || p >= i)) {  // expansion appends children behind their parents; anything else could loop
      flag(a.dev_status, SUBSPEC_DEV_BAD_PARENT);
      p = -1;
    }
    par[i] = p;
  }

  // rank by (cumulative probability desc, index asc); the root carries probability 1, NaN counts as -inf
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int r = i;
    if (!identity) {
      float pi = i == 0 ? 1.f : prob[i];
      pi = pi == pi ? pi : -INFINITY;
      r = 0;
      for (int j = 0; j < n; ++j) {
        float pj = j == 0 ? 1.f : prob[j];
        pj = pj == pj ? pj : -INFINITY;
        r += (pj > pi || (pj == pi && j < i)) ? 1 : 0;
      }
    }
    rank[i] = r;
    if (r < keep) old_of[r] = i;
  }
  // mask background: prefix columns "may attend", everything behind "masked"
  const MaskFmt mf = mask_fmt(a.mask_kind);
  const int skip = min(max(a.skip_nodes, 0), a.keep);
  int64_t prefix = a.prefix_length ? (int64_t)a.prefix_length[b] : 0;
  bool mask_ok = true;
  if (prefix < 0 || prefix + a.keep > fa.cols) {
    if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_INDEX);
    mask_ok = false;
  }
  uint8_t* mbase = reinterpret_cast<uint8_t*>(a.mask) + (size_t)b * fa.seq_stride * mf.esz;
  if (mask_ok) mask_fill_rows(mbase, fa.row_stride, a.keep - skip, fa.cols, prefix, mf);
  __syncthreads();
  const size_t ob = (size_t)b * a.keep;
  for (int r = threadIdx.x; r < keep; r += blockDim.x) {
    const int o = old_of[r];
    const int p = par[o];
    const int np = (p >= 0 && rank[p] < keep) ? rank[p] : -1;
    a.keep_idx[ob + r] = o;
    a.tokens[ob + r] = a.tree_tokens[tb + o];
    a.parents[ob + r] = np;
    const int d = o == 0 ? 0 : a.tree_depths[tb + o];
    a.depths[ob + r] = d;
    a.probs[ob + r] = o == 0 ? 1.f : prob[o];
    a.position_ids[ob + r] = (int64_t)d + (a.position_offset ? a.position_offset[b] : 0);
    // ancestor-or-self row (parents are smaller than their children, so the walk ends within n steps)
    if (mask_ok && r >= skip) {
      uint8_t* mrow = mbase + (size_t)(r - skip) * fa.row_stride * mf.esz;
      int cur = o, guard = 0;
      while (cur >= 0 && guard <= n) {
        if (rank[cur] < keep) mask_store(mrow, prefix + rank[cur], mf, true);
        cur = par[cur];
        ++guard;
      }
    }
  }
  for (int r = keep + threadIdx.x; r < a.keep; r += blockDim.x) {  // padding when the tree is smaller than `keep`
    a.keep_idx[ob + r] = -1;
    a.tokens[ob + r] = 0;
    a.parents[ob + r] = -1;
    a.depths[ob + r] = 0;
    a.probs[ob + r] = 0.f;
    a.position_ids[ob + r] = 0;
    // a padding row attends to itself only, so that a caller who runs all `keep` rows has no fully masked row
    if (mask_ok && r >= skip) mask_store(mbase + (size_t)(r - skip) * fa.row_stride * mf.esz, prefix + r, mf, true);
  }
  __syncthreads();
  // children CSR in new numbering; a node's children keep their original relative order
  // (ascending old index), as the reference's re-link loop leaves them (cpu_tree.py:196-199).
  // Every kept node counts its kept children, one thread adds the counts up, every node writes its list:
  // (one thread doing all of it read the parents keep x n times from global memory, 0.35 ms for 161 nodes).
  for (int r = threadIdx.x; r < keep; r += blockDim.x) {
    const int o = old_of[r];
    int cnt = 0;
    for (int c = 1; c < n; ++c) cnt += (par[c] == o && rank[c] < keep) ? 1 : 0;
    coff[r + 1] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    coff[0] = 0;
    for (int r = 0; r < keep; ++r) coff[r + 1] += coff[r];
  }
  __syncthreads();
  {
    int* off = a.child_off + (size_t)b * (a.keep + 1);
    int* idx = a.child_idx + ob;
    for (int r = threadIdx.x; r < keep; r += blockDim.x) {
      const int o = old_of[r];
      int w = coff[r];
      off[r] = w;
      for (int c = 1; c < n; ++c)
        if (par[c] == o && rank[c] < keep) idx[w++] = rank[c];
    }
    for (int r = keep + threadIdx.x; r <= a.keep; r += blockDim.x) off[r] = coff[keep];
    if (threadIdx.x == 0) a.n_out[b] = keep;
  }
}

size_t align_up(size_t x, size_t al) { return (x + al - 1) / al * al; }

template <typename T>
cudaError_t launch_expand(const KArgs& ka, int grid, cudaStream_t st) {
  if (ka.a.input_kind == SUBSPEC_IN_LOGITS)
    expand_rows_kernel<T, SUBSPEC_IN_LOGITS><<<grid, kThreads, 0, st>>>(ka);
  else
    expand_rows_kernel<T, SUBSPEC_IN_PROBS><<<grid, kThreads, 0, st>>>(ka);
  return cudaGetLastError();
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_expand_scratch_bytes(int32_t batch, int32_t leaves, int32_t k, size_t* bytes) {
  if (!bytes || batch < 0 || leaves < 1 || k < 1 || k > kMaxK) return SUBSPEC_EINVAL;
  const size_t rows = (size_t)batch * leaves;
  // sequence tickets + row tickets | row sums | row lists | slice sums | slice lists (rows may be cut into slices)
  *bytes = align_up(sizeof(int) * ((size_t)batch + rows), 256) + align_up(sizeof(RowOut) * rows, 256) +
           align_up(sizeof(Cand) * rows * k, 256) + align_up(sizeof(RowOut) * rows * kMaxRowSplits, 256) +
           sizeof(Cand) * rows * kMaxRowSplits * k;
  return SUBSPEC_OK;
}

extern "C" int subspec_expand_step(const subspec_expand_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_expand_args)) return SUBSPEC_EINVAL;
  const subspec_expand_args& a = *args;
  if (a.batch < 0 || a.leaves < 1 || a.vocab < 1 || a.k < 1) return SUBSPEC_EINVAL;
  if (a.k > kMaxK || a.k > a.vocab || a.vocab > (1 << 20) || (int64_t)a.leaves * a.vocab > INT_MAX ||
      a.leaves > kMaxK)
    return SUBSPEC_EUNSUPPORTED;
  if (a.dtype != SUBSPEC_F32 && a.dtype != SUBSPEC_BF16 && a.dtype != SUBSPEC_F16) return SUBSPEC_EINVAL;
  if (a.input_kind != SUBSPEC_IN_LOGITS && a.input_kind != SUBSPEC_IN_PROBS) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.scores || !a.out_tokens || !a.out_probs || !a.out_parents || !a.scratch) return SUBSPEC_EINVAL;
  if (!(a.temperature > 0.0)) return SUBSPEC_EINVAL;
  if (a.tree_tokens && (!a.tree_parents || !a.tree_probs || !a.tree_depths || a.level < 0 ||
                        1 + (int64_t)(a.level + 1) * a.k > a.tree_stride))
    return SUBSPEC_EINVAL;
  if (a.draft_mask) {
    if (!a.tree_tokens || !mask_kind_ok(a.draft_mask_kind) || a.draft_mask_cols < (int64_t)(a.level + 1) * a.k ||
        a.draft_mask_row_stride < 0 || a.draft_mask_seq_stride < 0 ||
        (a.draft_mask_row_stride && a.draft_mask_row_stride < a.draft_mask_cols) ||
        (reinterpret_cast<uintptr_t>(a.draft_mask) % mask_elem_bytes(a.draft_mask_kind)) != 0)
      return SUBSPEC_EINVAL;
  }
  size_t need = 0;
  subspec_expand_scratch_bytes(a.batch, a.leaves, a.k, &need);
  if (a.scratch_bytes < need || (reinterpret_cast<uintptr_t>(a.scratch) & 255u)) return SUBSPEC_ESCRATCH;
  KArgs ka;
  ka.a = a;
  ka.dm_row_stride = a.draft_mask_row_stride ? a.draft_mask_row_stride : a.draft_mask_cols;
  ka.dm_seq_stride = a.draft_mask_seq_stride ? a.draft_mask_seq_stride : (int64_t)a.k * ka.dm_row_stride;
  char* p = reinterpret_cast<char*>(a.scratch);
  const size_t rows = (size_t)a.batch * a.leaves;
  ka.ticket = reinterpret_cast<int*>(p);
  ka.rowticket = ka.ticket + a.batch;
  p += align_up(sizeof(int) * ((size_t)a.batch + rows), 256);
  ka.rowout = reinterpret_cast<RowOut*>(p);
  p += align_up(sizeof(RowOut) * rows, 256);
  ka.rowtop = reinterpret_cast<Cand*>(p);
  p += align_up(sizeof(Cand) * rows * a.k, 256);
  ka.partout = reinterpret_cast<RowOut*>(p);
  p += align_up(sizeof(RowOut) * rows * kMaxRowSplits, 256);
  ka.parttop = reinterpret_cast<Cand*>(p);
  const size_t esz = a.dtype == SUBSPEC_F32 ? 4 : 2;
  ka.prescale = (esz == 2 && a.input_kind == SUBSPEC_IN_LOGITS && a.temperature != 1.0) ? 1 : 0;
  ka.T = (float)a.temperature;
  ka.invT = 1.0f / ka.T;
  ka.kT = ka.prescale ? kLog2e : (float)(1.4426950408889634 / a.temperature);
  ka.vec_ok = ((reinterpret_cast<uintptr_t>(a.scores) & 15u) == 0) && ((a.seq_stride * esz) % 16 == 0) &&
              ((a.row_stride * esz) % 16 == 0);
  // Few rows: a row alone takes one CTA ~45 us whatever else runs (sixteen dependent iterations plus the
  // warm-up and the merges), so a single sequence's step cost almost what 32 sequences' did.  Cut every
  // row into slices while the slices of all rows still fit the machine at once and each has at least one
  // full iteration of vectors; at 4 x 148 rows and above nothing changes.
  ka.splits = 1;
  if (ka.vec_ok) {
    const int64_t slots = 4LL * kNumSMs;
    const int64_t iters = (a.vocab / (int)(16 / esz)) / (kThreads * kUnroll);  // full iterations in a row
    int64_t sp = slots / (int64_t)rows;
    if (sp > iters) sp = iters;
    if (sp > kMaxRowSplits) sp = kMaxRowSplits;
    if (sp >= 2) ka.splits = (int)sp;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = cuda_check(cudaMemsetAsync(ka.ticket, 0, sizeof(int) * ((size_t)a.batch + rows), st));
  if (rc) return rc;
  cudaError_t e;
  switch (a.dtype) {
    case SUBSPEC_F32:
      e = launch_expand<float>(ka, (int)rows * ka.splits, st);
      break;
    case SUBSPEC_BF16:
      e = launch_expand<__nv_bfloat16>(ka, (int)rows * ka.splits, st);
      break;
    default:
      e = launch_expand<__half>(ka, (int)rows * ka.splits, st);
      break;
  }
  return cuda_check(e);
}

extern "C" int subspec_tree_finalize(const subspec_tree_finalize_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_tree_finalize_args)) return SUBSPEC_EINVAL;
  const subspec_tree_finalize_args& a = *args;
  if (a.batch < 0 || a.n_nodes < 1 || a.keep < 1 || a.tree_stride < a.n_nodes) return SUBSPEC_EINVAL;
  if (a.n_nodes > 4096 || a.keep > 1024) return SUBSPEC_EUNSUPPORTED;
  if (a.skip_nodes < 0 || a.skip_nodes > a.keep || !mask_kind_ok(a.mask_kind)) return SUBSPEC_EINVAL;
  if (a.mask_cols < 0 || a.mask_row_stride < 0 || a.mask_seq_stride < 0) return SUBSPEC_EINVAL;
  if (a.mask_cols == 0 && a.prefix_length) return SUBSPEC_EINVAL;  // the host cannot size the rows from device values
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.tree_tokens || !a.tree_parents || !a.tree_probs || !a.tree_depths || !a.keep_idx || !a.tokens ||
      !a.parents || !a.depths || !a.probs || !a.position_ids || !a.mask || !a.child_off || !a.child_idx || !a.n_out)
    return SUBSPEC_EINVAL;
  FinArgs fa;
  fa.a = a;
  fa.cols = a.mask_cols ? a.mask_cols : a.keep;
  if (fa.cols < a.keep) return SUBSPEC_EINVAL;
  fa.row_stride = a.mask_row_stride ? a.mask_row_stride : fa.cols;
  if (fa.row_stride < fa.cols) return SUBSPEC_EINVAL;
  fa.seq_stride = a.mask_seq_stride ? a.mask_seq_stride : (int64_t)(a.keep - a.skip_nodes) * fa.row_stride;
  if ((reinterpret_cast<uintptr_t>(a.mask) % mask_elem_bytes(a.mask_kind)) != 0) return SUBSPEC_EINVAL;
  const size_t smem = sizeof(int) * (2 * (size_t)a.n_nodes + 2 * (size_t)a.keep + 1);
  tree_finalize_kernel<<<a.batch, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(fa);
  return cuda_check(cudaGetLastError());
}
