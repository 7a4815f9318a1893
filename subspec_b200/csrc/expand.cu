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

#include <type_traits>

#include <algorithm>

#include "common.cuh"
#include "mask.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;
constexpr int kMaxK = 32;
constexpr int kMaxRowSplits = 16;   // slices a row may be cut into when a launch has few rows

struct Cand {
  float v;
  int id;
};
__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
  return av > bv || (av == bv && ai < bi);
}

// Lanes that share one candidate in a rank count over n candidates by kThreads threads: the largest power of
// two (at most 32) that still gives every candidate its lanes in one sweep.  The latency of a rank count is
// the n / P compares one lane makes one after the other, and these counts sit between the stages of a CTA
// that has nothing else to do meanwhile.
__device__ __forceinline__ int lanes_per_candidate(int n) {
  int p = 1;
  while (p < 32 && 2 * p * n <= (int)blockDim.x) p <<= 1;
  return p;
}

// Rank (number of candidates that beat it) of candidate i = base + threadIdx.x / P among get(0..n), counted by
// its P lanes together; the same value in all of them.  Called by every thread of the CTA (it shuffles).
template <typename Get>
__device__ __forceinline__ int coop_rank(int n, int P, int i, const Cand& me, Get&& get) {
  const int part = threadIdx.x & (P - 1);
  int rank = 0;
  if (i < n && me.id != INT_MAX) {
#pragma unroll 4  // the loads of a group go out together: one after the other they are the whole cost
    for (int j = part; j < n; j += P) {
      const Cand o = get(j);
      rank += (o.id != INT_MAX && better(o.v, o.id, me.v, me.id)) ? 1 : 0;
    }
  }
  for (int off = P >> 1; off > 0; off >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, off);
  return rank;
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
  const int P = lanes_per_candidate(n);
  const int per_sweep = blockDim.x / P;
  for (int base = 0; base < n; base += per_sweep) {
    const int i = base + threadIdx.x / P;
    const Cand me = i < n ? get(i) : Cand{-INFINITY, INT_MAX};
    const int rank = coop_rank(n, P, i, me, get);
    if (i < n && me.id != INT_MAX && (threadIdx.x & (P - 1)) == 0 && rank < k) out[rank] = me;
  }
  __syncthreads();
}

struct RowOut {  // per (sequence, leaf) row, in scratch
  float c, s;    // softmax shift (log2 domain) and denominator; unused for probabilities in
};

struct KArgs {
  subspec_expand_args a;
  int* ticket;     // [batch]
  float kT;        // scale inside 2^(x * kT - c): log2(e) / temperature, or log2(e) when the logits are pre-scaled
  float invT, T;   // 16-bit dtypes with temperature != 1: the reference rounds logits / T to the dtype first
  int prescale;
  int vec_ok;
  // few rows: every row is cut into `splits` slices, one CTA each; the slices' lists and softmax sums meet
  // in scratch behind a ticket per row, and the last slice to arrive carries on as the row's CTA
  int splits;
  int64_t dm_row_stride, dm_seq_stride;  // draft-side mask geometry in elements, defaults resolved
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
  // filler for vectors past the end of a slice: the lowest finite value (and the smallest value above it)
  static __device__ __forceinline__ uint4 lowest() { return make_uint4(0xff7fffffu, 0xff7fffffu, 0xff7fffffu, 0xff7fffffu); }
  static __device__ __forceinline__ float above_lowest() { return __uint_as_float(0xff7ffffeu); }
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
  static __device__ __forceinline__ uint4 lowest() { return make_uint4(0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu); }
  static __device__ __forceinline__ float above_lowest() { return __uint_as_float(0xff7e0000u); }
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
  static __device__ __forceinline__ uint4 lowest() { return make_uint4(0xfbfffbffu, 0xfbfffbffu, 0xfbfffbffu, 0xfbfffbffu); }
  static __device__ __forceinline__ float above_lowest() { return -65472.f; }
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
// Candidates of a slice are 16-byte VECTORS, not elements: a vector whose maximum reaches the threshold goes,
// unordered, into a buffer in shared memory as (maximum, index of its first element) -- one atomic and one
// store, a dozen instructions, which matters because a warp with a single candidate lane pays for every
// instruction thirty-two-fold.  The threshold is seeded from the first stage (the k-th largest of the 256
// per-thread maxima is k distinct elements' worth of evidence that the slice's k-th best is at least that)
// and raised, the buffer cut back to its k best vectors, at the first stage boundary after the buffer has
// gathered k + kSlack entries: with the threshold at the k-th best of the m stages read so far, stage m + 1
// brings about k / m candidates.  Only when the slice has been read are the elements looked at: the vectors
// whose maximum reaches the k-th largest vector maximum are fetched again (a few dozen 16-byte loads, mostly
// L2 hits) and their elements at or above that value compete by rank counting.  Every element of the true
// top k sits in a vector that was pushed and kept: a vector is only dropped when k vectors with a better
// (maximum, index) exist, each of which holds an element that beats all of its elements.  A slice whose
// candidates outrun the buffer inside one stage (sorted input) is redone by the slow selector below.
// Rows that cannot be read as vectors, and the few elements behind a row's last whole vector, go through the
// same buffer as single elements.
constexpr int kStageVecs = kThreads * kUnroll;  // 16-byte vectors per TMA stage: one group per thread (16 KB)
constexpr int kStages = 3;                      // shared-memory ring depth
constexpr int kRingBytes = kStages * kStageVecs * 16;
constexpr int kCap = kThreads;  // candidate buffer entries: one per thread when the buffer is ranked
constexpr int kSlack = 48;   // the buffer is cut back to k entries once it has reached k + kSlack
constexpr int kMaxSeqCands = 4096;  // leaves x slices x k candidates the last CTA of a sequence merges (32 KB)
constexpr int kMaxSel = kRingBytes / 8 - kMaxSeqCands;  // of which so many may pass the pre-filter (16 KB)

// The elements of a 16-byte vector, two at a time, as floats: f(x0, x1) for pairs in vocabulary order.
template <typename T, typename F>
__device__ __forceinline__ void for_pairs(const uint4& q, F&& f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  if constexpr (sizeof(T) == 4) {
    f(__uint_as_float(w[0]), __uint_as_float(w[1]));
    f(__uint_as_float(w[2]), __uint_as_float(w[3]));
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f(v.x, v.y);
    }
  }
}

struct Slice {
  Cand* buf;
  int* cnt;
  int tighten_at;  // k + kSlack
  bool hot;        // this thread saw the buffer reach tighten_at
  __device__ __forceinline__ void push(float v, int id) {
    const int p = atomicAdd(cnt, 1);
    if (p < kCap) buf[p] = Cand{v, id};
    hot |= p >= tighten_at - 1;
  }
};

// all 32 lane values in descending order: lane i ends up with the i-th largest
__device__ __forceinline__ float warp_sort_desc(float v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const float o = __shfl_xor_sync(0xffffffffu, v, stride);
      const bool desc = (lane & size) == 0;
      const bool lower = (lane & stride) == 0;
      v = (desc == lower) ? fmaxf(v, o) : fminf(v, o);
    }
  }
  return v;
}

// A lower bound of the k-th largest of the CTA's 256 per-thread values (-inf = no value), nearly for free:
// with j = ceil(k / warps), every warp's j-th largest value has j values of that warp at or above it, so the
// smallest of them over the warps has warps * j >= k values of the CTA at or above it.  (The exact k-th largest
// by rank counting over the warps' sorted lists cost a tenth of a row's streaming instructions; this bound
// lets about one and a half times as many candidates through the first stage, which the first cut of the
// buffer mends.)  `tmp` holds kWarps floats.
__device__ __forceinline__ float cta_kth_lower_bound(float v, int k, float* tmp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j = (k + kWarps - 1) / kWarps;
  float jth = -INFINITY;
  for (int r = 0; r < j; ++r) {  // the warp's j-th largest: take the maximum out j times (one instance each time)
    float m = v;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    jth = m;
    const uint32_t holders = __ballot_sync(0xffffffffu, v == m);
    if (holders && lane == __ffs(holders) - 1) v = -INFINITY;
  }
  if (lane == 0) tmp[warp] = jth;
  __syncthreads();
  float bound = tmp[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) bound = fminf(bound, tmp[w]);
  return bound;
}

// The slow selector: the k best (value desc, index asc) of elements [lo, hi) of a row, one CTA-wide pass per
// entry (each pass finds the best element that comes after the previous pick in that order).  Only slices
// whose candidates overflowed the buffer come here.
template <typename T>
__device__ void select_slow(const T* rowp, int lo, int hi, int k, Cand* out, Cand* s_red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float pv = INFINITY;
  int pid = -1;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bid = INT_MAX;
    for (int i = lo + threadIdx.x; i < hi; i += kThreads) {
      const float x = to_f32<T>(rowp[i]);
      const bool after = x < pv || (x == pv && i > pid);
      if (after && better(x, i, bv, bid)) {
        bv = x;
        bid = i;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bid, off);
      if (better(ov, oi, bv, bid)) {
        bv = ov;
        bid = oi;
      }
    }
    __syncthreads();
    if (lane == 0) s_red[warp] = Cand{bv, bid};
    __syncthreads();
    bv = s_red[0].v;
    bid = s_red[0].id;
    for (int w = 1; w < kWarps; ++w)
      if (better(s_red[w].v, s_red[w].id, bv, bid)) {
        bv = s_red[w].v;
        bid = s_red[w].id;
      }
    if (threadIdx.x == 0) out[r] = Cand{bv, bid};
    pv = bid == INT_MAX ? -INFINITY : bv;
    pid = bid == INT_MAX ? INT_MAX : bid;
  }
  __syncthreads();
}

template <typename T, int KIND, bool PRESCALE>
__global__ void __launch_bounds__(kThreads, 4) expand_rows_kernel(const KArgs ka) {
  extern __shared__ __align__(128) unsigned char smem_raw[];  // the ring; after streaming, the merges' candidates
  __shared__ Cand s_buf[kCap];
  __shared__ Cand s_best[kMaxK];
  __shared__ Cand s_red[kWarps];
  __shared__ float s_tmp[kWarps * kMaxK];
  __shared__ float s_c[kWarps], s_s[kWarps];
  __shared__ __align__(8) uint64_t s_full[kStages];
  __shared__ float s_thr;
  __shared__ int s_cnt, s_cnt2, s_flag, s_abort;

  const subspec_expand_args& a = ka.a;
  const int L = a.leaves, V = a.vocab, k = a.k;
  const int S = ka.splits;
  const int row = blockIdx.x / S;
  const int split = blockIdx.x - row * S;
  const int b = row / L;
  const T* rowp = reinterpret_cast<const T*>(a.scores) + (size_t)b * a.seq_stride + (size_t)(row - b * L) * a.row_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int VN = Elem<T>::N;

  SoftAcc soft;
  soft.init(ka.kT);
  Slice sl{s_buf, &s_cnt, k + kSlack, false};
  if (threadIdx.x == 0) {
    s_cnt = 0;
    s_cnt2 = 0;
    s_abort = 0;
    for (int st = 0; st < kStages; ++st) mbar_init(&s_full[st], 1);
    mbar_init_fence();
  }
  fence_async_smem();
  __syncthreads();
  float thr = -INFINITY;
  bool overflow = false;  // the same in every thread

  // Raise the threshold at a stage boundary: the buffer is cut back to its k best entries (rank counting, every
  // entry against all others).  Called by the whole CTA between two stages, when nobody is pushing.
  auto tighten = [&]() {
    const int n = s_cnt;
    if (n > kCap) {  // candidates were dropped: this slice goes to the slow selector
      overflow = true;
      thr = INFINITY;
      __syncthreads();
    } else {
      const int P = lanes_per_candidate(n);  // n <= kCap = kThreads: one sweep
      const int i = threadIdx.x / P;
      const bool mine = i < n && (threadIdx.x & (P - 1)) == 0;
      const Cand me = i < n ? s_buf[i] : Cand{-INFINITY, INT_MAX};
      int rank = coop_rank(n, P, i, me, [&](int j) { return s_buf[j]; });
      if (!mine) rank = INT_MAX;
      __syncthreads();
      if (rank < k) s_buf[rank] = me;
      if (rank == k - 1) s_thr = me.v;
    }
    if (threadIdx.x == 0) s_cnt = overflow ? 0 : min(n, k);
    sl.hot = false;
    __syncthreads();
    if (!overflow && n >= k) thr = fmaxf(thr, s_thr);
  };

  const int nvec = ka.vec_ok ? V / VN : 0;
  // this CTA's slice of the row's vectors (the whole row when S == 1); the scalar tail goes with the last slice
  const int vec_per = (nvec + S - 1) / S;
  const int v0 = min(split * vec_per, nvec), v1 = min(v0 + vec_per, nvec);
  int lo_elem = v0 * VN, hi_elem = v1 * VN;  // what the slow selector would scan
  if (ka.vec_ok) {
    // The slice is staged through a ring of kStages 16 KB buffers by TMA bulk copies that thread 0 issues
    // kStages - 1 stages ahead; the barrier at the top of iteration st proves that stage st - 1 has been read
    // by everyone, so its buffer is refilled, and carries the vote on whether the buffer needs cutting back.
    const uint4* vp = reinterpret_cast<const uint4*>(rowp);
    uint4* ring = reinterpret_cast<uint4*>(smem_raw);
    const int nst = (v1 - v0 + kStageVecs - 1) / kStageVecs;
    auto issue = [&](int st) {
      const int a0 = v0 + st * kStageVecs;
      const uint32_t bytes = (uint32_t)(min(kStageVecs, v1 - a0) * 16);
      uint64_t* bar = &s_full[st % kStages];
      mbar_expect_tx(bar, bytes);
      bulk_g2s(ring + (size_t)(st % kStages) * kStageVecs, vp + a0, bytes, bar);
    };
    if (threadIdx.x == 0)
      for (int st = 0; st < kStages - 1 && st < nst; ++st) issue(st);
    for (int st = 0; st < nst; ++st) {
      const int need = __syncthreads_or(sl.hot ? 1 : 0);
      if (s_abort) break;
      if (need) tighten();
      if (threadIdx.x == 0 && st + kStages - 1 < nst) issue(st + kStages - 1);
      if (!mbar_wait_bounded(&s_full[st % kStages], (uint32_t)(st / kStages) & 1u)) s_abort = 1;
      const uint4* buf = ring + (size_t)(st % kStages) * kStageVecs;
      const int a0 = v0 + st * kStageVecs;
      const bool full = a0 + kStageVecs <= v1;  // all but a slice's last stage
      uint4 q[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; ++j)
        q[j] = (full || a0 + threadIdx.x + j * kThreads < v1) ? buf[threadIdx.x + j * kThreads] : Elem<T>::lowest();
      float m[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) m[j] = Elem<T>::vmax(q[j]);
      const float gm = fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
      if (st == 0) thr = fmaxf(thr, cta_kth_lower_bound(gm, k, s_tmp));
      if (KIND == SUBSPEC_IN_LOGITS) {
        // With pre-scaling the sums run over round(x / T); the multiply by 1 / T used here can differ from the
        // division by one fp32 ulp before rounding, which the k survivors (recomputed exactly below) never see.
        // Vectors past the end of a last, partial stage hold the lowest finite value: 2^y = 0 for them.
        soft.ensure(fmaxf(PRESCALE ? Elem<T>::round_to(gm * ka.invT) : gm, -1.0e30f));
#pragma unroll
        for (int j = 0; j < kUnroll; ++j)
          for_pairs<T>(q[j], [&](float x0, float x1) {
            if (PRESCALE) {
              x0 = Elem<T>::round_to(x0 * ka.invT);
              x1 = Elem<T>::round_to(x1 * ka.invT);
            }
            soft.add_pair(x0, x1);
          });
      }
      if (gm >= thr) {
        const float t = full ? thr : fmaxf(thr, Elem<T>::above_lowest());  // the filler never qualifies
#pragma unroll
        for (int j = 0; j < kUnroll; ++j)
          if (m[j] >= t) sl.push(m[j], (a0 + threadIdx.x + j * kThreads) * VN);
      }
    }
    if (split == S - 1) {  // scalar tail of an aligned row whose length is not a multiple of the vector
      hi_elem = V;
      const int i = nvec * VN + threadIdx.x;
      if (i < V) {
        const float x = to_f32<T>(rowp[i]);
        if (KIND == SUBSPEC_IN_LOGITS) {
          const float xs = PRESCALE ? Elem<T>::round_to(x * ka.invT) : x;
          soft.ensure(fmaxf(xs, -1.0e30f));
          soft.add_one(xs);
        }
        if (x >= thr) sl.push(x, i);
      }
    }
  } else {
    // Rows that do not start on 16-byte boundaries: the same scheme over "stages" of kThreads * 32 elements read
    // straight from global memory, thread t taking elements t, t + kThreads, ... of the stage.
    lo_elem = 0;
    hi_elem = V;
    constexpr int kPer = 32;
    for (int e0 = 0; e0 < V; e0 += kThreads * kPer) {
      const int need = __syncthreads_or(sl.hot ? 1 : 0);
      if (need) tighten();
      float gm = -INFINITY;
      for (int j = 0; j < kPer; ++j) {
        const int i = e0 + threadIdx.x + j * kThreads;
        if (i < V) gm = fmaxf(gm, to_f32<T>(rowp[i]));
      }
      if (e0 == 0) thr = fmaxf(thr, cta_kth_lower_bound(gm, k, s_tmp));
      if (KIND == SUBSPEC_IN_LOGITS && gm != -INFINITY)
        soft.ensure(fmaxf(PRESCALE ? Elem<T>::round_to(gm * ka.invT) : gm, -1.0e30f));
      for (int j = 0; j < kPer; ++j) {
        const int i = e0 + threadIdx.x + j * kThreads;
        if (i >= V) break;
        const float x = to_f32<T>(rowp[i]);
        if (KIND == SUBSPEC_IN_LOGITS) soft.add_one(PRESCALE ? Elem<T>::round_to(x * ka.invT) : x);
        if (x >= thr) sl.push(x, i);
      }
    }
  }
  {
    const int need = __syncthreads_or(sl.hot ? 1 : 0);  // every push is in
    if (s_abort) {  // a bulk copy never completed: report and leave together
      if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_TIMEOUT);
      return;
    }
    if (need && s_cnt > kCap) overflow = true;
  }

  // ---- the slice's k best, and its softmax sum ----
  Cand* s_cand = reinterpret_cast<Cand*>(smem_raw);  // 6144 entries: the ring is idle from here on
  if (overflow) {
    select_slow<T>(rowp, lo_elem, hi_elem, k, s_best, s_red);
  } else {
    // the k-th largest entry of the buffer bounds the k-th best element from below ...
    const int n = min(s_cnt, kCap);
    if (threadIdx.x == 0) s_thr = -INFINITY;
    __syncthreads();
    {
      const int P = lanes_per_candidate(n);
      const int i = threadIdx.x / P;
      const Cand me = i < n ? s_buf[i] : Cand{-INFINITY, INT_MAX};
      const int rank = coop_rank(n, P, i, me, [&](int j) { return s_buf[j]; });
      if (i < n && (threadIdx.x & (P - 1)) == 0 && rank == k - 1) s_thr = me.v;
    }
    __syncthreads();
    // ... and the elements at or above it, all of which sit in buffered vectors, compete
    const float tv = s_thr;
    const int vec_end = nvec * VN;  // entries from here on (and all entries of an unaligned row) are single elements
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const Cand u = s_buf[i];
      if (!(u.v >= tv)) continue;
      if (u.id < vec_end) {
        float x[VN];
        Elem<T>::unpack(reinterpret_cast<const uint4*>(rowp)[u.id / VN], x);
#pragma unroll
        for (int e = 0; e < VN; ++e)
          if (x[e] >= tv) s_cand[atomicAdd(&s_cnt2, 1)] = Cand{x[e], u.id + e};
      } else {
        s_cand[atomicAdd(&s_cnt2, 1)] = u;
      }
    }
    __syncthreads();
    cta_topk(s_cnt2, k, [&](int i) { return s_cand[i]; }, s_best);
  }
  {
    float c = soft.c, sm = soft.sum();
    if (KIND != SUBSPEC_IN_LOGITS) {
      c = 0.f;
      sm = 1.f;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float oc = __shfl_xor_sync(0xffffffffu, c, off);
      const float os = __shfl_xor_sync(0xffffffffu, sm, off);
      combine_soft(c, sm, oc, os);
    }
    if (lane == 0) {
      s_c[warp] = c;
      s_s[warp] = sm;
    }
  }
  __syncthreads();
  // ---- the slice's list and softmax sum go to scratch; the last slice of the SEQUENCE to arrive merges ----
  // (one ticket per sequence counts leaves x slices arrivals: the slices of a row do not meet first, which
  // would put a second fence / atomic / reload round trip on the path of every row)
  Cand* top_dst = ka.parttop + ((size_t)row * S + split) * k;
  if (threadIdx.x < k) top_dst[threadIdx.x] = s_best[threadIdx.x];
  if (threadIdx.x == 0) {
    float c = s_c[0], sm = s_s[0];
    for (int w = 1; w < kWarps; ++w) combine_soft(c, sm, s_c[w], s_s[w]);
    if (KIND != SUBSPEC_IN_LOGITS) {
      c = 0.f;
      sm = 1.f;
    }
    ka.partout[(size_t)row * S + split] = RowOut{c, sm};
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_flag = (atomicAdd(ka.ticket + b, 1) == L * S - 1);
    if (s_flag) ka.ticket[b] = 0;  // everybody has been: left as found, zero, for the next launch
  }
  __syncthreads();
  if (!s_flag) return;
  __threadfence();

  // ---- the last CTA of the sequence: scores with the reference's rounding, global top-k ----
  {
    // every row's softmax shift and denominator from its slices' (in slice order: the same bits on every run)
    if (threadIdx.x < L) {
      const volatile RowOut* po = ka.partout + ((size_t)b * L + threadIdx.x) * S;
      float c = po[0].c, sm = po[0].s;
      for (int i = 1; i < S; ++i) combine_soft(c, sm, po[i].c, po[i].s);
      s_tmp[threadIdx.x] = c;
      s_tmp[kMaxK + threadIdx.x] = sm;
    }
    __syncthreads();
    const int per_row = S * k;
    const int total = L * per_row;  // <= kMaxSeqCands (the host picks S accordingly)
    for (int t = threadIdx.x; t < total; t += kThreads) {
      const int l = t / per_row;
      const volatile Cand* src = ka.parttop + (size_t)b * total + t;
      const float xv = src->v;
      const int xi = src->id;
      Cand out{-INFINITY, INT_MAX};
      if (xi != INT_MAX) {
        float p = xv;
        if (KIND == SUBSPEC_IN_LOGITS) {
          // The survivors' probabilities in double precision: a 16-bit dtype rounds them next, and an error of
          // 1e-6 in fp32 arithmetic on an exponent near 20 would land on the other side of a rounding boundary
          // a few times per thousand values; what is left is the error of the fp32 denominator (~1e-7).
          const float xs = PRESCALE ? Elem<T>::round_to(__fdiv_rn(xv, ka.T)) : xv;
          p = (float)(exp2((double)xs * (double)ka.kT - (double)s_tmp[l]) / (double)s_tmp[kMaxK + l]);
        }
        p = Elem<T>::round_to(p);
        const float pp = a.parent_probs ? Elem<T>::load(a.parent_probs, (size_t)b * L + l) : 1.f;
        out = Cand{Elem<T>::round_to(p * pp), l * V + xi};
      }
      s_cand[t] = out;
    }
    __syncthreads();  // s_tmp is reused below
    if (threadIdx.x == 0) s_cnt2 = 0;
    __syncthreads();
    // A warp's k-th best score bounds the sequence's k-th best from below (k distinct candidates reach it):
    // the largest such bound over the warps lets a few dozen of the leaves x k candidates into the rank count.
    {
      float wk = -INFINITY;
      for (int t0 = 0; t0 < total; t0 += kThreads) {  // the same trips in every thread
        const int t = t0 + threadIdx.x;
        const float sorted = warp_sort_desc(t < total ? s_cand[t].v : -INFINITY);
        wk = fmaxf(wk, __shfl_sync(0xffffffffu, sorted, k - 1));
      }
      if (lane == 0) s_tmp[warp] = wk;
      __syncthreads();
      float bound = s_tmp[0];
      for (int w = 1; w < kWarps; ++w) bound = fmaxf(bound, s_tmp[w]);
      Cand* s_sel = s_cand + kMaxSeqCands;
      for (int t = threadIdx.x; t < total; t += kThreads) {
        const Cand cnd = s_cand[t];
        if (cnd.id != INT_MAX && cnd.v >= bound) {
          const int pos = atomicAdd(&s_cnt2, 1);
          if (pos < kMaxSel) s_sel[pos] = cnd;
        }
      }
      __syncthreads();
      if (s_cnt2 <= kMaxSel)
        cta_topk(s_cnt2, k, [&](int i) { return s_sel[i]; }, s_best);
      else  // thousands of candidates tied at the bound: rank them all
        cta_topk(total, k, [&](int i) { return s_cand[i]; }, s_best);
    }
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
  float* ps = reinterpret_cast<float*>(coff + keep + 1);  // [n] cumulative probabilities as they are ranked
  // The mask rows of a sequence are shared out between the gridDim.y CTAs of the sequence (a static buffer of
  // [max_verify, max_cache_len] is a quarter of a megabyte to fill); every CTA ranks the nodes for itself, CTA 0
  // also writes the per-node outputs and the children lists.
  const int slice = blockIdx.y, nslices = gridDim.y;
  const size_t tb = (size_t)b * a.tree_stride;
  const float* prob = a.tree_probs + tb;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int p = i == 0 ? -1 : a.tree_parents[tb + i];
    if (i > 0 && (p < 0 || p >= i)) {  // expansion appends children behind their parents; anything else could loop
      flag(a.dev_status, SUBSPEC_DEV_BAD_PARENT);
      p = -1;
    }
    par[i] = p;
    const float pr = i == 0 ? 1.f : prob[i];
    ps[i] = pr == pr ? pr : -INFINITY;  // the root carries probability 1, NaN counts as -inf
  }
  __syncthreads();

  // rank by (cumulative probability desc, index asc)
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int r = i;
    if (!identity) {
      const float pi = ps[i];
      r = 0;
      for (int j = 0; j < n; ++j) {
        const float pj = ps[j];
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
  const int mrows = a.keep - skip, per_slice = (mrows + nslices - 1) / nslices;
  const int r0 = min(slice * per_slice, mrows), r1 = min(r0 + per_slice, mrows);  // this CTA's mask rows
  if (mask_ok) mask_fill_rows(mbase + (size_t)r0 * fa.row_stride * mf.esz, fa.row_stride, r1 - r0, fa.cols, prefix, mf);
  __syncthreads();
  const size_t ob = (size_t)b * a.keep;
  for (int r = threadIdx.x; r < keep; r += blockDim.x) {
    const int o = old_of[r];
    const int p = par[o];
    if (slice == 0) {
      const int np = (p >= 0 && rank[p] < keep) ? rank[p] : -1;
      a.keep_idx[ob + r] = o;
      a.tokens[ob + r] = a.tree_tokens[tb + o];
      a.parents[ob + r] = np;
      const int d = o == 0 ? 0 : a.tree_depths[tb + o];
      a.depths[ob + r] = d;
      a.probs[ob + r] = o == 0 ? 1.f : prob[o];
      a.position_ids[ob + r] = (int64_t)d + (a.position_offset ? a.position_offset[b] : 0);
    }
    // ancestor-or-self row (parents are smaller than their children, so the walk ends within n steps)
    if (mask_ok && r >= skip && r - skip >= r0 && r - skip < r1) {
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
    if (slice == 0) {
      a.keep_idx[ob + r] = -1;
      a.tokens[ob + r] = 0;
      a.parents[ob + r] = -1;
      a.depths[ob + r] = 0;
      a.probs[ob + r] = 0.f;
      a.position_ids[ob + r] = 0;
    }
    // a padding row attends to itself only, so that a caller who runs all `keep` rows has no fully masked row
    if (mask_ok && r >= skip && r - skip >= r0 && r - skip < r1) mask_store(mbase + (size_t)(r - skip) * fa.row_stride * mf.esz, prefix + r, mf, true);
  }
  if (slice != 0) return;  // (the whole CTA: the children lists are CTA 0's)
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
  void (*kernel)(const KArgs) = expand_rows_kernel<T, SUBSPEC_IN_PROBS, false>;
  if (ka.a.input_kind == SUBSPEC_IN_LOGITS)
    kernel = ka.prescale ? expand_rows_kernel<T, SUBSPEC_IN_LOGITS, true> : expand_rows_kernel<T, SUBSPEC_IN_LOGITS, false>;
  // static + dynamic shared memory pass the 48 KB that need no opt-in
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
  if (e != cudaSuccess) return e;
  kernel<<<grid, kThreads, kRingBytes, st>>>(ka);
  return cudaGetLastError();
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_expand_scratch_bytes(int32_t batch, int32_t leaves, int32_t k, size_t* bytes) {
  if (!bytes || batch < 0 || leaves < 1 || k < 1 || k > kMaxK) return SUBSPEC_EINVAL;
  const size_t rows = (size_t)batch * leaves;
  // sequence tickets | slice sums | slice lists (rows may be cut into up to kMaxRowSplits slices)
  *bytes = align_up(sizeof(int) * (size_t)batch, 256) + align_up(sizeof(RowOut) * rows * kMaxRowSplits, 256) +
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
  p += align_up(sizeof(int) * (size_t)a.batch, 256);
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
  // A launch with fewer rows than the machine has CTA slots cuts every row into slices, one CTA each, so that
  // it still fills the machine (a single sequence's step: 16 rows); a slice is at least one 16 KB stage.
  // With a row per slot or more, rows stay whole: every slice pays the threshold's warm-up again (its own
  // first stage, and the k ln(stages) candidates after it), which costs more than the even finish buys.
  ka.splits = 1;
  if (ka.vec_ok) {
    const int64_t slots = 4LL * kNumSMs;
    const int64_t stages = ((a.vocab / (int)(16 / esz)) + kStageVecs - 1) / kStageVecs;
    int64_t sp = slots / (int64_t)rows;
    if (sp > stages) sp = stages;
    if (sp > kMaxRowSplits) sp = kMaxRowSplits;
    const int64_t mergeable = kMaxSeqCands / ((int64_t)a.leaves * a.k);  // what the sequence's last CTA can hold
    if (sp > mergeable) sp = mergeable;
    if (sp >= 2) ka.splits = (int)sp;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // The tickets have to be zero; every launch leaves them so (the last arrival resets its ticket), so a caller
  // who vouches for the buffer saves this node in front of the kernel.
  int rc = SUBSPEC_OK;
  if (!(a.flags & SUBSPEC_EXPAND_SCRATCH_CLEAN))
    rc = cuda_check(cudaMemsetAsync(ka.ticket, 0, sizeof(int) * (size_t)a.batch, st));
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
  const size_t smem = sizeof(int) * (3 * (size_t)a.n_nodes + 2 * (size_t)a.keep + 1);
  // CTAs per sequence: one per 32 KB of mask rows, at most 16, and no more than four waves' worth in all
  const int64_t mask_bytes = (int64_t)(a.keep - a.skip_nodes) * fa.cols * mask_elem_bytes(a.mask_kind);
  int slices = (int)std::min<int64_t>(16, std::max<int64_t>(1, mask_bytes / 32768));
  slices = std::max(1, std::min(slices, 4 * kNumSMs / std::max(a.batch, 1)));
  if (smem > 48 * 1024) {  // more than 3072 nodes: past the default limit of dynamic shared memory
    static const cudaError_t opted = cudaFuncSetAttribute(tree_finalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                          (int)(sizeof(int) * (3 * 4096 + 2 * 1024 + 1)));
    if (opted != cudaSuccess) return cuda_check(opted);
  }
  tree_finalize_kernel<<<dim3((unsigned)a.batch, (unsigned)slices), 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(fa);
  return cuda_check(cudaGetLastError());
}
