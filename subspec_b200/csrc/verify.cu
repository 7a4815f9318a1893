// Fused tree verify + accept for sm_100a.
//
// One launch per batch.  Each CTA streams one chunk of one [vocab] row with
// 128-bit loads and reduces, in a single pass over HBM:
//   - the first-index argmax (the greedy target token),
//   - the softmax denominator in the log2 domain,
//   - sum((x*k - c) * 2^(x*k - c))  from which the normalised entropy follows.
// The CTA that completes a row (an atomic ticket, no spinning) finalises the
// row statistics and gathers P[u, token(child)] for the node's children.  The
// CTA that completes the last row of a sequence then runs the accept walk for
// that sequence (exact walk, or the lossy reverse-index DP + top-down walk)
// out of shared memory while other CTAs keep streaming other sequences.
//
// Semantics follow the reference's verify_tree (tree_verify.py:49-163),
// _verify_step (classic_sd.py:111-116) and lossy_bottom_up_verify
// (lossy_tree_verify.py:9-291).
#include <limits.h>
#include <math.h>

#include "common.cuh"
#include "lm_head.cuh"
#include "tma.cuh"

namespace subspec {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;
constexpr int kStageVecs = kThreads * kUnroll;  // 16-byte vectors per TMA stage: one group per thread
constexpr int kStageBytes = kStageVecs * 16;    // 16 KB
constexpr int kStages = 3;                      // shared-memory ring depth
constexpr int kMaxSplits = 32;
constexpr int kMaxNodes = 1024;

// Row statistics relative to a shift `c` in the log2 domain:
//   s  = sum 2^(y),  t2 = sum y * 2^(y)   with y = x * k - c.
// In SUBSPEC_IN_PROBS mode c stays 0, s = sum p, t2 = sum p * log2(p).
struct RowStat {
  float c, s, t2, vmax;
  int amax;
};

__device__ __forceinline__ RowStat empty_stat(bool probs) {
  RowStat r;
  r.c = probs ? 0.f : -INFINITY;
  r.s = 0.f;
  r.t2 = 0.f;
  r.vmax = -INFINITY;
  r.amax = INT_MAX;
  return r;
}

__device__ __forceinline__ RowStat combine(const RowStat& a, const RowStat& b) {
  RowStat r;
  r.c = fmaxf(a.c, b.c);
  float fa = 0.f, fb = 0.f, ta = 0.f, tb = 0.f;
  if (a.c != -INFINITY) {
    const float d = a.c - r.c;
    fa = ex2f(d);
    ta = fa * fmaf(d, a.s, a.t2);
  }
  if (b.c != -INFINITY) {
    const float d = b.c - r.c;
    fb = ex2f(d);
    tb = fb * fmaf(d, b.s, b.t2);
  }
  r.s = a.s * fa + b.s * fb;
  r.t2 = ta + tb;
  const bool pick_a = (a.vmax > b.vmax) || (a.vmax == b.vmax && a.amax < b.amax);
  r.vmax = pick_a ? a.vmax : b.vmax;
  r.amax = pick_a ? a.amax : b.amax;
  return r;
}

__device__ __forceinline__ RowStat shfl_down_stat(const RowStat& v, int off) {
  RowStat r;
  r.c = __shfl_down_sync(0xffffffffu, v.c, off);
  r.s = __shfl_down_sync(0xffffffffu, v.s, off);
  r.t2 = __shfl_down_sync(0xffffffffu, v.t2, off);
  r.vmax = __shfl_down_sync(0xffffffffu, v.vmax, off);
  r.amax = __shfl_down_sync(0xffffffffu, v.amax, off);
  return r;
}

__device__ __forceinline__ RowStat warp_reduce(RowStat v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = combine(v, shfl_down_stat(v, off));
  return v;
}

// Headroom (log2 domain) a new row maximum may have over the thread's reference shift
// before the accumulators are rescaled: 2^64 * vocab still sits far below FLT_MAX.
constexpr float kRefHeadroom = 64.f;

// Per-thread accumulator.  SOFT = false keeps only the argmax.
//
// Logits mode keeps S = sum 2^y and T2 = sum y * 2^y with y = x * k - c in packed fp32x2
// lanes (even / odd elements).  The shift c is taken from the first maximum the thread
// meets and only moves when a later maximum exceeds it by kRefHeadroom; any c gives the
// same entropy and probabilities, it just has to keep 2^y inside the fp32 range.
template <int KIND, bool SOFT>
struct Acc {
  uint64_t s2, t2, k2, nc2;  // packed: (even, odd) lanes
  float c, vmax, k;
  // Where vmax was first met: rec >= 0 is the first vector index of a group of kUnroll vectors
  // (the position inside the group is looked up once, after streaming, by the threads that hold
  // the row maximum); rec < 0 is ~element_index, recorded exactly by the scalar path.
  int rec;

  __device__ __forceinline__ void init(float k_) {
    k = k_;
    k2 = f2_pack(k_, k_);
    c = (KIND == SUBSPEC_IN_PROBS) ? 0.f : -INFINITY;
    nc2 = f2_pack(-c, -c);
    s2 = t2 = f2_pack(0.f, 0.f);
    vmax = -INFINITY;
    rec = ~INT_MAX;
  }

  __device__ __forceinline__ void set_ref(float cn) {
    c = cn;
    nc2 = f2_pack(-cn, -cn);
  }

  // Move the shift to cn (first use, or a maximum that outgrew the headroom).
  __device__ __forceinline__ void move_ref(float cn) {
    if (c != -INFINITY) {
      const float d = c - cn;
      const float f = ex2f(d);
      float s0, s1, t0, t1;
      f2_unpack(s2, s0, s1);
      f2_unpack(t2, t0, t1);
      t2 = f2_pack(f * fmaf(d, s0, t0), f * fmaf(d, s1, t1));
      s2 = f2_pack(s0 * f, s1 * f);
    }
    set_ref(cn);
  }

  // Maximum `gm` of a group of vectors starting at vector index v0: branch-free bookkeeping.
  __device__ __forceinline__ void note_group(float gm, int v0) {
    const bool up = gm > vmax;
    vmax = up ? gm : vmax;
    rec = up ? v0 : rec;
    if (SOFT && KIND == SUBSPEC_IN_LOGITS) {
      if (fmaf(gm, k, -c) > kRefHeadroom) move_ref(gm * k);  // first group of the thread; otherwise almost never
    }
  }

  // Two logits (finite, reference already set).
  __device__ __forceinline__ void add_pair(float x0, float x1) {
    const uint64_t y2 = f2_fma(f2_pack(x0, x1), k2, nc2);
    float y0, y1;
    f2_unpack(y2, y0, y1);
    const uint64_t e2 = f2_pack(ex2f(y0), ex2f(y1));
    s2 = f2_add(s2, e2);
    t2 = f2_fma(y2, e2, t2);
  }

  // One value through the scalar path (probabilities, unaligned rows, tails, masked logits).
  __device__ __forceinline__ void one(float x, int idx) {
    if (KIND == SUBSPEC_IN_LOGITS) x = fmaxf(x, -1.0e30f);  // -inf (masked) must not turn 0 * inf into NaN
    if (x > vmax) {
      vmax = x;
      rec = ~idx;
      if (SOFT && KIND == SUBSPEC_IN_LOGITS && fmaf(x, k, -c) > kRefHeadroom) move_ref(x * k);
    }
    if (!SOFT) return;
    float s0, s1, t0, t1;
    f2_unpack(s2, s0, s1);
    f2_unpack(t2, t0, t1);
    if (KIND == SUBSPEC_IN_LOGITS) {
      const float y = fmaf(x, k, -c);
      const float e = ex2f(y);
      s0 += e;
      t0 = fmaf(y, e, t0);
    } else {
      const float l = x > 0.f ? lg2f(x) : 0.f;
      s0 += x;
      t0 = fmaf(x, l, t0);
    }
    s2 = f2_pack(s0, s1);
    t2 = f2_pack(t0, t1);
  }

  // `amax`: exact first index of vmax for this thread (INT_MAX when the thread cannot hold the row maximum).
  __device__ __forceinline__ RowStat stat(int amax) const {
    RowStat r;
    float s0, s1, t0, t1;
    f2_unpack(s2, s0, s1);
    f2_unpack(t2, t0, t1);
    r.c = (vmax == -INFINITY && KIND == SUBSPEC_IN_LOGITS) ? -INFINITY : c;
    r.s = s0 + s1;
    r.t2 = t0 + t1;
    r.vmax = vmax;
    r.amax = amax;
    return r;
  }
};

// ---- consumers of a group of kUnroll 16-byte vectors ----------------------------------------
// The group maximum is formed with packed 16-bit max instructions and compared with the
// running maximum once per group; only when it wins (a handful of times per thread) is the
// group searched for the first position of that value.  Vectors of a group are kThreads
// vectors apart and ascending, so "first in the group" is "lowest vocabulary index".
template <typename T>
struct Vec;

template <>
struct Vec<float> {
  static constexpr int N = 4;
  // Element index of the first value equal to gm in the group of vectors v0, v0 + kThreads, ...
  static __device__ __noinline__ int first_of(const uint4* vp, int v0, float gm) {
    for (int j = 0; j < kUnroll; ++j) {
      const uint4 q = vp[v0 + j * kThreads];
      const float x[4] = {__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w)};
      for (int i = 0; i < 4; ++i)
        if (x[i] == gm) return (v0 + j * kThreads) * N + i;
    }
    return INT_MAX;
  }
  template <int KIND, bool SOFT>
  static __device__ __forceinline__ void consume(Acc<KIND, SOFT>& a, const uint4 (&q)[kUnroll], int v0) {
    float gm = -INFINITY;
#pragma unroll
    for (int j = 0; j < kUnroll; ++j)
      gm = fmaxf(gm, fmaxf(fmaxf(__uint_as_float(q[j].x), __uint_as_float(q[j].y)),
                           fmaxf(__uint_as_float(q[j].z), __uint_as_float(q[j].w))));
    a.note_group(gm, v0);
    if (SOFT) {
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        a.add_pair(__uint_as_float(q[j].x), __uint_as_float(q[j].y));
        a.add_pair(__uint_as_float(q[j].z), __uint_as_float(q[j].w));
      }
    }
  }
};

template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __noinline__ int first_of(const uint4* vp, int v0, float gm) {
    for (int j = 0; j < kUnroll; ++j) {
      const uint4 q = vp[v0 + j * kThreads];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      for (int i = 0; i < 4; ++i) {
        if (__uint_as_float(w[i] << 16) == gm) return (v0 + j * kThreads) * N + 2 * i;
        if (__uint_as_float(w[i] & 0xffff0000u) == gm) return (v0 + j * kThreads) * N + 2 * i + 1;
      }
    }
    return INT_MAX;
  }
  template <int KIND, bool SOFT>
  static __device__ __forceinline__ void consume(Acc<KIND, SOFT>& a, const uint4 (&q)[kUnroll], int v0) {
    __nv_bfloat162 m[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[j]);
      m[j] = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    }
    const __nv_bfloat162 m2 = __hmax2(__hmax2(m[0], m[1]), __hmax2(m[2], m[3]));
    const float gm = fmaxf(__low2float(m2), __high2float(m2));
    a.note_group(gm, v0);
    if (SOFT) {
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) a.add_pair(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
      }
    }
  }
};

template <>
struct Vec<__half> {
  static constexpr int N = 8;
  static __device__ __noinline__ int first_of(const uint4* vp, int v0, float gm) {
    for (int j = 0; j < kUnroll; ++j) {
      const uint4 q = vp[v0 + j * kThreads];
      const __half2* h = reinterpret_cast<const __half2*>(&q);
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        if (f.x == gm) return (v0 + j * kThreads) * N + 2 * i;
        if (f.y == gm) return (v0 + j * kThreads) * N + 2 * i + 1;
      }
    }
    return INT_MAX;
  }
  template <int KIND, bool SOFT>
  static __device__ __forceinline__ void consume(Acc<KIND, SOFT>& a, const uint4 (&q)[kUnroll], int v0) {
    __half2 m[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const __half2* h = reinterpret_cast<const __half2*>(&q[j]);
      m[j] = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    }
    const __half2 m2 = __hmax2(__hmax2(m[0], m[1]), __hmax2(m[2], m[3]));
    const float gm = fmaxf(__low2float(m2), __high2float(m2));
    a.note_group(gm, v0);
    if (SOFT) {
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        const __half2* h = reinterpret_cast<const __half2*>(&q[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          a.add_pair(f.x, f.y);
        }
      }
    }
  }
};

struct Scratch {
  int* seq_ticket;   // [batch]
  int* row_ticket;   // [batch * max_nodes]
  RowStat* partial;  // [batch * max_nodes * kMaxSplits]
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ inline size_t ticket_bytes(int batch, int max_nodes) {
  return align_up(sizeof(int) * ((size_t)batch + (size_t)batch * max_nodes), 256);
}

__host__ __device__ inline Scratch carve(void* base, int batch, int max_nodes) {
  Scratch s;
  s.seq_ticket = reinterpret_cast<int*>(base);
  s.row_ticket = s.seq_ticket + batch;
  s.partial = reinterpret_cast<RowStat*>(reinterpret_cast<char*>(base) + ticket_bytes(batch, max_nodes));
  return s;
}

struct KArgs {
  subspec_verify_args a;
  Scratch sc;
  int splits;
  int vec_ok;  // every row start is 16-byte aligned
  float k;     // log2(e) / temperature
  float remove_below;  // nucleus filter: drop tokens while the ascending cumulative probability is <= this
  float kD;            // residual acceptance: log2(e) / draft temperature
  int dvec_ok;         // every draft row start is 16-byte aligned
  int wide_gates;      // row sampler without the histogram: also entropy and child probabilities (lossy + filters)
  int targets_only;    // row sampler: write node_target and stop, no walk
  int keep_target;     // streaming kernel: node_target already holds the (sampled) targets
};

// Node and row counts of a sequence as every kernel uses them: 0 <= n_rows <= n_nodes <= max_nodes.  Values
// outside that are clamped (the same way in every CTA, so the tickets still add up) and reported.
__device__ __forceinline__ void seq_counts(const subspec_verify_args& a, int b, int& n_nodes, int& n_rows) {
  const int nn = a.n_nodes[b], nr = a.n_rows[b];
  n_nodes = min(max(nn, 0), a.max_nodes);
  n_rows = min(max(nr, 0), n_nodes);
  if (n_nodes != nn || n_rows != nr) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
}
// The children of node u as a range of child_idx, kept inside [0, n_nodes] whatever child_off holds.
__device__ __forceinline__ void child_range(const subspec_verify_args& a, int b, int u, int n_nodes, int& cb, int& ce) {
  const int* coff = a.child_off + (size_t)b * (a.max_nodes + 1);
  const int lo = coff[u], hi = coff[u + 1];
  cb = min(max(lo, 0), n_nodes);
  ce = min(max(hi, cb), n_nodes);
  if (cb != lo || ce != hi) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
}
// A sequence without a decoded row launches no walk: its result is "nothing accepted, nothing emitted".
__device__ __forceinline__ void write_empty_result(const subspec_verify_args& a, int b) {
  int* meta = a.out_meta + (size_t)b * 4;
  meta[0] = meta[1] = meta[2] = meta[3] = 0;
  if (a.method == SUBSPEC_VERIFY_EXACT_AND_LOSSY && a.out2_meta) {
    int* m2 = a.out2_meta + (size_t)b * 4;
    m2[0] = m2[1] = m2[2] = m2[3] = 0;
  }
}

// ---- the accept walk, run by one CTA per sequence out of shared memory -----------
struct WalkSmem {
  int* tok;
  int* tgt;
  float* ent;
  float* cprob;
  int* coff;
  int* cidx;
  int* ea;
  int* bl;
  int* bn;
};

__device__ __forceinline__ WalkSmem carve_walk(unsigned char* base, int n) {
  WalkSmem w;
  int* p = reinterpret_cast<int*>(base);
  w.tok = p;
  p += n;
  w.tgt = p;
  p += n;
  w.ent = reinterpret_cast<float*>(p);
  p += n;
  w.cprob = reinterpret_cast<float*>(p);
  p += n;
  w.coff = p;
  p += n + 1;
  w.cidx = p;
  p += n;
  w.ea = p;
  p += n;
  w.bl = p;
  p += n;
  w.bn = p;
  return w;
}

__device__ void run_walk(const KArgs& ka, int b, unsigned char* smem_raw) {
  const subspec_verify_args& a = ka.a;
  const int N = a.max_nodes;
  int n_nodes, n_rows;
  seq_counts(a, b, n_nodes, n_rows);
  WalkSmem w = carve_walk(smem_raw, N);
  const size_t nb = (size_t)b * N;
  const bool lossy = a.method != SUBSPEC_VERIFY_EXACT;  // the lossy walk runs (alone, or after the exact one)

  for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) {
    w.tok[i] = a.token_ids[nb + i];
    int ci = a.child_idx[nb + i];
    if (ci < 0 || ci >= n_nodes) ci = 0;  // only entries below child_off[n_nodes] are ever read; those were checked
    w.cidx[i] = ci;
    w.ea[i] = 0;
    w.bl[i] = 0;
    w.bn[i] = -1;
    if (i < n_rows) {
      w.tgt[i] = __ldcg(a.node_target + nb + i);
      w.ent[i] = lossy ? __ldcg(a.node_entropy + nb + i) : 0.f;
    } else {
      w.tgt[i] = -1;
      w.ent[i] = 0.f;
    }
    w.cprob[i] = lossy ? __ldcg(a.node_child_prob + nb + i) : 0.f;
  }
  for (int i = threadIdx.x; i <= n_nodes; i += blockDim.x) {
    int o = a.child_off[(size_t)b * (N + 1) + i];
    if (o < 0 || o > n_nodes) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
      o = o < 0 ? 0 : n_nodes;
    }
    w.coff[i] = o;
  }
  __syncthreads();

  if (lossy) {
    // lossy_tree_verify.py:107-168, the reverse-index DP.  A node's (exact_after, best_len, best_next) depend
    // on its children's only, so instead of one thread walking the indices downwards the whole CTA
    // recomputes every node from the current values of its children until a round changes nothing: after
    // round r every node of height <= r holds its final values (the children of a node have larger indices,
    // so the induction is the sequential loop's), and the fixed point is the sequential result.  A tree of
    // height h takes h + 1 rounds; one sequence alone in a launch no longer waits for a 64-step serial loop.
    __shared__ int s_changed;
    const bool use_entropy = a.gate == SUBSPEC_GATE_ENTROPY;
    const double thr = a.threshold;
    const int window = a.window > 0 ? a.window : 0;
    bool settled = false;
    for (int round = 0; round <= n_nodes; ++round) {
      if (threadIdx.x == 0) s_changed = 0;
      __syncthreads();
      bool changed = false;
      for (int u = threadIdx.x; u < n_nodes; u += blockDim.x) {
        const int cb = w.coff[u], ce = w.coff[u + 1];
        if (ce == cb) continue;
        const int tgt = w.tgt[u];
        bool has_exact = false;
        int max_ea = 0;
        for (int e = cb; e < ce; ++e) {
          const int c = w.cidx[e];
          if (w.tok[c] == tgt) {
            has_exact = true;
            max_ea = max(max_ea, w.ea[c]);
          }
        }
        const int ea_u = has_exact ? 1 + max_ea : 0;
        int best_c = -1, best_total = 0;
        bool best_exact = false;
        float best_p = -1.f;
        const bool ent_blocks = use_entropy && ((double)w.ent[u] >= thr);
        for (int e = cb; e < ce; ++e) {
          const int c = w.cidx[e];
          const bool is_exact = w.tok[c] == tgt;
          float p = -1.f;
          if (!is_exact) {
            if (w.ea[c] < window) continue;
            if (ent_blocks) continue;
            p = w.cprob[c];
            if (!use_entropy && (double)p < thr) continue;
          }
          const int tl = 1 + w.bl[c];
          if (tl > best_total) {
            best_c = c;
            best_total = tl;
            best_exact = is_exact;
            best_p = p;
            continue;
          }
          if (tl == best_total) {
            if (is_exact && !best_exact) {
              best_c = c;
              best_exact = true;
              best_p = p;
            } else if (!is_exact && !best_exact && p > best_p) {
              best_c = c;
              best_p = p;
            }
          }
        }
        const int bn_u = (best_c >= 0 && best_total > 0) ? best_c : -1;
        const int bl_u = bn_u >= 0 ? best_total : 0;
        if (ea_u != w.ea[u] || bn_u != w.bn[u] || bl_u != w.bl[u]) {
          w.ea[u] = ea_u;
          w.bn[u] = bn_u;
          w.bl[u] = bl_u;
          changed = true;
        }
      }
      if (changed) s_changed = 1;
      __syncthreads();
      const int again = s_changed;
      __syncthreads();  // everybody has read the flag before the next round clears it
      if (!again) {
        settled = true;
        break;
      }
    }
    // a forest settles within height + 1 <= n_nodes rounds; children lists with a loop in them never do
    if (!settled && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
  }

  if (threadIdx.x == 0) {
    const int max_out = a.max_out;
    const int64_t eos = a.eos;
    int root = a.root[b];
    if (root < 0 || root >= n_rows) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_ROOT);
      root = 0;
    }
    // Pass 0: the exact walk; pass 1: the lossy DP and walk.  SUBSPEC_VERIFY_EXACT_AND_LOSSY runs both on
    // the same per-node targets (one pass over the logits): the exact results then go to the out2_* arrays.
    for (int pass = 0; pass < 2; ++pass) {
    const bool walk_lossy = pass == 1;
    if (walk_lossy ? a.method == SUBSPEC_VERIFY_EXACT : a.method == SUBSPEC_VERIFY_LOSSY) continue;
    const bool second = a.method == SUBSPEC_VERIFY_EXACT_AND_LOSSY && !walk_lossy;
    int64_t* out_tok = (second ? a.out2_tokens : a.out_tokens) + (size_t)b * a.max_out;
    int64_t* out_hid = (second ? a.out2_hidden : a.out_hidden) + (size_t)b * a.max_out;
    int L = 0, acc = 0, total = 0;
    if (!walk_lossy) {
      // tree_verify.py:61-104
      int cur = root;
      int bonus = -1;
      bool go = (w.coff[cur + 1] - w.coff[cur]) > 0;
      while (go) {
        if (total >= n_nodes) {  // a walk over a tree visits every node at most once: the children lists loop
          flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
          break;
        }
        ++total;
        const int s = w.tgt[cur];
        int match = -1;
        for (int e = w.coff[cur]; e < w.coff[cur + 1]; ++e) {
          const int c = w.cidx[e];
          if (w.tok[c] == s) {
            match = c;
            break;
          }
        }
        if (match < 0) {
          bonus = s;
          break;
        }
        ++acc;
        if (L < max_out) {
          out_tok[L] = s;
          out_hid[L] = cur;
        }
        ++L;
        if (eos >= 0 && (int64_t)s == eos) break;
        cur = match;
        const int cb = w.coff[cur], ce = w.coff[cur + 1];
        if (ce - cb == 0) break;
        int mn = INT_MAX;
        for (int e = cb; e < ce; ++e) mn = min(mn, w.cidx[e]);
        if (mn >= n_rows) break;
      }
      const bool ended_on_eos = (L > 0) && (eos >= 0) && (L - 1 < max_out) && (out_tok[L - 1] == eos);
      if (!ended_on_eos) {
        if (bonus < 0) bonus = w.tgt[cur];
        if (L < max_out) {
          out_tok[L] = bonus;
          out_hid[L] = cur;
        }
        ++L;
      }
    } else {
      // lossy_tree_verify.py:247-291: the walk along best_next (the DP has run above, by the whole CTA)
      int ctx = root;
      while (true) {
        const int nxt = w.bn[ctx];
        if (nxt < 0) break;
        if (acc >= n_nodes) {  // longer than any path of a tree: the children lists loop
          flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
          break;
        }
        const int t = w.tok[nxt];
        if (L < max_out) {
          out_tok[L] = t;
          out_hid[L] = ctx;
        }
        ++L;
        ++acc;
        if (eos >= 0 && (int64_t)t == eos) break;
        ctx = nxt;
      }
      const bool ended_on_eos = (L > 0) && (eos >= 0) && (L - 1 < max_out) && (out_tok[L - 1] == eos);
      if (!ended_on_eos) {
        if (L < max_out) {
          out_tok[L] = w.tgt[ctx];
          out_hid[L] = ctx;
        }
        ++L;
      }
      total = L;
    }
    int* meta = (second ? a.out2_meta : a.out_meta) + (size_t)b * 4;
    meta[0] = L < max_out ? L : max_out;
    meta[1] = acc;
    meta[2] = total;
    meta[3] = L > max_out ? 1 : 0;
    }
  }
  __syncthreads();
  if (lossy) {
    for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) {
      a.node_exact_after[nb + i] = w.ea[i];
      a.node_best_len[nb + i] = w.bl[i];
      a.node_best_next[nb + i] = w.bn[i];
    }
  }
}

// CTA-wide combine of the per-thread statistics into *out (shared memory); ends with a barrier.
template <int KIND>
__device__ __forceinline__ void block_reduce(RowStat st, RowStat* s_warp, RowStat* out) {
  st = warp_reduce(st);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // s_warp / *out may still be read from a previous round
  if (lane == 0) s_warp[warp] = st;
  __syncthreads();
  if (warp == 0) {
    st = lane < kWarps ? s_warp[lane] : empty_stat(KIND == SUBSPEC_IN_PROBS);
    st = warp_reduce(st);
    if (lane == 0) *out = st;
  }
  __syncthreads();
}

// ---- the streaming kernel --------------------------------------------------------
template <typename T, int KIND, bool SOFT>
__global__ void __launch_bounds__(kThreads, 4) verify_rows_kernel(const KArgs ka) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ RowStat s_warp[kWarps];
  __shared__ float s_max[kWarps];
  __shared__ __align__(8) uint64_t s_full[kStages];
  __shared__ int s_abort;
  __shared__ RowStat s_row;
  __shared__ int s_flag;

  const subspec_verify_args& a = ka.a;
  const int splits = ka.splits;
  const int row = blockIdx.x / splits;
  const int split = blockIdx.x - row * splits;
  const int b = row / a.max_nodes;
  const int u = row - b * a.max_nodes;
  // A kernel launched behind this one as a programmatic dependent (the KV compaction) may be scheduled once
  // every CTA of this grid has got here or left; it waits for this grid's completion before it reads anything.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int n_nodes, n_rows;
  seq_counts(a, b, n_nodes, n_rows);
  if (u >= n_rows) {
    if (n_rows == 0 && u == 0 && split == 0 && threadIdx.x == 0) write_empty_result(a, b);
    return;
  }

  const int V = a.vocab;
  const T* rowp = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.seq_stride + (size_t)u * a.row_stride;

  Acc<KIND, SOFT> acc;
  acc.init(ka.k);

  constexpr int VN = Vec<T>::N;
  // chunk of this split, in elements; boundaries are multiples of VN
  const int nvec_total = ka.vec_ok ? V / VN : 0;
  const int vec_per_split = (nvec_total + splits - 1) / splits;
  const int v0 = min(split * vec_per_split, nvec_total);
  const int v1 = min(v0 + vec_per_split, nvec_total);
  static_assert(kUnroll == 4, "the group consumers take four vectors");
  if (KIND == SUBSPEC_IN_LOGITS) {
    // The chunk [v0, v1) is staged through a ring of kStages shared-memory buffers by TMA bulk
    // copies that thread 0 issues kStages - 1 stages ahead; every thread then reads its group of
    // kUnroll vectors (kThreads apart, ascending) from shared memory.  The barrier at the top of
    // iteration k proves that stage k - 1 has been read by everyone, so its buffer is refilled.
    const uint4* vp = reinterpret_cast<const uint4*>(rowp);
    uint4* ring = reinterpret_cast<uint4*>(smem_raw);
    const int nst = (v1 - v0 + kStageVecs - 1) / kStageVecs;
    if (threadIdx.x == 0) {
      for (int st = 0; st < kStages; ++st) mbar_init(&s_full[st], 1);
      mbar_init_fence();
      s_abort = 0;
    }
    fence_async_smem();
    __syncthreads();
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
      __syncthreads();
      if (s_abort) break;
      if (threadIdx.x == 0 && st + kStages - 1 < nst) issue(st + kStages - 1);
      if (!mbar_wait_bounded(&s_full[st % kStages], (uint32_t)(st / kStages) & 1u)) s_abort = 1;
      const uint4* buf = ring + (size_t)(st % kStages) * kStageVecs;
      const int a0 = v0 + st * kStageVecs;
      const int i = a0 + threadIdx.x;
      if (a0 + kStageVecs <= v1) {
        uint4 q[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) q[j] = buf[threadIdx.x + j * kThreads];
        Vec<T>::template consume<KIND, SOFT>(acc, q, i);
      } else {
        // last, partial stage: its vectors go element by element through the scalar path
        for (int j = 0; j < kUnroll && i + j * kThreads < v1; ++j) {
          const uint4 q = buf[threadIdx.x + j * kThreads];
          const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
          for (int l = 0; l < VN; ++l) acc.one(to_f32<T>(e[l]), (i + j * kThreads) * VN + l);
        }
      }
    }
    __syncthreads();
    if (s_abort) {  // a bulk copy never completed: report and leave together
      if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_TIMEOUT);
      return;
    }
  } else {
    for (int i = v0 * VN + threadIdx.x; i < v1 * VN; i += kThreads) acc.one(to_f32<T>(rowp[i]), i);
  }
  // scalar remainder (and the whole row when it is not 16-byte aligned): last split only
  if (split == splits - 1) {
    for (int i = nvec_total * VN + threadIdx.x; i < V; i += kThreads) acc.one(to_f32<T>(rowp[i]), i);
  }

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Row (chunk) maximum first; only the threads that hold it look up where in their group it sits.
  {
    float m = acc.vmax;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) s_max[warp] = m;
    __syncthreads();
    m = s_max[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) m = fmaxf(m, s_max[w]);
    int amax = INT_MAX;
    if (acc.vmax == m && m != -INFINITY)
      amax = acc.rec < 0 ? ~acc.rec : Vec<T>::first_of(reinterpret_cast<const uint4*>(rowp), acc.rec, m);
    block_reduce<KIND>(acc.stat(amax), s_warp, &s_row);
  }

  if (splits > 1) {
    if (threadIdx.x == 0) {
      ka.sc.partial[(size_t)row * kMaxSplits + split] = s_row;
      __threadfence();
      const int t = atomicAdd(ka.sc.row_ticket + row, 1);
      s_flag = (t == splits - 1);
      if (s_flag) ka.sc.row_ticket[row] = 0;  // everybody has been: left as found, zero, for the next launch
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
    if (warp == 0) {
      RowStat p = empty_stat(KIND == SUBSPEC_IN_PROBS);
      if (lane < splits) {
        const volatile RowStat* src = ka.sc.partial + (size_t)row * kMaxSplits + lane;
        p.c = src->c;
        p.s = src->s;
        p.t2 = src->t2;
        p.vmax = src->vmax;
        p.amax = src->amax;
      }
      p = warp_reduce(p);
      if (lane == 0) s_row = p;
    }
    __syncthreads();
  }

  // A -inf (masked) logit makes the fast path produce 0 * inf = NaN.  Such rows are rare on this
  // path; the CTA that finalises the row streams it once more through the clamping scalar path.
  if (SOFT && KIND == SUBSPEC_IN_LOGITS && !(isfinite(s_row.s) && isfinite(s_row.t2))) {
    __syncthreads();
    acc.init(ka.k);
    for (int i = threadIdx.x; i < V; i += kThreads) acc.one(to_f32<T>(rowp[i]), i);
    block_reduce<KIND>(acc.stat(acc.rec == ~INT_MAX ? INT_MAX : ~acc.rec), s_warp, &s_row);
  }

  // ---- finalise the row ----
  const RowStat r = s_row;
  const size_t nb = (size_t)b * a.max_nodes;
  if (threadIdx.x == 0) {
    if (!ka.keep_target) a.node_target[nb + u] = r.amax == INT_MAX ? 0 : r.amax;
    float ent = 0.f;
    if (SOFT) {
      const float denom = V > 1 ? logf((float)V) : 1.f;
      if (KIND == SUBSPEC_IN_LOGITS)
        ent = kLn2 * (lg2f(r.s) - r.t2 / r.s) / denom;
      else
        ent = -kLn2 * r.t2 / denom;
    }
    a.node_entropy[nb + u] = ent;
    a.node_rowmax[nb + u] = r.c;
    a.node_rowsum[nb + u] = (KIND == SUBSPEC_IN_PROBS) ? 1.f : r.s;
  }
  if (SOFT) {
    // P[u, token(c)] for every child c of u
    int cb, ce;
    child_range(a, b, u, n_nodes, cb, ce);
    for (int e = cb + threadIdx.x; e < ce; e += kThreads) {
      const int c = a.child_idx[nb + e];
      if (c < 0 || c >= n_nodes) {
        flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
        continue;
      }
      const int tok = a.token_ids[nb + c];
      float p = 0.f;
      if (tok < 0 || tok >= V) {
        flag(a.dev_status, SUBSPEC_DEV_BAD_TOKEN);
      } else {
        const float x = to_f32<T>(rowp[tok]);
        p = (KIND == SUBSPEC_IN_PROBS) ? x : ex2f(fmaf(x, ka.k, -r.c)) / r.s;
      }
      a.node_child_prob[nb + c] = p;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(ka.sc.seq_ticket + b, 1);
    s_flag = (t == n_rows - 1);
    if (s_flag) ka.sc.seq_ticket[b] = 0;
  }
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  run_walk(ka, b, smem_raw);
}

// ---- sampled target tokens: temperature + nucleus (top-p) + inverse-CDF pick -----------------
//
// One CTA per [vocab] row of 16-bit logits.  A 16-bit float has only 65536 values, so a COUNT
// histogram over all of them (128 KB of shared memory, two 16-bit counters per word) describes the
// row's distribution exactly: the softmax denominator, the nucleus boundary value and how many
// of the tokens tied at that value fall outside the nucleus all follow from it, with one
// exponential per distinct value instead of one per token.  A second sweep over the row (served
// by L2) then adds up, chunk by chunk in vocabulary order, the mass that survives the filter, and
// the chunk / element where the cumulative mass passes u * Z is the sampled token.
//
// Filter semantics = transformers' TopPLogitsWarper (min_tokens_to_keep = 1) applied to
// logits / temperature, as the reference's _sample_token does (generators/base.py:57-62, 116-126):
// ascending stable sort, remove while the cumulative probability is <= 1 - top_p, never remove
// the last.  Among tokens tied at the boundary value the lowest vocabulary indices go first.
constexpr int kSThreads = 1024;
constexpr int kSWarps = kSThreads / 32;
constexpr int kHistWords = 32768;   // 65536 16-bit counters
constexpr int kChunkElems = 256;    // one warp sweep: 32 lanes x 8 elements
constexpr int kMaxChunks = (1 << 20) / kChunkElems;
constexpr size_t kSampleSmem = sizeof(uint32_t) * kHistWords + (sizeof(float) + sizeof(uint32_t)) * kMaxChunks;

template <typename T>
struct Bits16;
template <>
struct Bits16<__nv_bfloat16> {
  static constexpr uint32_t kNegInf = 0xFF80u;
  static __device__ __forceinline__ float value(uint32_t bits) { return __uint_as_float(bits << 16); }
};
template <>
struct Bits16<__half> {
  static constexpr uint32_t kNegInf = 0xFC00u;
  static __device__ __forceinline__ float value(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
  }
};
// order-preserving key of a 16-bit float pattern, and back
__device__ __forceinline__ uint32_t key_of(uint32_t bits) {
  return (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
}
__device__ __forceinline__ uint32_t bits_of(uint32_t key) {
  return (key & 0x8000u) ? (key & 0x7FFFu) : (~key & 0xFFFFu);
}
// The histogram is indexed by the RAW 16-bit pattern (no key arithmetic per counted element): counter
// `bits` is half (bits & 1) of word bits >> 1.  A "row" is 32 words = 64 consecutive patterns = 64
// consecutive keys (ascending patterns for positive floats, descending for negative ones), and thread t
// of the scans owns the row of keys [64 t, 64 t + 64).  Word w lives at hist_pos(w): the 16-byte groups
// of a row are XOR-rotated by the row number, so that the 128-bit loads of a quarter-warp (eight
// threads, eight consecutive rows) hit eight different bank groups.
__device__ __forceinline__ uint32_t hist_pos(uint32_t w) { return w ^ (((w >> 5) & 7u) << 2); }
// Eight consecutive raw 16-bit patterns starting at element i0 (a multiple of 8); elements at or beyond
// V read as -inf.
template <typename T>
__device__ __forceinline__ void load8(const T* rowp, int i0, int V, bool vec_ok, uint32_t (&b)[8]) {
  if (vec_ok && i0 + 8 <= V) {
    const uint4 q = *reinterpret_cast<const uint4*>(rowp + i0);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      b[2 * j] = w[j] & 0xFFFFu;
      b[2 * j + 1] = w[j] >> 16;
    }
  } else {
    const unsigned short* p = reinterpret_cast<const unsigned short*>(rowp);
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = (i0 + j < V) ? (uint32_t)p[i0 + j] : Bits16<T>::kNegInf;
  }
}

// The same eight patterns, still packed two to a word (element i0 + 2 j in the low half of word j).
template <typename T>
__device__ __forceinline__ uint4 load8_packed(const T* rowp, int i0, int V, bool vec_ok) {
  if (vec_ok && i0 + 8 <= V) return *reinterpret_cast<const uint4*>(rowp + i0);
  uint32_t b[8];
  load8<T>(rowp, i0, V, false, b);
  return make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16));
}
__device__ __forceinline__ void unpack8(const uint4& q, uint32_t (&b)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[2 * j] = w[j] & 0xFFFFu;
    b[2 * j + 1] = w[j] >> 16;
  }
}
// the eight values as floats, straight from the packed words
__device__ __forceinline__ void unpack8_values(const uint4& q, float (&v)[8], __nv_bfloat16) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void unpack8_values(const uint4& q, float (&v)[8], __half) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
constexpr int kSweepDepth = 4;  // chunks a warp has in flight in the two sweeps over the row

__device__ __forceinline__ double shfl_up_f64(double v, int d) {
  int lo = __double2loint(v), hi = __double2hiint(v);
  lo = __shfl_up_sync(0xffffffffu, lo, d);
  hi = __shfl_up_sync(0xffffffffu, hi, d);
  return __hiloint2double(hi, lo);
}
__device__ __forceinline__ double shfl_xor_f64(double v, int mask) {
  int lo = __double2loint(v), hi = __double2hiint(v);
  lo = __shfl_xor_sync(0xffffffffu, lo, mask);
  hi = __shfl_xor_sync(0xffffffffu, hi, mask);
  return __hiloint2double(hi, lo);
}
// inclusive scan over the warp
__device__ __forceinline__ double warp_scan_f64(double v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const double o = shfl_up_f64(v, d);
    if (lane >= d) v += o;
  }
  return v;
}
__device__ __forceinline__ int warp_scan_i32(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += o;
  }
  return v;
}

struct SampleShared {
  double warp_tot[kSWarps];
  double S, cum_before, Z;
  float c, e_b;
  double cbase;
  double T2;
  int kmax, k_b, r, n_b, finite, counted, flag, first, last_nz, cstar, T0, k_k, itotal, rank;
  int tie_chunk, tie_T0, tie_cut;  // where the run of values tied at the boundary is cut, in vocabulary order
  int warp_max[kSWarps];
};

// The whole row pipeline for row u of sequence b, run by one 1024-thread CTA: writes node_target (and the
// row statistics; entropy and child probabilities too unless the method is the exact walk) and ends with a
// CTA barrier.  False when the row could not be processed (reported through dev_status); every thread
// returns the same value.
template <typename T>
__device__ bool sample_row(const KArgs& ka, SampleShared& sh, unsigned char* smem_raw, int b, int u) {
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw);
  float* ch_mass = reinterpret_cast<float*>(hist + kHistWords);
  uint32_t* ch_ties = reinterpret_cast<uint32_t*>(ch_mass + kMaxChunks);

  const subspec_verify_args& a = ka.a;
  const int V = a.vocab;
  const T* rowp = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.seq_stride + (size_t)u * a.row_stride;
  const bool vec_ok = ka.vec_ok != 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float kT = ka.k;

  // ---- 0. clear the histogram ----
  for (int i = tid; i < kHistWords / 4; i += kSThreads) reinterpret_cast<uint4*>(hist)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    sh.finite = 0;
    sh.counted = 0;
    sh.k_k = 0;
  }
  __syncthreads();

  // ---- 1. count every value of the row (HBM pass) ----
  const int nchunks = (V + kChunkElems - 1) / kChunkElems;
  int n_finite = 0;
  // a warp keeps kSweepDepth chunk loads in flight: one 16-byte load per thread at a time would leave the
  // SM with 16 KB outstanding, a third of what its share of the HBM bandwidth needs
  constexpr uint32_t kNegInf2 = Bits16<T>::kNegInf | (Bits16<T>::kNegInf << 16);
  for (int c0 = warp; c0 < nchunks; c0 += kSweepDepth * kSWarps) {
    uint4 raw[kSweepDepth];
#pragma unroll
    for (int d = 0; d < kSweepDepth; ++d) {
      const int c = c0 + d * kSWarps;
      raw[d] = c < nchunks ? load8_packed<T>(rowp, c * kChunkElems + lane * 8, V, vec_ok)
                           : make_uint4(kNegInf2, kNegInf2, kNegInf2, kNegInf2);
    }
#pragma unroll
    for (int d = 0; d < kSweepDepth; ++d) {
      uint32_t bits[8];
      unpack8(raw[d], bits);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t bj = bits[j];
        if (bj != Bits16<T>::kNegInf) {  // masked: no mass, and often far too many to count
          atomicAdd(&hist[hist_pos(bj >> 1)], 1u + (bj & 1u) * 0xFFFFu);  // no return value: a reduction
          ++n_finite;
        }
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) n_finite += __shfl_xor_sync(0xffffffffu, n_finite, off);
  if (lane == 0 && n_finite) atomicAdd(&sh.finite, n_finite);
  __syncthreads();

  // ---- 2. the histogram: maximum, denominator, nucleus boundary ----
  // Thread t owns keys [64 t, 64 t + 64) = one row of raw patterns, walked downwards for the negative
  // floats (t < 512) and upwards for the positive ones.  visit(f) calls f(count, key) for the row's
  // non-empty counters in ascending key order; empty 16-byte groups and words cost one test each.
  const bool desc = tid < kSThreads / 2;
  const uint32_t rowi = desc ? (uint32_t)(kSThreads - 1 - tid) : (uint32_t)(tid - kSThreads / 2);
  const uint4* row4 = reinterpret_cast<const uint4*>(hist) + rowi * 8;
  auto visit = [&](auto&& f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int gi = desc ? 7 - i : i;
      const uint4 q = row4[gi ^ (int)(rowi & 7u)];
      if ((q.x | q.y | q.z | q.w) == 0u) continue;
      const uint32_t wd[4] = {desc ? q.w : q.x, desc ? q.z : q.y, desc ? q.y : q.z, desc ? q.x : q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w = wd[j];
        if (w == 0u) continue;
        const uint32_t c0 = desc ? (w >> 16) : (w & 0xFFFFu), c1 = desc ? (w & 0xFFFFu) : (w >> 16);
        const int key = tid * 64 + i * 8 + j * 2;
        if (c0) f(c0, key);
        if (c1) f(c1, key + 1);
      }
    }
  };
  auto count_of = [&](int key) -> int {  // one counter, by key
    const uint32_t pat = bits_of((uint32_t)key);
    const uint32_t w = hist[hist_pos(pat >> 1)];
    return (int)((pat & 1u) ? (w >> 16) : (w & 0xFFFFu));
  };
  // this thread's highest occupied key: the row's eight 16-byte groups in ascending key order, one compare
  // and select per counter, no branches
  int kmax = -1;
  int N_all = 0;  // elements in this thread's 64 counters
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gi = desc ? 7 - i : i;
    const uint4 q = row4[gi ^ (int)(rowi & 7u)];
    const uint32_t wd[4] = {desc ? q.w : q.x, desc ? q.z : q.y, desc ? q.y : q.z, desc ? q.x : q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = desc ? (wd[j] >> 16) : (wd[j] & 0xFFFFu), hi = desc ? (wd[j] & 0xFFFFu) : (wd[j] >> 16);
      kmax = lo ? i * 8 + j * 2 : kmax;
      kmax = hi ? i * 8 + j * 2 + 1 : kmax;
      N_all += (int)(lo + hi);
    }
  }
  if (kmax >= 0) kmax += tid * 64;
  // counter of this thread's m-th key (0..63, ascending), for the walks that one thread does alone
  auto counter_at = [&](int m) -> int {
    const int gi = desc ? 7 - (m >> 3) : (m >> 3);
    const int wj = desc ? 3 - ((m >> 1) & 3) : ((m >> 1) & 3);
    const uint32_t w = hist[(rowi * 8 + (uint32_t)(gi ^ (int)(rowi & 7u))) * 4 + (uint32_t)wj];
    const bool high = desc ? (m & 1) == 0 : (m & 1) != 0;
    return (int)(high ? (w >> 16) : (w & 0xFFFFu));
  };
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, off));
  if (lane == 0) sh.warp_max[warp] = kmax;
  __syncthreads();
  if (tid == 0) {
    int m = -1;
    for (int w = 0; w < kSWarps; ++w) m = max(m, sh.warp_max[w]);
    sh.kmax = m;
    sh.c = m >= 0 ? Bits16<T>::value(bits_of((uint32_t)m)) * kT : 0.f;
  }
  __syncthreads();
  const int K_max = sh.kmax;
  const size_t nb = (size_t)b * a.max_nodes;
  // ---- top-k (TopKLogitsWarper): every value below the k-th largest goes; k_k = lowest key that stays ----
  if (ka.a.top_k > 0 && K_max >= 0) {
    const int incl = warp_scan_i32(N_all);
    if (lane == 31) sh.warp_max[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int x = sh.warp_max[lane];
      const int xs = warp_scan_i32(x);
      sh.warp_max[lane] = xs - x;
      if (lane == 31) sh.itotal = xs;
    }
    __syncthreads();
    const int above = sh.itotal - (sh.warp_max[warp] + incl);  // elements with keys above this thread's range
    if (N_all > 0 && above < ka.a.top_k && ka.a.top_k <= above + N_all) {
      int need = ka.a.top_k - above;
      for (int m = 63; m >= 0; --m) {
        need -= counter_at(m);
        if (need <= 0) {
          sh.k_k = tid * 64 + m;
          break;
        }
      }
    }
    __syncthreads();
  }
  const int k_k = sh.k_k;
  if (K_max < 0) {  // nothing but -inf / empty: no distribution to sample from
    if (sh.finite != 0) {  // ... or 65536 copies of one value wrapped its counter to zero
      if (tid == 0) flag(a.dev_status, SUBSPEC_DEV_HIST_OVERFLOW);
      return false;
    }
    if (tid == 0) {
      a.node_target[nb + u] = 0;
      a.node_entropy[nb + u] = 0.f;
      a.node_rowmax[nb + u] = 0.f;
      a.node_rowsum[nb + u] = 0.f;
    }
    if (a.method != SUBSPEC_VERIFY_EXACT) {  // no child of this node has any probability
      int n_nodes, n_rows_unused, cb, ce;
      seq_counts(a, b, n_nodes, n_rows_unused);
      child_range(a, b, u, n_nodes, cb, ce);
      for (int e = cb + tid; e < ce; e += kSThreads) {
        const int cnode = a.child_idx[nb + e];
        if (cnode >= 0 && cnode < n_nodes) a.node_child_prob[nb + cnode] = 0.f;
      }
    }
  } else {
    const float c = sh.c;
    // Masses of this thread's values, ascending; and how many elements the counters hold.  Within a thread
    // (64 keys) the sums run in single precision; double precision, slow on this part, is kept for the
    // scan across threads and for the handful of scalars derived from it.
    // An empty 16-byte group costs one test; inside a non-empty one all eight counters are processed
    // without branches (an empty counter adds nothing), which gives the same partial sums as visiting the
    // non-empty ones alone.
    float m32 = 0.f;
    int N_t = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int gi = desc ? 7 - i : i;
      const uint4 q = row4[gi ^ (int)(rowi & 7u)];
      if ((q.x | q.y | q.z | q.w) == 0u) continue;
      const uint32_t wd[4] = {desc ? q.w : q.x, desc ? q.z : q.y, desc ? q.y : q.z, desc ? q.x : q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t c0 = desc ? (wd[j] >> 16) : (wd[j] & 0xFFFFu), c1 = desc ? (wd[j] & 0xFFFFu) : (wd[j] >> 16);
        const int key = tid * 64 + i * 8 + j * 2;
        const float e0 = ex2f(fmaf(Bits16<T>::value(bits_of((uint32_t)key)), kT, -c));
        const float e1 = ex2f(fmaf(Bits16<T>::value(bits_of((uint32_t)key + 1u)), kT, -c));
        const float s0 = fmaf((float)c0, e0, m32);
        m32 = (c0 && key >= k_k) ? s0 : m32;  // what top-k removed carries no mass
        const float s1 = fmaf((float)c1, e1, m32);
        m32 = (c1 && key + 1 >= k_k) ? s1 : m32;
        N_t += (int)(c0 + c1);
      }
    }
    const double M_t = (double)m32;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) N_t += __shfl_xor_sync(0xffffffffu, N_t, off);
    if (lane == 0 && N_t) atomicAdd(&sh.counted, N_t);
    // block exclusive scan of M_t in key order
    const double incl = warp_scan_f64(M_t);
    if (lane == 31) sh.warp_tot[warp] = incl;
    __syncthreads();
    if (sh.counted != sh.finite) {
      // a 16-bit counter wrapped (one value more than 65535 times in the row): the counters no longer add
      // up to the number of elements counted, whichever way the carry went
      if (tid == 0) flag(a.dev_status, SUBSPEC_DEV_HIST_OVERFLOW);
      return false;
    }
    // the 32 warp totals are scanned by one warp, not added up by every thread: double-precision adds are
    // the slowest instructions this kernel has
    if (warp == 0) {
      const double x = sh.warp_tot[lane];
      const double xs = warp_scan_f64(x);
      sh.warp_tot[lane] = xs - x;
      if (lane == 31) sh.S = xs;
    }
    __syncthreads();
    const double total = sh.S;
    const double P_t = sh.warp_tot[warp] + incl - M_t;
    const double thrS = (double)ka.remove_below * total;  // remove while cumulative mass <= thrS
    if (tid == 0) {
      // default: the filter is off, or the threshold is never passed (keep only the last of the maximum)
      sh.k_b = -1;
      sh.r = 0;
      sh.n_b = 0;
      sh.e_b = 0.f;
      sh.cum_before = 0.0;
    }
    __syncthreads();
    if (ka.remove_below > 0.f) {
      if (M_t > 0.0 && P_t <= thrS && thrS < P_t + M_t) {
        // the same single-precision partial sums as above, against the threshold's distance from this
        // thread's base; the boundary key is the first whose run of equal values passes it (the last
        // non-empty key if rounding lets none pass)
        const float rem = (float)(thrS - P_t);
        float loc = 0.f, loc_b = 0.f, e_k = 0.f;
        int key_b = -1, n_k = 0;
        bool found = false;
        visit([&](uint32_t cnt, int key) {
          if (found || key < k_k) return;
          const float e = ex2f(fmaf(Bits16<T>::value(bits_of((uint32_t)key)), kT, -c));
          const float nxt = fmaf((float)cnt, e, loc);
          key_b = key;
          n_k = (int)cnt;
          e_k = e;
          loc_b = loc;
          if (nxt > rem)
            found = true;
          else
            loc = nxt;
        });
        const double cum = P_t + (double)loc_b;
        int r = found ? (int)floor((thrS - cum) / (double)e_k) : n_k;
        r = min(max(r, 0), n_k);
        if (key_b == K_max) r = min(r, n_k - 1);
        sh.k_b = key_b;
        sh.r = r;
        sh.n_b = n_k;
        sh.e_b = e_k;
        sh.cum_before = cum;
      }
      __syncthreads();
      if (tid == 0 && sh.k_b < 0) {
        // thrS >= total (top_p ~ 0): everything below the maximum goes, and all but the last of the maximum
        sh.k_b = K_max;
        const int n = count_of(K_max);
        const float e = ex2f(fmaf(Bits16<T>::value(bits_of((uint32_t)K_max)), kT, -c));
        sh.n_b = n;
        sh.r = n - 1;
        sh.e_b = e;
        sh.cum_before = total - (double)n * (double)e;
      }
    }
    __syncthreads();
    if (tid == 0 && k_k > 0 && sh.k_b < k_k) {
      // no nucleus boundary above the top-k cut: the cut is the boundary, as a key just below it whose own
      // elements (if any) carry no mass
      sh.k_b = k_k - 1;
      sh.r = 0;
      sh.n_b = 0;
      sh.e_b = 0.f;
      sh.cum_before = 0.0;
    }
    __syncthreads();
    const int k_b = sh.k_b, r_rm = sh.r;
    const float e_b = sh.e_b;
    if (tid == 0) {
      sh.Z = sh.S - sh.cum_before - (double)r_rm * (double)e_b;
      sh.T2 = 0.0;
    }
    __syncthreads();

    // ---- 2b. lossy verification on sampled targets: entropy of the filtered distribution and the
    // filtered probability of every child's token (lossy_tree_verify.py:66-72, 135-146) ----
    if (a.method != SUBSPEC_VERIFY_EXACT) {
      // sum of e * y over the survivors (y = log2 of the unnormalised mass), from the histogram
      float t2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int gi = desc ? 7 - i : i;
        const uint4 q = row4[gi ^ (int)(rowi & 7u)];
        if ((q.x | q.y | q.z | q.w) == 0u) continue;
        const uint32_t wd[4] = {desc ? q.w : q.x, desc ? q.z : q.y, desc ? q.y : q.z, desc ? q.x : q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t cn[2] = {desc ? (wd[j] >> 16) : (wd[j] & 0xFFFFu), desc ? (wd[j] & 0xFFFFu) : (wd[j] >> 16)};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int key = tid * 64 + i * 8 + j * 2 + h;
            const float y = fmaf(Bits16<T>::value(bits_of((uint32_t)key)), kT, -c);
            // above the boundary everything stays; at it, what the nucleus filter left of the run of equal
            // values (nothing when the boundary is only the top-k cut, which has e_b = 0)
            const float wgt = key > k_b ? (float)cn[h]
                                        : ((key == k_b && e_b > 0.f) ? (float)max((int)cn[h] - r_rm, 0) : 0.f);
            t2 += wgt > 0.f ? wgt * ex2f(y) * y : 0.f;
          }
        }
      }
      double t2d = (double)t2;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) t2d += shfl_xor_f64(t2d, off);
      if (lane == 0 && t2d != 0.0) atomicAdd(&sh.T2, t2d);
      __syncthreads();
      const float Zf = (float)sh.Z;
      if (tid == 0) {
        const float denom = V > 1 ? logf((float)V) : 1.f;
        a.node_entropy[nb + u] = kLn2 * (lg2f(Zf) - (float)sh.T2 / Zf) / denom;
      }
      // children of u
      int n_nodes, n_rows_unused, cb, ce;
      seq_counts(a, b, n_nodes, n_rows_unused);
      child_range(a, b, u, n_nodes, cb, ce);
      for (int e = cb; e < ce; ++e) {  // the same trip count and decisions in every thread
        const int cnode = a.child_idx[nb + e];
        if (cnode < 0 || cnode >= n_nodes) {
          if (tid == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
          continue;
        }
        const int tok = a.token_ids[nb + cnode];
        float p = 0.f;
        if (tok < 0 || tok >= V) {
          if (tid == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_TOKEN);
        } else {
          const uint32_t pat = reinterpret_cast<const unsigned short*>(rowp)[tok];
          const int key = pat == Bits16<T>::kNegInf ? -1 : (int)key_of(pat);
          if (key > k_b) {
            p = ex2f(fmaf(Bits16<T>::value(pat), kT, -c)) / Zf;
          } else if (key == k_b && e_b > 0.f && r_rm < sh.n_b) {
            bool stays = r_rm == 0;
            if (!stays) {
              // part of the run of equal values stays: this token does if at least r_rm equal values
              // precede it in the vocabulary
              int before = 0;
              for (int i0 = tid * 8; i0 < tok; i0 += kSThreads * 8) {
                uint32_t bits[8];
                load8<T>(rowp, i0, V, vec_ok, bits);
#pragma unroll
                for (int j = 0; j < 8; ++j) before += (i0 + j < tok && bits[j] == pat) ? 1 : 0;
              }
#pragma unroll
              for (int off = 16; off > 0; off >>= 1) before += __shfl_xor_sync(0xffffffffu, before, off);
              if (tid == 0) sh.rank = 0;
              __syncthreads();
              if (lane == 0 && before) atomicAdd(&sh.rank, before);
              __syncthreads();
              stays = sh.rank >= r_rm;
              __syncthreads();
            }
            p = stays ? e_b / Zf : 0.f;
          }
        }
        if (tid == 0) a.node_child_prob[nb + cnode] = p;
      }
    }

    // ---- 3. second sweep: surviving mass and boundary ties per chunk, vocabulary order (L2 pass) ----
    // Survivors are the values above the boundary value, ties the values equal to it: float compares, except
    // when the boundary is one of the two zeros, which compare equal as floats but are two keys.
    const uint32_t pat_b = k_b >= 0 ? bits_of((uint32_t)k_b) : (uint32_t)Bits16<T>::kNegInf;
    const float v_b = Bits16<T>::value(pat_b);
    const bool zero_boundary = k_b >= 0 && (pat_b & 0x7FFFu) == 0u;
    for (int c0 = warp; c0 < nchunks; c0 += kSweepDepth * kSWarps) {
      uint4 raw[kSweepDepth];
#pragma unroll
      for (int d = 0; d < kSweepDepth; ++d) {
        const int cidx = c0 + d * kSWarps;
        raw[d] = cidx < nchunks ? load8_packed<T>(rowp, cidx * kChunkElems + lane * 8, V, vec_ok)
                                : make_uint4(kNegInf2, kNegInf2, kNegInf2, kNegInf2);
      }
      float mass[kSweepDepth];
      int ties[kSweepDepth];
#pragma unroll
      for (int d = 0; d < kSweepDepth; ++d) {
        mass[d] = 0.f;
        ties[d] = 0;
        if (!zero_boundary) {
          float v[8];
          unpack8_values(raw[d], v, T());
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (v[j] > v_b) mass[d] += ex2f(fmaf(v[j], kT, -c));
            ties[d] += (v[j] == v_b) ? 1 : 0;
          }
        } else {
          uint32_t bits[8];
          unpack8(raw[d], bits);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (bits[j] == Bits16<T>::kNegInf) continue;
            const int key = (int)key_of(bits[j]);
            if (key > k_b)
              mass[d] += ex2f(fmaf(Bits16<T>::value(bits[j]), kT, -c));
            else if (key == k_b)
              ++ties[d];
          }
        }
      }
      // the warp sums of the chunks in flight, their shuffle chains interleaved
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int d = 0; d < kSweepDepth; ++d) {
          mass[d] += __shfl_xor_sync(0xffffffffu, mass[d], off);
          ties[d] += __shfl_xor_sync(0xffffffffu, ties[d], off);
        }
      }
      if (lane < kSweepDepth) {
        const int cidx = c0 + lane * kSWarps;
        if (cidx < nchunks) {
          float m = mass[0];
          int t = ties[0];
#pragma unroll
          for (int d = 1; d < kSweepDepth; ++d)
            if (lane == d) {
              m = mass[d];
              t = ties[d];
            }
          ch_mass[cidx] = m;
          ch_ties[cidx] = (uint32_t)t;
        }
      }
    }
    __syncthreads();

    // ---- 4. locate the chunk where the cumulative surviving mass passes u * Z: the whole block, each
    // thread a run of `per` consecutive chunks (one, up to 262144 tokens), two block scans ----
    const double Z = sh.Z;
    const double target = (double)a.uniforms[nb + u] * Z;
    const int per = (nchunks + kSThreads - 1) / kSThreads;
    const int c0 = min(tid * per, nchunks), c1 = min(c0 + per, nchunks);
    int tl = 0;
    for (int cc = c0; cc < c1; ++cc) tl += (int)ch_ties[cc];
    if (tid == 0) {
      sh.first = kSThreads;
      sh.last_nz = -1;
      sh.tie_chunk = -1;
    }
    // exclusive block scan of the tie counts
    int T_thread0;
    {
      const int incl = warp_scan_i32(tl);
      if (lane == 31) sh.warp_max[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        const int x = sh.warp_max[lane];
        sh.warp_max[lane] = warp_scan_i32(x) - x;
      }
      __syncthreads();
      T_thread0 = sh.warp_max[warp] + incl - tl;
    }
    if (r_rm > 0 && r_rm < sh.n_b && T_thread0 <= r_rm && r_rm < T_thread0 + tl) {
      // the nucleus filter removes the first r_rm of the values tied at the boundary: the tie of rank r_rm
      // (the first that stays) is in one of this thread's chunks
      int Trun = T_thread0;
      for (int cc = c0; cc < c1; ++cc) {
        const int T1 = Trun + (int)ch_ties[cc];
        if (r_rm < T1) {
          sh.tie_chunk = cc;
          sh.tie_T0 = Trun;
          break;
        }
        Trun = T1;
      }
    }
    double local = 0.0;
    {
      int Trun = T_thread0;
      for (int cc = c0; cc < c1; ++cc) {
        const int T1 = Trun + (int)ch_ties[cc];
        local += (double)ch_mass[cc] + (double)e_b * (double)(max(T1 - r_rm, 0) - max(Trun - r_rm, 0));
        Trun = T1;
      }
    }
    // exclusive block scan of the surviving mass, thread order = vocabulary order
    double lbase;
    {
      const double incl = warp_scan_f64(local);
      if (lane == 31) sh.warp_tot[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        const double x = sh.warp_tot[lane];
        sh.warp_tot[lane] = warp_scan_f64(x) - x;
      }
      __syncthreads();
      lbase = sh.warp_tot[warp] + incl - local;
    }
    if (local > 0.0) {
      if (lbase + local > target) atomicMin(&sh.first, tid);
      atomicMax(&sh.last_nz, tid);
    }
    __syncthreads();
    // no crossing (u * Z rounds up to the total): the last token with surviving mass
    const bool pick_last = sh.first == kSThreads;
    const int L = pick_last ? max(sh.last_nz, 0) : sh.first;
    if (tid == L) {
      double cum = lbase;
      int Trun = T_thread0;
      int cstar = c0, T0 = Trun;
      double cbase = cum;
      for (int cc = c0; cc < c1; ++cc) {
        const int T1 = Trun + (int)ch_ties[cc];
        const double cm = (double)ch_mass[cc] + (double)e_b * (double)(max(T1 - r_rm, 0) - max(Trun - r_rm, 0));
        if (cm > 0.0) {  // candidate: the crossing chunk, or (pick_last) the last chunk with mass
          cstar = cc;
          T0 = Trun;
          cbase = cum;
          if (!pick_last && cum + cm > target) break;
        }
        cum += cm;
        Trun = T1;
      }
      sh.cstar = min(cstar, nchunks - 1);
      sh.T0 = T0;
      sh.cbase = cbase;
    }
    __syncthreads();

    // ---- 5. the element inside that chunk: one warp ----
    if (warp == 0) {
      const int cstar = sh.cstar, T0 = sh.T0;
      const double cbase = sh.cbase;

      uint32_t bits[8];
      load8<T>(rowp, cstar * kChunkElems + lane * 8, V, vec_ok, bits);
      int lt = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (bits[j] != Bits16<T>::kNegInf && (int)key_of(bits[j]) == k_b) ++lt;
      int trank = T0 + warp_scan_i32(lt) - lt;
      float km[8];
      double lsum = 0.0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        km[j] = 0.f;
        if (bits[j] == Bits16<T>::kNegInf) continue;
        const int key = (int)key_of(bits[j]);
        if (key > k_b) {
          km[j] = ex2f(fmaf(Bits16<T>::value(bits[j]), kT, -c));
        } else if (key == k_b) {
          km[j] = trank >= r_rm ? e_b : 0.f;
          ++trank;
        }
        lsum += (double)km[j];
      }
      const double eincl = warp_scan_f64(lsum);
      double run = cbase + eincl - lsum;
      int pick = -1, last = -1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (km[j] > 0.f) {
          last = lane * 8 + j;
          run += (double)km[j];
          if (pick < 0 && run > target) pick = lane * 8 + j;
        }
      }
      const uint32_t hit = __ballot_sync(0xffffffffu, pick >= 0);
      const uint32_t any = __ballot_sync(0xffffffffu, last >= 0);
      int within;
      if (hit && !pick_last) {
        within = __shfl_sync(0xffffffffu, pick, __ffs(hit) - 1);
      } else {
        within = any ? __shfl_sync(0xffffffffu, last, 31 - __clz(any)) : 0;
      }
      // vocabulary index from which the values tied at the boundary stay in the distribution
      int tie_cut = r_rm == 0 ? 0 : V;
      if (sh.tie_chunk >= 0) {
        uint32_t tb[8];
        load8<T>(rowp, sh.tie_chunk * kChunkElems + lane * 8, V, vec_ok, tb);
        int lt2 = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (tb[j] != Bits16<T>::kNegInf && (int)key_of(tb[j]) == k_b) ++lt2;
        int rank = sh.tie_T0 + warp_scan_i32(lt2) - lt2;
        int found = -1;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (tb[j] != Bits16<T>::kNegInf && (int)key_of(tb[j]) == k_b) {
            if (rank == r_rm && found < 0) found = sh.tie_chunk * kChunkElems + lane * 8 + j;
            ++rank;
          }
        const uint32_t who = __ballot_sync(0xffffffffu, found >= 0);
        if (who) tie_cut = __shfl_sync(0xffffffffu, found, __ffs(who) - 1);
      }
      if (lane == 0) sh.tie_cut = tie_cut;
      if (lane == 0) {
        a.node_target[nb + u] = min(cstar * kChunkElems + within, V - 1);
        if (a.method == SUBSPEC_VERIFY_EXACT) a.node_entropy[nb + u] = 0.f;
        a.node_rowmax[nb + u] = c;
        a.node_rowsum[nb + u] = (float)Z;
      }
    }
  }
  __syncthreads();
  return true;
}

// ---- sampled targets without the 16-bit histogram: fp32 logits, or probabilities of any type --------------
//
// A 32-bit float has too many values to count, so the filters' boundaries are found by searching the
// order-preserving 32-bit key space with counting passes over the row (served by L2 after the first): three
// thresholds per pass, seventeen passes per search.  top-k: the largest key t with count(key >= t) >= k;
// top-p: the largest key t with mass(key < t) <= (1 - top_p) Z.  Ties at the top-p boundary are cut in
// vocabulary order (lowest indices go first), as in the 16-bit pipeline.  Probabilities come in unfiltered
// (the reference's lossy_bottom_up_verify draws torch.multinomial(probs), lossy_tree_verify.py:75-77).
// Slower per row than the histogram pipeline; the walk-driven kernel samples only a handful of rows.
template <typename T>
struct WideRow;
template <>
struct WideRow<float> {
  static constexpr int E = 4;  // elements per lane and chunk
  static __device__ __forceinline__ void load(const float* rowp, int i0, int V, bool vec_ok, float (&v)[4]) {
    if (vec_ok && i0 + 4 <= V) {
      const float4 q = *reinterpret_cast<const float4*>(rowp + i0);
      v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = (i0 + j < V) ? rowp[i0 + j] : __uint_as_float(0xFFFFFFFFu);
    }
  }
};
template <typename T16>
struct WideRow16 {
  static constexpr int E = 8;
  static __device__ __forceinline__ void load(const T16* rowp, int i0, int V, bool vec_ok, float (&v)[8]) {
    unpack8_values(load8_packed<T16>(rowp, i0, V, vec_ok), v, T16());
    if (i0 + 8 > V) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i0 + j >= V) v[j] = __uint_as_float(0xFFFFFFFFu);
    }
  }
};
template <>
struct WideRow<__nv_bfloat16> : WideRow16<__nv_bfloat16> {};
template <>
struct WideRow<__half> : WideRow16<__half> {};

// Order-preserving key of a float.  Padding (the negative NaN of all ones) has key 0 and -inf has key
// 0x007FFFFF: everything with mass has a key of at least kKeyFloor.
__device__ __forceinline__ uint32_t key32(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float value_of_key32(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
constexpr uint32_t kKeyFloor = 0x00800000u;

// sum (or maximum) over the CTA of one double per thread; every thread gets the result
__device__ __forceinline__ double block_reduce_f64(double v, SampleShared& sh, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const double o = shfl_xor_f64(v, off);
    v = is_max ? fmax(v, o) : v + o;
  }
  __syncthreads();  // warp_tot may still be read from a previous round
  if (lane == 0) sh.warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double t = sh.warp_tot[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const double o = shfl_xor_f64(t, off);
      t = is_max ? fmax(t, o) : t + o;
    }
    if (lane == 0) sh.S = t;
  }
  __syncthreads();
  return sh.S;
}

// exclusive prefix over the CTA (thread order) of one double per thread, and the total
__device__ __forceinline__ double block_excl_scan_f64(double v, SampleShared& sh, double* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const double incl = warp_scan_f64(v);
  __syncthreads();
  if (lane == 31) sh.warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const double x = sh.warp_tot[lane];
    const double xi = warp_scan_f64(x);
    sh.warp_tot[lane] = xi - x;
    if (lane == 31) sh.S = xi;
  }
  __syncthreads();
  *total = sh.S;
  return sh.warp_tot[warp] + incl - v;
}

template <typename T, int KIND>
__device__ bool sample_row_wide(const KArgs& ka, SampleShared& sh, unsigned char* smem_raw, int b, int u) {
  using Row = WideRow<T>;
  constexpr int E = Row::E;
  constexpr int kElems = 32 * E;       // one warp sweep
  constexpr int kWideDepth = 16 / E;   // chunk loads a warp keeps in flight
  float* ch_mass = reinterpret_cast<float*>(smem_raw);           // up to 2^20 / 128 = 8192 chunks
  int* ch_cnt = reinterpret_cast<int*>(smem_raw) + (1 << 13);

  const subspec_verify_args& a = ka.a;
  const int V = a.vocab;
  const T* rowp = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.seq_stride + (size_t)u * a.row_stride;
  const bool vec_ok = ka.vec_ok != 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t nb = (size_t)b * a.max_nodes;
  const int nchunks = (V + kElems - 1) / kElems;
  const float kT = ka.k;
  constexpr bool kLogits = KIND == SUBSPEC_IN_LOGITS;

  // f(values, first index) for every chunk of the row, kWideDepth chunk loads in flight per warp
  auto sweep = [&](auto&& f) {
    for (int c0 = warp; c0 < nchunks; c0 += kWideDepth * kSWarps) {
      float v[kWideDepth][E];
#pragma unroll
      for (int d = 0; d < kWideDepth; ++d) {
        const int c = c0 + d * kSWarps;
        if (c < nchunks) Row::load(rowp, c * kElems + lane * E, V, vec_ok, v[d]);
      }
#pragma unroll
      for (int d = 0; d < kWideDepth; ++d) {
        const int c = c0 + d * kSWarps;
        if (c < nchunks) f(v[d], c);
      }
    }
  };

  // ---- 1. the row maximum (logits) ----
  uint32_t kmax = 0xFFFFFFFFu;
  float c = 0.f;
  if (kLogits) {
    uint32_t m = 0;
    sweep([&](const float(&v)[E], int) {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const uint32_t k = key32(v[j]);
        if (k <= 0xFF800000u) m = max(m, k);  // up to +inf; NaNs are left out
      }
    });
    kmax = (uint32_t)block_reduce_f64((double)m, sh, true);
    if (kmax < kKeyFloor) {  // nothing but -inf: no distribution to draw from
      if (tid == 0) {
        a.node_target[nb + u] = 0;
        if (a.method == SUBSPEC_VERIFY_EXACT) a.node_entropy[nb + u] = 0.f;
        a.node_rowmax[nb + u] = 0.f;
        a.node_rowsum[nb + u] = 0.f;
        if (ka.wide_gates) a.node_entropy[nb + u] = 0.f;
      }
      if (ka.wide_gates) {  // no distribution: every child has probability zero
        int n_nodes, n_rows_unused, cb, ce;
        seq_counts(a, b, n_nodes, n_rows_unused);
        child_range(a, b, u, n_nodes, cb, ce);
        for (int e = cb + tid; e < ce; e += kSThreads) {
          const int cn = a.child_idx[nb + e];
          if (cn >= 0 && cn < n_nodes) a.node_child_prob[nb + cn] = 0.f;
        }
      }
      __syncthreads();
      return true;
    }
    c = value_of_key32(kmax) * kT;
  }
  auto weight = [&](float x) -> float { return kLogits ? ex2f(fmaf(x, kT, -c)) : x; };

  // Largest key t in [lo, hi] for which pred_of(counts) holds, given that it holds at lo and is monotone
  // (true below, false above).  measure(v, t0, t1, t2, acc) adds a chunk's contribution for three thresholds.
  auto search = [&](uint32_t lo, uint32_t hi, auto&& measure, auto&& holds) -> uint32_t {
    uint64_t good = lo, bad = (uint64_t)hi + 1;  // holds at good, fails at bad (or bad is past the range)
    while (bad - good > 1) {
      const uint64_t span = bad - good;
      uint32_t t[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        uint64_t x = good + (span * (uint64_t)(j + 1)) / 4;
        if (x <= good) x = good + 1;
        if (x >= bad) x = bad - 1;
        t[j] = (uint32_t)x;
      }
      float acc[3] = {0.f, 0.f, 0.f};
      sweep([&](const float(&v)[E], int) { measure(v, t, acc); });
      double tot[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) tot[j] = block_reduce_f64((double)acc[j], sh, false);
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        if (holds(tot[j])) {
          if ((uint64_t)t[j] > good) good = t[j];
        } else {
          if ((uint64_t)t[j] < bad) bad = t[j];
        }
      }
    }
    return (uint32_t)good;
  };

  // ---- 2. top-k: everything below the k-th largest value goes, ties with it stay ----
  uint32_t kk = kKeyFloor;
  if (kLogits && a.top_k > 0 && a.top_k < V) {
    const double want = (double)a.top_k;
    const uint32_t kth = search(
        0u, kmax,
        [&](const float(&v)[E], const uint32_t(&t)[3], float(&acc)[3]) {
#pragma unroll
          for (int j = 0; j < E; ++j) {
            const uint32_t k = key32(v[j]);
            const bool counted = k != 0u && k <= 0xFF800000u;  // padding and NaNs are no candidates
#pragma unroll
            for (int q = 0; q < 3; ++q) acc[q] += (counted && k >= t[q]) ? 1.f : 0.f;
          }
        },
        [&](double n) { return n >= want; });
    kk = max(kth, kKeyFloor);
  }

  // ---- 3. the denominator over what top-k left ----
  double Z;
  {
    float acc = 0.f;
    sweep([&](const float(&v)[E], int) {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const uint32_t k = key32(v[j]);
        acc += (k >= kk && k <= kmax) ? weight(v[j]) : 0.f;
      }
    });
    Z = block_reduce_f64((double)acc, sh, false);
  }

  // ---- 4. top-p: drop the ascending prefix whose cumulative probability is <= 1 - top_p, keep the largest ----
  uint32_t kb = kk;   // smallest key that (partly) survives
  int tie_cut = 0;    // of the elements tied at kb, those from this vocabulary index on survive
  if (kLogits && ka.remove_below > 0.f) {
    const double thrZ = (double)ka.remove_below * Z;
    kb = search(
        kk, kmax,
        [&](const float(&v)[E], const uint32_t(&t)[3], float(&acc)[3]) {
#pragma unroll
          for (int j = 0; j < E; ++j) {
            const uint32_t k = key32(v[j]);
            const float w = (k >= kk && k <= kmax) ? weight(v[j]) : 0.f;
#pragma unroll
            for (int q = 0; q < 3; ++q) acc[q] += k < t[q] ? w : 0.f;
          }
        },
        [&](double m) { return m <= thrZ; });
    // at the boundary: mass strictly below, the number of ties, how many of them go
    float below = 0.f;
    sweep([&](const float(&v)[E], int cidx) {
      int n = 0;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const uint32_t k = key32(v[j]);
        below += (k >= kk && k < kb) ? weight(v[j]) : 0.f;
        n += k == kb;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) n += __shfl_xor_sync(0xffffffffu, n, off);
      if (lane == 0) ch_cnt[cidx] = n;
    });
    const double mass_below = block_reduce_f64((double)below, sh, false);  // its barriers publish ch_cnt
    const int per = (nchunks + kSThreads - 1) / kSThreads;
    const int c0 = min(tid * per, nchunks), c1 = min(c0 + per, nchunks);
    int local = 0;
    for (int cc = c0; cc < c1; ++cc) local += ch_cnt[cc];
    double n_b_d;
    const double before = block_excl_scan_f64((double)local, sh, &n_b_d);
    const int n_b = (int)n_b_d;
    const float e_b = weight(value_of_key32(kb));
    int r = 0;
    if (thrZ >= mass_below) r = e_b > 0.f ? (int)fmin(floor((thrZ - mass_below) / (double)e_b), 2.0e9) : n_b;
    r = min(r, kb == kmax ? n_b - 1 : n_b);
    r = max(r, 0);
    if (tid == 0) sh.tie_cut = 0;
    __syncthreads();
    if (r > 0) {
      // the r-th tie in vocabulary order (1-based): the cut sits right behind it
      if ((int)before < r && r <= (int)before + local) {
        int seen = (int)before, cstar = c0;
        for (int cc = c0; cc < c1; ++cc) {
          if (seen + ch_cnt[cc] >= r) {
            cstar = cc;
            break;
          }
          seen += ch_cnt[cc];
        }
        sh.cstar = cstar;
        sh.rank = r - seen;  // which tie inside that chunk
      }
      __syncthreads();
      if (warp == 0) {
        const int cstar = sh.cstar, want = sh.rank;
        float v[E];
        Row::load(rowp, cstar * kElems + lane * E, V, vec_ok, v);
        int n = 0;
#pragma unroll
        for (int j = 0; j < E; ++j) n += key32(v[j]) == kb;
        int seen = warp_scan_i32(n) - n;
#pragma unroll
        for (int j = 0; j < E; ++j)
          if (key32(v[j]) == kb) {
            ++seen;
            if (seen == want) sh.tie_cut = cstar * kElems + lane * E + j + 1;
          }
      }
      __syncthreads();
    }
    tie_cut = sh.tie_cut;
  }

  // ---- 5. the draw: inverse CDF over the survivors in vocabulary order ----
  auto kept = [&](float x, int idx) -> float {
    const uint32_t k = key32(x);
    const bool in = k <= kmax && (k > kb || (k == kb && k >= kKeyFloor && idx >= tie_cut));
    return in ? weight(x) : 0.f;
  };
  // (with the lossy gates wanted from this kernel: also T2 = sum of w * log2(w) over the survivors, for the
  // entropy of the filtered distribution)
  const bool gates = kLogits && ka.wide_gates != 0;
  float t2_acc = 0.f;
  sweep([&](const float(&v)[E], int cidx) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float w = kept(v[j], cidx * kElems + lane * E + j);
      m += w;
      if (gates) t2_acc += w > 0.f ? w * fmaf(v[j], kT, -c) : 0.f;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m += __shfl_xor_sync(0xffffffffu, m, off);
    if (lane == 0) ch_mass[cidx] = m;
  });
  const double T2 = gates ? block_reduce_f64((double)t2_acc, sh, false) : 0.0;
  if (tid == 0) {
    sh.first = kSThreads;
    sh.last_nz = -1;
  }
  __syncthreads();
  const int per = (nchunks + kSThreads - 1) / kSThreads;
  const int c0 = min(tid * per, nchunks), c1 = min(c0 + per, nchunks);
  double local = 0.0;
  for (int cc = c0; cc < c1; ++cc) local += (double)ch_mass[cc];
  double Zs;
  const double lbase = block_excl_scan_f64(local, sh, &Zs);
  const double target = (double)a.uniforms[nb + u] * Zs;
  if (local > 0.0) {
    if (lbase + local > target) atomicMin(&sh.first, tid);
    atomicMax(&sh.last_nz, tid);
  }
  __syncthreads();
  const bool pick_last = sh.first == kSThreads;
  const int Lt = pick_last ? max(sh.last_nz, 0) : sh.first;
  if (tid == Lt) {
    double cum = lbase, cbase = lbase;
    int cstar = c0;
    for (int cc = c0; cc < c1; ++cc) {
      const double cm = (double)ch_mass[cc];
      if (cm > 0.0) {
        cstar = cc;
        cbase = cum;
        if (!pick_last && cum + cm > target) break;
      }
      cum += cm;
    }
    sh.cstar = min(cstar, nchunks - 1);
    sh.cbase = cbase;
  }
  __syncthreads();
  if (warp == 0) {
    const int cstar = sh.cstar;
    const int i0 = cstar * kElems + lane * E;
    float v[E], m[E];
    Row::load(rowp, i0, V, vec_ok, v);
    double lsum = 0.0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      m[j] = kept(v[j], i0 + j);
      lsum += (double)m[j];
    }
    const double eincl = warp_scan_f64(lsum);
    double run = sh.cbase + eincl - lsum;
    int hit = -1, last = -1;
#pragma unroll
    for (int j = 0; j < E; ++j)
      if (m[j] > 0.f) {
        last = lane * E + j;
        run += (double)m[j];
        if (hit < 0 && run > target) hit = lane * E + j;
      }
    const uint32_t hits = __ballot_sync(0xffffffffu, hit >= 0);
    const uint32_t any = __ballot_sync(0xffffffffu, last >= 0);
    int within;
    if (hits && !pick_last)
      within = __shfl_sync(0xffffffffu, hit, __ffs(hits) - 1);
    else
      within = any ? __shfl_sync(0xffffffffu, last, 31 - __clz(any)) : 0;
    if (lane == 0) {
      a.node_target[nb + u] = min(cstar * kElems + within, V - 1);
      if (a.method == SUBSPEC_VERIFY_EXACT) a.node_entropy[nb + u] = 0.f;
      a.node_rowmax[nb + u] = c;
      a.node_rowsum[nb + u] = (float)Zs;
      if (gates) {  // entropy of the filtered distribution, normalised by ln V as the reference does
        const float denom = V > 1 ? logf((float)V) : 1.f;
        a.node_entropy[nb + u] = Zs > 0.0 ? (float)(0.6931471805599453 * (log2(Zs) - T2 / Zs)) / denom : 0.f;
      }
    }
  }
  if (gates) {
    // P[u, token(c)] under the filters, for every child c of u
    int n_nodes, n_rows_unused, cb, ce;
    seq_counts(a, b, n_nodes, n_rows_unused);
    child_range(a, b, u, n_nodes, cb, ce);
    const float invZ = Zs > 0.0 ? (float)(1.0 / Zs) : 0.f;
    for (int e = cb + tid; e < ce; e += kSThreads) {
      const int cn = a.child_idx[nb + e];
      if (cn < 0 || cn >= n_nodes) {
        flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
        continue;
      }
      const int tk = a.token_ids[nb + cn];
      float p = 0.f;
      if (tk < 0 || tk >= V)
        flag(a.dev_status, SUBSPEC_DEV_BAD_TOKEN);
      else
        p = kept(to_f32<T>(rowp[tk]), tk) * invZ;
      a.node_child_prob[nb + cn] = p;
    }
  }
  __syncthreads();
  return true;
}

// One CTA per decoded row; the CTA that finishes a sequence's last row runs the walk (lossy DP on sampled
// targets, or the exact walk when every row's target is wanted).
template <typename T, int KIND>
__global__ void __launch_bounds__(kSThreads, 1) verify_sample_rows_kernel(const KArgs ka) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ SampleShared sh;
  constexpr bool kWide = sizeof(T) == 4 || KIND == SUBSPEC_IN_PROBS;
  const subspec_verify_args& a = ka.a;
  const int row = blockIdx.x;
  const int b = row / a.max_nodes;
  const int u = row - b * a.max_nodes;
  int n_nodes, n_rows;
  seq_counts(a, b, n_nodes, n_rows);
  if (u >= n_rows) {
    if (n_rows == 0 && u == 0 && threadIdx.x == 0 && !ka.targets_only) write_empty_result(a, b);
    return;
  }
  if constexpr (kWide) {
    if (!sample_row_wide<T, KIND>(ka, sh, smem_raw, b, u)) return;
  } else {
    if (!sample_row<T>(ka, sh, smem_raw, b, u)) return;
  }
  if (ka.targets_only) return;  // the streaming kernel that follows takes the targets from node_target
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(ka.sc.seq_ticket + b, 1);
    sh.flag = (t == n_rows - 1);
    if (sh.flag) ka.sc.seq_ticket[b] = 0;
  }
  __syncthreads();
  if (!sh.flag) return;
  __threadfence();
  run_walk(ka, b, smem_raw);
}

// ---- residual (p - q) acceptance at one context: block-wide helpers ---------------------------------------
// The filtered target distribution of the row sample_row has just processed, evaluable per element:
// p(v) = 2^(x kT - c) / Z for a survivor of the filters, 0 otherwise.  Survivors are the values above the
// boundary value, and of the values tied at it those from vocabulary index tie_cut on.
template <typename T>
struct TargetDist {
  float kT, c, invZ, v_b;
  int k_b, tie_cut;
  bool ties_live, zero_boundary;
  __device__ __forceinline__ void from(const SampleShared& sh, float kT_) {
    kT = kT_;
    c = sh.c;
    invZ = (float)(1.0 / sh.Z);
    k_b = sh.k_b;
    const uint32_t pat_b = k_b >= 0 ? bits_of((uint32_t)k_b) : (uint32_t)Bits16<T>::kNegInf;
    v_b = Bits16<T>::value(pat_b);
    zero_boundary = k_b >= 0 && (pat_b & 0x7FFFu) == 0u;
    ties_live = k_b >= 0 && sh.e_b > 0.f;
    tie_cut = sh.tie_cut;
  }
  __device__ __forceinline__ bool tie_ok(uint32_t pat, int idx) const {
    if (zero_boundary) {  // the two zeros compare equal as floats but are two keys
      const int key = (int)key_of(pat);
      if (key != k_b) return key > k_b;
    }
    return ties_live && idx >= tie_cut;
  }
  __device__ __forceinline__ float p(uint32_t pat, float v, int idx) const {
    bool surv = v > v_b;
    if (v == v_b) surv = tie_ok(pat, idx);
    return surv ? ex2f(fmaf(v, kT, -c)) * invZ : 0.f;
  }
};

__device__ __forceinline__ double block_sum_f64(double v, SampleShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += shfl_xor_f64(v, off);
  __syncthreads();  // warp_tot may still be read from a previous round
  if (lane == 0) sh.warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double t = sh.warp_tot[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += shfl_xor_f64(t, off);
    if (lane == 0) sh.S = t;
  }
  __syncthreads();
  return sh.S;
}

// do_sample == 2: only the contexts the walk visits are sampled -- what the reference's walker does
// (tree_verify.py:61-104 with classic_sd.py:111-116 draws at the context it stands on) -- by one CTA per
// sequence that alternates the row pipeline with one step of the exact walk.  A sequence touches a
// handful of its rows instead of all of them.
template <typename T, int KIND>
__global__ void __launch_bounds__(kSThreads, 1) verify_sample_walk_kernel(const KArgs ka) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ SampleShared sh;
  constexpr bool kWide = sizeof(T) == 4 || KIND == SUBSPEC_IN_PROBS;  // no histogram pipeline, no residual mode
  __shared__ int s_cur, s_state;  // context to sample next; 1 = walk on, 2 = sample the bonus, 0 = done
  __shared__ int s_dec, s_pick;   // residual acceptance: the accepted child (-1: rejected); the bonus drawn
  __shared__ float s_a, s_zr, s_dmax;  // residual p' ~ max(p - a q, 0) / zr; maximum of the draft row
  const subspec_verify_args& a = ka.a;
  const int b = blockIdx.x, N = a.max_nodes;
  const size_t nb = (size_t)b * N;
  int n_nodes, n_rows;
  seq_counts(a, b, n_nodes, n_rows);
  const int* coff_raw = a.child_off + (size_t)b * (N + 1);
  // children offsets as read, kept inside [0, n_nodes]: whatever they hold, child_idx is read inside the sequence
  auto coff = [&](int i) { return min(max(coff_raw[i], 0), n_nodes); };
  for (int i = threadIdx.x; i <= n_nodes; i += kSThreads)
    if (coff_raw[i] < 0 || coff_raw[i] > n_nodes) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
  const int* cidx = a.child_idx + nb;
  const int* tok = a.token_ids + nb;
  for (int i = threadIdx.x; i < N; i += kSThreads) a.node_target[nb + i] = -1;  // not visited
  // walk state, thread 0 only
  int64_t* out_tok = a.out_tokens + (size_t)b * a.max_out;
  int64_t* out_hid = a.out_hidden + (size_t)b * a.max_out;
  const int max_out = a.max_out;
  const int64_t eos = a.eos;
  // (thread 0's walk state lives in shared memory: registers are short around the row pipeline)
  __shared__ int s_walk[5];
  int &L = s_walk[0], &acc = s_walk[1], &total = s_walk[2], &bonus = s_walk[3], &cur = s_walk[4];
  if (threadIdx.x == 0) {
    L = 0, acc = 0, total = 0, bonus = -1;
    cur = a.root[b];
    if (cur < 0 || cur >= n_rows) {
      flag(a.dev_status, SUBSPEC_DEV_BAD_ROOT);
      cur = 0;
    }
    const bool go = n_nodes > 0 && (coff(cur + 1) - coff(cur)) > 0;
    s_cur = cur;
    s_state = n_nodes > 0 ? (go ? 1 : 2) : 0;
  }
  __syncthreads();
  int visits = 0;  // the same count in every thread: one context per round of the loop
  while (s_state != 0) {
    if (++visits > n_nodes + 1) {  // a walk stands on every node at most once (plus the bonus draw): the lists loop
      if (threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
      break;
    }
    const int state = s_state, ctx = s_cur;
    int tgt = -1;
    if (ctx < n_rows) {
      if constexpr (kWide) {
        if (!sample_row_wide<T, KIND>(ka, sh, smem_raw, b, ctx)) return;
      } else {
        if (!sample_row<T>(ka, sh, smem_raw, b, ctx)) return;  // reported through dev_status
      }
      tgt = a.node_target[nb + ctx];  // written inside this CTA, before its last barrier
    }
    if constexpr (!kWide) if (a.acceptance == 1 && state == 1 && ctx < n_rows) {
      // ---- residual acceptance at this context (every branch below is taken by the whole CTA) ----
      const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
      const int V = a.vocab;
      const T* trow = reinterpret_cast<const T*>(a.logits) + (size_t)b * a.seq_stride + (size_t)ctx * a.row_stride;
      const T* drow = reinterpret_cast<const T*>(a.draft_logits) + (size_t)b * a.draft_seq_stride +
                      (size_t)ctx * a.draft_row_stride;
      const bool tvec = ka.vec_ok != 0, dvec = ka.dvec_ok != 0;
      const int nchunks = (V + kChunkElems - 1) / kChunkElems;
      float* ch_mass = reinterpret_cast<float*>(reinterpret_cast<uint32_t*>(smem_raw) + kHistWords);
      TargetDist<T> tp;
      tp.from(sh, ka.k);
      const float kD = ka.kD;
      // draft row: maximum, then the softmax denominator
      float dmax = -INFINITY;
      for (int cidx2 = warp; cidx2 < nchunks; cidx2 += kSWarps) {
        float v[8];
        unpack8_values(load8_packed<T>(drow, cidx2 * kChunkElems + lane * 8, V, dvec), v, T());
#pragma unroll
        for (int j = 0; j < 8; ++j) dmax = fmaxf(dmax, v[j]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, off));
      __syncthreads();  // warp_tot may still be read from the row pipeline
      if (lane == 0) sh.warp_tot[warp] = (double)dmax;
      __syncthreads();
      if (warp == 0) {
        float t = (float)sh.warp_tot[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
        if (lane == 0) s_dmax = fmaxf(t, -3.0e38f);
      }
      __syncthreads();
      const float cD = s_dmax * kD;
      double dsum = 0.0;
      {
        float acc32 = 0.f;
        for (int cidx2 = warp; cidx2 < nchunks; cidx2 += kSWarps) {
          float v[8];
          unpack8_values(load8_packed<T>(drow, cidx2 * kChunkElems + lane * 8, V, dvec), v, T());
#pragma unroll
          for (int j = 0; j < 8; ++j) acc32 += ex2f(fmaf(v[j], kD, -cD));
        }
        dsum = block_sum_f64((double)acc32, sh);
      }
      const float invS = (float)(1.0 / dsum);
      // residual mass sum_v max(p(v) - coef q(v), 0), and optionally its per-chunk parts
      auto residual_pass = [&](float coef, bool keep_chunks) -> double {
        float acc32 = 0.f;
        for (int cidx2 = warp; cidx2 < nchunks; cidx2 += kSWarps) {
          const int i0 = cidx2 * kChunkElems + lane * 8;
          uint32_t tb[8];
          float tv[8], dv[8];
          const uint4 tq = load8_packed<T>(trow, i0, V, tvec);
          unpack8(tq, tb);
          unpack8_values(tq, tv, T());
          unpack8_values(load8_packed<T>(drow, i0, V, dvec), dv, T());
          float m = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float q = ex2f(fmaf(dv[j], kD, -cD)) * invS;
            m += fmaxf(fmaf(-coef, q, tp.p(tb[j], tv[j], i0 + j)), 0.f);
          }
          if (keep_chunks) {
            float cm = m;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) cm += __shfl_xor_sync(0xffffffffu, cm, off);
            if (lane == 0) ch_mass[cidx2] = cm;
          }
          acc32 += m;
        }
        return block_sum_f64((double)acc32, sh);
      };
      if (tid == 0) {
        s_a = 0.f;
        s_zr = 1.f;
        s_dec = -1;
        ++total;
      }
      __syncthreads();
      const int cb = coff(ctx), ce = coff(ctx + 1);
      for (int e = cb; e < ce; ++e) {
        if (tid == 0) {
          const int cnode = cidx[e];
          int dec = -1;
          if (cnode < 0 || cnode >= n_nodes) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
          } else {
            const int x = tok[cnode];
            if (x < 0 || x >= V) {
              flag(a.dev_status, SUBSPEC_DEV_BAD_TOKEN);
            } else if (s_zr > 0.f) {
              const uint32_t tpat = reinterpret_cast<const unsigned short*>(trow)[x];
              const uint32_t dpat = reinterpret_cast<const unsigned short*>(drow)[x];
              const float px = tp.p(tpat, Bits16<T>::value(tpat), x);
              const float qx = ex2f(fmaf(Bits16<T>::value(dpat), kD, -cD)) * invS;
              const float r = fmaxf(fmaf(-s_a, qx, px), 0.f) / s_zr;
              const float ratio = qx > 0.f ? r / qx : (r > 0.f ? INFINITY : 0.f);
              if (a.accept_uniforms[nb + cnode] < fminf(1.f, ratio)) dec = cnode;
            }
          }
          s_dec = dec;
        }
        __syncthreads();
        if (s_dec >= 0) break;
        // rejected: p' <- normalise(max(p' - q, 0)), i.e. coefficient a + zr and a new normaliser
        const float coef = s_a + s_zr;
        const double z = residual_pass(coef, false);
        if (tid == 0) {
          s_a = coef;
          s_zr = (float)z;
        }
        __syncthreads();
      }
      if (s_dec < 0) {
        // no child accepted: the bonus is the inverse-CDF draw from the residual (from p itself when the
        // residual has no mass left), in vocabulary order
        int pick = tgt;
        if (s_a > 0.f && s_zr > 0.f) {
          const float coef = s_a;
          const double zsum = residual_pass(coef, true);
          const double target = (double)a.uniforms[nb + ctx] * zsum;
          // chunk: first whose inclusive cumulative mass passes the target
          const int per = (nchunks + kSThreads - 1) / kSThreads;
          const int c0 = min(tid * per, nchunks), c1 = min(c0 + per, nchunks);
          double local = 0.0;
          for (int cc = c0; cc < c1; ++cc) local += (double)ch_mass[cc];
          if (tid == 0) {
            sh.first = kSThreads;
            sh.last_nz = -1;
          }
          const double incl = warp_scan_f64(local);
          __syncthreads();
          if (lane == 31) sh.warp_tot[warp] = incl;
          __syncthreads();
          if (warp == 0) {
            const double x = sh.warp_tot[lane];
            sh.warp_tot[lane] = warp_scan_f64(x) - x;
          }
          __syncthreads();
          const double lbase = sh.warp_tot[warp] + incl - local;
          if (local > 0.0) {
            if (lbase + local > target) atomicMin(&sh.first, tid);
            atomicMax(&sh.last_nz, tid);
          }
          __syncthreads();
          const bool pick_last = sh.first == kSThreads;
          const int Lt = pick_last ? max(sh.last_nz, 0) : sh.first;
          if (tid == Lt) {
            double cum = lbase;
            int cstar = c0;
            double cbase = cum;
            for (int cc = c0; cc < c1; ++cc) {
              const double cm = (double)ch_mass[cc];
              if (cm > 0.0) {
                cstar = cc;
                cbase = cum;
                if (!pick_last && cum + cm > target) break;
              }
              cum += cm;
            }
            sh.cstar = min(cstar, nchunks - 1);
            sh.cbase = cbase;
          }
          __syncthreads();
          if (warp == 0) {
            const int cstar = sh.cstar;
            const int i0 = cstar * kChunkElems + lane * 8;
            uint32_t tb[8];
            float tv[8], dv[8], rm[8];
            const uint4 tq = load8_packed<T>(trow, i0, V, tvec);
            unpack8(tq, tb);
            unpack8_values(tq, tv, T());
            unpack8_values(load8_packed<T>(drow, i0, V, dvec), dv, T());
            double lsum = 0.0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float q = ex2f(fmaf(dv[j], kD, -cD)) * invS;
              rm[j] = fmaxf(fmaf(-coef, q, tp.p(tb[j], tv[j], i0 + j)), 0.f);
              lsum += (double)rm[j];
            }
            const double eincl = warp_scan_f64(lsum);
            double run = sh.cbase + eincl - lsum;
            int hit = -1, last = -1;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (rm[j] > 0.f) {
                last = lane * 8 + j;
                run += (double)rm[j];
                if (hit < 0 && run > target) hit = lane * 8 + j;
              }
            const uint32_t hits = __ballot_sync(0xffffffffu, hit >= 0);
            const uint32_t any = __ballot_sync(0xffffffffu, last >= 0);
            int within;
            if (hits && !pick_last)
              within = __shfl_sync(0xffffffffu, hit, __ffs(hits) - 1);
            else
              within = any ? __shfl_sync(0xffffffffu, last, 31 - __clz(any)) : 0;
            if (lane == 0) s_pick = min(cstar * kChunkElems + within, V - 1);
          }
          __syncthreads();
          pick = s_pick;
        }
        if (tid == 0) {
          if (L < max_out) {
            out_tok[L] = pick;
            out_hid[L] = ctx;
          }
          ++L;
          s_state = 0;
        }
      } else if (tid == 0) {
        // accepted child: emit its token, move there; a leaf or an undecoded level ends the walk with a
        // fresh draw at that context (state 2), as in the sample-and-match walk
        const int cnode = s_dec;
        const int x = tok[cnode];
        ++acc;
        if (L < max_out) {
          out_tok[L] = x;
          out_hid[L] = ctx;
        }
        ++L;
        cur = cnode;
        s_cur = cur;
        if (eos >= 0 && (int64_t)x == eos) {
          s_state = 0;
        } else {
          const int cb2 = coff(cur), ce2 = coff(cur + 1);
          bool more = ce2 - cb2 > 0;
          if (more) {
            int mn = INT_MAX;
            for (int e2 = cb2; e2 < ce2; ++e2) mn = min(mn, cidx[e2]);
            if (mn >= n_rows) more = false;
          }
          s_state = more ? 1 : 2;
        }
      }
      __syncthreads();
      continue;
    }
    if (threadIdx.x == 0) {
      if (state == 2) {  // the bonus token of the final context
        if (L < max_out) {
          out_tok[L] = tgt;
          out_hid[L] = ctx;
        }
        ++L;
        s_state = 0;
      } else {  // one step of tree_verify.py:61-104
        ++total;
        int match = -1;
        for (int e = coff(cur); e < coff(cur + 1); ++e) {
          const int c = cidx[e];
          if (c < 0 || c >= n_nodes) {
            flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
            continue;
          }
          if (tok[c] == tgt) {
            match = c;
            break;
          }
        }
        bool stop = false;
        if (match < 0) {
          bonus = tgt;
          stop = true;
        } else {
          ++acc;
          if (L < max_out) {
            out_tok[L] = tgt;
            out_hid[L] = cur;
          }
          ++L;
          if (eos >= 0 && (int64_t)tgt == eos) {
            stop = true;
          } else {
            cur = match;
            const int cb = coff(cur), ce = coff(cur + 1);
            if (ce - cb == 0) {
              stop = true;
            } else {
              int mn = INT_MAX;
              for (int e = cb; e < ce; ++e) mn = min(mn, cidx[e]);
              if (mn >= n_rows) stop = true;
            }
          }
        }
        if (!stop) {
          s_cur = cur;
        } else {
          const bool ended_on_eos = (L > 0) && (eos >= 0) && (L - 1 < max_out) && (out_tok[L - 1] == eos);
          if (ended_on_eos) {
            s_state = 0;
          } else if (bonus >= 0) {  // the draw that missed every child is the bonus
            if (L < max_out) {
              out_tok[L] = bonus;
              out_hid[L] = cur;
            }
            ++L;
            s_state = 0;
          } else {  // stopped on a context that has not drawn yet
            s_cur = cur;
            s_state = 2;
          }
        }
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int* meta = a.out_meta + (size_t)b * 4;
    meta[0] = L < max_out ? L : max_out;
    meta[1] = acc;
    meta[2] = total;
    meta[3] = L > max_out ? 1 : 0;
  }
}

template <typename T, int KIND>
cudaError_t launch_sample_walk(const KArgs& ka, int batch, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(verify_sample_walk_kernel<T, KIND>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSampleSmem);
  if (e != cudaSuccess) return e;
  verify_sample_walk_kernel<T, KIND><<<batch, kSThreads, kSampleSmem, st>>>(ka);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_rows(const KArgs& ka, int grid, size_t smem, cudaStream_t st) {
  const bool soft = ka.a.method != SUBSPEC_VERIFY_EXACT;
  const bool probs = ka.a.input_kind == SUBSPEC_IN_PROBS;
#define SUBSPEC_LAUNCH(KIND, SOFT)                                                                        \
  do {                                                                                                    \
    cudaError_t e_ = cudaFuncSetAttribute(verify_rows_kernel<T, KIND, SOFT>,                              \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    if (e_ != cudaSuccess) return e_;                                                                     \
    verify_rows_kernel<T, KIND, SOFT><<<grid, kThreads, smem, st>>>(ka);                                  \
  } while (0)
  if (probs) {
    if (soft)
      SUBSPEC_LAUNCH(SUBSPEC_IN_PROBS, true);
    else
      SUBSPEC_LAUNCH(SUBSPEC_IN_PROBS, false);
  } else {
    if (soft)
      SUBSPEC_LAUNCH(SUBSPEC_IN_LOGITS, true);
    else
      SUBSPEC_LAUNCH(SUBSPEC_IN_LOGITS, false);
  }
#undef SUBSPEC_LAUNCH
  return cudaGetLastError();
}

template <typename T, int KIND>
cudaError_t launch_sample(const KArgs& ka, int rows, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(verify_sample_rows_kernel<T, KIND>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSampleSmem);
  if (e != cudaSuccess) return e;
  verify_sample_rows_kernel<T, KIND><<<rows, kSThreads, kSampleSmem, st>>>(ka);
  return cudaGetLastError();
}

// the two sampling kernels by element type and input kind
template <bool WALK>
cudaError_t launch_sampler(const KArgs& ka, int n, cudaStream_t st) {
  const bool probs = ka.a.input_kind == SUBSPEC_IN_PROBS;
#define SUBSPEC_SAMPLER(T, KIND) \
  (WALK ? launch_sample_walk<T, KIND>(ka, n, st) : launch_sample<T, KIND>(ka, n, st))
  switch (ka.a.dtype) {
    case SUBSPEC_F32:
      return probs ? SUBSPEC_SAMPLER(float, SUBSPEC_IN_PROBS) : SUBSPEC_SAMPLER(float, SUBSPEC_IN_LOGITS);
    case SUBSPEC_BF16:
      return probs ? SUBSPEC_SAMPLER(__nv_bfloat16, SUBSPEC_IN_PROBS)
                   : SUBSPEC_SAMPLER(__nv_bfloat16, SUBSPEC_IN_LOGITS);
    default:
      return probs ? SUBSPEC_SAMPLER(__half, SUBSPEC_IN_PROBS) : SUBSPEC_SAMPLER(__half, SUBSPEC_IN_LOGITS);
  }
#undef SUBSPEC_SAMPLER
}

// ---- the tail behind the lm_head GEMM with a statistics epilogue --------------------------------
// One CTA per decoded row: the row's statistics are the combination of its per-tile records; the logits of
// the children's tokens, which the lossy gates need as probabilities, are 16-bit-rounded dot products of the
// row's hidden state with those tokens' weight rows (a few dozen per tree); then the same per-node outputs,
// the same ticket and the same walk as the streaming kernel's.
static_assert(sizeof(LmHeadStat) == sizeof(RowStat), "the GEMM's records are read as row statistics");
struct LmTailArgs {
  const LmHeadStat* partial;  // [batch * seq_rows, ntiles]
  int ntiles, seq_rows, dim;
  int half;  // 16-bit operands: 0 bf16, 1 fp16
  const uint16_t* hidden;
  int64_t hidden_stride;
  const uint16_t* weight;
  int64_t weight_stride;
};

// the two 16-bit floats of a word as fp32
__device__ __forceinline__ void pair_to_f32(uint32_t w, bool half, float& lo, float& hi) {
  if (half) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x, hi = f.y;
  } else {
    lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
  }
}

template <bool SOFT>
__global__ void __launch_bounds__(kThreads) lm_head_tail_kernel(const KArgs ka, const LmTailArgs lt) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ RowStat s_warp[kWarps];
  __shared__ RowStat s_row;
  __shared__ int s_flag;
  const subspec_verify_args& a = ka.a;
  const int row = blockIdx.x;
  const int b = row / a.max_nodes;
  const int u = row - b * a.max_nodes;
  int n_nodes, n_rows;
  seq_counts(a, b, n_nodes, n_rows);
  if (u >= n_rows) {
    if (n_rows == 0 && u == 0 && threadIdx.x == 0) write_empty_result(a, b);
    return;
  }
  // (a row count beyond the rows the caller laid out per sequence: reported, the row counts as empty)
  const bool have = u < lt.seq_rows;
  if (!have && threadIdx.x == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_COUNT);
  const size_t grow = (size_t)b * lt.seq_rows + (have ? u : 0);  // the row of the GEMM
  RowStat st = empty_stat(false);
  for (int i = threadIdx.x; have && i < lt.ntiles; i += kThreads) {
    const LmHeadStat p = lt.partial[grow * lt.ntiles + i];
    RowStat q;
    q.c = p.c, q.s = p.s, q.t2 = p.t2, q.vmax = p.vmax, q.amax = p.amax;
    st = combine(st, q);
  }
  block_reduce<SUBSPEC_IN_LOGITS>(st, s_warp, &s_row);
  const RowStat r = s_row;
  const size_t nb = (size_t)b * a.max_nodes;
  if (threadIdx.x == 0) {
    a.node_target[nb + u] = r.amax == INT_MAX ? 0 : r.amax;
    float ent = 0.f;
    if (SOFT) {
      const float denom = a.vocab > 1 ? logf((float)a.vocab) : 1.f;
      ent = kLn2 * (lg2f(r.s) - r.t2 / r.s) / denom;
    }
    a.node_entropy[nb + u] = ent;
    a.node_rowmax[nb + u] = r.c;
    a.node_rowsum[nb + u] = r.s;
  }
  if (SOFT) {
    int cb, ce;
    child_range(a, b, u, n_nodes, cb, ce);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* h = reinterpret_cast<const uint4*>(lt.hidden + grow * lt.hidden_stride);
    for (int e = cb + warp; e < ce; e += kWarps) {  // a warp per child
      const int c = a.child_idx[nb + e];
      if (c < 0 || c >= n_nodes) {
        if (lane == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_CHILD);
        continue;
      }
      const int tok = a.token_ids[nb + c];
      float p = 0.f;
      if (tok < 0 || tok >= a.vocab) {
        if (lane == 0) flag(a.dev_status, SUBSPEC_DEV_BAD_TOKEN);
      } else {
        const uint4* wv = reinterpret_cast<const uint4*>(lt.weight + (size_t)tok * lt.weight_stride);
        float acc = 0.f;
        for (int i = lane; i < lt.dim / 8; i += 32) {
          const uint4 hv = h[i], wq = wv[i];
          const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w}, ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float h0, h1, w0, w1;
            pair_to_f32(hw[j], lt.half != 0, h0, h1);
            pair_to_f32(ww[j], lt.half != 0, w0, w1);
            acc = fmaf(h0, w0, acc);
            acc = fmaf(h1, w1, acc);
          }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        const float x = lt.half ? __half2float(__float2half_rn(acc)) : __bfloat162float(__float2bfloat16_rn(acc));
        p = ex2f(fmaf(x, ka.k, -r.c)) / r.s;
      }
      if (lane == 0) a.node_child_prob[nb + c] = p;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(ka.sc.seq_ticket + b, 1);
    s_flag = (t == n_rows - 1);
    if (s_flag) ka.sc.seq_ticket[b] = 0;
  }
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  run_walk(ka, b, smem_raw);
}

// Dynamic shared memory: the TMA ring while streaming, reused for the walk's tree arrays afterwards.
size_t kernel_smem_bytes(int max_nodes) {
  const size_t walk = sizeof(int) * (9 * (size_t)max_nodes + 1);
  const size_t ring = (size_t)kStages * kStageBytes;
  return walk > ring ? walk : ring;
}

}  // namespace
}  // namespace subspec

using namespace subspec;

extern "C" int subspec_verify_scratch_bytes(int32_t batch, int32_t max_nodes, size_t* bytes) {
  if (!bytes || batch < 0 || max_nodes < 1 || max_nodes > kMaxNodes) return SUBSPEC_EINVAL;
  *bytes = ticket_bytes(batch, max_nodes) + sizeof(RowStat) * (size_t)batch * max_nodes * kMaxSplits;
  return SUBSPEC_OK;
}

extern "C" int subspec_verify_batched(const subspec_verify_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_verify_args)) return SUBSPEC_EINVAL;
  const subspec_verify_args& a = *args;
  if (a.batch < 0 || a.max_nodes < 1 || a.vocab < 1 || a.max_out < 2) return SUBSPEC_EINVAL;
  if (a.max_nodes > kMaxNodes || a.vocab > (1 << 20)) return SUBSPEC_EUNSUPPORTED;
  if (a.dtype != SUBSPEC_F32 && a.dtype != SUBSPEC_BF16 && a.dtype != SUBSPEC_F16) return SUBSPEC_EINVAL;
  if (a.input_kind != SUBSPEC_IN_LOGITS && a.input_kind != SUBSPEC_IN_PROBS) return SUBSPEC_EINVAL;
  if (a.method != SUBSPEC_VERIFY_EXACT && a.method != SUBSPEC_VERIFY_LOSSY &&
      a.method != SUBSPEC_VERIFY_EXACT_AND_LOSSY)
    return SUBSPEC_EINVAL;
  if (a.method == SUBSPEC_VERIFY_EXACT_AND_LOSSY && (!a.out2_tokens || !a.out2_hidden || !a.out2_meta))
    return SUBSPEC_EINVAL;
  if (a.gate != SUBSPEC_GATE_PROB && a.gate != SUBSPEC_GATE_ENTROPY) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!a.logits || !a.n_nodes || !a.n_rows || !a.token_ids || !a.child_off || !a.child_idx || !a.root ||
      !a.out_tokens || !a.out_hidden || !a.out_meta || !a.node_target || !a.node_entropy || !a.node_child_prob ||
      !a.node_rowmax || !a.node_rowsum || !a.node_exact_after || !a.node_best_len || !a.node_best_next ||
      !a.scratch)
    return SUBSPEC_EINVAL;
  // fp32 logits and probabilities go through the sampler without the 16-bit histogram
  const bool wide = a.dtype == SUBSPEC_F32 || a.input_kind == SUBSPEC_IN_PROBS;
  if (a.do_sample) {
    // sampled targets: the exact (sample-and-match) walk, or the lossy DP on the processed distribution
    if (!a.uniforms || !(a.temperature > 0.0) || !(a.top_p >= 0.0) || a.top_k < 0) return SUBSPEC_EINVAL;
    if (a.acceptance != 0 && a.acceptance != 1) return SUBSPEC_EINVAL;
    if (a.acceptance == 1) {  // residual acceptance: the exact walk, with the draft's logits of the same nodes
      if (a.method != SUBSPEC_VERIFY_EXACT || wide) return SUBSPEC_EUNSUPPORTED;
      if (!a.draft_logits || !a.accept_uniforms || !(a.draft_temperature > 0.0)) return SUBSPEC_EINVAL;
    }
    const bool filtered = a.top_k > 0 || a.top_p < 1.0;
    // probabilities are drawn from as they are (lossy_tree_verify.py:75-77)
    if (a.input_kind == SUBSPEC_IN_PROBS && (filtered || a.temperature != 1.0)) return SUBSPEC_EUNSUPPORTED;
    // (the lossy gates of a wide row come from the streaming kernel, which knows the temperature; with a
    // top-k / top-p filter on fp32 logits the sampler computes them itself)
  } else if (a.acceptance != 0) {
    return SUBSPEC_EINVAL;
  }
  size_t need = 0;
  subspec_verify_scratch_bytes(a.batch, a.max_nodes, &need);
  if (a.scratch_bytes < need || (reinterpret_cast<uintptr_t>(a.scratch) & 255u)) return SUBSPEC_ESCRATCH;
  if ((int64_t)a.batch * a.max_nodes > (int64_t)INT_MAX / kMaxSplits) return SUBSPEC_EUNSUPPORTED;

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  KArgs ka;
  ka.a = a;
  ka.sc = carve(a.scratch, a.batch, a.max_nodes);
  ka.k = a.do_sample ? (float)(1.4426950408889634 / a.temperature) : kLog2e;
  // transformers compares float32 cumulative probabilities with the Python double 1 - top_p cast to float32
  ka.remove_below = (a.do_sample && a.top_p < 1.0) ? (float)(1.0 - a.top_p) : 0.f;
  const size_t esz = a.dtype == SUBSPEC_F32 ? 4 : 2;
  ka.vec_ok = ((reinterpret_cast<uintptr_t>(a.logits) & 15u) == 0) && ((a.seq_stride * esz) % 16 == 0) &&
              ((a.row_stride * esz) % 16 == 0);
  ka.kD = a.acceptance == 1 ? (float)(1.4426950408889634 / a.draft_temperature) : 0.f;
  ka.dvec_ok = a.acceptance == 1 && ((reinterpret_cast<uintptr_t>(a.draft_logits) & 15u) == 0) &&
               ((a.draft_seq_stride * esz) % 16 == 0) && ((a.draft_row_stride * esz) % 16 == 0);
  // Fill the machine: with few rows, split every row over several CTAs.
  const int64_t rows = (int64_t)a.batch * a.max_nodes;
  const int64_t target = 4LL * kNumSMs;
  int splits = 1;
  if (rows < target) {
    // The launch lasts (waves of resident CTAs) x (a CTA's share of a row + its fixed cost): take the split
    // count that makes that smallest, with a small charge per split for the exchange of partials.  Rounding
    // the count up to "at least one CTA per slot" is wrong by a wave: 64 rows x 10 splits = 640 CTAs on 592
    // slots ran 48 CTAs behind everybody else, 5 us of a 20 us launch; nine splits fit.
    const int64_t vecs = a.vocab / (esz == 4 ? 4 : 8);
    int64_t max_s = vecs / (2 * kThreads) > 1 ? vecs / (2 * kThreads) : 1;
    if (max_s > kMaxSplits) max_s = kMaxSplits;
    // in units of the time one resident CTA needs for a whole row (its slot's share of the HBM bandwidth,
    // ~11 GB/s): ~1.5 us of fixed cost per CTA, ~0.1 us per split for the exchange
    const double row_us = (double)a.vocab * (double)esz / 11.0e3;
    const double per_cta = 1.5 / row_us, per_split = 0.1 / row_us;
    double best = 1e30;
    for (int sp = 1; sp <= (int)max_s; ++sp) {
      const int64_t waves = (rows * sp + target - 1) / target;
      const double cost = (double)waves * (1.0 / sp + per_cta) + per_split * sp;
      if (cost < best - 1e-12) {
        best = cost;
        splits = sp;
      }
    }
  }
  ka.splits = splits;

  // The tickets have to be zero; every launch leaves them so (the last arrival resets its ticket), so a caller
  // who vouches for the buffer (SUBSPEC_VERIFY_SCRATCH_CLEAN) saves this node in front of the kernel.
  int rc = SUBSPEC_OK;
  if (!(a.flags & SUBSPEC_VERIFY_SCRATCH_CLEAN))
    rc = cuda_check(cudaMemsetAsync(a.scratch, 0, ticket_bytes(a.batch, a.max_nodes), st));
  if (rc) return rc;
  cudaError_t e;
  ka.targets_only = 0;
  ka.keep_target = 0;
  ka.wide_gates = 0;
  if ((a.do_sample == 2 || a.acceptance == 1) && a.method == SUBSPEC_VERIFY_EXACT)
    return cuda_check(launch_sampler<true>(ka, a.batch, st));
  if (a.do_sample && wide && a.method != SUBSPEC_VERIFY_EXACT && (a.top_k > 0 || a.top_p < 1.0)) {
    ka.wide_gates = 1;  // fp32 logits, lossy, filtered: gates on the filtered distribution, one launch
    return cuda_check(launch_sampler<false>(ka, (int)rows, st));
  }
  if (a.do_sample && !(wide && a.method != SUBSPEC_VERIFY_EXACT))
    return cuda_check(launch_sampler<false>(ka, (int)rows, st));
  if (a.do_sample) {
    // wide rows, lossy DP: draw the targets first, then stream the rows for entropies and child
    // probabilities and run the DP on the targets already in node_target
    ka.targets_only = 1;
    e = launch_sampler<false>(ka, (int)rows, st);
    if (e != cudaSuccess) return cuda_check(e);
    ka.targets_only = 0;
    ka.keep_target = 1;
  }
  const int grid = (int)(rows * splits);
  const size_t smem = kernel_smem_bytes(a.max_nodes);
  switch (a.dtype) {
    case SUBSPEC_F32:
      e = launch_rows<float>(ka, grid, smem, st);
      break;
    case SUBSPEC_BF16:
      e = launch_rows<__nv_bfloat16>(ka, grid, smem, st);
      break;
    default:
      e = launch_rows<__half>(ka, grid, smem, st);
      break;
  }
  return cuda_check(e);
}

// ---- lm_head + verify without the logits in between ---------------------------------
static size_t lm_head_stats_bytes(int64_t rows, int vocab) {
  return align_up(sizeof(LmHeadStat) * (size_t)rows * (size_t)((vocab + kLmMinTileN - 1) / kLmMinTileN), 256);
}

extern "C" int subspec_lm_head_verify_scratch_bytes(int32_t batch, int32_t max_nodes, int32_t hidden_seq_rows,
                                                    int32_t vocab, size_t* bytes) {
  if (!bytes || batch < 0 || max_nodes < 1 || max_nodes > kMaxNodes || hidden_seq_rows < 1 || vocab < 1 ||
      vocab > (1 << 20))
    return SUBSPEC_EINVAL;
  *bytes = ticket_bytes(batch, max_nodes) + lm_head_stats_bytes((int64_t)batch * hidden_seq_rows, vocab);
  return SUBSPEC_OK;
}

extern "C" int subspec_lm_head_verify(const subspec_lm_head_verify_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_lm_head_verify_args) ||
      args->verify.struct_size != sizeof(subspec_verify_args))
    return SUBSPEC_EINVAL;
  const subspec_verify_args& a = args->verify;
  if (a.batch < 0 || a.max_nodes < 1 || a.vocab < 1 || a.max_out < 2 || args->hidden_dim < 8 ||
      args->hidden_seq_rows < 1)
    return SUBSPEC_EINVAL;
  if (a.max_nodes > kMaxNodes || a.vocab > (1 << 20) || args->hidden_dim % 8) return SUBSPEC_EUNSUPPORTED;
  // the dtype of hidden states and weight, and of the logits this call stands for
  if (a.dtype != SUBSPEC_BF16 && a.dtype != SUBSPEC_F16) return SUBSPEC_EUNSUPPORTED;
  if (a.do_sample || a.acceptance) return SUBSPEC_EUNSUPPORTED;  // sampled targets need the whole row
  if (a.method != SUBSPEC_VERIFY_EXACT && a.method != SUBSPEC_VERIFY_LOSSY &&
      a.method != SUBSPEC_VERIFY_EXACT_AND_LOSSY)
    return SUBSPEC_EINVAL;
  if (a.method == SUBSPEC_VERIFY_EXACT_AND_LOSSY && (!a.out2_tokens || !a.out2_hidden || !a.out2_meta))
    return SUBSPEC_EINVAL;
  if (a.gate != SUBSPEC_GATE_PROB && a.gate != SUBSPEC_GATE_ENTROPY) return SUBSPEC_EINVAL;
  if (a.batch == 0) return SUBSPEC_OK;
  if (!args->hidden || !args->weight || !a.n_nodes || !a.n_rows || !a.token_ids || !a.child_off || !a.child_idx ||
      !a.root || !a.out_tokens || !a.out_hidden || !a.out_meta || !a.node_target || !a.node_entropy ||
      !a.node_child_prob || !a.node_rowmax || !a.node_rowsum || !a.node_exact_after || !a.node_best_len ||
      !a.node_best_next || !a.scratch)
    return SUBSPEC_EINVAL;
  const int64_t rows = (int64_t)a.batch * args->hidden_seq_rows;
  if (rows > INT_MAX || (int64_t)a.batch * a.max_nodes > INT_MAX) return SUBSPEC_EUNSUPPORTED;
  size_t need = 0;
  subspec_lm_head_verify_scratch_bytes(a.batch, a.max_nodes, args->hidden_seq_rows, a.vocab, &need);
  if (a.scratch_bytes < need || (reinterpret_cast<uintptr_t>(a.scratch) & 255u)) return SUBSPEC_ESCRATCH;
  const int64_t hs = args->hidden_row_stride ? args->hidden_row_stride : args->hidden_dim;
  const int64_t ws = args->weight_row_stride ? args->weight_row_stride : args->hidden_dim;

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  KArgs ka = {};
  ka.a = a;
  ka.sc = carve(a.scratch, a.batch, a.max_nodes);
  ka.splits = 1;
  ka.k = kLog2e;
  const bool soft = a.method != SUBSPEC_VERIFY_EXACT;
  LmHeadGemmArgs ga;
  ga.half = a.dtype == SUBSPEC_F16 ? 1 : 0;
  ga.hidden = args->hidden, ga.hidden_stride = hs, ga.weight = args->weight, ga.weight_stride = ws;
  ga.rows = (int)rows, ga.vocab = a.vocab, ga.dim = args->hidden_dim;
  ga.soft = soft ? 1 : 0;
  ga.k = ka.k;
  ga.partial = reinterpret_cast<LmHeadStat*>(reinterpret_cast<char*>(a.scratch) + ticket_bytes(a.batch, a.max_nodes));
  ga.dev_status = a.dev_status;
  int rc = SUBSPEC_OK;
  if (!(a.flags & SUBSPEC_VERIFY_SCRATCH_CLEAN))
    rc = cuda_check(cudaMemsetAsync(a.scratch, 0, ticket_bytes(a.batch, a.max_nodes), st));
  if (rc) return rc;
  int ntiles = 0;
  cudaError_t e = launch_lm_head_stats(ga, st, &ntiles);
  if (e == cudaErrorInvalidValue) return SUBSPEC_EINVAL;  // addresses or strides not multiples of 16 bytes
  if (e != cudaSuccess) return cuda_check(e);
  LmTailArgs lt;
  lt.partial = ga.partial, lt.ntiles = ntiles, lt.seq_rows = args->hidden_seq_rows;
  lt.dim = args->hidden_dim;
  lt.half = ga.half;
  lt.hidden = reinterpret_cast<const uint16_t*>(args->hidden), lt.hidden_stride = hs;
  lt.weight = reinterpret_cast<const uint16_t*>(args->weight), lt.weight_stride = ws;
  const size_t smem = sizeof(int) * (9 * (size_t)a.max_nodes + 1);
  const int grid = a.batch * a.max_nodes;
  if (soft) {
    lm_head_tail_kernel<true><<<grid, kThreads, smem, st>>>(ka, lt);
  } else {
    lm_head_tail_kernel<false><<<grid, kThreads, smem, st>>>(ka, lt);
  }
  return cuda_check(cudaGetLastError());
}

// ---- no-allocation variant -------------------------------------------------------
// Scratch for subspec_verify_batched_static_scratch: room for the tickets and split
// partials of up to SUBSPEC_STATIC_SCRATCH_MAX_ROWS tree nodes per launch.  The array is
// part of the library image, so every GPU that loads the library holds it until the
// process exits.
namespace subspec {
namespace {
constexpr size_t kStaticRows = SUBSPEC_STATIC_SCRATCH_MAX_ROWS;
constexpr size_t kStaticScratchBytes =
    (sizeof(int) * 2 * kStaticRows + 255) / 256 * 256 + sizeof(RowStat) * kStaticRows * kMaxSplits;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal
}  // namespace
}  // namespace subspec

extern "C" int subspec_verify_batched_static_scratch(const subspec_verify_args* args, subspec_stream_t stream) {
  if (!args || args->struct_size != sizeof(subspec_verify_args)) return SUBSPEC_EINVAL;
  if (args->batch < 0 || args->max_nodes < 1) return SUBSPEC_EINVAL;
  if ((int64_t)args->batch * args->max_nodes > (int64_t)kStaticRows) return SUBSPEC_ETOOLARGE;
  int dev = -1;
  int rc = cuda_check(cudaGetDevice(&dev));
  if (rc) return rc;
  if (dev < 0 || dev >= kMaxDevices) return SUBSPEC_EUNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {
    // In host code `g_static_scratch` is only a handle for the symbol; the address a kernel can use
    // has to be asked for, with the device that will run the kernel current.
    void* p = nullptr;
    rc = cuda_check(cudaGetSymbolAddress(&p, g_static_scratch));
    if (rc) return rc;
    if (!p || (reinterpret_cast<uintptr_t>(p) & 255u)) return SUBSPEC_ESCRATCH;
    g_static_scratch_ptr[dev] = p;
  }
  subspec_verify_args a = *args;
  a.scratch = g_static_scratch_ptr[dev];
  a.scratch_bytes = kStaticScratchBytes;
  a.flags &= ~SUBSPEC_VERIFY_SCRATCH_CLEAN;  // nobody can vouch for this buffer: always cleared first
  return subspec_verify_batched(&a, stream);
}
