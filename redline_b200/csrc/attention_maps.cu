// Causal attention over the paged cache in its general form: key size D and value size DV of their
// own, M score maps per head over the same values (M = 2: differential attention), an optional
// tanh cap on the scores, a sliding window that keeps the first tokens of the sequence visible, and
// an optional unit-RMS norm of every head's output.  No positions enter the scores here (a rotary
// encoding would be applied to q and k before the cache write).
//
//   query row (h, m) of token i:   s_j = cap * tanh(scale * q_{h,m} . k_{g,m,j} / cap),  g = h / (H / G)
//   key j is visible from i when    j <= i and (i - j < window or j < keep_first)      (window 0: all)
//   a_{h,m} = softmax_j(s) V_g
//   M = 1:  o_h = a_{h,0};          M = 2:  o_h = a_{h,0} - lambda * a_{h,1}
//   sink:       a learned number per head joins the softmax's denominator, exp(sink_h) once, with no key and
//               no value (M = 1)
//   slopes:     a number per head times the distance is taken off the score, s_j <- s_j - slope_h * (i - j)
//   unit_norm:  o_h <- o_h / sqrt(mean(o_h^2) + eps)
//   o_h <- o_h * post_scale, and with a gate o_h <- o_h * sigmoid(gate), the gate one number per head
//   (gate_mode 1: gate[token, h]) or per entry (gate_mode 2: gate[token, h * DV + d])
//
// Layouts: q [tokens, q_stride] with row (h, m) at column (h * M + m) * D; the key cache
// [pages, G * M, page_size, D] (kv head g's map m is head g * M + m); the value cache
// [pages, G, page_size, VS] of which a row's first DV entries are the value (VS = DV unless the module is
// compiled with -DRL_V_STRIDE: a mixer whose values are the keys, or the leading part of them, hands the key
// cache in as the value cache with VS = D); out [tokens, out_stride] with head h at column h * DV.
//
// Scores, softmax, the combination of the maps and the norm are float32 for both element types.
// Single tokens: one CTA per (128-key partition, kv head and four of its query heads, item) over absolute partitions, so a row's
// sums do not depend on what else is in the launch; a second kernel merges the partitions of a head's
// maps, combines them and norms.  Prompt portions: both maps in turn over the visible key tiles,
// combination and norm in the epilogue; in bfloat16 with sizes that are multiples of 16 on the tensor
// cores (one CTA per 64 query rows and head), else on CUDA cores (one CTA per 32 query rows and head).
#include <cstring>

#include "common.cuh"

#if !defined(RL_QK_DIM) || !defined(RL_V_DIM) || !defined(RL_MAPS)
#error "compile with -DRL_QK_DIM=<key size> -DRL_V_DIM=<value size> -DRL_MAPS=<1 or 2>"
#endif

namespace rl {

#ifndef RL_V_STRIDE
#define RL_V_STRIDE RL_V_DIM
#endif
constexpr int kD = RL_QK_DIM, kDV = RL_V_DIM, kM = RL_MAPS, kVS = RL_V_STRIDE;
static_assert(kVS >= kDV, "a value row holds the value");
static_assert(kM == 1 || kM == 2, "one or two score maps");
// (up to 256 entries every kernel applies; longer rows, up to 576, go through the CUDA-core kernels only: what
// the single-token kernel keeps in static shared memory and the portion kernel in dynamic shared memory still fits)
static_assert(kD >= 1 && kD <= 576 && kDV >= 1 && kDV <= 512, "sizes out of range");
constexpr int kVQ = (kDV + 3) / 4;             // value columns of one of the four threads that share a query row
constexpr int kPart = 128;
constexpr int kThreads = 128;
constexpr int kLPK = 8;                      // lanes that share a key
constexpr int kKeysPerIter = kThreads / kLPK;
constexpr int kRows = 4;                     // query rows per pass over the keys

struct MaskArgs {
  int window, keep_first;
};

// What follows the softmax: a sink in the denominator, a gate on the output.
template <typename T>
struct TailArgs {
  const float* sink;     // [heads] or null
  const float* slopes;   // [heads] or null: slope_h * (i - j) is taken off the score of key j for query i
  const T* gate;         // rows of gate_stride entries, or null
  int gate_stride, gate_mode;
};
template <typename T>
__device__ __forceinline__ float gate_factor(const TailArgs<T>& t, size_t tok, int head, int d, int dv) {
  if (t.gate_mode == 0) return 1.f;
  const float g = to_float(t.gate[tok * t.gate_stride + (t.gate_mode == 1 ? head : head * dv + d)]);
  return 1.f / (1.f + expf(-g));
}

__device__ __forceinline__ bool key_visible(int j, int i, const MaskArgs& mk) {
  return j <= i && (mk.window <= 0 || i - j < mk.window || j < mk.keep_first);
}
// Whether key j is behind the window of position i and of every later one, and not kept: its page may have
// been given back, so it is not read at all (a masked weight of zero times a stray NaN would be NaN).
__device__ __forceinline__ bool dead_key(int j, int i, const MaskArgs& mk) {
  return mk.window > 0 && j >= mk.keep_first && j <= i - mk.window;
}
// Whether keys [lo, hi) hold one that position i sees.
__device__ __forceinline__ bool range_visible(int lo, int hi, int i, const MaskArgs& mk) {
  if (lo > i || lo >= hi) return false;
  if (mk.window <= 0) return true;
  return lo < mk.keep_first || hi > i - mk.window + 1;
}

template <typename T>
struct MapsDecodeArgs {
  const T* q;
  int q_stride;
  const T* kcache;
  const T* vcache;
  const int32_t* block_table;
  int max_blocks;
  const int4* items;     // (token index, sequence index, context length, 0)
  float* part_o;         // [items, H * M, max_parts, DV]
  float* part_ml;        // [items, H * M, max_parts, 2]
  int max_parts;
  T* out;
  int out_stride;
  int heads, kv_heads, page_size;
  MaskArgs mask;
  float scale, softcap, lambda, post_scale, eps;
  int unit_norm;
  TailArgs<T> tail;
};

// Lane l of the 8 that share a key takes elements l, l + 8, ... of the key in pieces of E elements.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maps_decode_kernel(const MapsDecodeArgs<T> a) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<T>::N;
  constexpr int E = (kD % VEC == 0) ? VEC : 1;          // piece of a key
  constexpr int CH = kD / E;
  constexpr int CPL = (CH + kLPK - 1) / kLPK;
  constexpr int EVV = (kDV % VEC == 0 && kVS % VEC == 0) ? VEC : 1;         // piece of a value row
  constexpr int CHV = kDV / EVV;
  constexpr int CPLV = (CHV + kLPK - 1) / kLPK;
  __shared__ float qs[kRows][kD];
  __shared__ float sc[kRows][kPart];
  __shared__ float red[kThreads / 32][kRows][kDV];
  __shared__ float stat_m[kRows], stat_l[kRows];

  // blockIdx.y: (kv head, group of up to kRows of its query heads): the groups of a kv head run side by side
  const int G = a.heads / a.kv_heads;
  const int groups = (G + kRows - 1) / kRows;
  const int part = blockIdx.x, kvh = blockIdx.y / groups, g0 = (blockIdx.y % groups) * kRows, item = blockIdx.z;
  const int4 info = a.items[item];
  const int tok = info.x, seq = info.y, ctx = info.z;
  const int me = ctx - 1;                                // the query's position
  const int base = part * kPart;
  const int j_hi = min(ctx, base + kPart);
  if (!range_visible(base, j_hi, me, a.mask)) return;
  const int lane8 = threadIdx.x % kLPK, slot = threadIdx.x / kLPK;
  const int warp = threadIdx.x >> 5;
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
  // the pages of this thread's keys (key base + it * 16 + slot), read once
  int pages[kPart / kKeysPerIter];
#pragma unroll
  for (int it = 0; it < kPart / kKeysPerIter; ++it) {
    const int j = base + it * kKeysPerIter + slot;
    pages[it] = (j < j_hi && key_visible(j, me, a.mask)) ? bt[j / a.page_size] : 0;
  }

  for (int m = 0; m < kM; ++m) {
    const int khead = kvh * kM + m;
    {
      const int ng = min(kRows, G - g0);
      __syncthreads();
      for (int i = threadIdx.x; i < kRows * kD; i += kThreads) {
        const int g = i / kD, d = i - g * kD;
        qs[g][d] = g < ng ? to_float(a.q[static_cast<size_t>(tok) * a.q_stride +
                                         ((kvh * G + g0 + g) * kM + m) * kD + d]) * a.scale
                          : 0.f;
      }
      __syncthreads();
      // ---- scores (every lane of a warp makes the same number of trips: the shuffles need all of them)
#pragma unroll
      for (int it = 0; it < kPart / kKeysPerIter; ++it) {
        const int j = base + it * kKeysPerIter + slot;
        const bool live = j < j_hi && key_visible(j, me, a.mask);
        const size_t page = live ? pages[it] : 0;
        const T* kp = a.kcache + ((page * (a.kv_heads * kM) + khead) * a.page_size + j % a.page_size) * kD;
        float dot[kRows];
#pragma unroll
        for (int g = 0; g < kRows; ++g) dot[g] = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          const int ch = lane8 + c * kLPK;
          if (live && ch < CH) {
            float kf[E];
            if (E == 1) kf[0] = to_float(kp[ch]);
            else load16(kp + ch * E, kf);
#pragma unroll
            for (int g = 0; g < kRows; ++g) {
#pragma unroll
              for (int e = 0; e < E; ++e) dot[g] += kf[e] * qs[g][ch * E + e];
            }
          }
        }
#pragma unroll
        for (int g = 0; g < kRows; ++g) {
          float v = dot[g];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if (lane8 == 0 && j < j_hi) {
            if (a.softcap > 0.f) v = a.softcap * tanhf(v * inv_cap);
            if (a.tail.slopes != nullptr && g < ng) v -= a.tail.slopes[kvh * G + g0 + g] * static_cast<float>(me - j);
            sc[g][j - base] = live ? v : -INFINITY;
          }
        }
      }
      __syncthreads();
      // ---- softmax statistics of this partition, one warp per row
      for (int g = warp; g < ng; g += kThreads / 32) {
        float mx = -INFINITY;
        for (int j = base + (threadIdx.x & 31); j < j_hi; j += 32) mx = fmaxf(mx, sc[g][j - base]);
        mx = warp_max(mx);
        float l = 0.f;
        for (int j = base + (threadIdx.x & 31); j < j_hi; j += 32) {
          const float p = expf(sc[g][j - base] - mx);      // masked keys: exp(-inf) = 0
          sc[g][j - base] = p;
          l += p;
        }
        l = warp_sum(l);
        if ((threadIdx.x & 31) == 0) {
          stat_m[g] = mx;
          stat_l[g] = l;
        }
      }
      __syncthreads();
      // ---- P V
      float acc[kRows][CPLV][EVV];
#pragma unroll
      for (int g = 0; g < kRows; ++g)
#pragma unroll
        for (int c = 0; c < CPLV; ++c)
#pragma unroll
          for (int e = 0; e < EVV; ++e) acc[g][c][e] = 0.f;
#pragma unroll
      for (int it = 0; it < kPart / kKeysPerIter; ++it) {
        const int j = base + it * kKeysPerIter + slot;
        if (j >= j_hi || !key_visible(j, me, a.mask)) continue;
        const size_t page = pages[it];
        const T* vp = a.vcache + ((page * a.kv_heads + kvh) * a.page_size + j % a.page_size) * kVS;
        float p[kRows];
#pragma unroll
        for (int g = 0; g < kRows; ++g) p[g] = g < ng ? sc[g][j - base] : 0.f;
#pragma unroll
        for (int c = 0; c < CPLV; ++c) {
          const int ch = lane8 + c * kLPK;
          if (ch < CHV) {
            float vf[EVV];
            if (EVV == 1) vf[0] = to_float(vp[ch]);
            else load16(vp + ch * EVV, vf);
#pragma unroll
            for (int g = 0; g < kRows; ++g)
#pragma unroll
              for (int e = 0; e < EVV; ++e) acc[g][c][e] += p[g] * vf[e];
          }
        }
      }
      // lanes 8 and 16 apart hold other keys of the same piece
#pragma unroll
      for (int g = 0; g < kRows; ++g)
#pragma unroll
        for (int c = 0; c < CPLV; ++c)
#pragma unroll
          for (int e = 0; e < EVV; ++e) {
            float v = acc[g][c][e];
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[g][c][e] = v;
          }
      if ((threadIdx.x & 31) < kLPK) {
#pragma unroll
        for (int g = 0; g < kRows; ++g)
#pragma unroll
          for (int c = 0; c < CPLV; ++c) {
            const int ch = lane8 + c * kLPK;
            if (ch < CHV) {
#pragma unroll
              for (int e = 0; e < EVV; ++e) red[warp][g][ch * EVV + e] = acc[g][c][e];
            }
          }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < ng * kDV; i += kThreads) {
        const int g = i / kDV, d = i - g * kDV;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) v += red[w][g][d];
        const int qrow = (kvh * G + g0 + g) * kM + m;
        const size_t row = (static_cast<size_t>(item) * (a.heads * kM) + qrow) * a.max_parts + part;
        a.part_o[row * kDV + d] = v;
        if (d == 0) {
          a.part_ml[row * 2] = stat_m[g];
          a.part_ml[row * 2 + 1] = stat_l[g];
        }
      }
    }
  }
}

// One CTA per (item, head): merges the visible partitions of each of the head's maps, combines the
// maps, norms, writes.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maps_merge_kernel(const MapsDecodeArgs<T> a) {
  pdl_launch();
  pdl_wait();
  __shared__ float o[kDV];
  __shared__ float scratch[32];
  const int item = blockIdx.x, head = blockIdx.y;
  const int4 info = a.items[item];
  const int tok = info.x, ctx = info.z;
  const int me = ctx - 1;
  const int p_hi = me / kPart;
  for (int d = threadIdx.x; d < kDV; d += kThreads) o[d] = 0.f;
  __syncthreads();
  for (int m = 0; m < kM; ++m) {
    const size_t row0 = (static_cast<size_t>(item) * (a.heads * kM) + head * kM + m) * a.max_parts;
    float mx = -INFINITY;
    for (int p = 0; p <= p_hi; ++p)
      if (range_visible(p * kPart, min(ctx, (p + 1) * kPart), me, a.mask)) mx = fmaxf(mx, a.part_ml[(row0 + p) * 2]);
    const float coef = m == 0 ? 1.f : -a.lambda;
    const bool sunk = kM == 1 && a.tail.sink != nullptr;
    if (sunk) mx = fmaxf(mx, a.tail.sink[head]);
    for (int d = threadIdx.x; d < kDV; d += kThreads) {
      float num = 0.f, den = sunk ? expf(a.tail.sink[head] - mx) : 0.f;
      for (int p = 0; p <= p_hi; ++p) {
        if (!range_visible(p * kPart, min(ctx, (p + 1) * kPart), me, a.mask)) continue;
        const float w = expf(a.part_ml[(row0 + p) * 2] - mx);
        num += w * a.part_o[(row0 + p) * kDV + d];
        den += w * a.part_ml[(row0 + p) * 2 + 1];
      }
      o[d] += coef * (num / den);
    }
  }
  __syncthreads();
  float r = a.post_scale;
  if (a.unit_norm) {
    float q = 0.f;
    for (int d = threadIdx.x; d < kDV; d += kThreads) q += o[d] * o[d];
    r *= rsqrtf(block_sum(q, scratch) / static_cast<float>(kDV) + a.eps);
  }
  for (int d = threadIdx.x; d < kDV; d += kThreads)
    a.out[static_cast<size_t>(tok) * a.out_stride + head * kDV + d] =
        from_float<T>(o[d] * r * gate_factor(a.tail, tok, head, d, kDV));
}

// ------------------------------------------------------------------ prompt portions
constexpr int kBQ = 32, kBK = 32;

template <typename T>
struct MapsPrefillArgs {
  const T* q;
  int q_stride;
  const T* kcache;
  const T* vcache;
  const int32_t* block_table;
  int max_blocks;
  const int32_t* tile_seq;
  const int32_t* tile_tok;
  const int32_t* tile_rows;
  const int32_t* positions;
  T* out;
  int out_stride;
  int heads, kv_heads, page_size, tile_quarters;
  MaskArgs mask;
  float scale, softcap, lambda, post_scale, eps;
  int unit_norm;
  TailArgs<T> tail;
};

// Thread t owns query row r = t / 4 and the columns c = t % 4 + 4 i of every tile.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maps_prefill_kernel(const MapsPrefillArgs<T> a) {
  pdl_launch();
  pdl_wait();
  constexpr int LDQ = kD + 1;
  extern __shared__ float smem[];
  float* Qs = smem;                  // [32][D+1], pre-scaled
  float* Ks = Qs + kBQ * LDQ;        // [32][D+1]
  float* Vs = Ks + kBK * LDQ;        // [32][DV]
  float* Ps = Vs + kBK * kDV;        // [32][33]

  const int tile = blockIdx.x / a.tile_quarters, quarter = blockIdx.x % a.tile_quarters, head = blockIdx.y;
  const int seq = a.tile_seq[tile], tok0 = a.tile_tok[tile] + quarter * kBQ;
  const int rows = min(a.tile_rows[tile] - quarter * kBQ, kBQ);
  if (rows <= 0) return;
  const int kvh = head / (a.heads / a.kv_heads);
  const int pos0 = a.positions[tok0];
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int r = threadIdx.x >> 2, cq = threadIdx.x & 3;
  const int my_pos = pos0 + r;
  const int k_end = pos0 + rows;     // exclusive
  const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
  const float slope = a.tail.slopes != nullptr ? a.tail.slopes[head] : 0.f;

  float o[kVQ];
#pragma unroll
  for (int i = 0; i < kVQ; ++i) o[i] = 0.f;

  for (int m = 0; m < kM; ++m) {
    __syncthreads();
    for (int i = threadIdx.x; i < kBQ * kD; i += kThreads) {
      const int rr = i / kD, d = i - rr * kD;
      Qs[rr * LDQ + d] = rr < rows ? to_float(a.q[static_cast<size_t>(tok0 + rr) * a.q_stride +
                                                  (head * kM + m) * kD + d]) * a.scale
                                   : 0.f;
    }
    float mx = -INFINITY, l = 0.f;
    float acc[kVQ];
#pragma unroll
    for (int i = 0; i < kVQ; ++i) acc[i] = 0.f;

    for (int k0 = 0; k0 < k_end; k0 += kBK) {
      // a tile that no row of this CTA sees is skipped: the rows' windows together reach back to
      // pos0 - window + 1, and the kept first tokens are seen by all
      const int t_hi = min(k0 + kBK, k_end);
      if (a.mask.window > 0 && k0 >= a.mask.keep_first && t_hi <= pos0 - a.mask.window + 1) continue;
      __syncthreads();
      for (int i = threadIdx.x; i < kBK * kD; i += kThreads) {
        const int key = i / kD, d = i - key * kD;
        const int j = k0 + key;
        float v = 0.f;
        if (j < k_end && !dead_key(j, pos0, a.mask)) {
          const size_t page = bt[j / a.page_size];
          v = to_float(a.kcache[((page * (a.kv_heads * kM) + kvh * kM + m) * a.page_size + j % a.page_size) * kD + d]);
        }
        Ks[key * LDQ + d] = v;
      }
      for (int i = threadIdx.x; i < kBK * kDV; i += kThreads) {
        const int key = i / kDV, d = i - key * kDV;
        const int j = k0 + key;
        float v = 0.f;
        if (j < k_end && !dead_key(j, pos0, a.mask)) {
          const size_t page = bt[j / a.page_size];
          v = to_float(a.vcache[((page * a.kv_heads + kvh) * a.page_size + j % a.page_size) * kVS + d]);
        }
        Vs[key * kDV + d] = v;
      }
      __syncthreads();
      float s[kBK / 4];
#pragma unroll
      for (int i = 0; i < kBK / 4; ++i) s[i] = 0.f;
      for (int d = 0; d < kD; ++d) {
        const float qv = Qs[r * LDQ + d];
#pragma unroll
        for (int i = 0; i < kBK / 4; ++i) s[i] += qv * Ks[(cq + 4 * i) * LDQ + d];
      }
      float tmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBK / 4; ++i) {
        const int kp = k0 + cq + 4 * i;
        const bool ok = (r < rows) && key_visible(kp, my_pos, a.mask);
        float v = s[i];
        if (a.softcap > 0.f) v = a.softcap * tanhf(v * inv_cap);
        v -= slope * static_cast<float>(my_pos - kp);
        s[i] = ok ? v : -INFINITY;
        tmax = fmaxf(tmax, s[i]);
      }
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const float m_new = fmaxf(mx, tmax);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (mx == -INFINITY) ? 0.f : expf(mx - m_use);
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < kBK / 4; ++i) {
        const float p = expf(s[i] - m_use);
        Ps[r * (kBK + 1) + cq + 4 * i] = p;
        psum += p;
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      l = l * alpha + psum;
      mx = m_new;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < kVQ; ++i) acc[i] *= alpha;
      for (int c = 0; c < kBK; ++c) {
        const float p = Ps[r * (kBK + 1) + c];
#pragma unroll
        for (int i = 0; i < kVQ; ++i)
          if (kDV % 4 == 0 || cq + 4 * i < kDV) acc[i] += p * Vs[c * kDV + cq + 4 * i];
      }
    }
    if (kM == 1 && a.tail.sink != nullptr && mx != -INFINITY) {
      // the sink joins the denominator; the reference maximum moves to it if it is the larger
      const float sk = a.tail.sink[head];
      const float m_new = fmaxf(mx, sk);
      const float alpha = expf(mx - m_new);
      l = l * alpha + expf(sk - m_new);
#pragma unroll
      for (int i = 0; i < kVQ; ++i) acc[i] *= alpha;
    }
    const float coef = (m == 0 ? 1.f : -a.lambda) / (l > 0.f ? l : 1.f);
#pragma unroll
    for (int i = 0; i < kVQ; ++i) o[i] += coef * acc[i];
  }
  float scale_out = a.post_scale;
  if (a.unit_norm) {
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kVQ; ++i) q += o[i] * o[i];
    q += __shfl_xor_sync(0xffffffffu, q, 1);
    q += __shfl_xor_sync(0xffffffffu, q, 2);
    scale_out *= rsqrtf(q / static_cast<float>(kDV) + a.eps);
  }
  if (r < rows) {
#pragma unroll
    for (int i = 0; i < kVQ; ++i)
      if (kDV % 4 == 0 || cq + 4 * i < kDV)
        a.out[static_cast<size_t>(tok0 + r) * a.out_stride + head * kDV + cq + 4 * i] =
            from_float<T>(o[i] * scale_out * gate_factor(a.tail, tok0 + r, head, cq + 4 * i, kDV));
  }
}

// ------------------------------------------------------------------ prompt portions on the tensor cores
// bfloat16, key and value sizes that are multiples of 16.  One CTA of four warps takes 64 query rows of a
// tile for one head; a warp takes 16 of them.  Keys and values come in tiles of 64 from the paged cache
// into shared memory (cp.async in 16-byte pieces; rows padded by 16 bytes so that fragment reads meet no
// bank twice; the ring may have two stages, see kStages).
// S = Q K^T with mma.sync.m16n8k16 (Q fragments straight from global memory, once per map), scale, cap,
// mask and online softmax in float32 in the accumulator layout; O += P V with V fragments from
// ldmatrix.trans.  The weights P are not cut to 16 bits: P = P_hi + P_lo (two bfloat16 operands, two MMAs
// into the same float32 accumulator), which keeps 16 bits of mantissa.  Both maps run in turn over the
// visible tiles; the first map's result waits in shared memory; combination, unit norm and the bfloat16
// store are the epilogue.
#if (RL_QK_DIM % 16 == 0) && (RL_V_DIM % 16 == 0) && (RL_V_STRIDE % 8 == 0) && (RL_QK_DIM <= 256) && (RL_V_DIM <= 256)
#define RL_MAPS_HAVE_MMA 1
constexpr int kTQ = 64, kTK = 64;
constexpr int kLDK = kD + 8, kLDV = kDV + 8;      // shared-memory row lengths in elements

__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// tanh with an ABSOLUTE error of a few 1e-7 (what a score needs: it goes into an exponential), from one
// fast exponential and one fast division; the hardware's tanh.approx is good to 2^-11 only.  (The odd series
// on the FMA pipe for small arguments was measured slower: 0.54 against 0.46 ms for 2,048 tokens of 16 heads.)
__device__ __forceinline__ float tanh_fast(float x) {
  return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);
}

// Stages of the K/V ring.  The kernel waits on dependent arithmetic, not on memory, with two warps per
// scheduler: what helps is a third CTA per SM, which one stage leaves room for (measured at 2,048 tokens,
// 16 heads, window 1,024: two stages and two CTAs 0.42 ms, one stage and three CTAs 0.32 ms).
constexpr int kStages = 1;

// (three CTAs to an SM cap a thread at 168 registers, which the query fragments and the output accumulators of
//  long rows do not fit: those sizes take two CTAs and up to 255 registers instead of spilling)
constexpr int kMmaCtas = (kD + kDV > 288) ? 2 : 3;

__global__ void __launch_bounds__(128, kMmaCtas)
maps_prefill_mma_kernel(const MapsPrefillArgs<bf16> a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Kst = reinterpret_cast<bf16*>(smem_raw);                // kStages x [64][D + 8]
  bf16* Vst = Kst + kStages * kTK * kLDK;                        // kStages x [64][DV + 8]
  float* O0 = reinterpret_cast<float*>(Vst + kStages * kTK * kLDV);   // [64][DV], the first map's result (two maps)

  const int halves = a.tile_quarters;                            // 64-row parts of a tile of the launch
  const int tile = blockIdx.x / halves, part = blockIdx.x % halves, head = blockIdx.y;
  const int seq = a.tile_seq[tile], tok0 = a.tile_tok[tile] + part * kTQ;
  const int rows = min(a.tile_rows[tile] - part * kTQ, kTQ);
  if (rows <= 0) return;
  const int kvh = head / (a.heads / a.kv_heads);
  const int pos0 = a.positions[tok0];
  const int k_end = pos0 + rows;
  const int32_t* bt = a.block_table + static_cast<size_t>(seq) * a.max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int r0 = warp * 16 + gid, r1 = r0 + 8;                   // this thread's two rows within the CTA's 64
  const int p0 = pos0 + r0, p1 = pos0 + r1;
  const bool ok0 = r0 < rows, ok1 = r1 < rows;
  const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
  const float slope = a.tail.slopes != nullptr ? a.tail.slopes[head] : 0.f;
  const int ps_shift = __ffs(a.page_size) - 1, ps_mask = a.page_size - 1;      // (pages hold a power of two of tokens)

  float o[kDV / 8][4];
  for (int m = 0; m < kM; ++m) {
    // ---- Q fragments of this map
    uint32_t qf[kD / 16][4];
    {
      const bf16* q0 = a.q + static_cast<size_t>(tok0 + r0) * a.q_stride + (head * kM + m) * kD + tig * 2;
      const bf16* q1 = a.q + static_cast<size_t>(tok0 + r1) * a.q_stride + (head * kM + m) * kD + tig * 2;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        qf[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16) : 0u;
        qf[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16) : 0u;
        qf[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8) : 0u;
        qf[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8) : 0u;
      }
    }
#pragma unroll
    for (int nd = 0; nd < kDV / 8; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // the visible key tiles in turn; the next one is on its way (cp.async) while this one is worked on
    auto next_visible = [&](int k0) {
      while (k0 < k_end && a.mask.window > 0 && k0 >= a.mask.keep_first &&
             min(k0 + kTK, k_end) <= pos0 - a.mask.window + 1)
        k0 += kTK;
      return k0;
    };
    auto issue = [&](int stage, int k0) {
      bf16* Kd = Kst + stage * kTK * kLDK;
      bf16* Vd = Vst + stage * kTK * kLDV;
      for (int i = threadIdx.x; i < kTK * (kD / 8); i += 128) {
        const int key = i / (kD / 8), c = i - key * (kD / 8);
        const int j = k0 + key;
        bf16* d = Kd + key * kLDK + c * 8;
        if (j < k_end && !dead_key(j, pos0, a.mask)) {
          const size_t page = bt[j >> ps_shift];
          cp_async16(d, a.kcache + ((page * (a.kv_heads * kM) + kvh * kM + m) * a.page_size + (j & ps_mask)) * kD + c * 8);
        } else {
          *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
      }
      for (int i = threadIdx.x; i < kTK * (kDV / 8); i += 128) {
        const int key = i / (kDV / 8), c = i - key * (kDV / 8);
        const int j = k0 + key;
        bf16* d = Vd + key * kLDV + c * 8;
        if (j < k_end && !dead_key(j, pos0, a.mask)) {
          const size_t page = bt[j >> ps_shift];
          cp_async16(d, a.vcache + ((page * a.kv_heads + kvh) * a.page_size + (j & ps_mask)) * kVS + c * 8);
        } else {
          *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
      }
    };
    int stage = 0;
    int k0 = next_visible(0);
    __syncthreads();                         // (the map before has left both stages)
    if (kStages == 2) {
      if (k0 < k_end) issue(0, k0);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    while (k0 < k_end) {
      const int k1 = next_visible(k0 + kTK);
      if (kStages == 2) {
        if (k1 < k_end) issue(stage ^ 1, k1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // this tile's copies have landed
      } else {
        issue(0, k0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
      const bf16* Ks = Kst + stage * kTK * kLDK;
      const bf16* Vs = Vst + stage * kTK * kLDV;
      // ---- S = Q K^T: 16 rows x 64 keys per warp
      float s[kTK / 8][4];
#pragma unroll
      for (int nt = 0; nt < kTK / 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const bf16* kr = Ks + (nt * 8 + gid) * kLDK + tig * 2;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          mma_16816(s[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kr + ks * 16),
                    *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8));
      }
      // ---- scale, cap, mask; the rows' maxima
      float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kTK / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = k0 + nt * 8 + tig * 2 + (e & 1);
          float v = s[nt][e] * a.scale;
          if (a.softcap > 0.f) v = a.softcap * tanh_fast(v * inv_cap);
          v -= slope * static_cast<float>(((e < 2) ? p0 : p1) - j);
          const bool vis = (e < 2) ? (ok0 && key_visible(j, p0, a.mask)) : (ok1 && key_visible(j, p1, a.mask));
          v = vis ? v : -INFINITY;
          s[nt][e] = v;
          if (e < 2) t0 = fmaxf(t0, v);
          else t1 = fmaxf(t1, v);
        }
      }
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      const float n0 = fmaxf(mx0, t0), n1 = fmaxf(mx1, t1);
      const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
      const float al0 = mx0 == -INFINITY ? 0.f : __expf(mx0 - u0), al1 = mx1 == -INFINITY ? 0.f : __expf(mx1 - u1);
      mx0 = n0;
      mx1 = n1;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < kTK / 8; ++nt) {
        s[nt][0] = __expf(s[nt][0] - u0);
        s[nt][1] = __expf(s[nt][1] - u0);
        s[nt][2] = __expf(s[nt][2] - u1);
        s[nt][3] = __expf(s[nt][3] - u1);
        sum0 += s[nt][0] + s[nt][1];
        sum1 += s[nt][2] + s[nt][3];
      }
      l0 = l0 * al0 + sum0;                  // (a quad's four partial sums are added at the end)
      l1 = l1 * al1 + sum1;
#pragma unroll
      for (int nd = 0; nd < kDV / 8; ++nd) {
        o[nd][0] *= al0;
        o[nd][1] *= al0;
        o[nd][2] *= al1;
        o[nd][3] *= al1;
      }
      // ---- O += P V, P as a high and a low bfloat16 part
#pragma unroll
      for (int kk = 0; kk < kTK / 16; ++kk) {
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const float x = s[2 * kk + (f >> 1)][(f & 1) * 2], y = s[2 * kk + (f >> 1)][(f & 1) * 2 + 1];
          const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
          ph[f] = *reinterpret_cast<const uint32_t*>(&h);
          pl[f] = pack_bf16(x - __low2float(h), y - __high2float(h));
        }
        const bf16* vrow = Vs + (kk * 16 + (lane & 15)) * kLDV + (lane >> 4) * 8;
#pragma unroll
        for (int nd = 0; nd < kDV / 8; nd += 2) {
          uint32_t b0, b1, b2, b3;
          const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(vrow + nd * 8));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
          mma_16816(o[nd], ph, b0, b1);
          mma_16816(o[nd + 1], ph, b2, b3);
          mma_16816(o[nd], pl, b0, b1);
          mma_16816(o[nd + 1], pl, b2, b3);
        }
      }
      __syncthreads();                       // every warp has read this stage: the tile after the next may land in it
      if (kStages == 2) stage ^= 1;
      k0 = k1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (kM == 1 && a.tail.sink != nullptr) {
      // the sink joins the denominators; a row's reference maximum moves to it if it is the larger
      const float sk = a.tail.sink[head];
      const float n0 = fmaxf(mx0, sk), n1 = fmaxf(mx1, sk);
      const float al0 = mx0 == -INFINITY ? 0.f : expf(mx0 - n0), al1 = mx1 == -INFINITY ? 0.f : expf(mx1 - n1);
      l0 = l0 * al0 + expf(sk - n0);
      l1 = l1 * al1 + expf(sk - n1);
#pragma unroll
      for (int nd = 0; nd < kDV / 8; ++nd) {
        o[nd][0] *= al0;
        o[nd][1] *= al0;
        o[nd][2] *= al1;
        o[nd][3] *= al1;
      }
    }
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (kM == 2 && m == 0) {
      // (every thread reads back exactly what it wrote: no barrier is needed for O0)
#pragma unroll
      for (int nd = 0; nd < kDV / 8; ++nd) {
        float* w0 = O0 + r0 * kDV + nd * 8 + tig * 2;
        float* w1 = O0 + r1 * kDV + nd * 8 + tig * 2;
        w0[0] = o[nd][0] * i0;
        w0[1] = o[nd][1] * i0;
        w1[0] = o[nd][2] * i1;
        w1[1] = o[nd][3] * i1;
      }
    } else if (kM == 2) {
#pragma unroll
      for (int nd = 0; nd < kDV / 8; ++nd) {
        const float* w0 = O0 + r0 * kDV + nd * 8 + tig * 2;
        const float* w1 = O0 + r1 * kDV + nd * 8 + tig * 2;
        o[nd][0] = w0[0] - a.lambda * o[nd][0] * i0;
        o[nd][1] = w0[1] - a.lambda * o[nd][1] * i0;
        o[nd][2] = w1[0] - a.lambda * o[nd][2] * i1;
        o[nd][3] = w1[1] - a.lambda * o[nd][3] * i1;
      }
    } else {
#pragma unroll
      for (int nd = 0; nd < kDV / 8; ++nd) {
        o[nd][0] *= i0;
        o[nd][1] *= i0;
        o[nd][2] *= i1;
        o[nd][3] *= i1;
      }
    }
  }
  float g0 = a.post_scale, g1 = a.post_scale;
  if (a.unit_norm) {
    float q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int nd = 0; nd < kDV / 8; ++nd) {
      q0 += o[nd][0] * o[nd][0] + o[nd][1] * o[nd][1];
      q1 += o[nd][2] * o[nd][2] + o[nd][3] * o[nd][3];
    }
    q0 += __shfl_xor_sync(0xffffffffu, q0, 1);
    q0 += __shfl_xor_sync(0xffffffffu, q0, 2);
    q1 += __shfl_xor_sync(0xffffffffu, q1, 1);
    q1 += __shfl_xor_sync(0xffffffffu, q1, 2);
    g0 *= rsqrtf(q0 / static_cast<float>(kDV) + a.eps);
    g1 *= rsqrtf(q1 / static_cast<float>(kDV) + a.eps);
  }
  if (a.tail.gate_mode == 1) {             // one gate per head: it joins the row's factor
    if (ok0) g0 *= gate_factor(a.tail, tok0 + r0, head, 0, kDV);
    if (ok1) g1 *= gate_factor(a.tail, tok0 + r1, head, 0, kDV);
  }
  const bool each = a.tail.gate_mode == 2;
#pragma unroll
  for (int nd = 0; nd < kDV / 8; ++nd) {
    const int d = nd * 8 + tig * 2;
    if (ok0)
      *reinterpret_cast<__nv_bfloat162*>(a.out + static_cast<size_t>(tok0 + r0) * a.out_stride + head * kDV + d) =
          __floats2bfloat162_rn(o[nd][0] * g0 * (each ? gate_factor(a.tail, tok0 + r0, head, d, kDV) : 1.f),
                                o[nd][1] * g0 * (each ? gate_factor(a.tail, tok0 + r0, head, d + 1, kDV) : 1.f));
    if (ok1)
      *reinterpret_cast<__nv_bfloat162*>(a.out + static_cast<size_t>(tok0 + r1) * a.out_stride + head * kDV + d) =
          __floats2bfloat162_rn(o[nd][2] * g1 * (each ? gate_factor(a.tail, tok0 + r1, head, d, kDV) : 1.f),
                                o[nd][3] * g1 * (each ? gate_factor(a.tail, tok0 + r1, head, d + 1, kDV) : 1.f));
  }
}
#endif  // sizes that are multiples of 16


// Whether this module's kernels have been allowed their dynamic shared memory.  File-scope statics on
// purpose: a static inside a function template is one object for the whole process, shared by every
// compiled variant of this file that is loaded, and a variant would then skip its own kernels.
static bool g_mma_attr_set = false;
static bool g_simt_attr_set[2] = {false, false};

template <typename T>
int launch_maps_decode(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt, int max_blocks,
                       const int32_t* items, float* part_o, float* part_ml, int max_parts, void* out, int out_stride,
                       int nitems, int heads, int kv_heads, int page_size, int window, int keep_first, float scale,
                       float softcap, float lambda, float post_scale, float eps, int unit_norm, const float* sink,
                       const float* slopes, const void* gate, int gate_stride, int gate_mode, cudaStream_t stream) {
  MapsDecodeArgs<T> a;
  a.tail.sink = sink;
  a.tail.slopes = slopes;
  a.tail.gate = static_cast<const T*>(gate);
  a.tail.gate_stride = gate_stride;
  a.tail.gate_mode = gate == nullptr ? 0 : gate_mode;
  a.q = static_cast<const T*>(q);
  a.q_stride = q_stride;
  a.kcache = static_cast<const T*>(kc);
  a.vcache = static_cast<const T*>(vc);
  a.block_table = bt;
  a.max_blocks = max_blocks;
  a.items = reinterpret_cast<const int4*>(items);
  a.part_o = part_o;
  a.part_ml = part_ml;
  a.max_parts = max_parts;
  a.out = static_cast<T*>(out);
  a.out_stride = out_stride;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.page_size = page_size;
  a.mask.window = window;
  a.mask.keep_first = keep_first;
  a.scale = scale;
  a.softcap = softcap;
  a.lambda = lambda;
  a.post_scale = post_scale;
  a.eps = eps;
  a.unit_norm = unit_norm;
  const int groups = (heads / kv_heads + kRows - 1) / kRows;
  cudaError_t e = launch_kernel(maps_decode_kernel<T>, dim3(max_parts, kv_heads * groups, nitems), dim3(kThreads), 0, stream,
                                a);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = launch_kernel(maps_merge_kernel<T>, dim3(nitems, heads), dim3(kThreads), 0, stream, a);
  return static_cast<int>(e);
}

template <typename T>
int launch_maps_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt, int max_blocks,
                        const int32_t* tile_seq, const int32_t* tile_tok, const int32_t* tile_rows,
                        const int32_t* positions, void* out, int out_stride, int tiles, int tile_rows_max, int heads,
                        int kv_heads, int page_size, int window, int keep_first, float scale, float softcap,
                        float lambda, float post_scale, float eps, int unit_norm, const float* sink,
                        const float* slopes, const void* gate, int gate_stride, int gate_mode, int impl,
                        cudaStream_t stream) {
  MapsPrefillArgs<T> a;
  a.tail.sink = sink;
  a.tail.slopes = slopes;
  a.tail.gate = static_cast<const T*>(gate);
  a.tail.gate_stride = gate_stride;
  a.tail.gate_mode = gate == nullptr ? 0 : gate_mode;
  a.q = static_cast<const T*>(q);
  a.q_stride = q_stride;
  a.kcache = static_cast<const T*>(kc);
  a.vcache = static_cast<const T*>(vc);
  a.block_table = bt;
  a.max_blocks = max_blocks;
  a.tile_seq = tile_seq;
  a.tile_tok = tile_tok;
  a.tile_rows = tile_rows;
  a.positions = positions;
  a.out = static_cast<T*>(out);
  a.out_stride = out_stride;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.page_size = page_size;
  a.tile_quarters = (tile_rows_max + kBQ - 1) / kBQ;
  a.mask.window = window;
  a.mask.keep_first = keep_first;
  a.scale = scale;
  a.softcap = softcap;
  a.lambda = lambda;
  a.post_scale = post_scale;
  a.eps = eps;
  a.unit_norm = unit_norm;
#ifdef RL_MAPS_HAVE_MMA
  if (sizeof(T) == 2 && impl != 1 && q_stride % 2 == 0 && out_stride % 2 == 0 && (page_size & (page_size - 1)) == 0 &&
      reinterpret_cast<uintptr_t>(q) % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0 &&
      reinterpret_cast<uintptr_t>(kc) % 16 == 0 && reinterpret_cast<uintptr_t>(vc) % 16 == 0) {
    MapsPrefillArgs<bf16> b;
    static_assert(sizeof(b) == sizeof(a), "one layout for both element types");
    memcpy(&b, &a, sizeof(b));
    b.tile_quarters = (tile_rows_max + kTQ - 1) / kTQ;
    const size_t need = kStages * (kTK * kLDK + kTK * kLDV) * sizeof(bf16) + (kM == 2 ? kTQ * kDV * sizeof(float) : 0);
    if (!g_mma_attr_set && need > 48 * 1024) {
      cudaFuncSetAttribute(maps_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(need));
      g_mma_attr_set = true;
    }
    return static_cast<int>(launch_kernel(maps_prefill_mma_kernel, dim3(tiles * b.tile_quarters, heads), dim3(128), need,
                                          stream, b));
  }
#endif
  if (impl == 2) return static_cast<int>(cudaErrorInvalidValue);      // the tensor-core kernel was asked for
  const size_t smem = (kBQ * (kD + 1) + kBK * (kD + 1) + kBK * kDV + kBQ * (kBK + 1)) * sizeof(float);
  bool& attr_set = g_simt_attr_set[sizeof(T) == 2 ? 1 : 0];
  if (!attr_set && smem > 48 * 1024) {
    cudaFuncSetAttribute(maps_prefill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    attr_set = true;
  }
  return static_cast<int>(launch_kernel(maps_prefill_kernel<T>, dim3(tiles * a.tile_quarters, heads), dim3(kThreads),
                                        smem, stream, a));
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_maps_partition() { return kPart; }

int rl_maps_decode(int dtype, const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                   int max_blocks, const int32_t* items, float* part_o, float* part_ml, int max_parts, void* out,
                   int out_stride, int nitems, int heads, int kv_heads, int page_size, int window, int keep_first,
                   float scale, float softcap, float lambda, float post_scale, float eps, int unit_norm,
                   const float* sink, const float* slopes, const void* gate, int gate_stride, int gate_mode,
                   cudaStream_t stream) {
  if (nitems <= 0 || max_parts <= 0) return 0;
  if (dtype == 0)
    return launch_maps_decode<float>(q, q_stride, kc, vc, bt, max_blocks, items, part_o, part_ml, max_parts, out,
                                     out_stride, nitems, heads, kv_heads, page_size, window, keep_first, scale, softcap,
                                     lambda, post_scale, eps, unit_norm, sink, slopes, gate, gate_stride, gate_mode, stream);
  return launch_maps_decode<bf16>(q, q_stride, kc, vc, bt, max_blocks, items, part_o, part_ml, max_parts, out,
                                  out_stride, nitems, heads, kv_heads, page_size, window, keep_first, scale, softcap,
                                  lambda, post_scale, eps, unit_norm, sink, slopes, gate, gate_stride, gate_mode, stream);
}

int rl_maps_prefill(int dtype, const void* q, int q_stride, const void* kc, const void* vc, const int32_t* bt,
                    int max_blocks, const int32_t* tile_seq, const int32_t* tile_tok, const int32_t* tile_rows,
                    const int32_t* positions, void* out, int out_stride, int tiles, int tile_rows_max, int heads,
                    int kv_heads, int page_size, int window, int keep_first, float scale, float softcap, float lambda,
                    float post_scale, float eps, int unit_norm, const float* sink, const float* slopes, const void* gate,
                    int gate_stride, int gate_mode, int impl, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (dtype == 0)
    return launch_maps_prefill<float>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows, positions,
                                      out, out_stride, tiles, tile_rows_max, heads, kv_heads, page_size, window,
                                      keep_first, scale, softcap, lambda, post_scale, eps, unit_norm, sink, slopes, gate, gate_stride,
                                      gate_mode, impl, stream);
  return launch_maps_prefill<bf16>(q, q_stride, kc, vc, bt, max_blocks, tile_seq, tile_tok, tile_rows, positions,
                                   out, out_stride, tiles, tile_rows_max, heads, kv_heads, page_size, window,
                                   keep_first, scale, softcap, lambda, post_scale, eps, unit_norm, sink, slopes, gate, gate_stride,
                                      gate_mode, impl, stream);
}

}  // extern "C"
