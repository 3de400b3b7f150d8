// Routed feed-forward (mixture of experts): the router, the grouping of (token, expert) pairs by
// expert, and the experts' two products as grouped matrix products.
//
//   router:   z = W_r x (float32 sums; in this kernel, or handed in as float32 logits), score = sigmoid(z) (or softmax over the experts); experts lie in
//             `groups` equal groups of neighbours; a group's score is the sum of its `group_top` best
//             scores; only experts of the best `keep` groups can be chosen; the `top` best of those are
//             the token's experts, weighted by their scores (optionally divided by their sum);
//             a choice bias per expert may be added to the scores for the choice alone (the weights are the
//             scores without it); the weights may be multiplied by a constant
//   identity: router outputs beyond the experts that have matrices stand for the input itself: their pairs
//             get no tiles, and the combine kernel takes the token's input row in place of a product
//   pairs:    pair p = token * top + k; `order` lists the pairs expert by expert, `tile_expert` /
//             `tile_begin` / `tile_rows` cut every expert's pairs into tiles of up to 64 rows
//   products: up:   act[p, :]  = f(W_up[e]   x[token(p), :])      f = activation
//             down: y[p, :]    =   W_down[e] act[p, :]
//   combine:  out[t, :] = sum_k weight[t, k] * y[t * top + k, :] (+ shared[t, :]), k in order
//
// A pair's results do not depend on which other pairs share its tile or on the order within the
// expert's list: every output element is one thread's sum over k in a fixed order.  All sums are float32.
// bfloat16 operands go through mma.sync (m16n8k16, float32 accumulators); float32 operands through
// FFMA only; steps of a handful of pairs stream the chosen experts' weights through FFMA in both types.
#include "common.cuh"

namespace rl {

enum { ACT_NONE = 0, ACT_RELU_SQ = 1, ACT_GELU_ERF = 2, ACT_SILU = 3, ACT_GELU_TANH = 4 };

__device__ __forceinline__ float moe_activate(float z, int mode) {
  switch (mode) {
    case ACT_RELU_SQ: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_GELU_ERF: return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
    case ACT_SILU: return z / (1.f + expf(-z));
    case ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    default: return z;
  }
}

// ------------------------------------------------------------------ router
// One warp per token.  Scores live in shared memory (experts floats per warp).  The largest score wins,
// the lower index among equals.
struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, a.v, o);
    const int i = __shfl_xor_sync(0xffffffffu, a.i, o);
    if (v > a.v || (v == a.v && i < a.i)) {
      a.v = v;
      a.i = i;
    }
  }
  return a;
}

template <typename TA, typename TW>
__global__ void moe_route_kernel(const TA* __restrict__ x, int ld, const TW* __restrict__ router, int tokens,
                                 int width, int experts, int groups, int keep, int group_top, int top, int softmax,
                                 int renorm, const float* __restrict__ bias, const float* __restrict__ choice_bias,
                                 float weight_scale, float renorm_floor, int32_t* __restrict__ choice,
                                 float* __restrict__ weight) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * warps + warp;
  if (t >= tokens) return;
  float* score = sm + warp * (2 * experts + 2 * groups);   // [experts] scores, [experts] working copy, 2 x [groups]
  float* work = score + experts;
  float* gscore = work + experts;
  float* gsel = gscore + groups;
  const TA* xr = x + static_cast<size_t>(t) * ld;
  if (router == nullptr) {
    // x holds the logits themselves [tokens, experts] (a matrix product before this kernel made them)
    for (int e = lane; e < experts; e += 32) score[e] = to_float(xr[e]);
  } else {
    for (int e = 0; e < experts; ++e) {
      const TW* w = router + static_cast<size_t>(e) * width;
      float s = 0.f;
      for (int c = lane; c < width; c += 32) s = fmaf(to_float(xr[c]), to_float(w[c]), s);
      s = warp_sum(s);
      if (lane == 0) score[e] = s;
    }
  }
  __syncwarp();
  if (bias != nullptr) {            // a bias of the router's logits
    for (int e = lane; e < experts; e += 32) score[e] += bias[e];
    __syncwarp();
  }
  if (softmax) {
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, score[e]);
    mx = warp_max(mx);
    float l = 0.f;
    for (int e = lane; e < experts; e += 32) l += expf(score[e] - mx);
    l = warp_sum(l);
    for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - mx) / l;
  } else {
    for (int e = lane; e < experts; e += 32) score[e] = 1.f / (1.f + expf(-score[e]));
  }
  __syncwarp();
  for (int e = lane; e < experts; e += 32) work[e] = score[e] + (choice_bias != nullptr ? choice_bias[e] : 0.f);
  __syncwarp();
  const int per = experts / groups;
  if (groups > 1 && keep < groups) {
    // a group's score: the sum of its group_top best scores
    for (int g = lane; g < groups; g += 32) {
      float total = 0.f;
      int taken_a = -1;                    // (group_top is small: the best, then the best of the rest, ...)
      float last = INFINITY;
      for (int k = 0; k < group_top && k < per; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = 0; e < per; ++e) {
          const float v = score[g * per + e];
          // next in the order (value descending, index ascending) after (last, taken_a)
          const bool after = v < last || (v == last && e > taken_a);
          if (after && (v > best || bi < 0)) {
            best = v;
            bi = e;
          }
        }
        total += best;
        last = best;
        taken_a = bi;
      }
      gscore[g] = total;
    }
    __syncwarp();
    // the best `keep` groups stay (the lower index among equals); the others' experts cannot be chosen
    for (int g = lane; g < groups; g += 32) gsel[g] = 0.f;
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      ArgMax a = {-INFINITY, 0x7fffffff};
      for (int g = lane; g < groups; g += 32) {
        const float v = gscore[g];
        if (gsel[g] == 0.f && (a.i == 0x7fffffff || v > a.v)) {
          a.v = v;
          a.i = g;
        }
      }
      a = warp_argmax(a);
      __syncwarp();
      if (lane == 0 && a.i < groups) gsel[a.i] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gsel[e / per] == 0.f) work[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    ArgMax a = {-INFINITY, 0x7fffffff};
    for (int e = lane; e < experts; e += 32) {
      const float v = work[e];
      if (v > a.v || (v == a.v && e < a.i)) {
        a.v = v;
        a.i = e;
      }
    }
    a = warp_argmax(a);
    __syncwarp();
    const bool found = a.i < experts;              // (false only if fewer experts are allowed than asked for)
    if (lane == 0) {
      choice[static_cast<size_t>(t) * top + k] = found ? a.i : 0;
      weight[static_cast<size_t>(t) * top + k] = found ? score[a.i] : 0.f;
      if (found) work[a.i] = -INFINITY;
    }
    if (found) total += score[a.i];
    __syncwarp();
  }
  if (lane == 0 && (renorm || weight_scale != 1.f)) {
    for (int k = 0; k < top; ++k) {
      float wk = weight[static_cast<size_t>(t) * top + k];
      if (renorm) wk /= total + renorm_floor;
      weight[static_cast<size_t>(t) * top + k] = wk * weight_scale;
    }
  }
}

// ------------------------------------------------------------------ pairs grouped by expert
// One CTA.  counts -> offsets -> order; then the tiles.  meta: [0] number of tiles.
constexpr int kTileRows = 64;

__global__ void moe_group_kernel(const int32_t* __restrict__ choice, int pairs, int experts, int tiled,
                                 int32_t* __restrict__ order, int32_t* __restrict__ tile_expert,
                                 int32_t* __restrict__ tile_begin, int32_t* __restrict__ tile_rows,
                                 int32_t* __restrict__ meta) {
  pdl_launch();
  pdl_wait();
  extern __shared__ int32_t cnt[];          // [experts] counts, then [experts + 1] offsets
  int32_t* off = cnt + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[choice[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = at;
      for (int r = 0; r < cnt[e] && e < tiled; r += kTileRows) {      // (experts from `tiled` on have no matrices)
        tile_expert[tiles] = e;
        tile_begin[tiles] = at + r;
        tile_rows[tiles] = min(kTileRows, cnt[e] - r);
        ++tiles;
      }
      at += cnt[e];
    }
    off[experts] = at;
    meta[0] = tiles;
  }
  __syncthreads();
  // a pair's place within its expert's list: the pairs of an expert in ascending order (a fixed order,
  // though no result depends on it)
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  if (pairs <= 4096) {
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      const int e = choice[p];
      int before = 0;
      for (int q = 0; q < p; ++q) before += choice[q] == e;
      order[off[e] + before] = p;
    }
  } else {
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      const int e = choice[p];
      order[off[e] + atomicAdd(&cnt[e], 1)] = p;
    }
  }
}

// ------------------------------------------------------------------ grouped products
// One CTA per (tile of up to 64 pairs of one expert, 64 output features).  Row r of the tile is pair
// order[begin + r]; its input row is src[pair / src_div] (src_div = top for the first product, whose
// input is the token's row; 1 for the second, whose input is the pair's own row); its output row is
// dst[pair].  W is [experts, n, k].
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
moe_gemm_simt_kernel(const TA* __restrict__ src, int ld_src, int src_div, const TW* __restrict__ w, int n, int k,
                     TA* __restrict__ dst, int ld_dst, const int32_t* __restrict__ order,
                     const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_begin,
                     const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ meta, int act) {
  pdl_launch();
  pdl_wait();
  constexpr int BM = kTileRows, BN = 64, BK = 32, RPT = BM / 8;
  __shared__ float As[BM][BK + 1];
  __shared__ float Ws[BN][BK + 1];
  __shared__ int32_t pair_of[BM];
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], begin = tile_begin[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.y * BN;
  const TW* we = w + static_cast<size_t>(e) * n * k;
  if (threadIdx.x < BM) pair_of[threadIdx.x] = threadIdx.x < rows ? order[begin + threadIdx.x] : -1;
  __syncthreads();
  // thread (ty, tx): rows ty * 8 .. + 7 (8 groups), columns tx, tx + 16, tx + 32, tx + 48
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  float acc[RPT][4];
#pragma unroll
  for (int i = 0; i < RPT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += BK) {
    __syncthreads();
    for (int i = threadIdx.x; i < BM * BK; i += 128) {
      const int r = i / BK, c = i - r * BK;
      const int p = pair_of[r];
      As[r][c] = (p >= 0 && k0 + c < k) ? to_float(src[static_cast<size_t>(p / src_div) * ld_src + k0 + c]) : 0.f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += 128) {
      const int r = i / BK, c = i - r * BK;
      Ws[r][c] = (n0 + r < n && k0 + c < k) ? to_float(we[static_cast<size_t>(n0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < BK; ++c) {
      float av[RPT], wv[4];
#pragma unroll
      for (int i = 0; i < RPT; ++i) av[i] = As[ty * RPT + i][c];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[tx + 16 * j][c];
#pragma unroll
      for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int p = pair_of[ty * RPT + i];
    if (p < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx + 16 * j;
      if (col < n) dst[static_cast<size_t>(p) * ld_dst + col] = from_float<TA>(moe_activate(acc[i][j], act));
    }
  }
}

// The tile on the tensor cores for bfloat16: 64 pairs x 128 output features per CTA, eight warps in a
// 2 x 4 grid (32 rows x 32 features each: 2 x 4 MMAs per 16 of k).  A (the pairs' rows) and W tiles of
// 32 k go through shared memory as bfloat16; the next k block's 16-byte pieces are asked for before the
// MMAs of the running one and stored after them.  mma.sync.m16n8k16, float32 accumulators, k ascending.
__device__ __forceinline__ void mma_bf16_16816(float* d, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

constexpr int kMmaCols = 128;

__global__ void __launch_bounds__(256)
moe_gemm_mma_kernel(const bf16* __restrict__ src, int ld_src, int src_div, const bf16* __restrict__ w, int n, int k,
                    bf16* __restrict__ dst, int ld_dst, const int32_t* __restrict__ order,
                    const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_begin,
                    const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ meta, int act) {
  pdl_launch();
  pdl_wait();
  constexpr int BM = kTileRows, BN = kMmaCols, BK = 32, LD = BK + 8;      // 80-byte rows: fragment reads hit distinct banks
  __shared__ __align__(16) bf16 As[BM][LD];
  __shared__ __align__(16) bf16 Ws[BN][LD];
  __shared__ int32_t pair_of[BM];
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], begin = tile_begin[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.y * BN;
  const bf16* we = w + static_cast<size_t>(e) * n * k;
  if (threadIdx.x < BM) pair_of[threadIdx.x] = threadIdx.x < rows ? order[begin + threadIdx.x] : -1;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;            // this warp's 32 rows and 32 features
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int f = 0; f < 4; ++f) acc[i][j][f] = 0.f;
  // this thread's pieces of a k block: one of A (64 rows x 4 pieces), two of W (128 rows x 4 pieces)
  const int ar = threadIdx.x >> 2, ac = (threadIdx.x & 3) * 8;
  const int ap = pair_of[ar];
  const bf16* a_src = ap >= 0 ? src + static_cast<size_t>(ap / src_div) * ld_src + ac : nullptr;
  const bf16* w_src[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = ar + h * 64;
    w_src[h] = n0 + r < n ? we + static_cast<size_t>(n0 + r) * k + ac : nullptr;
  }
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 pa = zero, pw[2] = {zero, zero};
  auto fetch = [&](int k0) {
    const bool in = k0 + ac < k;
    pa = (a_src != nullptr && in) ? *reinterpret_cast<const uint4*>(a_src + k0) : zero;
#pragma unroll
    for (int h = 0; h < 2; ++h) pw[h] = (w_src[h] != nullptr && in) ? *reinterpret_cast<const uint4*>(w_src[h] + k0) : zero;
  };
  fetch(0);
  for (int k0 = 0; k0 < k; k0 += BK) {
    __syncthreads();                                  // the block before has been read
    *reinterpret_cast<uint4*>(&As[ar][ac]) = pa;
    *reinterpret_cast<uint4*>(&Ws[ar][ac]) = pw[0];
    *reinterpret_cast<uint4*>(&Ws[ar + 64][ac]) = pw[1];
    __syncthreads();
    if (k0 + BK < k) fetch(k0 + BK);                  // on its way while the MMAs run
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t b[4][2];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bf16* wr = &Ws[wn * 32 + j * 8 + gid][kk + tig * 2];
        b[j][0] = *reinterpret_cast<const uint32_t*>(wr);
        b[j][1] = *reinterpret_cast<const uint32_t*>(wr + 8);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        uint32_t a[4];
        const bf16* arow = &As[wm * 32 + i * 16 + gid][kk + tig * 2];
        a[0] = *reinterpret_cast<const uint32_t*>(arow);
        a[1] = *reinterpret_cast<const uint32_t*>(arow + 8 * LD);
        a[2] = *reinterpret_cast<const uint32_t*>(arow + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(arow + 8 * LD + 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a, b[j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int p = pair_of[wm * 32 + i * 16 + gid + half * 8];
      if (p < 0) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + wn * 32 + j * 8 + tig * 2;
        const float v0 = moe_activate(acc[i][j][half * 2], act), v1 = moe_activate(acc[i][j][half * 2 + 1], act);
        bf16* d = dst + static_cast<size_t>(p) * ld_dst + col;
        if (col + 1 < n && (ld_dst % 2 == 0)) {
          *reinterpret_cast<__nv_bfloat162*>(d) = __floats2bfloat162_rn(v0, v1);
        } else {
          if (col < n) d[0] = __float2bfloat16_rn(v0);
          if (col + 1 < n) d[1] = __float2bfloat16_rn(v1);
        }
      }
    }
}

// For a handful of pairs (single-token steps) the products are bound by the stream of the chosen experts'
// weights: one CTA per (tile, 16 output features), a warp takes four features at once and streams their
// weight rows in 16-byte pieces, up to four of the tile's rows at a time (their input rows come from L1).
template <typename T>
__global__ void __launch_bounds__(128)
moe_gemv_kernel(const T* __restrict__ src, int ld_src, int src_div, const T* __restrict__ w, int n, int k,
                T* __restrict__ dst, int ld_dst, const int32_t* __restrict__ order,
                const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_begin,
                const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ meta, int act) {
  pdl_launch();
  pdl_wait();
  constexpr int VEC = Vec16<T>::N, NF = 4, NR = 4;
  const int tile = blockIdx.x;
  if (tile >= meta[0]) return;
  const int e = tile_expert[tile], begin = tile_begin[tile], rows = tile_rows[tile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.y * 16 + warp * NF;
  if (f0 >= n) return;
  const T* we = w + static_cast<size_t>(e) * n * k;
  const bool vec = (k % VEC == 0) && (ld_src % VEC == 0) && (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  for (int r0 = 0; r0 < rows; r0 += NR) {
    const int nr = min(NR, rows - r0);
    int pair[NR];
    const T* xr[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      pair[r] = r < nr ? order[begin + r0 + r] : 0;
      xr[r] = src + static_cast<size_t>(pair[r] / src_div) * ld_src;
    }
    float acc[NF][NR];
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int r = 0; r < NR; ++r) acc[f][r] = 0.f;
    if (vec) {
      for (int c = lane * VEC; c < k; c += 32 * VEC) {
        float wv[NF][VEC];
#pragma unroll
        for (int f = 0; f < NF; ++f) {
          if (f0 + f < n) load16(we + static_cast<size_t>(f0 + f) * k + c, wv[f]);
          else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) wv[f][i] = 0.f;
          }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          if (r < nr) {
            float xv[VEC];
            load16(xr[r] + c, xv);
#pragma unroll
            for (int f = 0; f < NF; ++f)
#pragma unroll
              for (int i = 0; i < VEC; ++i) acc[f][r] = fmaf(wv[f][i], xv[i], acc[f][r]);
          }
        }
      }
    } else {
      for (int c = lane; c < k; c += 32) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const float xv = r < nr ? to_float(xr[r][c]) : 0.f;
#pragma unroll
          for (int f = 0; f < NF; ++f)
            if (f0 + f < n) acc[f][r] = fmaf(to_float(we[static_cast<size_t>(f0 + f) * k + c]), xv, acc[f][r]);
        }
      }
    }
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float v = warp_sum(acc[f][r]);
        if (lane == 0 && r < nr && f0 + f < n)
          dst[static_cast<size_t>(pair[r]) * ld_dst + f0 + f] = from_float<T>(moe_activate(v, act));
      }
  }
}

// ------------------------------------------------------------------ combine
// out[t, c] = sum_k weight[t, k] * y[t * top + k, c] (+ shared[t, c])
template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const float* __restrict__ weight,
                                   const TA* __restrict__ shared, TA* __restrict__ out, int width, int top,
                                   const int32_t* __restrict__ choice, int real_experts, const TA* __restrict__ x,
                                   int ld_x) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t pair = static_cast<size_t>(t) * top + k;
      // (an identity expert's pair has no product: its term is the token's input row)
      const bool same = choice != nullptr && choice[pair] >= real_experts;
      s = fmaf(weight[pair], same ? to_float(x[static_cast<size_t>(t) * ld_x + c]) : to_float(y[pair * width + c]), s);
    }
    if (shared != nullptr) s += to_float(shared[static_cast<size_t>(t) * width + c]);
    out[static_cast<size_t>(t) * width + c] = from_float<TA>(s);
  }
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_moe_tile_rows() { return kTileRows; }

int rl_moe_route(const void* x, int act_dtype, int ld, const void* router, int w_dtype, int tokens, int width,
                 int experts, int groups, int keep, int group_top, int top, int softmax, int renorm, const float* bias,
                 const float* choice_bias, float weight_scale, float renorm_floor, int32_t* choice, float* weight,
                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * (2 * experts + 2 * groups) * sizeof(float);
  dim3 grid((tokens + warps - 1) / warps), block(warps * 32);
#define RL_CASE(TA, TW)                                                                                            \
  launch_kernel(moe_route_kernel<TA, TW>, grid, block, smem, stream, static_cast<const TA*>(x), ld,                \
                static_cast<const TW*>(router), tokens, width, experts, groups, keep, group_top, top, softmax,     \
                renorm, bias, choice_bias, weight_scale, renorm_floor, choice, weight)
  if (act_dtype == 0) RL_CASE(float, float);
  else if (w_dtype == 0) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_moe_group(const int32_t* choice, int pairs, int experts, int tiled, int32_t* order, int32_t* tile_expert,
                 int32_t* tile_begin, int32_t* tile_rows, int32_t* meta, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  launch_kernel(moe_group_kernel, dim3(1), dim3(256), (2 * experts + 1) * sizeof(int32_t), stream, choice, pairs,
                experts, tiled, order, tile_expert, tile_begin, tile_rows, meta);
  RL_LAUNCH_END();
}

// max_tiles: the most tiles the grouping can have made (pairs / 64 + experts); CTAs beyond the real
// number leave at once.  few_pairs: the weight-streaming kernel for a handful of pairs (single-token steps).
int rl_moe_gemm(int act_dtype, const void* src, int ld_src, int src_div, const void* w, int n, int k, void* dst,
                int ld_dst, const int32_t* order, const int32_t* tile_expert, const int32_t* tile_begin,
                const int32_t* tile_rows, const int32_t* meta, int max_tiles, int few_pairs, int act,
                cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (few_pairs) {
    dim3 g(max_tiles, (n + 15) / 16);
    if (act_dtype == 0)
      launch_kernel(moe_gemv_kernel<float>, g, dim3(128), 0, stream, static_cast<const float*>(src), ld_src, src_div,
                    static_cast<const float*>(w), n, k, static_cast<float*>(dst), ld_dst, order, tile_expert, tile_begin,
                    tile_rows, meta, act);
    else
      launch_kernel(moe_gemv_kernel<bf16>, g, dim3(128), 0, stream, static_cast<const bf16*>(src), ld_src, src_div,
                    static_cast<const bf16*>(w), n, k, static_cast<bf16*>(dst), ld_dst, order, tile_expert, tile_begin,
                    tile_rows, meta, act);
    RL_LAUNCH_END();
  }
  dim3 grid(max_tiles, (n + 63) / 64);
  if (act_dtype == 0) {
    launch_kernel(moe_gemm_simt_kernel<float, float>, grid, dim3(128), 0, stream, static_cast<const float*>(src),
                  ld_src, src_div, static_cast<const float*>(w), n, k, static_cast<float*>(dst), ld_dst, order,
                  tile_expert, tile_begin, tile_rows, meta, act);
  } else if (k % 8 == 0 && ld_src % 8 == 0 && (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
             (reinterpret_cast<uintptr_t>(w) % 16 == 0)) {
    launch_kernel(moe_gemm_mma_kernel, dim3(max_tiles, (n + kMmaCols - 1) / kMmaCols), dim3(256), 0, stream,
                  static_cast<const bf16*>(src), ld_src, src_div,
                  static_cast<const bf16*>(w), n, k, static_cast<bf16*>(dst), ld_dst, order, tile_expert, tile_begin,
                  tile_rows, meta, act);
  } else {
    launch_kernel(moe_gemm_simt_kernel<bf16, bf16>, grid, dim3(128), 0, stream, static_cast<const bf16*>(src), ld_src,
                  src_div, static_cast<const bf16*>(w), n, k, static_cast<bf16*>(dst), ld_dst, order, tile_expert,
                  tile_begin, tile_rows, meta, act);
  }
  RL_LAUNCH_END();
}

int rl_moe_combine(int act_dtype, const void* y, const float* weight, const void* shared, void* out, int tokens,
                   int width, int top, const int32_t* choice, int real_experts, const void* x, int ld_x,
                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  dim3 grid(min((width + 255) / 256, 32), tokens);
  if (act_dtype == 0)
    launch_kernel(moe_combine_kernel<float>, grid, dim3(256), 0, stream, static_cast<const float*>(y), weight,
                  static_cast<const float*>(shared), static_cast<float*>(out), width, top, choice, real_experts,
                  static_cast<const float*>(x), ld_x);
  else
    launch_kernel(moe_combine_kernel<bf16>, grid, dim3(256), 0, stream, static_cast<const bf16*>(y), weight,
                  static_cast<const bf16*>(shared), static_cast<bf16*>(out), width, top, choice, real_experts,
                  static_cast<const bf16*>(x), ld_x);
  RL_LAUNCH_END();
}

}  // extern "C"
