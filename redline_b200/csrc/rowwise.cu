// Row-wise kernels for blocks that norm a sublayer's input AND its output: layer norm (weight, no
// bias) fused with the add to the float32 residual stream and with the norm that follows; bias +
// activation over a range of columns; the write of any per-token tensor into its paged cache; the
// gated unit-RMS norm that closes a linear-attention mixer; a gated activation act(gate) * up; and what
// attention heads may need between their projection and the cache: an RMS norm of queries and keys
// (per head or over the whole projection), a rotation of pairs (neighbours, or entry i with entry
// i + half), a mix of the values with those of an earlier layer.
//
// Activations are float or bfloat16; means, variances, the stream and the activations'
// arithmetic are float.  The variance is the mean of squared deviations (two passes over a row
// held in shared memory), not E[x^2] - E[x]^2.
#include "common.cuh"

namespace rl {

enum { ACT_NONE = 0, ACT_RELU_SQ = 1, ACT_GELU_ERF = 2, ACT_SILU = 3, ACT_GELU_TANH = 4, ACT_SIGMOID = 5,
       ACT_CLAMPED_SWISH = 6 };

__device__ __forceinline__ float activate(float z, int mode) {
  switch (mode) {
    case ACT_RELU_SQ: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_GELU_ERF: return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
    case ACT_SILU: return z / (1.f + expf(-z));
    case ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.79788456080286536f * (z + 0.044715f * z * z * z)));
    case ACT_SIGMOID: return 1.f / (1.f + expf(-z));
    default: return z;
  }
}

// ------------------------------------------------ residual += LN(delta) * post_w;  out = LN(residual) * pre_w
// One CTA per row; the row lives in dynamic shared memory (hidden floats).
//   delta / post_w given:  the sublayer's output is normed and added to the stream (written back)
//   delta without post_w:  the sublayer's output is added as it is
//   out / pre_w given:     the (new) stream row is normed for the next sublayer
//   out without pre_w:     the (new) stream row is handed on as it is, in the activation type (blocks
//                          whose sublayers read the stream itself)
//   rows_idx given:        out row i comes from stream row rows_idx[i]; nothing is added (delta is null)
// kind: 0 layer norm (mean removed), 1 RMS norm; both with a weight and without a bias.
template <typename TA, typename TW>
__global__ void sandwich_norm_kernel(float* __restrict__ residual, const TA* __restrict__ delta, int ld_delta,
                                     const TW* __restrict__ post_w, const TW* __restrict__ pre_w,
                                     TA* __restrict__ out, int ld_out, const int32_t* __restrict__ rows_idx,
                                     int hidden, float eps, int kind) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows_idx ? rows_idx[r] : r;
  float* res = residual + static_cast<size_t>(src) * hidden;
  const float inv_n = 1.f / static_cast<float>(hidden);
  if (delta != nullptr && post_w == nullptr) {
    const TA* d = delta + static_cast<size_t>(src) * ld_delta;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = res[c] + to_float(d[c]);
      res[c] = v;
      row[c] = v;
    }
  } else if (delta != nullptr) {
    const TA* d = delta + static_cast<size_t>(src) * ld_delta;
    float s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = to_float(d[c]);
      row[c] = v;
      s += v;
    }
    const float mean = kind == 0 ? block_sum(s, scratch) * inv_n : 0.f;
    float q = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = row[c] - mean;
      q += v * v;
    }
    const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = res[c] + (row[c] - mean) * rstd * to_float(post_w[c]);
      res[c] = v;
      row[c] = v;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) row[c] = res[c];
  }
  if (out == nullptr) return;
  if (pre_w == nullptr) {
    TA* o = out + static_cast<size_t>(r) * ld_out;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_float<TA>(row[c]);
    return;
  }
  float s = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) s += row[c];
  const float mean = kind == 0 ? block_sum(s, scratch) * inv_n : 0.f;
  float q = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = row[c] - mean;
    q += v * v;
  }
  const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
  TA* o = out + static_cast<size_t>(r) * ld_out;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    o[c] = from_float<TA>((row[c] - mean) * rstd * to_float(pre_w[c]));
}

// The same for rows of up to EPT x blockDim elements, the row in registers: every global load (addend,
// stream, both weights) is asked for before the first sum, so that a row costs one round trip to memory
// and four block reductions.  Thread t holds elements t, t + blockDim, ...
template <typename TA, typename TW, int EPT>
__global__ void sandwich_norm_reg_kernel(float* __restrict__ residual, const TA* __restrict__ delta, int ld_delta,
                                         const TW* __restrict__ post_w, const TW* __restrict__ pre_w,
                                         TA* __restrict__ out, int ld_out, const int32_t* __restrict__ rows_idx,
                                         int hidden, float eps, int kind) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows_idx ? rows_idx[r] : r;
  float* res = residual + static_cast<size_t>(src) * hidden;
  const float inv_n = 1.f / static_cast<float>(hidden);
  float v[EPT], d[EPT], pw[EPT], nw[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    const bool in = c < hidden;
    v[i] = in ? res[c] : 0.f;
    d[i] = (in && delta != nullptr) ? to_float(delta[static_cast<size_t>(src) * ld_delta + c]) : 0.f;
    pw[i] = (in && post_w != nullptr) ? to_float(post_w[c]) : 0.f;
    nw[i] = (in && out != nullptr && pre_w != nullptr) ? to_float(pre_w[c]) : 0.f;
  }
  if (delta != nullptr) {
    if (post_w == nullptr) {
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] += d[i];
    } else {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < EPT; ++i) s += d[i];
      const float mean = kind == 0 ? block_sum(s, scratch) * inv_n : 0.f;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < EPT; ++i) {
        const float x = (threadIdx.x + i * blockDim.x < hidden) ? d[i] - mean : 0.f;
        q += x * x;
      }
      const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
#pragma unroll
      for (int i = 0; i < EPT; ++i) v[i] += (d[i] - mean) * rstd * pw[i];
    }
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < hidden) res[c] = v[i];
    }
  }
  if (out == nullptr) return;
  if (pre_w == nullptr) {
    TA* o = out + static_cast<size_t>(r) * ld_out;
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < hidden) o[c] = from_float<TA>(v[i]);
    }
    return;
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) s += v[i];
  const float mean = kind == 0 ? block_sum(s, scratch) * inv_n : 0.f;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const float x = (threadIdx.x + i * blockDim.x < hidden) ? v[i] - mean : 0.f;
    q += x * x;
  }
  const float rstd = rsqrtf(block_sum(q, scratch) * inv_n + eps);
  TA* o = out + static_cast<size_t>(r) * ld_out;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < hidden) o[c] = from_float<TA>((v[i] - mean) * rstd * nw[i]);
  }
}

// ------------------------------------------------ x[r, c] = act(x[r, c] + bias[c]) for c < cols
template <typename TA>
__global__ void bias_act_kernel(TA* __restrict__ x, int ld, const float* __restrict__ bias, int cols, int mode,
                                int vec_ok) {
  pdl_launch();
  pdl_wait();
  TA* p = x + static_cast<size_t>(blockIdx.y) * ld;
  constexpr int VEC = Vec16<TA>::N;
  if (vec_ok) {      // rows start on 16-byte boundaries and cols is a multiple of the piece
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC; c < cols; c += gridDim.x * blockDim.x * VEC) {
      float v[VEC];
      load16(p + c, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        if (bias != nullptr) v[i] = to_float(from_float<TA>(v[i] + bias[c + i]));
        v[i] = activate(v[i], mode);
      }
      store16(p + c, v);
    }
    return;
  }
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
    float v = to_float(p[c]);
    if (bias != nullptr) v = to_float(from_float<TA>(v + bias[c]));   // (the biased projection is what is stored)
    p[c] = from_float<TA>(activate(v, mode));
  }
}

// ------------------------------------------------ cache[page, head, offset, :] = src[t, col + head * dim : ...]
// `cache` is [pages, heads, page_size, dim]; slots[t] = page * page_size + offset, negative: no write;
// a slot beyond the pool is not written and sets bit 2 of *status.
template <typename TA>
__global__ void cache_store_kernel(const TA* __restrict__ src, int ld, int col, int heads, int dim,
                                   const int32_t* __restrict__ slots, TA* __restrict__ cache, int page_size,
                                   long long num_slots, int* status) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, 4);
    return;
  }
  const size_t page = slot / page_size, off = slot % page_size;
  const TA* s = src + static_cast<size_t>(t) * ld + col;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int h = i / dim, d = i - h * dim;
    cache[((page * heads + h) * page_size + off) * dim + d] = s[i];
  }
}

// ------------------------------------------------ out = o / rms(o) * w * sigmoid(gate)
// o is the float32 output of a recurrence [T, n]; gate lies in a projection buffer (row stride ld_gate).
template <typename TA, typename TW>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const TA* __restrict__ gate, int ld_gate,
                                     const TW* __restrict__ w, TA* __restrict__ out, int n, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float* orow = o + static_cast<size_t>(r) * n;
  float q = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) q += orow[c] * orow[c];
  const float rstd = rsqrtf(block_sum(q, scratch) / static_cast<float>(n) + eps);
  const TA* g = gate + static_cast<size_t>(r) * ld_gate;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float s = 1.f / (1.f + expf(-to_float(g[c])));
    out[static_cast<size_t>(r) * n + c] = from_float<TA>(orow[c] * rstd * to_float(w[c]) * s);
  }
}

// ------------------------------------------------ out[r, i] = act(gu[r, i]) * gu[r, inter + i]
// mode ACT_CLAMPED_SWISH: g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(slope g) (u + 1).
template <typename TA>
__global__ void gated_act_kernel(const TA* __restrict__ gu, int ld, TA* __restrict__ out, int inter, int mode,
                                 float limit, float slope, const float* __restrict__ bias) {
  pdl_launch();
  pdl_wait();
  const TA* g = gu + static_cast<size_t>(blockIdx.y) * ld;
  TA* o = out + static_cast<size_t>(blockIdx.y) * inter;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < inter; c += gridDim.x * blockDim.x) {
    // (a bias [gate | up] of the product before is added on the way in)
    const float gate = to_float(g[c]) + (bias != nullptr ? bias[c] : 0.f);
    const float up = to_float(g[inter + c]) + (bias != nullptr ? bias[inter + c] : 0.f);
    if (mode == ACT_CLAMPED_SWISH) {
      const float z = fminf(gate, limit);
      const float u = fminf(fmaxf(up, -limit), limit);
      o[c] = from_float<TA>(z / (1.f + expf(-slope * z)) * (u + 1.f));
    } else {
      o[c] = from_float<TA>(activate(gate, mode) * up);
    }
  }
}

// ------------------------------------------------ queries, keys and values between projection and cache
// In place on the rows of a projection buffer, one CTA per token.  Two sections of heads (queries at
// q_col, keys at k_col; `dim` entries a head) are, in float32,
//   normed:   x / sqrt(mean(x^2) + eps) * w, the mean over one head (norm_mode 1, w of `dim` entries for all
//             heads) or over the whole section (norm_mode 2, w of heads * dim entries); 0: not normed;
//   rotated:  entries (2i, 2i+1), i < rot_pairs, of every head turn by the angle whose cosine and sine are
//             cos[pos, i] and sin[pos, i] (tables [max_pos, rot_pairs]); the other entries stay.  With rot_half
//             the pairs are (i, i + rot_pairs) instead.
// The values (v_size entries at v_col) are, with vmix_mode 1, copied to v_first [tokens, v_size]; with
// vmix_mode 2 replaced by (1 - lam) v + lam v_first.  A position beyond the tables sets bit 1 of *status.
// With `slots` the finished keys and values also go to their paged caches ([pages, k_heads, page_size, dim]
// and [pages, v_heads, page_size, v_size / v_heads]) at slots[t] = page * page_size + offset (negative: no
// write; beyond the pool: not written, bit 2 of *status).
// Two neighbouring entries as one access (the address is a multiple of the pair's size).
__device__ __forceinline__ void load2(const float* p, float& a, float& b) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  a = v.x;
  b = v.y;
}
__device__ __forceinline__ void load2(const bf16* p, float& a, float& b) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
  a = __low2float(v);
  b = __high2float(v);
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

struct HeadPrepArgs {
  int ld, q_col, q_heads, k_col, k_heads, dim, norm_mode;
  float eps;
  int rot_pairs, max_pos, v_col, v_size, vmix_mode;
  float lam;
  const int32_t* slots;
  int v_heads, page_size;
  long long num_slots;
  int pairs_ok;       // every head starts on a pair's boundary in the buffer, the weights and the caches
  int rot_half;       // 1: entry i < rot_pairs is paired with entry i + rot_pairs instead of its neighbour
};

template <typename TA, typename TW>
__global__ void head_prep_kernel(TA* __restrict__ x, const int32_t* __restrict__ positions,
                                 const TW* __restrict__ q_w, const TW* __restrict__ k_w,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 TA* __restrict__ v_first, TA* __restrict__ k_cache, TA* __restrict__ v_cache,
                                 int* status, const HeadPrepArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float head_sq[];           // per head of both sections: the sum of squares
  const int t = blockIdx.x;
  TA* row = x + static_cast<size_t>(t) * a.ld;
  int pos = positions[t];
  if (a.rot_pairs > 0 && (pos < 0 || pos >= a.max_pos)) {
    if (threadIdx.x == 0) atomicOr(status, 2);
    pos = 0;
  }
  long long slot = a.slots != nullptr ? a.slots[t] : -1;
  if (slot >= a.num_slots) {
    if (threadIdx.x == 0) atomicOr(status, 4);
    slot = -1;
  }
  const size_t page = slot >= 0 ? slot / a.page_size : 0, off = slot >= 0 ? slot % a.page_size : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int all_heads = a.q_heads + a.k_heads;
  if (a.norm_mode != 0) {
    for (int h = warp; h < all_heads; h += nwarps) {
      const TA* p = h < a.q_heads ? row + a.q_col + h * a.dim : row + a.k_col + (h - a.q_heads) * a.dim;
      float q = 0.f;
      for (int d = lane; d < a.dim; d += 32) {
        const float v = to_float(p[d]);
        q += v * v;
      }
      q = warp_sum(q);
      if (lane == 0) head_sq[h] = q;
    }
    __syncthreads();
  }
  for (int sec = 0; sec < 2; ++sec) {
    const int heads = sec == 0 ? a.q_heads : a.k_heads;
    const int h0 = sec == 0 ? 0 : a.q_heads;
    TA* p = row + (sec == 0 ? a.q_col : a.k_col);
    const TW* w = sec == 0 ? q_w : k_w;
    float whole = 1.f;
    if (a.norm_mode == 2) {        // every thread adds the section's heads in the same order
      float q = 0.f;
      for (int h = 0; h < heads; ++h) q += head_sq[h0 + h];
      whole = rsqrtf(q / static_cast<float>(heads * a.dim) + a.eps);
    }
    TA* kc = (sec == 1 && slot >= 0) ? k_cache : nullptr;
    const int n = heads * a.dim;
    if (a.pairs_ok) {              // two entries per trip, each pair one access
      for (int i = 2 * threadIdx.x; i < n; i += 2 * blockDim.x) {
        const int h = i / a.dim, d = i - h * a.dim;
        const float r = a.norm_mode == 2 ? whole
                        : (a.norm_mode == 1 ? rsqrtf(head_sq[h0 + h] / static_cast<float>(a.dim) + a.eps) : 1.f);
        float u, v;
        load2(p + i, u, v);
        if (a.norm_mode != 0) {
          float wu, wv;
          load2(w + (a.norm_mode == 2 ? i : d), wu, wv);
          u *= r * wu;
          v *= r * wv;
        }
        if (d < 2 * a.rot_pairs) {
          const float cs = cos_t[static_cast<size_t>(pos) * a.rot_pairs + (d >> 1)];
          const float sn = sin_t[static_cast<size_t>(pos) * a.rot_pairs + (d >> 1)];
          const float ru = u * cs - v * sn, rv = v * cs + u * sn;
          u = ru;
          v = rv;
        } else if (a.norm_mode == 0 && kc == nullptr) {
          continue;                  // nothing changes and nothing is cached
        }
        store2(p + i, u, v);
        if (kc != nullptr) {
          float cu, cv;              // what was stored, so that cache and buffer hold the same rounded values
          load2(p + i, cu, cv);
          store2(kc + ((page * heads + h) * a.page_size + off) * a.dim + d, cu, cv);
        }
      }
      continue;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int h = i / a.dim, d = i - h * a.dim;
      const bool paired = d < 2 * a.rot_pairs;
      // the second entry of a pair goes with the first one
      if (paired && (a.rot_half ? d >= a.rot_pairs : (d & 1))) continue;
      const int other = a.rot_half ? a.rot_pairs : 1, pair = a.rot_half ? d : (d >> 1);
      const float r = a.norm_mode == 2 ? whole
                      : (a.norm_mode == 1 ? rsqrtf(head_sq[h0 + h] / static_cast<float>(a.dim) + a.eps) : 1.f);
      const int wi = a.norm_mode == 2 ? i : d;
      float u = to_float(p[i]) * r;
      if (a.norm_mode != 0) u *= to_float(w[wi]);
      TA* c = kc != nullptr ? kc + ((page * heads + h) * a.page_size + off) * a.dim + d : nullptr;
      if (!paired) {
        const TA o = from_float<TA>(u);
        if (a.norm_mode != 0) p[i] = o;
        if (c != nullptr) c[0] = o;
        continue;
      }
      float v = to_float(p[i + other]) * r;
      if (a.norm_mode != 0) v *= to_float(w[wi + other]);
      const float cs = cos_t[static_cast<size_t>(pos) * a.rot_pairs + pair];
      const float sn = sin_t[static_cast<size_t>(pos) * a.rot_pairs + pair];
      const TA o0 = from_float<TA>(u * cs - v * sn), o1 = from_float<TA>(v * cs + u * sn);
      p[i] = o0;
      p[i + other] = o1;
      if (c != nullptr) {
        c[0] = o0;
        c[other] = o1;
      }
    }
  }
  if (a.vmix_mode != 0 || slot >= 0) {
    TA* v = row + a.v_col;
    TA* f = v_first != nullptr ? v_first + static_cast<size_t>(t) * a.v_size : nullptr;
    const int vdim = a.v_size / max(a.v_heads, 1);
    for (int i = threadIdx.x; i < a.v_size; i += blockDim.x) {
      TA o = v[i];
      if (a.vmix_mode == 1) f[i] = o;
      else if (a.vmix_mode == 2) {
        o = from_float<TA>((1.f - a.lam) * to_float(o) + a.lam * to_float(f[i]));
        v[i] = o;
      }
      if (slot >= 0) {
        const int h = i / vdim, d = i - h * vdim;
        v_cache[((page * a.v_heads + h) * a.page_size + off) * vdim + d] = o;
      }
    }
  }
}

}  // namespace rl


using namespace rl;

extern "C" {

enum { RL_F32 = 0, RL_BF16 = 1 };

int rl_sandwich_norm(float* residual, const void* delta, int ld_delta, const void* post_w, const void* pre_w,
                     int w_dtype, void* out, int ld_out, int act_dtype, const int32_t* rows_idx, int rows, int hidden,
                     float eps, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  constexpr int EPT = 4;
  if (hidden <= EPT * 1024) {                      // the row fits the registers of one CTA
    const int th = min(1024, max(64, ((hidden + EPT - 1) / EPT + 31) / 32 * 32));
#define RL_REG_CASE(TA, TW)                                                                                       \
  launch_kernel(sandwich_norm_reg_kernel<TA, TW, EPT>, dim3(rows), dim3(th), 0, stream, residual,                \
                static_cast<const TA*>(delta), ld_delta, static_cast<const TW*>(post_w),                         \
                static_cast<const TW*>(pre_w), static_cast<TA*>(out), ld_out, rows_idx, hidden, eps, kind)
    if (act_dtype == RL_F32) RL_REG_CASE(float, float);
    else if (w_dtype == RL_F32) RL_REG_CASE(bf16, float);
    else RL_REG_CASE(bf16, bf16);
#undef RL_REG_CASE
    RL_LAUNCH_END();
  }
  const int th = hidden >= 2048 ? 512 : 256;
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
#define RL_CASE(TA, TW)                                                                                          \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(sandwich_norm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_kernel(sandwich_norm_kernel<TA, TW>, dim3(rows), dim3(th), smem, stream, residual,                    \
                  static_cast<const TA*>(delta), ld_delta, static_cast<const TW*>(post_w),                       \
                  static_cast<const TW*>(pre_w), static_cast<TA*>(out), ld_out, rows_idx, hidden, eps, kind);    \
  } while (0)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_bias_act(void* x, int act_dtype, int ld, const float* bias, int rows, int cols, int mode, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const int th = 256;
  const int vec = act_dtype == RL_F32 ? 4 : 8;
  const int vec_ok = (cols % vec == 0 && ld % vec == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) ? 1 : 0;
  const int per_thread = vec_ok ? vec : 1;
  dim3 grid(min((cols + th * per_thread - 1) / (th * per_thread), 64), rows);
  if (act_dtype == RL_F32)
    launch_kernel(bias_act_kernel<float>, grid, dim3(th), 0, stream, static_cast<float*>(x), ld, bias, cols, mode, vec_ok);
  else
    launch_kernel(bias_act_kernel<bf16>, grid, dim3(th), 0, stream, static_cast<bf16*>(x), ld, bias, cols, mode, vec_ok);
  RL_LAUNCH_END();
}

int rl_cache_store(const void* src, int act_dtype, int ld, int col, int heads, int dim, const int32_t* slots,
                   void* cache, int page_size, long long num_slots, int tokens, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int th = heads * dim >= 256 ? 256 : 128;
  if (act_dtype == RL_F32)
    launch_kernel(cache_store_kernel<float>, dim3(tokens), dim3(th), 0, stream, static_cast<const float*>(src), ld,
                  col, heads, dim, slots, static_cast<float*>(cache), page_size, num_slots, status);
  else
    launch_kernel(cache_store_kernel<bf16>, dim3(tokens), dim3(th), 0, stream, static_cast<const bf16*>(src), ld,
                  col, heads, dim, slots, static_cast<bf16*>(cache), page_size, num_slots, status);
  RL_LAUNCH_END();
}

int rl_gated_rmsnorm(const float* o, const void* gate, int ld_gate, const void* w, int w_dtype, void* out,
                     int act_dtype, int rows, int n, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int th = 256;
#define RL_CASE(TA, TW)                                                                                        \
  launch_kernel(gated_rmsnorm_kernel<TA, TW>, dim3(rows), dim3(th), 0, stream, o, static_cast<const TA*>(gate), \
                ld_gate, static_cast<const TW*>(w), static_cast<TA*>(out), n, eps)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_gated_act(const void* gu, int ld, void* out, int act_dtype, int rows, int inter, int mode, float limit,
                 float slope, const float* bias, cudaStream_t stream) {
  if (rows <= 0 || inter <= 0) return 0;
  const int th = 256;
  dim3 grid(min((inter + th - 1) / th, 64), rows);
  if (act_dtype == RL_F32)
    launch_kernel(gated_act_kernel<float>, grid, dim3(th), 0, stream, static_cast<const float*>(gu), ld,
                  static_cast<float*>(out), inter, mode, limit, slope, bias);
  else
    launch_kernel(gated_act_kernel<bf16>, grid, dim3(th), 0, stream, static_cast<const bf16*>(gu), ld,
                  static_cast<bf16*>(out), inter, mode, limit, slope, bias);
  RL_LAUNCH_END();
}

int rl_head_prep(void* x, int act_dtype, int ld, const int32_t* positions, int tokens, int q_col, int q_heads,
                 int k_col, int k_heads, int dim, const void* q_w, const void* k_w, int w_dtype, int norm_mode,
                 float eps, const float* cos_t, const float* sin_t, int rot_pairs, int max_pos, int v_col,
                 int v_size, void* v_first, int vmix_mode, float lam, const int32_t* slots, void* k_cache,
                 void* v_cache, int v_heads, int page_size, long long num_slots, int* status, int rot_half,
                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  HeadPrepArgs a;
  a.rot_half = rot_half;
  a.ld = ld; a.q_col = q_col; a.q_heads = q_heads; a.k_col = k_col; a.k_heads = k_heads; a.dim = dim;
  a.norm_mode = norm_mode; a.eps = eps; a.rot_pairs = rot_pairs; a.max_pos = max_pos; a.v_col = v_col;
  a.v_size = v_size; a.vmix_mode = vmix_mode; a.lam = lam;
  a.slots = slots; a.v_heads = v_heads; a.page_size = page_size; a.num_slots = num_slots;
  const size_t pair = act_dtype == RL_F32 ? 8 : 4, wpair = (act_dtype == RL_F32 || w_dtype == RL_F32) ? 8 : 4;
  a.pairs_ok = !(rot_half && rot_pairs > 0) && dim % 2 == 0 && ld % 2 == 0 && q_col % 2 == 0 && k_col % 2 == 0 &&
               reinterpret_cast<uintptr_t>(x) % pair == 0 && reinterpret_cast<uintptr_t>(k_cache) % pair == 0 &&
               reinterpret_cast<uintptr_t>(q_w) % wpair == 0 && reinterpret_cast<uintptr_t>(k_w) % wpair == 0;
  const int widest = max(q_heads, k_heads) * dim;
  const int th = widest >= 1024 ? 512 : (widest >= 256 ? 256 : 128);
  const size_t smem = static_cast<size_t>(max(q_heads + k_heads, 1)) * sizeof(float);
#define RL_CASE(TA, TW)                                                                                          \
  launch_kernel(head_prep_kernel<TA, TW>, dim3(tokens), dim3(th), smem, stream, static_cast<TA*>(x), positions, \
                static_cast<const TW*>(q_w), static_cast<const TW*>(k_w), cos_t, sin_t,                          \
                static_cast<TA*>(v_first), static_cast<TA*>(k_cache), static_cast<TA*>(v_cache), status, a)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

}  // extern "C"