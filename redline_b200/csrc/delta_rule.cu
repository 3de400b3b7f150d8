// The gated delta rule: a matrix state per head that every token first decays row by row, then
// corrects towards its value along its key, then reads with its query:
//
//     S <- diag(a_t) S            a_t one decay per key channel (row of S)
//     d  = beta_t (v_t - S^T k_t)
//     S <- S + k_t d^T
//     o_t = S^T q_t                (the read-out sees the token's own write)
//
// S is [D, DV] per (request, head) in float32, in the request's state slot: zero for a new request,
// carried from step to step.  Columns of S never mix, so a CTA owns a few columns of one (sequence, head)
// and walks the sequence's tokens in order; within a warp 32 / G columns x G groups of rows (long sequences: G = 4,
// 8 from key size 64 and 16 from 128 on; steps of single tokens: G = 4): a thread keeps D / G neighbouring rows of its
// column in registers.  With R = diag(a_t) S the read-out is o_t = R^T q_t + d (k_t . q_t), so a thread sums its
// part of R^T k, R^T q and k . q in one pass over its rows and one shuffle reduction finishes all three.  q, k and the decays of a few tokens at a time are staged in shared memory by asynchronous
// copies into one of two buffers while the tokens of the other are worked on.  Everything here is float32:
// q and k arrive as unit vectors, beta and the decays as numbers in (0, 1) (delta_prep_kernel makes them
// from the projections); v is read in the activation type.
//
// delta_prep_kernel, one CTA per token: q and k heads (already convolved and activated) to unit vectors
// x / sqrt(sum x^2 + floor), q times a constant; beta = sigmoid(z_b); a = exp(-exp(A_log_h) softplus(z_a + dt_bias)).
// head_gated_norm_kernel, one warp per (token, head): o / sqrt(mean(o^2) + eps) * w * sigmoid(gate).
//
// RL_DELTA_DIM is the key size D (1..256), fixed when the file is compiled.
#include "common.cuh"

#ifndef RL_DELTA_DIM
#define RL_DELTA_DIM 64
#endif

namespace rl {

constexpr int kD = RL_DELTA_DIM;
// Row groups a column is split into: many where sequences are long (a token's work is a chain that more
// groups shorten), few where a step is mostly state traffic (single tokens: a warp then covers 8 neighbouring
// columns of every row it loads and stores).
constexpr int kGroupsLong = kD >= 128 ? 16 : (kD >= 64 ? 8 : 4);
constexpr int kGroupsShort = kD > 128 ? 8 : 4;
constexpr int kThreads = 128;
constexpr bool kVec = kD % 4 == 0;                 // rows of q, k and the decays start on 16-byte boundaries

__device__ __forceinline__ void async_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void async_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void async_copies_done() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// First token index t in [0, n) with seq_of_token[t] >= s (sequences lie in order in a step).
__device__ __forceinline__ int first_token_of(const int32_t* __restrict__ seq_of_token, int n, int s) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (seq_of_token[mid] < s) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

template <typename T>
struct DeltaArgs {
  const float* q;          // [tokens, qk_heads * D] unit vectors, scaled
  const float* k;          // [tokens, qk_heads * D] unit vectors
  const T* v;              // [tokens, ld_v]: head h's values at h * DV
  int ld_v;
  const float* beta;       // [tokens, heads]
  const float* decay;      // [tokens, heads * D]
  const int32_t* seq_of_token;
  const int32_t* state_slot;
  float* state;            // [slots] x [heads, D, DV]
  long long slot_stride;   // floats from one slot to the next
  float* out;              // [tokens, heads * DV]
  int tokens, heads, qk_heads, dv;
  int vec_ok;              // q, k and decay are 16-byte aligned
  int v_ok;                // pairs of values start on 4-byte boundaries
};

// Row r of a staged vector lies at (r / kRows) * kStride + r % kRows: a thread's rows are contiguous.
template <typename T, int kGroups>
__global__ void __launch_bounds__(kThreads)
delta_rule_kernel(const DeltaArgs<T> a) {
  constexpr int kRows = ((kD + kGroups - 1) / kGroups + 3) / 4 * 4;  // rows a thread keeps (a multiple of 4: float4 loads)
  constexpr int kDP = kRows * kGroups;               // D rounded up; the rows beyond D stay zero
  constexpr int kStride = kRows + 4;                 // floats from one group's rows to the next in shared memory (spreads the banks)
  constexpr int kSm = kGroups * kStride;             // floats of one staged vector
  constexpr int kWarpCols = 32 / kGroups;            // columns of a warp
  constexpr int kCols = 4 * kWarpCols;               // columns of a CTA (4 warps)
  constexpr int kTok = kD > 128 ? 4 : 8;             // tokens staged at a time (two such buffers)
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float qs[2][kTok][kSm];
  __shared__ __align__(16) float ks[2][kTok][kSm];
  __shared__ __align__(16) float as[2][kTok][kSm];
  __shared__ __align__(16) T vs[2][kTok][kCols];
  __shared__ float bs[2][kTok];
  const int seq = blockIdx.z, head = blockIdx.y;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = lane / kWarpCols;                            // rows group * kRows .. group * kRows + kRows - 1
  const int local_col = warp * kWarpCols + (lane % kWarpCols);
  const int col = blockIdx.x * kCols + local_col;
  const bool mine = col < a.dv;
  const int t0 = first_token_of(a.seq_of_token, a.tokens, seq);
  const int t1 = first_token_of(a.seq_of_token, a.tokens, seq + 1);
  if (t0 >= t1) return;
  float* plane = a.state + static_cast<size_t>(a.state_slot[seq]) * a.slot_stride +
                 static_cast<size_t>(head) * kD * a.dv;
  float S[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const int row = group * kRows + i;
    S[i] = (mine && row < kD) ? plane[static_cast<size_t>(row) * a.dv + col] : 0.f;
  }
  if (kDP > kD) {          // the rows beyond D: k = q = 0 and decay 1, never overwritten
    for (int i = threadIdx.x; i < 2 * kTok * kSm; i += kThreads) {
      (&qs[0][0][0])[i] = 0.f;
      (&ks[0][0][0])[i] = 0.f;
      (&as[0][0][0])[i] = 1.f;
    }
    __syncthreads();
  }
  const bool vec = kVec && a.vec_ok;
  // q, k and the decays of tokens tb .. tb + nt - 1 on their way into buffer b (asynchronous copies)
  auto stage = [&](int b, int tb, int nt) {
    if (vec) {
      constexpr int per = kD / 4;
      for (int i = threadIdx.x; i < nt * per; i += kThreads) {
        const int tt = i / per, e = (i - tt * per) * 4;
        const int sm = (e / kRows) * kStride + e % kRows;
        const size_t t = tb + tt;
        async_copy16(&qs[b][tt][sm], a.q + (t * a.qk_heads + qk_head) * kD + e);
        async_copy16(&ks[b][tt][sm], a.k + (t * a.qk_heads + qk_head) * kD + e);
        async_copy16(&as[b][tt][sm], a.decay + (t * a.heads + head) * kD + e);
      }
    } else {
      for (int i = threadIdx.x; i < nt * kD; i += kThreads) {
        const int tt = i / kD, e = i - tt * kD;
        const int sm = (e / kRows) * kStride + e % kRows;
        const size_t t = tb + tt;
        async_copy4(&qs[b][tt][sm], a.q + (t * a.qk_heads + qk_head) * kD + e);
        async_copy4(&ks[b][tt][sm], a.k + (t * a.qk_heads + qk_head) * kD + e);
        async_copy4(&as[b][tt][sm], a.decay + (t * a.heads + head) * kD + e);
      }
    }
    // the values of this CTA's columns (as they are, in the activation type) and the betas
    const int col0 = blockIdx.x * kCols;
    if (a.v_ok) {
      constexpr int per_word = 4 / sizeof(T), words = kCols / per_word;       // 4-byte words of a token's values
      for (int i = threadIdx.x; i < nt * words; i += kThreads) {
        const int tt = i / words, c = (i - tt * words) * per_word;
        if (col0 + c < a.dv)
          async_copy4(reinterpret_cast<float*>(&vs[b][tt][c]),
                      reinterpret_cast<const float*>(a.v + static_cast<size_t>(tb + tt) * a.ld_v + head * a.dv + col0 + c));
      }
    } else {
      for (int i = threadIdx.x; i < nt * kCols; i += kThreads) {
        const int tt = i / kCols, c = i - tt * kCols;
        if (col0 + c < a.dv) vs[b][tt][c] = a.v[static_cast<size_t>(tb + tt) * a.ld_v + head * a.dv + col0 + c];
      }
    }
    if (threadIdx.x < nt) async_copy4(&bs[b][threadIdx.x], a.beta + static_cast<size_t>(tb + threadIdx.x) * a.heads + head);
  };
  {
    const int nt = min(kTok, t1 - t0);
    stage(0, t0, nt);
    async_copies_done();
    __syncthreads();
  }
  int b = 0;
  for (int tb = t0; tb < t1; tb += kTok, b ^= 1) {
    const int nt = min(kTok, t1 - tb);
    const int nn = min(kTok, t1 - tb - kTok);        // tokens of the batch after this one
    if (nn > 0) stage(b ^ 1, tb + kTok, nn);
    auto token = [&](int tt) {
      // With R = diag(a) S:  d = beta (v - R^T k),  S = R + k d^T,  o = S^T q = R^T q + d (k . q): the three inner
      // products over the rows are summed in one pass and finished by one shuffle reduction.
      const float4* a4 = reinterpret_cast<const float4*>(&as[b][tt][group * kStride]);
      const float4* k4 = reinterpret_cast<const float4*>(&ks[b][tt][group * kStride]);
      const float4* q4 = reinterpret_cast<const float4*>(&qs[b][tt][group * kStride]);
      float kk[kRows];
      float rk0 = 0.f, rk1 = 0.f, rq0 = 0.f, rq1 = 0.f, kq0 = 0.f, kq1 = 0.f;     // two chains each
#pragma unroll
      for (int i = 0; i < kRows; i += 4) {
        const float4 av = a4[i >> 2], kv = k4[i >> 2], qv = q4[i >> 2];
        kk[i] = kv.x; kk[i + 1] = kv.y; kk[i + 2] = kv.z; kk[i + 3] = kv.w;
        S[i] *= av.x;     rk0 = fmaf(S[i], kv.x, rk0);     rq0 = fmaf(S[i], qv.x, rq0);     kq0 = fmaf(kv.x, qv.x, kq0);
        S[i + 1] *= av.y; rk1 = fmaf(S[i + 1], kv.y, rk1); rq1 = fmaf(S[i + 1], qv.y, rq1); kq1 = fmaf(kv.y, qv.y, kq1);
        S[i + 2] *= av.z; rk0 = fmaf(S[i + 2], kv.z, rk0); rq0 = fmaf(S[i + 2], qv.z, rq0); kq0 = fmaf(kv.z, qv.z, kq0);
        S[i + 3] *= av.w; rk1 = fmaf(S[i + 3], kv.w, rk1); rq1 = fmaf(S[i + 3], qv.w, rq1); kq1 = fmaf(kv.w, qv.w, kq1);
      }
      float rk = rk0 + rk1, rq = rq0 + rq1, kq = kq0 + kq1;
#pragma unroll
      for (int off = kWarpCols; off < 32; off <<= 1) {
        rk += __shfl_xor_sync(0xffffffffu, rk, off);
        rq += __shfl_xor_sync(0xffffffffu, rq, off);
        kq += __shfl_xor_sync(0xffffffffu, kq, off);
      }
      const float d = bs[b][tt] * (to_float(vs[b][tt][local_col]) - rk);
#pragma unroll
      for (int i = 0; i < kRows; ++i) S[i] = fmaf(kk[i], d, S[i]);
      if (mine && group == 0) a.out[(static_cast<size_t>(tb + tt) * a.heads + head) * a.dv + col] = fmaf(d, kq, rq);
    };
    if (nt == kTok) {          // a full batch, unrolled: the next token's loads are asked for while this one's sums are finished
#pragma unroll
      for (int tt = 0; tt < kTok; ++tt) token(tt);
    } else {
      for (int tt = 0; tt < nt; ++tt) token(tt);
    }
    async_copies_done();
    __syncthreads();
  }
  if (mine) {
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int row = group * kRows + i;
      if (row < kD) plane[static_cast<size_t>(row) * a.dv + col] = S[i];
    }
  }
}

// ------------------------------------------------------------------ what the recurrence is fed
template <typename T>
struct PrepArgs {
  const T* x;              // [tokens, ld]: q heads at q_col, k heads at k_col (convolved, activated)
  int ld, q_col, k_col, qk_heads, heads;
  float q_scale, unit_floor;
  const float* zb;         // [tokens, heads]       projection for beta
  const float* za;         // [tokens, heads * D]   projection for the decays
  const float* dt_bias;    // [heads * D]
  const float* a_log;      // [heads]
  float* q;                // [tokens, qk_heads * D]
  float* k;
  float* beta;             // [tokens, heads]
  float* decay;            // [tokens, heads * D]
};

template <typename T>
__global__ void delta_prep_kernel(const PrepArgs<T> a) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = a.x + static_cast<size_t>(t) * a.ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < 2 * a.qk_heads; h += nwarps) {       // a warp per head: first the q heads, then the k heads
    const bool is_q = h < a.qk_heads;
    const int hh = is_q ? h : h - a.qk_heads;
    const T* p = row + (is_q ? a.q_col : a.k_col) + hh * kD;
    float ss = 0.f;
    for (int d = lane; d < kD; d += 32) {
      const float v = to_float(p[d]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + a.unit_floor) * (is_q ? a.q_scale : 1.f);
    float* o = (is_q ? a.q : a.k) + (static_cast<size_t>(t) * a.qk_heads + hh) * kD;
    for (int d = lane; d < kD; d += 32) o[d] = to_float(p[d]) * r;
  }
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x)
    a.beta[static_cast<size_t>(t) * a.heads + h] = 1.f / (1.f + expf(-a.zb[static_cast<size_t>(t) * a.heads + h]));
  const int n = a.heads * kD;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float z = a.za[static_cast<size_t>(t) * n + i] + a.dt_bias[i];
    const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
    a.decay[static_cast<size_t>(t) * n + i] = expf(-expf(a.a_log[i / kD]) * sp);
  }
}

// ------------------------------------------------------------------ per-head norm, weight and gate
template <typename T, typename TW>
__global__ void head_gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ld_gate,
                                       const TW* __restrict__ w, int w_per_head, T* __restrict__ out, int ld_out,
                                       int tokens, int heads, int dv, float eps) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= tokens * heads) return;
  const int t = item / heads, h = item - t * heads;
  const float* p = o + (static_cast<size_t>(t) * heads + h) * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss = fmaf(p[d], p[d], ss);
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / static_cast<float>(dv) + eps);
  for (int d = lane; d < dv; d += 32) {
    float y = p[d] * r * to_float(w[w_per_head ? h * dv + d : d]);
    if (gate != nullptr) y *= 1.f / (1.f + expf(-to_float(gate[static_cast<size_t>(t) * ld_gate + h * dv + d])));
    out[static_cast<size_t>(t) * ld_out + h * dv + d] = from_float<T>(y);
  }
}

}  // namespace rl

using namespace rl;

extern "C" {

enum { RL_F32 = 0, RL_BF16 = 1 };

int rl_delta_dim() { return kD; }

int rl_delta_prep(int act_dtype, const void* x, int ld, int q_col, int k_col, int qk_heads, int heads, float q_scale,
                  float unit_floor, const float* zb, const float* za, const float* dt_bias, const float* a_log,
                  float* q, float* k, float* beta, float* decay, int tokens, cudaStream_t stream) {
  if (tokens <= 0) return 0;
#define RL_CASE(T)                                                                                               \
  do {                                                                                                           \
    PrepArgs<T> a;                                                                                               \
    a.x = static_cast<const T*>(x); a.ld = ld; a.q_col = q_col; a.k_col = k_col; a.qk_heads = qk_heads;          \
    a.heads = heads; a.q_scale = q_scale; a.unit_floor = unit_floor; a.zb = zb; a.za = za; a.dt_bias = dt_bias;  \
    a.a_log = a_log; a.q = q; a.k = k; a.beta = beta; a.decay = decay;                                           \
    launch_kernel(delta_prep_kernel<T>, dim3(tokens), dim3(256), 0, stream, a);                                  \
  } while (0)
  if (act_dtype == RL_F32) RL_CASE(float);
  else RL_CASE(bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_delta_rule(int act_dtype, const float* q, const float* k, const void* v, int ld_v, const float* beta,
                  const float* decay, const int32_t* seq_of_token, const int32_t* state_slot, float* state,
                  long long slot_stride, float* out, int tokens, int sequences, int heads, int qk_heads, int dv,
                  cudaStream_t stream) {
  if (tokens <= 0 || sequences <= 0) return 0;
  // long sequences: many row groups, and a launch that waits for an empty machine (few CTAs that run long: begun
  // while the kernel before drains, they would share a few SMs); steps of (mostly) single tokens: few row groups
  const bool long_seqs = tokens >= 16 * sequences;
  const int cols = 4 * (32 / (long_seqs ? kGroupsLong : kGroupsShort));
  const dim3 grid((dv + cols - 1) / cols, heads, sequences);
#define RL_CASE(T)                                                                                               \
  do {                                                                                                           \
    DeltaArgs<T> a;                                                                                              \
    a.q = q; a.k = k; a.v = static_cast<const T*>(v); a.ld_v = ld_v; a.beta = beta; a.decay = decay;             \
    a.seq_of_token = seq_of_token; a.state_slot = state_slot; a.state = state; a.slot_stride = slot_stride;      \
    a.out = out; a.tokens = tokens; a.heads = heads; a.qk_heads = qk_heads; a.dv = dv;                           \
    a.vec_ok = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |                               \
                 reinterpret_cast<uintptr_t>(decay)) & 15) == 0;                                                 \
    a.v_ok = sizeof(T) == 4 || ((reinterpret_cast<uintptr_t>(v) & 3) == 0 && ld_v % 2 == 0 && dv % 2 == 0);     \
    if (long_seqs) launch_kernel_serial(delta_rule_kernel<T, kGroupsLong>, grid, dim3(kThreads), 0, stream, a);  \
    else launch_kernel(delta_rule_kernel<T, kGroupsShort>, grid, dim3(kThreads), 0, stream, a);                                          \
  } while (0)
  if (act_dtype == RL_F32) RL_CASE(float);
  else RL_CASE(bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_head_gated_norm(int act_dtype, const float* o, const void* gate, int ld_gate, const void* w, int w_dtype,
                       int w_per_head, void* out, int ld_out, int tokens, int heads, int dv, float eps,
                       cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int warps = 8;
  const dim3 grid((tokens * heads + warps - 1) / warps);
#define RL_CASE(T, TW)                                                                                          \
  launch_kernel(head_gated_norm_kernel<T, TW>, grid, dim3(warps * 32), 0, stream, o, static_cast<const T*>(gate), \
                ld_gate, static_cast<const TW*>(w), w_per_head, static_cast<T*>(out), ld_out, tokens, heads, dv, eps)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

}  // extern "C"
