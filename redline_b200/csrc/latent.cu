// Attention over a cached latent: what lies between the projections and the attention kernel, and the
// per-head products around it.
//
// A token's projection row holds, per head, a query [n | r] (n unrotated entries, r rotated ones) and, behind
// the queries, [c' | k_r]: the raw latent of `rank` entries and one rotated key part of r entries that all
// heads share.  Keys and values of head h are W_uk,h c and W_uv,h c with c = c' / rms(c') * w, so
//     q_n . (W_uk,h c) = (W_uk,h^T q_n) . c      and      sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j):
// attention runs over the cached rows [c | k_r] themselves, one key head for all query heads, with the query
// [W_uk,h^T q_n | q_r] and the row's first `rank` entries as the value; W_uv,h is applied to its result.
//
//   latent_prep   per token: c (RMS norm in float32, weight w), k_r and every head's q_r turned by the
//                 token's position (entry i with entry i + dims/2 of the first `dims` rotated entries, cos
//                 and sin from tables), [c | k_r] into the paged cache, q_r into the attention's query rows
//   head_linear   y[t, h, :] = W_h x[t, h, :] for every head h, W [heads, n, k], float32 sums in ascending k
//                 (a row's result does not depend on what else is in the launch); FFMA for float32, and
//                 mma.sync.m16n8k16 for bfloat16 operands whose sizes allow it
#include "common.cuh"

namespace rl {

struct LatentPrepArgs {
  int ld;            // row length of the projection buffer
  int heads, dn, dr, rank, rot_dims;
  int q_ld;          // row length of the attention's query buffer: heads * (rank + dr)
  float eps;
  int page_size;
  long long num_slots;
  int max_pos;       // rows of the tables
};

// One CTA per token.  A position beyond the tables sets bit 1 of *status, a slot beyond the pool bit 2
// (negative slot: no write).
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const TA* __restrict__ proj, const int32_t* __restrict__ positions, const TW* __restrict__ w,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, TA* __restrict__ qa,
                   const int32_t* __restrict__ slots, TA* __restrict__ cache, int* status, const LatentPrepArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int qsize = a.heads * (a.dn + a.dr);
  const TA* row = proj + static_cast<size_t>(t) * a.ld;
  const TA* craw = row + qsize;
  const int half = a.rot_dims / 2;
  int pos = positions[t];
  if (a.dr > 0 && (pos < 0 || pos >= a.max_pos)) {
    if (threadIdx.x == 0) atomicOr(status, 2);
    pos = 0;
  }
  const float* cs = cos_t + static_cast<size_t>(pos) * half;
  const float* sn = sin_t + static_cast<size_t>(pos) * half;
  // ---- the heads' rotated query parts
  TA* qrow = qa + static_cast<size_t>(t) * a.q_ld;
  for (int i = threadIdx.x; i < a.heads * a.dr; i += blockDim.x) {
    const int h = i / a.dr, d = i - h * a.dr;
    const TA* src = row + h * (a.dn + a.dr) + a.dn;
    float v = to_float(src[d]);
    if (d < half) v = v * cs[d] - to_float(src[d + half]) * sn[d];
    else if (d < a.rot_dims) v = v * cs[d - half] + to_float(src[d - half]) * sn[d - half];
    qrow[h * (a.rank + a.dr) + a.rank + d] = from_float<TA>(v);
  }
  // ---- the latent and the shared key part into the cache
  float q = 0.f;
  for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
    const float v = to_float(craw[i]);
    q += v * v;
  }
  const float r = rsqrtf(block_sum(q, scratch) / static_cast<float>(a.rank) + a.eps);
  const int slot = slots != nullptr ? slots[t] : -1;
  if (slot < 0) return;
  if (slot >= a.num_slots) {
    if (threadIdx.x == 0) atomicOr(status, 4);
    return;
  }
  TA* dst = cache + static_cast<size_t>(slot) * (a.rank + a.dr);     // one key head: [pages, 1, page, rank + dr]
  for (int i = threadIdx.x; i < a.rank; i += blockDim.x) dst[i] = from_float<TA>(to_float(craw[i]) * r * to_float(w[i]));
  for (int d = threadIdx.x; d < a.dr; d += blockDim.x) {
    const TA* src = craw + a.rank;
    float v = to_float(src[d]);
    if (d < half) v = v * cs[d] - to_float(src[d + half]) * sn[d];
    else if (d < a.rot_dims) v = v * cs[d - half] + to_float(src[d - half]) * sn[d - half];
    dst[a.rank + d] = from_float<TA>(v);
  }
}

// ------------------------------------------------------------------ per-head products
// y[t, y_col + h * y_head + j] = sum_k W[h, j, k] x[t, x_col + h * x_head + k]
struct HeadLinearArgs {
  int tokens, heads, n, k;
  int x_ld, x_col, x_head;
  int y_ld, y_col, y_head;
};

constexpr int kHlRows = 16, kHlCols = 128, kHlK = 32;

// CUDA cores: a CTA takes 16 tokens x 128 outputs of one head; thread j owns output column j for all 16 tokens.
template <typename TA, typename TW>
__global__ void __launch_bounds__(kHlCols)
head_linear_kernel(const TA* __restrict__ x, const TW* __restrict__ w, TA* __restrict__ y, const HeadLinearArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ float xs[kHlRows][kHlK];
  __shared__ float wsm[kHlK][kHlCols + 1];
  const int t0 = blockIdx.x * kHlRows, j0 = blockIdx.y * kHlCols, h = blockIdx.z;
  const int j = j0 + threadIdx.x;
  const TW* wh = w + static_cast<size_t>(h) * a.n * a.k;
  float acc[kHlRows];
#pragma unroll
  for (int r = 0; r < kHlRows; ++r) acc[r] = 0.f;
  for (int k0 = 0; k0 < a.k; k0 += kHlK) {
    __syncthreads();
    for (int i = threadIdx.x; i < kHlRows * kHlK; i += kHlCols) {
      const int r = i / kHlK, kk = i - r * kHlK;
      xs[r][kk] = (t0 + r < a.tokens && k0 + kk < a.k)
                      ? to_float(x[static_cast<size_t>(t0 + r) * a.x_ld + a.x_col + h * a.x_head + k0 + kk])
                      : 0.f;
    }
    for (int i = threadIdx.x; i < kHlCols * kHlK; i += kHlCols) {
      const int c = i / kHlK, kk = i - c * kHlK;
      wsm[kk][c] = (j0 + c < a.n && k0 + kk < a.k) ? to_float(wh[static_cast<size_t>(j0 + c) * a.k + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kHlK; ++kk) {
      const float wv = wsm[kk][threadIdx.x];
#pragma unroll
      for (int r = 0; r < kHlRows; ++r) acc[r] = fmaf(xs[r][kk], wv, acc[r]);
    }
  }
  if (j < a.n) {
#pragma unroll
    for (int r = 0; r < kHlRows; ++r)
      if (t0 + r < a.tokens)
        y[static_cast<size_t>(t0 + r) * a.y_ld + a.y_col + h * a.y_head + j] = from_float<TA>(acc[r]);
  }
}

// Tensor cores for bfloat16: a CTA of four warps takes 64 tokens x 64 outputs of one head, a warp 16 tokens;
// A fragments (x) and B fragments (W rows are the MMA's columns: W is [n, k] row-major, which is the "col"
// operand) come straight from global memory; k ascending in steps of 16.  Needs k % 16 == 0, n % 8 == 0 and
// even strides and columns (4-byte loads and stores).
__device__ __forceinline__ void hl_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kHmRows = 64, kHmCols = 64;

__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                       const HeadLinearArgs a) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int t0 = blockIdx.x * kHmRows + warp * 16, j0 = blockIdx.y * kHmCols, h = blockIdx.z;
  if (t0 >= a.tokens) return;
  const int r0 = t0 + gid, r1 = r0 + 8;
  const bool ok0 = r0 < a.tokens, ok1 = r1 < a.tokens;
  const bf16* x0 = x + static_cast<size_t>(ok0 ? r0 : t0) * a.x_ld + a.x_col + h * a.x_head + tig * 2;
  const bf16* x1 = x + static_cast<size_t>(ok1 ? r1 : t0) * a.x_ld + a.x_col + h * a.x_head + tig * 2;
  const bf16* wh = w + static_cast<size_t>(h) * a.n * a.k;
  float acc[kHmCols / 8][4];
#pragma unroll
  for (int nt = 0; nt < kHmCols / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll 4
  for (int k0 = 0; k0 < a.k; k0 += 16) {
    uint32_t af[4];
    af[0] = *reinterpret_cast<const uint32_t*>(x0 + k0);
    af[1] = *reinterpret_cast<const uint32_t*>(x1 + k0);
    af[2] = *reinterpret_cast<const uint32_t*>(x0 + k0 + 8);
    af[3] = *reinterpret_cast<const uint32_t*>(x1 + k0 + 8);
#pragma unroll
    for (int nt = 0; nt < kHmCols / 8; ++nt) {
      const int j = j0 + nt * 8 + gid;
      if (j0 + nt * 8 < a.n) {               // (n is a multiple of 8: a group of 8 columns is in or out as a whole)
        const bf16* wr = wh + static_cast<size_t>(j) * a.k + k0 + tig * 2;
        hl_mma(acc[nt], af, *reinterpret_cast<const uint32_t*>(wr), *reinterpret_cast<const uint32_t*>(wr + 8));
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < kHmCols / 8; ++nt) {
    const int j = j0 + nt * 8 + tig * 2;
    if (j0 + nt * 8 >= a.n) continue;
    if (ok0)
      *reinterpret_cast<__nv_bfloat162*>(y + static_cast<size_t>(r0) * a.y_ld + a.y_col + h * a.y_head + j) =
          __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
    if (ok1)
      *reinterpret_cast<__nv_bfloat162*>(y + static_cast<size_t>(r1) * a.y_ld + a.y_col + h * a.y_head + j) =
          __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
  }
}

}  // namespace rl

using namespace rl;

extern "C" {

int rl_latent_prep(int act_dtype, int w_dtype, const void* proj, int ld, const int32_t* positions, int tokens, int heads,
                   int dn, int dr, int rank, int rot_dims, const void* w, float eps, const float* cos_t,
                   const float* sin_t, int max_pos, void* qa, int q_ld, const int32_t* slots, void* cache, int page_size,
                   long long num_slots, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  LatentPrepArgs a;
  a.ld = ld;
  a.heads = heads;
  a.dn = dn;
  a.dr = dr;
  a.rank = rank;
  a.rot_dims = rot_dims;
  a.q_ld = q_ld;
  a.eps = eps;
  a.page_size = page_size;
  a.num_slots = num_slots;
  a.max_pos = max_pos;
#define RL_CASE(TA, TW)                                                                                          \
  launch_kernel(latent_prep_kernel<TA, TW>, dim3(tokens), dim3(128), 0, stream, static_cast<const TA*>(proj),    \
                positions, static_cast<const TW*>(w), cos_t, sin_t, static_cast<TA*>(qa), slots,                  \
                static_cast<TA*>(cache), status, a)
  if (act_dtype == 0) RL_CASE(float, float);
  else if (w_dtype == 0) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

// impl 0: the tensor cores where they apply; 1: CUDA cores.
int rl_head_linear(int act_dtype, int w_dtype, const void* x, int x_ld, int x_col, int x_head, const void* w, int heads,
                   int n, int k, void* y, int y_ld, int y_col, int y_head, int tokens, int impl, cudaStream_t stream) {
  if (tokens <= 0 || heads <= 0 || n <= 0) return 0;
  HeadLinearArgs a;
  a.tokens = tokens;
  a.heads = heads;
  a.n = n;
  a.k = k;
  a.x_ld = x_ld;
  a.x_col = x_col;
  a.x_head = x_head;
  a.y_ld = y_ld;
  a.y_col = y_col;
  a.y_head = y_head;
  const bool even = ((x_ld | x_col | x_head | y_ld | y_col | y_head) & 1) == 0 &&
                    reinterpret_cast<uintptr_t>(x) % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(w) % 4 == 0;
  if (act_dtype == 1 && w_dtype == 1 && impl == 0 && k % 16 == 0 && n % 8 == 0 && even) {
    launch_kernel(head_linear_mma_kernel, dim3((tokens + kHmRows - 1) / kHmRows, (n + kHmCols - 1) / kHmCols, heads),
                  dim3(128), 0, stream, static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<bf16*>(y), a);
    RL_LAUNCH_END();
  }
  dim3 grid((tokens + kHlRows - 1) / kHlRows, (n + kHlCols - 1) / kHlCols, heads);
#define RL_CASE(TA, TW)                                                                                       \
  launch_kernel(head_linear_kernel<TA, TW>, grid, dim3(kHlCols), 0, stream, static_cast<const TA*>(x),        \
                static_cast<const TW*>(w), static_cast<TA*>(y), a)
  if (act_dtype == 0) RL_CASE(float, float);
  else if (w_dtype == 0) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

}  // extern "C"
