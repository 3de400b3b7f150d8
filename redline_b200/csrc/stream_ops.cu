// Kernels around several residual streams (hyper-connections), the normed mean of two sublayer outputs,
// and the short causal convolution over time that some mixers put behind their projections.
//
// streams_step_kernel, one CTA per token, everything float32 but the sublayer's output y and the normed
// row handed to the next sublayer (activation type).  With n streams X_1 .. X_n of a token:
//   init given:     X_s <- init for every s (the embedding's row; the model's first sublayer)
//   y given:        X_t <- sum_s mix[s, t] X_s + out[t] * y   for all t from the old streams
//   read_in given:  u = sum_s read_in[s] X_s;  normed = u / sqrt(mean(u^2) + eps) * norm_w   (the next sublayer's input)
//   total given:    total = sum_s X_s   (what the model's final norm reads)
// The row u lives in dynamic shared memory (width floats).
//
// pair_norm_mean_kernel, one CTA per token: out = ca * N(a + bias_a, wa) + cb * N(b + bias_b, wb), N the RMS
// norm, the biases (float32, of the two products that made a and b) optional.
//
// short_conv_kernel, one thread per channel and token (eight tokens in a large step): y_t = act(sum_j w[c, j] (u_(t - taps + 1 + j) + bias_c)),
// over the tokens of the token's own sequence; tokens before the step's portion come from the request's state
// slot, which holds the last taps - 1 inputs (bias added) in float32: [taps - 1, channels], the oldest first,
// zeros for a new request.  short_conv_state_kernel then moves the slot on: the thread of a sequence's last
// token gathers the channel's last taps - 1 inputs (from the step, or from the old slot where the portion
// is shorter) and writes them back.  The two are separate launches because the first tokens of a portion
// read what the last one replaces; in a step where every sequence has one token the first kernel moves the
// slot on itself.
#include "common.cuh"

namespace rl {

constexpr int kMaxStreams = 8;
constexpr int kMaxTaps = 8;

enum { ACT_NONE = 0, ACT_SILU = 3 };

struct StreamsArgs {
  float* streams;          // [tokens, n, width]
  const float* init;       // [tokens, width] or null
  const float* mix;        // [n, n] (from, to) or null with y
  const float* out_w;      // [n]
  const float* read_in;    // [n] or null
  float* total;            // [tokens, width] or null
  int n, width, ld_y, ld_normed;
  float eps;
};

template <typename TA, typename TW>
__global__ void streams_step_kernel(const StreamsArgs a, const TA* __restrict__ y, const TW* __restrict__ norm_w,
                                    TA* __restrict__ normed) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float u_row[];
  __shared__ float red[32];
  __shared__ float coef[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  const int n = a.n;
  float* mix = coef;
  float* out_w = coef + kMaxStreams * kMaxStreams;
  float* read_in = out_w + kMaxStreams;
  if (threadIdx.x < n * n && y != nullptr) mix[threadIdx.x] = a.mix[threadIdx.x];
  if (threadIdx.x < n) {
    out_w[threadIdx.x] = y != nullptr ? a.out_w[threadIdx.x] : 0.f;
    read_in[threadIdx.x] = a.read_in != nullptr ? a.read_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const size_t t = blockIdx.x;
  float* X = a.streams + t * n * a.width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < a.width; c += blockDim.x) {
    float x[kMaxStreams];
    if (a.init != nullptr) {
      const float e = a.init[t * a.width + c];
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) x[s] = e;
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) x[s] = s < n ? X[static_cast<size_t>(s) * a.width + c] : 0.f;
    }
    if (y != nullptr) {
      const float yv = to_float(y[t * a.ld_y + c]);
      float nx[kMaxStreams];
#pragma unroll
      for (int to = 0; to < kMaxStreams; ++to) {
        float acc = 0.f;
        if (to < n) {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) acc = fmaf(mix[s * n + to], x[s], acc);
          acc = fmaf(out_w[to], yv, acc);
        }
        nx[to] = acc;
      }
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) x[s] = nx[s];
    }
    if (y != nullptr || a.init != nullptr) {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < n) X[static_cast<size_t>(s) * a.width + c] = x[s];
    }
    if (a.total != nullptr) {
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < n) sum += x[s];
      a.total[t * a.width + c] = sum;
    }
    if (a.read_in != nullptr) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < n) u = fmaf(read_in[s], x[s], u);
      u_row[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (a.read_in == nullptr) return;
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / static_cast<float>(a.width) + a.eps);
  for (int c = threadIdx.x; c < a.width; c += blockDim.x)       // (a thread reads back what it wrote itself)
    normed[t * a.ld_normed + c] = from_float<TA>(u_row[c] * r * to_float(norm_w[c]));
}

template <typename TA, typename TW>
__global__ void pair_norm_mean_kernel(const TA* __restrict__ a, int ld_a, const TW* __restrict__ wa, float ca,
                                      const TA* __restrict__ b, int ld_b, const TW* __restrict__ wb, float cb,
                                      TA* __restrict__ out, int ld_out, int width, float eps,
                                      const float* __restrict__ bias_a, const float* __restrict__ bias_b) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const size_t t = blockIdx.x;
  const TA* pa = a + t * ld_a;
  const TA* pb = b + t * ld_b;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_float(pa[c]) + (bias_a != nullptr ? bias_a[c] : 0.f);
    const float z = to_float(pb[c]) + (bias_b != nullptr ? bias_b[c] : 0.f);
    sa = fmaf(x, x, sa);
    sb = fmaf(z, z, sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ra = ca * rsqrtf(sa / static_cast<float>(width) + eps);
  const float rb = cb * rsqrtf(sb / static_cast<float>(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_float(pa[c]) + (bias_a != nullptr ? bias_a[c] : 0.f);
    const float z = to_float(pb[c]) + (bias_b != nullptr ? bias_b[c] : 0.f);
    out[t * ld_out + c] = from_float<TA>(x * ra * to_float(wa[c]) + z * rb * to_float(wb[c]));
  }
}

struct ConvArgs {
  int ld_x, col_x, ld_y, col_y, channels, taps, act, tokens;
  int tile;                      // consecutive tokens a thread of short_conv_kernel walks
  int own_state;                 // every sequence has one token in this step: the thread of the token moves the slot on itself
  const float* bias;             // [channels] or null
  const int32_t* seq_of_token;
  const int32_t* state_slot;
  float* state;                  // [slots] x [taps - 1, channels]
  long long slot_stride;
};

constexpr int kConvTile = 8;         // tokens a thread of short_conv_kernel walks in a step of many tokens (one in a small step)
constexpr int kStateTile = 32;       // tokens a thread of short_conv_state_kernel looks at

// Input u_s of channel c for the token at index s of the step, or, where s lies before the first token of
// the sequence in this step (index `first`), what the sequence's slot holds for it.
template <typename TA>
__device__ __forceinline__ float conv_input(const ConvArgs& a, const TA* __restrict__ x, const float* st, int s,
                                            int first, int c, float bias) {
  if (s >= first) return to_float(x[static_cast<size_t>(s) * a.ld_x + a.col_x + c]) + bias;
  return st[static_cast<size_t>(a.taps - 1 + (s - first)) * a.channels + c];
}

// Index of the first token of token t's sequence in this step, looking back at most `reach` tokens
// (t - reach if the sequence began earlier: nothing before that is asked for).
__device__ __forceinline__ int conv_first(const int32_t* __restrict__ seq_of_token, int t, int seq, int reach) {
  int first = t;
  while (first > 0 && t - first < reach && seq_of_token[first - 1] == seq) --first;
  return first;
}

// One thread per channel and a.tile consecutive tokens: the window of the last taps - 1 inputs slides in
// registers from token to token and is gathered anew where another sequence begins.
template <typename TA, typename TW>
__global__ void short_conv_kernel(const ConvArgs a, const TA* __restrict__ x, const TW* __restrict__ w,
                                  TA* __restrict__ y) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int t_begin = blockIdx.y * a.tile, t_end = min(t_begin + a.tile, a.tokens);
  const float bias = a.bias != nullptr ? a.bias[c] : 0.f;
  const int keep = a.taps - 1;
  float wt[kMaxTaps], win[kMaxTaps];     // win[j]: the input j + 1 tokens back, wt[j] its weight
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) {
    wt[j] = j < keep ? to_float(w[static_cast<size_t>(c) * a.taps + (keep - 1 - j)]) : 0.f;
    win[j] = 0.f;
  }
  const float w_now = to_float(w[static_cast<size_t>(c) * a.taps + keep]);
  int seq = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int sq = a.seq_of_token[t];
    if (sq != seq) {                     // the tile's first token, or another sequence begins: gather the window
      seq = sq;
      const int first = conv_first(a.seq_of_token, t, seq, keep);
      const float* st = a.state + static_cast<size_t>(a.state_slot[seq]) * a.slot_stride;
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j)
        if (j < keep) win[j] = conv_input(a, x, st, t - 1 - j, first, c, bias);
    }
    const float u = to_float(x[static_cast<size_t>(t) * a.ld_x + a.col_x + c]) + bias;
    float acc = 0.f;
#pragma unroll
    for (int j = kMaxTaps - 1; j >= 0; --j)                  // the oldest input first, as a sum over the taps in order
      if (j < keep) acc = fmaf(wt[j], win[j], acc);
    acc = fmaf(w_now, u, acc);
#pragma unroll
    for (int j = kMaxTaps - 1; j > 0; --j) win[j] = win[j - 1];
    win[0] = u;
    if (a.own_state) {                   // nobody else reads this sequence's slot in this step
      float* st = a.state + static_cast<size_t>(a.state_slot[seq]) * a.slot_stride;
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j)
        if (j < keep) st[static_cast<size_t>(keep - 1 - j) * a.channels + c] = win[j];
      seq = -1;                          // (the next token gathers its own window)
    }
    if (a.act == ACT_SILU) acc = acc / (1.f + expf(-acc));
    y[static_cast<size_t>(t) * a.ld_y + a.col_y + c] = from_float<TA>(acc);
  }
}

// Moves the slots on: the thread that meets a sequence's last token of the step gathers the channel's last
// taps - 1 inputs (from the step, or from the old slot where the portion is shorter) and writes them back.
template <typename TA>
__global__ void short_conv_state_kernel(const ConvArgs a, const TA* __restrict__ x) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int t_begin = blockIdx.y * kStateTile, t_end = min(t_begin + kStateTile, a.tokens);
  const float bias = a.bias != nullptr ? a.bias[c] : 0.f;
  const int keep = a.taps - 1;
  for (int t = t_begin; t < t_end; ++t) {
    const int seq = a.seq_of_token[t];
    if (t + 1 < a.tokens && a.seq_of_token[t + 1] == seq) continue;    // not the sequence's last token of the step
    float* st = a.state + static_cast<size_t>(a.state_slot[seq]) * a.slot_stride;
    const int first = conv_first(a.seq_of_token, t, seq, keep);
    float u[kMaxTaps];
#pragma unroll
    for (int back = 0; back < kMaxTaps; ++back)
      if (back < keep) u[back] = conv_input(a, x, st, t - back, first, c, bias);
#pragma unroll
    for (int back = 0; back < kMaxTaps; ++back)
      if (back < keep) st[static_cast<size_t>(keep - 1 - back) * a.channels + c] = u[back];
  }
}

}  // namespace rl

using namespace rl;

extern "C" {

enum { RL_F32 = 0, RL_BF16 = 1 };

int rl_streams_max() { return kMaxStreams; }
int rl_conv_max_taps() { return kMaxTaps; }

int rl_streams_step(float* streams, const float* init, const void* y, int ld_y, const float* mix, const float* out_w,
                    const float* read_in, const void* norm_w, int w_dtype, void* normed, int ld_normed,
                    int act_dtype, float* total, int tokens, int n, int width, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n < 1 || n > kMaxStreams) return static_cast<int>(cudaErrorInvalidValue);
  StreamsArgs a;
  a.streams = streams; a.init = init; a.mix = mix; a.out_w = out_w; a.read_in = read_in; a.total = total;
  a.n = n; a.width = width; a.ld_y = ld_y; a.ld_normed = ld_normed; a.eps = eps;
  const int th = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = read_in != nullptr ? static_cast<size_t>(width) * sizeof(float) : 0;
#define RL_CASE(TA, TW)                                                                                          \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(streams_step_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_kernel(streams_step_kernel<TA, TW>, dim3(tokens), dim3(th), smem, stream, a,                          \
                  static_cast<const TA*>(y), static_cast<const TW*>(norm_w), static_cast<TA*>(normed));          \
  } while (0)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_pair_norm_mean(int act_dtype, const void* a, int ld_a, const void* wa, float ca, const void* b, int ld_b,
                      const void* wb, float cb, int w_dtype, void* out, int ld_out, int tokens, int width, float eps,
                      const float* bias_a, const float* bias_b, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int th = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define RL_CASE(TA, TW)                                                                                       \
  launch_kernel(pair_norm_mean_kernel<TA, TW>, dim3(tokens), dim3(th), 0, stream, static_cast<const TA*>(a),  \
                ld_a, static_cast<const TW*>(wa), ca, static_cast<const TA*>(b), ld_b,                        \
                static_cast<const TW*>(wb), cb, static_cast<TA*>(out), ld_out, width, eps, bias_a, bias_b)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

int rl_short_conv(int act_dtype, const void* x, int ld_x, int col_x, const void* w, int w_dtype, const float* bias,
                  void* y, int ld_y, int col_y, int channels, int taps, int act, const int32_t* seq_of_token,
                  const int32_t* state_slot, float* state, long long slot_stride, int tokens, int single,
                  cudaStream_t stream) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps) return static_cast<int>(cudaErrorInvalidValue);
  ConvArgs a;
  a.ld_x = ld_x; a.col_x = col_x; a.ld_y = ld_y; a.col_y = col_y; a.channels = channels; a.taps = taps; a.act = act;
  a.tokens = tokens; a.bias = bias; a.seq_of_token = seq_of_token; a.state_slot = state_slot; a.state = state;
  a.slot_stride = slot_stride;
  a.own_state = (single && taps > 1) ? 1 : 0;
  const int th = 128;
  // enough threads for the machine first: a thread walks several tokens only where there are thousands of them
  a.tile = static_cast<long long>(channels) * tokens >= (1ll << 20) ? kConvTile : 1;
  const dim3 grid((channels + th - 1) / th, (tokens + a.tile - 1) / a.tile);
  const dim3 grid_state((channels + th - 1) / th, (tokens + kStateTile - 1) / kStateTile);
#define RL_CASE(TA, TW)                                                                                        \
  do {                                                                                                         \
    launch_kernel(short_conv_kernel<TA, TW>, grid, dim3(th), 0, stream, a, static_cast<const TA*>(x),          \
                  static_cast<const TW*>(w), static_cast<TA*>(y));                                             \
    if (taps > 1 && !single) launch_kernel(short_conv_state_kernel<TA>, grid_state, dim3(th), 0, stream, a, static_cast<const TA*>(x)); \
  } while (0)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

}  // extern "C"
