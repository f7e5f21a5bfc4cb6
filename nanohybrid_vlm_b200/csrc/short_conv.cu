// Short causal convolution over time, one filter per channel, with SiLU, for packed steps of several requests.
//
//   y[t, c] = silu(bias[c] + sum_{j < K} w[c, j] * x[t - (K - 1) + j, c])
//
// where t counts within the request: inputs before the request's first token are zero, and inputs before this
// step's portion come from the request's state, which holds its last K - 1 inputs (fp32, [slot][K - 1][C], oldest
// first).  A first kernel computes all outputs (reading the old state), a second one moves the state on; a
// request with q_start == 0 starts from zeros whatever its slot held.  Requests without a slot (slot < 0: the
// idle entries that pad a captured batch) read zeros and write nothing.
#include "nhv_common.cuh"

constexpr int SC_MAX_TAPS = 8;
constexpr int SC_TOKENS = 32;       // tokens per block of the output kernel in a long step (each input is read once for them);
                                    // a short step takes one token per block: finding a token's request is a chain of
                                    // dependent loads that the tokens of a block would go through one after another

template <typename T, typename TO>
__global__ void short_conv_silu_kernel(TO* __restrict__ y, int y_stride, const T* __restrict__ x, int x_stride,
                                       const T* __restrict__ w, const T* __restrict__ bias,
                                       const float* __restrict__ state, long state_stride,
                                       const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                       const int* __restrict__ slots, int n_seqs, int n_tokens, int C, int K,
                                       int tokens_per_block) {
  pdl_prologue();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * tokens_per_block;
  if (c >= C || t0 >= n_tokens) return;
  // the filter right-aligned in 8 places (the last one is the current token's), zeros before it
  constexpr int M = SC_MAX_TAPS - 1;
  float wr[SC_MAX_TAPS];
#pragma unroll
  for (int m = 0; m < SC_MAX_TAPS; ++m) wr[m] = m >= SC_MAX_TAPS - K ? to_f32<T>(w[(size_t)c * K + (m - (SC_MAX_TAPS - K))]) : 0.f;
  const float b = bias ? to_f32<T>(bias[c]) : 0.f;
  // the request of the tile's first token (binary search over the starts), then walk on
  int lo = 0, hi = n_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t0) lo = mid; else hi = mid - 1;
  }
  int s = lo;
  int seq_first = cu_q[s], next_first = cu_q[s + 1];
  float win[M];                                     // the inputs before the current token, the latest last
  // the window in front of token t of request s: earlier tokens of this portion, behind them the request's state
  auto fill = [&](int t) {
    const int i = t - seq_first;
    const int slot = slots[s];
    const bool has_past = slot >= 0 && q_start[s] > 0;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = 0.f;
      if (m >= M - (K - 1)) {
        const int rel = i - M + m;                  // index in the portion; negative: before it
        if (rel >= 0) v = to_f32<T>(x[(size_t)(t - M + m) * x_stride + c]);
        else if (has_past) v = state[(size_t)slot * state_stride + (size_t)(K - 1 + rel) * C + c];
      }
      win[m] = v;
    }
  };
  fill(t0);
  const int t_end = min(t0 + tokens_per_block, n_tokens);
  for (int t = t0; t < t_end; ++t) {
    if (t >= next_first) {                          // the next request begins (requests without tokens are passed over)
      while (s + 1 < n_seqs && cu_q[s + 1] <= t) ++s;
      seq_first = cu_q[s];
      next_first = cu_q[s + 1];
      fill(t);
    }
    const float xt = to_f32<T>(x[(size_t)t * x_stride + c]);
    float acc = fmaf(wr[M], xt, b);
#pragma unroll
    for (int m = 0; m < M; ++m) acc = fmaf(wr[m], win[m], acc);
#pragma unroll
    for (int m = 0; m + 1 < M; ++m) win[m] = win[m + 1];
    win[M - 1] = xt;
    y[(size_t)t * y_stride + c] = from_f32<TO>(acc / (1.0f + expf(-acc)));
  }
}

template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                        long state_stride, const int* __restrict__ cu_q,
                                        const int* __restrict__ q_start, const int* __restrict__ slots, int C, int K) {
  pdl_prologue();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slots[s];
  if (c >= C || slot < 0) return;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const bool has_past = q_start[s] > 0;
  float* st = state + (size_t)slot * state_stride;
  float keep[SC_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS - 1; ++j) {
    keep[j] = 0.f;
    if (j < K - 1) {
      const int rel = n - (K - 1) + j;              // the input that becomes entry j of the new state
      if (rel >= 0) keep[j] = to_f32<T>(x[(size_t)(first + rel) * x_stride + c]);
      else if (has_past) keep[j] = st[(size_t)(K - 1 + rel) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS - 1; ++j)
    if (j < K - 1) st[(size_t)j * C + c] = keep[j];
}

// The same filter without bias or activation, added to its own input, for one or two filters over one input:
//   y1[t, c] = x[t, c] + sum_{j < K} w1[c, j] * x[t - (K - 1) + j, c],   y2 likewise with w2 (y2, w2 may be null)
// Both read the same inputs, so one state (the request's last K - 1 inputs) serves both.
template <typename T>
__global__ void filter_add_kernel(T* __restrict__ y1, T* __restrict__ y2, int y_stride, const T* __restrict__ x,
                                  int x_stride, const T* __restrict__ w1, const T* __restrict__ w2,
                                  const float* __restrict__ state, long state_stride, const int* __restrict__ cu_q,
                                  const int* __restrict__ q_start, const int* __restrict__ slots, int n_seqs,
                                  int n_tokens, int C, int K, int tokens_per_block) {
  pdl_prologue();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * tokens_per_block;
  if (c >= C || t0 >= n_tokens) return;
  constexpr int M = SC_MAX_TAPS - 1;
  float wa[SC_MAX_TAPS], wb[SC_MAX_TAPS];
#pragma unroll
  for (int m = 0; m < SC_MAX_TAPS; ++m) {
    const bool in = m >= SC_MAX_TAPS - K;
    wa[m] = in ? to_f32<T>(w1[(size_t)c * K + (m - (SC_MAX_TAPS - K))]) : 0.f;
    wb[m] = in && w2 ? to_f32<T>(w2[(size_t)c * K + (m - (SC_MAX_TAPS - K))]) : 0.f;
  }
  int lo = 0, hi = n_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t0) lo = mid; else hi = mid - 1;
  }
  int s = lo;
  int seq_first = cu_q[s], next_first = cu_q[s + 1];
  float win[M];
  auto fill = [&](int t) {
    const int i = t - seq_first;
    const int slot = slots[s];
    const bool has_past = slot >= 0 && q_start[s] > 0;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = 0.f;
      if (m >= M - (K - 1)) {
        const int rel = i - M + m;
        if (rel >= 0) v = to_f32<T>(x[(size_t)(t - M + m) * x_stride + c]);
        else if (has_past) v = state[(size_t)slot * state_stride + (size_t)(K - 1 + rel) * C + c];
      }
      win[m] = v;
    }
  };
  fill(t0);
  const int t_end = min(t0 + tokens_per_block, n_tokens);
  for (int t = t0; t < t_end; ++t) {
    if (t >= next_first) {
      while (s + 1 < n_seqs && cu_q[s + 1] <= t) ++s;
      seq_first = cu_q[s];
      next_first = cu_q[s + 1];
      fill(t);
    }
    const float xt = to_f32<T>(x[(size_t)t * x_stride + c]);
    float a = wa[M] * xt, b = wb[M] * xt;               // oldest tap first, the current token last, then the input itself
    float ra = 0.f, rb = 0.f;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      ra = fmaf(wa[m], win[m], ra);
      rb = fmaf(wb[m], win[m], rb);
    }
#pragma unroll
    for (int m = 0; m + 1 < M; ++m) win[m] = win[m + 1];
    win[M - 1] = xt;
    y1[(size_t)t * y_stride + c] = from_f32<T>(xt + (ra + a));
    if (y2) y2[(size_t)t * y_stride + c] = from_f32<T>(xt + (rb + b));
  }
}

// y1 (and y2) [T, C] rows of y_stride; x [T, C] rows of x_stride; w1 (and w2) [C, K]; all of one type.  The state
// [slots][(K - 1) * C] fp32 is read and then moved on.
NHV_API int nhv_causal_filter_add(int dtype, void* y1, void* y2, int y_stride, const void* x, int x_stride, const void* w1,
                                  const void* w2, float* state, long state_stride, const int* cu_q, const int* q_start,
                                  const int* slots, int n_seqs, int n_tokens, int C, int K, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(C > 0 && K >= 1 && K <= SC_MAX_TAPS, "causal_filter: %d taps are beyond the supported %d", K, SC_MAX_TAPS);
  NHV_REQUIRE(K == 1 || (state && state_stride >= (long)(K - 1) * C), "causal_filter: the state holds fewer than (taps - 1) * channels floats");
  NHV_REQUIRE(y1 && w1 && (!y2) == (!w2), "causal_filter: a second output comes with a second filter");
  const int threads = 128;
  const int tokens_per_block = n_tokens <= 512 ? 1 : SC_TOKENS;
  dim3 grid((n_tokens + tokens_per_block - 1) / tokens_per_block, (C + threads - 1) / threads);
  dim3 grid2(n_seqs, (C + threads - 1) / threads);
#define LAUNCH(T)                                                                                                  \
  do {                                                                                                             \
    nhv_launch(filter_add_kernel<T>, grid, threads, 0, stream, (T*)y1, (T*)y2, y_stride, (const T*)x, x_stride,    \
               (const T*)w1, (const T*)w2, (const float*)state, state_stride, cu_q, q_start, slots, n_seqs,        \
               n_tokens, C, K, tokens_per_block);                                                                  \
    if (K > 1)                                                                                                     \
      nhv_launch(short_conv_state_kernel<T>, grid2, threads, 0, stream, (const T*)x, x_stride, state, state_stride, \
                 cu_q, q_start, slots, C, K);                                                                      \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "causal_filter: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("causal_filter");
  return 0;
}

// dtype: of x, the filters and the bias; out_dtype: of y (fp32 where a recurrence reads it next)
NHV_API int nhv_short_conv_silu(int dtype, int out_dtype, void* y, int y_stride, const void* x, int x_stride, const void* w,
                                const void* bias, float* state, long state_stride, const int* cu_q,
                                const int* q_start, const int* slots, int n_seqs, int n_tokens, int C, int K,
                                cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(out_dtype == dtype || out_dtype == NHV_F32, "short_conv: the output is of the input's type or fp32");
  NHV_REQUIRE(C > 0 && K >= 1 && K <= SC_MAX_TAPS, "short_conv: %d taps are beyond the supported %d", K, SC_MAX_TAPS);
  NHV_REQUIRE(K == 1 || (state && state_stride >= (long)(K - 1) * C), "short_conv: the state holds fewer than (taps - 1) * channels floats");
  const int threads = 128;
  const int tokens_per_block = n_tokens <= 512 ? 1 : SC_TOKENS;
  dim3 grid((n_tokens + tokens_per_block - 1) / tokens_per_block, (C + threads - 1) / threads);
  dim3 grid2(n_seqs, (C + threads - 1) / threads);
#define OUT(T, TO)                                                                                                 \
  nhv_launch(short_conv_silu_kernel<T, TO>, grid, threads, 0, stream, (TO*)y, y_stride, (const T*)x, x_stride,     \
             (const T*)w, (const T*)bias, (const float*)state, state_stride, cu_q, q_start, slots, n_seqs,         \
             n_tokens, C, K, tokens_per_block)
#define LAUNCH(T)                                                                                                  \
  do {                                                                                                             \
    if (out_dtype == NHV_F32) OUT(T, float);                                                                       \
    else OUT(T, T);                                                                                                \
    if (K > 1)                                                                                                     \
      nhv_launch(short_conv_state_kernel<T>, grid2, threads, 0, stream, (const T*)x, x_stride, state, state_stride, \
                 cu_q, q_start, slots, C, K);                                                                      \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "short_conv: unknown dtype %d", dtype);
#undef LAUNCH
#undef OUT
  NHV_CHECK_LAUNCH("short_conv");
  return 0;
}
