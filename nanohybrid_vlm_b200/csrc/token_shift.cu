// Mixes of a token's input with the input of the token before it, for packed steps of several requests:
//
//   out[s, t, c] = x[t, c] + (x[t - 1, c] - x[t, c]) * mu[s, c]        s < n_mix  (one contiguous [T, C] plane per mix)
//
// where t counts within the request: the token before a request's first token is zero, and the one before this step's
// portion is the request's state (fp32, [slot][C]: its last input).  A first kernel computes all mixes (reading the
// old state), a second one moves the state on; a request with q_start == 0 starts from zeros whatever its slot held.
// Requests without a slot (slot < 0: the idle entries that pad a captured batch) read zeros and write nothing.
// The arithmetic is fp32, rounded once to the storage type.
#include "nhv_common.cuh"

constexpr int TS_MAX_MIX = 8;
constexpr int TS_TOKENS = 16;

template <typename T>
__global__ void token_shift_mix_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ mu,
                                       const float* __restrict__ state, long state_stride,
                                       const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                       const int* __restrict__ slots, int n_seqs, int n_tokens, int C, int n_mix,
                                       int tokens_per_block) {
  pdl_prologue();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * tokens_per_block;
  if (c >= C || t0 >= n_tokens) return;
  float m[TS_MAX_MIX];
#pragma unroll
  for (int s = 0; s < TS_MAX_MIX; ++s) m[s] = s < n_mix ? to_f32<T>(mu[(size_t)s * C + c]) : 0.f;
  int lo = 0, hi = n_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t0) lo = mid; else hi = mid - 1;
  }
  int s = lo;
  int next_first = cu_q[s + 1];
  auto before = [&](int t) -> float {
    if (t > cu_q[s]) return to_f32<T>(x[(size_t)(t - 1) * C + c]);
    const int slot = slots[s];
    return slot >= 0 && q_start[s] > 0 ? state[(size_t)slot * state_stride + c] : 0.f;
  };
  float prev = before(t0);
  const int t_end = min(t0 + tokens_per_block, n_tokens);
  for (int t = t0; t < t_end; ++t) {
    if (t >= next_first) {                          // the next request begins (requests without tokens are passed over)
      while (s + 1 < n_seqs && cu_q[s + 1] <= t) ++s;
      next_first = cu_q[s + 1];
      prev = before(t);
    }
    const float xt = to_f32<T>(x[(size_t)t * C + c]);
    const float d = prev - xt;
    T* dst = out + (size_t)t * C + c;
#pragma unroll
    for (int k = 0; k < TS_MAX_MIX; ++k)
      if (k < n_mix) dst[(size_t)k * n_tokens * C] = from_f32<T>(fmaf(d, m[k], xt));
    prev = xt;
  }
}

template <typename T>
__global__ void token_shift_state_kernel(const T* __restrict__ x, float* __restrict__ state, long state_stride,
                                         const int* __restrict__ cu_q, const int* __restrict__ slots, int C) {
  pdl_prologue();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slots[s];
  const int last = cu_q[s + 1] - 1;
  if (c >= C || slot < 0 || last < cu_q[s]) return;
  state[(size_t)slot * state_stride + c] = to_f32<T>(x[(size_t)last * C + c]);
}

NHV_API int nhv_token_shift_mix(int dtype, void* out, const void* x, const void* mu, float* state, long state_stride,
                                const int* cu_q, const int* q_start, const int* slots, int n_seqs, int n_tokens, int C,
                                int n_mix, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(C > 0 && n_mix > 0 && n_mix <= TS_MAX_MIX, "token_shift_mix: 1 to %d mixes, got %d", TS_MAX_MIX, n_mix);
  NHV_REQUIRE(state && state_stride >= C, "token_shift_mix: the state holds one input per request");
  const int threads = C >= 256 ? 256 : 64;
  const int tokens_per_block = n_tokens >= 4 * TS_TOKENS ? TS_TOKENS : 1;
  dim3 grid((n_tokens + tokens_per_block - 1) / tokens_per_block, (C + threads - 1) / threads);
  dim3 sgrid(n_seqs, (C + threads - 1) / threads);
#define LAUNCH(T)                                                                                                     \
  do {                                                                                                                \
    nhv_launch(token_shift_mix_kernel<T>, grid, threads, 0, stream, (T*)out, (const T*)x, (const T*)mu, state,        \
               state_stride, cu_q, q_start, slots, n_seqs, n_tokens, C, n_mix, tokens_per_block);                     \
    nhv_launch(token_shift_state_kernel<T>, sgrid, threads, 0, stream, (const T*)x, state, state_stride, cu_q, slots, C); \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "token_shift_mix: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("token_shift_mix");
  return 0;
}
