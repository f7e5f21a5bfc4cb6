// Linear recurrences with a matrix state per head that decays per key channel, for packed steps of several requests:
//
//   S_t = diag(w_t) S_(t-1) + k_t v_t^T                      S [dk, dv] per head, fp32, one per live request
//   read before the update (a bonus b for the current token):  o_t = (S_(t-1) + diag(b) k_t v_t^T)^T r_t
//   read after the update:                                     o_t = S_t^T r_t
//
// Both reads are  o_t[v] = sum_k r'_k S_(t-1)[k, v] + c_t v_t[v]  with r' = r and c_t = sum_k r_k b_k k_k in the first
// form, r' = r * w_t and c_t = r_t . k_t in the second; r' and c_t are made once per token while it is staged, so the
// loop over the state has one multiply-add for the read and one for the update per element.
// The decay is a tensor per token and key channel (fp32, [T, H dk]) or one constant per head.  r, k and v come in the
// storage type (the projections' output), optionally through SiLU, and are widened once; everything else is fp32.
//
// decay_lowrank: w[t, c] = exp(-exp(w0[c] + sum_j tanh(inner[t, j]) w2[c, j])), the decay of the first form from the
// fp32 sums of its inner projection; the tanh stays fp32 and the small second product is summed in fp32 in a fixed order.
//
// Block = (request, head, 16 columns of the state); a column lives in 8 lanes (heads of up to 32 key channels) or 16,
// lane l holding the key channels 4 LANES i + 4 l .. + 3 of it in registers (KPL channels per lane).  Tokens are staged
// 16 at a time in shared memory (8 for the widest heads).
// State layout per slot: [H][dv][dk].  A request with q_start == 0 starts from zeros whatever its slot held; a request
// without a slot (slot < 0: the idle entries that pad a captured batch) gets zeros and keeps nothing.
#include <math.h>

#include "nhv_common.cuh"

constexpr int DS_COLS = 16;          // columns of the memory per block
constexpr int DS_TOKENS = 16;

// 16 bytes of the storage type, kept as they were read until they are needed (a register that is only the target of a
// read in flight does not hold the thread up; the first instruction that looks at it does)
template <typename T> struct DsVec;
template <> struct DsVec<float> {
  static constexpr int N = 4;
  __device__ static uint4 pack(const float (&x)[4]) {
    return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
  }
  __device__ static void unpack(float (&o)[4], const uint4& v) {
    o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
  }
};
template <> struct DsVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static uint4 pack(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (__float_as_uint(x[2 * i]) >> 16) | (__float_as_uint(x[2 * i + 1]) & 0xffff0000u);
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static void unpack(float (&o)[8], const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);             // a bfloat16 is the upper half of a float
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// SiLU of a projection's output.  float32 storage: the exact exponential and division.  bfloat16 storage: the input
// carries 8 bits, so the fast exponential and reciprocal (errors near 1e-6) are far below what it already lost.
template <typename T> __device__ __forceinline__ float ds_silu(float x) {
  if constexpr (sizeof(T) == 2) return x * __frcp_rn(1.0f + __expf(-x));
  else return x / (1.0f + expf(-x));
}

// A chunk of tokens travels in two steps: `fetch` reads it from global memory into registers (16-byte reads where the
// layout allows; issued before the chunk in shared memory is worked on, so the reads are in flight meanwhile), `put`
// writes it, widened and through SiLU if asked, into shared memory.
// CW: the decay is one constant per head (it is not staged per token and key channel).
// LANES: lanes that share a column (8 or 16); the block has DS_COLS * LANES threads.
template <typename T, int KPL, int LANES, bool CW>
__global__ void __launch_bounds__(DS_COLS * LANES) decay_scan_kernel(
    float* __restrict__ o, const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, int ld,
    const float* __restrict__ w_tok, const float* __restrict__ w_head, const T* __restrict__ bonus,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int H, int dk, int dv, int act_silu, int read_after, int vec_ok, int wvec_ok) {
  constexpr int DS_THREADS = DS_COLS * LANES, DS_LANES = LANES;
  constexpr int DKP = KPL * DS_LANES;                 // key channels with padding (zeros)
  constexpr int TOK = DKP >= 256 ? DS_TOKENS / 2 : DS_TOKENS;     // the widest heads stage fewer tokens (48 KB of static shared memory)
  constexpr int VN = DsVec<T>::N;
  constexpr int RK_VECS = TOK * DKP / VN;             // 16-byte pieces of r (and of k) in a chunk
  constexpr int RK_PER = (RK_VECS + DS_THREADS - 1) / DS_THREADS;
  constexpr int W_VECS = TOK * DKP / 4;               // float4 pieces of the decay in a chunk
  constexpr int W_PER = (W_VECS + DS_THREADS - 1) / DS_THREADS;
  constexpr int V_PER = (TOK * DS_COLS + DS_THREADS - 1) / DS_THREADS;
  __shared__ __align__(16) float rs[TOK][DKP];
  __shared__ __align__(16) float ks[TOK][DKP];
  __shared__ __align__(16) float ws[TOK][DKP];
  __shared__ float vs[TOK][DS_COLS];
  __shared__ float cs[TOK];
  pdl_prologue();
  const int seq = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * DS_COLS;
  const int first = cu_q[seq], n = cu_q[seq + 1] - first;
  if (n <= 0) return;
  const int tid = threadIdx.x, lane = tid & (DS_LANES - 1), cl = tid / DS_LANES;
  const int col = col0 + cl;
  const int slot = slots[seq];
  const bool col_ok = col < dv;
  float S[KPL];
  float* st = slot >= 0 ? state + (size_t)slot * state_stride + ((size_t)h * dv + (col_ok ? col : 0)) * dk : nullptr;
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int c = (i >> 2) * (4 * DS_LANES) + lane * 4 + (i & 3);
    S[i] = (st && col_ok && c < dk && q_start[seq] > 0) ? st[c] : 0.f;
  }
  const float wh = w_head ? w_head[h] : 1.f;
  const int warp = tid >> 5, wl = tid & 31;

  uint4 fr[RK_PER], fk[RK_PER];                       // as read: the first look at them is in put()
  float4 fw[W_PER];
  T fv[V_PER];
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int q = 0; q < RK_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      const int tt = idx / (DKP / VN), c = (idx - tt * (DKP / VN)) * VN;
      fr[q] = fk[q] = make_uint4(0, 0, 0, 0);
      if (idx < RK_VECS && tt < nt && c < dk) {
        const size_t at = (size_t)(first + t0 + tt) * ld + (size_t)h * dk + c;
        if (vec_ok) {
          fr[q] = *reinterpret_cast<const uint4*>(r + at);
          fk[q] = *reinterpret_cast<const uint4*>(k + at);
        } else {                                        // rows that are not on 16-byte boundaries: element by element
          float xr[VN], xk[VN];
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            xr[e] = c + e < dk ? to_f32<T>(r[at + e]) : 0.f;
            xk[e] = c + e < dk ? to_f32<T>(k[at + e]) : 0.f;
          }
          fr[q] = DsVec<T>::pack(xr);
          fk[q] = DsVec<T>::pack(xk);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < W_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      const int tt = idx / (DKP / 4), c = (idx - tt * (DKP / 4)) * 4;
      fw[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (CW) continue;
      if (idx < W_VECS && tt < nt && c < dk) {
        if (!w_tok) {
          fw[q] = make_float4(wh, c + 1 < dk ? wh : 0.f, c + 2 < dk ? wh : 0.f, c + 3 < dk ? wh : 0.f);
        } else {
          const float* src = w_tok + (size_t)(first + t0 + tt) * H * dk + (size_t)h * dk + c;
          if (wvec_ok) fw[q] = *reinterpret_cast<const float4*>(src);
          else fw[q] = make_float4(src[0], c + 1 < dk ? src[1] : 0.f, c + 2 < dk ? src[2] : 0.f, c + 3 < dk ? src[3] : 0.f);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < V_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      const int tt = idx / DS_COLS, c = idx - tt * DS_COLS;
      fv[q] = (idx < TOK * DS_COLS && tt < nt && col0 + c < dv) ? v[(size_t)(first + t0 + tt) * ld + (size_t)h * dv + col0 + c] : from_f32<T>(0.f);
    }
  };
  auto put = [&]() {
#pragma unroll
    for (int q = 0; q < RK_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      if (idx >= RK_VECS) continue;
      const int tt = idx / (DKP / VN), c = (idx - tt * (DKP / VN)) * VN;
      float xr[VN], xk[VN];
      DsVec<T>::unpack(xr, fr[q]);
      DsVec<T>::unpack(xk, fk[q]);
      if (act_silu) {
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          xr[e] = ds_silu<T>(xr[e]);
          xk[e] = ds_silu<T>(xk[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < VN; e += 4) {                 // 16-byte writes: no two lanes of a quarter warp in one bank
        *reinterpret_cast<float4*>(&rs[tt][c + e]) = make_float4(xr[e], xr[e + 1], xr[e + 2], xr[e + 3]);
        *reinterpret_cast<float4*>(&ks[tt][c + e]) = make_float4(xk[e], xk[e + 1], xk[e + 2], xk[e + 3]);
      }
    }
#pragma unroll
    for (int q = 0; q < W_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      if (CW || idx >= W_VECS) continue;
      const int tt = idx / (DKP / 4), c = (idx - tt * (DKP / 4)) * 4;
      *reinterpret_cast<float4*>(&ws[tt][c]) = fw[q];
    }
#pragma unroll
    for (int q = 0; q < V_PER; ++q) {
      const int idx = tid + q * DS_THREADS;
      const int tt = idx / DS_COLS, c = idx - tt * DS_COLS;
      const float x = to_f32<T>(fv[q]);
      if (idx < TOK * DS_COLS) vs[tt][c] = act_silu ? ds_silu<T>(x) : x;
    }
  };
  // the bonus of this lane's key channels in the per-token sums below (ones where there is none)
  float bon[DKP / 32];
#pragma unroll
  for (int i = 0; i < DKP / 32; ++i) {
    const int c = wl + 32 * i;
    bon[i] = (!read_after && bonus && c < dk) ? to_f32<T>(bonus[(size_t)h * dk + c]) : 1.f;
  }

  fetch(0, min(TOK, n));
  for (int t0 = 0; t0 < n; t0 += TOK) {
    const int nt = min(TOK, n - t0);
    __syncthreads();                                    // the chunk before has been worked on
    put();
    __syncthreads();
    // per token: the current token's own weight c_t (a fixed order of summation), then r' in place of r
    for (int tt = warp; tt < nt; tt += DS_THREADS / 32) {
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < DKP / 32; ++i) part = fmaf(rs[tt][wl + 32 * i] * bon[i], ks[tt][wl + 32 * i], part);
      part = warp_sum(part);
      if (wl == 0) cs[tt] = part;
      if (read_after) {
#pragma unroll
        for (int i = 0; i < DKP / 32; ++i) rs[tt][wl + 32 * i] *= CW ? wh : ws[tt][wl + 32 * i];
      }
    }
    if (t0 + TOK < n) fetch(t0 + TOK, min(TOK, n - t0 - TOK));      // the next chunk's reads fly while this one is worked on
    __syncthreads();
    // tokens in turn; only the memory's update is carried from one to the next, so four tokens' reads overlap
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float vt = vs[tt][cl];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int j = 0; j < KPL / 4; ++j) {
        const float4 r4 = *reinterpret_cast<const float4*>(&rs[tt][j * (4 * DS_LANES) + lane * 4]);
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][j * (4 * DS_LANES) + lane * 4]);
        // (padded key channels decay by the constant too: their memory is zero and their keys are zero)
        const float4 w4 = CW ? make_float4(wh, wh, wh, wh) : *reinterpret_cast<const float4*>(&ws[tt][j * (4 * DS_LANES) + lane * 4]);
        acc0 = fmaf(r4.x, S[4 * j + 0], acc0);
        acc1 = fmaf(r4.y, S[4 * j + 1], acc1);
        acc0 = fmaf(r4.z, S[4 * j + 2], acc0);
        acc1 = fmaf(r4.w, S[4 * j + 3], acc1);
        S[4 * j + 0] = fmaf(w4.x, S[4 * j + 0], k4.x * vt);
        S[4 * j + 1] = fmaf(w4.y, S[4 * j + 1], k4.y * vt);
        S[4 * j + 2] = fmaf(w4.z, S[4 * j + 2], k4.z * vt);
        S[4 * j + 3] = fmaf(w4.w, S[4 * j + 3], k4.w * vt);
      }
      float acc = acc0 + acc1;
      if (DS_LANES == 16) acc += __shfl_xor_sync(0xffffffffu, acc, 8);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (lane == 0 && col_ok) o[(size_t)(first + t0 + tt) * H * dv + (size_t)h * dv + col] = fmaf(cs[tt], vt, acc);
    }
  }
  if (st && col_ok) {
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      const int c = (i >> 2) * (4 * DS_LANES) + lane * 4 + (i & 3);
      if (c < dk) st[c] = S[i];
    }
  }
}

NHV_API int nhv_decay_scan(int dtype, float* o, const void* r, const void* k, const void* v, int ld, const float* w_tok,
                           const float* w_head, const void* bonus, float* state, long state_stride, const int* cu_q,
                           const int* q_start, const int* slots, int n_seqs, int n_tokens, int H, int dk, int dv,
                           int act_silu, int read_after, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(H > 0 && dk > 0 && dv > 0 && dk <= 256, "decay_scan: key heads of 1 to 256 channels, got %d", dk);
  NHV_REQUIRE((w_tok != nullptr) != (w_head != nullptr), "decay_scan: the decay is a tensor per token or a constant per head");
  NHV_REQUIRE(state && state_stride >= (long)H * dk * dv, "decay_scan: the state holds H dk dv floats per request");
  dim3 grid((dv + DS_COLS - 1) / DS_COLS, H, n_seqs);
  // 16-byte reads of r and k (rows and heads on 16-byte boundaries) and of the decay tensor
  const size_t esize = dtype == NHV_F32 ? 4 : 2;
  const int per16 = (int)(16 / esize);
  const int vec_ok = ld % per16 == 0 && dk % per16 == 0 && ((uintptr_t)r % 16) == 0 && ((uintptr_t)k % 16) == 0;
  const int wvec_ok = w_tok && dk % 4 == 0 && ((uintptr_t)w_tok % 16) == 0;
#define LAUNCH(T, KPL, LANES)                    \
  do {                                           \
    if (w_head) LAUNCH_W(T, KPL, LANES, true);   \
    else LAUNCH_W(T, KPL, LANES, false);         \
  } while (0)
#define LAUNCH_W(T, KPL, LANES, CW)                                                                                  \
  nhv_launch(decay_scan_kernel<T, KPL, LANES, CW>, grid, DS_COLS * LANES, 0, stream, o, (const T*)r, (const T*)k,    \
             (const T*)v, ld,                                                                                        \
             w_tok, w_head, (const T*)bonus, state, state_stride, cu_q, q_start, slots, H, dk, dv, act_silu, read_after,  \
             vec_ok, wvec_ok)
#define LAUNCH_K(T)                    \
  do {                                 \
    if (dk <= 32) LAUNCH(T, 4, 8);          \
    else if (dk <= 64) LAUNCH(T, 4, 16);    \
    else if (dk <= 128) LAUNCH(T, 8, 16);   \
    else LAUNCH(T, 16, 16);                 \
  } while (0)
  if (dtype == NHV_F32) LAUNCH_K(float);
  else if (dtype == NHV_BF16) LAUNCH_K(__nv_bfloat16);
  else NHV_REQUIRE(false, "decay_scan: unknown dtype %d", dtype);
#undef LAUNCH_K
#undef LAUNCH
#undef LAUNCH_W
  NHV_CHECK_LAUNCH("decay_scan");
  return 0;
}

constexpr int DL_TOKENS = 16;       // tokens per block of decay_lowrank: a row of w2 is read once for all of them

template <typename T>
__global__ void decay_lowrank_kernel(float* __restrict__ w, const float* __restrict__ inner, int inner_stride,
                                     const T* __restrict__ w2, const T* __restrict__ w0, int n_tokens, int n, int rank) {
  extern __shared__ float th[];                       // [DL_TOKENS][rank]: tanh of the tokens' inner projections
  pdl_prologue();
  const int t0 = blockIdx.x * DL_TOKENS;
  const int nt = min(DL_TOKENS, n_tokens - t0);
  for (int i = threadIdx.x; i < nt * rank; i += blockDim.x) {
    const int tt = i / rank, j = i - tt * rank;
    th[i] = tanhf(inner[(size_t)(t0 + tt) * inner_stride + j]);
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float z[DL_TOKENS];
  const float z0 = to_f32<T>(w0[c]);
#pragma unroll
  for (int tt = 0; tt < DL_TOKENS; ++tt) z[tt] = z0;
  const T* row = w2 + (size_t)c * rank;
  for (int j = 0; j < rank; ++j) {                    // every token's sum runs over j in ascending order
    const float wj = to_f32<T>(row[j]);
#pragma unroll
    for (int tt = 0; tt < DL_TOKENS; ++tt)
      if (tt < nt) z[tt] = fmaf(th[tt * rank + j], wj, z[tt]);
  }
#pragma unroll
  for (int tt = 0; tt < DL_TOKENS; ++tt)
    if (tt < nt) w[(size_t)(t0 + tt) * n + c] = expf(-expf(z[tt]));
}

NHV_API int nhv_decay_lowrank(int dtype, float* w, const float* inner, int inner_stride, const void* w2, const void* w0,
                              int n_tokens, int n, int rank, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n > 0 && rank > 0 && rank <= 2048 && inner_stride >= rank, "decay_lowrank: bad sizes (n %d, rank %d)", n, rank);
  const int threads = 128;
  dim3 grid((n_tokens + DL_TOKENS - 1) / DL_TOKENS, (n + threads - 1) / threads);
  NHV_REQUIRE(grid.y <= 65535, "decay_lowrank: %d channels are beyond the grid's reach", n);
  const size_t smem = (size_t)DL_TOKENS * rank * sizeof(float);
#define LAUNCH(T)                                                                                                     \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      NHV_CUDA(cudaFuncSetAttribute(decay_lowrank_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), \
               "decay_lowrank");                                                                                      \
    nhv_launch(decay_lowrank_kernel<T>, grid, threads, smem, stream, w, inner, inner_stride, (const T*)w2,            \
               (const T*)w0, n_tokens, n, rank);                                                                      \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "decay_lowrank: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("decay_lowrank");
  return 0;
}
