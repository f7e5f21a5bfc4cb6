// The generalised delta rule as a recurrence over a packed step of several requests.
//
// Per head, with the state S [d, d] (fp32, carried per request; rows: key channels, columns: value channels):
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,     o_t = S_t^T r_t
// where u_t = k_t / sqrt(sum k_t^2 + 1e-6) is the unit key, w_t a decay per key channel and a_t a removal rate per key
// channel:  w_t = exp(-decay_floor * sigmoid(e_t + w0)),  a_t = sigmoid(y_t + b), with e_t = W2 tanh(z_t) and y_t [H d]
// projections of the token that the caller gives in fp32 (z_t [rank] a small projection; general_delta_tanh makes
// tanh(z_t) in the storage type for the product with W2).  Decay and removal both read the state of the token before.
//
// general_delta_prepare: one warp per (token, head): u, a * u, r * w, w, k widened to fp32, the two scalars
//                r . (a * u) and r . k, and v in fp32.
// general_delta_scan:    the columns of S are independent of one another.  Column j (a vector s over the key channels):
//                  A = u . s,  B = (r * w) . s          (both over the old column, side by side)
//                  s <- w * s - (a * u) A + k v_j
//                  o_j = B - A (r . (a * u)) + v_j (r . k)
//                which is the read-out after the write.  A block takes (request, head, 16 columns); a column lives in
//                the registers of 8 lanes, each with d / 8 rows in groups of four; tokens pass through shared memory 16
//                at a time.  The token order per column is fixed, so a position's result does not depend on how the
//                tokens were cut into steps.
// The state of a slot is stored transposed, [head][column][row].  A request with q_start == 0 starts from zeros; one
// without a slot (slot < 0) is skipped and its outputs are cleared.  o is written in fp32; its norm and gate follow in
// nhv_gated_rmsnorm.
#include <math.h>

#include "nhv_common.cuh"

constexpr int GD_WARPS = 4;
constexpr int GD_MAX_D = 256;
constexpr int GD_CHUNK = 16;
constexpr int GD_LANES = 8;
constexpr int GD_THREADS = 128;
constexpr int GD_COLS = GD_THREADS / GD_LANES;

// out[t, j] = tanh(in[t, j]) in the storage type, in [T, cols] fp32 with rows in_stride apart.
template <typename T>
__global__ void general_delta_tanh_kernel(T* __restrict__ out, const float* __restrict__ in, int in_stride, int cols,
                                          size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / cols;
    out[i] = from_f32<T>(tanhf(in[t * in_stride + (i - t * cols)]));
  }
}

// proj [T, 4 n] rows of proj_stride: r, k, v (then the gate, not read here); aw [T, >= n] fp32: y; dec [T, n] fp32: e.
// vec [5][T, H, d] fp32: u, a*u, r*w, w, k; sc [T, H, 2]: r.(a*u), r.k; v32 [T, H, d].
template <typename T>
__global__ void general_delta_prepare_kernel(float* __restrict__ vec, float* __restrict__ sc, float* __restrict__ v32,
                                             const T* __restrict__ proj, int proj_stride, const float* __restrict__ aw,
                                             int aw_stride, const T* __restrict__ a_bias, const float* __restrict__ dec,
                                             const T* __restrict__ w0, int n_tokens, int H, int d,
                                             float decay_floor) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * GD_WARPS + warp;
  if (item >= (long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  const int n = H * d;
  const T* row = proj + (size_t)t * proj_stride;
  const float* awr = aw + (size_t)t * aw_stride;
  float kk[GD_MAX_D / 32], ss = 0.f;
#pragma unroll
  for (int i = 0; i < GD_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    kk[i] = c < d ? to_f32<T>(row[n + h * d + c]) : 0.f;
    ss = fmaf(kk[i], kk[i], ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + 1e-6f);
  const size_t plane = (size_t)n_tokens * n, at = (size_t)t * n + (size_t)h * d;
  float ra = 0.f, rk = 0.f;
#pragma unroll
  for (int i = 0; i < GD_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < d) {
      const int col = h * d + c;
      const float z = dec[(size_t)t * n + col] + to_f32<T>(w0[col]);
      const float decay = expf(-decay_floor / (1.0f + expf(-z)));
      const float rate = 1.0f / (1.0f + expf(-(awr[col] + to_f32<T>(a_bias[col]))));
      const float r = to_f32<T>(row[col]);
      const float u = kk[i] * inv, au = rate * u;
      vec[at + c] = u;
      vec[plane + at + c] = au;
      vec[2 * plane + at + c] = r * decay;
      vec[3 * plane + at + c] = decay;
      vec[4 * plane + at + c] = kk[i];
      v32[at + c] = to_f32<T>(row[2 * n + col]);
      ra = fmaf(r, au, ra);
      rk = fmaf(r, kk[i], rk);
    }
  }
  ra = warp_sum(ra);
  rk = warp_sum(rk);
  if (lane == 0) {
    sc[(size_t)item * 2] = ra;
    sc[(size_t)item * 2 + 1] = rk;
  }
}

__device__ __forceinline__ void gd_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void gd_cp_async8(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void gd_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void gd_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// R: rows of a column per lane (a multiple of 4, 8 R >= d).  ASYNC (d a multiple of 4): the tokens reach shared memory
// by cp.async, 16 at a time, the next 16 while these are worked on; otherwise by plain loads, one stage.
template <int R, bool ASYNC>
__global__ void __launch_bounds__(GD_THREADS) general_delta_scan_kernel(
    float* __restrict__ o_out, const float* __restrict__ vec, const float* __restrict__ sc, const float* __restrict__ v32,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int n_tokens, int H, int d) {
  extern __shared__ __align__(16) float smem[];
  pdl_prologue();
  constexpr int DP = R * GD_LANES;                    // a vector in shared memory: d floats, then zeros
  constexpr int STAGE = 5 * GD_CHUNK * DP + GD_CHUNK * GD_COLS + GD_CHUNK * 2;
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GD_COLS;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(GD_COLS, d - col0);
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += GD_THREADS)
      o_out[((size_t)(first + i / ncol) * H + h) * d + col0 + i % ncol] = 0.f;
    return;
  }
  const int cl = tid / GD_LANES, part = tid % GD_LANES;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * d + col) * d;
  float S[R];
  const bool fresh = q_start[s] == 0;
#pragma unroll
  for (int j = 0; j < R / 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * (part + GD_LANES * j) + e;
      S[4 * j + e] = (live && !fresh && i < d) ? st[i] : 0.f;
    }
  const size_t plane = (size_t)n_tokens * H * d;
  if constexpr (ASYNC) {                              // what no copy writes: the zeros behind a vector, the columns past d
    for (int i = tid; i < 2 * STAGE; i += GD_THREADS) smem[i] = 0.f;
    __syncthreads();
  }
  // tokens [c0, c0 + cn) of the request into a stage: [5][CHUNK][DP] u, a*u, r*w, w, k; [CHUNK][COLS] v; [CHUNK][2]
  auto fetch = [&](int c0, int stage) {
    float* base = smem + stage * STAGE;
    const int cn = min(GD_CHUNK, n - c0);
    if constexpr (ASYNC) {
      const int quads = d >> 2, per = cn * quads;
      for (int i = tid; i < 5 * per; i += GD_THREADS) {
        const int which = i / per, rem = i - which * per;
        const int tt = rem / quads, c = rem - tt * quads;
        gd_cp_async16(base + (which * GD_CHUNK + tt) * DP + 4 * c,
                      vec + which * plane + ((size_t)(first + c0 + tt) * H + h) * d + 4 * c);
      }
      const int vq = ncol >> 2;
      for (int i = tid; i < cn * vq; i += GD_THREADS) {
        const int tt = i / vq, c = i - tt * vq;
        gd_cp_async16(base + 5 * GD_CHUNK * DP + tt * GD_COLS + 4 * c,
                      v32 + ((size_t)(first + c0 + tt) * H + h) * d + col0 + 4 * c);
      }
      for (int tt = tid; tt < cn; tt += GD_THREADS)
        gd_cp_async8(base + 5 * GD_CHUNK * DP + GD_CHUNK * GD_COLS + tt * 2, sc + ((size_t)(first + c0 + tt) * H + h) * 2);
    } else {
      for (int i = tid; i < 5 * cn * DP; i += GD_THREADS) {
        const int which = i / (cn * DP), rem = i - which * (cn * DP);
        const int tt = rem / DP, c = rem - tt * DP;
        base[(which * GD_CHUNK + tt) * DP + c] =
            c < d ? vec[which * plane + ((size_t)(first + c0 + tt) * H + h) * d + c] : 0.f;
      }
      for (int i = tid; i < cn * GD_COLS; i += GD_THREADS) {
        const int tt = i / GD_COLS, c = i - tt * GD_COLS;
        base[5 * GD_CHUNK * DP + i] = c < ncol ? v32[((size_t)(first + c0 + tt) * H + h) * d + col0 + c] : 0.f;
      }
      for (int i = tid; i < cn * 2; i += GD_THREADS)
        base[5 * GD_CHUNK * DP + GD_CHUNK * GD_COLS + i] = sc[((size_t)(first + c0 + (i >> 1)) * H + h) * 2 + (i & 1)];
    }
  };
  const int n_chunks = (n + GD_CHUNK - 1) / GD_CHUNK;
  if constexpr (ASYNC) {
    fetch(0, 0);
    gd_cp_async_commit();
  }
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * GD_CHUNK;
    const int cn = min(GD_CHUNK, n - c0);
    const int stage = ASYNC ? (ci & 1) : 0;
    if constexpr (ASYNC) {
      if (ci + 1 < n_chunks) fetch(c0 + GD_CHUNK, stage ^ 1);
      gd_cp_async_commit();                           // one group per pass, empty or not
      gd_cp_async_wait<1>();
    } else {
      __syncthreads();
      fetch(c0, 0);
    }
    __syncthreads();
    const float* vs_u = smem + stage * STAGE;
    const float* vs_v = vs_u + 5 * GD_CHUNK * DP;
    const float* vs_s = vs_v + GD_CHUNK * GD_COLS;
    // the sums over a lane's rows run as two chains each (even and odd rows), fixed whatever the step's shape; the
    // loop is unrolled so that the next tokens' vectors are on their way while this token's sums cross the lanes
#pragma unroll(R <= 8 ? 4 : (R <= 16 ? 2 : 1))
    for (int tt = 0; tt < cn; ++tt) {
      const float* base = vs_u + tt * DP + 4 * part;
      float A = 0.f, B = 0.f, A2 = 0.f, B2 = 0.f;
      float4 w4[R / 4], au4[R / 4], k4[R / 4];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 u = *reinterpret_cast<const float4*>(base + 4 * GD_LANES * j);
        const float4 rw = *reinterpret_cast<const float4*>(base + 2 * GD_CHUNK * DP + 4 * GD_LANES * j);
        au4[j] = *reinterpret_cast<const float4*>(base + GD_CHUNK * DP + 4 * GD_LANES * j);
        w4[j] = *reinterpret_cast<const float4*>(base + 3 * GD_CHUNK * DP + 4 * GD_LANES * j);
        k4[j] = *reinterpret_cast<const float4*>(base + 4 * GD_CHUNK * DP + 4 * GD_LANES * j);
        A = fmaf(u.x, S[4 * j], A);        B = fmaf(rw.x, S[4 * j], B);
        A2 = fmaf(u.y, S[4 * j + 1], A2);  B2 = fmaf(rw.y, S[4 * j + 1], B2);
        A = fmaf(u.z, S[4 * j + 2], A);    B = fmaf(rw.z, S[4 * j + 2], B);
        A2 = fmaf(u.w, S[4 * j + 3], A2);  B2 = fmaf(rw.w, S[4 * j + 3], B2);
      }
      A += A2;
      B += B2;
#pragma unroll
      for (int off = 1; off < GD_LANES; off <<= 1) {
        A += __shfl_xor_sync(0xffffffffu, A, off);
        B += __shfl_xor_sync(0xffffffffu, B, off);
      }
      const float vt = vs_v[tt * GD_COLS + cl];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        S[4 * j] = fmaf(k4[j].x, vt, fmaf(-au4[j].x, A, w4[j].x * S[4 * j]));
        S[4 * j + 1] = fmaf(k4[j].y, vt, fmaf(-au4[j].y, A, w4[j].y * S[4 * j + 1]));
        S[4 * j + 2] = fmaf(k4[j].z, vt, fmaf(-au4[j].z, A, w4[j].z * S[4 * j + 2]));
        S[4 * j + 3] = fmaf(k4[j].w, vt, fmaf(-au4[j].w, A, w4[j].w * S[4 * j + 3]));
      }
      if (live && part == 0)
        o_out[((size_t)(first + c0 + tt) * H + h) * d + col] = fmaf(vt, vs_s[tt * 2 + 1], fmaf(-A, vs_s[tt * 2], B));
    }
    if constexpr (ASYNC) __syncthreads();             // the stage is free for the fetch after next
  }
  if constexpr (ASYNC) gd_cp_async_wait<0>();
  if (live) {
#pragma unroll
    for (int j = 0; j < R / 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * (part + GD_LANES * j) + e;
        if (i < d) st[i] = S[4 * j + e];
      }
  }
}

// out [rows, cols] of type `dtype` = tanh(in), in fp32 with rows in_stride apart (the decay's inner projection).
NHV_API int nhv_general_delta_tanh(int dtype, void* out, const float* in, int in_stride, int rows, int cols,
                                   cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  NHV_REQUIRE(rows > 0 && cols > 0 && in_stride >= cols, "general_delta_tanh: bad sizes");
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (dtype == NHV_F32)
    nhv_launch(general_delta_tanh_kernel<float>, blocks, 256, 0, stream, (float*)out, in, in_stride, cols, total);
  else if (dtype == NHV_BF16)
    nhv_launch(general_delta_tanh_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, in, in_stride, cols, total);
  else
    NHV_REQUIRE(false, "general_delta_tanh: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("general_delta_tanh");
  return 0;
}

// o_out [T, H, d] fp32.  proj [T, >= 3 H d] (r, k, v) of type `dtype`; aw [T, >= H d] fp32 (the removal rate's
// projection); dec [T, H d] fp32 (the decay's projection W2 tanh(z)); a_bias, w0 [H d] of type `dtype`.
// Scratch given by the caller, all fp32: vec [5][T, H, d]; sc [T, H, 2]; v32 [T, H, d].
NHV_API int nhv_general_delta(int dtype, float* o_out, const void* proj, int proj_stride, const float* aw, int aw_stride,
                              const void* a_bias, const float* dec, const void* w0, float* state, long state_stride,
                              float* vec, float* sc, float* v32, const int* cu_q, const int* q_start, const int* slots,
                              int n_seqs, int n_tokens, int H, int d, float decay_floor, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(H > 0 && d > 0 && d <= GD_MAX_D, "general_delta: a head of %d channels is beyond the supported %d", d, GD_MAX_D);
  NHV_REQUIRE(proj_stride >= 3 * H * d && aw_stride >= H * d, "general_delta: rows too short for r, k, v / the rate");
  NHV_REQUIRE(state_stride >= (long)H * d * d, "general_delta: the state holds fewer than heads * d * d floats");
  const long items = (long)n_tokens * H;
  const int pblocks = (int)((items + GD_WARPS - 1) / GD_WARPS);
  if (dtype == NHV_F32)
    nhv_launch(general_delta_prepare_kernel<float>, pblocks, GD_WARPS * 32, 0, stream, vec, sc, v32, (const float*)proj,
               proj_stride, aw, aw_stride, (const float*)a_bias, dec, (const float*)w0, n_tokens, H, d, decay_floor);
  else if (dtype == NHV_BF16)
    nhv_launch(general_delta_prepare_kernel<__nv_bfloat16>, pblocks, GD_WARPS * 32, 0, stream, vec, sc, v32,
               (const __nv_bfloat16*)proj, proj_stride, aw, aw_stride, (const __nv_bfloat16*)a_bias, dec,
               (const __nv_bfloat16*)w0, n_tokens, H, d, decay_floor);
  else
    NHV_REQUIRE(false, "general_delta: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("general_delta_prepare");
  dim3 grid(n_seqs, H, (d + GD_COLS - 1) / GD_COLS);
  // cp.async wants 16-byte aligned sources: d a multiple of 4 and scratch that starts on such a boundary
  const bool async = d % 4 == 0 && (((uintptr_t)vec | (uintptr_t)sc | (uintptr_t)v32) & 15) == 0;
#define SCAN_AS(R, A)                                                                                               \
  do {                                                                                                              \
    const size_t smem = (size_t)(A ? 2 : 1) * (5 * GD_CHUNK * R * GD_LANES + GD_CHUNK * GD_COLS + GD_CHUNK * 2) *   \
                        sizeof(float);                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      NHV_CUDA(cudaFuncSetAttribute(general_delta_scan_kernel<R, A>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                    (int)smem), "general_delta");                                                   \
    nhv_launch(general_delta_scan_kernel<R, A>, grid, GD_THREADS, smem, stream, o_out, (const float*)vec,           \
               (const float*)sc, (const float*)v32, state, state_stride, cu_q, q_start, slots, n_tokens, H, d);     \
  } while (0)
#define SCAN(R)              \
  do {                       \
    if (async) SCAN_AS(R, true); \
    else SCAN_AS(R, false);  \
  } while (0)
  if (d <= 32) SCAN(4);
  else if (d <= 64) SCAN(8);
  else if (d <= 128) SCAN(16);
  else SCAN(32);
#undef SCAN
#undef SCAN_AS
  NHV_CHECK_LAUNCH("general_delta_scan");
  return 0;
}
