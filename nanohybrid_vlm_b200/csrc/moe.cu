// Mixture of experts: the router, the ordering of (token, choice) slots by expert, the experts' products over that
// order for any storage type, and the weighted sum that brings the choices of a token together again.
//
//   moe_route     per token, from fp32 router logits z over N outputs (experts, then identity experts):
//                 s = softmax(z); choice score c = s + correction; the outputs form n_groups equal groups of
//                 neighbours, a group's score is its largest c, and only outputs of the `keep` best groups can be
//                 chosen (the others count as -inf); the `top` outputs with the largest c are chosen; their weights
//                 are their s, divided by the sum of the chosen s (+ 1e-20).  One warp per token, all in fp32.
//                 sigmoid_scores: s = sigmoid(z) instead of the softmax; renorm 0: the weights are the chosen s as
//                 they are.
//   moe_align     slots (t, k) whose choice is a real expert are grouped by expert; each expert's run is padded to
//                 a multiple of the row tile, so that a tile of rows has one expert.  Writes sorted_slots (slot per
//                 row, -1 for padding), slot_pos (row per slot, -1 for identity choices) and tile_expert.
//   moe_gemm      (any type, CUDA cores, fixed order of summation over k) the products over the sorted rows:
//                 first: act[row] = glu(x[token(row)] Wg[e]^T, x[token(row)] Wu[e]^T), second: y[row] = act[row] Wd[e]^T.
//                 row_scale [slots] (optional): a factor on the expert's input, one per (token, choice) slot; it is
//                 applied to both first products' fp32 sums, which equals scaling the input.
//   moe_combine   out[t] = sum_k w[t,k] * (choice is an expert ? y[row(t,k)] : x[t]) + sigmoid(sg[t]) * shared[t];
//                 without weights every choice counts fully (the weights went into the experts' inputs).
//
// A row's result does not depend on where in its expert's run it stands, so the order in which moe_align hands out
// rows (atomics) does not show in the numbers.
#include <math.h>

#include "nhv_common.cuh"
#include "nhv_vec8.cuh"

// ---------------------------------------------------------------- router
constexpr int MR_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
}

__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(
    int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits, int ld,
    const float* __restrict__ correction, int n_tokens, int N, int n_groups, int keep, int top, int sigmoid_scores,
    int renorm) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * MR_WARPS + warp;
  if (t >= n_tokens) return;
  float* s = smem + (size_t)warp * 3 * N;    // scores
  float* c = s + N;                          // choice scores
  float* gs = c + N;                         // group scores
  const float* z = logits + (size_t)t * ld;
  if (sigmoid_scores) {
    for (int j = lane; j < N; j += 32) {
      const float v = 1.0f / (1.0f + expf(-z[j]));
      s[j] = v;
      c[j] = v + (correction ? correction[j] : 0.f);
    }
  } else {
    float mx = -INFINITY;
    for (int j = lane; j < N; j += 32) mx = fmaxf(mx, z[j]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = lane; j < N; j += 32) {
      const float e = expf(z[j] - mx);
      s[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int j = lane; j < N; j += 32) {
      const float v = s[j] / sum;
      s[j] = v;
      c[j] = v + (correction ? correction[j] : 0.f);
    }
  }
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int gsz = N / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float best = -INFINITY;
      for (int j = 0; j < gsz; ++j) best = fmaxf(best, c[g * gsz + j]);
      gs[g] = best;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      if (lane == 0 && bi < n_groups) gs[bi] = INFINITY;       // +inf marks a kept group
      __syncwarp();
    }
    for (int j = lane; j < N; j += 32)
      if (gs[j / gsz] != INFINITY) c[j] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = lane; j < N; j += 32) {
      const float v = c[j];
      if (v > bv || (v == bv && j < bi)) { bv = v; bi = j; }
    }
    warp_argmax(bv, bi);
    if (bi >= N) bi = 0;                                       // nothing left to choose: a configuration fault
    const float w = s[bi];
    wsum += w;
    if (lane == 0) {
      ids[(size_t)t * top + r] = bi;
      weights[(size_t)t * top + r] = w;
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (!renorm) return;
  const float inv = 1.0f / (wsum + 1e-20f);
  for (int r = lane; r < top; r += 32) weights[(size_t)t * top + r] *= inv;
}

NHV_API int nhv_moe_route(int* ids, float* weights, const float* logits, int ld, const float* correction, int n_tokens, int N,
                          int n_groups, int keep, int top, int sigmoid_scores, int renorm, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(N > 0 && N <= 4096 && top > 0 && top <= N && ld >= N, "moe_route: bad sizes (N %d, top %d)", N, top);
  NHV_REQUIRE(n_groups > 0 && N % n_groups == 0 && keep > 0 && keep <= n_groups,
              "moe_route: %d outputs do not form %d equal groups of which %d are kept", N, n_groups, keep);
  NHV_REQUIRE((long)keep * (N / n_groups) >= top, "moe_route: the kept groups hold fewer than top = %d outputs", top);
  const size_t smem = (size_t)MR_WARPS * 3 * N * sizeof(float);
  if (smem > 48 * 1024)
    NHV_CUDA(cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "moe_route");
  nhv_launch(moe_route_kernel, (n_tokens + MR_WARPS - 1) / MR_WARPS, MR_WARPS * 32, smem, stream, ids, weights, logits, ld,
             correction, n_tokens, N, n_groups, keep, top, sigmoid_scores, renorm);
  NHV_CHECK_LAUNCH("moe_route");
  return 0;
}

// ---------------------------------------------------------------- order by expert
constexpr int MA_THREADS = 1024;
constexpr int MA_MAX_EXPERTS = 2048;

__global__ void __launch_bounds__(MA_THREADS) moe_align_kernel(
    const int* __restrict__ ids, int n_slots, int E, int BM, int cap, int max_tiles, int* __restrict__ sorted_slots,
    int* __restrict__ slot_pos, int* __restrict__ tile_expert) {
  __shared__ int count[MA_MAX_EXPERTS];
  __shared__ int start[MA_MAX_EXPERTS + 1];
  pdl_prologue();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += MA_THREADS) count[e] = 0;
  for (int i = tid; i < cap; i += MA_THREADS) sorted_slots[i] = -1;
  for (int i = tid; i < max_tiles; i += MA_THREADS) tile_expert[i] = -1;
  __syncthreads();
  for (int i = tid; i < n_slots; i += MA_THREADS) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      at += (count[e] + BM - 1) / BM * BM;
    }
    start[E] = at;
  }
  __syncthreads();
  for (int e = tid; e < E; e += MA_THREADS) {
    for (int r = start[e]; r < start[e + 1]; r += BM) tile_expert[r / BM] = e;
    count[e] = 0;                                              // now the cursor of the expert's run
  }
  __syncthreads();
  for (int i = tid; i < n_slots; i += MA_THREADS) {
    const int e = ids[i];
    int pos = -1;
    if (e >= 0 && e < E) {
      pos = start[e] + atomicAdd(&count[e], 1);
      sorted_slots[pos] = i;
    }
    slot_pos[i] = pos;
  }
}

// Rows that the ordering can need: every slot, and up to BM - 1 rows of padding for each expert that can be hit.
NHV_API int nhv_moe_sorted_rows(int n_slots, int E, int BM) {
  const int hit = n_slots < E ? n_slots : E;
  const long rows = (long)n_slots + (long)hit * (BM - 1);
  return (int)((rows + BM - 1) / BM * BM);
}

NHV_API int nhv_moe_align(const int* ids, int n_slots, int E, int BM, int* sorted_slots, int* slot_pos, int* tile_expert,
                          cudaStream_t stream) {
  if (n_slots == 0) return 0;
  NHV_REQUIRE(E > 0 && E <= MA_MAX_EXPERTS && BM > 0, "moe_align: %d experts are beyond the supported %d", E, MA_MAX_EXPERTS);
  const int cap = nhv_moe_sorted_rows(n_slots, E, BM);
  nhv_launch(moe_align_kernel, 1, MA_THREADS, 0, stream, ids, n_slots, E, BM, cap, cap / BM, sorted_slots, slot_pos,
             tile_expert);
  NHV_CHECK_LAUNCH("moe_align");
  return 0;
}

// ---------------------------------------------------------------- the experts' products, any type
constexpr int MG_BM = 16;
constexpr int MG_BN = 64;
constexpr int MG_BK = 32;

#include "nhv_glu.cuh"


// FIRST: A rows are x[sorted_slots[row] / top], B = (Wg[e], Wu[e]) [N, K] each, out = glu.  Else: A rows are
// a[row], B = Wd[e] [N, K].  256 threads: thread (ty, tx) has rows ty * 4 .. + 3 of column tx.
template <typename T, bool FIRST>
__global__ void __launch_bounds__(256) moe_gemm_simt_kernel(
    T* __restrict__ out, const T* __restrict__ A, int lda, const T* __restrict__ W0, const T* __restrict__ W1,
    const int* __restrict__ sorted_slots, const int* __restrict__ tile_expert, int top, int N, int K, float limit,
    float alpha, float up_shift, const float* __restrict__ row_scale) {
  __shared__ float As[MG_BM][MG_BK + 1];
  __shared__ float ascale[MG_BM];
  __shared__ float B0[MG_BN][MG_BK + 1];
  __shared__ float B1[FIRST ? MG_BN : 1][MG_BK + 1];
  __shared__ int arow[MG_BM];
  pdl_prologue();
  const int tile = blockIdx.x, n0 = blockIdx.y * MG_BN;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int tid = threadIdx.x, tx = tid % MG_BN, ty = tid / MG_BN;
  if (tid < MG_BM) {
    const int row = tile * MG_BM + tid;
    const int slot = sorted_slots[row];
    arow[tid] = slot < 0 ? -1 : (FIRST ? slot / top : row);
    ascale[tid] = (FIRST && row_scale && slot >= 0) ? row_scale[slot] : 1.f;
  }
  __syncthreads();
  const T* w0 = W0 + (size_t)e * N * K;
  const T* w1 = FIRST ? W1 + (size_t)e * N * K : nullptr;
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    for (int i = tid; i < MG_BM * MG_BK; i += 256) {
      const int r = i / MG_BK, c = i - r * MG_BK;
      const int src = arow[r];
      As[r][c] = (src >= 0 && k0 + c < K) ? to_f32<T>(A[(size_t)src * lda + k0 + c]) : 0.f;
    }
    for (int i = tid; i < MG_BN * MG_BK; i += 256) {
      const int r = i / MG_BK, c = i - r * MG_BK;
      const bool ok = n0 + r < N && k0 + c < K;
      B0[r][c] = ok ? to_f32<T>(w0[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
      if (FIRST) B1[r][c] = ok ? to_f32<T>(w1[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < MG_BK; ++c) {
      const float b0 = B0[tx][c];
      const float b1 = FIRST ? B1[tx][c] : 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float a = As[ty * 4 + r][c];
        acc0[r] = fmaf(a, b0, acc0[r]);
        if (FIRST) acc1[r] = fmaf(a, b1, acc1[r]);
      }
    }
    __syncthreads();
  }
  if (n0 + tx >= N) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int lr = ty * 4 + r;
    if (arow[lr] < 0) continue;
    const size_t row = (size_t)tile * MG_BM + lr;
    // the storage type's rounding of gate and up comes first, as a separate product would leave it
    const float sc = ascale[lr];          // a factor on the expert's input is a factor on both first products
    const float v = FIRST ? nhv_glu(round_to<T>(sc * acc0[r]), round_to<T>(sc * acc1[r]), limit, alpha, up_shift) : acc0[r];
    out[row * N + n0 + tx] = from_f32<T>(v);
  }
}

NHV_API int nhv_moe_simt_tile() { return MG_BM; }

// first != 0: out [rows, N] = glu over x [T, K] gathered by sorted_slots, W0 / W1 [E, N, K].  first == 0: out [rows, N]
// = a [rows, K] times W0 [E, N, K].  max_tiles: the tiles of the ordering (rows / tile).
NHV_API int nhv_moe_gemm_simt(int dtype, int first, void* out, const void* A, int lda, const void* W0, const void* W1,
                              const int* sorted_slots, const int* tile_expert, int max_tiles, int top, int N, int K,
                              float limit, float alpha, float up_shift, const float* row_scale, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  NHV_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && top > 0, "moe_gemm: bad sizes");
  dim3 grid(max_tiles, (N + MG_BN - 1) / MG_BN);
  NHV_REQUIRE(grid.y <= 65535, "moe_gemm: %d output columns are beyond the grid's reach", N);
#define GO(T, F)                                                                                                 \
  nhv_launch(moe_gemm_simt_kernel<T, F>, grid, 256, 0, stream, (T*)out, (const T*)A, lda, (const T*)W0, (const T*)W1, \
             sorted_slots, tile_expert, top, N, K, limit, alpha, up_shift, row_scale)
  if (dtype == NHV_F32) { if (first) GO(float, true); else GO(float, false); }
  else if (dtype == NHV_BF16) { if (first) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else NHV_REQUIRE(false, "moe_gemm: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("moe_gemm");
  return 0;
}

// ---------------------------------------------------------------- the weighted sum
// VEC: eight columns per thread and step (width in steps of 8, rows on 16-byte boundaries); the sums run in the same
// order either way.
template <typename T, bool VEC>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const T* __restrict__ x,
                                   const T* __restrict__ shared, const float* __restrict__ shared_gate, int gate_stride,
                                   const int* __restrict__ ids, const float* __restrict__ weights,
                                   const int* __restrict__ slot_pos, int top, int E, int width) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int t = blockIdx.x;
  float* w = smem;                            // [top]
  int* pos = reinterpret_cast<int*>(smem + top);
  for (int k = threadIdx.x; k < top; k += blockDim.x) {
    w[k] = weights ? weights[(size_t)t * top + k] : 1.f;
    const int e = ids[(size_t)t * top + k];
    pos[k] = e < E ? slot_pos[(size_t)t * top + k] : -2;      // -2: an identity expert
  }
  __syncthreads();
  float sg = 0.f;
  if (shared) sg = shared_gate ? 1.0f / (1.0f + expf(-shared_gate[(size_t)t * gate_stride])) : 1.0f;
  if constexpr (VEC) {
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, xv[8], v[8];
      nhv_load8(xv, x + (size_t)t * width + c);
      for (int k = 0; k < top; ++k) {
        const int p = pos[k];
        if (p >= 0) {
          nhv_load8(v, y + (size_t)p * width + c);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[k], v[i], acc[i]);
        } else if (p == -2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[k], xv[i], acc[i]);
        }
      }
      if (shared) {
        nhv_load8(v, shared + (size_t)t * width + c);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(sg, v[i], acc[i]);
      }
      nhv_store8(out + (size_t)t * width + c, acc);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float acc = 0.f;
      const float xv = to_f32<T>(x[(size_t)t * width + c]);
      for (int k = 0; k < top; ++k) {
        const int p = pos[k];
        if (p >= 0) acc = fmaf(w[k], to_f32<T>(y[(size_t)p * width + c]), acc);
        else if (p == -2) acc = fmaf(w[k], xv, acc);
      }
      if (shared) acc = fmaf(sg, to_f32<T>(shared[(size_t)t * width + c]), acc);
      out[(size_t)t * width + c] = from_f32<T>(acc);
    }
  }
}

NHV_API int nhv_moe_combine(int dtype, void* out, const void* y, const void* x, const void* shared, const float* shared_gate,
                            int gate_stride, const int* ids, const float* weights, const int* slot_pos, int n_tokens,
                            int top, int E, int width, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(top > 0 && top <= 1024 && width > 0, "moe_combine: bad sizes");
  const bool vec = width % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)x % 16) == 0 &&
                   ((uintptr_t)shared % 16) == 0;
  const int threads = vec ? (width >= 2048 ? 256 : 128) : (width >= 1024 ? 256 : 128);
  const size_t smem = (size_t)top * 8;
#define GO(T, V)                                                                                                 \
  nhv_launch(moe_combine_kernel<T, V>, n_tokens, threads, smem, stream, (T*)out, (const T*)y, (const T*)x, (const T*)shared, \
             shared_gate, gate_stride, ids, weights, slot_pos, top, E, width)
  if (dtype == NHV_F32) { if (vec) GO(float, true); else GO(float, false); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else NHV_REQUIRE(false, "moe_combine: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("moe_combine");
  return 0;
}
