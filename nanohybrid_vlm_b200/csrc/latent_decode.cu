// Attention over one latent per token for steps of few tokens (decoding), bfloat16, on the tensor cores (mma.sync).
//
// A cache row holds a token's latent [rank] and the rotated key part [dr]; the row is the key of every head and its
// leading `rank` elements are the value of every head.  A query is [row] per head (the key expansion folded into it
// beforehand) and the result is a weighted sum of latents per head, [rank], which the caller expands into values.
//
// The heads of one token are the 16 rows of an mma tile, so the keys of a request are read once for up to 16 heads.
// The keys a token sees are cut into `n_splits` runs of whole tiles of 64 keys; block (split, token, group of 16
// heads) writes an unnormalised partial sum with its running maximum and denominator, and a second kernel merges the
// partial sums of a token and head, where the sink (exp(sink) in the denominator, once) joins.  The cutting depends
// on the token's position and on `n_splits` only.
//
// Block: 16 warps.  Q.K^T: warps w and w + 8 own keys 8 w .. 8 w + 7 of a tile, all 16 heads, each one half of the
// row's elements in steps of 16 (even and odd steps in two chains of products); the upper warp hands its partial
// scores to the lower one through shared memory.  The running maximum is shared through shared memory; P goes to
// shared memory as bfloat16; P.V: warp w owns a sixteenth of the latent's columns (NT tiles of 8), all 64 keys.  Tiles arrive by cp.async, the next while this one is
// worked on.  Shared-memory rows are round_up(row, 16) + 8 elements, an odd number of 16-byte chunks, so that ldmatrix
// meets no bank conflicts; what no copy writes stays zero.
#include <cuda_bf16.h>
#include <math.h>

#include "nhv_common.cuh"

typedef __nv_bfloat16 bf16;

constexpr int LD_BN = 64;            // keys per tile
constexpr int LD_THREADS = 512;
constexpr int LD_WARPS = LD_THREADS / 32;
constexpr int LD_KG = LD_BN / 8;       // groups of 8 keys in a tile
constexpr int LD_PS = LD_BN + 8;     // a row of P in shared memory
constexpr float LD_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void ld_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ld_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void ld_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ld_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ld_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ld_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ld_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// NT: tiles of 8 latent columns per warp (an even number; 16 NT 8 >= rank).
template <int NT>
__global__ void __launch_bounds__(LD_THREADS, 1) latent_decode_kernel(
    float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q, int q_stride,
    const bf16* __restrict__ pages, const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
    const int* __restrict__ kv_len, int n_seqs, int H, int rank, int row, int page_size, int n_pages, float scale) {
  extern __shared__ __align__(16) unsigned char ld_smem[];
  pdl_prologue();
  const int split = blockIdx.x, n_splits = gridDim.x, tok = blockIdx.y, h0 = blockIdx.z * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int RS = (row + 15) / 16 * 16 + 8;              // elements of a row in shared memory
  const int ksteps = (row + 15) / 16;
  bf16* Qs = reinterpret_cast<bf16*>(ld_smem);          // [16][RS]
  bf16* Ks = Qs + 16 * RS;                              // [2][64][RS]
  bf16* Ps = Ks + 2 * LD_BN * RS;                       // [16][LD_PS]
  float* red = reinterpret_cast<float*>(Ps + 16 * LD_PS);   // [16][16]
  float4* sred = reinterpret_cast<float4*>(red + LD_WARPS * 16);   // [8][32]: partial scores of the upper warps

  // the request of this token and the token's position
  int seq = 0;
  while (seq + 1 < n_seqs && cu_q[seq + 1] <= tok) ++seq;
  const int pos = kv_len[seq] - (cu_q[seq + 1] - tok);  // it sees keys 0 .. pos
  const int tiles_total = pos / LD_BN + 1;
  const int per = (tiles_total + n_splits - 1) / n_splits;
  const int tile0 = split * per, tile1 = min(tile0 + per, tiles_total);
  const size_t part = ((size_t)tok * H) * n_splits + split;     // + h * n_splits
  if (tile0 >= tile1 || pos < 0) {                      // nothing for this block: a partial sum that weighs nothing
    for (int r = tid; r < 16 && h0 + r < H; r += LD_THREADS) {
      part_ml[(part + (size_t)(h0 + r) * n_splits) * 2] = -INFINITY;
      part_ml[(part + (size_t)(h0 + r) * n_splits) * 2 + 1] = 0.f;
    }
    return;
  }
  {                                                     // zeros where no copy writes (padding behind a row, heads past H)
    uint4* z = reinterpret_cast<uint4*>(ld_smem);
    const int n16 = ((16 + 2 * LD_BN) * RS + 16 * LD_PS) * (int)sizeof(bf16) / 16;
    for (int i = tid; i < n16; i += LD_THREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const int cpr = row >> 3;                             // 16-byte chunks of a row
  const int* table = block_table + (size_t)seq * bt_stride;
  auto fetch = [&](int tile, int stage) {
    bf16* dst = Ks + (size_t)stage * LD_BN * RS;
    int mine = -1;                                      // lane i looks up the page of key warp + 16 i
    {
      const int j = tile * LD_BN + warp + LD_WARPS * (lane % (LD_BN / LD_WARPS));
      if (j <= pos) mine = table[j / page_size];
    }
#pragma unroll
    for (int i = 0; i < LD_BN / LD_WARPS; ++i) {
      const int kk = warp + LD_WARPS * i, j = tile * LD_BN + kk;
      bf16* d = dst + kk * RS;
      const int page = __shfl_sync(0xffffffffu, mine, i);
      if (page >= 0 && page < n_pages) {
        const bf16* src = pages + ((size_t)page * page_size + j % page_size) * row;
        for (int c = lane; c < cpr; c += 32) ld_cp_async16(d + 8 * c, src + 8 * c);
      } else {                                          // a key the token does not see: its value must not be stale memory
        for (int c = lane; c < cpr; c += 32) *reinterpret_cast<uint4*>(d + 8 * c) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  fetch(tile0, 0);
  for (int r = warp; r < 16; r += LD_WARPS)             // the queries of 16 heads
    if (h0 + r < H) {
      const bf16* src = q + (size_t)tok * q_stride + (size_t)(h0 + r) * row;
      for (int c = lane; c < cpr; c += 32) ld_cp_async16(Qs + r * RS + 8 * c, src + 8 * c);
    }
  ld_cp_async_commit();

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};      // rows g and g + 8
  const float sc2 = scale * LD_LOG2E;
  const int ntw = (((rank >> 3) + LD_WARPS - 1) / LD_WARPS + 1) & ~1;   // tiles of 8 columns per warp, even
  const int kg = warp & (LD_KG - 1);                    // this warp's group of 8 keys in Q.K^T
  const bool upper = warp >= LD_KG;                     // the warp with the upper half of the row's steps
  const int ksplit = (ksteps + 3) / 4 * 2;              // an even number of steps for the lower warp
  const int col_base = warp * ntw * 8;

  for (int tile = tile0; tile < tile1; ++tile) {
    const int stage = (tile - tile0) & 1;
    ld_cp_async_wait<0>();
    __syncthreads();                                    // the tile is here; the other stage and P are free
    if (tile + 1 < tile1) fetch(tile + 1, stage ^ 1);
    ld_cp_async_commit();
    const bf16* Kt = Ks + (size_t)stage * LD_BN * RS;
    // scores of 16 heads x this warp's 8 keys over its half of the steps; one load of the keys serves two steps
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      float s2[4] = {0.f, 0.f, 0.f, 0.f};
      const bf16* qa = Qs + (lane & 15) * RS + (lane >> 4) * 8;
      const bf16* kb = Kt + (kg * 8 + (lane & 7)) * RS + (lane >> 3) * 8;
      const int ks0 = upper ? ksplit : 0, ks1 = upper ? ksteps : min(ksplit, ksteps);
      for (int ks = ks0; ks < ks1; ks += 2) {
        uint32_t a[4], b[4];
        ld_ldmatrix_x4(b, kb + ks * 16);                // behind an odd last step it reads on into memory that is not used
        ld_ldmatrix_x4(a, qa + ks * 16);
        ld_mma(s, a, b[0], b[1]);
        if (ks + 1 < ksteps) {
          ld_ldmatrix_x4(a, qa + ks * 16 + 16);
          ld_mma(s2, a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) s[e] += s2[e];
    }
    if (upper) sred[kg * 32 + lane] = make_float4(s[0], s[1], s[2], s[3]);
    __syncthreads();
    float mx[2] = {-INFINITY, -INFINITY};
    if (!upper) {
      const float4 other = sred[kg * 32 + lane];
      s[0] += other.x; s[1] += other.y; s[2] += other.z; s[3] += other.w;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = tile * LD_BN + kg * 8 + 2 * t4 + (e & 1);
        s[e] = j <= pos ? s[e] * sc2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[e]);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if (t4 == 0 && !upper) {
      red[kg * 16 + g] = mx[0];
      red[kg * 16 + g + 8] = mx[1];
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rr = g + 8 * r;
      float m_new = m_run[r];
#pragma unroll
      for (int w = 0; w < LD_KG; ++w) m_new = fmaxf(m_new, red[w * 16 + rr]);
      alpha[r] = exp2f(m_run[r] - m_new);               // the first tile has a key that is seen: m_new is finite
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
    if (!upper) {
      const float p0 = exp2f(s[0] - m_run[0]), p1 = exp2f(s[1] - m_run[0]);
      const float p2 = exp2f(s[2] - m_run[1]), p3 = exp2f(s[3] - m_run[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      const int c = kg * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(Ps + g * LD_PS + c) = ld_pack(p0, p1);
      *reinterpret_cast<uint32_t*>(Ps + (g + 8) * LD_PS + c) = ld_pack(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    __syncthreads();
    // weighted sum of the tile's latents: this warp's columns, all 64 keys
    {
      const bf16* pa = Ps + (lane & 15) * LD_PS + (lane >> 4) * 8;
      const bf16* vb = Kt + (lane & 15) * RS + (lane >> 4) * 8 + col_base;
#pragma unroll
      for (int kk = 0; kk < LD_BN / 16; ++kk) {
        uint32_t a[4];
        ld_ldmatrix_x4(a, pa + kk * 16);
#pragma unroll
        for (int i = 0; i < NT; i += 2) {
          if (i < ntw && col_base + i * 8 < rank) {
            uint32_t b[4];
            ld_ldmatrix_x4_trans(b, vb + (size_t)kk * 16 * RS + i * 8);
            ld_mma(o[i], a, b[0], b[1]);
            ld_mma(o[i + 1], a, b[2], b[3]);
          }
        }
      }
    }
  }
  ld_cp_async_wait<0>();
  // the denominators: over the quad, then over the warps
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __syncthreads();
  if (t4 == 0) {
    red[warp * 16 + g] = l_run[0];
    red[warp * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
  if (tid < 16 && h0 + tid < H) {
    const size_t at = (part + (size_t)(h0 + tid) * n_splits) * 2;
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < LD_WARPS; ++w) l += red[w * 16 + tid];
    part_ml[at + 1] = l;
  }
  if (warp == 0 && t4 == 0) {                           // every thread holds the maxima of its two rows
#pragma unroll
    for (int r = 0; r < 2; ++r)
      if (h0 + g + 8 * r < H) part_ml[(part + (size_t)(h0 + g + 8 * r) * n_splits) * 2] = m_run[r];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int c = col_base + i * 8 + 2 * t4;
    if (i < ntw && c < rank) {
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (h0 + g + 8 * r < H) {
          float* dst = part_o + (part + (size_t)(h0 + g + 8 * r) * n_splits) * rank + c;
          *reinterpret_cast<float2*>(dst) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
        }
    }
  }
}

// out[tok, h, :] = sum over splits of part_o * 2^(m - M) / (sum of l * 2^(m - M) + 2^(sink - M)); one block per (tok, h).
__global__ void latent_decode_merge_kernel(bf16* __restrict__ out, int out_stride, const float* __restrict__ part_o,
                                           const float* __restrict__ part_ml, const float* __restrict__ sinks, int H,
                                           int rank, int n_splits) {
  pdl_prologue();
  const int tok = blockIdx.x / H, h = blockIdx.x % H;
  const size_t base = ((size_t)tok * H + h) * n_splits;
  float M = sinks ? sinks[h] * LD_LOG2E : -INFINITY;
  for (int i = 0; i < n_splits; ++i)
    if (part_ml[(base + i) * 2 + 1] > 0.f) M = fmaxf(M, part_ml[(base + i) * 2]);
  float L = sinks ? exp2f(sinks[h] * LD_LOG2E - M) : 0.f;
  for (int i = 0; i < n_splits; ++i) {
    const float l = part_ml[(base + i) * 2 + 1];
    if (l > 0.f) L += l * exp2f(part_ml[(base + i) * 2] - M);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float l = part_ml[(base + i) * 2 + 1];
      if (l > 0.f) acc = fmaf(part_o[(base + i) * rank + c], exp2f(part_ml[(base + i) * 2] - M), acc);
    }
    out[(size_t)tok * out_stride + (size_t)h * rank + c] = __float2bfloat16_rn(acc * inv);
  }
}

NHV_API int nhv_latent_decode_supports(int H, int rank, int row) {
  const int RS = (row + 15) / 16 * 16 + 8;
  const size_t smem = (size_t)((16 + 2 * LD_BN) * RS + 16 * LD_PS) * sizeof(bf16) + (LD_WARPS * 16 + LD_KG * 32 * 4) * sizeof(float);
  return H > 0 && rank > 0 && rank % 8 == 0 && row % 8 == 0 && row >= rank && rank <= 512 && smem <= 227 * 1024;
}

// part_o: [T, H, n_splits, rank] floats, part_ml: [T, H, n_splits, 2] floats (scratch).  q: [T, H, row] with rows
// q_stride apart; out: [T, H, rank] with rows out_stride apart.
NHV_API int nhv_latent_decode(void* out, int out_stride, const void* q, int q_stride, const void* pages,
                              const int* block_table, int bt_stride, const int* cu_q, const int* kv_len, int n_seqs,
                              int n_tokens, int H, int rank, int row, int page_size, int n_pages, float scale,
                              const float* sinks, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(nhv_latent_decode_supports(H, rank, row), "latent_decode: %d heads, a latent of %d in rows of %d: not taken", H, rank, row);
  NHV_REQUIRE(n_splits > 0 && page_size > 0 && n_pages > 0 && bt_stride > 0 && q_stride % 8 == 0 &&
              ((uintptr_t)q & 15) == 0 && ((uintptr_t)pages & 15) == 0, "latent_decode: bad geometry or alignment");
  const int RS = (row + 15) / 16 * 16 + 8;
  const size_t smem = (size_t)((16 + 2 * LD_BN) * RS + 16 * LD_PS) * sizeof(bf16) + (LD_WARPS * 16 + LD_KG * 32 * 4) * sizeof(float);
  dim3 grid(n_splits, n_tokens, (H + 15) / 16);
#define LAUNCH(NT)                                                                                                   \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      NHV_CUDA(cudaFuncSetAttribute(latent_decode_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), \
               "latent_decode");                                                                                     \
    nhv_launch(latent_decode_kernel<NT>, grid, LD_THREADS, smem, stream, part_o, part_ml, (const bf16*)q, q_stride,  \
               (const bf16*)pages, block_table, bt_stride, cu_q, kv_len, n_seqs, H, rank, row, page_size, n_pages,   \
               scale);                                                                                               \
  } while (0)
  const int ntw = (((rank >> 3) + LD_WARPS - 1) / LD_WARPS + 1) & ~1;
  if (ntw <= 2) LAUNCH(2);
  else LAUNCH(4);
#undef LAUNCH
  NHV_CHECK_LAUNCH("latent_decode");
  nhv_launch(latent_decode_merge_kernel, dim3(n_tokens * H), dim3(128), 0, stream, (bf16*)out, out_stride,
             (const float*)part_o, (const float*)part_ml, sinks, H, rank, n_splits);
  NHV_CHECK_LAUNCH("latent_decode_merge");
  return 0;
}
