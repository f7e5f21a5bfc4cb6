// The experts' products of a mixture of experts over rows ordered by expert, in bfloat16 on the tensor cores
// (mma.sync m16n8k16, fp32 accumulators), with the experts' gated unit in the epilogue of the first product.
//
// Rows are those of moe_align (csrc/moe.cu): every tile of BM rows belongs to one expert (tile_expert), a row is a
// (token, choice) slot (sorted_slots) or padding (-1).  A block takes one tile of rows and a panel of output columns:
//   first:  act[row, c] = glu(x[token(row)] . Wg[e][c], x[token(row)] . Wu[e][c])   64 columns: 64 gate rows and the 64
//           up rows of the same columns lie in one 128-row tile of B, and a warp's fragments hold gate and up of the
//           same (row, column) in the same thread, so the unit is applied without leaving the registers;
//   second: y[row, c] = act[row] . Wd[e][c]                                          128 columns.
// A rows are gathered by token on their way into shared memory.  Operands travel by cp.async in a ring of three
// stages of 32 columns of K (small stages: several blocks fit an SM, and the tensor pipe needs many warps to stay
// busy); a row's sum over K runs in the same order wherever the row stands, so results do not depend on the
// ordering.  BM is 16 where experts see few rows (decoding: the kernel streams each expert's weights once), 64 or
// 128 (eight warps, each panel of weights read for twice the rows) for prompts.
#include <cuda_bf16.h>
#include <math.h>

#include "nhv_common.cuh"
#include "nhv_glu.cuh"

typedef __nv_bfloat16 bf16;

constexpr int MM_BK = 32;
constexpr int MM_LDS = MM_BK + 8;       // a row of a stage in shared memory, padded against bank conflicts
constexpr int MM_STAGES = 3;
constexpr int MM_BROWS = 128;

__device__ __forceinline__ void mm_cp_async16(void* smem, const void* gmem, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem),
               "r"(bytes));
}
__device__ __forceinline__ void mm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N_> __device__ __forceinline__ void mm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N_)); }

__device__ __forceinline__ void mm_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float mm_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int BM> struct MmShape {
  static constexpr int WM = BM >= 64 ? 64 : 16;        // rows per warp
  static constexpr int THREADS = (BM / WM) * 4 * 32;   // warps: BM / WM along the rows x 4 along the columns
};

template <int BM, bool FIRST>
__global__ void __launch_bounds__(MmShape<BM>::THREADS) moe_gemm_mma_kernel(
    bf16* __restrict__ out, const bf16* __restrict__ A, int lda, const bf16* __restrict__ W0, const bf16* __restrict__ W1,
    const int* __restrict__ sorted_slots, const int* __restrict__ tile_expert, int top, int N, int K, float limit,
    float alpha, float up_shift, const float* __restrict__ row_scale) {
  constexpr int MT = MmShape<BM>::WM / 16, MM_THREADS = MmShape<BM>::THREADS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* As = reinterpret_cast<bf16*>(smem_raw);              // [STAGES][BM][LDS]
  bf16* Bs = As + MM_STAGES * BM * MM_LDS;                   // [STAGES][BROWS][LDS]
  __shared__ int arow[BM];
  __shared__ float ascale[BM];                              // a factor on the expert's input, per row (1 without)
  pdl_prologue();
  // panels of one tile of rows are neighbours in the grid: they run together and share the tile's rows in L2
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.x * (FIRST ? 64 : 128);
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = (tid >> 5) & 3, row0 = (tid >> 7) * MmShape<BM>::WM;       // column quarter, first row of the warp
  if (tid < BM) {
    const int row = tile * BM + tid;
    const int slot = sorted_slots[row];
    arow[tid] = slot < 0 ? -1 : (FIRST ? slot / top : row);
    ascale[tid] = (FIRST && row_scale && slot >= 0) ? row_scale[slot] : 1.f;
  }
  __syncthreads();
  const bf16* w0 = W0 + (size_t)e * N * K;
  const bf16* w1 = FIRST ? W1 + (size_t)e * N * K : nullptr;
  const int KT = (K + MM_BK - 1) / MM_BK;

  auto load_stage = [&](int stage, int kt) {
    const int k0 = kt * MM_BK;
    constexpr int CH = MM_BK / 8;                              // 16-byte pieces of a row of a stage
    for (int i = tid; i < BM * CH; i += MM_THREADS) {
      const int r = i / CH, c = i % CH, k = k0 + c * 8;
      const int src = arow[r];
      const bool ok = src >= 0 && k < K;
      mm_cp_async16(As + ((size_t)stage * BM + r) * MM_LDS + c * 8, ok ? A + (size_t)src * lda + k : A, ok ? 16 : 0);
    }
    for (int i = tid; i < MM_BROWS * CH; i += MM_THREADS) {
      const int r = i / CH, c = i % CH, k = k0 + c * 8;
      const int n = FIRST ? n0 + (r & 63) : n0 + r;
      const bf16* base = (FIRST && r >= 64) ? w1 : w0;
      const bool ok = n < N && k < K;
      mm_cp_async16(Bs + ((size_t)stage * MM_BROWS + r) * MM_LDS + c * 8, ok ? base + (size_t)n * K + k : base, ok ? 16 : 0);
    }
  };

  float acc[MT][4][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][j][i] = 0.f;

#pragma unroll
  for (int s = 0; s < MM_STAGES - 1; ++s) {
    if (s < KT) load_stage(s, s);
    mm_commit();
  }
  // the rows of B that this warp's four column tiles read, two tiles (16 rows) per ldmatrix
  const int brow0 = FIRST ? warp * 16 : warp * 32;
  const int brow1 = FIRST ? 64 + warp * 16 : warp * 32 + 16;
  const int b_r = (lane & 7) + ((lane >> 4) << 3), b_k = ((lane >> 3) & 1) * 8;
  const int a_r = lane & 15, a_k = (lane >> 4) * 8;
  for (int kt = 0; kt < KT; ++kt) {
    mm_wait<MM_STAGES - 2>();
    __syncthreads();
    const int nxt = kt + MM_STAGES - 1;
    if (nxt < KT) load_stage(nxt % MM_STAGES, nxt);
    mm_commit();
    const bf16* as = As + (size_t)(kt % MM_STAGES) * BM * MM_LDS;
    const bf16* bs = Bs + (size_t)(kt % MM_STAGES) * MM_BROWS * MM_LDS;
#pragma unroll
    for (int kk = 0; kk < MM_BK / 16; ++kk) {
      uint32_t b[2][4];
      mm_ldmatrix_x4(b[0], bs + (size_t)(brow0 + b_r) * MM_LDS + kk * 16 + b_k);
      mm_ldmatrix_x4(b[1], bs + (size_t)(brow1 + b_r) * MM_LDS + kk * 16 + b_k);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        mm_ldmatrix_x4(a, as + (size_t)(row0 + mt * 16 + a_r) * MM_LDS + kk * 16 + a_k);
        mm_mma(acc[mt][0], a, b[0][0], b[0][1]);
        mm_mma(acc[mt][1], a, b[0][2], b[0][3]);
        mm_mma(acc[mt][2], a, b[1][0], b[1][1]);
        mm_mma(acc[mt][3], a, b[1][2], b[1][3]);
      }
    }
  }
  mm_wait<0>();

  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int lr = row0 + mt * 16 + g + 8 * half;
      if (arow[lr] < 0) continue;
      const float sc = ascale[lr];
      bf16* orow = out + ((size_t)tile * BM + lr) * N;
#pragma unroll
      for (int j = 0; j < (FIRST ? 2 : 4); ++j) {
        const int col = n0 + (FIRST ? warp * 16 : warp * 32) + j * 8 + 2 * tq;
        if (col >= N) continue;
        float v0, v1;
        if (FIRST) {
          // gate and up rounded to the storage type first, as a separate product would leave them
          v0 = nhv_glu(mm_round(sc * acc[mt][j][2 * half]), mm_round(sc * acc[mt][j + 2][2 * half]), limit, alpha, up_shift);
          v1 = nhv_glu(mm_round(sc * acc[mt][j][2 * half + 1]), mm_round(sc * acc[mt][j + 2][2 * half + 1]), limit, alpha, up_shift);
        } else {
          v0 = acc[mt][j][2 * half];
          v1 = acc[mt][j][2 * half + 1];
        }
        if (col + 1 < N) *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(v0, v1);
        else orow[col] = __float2bfloat16_rn(v0);
      }
    }
  }
}

template <int BM>
static size_t mm_smem_bytes() { return (size_t)MM_STAGES * (BM + MM_BROWS) * MM_LDS * sizeof(bf16); }

// tile: 16, 64 or 128, the row tile that moe_align was called with.  first != 0: out [rows, N] = glu over x [T, K] gathered
// by sorted_slots, W0 / W1 [E, N, K]; first == 0: out [rows, N] = a [rows, K] times W0 [E, N, K].
NHV_API int nhv_moe_gemm_mma(int tile, int first, void* out, const void* A, int lda, const void* W0, const void* W1,
                             const int* sorted_slots, const int* tile_expert, int max_tiles, int top, int N, int K,
                             float limit, float alpha, float up_shift, const float* row_scale, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  NHV_REQUIRE(tile == 16 || tile == 64 || tile == 128, "moe_gemm (mma): the row tile is 16, 64 or 128, not %d", tile);
  NHV_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && top > 0, "moe_gemm (mma): bad sizes");
  NHV_REQUIRE(K % 8 == 0 && lda % 8 == 0 && N % 2 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W0 % 16) == 0 &&
                  (!first || ((uintptr_t)W1 % 16) == 0) && ((uintptr_t)out % 4) == 0,
              "moe_gemm (mma): rows of A and of the weights must start on 16-byte boundaries (K %d, lda %d)", K, lda);
  dim3 grid((N + (first ? 64 : 128) - 1) / (first ? 64 : 128), max_tiles);
  NHV_REQUIRE(grid.y <= 65535, "moe_gemm (mma): %d tiles of rows are beyond the grid's reach", max_tiles);
#define GO(BM, F)                                                                                                     \
  do {                                                                                                                \
    static bool attr = false;                                                                                         \
    if (!attr) {                                                                                                      \
      NHV_CUDA(cudaFuncSetAttribute(moe_gemm_mma_kernel<BM, F>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                    (int)mm_smem_bytes<BM>()), "moe_gemm (mma)");                                     \
      attr = true;                                                                                                    \
    }                                                                                                                 \
    nhv_launch(moe_gemm_mma_kernel<BM, F>, grid, MmShape<BM>::THREADS, mm_smem_bytes<BM>(), stream, (bf16*)out, (const bf16*)A, \
               lda, (const bf16*)W0, (const bf16*)W1, sorted_slots, tile_expert, top, N, K, limit, alpha, up_shift,   \
               row_scale);                                                                                            \
  } while (0)
  if (tile == 16) { if (first) GO(16, true); else GO(16, false); }
  else if (tile == 64) { if (first) GO(64, true); else GO(64, false); }
  else { if (first) GO(128, true); else GO(128, false); }
#undef GO
  NHV_CHECK_LAUNCH("moe_gemm (mma)");
  return 0;
}
