// The experts' products of a mixture of experts over rows ordered by expert, for prompts, on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory, operands brought by TMA.
//
// Rows are those of moe_align (csrc/moe.cu) with tiles of 128 rows: every tile belongs to one expert.  A block takes
// one tile of rows and a panel of 128 rows of that expert's weights.  The weights sit on the MMA's M axis, the tile's
// 128 rows on its N axis, so D [128 x 128] (fp32) fills 128 columns of tensor memory, one weight row per lane.
//   first:  the panel is 64 rows of the gate matrix and the 64 rows of the up matrix of the same output columns;
//           act[row, c] = glu(gate, up): the lanes that hold up hand their numbers to the lanes that hold gate through
//           shared memory (the ring, which is free by then);
//   second: y[row, c] = act[row] . Wd[e][c], 128 output columns.
// The first product reads its A rows from a copy of x gathered into the order of the rows (moe_gather_rows below), so
// that a tile of rows is one TMA box.
//
// Warp roles as in gemm_tcgen05.cu: warp 0 lane 0 issues the TMA loads into a ring of stages (64 columns of K each,
// 128-byte swizzle) and arms each stage's mbarrier; warp 1 allocates tensor memory and its lane 0 issues the MMAs and
// commits them to the stage's "empty" barrier, at the end to the accumulator's barrier; warps 2-5 read their quarter
// of the lanes with tcgen05.ld and write the outputs.  Every wait is bounded; one that runs out sets the file's error
// word and the block leaves through the common exit, which frees its tensor memory.
#include <mutex>
#include <unordered_map>

#define NHV_WAIT_LIMIT (1u << 22)
#include "nhv_async.cuh"
#include "nhv_glu.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int PANEL = 128;             // weight rows per block = MMA M
constexpr int ROWS = 128;              // rows of the ordering per block = MMA N
constexpr int BK = 64;                 // columns per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int THREADS = 192;           // producer warp, MMA warp, four epilogue warps
constexpr int EPI_THREADS = 128;
constexpr int W_BYTES = PANEL * 128, A_BYTES = ROWS * 128, STAGE_BYTES = W_BYTES + A_BYTES;
constexpr uint32_t TMEM_COLS = 128;
constexpr int PARK_LD = 33;            // a parked row of 32 columns, padded

__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major bfloat16
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// Shared-memory matrix descriptor of a K-major bf16 operand tile in the 128-byte swizzle (rows of 128 bytes, groups of
// 8 rows 1024 bytes apart; the tile starts on a 1024-byte boundary; `addr` may point 32, 64 or 96 bytes into the
// first row to select the K=16 slice).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both K-major, M x N.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(EPI_THREADS) : "memory"); }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct alignas(64) Params {
  CUtensorMap w0_map;   // first: gate [E * N, K], box 64 columns x 64 rows; second: down [E * N, K], box 64 x 128
  CUtensorMap w1_map;   // first: up, as gate
  CUtensorMap a_map;    // the rows [rows, K], box 64 columns x 128 rows
  bf16* out;            // [rows, N]
  const int* sorted_slots;
  const int* tile_expert;
  int N, K;
  float limit, alpha, up_shift;
  const float* row_scale;     // a factor on the expert's input per (token, choice) slot, or null
};

template <bool FIRST>
__global__ void __launch_bounds__(THREADS, 1) moe_tcgen05_kernel(const __grid_constant__ Params p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = smem_unaligned + ((1024 - (smem_u32(smem_unaligned) & 1023)) & 1023);
  unsigned char* ring = smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  __shared__ int s_abort;
  __shared__ int s_epi_abort;             // set by epilogue threads only, read by them after their barrier: one answer for all
  __shared__ float s_scale[ROWS];         // the row's factor on the expert's input (1 without)
  __shared__ int s_live[ROWS];            // 1 where the row of the tile is a slot, 0 where it is padding

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // panels of one tile of rows are neighbours in the grid: they run together and share the tile's rows in L2, and the
  // tiles of one expert follow one another, so its weights stay there too
  const int tile = blockIdx.y;
  const int n0 = blockIdx.x * (FIRST ? PANEL / 2 : PANEL);
  const int kb_n = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    s_abort = 0;
    s_epi_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                                                   // the ordering and the rows are the work of kernels before
  const int e = p.tile_expert[tile];                            // block-uniform: a tile without an expert has no work

  if (e >= 0) {
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        const int w_row = e * p.N + n0;
        for (int kb = 0; kb < kb_n; ++kb) {
          const int s = kb % STAGES;
          if (kb >= STAGES && !mbar_wait(&empty[s], (uint32_t)((kb / STAGES) - 1) & 1, 1)) { s_abort = 1; break; }
          unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);                // zero-filled parts of a box count too
          if (FIRST) {
            tma_load_2d(dst, &p.w0_map, kb * BK, w_row, &full[s]);
            tma_load_2d(dst + W_BYTES / 2, &p.w1_map, kb * BK, w_row, &full[s]);
          } else {
            tma_load_2d(dst, &p.w0_map, kb * BK, w_row, &full[s]);
          }
          tma_load_2d(dst + W_BYTES, &p.a_map, kb * BK, tile * ROWS, &full[s]);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        const uint32_t idesc = instr_desc(PANEL, ROWS);
        bool ok = true;
        for (int kb = 0; kb < kb_n && ok; ++kb) {
          const int s = kb % STAGES;
          ok = mbar_wait(&full[s], (uint32_t)(kb / STAGES) & 1, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + (size_t)s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + W_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            tc_mma(tmem_base, smem_desc_sw128(a_addr + kk * UMMA_K * 2), smem_desc_sw128(b_addr + kk * UMMA_K * 2), idesc,
                   (kb == 0 && kk == 0) ? 0u : 1u);
          tc_commit(&empty[s]);                                 // the stage is free once these MMAs have read it
        }
        if (ok) tc_commit(acc_full);
        else s_abort = 1;
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
      const int tid = threadIdx.x - 64;                         // 0..127
      const int quarter = warp & 3;                             // the tensor-memory lanes this warp may read
      const int lane_row = quarter * 32 + lane;                 // the weight row of the panel that this thread holds
      {
        const int slot = p.sorted_slots[(size_t)tile * ROWS + tid];
        s_live[tid] = slot >= 0;
        s_scale[tid] = (FIRST && p.row_scale && slot >= 0) ? p.row_scale[slot] : 1.f;
      }
      if (!mbar_wait(acc_full, 0, 4)) s_epi_abort = 1;
      epi_sync();
      const bool ok = s_epi_abort == 0;                         // the same for all 128: they meet at barriers below
      if (!ok) s_abort = 1;
      tc_fence_after();
      if (ok) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float* park = reinterpret_cast<float*>(ring);           // [64][PARK_LD]: the ring is free once the MMAs are done
        for (int c0 = 0; c0 < ROWS; c0 += 32) {
          float v[32];
          tmem_ld32(v, taddr + c0);
          if (FIRST) {
            if (lane_row >= PANEL / 2) {
#pragma unroll
              for (int j = 0; j < 32; ++j) park[(lane_row - PANEL / 2) * PARK_LD + j] = v[j];
            }
            epi_sync();
            const int n = n0 + lane_row;
            if (lane_row < PANEL / 2 && n < p.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (s_live[c0 + j]) {
                  // gate and up rounded to the storage type first, as a separate product would leave them
                  const float sc = s_scale[c0 + j];
                  const float a = nhv_glu(round_bf16(sc * v[j]), round_bf16(sc * park[lane_row * PARK_LD + j]), p.limit, p.alpha,
                                          p.up_shift);
                  p.out[((size_t)tile * ROWS + c0 + j) * p.N + n] = __float2bfloat16_rn(a);
                }
            }
            epi_sync();                                         // the parked columns are overwritten by the next 32
          } else {
            const int n = n0 + lane_row;
            if (n < p.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (s_live[c0 + j]) p.out[((size_t)tile * ROWS + c0 + j) * p.N + n] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
      tc_fence_before();
    }
  }
  // ------------------------------------------------------------------ common exit
  __syncthreads();
  if (s_abort) give_up_delay();                                 // let copies that may still be in flight land
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8 + 16;

struct MapKey {
  const void* base;
  long long rows;
  int cols, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols << 20) ^ (size_t)k.box_rows;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_weight_maps;   // weights do not move: one map per stack
std::mutex g_maps_mutex;

bool weight_map(CUtensorMap* out, const void* base, long long rows, int cols, int box_rows) {
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  const MapKey key{base, rows, cols, box_rows};
  auto it = g_weight_maps.find(key);
  if (it == g_weight_maps.end()) {
    CUtensorMap m;
    if (!nhv_make_map_bf16(&m, base, rows, cols, cols, BK, box_rows)) return false;
    it = g_weight_maps.emplace(key, m).first;
  }
  *out = it->second;
  return true;
}

// One block per row of the ordering: the token's row of x, or zeros for padding.
__global__ void moe_gather_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, const int* __restrict__ sorted_slots,
                                       int top, int pieces) {
  pdl_prologue();
  const int slot = sorted_slots[blockIdx.x];
  uint4* dst = out + (size_t)blockIdx.x * pieces;
  if (slot < 0) {
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = x + (size_t)(slot / top) * pieces;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) dst[i] = src[i];
}

}  // namespace

NHV_API int nhv_moe_tcgen05_error() { return nhv_wait_error_take(); }
NHV_API void* nhv_moe_tcgen05_error_word() { return nhv_wait_error_address(); }
NHV_API int nhv_moe_tcgen05_tile() { return ROWS; }

// out [rows, width] (bfloat16) = x[sorted_slots[row] / top], zeros where the row is padding.
NHV_API int nhv_moe_gather_rows(void* out, const void* x, const int* sorted_slots, int rows, int top, int width,
                                cudaStream_t stream) {
  if (rows == 0) return 0;
  NHV_REQUIRE(width % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)x % 16) == 0 && top > 0,
              "moe_gather_rows: rows of %d elements do not start on 16-byte boundaries", width);
  NHV_CUDA(nhv_launch(moe_gather_rows_kernel, dim3(rows), dim3(128), 0, stream, (uint4*)out, (const uint4*)x, sorted_slots, top,
                      width / 8), "moe_gather_rows");
  return 0;
}

// first != 0: out [rows, N] = glu(A W0[e]^T, A W1[e]^T) with A [rows, K] (the gathered rows) and W0 / W1 [E, N, K];
// first == 0: out [rows, N] = A W0[e]^T.  rows = tiles * 128, the ordering of moe_align with tiles of 128 rows.
NHV_API int nhv_moe_gemm_tcgen05(int first, void* out, const void* A, const void* W0, const void* W1, int n_experts,
                                 const int* sorted_slots, const int* tile_expert, int tiles, int N, int K, float limit,
                                 float alpha, float up_shift, const float* row_scale, cudaStream_t stream) {
  if (tiles == 0) return 0;
  NHV_REQUIRE(tiles > 0 && N > 0 && K > 0 && K % 8 == 0 && n_experts > 0, "moe_gemm (tcgen05): K must be a multiple of 8 (N=%d K=%d)", N, K);
  NHV_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W0 % 16) == 0 && (!first || ((uintptr_t)W1 % 16) == 0),
              "moe_gemm (tcgen05): operands must be 16-byte aligned");
  NHV_REQUIRE((long long)n_experts * N < (1LL << 31) && (long long)tiles * ROWS < (1LL << 31), "moe_gemm (tcgen05): too many rows");
  Params p;
  const int box = first ? PANEL / 2 : PANEL;
  NHV_REQUIRE(weight_map(&p.w0_map, W0, (long long)n_experts * N, K, box), "moe_gemm (tcgen05): cannot encode the weights' tensor map");
  if (first) NHV_REQUIRE(weight_map(&p.w1_map, W1, (long long)n_experts * N, K, box), "moe_gemm (tcgen05): cannot encode the weights' tensor map");
  else p.w1_map = p.w0_map;
  NHV_REQUIRE(nhv_make_map_bf16(&p.a_map, A, (long long)tiles * ROWS, K, K, BK, ROWS), "moe_gemm (tcgen05): cannot encode the rows' tensor map");
  p.out = (bf16*)out;
  p.sorted_slots = sorted_slots;
  p.tile_expert = tile_expert;
  p.N = N;
  p.K = K;
  p.limit = limit;
  p.alpha = alpha;
  p.up_shift = up_shift;
  p.row_scale = row_scale;
  dim3 grid((N + box - 1) / box, tiles);
  NHV_REQUIRE(grid.y <= 65535, "moe_gemm (tcgen05): %d tiles of rows are beyond the grid's reach", tiles);
  static bool attr_set = false;
  if (!attr_set) {
    NHV_CUDA(cudaFuncSetAttribute(moe_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES), "moe_gemm (tcgen05)");
    NHV_CUDA(cudaFuncSetAttribute(moe_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES), "moe_gemm (tcgen05)");
    attr_set = true;
  }
  if (first) NHV_CUDA(nhv_launch(moe_tcgen05_kernel<true>, grid, dim3(THREADS), SMEM_BYTES, stream, p), "moe_gemm (tcgen05)");
  else NHV_CUDA(nhv_launch(moe_tcgen05_kernel<false>, grid, dim3(THREADS), SMEM_BYTES, stream, p), "moe_gemm (tcgen05)");
  return 0;
}
