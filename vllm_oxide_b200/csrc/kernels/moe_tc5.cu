// The experts' products of a mixture of experts for steps of many tokens, in bfloat16 on the fifth-generation tensor
// cores: tcgen05.mma with the accumulator in tensor memory.
//
// The step's (token, choice) pairs lie sorted by expert (moe.cu: moe_align), every expert's rows padded to a tile of 128,
// so a row tile belongs to one expert: C[rows of the tile] = f(A[rows] W_e^T) with W stacked [experts * N, K].  As in the
// product for 17 to 128 tokens (gemm_tc5.cu) the weights are the 128-row operand: a work item is 128 rows of W_e against
// the 128 rows of a row tile, D[128 x 128] in float lives in tensor memory.  Persistent blocks, one per SM, walk the items
// (row tile major, so the blocks that run side by side share a tile's rows and an expert's matrix stays in L2 for its next
// row tile); items of row tiles past the end (tile_expert < 0) are skipped.
//   warp 0      producer: per 64 columns of K one TMA copy of the W tile [128 x 64] and one of the rows [128 x 64]
//               (128-byte swizzle) into a ring of stages;
//   warp 1      allocates tensor memory (two accumulators) and issues the MMAs: four tcgen05.mma (K = 16 each) per stage;
//               tcgen05.commit hands a stage back to the producer and, after an item's last, the accumulator to the epilogue;
//   warps 2-5   epilogue: tcgen05.ld brings the accumulator to registers (a thread owns one output feature for all rows of
//               the tile), applies f (identity into float, the squared relu into bfloat16, or, rows of W in (gate, up)
//               pairs, SiLU(gate) * up into bfloat16 feature / 2: the up value comes from the neighbouring lane) and stores
//               the rows that name a token; the next item's MMAs run meanwhile into the other accumulator.
// Which items exist is only known on the device (the sorting kernel ran just before), so nothing is copied before the wait
// for the kernels ahead.  Every wait on an mbarrier is bounded; on a timeout the block sets an error bit, stops issuing
// work, and still frees its tensor memory before it returns.
#define VOB_TIMEOUT_WHERE 0x2000
#include "tcgen05.cuh"

namespace vob {

constexpr int MT_ROWS = 128;      // rows of W per item (the MMA's M)
constexpr int MT_NT = 128;        // rows of a row tile (the MMA's N)
constexpr int MT_KC = 64;         // columns of K per stage: one 128-byte swizzle atom
constexpr int MT_THREADS = 192;
constexpr int MT_EPI_WARPS = 4;
constexpr int MT_STAGE_BYTES = (MT_ROWS + MT_NT) * 128;
constexpr int MT_S = 6;
constexpr int MT_NUM_BARRIERS = 2 * MT_S + 4;
constexpr int MT_SMEM = 1024 + MT_S * MT_STAGE_BYTES + MT_NUM_BARRIERS * 8 + 16;

enum { MT_EPI_RELU2_BF16 = 0, MT_EPI_F32 = 1, MT_EPI_SILU_PAIRS_BF16 = 2 };

// tmW: W [experts * N, K] as 2-D map with box [128 rows, 64 columns]; tmX: the sorted rows [max_rows, K], same box.
// tile_expert: one entry per 64 rows (the sorting kernel's granularity); row_token: one per row, -1 for padding.
template <int EPI>
__global__ void __launch_bounds__(MT_THREADS, 1)
moe_tc5_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, void* out, long ldo,
               const int* row_token, const int* tile_expert, int row_tiles, int N, int K, float glu_limit, int* err) {
  constexpr int S = MT_S, A_BYTES = MT_ROWS * 128, STAGE_BYTES = MT_STAGE_BYTES;
  constexpr int TMEM_COLS = 2 * MT_NT;
  extern __shared__ __align__(1024) char smem_raw[];
  char* stages = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + S * STAGE_BYTES);
  uint64_t* empty = full + S;
  uint64_t* acc_full = empty + S;       // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;   // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (K + MT_KC - 1) / MT_KC;
  const int n_tiles = (N + MT_ROWS - 1) / MT_ROWS;
  const long total = (long)row_tiles * n_tiles;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], MT_EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    tma_prefetch_map(&tmW);
    tma_prefetch_map(&tmX);
  }
  if (warp == 1) t5_alloc(tmem_slot, TMEM_COLS);
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                       // which items exist, and the rows themselves, come from the kernels ahead

  if (warp == 0) {
    // ------------------------------------------------ producer (one thread)
    if (lane == 0) {
      long p_it = 0;
      bool ok = true;
      for (long item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int mt = (int)(item / n_tiles), nt = (int)(item % n_tiles);
        const int e = tile_expert[mt * (MT_NT / 64)];
        if (e < 0) continue;
        for (int kb = 0; kb < k_iters; ++kb, ++p_it) {
          const int s = (int)(p_it % S);
          if (p_it >= S) {
            ok = mbar_wait(&empty[s], (unsigned)(((p_it / S) - 1) & 1), abort_flag, err);
            if (!ok) break;
          }
          mbar_expect_tx(&full[s], (unsigned)STAGE_BYTES);
          tma_load_2d(stages + s * STAGE_BYTES, &tmW, kb * MT_KC, e * N + nt * MT_ROWS, &full[s]);
          tma_load_2d(stages + s * STAGE_BYTES + A_BYTES, &tmX, kb * MT_KC, mt * MT_NT, &full[s]);
        }
      }
      const long first = p_it > S ? p_it - S : 0;       // copies in flight must land before the block exits
      for (long j = first; j < p_it; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % S], (unsigned)((j / S) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = t5_instr_desc(MT_ROWS, MT_NT);
      long it = 0;
      int lt = 0;
      bool ok = true;
      for (long item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int mt = (int)(item / n_tiles);
        if (tile_expert[mt * (MT_NT / 64)] < 0) continue;
        const int a = lt & 1;
        if (lt >= 2) {   // the epilogue must have drained this accumulator (two items ago)
          ok = mbar_wait(&acc_empty[a], (unsigned)(((lt >> 1) - 1) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * MT_NT);
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = (int)(it % S);
          ok = mbar_wait(&full[s], (unsigned)((it / S) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
          const char* st = stages + s * STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < MT_KC / 16; ++k)      // 16 columns = 32 bytes further into the swizzle atom
            t5_mma(d_tmem, t5_smem_desc(st + k * 32), t5_smem_desc(st + A_BYTES + k * 32), idesc, (kb | k) ? 1u : 0u);
          t5_commit(&empty[s]);                      // the stage is free once these MMAs have read it
        }
        if (ok) t5_commit(&acc_full[a]);             // the accumulator is complete once they have all finished
        ++lt;
      }
    }
  } else {
    // ------------------------------------------------ epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +31
    const int q = warp & 3;
    const int row = q * 32 + lane;                                // this thread's row of the W tile
    int lt = 0;
    for (long item = blockIdx.x; item < total; item += gridDim.x) {
      const int mt = (int)(item / n_tiles), nt = (int)(item % n_tiles);
      if (tile_expert[mt * (MT_NT / 64)] < 0) continue;
      const int a = lt & 1;
      bool ok = mbar_wait(&acc_full[a], (unsigned)((lt >> 1) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      t5_fence_after();
      const long n = (long)nt * MT_ROWS + row;                    // one output feature
#pragma unroll
      for (int c0 = 0; c0 < MT_NT; c0 += 32) {
        float v[32];
        t5_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * MT_NT + c0), v);
        const int tok = row_token[mt * MT_NT + c0 + lane];        // lane j's entry belongs to column c0 + j
        if (EPI == MT_EPI_SILU_PAIRS_BF16) {
          // Two lanes hold a (gate, up) pair of features.  They finish two token columns at a time, the even lane column
          // j and the odd lane column j + 1, so every lane takes one exponential for two columns and one exchange
          // serves both.
          const bool odd = lane & 1;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const bool live0 = __shfl_sync(0xffffffffu, tok, j) >= 0, live1 = __shfl_sync(0xffffffffu, tok, j + 1) >= 0;
            if (!live0 && !live1) continue;                       // the same for every lane of the warp
            const float got = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[j + 1], 1);
            const float gate = odd ? got : v[j], up = odd ? v[j + 1] : got;
            if ((odd ? live1 : live0) && (n | 1) < N) {
              const long m = (long)mt * MT_NT + c0 + j + (odd ? 1 : 0);
              reinterpret_cast<__nv_bfloat16*>(out)[m * ldo + (n >> 1)] =
                  __float2bfloat16_rn(glu_limit > 0.f
                                          ? __fdividef(fminf(gate, glu_limit), 1.f + __expf(-1.702f * fminf(gate, glu_limit))) *
                                                (fminf(fmaxf(up, -glu_limit), glu_limit) + 1.f)
                                          : __fdividef(gate, 1.f + __expf(-gate)) * up);
            }
          }
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const bool live = __shfl_sync(0xffffffffu, tok, j) >= 0;
          if (live && n < N) {
            const long m = (long)mt * MT_NT + c0 + j;
            if (EPI == MT_EPI_F32) {
              reinterpret_cast<float*>(out)[m * ldo + n] = v[j];
            } else {
              const float r = fmaxf(v[j], 0.f);
              reinterpret_cast<__nv_bfloat16*>(out)[m * ldo + n] = __float2bfloat16_rn(r * r);
            }
          }
        }
      }
      t5_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
      ++lt;
    }
  }
  // every path ends here: the tensor memory goes back before the block exits
  t5_fence_before();
  __syncthreads();
  if (warp == 1) {
    t5_fence_after();
    t5_dealloc(tmem_base, TMEM_COLS);
  }
}

// xs[row] = x[row_token[row]] (rows that name no token are left as they are); D a multiple of 8, 16-byte aligned rows.
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const __nv_bfloat16* x, long ldx, __nv_bfloat16* xs, const int* row_token, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int tok = row_token[row];
  if (tok < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * D);
  for (int i = threadIdx.x; i < D / 8; i += 128) dst[i] = src[i];
}

}  // namespace vob

using namespace vob;

VOB_API int vob_moe_tc5_row_tile() { return MT_NT; }

// map_w: tensor map of W [experts * N, K] with box 128 rows; map_x: tensor map of the sorted rows [max_rows, K] with box 128
// rows (vob_tensor_map_bf16_2d).  out [max_rows, ldo]: bfloat16 with the squared relu (epilogue 0), float (1), or bfloat16
// SiLU(gate) * up over rows of W in (gate, up) pairs (2: N / 2 columns; with glu_limit > 0 the clamped form
// min(gate, limit) * sigmoid(1.702 min(gate, limit)) * (clamp(up, -limit, limit) + 1)).
VOB_API int vob_moe_gemm_tc5(const void* map_w, const void* map_x, void* out, long ldo, const int* row_token,
                             const int* tile_expert, int max_rows, int N, int K, int epilogue, float glu_limit, int* err,
                             cudaStream_t stream) {
  if (max_rows <= 0 || N <= 0) return 0;
  if (!map_w || !map_x || K <= 0 || K % 8 || max_rows % MT_NT) return VOB_BAD_ARGUMENT;
  const int row_tiles = max_rows / MT_NT;
  const long total = (long)row_tiles * ((N + MT_ROWS - 1) / MT_ROWS);
  const int blocks = (int)(total < sm_count() ? total : sm_count());
  static bool configured[3] = {false, false, false};
#define VOB_MT(EPI)                                                                                                        \
  do {                                                                                                                     \
    if (!configured[EPI]) {                                                                                                \
      cudaError_t e = cudaFuncSetAttribute(moe_tc5_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, MT_SMEM);     \
      if (e != cudaSuccess) return (int)e;                                                                                 \
      configured[EPI] = true;                                                                                              \
    }                                                                                                                      \
    return launch_kernel(moe_tc5_kernel<EPI>, dim3(blocks), MT_THREADS, MT_SMEM, stream, *(const CUtensorMap*)map_w,       \
                         *(const CUtensorMap*)map_x, out, ldo, row_token, tile_expert, row_tiles, N, K, glu_limit, err);          \
  } while (0)
  if (epilogue == MT_EPI_RELU2_BF16) VOB_MT(MT_EPI_RELU2_BF16);
  if (epilogue == MT_EPI_F32) VOB_MT(MT_EPI_F32);
  if (epilogue == MT_EPI_SILU_PAIRS_BF16 && N % 2 == 0) VOB_MT(MT_EPI_SILU_PAIRS_BF16);
#undef VOB_MT
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_moe_gather_rows(const void* x, long ldx, void* xs, const int* row_token, int max_rows, int D, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (D % 8 || ((uintptr_t)x | (uintptr_t)xs) % 16 || (ldx * 2) % 16) return VOB_UNSUPPORTED;
  return launch_kernel(moe_gather_rows_kernel, dim3(max_rows), 128, 0, stream, (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)xs,
                       row_token, D);
}
