// A mixture of experts inside a feed-forward: routing, the experts' products over tokens sorted by expert, the weighted sum.
//
//   moe_route     z = W_r h in float (one chain of additions a logit, whatever the batch), s = softmax(z) over all experts;
//                 the choice is by s + correction, among the experts of the `keep` groups (of `count` equal groups of
//                 neighbours) whose best choice score is largest; the `top` best are taken and weighted by their plain s,
//                 as it is (no renormalisation).  Ties go to the lower index.  Options: scores may be sigmoid(z) instead of
//                 the softmax; there may be no correction; a group may count by the sum of its two best choice scores
//                 instead of its best; the chosen scores may be divided by their sum (+ 1e-20); and a factor may scale them.
//   moe_align     sorts the step's (token, choice) pairs by expert: every expert's rows start on a multiple of the product's
//                 row tile (padding rows name no token), and each row tile knows its expert.  Everything stays on the
//                 device: the grid of the products is sized for the worst case and tiles past the end return at once.
//   moe_gemm      C[row] = f(A[row] W_e^T) for the rows of expert e, W stacked [experts, N, K]; A is either gathered by the
//                 row's token (the first product) or read in place (the second); f is the identity, the squared relu, or
//                 (rows of W in pairs: gate row, up row) SiLU(gate) * up, which halves the output's width.
//                 Float accumulation, one chain of fused multiply-adds over k in ascending order for every output element
//                 (the float path's product, with a tile's expert in front of it).
//   moe_combine   out[t] = sum_j weight[t, j] * y[row of (t, j)], j in order, in float.
//   relu_squared  out = max(x, 0)^2 (the dense feed-forward's activation).
#include "common.cuh"

namespace vob {

constexpr int MOE_TM = 64;       // rows of a product tile; experts' row ranges are padded to it

// What a (gate, up) pair of features becomes: SiLU(gate) * up, or with a clamp (`limit` > 0)
// g = min(gate, limit), u = clamp(up, -limit, limit): g * sigmoid(1.702 g) * (u + 1).
__device__ __forceinline__ float gated_pair(float gate, float up, float limit) {
  if (limit > 0.f) {
    const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
  }
  return gate / (1.f + expf(-gate)) * up;
}

// ---------------------------------------------------------------- routing
struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}

constexpr int ROUTE_NT = 256;

constexpr int ROUTE_TOKENS = 4;   // tokens a block: the router's rows are read once for all of them

template <typename T>
__global__ void __launch_bounds__(ROUTE_NT)
moe_route_kernel(const T* h, const float* __restrict__ w_router, const float* __restrict__ router_bias,
                 const float* __restrict__ correction, int* ids, float* weights,
                 int W, int E, int top, int count, int keep, int sigmoid_scores, int group_top, int normalise, float weight_scale,
                 int num_tokens, int per_block) {
  extern __shared__ __align__(16) float route_smem[];
  float* hrows = route_smem;                        // [per_block][W]
  float* lists = hrows + (size_t)per_block * W;     // per token: [E] scores, [E] choice scores, [count] group scores
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * per_block, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int here = min(per_block, num_tokens - t0);
  for (int d = threadIdx.x; d < here * W; d += ROUTE_NT) hrows[d] = to_f<T>(h[(size_t)t0 * W + d]);
  __syncthreads();
  // a warp takes experts warp, warp + 8, ...; a lane sums four elements at a time into four chains (one chain where the
  // width is no multiple of 4): the order of a logit's additions depends on the width alone, not on the tokens beside it
  const bool vec = W % 4 == 0 && ((uintptr_t)w_router % 16) == 0;
  for (int e = warp; e < E; e += ROUTE_NT / 32) {
    const float* wr = w_router + (size_t)e * W;
    float z[ROUTE_TOKENS];
    if (vec) {
      float z4[ROUTE_TOKENS][4];
#pragma unroll
      for (int k = 0; k < ROUTE_TOKENS; ++k) z4[k][0] = z4[k][1] = z4[k][2] = z4[k][3] = 0.f;
      for (int d = lane * 4; d < W; d += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(wr + d);
#pragma unroll
        for (int k = 0; k < ROUTE_TOKENS; ++k) {
          if (k < here) {
            const float4 hv = *reinterpret_cast<const float4*>(hrows + (size_t)k * W + d);
            z4[k][0] = fmaf(hv.x, wv.x, z4[k][0]); z4[k][1] = fmaf(hv.y, wv.y, z4[k][1]);
            z4[k][2] = fmaf(hv.z, wv.z, z4[k][2]); z4[k][3] = fmaf(hv.w, wv.w, z4[k][3]);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < ROUTE_TOKENS; ++k) z[k] = (z4[k][0] + z4[k][1]) + (z4[k][2] + z4[k][3]);
    } else {
#pragma unroll
      for (int k = 0; k < ROUTE_TOKENS; ++k) z[k] = 0.f;
      for (int d = lane; d < W; d += 32) {
        const float wv = wr[d];
#pragma unroll
        for (int k = 0; k < ROUTE_TOKENS; ++k)
          if (k < here) z[k] = fmaf(hrows[(size_t)k * W + d], wv, z[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < ROUTE_TOKENS; ++k) {
      const float sum = warp_sum(z[k]);
      if (lane == 0 && k < here) lists[(size_t)k * (2 * E + count) + e] = router_bias ? sum + router_bias[e] : sum;
    }
  }
  __syncthreads();
  // warp k chooses for token k
  if (warp >= here) return;
  const int t = t0 + warp;
  float* score = lists + (size_t)warp * (2 * E + count);   // [E] softmax or sigmoid
  float* choice = score + E;                               // [E] score + correction, -inf once taken or shut out
  float* gbest = choice + E;                               // [count]
  if (sigmoid_scores) {
    for (int e = lane; e < E; e += 32) {
      const float s = 1.f / (1.f + expf(-score[e]));
      score[e] = s;
      choice[e] = correction ? s + correction[e] : s;
    }
  } else {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, score[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(score[e] - m);
    sum = warp_sum(sum);
    // Without a correction the choice is by the logit itself where that gives the same order (it does unless groups count
    // by a sum of scores): logits far below the largest all become a score of zero, and would tie.
    const bool by_logit = !correction && (keep >= count || group_top < 2);
    for (int e = lane; e < E; e += 32) {
      const float z = score[e] - m;
      const float s = expf(z) / sum;
      score[e] = s;
      choice[e] = correction ? s + correction[e] : (by_logit ? z : s);
    }
  }
  __syncwarp();
  const int per = E / count;
  if (keep < count) {
    for (int g = lane; g < count; g += 32) {
      float b = -INFINITY, b2 = -INFINITY;     // the group's best and second best choice score
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > b) { b2 = b; b = c; } else if (c > b2) { b2 = c; }
      }
      gbest[g] = (group_top >= 2 && per >= 2) ? b + b2 : b;
    }
    __syncwarp();
    // the `keep` best groups are marked by +inf; then every expert of an unmarked group is shut out
    for (int it = 0; it < keep; ++it) {
      Best x{-INFINITY, 0x7fffffff};
      for (int g = lane; g < count; g += 32)
        if (gbest[g] != INFINITY) x = better(x, Best{gbest[g], g});
      x = warp_best(x);
      __syncwarp();
      if (lane == 0 && x.i < count) gbest[x.i] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gbest[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    Best x{-INFINITY, 0x7fffffff};
    for (int e = lane; e < E; e += 32) x = better(x, Best{choice[e], e});
    x = warp_best(x);
    __syncwarp();
    if (lane == 0) {
      const int e = x.i < E ? x.i : 0;
      ids[(size_t)t * top + j] = e;
      weights[(size_t)t * top + j] = x.i < E ? score[e] : 0.f;
      choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0 && (normalise || weight_scale != 1.f)) {
    float* wt = weights + (size_t)t * top;
    float sum = 0.f;
    for (int j = 0; j < top; ++j) sum += wt[j];
    for (int j = 0; j < top; ++j) wt[j] = (normalise ? wt[j] / (sum + 1e-20f) : wt[j]) * weight_scale;
  }
}

// ---------------------------------------------------------------- sorting by expert
// One block.  n = tokens * top pairs; slot_of[n]: the row of a pair; row_token[max_rows]: a row's token (-1: padding);
// tile_expert[max_rows / MOE_TM]: the expert of every MOE_TM rows (-1: past the end).  An expert's rows are padded to a
// multiple of `pad`, itself a multiple of MOE_TM (a product with larger row tiles asks for more).
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* ids, int* slot_of, int* row_token, int* tile_expert, int n, int top, int E, int max_rows, int pad) {
  extern __shared__ int align_smem[];
  int* counts = align_smem;          // [E]
  int* offsets = counts + E;         // [E]
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_token[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = off;
      const int padded = (counts[e] + pad - 1) / pad * pad;
      for (int tile = off / MOE_TM; tile < (off + padded) / MOE_TM; ++tile) tile_expert[tile] = e;
      off += padded;
      counts[e] = 0;      // now the expert's cursor
    }
    for (int tile = off / MOE_TM; tile < max_rows / MOE_TM; ++tile) tile_expert[tile] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= E) { slot_of[i] = -1; continue; }
    const int row = offsets[e] + atomicAdd(&counts[e], 1);
    slot_of[i] = row;
    row_token[row] = i / top;
  }
}

// ---------------------------------------------------------------- the experts' products
constexpr int MG_N = 64, MG_K = 16;

// EPI 0: as it is; 1: squared relu; 2: gated_pair(even column, odd column) into column / 2.  GATHER: row r of A is
// a[row_token[r]], else a[r].
template <typename TA, typename TC, int EPI, bool GATHER>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* A, long lda, const TA* __restrict__ W, TC* C, long ldc, const int* row_token,
                const int* tile_expert, int N, int K, float glu_limit) {
  __shared__ float As[MG_K][MOE_TM + 4];
  __shared__ float Ws[MG_K][MG_N + 4];
  __shared__ int src[MOE_TM];
  pdl_launch_dependents();
  pdl_wait();
  const int e = tile_expert[blockIdx.y];
  if (e < 0) return;
  const int m0 = blockIdx.y * MOE_TM, n0 = blockIdx.x * MG_N;
  const int tid = threadIdx.x;
  if (tid < MOE_TM) {
    const int tok = row_token[m0 + tid];
    src[tid] = tok < 0 ? -1 : (GATHER ? tok : m0 + tid);
  }
  __syncthreads();
  const TA* We = W + (size_t)e * N * K;
  const int tx = tid % 16, ty = tid / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const int arow = src[lr];
  for (int k0 = 0; k0 < K; k0 += MG_K) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int wn = n0 + lr;
      As[lk + j][lr] = (arow >= 0 && k < K) ? to_f<TA>(A[(size_t)arow * lda + k]) : 0.f;
      Ws[lk + j][lr] = (wn < N && k < K) ? to_f<TA>(We[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MG_K; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (src[ty * 4 + i] < 0) continue;
    const int m = m0 + ty * 4 + i;
    if (EPI == 2) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 >= N) continue;
        const float g = acc[i][j];
        C[(size_t)m * ldc + n / 2] = from_f<TC>(gated_pair(g, acc[i][j + 1], glu_limit));
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (EPI == 1) { v = fmaxf(v, 0.f); v = v * v; }
      C[(size_t)m * ldc + n] = from_f<TC>(v);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* y, const int* slot_of, const float* weights, T* out, int D, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += 256) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int row = slot_of ? slot_of[(size_t)t * top + j] : t * top + j;
      if (row >= 0) acc = fmaf(weights[(size_t)t * top + j], y[(size_t)row * D + d], acc);
    }
    out[(size_t)t * D + d] = from_f<T>(acc);
  }
}

// ---------------------------------------------------------------- steps of few tokens (bfloat16)
// While decoding, a step has fewer (token, choice) pairs than a row tile has rows, and the products are bound by the
// experts' weights, not by arithmetic.  moe_order lists the pairs by expert, without padding; moe_gemv gives a pair a
// block per 64 output features: the pair's input row lies in shared memory, a warp streams four rows of W_e at a time
// with 16-byte loads and sums in float.  Pairs of one expert run side by side, so its rows come from DRAM once.
__global__ void __launch_bounds__(256)
moe_order_kernel(const int* ids, int* order, int n, int E) {
  extern __shared__ int order_smem[];
  int* counts = order_smem;          // [E], then the experts' cursors
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      counts[e] = off;
      off += c;
    }
    for (int j = off; j < n; ++j) order[j] = -1;      // pairs that name no expert
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) order[atomicAdd(&counts[e], 1)] = i;
  }
}

constexpr int MV_ROWS = 64;       // output features a block

// EPI 0: float as it is; 1: squared relu into bfloat16; 2: SiLU(even row) * odd row into bfloat16 column row / 2.  BY_TOKEN: a pair's input row is its token's (pair / top), else its own.
template <int EPI, bool BY_TOKEN>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(const __nv_bfloat16* A, long lda, const __nv_bfloat16* __restrict__ W, void* C, long ldc, const int* ids,
                const int* order, int top, int N, int K, float glu_limit) {
  extern __shared__ uint4 gemv_smem[];     // the input row: K bfloat16
  pdl_launch_dependents();
  pdl_wait();
  const int pair = order[blockIdx.y];
  if (pair < 0) return;
  const int e = ids[pair];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = K / 8;
  const uint4* arow = reinterpret_cast<const uint4*>(A + (size_t)(BY_TOKEN ? pair / top : pair) * lda);
  for (int c = threadIdx.x; c < chunks; c += 256) gemv_smem[c] = arow[c];
  __syncthreads();
  const int n0 = blockIdx.x * MV_ROWS + warp * 8;
#pragma unroll
  for (int rg = 0; rg < 2; ++rg) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4* wrow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = min(n0 + rg * 4 + r, N - 1);
      wrow[r] = reinterpret_cast<const uint4*>(W + ((size_t)e * N + n) * K);
    }
    for (int c = lane; c < chunks; c += 32) {
      uint4 wv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) wv[r] = wrow[r][c];
      const uint4 xv = gemv_smem[c];
      const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = __bfloat1622float2(w2[j]), xf = __bfloat1622float2(x2[j]);
          acc[r] = fmaf(wf.x, xf.x, acc[r]);
          acc[r] = fmaf(wf.y, xf.y, acc[r]);
        }
      }
    }
    if (EPI == 2) {
      float v[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) v[r] = warp_sum(acc[r]);
#pragma unroll
      for (int r = 0; r < 4; r += 2) {
        const int n = n0 + rg * 4 + r;
        if (lane == 0 && n + 1 < N)
          reinterpret_cast<__nv_bfloat16*>(C)[(size_t)pair * ldc + n / 2] = __float2bfloat16_rn(gated_pair(v[r], v[r + 1], glu_limit));
      }
      continue;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float v = warp_sum(acc[r]);
      const int n = n0 + rg * 4 + r;
      if (lane == 0 && n < N) {
        if (EPI == 1) {
          const float p = fmaxf(v, 0.f);
          reinterpret_cast<__nv_bfloat16*>(C)[(size_t)pair * ldc + n] = __float2bfloat16_rn(p * p);
        } else {
          reinterpret_cast<float*>(C)[(size_t)pair * ldc + n] = v;
        }
      }
    }
  }
}

template <typename T>
__global__ void relu_squared_kernel(const T* x, T* out, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_f<T>(x[i]), 0.f);
    out[i] = from_f<T>(v * v);
  }
}

// The same with 16-byte accesses (bfloat16, a multiple of 8 elements, aligned).
__global__ void relu_squared_vec_kernel(const uint4* x, uint4* out, size_t chunks) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (size_t)gridDim.x * blockDim.x) {
    uint4 v = x[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
      h[j] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
    }
    out[i] = v;
  }
}

}  // namespace vob

using namespace vob;

VOB_API int vob_moe_row_tile() { return MOE_TM; }

// correction may be null; sigmoid_scores: scores are sigmoid(z), not the softmax; group_top 2: a group counts by its two best;
// normalise: the chosen scores are divided by their sum; weight_scale: a factor on the weights.
VOB_API int vob_moe_route(const void* h, const float* w_router, const float* router_bias, const float* correction, int* ids,
                          float* weights, int T, int W,
                          int E, int top, int count, int keep, int sigmoid_scores, int group_top, int normalise,
                          float weight_scale, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || count <= 0 || E % count || keep <= 0 || keep > count || (long)(E / count) * keep < top)
    return VOB_BAD_ARGUMENT;
  // as many tokens a block as 96 KB hold (up to ROUTE_TOKENS) while the blocks still fill the device twice; one where the
  // width is no multiple of 4 (rows stay aligned).  A token's arithmetic does not depend on how many share its block.
  int per_block = (int)std::min<long>(ROUTE_TOKENS, std::max<long>(1, T / (2L * sm_count())));
  while (per_block > 1 && ((size_t)per_block * (W + 2 * E + count) * sizeof(float) > 96 * 1024 || W % 4)) --per_block;
  const size_t smem = (size_t)per_block * (W + 2 * E + count) * sizeof(float);
  if (smem > 200 * 1024) return VOB_UNSUPPORTED;
#define VOB_ROUTE(TYPE)                                                                                                  \
  do {                                                                                                                   \
    if (smem > 48 * 1024)                                                                                                \
      cudaFuncSetAttribute(moe_route_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
    return launch_kernel(moe_route_kernel<TYPE>, dim3((T + per_block - 1) / per_block), ROUTE_NT, smem, stream,          \
                         (const TYPE*)h, w_router, router_bias, correction, ids, weights, W, E, top, count, keep, sigmoid_scores,     \
                         group_top, normalise, weight_scale, T, per_block);                                              \
  } while (0)
  if (dtype == VOB_F32) VOB_ROUTE(float);
  if (dtype == VOB_BF16) VOB_ROUTE(__nv_bfloat16);
#undef VOB_ROUTE
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_moe_align(const int* ids, int* slot_of, int* row_token, int* tile_expert, int n, int top, int E, int max_rows,
                          int pad, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (pad <= 0 || pad % MOE_TM || max_rows % pad || E <= 0 || E > 4096) return VOB_BAD_ARGUMENT;
  return launch_kernel(moe_align_kernel, dim3(1), 1024, (size_t)2 * E * sizeof(int), stream, ids, slot_of, row_token, tile_expert,
                       n, top, E, max_rows, pad);
}

// A: rows of lda elements (`gather`: indexed by the row's token); W [experts, N, K]; C [max_rows, ldc] of `dtype`, or float
// with `c_float`.  epilogue 0: as it is, 1: squared relu, 2: SiLU(gate) * up over rows of W in (gate, up) pairs: C has N / 2
// columns.
VOB_API int vob_moe_gemm(const void* A, long lda, const void* W, void* C, long ldc, const int* row_token, const int* tile_expert,
                         int max_rows, int N, int K, int epilogue, int gather, int c_float, float glu_limit, int dtype,
                         cudaStream_t stream) {
  if (max_rows <= 0 || N <= 0) return 0;
  if (K <= 0 || max_rows % MOE_TM) return VOB_BAD_ARGUMENT;
  dim3 grid((N + MG_N - 1) / MG_N, max_rows / MOE_TM);
  if (grid.y > 65535) return VOB_UNSUPPORTED;
#define VOB_MG(TA, TC, EPI, G)                                                                                       \
  return launch_kernel(moe_gemm_kernel<TA, TC, EPI, G>, grid, 256, 0, stream, (const TA*)A, lda, (const TA*)W, (TC*)C, ldc, \
                       row_token, tile_expert, N, K, glu_limit)
#define VOB_MG_TYPE(TA)                                                   \
  if (epilogue == 1 && gather && !c_float) VOB_MG(TA, TA, 1, true);       \
  if (epilogue == 2 && gather && !c_float) VOB_MG(TA, TA, 2, true);       \
  if (epilogue == 0 && !gather && c_float) VOB_MG(TA, float, 0, false);   \
  return VOB_UNSUPPORTED
  if (dtype == VOB_F32) { VOB_MG_TYPE(float); }
  if (dtype == VOB_BF16) { VOB_MG_TYPE(__nv_bfloat16); }
#undef VOB_MG_TYPE
#undef VOB_MG
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_moe_order(const int* ids, int* order, int n, int E, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > 4096) return VOB_BAD_ARGUMENT;
  return launch_kernel(moe_order_kernel, dim3(1), 256, (size_t)E * sizeof(int), stream, ids, order, n, E);
}

// A: bfloat16 rows of lda elements, a token's (`by_token`) or a pair's; W bfloat16 [experts, N, K], K a multiple of 8;
// C [pairs, ldc]: bfloat16 with the squared relu (`epilogue` 1) or with SiLU(gate) * up over rows of W in (gate, up) pairs
// (2: N / 2 columns), or float (0).  order: the pairs by expert (vob_moe_order).
VOB_API int vob_moe_gemv(const void* A, long lda, const void* W, void* C, long ldc, const int* ids, const int* order, int n,
                         int top, int N, int K, int epilogue, int by_token, float glu_limit, cudaStream_t stream) {
  if (n <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (lda * 2) % 16 || ((uintptr_t)A | (uintptr_t)W) % 16 || n > 65535) return VOB_UNSUPPORTED;
  const size_t smem = (size_t)K * 2;
  if (smem > 96 * 1024) return VOB_UNSUPPORTED;
  dim3 grid((N + MV_ROWS - 1) / MV_ROWS, n);
#define VOB_MV(EPI, BT)                                                                                                     \
  do {                                                                                                                      \
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_gemv_kernel<EPI, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return launch_kernel(moe_gemv_kernel<EPI, BT>, grid, 256, smem, stream, (const __nv_bfloat16*)A, lda,                   \
                         (const __nv_bfloat16*)W, C, ldc, ids, order, top, N, K, glu_limit);                                       \
  } while (0)
  if (epilogue == 1 && by_token) VOB_MV(1, true);
  if (epilogue == 2 && by_token && N % 2 == 0) VOB_MV(2, true);
  if (epilogue == 0 && !by_token) VOB_MV(0, false);
#undef VOB_MV
  return VOB_UNSUPPORTED;
}

VOB_API int vob_moe_combine(const float* y, const int* slot_of, const float* weights, void* out, int T, int D, int top, int dtype,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == VOB_F32)
    return launch_kernel(moe_combine_kernel<float>, dim3(T), 256, 0, stream, y, slot_of, weights, (float*)out, D, top);
  if (dtype == VOB_BF16)
    return launch_kernel(moe_combine_kernel<__nv_bfloat16>, dim3(T), 256, 0, stream, y, slot_of, weights, (__nv_bfloat16*)out, D, top);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_relu_squared(const void* x, void* out, long total, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == VOB_F32)
    return launch_kernel(relu_squared_kernel<float>, dim3(blocks), 256, 0, stream, (const float*)x, (float*)out, (size_t)total);
  if (dtype == VOB_BF16 && total % 8 == 0 && ((uintptr_t)x | (uintptr_t)out) % 16 == 0) {
    const long chunks = total / 8;
    const int vblocks = (int)((chunks + 255) / 256 < 148 * 16 ? (chunks + 255) / 256 : 148 * 16);
    return launch_kernel(relu_squared_vec_kernel, dim3(vblocks), 256, 0, stream, (const uint4*)x, (uint4*)out, (size_t)chunks);
  }
  if (dtype == VOB_BF16)
    return launch_kernel(relu_squared_kernel<__nv_bfloat16>, dim3(blocks), 256, 0, stream, (const __nv_bfloat16*)x,
                         (__nv_bfloat16*)out, (size_t)total);
  return VOB_BAD_ARGUMENT;
}
