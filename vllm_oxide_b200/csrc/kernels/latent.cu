// Attention through a latent: what surrounds the paged attention kernels when keys and values are kept as one
// low-rank row per token.
//
//   latent_prep:   the down-projected row of a token is split into the query latent, the key/value latent and a rotated
//                  key part that every head uses; both latents are normalised (vector weights), the shared part is
//                  rotated by the token's position, and [latent | rotated part | zeros] is written to the token's slot
//                  of the cache plane.  A layer that borrows another layer's plane only gets its query latent.
//   head_linear:   y[t, h, :] = W_h x[t, h, :] for per-head matrices W_h: queries carried into the latent's space (so
//                  that a score is a dot product with the cached row itself) and attention results carried from the
//                  latent's space to the value heads.
//   latent_query_rotate: the rotated part of every query head, behind its latent part, and zeros up to the row width.
//
// Pairs are neighbours (2i, 2i + 1) or, with `halves`, (i, i + rotary / 2).  The angle of pair i at position p is float(p) * frequency[i], computed where it is used (no table, no position limit);
// cos and sin are multiplied by an amplitude.  Norms, angles and rotation are float; rows are of the model's type T.
#include "common.cuh"

namespace vob {

// (a, b) turned by `angle`, amplitude `amp`; products and sums are spelled out so that every kernel rounds alike.
__device__ __forceinline__ void turn_pair(float a, float b, float angle, float amp, float& ra, float& rb) {
  const float c = __fmul_rn(cosf(angle), amp), s = __fmul_rn(sinf(angle), amp);
  ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}

constexpr int LP_NT = 128;

template <typename T>
__global__ void __launch_bounds__(LP_NT)
latent_prep_kernel(const T* down, long stride, const float* __restrict__ wq, const float* __restrict__ wkv,
                   const float* __restrict__ freq, float amp, const int* __restrict__ positions, const int* __restrict__ slots,
                   T* cq, T* cache, int q_rank, int kv_rank, int rot, int rotary, int row_width, long num_slots, float eps,
                   int has_kv, int halves, int* err) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = has_kv ? slots[t] : -1;
  pdl_wait();
  const T* row = down + (size_t)t * stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += LP_NT) {
    const float v = to_f<T>(row[i]);
    ss += v * v;
  }
  float denom = sqrtf(block_sum<LP_NT>(ss, scratch) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += LP_NT) cq[(size_t)t * q_rank + i] = from_f<T>(to_f<T>(row[i]) / denom * wq[i]);
  if (!has_kv || slot < 0) return;       // a borrowed plane, or a padded row of a fixed-size launch
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const T* kv = row + q_rank;
  T* dst = cache + (size_t)slot * row_width;
  ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += LP_NT) {
    const float v = to_f<T>(kv[i]);
    ss += v * v;
  }
  denom = sqrtf(block_sum<LP_NT>(ss, scratch) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += LP_NT) dst[i] = from_f<T>(to_f<T>(kv[i]) / denom * wkv[i]);
  const T* kr = kv + kv_rank;
  if (halves) {
    // element i pairs with element i + rotary / 2; what lies behind the rotated elements passes as it is
    const int half = rotary / 2;
    for (int i = threadIdx.x; i < rot; i += LP_NT) {
      float v = to_f<T>(kr[i]);
      if (i < rotary) {
        const int p = i < half ? i : i - half;
        float ra, rb;
        turn_pair(to_f<T>(kr[p]), to_f<T>(kr[p + half]), __fmul_rn((float)pos, freq[p]), amp, ra, rb);
        v = i < half ? ra : rb;
      }
      dst[kv_rank + i] = from_f<T>(v);
    }
    for (int i = kv_rank + rot + threadIdx.x; i < row_width; i += LP_NT) dst[i] = from_f<T>(0.f);
    return;
  }
  for (int p = threadIdx.x; p < rot / 2; p += LP_NT) {
    float a = to_f<T>(kr[2 * p]), b = to_f<T>(kr[2 * p + 1]);
    if (2 * p + 1 < rotary) turn_pair(a, b, __fmul_rn((float)pos, freq[p]), amp, a, b);
    dst[kv_rank + 2 * p] = from_f<T>(a);
    dst[kv_rank + 2 * p + 1] = from_f<T>(b);
  }
  if ((rot & 1) && threadIdx.x == 0) dst[kv_rank + rot - 1] = kr[rot - 1];
  for (int i = kv_rank + rot + threadIdx.x; i < row_width; i += LP_NT) dst[i] = from_f<T>(0.f);
}

// q [tokens, heads, dk + rot] -> qa[t, h, offset + i] = rotated part (i < rot), 0 (offset + i < row_width).
template <typename T>
__global__ void latent_query_rotate_kernel(const T* q, T* qa, const float* __restrict__ freq, float amp,
                                           const int* __restrict__ positions, int heads, int dk, int rot, int rotary, int offset,
                                           int row_width, int halves) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  pdl_wait();
  const int tail = row_width - offset;
  for (int idx = threadIdx.x; idx < heads * tail; idx += blockDim.x) {
    const int h = idx / tail, i = idx % tail;
    float v = 0.f;
    if (i < rot) {
      const T* src = q + ((size_t)t * heads + h) * (dk + rot) + dk;
      v = to_f<T>(src[i]);
      if (halves && i < rotary) {
        const int half = rotary / 2, p = i < half ? i : i - half;
        float ra, rb;
        turn_pair(to_f<T>(src[p]), to_f<T>(src[p + half]), __fmul_rn((float)pos, freq[p]), amp, ra, rb);
        v = i < half ? ra : rb;
      } else if (!halves && (i | 1) < rotary) {
        float a = to_f<T>(src[i & ~1]), b = to_f<T>(src[i | 1]), ra, rb;
        turn_pair(a, b, __fmul_rn((float)pos, freq[i >> 1]), amp, ra, rb);
        v = (i & 1) ? rb : ra;
      }
    }
    qa[((size_t)t * heads + h) * row_width + offset + i] = from_f<T>(v);
  }
}

// y[t, h, o] = sum_i w[h][i][o] * x[t, h, i]; w is [heads, I, O] with O contiguous.  A block takes HL_TT tokens, one head and 32
// outputs; the tokens' inputs wait in shared memory as floats.  Warp k multiplies the inputs i = k, k + 8, ... (its loads of
// w do not depend on one another, so many are in flight: with a few tokens the kernel is a chain of memory latencies, and
// eight short chains side by side end eight times sooner than one); the eight partial sums of an output are then added in
// the order of the warps.  The order of operations of an output depends on I alone, not on the tile it falls into.
constexpr int HL_TT = 8, HL_WARPS = 8, HL_O = 32;

template <typename T>
__global__ void __launch_bounds__(HL_WARPS * 32)
head_linear_kernel(const T* x, long x_ts, long x_hs, const T* __restrict__ w, T* y, long y_ts, long y_hs, int tokens, int I, int O) {
  extern __shared__ float xs[];                 // [HL_TT][I], then the partial sums [HL_WARPS][HL_TT][HL_O]
  float* part = xs + HL_TT * I;
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, t0 = blockIdx.z * HL_TT, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int o = blockIdx.x * HL_O + lane;
  const int n = min(HL_TT, tokens - t0);
  for (int idx = threadIdx.x; idx < HL_TT * I; idx += HL_WARPS * 32) {
    const int tt = idx / I, i = idx % I;
    xs[idx] = tt < n ? to_f<T>(x[(size_t)(t0 + tt) * x_ts + (size_t)h * x_hs + i]) : 0.f;
  }
  __syncthreads();
  float acc[HL_TT];
#pragma unroll
  for (int tt = 0; tt < HL_TT; ++tt) acc[tt] = 0.f;
  if (o < O) {
    const T* wh = w + (size_t)h * I * O + o;
#pragma unroll 8
    for (int i = warp; i < I; i += HL_WARPS) {
      const float wv = to_f<T>(wh[(size_t)i * O]);
#pragma unroll
      for (int tt = 0; tt < HL_TT; ++tt) acc[tt] = fmaf(wv, xs[tt * I + i], acc[tt]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < HL_TT; ++tt) part[(warp * HL_TT + tt) * HL_O + lane] = acc[tt];
  __syncthreads();
  const int tt = warp;                          // eight warps, eight tokens: warp k sums token k's partial sums
  if (o < O && tt < n) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < HL_WARPS; ++k) s += part[(k * HL_TT + tt) * HL_O + lane];
    y[(size_t)(t0 + tt) * y_ts + (size_t)h * y_hs + o] = from_f<T>(s);
  }
}

// x[t, i] *= sigmoid(gate[t, i]) for the first `width` elements of every row (rows of x_stride / gate_stride elements).
template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* x, long x_stride, const T* gate, long gate_stride, int width, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / width, i = idx % width;
  const float g = to_f<T>(gate[t * gate_stride + i]);
  T* px = x + t * x_stride + i;
  *px = from_f<T>(to_f<T>(*px) / (1.f + expf(-g)));
}

template <typename T>
__global__ void sigmoid_gate_mul_vec_kernel(T* x, long x_stride, const T* gate, long gate_stride, int width, size_t chunks) {
  constexpr int N = Wide16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const int per_row = width / N;
  const size_t t = idx / per_row;
  const int i = (int)(idx % per_row) * N;
  float v[N], g[N];
  Wide16<T>::load(x + t * x_stride + i, v);
  Wide16<T>::load(gate + t * gate_stride + i, g);
#pragma unroll
  for (int j = 0; j < N; ++j) {
    // bfloat16 rows: the hardware's exponential and division (a float unit or two before a rounding to 8 bits)
    if (sizeof(T) == 2) v[j] = __fdividef(v[j], 1.f + __expf(-g[j]));
    else v[j] = v[j] / (1.f + expf(-g[j]));
  }
  Wide16<T>::store(x + t * x_stride + i, v);
}

}  // namespace vob

using namespace vob;

VOB_API int vob_sigmoid_gate_mul(void* x, long x_stride, const void* gate, long gate_stride, int T, int width, int dtype,
                                 cudaStream_t stream) {
  if (T <= 0 || width <= 0) return 0;
  const size_t total = (size_t)T * width;
  const int n = dtype == VOB_F32 ? 4 : 8;
  if (width % n == 0 && x_stride % n == 0 && gate_stride % n == 0 && (((uintptr_t)x | (uintptr_t)gate) & 15) == 0) {
    const size_t chunks = total / n;
    const dim3 vgrid((unsigned)((chunks + 255) / 256));
    if (dtype == VOB_F32)
      return launch_kernel(sigmoid_gate_mul_vec_kernel<float>, vgrid, dim3(256), 0, stream, (float*)x, x_stride,
                           (const float*)gate, gate_stride, width, chunks);
    if (dtype == VOB_BF16)
      return launch_kernel(sigmoid_gate_mul_vec_kernel<__nv_bfloat16>, vgrid, dim3(256), 0, stream, (__nv_bfloat16*)x, x_stride,
                           (const __nv_bfloat16*)gate, gate_stride, width, chunks);
  }
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == VOB_F32)
    return launch_kernel(sigmoid_gate_mul_kernel<float>, grid, dim3(256), 0, stream, (float*)x, x_stride, (const float*)gate,
                         gate_stride, width, total);
  if (dtype == VOB_BF16)
    return launch_kernel(sigmoid_gate_mul_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, x_stride,
                         (const __nv_bfloat16*)gate, gate_stride, width, total);
  return VOB_BAD_ARGUMENT;
}

// down [T, >= q_rank (+ kv_rank + rot)] rows of `stride` elements; wq [q_rank], wkv [kv_rank], freq [rotary/2] float;
// cq [T, q_rank]; cache: rows of row_width elements, one per slot; slots [T] (-1: skip).
VOB_API int vob_latent_prep(const void* down, long stride, const float* wq, const float* wkv, const float* freq, float amp,
                            const int* positions, const int* slots, void* cq, void* cache, int T, int q_rank, int kv_rank, int rot,
                            int rotary, int row_width, long num_slots, float eps, int has_kv, int halves, int dtype, int* err,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || (has_kv && (kv_rank <= 0 || rot < 0 || rotary > rot || (rotary & 1) || row_width < kv_rank + rot)))
    return VOB_BAD_ARGUMENT;
  if (dtype == VOB_F32)
    return launch_kernel(latent_prep_kernel<float>, dim3(T), dim3(LP_NT), 0, stream, (const float*)down, stride, wq, wkv, freq, amp,
                         positions, slots, (float*)cq, (float*)cache, q_rank, kv_rank, rot, rotary, row_width, num_slots, eps, has_kv,
                         halves, err);
  if (dtype == VOB_BF16)
    return launch_kernel(latent_prep_kernel<__nv_bfloat16>, dim3(T), dim3(LP_NT), 0, stream, (const __nv_bfloat16*)down, stride, wq,
                         wkv, freq, amp, positions, slots, (__nv_bfloat16*)cq, (__nv_bfloat16*)cache, q_rank, kv_rank, rot, rotary,
                         row_width, num_slots, eps, has_kv, halves, err);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_latent_query_rotate(const void* q, void* qa, const float* freq, float amp, const int* positions, int T, int heads,
                                    int dk, int rot, int rotary, int offset, int row_width, int halves, int dtype,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rotary > rot || (rotary & 1) || offset + rot > row_width) return VOB_BAD_ARGUMENT;
  if (row_width == offset) return 0;
  if (dtype == VOB_F32)
    return launch_kernel(latent_query_rotate_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)q, (float*)qa, freq, amp,
                         positions, heads, dk, rot, rotary, offset, row_width, halves);
  if (dtype == VOB_BF16)
    return launch_kernel(latent_query_rotate_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)q,
                         (__nv_bfloat16*)qa, freq, amp, positions, heads, dk, rot, rotary, offset, row_width, halves);
  return VOB_BAD_ARGUMENT;
}

// x: token stride x_ts, head stride x_hs (elements); w [heads, I, O]; y likewise.
VOB_API int vob_head_linear(const void* x, long x_ts, long x_hs, const void* w, void* y, long y_ts, long y_hs, int T, int heads,
                            int I, int O, int dtype, cudaStream_t stream) {
  if (T <= 0 || heads <= 0 || O <= 0) return 0;
  if (I <= 0) return VOB_BAD_ARGUMENT;
  const size_t smem = ((size_t)HL_TT * I + (size_t)HL_WARPS * HL_TT * HL_O) * sizeof(float);
  dim3 grid((O + HL_O - 1) / HL_O, heads, (T + HL_TT - 1) / HL_TT);
  if (smem > 48 * 1024 || grid.y > 65535 || grid.z > 65535) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return launch_kernel(head_linear_kernel<float>, grid, dim3(HL_WARPS * 32), smem, stream, (const float*)x, x_ts, x_hs, (const float*)w,
                         (float*)y, y_ts, y_hs, T, I, O);
  if (dtype == VOB_BF16)
    return launch_kernel(head_linear_kernel<__nv_bfloat16>, grid, dim3(HL_WARPS * 32), smem, stream, (const __nv_bfloat16*)x, x_ts, x_hs,
                         (const __nv_bfloat16*)w, (__nv_bfloat16*)y, y_ts, y_hs, T, I, O);
  return VOB_BAD_ARGUMENT;
}
