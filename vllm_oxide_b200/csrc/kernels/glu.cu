// A gated feed-forward's activation with clamps, and a bias added to rows.
//
//   clamped_glu:  g = min(gate + b_gate, limit);  u = clamp(up + b_up, -limit, limit);  out = g * sigmoid(alpha * g) * (u + 1).
//                 The input row holds the gate's columns, then the up columns; the biases (float, optional) lie alike.
//   add_bias:     x[t, :] += b  (float b, x of the model's type).
//
// The arithmetic is float; inputs and outputs are of the model's type T.
#include "common.cuh"

namespace vob {

template <typename T>
__global__ void clamped_glu_kernel(const T* gu, long gu_stride, const float* __restrict__ bias, T* out, int I, float limit,
                                   float alpha, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I, i = idx % I;
  float g = to_f<T>(gu[t * gu_stride + i]), u = to_f<T>(gu[t * gu_stride + I + i]);
  if (bias) { g += bias[i]; u += bias[I + i]; }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  out[idx] = from_f<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// The same, a 16-byte access of gate, up and out a thread (I a multiple of the access, rows that start on 16-byte boundaries).
template <typename T>
__global__ void clamped_glu_vec_kernel(const T* gu, long gu_stride, const float* __restrict__ bias, T* out, int I, float limit,
                                       float alpha, size_t chunks) {
  constexpr int N = Wide16<T>::N;
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const int per_row = I / N;
  const size_t t = idx / per_row;
  const int i = (int)(idx % per_row) * N;
  float g[N], u[N], y[N];
  Wide16<T>::load(gu + t * gu_stride + i, g);
  Wide16<T>::load(gu + t * gu_stride + I + i, u);
  if (bias) {
    // (I and i are multiples of four: the biases come four at a time)
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      const float4 bg = *reinterpret_cast<const float4*>(bias + i + j), bu = *reinterpret_cast<const float4*>(bias + I + i + j);
      g[j] += bg.x; g[j + 1] += bg.y; g[j + 2] += bg.z; g[j + 3] += bg.w;
      u[j] += bu.x; u[j + 1] += bu.y; u[j + 2] += bu.z; u[j + 3] += bu.w;
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float a = fminf(g[j], limit), b = fminf(fmaxf(u[j], -limit), limit);
    // bfloat16 rows: the hardware's exponential and division, as SiLU * up takes them for portions (a float unit or two
    // before a rounding to 8 bits); float rows: the accurate ones
    if (sizeof(T) == 2) y[j] = __fdividef(a, 1.f + __expf(-alpha * a)) * (b + 1.f);
    else y[j] = a / (1.f + expf(-alpha * a)) * (b + 1.f);
  }
  Wide16<T>::store(out + t * I + i, y);
}

template <typename T>
__global__ void add_bias_kernel(T* x, const float* __restrict__ bias, int D, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  x[idx] = from_f<T>(to_f<T>(x[idx]) + bias[idx % D]);
}

}  // namespace vob

using namespace vob;

// gu [T, 2 * I] rows of gu_stride elements; bias float [2 * I] or null; out [T, I] contiguous.
VOB_API int vob_clamped_glu(const void* gu, long gu_stride, const float* bias, void* out, int T, int I, float limit, float alpha,
                            int dtype, cudaStream_t stream) {
  if (T <= 0 || I <= 0) return 0;
  if (!(limit > 0.f)) return VOB_BAD_ARGUMENT;
  const size_t total = (size_t)T * I;
  const int n = dtype == VOB_F32 ? 4 : 8;
  if (I % n == 0 && gu_stride % n == 0 && (((uintptr_t)gu | (uintptr_t)out | (uintptr_t)bias) & 15) == 0) {
    const size_t chunks = total / n;
    const dim3 vgrid((unsigned)((chunks + 255) / 256));
    if (dtype == VOB_F32)
      return launch_kernel(clamped_glu_vec_kernel<float>, vgrid, dim3(256), 0, stream, (const float*)gu, gu_stride, bias,
                           (float*)out, I, limit, alpha, chunks);
    if (dtype == VOB_BF16)
      return launch_kernel(clamped_glu_vec_kernel<__nv_bfloat16>, vgrid, dim3(256), 0, stream, (const __nv_bfloat16*)gu, gu_stride,
                           bias, (__nv_bfloat16*)out, I, limit, alpha, chunks);
  }
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == VOB_F32)
    return launch_kernel(clamped_glu_kernel<float>, grid, dim3(256), 0, stream, (const float*)gu, gu_stride, bias, (float*)out, I,
                         limit, alpha, total);
  if (dtype == VOB_BF16)
    return launch_kernel(clamped_glu_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)gu, gu_stride, bias,
                         (__nv_bfloat16*)out, I, limit, alpha, total);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_add_bias(void* x, const float* bias, int T, int D, int dtype, cudaStream_t stream) {
  if (T <= 0 || D <= 0) return 0;
  const size_t total = (size_t)T * D;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == VOB_F32)
    return launch_kernel(add_bias_kernel<float>, grid, dim3(256), 0, stream, (float*)x, bias, D, total);
  if (dtype == VOB_BF16)
    return launch_kernel(add_bias_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, bias, D, total);
  return VOB_BAD_ARGUMENT;
}
