// One float residual stream around layers whose two sublayers read ONE norm ("parallel" layers):
//
//     h = LayerNorm(x) * w + b;      x <- x + (mixer(h) + feed_forward(h))
//
// One launch does, for every token, in a single pass over the row:
//   (1) x = 0 (`init`: the row begins here, with the embedded token as y1) or x = stream[token];
//   (2) x += (y1 + y2)        the outputs of the layer before, either may be absent; the bracket is summed first;
//   (3) x is stored to the stream if (1)-(2) changed it;
//   (4) with w:  out = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b      (b may be absent).
// With a list of rows, (4) is computed for those source rows only and nothing is stored (the model's last norm on the
// rows whose logits are wanted).
//
// The stream, the mean, the variance and the sums are float on both paths; y1, y2 and out are of the model's type T.  The
// variance is the mean of the squared deviations from the mean (two passes over the row, which lies in shared memory).
// A block of fixed size takes a row, so the order of additions depends on the row's width only.
#include "common.cuh"

namespace vob {

constexpr int PN_NT = 256;

// Four neighbouring elements of the model's type as floats, by one access.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T>
__global__ void __launch_bounds__(PN_NT)
layer_norm_step_kernel(float* stream, const T* y1, const T* y2, const float* __restrict__ w, const float* __restrict__ b,
                       T* out, const int* __restrict__ rows, int num_src_rows, int D, float eps, int init, int* err, int wide) {
  extern __shared__ __align__(16) float pn_row[];    // [D] the new row
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  int src = r;
  if (rows) {
    src = rows[r];
    if (src < 0 || src >= num_src_rows) {
      if (threadIdx.x == 0) atomicOr(err, VOB_ERR_ROW);
      return;
    }
  }
  const size_t base = (size_t)src * D;
  const bool changed = init || y1 || y2;
  const bool store = rows == nullptr && changed;
  if (wide) {
    // widths that are a multiple of 4 (every pointer 16-byte aligned): a thread takes four neighbours an access; the order
    // of a row's additions still depends on its width alone
    float sum = 0.f;
    for (int d = threadIdx.x * 4; d < D; d += PN_NT * 4) {
      float x[4] = {0.f, 0.f, 0.f, 0.f}, a[4], c[4];
      if (!init) load4(stream + base + d, x);
      if (y1) load4(y1 + base + d, a);
      if (y2) load4(y2 + base + d, c);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (y1 && y2) x[i] += a[i] + c[i];
        else if (y1) x[i] += a[i];
        else if (y2) x[i] += c[i];
        sum += x[i];
      }
      if (store) store4(stream + base + d, x);
      store4(pn_row + d, x);
    }
    if (!out) return;
    const float mean = block_sum<PN_NT>(sum, scratch) / (float)D;
    float sq = 0.f;
    for (int d = threadIdx.x * 4; d < D; d += PN_NT * 4) {
      float x[4];
      load4(pn_row + d, x);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float c = x[i] - mean; sq = fmaf(c, c, sq); }
    }
    const float inv = 1.f / sqrtf(block_sum<PN_NT>(sq, scratch) / (float)D + eps);
    for (int d = threadIdx.x * 4; d < D; d += PN_NT * 4) {
      float x[4], g[4], o[4], bias[4] = {0.f, 0.f, 0.f, 0.f};
      load4(pn_row + d, x);
      load4(w + d, g);
      if (b) load4(b + d, bias);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = (x[i] - mean) * inv * g[i] + bias[i];
      store4(out + (size_t)r * D + d, o);
    }
    return;
  }
  float sum = 0.f;
  for (int d = threadIdx.x; d < D; d += PN_NT) {
    float x = init ? 0.f : stream[base + d];
    if (y1 && y2) x += to_f<T>(y1[base + d]) + to_f<T>(y2[base + d]);
    else if (y1) x += to_f<T>(y1[base + d]);
    else if (y2) x += to_f<T>(y2[base + d]);
    if (store) stream[base + d] = x;
    pn_row[d] = x;
    sum += x;
  }
  if (!out) return;
  const float mean = block_sum<PN_NT>(sum, scratch) / (float)D;
  float sq = 0.f;
  for (int d = threadIdx.x; d < D; d += PN_NT) {
    const float c = pn_row[d] - mean;
    sq = fmaf(c, c, sq);
  }
  const float inv = 1.f / sqrtf(block_sum<PN_NT>(sq, scratch) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += PN_NT) {
    const float o = (pn_row[d] - mean) * inv * w[d] + (b ? b[d] : 0.f);
    out[(size_t)r * D + d] = from_f<T>(o);
  }
}


// The same pass with an RMS norm instead: x = y1 * open_scale (`init`: the row begins here with the embedded token) or
// x = stream[token] + mult * (y1 + y2); the row is stored; out = x / sqrt(mean(x^2) + eps) * (gain_offset + w)
// (gain_offset 1: a gain stored around zero; 0: a plain gain).  Float throughout; y1, y2, out of the model's type T.
template <typename T>
__global__ void __launch_bounds__(PN_NT)
rms_norm_step_kernel(float* stream, const T* y1, const T* y2, const float* __restrict__ w, T* out, const int* __restrict__ rows,
                     int num_src_rows, int D, float eps, int init, float mult, float open_scale, float gain_offset, int* err,
                     int wide) {
  extern __shared__ __align__(16) float pn_row[];    // [D] the new row
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  int src = r;
  if (rows) {
    src = rows[r];
    if (src < 0 || src >= num_src_rows) {
      if (threadIdx.x == 0) atomicOr(err, VOB_ERR_ROW);
      return;
    }
  }
  const size_t base = (size_t)src * D;
  const bool store = rows == nullptr && (init || y1 || y2);
  float sq = 0.f;
  const int step = wide ? 4 : 1;
  for (int d = threadIdx.x * step; d < D; d += PN_NT * step) {
    float x[4] = {0.f, 0.f, 0.f, 0.f}, a[4] = {0.f, 0.f, 0.f, 0.f}, c[4] = {0.f, 0.f, 0.f, 0.f};
    if (wide) {
      if (!init) load4(stream + base + d, x);
      if (y1) load4(y1 + base + d, a);
      if (y2) load4(y2 + base + d, c);
    } else {
      if (!init) x[0] = stream[base + d];
      if (y1) a[0] = to_f<T>(y1[base + d]);
      if (y2) c[0] = to_f<T>(y2[base + d]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i >= step) break;
      if (init) x[i] = __fmul_rn(a[i], open_scale);
      else if (y1 || y2) x[i] = __fadd_rn(x[i], __fmul_rn(mult, __fadd_rn(a[i], c[i])));
      sq = fmaf(x[i], x[i], sq);
      pn_row[d + i] = x[i];
    }
    if (store) {
      if (wide) store4(stream + base + d, x);
      else stream[base + d] = x[0];
    }
  }
  if (!out) return;
  const float inv = 1.f / sqrtf(block_sum<PN_NT>(sq, scratch) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += PN_NT)
    out[(size_t)r * D + d] = from_f<T>(pn_row[d] * inv * (gain_offset + w[d]));
}

// out = 0.5 * (a / rms(a) * wa + b / rms(b) * wb): two mixers side by side over the same input, each with an RMS norm over
// the width (plain gains), then their mean.  One block a token; float sums.
template <typename T>
__global__ void __launch_bounds__(PN_NT)
pair_norm_mean_kernel(const T* a, const T* b, const float* __restrict__ wa, const float* __restrict__ wb, T* out, int D,
                      float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * D;
  float sa = 0.f, sb = 0.f;
  for (int d = threadIdx.x; d < D; d += PN_NT) {
    const float x = to_f<T>(a[base + d]), y = to_f<T>(b[base + d]);
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  const float ia = 1.f / sqrtf(block_sum<PN_NT>(sa, scratch) / (float)D + eps);
  const float ib = 1.f / sqrtf(block_sum<PN_NT>(sb, scratch) / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += PN_NT)
    out[base + d] = from_f<T>(0.5f * (to_f<T>(a[base + d]) * ia * wa[d] + to_f<T>(b[base + d]) * ib * wb[d]));
}

}  // namespace vob

using namespace vob;

// stream [num_src_rows, D] float; y1, y2 [num_src_rows, D] and out [n_out, D] of `dtype`; w, b [D] float; rows [n_out]
// source rows or null (then n_out == num_src_rows).  Any of y1, y2, b and w / out may be null.
VOB_API int vob_layer_norm_step(float* stream, const void* y1, const void* y2, const float* w, const float* b, void* out,
                                const int* rows, int n_out, int num_src_rows, int D, float eps, int init, int dtype, int* err,
                                cudaStream_t stream_) {
  if (n_out <= 0) return 0;
  if (D <= 0 || (rows && !out) || (out && !w)) return VOB_BAD_ARGUMENT;
  const size_t smem = (size_t)D * sizeof(float);
  if (smem > 200 * 1024) return VOB_UNSUPPORTED;
  const int wide = D % 4 == 0 && (((uintptr_t)stream | (uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
#define VOB_PN_LAUNCH(TYPE)                                                                                             \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(layer_norm_step_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    return launch_kernel(layer_norm_step_kernel<TYPE>, dim3(n_out), PN_NT, smem, stream_, stream, (const TYPE*)y1,      \
                         (const TYPE*)y2, w, b, (TYPE*)out, rows, num_src_rows, D, eps, init, err, wide);                     \
  } while (0)
  if (dtype == VOB_F32) VOB_PN_LAUNCH(float);
  if (dtype == VOB_BF16) VOB_PN_LAUNCH(__nv_bfloat16);
#undef VOB_PN_LAUNCH
  return VOB_BAD_ARGUMENT;
}

// As vob_layer_norm_step with an RMS norm: see rms_norm_step_kernel.  w [D] float; b is not taken.
VOB_API int vob_rms_norm_step(float* stream, const void* y1, const void* y2, const float* w, void* out, const int* rows, int n_out,
                              int num_src_rows, int D, float eps, int init, float mult, float open_scale, float gain_offset,
                              int dtype, int* err, cudaStream_t stream_) {
  if (n_out <= 0) return 0;
  if (D <= 0 || (rows && !out) || (out && !w) || (init && !y1)) return VOB_BAD_ARGUMENT;
  const size_t smem = (size_t)D * sizeof(float);
  if (smem > 200 * 1024) return VOB_UNSUPPORTED;
  const int wide = D % 4 == 0 && (((uintptr_t)stream | (uintptr_t)y1 | (uintptr_t)y2) & 15) == 0;
#define VOB_RN_LAUNCH(TYPE)                                                                                             \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(rms_norm_step_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    return launch_kernel(rms_norm_step_kernel<TYPE>, dim3(n_out), PN_NT, smem, stream_, stream, (const TYPE*)y1,        \
                         (const TYPE*)y2, w, (TYPE*)out, rows, num_src_rows, D, eps, init, mult, open_scale, gain_offset, \
                         err, wide);                                                                                    \
  } while (0)
  if (dtype == VOB_F32) VOB_RN_LAUNCH(float);
  if (dtype == VOB_BF16) VOB_RN_LAUNCH(__nv_bfloat16);
#undef VOB_RN_LAUNCH
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_pair_norm_mean(const void* a, const void* b, const float* wa, const float* wb, void* out, int T, int D, float eps,
                               int dtype, cudaStream_t stream) {
  if (T <= 0 || D <= 0) return 0;
  if (dtype == VOB_F32)
    return launch_kernel(pair_norm_mean_kernel<float>, dim3(T), PN_NT, 0, stream, (const float*)a, (const float*)b, wa, wb,
                         (float*)out, D, eps);
  if (dtype == VOB_BF16)
    return launch_kernel(pair_norm_mean_kernel<__nv_bfloat16>, dim3(T), PN_NT, 0, stream, (const __nv_bfloat16*)a,
                         (const __nv_bfloat16*)b, wa, wb, (__nv_bfloat16*)out, D, eps);
  return VOB_BAD_ARGUMENT;
}
