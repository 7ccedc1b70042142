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

template <typename T>
__global__ void __launch_bounds__(PN_NT)
layer_norm_step_kernel(float* stream, const T* y1, const T* y2, const float* __restrict__ w, const float* __restrict__ b,
                       T* out, const int* __restrict__ rows, int num_src_rows, int D, float eps, int init, int* err) {
  extern __shared__ float pn_row[];    // [D] the new row
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
#define VOB_PN_LAUNCH(TYPE)                                                                                             \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(layer_norm_step_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    return launch_kernel(layer_norm_step_kernel<TYPE>, dim3(n_out), PN_NT, smem, stream_, stream, (const TYPE*)y1,      \
                         (const TYPE*)y2, w, b, (TYPE*)out, rows, num_src_rows, D, eps, init, err);                     \
  } while (0)
  if (dtype == VOB_F32) VOB_PN_LAUNCH(float);
  if (dtype == VOB_BF16) VOB_PN_LAUNCH(__nv_bfloat16);
#undef VOB_PN_LAUNCH
  return VOB_BAD_ARGUMENT;
}
