// What stands between short convolutions and paged attention when q, k and v come out of per-channel filters as floats:
//
//   unit_qk_kv_write:  a token's row [q heads | k heads | v heads] (float, the filters' output).  Every q head and every k
//                      head is divided by its root mean square over the head (x / sqrt(mean(x^2) + eps), no gain; `unit` 0
//                      leaves them as they are); q goes to a row of the model's type, k and v to the token's slot of the
//                      key plane [pages, kv heads, page, dim] and the value plane [pages, kv heads, page, vdim].  Heads in
//                      the planes may be wider than dim / vdim (`kd_row`, `vd_row`: heads padded for the tensor-core
//                      kernels): the tail is written as zeros, and q's heads are padded alike.
//
// The sums are float; a warp takes a head, so the order of additions depends on the head's size alone.
#include "common.cuh"

namespace vob {

template <typename T>
__global__ void __launch_bounds__(128)
unit_qk_kv_write_kernel(const float* x, const int* __restrict__ slots, T* q_out, T* kcache, T* vcache, int nh, int kvh, int dim,
                        int vdim, int kd_row, int vd_row, int block_size, long num_slots, float eps, int unit, int write_kv,
                        int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = write_kv ? slots[t] : -1;
  pdl_wait();
  const int C = (nh + kvh) * dim + kvh * vdim;
  const float* row = x + (size_t)t * C;
  if (write_kv && slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
  }
  const bool store_kv = write_kv && slot >= 0 && slot < num_slots;
  const long page = store_kv ? slot / block_size : 0, off = store_kv ? slot % block_size : 0;
  for (int head = warp; head < nh + 2 * kvh; head += 4) {
    if (head < nh + kvh) {
      const float* src = row + (size_t)head * dim;
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(src[d], src[d], ss);
      ss = warp_sum(ss);
      const float inv = unit ? 1.f / sqrtf(ss / (float)dim + eps) : 1.f;
      T* dst;
      if (head < nh) dst = q_out + ((size_t)t * nh + head) * kd_row;
      else if (store_kv) dst = kcache + ((page * kvh + (head - nh)) * block_size + off) * (long)kd_row;
      else continue;
      for (int d = lane; d < kd_row; d += 32) dst[d] = from_f<T>(d < dim ? src[d] * inv : 0.f);
    } else if (store_kv) {
      const int vh = head - nh - kvh;
      const float* src = row + (size_t)(nh + kvh) * dim + (size_t)vh * vdim;
      T* dst = vcache + ((page * kvh + vh) * block_size + off) * (long)vd_row;
      for (int d = lane; d < vd_row; d += 32) dst[d] = from_f<T>(d < vdim ? src[d] : 0.f);
    }
  }
}

}  // namespace vob

using namespace vob;

// x float [T, (nh + kvh) * dim + kvh * vdim]; slots [T] (-1: nothing is written); q_out [T, nh * kd_row];
// kcache [pages, kvh, block_size, kd_row]; vcache [pages, kvh, block_size, vd_row].
VOB_API int vob_unit_qk_kv_write(const float* x, const int* slots, void* q_out, void* kcache, void* vcache, int T, int nh, int kvh,
                                 int dim, int vdim, int kd_row, int vd_row, int block_size, long num_slots, float eps, int unit,
                                 int write_kv, int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nh <= 0 || kvh <= 0 || dim <= 0 || vdim <= 0 || kd_row < dim || vd_row < vdim || block_size <= 0) return VOB_BAD_ARGUMENT;
  if (dtype == VOB_F32)
    return launch_kernel(unit_qk_kv_write_kernel<float>, dim3(T), dim3(128), 0, stream, x, slots, (float*)q_out, (float*)kcache,
                         (float*)vcache, nh, kvh, dim, vdim, kd_row, vd_row, block_size, num_slots, eps, unit, write_kv, err);
  if (dtype == VOB_BF16)
    return launch_kernel(unit_qk_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, x, slots, (__nv_bfloat16*)q_out,
                         (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, kvh, dim, vdim, kd_row, vd_row, block_size, num_slots,
                         eps, unit, write_kv, err);
  return VOB_BAD_ARGUMENT;
}
