// What lies between the merged q|k|v product and attention, for mixers whose keys and values have sizes of their own, and
// what lies behind attention for heads that are the difference of two softmax maps.
//
//   rownorm_rope_kv_write   A token's row holds nh query heads and kvh key heads of kd elements, then vh value heads of vd
//                           elements (whatever follows is not touched).  With norm weights, q (all nh * kd elements at
//                           once) and k (all kvh * kd) each pass an RMS norm with a gain: x / sqrt(mean(x^2) + eps) * w
//                           (the mean counts kd_norm elements a head: heads padded with zeros behind them count as
//                           their own size).
//                           Then the first rot_dim elements of every q and k head turn by the angle float(position) *
//                           freq[i]: element 2i with 2i + 1 (`interleaved`) or i with i + rot_dim/2.  q is written back in
//                           place; k goes to the key plane [pages, kvh, block_size, kd] and v, as projected, to the value
//                           plane [pages, vh, block_size, vd], at the token's slot (-1 writes nothing).  Sums, norms, angles
//                           and the rotation are float on both paths and spelled out with rounding intrinsics.
//   diff_heads_combine      o = a1 - lambda * a2 per head (float), o / sqrt(mean(o^2) + eps) * post, times
//                           sigmoid(gate) element by element where a gate is given.  a holds, per key/value head, the
//                           first maps of its r query heads and then their second maps (the order in which attention ran
//                           them as 2 * heads plain heads); the output is in the heads' own order.
#include "common.cuh"

namespace vob {

constexpr int QP_NT = 256;
constexpr int QP_MAX_ROT = 512;   // the most elements of a head that turn

template <typename T>
__global__ void __launch_bounds__(QP_NT)
rownorm_rope_kv_write_kernel(T* qkv, long row_stride, const int* __restrict__ positions, const int* __restrict__ slots,
                             const float* __restrict__ wq, const float* __restrict__ wk, const float* __restrict__ freq,
                             T* kcache, T* vcache, int nh, int kvh, int kd, int vh, int vd, int rot_dim, int interleaved,
                             float eps, long num_slots, int block_size, int write_kv, int* err, int kd_norm) {
  __shared__ float scratch[32];
  __shared__ float2 turn[QP_MAX_ROT / 2];               // (cos, sin) of every angle
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  pdl_wait();
  if (pos < 0) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_POSITION);
    return;
  }
  const bool put = write_kv && slot >= 0;
  if (put && slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  T* row = qkv + (size_t)t * row_stride;
  const int nq = nh * kd, nk = kvh * kd, nv = vh * vd;
  const int half = rot_dim >> 1;
  // 16-bit rows whose heads and rotated parts are whole groups of 8 elements, with neighbours turning together, move by
  // 16-byte accesses (same arithmetic)
  const bool wide = sizeof(T) == 2 && kd % 8 == 0 && vd % 8 == 0 && rot_dim % 8 == 0 && (interleaved || rot_dim == 0) &&
                    row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0;
  // the angles' sines and cosines, once a token (every head turns by the same ones)
  for (int j = threadIdx.x; j < half; j += QP_NT) sincosf(__fmul_rn((float)pos, freq[j]), &turn[j].y, &turn[j].x);
  float inv_q = 1.f, inv_k = 1.f;
  if (wq) {
    // the sums of squares of q and of k, each added up in the same order whatever else the step holds
    float sq = 0.f, sk = 0.f;
    if (wide) {
      for (int i = threadIdx.x * 8; i < nq + nk; i += QP_NT * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) { const float x = __bfloat162float(e[c]); ss = fmaf(x, x, ss); }
        if (i < nq) sq += ss; else sk += ss;
      }
    } else {
      for (int i = threadIdx.x; i < nq; i += QP_NT) { const float x = to_f<T>(row[i]); sq = fmaf(x, x, sq); }
      for (int i = threadIdx.x; i < nk; i += QP_NT) { const float x = to_f<T>(row[nq + i]); sk = fmaf(x, x, sk); }
    }
    inv_q = 1.f / sqrtf(block_sum<QP_NT>(sq, scratch) / (float)(nh * kd_norm) + eps);
    inv_k = 1.f / sqrtf(block_sum<QP_NT>(sk, scratch) / (float)(kvh * kd_norm) + eps);
  } else {
    __syncthreads();                                    // the angles are there
  }
  const size_t page = put ? (size_t)(slot / block_size) : 0;
  const int in_page = put ? slot % block_size : 0;
  if (wide) {
    if constexpr (sizeof(T) == 2) {
      const int chunks = kd / 8;
      for (int it = threadIdx.x; it < (nh + kvh) * chunks; it += QP_NT) {
        const int head = it / chunks, a0 = it % chunks * 8;
        const bool is_q = head < nh;
        if (!is_q && !put) continue;
        if (is_q && !wq && a0 >= rot_dim) continue;            // nothing changes it
        const float inv = is_q ? inv_q : inv_k;
        const float* w = is_q ? wq : wk;
        const int hoff = is_q ? head * kd : (head - nh) * kd;
        T* src = row + (is_q ? 0 : nq) + hoff;
        T* dst = is_q ? src : kcache + ((page * kvh + (head - nh)) * block_size + in_page) * (size_t)kd;
        auto normed = [&](int at, float (&x)[8]) {
          const uint4 raw = *reinterpret_cast<const uint4*>(src + at);
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
          for (int c = 0; c < 8; ++c) x[c] = __bfloat162float(e[c]);
          if (w) {
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(w + hoff + at));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(w + hoff + at) + 1);
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) x[c] = __fmul_rn(__fmul_rn(x[c], inv), g[c]);
          }
        };
        float x[8], y[8];
        normed(a0, x);
        if (a0 < rot_dim) {
#pragma unroll
          for (int c = 0; c < 8; c += 2) {
            const float2 cs = turn[(a0 + c) >> 1];
            y[c] = __fsub_rn(__fmul_rn(x[c], cs.x), __fmul_rn(x[c + 1], cs.y));
            y[c + 1] = __fadd_rn(__fmul_rn(x[c + 1], cs.x), __fmul_rn(x[c], cs.y));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) y[c] = x[c];
        }
        uint4 packed;
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int c = 0; c < 4; ++c) p2[c] = __floats2bfloat162_rn(y[2 * c], y[2 * c + 1]);
        *reinterpret_cast<uint4*>(dst + a0) = packed;
      }
      if (put)
        for (int i = threadIdx.x * 8; i < nv; i += QP_NT * 8) {
          const int head = i / vd, d = i % vd;
          *reinterpret_cast<uint4*>(vcache + ((page * vh + head) * block_size + in_page) * (size_t)vd + d) =
              *reinterpret_cast<const uint4*>(row + nq + nk + i);
        }
    }
    return;
  }
  // q and k: a thread takes a pair of elements that turn together, or a single element behind the rotated part
  const int per_head = half + (kd - rot_dim);          // work items of a head
  const int items = (nh + kvh) * per_head;
  for (int it = threadIdx.x; it < items; it += QP_NT) {
    const int head = it / per_head, j = it % per_head;
    const bool is_q = head < nh;
    if (!is_q && !put) continue;
    const float inv = is_q ? inv_q : inv_k;
    const float* w = is_q ? wq : wk;
    const int hoff = is_q ? head * kd : (head - nh) * kd;       // offset within q, or within k
    T* src = row + (is_q ? 0 : nq) + hoff;
    T* dst = is_q ? src : kcache + ((page * kvh + (head - nh)) * block_size + in_page) * (size_t)kd;
    if (j < half) {
      const int a = interleaved ? 2 * j : j, b = interleaved ? 2 * j + 1 : j + half;
      float u = to_f<T>(src[a]), v = to_f<T>(src[b]);
      if (w) { u = __fmul_rn(__fmul_rn(u, inv), w[hoff + a]); v = __fmul_rn(__fmul_rn(v, inv), w[hoff + b]); }
      const float cs = turn[j].x, sn = turn[j].y;
      dst[a] = from_f<T>(__fsub_rn(__fmul_rn(u, cs), __fmul_rn(v, sn)));
      dst[b] = from_f<T>(__fadd_rn(__fmul_rn(v, cs), __fmul_rn(u, sn)));
    } else {
      const int a = rot_dim + (j - half);
      float u = to_f<T>(src[a]);
      if (w) u = __fmul_rn(__fmul_rn(u, inv), w[hoff + a]);
      if (w || !is_q) dst[a] = from_f<T>(u);
    }
  }
  if (put)
    for (int i = threadIdx.x; i < nv; i += QP_NT) {
      const int head = i / vd, d = i % vd;
      vcache[((page * vh + head) * block_size + in_page) * (size_t)vd + d] = row[nq + nk + i];
    }
}

// One warp a (token, head).  a: [tokens, 2 * heads * vd] of TA; out [tokens, heads * vd] of T; gate rows of gate_stride.
template <typename T, typename TA>
__global__ void __launch_bounds__(128)
diff_heads_combine_kernel(const TA* a, const T* gate, long gate_stride, T* out, int heads, int group, int vd, float lambda,
                          float post, float eps, int vd_norm) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * 4 + warp;
  if (h >= heads) return;
  const int g = h / group, hl = h % group;
  const TA* a1 = a + ((size_t)t * 2 * heads + (size_t)g * 2 * group + hl) * vd;
  const TA* a2 = a1 + (size_t)group * vd;
  float ss = 0.f;
  for (int d = lane; d < vd; d += 32) {
    const float o = __fsub_rn(to_f<TA>(a1[d]), __fmul_rn(lambda, to_f<TA>(a2[d])));
    ss = fmaf(o, o, ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)vd_norm + eps);
  for (int d = lane; d < vd; d += 32) {
    float o = __fsub_rn(to_f<TA>(a1[d]), __fmul_rn(lambda, to_f<TA>(a2[d]))) * inv * post;
    if (gate) o *= 1.f / (1.f + expf(-to_f<T>(gate[(size_t)t * gate_stride + (size_t)h * vd + d])));
    out[((size_t)t * heads + h) * vd + d] = from_f<T>(o);
  }
}

}  // namespace vob

using namespace vob;

VOB_API int vob_rownorm_rope_kv_write(void* qkv, long row_stride, const int* positions, const int* slots, const float* wq,
                                      const float* wk, const float* freq, void* kcache, void* vcache, int T, int nh, int kvh,
                                      int kd, int vh, int vd, int rot_dim, int interleaved, float eps, long num_slots,
                                      int block_size, int write_kv, int dtype, int kd_norm, int* err, cudaStream_t stream) {
  if (kd_norm <= 0 || kd_norm > kd) return VOB_BAD_ARGUMENT;
  if (T <= 0) return 0;
  if (kd <= 0 || vd <= 0 || nh <= 0 || kvh <= 0 || vh <= 0 || block_size <= 0 || rot_dim < 0 || rot_dim > kd || rot_dim % 2 ||
      (rot_dim > 0 && !freq) || (wq == nullptr) != (wk == nullptr) ||
      rot_dim > QP_MAX_ROT)
    return VOB_BAD_ARGUMENT;
  if (dtype == VOB_F32)
    return launch_kernel(rownorm_rope_kv_write_kernel<float>, dim3(T), QP_NT, 0, stream, (float*)qkv, row_stride, positions,
                         slots, wq, wk, freq, (float*)kcache, (float*)vcache, nh, kvh, kd, vh, vd, rot_dim, interleaved, eps,
                         num_slots, block_size, write_kv, err, kd_norm);
  if (dtype == VOB_BF16)
    return launch_kernel(rownorm_rope_kv_write_kernel<__nv_bfloat16>, dim3(T), QP_NT, 0, stream, (__nv_bfloat16*)qkv,
                         row_stride, positions, slots, wq, wk, freq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, kvh,
                         kd, vh, vd, rot_dim, interleaved, eps, num_slots, block_size, write_kv, err, kd_norm);
  return VOB_BAD_ARGUMENT;
}

// a: float (`a_float`) or `dtype`; gate (null: none) and out of `dtype`.  The mean counts vd_norm elements of a head (heads
// padded with zeros count as their own size).
VOB_API int vob_diff_heads_combine(const void* a, int a_float, const void* gate, long gate_stride, void* out, int T, int heads,
                                   int group, int vd, float lambda, float post, float eps, int dtype, int vd_norm,
                                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || group <= 0 || heads % group || vd <= 0 || vd_norm <= 0 || vd_norm > vd) return VOB_BAD_ARGUMENT;
  dim3 grid(T, (heads + 3) / 4);
#define VOB_DC(TYPE, TA)                                                                                              \
  return launch_kernel(diff_heads_combine_kernel<TYPE, TA>, grid, 128, 0, stream, (const TA*)a, (const TYPE*)gate,    \
                       gate_stride, (TYPE*)out, heads, group, vd, lambda, post, eps, vd_norm)
  if (dtype == VOB_F32) { VOB_DC(float, float); }
  if (dtype == VOB_BF16) {
    if (a_float) { VOB_DC(__nv_bfloat16, float); }
    VOB_DC(__nv_bfloat16, __nv_bfloat16);
  }
#undef VOB_DC
  return VOB_BAD_ARGUMENT;
}
