// Causal grouped-query attention over the paged cache, for any mix of prompt portions and
// single decoded tokens: the plain kernel.  It serves the true 32-bit path and every size the
// faster kernels refuse.
//
// One block per (token, query head).  The keys a query may read are lo..pos, with
// pos the query's position and lo = max(0, pos - window + 1) (0 without a window).  They are
// walked in tiles of 32 ALIGNED TO ABSOLUTE POSITIONS; tile j belongs to warp j % 4.  Any head size up to 512 (16-byte
// loads where a head's rows allow them).  Each
// warp keeps a running maximum, sum and weighted value sum in float (an online softmax), and
// the four warps are merged in a fixed order.  So the sequence of float operations for a
// query depends only on (lo, pos) and on the cache's contents at those positions: not on how
// the tokens were cut into steps, not on what else is in the batch, not on which pages hold
// the keys.  Scale 1/sqrt(hd) is applied to the score as the reference does
// (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:204-209); query head h reads key/value
// head h / (nh/kvh).
//
// Options that other mixers use: the value plane may have its own head size and fewer heads than the key plane (value
// head = key head * vkvh / kvh: neighbouring key heads share a value head); `softcap` > 0 bends the scaled score to
// softcap * tanh(score / softcap); `chunk` > 0 moves lo to the start of the query's block of `chunk` positions (blocks
// counted from position 0), so a query sees only keys of its own block; the output may be stored as float whatever T;
// `keep_first` > 0 lets every query also see the keys at positions below it, whatever the window or block (they keep their
// own positions); `dist_bias` [nh, dist_rows] float adds dist_bias[h][min(pos - key, dist_rows - 1)] to the scaled
// (and capped) score: a learned bias by distance.
#include "common.cuh"

namespace vob {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAXD = 16;  // value dims per lane: hd <= 512

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* q, const float* k, int hd) {
  float s = 0.f;
  if (hd % 4) {                        // rows that do not start on 16-byte boundaries: element by element
    for (int i = 0; i < hd; ++i) s += q[i] * k[i];
    return s;
  }
  const float4* k4 = reinterpret_cast<const float4*>(k);
  for (int i = 0; i < hd / 4; ++i) {
    const float4 v = k4[i];
    s += q[4 * i] * v.x; s += q[4 * i + 1] * v.y; s += q[4 * i + 2] * v.z; s += q[4 * i + 3] * v.w;
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* q, const __nv_bfloat16* k,
                                                         int hd) {
  float s = 0.f;
  if (hd % 8) {                        // rows that do not start on 16-byte boundaries: element by element
    for (int i = 0; i < hd; ++i) s += q[i] * __bfloat162float(k[i]);
    return s;
  }
  const uint4* k8 = reinterpret_cast<const uint4*>(k);
  for (int i = 0; i < hd / 8; ++i) {
    const uint4 raw = k8[i];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      s += q[8 * i + 2 * j] * f.x;
      s += q[8 * i + 2 * j + 1] * f.y;
    }
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_generic_kernel(const T* q, long q_stride, T* out,
                               const T* kcache, const T* vcache,
                               const int* __restrict__ block_tables, int table_stride,
                               const int* __restrict__ token_req, const int* __restrict__ positions,
                               const int* __restrict__ skip_single_cu_q, int nh, int kvh, int hd, int vd, int block_size,
                               int window, float scale, long num_pages, int sink, const T* gate, long gate_stride,
                               int vkvh, int v_row, float softcap, int chunk, int out_float, int keep_first,
                               const float* __restrict__ dist_bias, int dist_rows, int* err) {
  extern __shared__ float smem[];
  float* qs = smem;                        // [hd]
  float* accs = smem + hd;                 // [ATT_WARPS][vd]
  __shared__ float ms[ATT_WARPS], ls[ATT_WARPS];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int req = token_req[t];
  if (req < 0) return;
  if (skip_single_cu_q && skip_single_cu_q[req + 1] - skip_single_cu_q[req] == 1) return;  // the decode kernel's
  const int pos = positions[t];
  const int kh = h / (nh / kvh);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vh = (int)((long)kh * vkvh / kvh);
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (chunk > 0) lo = max(lo, pos / chunk * chunk);
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) qs[i] = to_f<T>(qrow[i]);
  __syncthreads();
  const int* table = block_tables + (size_t)req * table_stride;

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAXD];
#pragma unroll
  for (int j = 0; j < ATT_MAXD; ++j) acc[j] = 0.f;

  // kept first keys: the tiles that hold them are walked too, the ones between them and the window are passed over
  const int keep = min(max(keep_first, 0), lo);
  const int first_tile = keep > 0 ? 0 : lo / 32;
  for (int tile = first_tile + ((warp - first_tile % ATT_WARPS + ATT_WARPS) % ATT_WARPS); tile <= pos / 32; tile += ATT_WARPS) {
    if (tile * 32 >= keep && tile * 32 + 31 < lo) continue;
    const int key = tile * 32 + lane;
    const bool valid = (key >= lo || key < keep) && key <= pos;
    long row = -1;  // element offset of this key's row for kv head kh
    int page = -1;
    if (valid) {
      page = table[key / block_size];
      if (page < 0 || page >= num_pages) { atomicOr(err, VOB_ERR_PAGE); page = -1; }
      else row = (((long)page * kvh + kh) * block_size + key % block_size) * (long)hd;
    }
    float s = -INFINITY;
    if (row >= 0) {
      s = dot_row<T>(qs, kcache + row, hd) * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      if (dist_bias) s += dist_bias[(size_t)h * dist_rows + min(pos - key, dist_rows - 1)];
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (row >= 0) ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < ATT_MAXD; ++j) acc[j] *= corr;
    for (int kk = 0; kk < 32; ++kk) {
      const int pg = __shfl_sync(0xffffffffu, page, kk);
      if (pg < 0) continue;
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const T* vrow = vcache + (((long)pg * vkvh + vh) * block_size + (tile * 32 + kk) % block_size) * (long)v_row;
#pragma unroll
      for (int j = 0; j < ATT_MAXD; ++j) {
        const int d = lane + 32 * j;
        if (d < vd) acc[j] += pk * to_f<T>(vrow[d]);
      }
    }
    m = m_new;
  }
  if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
  for (int j = 0; j < ATT_MAXD; ++j) {
    const int d = lane + 32 * j;
    if (d < vd) accs[warp * vd + d] = acc[j];
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, ms[w]);
  // a sink is one more entry of score 0 that has no value: it adds exp(0 - max) to the denominator and nothing else
  if (sink) mm = fmaxf(mm, 0.f);
  float f[ATT_WARPS], lt = sink ? expf(-mm) : 0.f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) {
    f[w] = (ms[w] == -INFINITY) ? 0.f : expf(ms[w] - mm);
    lt += ls[w] * f[w];
  }
  // a gate: the head's output times sigmoid of one number of the token's row
  const float gt = gate ? 1.f / (1.f + expf(-to_f<T>(gate[(size_t)t * gate_stride + h]))) : 1.f;
  const size_t obase = (size_t)t * nh * vd + (size_t)h * vd;
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += accs[w * vd + d] * f[w];
    o = lt > 0.f ? o / lt * gt : 0.f;
    if (out_float) reinterpret_cast<float*>(out)[obase + d] = o;
    else out[obase + d] = from_f<T>(o);
  }
}

}  // namespace vob

using namespace vob;

// q: rows of q_stride elements, head h at h*hd; out [T, nh*vd]; caches [num_pages, kvh, block_size, hd];
// block_tables [B, table_stride]; token_req [T] (-1: padding); positions [T].  Of a value row the first vd elements are
// read (vd = hd: all of it; less when keys and values are one row and the key is the longer one).  `sink`: the softmax
// has a silent extra entry of score 0 (weights exp(s) / (1 + sum exp(s))); `gate` (rows of gate_stride elements, one
// number a head): head h of token t is multiplied by sigmoid(gate[t, h]).
// vkvh, v_row: heads and head size of the value plane [num_pages, vkvh, block_size, v_row] (0: those of the key plane);
// softcap, chunk, keep_first, dist_bias: see above (0 / null: off); out_float: out is float whatever `dtype`.
VOB_API int vob_paged_attention_generic(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                        const int* block_tables, int table_stride, const int* token_req,
                                        const int* positions, const int* skip_single_cu_q, int T, int nh, int kvh, int hd,
                                        int vd, int block_size,
                                        int window, float scale, long num_pages, int sink, const void* gate,
                                        long gate_stride, int vkvh, int v_row, float softcap, int chunk, int out_float,
                                        int keep_first, const float* dist_bias, int dist_rows,
                                        int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (vkvh <= 0) vkvh = kvh;
  if (v_row <= 0) v_row = hd;
  if (hd <= 0 || hd > 512 || kvh <= 0 || nh % kvh || block_size <= 0 || vd <= 0 || vd > v_row || vd > 512 || kvh % vkvh ||
      softcap < 0.f || chunk < 0 || keep_first < 0 || (dist_bias && dist_rows <= 0))
    return VOB_UNSUPPORTED;
  dim3 grid(T, nh);
  const size_t smem = (size_t)(hd + ATT_WARPS * vd) * sizeof(float);
  if (dtype == VOB_F32)
    return launch_kernel(paged_attention_generic_kernel<float>, grid, ATT_WARPS * 32, smem, stream, (const float*)q, q_stride,
                         (float*)out, (const float*)kcache, (const float*)vcache, block_tables, table_stride, token_req,
                         positions, skip_single_cu_q, nh, kvh, hd, vd, block_size, window, scale, num_pages, sink,
                         (const float*)gate, gate_stride, vkvh, v_row, softcap, chunk, out_float, keep_first, dist_bias, dist_rows, err);
  if (dtype == VOB_BF16)
    return launch_kernel(paged_attention_generic_kernel<__nv_bfloat16>, grid, ATT_WARPS * 32, smem, stream,
                         (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache,
                         (const __nv_bfloat16*)vcache, block_tables, table_stride, token_req, positions, skip_single_cu_q,
                         nh, kvh, hd, vd, block_size, window, scale, num_pages, sink, (const __nv_bfloat16*)gate,
                         gate_stride, vkvh, v_row, softcap, chunk, out_float, keep_first, dist_bias, dist_rows, err);
  return VOB_BAD_ARGUMENT;
}
