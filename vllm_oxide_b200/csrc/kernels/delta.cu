// The gated delta rule: a matrix state per head that forgets by a decay and is corrected toward each new value.
//
// Per head, with S [dim, vdim] float, carried from token to token in the request's state slot (stored [vdim][dim]):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
// q and k are unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2); beta = sigmoid(b);
// g = exp(-exp(A_log) * softplus(a + dt_bias)): one number a head, or (`channel_decay`) one a head and key channel, which
// multiplies that row of S (a and dt_bias are then [heads, dim]).  q, k and v come out of short causal convolutions over time (one filter a
// channel, `taps` taps, the last one the current token's) followed by SiLU; the last taps - 1 inputs of every channel are
// part of the request's state, behind S in the same slot.  Query/key head h / (heads / kv_heads) serves value head h.
//
// Four kernels (short_conv_step is the first two in one, for steps of short portions):
//   short_conv_silu    out[t, c] = f(sum_j w[c, j] x[t - (taps-1) + j, c]), inputs before the portion's start from the slot;
//                      f is SiLU or (`act` 0) the identity
//   short_conv_state   the slot's taps - 1 inputs after this portion (run after the first: it overwrites what that one reads)
//   delta_scan         the recurrence.  A column of S lives in the registers of LANES threads (ROWS rows each, rows
//                      interleaved so that a warp's loads of the state fill whole sectors); a block takes the columns
//                      c0.. of one (request, head) and walks the request's tokens in order, while half of its warps
//                      prepare the next tokens in shared memory (unit vectors, decay and beta are made there, in float).
//   delta_out_norm     o / sqrt(mean(o^2) + eps) * w * SiLU(gate) (or * sigmoid(gate)), per head over vdim
// Everything but the inputs' type T is float on both paths.  The chain of operations of an output depends only on the
// request's tokens and the state it starts from, not on the cut, the batch or the slot.
#include "common.cuh"

namespace vob {

constexpr int DELTA_MAX_TAPS = 9;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

constexpr int CONV_TOKENS = 8;    // tokens a thread walks in a large step: the filter's window slides through registers

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_silu_kernel(const T* x, long x_stride, const float* __restrict__ w, const float* state, long state_stride,
                       long conv_off, const int* __restrict__ token_req, const int* __restrict__ cu_q,
                       const int* __restrict__ state_slots, float* out, int num_tokens, int walk, int C, int taps, long num_slots,
                       int act, int* err) {
  pdl_launch_dependents();
  const int t_first = blockIdx.x * walk;
  const int c = blockIdx.y * 128 + threadIdx.x;
  float wt[DELTA_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS; ++s) wt[s] = (c < C && s < taps) ? w[(size_t)c * taps + s] : 0.f;
  const float w_now = c < C ? w[(size_t)c * taps + taps - 1] : 0.f;      // the current token's tap
  pdl_wait();
  if (c >= C) return;
  float win[DELTA_MAX_TAPS - 1];      // win[s]: the input taps - 1 - s tokens back
  bool have = false;
  for (int tt = 0; tt < walk; ++tt) {
    const int t = t_first + tt;
    if (t >= num_tokens) break;
    const int req = token_req[t];
    if (req < 0) { have = false; continue; }
    const int j = t - cu_q[req];
    if (!have || j == 0) {            // the window is filled anew at the start of the thread's tokens and of a portion
      const int slot = state_slots[req];
      if (slot < 0 || slot >= num_slots) {
        atomicOr(err, VOB_ERR_SLOT);
        have = false;
        continue;
      }
      const float* st = state + (size_t)slot * state_stride + conv_off;
#pragma unroll
      for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) {
        if (s < taps - 1) {
          const int rel = j - (taps - 1) + s;      // place within the portion; before its start the slot has the input
          win[s] = rel >= 0 ? to_f<T>(x[(size_t)(t - (taps - 1) + s) * x_stride + c]) : st[(size_t)(taps - 1 + rel) * C + c];
        }
      }
      have = true;
    }
    const float cur = to_f<T>(x[(size_t)t * x_stride + c]);
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s)
      if (s < taps - 1) acc = fmaf(wt[s], win[s], acc);          // oldest input first
    acc = fmaf(w_now, cur, acc);
    out[(size_t)t * C + c] = act ? silu_f(acc) : acc;
#pragma unroll
    for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) {
      if (s < taps - 2) win[s] = win[s + 1 < DELTA_MAX_TAPS - 1 ? s + 1 : s];
      else if (s == taps - 2) win[s] = cur;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_state_kernel(const T* x, long x_stride, float* state, long state_stride, long conv_off,
                        const int* __restrict__ cu_q, const int* __restrict__ state_slots, int C, int taps, long num_slots) {
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int t0 = cu_q[b], n = cu_q[b + 1] - t0;
  const int slot = state_slots[b];
  pdl_wait();
  if (n <= 0 || slot < 0 || slot >= num_slots || c >= C) return;
  float* st = state + (size_t)slot * state_stride + conv_off;
  float nv[DELTA_MAX_TAPS - 1];
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) {
    if (s < taps - 1) {
      const int rel = n - (taps - 1) + s;     // place within the portion of the input that entry s holds afterwards
      nv[s] = rel >= 0 ? to_f<T>(x[(size_t)(t0 + rel) * x_stride + c]) : st[(size_t)(s + n) * C + c];
    }
  }
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s)
    if (s < taps - 1) st[(size_t)s * C + c] = nv[s];
}

// Both of the above in one launch for steps whose portions are short (decoding): a thread owns one channel of one request,
// takes its window from the slot, walks the request's few tokens and leaves the window in the slot.  The same sums in the
// same order as the two kernels.
template <typename T>
__global__ void __launch_bounds__(128)
short_conv_step_kernel(const T* x, long x_stride, const float* __restrict__ w, float* state, long state_stride, long conv_off,
                       const int* __restrict__ cu_q, const int* __restrict__ state_slots, float* out, int C, int taps,
                       long num_slots, int act, int* err) {
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int t0 = cu_q[b], n = cu_q[b + 1] - t0;
  const int slot = state_slots[b];
  float wt[DELTA_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS; ++s) wt[s] = (c < C && s < taps) ? w[(size_t)c * taps + s] : 0.f;
  const float w_now = c < C ? w[(size_t)c * taps + taps - 1] : 0.f;
  pdl_wait();
  if (n <= 0) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  if (c >= C) return;
  float* st = state + (size_t)slot * state_stride + conv_off;
  float win[DELTA_MAX_TAPS - 1];
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) win[s] = s < taps - 1 ? st[(size_t)s * C + c] : 0.f;
  for (int i = 0; i < n; ++i) {
    const float cur = to_f<T>(x[(size_t)(t0 + i) * x_stride + c]);
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s)
      if (s < taps - 1) acc = fmaf(wt[s], win[s], acc);
    acc = fmaf(w_now, cur, acc);
    out[(size_t)(t0 + i) * C + c] = act ? silu_f(acc) : acc;
#pragma unroll
    for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) {
      if (s < taps - 2) win[s] = win[s + 1 < DELTA_MAX_TAPS - 1 ? s + 1 : s];
      else if (s == taps - 2) win[s] = cur;
    }
  }
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s)
    if (s < taps - 1) st[(size_t)s * C + c] = win[s];
}

// ---------------------------------------------------------------- the recurrence
constexpr int DS_COMPUTE = 128;   // threads that hold the state
constexpr int DS_LOADERS = 128;   // threads that prepare the next tokens meanwhile
constexpr int DS_THREADS = DS_COMPUTE + DS_LOADERS;

__device__ __forceinline__ void named_sync(int id, int count) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;\n" ::"r"(id), "r"(count) : "memory"); }

// qkv: float [tokens, 2 * kvh * dim + heads * vdim] (q heads, k heads, v heads: the convolutions' output);
// ab: rows of ab_stride elements of T, beta's pre-activation of head h at b_off + h, the decay's at a_off + h.
// A column of the state is held by LANES neighbouring threads, ROWS rows each (LANES * ROWS >= dim); 128 such threads
// walk the tokens, CH at a time from one of two buffers in shared memory, while four more warps fill the other buffer:
// unit vectors (laid out so that a thread finds its rows side by side), decay, beta and the block's slice of the values.
// The two groups meet on named barriers: "full" when a buffer is ready, "empty" when its tokens have been walked.
template <typename T, int LANES, int ROWS, bool CHD>
__global__ void __launch_bounds__(DS_THREADS)
delta_scan_kernel(const float* qkv, const T* ab, long ab_stride, int b_off, int a_off, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, float* state, long state_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, float* raw, int heads, int kvh, int dim, int vdim, long num_slots,
                  int* err) {
  constexpr int COLS = DS_COMPUTE / LANES;
  constexpr int RS = ROWS + 4;                 // a thread's rows in shared memory, 16 bytes apart from the next thread's:
  constexpr int KW = LANES * RS;               // the 16-byte reads of a column's LANES threads then fall into different banks
  constexpr int CH = ROWS > 16 ? 8 : 16;       // tokens a buffer holds
  constexpr int BUF = CH * ((CHD ? 3 : 2) * KW + COLS + 2);     // CHD: a decay for every row of the head beside k and q
  extern __shared__ __align__(16) float ds_smem[];
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int tid = threadIdx.x, lane = tid & 31;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int slot = state_slots[b];
  const float neg_rate = -expf(A_log[h]), bias = CHD ? 0.f : dt_bias[h];
  pdl_wait();
  if (t1 <= t0) return;
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const int kh = h / (heads / kvh);
  const int C = 2 * kvh * dim + heads * vdim;
  const int chunks = (t1 - t0 + CH - 1) / CH;
  if (tid >= DS_COMPUTE) {
    // ------------------------------------------------ loaders
    const int lw = (tid - DS_COMPUTE) >> 5;
    const float qscale = 1.f / sqrtf((float)dim);
    for (int c = 0; c < chunks; ++c) {
      float* ks = ds_smem + (c & 1) * BUF;
      float* qs = ks + CH * KW;
      float* vs = qs + CH * KW;
      float* gs = vs + CH * COLS;
      float* bs = gs + CH;
      float* gv = bs + CH;                                    // CHD: [CH][KW], laid out as ks
      if (c >= 2) named_sync(3 + (c & 1), DS_THREADS);        // the walkers have left this buffer
      const int base = t0 + c * CH, n = min(CH, t1 - base);
      // a warp takes tokens lw, lw + 4, ...: all their loads are issued before the first sum is taken
      constexpr int NV = (LANES * ROWS + 31) / 32, TPW = CH / (DS_LOADERS / 32);
      float qv[TPW][NV], kv[TPW][NV], av[CHD ? TPW : 1][CHD ? NV : 1];
#pragma unroll
      for (int tt = 0; tt < TPW; ++tt) {
        const int i = lw + tt * (DS_LOADERS / 32);
        const float* qrow = qkv + (size_t)(base + min(i, n - 1)) * C + (size_t)kh * dim;
        const float* krow = qrow + (size_t)kvh * dim;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int d = lane + 32 * j;
          const bool ok = i < n && d < dim;
          qv[tt][j] = ok ? qrow[d] : 0.f;
          kv[tt][j] = ok ? krow[d] : 0.f;
          if constexpr (CHD)      // the decay's pre-activation of (head h, key channel d), with its bias
            av[tt][j] = ok ? to_f<T>(ab[(size_t)(base + i) * ab_stride + a_off + (size_t)h * dim + d]) + dt_bias[(size_t)h * dim + d]
                           : 0.f;
        }
      }
      if (lane < TPW && lw + lane * (DS_LOADERS / 32) < n) {
        const int i = lw + lane * (DS_LOADERS / 32);
        const T* abrow = ab + (size_t)(base + i) * ab_stride;
        const float bv = to_f<T>(abrow[b_off + h]);
        bs[i] = 1.f / (1.f + expf(-bv));
        if (!CHD) {
          const float a1 = to_f<T>(abrow[a_off + h]) + bias;
          const float sp = a1 > 20.f ? a1 : log1pf(expf(a1));
          gs[i] = expf(neg_rate * sp);
        }
      }
#pragma unroll
      for (int tt = 0; tt < TPW; ++tt) {
        const int i = lw + tt * (DS_LOADERS / 32);
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          sq = fmaf(qv[tt][j], qv[tt][j], sq);
          sk = fmaf(kv[tt][j], kv[tt][j], sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (i >= n) continue;
        const float iq = qscale / sqrtf(sq + 1e-6f), ik = 1.f / sqrtf(sk + 1e-6f);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int d = lane + 32 * j;                       // head row d lies at shared index (d % LANES) * RS + d / LANES
          if (d < LANES * ROWS) {
            const int idx = (d % LANES) * RS + d / LANES;
            qs[i * KW + idx] = qv[tt][j] * iq;               // rows past dim were read as zeros
            ks[i * KW + idx] = kv[tt][j] * ik;
            if constexpr (CHD) {
              const float a1 = av[tt][j];
              gv[i * KW + idx] = expf(neg_rate * (a1 > 20.f ? a1 : log1pf(expf(a1))));
            }
          }
        }
      }
      for (int i = tid - DS_COMPUTE; i < n * COLS; i += DS_LOADERS) {
        const int tk = i / COLS, cc = i % COLS;
        vs[tk * COLS + cc] = c0 + cc < vdim ? qkv[(size_t)(base + tk) * C + (size_t)2 * kvh * dim + (size_t)h * vdim + c0 + cc] : 0.f;
      }
      __threadfence_block();
      named_arrive(1 + (c & 1), DS_THREADS);
    }
    return;
  }
  // -------------------------------------------------- walkers
  const int colb = tid / LANES, seg = tid % LANES;
  const int col = c0 + colb;
  const bool live = col < vdim;
  // this thread's rows of its column: seg, seg + LANES, ... (row r of the thread is row seg + LANES * r of the head)
  float S[ROWS];
  // (the slot keeps a head's matrix column by column, [vdim][dim]: the LANES threads of a column then read neighbours)
  float* mine = state + (size_t)slot * state_stride + ((size_t)h * vdim + col) * dim;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = seg + LANES * r;
    S[r] = (live && row < dim) ? mine[row] : 0.f;
  }
  for (int c = 0; c < chunks; ++c) {
    const float* ks = ds_smem + (c & 1) * BUF;
    const float* qs = ks + CH * KW;
    const float* vs = qs + CH * KW;
    const float* gs = vs + CH * COLS;
    const float* bs = gs + CH;
    const float* gv = bs + CH;
    const int base = t0 + c * CH, n = min(CH, t1 - base);
    named_sync(1 + (c & 1), DS_THREADS);
    for (int i = 0; i < n; ++i) {
      const float g = CHD ? 1.f : gs[i], beta = bs[i];
      const float4* g4 = reinterpret_cast<const float4*>(gv + i * KW + seg * RS);
      const float4* k4 = reinterpret_cast<const float4*>(ks + i * KW + seg * RS);
      const float4* q4 = reinterpret_cast<const float4*>(qs + i * KW + seg * RS);
      float kr[ROWS];
      float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < ROWS / 4; ++r) {
        const float4 kv = k4[r];
        kr[4 * r] = kv.x; kr[4 * r + 1] = kv.y; kr[4 * r + 2] = kv.z; kr[4 * r + 3] = kv.w;
        float gr[4] = {g, g, g, g};
        if constexpr (CHD) { const float4 t4 = g4[r]; gr[0] = t4.x; gr[1] = t4.y; gr[2] = t4.z; gr[3] = t4.w; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[4 * r + j] *= gr[j];
          a[j] = fmaf(S[4 * r + j], kr[4 * r + j], a[j]);
        }
      }
      float dot = (a[0] + a[1]) + (a[2] + a[3]);
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = beta * (vs[i * COLS + colb] - dot);
      float out4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < ROWS / 4; ++r) {
        const float4 qv = q4[r];
        const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[4 * r + j] = fmaf(kr[4 * r + j], u, S[4 * r + j]);
          out4[j] = fmaf(S[4 * r + j], qq[j], out4[j]);
        }
      }
      float o_ = (out4[0] + out4[1]) + (out4[2] + out4[3]);
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) o_ += __shfl_xor_sync(0xffffffffu, o_, o);
      if (seg == 0 && live) raw[(size_t)(base + i) * heads * vdim + (size_t)h * vdim + col] = o_;
    }
    if (c + 2 < chunks) named_arrive(3 + (c & 1), DS_THREADS);
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = seg + LANES * r;
    if (live && row < dim) mine[row] = S[r];
  }
}

// out[t, h, :] = raw[t, h, :] / sqrt(mean(raw[t, h, :]^2) + eps) * w * SiLU(gate[t, h, :]); one warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
delta_out_norm_kernel(const float* raw, const T* gate, long gate_stride, const float* __restrict__ w, T* out, int heads,
                      int vdim, float eps, int total, int gate_sigmoid) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= total) return;
  const int t = idx / heads, h = idx % heads;
  const float* o = raw + ((size_t)t * heads + h) * vdim;
  float ss = 0.f;
  for (int d = lane; d < vdim; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  const T* grow = gate + (size_t)t * gate_stride + (size_t)h * vdim;
  T* orow = out + ((size_t)t * heads + h) * vdim;
  for (int d = lane; d < vdim; d += 32) {
    const float gv = to_f<T>(grow[d]);
    orow[d] = from_f<T>(o[d] * inv * w[d] * (gate_sigmoid ? 1.f / (1.f + expf(-gv)) : silu_f(gv)));
  }
}

}  // namespace vob

using namespace vob;

// x: rows of x_stride elements of `dtype`, the C channels first; w float [C, taps]; state float [num_slots, state_stride]
// with the convolutions' part ((taps - 1) x C) at conv_off; out float [T, C].
VOB_API int vob_short_conv_silu(const void* x, long x_stride, const float* w, const float* state, long state_stride,
                                long conv_off, const int* token_req, const int* cu_q, const int* state_slots, float* out,
                                int T, int C, int taps, long num_slots, int act, int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > DELTA_MAX_TAPS) return VOB_UNSUPPORTED;
  const int walk = T >= 32 * CONV_TOKENS ? CONV_TOKENS : 1;      // few tokens (decoding): one each, nothing to slide
  dim3 grid((T + walk - 1) / walk, (C + 127) / 128);
  if (grid.y > 65535) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return launch_kernel(short_conv_silu_kernel<float>, grid, 128, 0, stream, (const float*)x, x_stride, w, state, state_stride,
                         conv_off, token_req, cu_q, state_slots, out, T, walk, C, taps, num_slots, act, err);
  if (dtype == VOB_BF16)
    return launch_kernel(short_conv_silu_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_stride, w,
                         state, state_stride, conv_off, token_req, cu_q, state_slots, out, T, walk, C, taps, num_slots, act, err);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_short_conv_state(const void* x, long x_stride, float* state, long state_stride, long conv_off,
                                 const int* cu_q, const int* state_slots, int B, int C, int taps, long num_slots, int dtype,
                                 cudaStream_t stream) {
  if (B <= 0 || taps <= 1) return 0;
  if (C <= 0 || taps > DELTA_MAX_TAPS) return VOB_UNSUPPORTED;
  dim3 grid((C + 127) / 128, B);
  if (dtype == VOB_F32)
    return launch_kernel(short_conv_state_kernel<float>, grid, 128, 0, stream, (const float*)x, x_stride, state, state_stride,
                         conv_off, cu_q, state_slots, C, taps, num_slots);
  if (dtype == VOB_BF16)
    return launch_kernel(short_conv_state_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_stride,
                         state, state_stride, conv_off, cu_q, state_slots, C, taps, num_slots);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_short_conv_step(const void* x, long x_stride, const float* w, float* state, long state_stride, long conv_off,
                                const int* cu_q, const int* state_slots, float* out, int B, int C, int taps, long num_slots,
                                int act, int dtype, int* err, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > DELTA_MAX_TAPS || B > 65535) return VOB_UNSUPPORTED;
  dim3 grid((C + 127) / 128, B);
  if (dtype == VOB_F32)
    return launch_kernel(short_conv_step_kernel<float>, grid, 128, 0, stream, (const float*)x, x_stride, w, state, state_stride,
                         conv_off, cu_q, state_slots, out, C, taps, num_slots, act, err);
  if (dtype == VOB_BF16)
    return launch_kernel(short_conv_step_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_stride, w,
                         state, state_stride, conv_off, cu_q, state_slots, out, C, taps, num_slots, act, err);
  return VOB_BAD_ARGUMENT;
}

template <typename T>
static int launch_delta_scan(const float* qkv, const void* ab, long ab_stride, int b_off, int a_off, const float* A_log,
                             const float* dt_bias, float* state, long state_stride, const int* cu_q, const int* state_slots,
                             float* raw, int B, int heads, int kvh, int dim, int vdim, long num_slots, int channel_decay,
                             int* err, cudaStream_t stream) {
  // rows a thread keeps, and threads a column: the fewest threads whose rows cover the head
  const int rows = dim <= 128 ? 16 : 32;
  const int lanes = dim <= rows ? 1 : (dim <= 2 * rows ? 2 : (dim <= 4 * rows ? 4 : 8));
#define VOB_DS(L, R)                                                                                                       \
  if (lanes == L && rows == R) {                                                                                           \
    constexpr int cols = DS_COMPUTE / L, ch = R > 16 ? 8 : 16;                                                             \
    dim3 grid((vdim + cols - 1) / cols, heads, B);                                                                         \
    if (channel_decay) {                                                                                                   \
      const size_t smem = (size_t)2 * ch * (3 * L * (R + 4) + cols + 2) * sizeof(float);                                   \
      if (smem > 48 * 1024)                                                                                                \
        cudaFuncSetAttribute(delta_scan_kernel<T, L, R, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
      return launch_kernel(delta_scan_kernel<T, L, R, true>, grid, DS_THREADS, smem, stream, qkv, (const T*)ab, ab_stride, \
                           b_off, a_off, A_log, dt_bias, state, state_stride, cu_q, state_slots, raw, heads, kvh, dim,     \
                           vdim, num_slots, err);                                                                          \
    }                                                                                                                      \
    const size_t smem = (size_t)2 * ch * (2 * L * (R + 4) + cols + 2) * sizeof(float);                                     \
    return launch_kernel(delta_scan_kernel<T, L, R, false>, grid, DS_THREADS, smem, stream, qkv, (const T*)ab, ab_stride,  \
                         b_off, a_off, A_log, dt_bias, state, state_stride, cu_q, state_slots, raw, heads, kvh, dim, vdim, \
                         num_slots, err);                                                                                  \
  }
  VOB_DS(1, 16) VOB_DS(2, 16) VOB_DS(4, 16) VOB_DS(8, 16) VOB_DS(8, 32)
#undef VOB_DS
  return VOB_UNSUPPORTED;
}

VOB_API int vob_delta_scan(const float* qkv, const void* ab, long ab_stride, int b_off, int a_off, const float* A_log,
                           const float* dt_bias, float* state, long state_stride, const int* cu_q, const int* state_slots,
                           float* raw, int B, int heads, int kvh, int dim, int vdim, long num_slots, int channel_decay,
                           int dtype, int* err, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || dim > 256 || vdim <= 0 || B > 65535) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return launch_delta_scan<float>(qkv, ab, ab_stride, b_off, a_off, A_log, dt_bias, state, state_stride, cu_q, state_slots, raw,
                                    B, heads, kvh, dim, vdim, num_slots, channel_decay, err, stream);
  if (dtype == VOB_BF16)
    return launch_delta_scan<__nv_bfloat16>(qkv, ab, ab_stride, b_off, a_off, A_log, dt_bias, state, state_stride, cu_q,
                                            state_slots, raw, B, heads, kvh, dim, vdim, num_slots, channel_decay, err, stream);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_delta_out_norm(const float* raw, const void* gate, long gate_stride, const float* w, void* out, int T, int heads,
                               int vdim, float eps, int gate_sigmoid, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int total = T * heads;
  dim3 grid((total + 3) / 4);
  if (dtype == VOB_F32)
    return launch_kernel(delta_out_norm_kernel<float>, grid, 128, 0, stream, raw, (const float*)gate, gate_stride, w,
                         (float*)out, heads, vdim, eps, total, gate_sigmoid);
  if (dtype == VOB_BF16)
    return launch_kernel(delta_out_norm_kernel<__nv_bfloat16>, grid, 128, 0, stream, raw, (const __nv_bfloat16*)gate,
                         gate_stride, w, (__nv_bfloat16*)out, heads, vdim, eps, total, gate_sigmoid);
  return VOB_BAD_ARGUMENT;
}
