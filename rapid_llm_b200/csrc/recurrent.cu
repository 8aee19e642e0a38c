// Kernels of the mixers that carry a state of fixed size per request instead of (or beside) cached
// keys: short causal convolutions, decays and step sizes, the recurrence itself, the norm and gate
// that follow it, and the activation of the dense feed-forward.
//
// A step is a packed ragged batch: entry e owns rows cu_seqlens[e] .. cu_seqlens[e + 1] - 1, its
// request sits in slot entry_slot[e] and had entry_start[e] tokens before this step.  State lives in
// one float32 row per slot (`state + slot * state_stride + offset`); a request at position 0 starts
// from zeros whatever the row holds, so a slot needs no clearing when it changes hands.  Everything a
// recurrence consumes (decays, step sizes, gates, unit vectors, the state) is float32 in both engine
// precisions; the recurrence runs token by token in a fixed order, so a row's result does not depend
// on how the tokens were cut into steps or on what else is in the batch.
//
// Pointers to what an earlier kernel of the same step wrote (activations, the state) carry no `__restrict__`:
// a load through a const restrict pointer counts as invariant and may be moved above the wait for the
// kernel before (seen: a convolution that read its rows before the product that writes them had finished,
// once its loads no longer depended on anything else).  Weights and the step's uploaded metadata keep it.
#include <type_traits>

#include "common.cuh"

namespace rl {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

constexpr int kMaxTaps = 16;

// ------------------------------------------------------------ short causal convolution
// out[t, c] = silu(bias[c] + sum_d taps[c, K - 1 - d] * x[t - d, c]) over the request's own tokens:
// those of this step from the rows of x, the K - 1 before them from the slot's tail (float32,
// [K - 1, C], oldest first), zeros before position 0.  x is columns col0 .. col0 + C - 1 of rows of
// length x_stride.
constexpr int kConvRows = 8;

template <typename T>
__device__ __forceinline__ float2 load_pair(const T* p);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// A thread owns kLanes (1 or 2) neighbouring channels over kConvRows consecutive packed rows and slides the taps'
// window down them, so a row of x is fetched once, not once per tap.  kLanes == 2 wants even C, col0 and x_stride.
// kTaps > 0: the taps' number is known when compiling and the window lives in registers; 0: any number up to kMaxTaps.
template <typename T, int kLanes, int kTaps>
__global__ void causal_conv_silu_kernel(const T* x, int x_stride, int col0,
                                        const float* __restrict__ taps, const float* __restrict__ bias,
                                        const float* state, long long state_stride, int state_off,
                                        float* __restrict__ out, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ entry_slot, const int* __restrict__ entry_start,
                                        int entries, int tokens, int C, int taps_given, int slots, int* __restrict__ fault,
                                        int act) {
  pdl_trigger();
  const int K = kTaps > 0 ? kTaps : taps_given;
  constexpr int kHeld = kTaps > 0 ? kTaps : kMaxTaps;
  const int groups = C / kLanes, tiles = (tokens + kConvRows - 1) / kConvRows;
  const long long total = static_cast<long long>(tiles) * groups;
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= total) {
    pdl_wait();
    return;
  }
  const int tile = static_cast<int>(idx / groups), c = static_cast<int>(idx - static_cast<long long>(tile) * groups) * kLanes;
  float w[kLanes][kHeld], b[kLanes];
#pragma unroll
  for (int l = 0; l < kLanes; ++l) {
    b[l] = bias ? bias[c + l] : 0.0f;
#pragma unroll
    for (int d = 0; d < kHeld; ++d)
      if (d < K) w[l][d] = taps[static_cast<size_t>(c + l) * K + d];     // w[K - 1] is the current token's
  }
  const int t0 = tile * kConvRows;
  int e = entry_of(cu_seqlens, entries, t0);
  pdl_wait();
  // this tile's own rows, asked for at once (every row needs its own input, whatever entry it belongs to)
  float own[kLanes][kConvRows];
#pragma unroll
  for (int r = 0; r < kConvRows; ++r) {
    if (t0 + r < tokens) {
      if constexpr (kLanes == 2) {
        const float2 v = load_pair(x + static_cast<size_t>(t0 + r) * x_stride + col0 + c);
        own[0][r] = v.x; own[1][r] = v.y;
      } else {
        own[0][r] = to_float(x[static_cast<size_t>(t0 + r) * x_stride + col0 + c]);
      }
    }
  }
  // the window: hist[d] is the input d rows back (hist[0] the current row's)
  float hist[kLanes][kHeld];
  int filled_for = -1;      // the entry the window was filled for
#pragma unroll
  for (int r = 0; r < kConvRows; ++r) {
    const int t = t0 + r;
    if (t >= tokens) break;
    while (t >= cu_seqlens[e + 1]) ++e;
    const int local = t - cu_seqlens[e], start = entry_start[e];
    if (filled_for != e) {      // first row of this tile that belongs to entry e: fetch the K - 1 inputs before it
      int slot = entry_slot[e];
      if (slot < 0 || slot >= slots) {
        atomicOr(fault, kFaultSlot);
        slot = 0;
      }
      const float* tail = state + slot * state_stride + state_off;
#pragma unroll
      for (int d = 1; d < kHeld; ++d) {
        if (d >= K) break;
        const int at = local - d;
#pragma unroll
        for (int l = 0; l < kLanes; ++l) hist[l][d] = 0.0f;
        if (at >= 0) {
          if constexpr (kLanes == 2) {
            const float2 v = load_pair(x + static_cast<size_t>(t - d) * x_stride + col0 + c);
            hist[0][d] = v.x; hist[1][d] = v.y;
          } else {
            hist[0][d] = to_float(x[static_cast<size_t>(t - d) * x_stride + col0 + c]);
          }
        } else if (start + at >= 0) {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) hist[l][d] = tail[static_cast<size_t>(K - 1 + at) * C + c + l];
        }
      }
      filled_for = e;
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) hist[l][0] = own[l][r];
    float acc[kLanes];
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      acc[l] = b[l];
#pragma unroll
      for (int d = 0; d < kHeld; ++d)
        if (d < K) acc[l] += w[l][K - 1 - d] * hist[l][d];
      if (act) acc[l] = silu_f(acc[l]);      // act 0: the convolution's plain result
    }
    if constexpr (kLanes == 2) {
      *reinterpret_cast<float2*>(out + static_cast<size_t>(t) * C + c) = make_float2(acc[0], acc[1]);
    } else {
      out[static_cast<size_t>(t) * C + c] = acc[0];
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
#pragma unroll
      for (int d = kHeld - 1; d > 0; --d)
        if (d < K) hist[l][d] = hist[l][d - 1];
    }
  }
}

// The slot's tail after the step: the last K - 1 inputs of the request, taken from this step's rows
// and, where the step brought fewer, from the old tail.  A thread reads all it needs before it writes.
template <typename T>
__global__ void conv_tail_update_kernel(const T* x, int x_stride, int col0,
                                        float* __restrict__ state, long long state_stride, int state_off,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ entry_slot,
                                        const int* __restrict__ entry_start, int entries, int C, int K, int slots) {
  pdl_trigger();
  pdl_wait();
  const long long total = static_cast<long long>(entries) * C;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = static_cast<int>(idx / C), c = static_cast<int>(idx - static_cast<long long>(e) * C);
    const int slot = entry_slot[e];
    if (slot < 0 || slot >= slots) continue;
    const int first = cu_seqlens[e], length = cu_seqlens[e + 1] - first, start = entry_start[e];
    float* tail = state + slot * state_stride + state_off;
    float fresh[kMaxTaps];
    for (int j = 0; j < K - 1; ++j) {
      const int at = length - (K - 1) + j;      // index among this step's tokens of the request
      float v = 0.0f;
      if (at >= 0) {
        v = to_float(x[static_cast<size_t>(first + at) * x_stride + col0 + c]);
      } else if (start + at >= 0) {
        v = tail[static_cast<size_t>(K - 1 + at) * C + c];
      }
      fresh[j] = v;
    }
    for (int j = 0; j < K - 1; ++j) tail[static_cast<size_t>(j) * C + c] = fresh[j];
  }
}

// ------------------------------------------------------------ activation into float32 rows
// out[t, c] = act(x[t, col0 + c]) as float32 (act 0: the value itself, 1: SiLU): what a mixer without a
// convolution feeds into its recurrence.
template <typename T>
__global__ void activate_rows_kernel(const T* x, int x_stride, int col0, float* __restrict__ out, int tokens, int C,
                                     int act) {
  pdl_trigger();
  pdl_wait();
  const long long total = static_cast<long long>(tokens) * C;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / C;
    const int c = static_cast<int>(idx - t * C);
    const float v = to_float(x[static_cast<size_t>(t) * x_stride + col0 + c]);
    out[idx] = act ? silu_f(v) : v;
  }
}

// ------------------------------------------------------------ decays and step sizes
// step[t, c] = softplus(x[t, c] + bias[c]); decay[t, c] = exp(-rate[c / per] * step[t, c]), rate = exp(A_log)
// (taken once when the weights are loaded).  kWide: four columns a thread, 8- and 16-byte accesses.
template <typename T, bool kWide>
__global__ void decay_gate_kernel(const T* x, int x_stride, int col0, const float* __restrict__ rate,
                                  const float* __restrict__ bias, int per, float* __restrict__ decay,
                                  float* __restrict__ step, int tokens, int C) {
  pdl_trigger();
  pdl_wait();
  constexpr int kEach = kWide ? 4 : 1;
  const int per_row = C / kEach;
  const long long total = static_cast<long long>(tokens) * per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / per_row), c = static_cast<int>(idx - static_cast<long long>(t) * per_row) * kEach;
    const T* in = x + static_cast<size_t>(t) * x_stride + col0 + c;
    float raw[kEach], dt[kEach], d[kEach];
    if constexpr (kWide && sizeof(T) == 2) {
      const uint2 packed = *reinterpret_cast<const uint2*>(in);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
      const float2 lo = __bfloat1622float2(h[0]), hi = __bfloat1622float2(h[1]);
      raw[0] = lo.x; raw[1] = lo.y; raw[2] = hi.x; raw[3] = hi.y;
    } else if constexpr (kWide) {
      const float4 f = *reinterpret_cast<const float4*>(in);
      raw[0] = f.x; raw[1] = f.y; raw[2] = f.z; raw[3] = f.w;
    } else {
      raw[0] = to_float(in[0]);
    }
#pragma unroll
    for (int j = 0; j < kEach; ++j) {
      dt[j] = softplus_f(raw[j] + (bias ? bias[c + j] : 0.0f));
      d[j] = expf(-rate[(c + j) / per] * dt[j]);
    }
    float* to = decay + static_cast<size_t>(t) * C + c;
    if constexpr (kWide) {
      *reinterpret_cast<float4*>(to) = make_float4(d[0], d[1], d[2], d[3]);
      if (step) *reinterpret_cast<float4*>(step + static_cast<size_t>(t) * C + c) = make_float4(dt[0], dt[1], dt[2], dt[3]);
    } else {
      to[0] = d[0];
      if (step) step[static_cast<size_t>(t) * C + c] = dt[0];
    }
  }
}

// ------------------------------------------------------------ decay from a double exponential
// decay[t, c] = exp(-exp(x[t, c] + bias[c])), float32: a decay per token and channel that stays inside (0, 1).
template <typename T>
__global__ void exp_decay_kernel(const T* x, int x_stride, int col0, const float* __restrict__ bias,
                                 float* __restrict__ decay, int tokens, int C) {
  pdl_trigger();
  pdl_wait();
  const long long total = static_cast<long long>(tokens) * C;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / C;
    const int c = static_cast<int>(idx - t * C);
    const float v = to_float(x[static_cast<size_t>(t) * x_stride + col0 + c]) + (bias ? bias[c] : 0.0f);
    decay[idx] = expf(-expf(v));
  }
}

// ------------------------------------------------------------ tanh of rows, in the rows' own type
// out[i] = tanh(x[i]) in float32, rounded once: the activation between the two halves of a low-rank product.
template <typename T>
__global__ void tanh_rows_kernel(const T* x, T* out, long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x)
    out[idx] = from_float<T>(tanhf(to_float(x[idx])));
}

// ------------------------------------------------------------ blends of a row with the row before it
// out[s][t][c] = x[t][c] + (before[t][c] - x[t][c]) * mu[s][c] for `mixes` vectors mu, float32 arithmetic, one
// rounding at the store; out is `mixes` planes of [tokens, C].  `before` is the request's previous row: row t - 1 of
// the same entry, the slot's kept row (float32) for the entry's first row, zeros at position 0.  The block of an
// entry's first row also brings the kept row up to date (the entry's last row), each thread after it has read
// what it needs; no other block touches the slot's row.
template <typename T>
__global__ void shift_mix_kernel(const T* x, int x_stride, const float* __restrict__ mu, int mixes, T* out,
                                 float* kept, long long kept_stride, int kept_off,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ entry_slot,
                                 const int* __restrict__ entry_start, int entries, int tokens, int C, int slots,
                                 int* __restrict__ fault) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int e = entry_of(cu_seqlens, entries, t);
  const int first = cu_seqlens[e], last = cu_seqlens[e + 1] - 1;
  int slot = entry_slot[e];
  const bool slot_ok = slot >= 0 && slot < slots;
  if (!slot_ok) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultSlot);
    slot = 0;
  }
  const bool opens = t == first;
  const bool from_kept = opens && entry_start[e] > 0;
  float* kr = kept + slot * kept_stride + kept_off;
  const T* xr = x + static_cast<size_t>(t) * x_stride;
  const T* pr = xr - x_stride;
  const T* lr = x + static_cast<size_t>(last) * x_stride;
  const size_t plane = static_cast<size_t>(tokens) * C;
  pdl_wait();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float now = to_float(xr[c]);
    float before = 0.0f;
    if (from_kept) before = kr[c];
    else if (!opens) before = to_float(pr[c]);
    if (opens && slot_ok) kr[c] = to_float(lr[c]);
    const float step = before - now;
    for (int s = 0; s < mixes; ++s)
      out[s * plane + static_cast<size_t>(t) * C + c] = from_float<T>(fmaf(step, mu[static_cast<size_t>(s) * C + c], now));
  }
}

// ------------------------------------------------------------ unit vectors per head, write strengths
// Heads of `dim` floats, `heads` of them side by side from column col0 of a float32 row: each becomes
// x / sqrt(sum(x^2) + eps) times scale_low (heads below `split`) or scale_high.  One warp a head.
// Beside it, sigmoid of `gates` columns of a row of the engine's dtype into a float32 [T, gates].
template <typename T>
__global__ void unit_heads_kernel(float* __restrict__ rows, int stride, int col0, int heads, int dim, float eps,
                                  int split, float scale_low, float scale_high, const T* gate_in,
                                  int gate_stride, int gate_col0, int gates, float* __restrict__ gate_out, int tokens) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  if (t >= tokens) return;
  for (int head = warp; head < heads; head += warps) {
    float* v = rows + static_cast<size_t>(t) * stride + col0 + static_cast<size_t>(head) * dim;
    float sum_sq = 0.0f;
    for (int i = lane; i < dim; i += 32) sum_sq += v[i] * v[i];
    sum_sq = warp_sum(sum_sq);
    const float factor = (head < split ? scale_low : scale_high) / sqrtf(sum_sq + eps);
    for (int i = lane; i < dim; i += 32) v[i] *= factor;
  }
  for (int i = threadIdx.x; i < gates; i += blockDim.x)
    gate_out[static_cast<size_t>(t) * gates + i] =
        sigmoid_f(to_float(gate_in[static_cast<size_t>(t) * gate_stride + gate_col0 + i]));
}

// ------------------------------------------------------------ rotation for heads without a cache
// in: a row of the engine's dtype with `heads` query heads of `dim` from column q_col0, as many key
// heads from k_col0 and `heads * vdim` values from v_col0.  out (float32): [q | k | v]; q and k with
// their first `rot` entries rotated by position (entry i paired with i + rot / 2, angle = position *
// inv_freq[i], all float32), k times k_scale after the rotation.
template <typename T>
__global__ void rotate_heads_kernel(const T* in, int in_stride, int q_col0, int k_col0, int v_col0,
                                    float* __restrict__ out, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int heads, int dim, int vdim, int rot,
                                    float k_scale, int tokens, int wide) {
  extern __shared__ __align__(16) float angles[];      // cos, then sin, of the token's rot / 2 angles: the same for every head
  pdl_trigger();
  const int t = blockIdx.x;
  const int qk = heads * dim, half = rot >> 1;
  const float pos = static_cast<float>(positions[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &angles[half + i], &angles[i]);
  pdl_wait();
  __syncthreads();
  const T* row = in + static_cast<size_t>(t) * in_stride;
  float* o = out + static_cast<size_t>(t) * (2 * qk + heads * vdim);
  if (wide) {
    // four neighbouring entries of a head and their partners at once: every input is read once, 8 or 16 bytes at a time
    auto load4 = [](const T* p, float (&v)[4]) {
      if constexpr (sizeof(T) == 2) {
        const uint2 packed = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
        const float2 lo = __bfloat1622float2(h[0]), hi = __bfloat1622float2(h[1]);
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
      } else {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      }
    };
    const int quads_rot = half >> 2, quads_rest = (dim - rot) >> 2, per_head = quads_rot + quads_rest;
    for (int idx = threadIdx.x; idx < 2 * heads * per_head; idx += blockDim.x) {
      const int head2 = idx / per_head, j = idx - head2 * per_head;      // head2: query heads, then key heads
      const bool is_k = head2 >= heads;
      const int head = is_k ? head2 - heads : head2;
      const T* src = row + (is_k ? k_col0 : q_col0) + head * dim;
      float* dst = o + (is_k ? qk : 0) + head * dim;
      const float scale = is_k ? k_scale : 1.0f;
      if (j < quads_rot) {
        const int i = j << 2;
        float x1[4], x2[4];
        load4(src + i, x1);
        load4(src + i + half, x2);
        const float4 c = *reinterpret_cast<const float4*>(angles + i), sn = *reinterpret_cast<const float4*>(angles + half + i);
        const float cs[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
        float o1[4], o2[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          o1[n] = (x1[n] * cs[n] - x2[n] * ss[n]) * scale;
          o2[n] = (x2[n] * cs[n] + x1[n] * ss[n]) * scale;
        }
        *reinterpret_cast<float4*>(dst + i) = make_float4(o1[0], o1[1], o1[2], o1[3]);
        *reinterpret_cast<float4*>(dst + i + half) = make_float4(o2[0], o2[1], o2[2], o2[3]);
      } else {
        const int i = rot + ((j - quads_rot) << 2);
        float v[4];
        load4(src + i, v);
        *reinterpret_cast<float4*>(dst + i) = make_float4(v[0] * scale, v[1] * scale, v[2] * scale, v[3] * scale);
      }
    }
    for (int idx = threadIdx.x * 4; idx < heads * vdim; idx += blockDim.x * 4) {
      float v[4];
      load4(row + v_col0 + idx, v);
      *reinterpret_cast<float4*>(o + 2 * qk + idx) = make_float4(v[0], v[1], v[2], v[3]);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < 2 * qk; idx += blockDim.x) {
    const bool is_k = idx >= qk;
    const int within = is_k ? idx - qk : idx;
    const int i = within % dim;
    const T* src = row + (is_k ? k_col0 : q_col0) + (within - i);
    float v = to_float(src[i]);
    if (i < rot) {
      const int pair = i < half ? i : i - half;
      const float c = angles[pair], sn = angles[half + pair];
      v = i < half ? v * c - to_float(src[i + half]) * sn : v * c + to_float(src[i - half]) * sn;
    }
    o[idx] = is_k ? v * k_scale : v;
  }
  for (int idx = threadIdx.x; idx < heads * vdim; idx += blockDim.x) o[2 * qk + idx] = to_float(row[v_col0 + idx]);
}

// ------------------------------------------------------------ the recurrence
// Per head a state S of dim x vdim floats; per token, in this order:
//   S <- decay * S                  decay: one number per head (mode 0), per token and head (mode 1),
//                                   or per token, head and row of S (mode 2)
//   u = beta * (v - S^T k)          with beta (the delta rule), else u = v_scale * v (v_scale may be null)
//   S <- S + k u^T
//   out = S^T q (+ skip * v)
// With `bonus` (one number per head and row of S) the read-out comes first and the token's own pair enters it
// weighed, before the state decays and takes the pair:
//   out = (S + diag(bonus) k v^T)^T q;   S <- decay * S + k v^T
// Query/key head of head h is h / (heads / kv_heads).
//
// A block owns (entry, head, a tile of columns of S) and walks the entry's tokens in order.  A column
// is shared by `partners` lanes of one warp, each holding kRows consecutive rows of it in registers;
// sums over rows end in a fixed tree of shuffles, so a token's result depends on nothing but the
// tokens before it.  q, k, row decays, v and the per-token numbers of a run of tokens are brought into
// shared memory by asynchronous copies while the run before is walked.  In the slot's row a head's
// state lies column by column (S^T, [vdim][dim]), so that a lane's rows are consecutive floats.
struct ScanArgs {
  const float* q; int q_stride;
  const float* k; int k_stride;
  const float* v; int v_stride;
  const float* decay; int decay_mode;
  const float* beta;
  const float* v_scale;
  const float* skip;
  const float* bonus;   // [heads, dim] or null: the read-out comes before the update and weighs the token's own pair
  float* out; int out_stride;
  float* state; long long state_stride; int state_off;
  const int* cu_seqlens; const int* entry_slot; const int* entry_start;
  int heads, kv_heads, dim, vdim, slots;
  int partners, run;
  int wide_in;      // q, k, v (and row decays) can be fetched 16 bytes at a time
  int* fault;
};

constexpr int kScanThreads = 256;

__device__ __forceinline__ void copy_async4(float* shared, const float* global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(shared))),
               "l"(global) : "memory");
}
__device__ __forceinline__ void copy_async16(float* shared, const float* global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<unsigned>(__cvta_generic_to_shared(shared))),
               "l"(global) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

template <int kRows, int kPartners>
__global__ void __launch_bounds__(kScanThreads) linear_scan_kernel(const ScanArgs a) {
  extern __shared__ __align__(16) float staged[];
  // Its successor is let in only when the walk is over (below): a kernel that waits at its start still holds
  // warp slots, and the walk is bound by its own latencies, which more resident warps do not shorten.
  const int e = blockIdx.x, head = blockIdx.y;
  constexpr int partners = kPartners, cols_per_warp = 32 / kPartners;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = lane / cols_per_warp, col_in_warp = lane - part * cols_per_warp;
  constexpr int tile_cols = (kScanThreads / 32) * cols_per_warp;
  const int col_in_tile = warp * cols_per_warp + col_in_warp;
  const int col = blockIdx.z * tile_cols + col_in_tile;
  const bool col_ok = col < a.vdim;
  const int row0 = part * kRows;
  constexpr int dim_padded = partners * kRows;
  const int kv_head = head / (a.heads / a.kv_heads);

  const int first = a.cu_seqlens[e], length = a.cu_seqlens[e + 1] - first, start = a.entry_start[e];
  int slot = a.entry_slot[e];
  const bool slot_ok = slot >= 0 && slot < a.slots;
  if (!slot_ok) {
    if (threadIdx.x == 0) atomicOr(a.fault, kFaultSlot);
    slot = 0;
  }
  float* home = a.state + slot * a.state_stride + a.state_off + static_cast<size_t>(head) * a.dim * a.vdim +
                static_cast<size_t>(col_ok ? col : 0) * a.dim + row0;
  const bool wide = (a.dim & 3) == 0 && (reinterpret_cast<uintptr_t>(home) & 15) == 0;   // kRows is a multiple of 4

  // two buffers, each: k, q (and row decays) [run][dim_padded]; v [run][tile_cols]; write strength, decay [run]
  const int run = a.run;
  const int per_token = (a.decay_mode == 2 ? 3 : 2) * dim_padded + tile_cols + 2;
  const int buffer_floats = (run * per_token + 3) & ~3;      // both buffers start on 16 bytes
  const float fixed_decay = a.decay_mode == 0 ? a.decay[head] : 1.0f;
  const float skip = a.skip ? a.skip[head] : 0.0f;
  const float* strength = a.beta ? a.beta : a.v_scale;

  auto stage = [&](int base, float* buffer) {
    const int count = min(run, length - base);
    float* sk = buffer;
    float* sq = sk + run * dim_padded;
    float* sg = sq + run * dim_padded;
    float* sv = sg + (a.decay_mode == 2 ? run * dim_padded : 0);
    float* sbeta = sv + run * tile_cols;
    float* sdecay = sbeta + run;
    if (a.wide_in) {
      const int quads = dim_padded >> 2, tile_quads = tile_cols >> 2;
      for (int idx = threadIdx.x; idx < count * quads; idx += kScanThreads) {
        const int tt = idx / quads, i = (idx - tt * quads) << 2;
        const size_t t = static_cast<size_t>(first + base + tt);
        const int at = tt * dim_padded + i;
        if (i < a.dim) {
          copy_async16(sk + at, a.k + t * a.k_stride + kv_head * a.dim + i);
          copy_async16(sq + at, a.q + t * a.q_stride + kv_head * a.dim + i);
          if (a.decay_mode == 2) copy_async16(sg + at, a.decay + (t * a.heads + head) * a.dim + i);
        } else {
          *reinterpret_cast<float4*>(sk + at) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          *reinterpret_cast<float4*>(sq + at) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (a.decay_mode == 2) *reinterpret_cast<float4*>(sg + at) = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        }
      }
      for (int idx = threadIdx.x; idx < count * tile_quads; idx += kScanThreads) {
        const int tt = idx / tile_quads, j = (idx - tt * tile_quads) << 2;
        const int c = blockIdx.z * tile_cols + j;
        float* to = sv + tt * tile_cols + j;
        if (c < a.vdim) copy_async16(to, a.v + static_cast<size_t>(first + base + tt) * a.v_stride + head * a.vdim + c);
        else *reinterpret_cast<float4*>(to) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    } else {
      for (int idx = threadIdx.x; idx < count * dim_padded; idx += kScanThreads) {
        const int tt = idx / dim_padded, i = idx - tt * dim_padded;
        const size_t t = static_cast<size_t>(first + base + tt);
        if (i < a.dim) {
          copy_async4(sk + idx, a.k + t * a.k_stride + kv_head * a.dim + i);
          copy_async4(sq + idx, a.q + t * a.q_stride + kv_head * a.dim + i);
          if (a.decay_mode == 2) copy_async4(sg + idx, a.decay + (t * a.heads + head) * a.dim + i);
        } else {
          sk[idx] = 0.0f;
          sq[idx] = 0.0f;
          if (a.decay_mode == 2) sg[idx] = 1.0f;
        }
      }
      for (int idx = threadIdx.x; idx < count * tile_cols; idx += kScanThreads) {
        const int tt = idx / tile_cols, j = idx - tt * tile_cols;
        const int c = blockIdx.z * tile_cols + j;
        if (c < a.vdim) copy_async4(sv + idx, a.v + static_cast<size_t>(first + base + tt) * a.v_stride + head * a.vdim + c);
        else sv[idx] = 0.0f;
      }
    }
    for (int tt = threadIdx.x; tt < count; tt += kScanThreads) {
      const size_t at = static_cast<size_t>(first + base + tt) * a.heads + head;
      if (strength) copy_async4(sbeta + tt, strength + at); else sbeta[tt] = 1.0f;
      if (a.decay_mode == 1) copy_async4(sdecay + tt, a.decay + at); else sdecay[tt] = fixed_decay;
    }
    copy_async_commit();
  };

  pdl_wait();
  if (length > 0) stage(0, staged);
  float S[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) S[r] = 0.0f;
  if (start > 0 && col_ok) {
    if (wide) {
#pragma unroll
      for (int r = 0; r < kRows; r += 4) {
        if (row0 + r < a.dim) {
          const float4 four = *reinterpret_cast<const float4*>(home + r);
          S[r] = four.x; S[r + 1] = four.y; S[r + 2] = four.z; S[r + 3] = four.w;
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (row0 + r < a.dim) S[r] = home[r];
    }
  }

  float bonus[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
    bonus[r] = (a.bonus && row0 + r < a.dim) ? a.bonus[static_cast<size_t>(head) * a.dim + row0 + r] : 0.0f;

  int flip = 0;
  for (int base = 0; base < length; base += run, flip ^= 1) {
    const int count = min(run, length - base);
    float* buffer = staged + flip * buffer_floats;
    if (base + run < length) {
      stage(base + run, staged + (flip ^ 1) * buffer_floats);   // the next run, while this one is walked
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const float* sk = buffer;
    const float* sq = sk + run * dim_padded;
    const float* sg = sq + run * dim_padded;
    const float* sv = sg + (a.decay_mode == 2 ? run * dim_padded : 0);
    const float* sbeta = sv + run * tile_cols;
    const float* sdecay = sbeta + run;
    // a lane's rows are 16-byte aligned runs of shared memory: fetched four at a time, no two lanes of a
    // quarter-warp meet in a bank; every pointer of the walk moves by a constant per token
    const float* kp = sk + row0;
    const float* qp = sq + row0;
    const float* gp = sg + row0;
    const float* vp = sv + col_in_tile;
    float* op = a.out + static_cast<size_t>(first + base) * a.out_stride + head * a.vdim + (col_ok ? col : 0);
    const bool writes = part == 0 && col_ok;
    // Tokens are walked in groups of four: the state passes from one to the next, but their read-outs' sums over
    // lanes are independent and run side by side after the group, one shuffle's wait for four.  A token's own
    // arithmetic is the same whatever group it falls into.
    auto walk = [&](auto group_size, int tt) {
      constexpr int kGroup = decltype(group_size)::value;
      float o[kGroup], vv[kGroup];
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        float kk[kRows], qq[kRows];
#pragma unroll
        for (int r = 0; r < kRows; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kp + g * dim_padded + r);
          const float4 q4 = *reinterpret_cast<const float4*>(qp + g * dim_padded + r);
          kk[r] = k4.x; kk[r + 1] = k4.y; kk[r + 2] = k4.z; kk[r + 3] = k4.w;
          qq[r] = q4.x; qq[r + 1] = q4.y; qq[r + 2] = q4.z; qq[r + 3] = q4.w;
        }
        const float vj = vp[g * tile_cols];
        if (a.bonus) {
          // read the state as the tokens before left it, the token's own pair weighed by the bonus; then decay and add
          float gg[kRows];
          if (a.decay_mode == 2) {
#pragma unroll
            for (int r = 0; r < kRows; r += 4) {
              const float4 g4 = *reinterpret_cast<const float4*>(gp + g * dim_padded + r);
              gg[r] = g4.x; gg[r + 1] = g4.y; gg[r + 2] = g4.z; gg[r + 3] = g4.w;
            }
          } else {
            const float d = sdecay[tt + g];
#pragma unroll
            for (int r = 0; r < kRows; ++r) gg[r] = d;
          }
          const float uj = sbeta[tt + g] * vj;
          float even = 0.0f, odd = 0.0f;
#pragma unroll
          for (int r = 0; r < kRows; r += 2) {
            const float kv0 = kk[r] * uj, kv1 = kk[r + 1] * uj;
            even += (S[r] + bonus[r] * kv0) * qq[r];
            odd += (S[r + 1] + bonus[r + 1] * kv1) * qq[r + 1];
            S[r] = S[r] * gg[r] + kv0;
            S[r + 1] = S[r + 1] * gg[r + 1] + kv1;
          }
          o[g] = even + odd;
          vv[g] = vj;
          continue;
        }
        if (a.decay_mode == 2) {
#pragma unroll
          for (int r = 0; r < kRows; r += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(gp + g * dim_padded + r);
            S[r] *= g4.x; S[r + 1] *= g4.y; S[r + 2] *= g4.z; S[r + 3] *= g4.w;
          }
        } else {
          const float d = sdecay[tt + g];
#pragma unroll
          for (int r = 0; r < kRows; ++r) S[r] *= d;
        }
        float u;
        if (a.beta) {
          float seen = 0.0f, seen_odd = 0.0f;
#pragma unroll
          for (int r = 0; r < kRows; r += 2) {
            seen += S[r] * kk[r];
            seen_odd += S[r + 1] * kk[r + 1];
          }
          seen += seen_odd;
#pragma unroll
          for (int offset = cols_per_warp; offset < 32; offset <<= 1) seen += __shfl_xor_sync(0xffffffffu, seen, offset);
          u = sbeta[tt + g] * (vj - seen);
        } else {
          u = sbeta[tt + g] * vj;
        }
        float even = 0.0f, odd = 0.0f;
#pragma unroll
        for (int r = 0; r < kRows; r += 2) {
          S[r] += kk[r] * u;
          S[r + 1] += kk[r + 1] * u;
          even += S[r] * qq[r];
          odd += S[r + 1] * qq[r + 1];
        }
        o[g] = even + odd;
        vv[g] = vj;
      }
#pragma unroll
      for (int offset = cols_per_warp; offset < 32; offset <<= 1) {
#pragma unroll
        for (int g = 0; g < kGroup; ++g) o[g] += __shfl_xor_sync(0xffffffffu, o[g], offset);
      }
      if (writes) {
#pragma unroll
        for (int g = 0; g < kGroup; ++g) op[static_cast<size_t>(g) * a.out_stride] = o[g] + skip * vv[g];
      }
      kp += kGroup * dim_padded; qp += kGroup * dim_padded; gp += kGroup * dim_padded; vp += kGroup * tile_cols;
      op += static_cast<size_t>(kGroup) * a.out_stride;
    };
    int tt = 0;
    for (; tt + 4 <= count; tt += 4) walk(std::integral_constant<int, 4>{}, tt);
    for (; tt < count; ++tt) walk(std::integral_constant<int, 1>{}, tt);
    __syncthreads();     // the buffer is free for the run after the next
  }
  pdl_trigger();
  if (slot_ok && col_ok) {
    if (wide) {
#pragma unroll
      for (int r = 0; r < kRows; r += 4)
        if (row0 + r < a.dim) *reinterpret_cast<float4*>(home + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
    } else {
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (row0 + r < a.dim) home[r] = S[r];
    }
  }
}

// ------------------------------------------------------------ norm and gate after a mixer
// y: [T, C] in groups of `group` columns.  gate = act(g[t, g_col0 + c]) with act 0 none, 1 sigmoid,
// 2 SiLU.  With `gate_first` the gate multiplies before the norm, else after it.  The norm (if `norm`)
// divides a group by sqrt(mean(z^2) + eps) and multiplies by weight[c % weight_period] (or nothing).
// One block per (token, group); float32 arithmetic, one rounding at the store.
template <typename TY, typename T>
__global__ void gated_norm_kernel(const TY* y, int y_stride, const T* g, int g_stride,
                                  int g_col0, int act, int gate_first, int norm, const float* __restrict__ weight,
                                  int weight_period, float eps, T* __restrict__ out, int group, int groups) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, part = blockIdx.y;
  const TY* yr = y + static_cast<size_t>(t) * y_stride + static_cast<size_t>(part) * group;
  const T* gr = g ? g + static_cast<size_t>(t) * g_stride + g_col0 + static_cast<size_t>(part) * group : nullptr;
  T* o = out + (static_cast<size_t>(t) * groups + part) * group;
  auto gate_at = [&](int i) {
    if (!gr || act == 0) return 1.0f;
    const float raw = to_float(gr[i]);
    return act == 1 ? sigmoid_f(raw) : silu_f(raw);
  };
  float inv = 1.0f;
  if (norm) {
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
      float z = to_float(yr[i]);
      if (gate_first) z *= gate_at(i);
      sum_sq += z * z;
    }
    sum_sq = block_sum(sum_sq, scratch);
    inv = 1.0f / sqrtf(sum_sq / static_cast<float>(group) + eps);
  }
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const float gate = gate_at(i);
    float z = to_float(yr[i]);
    if (gate_first) z *= gate;
    z *= inv;
    if (norm && weight) z *= weight[(part * group + i) % weight_period];
    if (!gate_first) z *= gate;
    o[i] = from_float<T>(z);
  }
}

// The same with one warp per (token, group), for groups that are a multiple of 4 columns: four columns a lane and
// step, no shared memory, no barrier; the second pass finds its rows in L1.
template <typename TY, typename T>
__global__ void gated_norm_warp_kernel(const TY* y, int y_stride, const T* g, int g_stride,
                                       int g_col0, int act, int gate_first, int norm, const float* __restrict__ weight,
                                       int weight_period, float eps, T* __restrict__ out, int group, int groups,
                                       long long total, int wide) {
  pdl_trigger();
  pdl_wait();
  const long long index = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (index >= total) return;
  const int lane = threadIdx.x & 31;
  const long long t = index / groups;
  const int part = static_cast<int>(index - t * groups);
  const TY* yr = y + static_cast<size_t>(t) * y_stride + static_cast<size_t>(part) * group;
  const T* gr = (g && act != 0) ? g + static_cast<size_t>(t) * g_stride + g_col0 + static_cast<size_t>(part) * group : nullptr;
  T* o = out + (static_cast<size_t>(t) * groups + part) * group;
  auto load4 = [&](const auto* p, float (&v)[4]) {      // `wide`: every run of four starts on a vector's boundary
    using E = std::remove_cv_t<std::remove_reference_t<decltype(*p)>>;
    if (wide) {
      if constexpr (sizeof(E) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 lo = __bfloat1622float2(h[0]), hi = __bfloat1622float2(h[1]);
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_float(p[j]);
    }
  };
  auto four = [&](int i, float (&z)[4], float (&gate)[4]) {
    load4(yr + i, z);
    float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (gr) load4(gr + i, raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gate[j] = gr ? (act == 1 ? sigmoid_f(raw[j]) : silu_f(raw[j])) : 1.0f;
      if (gate_first) z[j] *= gate[j];
    }
  };
  float inv = 1.0f;
  if (norm) {
    float sum_sq = 0.0f;
    for (int i = lane * 4; i < group; i += 128) {
      float z[4], gate[4];
      four(i, z, gate);
      sum_sq += z[0] * z[0] + z[1] * z[1] + z[2] * z[2] + z[3] * z[3];
    }
    sum_sq = warp_sum(sum_sq);
    inv = 1.0f / sqrtf(sum_sq / static_cast<float>(group) + eps);
  }
  for (int i = lane * 4; i < group; i += 128) {
    float z[4], gate[4];
    four(i, z, gate);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      z[j] *= inv;
      if (norm && weight) z[j] *= weight[(part * group + i + j) % weight_period];
      if (!gate_first) z[j] *= gate[j];
    }
    if (wide) {
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(o + i) = make_float4(z[0], z[1], z[2], z[3]);
      } else {
        uint2 packed;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
        h[0] = __floats2bfloat162_rn(z[0], z[1]);
        h[1] = __floats2bfloat162_rn(z[2], z[3]);
        *reinterpret_cast<uint2*>(o + i) = packed;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i + j] = from_float<T>(z[j]);
    }
  }
}

// ------------------------------------------------------------ xIELU
// z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2;  pq = {p, q}.
template <typename T>
__global__ void xielu_kernel(const T* in, T* __restrict__ out, const float* __restrict__ pq, size_t n,
                             int vector) {
  pdl_trigger();
  const float up = softplus_f(pq[0]), down = 0.5f + softplus_f(pq[1]);
  pdl_wait();
  auto one = [&](float z) {
    // exp(z) - 1 - z loses digits for small |z|, but beside z / 2 what is lost is below a sixteen-bit result's last
    // place; the 32-bit engine takes expm1f
    const float grown = sizeof(T) == 2 ? __expf(z) - 1.0f : expm1f(z);
    return z > 0.0f ? up * z * z + 0.5f * z : down * (grown - z) + 0.5f * z;
  };
  const size_t quads = vector ? n >> 2 : 0;      // four at a time where both rows start on 16 bytes
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < quads;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float z[4];
    if constexpr (sizeof(T) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(in + idx * 4);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 lo = __bfloat1622float2(h[0]), hi = __bfloat1622float2(h[1]);
      z[0] = lo.x; z[1] = lo.y; z[2] = hi.x; z[3] = hi.y;
      uint2 packed;
      __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&packed);
      ph[0] = __floats2bfloat162_rn(one(z[0]), one(z[1]));
      ph[1] = __floats2bfloat162_rn(one(z[2]), one(z[3]));
      *reinterpret_cast<uint2*>(out + idx * 4) = packed;
    } else {
      const float4 v = *reinterpret_cast<const float4*>(in + idx * 4);
      *reinterpret_cast<float4*>(out + idx * 4) = make_float4(one(v.x), one(v.y), one(v.z), one(v.w));
    }
  }
  for (size_t idx = (quads << 2) + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[idx] = from_float<T>(one(to_float(in[idx])));
}

// weighted sum of two results: out = a_scale * a + b_scale * b (float32 arithmetic)
template <typename T>
__global__ void scaled_sum_kernel(const T* a, const T* b, float a_scale, float b_scale,
                                  T* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[idx] = from_float<T>(a_scale * to_float(a[idx]) + b_scale * to_float(b[idx]));
}

inline unsigned flat_blocks(long long total, int threads) {
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks);
}

}  // namespace rl

extern "C" {

// out = silu(conv(x)) for every row of the step, then the slots' tails are brought up to date.
int rl_causal_conv_silu(int dtype, const void* x, int x_stride, int col0, const float* taps, const float* bias,
                        float* state, long long state_stride, int state_off, float* out, const int* cu_seqlens,
                        const int* entry_slot, const int* entry_start, int entries, int tokens, int channels,
                        int width, int slots, int* fault, int act, int pdl, cudaStream_t stream) {
  if (tokens == 0 || channels == 0) return 0;
  if (width < 1 || width > rl::kMaxTaps || entries < 1 || act < 0 || act > 1) return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    const bool pairs = channels % 2 == 0 && col0 % 2 == 0 && x_stride % 2 == 0 &&
                       (reinterpret_cast<uintptr_t>(x) & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0;
    const long long tiles = (tokens + rl::kConvRows - 1) / rl::kConvRows;
    const long long threads = tiles * (pairs ? channels / 2 : channels);
    auto kernel = pairs ? rl::causal_conv_silu_kernel<scalar_t, 2, 0> : rl::causal_conv_silu_kernel<scalar_t, 1, 0>;
    if (pairs && width == 4) kernel = rl::causal_conv_silu_kernel<scalar_t, 2, 4>;
    if (pairs && width == 3) kernel = rl::causal_conv_silu_kernel<scalar_t, 2, 3>;
    if (pairs && width == 2) kernel = rl::causal_conv_silu_kernel<scalar_t, 2, 2>;
    int code = rl::launch_kernel(kernel, dim3(static_cast<unsigned>((threads + 127) / 128)), dim3(128), 0,
                                 stream, pdl != 0, static_cast<const scalar_t*>(x), x_stride, col0, taps, bias,
                                 static_cast<const float*>(state), state_stride, state_off, out, cu_seqlens,
                                 entry_slot, entry_start, entries, tokens, channels, width, slots, fault, act);
    if (code != 0 || width == 1) return code;
    return rl::launch_kernel(rl::conv_tail_update_kernel<scalar_t>,
                             dim3(rl::flat_blocks(static_cast<long long>(entries) * channels, 256)), dim3(256), 0,
                             stream, pdl != 0, static_cast<const scalar_t*>(x), x_stride, col0, state, state_stride,
                             state_off, cu_seqlens, entry_slot, entry_start, entries, channels, width, slots);
  });
  return 0;
}

int rl_activate_rows(int dtype, const void* x, int x_stride, int col0, float* out, int tokens, int channels, int act,
                     int pdl, cudaStream_t stream) {
  if (tokens == 0 || channels == 0) return 0;
  if (act < 0 || act > 1) return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::activate_rows_kernel<scalar_t>,
                             dim3(rl::flat_blocks(static_cast<long long>(tokens) * channels, 256)), dim3(256), 0, stream,
                             pdl != 0, static_cast<const scalar_t*>(x), x_stride, col0, out, tokens, channels, act);
  });
  return 0;
}

int rl_decay_gate(int dtype, const void* x, int x_stride, int col0, const float* rate, const float* bias, int per,
                  float* decay, float* step, int tokens, int channels, int pdl, cudaStream_t stream) {
  if (tokens == 0 || channels == 0) return 0;
  if (per < 1) return static_cast<int>(cudaErrorInvalidValue);
  const bool wide = channels % 4 == 0 && x_stride % 4 == 0 && col0 % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(decay) | reinterpret_cast<uintptr_t>(step)) & 15) == 0;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = wide ? rl::decay_gate_kernel<scalar_t, true> : rl::decay_gate_kernel<scalar_t, false>;
    return rl::launch_kernel(kernel, dim3(rl::flat_blocks(static_cast<long long>(tokens) * channels / (wide ? 4 : 1), 256)),
                             dim3(256), 0, stream, pdl != 0, static_cast<const scalar_t*>(x), x_stride, col0, rate, bias,
                             per, decay, step, tokens, channels);
  });
  return 0;
}

int rl_exp_decay(int dtype, const void* x, int x_stride, int col0, const float* bias, float* decay, int tokens,
                 int channels, int pdl, cudaStream_t stream) {
  if (tokens == 0 || channels == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::exp_decay_kernel<scalar_t>,
                             dim3(rl::flat_blocks(static_cast<long long>(tokens) * channels, 256)), dim3(256), 0, stream,
                             pdl != 0, static_cast<const scalar_t*>(x), x_stride, col0, bias, decay, tokens, channels);
  });
  return 0;
}

int rl_tanh_rows(int dtype, const void* x, void* out, long long total, int pdl, cudaStream_t stream) {
  if (total == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::tanh_rows_kernel<scalar_t>, dim3(rl::flat_blocks(total, 256)), dim3(256), 0, stream,
                             pdl != 0, static_cast<const scalar_t*>(x), static_cast<scalar_t*>(out), total);
  });
  return 0;
}

int rl_shift_mix(int dtype, const void* x, int x_stride, const float* mu, int mixes, void* out, float* kept,
                 long long kept_stride, int kept_off, const int* cu_seqlens, const int* entry_slot,
                 const int* entry_start, int entries, int tokens, int channels, int slots, int* fault, int pdl,
                 cudaStream_t stream) {
  if (tokens == 0 || channels == 0) return 0;
  if (mixes < 1 || entries < 1) return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::shift_mix_kernel<scalar_t>, dim3(tokens), dim3(channels >= 1024 ? 256 : 128), 0, stream,
                             pdl != 0, static_cast<const scalar_t*>(x), x_stride, mu, mixes, static_cast<scalar_t*>(out),
                             kept, kept_stride, kept_off, cu_seqlens, entry_slot, entry_start, entries, tokens, channels,
                             slots, fault);
  });
  return 0;
}

int rl_unit_heads(int dtype, float* rows, int stride, int col0, int heads, int dim, float eps, int split,
                  float scale_low, float scale_high, const void* gate_in, int gate_stride, int gate_col0, int gates,
                  float* gate_out, int tokens, int pdl, cudaStream_t stream) {
  if (tokens == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::unit_heads_kernel<scalar_t>, dim3(tokens), dim3(128), 0, stream, pdl != 0, rows,
                             stride, col0, heads, dim, eps, split, scale_low, scale_high,
                             static_cast<const scalar_t*>(gate_in), gate_stride, gate_col0, gates, gate_out, tokens);
  });
  return 0;
}

int rl_rotate_heads(int dtype, const void* in, int in_stride, int q_col0, int k_col0, int v_col0, float* out,
                    const int* positions, const float* inv_freq, int heads, int dim, int vdim, int rot, float k_scale,
                    int tokens, int pdl, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (rot < 0 || rot > dim || (rot & 1)) return static_cast<int>(cudaErrorInvalidValue);
  const bool wide = rot % 8 == 0 && dim % 4 == 0 && vdim % 4 == 0 && in_stride % 4 == 0 && q_col0 % 4 == 0 &&
                    k_col0 % 4 == 0 && v_col0 % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::rotate_heads_kernel<scalar_t>, dim3(tokens), dim3(256), rot * sizeof(float), stream, pdl != 0,
                             static_cast<const scalar_t*>(in), in_stride, q_col0, k_col0, v_col0, out, positions,
                             inv_freq, heads, dim, vdim, rot, k_scale, tokens, static_cast<int>(wide));
  });
  return 0;
}

int rl_linear_scan(const float* q, int q_stride, const float* k, int k_stride, const float* v, int v_stride,
                   const float* decay, int decay_mode, const float* beta, const float* v_scale, const float* skip,
                   const float* bonus, float* out, int out_stride, float* state, long long state_stride, int state_off,
                   const int* cu_seqlens, const int* entry_slot, const int* entry_start, int entries, int heads,
                   int kv_heads, int dim, int vdim, int slots, int* fault, int pdl, cudaStream_t stream) {
  if (entries == 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || dim < 1 || dim > 1024 || vdim < 1 || decay_mode < 0 ||
      decay_mode > 2 || decay == nullptr || (bonus != nullptr && beta != nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  // rows a lane holds: few, so that a column's work spreads over many lanes; as many lanes a column as it takes
  const int rows = dim <= 32 ? 4 : (dim <= 256 ? 8 : (dim <= 512 ? 16 : 32));
  int partners = 1;
  while (partners * rows < dim) partners *= 2;
  rl::ScanArgs a;
  a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
  a.decay = decay; a.decay_mode = decay_mode; a.beta = beta; a.v_scale = v_scale; a.skip = skip; a.bonus = bonus;
  a.out = out; a.out_stride = out_stride; a.state = state; a.state_stride = state_stride; a.state_off = state_off;
  a.cu_seqlens = cu_seqlens; a.entry_slot = entry_slot; a.entry_start = entry_start;
  a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.slots = slots; a.partners = partners;
  a.fault = fault;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  a.wide_in = dim % 4 == 0 && vdim % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 &&
              aligned(q) && aligned(k) && aligned(v) && (decay_mode != 2 || aligned(decay));
  const int tile_cols = (rl::kScanThreads / 32) * (32 / partners);
  const int dim_padded = partners * rows;
  const int per_token = (decay_mode == 2 ? 3 : 2) * dim_padded + tile_cols + 2;
  int run = (20 * 1024 / 4) / per_token;      // two buffers of a run each within 40 KB
  a.run = run > 16 ? 16 : (run < 1 ? 1 : run);
  const size_t smem = 2 * static_cast<size_t>((a.run * per_token + 3) & ~3) * sizeof(float);
  const dim3 grid(entries, heads, (vdim + tile_cols - 1) / tile_cols), block(rl::kScanThreads);
#define RL_SCAN(R, P) \
  if (rows == R && partners == P) return rl::launch_kernel(rl::linear_scan_kernel<R, P>, grid, block, smem, stream, pdl != 0, a)
  RL_SCAN(4, 1); RL_SCAN(4, 2); RL_SCAN(4, 4); RL_SCAN(4, 8);
  RL_SCAN(8, 8); RL_SCAN(8, 16); RL_SCAN(8, 32);
  RL_SCAN(16, 32); RL_SCAN(32, 32);
#undef RL_SCAN
  return static_cast<int>(cudaErrorInvalidValue);
}

// y_f32: y is float32 whatever the engine's dtype (the result of a recurrence); else y has the engine's dtype.
int rl_gated_norm(int dtype, int y_f32, const void* y, int y_stride, const void* g, int g_stride, int g_col0, int act,
                  int gate_first, int norm, const float* weight, int weight_period, float eps, void* out, int tokens,
                  int group, int groups, int pdl, cudaStream_t stream) {
  if (tokens == 0 || groups == 0) return 0;
  if (group < 1 || act < 0 || act > 2 || (weight != nullptr && weight_period < 1))
    return static_cast<int>(cudaErrorInvalidValue);
  int threads = 32;
  while (threads < 256 && threads * 2 <= group) threads *= 2;
  const dim3 grid(tokens, groups), block(threads);
  // a warp per (token, group) while a group is a warp's work; a group of thousands of columns (one norm over all
  // heads) takes a block, or the few warps of a small step would each walk it alone
  if (group % 4 == 0 && group <= 512) {
    const long long total = static_cast<long long>(tokens) * groups;
    const dim3 warp_grid(static_cast<unsigned>((total + 7) / 8)), warp_block(256);
    const bool wide = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                      y_stride % 4 == 0 && g_stride % 4 == 0 && g_col0 % 4 == 0;
    RL_DISPATCH_DTYPE(dtype, {
      if (y_f32)
        return rl::launch_kernel(rl::gated_norm_warp_kernel<float, scalar_t>, warp_grid, warp_block, 0, stream, pdl != 0,
                                 static_cast<const float*>(y), y_stride, static_cast<const scalar_t*>(g), g_stride,
                                 g_col0, act, gate_first, norm, weight, weight_period, eps,
                                 static_cast<scalar_t*>(out), group, groups, total, static_cast<int>(wide));
      return rl::launch_kernel(rl::gated_norm_warp_kernel<scalar_t, scalar_t>, warp_grid, warp_block, 0, stream, pdl != 0,
                               static_cast<const scalar_t*>(y), y_stride, static_cast<const scalar_t*>(g), g_stride,
                               g_col0, act, gate_first, norm, weight, weight_period, eps,
                               static_cast<scalar_t*>(out), group, groups, total, static_cast<int>(wide));
    });
  }
  RL_DISPATCH_DTYPE(dtype, {
    if (y_f32)
      return rl::launch_kernel(rl::gated_norm_kernel<float, scalar_t>, grid, block, 0, stream, pdl != 0,
                               static_cast<const float*>(y), y_stride, static_cast<const scalar_t*>(g), g_stride,
                               g_col0, act, gate_first, norm, weight, weight_period, eps, static_cast<scalar_t*>(out),
                               group, groups);
    return rl::launch_kernel(rl::gated_norm_kernel<scalar_t, scalar_t>, grid, block, 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(y), y_stride, static_cast<const scalar_t*>(g), g_stride,
                             g_col0, act, gate_first, norm, weight, weight_period, eps, static_cast<scalar_t*>(out),
                             group, groups);
  });
  return 0;
}

int rl_xielu(int dtype, const void* in, void* out, const float* pq, long long n, int pdl, cudaStream_t stream) {
  if (n == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::xielu_kernel<scalar_t>, dim3(rl::flat_blocks((n + 3) / 4, 256)), dim3(256), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(in), static_cast<scalar_t*>(out), pq, static_cast<size_t>(n),
                             static_cast<int>(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0));
  });
  return 0;
}

int rl_scaled_sum(int dtype, const void* a, const void* b, float a_scale, float b_scale, void* out, long long n,
                  int pdl, cudaStream_t stream) {
  if (n == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::scaled_sum_kernel<scalar_t>, dim3(rl::flat_blocks(n, 256)), dim3(256), 0, stream,
                             pdl != 0, static_cast<const scalar_t*>(a), static_cast<const scalar_t*>(b), a_scale,
                             b_scale, static_cast<scalar_t*>(out), static_cast<size_t>(n));
  });
  return 0;
}

}  // extern "C"
