// Kernels of attention over a cached latent: the keys and values of every head are products of one
// short row per token (the latent c, kv_rank numbers) and the only other thing a key holds is a rotated part
// shared by all heads (rot numbers).  The cache keeps one row [c | rotated part | zeros] of D numbers per token,
// D a multiple of 16.  With W_uk and W_uv the per-head matrices that would expand c into keys and values,
//   score(t, j, h) = (W_uk_h^T q_h) . c_j + q_rot_h . k_rot_j        o_h = W_uv_h (sum_j p_j c_j)
// so a step moves W_uk to the query side and W_uv behind the attention, and the attention itself is one
// key/value head of width D shared by all query heads, with values read from the keys' rows.
//
// All arithmetic here is float32 with one rounding at the store; angles are position * frequency in float32.
#include "common.cuh"

namespace rl {

__device__ __forceinline__ float sigmoid_exact(float x) { return 1.0f / (1.0f + expf(-x)); }

// Rotation of `rot` numbers by position.  layout 0: entry i pairs with entry i + rot / 2; layout 1: entry 2i
// pairs with entry 2i + 1.  The pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a) * magnitude with
// a = position * freq[i].
__device__ __forceinline__ void pair_places(int i, int rot, int layout, int& lo, int& hi) {
  if (layout == 0) { lo = i; hi = i + rot / 2; } else { lo = 2 * i; hi = 2 * i + 1; }
}

// ------------------------------------------------------------ norms of the two latents, the cache row
// One block per token.  `down` holds [query latent (q_rank) | ... | c (kv_rank) | key part (rot)] at the given
// columns (q_rank 0: there is no query latent, and q_out is not touched).  q_out = RMS norm of the query latent with
// weight wq; the cache row at kv_dest[t] receives
// [RMS norm of c with weight wc | rotated key part | zeros up to D].
template <typename T>
__global__ void latent_norm_write_kernel(const T* __restrict__ down, int down_stride, int q_col0, int q_rank,
                                         int c_col0, int kv_rank, int rot, const float* __restrict__ wq,
                                         const float* __restrict__ wc, float eps, T* __restrict__ q_out,
                                         T* __restrict__ cache, const int* __restrict__ kv_dest, long long cache_rows,
                                         int D, const int* __restrict__ positions, const float* __restrict__ freq,
                                         float magnitude, int layout, int* __restrict__ fault) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int t = blockIdx.x;
  const T* row = down + static_cast<size_t>(t) * down_stride;
  pdl_wait();
  float sum_q = 0.0f, sum_c = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_float(row[q_col0 + i]);
    sum_q += v * v;
  }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float v = to_float(row[c_col0 + i]);
    sum_c += v * v;
  }
  sum_q = block_sum(sum_q, scratch);
  sum_c = block_sum(sum_c, scratch);
  const float inv_q = rsqrtf(sum_q / static_cast<float>(max(q_rank, 1)) + eps);
  const float inv_c = rsqrtf(sum_c / static_cast<float>(kv_rank) + eps);
  T* qo = q_out + static_cast<size_t>(t) * q_rank;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) qo[i] = from_float<T>(to_float(row[q_col0 + i]) * inv_q * wq[i]);
  const long long dest = kv_dest[t];
  if (dest < 0 || dest >= cache_rows) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultPageId);
    return;
  }
  T* out = cache + static_cast<size_t>(dest) * D;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) out[i] = from_float<T>(to_float(row[c_col0 + i]) * inv_c * wc[i]);
  const float p = static_cast<float>(positions[t]);
  const T* kr = row + c_col0 + kv_rank;
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    int lo, hi;
    pair_places(i, rot, layout, lo, hi);
    const float a = p * freq[i];
    const float c = cosf(a) * magnitude, s = sinf(a) * magnitude;
    const float u = to_float(kr[lo]), v = to_float(kr[hi]);
    out[kv_rank + lo] = from_float<T>(u * c - v * s);
    out[kv_rank + hi] = from_float<T>(v * c + u * s);
  }
  for (int i = kv_rank + rot + threadIdx.x; i < D; i += blockDim.x) out[i] = from_float<T>(0.0f);
}

// ------------------------------------------------------------ the queries' rotated parts
// q: [T, heads * (dim + rot)], a head's last `rot` numbers are its rotated part.  wide: [T, heads * D]; a head's
// columns [kv_rank, kv_rank + rot) receive the rotation, the columns behind them zeros.  One block per token.
template <typename T>
__global__ void latent_rotate_queries_kernel(const T* __restrict__ q, int heads, int dim, int rot,
                                             T* __restrict__ wide, int kv_rank, int D,
                                             const int* __restrict__ positions, const float* __restrict__ freq,
                                             float magnitude, int layout) {
  pdl_trigger();
  const int t = blockIdx.x;
  const float p = static_cast<float>(positions[t]);
  const int half = rot / 2, tail = D - kv_rank - rot;
  const T* qr = q + static_cast<size_t>(t) * heads * (dim + rot);
  T* wr = wide + static_cast<size_t>(t) * heads * D;
  pdl_wait();
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    int lo, hi;
    pair_places(i, rot, layout, lo, hi);
    const float a = p * freq[i];
    const float c = cosf(a) * magnitude, s = sinf(a) * magnitude;
    const T* src = qr + static_cast<size_t>(h) * (dim + rot) + dim;
    const float u = to_float(src[lo]), v = to_float(src[hi]);
    T* dst = wr + static_cast<size_t>(h) * D + kv_rank;
    dst[lo] = from_float<T>(u * c - v * s);
    dst[hi] = from_float<T>(v * c + u * s);
  }
  for (int idx = threadIdx.x; idx < heads * tail; idx += blockDim.x) {
    const int h = idx / tail, i = idx - h * tail;
    wr[static_cast<size_t>(h) * D + kv_rank + rot + i] = from_float<T>(0.0f);
  }
}

// ------------------------------------------------------------ one number per head as a sigmoid gate
// rows[t, h, 0:width] *= sigmoid(gate[t, gate_col0 + h]), in place.
// kVec elements (16 bytes) a thread and round where a head's width is a multiple of kVec; else one.
template <typename T, int kVec>
__global__ void sigmoid_scale_heads_kernel(T* __restrict__ rows, int heads, int width, const T* __restrict__ gate,
                                           int gate_stride, int gate_col0, long long total) {
  pdl_trigger();
  pdl_wait();
  if constexpr (kVec > 1) {
    const int per_head = width / kVec;
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total / kVec;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long head_at = idx / per_head;
      const long long t = head_at / heads;
      const int h = static_cast<int>(head_at - t * heads);
      const float g = sigmoid_exact(to_float(gate[static_cast<size_t>(t) * gate_stride + gate_col0 + h]));
      uint4 raw = reinterpret_cast<const uint4*>(rows)[idx];
      T* part = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < kVec; ++i) part[i] = from_float<T>(to_float(part[i]) * g);
      reinterpret_cast<uint4*>(rows)[idx] = raw;
    }
    return;
  }
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long head_at = idx / width;
    const long long t = head_at / heads;
    const int h = static_cast<int>(head_at - t * heads);
    const float g = sigmoid_exact(to_float(gate[static_cast<size_t>(t) * gate_stride + gate_col0 + h]));
    rows[idx] = from_float<T>(to_float(rows[idx]) * g);
  }
}

// ------------------------------------------------------------ a product per head
// out[t, h, 0:N] = x[t, h, x_col0 : x_col0 + K] @ w[h]^T with w [heads, N, K]; x rows hold `heads` heads of
// x_width numbers, out rows `heads` heads of out_width.  Tiles of 64 x 64 outputs, the inner range in steps of
// 16 through shared memory, a 4 x 4 patch a thread, float32 sums in a fixed order (true 32-bit for float32 inputs).
constexpr int kHeadTile = 64, kHeadStep = 16;

template <typename T>
__global__ void __launch_bounds__(256) heads_linear_kernel(const T* __restrict__ x, int x_width, int x_col0,
                                                           const T* __restrict__ w, T* __restrict__ out,
                                                           int out_width, int tokens, int heads, int N, int K) {
  __shared__ float xs[kHeadStep][kHeadTile + 4];
  __shared__ float ws[kHeadStep][kHeadTile + 4];
  pdl_trigger();
  const int h = blockIdx.z;
  const int t0 = blockIdx.x * kHeadTile, n0 = blockIdx.y * kHeadTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // tx: output columns, ty: tokens
  const T* wh = w + static_cast<size_t>(h) * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += kHeadStep) {
    for (int idx = threadIdx.x; idx < kHeadTile * kHeadStep; idx += 256) {
      const int r = idx / kHeadStep, kk = idx - r * kHeadStep;
      const int t = t0 + r, n = n0 + r, k = k0 + kk;
      xs[kk][r] = (t < tokens && k < K)
                      ? to_float(x[(static_cast<size_t>(t) * heads + h) * x_width + x_col0 + k]) : 0.0f;
      ws[kk][r] = (n < N && k < K) ? to_float(wh[static_cast<size_t>(n) * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kHeadStep; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(static_cast<size_t>(t) * heads + h) * out_width + n] = from_float<T>(acc[i][j]);
    }
  }
}

// The same product for a step of few tokens, where a 64 x 64 tile would be mostly empty rows and the heads x
// columns / 64 CTAs too few: a warp per output column.  The warp keeps its weight row in registers (lane l holds
// k = l, l + 32, ..., so K <= 32 * kHeadRowRegs), and for every token multiplies it with the token's row (read
// through L1 by the eight warps of a CTA) and adds the lanes' sums down a fixed tree.
// A CTA takes kHeadTokensPerCta tokens, so a step of 64 tokens is eight times the CTAs and not eight times the walk.
// bfloat16 only: float32 keeps the tiles at every size, so that its sums have one order however a prompt is cut.
constexpr int kHeadRowRegs = 8, kHeadColumnsPerCta = 8, kHeadTokensPerCta = 8;

template <typename T>
__global__ void __launch_bounds__(32 * kHeadColumnsPerCta) heads_linear_few_kernel(
    const T* __restrict__ x, int x_width, int x_col0, const T* __restrict__ w, T* __restrict__ out, int out_width,
    int tokens, int heads, int N, int K) {
  pdl_trigger();
  const int h = blockIdx.x, lane = threadIdx.x & 31;
  const int n = blockIdx.y * kHeadColumnsPerCta + (threadIdx.x >> 5);
  if (n >= N) return;
  const T* row = w + (static_cast<size_t>(h) * N + n) * K;
  float wr[kHeadRowRegs];
#pragma unroll
  for (int i = 0; i < kHeadRowRegs; ++i) {
    const int k = lane + 32 * i;
    wr[i] = k < K ? to_float(row[k]) : 0.0f;         // weights: no kernel of the step wrote them
  }
  pdl_wait();
  const int t_end = min(tokens, (static_cast<int>(blockIdx.z) + 1) * kHeadTokensPerCta);
  for (int t = blockIdx.z * kHeadTokensPerCta; t < t_end; ++t) {
    const T* xr = x + (static_cast<size_t>(t) * heads + h) * x_width + x_col0;
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kHeadRowRegs; ++i) {
      const int k = lane + 32 * i;
      if (k < K) sum = fmaf(to_float(xr[k]), wr[i], sum);
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    if (lane == 0) out[(static_cast<size_t>(t) * heads + h) * out_width + n] = from_float<T>(sum);
  }
}

inline unsigned flat_grid(long long total, int threads) {
  const long long blocks = (total + threads - 1) / threads;
  return static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace rl

extern "C" {

int rl_latent_norm_write(int dtype, const void* down, int down_stride, int q_col0, int q_rank, int c_col0, int kv_rank,
                         int rot, const float* wq, const float* wc, float eps, void* q_out, void* cache,
                         const int* kv_dest, long long cache_rows, int D, const int* positions, const float* freq,
                         float magnitude, int layout, int tokens, int* fault, int pdl, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (q_rank < 0 || kv_rank < 1 || rot < 0 || rot % 2 || kv_rank + rot > D || layout < 0 || layout > 1 ||
      (rot > 0 && freq == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::latent_norm_write_kernel<scalar_t>, dim3(tokens), dim3(128), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(down), down_stride, q_col0, q_rank, c_col0, kv_rank, rot, wq, wc,
                             eps, static_cast<scalar_t*>(q_out), static_cast<scalar_t*>(cache), kv_dest, cache_rows, D,
                             positions, freq, magnitude, layout, fault);
  });
  return 0;
}

int rl_latent_rotate_queries(int dtype, const void* q, int heads, int dim, int rot, void* wide, int kv_rank, int D,
                             const int* positions, const float* freq, float magnitude, int layout, int tokens, int pdl,
                             cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (heads < 1 || dim < 0 || rot < 0 || rot % 2 || kv_rank + rot > D || layout < 0 || layout > 1 ||
      (rot > 0 && freq == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::latent_rotate_queries_kernel<scalar_t>, dim3(tokens), dim3(128), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(q), heads, dim, rot, static_cast<scalar_t*>(wide), kv_rank, D,
                             positions, freq, magnitude, layout);
  });
  return 0;
}

int rl_sigmoid_scale_heads(int dtype, void* rows, int heads, int width, const void* gate, int gate_stride,
                           int gate_col0, int tokens, int pdl, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * heads * width;
  if (total == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    constexpr int kVec = 16 / static_cast<int>(sizeof(scalar_t));
    if (width % kVec == 0 && reinterpret_cast<uintptr_t>(rows) % 16 == 0)
      return rl::launch_kernel(rl::sigmoid_scale_heads_kernel<scalar_t, kVec>, dim3(rl::flat_grid(total / kVec, 256)),
                               dim3(256), 0, stream, pdl != 0, static_cast<scalar_t*>(rows), heads, width,
                               static_cast<const scalar_t*>(gate), gate_stride, gate_col0, total);
    return rl::launch_kernel(rl::sigmoid_scale_heads_kernel<scalar_t, 1>, dim3(rl::flat_grid(total, 256)), dim3(256), 0,
                             stream, pdl != 0, static_cast<scalar_t*>(rows), heads, width,
                             static_cast<const scalar_t*>(gate), gate_stride, gate_col0, total);
  });
  return 0;
}

int rl_heads_linear(int dtype, const void* x, int x_width, int x_col0, const void* w, void* out, int out_width,
                    int tokens, int heads, int n_out, int k, int pdl, cudaStream_t stream) {
  if (tokens == 0 || n_out == 0) return 0;
  if (heads < 1 || heads > 65535 || k < 1 || x_col0 < 0 || x_col0 + k > x_width || n_out > out_width)
    return static_cast<int>(cudaErrorInvalidValue);
  if (dtype == rl::kBF16 && tokens <= rl::kHeadTile && k <= 32 * rl::kHeadRowRegs) {
    const dim3 few(heads, (n_out + rl::kHeadColumnsPerCta - 1) / rl::kHeadColumnsPerCta,
                   (tokens + rl::kHeadTokensPerCta - 1) / rl::kHeadTokensPerCta);
    RL_DISPATCH_DTYPE(dtype, {
      return rl::launch_kernel(rl::heads_linear_few_kernel<scalar_t>, few, dim3(32 * rl::kHeadColumnsPerCta), 0, stream,
                               pdl != 0, static_cast<const scalar_t*>(x), x_width, x_col0, static_cast<const scalar_t*>(w),
                               static_cast<scalar_t*>(out), out_width, tokens, heads, n_out, k);
    });
    return 0;
  }
  const dim3 grid((tokens + rl::kHeadTile - 1) / rl::kHeadTile, (n_out + rl::kHeadTile - 1) / rl::kHeadTile, heads);
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::heads_linear_kernel<scalar_t>, grid, dim3(256), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(x), x_width, x_col0, static_cast<const scalar_t*>(w),
                             static_cast<scalar_t*>(out), out_width, tokens, heads, n_out, k);
  });
  return 0;
}

}  // extern "C"
