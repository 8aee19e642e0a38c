// Embedding gather, residual-add + RMSNorm, SiLU(gate)*up.
//
// The reference runs these as a library gather (rapid_llm/modules/vocab_parallel.py:101-103),
// Triton row kernels (rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:22-85,197-240) and a
// Triton SwiGLU kernel (rapid_llm/kernels/ops/activation/swiglu.py:91-121).  Here the
// residual stream is a float32 buffer in both engine precisions: the sum x + r is formed
// and kept in 32-bit, and the norm's statistics, scaling and weight product are 32-bit
// with one rounding at the store.
//
// Rows whose length is a multiple of 8 move in 16- and 32-byte accesses; other lengths take
// the element-by-element path of the same kernel.  The order of every sum is fixed by the
// row length and the block size alone, so a row's result does not depend on the batch.
#include "common.cuh"

namespace rl {

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ---------------------------------------------------------------- embedding
// An id -(r + 1) stands for "the token in feedback[r]": the id the previous step sampled into
// row r of its result, which the host may not have read yet.
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, const int* __restrict__ feedback,
                                 int feedback_rows, int hidden, int vocab, int* __restrict__ fault,
                                 float scale, float* __restrict__ stream) {
  pdl_trigger();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 && feedback != nullptr && -(id + 1) < feedback_rows) id = feedback[-(id + 1)];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultTokenId);
    id = 0;
  }
  const T* src = table + static_cast<size_t>(id) * hidden;
  T* dst = out + static_cast<size_t>(row) * hidden;
  constexpr int kVec = 16 / sizeof(T);
  pdl_wait();   // the output buffer may still be read by the previous step's kernels
  if (scale != 1.0f || stream != nullptr) {
    // a scaled embedding: the float32 product opens the residual stream, `out` is its rounding
    float* sr = stream ? stream + static_cast<size_t>(row) * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = to_float(src[i]) * scale;
      if (sr) sr[i] = v;
      dst[i] = from_float<T>(v);
    }
    return;
  }
  if (hidden % kVec == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < hidden / kVec; i += blockDim.x) d[i] = s[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

// ------------------------------------------------------------ token + token-pair + position rows
// out[t] = table[id] + pair_table[row] + position_table[p], a float32 sum that also opens the residual stream.
// The pair's row is (previous id * mul_prev + id * mul_cur) mod buckets; a request's first token has no previous
// one and takes row `buckets`, the table's last.  The previous id of a row is the row before it in the same entry;
// for an entry's first row it is the id the request's slot keeps in `last_token`, which that same block then
// brings up to date (the entry's last id), so that no other block touches the slot's word.
template <typename T>
__global__ void embedding_sum_kernel(T* __restrict__ out, float* __restrict__ stream, const T* __restrict__ table,
                                     const T* __restrict__ pair_table, const T* __restrict__ position_table,
                                     const int* __restrict__ ids, const int* __restrict__ feedback, int feedback_rows,
                                     const int* __restrict__ positions, const int* __restrict__ cu_seqlens,
                                     const int* __restrict__ entry_slot, int entries, int* last_token, int slots,
                                     int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur,
                                     int max_positions, int* __restrict__ fault) {
  pdl_trigger();
  const int t = blockIdx.x;
  auto id_of = [&](int row) {
    int id = ids[row];
    if (id < 0 && feedback != nullptr && -(id + 1) < feedback_rows) id = feedback[-(id + 1)];
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) atomicOr(fault, kFaultTokenId);
      id = 0;
    }
    return id;
  };
  const int e = entry_of(cu_seqlens, entries, t);
  const int first = cu_seqlens[e], last = cu_seqlens[e + 1] - 1;
  int slot = entry_slot[e];
  const bool slot_ok = slot >= 0 && slot < slots;
  int pos = positions[t];
  if (pos < 0 || pos >= max_positions) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultPosition);
    pos = 0;
  }
  if (!slot_ok && threadIdx.x == 0) atomicOr(fault, kFaultSlot);
  const int id = id_of(t);
  long long row = buckets;
  if (pos > 0) {
    const int before = t > first ? id_of(t - 1) : (slot_ok ? last_token[slot] : 0);
    row = (before * mul_prev + id * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  __syncthreads();      // every thread has read the kept id before one of them replaces it
  if (t == first && slot_ok && threadIdx.x == 0) last_token[slot] = id_of(last);
  const T* a = table + static_cast<size_t>(id) * hidden;
  const T* b = pair_table + static_cast<size_t>(row) * hidden;
  const T* c = position_table + static_cast<size_t>(pos) * hidden;
  T* dst = out + static_cast<size_t>(t) * hidden;
  float* sr = stream ? stream + static_cast<size_t>(t) * hidden : nullptr;
  pdl_wait();
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_float(a[i]) + to_float(b[i]) + to_float(c[i]);
    if (sr) sr[i] = v;
    dst[i] = from_float<T>(v);
  }
}

// ------------------------------------------------------------ add + RMSNorm
// One block per output row.  Row i of the output reads input row `row_index[i]`
// (or i when row_index is null).
//   mode 0: r = x                 (first layer: the residual stream starts here)
//   mode 1: r = x + residual
//   mode 2: r = x, residual untouched and may be null (a plain norm)
//   mode 3: r = residual, x unread (the norm of the stream itself, for models whose sublayers add
//           their normed outputs to it)
//   mode 4: the norm sits on a sublayer's output: y = x * rsqrt(mean(x^2) + eps) * weight joins the
//           stream, residual += y (stored), and out = the new residual rounded to the engine's dtype,
//           which is what the next sublayer reads
//   mode 5: as mode 4, and then the norm in front of the next sublayer at once: out = the new residual
//           * rsqrt(mean(residual^2) + eps) * extra_vector, where `extra_vector` is that second norm's weight
//           (no addend goes with this mode)
// With `write_residual` the sum is stored back to `residual` (float32).
// `extra_rows` (a row per token, the dtype of x) and `extra_vector` (float32, one row for all
// tokens), where given, are added to r in that order before it is stored or normed: what a model
// feeds into the stream between two layers.
// out = r * rsqrt(mean(r^2) + eps) * weight, all in float32, rounded once.
//
// kVector: hidden is a multiple of 8 and the block has at least hidden / 8 threads; a thread
// keeps its eight values (and the weights, fetched before the sum) in registers.
template <typename TX, typename TOut, bool kVector>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, TOut* __restrict__ out,
                                   const int* __restrict__ row_index, int hidden, float eps,
                                   int mode, int write_residual, const TX* extra_rows,
                                   const float* __restrict__ extra_vector) {
  extern __shared__ float row_values[];  // [hidden] on the element-by-element path
  __shared__ float scratch[32];
  pdl_trigger();
  const int out_row = blockIdx.x;
  const int in_row = row_index ? row_index[out_row] : out_row;
  const TX* xr = x + static_cast<size_t>(in_row) * hidden;
  float* rr = residual ? residual + static_cast<size_t>(in_row) * hidden : nullptr;
  const TX* er = extra_rows ? extra_rows + static_cast<size_t>(in_row) * hidden : nullptr;
  TOut* o = out + static_cast<size_t>(out_row) * hidden;

  if constexpr (kVector) {
    const int at = threadIdx.x * 8;
    const bool active = at < hidden;
    float w[8], v[8];
    if (active) load8(weight + at, w);
    pdl_wait();
    float sum_sq = 0.0f;
    if (active) {
      if (mode == 3) load8(rr + at, v); else load8(xr + at, v);
      if (mode == 1) {
        float r[8];
        load8(rr + at, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += r[i];
      }
      if (er) {
        float extra[8];
        load8(er + at, extra);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += extra[i];
      }
      if (extra_vector && mode != 5) {
        float extra[8];
        load8(extra_vector + at, extra);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += extra[i];
      }
      if (write_residual && mode < 4) store8(rr + at, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum_sq += v[i] * v[i];
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float inv_rms = rsqrtf(sum_sq / static_cast<float>(hidden) + eps);
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * inv_rms * w[i];
      if (mode >= 4) {
        float r[8];
        load8(rr + at, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += r[i];
        store8(rr + at, v);
      }
      if (mode != 5) store8(o + at, v);
    }
    if (mode == 5) {
      float again = 0.0f;
      if (active) {
#pragma unroll
        for (int i = 0; i < 8; ++i) again += v[i] * v[i];
      }
      again = block_sum(again, scratch);
      const float inv_next = rsqrtf(again / static_cast<float>(hidden) + eps);
      if (active) {
        load8(extra_vector + at, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] * inv_next * w[i];
        store8(o + at, v);
      }
    }
  } else {
    pdl_wait();
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = mode == 3 ? rr[i] : to_float(xr[i]);
      if (mode == 1) v += rr[i];
      if (er) v += to_float(er[i]);
      if (extra_vector && mode != 5) v += extra_vector[i];
      if (write_residual && mode < 4) rr[i] = v;
      row_values[i] = v;
      sum_sq += v * v;
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float inv_rms = rsqrtf(sum_sq / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = row_values[i] * inv_rms * weight[i];
      if (mode >= 4) {
        v += rr[i];
        rr[i] = v;
      }
      if (mode == 5) row_values[i] = v; else o[i] = from_float<TOut>(v);
    }
    if (mode == 5) {
      float again = 0.0f;
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) again += row_values[i] * row_values[i];
      again = block_sum(again, scratch);
      const float inv_next = rsqrtf(again / static_cast<float>(hidden) + eps);
      for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = from_float<TOut>(row_values[i] * inv_next * extra_vector[i]);
    }
  }
}

// ------------------------------------------------------------ layer norm (mean, variance, weight, bias)
// One block per output row; row i reads input row `row_index[i]` (or i).  With r = x + res_scale * residual
// (either operand may be absent), the norm is n = (r - mean(r)) * rsqrt(var(r) + eps) * weight + bias, the
// variance being the mean of the squared deviations (formed in a second pass over the row's values, which stay
// in registers or shared memory), all float32.  `store` 1 puts the sum r back into `residual` (a norm in front
// of a sublayer), 2 puts the norm n there (a norm behind the sum: the stream's new value is the norm itself).
// out = n * gain, rounded once to the engine's dtype.
template <typename T, bool kVector>
__global__ void layernorm_kernel(const T* __restrict__ x, float* __restrict__ residual,
                                 const float* __restrict__ weight, const float* __restrict__ bias,
                                 T* __restrict__ out, const int* __restrict__ row_index, int hidden, float eps,
                                 float res_scale, int store, float gain) {
  extern __shared__ float row_values[];  // [hidden] on the element-by-element path
  __shared__ float scratch[32];
  pdl_trigger();
  const int out_row = blockIdx.x;
  const int in_row = row_index ? row_index[out_row] : out_row;
  const T* xr = x ? x + static_cast<size_t>(in_row) * hidden : nullptr;
  float* rr = residual ? residual + static_cast<size_t>(in_row) * hidden : nullptr;
  T* o = out + static_cast<size_t>(out_row) * hidden;
  const float count = static_cast<float>(hidden);
  if constexpr (kVector) {
    const int at = threadIdx.x * 8;
    const bool active = at < hidden;
    float w[8], b[8], v[8];
    if (active) {
      load8(weight + at, w);
      if (bias) load8(bias + at, b);
    }
    pdl_wait();
    float sum = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
      if (xr) load8(xr + at, v);
      if (rr) {
        float r[8];
        load8(rr + at, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fmaf(res_scale, r[i], v[i]);
      }
      if (store == 1) store8(rr + at, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[i];
    }
    const float mean = block_sum(sum, scratch) / count;
    float dev = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] -= mean;
        dev += v[i] * v[i];
      }
    }
    const float inv = rsqrtf(block_sum(dev, scratch) / count + eps);
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * w[i] + (bias ? b[i] : 0.0f);
      if (store == 2) store8(rr + at, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= gain;
      store8(o + at, v);
    }
  } else {
    pdl_wait();
    float sum = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = xr ? to_float(xr[i]) : 0.0f;
      if (rr) v = fmaf(res_scale, rr[i], v);
      if (store == 1) rr[i] = v;
      row_values[i] = v;
      sum += v;
    }
    const float mean = block_sum(sum, scratch) / count;
    float dev = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = row_values[i] - mean;
      dev += d * d;
    }
    const float inv = rsqrtf(block_sum(dev, scratch) / count + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float n = (row_values[i] - mean) * inv * weight[i] + (bias ? bias[i] : 0.0f);
      if (store == 2) rr[i] = n;
      o[i] = from_float<T>(n * gain);
    }
  }
}

// ------------------------------------------------------------ a sigmoid gate, entry by entry
// out[t, c] = rows[t, c] * sigmoid(gate[t, c]), float32 arithmetic, one rounding; `gate` may be a view of some
// columns of wider rows (gate_stride).  kVector: eight entries (16 bytes of bfloat16) a thread and step.
template <typename T, bool kVector>
__global__ void sigmoid_gate_kernel(const T* __restrict__ rows, const T* __restrict__ gate, int gate_stride,
                                    T* __restrict__ out, int tokens, int width) {
  pdl_trigger();
  pdl_wait();
  constexpr int kStep = kVector ? 8 : 1;
  const size_t per_row = static_cast<size_t>(width / kStep);
  const size_t total = static_cast<size_t>(tokens) * per_row;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = idx / per_row;
    const int c = static_cast<int>(idx - t * per_row) * kStep;
    if constexpr (kVector) {
      float v[8], g[8];
      load8(rows + t * width + c, v);
      load8(gate + t * gate_stride + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] / (1.0f + expf(-g[i]));
      store8(out + t * width + c, v);
    } else {
      const float g = to_float(gate[t * gate_stride + c]);
      out[t * width + c] = from_float<T>(to_float(rows[t * width + c]) / (1.0f + expf(-g)));
    }
  }
}

// ---------------------------------------------------------------- SiLU * up
// gate_up is [rows, 2 * inter] with the gate in columns [0, inter) and up in
// [inter, 2 * inter); out[r, c] = silu(gate) * up with silu(z) = z * sigmoid(z), in float32.
// Sixteen-bit outputs keep 8 bits of mantissa: the fast exponential and division (a few units in
// the last place of float32) change no result; the 32-bit engine takes the exact ones.
template <typename T>
__device__ __forceinline__ float silu_times(float gate, float up) {
  if constexpr (sizeof(T) == 2) {
    return __fdividef(gate, 1.0f + __expf(-gate)) * up;
  } else {
    return gate / (1.0f + expf(-gate)) * up;
  }
}

template <typename T, bool kVector>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows,
                                int inter) {
  pdl_trigger();
  pdl_wait();
  constexpr int kStep = kVector ? 8 : 1;
  const size_t per_row = static_cast<size_t>(inter / kStep);
  const size_t total = static_cast<size_t>(rows) * per_row;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / per_row;
    const int c = static_cast<int>(idx - r * per_row) * kStep;
    const T* gate = gate_up + r * 2 * inter + c;
    if constexpr (kVector) {
      float g[8], u[8];
      load8(gate, g);
      load8(gate + inter, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = silu_times<T>(g[i], u[i]);
      store8(out + r * inter + c, g);
    } else {
      const float g = to_float(gate[0]);
      const float u = to_float(gate[inter]);
      out[r * inter + c] = from_float<T>(silu_times<T>(g, u));
    }
  }
}

// ------------------------------------------------------- clamped gate * (up + 1)
// gate_up as above; g = min(gate, limit), u = clamp(up, -limit, limit);
// out = g * sigmoid(alpha * g) * (u + 1), in float32, rounded once.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter,
                                   float limit, float alpha) {
  pdl_trigger();
  pdl_wait();
  const size_t total = static_cast<size_t>(rows) * inter;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / inter;
    const size_t c = idx - r * inter;
    const float g = fminf(to_float(gate_up[r * 2 * inter + c]), limit);
    const float u = fminf(fmaxf(to_float(gate_up[r * 2 * inter + inter + c]), -limit), limit);
    out[idx] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
  }
}

// -------------------------------------------------------------- conversions
template <typename TIn>
__global__ void to_float_kernel(const TIn* __restrict__ in, float* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[idx] = to_float(in[idx]);
}

// ------------------------------------------------------------ block-table rows
// table[slots[i], :] = rows[i, :]: the block-table rows that changed on the host, brought over
// with the step's metadata instead of one copy per row.
__global__ void scatter_rows_kernel(int* __restrict__ table, int row_len, int table_rows,
                                    const int* __restrict__ slots, const int* __restrict__ rows,
                                    int* __restrict__ fault) {
  const int slot = slots[blockIdx.x];
  if (slot < 0 || slot >= table_rows) {
    if (threadIdx.x == 0) atomicOr(fault, kFaultSlot);
    return;
  }
  for (int c = threadIdx.x; c < row_len; c += blockDim.x)
    table[static_cast<size_t>(slot) * row_len + c] = rows[static_cast<size_t>(blockIdx.x) * row_len + c];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace rl

extern "C" {

int rl_embedding(int dtype, void* out, const void* table, const int* ids, const int* feedback,
                 int feedback_rows, int rows, int hidden, int vocab, int* fault, float scale, float* stream_out,
                 int pdl, cudaStream_t stream) {
  if (rows == 0) return 0;
  RL_DISPATCH_DTYPE(dtype, {
    const int threads = hidden >= 2048 ? 256 : 128;
    return rl::launch_kernel(rl::embedding_kernel<scalar_t>, dim3(rows), dim3(threads), 0, stream, pdl != 0,
                             static_cast<scalar_t*>(out), static_cast<const scalar_t*>(table), ids, feedback,
                             feedback_rows, hidden, vocab, fault, scale, stream_out);
  });
  return 0;
}

int rl_embedding_sum(int dtype, void* out, float* stream_out, const void* table, const void* pair_table,
                     const void* position_table, const int* ids, const int* feedback, int feedback_rows,
                     const int* positions, const int* cu_seqlens, const int* entry_slot, int entries, int* last_token,
                     int slots, int rows, int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur,
                     int max_positions, int* fault, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (entries < 1 || buckets < 1 || hidden < 1) return static_cast<int>(cudaErrorInvalidValue);
  RL_DISPATCH_DTYPE(dtype, {
    const int threads = hidden >= 2048 ? 256 : 128;
    return rl::launch_kernel(rl::embedding_sum_kernel<scalar_t>, dim3(rows), dim3(threads), 0, stream, false,
                             static_cast<scalar_t*>(out), stream_out, static_cast<const scalar_t*>(table),
                             static_cast<const scalar_t*>(pair_table), static_cast<const scalar_t*>(position_table),
                             ids, feedback, feedback_rows, positions, cu_seqlens, entry_slot, entries, last_token, slots,
                             hidden, vocab, buckets, mul_prev, mul_cur, max_positions, fault);
  });
  return 0;
}

// x and out are `dtype`; residual and weight are float32.
int rl_add_rmsnorm(int dtype, const void* x, float* residual, const float* weight, void* out,
                   const int* row_index, int rows, int hidden, float eps, int mode,
                   int write_residual, const void* extra_rows, const float* extra_vector, int pdl,
                   cudaStream_t stream) {
  if (rows == 0) return 0;
  if (mode < 0 || mode > 5 || ((mode == 1 || mode >= 3) && residual == nullptr) ||
      (mode == 5 && (extra_vector == nullptr || extra_rows != nullptr)) ||
      (write_residual && residual == nullptr) || hidden <= 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const bool vector = hidden % 8 == 0 && hidden <= 8 * 1024 && rl::aligned16(x) && rl::aligned16(out) &&
                      rl::aligned16(weight) && (residual == nullptr || rl::aligned16(residual)) &&
                      rl::aligned16(extra_rows) && rl::aligned16(extra_vector);
  RL_DISPATCH_DTYPE(dtype, {
    if (vector) {
      const int threads = (hidden / 8 + 31) / 32 * 32;
      return rl::launch_kernel(rl::add_rmsnorm_kernel<scalar_t, scalar_t, true>, dim3(rows), dim3(threads), 0,
                               stream, pdl != 0, static_cast<const scalar_t*>(x), residual, weight,
                               static_cast<scalar_t*>(out), row_index, hidden, eps, mode, write_residual,
                               static_cast<const scalar_t*>(extra_rows), extra_vector);
    }
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
    int threads = 128;
    while (threads < 1024 && threads * 8 < hidden) threads *= 2;
    auto kernel = rl::add_rmsnorm_kernel<scalar_t, scalar_t, false>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(kernel, dim3(rows), dim3(threads), smem, stream, pdl != 0,
                             static_cast<const scalar_t*>(x), residual, weight, static_cast<scalar_t*>(out),
                             row_index, hidden, eps, mode, write_residual,
                             static_cast<const scalar_t*>(extra_rows), extra_vector);
  });
  return 0;
}

// x and out are `dtype` (x may be null: the norm of the stream alone); residual, weight and bias are float32.
int rl_layernorm(int dtype, const void* x, float* residual, const float* weight, const float* bias, void* out,
                 const int* row_index, int rows, int hidden, float eps, float res_scale, int store, float gain,
                 int pdl, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (store < 0 || store > 2 || (store != 0 && residual == nullptr) || (x == nullptr && residual == nullptr) ||
      hidden <= 0 || weight == nullptr || out == nullptr)
    return static_cast<int>(cudaErrorInvalidValue);
  const bool vector = hidden % 8 == 0 && hidden <= 8 * 1024 && rl::aligned16(x) && rl::aligned16(out) &&
                      rl::aligned16(weight) && rl::aligned16(bias) && (residual == nullptr || rl::aligned16(residual));
  RL_DISPATCH_DTYPE(dtype, {
    if (vector) {
      const int threads = (hidden / 8 + 31) / 32 * 32;
      return rl::launch_kernel(rl::layernorm_kernel<scalar_t, true>, dim3(rows), dim3(threads), 0, stream, pdl != 0,
                               static_cast<const scalar_t*>(x), residual, weight, bias, static_cast<scalar_t*>(out),
                               row_index, hidden, eps, res_scale, store, gain);
    }
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
    int threads = 128;
    while (threads < 1024 && threads * 8 < hidden) threads *= 2;
    auto kernel = rl::layernorm_kernel<scalar_t, false>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(kernel, dim3(rows), dim3(threads), smem, stream, pdl != 0,
                             static_cast<const scalar_t*>(x), residual, weight, bias, static_cast<scalar_t*>(out),
                             row_index, hidden, eps, res_scale, store, gain);
  });
  return 0;
}

int rl_sigmoid_gate(int dtype, const void* rows, const void* gate, int gate_stride, void* out, int tokens, int width,
                    int pdl, cudaStream_t stream) {
  if (tokens == 0 || width == 0) return 0;
  if (width < 0 || gate_stride < width) return static_cast<int>(cudaErrorInvalidValue);
  const bool vector = width % 8 == 0 && gate_stride % 8 == 0 && rl::aligned16(rows) && rl::aligned16(gate) && rl::aligned16(out);
  const size_t total = static_cast<size_t>(tokens) * (vector ? width / 8 : width);
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = vector ? rl::sigmoid_gate_kernel<scalar_t, true> : rl::sigmoid_gate_kernel<scalar_t, false>;
    return rl::launch_kernel(kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(rows), static_cast<const scalar_t*>(gate), gate_stride,
                             static_cast<scalar_t*>(out), tokens, width);
  });
  return 0;
}

int rl_silu_mul(int dtype, const void* gate_up, void* out, int rows, int inter, int pdl,
                cudaStream_t stream) {
  if (rows == 0) return 0;
  const bool vector = inter % 8 == 0 && rl::aligned16(gate_up) && rl::aligned16(out);
  const size_t total = static_cast<size_t>(rows) * (vector ? inter / 8 : inter);
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = vector ? rl::silu_mul_kernel<scalar_t, true> : rl::silu_mul_kernel<scalar_t, false>;
    return rl::launch_kernel(kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, stream, pdl != 0,
                             static_cast<const scalar_t*>(gate_up), static_cast<scalar_t*>(out), rows, inter);
  });
  return 0;
}

int rl_clamped_glu(int dtype, const void* gate_up, void* out, int rows, int inter, float limit, float alpha,
                   int pdl, cudaStream_t stream) {
  if (rows == 0 || inter == 0) return 0;
  const size_t total = static_cast<size_t>(rows) * inter;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::clamped_glu_kernel<scalar_t>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                             stream, pdl != 0, static_cast<const scalar_t*>(gate_up), static_cast<scalar_t*>(out),
                             rows, inter, limit, alpha);
  });
  return 0;
}

int rl_scatter_rows(int* table, int row_len, int table_rows, const int* slots, const int* rows, int count,
                    int* fault, cudaStream_t stream) {
  if (count == 0 || row_len == 0) return 0;
  if (count < 0 || row_len < 0 || table_rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  rl::scatter_rows_kernel<<<count, 128, 0, stream>>>(table, row_len, table_rows, slots, rows, fault);
  return rl::launch_status();
}

int rl_to_float(int dtype, const void* in, float* out, long long n, int pdl, cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  size_t blocks = (static_cast<size_t>(n) + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::to_float_kernel<scalar_t>, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0,
                             stream, pdl != 0, static_cast<const scalar_t*>(in), out, static_cast<size_t>(n));
  });
  return 0;
}

}  // extern "C"
