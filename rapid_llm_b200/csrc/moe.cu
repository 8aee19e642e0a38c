// Routed feed-forward: router scores and top-k, grouping of the step's (token, expert) pairs by
// expert, products over the groups, and the sum over a token's experts.
//
// A step's T tokens each choose `top` of E experts; pair i = t * top + j is token t's j-th choice.
//   rl_router_topk    z = W_r h in float32 (W_r float32, h the engine's dtype), s = sigmoid(z), the
//                     `top` largest per token, chosen on z (sigmoid keeps the order; ties: the lower
//                     index) with their s as weights; extra rows of W_r behind the experts' give
//                     sigmoid gates per token (a shared expert's).  Another weighting (`weigh` 2): s = softmax(z)
//                     over all router rows; the choice is made on s + correction, among the rows of the `keep`
//                     best of `groups` equal groups of neighbours (a group ranks by its largest corrected
//                     score); the weights are the chosen rows' s over their sum.  Router rows behind the experts
//                     that have tensors are identity experts: rl_moe_plan leaves their pairs out of every tile
//                     and rl_moe_combine adds weight * the token's own row for them.
//   rl_moe_plan       counts the pairs per expert and lays them out expert by expert in tiles of
//                     kTileM rows: sorted[p] = i, tile tables, all on the device (no host round trip).
//   rl_grouped_linear out rows = A rows @ W[e]^T over the tiles; A rows are fetched by token
//                     (pair i reads row i / top) or by place p; with `gated`, W[e] is [2 F, K] (gate
//                     rows, then up rows) and out = silu(w g) * (w u), w the pair's weight: the weight
//                     scales the expert's input, and W (w h) = w (W h).  With glu_limit > 0 the unit is the
//                     clamped one: g' = min(g, limit), u' = clamp(u, +-limit), out = g' sigmoid(alpha g') (u' + 1).
//   rl_moe_combine    out[t] = sum_j y[t * top + j] (+ gate[t] * shared[t]), j in order, float32 sums.
//   rl_moe_combine_layernorm  the same sum, and at once the layer norm that closes it in an arrangement with the norm
//                     behind the sum: stream[t] <- LN(res_scale * stream[t] + sum), out[t] its rounding.
// A row's result does not depend on its tile's other rows or on the order in which the pairs of an
// expert were laid out: the inner sums run over k in a fixed order per row.
//
// Three product kernels: float32 FMA tiles (the 32-bit engine; any sizes), mma.sync m16n8k16 tiles for
// bfloat16 (float32 accumulators; any sizes), and the same instruction behind a cp.async ring with
// ldmatrix fragments on tiles of 64 pairs for bfloat16 operands whose rows are multiples of 16 bytes.
// The plan is made for the tile the product kernels will use (`tile_m`).
#include "common.cuh"

namespace rl {

constexpr int kMoeTileM = 32;     // pairs per tile
constexpr int kMoeTileN = 64;     // output columns per block
constexpr int kMoeTileK = 32;
constexpr int kMoeThreads = 256;
constexpr int kMoeWideM = 64;     // pairs per tile of the pipelined bfloat16 kernel
constexpr int kMoeWideK = 64;
constexpr int kMoeStages = 3;

__device__ __forceinline__ float moe_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// The gated unit of an expert from its two float32 products: SiLU(g) * u, or with limit > 0 the clamped unit
// min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1).
__device__ __forceinline__ float moe_unit(float g, float u, float limit, float alpha) {
  if (limit > 0.0f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
  }
  return g / (1.0f + expf(-g)) * u;
}

// ------------------------------------------------------------------ router
// One block per kRouterTokens tokens.  The block's warps share the inner range: warp w forms, for every router row
// and each of the block's tokens, the part of the product over its slice of k (the row's slice is read once for all
// the tokens; 16-byte loads where sizes and addresses allow), so a step's loads are all in flight at once instead
// of one row after the other.  The parts meet in shared memory and are added in the order of the warps.  A token's
// logits thus have a fixed order of sums, whatever else is in the block or the step.  Warp t then picks token t's
// experts.
constexpr int kRouterTokens = 4;
constexpr int kRouterWarps = 8;

__device__ __forceinline__ void router_load4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void router_load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 packed = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
  const float2 lo = __bfloat1622float2(h[0]), hi = __bfloat1622float2(h[1]);
  v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}

template <typename T>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const T* x, int x_stride, const float* __restrict__ w, int hidden, int experts,
                   int gates, int top, int* __restrict__ ids, float* __restrict__ weights,
                   float* __restrict__ gate_out, float* __restrict__ scores_out, int tokens, int wide,
                   const float* __restrict__ bias, int weigh, const float* __restrict__ correction, int groups,
                   int keep) {
  extern __shared__ float moe_scores[];      // [kRouterTokens][rows] logits, then [kRouterWarps][kRouterTokens][rows] parts
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * kRouterTokens;
  const int rows = experts + gates;
  float* parts = moe_scores + kRouterTokens * rows;
  // the warp's slice of k: whole steps of 128, so that a lane's four neighbours stay together
  const int steps = (hidden + 127) / 128, per_warp = (steps + kRouterWarps - 1) / kRouterWarps;
  const int k_begin = min(hidden, warp * per_warp * 128), k_end = min(hidden, (warp + 1) * per_warp * 128);
  pdl_wait();
  const T* xr[kRouterTokens];
#pragma unroll
  for (int i = 0; i < kRouterTokens; ++i)
    xr[i] = x + static_cast<size_t>(min(t0 + i, tokens - 1)) * x_stride;      // rows past the end repeat the last one
  if (wide) {
    // eight router rows at a time: their loads leave together (a row after the other would wait for memory once per row)
    constexpr int kRowsAtOnce = 8;
    for (int e0 = 0; e0 < rows; e0 += kRowsAtOnce) {
      float acc[kRowsAtOnce][kRouterTokens];
#pragma unroll
      for (int j = 0; j < kRowsAtOnce; ++j)
#pragma unroll
        for (int i = 0; i < kRouterTokens; ++i) acc[j][i] = 0.0f;
      for (int k = k_begin + lane * 4; k < k_end; k += 128) {
        float4 wv[kRowsAtOnce];
#pragma unroll
        for (int j = 0; j < kRowsAtOnce; ++j)
          wv[j] = *reinterpret_cast<const float4*>(w + static_cast<size_t>(min(e0 + j, rows - 1)) * hidden + k);
        float xv[kRouterTokens][4];
#pragma unroll
        for (int i = 0; i < kRouterTokens; ++i) router_load4(xr[i] + k, xv[i]);
#pragma unroll
        for (int j = 0; j < kRowsAtOnce; ++j)
#pragma unroll
          for (int i = 0; i < kRouterTokens; ++i) {
            acc[j][i] = fmaf(wv[j].x, xv[i][0], acc[j][i]);
            acc[j][i] = fmaf(wv[j].y, xv[i][1], acc[j][i]);
            acc[j][i] = fmaf(wv[j].z, xv[i][2], acc[j][i]);
            acc[j][i] = fmaf(wv[j].w, xv[i][3], acc[j][i]);
          }
      }
#pragma unroll
      for (int j = 0; j < kRowsAtOnce; ++j)
#pragma unroll
        for (int i = 0; i < kRouterTokens; ++i) {
          const float total = warp_sum(acc[j][i]);
          if (lane == 0 && e0 + j < rows) parts[(warp * kRouterTokens + i) * rows + e0 + j] = total;
        }
    }
  } else {
    for (int e = 0; e < rows; ++e) {
      const float* wr = w + static_cast<size_t>(e) * hidden;
      float acc[kRouterTokens];
#pragma unroll
      for (int i = 0; i < kRouterTokens; ++i) acc[i] = 0.0f;
      for (int k = k_begin + lane; k < k_end; k += 32) {
        const float wv = wr[k];
#pragma unroll
        for (int i = 0; i < kRouterTokens; ++i) acc[i] = fmaf(wv, to_float(xr[i][k]), acc[i]);
      }
#pragma unroll
      for (int i = 0; i < kRouterTokens; ++i) {
        const float total = warp_sum(acc[i]);
        if (lane == 0) parts[(warp * kRouterTokens + i) * rows + e] = total;
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kRouterTokens * rows; idx += blockDim.x) {
    float total = 0.0f;
#pragma unroll
    for (int part = 0; part < kRouterWarps; ++part) total += parts[part * kRouterTokens * rows + idx];
    // the logit: the choice is made on it (sigmoid keeps the order, and does not saturate into ties)
    const int row = idx % rows;
    moe_scores[idx] = total + ((bias && row < experts) ? bias[row] : 0.0f);
  }
  __syncthreads();
  if (warp >= kRouterTokens || t0 + warp >= tokens) return;
  const int t = t0 + warp;
  float* s = moe_scores + warp * rows;
  if (scores_out && weigh != 2)
    for (int e = lane; e < experts; e += 32) scores_out[static_cast<size_t>(t) * experts + e] = moe_sigmoid(s[e]);
  for (int g = lane; g < gates; g += 32) gate_out[static_cast<size_t>(t) * gates + g] = moe_sigmoid(s[experts + g]);
  __syncwarp();
  // what the choice is made on: the logits, or (weigh 2) the softmax over all rows plus a correction per row,
  // with the rows outside the `keep` best groups at minus infinity.  The parts' memory is free by now.
  float* pick = s;
  if (weigh == 2) {
    float* choice = parts + warp * rows;
    float* group_best = parts + (kRouterTokens + warp) * rows;
    float* group_kept = parts + (2 * kRouterTokens + warp) * rows;
    float largest = -INFINITY;
    for (int e = lane; e < experts; e += 32) largest = fmaxf(largest, s[e]);
    largest = warp_max(largest);
    float total = 0.0f;
    for (int e = lane; e < experts; e += 32) total += expf(s[e] - largest);
    total = warp_sum(total);
    __syncwarp();
    for (int e = lane; e < experts; e += 32) {
      const float p = expf(s[e] - largest) / total;
      s[e] = p;                                            // the plain score: what the weights are made of
      if (scores_out) scores_out[static_cast<size_t>(t) * experts + e] = p;
      choice[e] = p + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    if (groups > 1) {
      const int per = experts / groups;
      for (int g = lane; g < groups; g += 32) {
        float m = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, choice[e]);
        group_best[g] = m;
        group_kept[g] = 0.0f;
      }
      __syncwarp();
      for (int r = 0; r < keep; ++r) {
        float best = -INFINITY;
        int best_g = 0x7fffffff;
        for (int g = lane; g < groups; g += 32) {
          if (group_kept[g] == 0.0f && (group_best[g] > best || best_g == 0x7fffffff)) { best = group_best[g]; best_g = g; }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
          const float other = __shfl_xor_sync(0xffffffffu, best, offset);
          const int other_g = __shfl_xor_sync(0xffffffffu, best_g, offset);
          if (other_g != 0x7fffffff && (best_g == 0x7fffffff || other > best || (other == best && other_g < best_g))) {
            best = other;
            best_g = other_g;
          }
        }
        if (lane == 0 && best_g != 0x7fffffff) group_kept[best_g] = 1.0f;
        __syncwarp();
      }
      for (int e = lane; e < experts; e += 32)
        if (group_kept[e / per] == 0.0f) choice[e] = -INFINITY;
      __syncwarp();
    }
    pick = choice;
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = pick[e];
      if (v > best) { best = v; best_e = e; }      // a lane's lowest index wins its ties
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (best_e == 0x7fffffff) best_e = 0;      // every logit left is not a number: keep the index inside the table
    if (lane == 0) {
      ids[static_cast<size_t>(t) * top + j] = best_e;
      weights[static_cast<size_t>(t) * top + j] = weigh == 2 ? s[best_e] : (weigh == 1 ? best : moe_sigmoid(best));
      pick[best_e] = -INFINITY;      // taken
    }
    __syncwarp();
  }
  if (weigh == 1 && lane == 0) {
    // the weights are the softmax over the chosen logits alone; the first chosen is the largest
    float* w = weights + static_cast<size_t>(t) * top;
    const float largest = w[0];
    float sum = 0.0f;
    for (int j = 0; j < top; ++j) {
      w[j] = expf(w[j] - largest);
      sum += w[j];
    }
    for (int j = 0; j < top; ++j) w[j] = w[j] / sum;
  }
  if (weigh == 2 && lane == 0) {
    // the chosen rows' scores over their sum, added up in the order of the choices
    float* w = weights + static_cast<size_t>(t) * top;
    float sum = 0.0f;
    for (int j = 0; j < top; ++j) sum += w[j];
    sum += 1e-20f;
    for (int j = 0; j < top; ++j) w[j] = w[j] / sum;
  }
}

// ------------------------------------------------------------------ plan
// One block.  meta: [0] tiles, then per tile (expert, first place, rows).  `sorted` [pairs] receives pair
// indices expert by expert.  `place_of` [pairs]: where pair i went (the inverse of sorted).
__global__ void moe_plan_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ sorted,
                                int* __restrict__ place_of, int* __restrict__ meta, int max_tiles, int tile_m,
                                int* __restrict__ fault) {
  extern __shared__ int moe_counts[];      // [experts] counts, [experts] cursors
  pdl_trigger();
  int* counts = moe_counts;
  int* cursor = moe_counts + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  pdl_wait();
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = at;
      for (int row = 0; row < counts[e]; row += tile_m) {
        if (tiles < max_tiles) {
          meta[1 + 3 * tiles] = e;
          meta[2 + 3 * tiles] = at + row;
          meta[3 + 3 * tiles] = min(tile_m, counts[e] - row);
        }
        ++tiles;
      }
      at += counts[e];
    }
    if (tiles > max_tiles) {
      atomicOr(fault, kFaultSlot);
      tiles = max_tiles;
    }
    meta[0] = tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= experts) continue;
    const int p = atomicAdd(&cursor[e], 1);
    sorted[p] = i;
    place_of[i] = p;
  }
}

// ------------------------------------------------------------------ products over the groups, float32 FMA
// grid: (column blocks, max tiles).  A: rows of `a` (engine dtype) found by pair: by_token ? pair / top : place.
// W: [experts, n_rows_w, K] with n_rows_w = gated ? 2 N : N.  out: gated ? act[place, N] (engine dtype)
// : y[pair, N] (float32).
template <typename T, bool kGated>
__global__ void __launch_bounds__(kMoeThreads)
grouped_linear_fma_kernel(const T* a, int a_stride, const T* __restrict__ w, const int* __restrict__ sorted,
                          const int* __restrict__ meta, const float* __restrict__ pair_weight, int top, int by_token,
                          int n, int k, T* out_act, float* out_y, float glu_limit, float glu_alpha) {
  __shared__ float sa[kMoeTileM][kMoeTileK + 1];
  __shared__ float sw[kGated ? 2 : 1][kMoeTileN][kMoeTileK + 1];
  __shared__ int s_pair[kMoeTileM];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int expert = meta[1 + 3 * tile], place0 = meta[2 + 3 * tile], rows = meta[3 + 3 * tile];
  const int n0 = blockIdx.x * kMoeTileN;
  const int tid = threadIdx.x;
  if (tid < kMoeTileM) s_pair[tid] = tid < rows ? sorted[place0 + tid] : -1;
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads: 4 columns x 2 rows each
  float acc[kGated ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[g][r][c] = 0.0f;
  const size_t w_rows = kGated ? 2 * static_cast<size_t>(n) : static_cast<size_t>(n);
  const T* we = w + static_cast<size_t>(expert) * w_rows * k;
  for (int k0 = 0; k0 < k; k0 += kMoeTileK) {
    for (int idx = tid; idx < kMoeTileM * kMoeTileK; idx += kMoeThreads) {
      const int r = idx / kMoeTileK, c = idx - r * kMoeTileK;
      float v = 0.0f;
      const int pair = s_pair[r];
      if (pair >= 0 && k0 + c < k) {
        const size_t row = by_token ? static_cast<size_t>(pair / top) : static_cast<size_t>(place0 + r);
        v = to_float(a[row * a_stride + k0 + c]);
      }
      sa[r][c] = v;
    }
    for (int idx = tid; idx < kMoeTileN * kMoeTileK; idx += kMoeThreads) {
      const int r = idx / kMoeTileK, c = idx - r * kMoeTileK;
      const bool ok = n0 + r < n && k0 + c < k;
      sw[0][r][c] = ok ? to_float(we[static_cast<size_t>(n0 + r) * k + k0 + c]) : 0.0f;
      if constexpr (kGated) sw[1][r][c] = ok ? to_float(we[(static_cast<size_t>(n) + n0 + r) * k + k0 + c]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kMoeTileK; ++kk) {
      const float a0 = sa[ty * 2][kk], a1 = sa[ty * 2 + 1][kk];
#pragma unroll
      for (int g = 0; g < (kGated ? 2 : 1); ++g) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float wv = sw[g][tx * 4 + c][kk];
          acc[g][0][c] = fmaf(a0, wv, acc[g][0][c]);
          acc[g][1][c] = fmaf(a1, wv, acc[g][1][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = ty * 2 + r;
    const int pair = s_pair[row];
    if (pair < 0) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = n0 + tx * 4 + c;
      if (col >= n) continue;
      if constexpr (kGated) {
        const float scale = pair_weight ? pair_weight[pair] : 1.0f;
        const float g = acc[0][r][c] * scale, u = acc[1][r][c] * scale;
        out_act[static_cast<size_t>(place0 + row) * n + col] = from_float<T>(moe_unit(g, u, glu_limit, glu_alpha));
      } else {
        out_y[static_cast<size_t>(pair) * n + col] = acc[0][r][c];
      }
    }
  }
}

// ------------------------------------------------------------------ products over the groups, bfloat16 mma.sync
// The same tiles on the tensor cores: 8 warps, warp (wm, wn) owns rows 16 wm .. and columns 16 wn .. of the
// 32 x 64 tile (two m16n8 accumulators, twice that when gated).  Operands pass through shared memory in
// chunks of 32 of k; float32 accumulators; k runs upward in steps of 16 per row, whatever the tile holds.
__device__ __forceinline__ void moe_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kGated>
__global__ void __launch_bounds__(kMoeThreads)
grouped_linear_mma_kernel(const __nv_bfloat16* a, int a_stride, const __nv_bfloat16* __restrict__ w,
                          const int* __restrict__ sorted, const int* __restrict__ meta,
                          const float* __restrict__ pair_weight, int top, int by_token, int n, int k,
                          __nv_bfloat16* out_act, float* out_y, float glu_limit, float glu_alpha) {
  constexpr int kStride = kMoeTileK + 8;      // elements; rows stay 16-byte aligned and spread over the banks
  __shared__ __align__(16) __nv_bfloat16 sa[kMoeTileM][kStride];
  __shared__ __align__(16) __nv_bfloat16 sw[kGated ? 2 : 1][kMoeTileN][kStride];
  __shared__ int s_pair[kMoeTileM];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int expert = meta[1 + 3 * tile], place0 = meta[2 + 3 * tile], rows = meta[3 + 3 * tile];
  const int n0 = blockIdx.x * kMoeTileN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kMoeTileM) s_pair[tid] = tid < rows ? sorted[place0 + tid] : -1;
  __syncthreads();
  const int wm = warp & 1, wn = warp >> 1;      // 2 x 4 warps: 16 rows x 16 columns each
  float acc[kGated ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[g][t][c] = 0.0f;
  const size_t w_rows = kGated ? 2 * static_cast<size_t>(n) : static_cast<size_t>(n);
  const __nv_bfloat16* we = w + static_cast<size_t>(expert) * w_rows * k;
  const bool wide = (k % 8 == 0) && (a_stride % 8 == 0) && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
  for (int k0 = 0; k0 < k; k0 += kMoeTileK) {
    if (wide) {
      // 16-byte pieces: 4 per row of 32
      for (int idx = tid; idx < kMoeTileM * 4; idx += kMoeThreads) {
        const int r = idx >> 2, c = (idx & 3) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        const int pair = s_pair[r];
        if (pair >= 0 && k0 + c < k) {
          const size_t row = by_token ? static_cast<size_t>(pair / top) : static_cast<size_t>(place0 + r);
          v = *reinterpret_cast<const uint4*>(a + row * a_stride + k0 + c);
        }
        *reinterpret_cast<uint4*>(&sa[r][c]) = v;
      }
      for (int idx = tid; idx < kMoeTileN * 4; idx += kMoeThreads) {
        const int r = idx >> 2, c = (idx & 3) * 8;
        const bool ok = n0 + r < n && k0 + c < k;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ok) v = *reinterpret_cast<const uint4*>(we + static_cast<size_t>(n0 + r) * k + k0 + c);
        *reinterpret_cast<uint4*>(&sw[0][r][c]) = v;
        if constexpr (kGated) {
          uint4 u = make_uint4(0, 0, 0, 0);
          if (ok) u = *reinterpret_cast<const uint4*>(we + (static_cast<size_t>(n) + n0 + r) * k + k0 + c);
          *reinterpret_cast<uint4*>(&sw[1][r][c]) = u;
        }
      }
    } else {
      for (int idx = tid; idx < kMoeTileM * kMoeTileK; idx += kMoeThreads) {
        const int r = idx / kMoeTileK, c = idx - r * kMoeTileK;
        __nv_bfloat16 v = zero;
        const int pair = s_pair[r];
        if (pair >= 0 && k0 + c < k) {
          const size_t row = by_token ? static_cast<size_t>(pair / top) : static_cast<size_t>(place0 + r);
          v = a[row * a_stride + k0 + c];
        }
        sa[r][c] = v;
      }
      for (int idx = tid; idx < kMoeTileN * kMoeTileK; idx += kMoeThreads) {
        const int r = idx / kMoeTileK, c = idx - r * kMoeTileK;
        const bool ok = n0 + r < n && k0 + c < k;
        sw[0][r][c] = ok ? we[static_cast<size_t>(n0 + r) * k + k0 + c] : zero;
        if constexpr (kGated) sw[1][r][c] = ok ? we[(static_cast<size_t>(n) + n0 + r) * k + k0 + c] : zero;
      }
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < kMoeTileK; ks += 16) {
      // A fragment (m16 x k16, row major): a0 (row g, k 2q..), a1 (row g + 8), a2 (row g, k + 8), a3 (row g + 8, k + 8)
      const int gr = lane >> 2, q = (lane & 3) * 2;
      uint32_t af[4];
      af[0] = *reinterpret_cast<const uint32_t*>(&sa[wm * 16 + gr][ks + q]);
      af[1] = *reinterpret_cast<const uint32_t*>(&sa[wm * 16 + gr + 8][ks + q]);
      af[2] = *reinterpret_cast<const uint32_t*>(&sa[wm * 16 + gr][ks + q + 8]);
      af[3] = *reinterpret_cast<const uint32_t*>(&sa[wm * 16 + gr + 8][ks + q + 8]);
#pragma unroll
      for (int g = 0; g < (kGated ? 2 : 1); ++g) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          // B fragment (k16 x n8, "col"): b0 (k 2q.., column gr), b1 (k + 8): W rows are the columns
          const int col = wn * 16 + t * 8 + gr;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&sw[g][col][ks + q]);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&sw[g][col][ks + q + 8]);
          moe_mma_bf16(acc[g][t], af, b0, b1);
        }
      }
    }
    __syncthreads();
  }
  // C fragment: c0, c1: row gr, columns 2q, 2q + 1; c2, c3: row gr + 8
  const int gr = lane >> 2, q = (lane & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = wm * 16 + gr + 8 * half;
    const int pair = s_pair[row];
    if (pair < 0) continue;
    const float scale = (kGated && pair_weight) ? pair_weight[pair] : 1.0f;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = n0 + wn * 16 + t * 8 + q + c;
        if (col >= n) continue;
        if constexpr (kGated) {
          const float g = acc[0][t][2 * half + c] * scale, u = acc[1][t][2 * half + c] * scale;
          out_act[static_cast<size_t>(place0 + row) * n + col] = __float2bfloat16_rn(moe_unit(g, u, glu_limit, glu_alpha));
        } else {
          out_y[static_cast<size_t>(pair) * n + col] = acc[0][t][2 * half + c];
        }
      }
    }
  }
}

// ------------------------------------------------------------------ the same, pipelined (bfloat16, aligned operands)
// Tiles of 64 pairs x 64 columns (twice 64 weight rows when gated), k in chunks of 64 through a ring of three
// stages filled by cp.async (16 bytes a copy; rows of pairs beyond the tile and columns beyond k arrive as zeros),
// fragments by ldmatrix.  8 warps as 2 x 4: a warp owns 32 rows x 16 columns.  Wants k a multiple of 8 and
// 16-byte aligned operands; the host falls back to the plain tiles otherwise.
__device__ __forceinline__ void moe_cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void moe_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <bool kGated>
constexpr int moe_wide_smem_bytes() {
  return kMoeStages * (kMoeWideM + (kGated ? 2 : 1) * kMoeTileN) * (kMoeWideK + 8) * 2;
}

template <bool kGated>
__global__ void __launch_bounds__(kMoeThreads)
grouped_linear_wide_kernel(const __nv_bfloat16* a, int a_stride, const __nv_bfloat16* __restrict__ w,
                           const int* __restrict__ sorted, const int* __restrict__ meta,
                           const float* __restrict__ pair_weight, int top, int by_token, int n, int k,
                           __nv_bfloat16* out_act, float* out_y, float glu_limit, float glu_alpha) {
  constexpr int kStride = kMoeWideK + 8;
  constexpr int kWRows = (kGated ? 2 : 1) * kMoeTileN;
  constexpr int kStageElems = (kMoeWideM + kWRows) * kStride;
  extern __shared__ __align__(16) unsigned char moe_wide_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(moe_wide_smem);
  __shared__ int s_pair[kMoeWideM];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int expert = meta[1 + 3 * tile], place0 = meta[2 + 3 * tile], rows = meta[3 + 3 * tile];
  const int n0 = blockIdx.x * kMoeTileN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kMoeWideM) s_pair[tid] = tid < rows ? sorted[place0 + tid] : -1;
  __syncthreads();
  const size_t w_rows = kGated ? 2 * static_cast<size_t>(n) : static_cast<size_t>(n);
  const __nv_bfloat16* we = w + static_cast<size_t>(expert) * w_rows * k;

  // what this thread copies per stage: 2 pieces of the pairs' rows, 2 (4) pieces of the weight rows
  const __nv_bfloat16* a_src[2];
  bool a_ok[2];
  int a_dst[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = tid + i * kMoeThreads, r = idx >> 3, c = (idx & 7) * 8;
    const int pair = s_pair[r];
    a_ok[i] = pair >= 0;
    const size_t row = a_ok[i] ? (by_token ? static_cast<size_t>(pair / top) : static_cast<size_t>(place0 + r)) : 0;
    a_src[i] = a + row * a_stride + c;
    a_dst[i] = r * kStride + c;
  }
  constexpr int kWPieces = kWRows * 8 / kMoeThreads;
  const __nv_bfloat16* w_src[kWPieces];
  bool w_ok[kWPieces];
  int w_dst[kWPieces];
#pragma unroll
  for (int i = 0; i < kWPieces; ++i) {
    const int idx = tid + i * kMoeThreads, r = idx >> 3, c = (idx & 7) * 8;
    const int col = n0 + (r & (kMoeTileN - 1));
    w_ok[i] = col < n;
    const size_t row = w_ok[i] ? static_cast<size_t>(col) + (r >= kMoeTileN ? static_cast<size_t>(n) : 0) : 0;
    w_src[i] = we + row * k + c;
    w_dst[i] = (kMoeWideM + r) * kStride + c;
  }
  const int chunks = (k + kMoeWideK - 1) / kMoeWideK;
  auto fill = [&](int chunk) {
    __nv_bfloat16* stage = ring + (chunk % kMoeStages) * kStageElems;
    const int k0 = chunk * kMoeWideK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool ok = a_ok[i] && k0 + ((tid + i * kMoeThreads) & 7) * 8 < k;
      moe_cp_async16(stage + a_dst[i], ok ? a_src[i] + k0 : a, ok);
    }
#pragma unroll
    for (int i = 0; i < kWPieces; ++i) {
      const bool ok = w_ok[i] && k0 + ((tid + i * kMoeThreads) & 7) * 8 < k;
      moe_cp_async16(stage + w_dst[i], ok ? w_src[i] + k0 : w, ok);
    }
  };
#pragma unroll
  for (int s = 0; s < kMoeStages - 1; ++s) {
    if (s < chunks) fill(s);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  const int wm = warp & 1, wn = warp >> 1;      // 2 x 4 warps: 32 rows x 16 columns each
  float acc[kGated ? 2 : 1][2][2][4];
#pragma unroll
  for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][mt][nt][c] = 0.0f;
  for (int chunk = 0; chunk < chunks; ++chunk) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kMoeStages - 2));
    __syncthreads();      // the chunk has landed for every thread, and the stage about to be refilled has been read
    if (chunk + kMoeStages - 1 < chunks) fill(chunk + kMoeStages - 1);
    asm volatile("cp.async.commit_group;\n" ::);
    const __nv_bfloat16* sa = ring + (chunk % kMoeStages) * kStageElems;
    const __nv_bfloat16* sw = sa + kMoeWideM * kStride;
#pragma unroll
    for (int ks = 0; ks < kMoeWideK; ks += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        moe_ldmatrix_x4(af[mt], sa + (wm * 32 + mt * 16 + (lane & 15)) * kStride + ks + (lane >> 4) * 8);
#pragma unroll
      for (int g = 0; g < (kGated ? 2 : 1); ++g) {
        uint32_t bf[4];      // (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
        moe_ldmatrix_x4(bf, sw + (g * kMoeTileN + wn * 16 + (lane & 7) + ((lane >> 4) << 3)) * kStride + ks +
                                ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          moe_mma_bf16(acc[g][mt][0], af[mt], bf[0], bf[1]);
          moe_mma_bf16(acc[g][mt][1], af[mt], bf[2], bf[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  const int gr = lane >> 2, q = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = wm * 32 + mt * 16 + gr + 8 * half;
      const int pair = s_pair[row];
      if (pair < 0) continue;
      const float scale = (kGated && pair_weight) ? pair_weight[pair] : 1.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + wn * 16 + nt * 8 + q + c;
          if (col >= n) continue;
          if constexpr (kGated) {
            const float g = acc[0][mt][nt][2 * half + c] * scale, u = acc[1][mt][nt][2 * half + c] * scale;
            out_act[static_cast<size_t>(place0 + row) * n + col] = __float2bfloat16_rn(moe_unit(g, u, glu_limit, glu_alpha));
          } else {
            out_y[static_cast<size_t>(pair) * n + col] = acc[0][mt][nt][2 * half + c];
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ combine
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, int top, const T* shared, const float* __restrict__ gate,
                                   int gate_stride, T* __restrict__ out, int tokens, int hidden, const float* weights,
                                   const int* __restrict__ ids, int experts, const T* __restrict__ x, int x_stride) {
  pdl_trigger();
  pdl_wait();
  const long long total = static_cast<long long>(tokens) * hidden;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / hidden;
    const int c = static_cast<int>(idx - t * hidden);
    float sum = 0.0f;
    if (ids) {
      // a choice at or behind `experts` is an identity expert: its result is the token's own row, and no tile wrote y
      const float own = to_float(x[t * x_stride + c]);
      for (int j = 0; j < top; ++j) {
        const float v = ids[t * top + j] >= experts ? own : y[(t * top + j) * hidden + c];
        sum = weights ? fmaf(weights[t * top + j], v, sum) : sum + v;
      }
    } else if (weights) {
      for (int j = 0; j < top; ++j) sum = fmaf(weights[t * top + j], y[(t * top + j) * hidden + c], sum);
    } else {
      for (int j = 0; j < top; ++j) sum += y[(t * top + j) * hidden + c];
    }
    if (shared) sum += (gate ? gate[t * gate_stride] : 1.0f) * to_float(shared[idx]);
    out[idx] = from_float<T>(sum);
  }
}

// ------------------------------------------------------------------ combine, and the layer norm behind the sum
// One block per token.  s = sum_j (w_j *) y_j as in moe_combine_kernel (an identity expert's y_j is the token's own
// row), r = res_scale * stream + s, n = (r - mean r) * rsqrt(var r + eps) * ln_weight + ln_bias with the variance
// as the mean of squared deviations; the stream takes n, out its rounding.  The row waits in shared memory between
// the passes; the sums run down the block's fixed tree.
template <typename T>
__global__ void moe_combine_layernorm_kernel(const float* __restrict__ y, int top, const float* __restrict__ weights,
                                             const int* __restrict__ ids, int experts, const T* __restrict__ x,
                                             int x_stride, float* __restrict__ stream, float res_scale,
                                             const float* __restrict__ ln_weight, const float* __restrict__ ln_bias,
                                             float eps, T* __restrict__ out, int hidden) {
  extern __shared__ float combine_row[];
  __shared__ float scratch[32];
  pdl_trigger();
  const long long t = blockIdx.x;
  pdl_wait();
  float sum = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float own = ids ? to_float(x[t * x_stride + c]) : 0.0f;
    float s = 0.0f;
    for (int j = 0; j < top; ++j) {
      const float v = (ids && ids[t * top + j] >= experts) ? own : y[(t * top + j) * hidden + c];
      s = weights ? fmaf(weights[t * top + j], v, s) : s + v;
    }
    const float r = fmaf(res_scale, stream[t * hidden + c], s);
    combine_row[c] = r;
    sum += r;
  }
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float dev = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float d = combine_row[c] - mean;
    dev += d * d;
  }
  const float inv = rsqrtf(block_sum(dev, scratch) / static_cast<float>(hidden) + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float n = (combine_row[c] - mean) * inv * ln_weight[c] + (ln_bias ? ln_bias[c] : 0.0f);
    stream[t * hidden + c] = n;
    out[t * hidden + c] = from_float<T>(n);
  }
}

}  // namespace rl

extern "C" {

int rl_moe_tile_rows(int wide) { return wide ? rl::kMoeWideM : rl::kMoeTileM; }

int rl_router_topk(int dtype, const void* x, int x_stride, const float* w, int hidden, int experts, int gates, int top,
                   int* ids, float* weights, float* gate_out, float* scores_out, int tokens, const float* bias,
                   int weigh, const float* correction, int groups, int keep, int pdl, cudaStream_t stream) {
  // bias: one float per expert added to its logit, or null.  weigh 0: a chosen expert's weight is the sigmoid of its
  // logit; 1: the softmax over the chosen logits; 2: the softmax over all rows, chosen on it plus `correction` (one
  // float per row, or null) within the `keep` best of `groups` groups, the chosen scores divided by their sum.
  if (tokens == 0) return 0;
  if (experts < 1 || top < 1 || top > experts || gates < 0 || (gates > 0 && gate_out == nullptr) || hidden < 1 ||
      weigh < 0 || weigh > 2)
    return static_cast<int>(cudaErrorInvalidValue);
  if (weigh == 2 && (groups < 1 || experts % groups != 0 || keep < 1 || keep > groups || bias != nullptr ||
                     top > keep * (experts / groups)))
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t smem = static_cast<size_t>(rl::kRouterTokens) * (rl::kRouterWarps + 1) * (experts + gates) * sizeof(float);
  if (smem > 200 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  // whole rows in 16-byte pieces: which order a row's sum runs in depends on the sizes and addresses alone
  const int wide = hidden % 4 == 0 && x_stride % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  RL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(rl::router_topk_kernel<scalar_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(rl::router_topk_kernel<scalar_t>,
                             dim3((tokens + rl::kRouterTokens - 1) / rl::kRouterTokens), dim3(rl::kRouterWarps * 32),
                             smem, stream, pdl != 0, static_cast<const scalar_t*>(x), x_stride, w, hidden, experts,
                             gates, top, ids, weights, gate_out, scores_out, tokens, wide, bias, weigh, correction,
                             groups, keep);
  });
  return 0;
}

int rl_moe_plan(const int* ids, int pairs, int experts, int* sorted, int* place_of, int* meta, int max_tiles,
                int tile_m, int* fault, int pdl, cudaStream_t stream) {
  if (pairs == 0) return 0;
  const size_t smem = 2 * static_cast<size_t>(experts) * sizeof(int);
  if (experts < 1 || smem > 48 * 1024 || max_tiles < 1 || (tile_m != rl::kMoeTileM && tile_m != rl::kMoeWideM))
    return static_cast<int>(cudaErrorInvalidValue);
  return rl::launch_kernel(rl::moe_plan_kernel, dim3(1), dim3(1024), smem, stream, pdl != 0, ids, pairs, experts,
                           sorted, place_of, meta, max_tiles, tile_m, fault);
}

// a: engine dtype rows; w: [experts, (gated ? 2 n : n), k] engine dtype; gated: out_act [pairs, n] engine dtype by
// place; else out_y [pairs, n] float32 by pair.
}  // extern "C"

template <bool kGated>
static int launch_grouped_wide(dim3 grid, cudaStream_t stream, bool pdl, const __nv_bfloat16* a, int a_stride,
                               const __nv_bfloat16* w, const int* sorted, const int* meta, const float* pair_weight,
                               int top, int by_token, int n, int k, __nv_bfloat16* out_act, float* out_y,
                               float glu_limit, float glu_alpha) {
  static bool configured = false;
  auto kernel = rl::grouped_linear_wide_kernel<kGated>;
  constexpr int smem = rl::moe_wide_smem_bytes<kGated>();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return rl::launch_kernel(kernel, grid, dim3(rl::kMoeThreads), smem, stream, pdl, a, a_stride, w, sorted, meta,
                           pair_weight, top, by_token, n, k, out_act, out_y, glu_limit, glu_alpha);
}

extern "C" {

// tile_m: the rows of a tile the plan was made with; kMoeWideM selects the pipelined bfloat16 kernel.
int rl_grouped_linear(int dtype, const void* a, int a_stride, const void* w, const int* sorted, const int* meta,
                      const float* pair_weight, int top, int by_token, int n, int k, int gated, void* out_act,
                      float* out_y, int max_tiles, int tile_m, float glu_limit, float glu_alpha, int pdl,
                      cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  if (tile_m == rl::kMoeWideM) {
    using bf = __nv_bfloat16;
    if (dtype != rl::kBF16 || k % 8 != 0 || a_stride % 8 != 0 || n < 1 || max_tiles > 65535 ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
      return static_cast<int>(cudaErrorInvalidValue);
    const dim3 wide_grid((n + rl::kMoeTileN - 1) / rl::kMoeTileN, max_tiles);
    if (gated)
      return launch_grouped_wide<true>(wide_grid, stream, pdl != 0, static_cast<const bf*>(a), a_stride,
                                       static_cast<const bf*>(w), sorted, meta, pair_weight, top, by_token, n, k,
                                       static_cast<bf*>(out_act), out_y, glu_limit, glu_alpha);
    return launch_grouped_wide<false>(wide_grid, stream, pdl != 0, static_cast<const bf*>(a), a_stride,
                                      static_cast<const bf*>(w), sorted, meta, pair_weight, top, by_token, n, k,
                                      static_cast<bf*>(out_act), out_y, glu_limit, glu_alpha);
  }
  if (tile_m != rl::kMoeTileM) return static_cast<int>(cudaErrorInvalidValue);
  if (n < 1 || k < 1 || top < 1 || (gated && out_act == nullptr) || (!gated && out_y == nullptr) || max_tiles > 65535)
    return static_cast<int>(cudaErrorInvalidValue);
  const dim3 grid((n + rl::kMoeTileN - 1) / rl::kMoeTileN, max_tiles), block(rl::kMoeThreads);
  if (dtype == rl::kBF16) {
    using bf = __nv_bfloat16;
    if (gated)
      return rl::launch_kernel(rl::grouped_linear_mma_kernel<true>, grid, block, 0, stream, pdl != 0,
                               static_cast<const bf*>(a), a_stride, static_cast<const bf*>(w), sorted, meta, pair_weight,
                               top, by_token, n, k, static_cast<bf*>(out_act), out_y, glu_limit, glu_alpha);
    return rl::launch_kernel(rl::grouped_linear_mma_kernel<false>, grid, block, 0, stream, pdl != 0,
                             static_cast<const bf*>(a), a_stride, static_cast<const bf*>(w), sorted, meta, pair_weight,
                             top, by_token, n, k, static_cast<bf*>(out_act), out_y, glu_limit, glu_alpha);
  }
  if (dtype != rl::kF32) return static_cast<int>(cudaErrorInvalidValue);
  if (gated)
    return rl::launch_kernel(rl::grouped_linear_fma_kernel<float, true>, grid, block, 0, stream, pdl != 0,
                             static_cast<const float*>(a), a_stride, static_cast<const float*>(w), sorted, meta,
                             pair_weight, top, by_token, n, k, static_cast<float*>(out_act), out_y, glu_limit, glu_alpha);
  return rl::launch_kernel(rl::grouped_linear_fma_kernel<float, false>, grid, block, 0, stream, pdl != 0,
                           static_cast<const float*>(a), a_stride, static_cast<const float*>(w), sorted, meta,
                           pair_weight, top, by_token, n, k, static_cast<float*>(out_act), out_y, glu_limit, glu_alpha);
}

// weights: one float per (token, choice) that multiplies the choice's row in the sum, or null.  ids (with x, the
// experts' input rows): a choice whose id is `experts` or more is an identity expert and contributes x's row.
int rl_moe_combine(int dtype, const float* y, int top, const void* shared, const float* gate, int gate_stride,
                   void* out, int tokens, int hidden, const float* weights, const int* ids, int experts, const void* x,
                   int x_stride, int pdl, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (ids != nullptr && x == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const long long total = static_cast<long long>(tokens) * hidden;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  RL_DISPATCH_DTYPE(dtype, {
    return rl::launch_kernel(rl::moe_combine_kernel<scalar_t>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream,
                             pdl != 0, y, top, static_cast<const scalar_t*>(shared), gate, gate_stride,
                             static_cast<scalar_t*>(out), tokens, hidden, weights, ids, experts,
                             static_cast<const scalar_t*>(x), x_stride);
  });
  return 0;
}

// The sum over a token's choices and the layer norm that closes it: stream (float32, [tokens, hidden]) is read and
// replaced, out is its rounding.  ids with x as for rl_moe_combine.
int rl_moe_combine_layernorm(int dtype, const float* y, int top, const float* weights, const int* ids, int experts,
                             const void* x, int x_stride, float* stream, float res_scale, const float* ln_weight,
                             const float* ln_bias, float eps, void* out, int tokens, int hidden, int pdl,
                             cudaStream_t stream_handle) {
  if (tokens == 0) return 0;
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (hidden < 1 || top < 1 || stream == nullptr || ln_weight == nullptr || (ids != nullptr && x == nullptr) ||
      smem > 200 * 1024)
    return static_cast<int>(cudaErrorInvalidValue);
  int threads = 128;
  while (threads < 1024 && threads * 4 < hidden) threads *= 2;
  RL_DISPATCH_DTYPE(dtype, {
    auto kernel = rl::moe_combine_layernorm_kernel<scalar_t>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    return rl::launch_kernel(kernel, dim3(tokens), dim3(threads), smem, stream_handle, pdl != 0, y, top, weights, ids,
                             experts, static_cast<const scalar_t*>(x), x_stride, stream, res_scale, ln_weight, ln_bias,
                             eps, static_cast<scalar_t*>(out), hidden);
  });
  return 0;
}

}  // extern "C"
