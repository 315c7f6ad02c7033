// Routed feed-forward (mixture of experts) on CUDA cores: router, grouping of the step's (token, choice)
// pairs by expert, per-expert products, and the weighted sum. Everything has fixed shapes given the
// number of tokens, so a step can be recorded as a CUDA graph.
//
//   route     z = Wr x + b in float32; the `top` largest logits (the lower index wins a tie); their weights
//             are the softmax over the chosen logits only
//   group     pairs (token * top + choice) sorted by expert into tiles of `tile` rows; a tile holds rows of
//             one expert (the last tile of an expert is padded with -1); tile_expert[i] = -1 for unused tiles
//   product   for every tile: rows of a (picked by pair / a_div) times the expert's matrix; the result row
//             is written at the pair's index, so no inverse permutation is needed. Epilogue: the exact
//             (erf) gelu, or the pair's weight
//   combine   out[t] = sum over the token's choices, in index order
#include "common.cuh"

#include <cfloat>
#include <cmath>

namespace {

template <typename T>
__global__ void route_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ wr, const float* __restrict__ bias,
                             int D, int E, int top, int* __restrict__ idx, float* __restrict__ share) {
  extern __shared__ float z[];  // E
  dep_launch();
  dep_wait();
  const int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T* xr = x + (size_t)tok * ldx;
  const bool vec = D % 8 == 0 && sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0 && (reinterpret_cast<uintptr_t>(wr) & 15u) == 0;
  for (int e = warp; e < E; e += nw) {
    const T* w = wr + (size_t)e * D;
    float acc = 0.f;
    if (vec) {  // bfloat16 rows, 16 bytes a lane a step
      for (int k = lane * 8; k < D; k += 256) {
        const uint4 xa = *reinterpret_cast<const uint4*>(xr + k), wa = *reinterpret_cast<const uint4*>(w + k);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xa);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wa);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __bfloat1622float2(xh[i]), wf = __bfloat1622float2(wh[i]);
          acc = fmaf(xf.x, wf.x, acc);
          acc = fmaf(xf.y, wf.y, acc);
        }
      }
    } else {
      for (int k = lane; k < D; k += 32) acc = fmaf(to_f32(xr[k]), to_f32(w[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  // warp 0 picks the largest `top` times; lanes scan strided, ties go to the lower index
  float zmax = 0.f, denom = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (k == 0) zmax = best;
    const float p = expf(best - zmax);
    denom += p;
    if (lane == 0) {
      idx[(size_t)tok * top + k] = bi;
      share[(size_t)tok * top + k] = p;
      z[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top) share[(size_t)tok * top + lane] /= denom;
}

// The router with scores over ALL experts and a limit on groups of experts:
//   s = softmax(z) over the E experts;  choice = s + correction;  experts form n_groups equal groups of neighbours, a group's
//   score is its largest choice score, and only experts of the `keep` best groups can be chosen (the others count as minus
//   infinity); the `top` largest choice scores win (the lower index wins a tie); their weights are s (without the correction)
//   divided by (their sum + norm_eps).
template <typename T>
__global__ void route_grouped_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ wr, const float* __restrict__ correction,
                                     int D, int E, int top, int n_groups, int keep, float norm_eps, int* __restrict__ idx,
                                     float* __restrict__ share, int score_mode, int group_top, int normalize, float weight_scale,
                                     float* __restrict__ gate_out) {
  extern __shared__ float sh_r[];  // s[E + 1], choice[E], group score[n_groups]
  float* s = sh_r;
  float* choice = sh_r + E + 1;
  float* gscore = sh_r + 2 * E + 1;
  dep_launch();
  dep_wait();
  const int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T* xr = x + (size_t)tok * ldx;
  const bool vec = D % 8 == 0 && sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0 && (reinterpret_cast<uintptr_t>(wr) & 15u) == 0;
  const int n_rows = E + (gate_out ? 1 : 0);  // with gate_out, one more row behind the router's: a gate's logit, no expert
  for (int e = warp; e < n_rows; e += nw) {
    const T* w = wr + (size_t)e * D;
    float acc = 0.f;
    if (vec) {  // bfloat16 rows, 16 bytes a lane a step
      for (int k = lane * 8; k < D; k += 256) {
        const uint4 xa = *reinterpret_cast<const uint4*>(xr + k), wa = *reinterpret_cast<const uint4*>(w + k);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xa);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wa);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __bfloat1622float2(xh[i]), wf = __bfloat1622float2(wh[i]);
          acc = fmaf(xf.x, wf.x, acc);
          acc = fmaf(xf.y, wf.y, acc);
        }
      }
    } else {
      for (int k = lane; k < D; k += 32) acc = fmaf(to_f32(xr[k]), to_f32(w[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) s[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  if (gate_out && lane == 0) gate_out[tok] = 1.0f / (1.0f + expf(-s[E]));
  if (score_mode == 1) {  // every expert's score by itself: sigmoid of its logit
    for (int e = lane; e < E; e += 32) {
      const float p = 1.0f / (1.0f + expf(-s[e]));
      s[e] = p;
      choice[e] = p + (correction ? correction[e] : 0.f);
    }
  } else {
    float zmax = -INFINITY;
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, s[e]);
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(s[e] - zmax);
      s[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
      const float p = s[e] / sum;
      s[e] = p;
      choice[e] = p + (correction ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  const int per = E / n_groups;
  if (keep < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      // the group's largest choice score, or (group_top 2) the sum of its two largest
      float best = -INFINITY, second = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = choice[e];
        if (v > best) { second = best; best = v; }
        else if (v > second) second = v;
      }
      gscore[g] = (group_top >= 2 && per >= 2) ? best + second : best;
    }
    __syncwarp();
    // a group stays if fewer than `keep` groups come before it (larger score, or the same score and a lower index)
    for (int g = lane; g < n_groups; g += 32) {
      const float mine = gscore[g];
      int before = 0;
      for (int o = 0; o < n_groups; ++o) before += (gscore[o] > mine || (gscore[o] == mine && o < g)) ? 1 : 0;
      if (before >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;  // fewer candidates than `top` (refused on the host; never read out of range)
    const float p = s[bi];
    total += p;
    if (lane == 0) {
      idx[(size_t)tok * top + k] = bi;
      share[(size_t)tok * top + k] = p;
      choice[bi] = -INFINITY;
    }
    __syncwarp();
  }
  __syncwarp();
  if (lane < top) {
    float p = share[(size_t)tok * top + lane];
    if (normalize) p /= (total + norm_eps);
    share[(size_t)tok * top + lane] = p * weight_scale;  // a scale of 1 changes nothing
  }
}

// One block. counts -> tiles per expert -> scatter. The order of an expert's rows depends on timing;
// every row's result is computed on its own, so nothing depends on that order.
// Experts from `real` on have no matrices (their pairs are dealt with where the results are added): they get no tiles.
__global__ void group_kernel(const int* __restrict__ idx, int n_pairs, int E, int real, int tile, int max_tiles, int* __restrict__ tile_expert,
                             int* __restrict__ tile_rows) {
  extern __shared__ int sh[];  // counts[E], start[E] (in rows, tile-aligned), cursor[E]
  int* counts = sh;
  int* start = sh + E;
  int* cursor = sh + 2 * E;
  dep_launch();
  dep_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) tile_rows[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = e < real ? at * tile : -1;
      const int nt = e < real ? (counts[e] + tile - 1) / tile : 0;
      for (int k = 0; k < nt; ++k) tile_expert[at + k] = e;
      at += nt;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = idx[i];
    if (start[e] >= 0) tile_rows[start[e] + atomicAdd(&cursor[e], 1)] = i;
  }
}

constexpr int RP_WARPS = 4, RP_ROWS = 8;  // rows of a tile of the CUDA-core product

// epilogue 0: exact gelu; 1: times share[pair]; 2: w holds 2 N rows, row 2 n a gate and row 2 n + 1 its up row:
// out[p, n] = gated_value(gate, up) with the activation (act, p0, p1) of common.cuh: silu(gate) * up, or both sides limited
template <typename TA, typename TO>
__global__ void __launch_bounds__(RP_WARPS * 32)
    routed_product_kernel(const TA* __restrict__ a, long long lda, int a_div, const TA* __restrict__ w, long long w_stride, int N, int K,
                          const int* __restrict__ tile_expert, const int* __restrict__ tile_rows, TO* __restrict__ out, long long ldo,
                          int epilogue, const float* __restrict__ share, int act, float p0, float p1) {
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = tile_expert[blockIdx.y];
  const int n = blockIdx.x * RP_WARPS + warp;
  if (e < 0 || n >= N) return;
  const int* rows = tile_rows + (size_t)blockIdx.y * RP_ROWS;
  int pair[RP_ROWS];
  const TA* ar[RP_ROWS];
#pragma unroll
  for (int i = 0; i < RP_ROWS; ++i) {
    pair[i] = rows[i];
    ar[i] = pair[i] >= 0 ? a + (size_t)(pair[i] / a_div) * lda : nullptr;
  }
  const TA* wrow = w + (size_t)e * w_stride + (size_t)(epilogue == 2 ? 2 * n : n) * K;
  float acc[RP_ROWS], acc2[RP_ROWS];
#pragma unroll
  for (int i = 0; i < RP_ROWS; ++i) acc[i] = acc2[i] = 0.f;
  if (epilogue == 2) {
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f32(wrow[k]), wu = to_f32(wrow[K + k]);
#pragma unroll
      for (int i = 0; i < RP_ROWS; ++i)
        if (ar[i]) {
          const float av = to_f32(ar[i][k]);
          acc[i] = fmaf(av, wv, acc[i]);
          acc2[i] = fmaf(av, wu, acc2[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < RP_ROWS; ++i) {
      const float g = warp_sum(acc[i]), u = warp_sum(acc2[i]);
      acc[i] = gated_value(g, u, act, p0, p1);
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f32(wrow[k]);
#pragma unroll
      for (int i = 0; i < RP_ROWS; ++i)
        if (ar[i]) acc[i] = fmaf(to_f32(ar[i][k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < RP_ROWS; ++i) acc[i] = warp_sum(acc[i]);
  }
  if (lane < RP_ROWS) {
    float v = 0.f;
    int p = -1;
#pragma unroll
    for (int i = 0; i < RP_ROWS; ++i)
      if (i == lane) { v = acc[i]; p = pair[i]; }
    if (p >= 0) {
      if (epilogue == 0) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
      else if (epilogue == 1) v *= share[p];
      out[(size_t)p * ldo + n] = from_f32<TO>(v);
    }
  }
}

// idx (with x, share, real): a choice of an expert from `real` on is an identity expert, whose result is the token's own
// input row times the choice's weight. b (with gate): float32 partial sums of an expert that every token uses, added after
// the chosen ones, times gate[token].
template <typename T>
__global__ void combine_kernel(const float* __restrict__ y, float* __restrict__ out, int top, int D, size_t total, const int* __restrict__ idx,
                               const float* __restrict__ share, int real, const T* __restrict__ x, long long ldx, const float* __restrict__ b,
                               int nb, size_t sb, const float* __restrict__ gate) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / D;
  const int c = (int)(i - t * D);
  float s = 0.f;
  for (int k = 0; k < top; ++k) {
    if (idx && idx[t * top + k] >= real) s += share[t * top + k] * to_f32(x[t * ldx + c]);
    else s += y[(t * top + k) * D + c];
  }
  if (b) {
    float v = b[i];
    for (int p = 1; p < nb; ++p) v += b[(size_t)p * sb + i];
    s += gate ? gate[t] * v : v;
  }
  out[i] = s;
}

}  // namespace

extern "C" int llm_route(const void* x, long long ldx, const void* wr, const float* bias, int n_tokens, int D, int E, int top,
                         int* idx, float* share, int dtype, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && top > 0 && top <= E, "route: bad sizes experts=%d top=%d", E, top);
  LLM_REQUIRE(top <= 32 && E <= 8192, "route: at most 32 of 8192 experts a token (got %d of %d)", top, E);
  const size_t smem = (size_t)E * sizeof(float);
  if (dtype == LLM_F32)
    launch_kernel(route_kernel<float>, n_tokens, 256, smem, stream, (const float*)x, ldx, (const float*)wr, bias, D, E, top, idx, share);
  else if (dtype == LLM_BF16)
    launch_kernel(route_kernel<bf16>, n_tokens, 256, smem, stream, (const bf16*)x, ldx, (const bf16*)wr, bias, D, E, top, idx, share);
  else
    LLM_REQUIRE(false, "route: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("route");
  return LLM_OK;
}

extern "C" int llm_route_grouped(const void* x, long long ldx, const void* wr, const float* correction, int n_tokens, int D, int E, int top,
                                 int n_groups, int keep, float norm_eps, int* idx, float* share, int dtype, int score_mode, int group_top, int normalize,
                                 float weight_scale, float* gate_out, cudaStream_t stream) {
  // weight_scale: the weights are multiplied by it at the end. gate_out (optional, float32 [tokens]): wr holds one more row behind the
  // E router rows, and gate_out[t] = sigmoid(that row . x[t]), formed in float32 like the router's logits
  // score_mode 0: softmax over all experts, 1: sigmoid of each logit; group_top: a group's score is its largest choice score (1) or
  // the sum of its two largest (2); normalize 0: the chosen experts' scores are the weights as they are
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE((score_mode == 0 || score_mode == 1) && (group_top == 1 || group_top == 2), "route: unknown score mode %d or group score over %d", score_mode, group_top);
  LLM_REQUIRE(n_tokens > 0 && D > 0 && E > 0 && top > 0 && top <= E, "route: bad sizes experts=%d top=%d", E, top);
  LLM_REQUIRE(top <= 32 && E <= 4096, "route: at most 32 of 4096 experts a token (got %d of %d)", top, E);
  LLM_REQUIRE(n_groups >= 1 && keep >= 1 && keep <= n_groups && E % n_groups == 0, "route: %d experts do not form %d equal groups of which %d stay", E, n_groups, keep);
  LLM_REQUIRE((long long)keep * (E / n_groups) >= top, "route: %d groups of %d experts cannot give %d choices", keep, E / n_groups, top);
  const size_t smem = (size_t)(2 * E + 1 + n_groups) * sizeof(float);
  if (dtype == LLM_F32)
    launch_kernel(route_grouped_kernel<float>, n_tokens, 256, smem, stream, (const float*)x, ldx, (const float*)wr, correction, D, E, top, n_groups,
                  keep, norm_eps, idx, share, score_mode, group_top, normalize, weight_scale, gate_out);
  else if (dtype == LLM_BF16)
    launch_kernel(route_grouped_kernel<bf16>, n_tokens, 256, smem, stream, (const bf16*)x, ldx, (const bf16*)wr, correction, D, E, top, n_groups,
                  keep, norm_eps, idx, share, score_mode, group_top, normalize, weight_scale, gate_out);
  else
    LLM_REQUIRE(false, "route: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("route_grouped");
  return LLM_OK;
}

extern "C" int llm_routed_tiles(int n_pairs, int E, int tile) { return (n_pairs + tile - 1) / tile + E; }

extern "C" int llm_routed_group(const int* idx, int n_pairs, int E, int tile, int max_tiles, int* tile_expert, int* tile_rows,
                                int real_experts, cudaStream_t stream) {
  // real_experts: idx may name experts real_experts .. E - 1 that have no matrices; their pairs enter no tile
  if (n_pairs == 0) return LLM_OK;
  LLM_REQUIRE(n_pairs > 0 && E > 0 && tile > 0 && E <= 4096 && real_experts >= 0 && real_experts <= E, "routed_group: bad sizes");
  LLM_REQUIRE(max_tiles >= llm_routed_tiles(n_pairs, E, tile), "routed_group: room for %d tiles, %d may be needed", max_tiles,
              llm_routed_tiles(n_pairs, E, tile));
  launch_kernel(group_kernel, 1, 1024, (size_t)3 * E * sizeof(int), stream, idx, n_pairs, E, real_experts, tile, max_tiles, tile_expert, tile_rows);
  LLM_CHECK_LAUNCH("routed_group");
  return LLM_OK;
}

// a: rows picked by pair / a_div; w [E, N, K]; out rows at the pair's index. in_dtype: a and w; out_dtype: out.
extern "C" int llm_routed_product(const void* a, long long lda, int a_div, const void* w, int N, int K, const int* tile_expert,
                                  const int* tile_rows, int max_tiles, void* out, long long ldo, int epilogue, const float* share,
                                  int in_dtype, int out_dtype, int act, float p0, float p1, cudaStream_t stream) {
  // act, p0, p1: the activation of epilogue 2 (0: silu; 2: both sides limited by p0, slope p1)
  if (max_tiles == 0) return LLM_OK;
  LLM_REQUIRE(N > 0 && K > 0 && a_div > 0 && max_tiles > 0 && max_tiles <= 65535, "routed_product: bad sizes");
  LLM_REQUIRE(epilogue == 0 || (epilogue == 1 && share) || (epilogue == 2 && N % 2 == 0), "routed_product: unknown epilogue %d", epilogue);
  LLM_REQUIRE(act >= 0 && act <= 2, "routed_product: unknown activation %d", act);
  const long long ws = (long long)N * K;
  if (epilogue == 2) N /= 2;  // outputs: one for every (gate, up) pair of rows
  dim3 grid(ceil_div(N, RP_WARPS), max_tiles);
#define LLM_RP(TA, TO)                                                                                                         \
  launch_kernel(routed_product_kernel<TA, TO>, grid, RP_WARPS * 32, 0, stream, (const TA*)a, lda, a_div, (const TA*)w, ws, N, K, \
                tile_expert, tile_rows, (TO*)out, ldo, epilogue, share, act, p0, p1)
  if (in_dtype == LLM_F32 && out_dtype == LLM_F32) LLM_RP(float, float);
  else if (in_dtype == LLM_BF16 && out_dtype == LLM_BF16) LLM_RP(bf16, bf16);
  else if (in_dtype == LLM_BF16 && out_dtype == LLM_F32) LLM_RP(bf16, float);
  else LLM_REQUIRE(false, "routed_product: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LLM_RP
  LLM_CHECK_LAUNCH("routed_product");
  return LLM_OK;
}

extern "C" int llm_routed_product_rows() { return RP_ROWS; }

extern "C" int llm_routed_combine(const float* y, float* out, int n_tokens, int top, int D, const int* idx, const float* share, int real_experts,
                                  const void* x, long long ldx, int x_dtype, const float* b, int nb, long long sb, const float* gate,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && top > 0 && D > 0, "routed_combine: bad sizes");
  LLM_REQUIRE(idx == nullptr || (share && x), "routed_combine: identity experts need the weights and the input rows");
  LLM_REQUIRE(b == nullptr || nb >= 1, "routed_combine: bad partial sums");
  const size_t total = (size_t)n_tokens * D;
  if (x_dtype == LLM_BF16)
    launch_kernel(combine_kernel<bf16>, ceil_div((long long)total, 256), 256, 0, stream, y, out, top, D, total, idx, share, real_experts,
                  (const bf16*)x, ldx, b, nb, (size_t)sb, gate);
  else
    launch_kernel(combine_kernel<float>, ceil_div((long long)total, 256), 256, 0, stream, y, out, top, D, total, idx, share, real_experts,
                  (const float*)x, ldx, b, nb, (size_t)sb, gate);
  LLM_CHECK_LAUNCH("routed_combine");
  return LLM_OK;
}
