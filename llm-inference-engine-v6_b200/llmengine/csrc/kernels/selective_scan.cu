// A recurrent mixer with input-dependent decay ("selective scan") over the step's flat ragged batch, float32 arithmetic.
// Per request the state lives in its slot: the last K - 1 inputs of the causal convolution [slots, K - 1, C] and the
// recurrent state [slots, C, N], both float32, zero when the request starts.
//
//   conv        xc[t, c] = silu(bias[c] + sum_j w[c, j] * x[t - (K - 1) + j, c]); inputs before the step's portion come
//               from the slot, inputs before the sequence are zero (the slot starts at zero)
//   conv_state  afterwards the slot holds the last K - 1 inputs again
//   dt          dt[t, c] = softplus(bias[c] + sum_r Wdt[c, r] * low[t, r])
//   scan        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = y * silu(z)
//               with A = -exp(A_log); token after token of a request, the request's state read from and written to its slot
//
// x and z are columns of a product given as float32 partial sums [parts, tokens, width] (added in index order); low, B and C
// are columns of a float32 product [tokens, ld]. A token's result depends on the tokens before it in its request alone.
#include "common.cuh"

#include <cmath>

namespace {

__device__ __forceinline__ float parts_sum(const float* __restrict__ p, int n_parts, size_t pstride, size_t i) {
  float s = p[i];
  for (int k = 1; k < n_parts; ++k) s += p[(size_t)k * pstride + i];
  return s;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// exp(x) - 1 for x <= 0 (a decay's distance from 1): close to 0 by its series (the next term is below x^7 / 5040, under a
// float's rounding for |x| < 1/8), elsewhere from expf, whose error is then small beside 1 - exp(x) >= 0.117 and meets a state
// that is forgotten within a few tokens. A quarter of the instructions of expm1f, which the scan spends most of its time in.
__device__ __forceinline__ float decay_minus_one(float x) {
  if (x > -0.125f) {
    float p = fmaf(x, 1.0f / 720.0f, 1.0f / 120.0f);
    p = fmaf(x, p, 1.0f / 24.0f);
    p = fmaf(x, p, 1.0f / 6.0f);
    p = fmaf(x, p, 0.5f);
    p = fmaf(x, p, 1.0f);
    return x * p;
  }
  return expf(x) - 1.0f;
}

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void conv_silu_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int x_off, int C, int K,
                                 const T* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ conv_state,
                                 const int* __restrict__ token_seq, const int* __restrict__ seq_qoff, const int* __restrict__ seq_slot,
                                 T* __restrict__ out, int n_tokens) {
  dep_launch();
  dep_wait();
  // a block: one token (or, beyond the grid's height, every gridDim.y-th), 256 channels; no division on the way to an index
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  for (int tok = blockIdx.y; tok < n_tokens; tok += gridDim.y) {
    const size_t i = (size_t)tok * C + c;
    const int seq = token_seq[tok];
    const int first = seq_qoff[seq];
    const float* st = conv_state + (size_t)seq_slot[seq] * (K - 1) * C;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < K; ++j) {
      const int src = tok - (K - 1) + j;  // flat row of the tap's input, if it is part of this step
      float v;
      if (src >= first) v = parts_sum(parts, n_parts, pstride, (size_t)src * width + x_off + c);
      else v = st[(size_t)((K - 1) + (src - first)) * C + c];  // src - first in [-(K-1), -1]
      acc = fmaf(to_f32(w[(size_t)c * K + j]), v, acc);
    }
    out[i] = from_f32<T>(silu_f(acc));
  }
}

__global__ void conv_state_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int x_off, int C, int K,
                                  float* __restrict__ conv_state, const int* __restrict__ seq_qoff, const int* __restrict__ seq_ntok,
                                  const int* __restrict__ seq_slot, int n_seqs) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_seqs * C) return;
  const int seq = (int)(i / C), c = (int)(i - (size_t)seq * C);
  const int first = seq_qoff[seq], n = seq_ntok[seq];
  float* st = conv_state + (size_t)seq_slot[seq] * (K - 1) * C;
  float keep[MAX_TAPS];
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k < K - 1) {
      const int rel = n - (K - 1) + k;  // which of the step's tokens, or (negative) how far back in the old state
      keep[k] = rel >= 0 ? parts_sum(parts, n_parts, pstride, (size_t)(first + rel) * width + x_off + c) : st[(size_t)(k + n) * C + c];
    }
  }
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k)
    if (k < K - 1) st[(size_t)k * C + c] = keep[k];
}

constexpr int DT_THREADS = 128;

// The low-rank map's two ends. in_act 1: tanh of the low-rank numbers before the map. out_act 0: softplus(z) (a step size);
// 1: sigmoid(z)^(1/p) = exp(-softplus(-z) / p) (a decay in (0, 1), p its temperature); 2: exp(-exp(z)) (a decay in (0, 1)).
__device__ __forceinline__ float low_in(float v, int in_act) { return in_act == 1 ? tanhf(v) : v; }
__device__ __forceinline__ float low_out(float z, int out_act, float p) {
  if (out_act == 1) return expf(-(z < -20.0f ? -z : log1pf(expf(-z))) / p);
  if (out_act == 2) return expf(-expf(z));
  return z > 20.0f ? z : log1pf(expf(z));
}

// wt: the step-size map stored [R, C] (transposed when loaded), so that neighbouring channels read neighbouring words.
// A block: 128 channels x TOK tokens; the tokens' low-rank rows lie in shared memory as [R][TOK], so that one 16-byte read
// feeds four multiply-adds.
template <typename T, int TOK>
__global__ void __launch_bounds__(DT_THREADS)
    dt_softplus_kernel(const float* __restrict__ proj, long long ld, int R, const T* __restrict__ wt, const float* __restrict__ bias, int C,
                       float* __restrict__ dt, int n_tokens, int in_act, int out_act, float param) {
  extern __shared__ __align__(16) float low[];  // [R][TOK]
  dep_launch();
  dep_wait();
  const int t0 = blockIdx.y * TOK;
  for (int i = threadIdx.x; i < TOK * R; i += blockDim.x) {
    const int tl = i / R, r = i - tl * R;
    low[r * TOK + tl] = t0 + tl < n_tokens ? low_in(proj[(size_t)(t0 + tl) * ld + r], in_act) : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float acc[TOK];
#pragma unroll
  for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int r = 0; r < R; ++r) {
    const float wv = to_f32(wt[(size_t)r * C + c]);
    const float4* row = reinterpret_cast<const float4*>(low + r * TOK);
#pragma unroll
    for (int i = 0; i < TOK / 4; ++i) {
      const float4 v = row[i];
      acc[4 * i] = fmaf(wv, v.x, acc[4 * i]);
      acc[4 * i + 1] = fmaf(wv, v.y, acc[4 * i + 1]);
      acc[4 * i + 2] = fmaf(wv, v.z, acc[4 * i + 2]);
      acc[4 * i + 3] = fmaf(wv, v.w, acc[4 * i + 3]);
    }
  }
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int i = 0; i < TOK; ++i) {
    const int t = t0 + i;
    if (t < n_tokens) {
      dt[(size_t)t * C + c] = low_out(acc[i] + b, out_act, param);
    }
  }
}

// The same map for steps of up to 8 tokens, where there is nothing but latency to hide: a block has 32 channels, its four warps
// take a quarter of the rank each (so four times as many weight loads are on their way) and warp 0 adds the quarters in index order.
template <typename T>
__global__ void __launch_bounds__(128)
    dt_softplus_few_kernel(const float* __restrict__ proj, long long ld, int R, const T* __restrict__ wt, const float* __restrict__ bias, int C,
                           float* __restrict__ dt, int n_tokens, int in_act, int out_act, float param) {
  extern __shared__ __align__(16) float sm_few[];  // low [R][8], then quarters [4][32][8]
  float* low = sm_few;
  float* quarter = sm_few + (size_t)R * 8;
  dep_launch();
  dep_wait();
  const int t0 = blockIdx.y * 8;
#pragma unroll 4
  for (int i = threadIdx.x; i < 8 * R; i += 128) {
    const int tl = i / R, r = i - tl * R;
    low[r * 8 + tl] = t0 + tl < n_tokens ? low_in(proj[(size_t)(t0 + tl) * ld + r], in_act) : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int c = min(blockIdx.x * 32 + lane, C - 1);
  const int per = (R + 3) / 4, r_end = min(R, (part + 1) * per);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 8
  for (int r = part * per; r < r_end; ++r) {
    const float wv = to_f32(wt[(size_t)r * C + c]);
    const float4 v0 = *reinterpret_cast<const float4*>(low + r * 8), v1 = *reinterpret_cast<const float4*>(low + r * 8 + 4);
    acc[0] = fmaf(wv, v0.x, acc[0]); acc[1] = fmaf(wv, v0.y, acc[1]); acc[2] = fmaf(wv, v0.z, acc[2]); acc[3] = fmaf(wv, v0.w, acc[3]);
    acc[4] = fmaf(wv, v1.x, acc[4]); acc[5] = fmaf(wv, v1.y, acc[5]); acc[6] = fmaf(wv, v1.z, acc[6]); acc[7] = fmaf(wv, v1.w, acc[7]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) quarter[(part * 32 + lane) * 8 + i] = acc[i];
  __syncthreads();
  if (part != 0 || blockIdx.x * 32 + lane >= C) return;
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = t0 + i;
    if (t < n_tokens) {
      const float z = ((quarter[lane * 8 + i] + quarter[(32 + lane) * 8 + i]) + quarter[(64 + lane) * 8 + i]) + quarter[(96 + lane) * 8 + i] + b;
      dt[(size_t)t * C + c] = low_out(z, out_act, param);
    }
  }
}

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_CHUNK = 64;  // tokens of a piece when a long portion is cut into pieces that run side by side

// How many pieces the requests before `seq` have (every request's portion is cut on its own).
__device__ __forceinline__ int pieces_before(const int* __restrict__ seq_ntok, int seq, int piece) {
  int n = 0;
  for (int s = 0; s < seq; ++s) n += (seq_ntok[s] + piece - 1) / piece;
  return n;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// TPC threads share a channel, each with NS of its N state numbers (n = part * NS + i). A block walks tokens of one request:
// MODE 0  the whole portion, from the request's slot and back into it;
// MODE 1  piece blockIdx.y of the portion, from a state of zero: leaves the piece's end state and the sum of its step sizes
//         (the decay over the piece is exp(A * that sum)), no outputs;
// MODE 2  the same piece again, from the state that the carry kernel has put at the piece's start: writes the outputs.
// FAST (the bfloat16 engine): the decay is one ex2.approx of dt * (A log2 e), float32 with a relative error of 2^-22 like expf's;
// otherwise (the 32-bit engine) exp(dA) - 1 is formed without the rounding of a decay near 1 (decay_minus_one).
template <typename T, int NS, int MODE, bool FAST>
__global__ void __launch_bounds__(SCAN_THREADS)
    selective_scan_kernel(const T* __restrict__ xc, const float* __restrict__ dt, const float* __restrict__ proj, long long ld, int b_off,
                          int c_off, const float* __restrict__ zparts, int n_parts, size_t pstride, int zwidth, int z_off,
                          const float* __restrict__ a_log, const float* __restrict__ dskip, float* __restrict__ state,
                          const int* __restrict__ seq_qoff, const int* __restrict__ seq_ntok, const int* __restrict__ seq_slot, int C, int N,
                          int tpc, T* __restrict__ out, float* __restrict__ piece_state, float* __restrict__ piece_sumdt,
                          const float* __restrict__ dt_bias, int dt_raw) {
  dep_launch();
  dep_wait();
  const int seq = blockIdx.z;
  int first = seq_qoff[seq], n_tok = seq_ntok[seq];
  size_t piece = 0;
  if (MODE != 0) {
    first += blockIdx.y * SCAN_CHUNK;
    n_tok = min(SCAN_CHUNK, n_tok - (int)blockIdx.y * SCAN_CHUNK);
    if (n_tok <= 0) return;
    piece = (size_t)pieces_before(seq_ntok, seq, SCAN_CHUNK) + blockIdx.y;
  }
  const int per_block = SCAN_THREADS / tpc;
  const int c = blockIdx.x * per_block + threadIdx.x / tpc;
  const int part = threadIdx.x % tpc;
  const bool live = c < C;
  const int cc = live ? c : C - 1;  // threads past the last channel compute along (the shuffles need them) and write nothing
  float* st = MODE == 0 ? state + ((size_t)seq_slot[seq] * C + cc) * N : piece_state + (piece * C + cc) * N;
  const int n0 = part * NS;
  float S[NS], A[NS];
#pragma unroll
  for (int i = 0; i < NS; ++i) {
    const int n = n0 + i;
    S[i] = (n < N && MODE != 1) ? st[n] : 0.f;
    A[i] = n < N ? -expf(a_log[(size_t)cc * N + n]) * (FAST ? 1.4426950408889634f : 1.0f) : 0.f;
  }
  const float dsk = dskip ? dskip[cc] : 0.f;
  // the token's B and C rows by 16-byte reads where this thread's numbers are whole, aligned groups of four
  const bool vec = NS % 4 == 0 && n0 + NS <= N && ((b_off + n0) % 4) == 0 && ((c_off + n0) % 4) == 0 && (ld % 4) == 0 &&
                   (reinterpret_cast<uintptr_t>(proj) & 15u) == 0;
  float sum_dt = 0.f;
  const float dtb = (dt_raw && dt_bias) ? dt_bias[cc] : 0.f;
  // a token's inputs: loaded one token ahead, so that their way from memory lies behind the arithmetic of the token before
  float n_d = 0.f, n_x = 0.f, n_z = 0.f, n_bv[NS], n_cv[NS];
  auto fetch = [&](int j) {
    const size_t t = (size_t)(first + j);
    n_d = dt[t * C + cc];
    n_x = to_f32(xc[t * C + cc]);
    if (MODE != 1) n_z = parts_sum(zparts, n_parts, pstride, t * zwidth + z_off + cc);
    const float* pr = proj + t * ld;
    if (vec) {
#pragma unroll
      for (int i = 0; i < NS / 4; ++i) {
        const float4 b4 = *reinterpret_cast<const float4*>(pr + b_off + n0 + 4 * i);
        n_bv[4 * i] = b4.x; n_bv[4 * i + 1] = b4.y; n_bv[4 * i + 2] = b4.z; n_bv[4 * i + 3] = b4.w;
        if (MODE != 1) {
          const float4 c4 = *reinterpret_cast<const float4*>(pr + c_off + n0 + 4 * i);
          n_cv[4 * i] = c4.x; n_cv[4 * i + 1] = c4.y; n_cv[4 * i + 2] = c4.z; n_cv[4 * i + 3] = c4.w;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        n_bv[i] = n0 + i < N ? pr[b_off + n0 + i] : 0.f;
        n_cv[i] = (MODE != 1 && n0 + i < N) ? pr[c_off + n0 + i] : 0.f;
      }
    }
  };
  fetch(0);
  for (int j = 0; j < n_tok; ++j) {
    const size_t t = (size_t)(first + j);
    float d = n_d;
    const float x = n_x, z = n_z;
    float bv[NS], cv[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) { bv[i] = n_bv[i]; cv[i] = n_cv[i]; }
    if (j + 1 < n_tok) fetch(j + 1);
    if (dt_raw) {  // the step size still is the product's sum: bias and softplus here
      d += dtb;
      d = d > 20.0f ? d : log1pf(expf(d));
    }
    const float dx = d * x;
    float y = 0.f;
    sum_dt += d;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (FAST) {
        S[i] = fmaf(ex2_approx(d * A[i]), S[i], dx * bv[i]);
      } else {
        // exp(dA) S + dt x B as S + ((exp(dA) - 1) S + dt x B): a decay close to 1 is not rounded to the grid of floats around
        // 1 first, an error of the same sign token after token that would grow along a sequence where dA is small
        S[i] += fmaf(decay_minus_one(d * A[i]), S[i], dx * bv[i]);
      }
      if (MODE != 1) y = fmaf(S[i], cv[i], y);
    }
    if (MODE != 1) {
      for (int o = tpc >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (part == 0 && live) out[t * C + cc] = from_f32<T>((y + dsk * x) * silu_f(z));
    }
  }
  if (live && MODE != 2) {
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      const int n = n0 + i;
      if (n < N) st[n] = S[i];
    }
    if (MODE == 1 && part == 0) piece_sumdt[piece * C + cc] = sum_dt;
  }
}

// Between the two passes over the pieces: a thread a (request, channel, state number) carries the state from the request's slot
// through its pieces, S <- exp(A * sum of the piece's step sizes) S + (the piece's end state from zero), leaves at every piece
// the state at its START (in place of the piece's own end state), and puts the last state back into the slot.
__global__ void scan_carry_kernel(const float* __restrict__ a_log, float* __restrict__ state, float* __restrict__ piece_state,
                                  const float* __restrict__ piece_sumdt, const int* __restrict__ seq_ntok, const int* __restrict__ seq_slot,
                                  int C, int N, int n_seqs) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t per_seq = (size_t)C * N;
  if (i >= per_seq * n_seqs) return;
  const int seq = (int)(i / per_seq);
  const size_t cn = i - (size_t)seq * per_seq;
  const int c = (int)(cn / N);
  const int pieces = (seq_ntok[seq] + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const size_t base = (size_t)pieces_before(seq_ntok, seq, SCAN_CHUNK);
  const float A = -expf(a_log[cn]);
  float* slot = state + (size_t)seq_slot[seq] * per_seq + cn;
  float S = *slot;
  for (int j0 = 0; j0 < pieces; j0 += 8) {  // eight pieces' loads on their way at a time; the carry itself goes piece by piece
    float local[8], sd[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool in = j0 + u < pieces;
      local[u] = in ? piece_state[(base + j0 + u) * per_seq + cn] : 0.f;
      sd[u] = in ? piece_sumdt[(base + j0 + u) * C + c] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < pieces) {
        piece_state[(base + j0 + u) * per_seq + cn] = S;
        S += fmaf(expm1f(A * sd[u]), S, local[u]);  // (once a piece: the library's expm1f)
      }
    }
  }
  *slot = S;
}

}  // namespace

extern "C" int llm_conv_silu(const float* parts, int n_parts, long long pstride, int width, int x_off, int C, int K, const void* w,
                             const float* bias, float* conv_state, const int* token_seq, const int* seq_qoff, const int* seq_ntok,
                             const int* seq_slot, void* out, int dtype, int n_tokens, int n_seqs, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_parts >= 1 && C > 0 && K >= 1 && K <= MAX_TAPS, "conv_silu: bad sizes (taps %d, at most %d)", K, MAX_TAPS);
  LLM_REQUIRE(x_off >= 0 && x_off + C <= width, "conv_silu: columns outside the product");
  dim3 grid(ceil_div(C, 256), n_tokens < 65535 ? n_tokens : 65535);
  if (dtype == LLM_F32)
    launch_kernel(conv_silu_kernel<float>, grid, 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  (const float*)w, bias, (const float*)conv_state, token_seq, seq_qoff, seq_slot, (float*)out, n_tokens);
  else if (dtype == LLM_BF16)
    launch_kernel(conv_silu_kernel<bf16>, grid, 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  (const bf16*)w, bias, (const float*)conv_state, token_seq, seq_qoff, seq_slot, (bf16*)out, n_tokens);
  else
    LLM_REQUIRE(false, "conv_silu: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("conv_silu");
  if (K > 1) {
    launch_kernel(conv_state_kernel, ceil_div((long long)n_seqs * C, 256), 256, 0, stream, parts, n_parts, (size_t)pstride, width, x_off, C, K,
                  conv_state, seq_qoff, seq_ntok, seq_slot, n_seqs);
    LLM_CHECK_LAUNCH("conv_state");
  }
  return LLM_OK;
}

// dt[t, c] = out_act(bias[c] + sum_r wt[r, c] * in_act(proj[t, r])): the step-size map of the selective scan (in_act 0, out_act 0) and
// the decay maps of the linear-state mixers (low_in / low_out above)
extern "C" int llm_lowrank_map(const float* proj, long long ld, int R, const void* wt, const float* bias, int C, float* dt, int dtype,
                               int n_tokens, int in_act, int out_act, float param, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE((in_act == 0 || in_act == 1) && out_act >= 0 && out_act <= 2 && (out_act != 1 || param > 0.f), "lowrank_map: unknown activation %d / %d", in_act, out_act);
  LLM_REQUIRE(n_tokens > 0 && R > 0 && C > 0 && R <= ld, "dt_softplus: bad sizes");
  LLM_REQUIRE(dtype == LLM_F32 || dtype == LLM_BF16, "dt_softplus: unknown dtype %d", dtype);
  if (n_tokens <= 8) {  // single decoded tokens
    const size_t smem_few = ((size_t)R * 8 + 4 * 32 * 8) * sizeof(float);
    LLM_REQUIRE(smem_few <= 48 * 1024, "dt_softplus: a step-size rank of %d exceeds one block's shared memory", R);
    dim3 grid_few(ceil_div(C, 32), ceil_div(n_tokens, 8));
    if (dtype == LLM_F32)
      launch_kernel(dt_softplus_few_kernel<float>, grid_few, 128, smem_few, stream, proj, ld, R, (const float*)wt, bias, C, dt, n_tokens, in_act, out_act, param);
    else
      launch_kernel(dt_softplus_few_kernel<bf16>, grid_few, 128, smem_few, stream, proj, ld, R, (const bf16*)wt, bias, C, dt, n_tokens, in_act, out_act, param);
    LLM_CHECK_LAUNCH("dt_softplus");
    return LLM_OK;
  }
  const int tok = 32;
  const size_t smem = (size_t)tok * R * sizeof(float);
  LLM_REQUIRE(smem <= 48 * 1024, "dt_softplus: a step-size rank of %d exceeds one block's shared memory", R);
  const int threads = DT_THREADS;
  dim3 grid(ceil_div(C, threads), ceil_div(n_tokens, tok));
  LLM_REQUIRE(grid.y <= 65535, "dt_softplus: too many tokens in one step (%d)", n_tokens);
#define LLM_DT(T, TOK) launch_kernel(dt_softplus_kernel<T, TOK>, grid, threads, smem, stream, proj, ld, R, (const T*)wt, bias, C, dt, n_tokens, in_act, out_act, param)
  if (dtype == LLM_F32) LLM_DT(float, 32); else LLM_DT(bf16, 32);
#undef LLM_DT
  LLM_CHECK_LAUNCH("dt_softplus");
  return LLM_OK;
}

extern "C" int llm_dt_softplus(const float* proj, long long ld, int R, const void* wt, const float* bias, int C, float* dt, int dtype,
                               int n_tokens, cudaStream_t stream) {
  return llm_lowrank_map(proj, ld, R, wt, bias, C, dt, dtype, n_tokens, 0, 0, 0.f, stream);
}

extern "C" int llm_selective_scan_piece() { return SCAN_CHUNK; }

// dt_raw != 0: dt holds the step-size product's sums, and softplus(dt + dt_bias) is applied here; else dt holds finished step sizes.
// pieces > 0: the portions are cut into pieces of llm_selective_scan_piece() tokens that run side by side (two passes and a carry
// between them); piece_state holds pieces * C * N floats and piece_sumdt pieces * C, pieces >= the sum over the requests of
// ceil(tokens / piece), max_new_tokens = the longest portion. pieces == 0: every portion is walked by one block a channel tile.
extern "C" int llm_selective_scan(const void* xc, const float* dt, const float* proj, long long ld, int b_off, int c_off,
                                  const float* zparts, int n_parts, long long pstride, int zwidth, int z_off, const float* a_log,
                                  const float* dskip, float* state, const int* seq_qoff, const int* seq_ntok, const int* seq_slot, int C,
                                  int N, void* out, int dtype, int n_seqs, int max_new_tokens, int pieces, float* piece_state,
                                  float* piece_sumdt, const float* dt_bias, int dt_raw, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && C > 0 && N > 0 && N <= 256, "selective_scan: bad sizes (state %d, at most 256)", N);
  LLM_REQUIRE(b_off >= 0 && c_off >= 0 && b_off + N <= ld && c_off + N <= ld && z_off >= 0 && z_off + C <= zwidth, "selective_scan: columns outside the products");
  LLM_REQUIRE(pieces == 0 || (piece_state && piece_sumdt && max_new_tokens > 0), "selective_scan: pieces need their scratch");
  // numbers of a channel's state a thread: few where single tokens leave little else to run side by side, many where pieces do
  const int ns = pieces ? (N <= 16 ? 16 : (N <= 128 ? 8 : 16)) : (N <= 128 ? 4 : 8);
  int tpc = 1;
  while (tpc * ns < N) tpc <<= 1;  // a power of two up to 32
  LLM_REQUIRE(tpc <= 32, "selective_scan: state %d too large", N);
  const int per_seq_pieces = pieces ? ceil_div(max_new_tokens, SCAN_CHUNK) : 1;
  LLM_REQUIRE(per_seq_pieces <= 65535, "selective_scan: portion too long");
  dim3 grid(ceil_div(C, SCAN_THREADS / tpc), per_seq_pieces, n_seqs);
  LLM_REQUIRE(dtype == LLM_F32 || dtype == LLM_BF16, "selective_scan: unknown dtype %d", dtype);
#define LLM_SCAN(T, NS, MODE, FAST)                                                                                                    \
  launch_kernel(selective_scan_kernel<T, NS, MODE, FAST>, grid, SCAN_THREADS, 0, stream, (const T*)xc, dt, proj, ld, b_off, c_off, zparts, \
                n_parts, (size_t)pstride, zwidth, z_off, a_log, dskip, state, seq_qoff, seq_ntok, seq_slot, C, N, tpc, (T*)out, piece_state, \
                piece_sumdt, dt_bias, dt_raw)
#define LLM_SCAN_T(MODE)                                                                                             \
  if (dtype == LLM_F32) {                                                                                            \
    if (ns == 4) LLM_SCAN(float, 4, MODE, false); else if (ns == 8) LLM_SCAN(float, 8, MODE, false); else LLM_SCAN(float, 16, MODE, false); \
  } else {                                                                                                           \
    if (ns == 4) LLM_SCAN(bf16, 4, MODE, true); else if (ns == 8) LLM_SCAN(bf16, 8, MODE, true); else LLM_SCAN(bf16, 16, MODE, true);       \
  }
  if (pieces == 0) {
    LLM_SCAN_T(0);
  } else {
    LLM_SCAN_T(1);
    LLM_CHECK_LAUNCH("selective_scan (pieces)");
    launch_kernel(scan_carry_kernel, ceil_div((long long)n_seqs * C * N, 256), 256, 0, stream, a_log, state, piece_state,
                  (const float*)piece_sumdt, seq_ntok, seq_slot, C, N, n_seqs);
    LLM_CHECK_LAUNCH("selective_scan (carry)");
    LLM_SCAN_T(2);
  }
#undef LLM_SCAN_T
#undef LLM_SCAN
  LLM_CHECK_LAUNCH("selective_scan");
  return LLM_OK;
}
