// Grouped-query attention with the options of the "gated attention" mixer, on CUDA cores in float32 arithmetic (both engine
// precisions, any sizes):
//
//   qkv_prep   per token, from the float32 sums of the [Wq; Wk; Wv; Wg] product: RMS norm of every query and key head over its
//              dk numbers with one weight for all heads (optional; or, `norm_wide`, one RMS norm over all query heads' numbers at
//              once and one over all key heads', with a weight a number), rotation of the first rot_dims numbers of a head in the
//              half-split layout from (cos, sin) tables, value mixing v <- (1 - lambda) v + lambda v_first with the values that
//              an earlier layer of the same step left for these tokens (or leaving them), and the write of k and v into the
//              token's page. Keys have dk numbers a head, values dv.
//   attention  one warp a (token, query head): keys lo..pos of the request through its block table, lo = the later of the
//              window's and the chunk's start (a chunk is [c * size, (c + 1) * size) in absolute positions); softmax in float32
//              whose denominator also holds exp(sink[head]) (optional: a learned term of the denominator alone); the result times
//              sigmoid(gate) (optional, float32 partial sums of the same product; a gate a number or one a head) before it is rounded.
//
// Keys are walked in chunks of 32 aligned to absolute positions, so a token's result does not depend on how its request was
// cut into steps, on the rest of the batch or on page numbers.
#include "common.cuh"

#include <cfloat>
#include <cmath>

namespace {

__device__ __forceinline__ float parts_sum(const float* __restrict__ p, int n_parts, size_t pstride, size_t i) {
  float s = p[i];
  for (int k = 1; k < n_parts; ++k) s += p[(size_t)k * pstride + i];
  return s;
}

constexpr int PREP_WARPS = 4;

// mix_role 0: values as they are; 1: they are also left in v_first; 2: mixed with v_first by *lambda.
template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
    qkv_prep_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int H, int G, int dk, int dv, int rot_dims,
                    const float* __restrict__ wq, const float* __restrict__ wk, float eps, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, const int* __restrict__ positions, const int* __restrict__ token_seq,
                    const int* __restrict__ block_table, int max_blocks, T* __restrict__ q_out, long long ld_q, T* __restrict__ kcache,
                    T* __restrict__ vcache, int page_size, int mix_role, const float* __restrict__ lambda, float* __restrict__ v_first,
                    int norm_wide) {
  extern __shared__ float sh[];  // PREP_WARPS rows of dk
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[tok];
  const size_t row = (size_t)tok * width;
  const int half = rot_dims / 2;
  const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
  const int page = block_table[(size_t)token_seq[tok] * max_blocks + pos / page_size];
  const int in_page = pos % page_size;
  float* buf = sh + (size_t)warp * dk;
  // norm_wide: the norm's statistic is over the whole projection, so every block of the token forms both sums of squares
  // first (the block's threads in turn, then block_sum: an order that depends on the sizes alone)
  float inv_q = 1.f, inv_k = 1.f;
  if (norm_wide) {
    if (wq) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < H * dk; i += blockDim.x) {
        const float v = parts_sum(parts, n_parts, pstride, row + i);
        ss += v * v;
      }
      inv_q = 1.0f / sqrtf(block_sum(ss, red) / (float)(H * dk) + eps);
    }
    if (wk && G > 0) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < G * dk; i += blockDim.x) {
        const float v = parts_sum(parts, n_parts, pstride, row + (size_t)H * dk + i);
        ss += v * v;
      }
      inv_k = 1.0f / sqrtf(block_sum(ss, red) / (float)(G * dk) + eps);
    }
  }
  // query heads 0..H-1, then key heads H..H+G-1: a warp a head; the blocks of a token (blockIdx.y) share its heads and values
  for (int head = blockIdx.y * PREP_WARPS + warp; head < H + G; head += gridDim.y * PREP_WARPS) {
    const bool is_q = head < H;
    const size_t col0 = is_q ? (size_t)head * dk : (size_t)H * dk + (size_t)(head - H) * dk;
    const float* w = is_q ? wq : wk;
    if (w && norm_wide) w += (size_t)(is_q ? head : head - H) * dk;  // a weight a number of the projection
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) {
      const float v = parts_sum(parts, n_parts, pstride, row + col0 + d);
      buf[d] = v;
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = !w ? 1.0f : norm_wide ? (is_q ? inv_q : inv_k) : 1.0f / sqrtf(ss / (float)dk + eps);
    __syncwarp();
    for (int d = lane; d < dk; d += 32) buf[d] = w ? buf[d] * inv * w[d] : buf[d];
    __syncwarp();
    T* dst;
    if (is_q) dst = q_out + (size_t)tok * ld_q + (size_t)head * dk;
    else dst = kcache ? kcache + (((size_t)page * G + (head - H)) * page_size + in_page) * dk : nullptr;
    if (dst) {
      for (int d = lane; d < dk; d += 32) {
        float v = buf[d];
        if (d < half) v = buf[d] * cs[d] - buf[d + half] * sn[d];
        else if (d < rot_dims) v = buf[d] * cs[d - half] + buf[d - half] * sn[d - half];
        dst[d] = from_f32<T>(v);
      }
    }
    __syncwarp();
  }
  // values
  const size_t vcol0 = (size_t)(H + G) * dk;
  const float lam = mix_role == 2 ? *lambda : 0.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < G * dv; i += gridDim.y * blockDim.x) {
    float v = parts_sum(parts, n_parts, pstride, row + vcol0 + i);
    if (mix_role == 1) v_first[(size_t)tok * G * dv + i] = v;
    else if (mix_role == 2) v = (1.0f - lam) * v + lam * v_first[(size_t)tok * G * dv + i];
    if (vcache) {
      const int g = i / dv, d = i - g * dv;
      vcache[(((size_t)page * G + g) * page_size + in_page) * dv + d] = from_f32<T>(v);
    }
  }
}

// The same work for norm_wide when a token's whole [q | k] row fits shared memory: ONE block a token forms the row's sums once
// (the parts added in their order), leaves them in shared memory with both sums of squares, and then a warp a head normalises,
// rotates and writes. A step of few tokens runs it with many warps (a head a warp at once); the other kernel would read every
// part twice and repeat the statistic in each of a token's blocks.
template <typename T>
__global__ void __launch_bounds__(512)
    qkv_prep_wide_kernel(const float* __restrict__ parts, int n_parts, size_t pstride, int width, int H, int G, int dk, int dv, int rot_dims,
                         const float* __restrict__ wq, const float* __restrict__ wk, float eps, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int max_blocks, T* __restrict__ q_out, long long ld_q, T* __restrict__ kcache,
                         T* __restrict__ vcache, int page_size) {
  extern __shared__ float row_s[];  // (H + G) * dk
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int tok = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int pos = positions[tok];
  const size_t row = (size_t)tok * width;
  const int half = rot_dims / 2, nq = H * dk, nk = G * dk;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const float v = parts_sum(parts, n_parts, pstride, row + i);
    row_s[i] = v;
    if (i < nq) ssq += v * v;
    else ssk += v * v;
  }
  const float inv_q = wq ? 1.0f / sqrtf(block_sum(ssq, red) / (float)nq + eps) : 1.0f;
  const float inv_k = (wk && G > 0) ? 1.0f / sqrtf(block_sum(ssk, red) / (float)nk + eps) : 1.0f;
  __syncthreads();
  const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
  const int page = block_table[(size_t)token_seq[tok] * max_blocks + pos / page_size];
  const int in_page = pos % page_size;
  for (int head = warp; head < H + G; head += n_warps) {
    const bool is_q = head < H;
    const float* w = is_q ? wq : wk;
    const float inv = is_q ? inv_q : inv_k;
    const float* buf = row_s + (size_t)head * dk;  // key heads lie right behind the query heads, in the row as in the product
    const float* wh = w ? w + (size_t)(is_q ? head : head - H) * dk : nullptr;
    T* dst;
    if (is_q) dst = q_out + (size_t)tok * ld_q + (size_t)head * dk;
    else dst = kcache ? kcache + (((size_t)page * G + (head - H)) * page_size + in_page) * dk : nullptr;
    if (!dst) continue;
    for (int d = lane; d < dk; d += 32) {
      const float x = wh ? buf[d] * inv * wh[d] : buf[d];
      float v = x;
      if (d < half) {
        const float y = wh ? buf[d + half] * inv * wh[d + half] : buf[d + half];
        v = x * cs[d] - y * sn[d];
      } else if (d < rot_dims) {
        const float y = wh ? buf[d - half] * inv * wh[d - half] : buf[d - half];
        v = x * cs[d - half] + y * sn[d - half];
      }
      dst[d] = from_f32<T>(v);
    }
  }
  if (vcache) {
    const size_t vcol0 = (size_t)(H + G) * dk;
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
      const float v = parts_sum(parts, n_parts, pstride, row + vcol0 + i);
      const int g = i / dv, d = i - g * dv;
      vcache[(((size_t)page * G + g) * page_size + in_page) * dv + d] = from_f32<T>(v);
    }
  }
}

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T, int R>  // R = ceil(dv / 32) output registers a lane
__global__ void __launch_bounds__(WARPS * 32)
    gated_attention_simt_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ kcache, const T* __restrict__ vcache,
                                const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                int max_blocks, T* __restrict__ out, long long ld_out, int n_tokens, int nq, int nkv, int dk, int dv,
                                int page_size, float scale, int window, int chunk, const float* __restrict__ sink,
                                const float* __restrict__ gate, int g_parts, size_t g_pstride, int g_width, int g_off, int g_head) {
  __shared__ float q_s[WARPS][MAX_HD];
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)n_tokens * nq) return;
  const int tok = (int)(item / nq), head = (int)(item - (long long)tok * nq);
  const int kvh = head / (nq / nkv);
  const int pos = positions[tok];
  int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
  const int* table = block_table + (size_t)token_seq[tok] * max_blocks;

  const T* qv = q + (size_t)tok * ld_q + (size_t)head * dk;
  for (int d = lane; d < dk; d += 32) q_s[warp][d] = to_f32(qv[d]);
  __syncwarp();

  float acc[R];
#pragma unroll
  for (int i = 0; i < R; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c = lo / 32; c <= pos / 32; ++c) {
    const int t = c * 32 + lane;
    const bool valid = (t >= lo) && (t <= pos);
    float s = -INFINITY;
    size_t v_off = 0;
    if (valid) {
      const int page = table[t / page_size];
      const size_t slot = ((size_t)page * nkv + kvh) * page_size + (size_t)(t % page_size);
      v_off = slot * dv;
      const T* kr = kcache + slot * dk;
      float dot = 0.f;
      for (int d = 0; d < dk; ++d) dot = fmaf(q_s[warp][d], to_f32(kr[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i] *= alpha;
    const int j_end = min(32, pos - c * 32 + 1);
    const int j_begin = max(0, lo - c * 32);
    for (int j = j_begin; j < j_end; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off_j = __shfl_sync(0xffffffffu, (unsigned long long)v_off, j);
      const T* vr = vcache + off_j;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  if (sink) {  // one more term of the denominator, with no value
    const float sk = sink[head];
    const float m_new = fmaxf(m, sk);
    const float alpha = expf(m - m_new);
    l = l * alpha + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i] *= alpha;
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)tok * ld_out + (size_t)head * dv;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = lane + 32 * i;
    if (d < dv) {
      float v = acc[i] * inv;
      if (gate) {
        const float g = parts_sum(gate, g_parts, g_pstride, (size_t)tok * g_width + g_off + (g_head ? (size_t)head : (size_t)head * dv + d));
        v = v / (1.0f + expf(-g));
      }
      o[d] = from_f32<T>(v);
    }
  }
}

}  // namespace

extern "C" int llm_qkv_prep(const float* parts, int n_parts, long long pstride, int width, int H, int G, int dk, int dv, int rot_dims,
                            const float* wq, const float* wk, float eps, const float* cos_t, const float* sin_t, const int* positions,
                            const int* token_seq, const int* block_table, int max_blocks, void* q_out, long long ld_q, void* kcache,
                            void* vcache, int page_size, int mix_role, const float* lambda, float* v_first, int dtype, int n_tokens,
                            int norm_wide, cudaStream_t stream) {
  // G 0: the product holds queries alone (a layer that reads another layer's keys and values): nothing is written to a cache.
  // norm_wide: wq [H * dk] and wk [G * dk], one RMS norm over each whole projection instead of one a head
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_parts >= 1 && H > 0 && G >= 0 && dk > 0 && dv > 0, "qkv_prep: bad sizes");
  LLM_REQUIRE(G > 0 || (kcache == nullptr && mix_role == 0), "qkv_prep: a product without keys and values writes none");
  LLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk, "qkv_prep: %d rotated dimensions do not fit a head of %d", rot_dims, dk);
  LLM_REQUIRE(rot_dims == 0 || (cos_t && sin_t), "qkv_prep: rotation tables missing");
  LLM_REQUIRE((size_t)(H + G) * dk + (size_t)G * dv <= (size_t)width, "qkv_prep: columns outside the product");
  LLM_REQUIRE((kcache == nullptr) == (vcache == nullptr), "qkv_prep: keys and values are written together");
  LLM_REQUIRE(mix_role == 0 || (v_first && (mix_role == 1 || (mix_role == 2 && lambda))), "qkv_prep: value mixing needs its buffer and weight");
  const size_t smem = (size_t)PREP_WARPS * dk * sizeof(float);
  LLM_REQUIRE(smem <= 48 * 1024, "qkv_prep: a head of %d numbers exceeds one block's shared memory", dk);
  const size_t wide_smem = (size_t)(H + G) * dk * sizeof(float);
  if (norm_wide && mix_role == 0 && wide_smem <= 40 * 1024) {
    // a block a token; with few tokens as many warps as there are heads (up to 16), with many tokens four
    int warps = n_tokens >= 512 ? 4 : min(16, max(4, H + G));
#define LLM_PREP_WIDE(T)                                                                                                             \
  launch_kernel(qkv_prep_wide_kernel<T>, n_tokens, warps * 32, wide_smem, stream, parts, n_parts, (size_t)pstride, width, H, G, dk, dv, \
                rot_dims, wq, wk, eps, cos_t, sin_t, positions, token_seq, block_table, max_blocks, (T*)q_out, ld_q, (T*)kcache,       \
                (T*)vcache, page_size)
    if (dtype == LLM_F32) LLM_PREP_WIDE(float);
    else if (dtype == LLM_BF16) LLM_PREP_WIDE(bf16);
    else LLM_REQUIRE(false, "qkv_prep: unknown dtype %d", dtype);
#undef LLM_PREP_WIDE
    LLM_CHECK_LAUNCH("qkv_prep");
    return LLM_OK;
  }
  // few tokens: the heads of a token are spread over several blocks, so that the sums of many parts are read side by side
  dim3 grid(n_tokens, n_tokens >= 512 ? 1 : min(ceil_div(H + G, PREP_WARPS), 8));
#define LLM_PREP(T)                                                                                                                  \
  launch_kernel(qkv_prep_kernel<T>, grid, PREP_WARPS * 32, smem, stream, parts, n_parts, (size_t)pstride, width, H, G, dk, dv,    \
                rot_dims, wq, wk, eps, cos_t, sin_t, positions, token_seq, block_table, max_blocks, (T*)q_out, ld_q, (T*)kcache,       \
                (T*)vcache, page_size, mix_role, lambda, v_first, norm_wide)
  if (dtype == LLM_F32) LLM_PREP(float);
  else if (dtype == LLM_BF16) LLM_PREP(bf16);
  else LLM_REQUIRE(false, "qkv_prep: unknown dtype %d", dtype);
#undef LLM_PREP
  LLM_CHECK_LAUNCH("qkv_prep");
  return LLM_OK;
}

extern "C" int llm_gated_attention_simt(const void* q, long long ld_q, const void* kcache, const void* vcache, int dtype,
                                        const int* positions, const int* token_seq, const int* block_table, int max_blocks, void* out,
                                        long long ld_out, int n_tokens, int nq, int nkv, int dk, int dv, int page_size, float scale,
                                        int window, int chunk, const float* sink, const float* gate, int g_parts, long long g_pstride,
                                        int g_width, int g_off, int g_head, cudaStream_t stream) {
  // g_head 0: a gate a number of the result (columns g_off + head * dv + d); 1: one gate a head (column g_off + head)
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  LLM_REQUIRE(dk > 0 && dk <= MAX_HD && dv > 0 && dv <= MAX_HD, "attention: head sizes %d / %d not in 1..%d", dk, dv, MAX_HD);
  LLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && chunk >= 0, "attention: bad page_size/max_blocks/window/chunk");
  LLM_REQUIRE(gate == nullptr || (g_parts >= 1 && g_off >= 0 && (long long)g_off + (long long)nq * (g_head ? 1 : dv) <= g_width), "attention: gate columns outside the product");
  const long long items = (long long)n_tokens * nq;
  const int grid = ceil_div(items, WARPS);
#define LLM_GA(T, R)                                                                                                                 \
  launch_kernel(gated_attention_simt_kernel<T, R>, grid, WARPS * 32, 0, stream, (const T*)q, ld_q, (const T*)kcache, (const T*)vcache, \
                positions, token_seq, block_table, max_blocks, (T*)out, ld_out, n_tokens, nq, nkv, dk, dv, page_size, scale, window,   \
                chunk, sink, gate, g_parts, (size_t)g_pstride, g_width, g_off, g_head)
#define LLM_GA_R(T)            \
  if (dv <= 32) LLM_GA(T, 1);  \
  else if (dv <= 64) LLM_GA(T, 2); \
  else if (dv <= 128) LLM_GA(T, 4); \
  else LLM_GA(T, 8)
  if (dtype == LLM_F32) { LLM_GA_R(float); }
  else if (dtype == LLM_BF16) { LLM_GA_R(bf16); }
  else LLM_REQUIRE(false, "attention: unknown dtype %d", dtype);
#undef LLM_GA_R
#undef LLM_GA
  LLM_CHECK_LAUNCH("gated_attention_simt");
  return LLM_OK;
}
