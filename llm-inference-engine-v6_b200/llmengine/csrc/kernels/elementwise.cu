// Embedding gather, RMSNorm (with the residual sum fused in), SiLU*up, residual add, sums of
// K-split partials. The residual stream is float32 in both engine precisions; sums of squares, the
// reciprocal root and the activation are computed in float32.
//
// Formulas follow the reference CPU ops: rmsnorm_f32 (src/kernels.cpp:18-24: out = w*x*inv_rms,
// inv_rms = 1/sqrt(sum(x^2)/dim + eps)), silu_f32 (src/kernels.cpp:26-31: v/(1+exp(-v))) with the
// product by `up` as a separate multiply (src/engine.cpp:388-389), embed_lookup_f32
// (src/kernels.cpp:59-66).
#include "common.cuh"

// ------------------------------------------------------------------------------------ embedding
// sumsq (may be null): sumsq[row] = sum of the squares of the row, for a norm that is folded into
// the product after it; scaled (may be null): the row times next_w in bfloat16, that product's operand.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, float* __restrict__ sumsq, int dim, int vocab,
                             const float* __restrict__ next_w, bf16* __restrict__ scaled, long long ld_scaled, float scale) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; never read out of range
  const T* src = table + (size_t)id * dim;
  float* dst = out + (size_t)row * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = to_f32(src[i]) * scale;  // scale 1 leaves the row as it is
    dst[i] = v;
    ss += v * v;
    if (scaled) scaled[(size_t)row * ld_scaled + i] = __float2bfloat16_rn(v * next_w[i]);
  }
  if (sumsq) {
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) sumsq[row] = ss;
  }
}

// next_w, scaled (both or neither): scaled [rows, ld_scaled] bf16 = next_w * row, the operand of the
// product behind a norm with weight next_w whose 1/rms the product's consumer applies from sumsq.
extern "C" int llm_embed(const void* table, int table_dtype, const int* ids, float* out, float* sumsq, int n_rows,
                         int dim, int vocab, const float* next_w, void* scaled, long long ld_scaled, float scale, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE((next_w == nullptr) == (scaled == nullptr), "embed: the scaled copy needs the weight it is scaled with");
  LLM_REQUIRE(n_rows > 0 && dim > 0 && vocab > 0, "embed: bad sizes rows=%d dim=%d vocab=%d", n_rows, dim, vocab);
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == LLM_F32)
    launch_kernel(embed_kernel<float>, n_rows, threads, 0, stream, (const float*)table, ids, out, sumsq, dim, vocab, next_w, (bf16*)scaled, ld_scaled, scale);
  else if (table_dtype == LLM_BF16)
    launch_kernel(embed_kernel<bf16>, n_rows, threads, 0, stream, (const bf16*)table, ids, out, sumsq, dim, vocab, next_w, (bf16*)scaled, ld_scaled, scale);
  else
    LLM_REQUIRE(false, "embed: unknown table dtype %d", table_dtype);
  LLM_CHECK_LAUNCH("embed");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ RMSNorm
// One block per output row. Source row r = rows ? rows[blockIdx.x] : blockIdx.x.
// x = h[r] + sum_p delta[p][r] (partials added in index order); if write_back, h[r] = x.
// out[blockIdx.x] = (w * x) * inv_rms. With `center` (a layer norm without bias) the row's mean is taken off first:
// out = w * (x - mean) / sqrt(mean((x - mean)^2) + eps), the variance from the deviations themselves (two passes over
// the row in registers), never from sum(x^2) - mean^2.
template <typename T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

// dim % 4 == 0 and dim <= 4 * R * blockDim: the row stays in registers between the two passes.
template <typename TOut, int R>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                           size_t partial_stride, const float* __restrict__ w,
                                                           const int* __restrict__ rows, TOut* __restrict__ out, int dim,
                                                           float eps, int write_back, int center) {
  __shared__ float red[33];
  dep_launch();
  float4 wv[R];
#pragma unroll
  for (int k = 0; k < R; ++k) {  // the norm weight is not produced by the stream: fetch it before waiting
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    wv[k] = i < dim ? *reinterpret_cast<const float4*>(w + i) : make_float4(0, 0, 0, 0);
  }
  dep_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* hr = h + (size_t)r * dim;
  const float* dr = delta ? delta + (size_t)r * dim : nullptr;
  float4 x[R];
  float ss = 0.f;
  if (R > 1 && dr && n_partials == 1) {
    // many rows a launch (a prompt), one product to add: every load of the thread is asked for before
    // any is used, so that a row costs one trip to memory, not one per quarter of it
    float4 d[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      x[k] = i < dim ? *reinterpret_cast<const float4*>(hr + i) : make_float4(0, 0, 0, 0);
      d[k] = i < dim ? *reinterpret_cast<const float4*>(dr + i) : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      x[k].x += d[k].x; x[k].y += d[k].y; x[k].z += d[k].z; x[k].w += d[k].w;
      if (i < dim) {
        if (write_back) *reinterpret_cast<float4*>(hr + i) = x[k];
        ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
      }
    }
  } else
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    x[k] = make_float4(0, 0, 0, 0);
    if (i < dim) {
      x[k] = *reinterpret_cast<const float4*>(hr + i);
      if (dr) {
        for (int p0 = 0; p0 < n_partials; p0 += 8) {  // eight loads in flight, then added in index order
          float4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            d[u] = (p0 + u < n_partials) ? *reinterpret_cast<const float4*>(dr + (size_t)(p0 + u) * partial_stride + i)
                                         : make_float4(0, 0, 0, 0);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (p0 + u < n_partials) { x[k].x += d[u].x; x[k].y += d[u].y; x[k].z += d[u].z; x[k].w += d[u].w; }
          }
        }
        if (write_back) *reinterpret_cast<float4*>(hr + i) = x[k];
      }
      ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
    }
  }
  if (center) {
    float sm = 0.f;
#pragma unroll
    for (int k = 0; k < R; ++k) sm += (x[k].x + x[k].y) + (x[k].z + x[k].w);  // lanes beyond the row hold zeros
    const float mean = block_sum(sm, red) / (float)dim;
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      if (i < dim) {
        x[k].x -= mean; x[k].y -= mean; x[k].z -= mean; x[k].w -= mean;
        ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TOut* o = out + (size_t)blockIdx.x * dim;
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    if (i < dim)
      store4<TOut>(o + i, (wv[k].x * x[k].x) * inv, (wv[k].y * x[k].y) * inv, (wv[k].z * x[k].z) * inv, (wv[k].w * x[k].w) * inv);
  }
}

template <typename TOut>
__global__ void rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                               size_t partial_stride, const float* __restrict__ w,
                               const int* __restrict__ rows, TOut* __restrict__ out, int dim, float eps,
                               int write_back, int center) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* hr = h + (size_t)r * dim;
  const float* dr = delta ? delta + (size_t)r * dim : nullptr;
  float ss = 0.f, sm = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float x = hr[i];
    if (dr) {
      for (int p = 0; p < n_partials; ++p) x += dr[(size_t)p * partial_stride + i];
      if (write_back) hr[i] = x;
    }
    ss += x * x;
    sm += x;
  }
  const bool again = dr && !write_back;  // the sum was not kept: it is formed again, the same additions in the same order
  float mean = 0.f;
  if (center) {
    mean = block_sum(sm, red) / (float)dim;
    ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      float x = hr[i];
      if (again)
        for (int p = 0; p < n_partials; ++p) x += dr[(size_t)p * partial_stride + i];
      ss += (x - mean) * (x - mean);
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TOut* o = out + (size_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float x = hr[i];
    if (again)
      for (int p = 0; p < n_partials; ++p) x += dr[(size_t)p * partial_stride + i];
    o[i] = from_f32<TOut>((w[i] * (x - mean)) * inv);
  }
}

template <typename TOut>
static void launch_rmsnorm(float* h, const float* delta, int n_partials, size_t partial_stride, const float* w, const int* rows,
                           TOut* out, int n_out_rows, int dim, float eps, int write_back, int center, cudaStream_t stream) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec = dim % 4 == 0 && dim <= 16384 && al(h) && al(w) && al(out) && (!delta || (al(delta) && partial_stride % 4 == 0));
  if (vec) {
    const int quads = dim / 4;
    int threads = quads <= 1024 ? ((quads + 31) / 32) * 32 : 1024;
    // Many rows (a prompt): a quarter of the threads with four float4 each, so that every row of the
    // launch is resident at once and all of its bytes are on their way together.
    if (n_out_rows >= 512 && quads >= 256 && quads <= 4096) threads = ((quads / 4 + 31) / 32) * 32;
    const int per_thread = (quads + threads - 1) / threads;
    if (per_thread == 1)
      launch_kernel(rmsnorm_vec_kernel<TOut, 1>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back, center);
    else if (per_thread == 2)
      launch_kernel(rmsnorm_vec_kernel<TOut, 2>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back, center);
    else
      launch_kernel(rmsnorm_vec_kernel<TOut, 4>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back, center);
    return;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < dim) threads *= 2;
  launch_kernel(rmsnorm_kernel<TOut>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back, center);
}

extern "C" int llm_rmsnorm(float* h, const float* delta, int n_partials, long long partial_stride,
                           const float* w, const int* rows, void* out, int out_dtype, int n_out_rows,
                           int dim, float eps, int write_back, int center, cudaStream_t stream) {
  if (n_out_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_out_rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", n_out_rows, dim);
  LLM_REQUIRE(!(rows && write_back), "rmsnorm: write_back with a row list is not allowed");
  LLM_REQUIRE(!delta || n_partials >= 1, "rmsnorm: delta needs n_partials >= 1");
  if (out_dtype == LLM_F32)
    launch_rmsnorm<float>(h, delta, n_partials, (size_t)partial_stride, w, rows, (float*)out, n_out_rows, dim, eps, write_back, center, stream);
  else if (out_dtype == LLM_BF16)
    launch_rmsnorm<bf16>(h, delta, n_partials, (size_t)partial_stride, w, rows, (bf16*)out, n_out_rows, dim, eps, write_back, center, stream);
  else
    LLM_REQUIRE(false, "rmsnorm: unknown out dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("rmsnorm");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ residual add
__global__ void residual_add_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                    size_t partial_stride, size_t n) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float x = h[i];
  for (int p = 0; p < n_partials; ++p) x += delta[(size_t)p * partial_stride + i];
  h[i] = x;
}

extern "C" int llm_residual_add(float* h, const float* delta, int n_partials, long long partial_stride,
                                long long n, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && n_partials >= 1, "residual_add: bad sizes");
  launch_kernel(residual_add_kernel, ceil_div(n, 256), 256, 0, stream, h, delta, n_partials, (size_t)partial_stride, (size_t)n);
  LLM_CHECK_LAUNCH("residual_add");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ SiLU(gate) * up
// in: [rows, 2*ff]; out: [rows, ff]. Column layout of `in`: block == 0: gate in columns [0,ff), up in
// [ff,2ff); block == b > 0: blocks of 2b columns, b of gate followed by the b matching ones of up.
__device__ __forceinline__ void gate_up_columns(int c, int ff, int block, size_t* gate, size_t* up) {
  if (block == 0) {
    *gate = c;
    *up = (size_t)ff + c;
  } else {
    *gate = (size_t)(c / block) * 2 * block + (c % block);
    *up = *gate + block;
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int ff, size_t total, int block, int act, float p0, float p1) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / ff;
  const int c = (int)(i - r * ff);
  size_t gc, uc;
  gate_up_columns(c, ff, block, &gc, &uc);
  const float g = to_f32(in[r * 2 * ff + gc]);
  const float u = to_f32(in[r * 2 * ff + uc]);
  out[i] = from_f32<T>(gated_value(g, u, act, p0, p1));
}

extern "C" int llm_silu_mul(const void* in, void* out, int dtype, int n_rows, int ff, int block, int act, float p0, float p1, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && ff > 0, "silu_mul: bad sizes rows=%d ff=%d", n_rows, ff);
  LLM_REQUIRE(block >= 0 && (block == 0 || ff % block == 0), "silu_mul: column block %d does not divide %d", block, ff);
  LLM_REQUIRE(act >= 0 && act <= 2, "silu_mul: unknown activation %d", act);
  const size_t total = (size_t)n_rows * ff;
  const int blocks = ceil_div((long long)total, 256);
  if (dtype == LLM_F32)
    launch_kernel(silu_mul_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, ff, total, block, act, p0, p1);
  else if (dtype == LLM_BF16)
    launch_kernel(silu_mul_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, ff, total, block, act, p0, p1);
  else
    LLM_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("silu_mul");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ partial sums
// K-split matrix products leave float32 partials [parts, rows, width]; these kernels add them in
// index order (a fixed order: the result does not depend on timing) while doing their own work.
template <typename T>
__global__ void reduce_partials_kernel(const float* __restrict__ partials, int n_partials, size_t stride,
                                       T* __restrict__ out, size_t total) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float x = partials[i];
  for (int p = 1; p < n_partials; ++p) x += partials[(size_t)p * stride + i];
  out[i] = from_f32<T>(x);
}

extern "C" int llm_reduce_partials(const float* partials, int n_partials, long long stride, void* out, int out_dtype,
                                   long long total, cudaStream_t stream) {
  if (total == 0) return LLM_OK;
  LLM_REQUIRE(total > 0 && n_partials >= 1, "reduce_partials: bad sizes");
  const int blocks = ceil_div(total, 256);
  if (out_dtype == LLM_F32)
    launch_kernel(reduce_partials_kernel<float>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (float*)out, (size_t)total);
  else if (out_dtype == LLM_BF16)
    launch_kernel(reduce_partials_kernel<bf16>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (bf16*)out, (size_t)total);
  else
    LLM_REQUIRE(false, "reduce_partials: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("reduce_partials");
  return LLM_OK;
}

// partials: [parts, rows, 2*ff] float32 (gate | up); out [rows, ff] = silu(sum gate) * (sum up).
template <typename T>
__global__ void silu_mul_partials_kernel(const float* __restrict__ partials, int n_partials, size_t stride,
                                         T* __restrict__ out, int ff, size_t total, int block, const RowScale rs, int act, float p0, float p1) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / ff;
  const int c = (int)(i - r * ff);
  size_t gc, uc;
  gate_up_columns(c, ff, block, &gc, &uc);
  const size_t gi = r * 2 * ff + gc, ui = r * 2 * ff + uc;
  float g = 0.f, u = 0.f;
  for (int p0 = 0; p0 < n_partials; p0 += 4) {  // four parts' loads in flight, added in index order
    float gv[4], uv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool in = p0 + k < n_partials;
      gv[k] = in ? partials[(size_t)(p0 + k) * stride + gi] : 0.f;
      uv[k] = in ? partials[(size_t)(p0 + k) * stride + ui] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      g += gv[k];
      u += uv[k];
    }
  }
  const float sc = row_scale(rs, r);  // the norm before the product, when its 1/rms is still owed
  g *= sc;
  u *= sc;
  out[i] = from_f32<T>(gated_value(g, u, act, p0, p1));
}

extern "C" int llm_silu_mul_partials(const float* partials, int n_partials, long long stride, void* out, int out_dtype,
                                     int n_rows, int ff, int block, const float* sumsq, int n_sumsq, float inv_dim, float eps,
                                     int act, float p0, float p1, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(act >= 0 && act <= 2, "silu_mul_partials: unknown activation %d", act);
  const RowScale rs{sumsq, n_sumsq, inv_dim, eps};
  LLM_REQUIRE(n_rows > 0 && ff > 0 && n_partials >= 1, "silu_mul_partials: bad sizes");
  LLM_REQUIRE(block >= 0 && (block == 0 || ff % block == 0), "silu_mul_partials: column block %d does not divide %d", block, ff);
  const size_t total = (size_t)n_rows * ff;
  const int blocks = ceil_div((long long)total, 256);
  if (out_dtype == LLM_F32)
    launch_kernel(silu_mul_partials_kernel<float>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (float*)out, ff, total, block, rs, act, p0, p1);
  else if (out_dtype == LLM_BF16)
    launch_kernel(silu_mul_partials_kernel<bf16>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (bf16*)out, ff, total, block, rs, act, p0, p1);
  else
    LLM_REQUIRE(false, "silu_mul_partials: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("silu_mul_partials");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ token side input
// out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j]: a gate computed from the stream times the
// token's own row of a second embedding table (columns col0 .. col0 + dim).
template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ z, const T* __restrict__ table, long long ld_table, int col0,
                                  const int* __restrict__ ids, int vocab, T* __restrict__ out, int dim, size_t total) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / dim;
  const int j = (int)(i - t * dim);
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  out[i] = from_f32<T>(gate_activation(to_f32(z[i]), 1) * to_f32(table[(size_t)id * ld_table + col0 + j]));
}

extern "C" int llm_token_gate(const void* z, const void* table, long long ld_table, int col0, const int* ids, int vocab, void* out,
                              int n_rows, int dim, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && dim > 0 && col0 >= 0 && col0 + dim <= ld_table && vocab > 0, "token_gate: bad sizes");
  const size_t total = (size_t)n_rows * dim;
  const int blocks = ceil_div((long long)total, 256);
  if (dtype == LLM_F32)
    launch_kernel(token_gate_kernel<float>, blocks, 256, 0, stream, (const float*)z, (const float*)table, ld_table, col0, ids, vocab, (float*)out, dim, total);
  else if (dtype == LLM_BF16)
    launch_kernel(token_gate_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)z, (const bf16*)table, ld_table, col0, ids, vocab, (bf16*)out, dim, total);
  else
    LLM_REQUIRE(false, "token_gate: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("token_gate");
  return LLM_OK;
}

// h += a (+ b), each float32 [parts, rows, dim] partial sums added in index order, a before b; then
// copy (may be null) = h in the engine's dtype: the stream as the operand of a product.
template <typename T>
__global__ void stream_add_kernel(float* __restrict__ h, const float* __restrict__ a, int na, size_t sa, const float* __restrict__ b,
                                  int nb, size_t sb, T* __restrict__ copy, size_t total) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float x = h[i];
  if (a) {
    float d = a[i];
    for (int p = 1; p < na; ++p) d += a[(size_t)p * sa + i];
    x += d;
  }
  if (b) {
    float d = b[i];
    for (int p = 1; p < nb; ++p) d += b[(size_t)p * sb + i];
    x += d;
  }
  h[i] = x;
  if (copy) copy[i] = from_f32<T>(x);
}

extern "C" int llm_stream_add(float* h, const float* a, int na, long long sa, const float* b, int nb, long long sb, void* copy,
                              int copy_dtype, long long total, cudaStream_t stream) {
  if (total == 0) return LLM_OK;
  LLM_REQUIRE(total > 0 && (a == nullptr || na >= 1) && (b == nullptr || nb >= 1), "stream_add: bad sizes");
  const int blocks = ceil_div(total, 256);
  if (copy_dtype == LLM_F32)
    launch_kernel(stream_add_kernel<float>, blocks, 256, 0, stream, h, a, na, (size_t)sa, b, nb, (size_t)sb, (float*)copy, (size_t)total);
  else if (copy_dtype == LLM_BF16)
    launch_kernel(stream_add_kernel<bf16>, blocks, 256, 0, stream, h, a, na, (size_t)sa, b, nb, (size_t)sb, (bf16*)copy, (size_t)total);
  else
    LLM_REQUIRE(false, "stream_add: unknown dtype %d", copy_dtype);
  LLM_CHECK_LAUNCH("stream_add");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ norm of a sub-layer's output
// A block whose norms sit on the sub-layers' OUTPUTS: y = a (+ b), float32 [n, dim] or partial sums [parts, n, dim] added in
// index order; h[r] += ((y / sqrt(mean(y^2) + eps)) * w) * ls  (ls: an optional per-column layer scale); copy[r] (optional) =
// the new h[r] in the engine dtype, the operand of the products that read the stream next. One block a row, float32.
namespace {
constexpr int NA_MAX = 8;  // elements of a row that a thread keeps between the two passes

template <typename T, bool KEEP>  // KEEP: dim <= NA_MAX * blockDim, the row's sums stay in registers
__global__ void norm_add_kernel(float* __restrict__ h, const float* __restrict__ a, int na, size_t sa, const float* __restrict__ b, int nb,
                                size_t sb, const float* __restrict__ w, const float* __restrict__ ls, float eps, T* __restrict__ copy, int dim) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const size_t base = (size_t)blockIdx.x * dim;
  auto sum_at = [&](int i) {
    float y = a[base + i];
    for (int p = 1; p < na; ++p) y += a[(size_t)p * sa + base + i];
    if (b) {
      float d = b[base + i];
      for (int p = 1; p < nb; ++p) d += b[(size_t)p * sb + base + i];
      y += d;
    }
    return y;
  };
  float keep[NA_MAX];
  float ss = 0.f;
  if (KEEP) {
    // part after part for all of the thread's elements at once: NA_MAX loads on their way at a time, and every element still
    // adds its parts in index order (a before b)
#pragma unroll
    for (int k = 0; k < NA_MAX; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      keep[k] = i < dim ? a[base + i] : 0.f;
    }
    for (int p = 1; p < na; ++p) {
#pragma unroll
      for (int k = 0; k < NA_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < dim) keep[k] += a[(size_t)p * sa + base + i];
      }
    }
    if (b) {
      float other[NA_MAX];
#pragma unroll
      for (int k = 0; k < NA_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        other[k] = i < dim ? b[base + i] : 0.f;
      }
      for (int p = 1; p < nb; ++p) {
#pragma unroll
        for (int k = 0; k < NA_MAX; ++k) {
          const int i = threadIdx.x + k * blockDim.x;
          if (i < dim) other[k] += b[(size_t)p * sb + base + i];
        }
      }
#pragma unroll
      for (int k = 0; k < NA_MAX; ++k) keep[k] += other[k];
    }
#pragma unroll
    for (int k = 0; k < NA_MAX; ++k) ss += keep[k] * keep[k];
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      const float y = sum_at(i);
      ss += y * y;
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  auto finish = [&](int i, float y) {
    float v = y * inv * w[i];
    if (ls) v *= ls[i];
    const float x = h[base + i] + v;
    h[base + i] = x;
    if (copy) copy[base + i] = from_f32<T>(x);
  };
  if (KEEP) {
#pragma unroll
    for (int k = 0; k < NA_MAX; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < dim) finish(i, keep[k]);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) finish(i, sum_at(i));
  }
}
}  // namespace

namespace {
// The same for rows of a multiple of 4 numbers behind 16-byte aligned pointers: a thread has up to two groups of four
// neighbouring numbers and moves them by 16-byte loads and stores; every number still adds its parts in index order.
template <typename T>
__global__ void __launch_bounds__(1024)
    norm_add_vec_kernel(float* __restrict__ h, const float* __restrict__ a, int na, size_t sa, const float* __restrict__ b, int nb, size_t sb,
                        const float* __restrict__ w, const float* __restrict__ ls, float eps, T* __restrict__ copy, int dim) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const size_t base = (size_t)blockIdx.x * dim;
  const int groups = dim / 4;
  float4 y[2];
  bool has[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int g = threadIdx.x + k * blockDim.x;
    has[k] = g < groups;
    y[k] = has[k] ? *reinterpret_cast<const float4*>(a + base + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int p = 1; p < na; ++p) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (has[k]) {
        const float4 v = *reinterpret_cast<const float4*>(a + (size_t)p * sa + base + 4 * (threadIdx.x + k * blockDim.x));
        y[k].x += v.x; y[k].y += v.y; y[k].z += v.z; y[k].w += v.w;
      }
    }
  }
  if (b) {
    float4 o[2];
#pragma unroll
    for (int k = 0; k < 2; ++k)
      o[k] = has[k] ? *reinterpret_cast<const float4*>(b + base + 4 * (threadIdx.x + k * blockDim.x)) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 1; p < nb; ++p) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (has[k]) {
          const float4 v = *reinterpret_cast<const float4*>(b + (size_t)p * sb + base + 4 * (threadIdx.x + k * blockDim.x));
          o[k].x += v.x; o[k].y += v.y; o[k].z += v.z; o[k].w += v.w;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) { y[k].x += o[k].x; y[k].y += o[k].y; y[k].z += o[k].z; y[k].w += o[k].w; }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) ss += y[k].x * y[k].x + y[k].y * y[k].y + y[k].z * y[k].z + y[k].w * y[k].w;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (!has[k]) continue;
    const int i = 4 * (threadIdx.x + k * blockDim.x);
    const float4 wv = *reinterpret_cast<const float4*>(w + i);
    float4 v = make_float4(y[k].x * inv * wv.x, y[k].y * inv * wv.y, y[k].z * inv * wv.z, y[k].w * inv * wv.w);
    if (ls) {
      const float4 l = *reinterpret_cast<const float4*>(ls + i);
      v.x *= l.x; v.y *= l.y; v.z *= l.z; v.w *= l.w;
    }
    float4 x = *reinterpret_cast<const float4*>(h + base + i);
    x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
    *reinterpret_cast<float4*>(h + base + i) = x;
    if (copy) store4<T>(copy + base + i, x.x, x.y, x.z, x.w);
  }
}
}  // namespace

extern "C" int llm_norm_add(float* h, const float* a, int na, long long sa, const float* b, int nb, long long sb, const float* w,
                            const float* ls, float eps, void* copy, int copy_dtype, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && dim > 0 && a != nullptr && na >= 1 && (b == nullptr || nb >= 1) && w != nullptr, "norm_add: bad arguments");
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  LLM_REQUIRE(copy_dtype == LLM_F32 || copy_dtype == LLM_BF16, "norm_add: unknown dtype %d", copy_dtype);
#define LLM_NA(T, KEEP) \
  launch_kernel(norm_add_kernel<T, KEEP>, n_rows, threads, 0, stream, h, a, na, (size_t)sa, b, nb, (size_t)sb, w, ls, eps, (T*)copy, dim)
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (dim % 4 == 0 && dim / 4 <= 2048 && al16(h) && al16(a) && al16(b) && al16(w) && al16(ls) && al16(copy) && sa % 4 == 0 && sb % 4 == 0) {
    int vt = ((dim / 4 + 1) / 2 + 31) / 32 * 32;  // two groups of four a thread
    vt = vt < 64 ? 64 : vt;
    if (copy_dtype == LLM_F32)
      launch_kernel(norm_add_vec_kernel<float>, n_rows, vt, 0, stream, h, a, na, (size_t)sa, b, nb, (size_t)sb, w, ls, eps, (float*)copy, dim);
    else
      launch_kernel(norm_add_vec_kernel<bf16>, n_rows, vt, 0, stream, h, a, na, (size_t)sa, b, nb, (size_t)sb, w, ls, eps, (bf16*)copy, dim);
    LLM_CHECK_LAUNCH("norm_add");
    return LLM_OK;
  }
  const bool keep = dim <= NA_MAX * threads;
  if (copy_dtype == LLM_F32) { if (keep) LLM_NA(float, true); else LLM_NA(float, false); }
  else { if (keep) LLM_NA(bf16, true); else LLM_NA(bf16, false); }
#undef LLM_NA
  LLM_CHECK_LAUNCH("norm_add");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ two branches into one
// out[r] = ca * fa(a[r]) + cb * fb(b[r]) for two sets of float32 sums (parts added in index order): f is the identity, or, with a
// weight, the row divided by its root mean square (eps inside the root) times that weight. One block a row, float32.
namespace {
__global__ void __launch_bounds__(256)
    pair_combine_kernel(const float* __restrict__ a, int na, size_t sa, const float* __restrict__ b, int nb, size_t sb,
                        const float* __restrict__ wa, const float* __restrict__ wb, float ca, float cb, float eps, float* __restrict__ out, int dim) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const size_t base = (size_t)blockIdx.x * dim;
  auto sum_of = [&](const float* p, int n, size_t stride, int i) {
    float y = p[base + i];
    for (int k = 1; k < n; ++k) y += p[(size_t)k * stride + base + i];
    return y;
  };
  float inv_a = 1.0f, inv_b = 1.0f;
  if (wa) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float y = sum_of(a, na, sa, i); ss += y * y; }
    inv_a = 1.0f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  }
  if (wb) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float y = sum_of(b, nb, sb, i); ss += y * y; }
    inv_b = 1.0f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  }
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float ya = sum_of(a, na, sa, i), yb = sum_of(b, nb, sb, i);
    if (wa) ya = ya * inv_a * wa[i];
    if (wb) yb = yb * inv_b * wb[i];
    out[base + i] = ca * ya + cb * yb;
  }
}
}  // namespace

extern "C" int llm_pair_combine(const float* a, int na, long long sa, const float* b, int nb, long long sb, const float* wa, const float* wb,
                                float ca, float cb, float eps, float* out, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && dim > 0 && a && b && na >= 1 && nb >= 1 && out, "pair_combine: bad arguments");
  launch_kernel(pair_combine_kernel, n_rows, 256, 0, stream, a, na, (size_t)sa, b, nb, (size_t)sb, wa, wb, ca, cb, eps, out, dim);
  LLM_CHECK_LAUNCH("pair_combine");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ capped logits
// x <- cap * tanh(x / cap), float32 in place: logits squeezed smoothly into (-cap, cap) before anything reads them.
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap, float inv_cap) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] = cap * tanhf(x[i] * inv_cap);
}

extern "C" int llm_softcap(float* x, long long total, float cap, cudaStream_t stream) {
  if (total == 0) return LLM_OK;
  LLM_REQUIRE(total > 0 && cap > 0.f, "softcap: needs a positive cap");
  launch_kernel(softcap_kernel, ceil_div(total, 256), 256, 0, stream, x, (size_t)total, cap, 1.0f / cap);
  LLM_CHECK_LAUNCH("softcap");
  return LLM_OK;
}
