// Per-expert products of the routed feed-forward on tensor cores (bfloat16 operands, float32 accumulators).
//
// The step's (token, choice) pairs arrive sorted by expert in tiles of 64 rows of one expert (routed.cu: group).
// A CTA owns one tile of rows and 64 output columns: its A rows are gathered through the tile's row list (row =
// pair / a_div of the operand), its B rows are 64 rows of the expert's matrix [N, K]. K is walked in blocks of 64
// with cp.async through a ring of three stages in shared memory; four warps of 16 rows each (m16n8k16). Every output row is
// written at its pair's own index; a row's sum depends on K alone, not on the rest of its tile.
// Epilogue 0: the exact (erf) gelu, bfloat16 out; 1: times the pair's router weight, float32 out; 2: the matrix holds a gate
// row and its up row in turn (an even number of rows), out[p, n / 2] = act(gate, up) (silu(gate) * up, or both sides limited: common.cuh), bfloat16 out.
// heads_product_mma: the same tile loop for a product per head over all tokens (the key and value maps of latent attention).
#include "common.cuh"
#include "mma_common.cuh"

#include <cmath>

namespace {

constexpr int RM_ROWS = 64, RM_COLS = 64, RM_BK = 64, RM_LD = RM_BK + 8, RM_THREADS = 128, RM_STAGES = 3;
constexpr size_t RM_SMEM = (size_t)RM_STAGES * (RM_ROWS + RM_COLS) * RM_LD * sizeof(bf16);

// WM 1: a tile of 64 rows x 64 columns, four warps of 16 x 64. WM 2 (many rows an expert): 128 x 128, eight warps of
// 32 x 64 (four along the rows, two along the columns): six ldmatrix feed sixteen mma instead of five feeding eight,
// and a row of the expert's matrix is fetched for twice as many rows.
template <typename TO, int EPI, int WM>
__global__ void __launch_bounds__(RM_THREADS * WM)
    routed_product_mma_kernel(const bf16* __restrict__ a, long long lda, int a_div, const bf16* __restrict__ w, long long w_stride, int N,
                              int K, const int* __restrict__ tile_expert, const int* __restrict__ tile_rows, TO* __restrict__ out,
                              long long ldo, const float* __restrict__ share, int act, float p0, float p1) {
  constexpr int ROWS = RM_ROWS * WM, COLS = RM_COLS * WM, THREADS = RM_THREADS * WM;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16 (*a_s)[ROWS][RM_LD] = reinterpret_cast<bf16 (*)[ROWS][RM_LD]>(smem_raw);
  bf16 (*w_s)[COLS][RM_LD] = reinterpret_cast<bf16 (*)[COLS][RM_LD]>(smem_raw + (size_t)RM_STAGES * ROWS * RM_LD * sizeof(bf16));
  __shared__ int rows_s[ROWS];
  dep_launch();
  dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp % 4, warp_n = warp / 4;
  const int e = tile_expert[blockIdx.y];
  if (e < 0) return;
  const int n0 = blockIdx.x * COLS;
  if (tid < ROWS) rows_s[tid] = tile_rows[(size_t)blockIdx.y * ROWS + tid];
  __syncthreads();
  const bf16* we = w + (size_t)e * w_stride;

  auto load = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < ROWS * (RM_BK / 8) / THREADS; ++i) {
      const int c = tid + i * THREADS, r = c / (RM_BK / 8), ch = c % (RM_BK / 8);
      const int k = kt * RM_BK + ch * 8;
      const int pair = rows_s[r];
      const bool va = pair >= 0 && k < K;
      cp_async16(&a_s[buf][r][ch * 8], a + (va ? (size_t)(pair / a_div) * lda + k : 0), va);
      const bool vw = n0 + r < N && k < K;
      cp_async16(&w_s[buf][r][ch * 8], we + (vw ? (size_t)(n0 + r) * K + k : 0), vw);
    }
  };

  float acc[WM][RM_COLS / 8][4];
#pragma unroll
  for (int i = 0; i < WM; ++i)
#pragma unroll
    for (int j = 0; j < RM_COLS / 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const int k_tiles = (K + RM_BK - 1) / RM_BK;
#pragma unroll
  for (int st = 0; st < RM_STAGES - 1; ++st) {  // the ring's first stages
    if (st < k_tiles) load(st, st);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    const int buf = kt % RM_STAGES;
    cp_async_wait<RM_STAGES - 2>();
    __syncthreads();  // block kt has landed, and everyone is done with the stage that block kt + STAGES - 1 overwrites
    if (kt + RM_STAGES - 1 < k_tiles) load(kt + RM_STAGES - 1, (kt + RM_STAGES - 1) % RM_STAGES);
    cp_async_commit();
#pragma unroll
    for (int ks = 0; ks < RM_BK / 16; ++ks) {
      uint32_t af[WM][4];
#pragma unroll
      for (int i = 0; i < WM; ++i) ldmatrix_x4(af[i], &a_s[buf][(warp_m * WM + i) * 16 + (lane % 16)][ks * 16 + (lane / 16) * 8]);
#pragma unroll
      for (int j2 = 0; j2 < RM_COLS / 16; ++j2) {
        uint32_t b[4];
        ldmatrix_x4(b, &w_s[buf][warp_n * RM_COLS + j2 * 16 + (lane % 8) + (lane / 16) * 8][ks * 16 + ((lane / 8) % 2) * 8]);
#pragma unroll
        for (int i = 0; i < WM; ++i) {
          mma_bf16(acc[i][2 * j2], af[i], b[0], b[1]);
          mma_bf16(acc[i][2 * j2 + 1], af[i], b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < WM; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int pair = rows_s[(warp_m * WM + i) * 16 + lane / 4 + half * 8];
      if (pair < 0) continue;
      const float sc = EPI == 1 ? share[pair] : 1.0f;
      TO* dst = out + (size_t)pair * ldo;
#pragma unroll
      for (int j = 0; j < RM_COLS / 8; ++j) {
#pragma unroll
        for (int el = 0; el < 2; ++el) {
          const int n = n0 + warp_n * RM_COLS + j * 8 + 2 * (lane % 4) + el;
          if (n >= N) continue;
          float v = acc[i][j][2 * half + el];
          if (EPI == 2) {  // the thread holds a gate column and, right of it, its up column
            if (el == 0) {
              const float u = acc[i][j][2 * half + 1];
              dst[n / 2] = from_f32<TO>(gated_value(v, u, act, p0, p1));
            }
            continue;
          }
          if (EPI == 0) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
          else v *= sc;
          dst[n] = from_f32<TO>(v);
        }
      }
    }
  }
}


// Few rows an expert (steps of single tokens): a tile of 16 rows x 64 columns, the four warps side by side along the
// columns, and a ring of six stages: the expert's matrix is all that moves, and what bounds the kernel is how many of
// its bytes are on their way to an SM at a time (a stage holds 9 KB of it and 2 KB of rows).
constexpr int RS_ROWS = 16, RS_STAGES = 6;
constexpr size_t RS_SMEM = (size_t)RS_STAGES * (RS_ROWS + RM_COLS) * RM_LD * sizeof(bf16);

template <typename TO, int EPI>
__global__ void __launch_bounds__(RM_THREADS)
    routed_product_mma_few_kernel(const bf16* __restrict__ a, long long lda, int a_div, const bf16* __restrict__ w, long long w_stride, int N,
                                  int K, const int* __restrict__ tile_expert, const int* __restrict__ tile_rows, TO* __restrict__ out,
                                  long long ldo, const float* __restrict__ share, int act, float p0, float p1) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16 (*a_s)[RS_ROWS][RM_LD] = reinterpret_cast<bf16 (*)[RS_ROWS][RM_LD]>(smem_raw);
  bf16 (*w_s)[RM_COLS][RM_LD] = reinterpret_cast<bf16 (*)[RM_COLS][RM_LD]>(smem_raw + (size_t)RS_STAGES * RS_ROWS * RM_LD * sizeof(bf16));
  __shared__ int rows_s[RS_ROWS];
  dep_launch();
  dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = tile_expert[blockIdx.y];
  if (e < 0) return;
  const int n0 = blockIdx.x * RM_COLS;
  if (tid < RS_ROWS) rows_s[tid] = tile_rows[(size_t)blockIdx.y * RS_ROWS + tid];
  __syncthreads();
  const bf16* we = w + (size_t)e * w_stride;

  auto load = [&](int kt, int buf) {
    {  // rows: 16 x 8 chunks, one a thread
      const int r = tid / (RM_BK / 8), ch = tid % (RM_BK / 8);
      const int k = kt * RM_BK + ch * 8;
      const int pair = rows_s[r];
      const bool va = pair >= 0 && k < K;
      cp_async16(&a_s[buf][r][ch * 8], a + (va ? (size_t)(pair / a_div) * lda + k : 0), va);
    }
#pragma unroll
    for (int i = 0; i < RM_COLS * (RM_BK / 8) / RM_THREADS; ++i) {
      const int c = tid + i * RM_THREADS, r = c / (RM_BK / 8), ch = c % (RM_BK / 8);
      const int k = kt * RM_BK + ch * 8;
      const bool vw = n0 + r < N && k < K;
      cp_async16(&w_s[buf][r][ch * 8], we + (vw ? (size_t)(n0 + r) * K + k : 0), vw);
    }
  };

  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  const int k_tiles = (K + RM_BK - 1) / RM_BK;
#pragma unroll
  for (int st = 0; st < RS_STAGES - 1; ++st) {
    if (st < k_tiles) load(st, st);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    const int buf = kt % RS_STAGES;
    cp_async_wait<RS_STAGES - 2>();
    __syncthreads();
    if (kt + RS_STAGES - 1 < k_tiles) load(kt + RS_STAGES - 1, (kt + RS_STAGES - 1) % RS_STAGES);
    cp_async_commit();
#pragma unroll
    for (int ks = 0; ks < RM_BK / 16; ++ks) {
      uint32_t af[4], b[4];
      ldmatrix_x4(af, &a_s[buf][lane % 16][ks * 16 + (lane / 16) * 8]);
      ldmatrix_x4(b, &w_s[buf][warp * 16 + (lane % 8) + (lane / 16) * 8][ks * 16 + ((lane / 8) % 2) * 8]);
      mma_bf16(acc[0], af, b[0], b[1]);
      mma_bf16(acc[1], af, b[2], b[3]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int pair = rows_s[lane / 4 + half * 8];
    if (pair < 0) continue;
    const float sc = EPI == 1 ? share[pair] : 1.0f;
    TO* dst = out + (size_t)pair * ldo;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int el = 0; el < 2; ++el) {
        const int n = n0 + warp * 16 + j * 8 + 2 * (lane % 4) + el;
        if (n >= N) continue;
        float v = acc[j][2 * half + el];
        if (EPI == 2) {
          if (el == 0) {
            const float u = acc[j][2 * half + 1];
            dst[n / 2] = from_f32<TO>(gated_value(v, u, act, p0, p1));
          }
          continue;
        }
        if (EPI == 0) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
        else v *= sc;
        dst[n] = from_f32<TO>(v);
      }
    }
  }
}

// The same main loop for a product per head over ALL tokens: out[t, h, :] = w[h] a[t, h, :] (a rows lda apart, a head's
// columns lda_h apart; out likewise), optionally times sigmoid of a gate given as float32 partial sums
// [parts, tokens, gwidth] at columns g_off + h * N + n. grid (N / 64, tokens / 64, heads).
__global__ void __launch_bounds__(RM_THREADS)
    heads_product_mma_kernel(const bf16* __restrict__ a, long long lda, long long lda_h, const bf16* __restrict__ w, int T_, int N, int K,
                             bf16* __restrict__ out, long long ldo, long long ldo_h, const float* __restrict__ gate, int n_parts,
                             size_t pstride, int gwidth, int g_off) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16 (*a_s)[RM_ROWS][RM_LD] = reinterpret_cast<bf16 (*)[RM_ROWS][RM_LD]>(smem_raw);
  bf16 (*w_s)[RM_COLS][RM_LD] = reinterpret_cast<bf16 (*)[RM_COLS][RM_LD]>(smem_raw + (size_t)RM_STAGES * RM_ROWS * RM_LD * sizeof(bf16));
  dep_launch();
  dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.z, t0 = blockIdx.y * RM_ROWS, n0 = blockIdx.x * RM_COLS;
  const bf16* ah = a + (size_t)h * lda_h;
  const bf16* wh = w + (size_t)h * N * K;

  auto load = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < RM_ROWS * (RM_BK / 8) / RM_THREADS; ++i) {
      const int c = tid + i * RM_THREADS, r = c / (RM_BK / 8), ch = c % (RM_BK / 8);
      const int k = kt * RM_BK + ch * 8;
      const bool va = t0 + r < T_ && k < K;
      cp_async16(&a_s[buf][r][ch * 8], ah + (va ? (size_t)(t0 + r) * lda + k : 0), va);
      const bool vw = n0 + r < N && k < K;
      cp_async16(&w_s[buf][r][ch * 8], wh + (vw ? (size_t)(n0 + r) * K + k : 0), vw);
    }
  };

  float acc[RM_COLS / 8][4];
#pragma unroll
  for (int j = 0; j < RM_COLS / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int k_tiles = (K + RM_BK - 1) / RM_BK;
#pragma unroll
  for (int st = 0; st < RM_STAGES - 1; ++st) {
    if (st < k_tiles) load(st, st);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    const int buf = kt % RM_STAGES;
    cp_async_wait<RM_STAGES - 2>();
    __syncthreads();
    if (kt + RM_STAGES - 1 < k_tiles) load(kt + RM_STAGES - 1, (kt + RM_STAGES - 1) % RM_STAGES);
    cp_async_commit();
#pragma unroll
    for (int ks = 0; ks < RM_BK / 16; ++ks) {
      uint32_t af[4];
      ldmatrix_x4(af, &a_s[buf][warp * 16 + (lane % 16)][ks * 16 + (lane / 16) * 8]);
#pragma unroll
      for (int j2 = 0; j2 < RM_COLS / 16; ++j2) {
        uint32_t b[4];
        ldmatrix_x4(b, &w_s[buf][j2 * 16 + (lane % 8) + (lane / 16) * 8][ks * 16 + ((lane / 8) % 2) * 8]);
        mma_bf16(acc[2 * j2], af, b[0], b[1]);
        mma_bf16(acc[2 * j2 + 1], af, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t = t0 + warp * 16 + lane / 4 + half * 8;
    if (t >= T_) continue;
    bf16* dst = out + (size_t)t * ldo + (size_t)h * ldo_h;
#pragma unroll
    for (int j = 0; j < RM_COLS / 8; ++j) {
#pragma unroll
      for (int el = 0; el < 2; ++el) {
        const int n = n0 + j * 8 + 2 * (lane % 4) + el;
        if (n >= N) continue;
        float v = acc[j][2 * half + el];
        if (gate) {
          const size_t gi = (size_t)t * gwidth + g_off + (size_t)h * N + n;
          float g = gate[gi];
          for (int q = 1; q < n_parts; ++q) g += gate[(size_t)q * pstride + gi];  // index order
          v *= 1.0f / (1.0f + expf(-g));
        }
        dst[n] = __float2bfloat16_rn(v);
      }
    }
  }
}

}  // namespace

// Rows of a tile: 64; 128 when an expert gets about that many rows or more; 16 when it gets a few.
extern "C" int llm_routed_product_mma_rows(int rows_per_expert) {
  return rows_per_expert >= 96 ? 2 * RM_ROWS : (rows_per_expert <= 8 ? RS_ROWS : RM_ROWS);
}

// Whether the tensor-core kernel takes these operands: 16-byte aligned rows of K % 8 == 0.
extern "C" int llm_routed_product_mma_supported(const void* a, long long lda, const void* w, int K) {
  return K > 0 && K % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0;
}

template <typename TO, int EPI, int WM>
int launch_routed(dim3 grid, cudaStream_t stream, const void* a, long long lda, int a_div, const void* w, long long ws, int N, int K,
                  const int* tile_expert, const int* tile_rows, void* out, long long ldo, const float* share, int act, float p0, float p1) {
  static bool raised = false;
  if (!raised) {
    if (cudaFuncSetAttribute(routed_product_mma_kernel<TO, EPI, WM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(RM_SMEM * WM)) != cudaSuccess)
      return 1;
    raised = true;
  }
  launch_kernel(routed_product_mma_kernel<TO, EPI, WM>, grid, RM_THREADS * WM, RM_SMEM * WM, stream, (const bf16*)a, lda, a_div, (const bf16*)w,
                ws, N, K, tile_expert, tile_rows, (TO*)out, ldo, share, act, p0, p1);
  return 0;
}

// tile: the rows of a tile of tile_rows (64 or 128, as llm_routed_product_mma_rows said when the pairs were grouped).
extern "C" int llm_routed_product_mma(const void* a, long long lda, int a_div, const void* w, int N, int K, const int* tile_expert,
                                      const int* tile_rows, int max_tiles, int tile, void* out, long long ldo, int epilogue,
                                      const float* share, int act, float p0, float p1, cudaStream_t stream) {
  // act, p0, p1: the activation of epilogue 2 (0: silu; 2: both sides limited by p0, slope p1)
  if (max_tiles == 0) return LLM_OK;
  LLM_REQUIRE(act >= 0 && act <= 2, "routed_product_mma: unknown activation %d", act);
  LLM_REQUIRE(llm_routed_product_mma_supported(a, lda, w, K), "routed_product_mma: operands must be 16-byte aligned with K and the row stride multiples of 8");
  LLM_REQUIRE(N > 0 && a_div > 0 && max_tiles > 0 && max_tiles <= 65535, "routed_product_mma: bad sizes");
  LLM_REQUIRE(tile == RS_ROWS || tile == RM_ROWS || tile == 2 * RM_ROWS, "routed_product_mma: tiles of %d rows (16, 64 or 128)", tile);
  LLM_REQUIRE(epilogue == 0 || (epilogue == 1 && share) || (epilogue == 2 && N % 2 == 0), "routed_product_mma: unknown epilogue %d", epilogue);
  if (tile == RS_ROWS) {
    static bool raised_few = false;
    if (!raised_few) {
      LLM_REQUIRE(cudaFuncSetAttribute(routed_product_mma_few_kernel<bf16, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RS_SMEM) == cudaSuccess &&
                  cudaFuncSetAttribute(routed_product_mma_few_kernel<bf16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RS_SMEM) == cudaSuccess &&
                  cudaFuncSetAttribute(routed_product_mma_few_kernel<float, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RS_SMEM) == cudaSuccess,
                  "routed_product_mma: cannot raise the shared memory limit");
      raised_few = true;
    }
    dim3 grid_few(ceil_div(N, RM_COLS), max_tiles);
    const long long wsf = (long long)N * K;
    if (epilogue == 0)
      launch_kernel(routed_product_mma_few_kernel<bf16, 0>, grid_few, RM_THREADS, RS_SMEM, stream, (const bf16*)a, lda, a_div, (const bf16*)w, wsf,
                    N, K, tile_expert, tile_rows, (bf16*)out, ldo, share, act, p0, p1);
    else if (epilogue == 2)
      launch_kernel(routed_product_mma_few_kernel<bf16, 2>, grid_few, RM_THREADS, RS_SMEM, stream, (const bf16*)a, lda, a_div, (const bf16*)w, wsf,
                    N, K, tile_expert, tile_rows, (bf16*)out, ldo, share, act, p0, p1);
    else
      launch_kernel(routed_product_mma_few_kernel<float, 1>, grid_few, RM_THREADS, RS_SMEM, stream, (const bf16*)a, lda, a_div, (const bf16*)w, wsf,
                    N, K, tile_expert, tile_rows, (float*)out, ldo, share, act, p0, p1);
    LLM_CHECK_LAUNCH("routed_product_mma");
    return LLM_OK;
  }
  const int wm = tile / RM_ROWS;
  dim3 grid(ceil_div(N, RM_COLS * wm), max_tiles);
  const long long ws = (long long)N * K;
  int rc;
  if (epilogue == 0)
    rc = wm == 2 ? launch_routed<bf16, 0, 2>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1)
                 : launch_routed<bf16, 0, 1>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1);
  else if (epilogue == 2)
    rc = wm == 2 ? launch_routed<bf16, 2, 2>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1)
                 : launch_routed<bf16, 2, 1>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1);
  else
    rc = wm == 2 ? launch_routed<float, 1, 2>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1)
                 : launch_routed<float, 1, 1>(grid, stream, a, lda, a_div, w, ws, N, K, tile_expert, tile_rows, out, ldo, share, act, p0, p1);
  LLM_REQUIRE(rc == 0, "routed_product_mma: cannot raise the shared memory limit");
  LLM_CHECK_LAUNCH("routed_product_mma");
  return LLM_OK;
}

// Whether heads_product_mma takes these operands (all of bfloat16): 16-byte aligned rows and head offsets, K % 8 == 0.
extern "C" int llm_heads_product_mma_supported(const void* a, long long lda, long long lda_h, const void* w, int K) {
  return K > 0 && K % 8 == 0 && lda % 8 == 0 && lda_h % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(w) & 15u) == 0;
}

extern "C" int llm_heads_product_mma(const void* a, long long lda, long long lda_h, const void* w, void* out, long long ldo, long long ldo_h,
                                     int n_tokens, int H, int N, int K, const float* gate, int n_parts, long long pstride, int gwidth,
                                     int g_off, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(llm_heads_product_mma_supported(a, lda, lda_h, w, K), "heads_product_mma: operands must be 16-byte aligned with K and the strides multiples of 8");
  LLM_REQUIRE(n_tokens > 0 && H > 0 && N > 0 && H <= 65535 && ceil_div(n_tokens, RM_ROWS) <= 65535, "heads_product_mma: bad sizes");
  static bool raised = false;
  if (!raised) {
    LLM_REQUIRE(cudaFuncSetAttribute(heads_product_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RM_SMEM) == cudaSuccess,
                "heads_product_mma: cannot raise the shared memory limit");
    raised = true;
  }
  dim3 grid(ceil_div(N, RM_COLS), ceil_div(n_tokens, RM_ROWS), H);
  launch_kernel(heads_product_mma_kernel, grid, RM_THREADS, RM_SMEM, stream, (const bf16*)a, lda, lda_h, (const bf16*)w, n_tokens, N, K,
                (bf16*)out, ldo, ldo_h, gate, n_parts, (size_t)pstride, gwidth, g_off);
  LLM_CHECK_LAUNCH("heads_product_mma");
  return LLM_OK;
}
