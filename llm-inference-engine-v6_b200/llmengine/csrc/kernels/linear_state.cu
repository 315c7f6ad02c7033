// Mixers whose memory is a matrix per head ("linear state"): S [dk, dv] per request and head, float32, kept in the request's state
// slot, updated token after token by a rank-one write k v^T and read by a query. Three update rules share one kernel:
//
//   MODE 0  decay a key channel, write, read:   S <- diag(a_t) S + k_t v_t^T;              o_t = S^T q_t
//   MODE 1  read with a bonus, decay, write:    o_t = (S + diag(u) k_t v_t^T)^T q_t;       S <- diag(a_t) S + k_t v_t^T
//   MODE 2  delta rule with a decay a head:     S <- g_t S;  w = beta_t (v_t - S^T k_t);   S <- S + k_t w^T;   o_t = S^T q_t
//           (q and k made unit vectors per head first: x / sqrt(sum x^2 + unit_eps))
//
// Every column S[:, j] evolves by itself, so a block takes a (request, head, tile of columns) and walks the request's tokens of the
// step in order; a column's dk numbers are spread over R lanes of a warp (KPT = 16 numbers a lane), the two dot products of a
// token are sums over a lane's numbers and then over the R lanes (xor shuffles, a fixed order). The tokens' q, k, decays and v
// come through shared memory in tiles of a few tokens that warps of their own fetch ahead of the walk (the sums of the products'
// parts, the unit norms and the query's scale are applied there), so the walk itself only syncs once a tile. Results never depend
// on how a request was cut into steps, on the batch or on the slot: the same additions happen in the same order.
//
// In the slot a head's matrix is stored as the threads hold it: number (m, column j, lane r) at ((m * dv + j) * R + r), which is
// S[channel_of(m, r, R), j]; loads and stores of a warp are then 128 contiguous bytes. R = the power of two >= dk / 16.
//
// Beside it: token_shift (every projection's own blend of a token's input with the previous token's, the previous token of a
// portion's first token coming from the slot), delta_gates (the delta rule's decay and write strength per head) and
// head_norm_gate (every head's result divided by its root mean square, times a weight, times silu of a gate).
#include "common.cuh"

#include <cmath>

namespace {

constexpr int KPT = 16;       // state numbers of a column that one lane holds
constexpr int LS_THREADS = 128;   // threads that hold the state, at most: fewer when the blocks would not fill the device
constexpr int LS_FETCHERS = 128;  // threads behind them that fetch the tiles of tokens ahead
constexpr int LS_BLOCK = LS_THREADS + LS_FETCHERS;
constexpr int LS_BUFFERS = 3;    // tiles in shared memory: walked, landing, issued

__device__ __forceinline__ float parts_sum(const float* __restrict__ p, int n_parts, size_t pstride, size_t i) {
  float s = p[i];
  for (int k = 1; k < n_parts; ++k) s += p[(size_t)k * pstride + i];
  return s;
}

struct Sums {  // columns off.. of float32 sums [parts, rows, width]
  const float* p; int n; size_t stride; int width, off;
};

struct LinearStateParams {
  Sums q, k, v;
  const float* decay; int decay_width, decay_off;  // float32 rows: MODE 0/1 a number a (head, key channel); MODE 2 [g: H | beta: H]
  const float* bonus;                              // MODE 1: [H, dk]
  float* state;                                    // [slots, H, R * KPT, dv] in the layout above
  const int* seq_qoff; const int* seq_ntok; const int* seq_slot;
  float* out;                                      // [tokens, H * dv]
  int H, G, dk, dv, R, tile;
  float q_scale, unit_eps;
  int walkers;   // threads of a block that hold the state (a multiple of 32 and of R); LS_FETCHERS more fetch
  int one_part;  // every product comes in one part
  int vec4;      // every row and column offset is a multiple of four numbers on a 16-byte boundary
};

// Key channel of a lane's number m: the lane holds four groups of four neighbouring channels, group c of lane r being channels
// 4 (c R + r) .. + 3, so that a lane reads a group with one 16-byte load and the R lanes of a column read 16 R contiguous bytes.
__device__ __forceinline__ int channel_of(int m, int lane_r, int R) { return (((m >> 2) * R + lane_r) << 2) + (m & 3); }

template <int R>
__device__ __forceinline__ void load16(float (&x)[KPT], const float* __restrict__ row) {
#pragma unroll
  for (int c = 0; c < KPT / 4; ++c) {
    const float4 t = *reinterpret_cast<const float4*>(row + 4 * c * R);
    x[4 * c] = t.x; x[4 * c + 1] = t.y; x[4 * c + 2] = t.z; x[4 * c + 3] = t.w;
  }
}

template <int R>
__device__ __forceinline__ float lanes_sum(float x) {  // over the R lanes of a column, a fixed order
#pragma unroll
  for (int o = R >> 1; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

struct TileRows {  // a tile of tokens in shared memory
  float* q;  // [tile][dkp]
  float* k;  // [tile][dkp]
  float* a;  // [tile][dkp] (MODE 0/1) or [tile][2] (MODE 2)
  float* v;  // [tile][dv]
};

// A tile of tokens through the rule: s the thread's numbers of its column, v[tt * dv + col] the column's value; out points at the
// column's result of the tile's first token. A lane's sixteen products are summed as four interleaved chains ((c0 + c1) +
// (c2 + c3), chain i taking m = i, i + 4, ...), which shortens the dependent chain of a token fourfold; the order is fixed, so a
// token's result is the same in every step that computes it. What the state does not wait for is moved out of its way: the next
// token's rows are read while this one is computed, and a result's sum over the lanes and its store happen one token late.
template <int MODE, int R>
__device__ __forceinline__ void walk_tile(float (&s)[KPT], const float (&u)[KPT], const TileRows& rows, int dv, int col, int cnt, int lane_r,
                                          bool live, float* __restrict__ out, size_t out_stride) {
  constexpr int dkp = R * KPT, a_stride = MODE == 2 ? 2 : dkp;
  float kk[KPT], qq[KPT], aa[KPT], vj, g = 0.f, beta = 0.f;
  auto read = [&](int tt, float (&k_)[KPT], float (&q_)[KPT], float (&a_)[KPT], float& v_, float& g_, float& b_) {
    load16<R>(k_, rows.k + tt * dkp + 4 * lane_r);
    load16<R>(q_, rows.q + tt * dkp + 4 * lane_r);
    if (MODE != 2) {
      load16<R>(a_, rows.a + tt * a_stride + 4 * lane_r);
    } else {
      g_ = rows.a[tt * a_stride];
      b_ = rows.a[tt * a_stride + 1];
    }
    v_ = live ? rows.v[tt * dv + col] : 0.f;
  };
  read(0, kk, qq, aa, vj, g, beta);
  float pend = 0.f;
#pragma unroll 4
  for (int tt = 0; tt < cnt; ++tt) {
    float kn[KPT], qn[KPT], an[KPT], vn, gn = 0.f, bn = 0.f;
    read(min(tt + 1, cnt - 1), kn, qn, an, vn, gn, bn);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (MODE == 0) {
#pragma unroll
      for (int m = 0; m < KPT; ++m) {
        s[m] = fmaf(kk[m], vj, aa[m] * s[m]);
        acc[m & 3] = fmaf(s[m], qq[m], acc[m & 3]);
      }
    } else if (MODE == 1) {
#pragma unroll
      for (int m = 0; m < KPT; ++m) {
        const float kv = kk[m] * vj;
        acc[m & 3] = fmaf(fmaf(u[m], kv, s[m]), qq[m], acc[m & 3]);
        s[m] = fmaf(aa[m], s[m], kv);
      }
    } else {
      float dot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int m = 0; m < KPT; ++m) {
        s[m] *= g;
        dot[m & 3] = fmaf(s[m], kk[m], dot[m & 3]);
      }
      const float d = lanes_sum<R>((dot[0] + dot[1]) + (dot[2] + dot[3]));
      const float w = beta * (vj - d);
#pragma unroll
      for (int m = 0; m < KPT; ++m) {
        s[m] = fmaf(kk[m], w, s[m]);
        acc[m & 3] = fmaf(s[m], qq[m], acc[m & 3]);
      }
    }
    if (tt > 0) {
      const float o = lanes_sum<R>(pend);
      if (live && lane_r == 0) out[(size_t)(tt - 1) * out_stride] = o;
    }
    pend = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
      kk[m] = kn[m];
      qq[m] = qn[m];
      if (MODE != 2) aa[m] = an[m];
    }
    vj = vn; g = gn; beta = bn;
  }
  const float o = lanes_sum<R>(pend);
  if (live && lane_r == 0) out[(size_t)(cnt - 1) * out_stride] = o;
}

__device__ __forceinline__ void copy4_async(float* smem_dst, const float* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy16_async(float* smem_dst, const float* gmem_src) {  // both on 16-byte boundaries
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copies_wait_but_last() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// A tile's rows into shared memory by the n_thr fetching threads (thread `tid` of them), in two steps so that two tiles can be
// on their way while a third is walked. fetch_issue: every thread takes elements of the whole tile in turn. Products in one
// part (a prompt's portion) are copied asynchronously (16 bytes a copy where every address allows it), no registers held, and
// the copies of a tile are one group. Products in several parts (few tokens, K cut) go through registers, a few elements at a
// time, the parts added in their order. fetch_finish, once the tile's group has landed: the thread scales its own queries; the
// delta rule's unit norms need a token's whole row, so the fetchers meet (barrier 1 is theirs alone) and a warp a token
// scales what was stored.
template <int MODE>
__device__ __forceinline__ void fetch_issue(const LinearStateParams& p, size_t row0, int cnt, int head, int kvh, int dk, int dkp, int dv,
                                            int tid, int n_thr, const TileRows& rows) {
  const bool unit = MODE == 2 && p.unit_eps >= 0.f;
  const float qmul = unit ? 1.0f : p.q_scale;
  const int lg = __ffs(dkp) - 1;  // dkp is a power of two
  const int n_qk = cnt * dkp, n_v = cnt * dv;
  if (p.one_part) {
    if (p.vec4) {
      for (int e = tid; e < (n_qk >> 2); e += n_thr) {
        const int tt = e >> (lg - 2), i = (e << 2) & (dkp - 1);
        const size_t row = row0 + tt;
        if (i < dk) {
          copy16_async(rows.q + 4 * e, p.q.p + row * p.q.width + p.q.off + (size_t)kvh * dk + i);
          copy16_async(rows.k + 4 * e, p.k.p + row * p.k.width + p.k.off + (size_t)kvh * dk + i);
          if (MODE != 2) copy16_async(rows.a + 4 * e, p.decay + row * p.decay_width + p.decay_off + (size_t)head * dk + i);
        } else {
          const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<float4*>(rows.q + 4 * e) = z;
          *reinterpret_cast<float4*>(rows.k + 4 * e) = z;
          if (MODE != 2) *reinterpret_cast<float4*>(rows.a + 4 * e) = z;
        }
      }
      const int dv4 = dv >> 2;
      for (int e = tid; e < (n_v >> 2); e += n_thr) {
        const int tt = e / dv4, j = (e - tt * dv4) << 2;
        copy16_async(rows.v + 4 * e, p.v.p + (row0 + tt) * p.v.width + p.v.off + (size_t)head * dv + j);
      }
    } else {
      for (int e = tid; e < n_qk; e += n_thr) {
        const int tt = e >> lg, i = e & (dkp - 1);
        const size_t row = row0 + tt;
        if (i < dk) {
          copy4_async(rows.q + e, p.q.p + row * p.q.width + p.q.off + (size_t)kvh * dk + i);
          copy4_async(rows.k + e, p.k.p + row * p.k.width + p.k.off + (size_t)kvh * dk + i);
          if (MODE != 2) copy4_async(rows.a + e, p.decay + row * p.decay_width + p.decay_off + (size_t)head * dk + i);
        } else {
          rows.q[e] = rows.k[e] = 0.f;
          if (MODE != 2) rows.a[e] = 0.f;
        }
      }
      for (int e = tid; e < n_v; e += n_thr) {
        const int tt = e / dv, j = e - tt * dv;
        copy4_async(rows.v + e, p.v.p + (row0 + tt) * p.v.width + p.v.off + (size_t)head * dv + j);
      }
    }
    if (MODE == 2)
      for (int e = tid; e < 2 * cnt; e += n_thr)
        copy4_async(rows.a + e, p.decay + (row0 + (e >> 1)) * p.decay_width + p.decay_off + (e & 1) * p.H + head);
    return;
  }
  constexpr int U = 4;  // elements a thread has in flight: their loads are issued together, part after part in the parts' order
  for (int e0 = tid; e0 < n_qk; e0 += U * n_thr) {
    float qv[U], kv[U], av[U];
    size_t qi[U], ki[U];
    bool ok[U];
#pragma unroll
    for (int x = 0; x < U; ++x) {
      const int e = e0 + x * n_thr, tt = e >> lg, i = e & (dkp - 1);
      const size_t row = row0 + tt;
      ok[x] = e < n_qk && i < dk;
      qi[x] = row * p.q.width + p.q.off + (size_t)kvh * dk + i;
      ki[x] = row * p.k.width + p.k.off + (size_t)kvh * dk + i;
      qv[x] = kv[x] = 0.f;
      av[x] = (MODE != 2 && ok[x]) ? p.decay[row * p.decay_width + p.decay_off + (size_t)head * dk + i] : 0.f;
    }
    for (int part = 0; part < p.q.n; ++part) {
#pragma unroll
      for (int x = 0; x < U; ++x)
        if (ok[x]) qv[x] += p.q.p[(size_t)part * p.q.stride + qi[x]];
    }
    for (int part = 0; part < p.k.n; ++part) {
#pragma unroll
      for (int x = 0; x < U; ++x)
        if (ok[x]) kv[x] += p.k.p[(size_t)part * p.k.stride + ki[x]];
    }
#pragma unroll
    for (int x = 0; x < U; ++x) {
      const int e = e0 + x * n_thr;
      if (e < n_qk) {
        rows.q[e] = qv[x] * qmul;
        rows.k[e] = kv[x];
        if (MODE != 2) rows.a[e] = av[x];
      }
    }
  }
  for (int e0 = tid; e0 < n_v; e0 += U * n_thr) {
    float vv[U];
    size_t vi[U];
#pragma unroll
    for (int x = 0; x < U; ++x) {
      const int e = min(e0 + x * n_thr, n_v - 1), tt = e / dv, j = e - tt * dv;
      vi[x] = (row0 + tt) * p.v.width + p.v.off + (size_t)head * dv + j;
      vv[x] = 0.f;
    }
    for (int part = 0; part < p.v.n; ++part) {
#pragma unroll
      for (int x = 0; x < U; ++x) vv[x] += p.v.p[(size_t)part * p.v.stride + vi[x]];
    }
#pragma unroll
    for (int x = 0; x < U; ++x)
      if (e0 + x * n_thr < n_v) rows.v[e0 + x * n_thr] = vv[x];
  }
  if (MODE == 2)
    for (int e = tid; e < 2 * cnt; e += n_thr) rows.a[e] = p.decay[(row0 + (e >> 1)) * p.decay_width + p.decay_off + (e & 1) * p.H + head];
}

template <int MODE>
__device__ __forceinline__ void fetch_finish(const LinearStateParams& p, int cnt, int dk, int dkp, int tid, int n_thr, const TileRows& rows) {
  const bool unit = MODE == 2 && p.unit_eps >= 0.f;
  const float qmul = unit ? 1.0f : p.q_scale;
  if (p.one_part && qmul != 1.0f) {  // the thread's own copies, as fetch_issue dealt them
    const int n_qk = cnt * dkp;
    if (p.vec4) {
      for (int e = tid; e < (n_qk >> 2); e += n_thr) {
        float4 t = *reinterpret_cast<float4*>(rows.q + 4 * e);
        t.x *= qmul; t.y *= qmul; t.z *= qmul; t.w *= qmul;
        *reinterpret_cast<float4*>(rows.q + 4 * e) = t;
      }
    } else {
      for (int e = tid; e < n_qk; e += n_thr) rows.q[e] *= qmul;
    }
  }
  if (unit) {
    asm volatile("bar.sync 1, %0;" ::"r"(n_thr) : "memory");
    const int lane = tid & 31;
    for (int tt = tid >> 5; tt < cnt; tt += n_thr >> 5) {
      float ssq = 0.f, ssk = 0.f;
      for (int i = lane; i < dkp; i += 32) {
        ssq = fmaf(rows.q[tt * dkp + i], rows.q[tt * dkp + i], ssq);
        ssk = fmaf(rows.k[tt * dkp + i], rows.k[tt * dkp + i], ssk);
      }
      ssq = warp_sum(ssq);
      ssk = warp_sum(ssk);
      const float qm = p.q_scale / sqrtf(ssq + p.unit_eps), km = 1.0f / sqrtf(ssk + p.unit_eps);
      for (int i = lane; i < dkp; i += 32) {  // the lane's own numbers again
        rows.q[tt * dkp + i] *= qm;
        rows.k[tt * dkp + i] *= km;
      }
    }
  }
}

// Threads 0 .. p.walkers - 1 hold the state and walk; the LS_FETCHERS threads behind them only fetch. Three buffers: while the walkers are in
// tile i of the request's tokens, tile i + 1 lands and is finished and the copies of tile i + 2 are issued; the block meets once
// a tile. (A decode step has one tile of one token; the walkers read their state while it is fetched.)
// FEW: for steps of about a token a request (decoding). The same code held to half the registers, so that two blocks share a
// multiprocessor: such a step is a state's trip to memory and back, and more blocks in flight hide more of it.
template <int MODE, int R, bool FEW>
__global__ void __launch_bounds__(LS_BLOCK, FEW ? 2 : 1) linear_state_kernel(const LinearStateParams p) {
  extern __shared__ __align__(16) float sh_ls[];
  dep_launch();
  dep_wait();
  const int seq = blockIdx.z, head = blockIdx.y, dk = p.dk, dv = p.dv;
  const int n_tok = p.seq_ntok[seq];
  if (n_tok <= 0) return;
  const int first = p.seq_qoff[seq];
  constexpr int dkp = R * KPT, a_stride = MODE == 2 ? 2 : dkp;
  const int kvh = head / (p.H / p.G);
  const bool walker = threadIdx.x < p.walkers;
  const int lane_r = threadIdx.x & (R - 1);
  const int col = blockIdx.x * (p.walkers / R) + threadIdx.x / R;
  const bool live = walker && col < dv;
  const int tile = p.tile, n_tiles = (n_tok + tile - 1) / tile;
  const size_t a_floats = ((size_t)tile * a_stride + 3) & ~(size_t)3;
  const size_t buf_floats = ((size_t)tile * (2 * dkp + dv) + a_floats + 3) & ~(size_t)3;  // every region starts on 16 bytes
  auto rows_of = [&](int i) {
    TileRows r;
    r.q = sh_ls + (size_t)(i % LS_BUFFERS) * buf_floats;
    r.k = r.q + (size_t)tile * dkp;
    r.a = r.k + (size_t)tile * dkp;
    r.v = r.a + a_floats;
    return r;
  };
  const int ftid = threadIdx.x - p.walkers, n_fetch = LS_FETCHERS;
  auto issue = [&](int i) {  // a group of copies a call, empty behind the last tile
    if (i < n_tiles)
      fetch_issue<MODE>(p, (size_t)(first + i * tile), min(tile, n_tok - i * tile), head, kvh, dk, dkp, dv, ftid, n_fetch, rows_of(i));
    copies_commit();
  };
  auto finish = [&](int i) {
    if (i < n_tiles) fetch_finish<MODE>(p, min(tile, n_tok - i * tile), dk, dkp, ftid, n_fetch, rows_of(i));
  };

  float* st = p.state + ((size_t)p.seq_slot[seq] * p.H + head) * (size_t)dkp * dv;
  float s[KPT], u[KPT];
  if (walker) {
#pragma unroll
    for (int m = 0; m < KPT; ++m) {
      s[m] = live ? st[((size_t)m * dv + col) * R + lane_r] : 0.f;
      const int i = channel_of(m, lane_r, R);
      u[m] = (MODE == 1 && i < dk) ? p.bonus[(size_t)head * dk + i] : 0.f;
    }
  } else {
    issue(0);
    issue(1);
    copies_wait_but_last();
    finish(0);
  }
  __syncthreads();
  for (int i = 0; i < n_tiles; ++i) {
    if (walker) {
      const int t0 = i * tile;
      walk_tile<MODE, R>(s, u, rows_of(i), dv, col, min(tile, n_tok - t0), lane_r, live,
                         p.out + (size_t)(first + t0) * p.H * dv + (size_t)head * dv + col, (size_t)p.H * dv);
    } else {
      issue(i + 2);
      copies_wait_but_last();
      finish(i + 1);
    }
    __syncthreads();  // tile i has been used up, tile i + 1 is in place
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < KPT; ++m) st[((size_t)m * dv + col) * R + lane_r] = s[m];
  }
}

// out[s][t, c] = x[t, c] + (prev[c] - x[t, c]) * mu[s, c], prev = the request's token before t (of this step, or from the slot)
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mu, int n_out, const float* __restrict__ shift_state,
                                   const int* __restrict__ token_seq, const int* __restrict__ seq_qoff, const int* __restrict__ seq_slot,
                                   T* __restrict__ out, int n_tokens, int D) {
  dep_launch();
  dep_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  for (int tok = blockIdx.y; tok < n_tokens; tok += gridDim.y) {
    const int seq = token_seq[tok];
    const float cur = to_f32(x[(size_t)tok * D + c]);
    const float prev = tok > seq_qoff[seq] ? to_f32(x[(size_t)(tok - 1) * D + c]) : shift_state[(size_t)seq_slot[seq] * D + c];
    const float d = prev - cur;
    for (int s = 0; s < n_out; ++s) out[((size_t)s * n_tokens + tok) * D + c] = from_f32<T>(fmaf(d, mu[(size_t)s * D + c], cur));
  }
}

template <typename T>
__global__ void token_shift_state_kernel(const T* __restrict__ x, float* __restrict__ shift_state, const int* __restrict__ seq_qoff,
                                         const int* __restrict__ seq_ntok, const int* __restrict__ seq_slot, int n_seqs, int D) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_seqs * D) return;
  const int seq = (int)(i / D), c = (int)(i - (size_t)seq * D);
  const int n = seq_ntok[seq];
  if (n > 0) shift_state[(size_t)seq_slot[seq] * D + c] = to_f32(x[(size_t)(seq_qoff[seq] + n - 1) * D + c]);
}

// out[t] = [g: H | beta: H], g = exp(-exp(a_log[h]) * softplus(a[t, h] + dt_bias[h])), beta = sigmoid(b[t, h])
__global__ void delta_gates_kernel(const Sums a, const Sums b, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ out, int n_tokens, int H) {
  dep_launch();
  dep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * H) return;
  const size_t tok = i / H;
  const int h = (int)(i - tok * H);
  const float z = parts_sum(a.p, a.n, a.stride, tok * a.width + a.off + h) + dt_bias[h];
  const float sp = z > 20.0f ? z : log1pf(expf(z));
  out[tok * 2 * H + h] = expf(-expf(a_log[h]) * sp);
  out[tok * 2 * H + H + h] = 1.0f / (1.0f + expf(-parts_sum(b.p, b.n, b.stride, tok * b.width + b.off + h)));
}

// a warp a (token, head): out = o / sqrt(mean(o^2) + eps) * weight * silu(gate); weight [dv] for all heads or [H * dv]
template <typename T>
__global__ void __launch_bounds__(128)
    head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, int weight_per_head, const Sums gate, float eps,
                          T* __restrict__ out, int n_tokens, int H, int dv) {
  dep_launch();
  dep_wait();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * H) return;
  const int lane = threadIdx.x & 31;
  const size_t tok = (size_t)(item / H);
  const int head = (int)(item - (long long)tok * H);
  const float* row = o + tok * (size_t)H * dv + (size_t)head * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss = fmaf(row[d], row[d], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) {
    float v = row[d] * inv * weight[weight_per_head ? (size_t)head * dv + d : d];
    if (gate.p) {
      const float g = parts_sum(gate.p, gate.n, gate.stride, tok * gate.width + gate.off + (size_t)head * dv + d);
      v *= g / (1.0f + expf(-g));
    }
    out[tok * (size_t)H * dv + (size_t)head * dv + d] = from_f32<T>(v);
  }
}

int device_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// Rotation of float32 sums for mixers whose recurrence reads rotated queries and keys: for every token and each of `heads` heads
// of dk numbers that lie side by side from column `off` of the sums, the pair (i, i + rot_dims / 2) of the head's first rot_dims
// numbers turns by the token's position (cos / sin tables [positions, rot_dims / 2]); heads from `scaled_from` on are then
// multiplied by `scale`. out [tokens, heads * dk] float32: nothing is rounded on the way.
__global__ void rotate_sums_kernel(Sums x, int heads, int dk, int rot_dims, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   const int* __restrict__ positions, float* __restrict__ out, int n_tokens, int scaled_from, float scale) {
  dep_launch();
  dep_wait();
  // a thread a pair of the rotated part, or a single number behind it: dk - half items a head, every number read and written once
  const int half = rot_dims / 2, items = dk - half, per = heads * items;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * per) return;
  const int tok = (int)(i / per), c = (int)(i - (size_t)tok * per), head = c / items, j = c - head * items;
  const float mul = head >= scaled_from ? scale : 1.0f;
  const size_t src = (size_t)tok * x.width + x.off + (size_t)head * dk, dst = ((size_t)tok * heads + head) * dk;
  if (j < half) {
    const float u = parts_sum(x.p, x.n, x.stride, src + j), v = parts_sum(x.p, x.n, x.stride, src + j + half);
    const float cs = cos_t[(size_t)positions[tok] * half + j], sn = sin_t[(size_t)positions[tok] * half + j];
    out[dst + j] = (u * cs - v * sn) * mul;
    out[dst + j + half] = (v * cs + u * sn) * mul;
  } else {
    out[dst + j + half] = parts_sum(x.p, x.n, x.stride, src + j + half) * mul;
  }
}

int lanes_for(int dk) {
  int r = 1;
  while (r * KPT < dk) r *= 2;
  return r;
}

}  // namespace

// Lanes a column of the state is spread over (the slot holds lanes * 16 rows a head); 0 if dk is beyond the kernel.
extern "C" int llm_linear_state_lanes(int dk) {
  if (dk <= 0 || dk > 32 * KPT) return 0;
  return lanes_for(dk);
}

extern "C" int llm_linear_state(int mode, const float* q, int qn, long long qs, int qw, int qo, const float* k, int kn, long long ks, int kw,
                                int ko, const float* v, int vn, long long vs, int vw, int vo, const float* decay, int decay_width,
                                int decay_off, const float* bonus, float* state, const int* seq_qoff, const int* seq_ntok,
                                const int* seq_slot, float* out, int n_tokens, int n_seqs, int H, int G, int dk, int dv, float q_scale,
                                float unit_eps, int decay_const, cudaStream_t stream) {
  // decay_const: `decay` is one row that holds for every token (decays that are constants of the model)
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(mode >= 0 && mode <= 2, "linear_state: unknown update rule %d", mode);
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && H > 0 && H <= 65535 && G > 0 && H % G == 0 && dv > 0, "linear_state: bad sizes");
  LLM_REQUIRE(llm_linear_state_lanes(dk) > 0, "linear_state: a key size of %d is not in 1..%d", dk, 32 * KPT);
  LLM_REQUIRE(mode == 2 || G == H, "linear_state: only the delta rule shares query/key heads");
  LLM_REQUIRE(q && k && v && decay && state && out && qn >= 1 && kn >= 1 && vn >= 1 && (mode != 1 || bonus), "linear_state: missing tensors");
  LLM_REQUIRE(qo + G * dk <= qw && ko + G * dk <= kw && vo + H * dv <= vw && decay_off + (mode == 2 ? 2 * H : H * dk) <= decay_width,
              "linear_state: columns outside their rows");
  LinearStateParams p;
  p.q = Sums{q, qn, (size_t)qs, qw, qo}; p.k = Sums{k, kn, (size_t)ks, kw, ko}; p.v = Sums{v, vn, (size_t)vs, vw, vo};
  p.decay = decay; p.decay_width = decay_const ? 0 : decay_width; p.decay_off = decay_off; p.bonus = bonus; p.state = state;
  p.seq_qoff = seq_qoff; p.seq_ntok = seq_ntok; p.seq_slot = seq_slot; p.out = out;
  p.H = H; p.G = G; p.dk = dk; p.dv = dv; p.R = lanes_for(dk); p.q_scale = q_scale; p.unit_eps = unit_eps;
  const int dkp = p.R * KPT;
  const int a_stride = mode == 2 ? 2 : dkp;
  auto smem_for = [&](int tile) {  // as the kernel lays a buffer out
    const size_t a_floats = ((size_t)tile * a_stride + 3) & ~(size_t)3;
    return LS_BUFFERS * ((((size_t)tile * (2 * dkp + dv) + a_floats + 3) & ~(size_t)3) * sizeof(float));
  };
  const bool few = n_tokens <= 2 * n_seqs;
  p.tile = few ? 2 : 16;
  while (p.tile > 1 && smem_for(p.tile) > 48 * 1024) p.tile /= 2;
  LLM_REQUIRE(smem_for(p.tile) <= 48 * 1024, "linear_state: heads of %d / %d numbers exceed one block's shared memory", dk, dv);
  p.one_part = qn == 1 && kn == 1 && vn == 1;
  auto quads = [](const void* ptr, long long width, long long off) { return ((uintptr_t)ptr & 15) == 0 && width % 4 == 0 && off % 4 == 0; };
  p.vec4 = dk % 4 == 0 && dv % 4 == 0 && quads(q, qw, qo) && quads(k, kw, ko) && quads(v, vw, vo) && (mode == 2 || quads(decay, p.decay_width, decay_off));
  // the walk is bound by what a multiprocessor's shared memory delivers a token, so few blocks are cut into more, down to a warp of walkers
  p.walkers = LS_THREADS;
  const long long per_column_block = (long long)H * n_seqs;
  while (p.walkers > 32 && 2 * per_column_block * ceil_div(dv, p.walkers / p.R) <= device_sms()) p.walkers /= 2;
  dim3 grid(ceil_div(dv, p.walkers / p.R), H, n_seqs);
  const size_t smem = smem_for(p.tile);
#define LS_LAUNCH(M, RR)                                                                                        \
  if (few) launch_kernel(linear_state_kernel<M, RR, true>, grid, p.walkers + LS_FETCHERS, smem, stream, p);     \
  else launch_kernel(linear_state_kernel<M, RR, false>, grid, p.walkers + LS_FETCHERS, smem, stream, p)
#define LS_LANES(M)                  \
  switch (p.R) {                     \
    case 1: LS_LAUNCH(M, 1); break;  \
    case 2: LS_LAUNCH(M, 2); break;  \
    case 4: LS_LAUNCH(M, 4); break;  \
    case 8: LS_LAUNCH(M, 8); break;  \
    case 16: LS_LAUNCH(M, 16); break; \
    default: LS_LAUNCH(M, 32); break; \
  }
  if (mode == 0) { LS_LANES(0) } else if (mode == 1) { LS_LANES(1) } else { LS_LANES(2) }
#undef LS_LANES
#undef LS_LAUNCH
  LLM_CHECK_LAUNCH("linear_state");
  return LLM_OK;
}

extern "C" int llm_token_shift(const void* x, const float* mu, int n_out, float* shift_state, const int* token_seq, const int* seq_qoff,
                               const int* seq_ntok, const int* seq_slot, void* out, int dtype, int n_tokens, int n_seqs, int D,
                               cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && D > 0 && n_out >= 1, "token_shift: bad sizes");
  LLM_REQUIRE(dtype == LLM_F32 || dtype == LLM_BF16, "token_shift: unknown dtype %d", dtype);
  dim3 grid(ceil_div(D, 256), n_tokens < 65535 ? n_tokens : 65535);
  const int sblocks = ceil_div((long long)n_seqs * D, 256);
  if (dtype == LLM_F32) {
    launch_kernel(token_shift_kernel<float>, grid, 256, 0, stream, (const float*)x, mu, n_out, (const float*)shift_state, token_seq, seq_qoff,
                  seq_slot, (float*)out, n_tokens, D);
    launch_kernel(token_shift_state_kernel<float>, sblocks, 256, 0, stream, (const float*)x, shift_state, seq_qoff, seq_ntok, seq_slot, n_seqs, D);
  } else {
    launch_kernel(token_shift_kernel<bf16>, grid, 256, 0, stream, (const bf16*)x, mu, n_out, (const float*)shift_state, token_seq, seq_qoff,
                  seq_slot, (bf16*)out, n_tokens, D);
    launch_kernel(token_shift_state_kernel<bf16>, sblocks, 256, 0, stream, (const bf16*)x, shift_state, seq_qoff, seq_ntok, seq_slot, n_seqs, D);
  }
  LLM_CHECK_LAUNCH("token_shift");
  return LLM_OK;
}

extern "C" int llm_delta_gates(const float* a, int an, long long as, int aw, int ao, const float* b, int bn, long long bs, int bw, int bo,
                               const float* a_log, const float* dt_bias, float* out, int n_tokens, int H, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && H > 0 && a && b && a_log && dt_bias && out && an >= 1 && bn >= 1, "delta_gates: bad arguments");
  LLM_REQUIRE(ao + H <= aw && bo + H <= bw, "delta_gates: columns outside their rows");
  launch_kernel(delta_gates_kernel, ceil_div((long long)n_tokens * H, 128), 128, 0, stream, Sums{a, an, (size_t)as, aw, ao},
                Sums{b, bn, (size_t)bs, bw, bo}, a_log, dt_bias, out, n_tokens, H);
  LLM_CHECK_LAUNCH("delta_gates");
  return LLM_OK;
}

extern "C" int llm_head_norm_gate(const float* o, const float* weight, int weight_per_head, const float* gate, int gn, long long gs, int gw,
                                  int go, float eps, void* out, int dtype, int n_tokens, int H, int dv, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && H > 0 && dv > 0 && o && weight && out, "head_norm_gate: bad arguments");
  LLM_REQUIRE(gate == nullptr || (gn >= 1 && go >= 0 && go + H * dv <= gw), "head_norm_gate: gate columns outside the product");
  const Sums g{gate, gn, (size_t)gs, gw, go};
  const int blocks = ceil_div((long long)n_tokens * H, 4);
  if (dtype == LLM_F32)
    launch_kernel(head_norm_gate_kernel<float>, blocks, 128, 0, stream, o, weight, weight_per_head, g, eps, (float*)out, n_tokens, H, dv);
  else if (dtype == LLM_BF16)
    launch_kernel(head_norm_gate_kernel<bf16>, blocks, 128, 0, stream, o, weight, weight_per_head, g, eps, (bf16*)out, n_tokens, H, dv);
  else
    LLM_REQUIRE(false, "head_norm_gate: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("head_norm_gate");
  return LLM_OK;
}

extern "C" int llm_rotate_sums(const float* x, int xn, long long xs, int xw, int xo, int heads, int dk, int rot_dims, const float* cos_t,
                               const float* sin_t, const int* positions, float* out, int n_tokens, int scaled_from, float scale,
                               cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && heads > 0 && dk > 0 && x && out && xn >= 1 && xo >= 0 && (long long)xo + (long long)heads * dk <= xw, "rotate_sums: bad arguments");
  LLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || (cos_t && sin_t && positions)), "rotate_sums: %d rotated numbers in a head of %d", rot_dims, dk);
  launch_kernel(rotate_sums_kernel, ceil_div((long long)n_tokens * heads * (dk - rot_dims / 2), 256), 256, 0, stream, Sums{x, xn, (size_t)xs, xw, xo}, heads, dk,
                rot_dims, cos_t, sin_t, positions, out, n_tokens, scaled_from, scale);
  LLM_CHECK_LAUNCH("rotate_sums");
  return LLM_OK;
}
