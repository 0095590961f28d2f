// Routed experts: a router that picks `top` of E small feed-forwards per token, and the products over the tokens
// of each expert.
//
//   qe_moe_route       z = W_r h + b in float32 per token; the `top` largest (the lower index wins a tie); weights =
//                      softmax over the chosen logits alone.  Second scoring: s = softmax(z) over all outputs, the `top`
//                      largest of s + correction are chosen, the weights are their s as it is
//   qe_moe_sort        the (token, choice) pairs ordered by expert: offsets[E + 1], the pairs of every expert side by
//                      side, and where each pair went.  One CTA.  Which pair of an expert comes first is not fixed
//                      (atomics); nothing depends on it, since every pair's row is computed alone
//   qe_moe_gate_up     act[p, :] = glu(W_gate_e x_t, W_up_e x_t) for the pair p = (t, e) in sorted order
//   qe_moe_down        y[p, :] = W_down_e act[p, :], float32
//   qe_moe_combine     out[t, :] = sum over the token's choices, in their order, of weight x y[place of the pair]; a choice
//                      at or beyond the experts that have weights stands for an expert that hands its input on: x[t, :]
//
// The grids of the two products are sized for the worst case (every expert's rows end in a tile of their own):
// nothing of a step's shape depends on the routing, so a step can be replayed from a CUDA graph.
#include "tile_product.cuh"
#include <math.h>

#define MOE_MAX_E 1024
#define MOE_MAX_TOP 32

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                 int* __restrict__ top_idx, float* __restrict__ top_w, int T_tokens, int W, int E, int top, int scoring,
                 const float* __restrict__ correction) {
  extern __shared__ float route_smem[];             // the token's row [W], then its logits [E]
  float* xs = route_smem;
  float* z = route_smem + ((W + 3) & ~3);
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * W;
  for (int d = threadIdx.x; d < W; d += blockDim.x) xs[d] = to_f32(xr[d]);
  __syncthreads();
  // a warp per expert in turn; a lane's share of the row in four sums that do not wait for each other, then the lanes' sums
  // in a fixed order: a logit's bits depend on W alone
  for (int e = warp; e < E; e += warps) {
    const float* wr = w + (size_t)e * W;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int d = lane;
    if ((W & 3) == 0 && (((uintptr_t)wr) & 15) == 0) {
      // 16 bytes of the weights a lane and turn, eight turns on their way at a time (a turn alone would wait for memory every time)
      const int W4 = W >> 2;
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 8
      for (int i = lane; i < W4; i += 32) {
        const float4 wv = __ldg(w4 + i), xv = x4[i];
        a0 = fmaf(xv.x, wv.x, a0); a1 = fmaf(xv.y, wv.y, a1); a2 = fmaf(xv.z, wv.z, a2); a3 = fmaf(xv.w, wv.w, a3);
      }
      d = W;
    }
    for (; d + 96 < W; d += 128) {
      a0 = fmaf(xs[d], wr[d], a0);
      a1 = fmaf(xs[d + 32], wr[d + 32], a1);
      a2 = fmaf(xs[d + 64], wr[d + 64], a2);
      a3 = fmaf(xs[d + 96], wr[d + 96], a3);
    }
    for (; d < W; d += 32) a0 = fmaf(xs[d], wr[d], a0);
    const float acc = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) z[e] = acc + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  if (scoring == 1) {
    // scores over all outputs: the largest logit and the sum of the exponentials lane by lane, then over the lanes in a
    // fixed order; the choice looks at score + correction, the weight is the score
    float* sc = z + E;                               // the scores, behind the logits (which become the choice values)
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - m); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) { const float p = sc[e] * inv; sc[e] = p; z[e] = p + (correction ? correction[e] : 0.f); }
    __syncwarp();
    for (int j = 0; j < top; ++j) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int e = lane; e < E; e += 32) { const float v = z[e]; if (v > best) { best = v; at = e; } }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at == 0x7fffffff) at = 0;
      if (lane == 0) { top_idx[(size_t)t * top + j] = at; top_w[(size_t)t * top + j] = sc[at]; z[at] = -INFINITY; }
      __syncwarp();
    }
    return;
  }
  float chosen[MOE_MAX_TOP];
  float zmax = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) { const float v = z[e]; if (v > best) { best = v; at = e; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;                  // (only logits that are not numbers: the row is lost anyway)
    chosen[j] = best;
    if (j == 0) zmax = best;
    if (lane == 0) { top_idx[(size_t)t * top + j] = at; z[at] = -INFINITY; }
    __syncwarp();
  }
  if (scoring == 2) {
    // every expert scored alone: sigmoid(z); the largest logits are the largest scores; the weights are the scores as they are
    if (lane == 0) for (int j = 0; j < top; ++j) top_w[(size_t)t * top + j] = 1.f / (1.f + expf(-chosen[j]));
    return;
  }
  float sum = 0.f;
  for (int j = 0; j < top; ++j) { chosen[j] = expf(chosen[j] - zmax); sum += chosen[j]; }
  if (lane == 0) for (int j = 0; j < top; ++j) top_w[(size_t)t * top + j] = chosen[j] / sum;
}

extern "C" int qe_moe_route(const void* x, const float* w, const float* bias, int* top_idx, float* top_w, int T, int W,
                            int E, int top, int dtype, int scoring, const float* correction, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > MOE_MAX_E || top < 1 || top > MOE_MAX_TOP || top > E) QE_REFUSE("moe_route: %d of %d experts", top, E);
  if (scoring < 0 || scoring > 2) QE_REFUSE("moe_route: unknown scoring %d", scoring);
  const size_t smem = ((size_t)((W + 3) & ~3) + 2 * (size_t)E) * sizeof(float);
  if (smem > 160 * 1024) QE_REFUSE("moe_route: a row of %d channels does not fit shared memory", W);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) QE_REFUSE("moe_route: shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
#define MR(TT) qe_launch(moe_route_kernel<TT>, dim3(T), dim3(128), smem, stream, (const TT*)x, w, bias, top_idx, top_w, T, W, E, top, scoring, correction)
  if (dtype == QE_DTYPE_F32) MR(float);
  else if (dtype == QE_DTYPE_BF16) MR(__nv_bfloat16);
  else QE_REFUSE("moe_route: unknown dtype %d", dtype);
#undef MR
  QE_CHECK_LAUNCH("moe_route");
  return 0;
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ top_idx, int* __restrict__ offsets, int* __restrict__ sorted_pair,
                int* __restrict__ place_of_pair, int P, int E) {
  __shared__ int cnt[MOE_MAX_E + 1];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[top_idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { const int c = cnt[e]; offsets[e] = run; cnt[e] = run; run += c; }
    offsets[E] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int at = atomicAdd(&cnt[top_idx[p]], 1);
    sorted_pair[at] = p;
    place_of_pair[p] = at;
  }
}

extern "C" int qe_moe_sort(const int* top_idx, int* offsets, int* sorted_pair, int* place_of_pair, int P, int E,
                           cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E < 1 || E > MOE_MAX_E) QE_REFUSE("moe_sort: %d experts", E);
  qe_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, top_idx, offsets, sorted_pair, place_of_pair, P, E);
  QE_CHECK_LAUNCH("moe_sort");
  return 0;
}

// the expert and the first sorted place of row tile `tile`: experts' tiles are numbered one expert after the other
__device__ __forceinline__ bool moe_find_tile(const int* __restrict__ offsets, int E, int tile, int BM, int* expert, int* first, int* rows) {
  int seen = 0;
  for (int e = 0; e < E; ++e) {
    const int lo = offsets[e], n = offsets[e + 1] - lo;
    const int tiles = (n + BM - 1) / BM;
    if (tile < seen + tiles) {
      const int i = tile - seen;
      *expert = e; *first = lo + i * BM; *rows = min(BM, n - i * BM);
      return true;
    }
    seen += tiles;
  }
  return false;
}

// the activation of a gated feed-forward on a product's float32 sums, gate and up rounded as if stored
template <typename T>
__device__ __forceinline__ float moe_glu(float v0, float v1, int act) {
  const float g = to_f32(from_f32<T>(v0)), u = to_f32(from_f32<T>(v1));
  if (act > 1) {
    const float lim = __int_as_float(act);
    const float gl = fminf(g, lim), ul = fminf(fmaxf(u, -lim), lim);
    return gl / (1.f + expf(-QE_GLU_SIGMOID_SLOPE * gl)) * (ul + 1.f);
  }
  if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  return g / (1.f + expf(-g)) * u;
}

// GLU = true: w [E, 2 I, K] (gate rows, then up rows), rows gathered from x by pair / top, out [P, I] in the compute type
// GLU = false: w [E, N, K], rows are x[p], out float32 [P, N]
template <typename T, bool GLU>
__global__ void __launch_bounds__(TP_THREADS)
moe_product_kernel(const T* __restrict__ x, const T* __restrict__ w, const int* __restrict__ offsets,
                   const int* __restrict__ sorted_pair, void* __restrict__ out_, int E, int N, int K, int top, int act,
                   const float* __restrict__ pair_w) {
  __shared__ TpSmem<T, GLU ? 2 : 1> sm;
  __shared__ int s_tile[4];
  TpAcc<T, GLU ? 2 : 1> acc;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int e = 0, first = 0, rows = 0;
    const bool ok = moe_find_tile(offsets, E, blockIdx.x, TP_BM, &e, &first, &rows);
    s_tile[0] = ok ? e : -1; s_tile[1] = first; s_tile[2] = rows;
  }
  __syncthreads();
  const int e = s_tile[0], first = s_tile[1], rows = s_tile[2];
  if (e < 0) return;
  const int n0 = blockIdx.y * TP_BN;
  const T* we = w + (size_t)e * (GLU ? 2 : 1) * N * K;
  tile_product<T, GLU ? 2 : 1>(sm, acc, K,
      [&](int r) -> const T* {
        if (r >= rows) return nullptr;
        return GLU ? x + (size_t)(sorted_pair[first + r] / top) * K : x + (size_t)(first + r) * K;
      },
      [&](int m, int n) -> const T* { return n0 + n < N ? we + ((size_t)m * N + n0 + n) * K : nullptr; });
  tile_for_each<T, GLU ? 2 : 1>(acc, [&](int r, int n, float v0, float v1) {
    if (r >= rows || n0 + n >= N) return;
    const size_t at = (size_t)(first + r) * N + n0 + n;
    if constexpr (GLU) {
      // an expert that reads its weight times the token's row: the products are linear, so the weight meets their sums
      const float pw = pair_w ? pair_w[sorted_pair[first + r]] : 1.f;
      const float y = moe_glu<T>(v0 * pw, v1 * pw, act);
      ((T*)out_)[at] = from_f32<T>(y);
    } else {
      ((float*)out_)[at] = v0;
    }
  });
}

// The same two products for bfloat16 rows on 16-byte boundaries, on the pipelined tile of 128 rows (tile_product.cuh).
// K may be cut into gridDim.z shares of k_share channels (GLU = false only): share z adds up its channels alone and writes
// its sums to out + z * P * N; the combining kernel adds the shares in their order.
template <bool GLU>
__global__ void __launch_bounds__(FP_THREADS)
moe_product_fast_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                        const int* __restrict__ sorted_pair, void* __restrict__ out_, int E, int N, int K, int top, int act,
                        int k_share, long share_stride, const float* __restrict__ pair_w) {
  extern __shared__ __align__(16) unsigned char fp_smem[];
  __shared__ int s_tile[4];
  FpAcc acc;
  constexpr int NB = GLU ? 2 : 1;
  constexpr int BN = FpShape<NB>::BN;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int e = 0, first = 0, rows = 0;
    const bool ok = moe_find_tile(offsets, E, blockIdx.x, FP_BM, &e, &first, &rows);
    s_tile[0] = ok ? e : -1; s_tile[1] = first; s_tile[2] = rows;
  }
  __syncthreads();
  const int e = s_tile[0], first = s_tile[1], rows = s_tile[2];
  if (e < 0) return;
  const int n0 = blockIdx.y * BN;
  const int k_first = blockIdx.z * k_share;
  const int k_len = min(k_share, K - k_first);
  const __nv_bfloat16* we = w + (size_t)e * NB * N * K + k_first;
  fast_tile_product<NB>(fp_smem, acc, k_len, w, rows,
      [&](int r) -> const __nv_bfloat16* {
        if (r >= rows) return nullptr;
        return GLU ? x + (size_t)(sorted_pair[first + r] / top) * K : x + (size_t)(first + r) * K + k_first;
      },
      [&](int m, int n) -> const __nv_bfloat16* { return n0 + n < N ? we + ((size_t)m * N + n0 + n) * K : nullptr; });
  fast_tile_for_each<NB>(acc, [&](int r, int n, float v0, float v1) {
    if (r >= rows || n0 + n >= N) return;
    const size_t at = (size_t)(first + r) * N + n0 + n;
    if constexpr (GLU) {
      const float pw = pair_w ? pair_w[sorted_pair[first + r]] : 1.f;
      ((__nv_bfloat16*)out_)[at] = __float2bfloat16_rn(moe_glu<__nv_bfloat16>(v0 * pw, v1 * pw, act));
    }
    else ((float*)out_)[(size_t)blockIdx.z * share_stride + at] = v0;
  });
}

static int moe_tiles(int P, int E, int BM = TP_BM) { return (P + BM - 1) / BM + (E < P ? E : P); }

template <bool GLU>
static int moe_fast_launch(const void* x, const void* w, const int* offsets, const int* sorted_pair, void* out, int P, int E, int N,
                           int K, int top, int act, int shares, cudaStream_t stream, const float* pair_w = nullptr) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_product_fast_kernel<GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM_BYTES);
    if (e != cudaSuccess) QE_REFUSE("moe: shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  constexpr int BN = FpShape<GLU ? 2 : 1>::BN;
  dim3 grid(moe_tiles(P, E, FP_BM), (N + BN - 1) / BN, shares);
  const int k_share = shares > 1 ? ((K + shares - 1) / shares + FP_BK - 1) / FP_BK * FP_BK : K;
  qe_launch(moe_product_fast_kernel<GLU>, grid, dim3(FP_THREADS), FP_SMEM_BYTES, stream, (const __nv_bfloat16*)x,
            (const __nv_bfloat16*)w, offsets, sorted_pair, out, E, N, K, top, act, k_share, (long)P * N, pair_w);
  return 0;
}
static bool moe_fast_applies(const void* x, const void* w, int K, int dtype) {
  return dtype == QE_DTYPE_BF16 && K % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
}

extern "C" int qe_moe_gate_up(const void* x, const void* w, const int* offsets, const int* sorted_pair, void* act_out,
                              int P, int E, int I, int K, int top, int act, int dtype, const float* pair_w, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (moe_fast_applies(x, w, K, dtype)) {
    if (int rc = moe_fast_launch<true>(x, w, offsets, sorted_pair, act_out, P, E, I, K, top, act, 1, stream, pair_w)) return rc;
    QE_CHECK_LAUNCH("moe_gate_up");
    return 0;
  }
  dim3 grid(moe_tiles(P, E), (I + TP_BN - 1) / TP_BN);
#define MP(TT) qe_launch(moe_product_kernel<TT, true>, grid, dim3(TP_THREADS), 0, stream, (const TT*)x, (const TT*)w, offsets, \
                         sorted_pair, act_out, E, I, K, top, act, pair_w)
  if (dtype == QE_DTYPE_F32) MP(float);
  else if (dtype == QE_DTYPE_BF16) MP(__nv_bfloat16);
  else QE_REFUSE("moe_gate_up: unknown dtype %d", dtype);
#undef MP
  QE_CHECK_LAUNCH("moe_gate_up");
  return 0;
}

// In how many shares the down product cuts K: one for steps of many rows; for a few rows (decoded tokens) one per 256
// channels, up to 8, so that enough CTAs pull the weights.  A function of P's class and K alone.
extern "C" int qe_moe_down_shares(int P, int K, int dtype) {
  if (dtype != QE_DTYPE_BF16 || K % 8 || P > 256) return 1;
  const int s = K / 256;
  return s < 1 ? 1 : s > 8 ? 8 : s;
}

// y: float32 [shares, P, N] (shares as qe_moe_down_shares says, or 1), share z holding the sums over its channels
extern "C" int qe_moe_down(const void* act_in, const void* w, const int* offsets, float* y, int P, int E, int N, int K,
                           int shares, int dtype, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (shares < 1 || shares > 8) QE_REFUSE("moe_down: %d shares of K", shares);
  if (moe_fast_applies(act_in, w, K, dtype)) {
    if (int rc = moe_fast_launch<false>(act_in, w, offsets, nullptr, (void*)y, P, E, N, K, 1, 0, shares, stream)) return rc;
    QE_CHECK_LAUNCH("moe_down");
    return 0;
  }
  // (the plain kernel adds up all of K: the other shares are zeros)
  if (shares > 1) cudaMemsetAsync(y + (size_t)P * N, 0, (size_t)(shares - 1) * P * N * sizeof(float), stream);
  dim3 grid(moe_tiles(P, E), (N + TP_BN - 1) / TP_BN);
#define MP(TT) qe_launch(moe_product_kernel<TT, false>, grid, dim3(TP_THREADS), 0, stream, (const TT*)act_in, (const TT*)w, offsets, \
                         (const int*)nullptr, (void*)y, E, N, K, 1, 0, (const float*)nullptr)
  if (dtype == QE_DTYPE_F32) MP(float);
  else if (dtype == QE_DTYPE_BF16) MP(__nv_bfloat16);
  else QE_REFUSE("moe_down: unknown dtype %d", dtype);
#undef MP
  QE_CHECK_LAUNCH("moe_down");
  return 0;
}

template <typename T, typename TX>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place_of_pair,
                                   const float* __restrict__ top_w, T* __restrict__ out, long total, int N, int top,
                                   int shares, long share_stride, const int* __restrict__ top_idx, int E,
                                   const TX* __restrict__ x) {
  pdl_launch_dependents();
  pdl_wait();
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long t = e / N;
    const int n = (int)(e - t * N);
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      float v;
      if (top_idx && top_idx[t * top + j] >= E) {
        v = to_f32(x[e]);                            // an expert that hands its input on
      } else {
        const float* src = y + (size_t)place_of_pair[t * top + j] * N + n;
        v = src[0];
        for (int z = 1; z < shares; ++z) v += src[(size_t)z * share_stride];
      }
      acc = top_w ? fmaf(top_w[t * top + j], v, acc) : acc + v;
    }
    out[e] = from_f32<T>(acc);
  }
}

// top_idx, E, x (null: every choice has weights): choices at or beyond E hand x[t] on (x [T, N] in x_dtype)
extern "C" int qe_moe_combine(const float* y, const int* place_of_pair, const float* top_w, void* out, int T, int N, int top,
                              int shares, int dtype, const int* top_idx, int E, const void* x, int x_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((top_idx != nullptr) != (x != nullptr)) QE_REFUSE("moe_combine: identity experts need the choices and the input");
  const long total = (long)T * N;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define MC(TT, TX) qe_launch(moe_combine_kernel<TT, TX>, dim3(blocks), dim3(256), 0, stream, y, place_of_pair, top_w, (TT*)out, total, N, top, shares, (long)T * top * N, top_idx, E, (const TX*)x)
  if (dtype == QE_DTYPE_F32 && (!x || x_dtype == QE_DTYPE_F32)) MC(float, float);
  else if (dtype == QE_DTYPE_BF16 && (!x || x_dtype == QE_DTYPE_BF16)) MC(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == QE_DTYPE_F32 && x_dtype == QE_DTYPE_BF16) MC(float, __nv_bfloat16);
  else QE_REFUSE("moe_combine: unknown dtypes %d, %d", dtype, x_dtype);
#undef MC
  QE_CHECK_LAUNCH("moe_combine");
  return 0;
}
