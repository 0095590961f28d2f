// How sublayers are wired to a float32 residual stream in designs that norm a sublayer's result instead of its input:
//
//   qe_stream_conv       what a sublayer reads: the stream's rows, and the rows plus a short causal convolution of them
//                        over the tokens of each request (channel by channel), both rounded once to the compute type;
//                        the last taps - 1 rows of a request are its state
//   qe_gated_norm_add    a sublayer's way back: dst = src + rmsnorm(branch * sigmoid(gate + bias)) * w, one pass over a row
//   qe_token_side_gate   a second embedding's row times gelu_tanh of a gate
//   qe_depth_mix         a weighted sum of the results of all layers so far
//
// Everything is float32 arithmetic; sums over a row run in an order that depends on the row's length alone.
#include "common.cuh"
#include <math.h>

#define SW_MAX_TAPS 16
#define SW_TOKENS 16            // tokens of a request a CTA takes: at least as many as a window holds rows of the past
#define SW_GROUPS 32            // channel groups a CTA takes
#define SW_TPT 4                // consecutive tokens a thread takes (its channels' weights are fetched once for them)

// out_plain[t, c] = x[t, c]; out_conv[t, c] = x[t, c] + sum_j w[c, j] x[t - (taps - 1) + j, c].  A thread takes SW_TPT
// consecutive tokens and CH neighbouring channels (one 16-byte load a row where CH = 4); the rows it shares with its
// neighbours come from L1/L2.  Rows before the step's first come from the request's state (zeros for a request without
// context).  The CTA of a request's first tokens is the only reader of the state and, behind a barrier, also its writer (a
// portion shorter than the window shifts the old rows: they are read before the barrier and written after it).
template <int CH> struct SwVec { float v[CH]; };

template <int CH>
__device__ __forceinline__ SwVec<CH> sw_ld(const float* p) {
  SwVec<CH> r;
  if constexpr (CH == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
  else r.v[0] = p[0];
  return r;
}
template <typename T, int CH>
__device__ __forceinline__ void sw_st(T* p, const SwVec<CH>& a) {
  if constexpr (CH == 4 && sizeof(T) == 2) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.v[0], a.v[1]), hi = __floats2bfloat162_rn(a.v[2], a.v[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else if constexpr (CH == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
  } else {
    p[0] = from_f32<T>(a.v[0]);
  }
}

__device__ __forceinline__ void sw_unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 sw_pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// TAPS 1 to 4: the window's length is known to the compiler, and a thread fetches each of the SW_TPT + TAPS - 1 rows that
// its tokens read once, all of them requested before the first product.  TAPS 0: any length, row by row.  Both add the
// products in the same order, so they agree to the bit.
template <typename T, int CH, int TAPS>
__global__ void __launch_bounds__(SW_TOKENS / SW_TPT * SW_GROUPS)
stream_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ state,
                   const int* __restrict__ cu_q, const int* __restrict__ ctx_lens, const int* __restrict__ slot_ids,
                   T* __restrict__ out_plain, T* __restrict__ out_conv, int C, int taps, int write_state) {
  constexpr int NCH = SW_GROUPS * CH;                 // channels of a CTA
  __shared__ __align__(16) float ws[SW_MAX_TAPS * NCH];   // their weights, tap by tap: ws[j][channel]
  pdl_launch_dependents();
  const int grp = threadIdx.x % SW_GROUPS, quad = threadIdx.x / SW_GROUPS;
  const int c0 = blockIdx.x * NCH;
  const int c = c0 + grp * CH;
  const int req = blockIdx.y;
  const int hist = taps - 1;
  const bool in_c = c < C;
  // the channels' weights depend on nothing a kernel writes: one pass over the CTA's rows of w (they lie side by side)
  {
    const int n_w = min(NCH, C - c0) * taps;
    const float* wsrc = w + (size_t)c0 * taps;
    for (int i = threadIdx.x; i < n_w; i += blockDim.x) ws[(i % taps) * NCH + i / taps] = wsrc[i];
  }
  pdl_wait();
  __syncthreads();
  const int row0 = cu_q[req], n = cu_q[req + 1] - row0;
  if (blockIdx.z * SW_TOKENS >= n) return;            // (the whole CTA)
  const int ctx = ctx_lens[req];
  float* st = (hist > 0 && in_c) ? state + (size_t)slot_ids[req] * hist * C + c : nullptr;      // [hist][C]: the oldest row first
  const float* wmine = ws + grp * CH;
  if constexpr (TAPS > 0) {
    constexpr int HIST = TAPS - 1;
    const int t0 = blockIdx.z * SW_TOKENS + quad * SW_TPT;
    if (in_c && t0 < n) {
      SwVec<CH> r[SW_TPT + HIST];
#pragma unroll
      for (int i = 0; i < SW_TPT + HIST; ++i) {
        const int t = t0 - HIST + i;                  // (a row of the state where negative: HIST + t is its place there)
#pragma unroll
        for (int e = 0; e < CH; ++e) r[i].v[e] = 0.f;
        if (t >= 0) { if (t < n) r[i] = sw_ld<CH>(x + (size_t)(row0 + t) * C + c); }
        else if (ctx > 0) r[i] = sw_ld<CH>(st + (size_t)(HIST + t) * C);
      }
      SwVec<CH> wj[TAPS];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) wj[j] = sw_ld<CH>(wmine + j * NCH);
#pragma unroll
      for (int i = 0; i < SW_TPT; ++i) {
        if (t0 + i >= n) break;
        SwVec<CH> acc;
#pragma unroll
        for (int e = 0; e < CH; ++e) acc.v[e] = 0.f;
#pragma unroll
        for (int j = 0; j < HIST; ++j) {
#pragma unroll
          for (int e = 0; e < CH; ++e) acc.v[e] = fmaf(wj[j].v[e], r[i + j].v[e], acc.v[e]);
        }
        const SwVec<CH>& cur = r[i + HIST];
#pragma unroll
        for (int e = 0; e < CH; ++e) acc.v[e] = cur.v[e] + fmaf(wj[HIST].v[e], cur.v[e], acc.v[e]);
        const size_t at = (size_t)(row0 + t0 + i) * C + c;
        if (out_plain) sw_st<T, CH>(out_plain + at, cur);
        sw_st<T, CH>(out_conv + at, acc);
      }
    }
  } else
#pragma unroll
  for (int i = 0; i < SW_TPT; ++i) {
    const int t = blockIdx.z * SW_TOKENS + quad * SW_TPT + i;
    if (in_c && t < n) {
      SwVec<CH> acc;
#pragma unroll
      for (int e = 0; e < CH; ++e) acc.v[e] = 0.f;
      // taps in the order of time: the oldest row first, the token itself last
#pragma unroll 4
      for (int j = 0; j < hist; ++j) {
        const int back = t - hist + j;
        SwVec<CH> r;
        if (back >= 0) r = sw_ld<CH>(x + (size_t)(row0 + back) * C + c);
        else if (ctx > 0 && hist + back >= 0) r = sw_ld<CH>(st + (size_t)(hist + back) * C);
        else {
#pragma unroll
          for (int e = 0; e < CH; ++e) r.v[e] = 0.f;
        }
        const SwVec<CH> wj = sw_ld<CH>(wmine + j * NCH);
#pragma unroll
        for (int e = 0; e < CH; ++e) acc.v[e] = fmaf(wj.v[e], r.v[e], acc.v[e]);
      }
      const size_t at = (size_t)(row0 + t) * C + c;
      const SwVec<CH> cur = sw_ld<CH>(x + at);
      const SwVec<CH> wl = sw_ld<CH>(wmine + hist * NCH);
#pragma unroll
      for (int e = 0; e < CH; ++e) acc.v[e] = cur.v[e] + fmaf(wl.v[e], cur.v[e], acc.v[e]);
      if (out_plain) sw_st<T, CH>(out_plain + at, cur);
      sw_st<T, CH>(out_conv + at, acc);
    }
  }
  if (blockIdx.z == 0 && write_state && hist > 0) {
    // the last taps - 1 rows: from this step's rows and, where they are fewer, from the state as it was; thread (quad, grp)
    // moves rows quad, quad + 4, ... of the state
    SwVec<CH> v[SW_TPT];
#pragma unroll
    for (int i = 0; i < SW_TPT; ++i) {
      const int j = quad + i * (SW_TOKENS / SW_TPT);
      const int from = n - hist + j;                  // the step's row that lands in place j
#pragma unroll
      for (int e = 0; e < CH; ++e) v[i].v[e] = 0.f;
      if (in_c && j < hist) {
        if (from >= 0) v[i] = sw_ld<CH>(x + (size_t)(row0 + from) * C + c);
        else if (ctx > 0) v[i] = sw_ld<CH>(st + (size_t)(hist + from) * C);
      }
    }
    __syncthreads();                                  // every read of the old rows is done
#pragma unroll
    for (int i = 0; i < SW_TPT; ++i) {
      const int j = quad + i * (SW_TOKENS / SW_TPT);
      if (in_c && j < hist) sw_st<float, CH>(st + (size_t)j * C, v[i]);
    }
  }
}

extern "C" int qe_stream_conv(const float* x, const float* w, float* state, const int* cu_q, const int* ctx_lens,
                              const int* slot_ids, void* out_plain, void* out_conv, int R, int max_q_len, int C, int taps,
                              int write_state, int dtype, cudaStream_t stream) {
  if (R <= 0 || C <= 0 || max_q_len <= 0) return 0;
  if (taps < 1 || taps > SW_MAX_TAPS) QE_REFUSE("stream_conv: %d taps are outside 1..%d", taps, SW_MAX_TAPS);
  if (taps > 1 && !state) QE_REFUSE("stream_conv: %d taps need a state", taps);
  if (R > 65535) QE_REFUSE("stream_conv: %d requests", R);
  const bool vec = C % 4 == 0 && (((uintptr_t)x | (uintptr_t)state | (uintptr_t)out_plain | (uintptr_t)out_conv) & 15) == 0;
  const int per = vec ? 4 : 1;
  dim3 grid(((C + per - 1) / per + SW_GROUPS - 1) / SW_GROUPS, R, (max_q_len + SW_TOKENS - 1) / SW_TOKENS);
  if (grid.z > 65535) QE_REFUSE("stream_conv: a portion of %d tokens is too long", max_q_len);
#define SCK(TT, CH, TP) qe_launch(stream_conv_kernel<TT, CH, TP>, grid, dim3(SW_TOKENS / SW_TPT * SW_GROUPS), 0, stream, x, w, state, \
                                  cu_q, ctx_lens, slot_ids, (TT*)out_plain, (TT*)out_conv, C, taps, write_state)
#define SCL(TT, CH) do { switch (taps) { case 1: SCK(TT, CH, 1); break; case 2: SCK(TT, CH, 2); break; case 3: SCK(TT, CH, 3); break; \
                                         case 4: SCK(TT, CH, 4); break; default: SCK(TT, CH, 0); } } while (0)
  if (dtype == QE_DTYPE_F32) { if (vec) SCL(float, 4); else SCL(float, 1); }
  else if (dtype == QE_DTYPE_BF16) { if (vec) SCL(__nv_bfloat16, 4); else SCL(__nv_bfloat16, 1); }
  else QE_REFUSE("stream_conv: unknown dtype %d", dtype);
#undef SCL
#undef SCK
  QE_CHECK_LAUNCH("stream_conv");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// dst[t] = src[t] + v / sqrt(mean(v^2) + eps) * w with v = branch[t] * sigmoid(gate[t] + bias) (gate null: v = branch[t]).
// A CTA per row; the row's v stays in shared memory between the sum and the scaling.  With `history` (float32
// [count, T, W], dst being its last entry's row) the row also leaves as the weighted sum over the entries,
// mixed[t] = sum_j mix_w[j] history[j][t], in the order of j: the layers' results so far, this one included.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float sw_load(const void* p, int dtype, size_t at) {
  return dtype == QE_DTYPE_F32 ? ((const float*)p)[at] : __bfloat162float(((const __nv_bfloat16*)p)[at]);
}

struct GnaArgs {
  const float* src; const void* branch; int branch_dtype; const void* gate; int gate_dtype; const float* gate_bias;
  const float* w; float eps; float* dst; void* dst_cast; int cast_dtype; int W;
  const float* history; const float* mix_w; int count; long entry_stride; float* mixed;
};

__global__ void __launch_bounds__(256)
gated_norm_add_kernel(GnaArgs A) {
  extern __shared__ float sw_row[];                 // [W], then 33 floats for the sum
  const int W = A.W;
  float* scratch = sw_row + W;
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    float v = sw_load(A.branch, A.branch_dtype, base + d);
    if (A.gate) {
      const float z = sw_load(A.gate, A.gate_dtype, base + d) + (A.gate_bias ? A.gate_bias[d] : 0.f);
      v *= 1.f / (1.f + expf(-z));
    }
    sw_row[d] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)W + A.eps);
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    const float o = A.src[base + d] + sw_row[d] * rstd * A.w[d];
    A.dst[base + d] = o;
    if (A.dst_cast) {
      if (A.cast_dtype == QE_DTYPE_F32) ((float*)A.dst_cast)[base + d] = o;
      else ((__nv_bfloat16*)A.dst_cast)[base + d] = __float2bfloat16_rn(o);
    }
    if (A.history) {
      float acc = 0.f;
      for (int j = 0; j + 1 < A.count; ++j) acc = fmaf(A.mix_w[j], A.history[(size_t)j * A.entry_stride + base + d], acc);
      A.mixed[base + d] = fmaf(A.mix_w[A.count - 1], o, acc);
    }
  }
}

// The same for bfloat16 branch, gate and copy on 8-byte boundaries with W a multiple of 4: four channels a thread and turn,
// ITER turns a thread, everything a turn reads requested before anything is used (the row never leaves the registers).
// PRE: the norm's weights and the gate's bias are fetched before the wait for the kernel ahead (steps of a few rows, where the
// launch chain's gaps count); otherwise they are fetched where they are used, from L1, and the registers they would hold
// while the row's loads are on their way go to more resident CTAs (steps of many rows, where bytes on their way count).
template <int ITER, bool PRE>
__global__ void __launch_bounds__(256)
gated_norm_add_bf16x4_kernel(GnaArgs A) {
  __shared__ float scratch[33];
  const int W4 = A.W >> 2;
  pdl_launch_dependents();
  const float4* w4 = reinterpret_cast<const float4*>(A.w);
  const float4* gb = reinterpret_cast<const float4*>(A.gate_bias);
  float4 ww[PRE ? ITER : 1], bb[PRE ? ITER : 1];
  if constexpr (PRE) {
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      ww[i] = d < W4 ? w4[d] : make_float4(0.f, 0.f, 0.f, 0.f);
      bb[i] = (gb && A.gate && d < W4) ? gb[d] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  const size_t base4 = (size_t)blockIdx.x * W4;
  const uint2* br = reinterpret_cast<const uint2*>(A.branch) + base4;
  const uint2* gt = A.gate ? reinterpret_cast<const uint2*>(A.gate) + base4 : nullptr;
  const float4* src4 = reinterpret_cast<const float4*>(A.src) + base4;
  auto unpack = [](uint2 u) {
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
  };
  uint2 rb[ITER], rg[ITER];
  float4 s4[ITER];
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    rb[i] = make_uint2(0u, 0u); rg[i] = make_uint2(0u, 0u); s4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d < W4) { rb[i] = br[d]; if (gt) rg[i] = gt[d]; s4[i] = src4[d]; }
  }
  float4 v[ITER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    v[i] = unpack(rb[i]);
    if (gt) {
      float4 z = unpack(rg[i]);
      const int d = threadIdx.x + i * blockDim.x;
      const float4 b = PRE ? bb[i] : ((gb && d < W4) ? __ldg(gb + d) : make_float4(0.f, 0.f, 0.f, 0.f));
      z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w;
      // (the gate's logits are bfloat16 roundings: the hardware's exponential and quotient change nothing that counts)
      v[i].x = __fdividef(v[i].x, 1.f + __expf(-z.x)); v[i].y = __fdividef(v[i].y, 1.f + __expf(-z.y));
      v[i].z = __fdividef(v[i].z, 1.f + __expf(-z.z)); v[i].w = __fdividef(v[i].w, 1.f + __expf(-z.w));
    }
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)A.W + A.eps);
  float4* dst4 = reinterpret_cast<float4*>(A.dst) + base4;
  uint2* cast = A.dst_cast ? reinterpret_cast<uint2*>(A.dst_cast) + base4 : nullptr;
  const long stride4 = A.entry_stride >> 2;
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= W4) continue;
    const float4 wv = PRE ? ww[i] : __ldg(w4 + d);
    float4 o;
    o.x = s4[i].x + v[i].x * rstd * wv.x; o.y = s4[i].y + v[i].y * rstd * wv.y;
    o.z = s4[i].z + v[i].z * rstd * wv.z; o.w = s4[i].w + v[i].w * rstd * wv.w;
    dst4[d] = o;
    if (cast) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
      uint2 u;
      u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
      cast[d] = u;
    }
    if (A.history) {
      const float4* h4 = reinterpret_cast<const float4*>(A.history) + base4 + d;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j + 1 < A.count; ++j) {
        const float4 hv = h4[(size_t)j * stride4];
        const float a = A.mix_w[j];
        acc.x = fmaf(a, hv.x, acc.x); acc.y = fmaf(a, hv.y, acc.y); acc.z = fmaf(a, hv.z, acc.z); acc.w = fmaf(a, hv.w, acc.w);
      }
      const float a = A.mix_w[A.count - 1];
      acc.x = fmaf(a, o.x, acc.x); acc.y = fmaf(a, o.y, acc.y); acc.z = fmaf(a, o.z, acc.z); acc.w = fmaf(a, o.w, acc.w);
      reinterpret_cast<float4*>(A.mixed)[base4 + d] = acc;
    }
  }
}

extern "C" int qe_gated_norm_add(const float* src, const void* branch, int branch_dtype, const void* gate, int gate_dtype,
                                 const float* gate_bias, const float* w, float eps, float* dst, void* dst_cast, int cast_dtype,
                                 int T, int W, const float* history, const float* mix_w, int count, float* mixed,
                                 cudaStream_t stream) {
  if (T <= 0 || W <= 0) return 0;
  const size_t smem = ((size_t)W + 33) * sizeof(float);
  if (smem > 48 * 1024) QE_REFUSE("gated_norm_add: a row of %d channels does not fit shared memory", W);
  if (history && (count < 1 || !mix_w || !mixed || dst != history + (size_t)(count - 1) * T * W))
    QE_REFUSE("gated_norm_add: the weighted sum needs its weights, its output and dst as the last of %d entries", count);
  GnaArgs A{src, branch, branch_dtype, gate, gate_dtype, gate_bias, w, eps, dst, dst_cast, cast_dtype, W,
            history, mix_w, count, (long)T * W, mixed};
  const int threads = W >= 1024 ? 256 : W >= 256 ? 128 : 64;
  const uintptr_t all = (uintptr_t)src | (uintptr_t)dst | (uintptr_t)w | (uintptr_t)gate_bias | (uintptr_t)history | (uintptr_t)mixed;
  const uintptr_t half = (uintptr_t)branch | (uintptr_t)gate | (uintptr_t)dst_cast;
  if (W % 4 == 0 && W <= 8192 && branch_dtype == QE_DTYPE_BF16 && (!gate || gate_dtype == QE_DTYPE_BF16) &&
      (!dst_cast || cast_dtype == QE_DTYPE_BF16) && (all & 15) == 0 && (half & 7) == 0) {
    // two turns a thread where the row allows (more loads on their way a thread, fewer threads to meet at the sum)
    const int W4 = W / 4;
    const int vthreads = W4 <= 64 ? 32 : W4 <= 128 ? 64 : W4 <= 512 ? 128 : 256;
    const int iters = (W4 + vthreads - 1) / vthreads;
#define GNA(IT) do { if (T <= 512) qe_launch(gated_norm_add_bf16x4_kernel<IT, true>, dim3(T), dim3(vthreads), 0, stream, A); \
                     else qe_launch(gated_norm_add_bf16x4_kernel<IT, false>, dim3(T), dim3(vthreads), 0, stream, A); } while (0)
    if (iters <= 1) GNA(1);
    else if (iters <= 2) GNA(2);
    else if (iters <= 4) GNA(4);
    else GNA(8);
#undef GNA
  } else
    qe_launch(gated_norm_add_kernel, dim3(T), dim3(threads), smem, stream, A);
  QE_CHECK_LAUNCH("gated_norm_add");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// out[t, j] = gelu_tanh(gate[t, j]) * table[ids[t], j]
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void token_side_gate_kernel(const T* __restrict__ gate, const T* __restrict__ table, const int* __restrict__ ids,
                                       T* __restrict__ out, long total, int d, int V) {
  pdl_launch_dependents();
  pdl_wait();
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long t = e / d;
    const int j = (int)(e - t * d);
    const int id = ids[t];
    const float g = to_f32(gate[e]);
    const float a = 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    const float row = (id >= 0 && id < V) ? to_f32(table[(size_t)id * d + j]) : __int_as_float(0x7fc00000);
    out[e] = from_f32<T>(a * row);
  }
}

// bfloat16 rows whose d is a multiple of 8, on 16-byte boundaries: a 16-byte piece a thread and turn, two turns' loads on
// their way together; gelu_tanh(g) = g sigmoid(2 u) with u = sqrt(2/pi) (g + 0.044715 g^3), by the hardware's exponential
// and quotient (the result is rounded to bfloat16)
__global__ void token_side_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ table,
                                              const int* __restrict__ ids, __nv_bfloat16* __restrict__ out, unsigned total8,
                                              unsigned d8, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned stride = gridDim.x * blockDim.x;
  const uint4* g4 = reinterpret_cast<const uint4*>(gate);
  const uint4* t4 = reinterpret_cast<const uint4*>(table);
  uint4* o4 = reinterpret_cast<uint4*>(out);
  const uint4 nan4 = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
  for (unsigned e0 = blockIdx.x * blockDim.x + threadIdx.x; e0 < total8; e0 += 2 * stride) {
    const unsigned e1 = e0 + stride;
    const bool two = e1 < total8 && e1 > e0;
    const unsigned r0 = e0 / d8, r1 = two ? e1 / d8 : r0;
    const int id0 = __ldg(ids + r0), id1 = __ldg(ids + r1);
    const uint4 rg0 = __ldcg(g4 + e0), rg1 = __ldcg(g4 + (two ? e1 : e0));
    const uint4 rt0 = (id0 >= 0 && id0 < V) ? __ldg(t4 + (size_t)id0 * d8 + (e0 - r0 * d8)) : nan4;
    const uint4 rt1 = (id1 >= 0 && id1 < V) ? __ldg(t4 + (size_t)id1 * d8 + ((two ? e1 : e0) - r1 * d8)) : nan4;
    float g[8], e[8];
    sw_unpack8(rg0, g);
    sw_unpack8(rt0, e);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float u = 0.7978845608028654f * (g[k] + 0.044715f * g[k] * g[k] * g[k]);
      g[k] = __fdividef(g[k], 1.f + __expf(-2.f * u)) * e[k];
    }
    o4[e0] = sw_pack8(g);
    if (two) {
      sw_unpack8(rg1, g);
      sw_unpack8(rt1, e);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float u = 0.7978845608028654f * (g[k] + 0.044715f * g[k] * g[k] * g[k]);
        g[k] = __fdividef(g[k], 1.f + __expf(-2.f * u)) * e[k];
      }
      o4[e1] = sw_pack8(g);
    }
  }
}

extern "C" int qe_token_side_gate(const void* gate, const void* table, const int* ids, void* out, int T, int d, int V, int dtype,
                                  cudaStream_t stream) {
  if (T <= 0 || d <= 0) return 0;
  const long total = (long)T * d;
  if (dtype == QE_DTYPE_BF16 && d % 8 == 0 && total / 8 < (1L << 30) &&
      (((uintptr_t)gate | (uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    const unsigned total8 = (unsigned)(total / 8);
    const unsigned vblocks = (total8 + 255) / 256 < 148 * 8 ? (total8 + 255) / 256 : 148 * 8;
    qe_launch(token_side_gate_bf16x8_kernel, dim3(vblocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate,
              (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, total8, (unsigned)(d / 8), V);
    QE_CHECK_LAUNCH("token_side_gate");
    return 0;
  }
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define TS(TT) qe_launch(token_side_gate_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)gate, (const TT*)table, ids, (TT*)out, total, d, V)
  if (dtype == QE_DTYPE_F32) TS(float);
  else if (dtype == QE_DTYPE_BF16) TS(__nv_bfloat16);
  else QE_REFUSE("token_side_gate: unknown dtype %d", dtype);
#undef TS
  QE_CHECK_LAUNCH("token_side_gate");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// out[e] = sum over j < count, in the order of j, of weights[j] * history[j * total + e]
// ---------------------------------------------------------------------------------------------------------
#define DM_MAX 256
__global__ void depth_mix_kernel(const float* __restrict__ history, const float* __restrict__ weights, int count,
                                 float* __restrict__ out, long total4) {
  __shared__ float wj[DM_MAX];
  pdl_launch_dependents();
  for (int j = threadIdx.x; j < count; j += blockDim.x) wj[j] = weights[j];
  pdl_wait();
  __syncthreads();
  const float4* h4 = reinterpret_cast<const float4*>(history);
  float4* o4 = reinterpret_cast<float4*>(out);
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < count; ++j) {
      const float4 v = h4[(size_t)j * total4 + e];
      const float a = wj[j];
      acc.x = fmaf(a, v.x, acc.x); acc.y = fmaf(a, v.y, acc.y); acc.z = fmaf(a, v.z, acc.z); acc.w = fmaf(a, v.w, acc.w);
    }
    o4[e] = acc;
  }
}

__global__ void depth_mix_scalar_kernel(const float* __restrict__ history, const float* __restrict__ weights, int count,
                                        float* __restrict__ out, long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < count; ++j) acc = fmaf(weights[j], history[(size_t)j * total + e], acc);
    out[e] = acc;
  }
}

extern "C" int qe_depth_mix(const float* history, const float* weights, int count, float* out, long total, cudaStream_t stream) {
  if (total <= 0 || count <= 0) return 0;
  if (count <= DM_MAX && total % 4 == 0 && (((uintptr_t)history | (uintptr_t)out) & 15) == 0) {
    const long total4 = total / 4;
    const unsigned blocks = (unsigned)((total4 + 255) / 256 < 148 * 16 ? (total4 + 255) / 256 : 148 * 16);
    qe_launch(depth_mix_kernel, dim3(blocks), dim3(256), 0, stream, history, weights, count, out, total4);
  } else {
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    qe_launch(depth_mix_scalar_kernel, dim3(blocks), dim3(256), 0, stream, history, weights, count, out, total);
  }
  QE_CHECK_LAUNCH("depth_mix");
  return 0;
}
