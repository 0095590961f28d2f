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
#define SW_TOKENS 32

// out_plain[t, c] = x[t, c]; out_conv[t, c] = x[t, c] + sum_j w[c, j] x[t - (taps - 1) + j, c].  A thread per channel
// walks up to SW_TOKENS tokens of one request with the window in registers.  Rows before the step's first come from the
// request's state (zeros for a request without context).  The CTA of a request's first tokens is the only reader of the
// state and also its writer.
template <typename T>
__global__ void __launch_bounds__(128)
stream_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ state,
                   const int* __restrict__ cu_q, const int* __restrict__ ctx_lens, const int* __restrict__ slot_ids,
                   T* __restrict__ out_plain, T* __restrict__ out_conv, int C, int taps, int write_state) {
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.y;
  float wt[SW_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SW_MAX_TAPS; ++j) wt[j] = (c < C && j < taps) ? w[(size_t)c * taps + j] : 0.f;
  pdl_wait();
  if (c >= C) return;
  const int row0 = cu_q[req], n = cu_q[req + 1] - row0;
  const int t0 = blockIdx.z * SW_TOKENS;
  if (t0 >= n) return;
  const int ctx = ctx_lens[req];
  const int hist = taps - 1;
  float* st = hist > 0 ? state + (size_t)slot_ids[req] * hist * C + c : nullptr;      // [hist][C]: the oldest row first
  auto input = [&](int t) -> float {
    if (t >= 0) return x[(size_t)(row0 + t) * C + c];
    return (ctx > 0 && hist + t >= 0) ? st[(size_t)(hist + t) * C] : 0.f;
  };
  float win[SW_MAX_TAPS];                                          // win[j]: the row taps - 1 - j tokens back
#pragma unroll
  for (int j = 0; j < SW_MAX_TAPS; ++j) win[j] = (j < hist) ? input(t0 - hist + j) : 0.f;
  float old_tail[SW_MAX_TAPS];
  const bool keeper = blockIdx.z == 0 && write_state && hist > 0;
  if (keeper) {
#pragma unroll
    for (int j = 0; j < SW_MAX_TAPS; ++j) old_tail[j] = (j < hist) ? win[j] : 0.f;    // the state as it was (zeros without context)
  }
  const int t1 = min(n, t0 + SW_TOKENS);
  for (int t = t0; t < t1; ++t) {
    const size_t at = (size_t)(row0 + t) * C + c;
    const float cur = x[at];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < SW_MAX_TAPS; ++j) {
      if (j < hist) acc = fmaf(wt[j], win[j], acc);
    }
    acc = fmaf(wt[hist], cur, acc);
    if (out_plain) out_plain[at] = from_f32<T>(cur);
    out_conv[at] = from_f32<T>(cur + acc);
#pragma unroll
    for (int j = 0; j < SW_MAX_TAPS - 1; ++j) win[j] = win[j + 1];
    if (hist > 0) {
#pragma unroll
      for (int j = 0; j < SW_MAX_TAPS; ++j) if (j == hist - 1) win[j] = cur;
    }
  }
  if (keeper) {
    for (int j = 0; j < hist; ++j) {
      const int t = n - hist + j;                                   // the step's row that lands in place j
      float v;
      if (t >= 0) v = x[(size_t)(row0 + t) * C + c];
      else {
        v = 0.f;
#pragma unroll
        for (int i = 0; i < SW_MAX_TAPS; ++i) if (i == hist + t) v = old_tail[i];
      }
      st[(size_t)j * C] = v;
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
  dim3 grid((C + 127) / 128, R, (max_q_len + SW_TOKENS - 1) / SW_TOKENS);
  if (grid.z > 65535) QE_REFUSE("stream_conv: a portion of %d tokens is too long", max_q_len);
#define SCL(TT) qe_launch(stream_conv_kernel<TT>, grid, dim3(128), 0, stream, x, w, state, cu_q, ctx_lens, slot_ids, \
                          (TT*)out_plain, (TT*)out_conv, C, taps, write_state)
  if (dtype == QE_DTYPE_F32) SCL(float);
  else if (dtype == QE_DTYPE_BF16) SCL(__nv_bfloat16);
  else QE_REFUSE("stream_conv: unknown dtype %d", dtype);
#undef SCL
  QE_CHECK_LAUNCH("stream_conv");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// dst[t] = src[t] + v / sqrt(mean(v^2) + eps) * w with v = branch[t] * sigmoid(gate[t] + bias) (gate null: v = branch[t]).
// A CTA per row; the row's v stays in shared memory between the sum and the scaling.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float sw_load(const void* p, int dtype, size_t at) {
  return dtype == QE_DTYPE_F32 ? ((const float*)p)[at] : __bfloat162float(((const __nv_bfloat16*)p)[at]);
}

__global__ void __launch_bounds__(256)
gated_norm_add_kernel(const float* __restrict__ src, const void* __restrict__ branch, int branch_dtype,
                      const void* __restrict__ gate, int gate_dtype, const float* __restrict__ gate_bias,
                      const float* __restrict__ w, float eps, float* __restrict__ dst, void* __restrict__ dst_cast,
                      int cast_dtype, int W) {
  extern __shared__ float sw_row[];                 // [W], then 33 floats for the sum
  float* scratch = sw_row + W;
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    float v = sw_load(branch, branch_dtype, base + d);
    if (gate) {
      const float z = sw_load(gate, gate_dtype, base + d) + (gate_bias ? gate_bias[d] : 0.f);
      v *= 1.f / (1.f + expf(-z));
    }
    sw_row[d] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)W + eps);
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    const float o = src[base + d] + sw_row[d] * rstd * w[d];
    dst[base + d] = o;
    if (dst_cast) {
      if (cast_dtype == QE_DTYPE_F32) ((float*)dst_cast)[base + d] = o;
      else ((__nv_bfloat16*)dst_cast)[base + d] = __float2bfloat16_rn(o);
    }
  }
}

extern "C" int qe_gated_norm_add(const float* src, const void* branch, int branch_dtype, const void* gate, int gate_dtype,
                                 const float* gate_bias, const float* w, float eps, float* dst, void* dst_cast, int cast_dtype,
                                 int T, int W, cudaStream_t stream) {
  if (T <= 0 || W <= 0) return 0;
  const size_t smem = ((size_t)W + 33) * sizeof(float);
  if (smem > 48 * 1024) QE_REFUSE("gated_norm_add: a row of %d channels does not fit shared memory", W);
  const int threads = W >= 1024 ? 256 : W >= 256 ? 128 : 64;
  qe_launch(gated_norm_add_kernel, dim3(T), dim3(threads), smem, stream, src, branch, branch_dtype, gate, gate_dtype, gate_bias, w,
            eps, dst, dst_cast, cast_dtype, W);
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

extern "C" int qe_token_side_gate(const void* gate, const void* table, const int* ids, void* out, int T, int d, int V, int dtype,
                                  cudaStream_t stream) {
  if (T <= 0 || d <= 0) return 0;
  const long total = (long)T * d;
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
