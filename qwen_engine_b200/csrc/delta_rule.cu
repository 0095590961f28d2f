// The gated delta rule as a recurrence over tokens, with its state in float32, and the short causal convolution
// in front of it.  Per head, with S: key channels x value channels,
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// (o is read after the token's own update).  A value channel's column of S evolves on its own: thread (j, l) keeps DC
// consecutive key channels of column j in registers, L threads a column within one warp (as the scan of gated linear
// attention).  Per token a column needs k.s and q.s of the decayed column; q.k is the same for all columns, and
// o = q.s + (q.k) u, so the three sums are formed in one pass and reduced together.  The order of every sum depends on
// the sizes alone: a prompt cut anywhere gives the same bits.  g null: one constant decay per head (head_decay) or none.
// hd_in [T, H] (compute type): on top of either, one decay per token and head that the CTA forms itself while it stages
// the token, exp(-exp(hd_rate[h]) softplus(hd_in[t, h] + hd_bias[h])) in float32.
// q, k [T, G dk] (head h reads group h / (H / G)), v [T, H dv], g [T, H dk], beta [T, H]: float32; state float32
// [slot][head][value channel][key channel]; a request without context starts from zero whatever its slot holds.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------------------------------------------------
// y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1) + j, c]): a convolution over the tokens of each request, channel by
// channel; inputs before the step's first token come from the request's state (its last taps - 1 inputs; zeros for a
// request without context), and the state is moved on.  x in the compute type, rows strided; y, w, state float32.
// ---------------------------------------------------------------------------------------------------------
#define SC_MAX_TAPS 16
#define SC_TOKENS 32

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T* __restrict__ x, long ldx, const float* __restrict__ w, float* __restrict__ state,
                  const int* __restrict__ cu_q, const int* __restrict__ ctx_lens, const int* __restrict__ slot_ids,
                  float* __restrict__ y, int C, int taps, int write_state, int silu) {
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.y;
  float wt[SC_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS; ++j) wt[j] = (c < C && j < taps) ? w[(size_t)c * taps + j] : 0.f;
  pdl_wait();
  if (c >= C) return;
  const int row0 = cu_q[req], n = cu_q[req + 1] - row0;
  const int t0 = blockIdx.z * SC_TOKENS;
  if (t0 >= n) return;
  const int ctx = ctx_lens[req];
  const int hist = taps - 1;
  float* st = state + (size_t)slot_ids[req] * hist * C + c;         // [hist][C]: the oldest input first
  // the input `back` tokens before the step's token t (back >= 1)
  auto input = [&](int t) -> float {
    if (t >= 0) return to_f32(x[(size_t)(row0 + t) * ldx + c]);
    return (ctx > 0 && hist + t >= 0) ? st[(size_t)(hist + t) * C] : 0.f;
  };
  float win[SC_MAX_TAPS];                                          // win[j]: the input taps - 1 - j tokens back
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS; ++j) win[j] = (j < hist) ? input(t0 - hist + j) : 0.f;
  float old_tail[SC_MAX_TAPS];
  if (blockIdx.z == 0 && write_state) {
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; ++j) old_tail[j] = (j < hist) ? win[j] : 0.f;    // state as it was (zeros without context)
  }
  const int t1 = min(n, t0 + SC_TOKENS);
  for (int t = t0; t < t1; ++t) {
    const float cur = to_f32(x[(size_t)(row0 + t) * ldx + c]);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; ++j) {
      if (j < hist) acc = fmaf(wt[j], win[j], acc);
    }
    acc = fmaf(wt[hist], cur, acc);
    y[(size_t)(row0 + t) * C + c] = silu ? acc / (1.f + expf(-acc)) : acc;
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS - 1; ++j) win[j] = win[j + 1];
    if (hist > 0) {
#pragma unroll
      for (int j = 0; j < SC_MAX_TAPS; ++j) if (j == hist - 1) win[j] = cur;
    }
  }
  // the CTA of the request's first tokens is the only one that read the state; it also writes it: the last
  // taps - 1 inputs, from this step's rows and, where they are fewer, from the state as it was
  if (blockIdx.z == 0 && write_state) {
    for (int j = 0; j < hist; ++j) {
      const int t = n - hist + j;                                   // the step's token that lands in place j
      float v;
      if (t >= 0) v = to_f32(x[(size_t)(row0 + t) * ldx + c]);
      else {
        v = 0.f;
#pragma unroll
        for (int i = 0; i < SC_MAX_TAPS; ++i) if (i == hist + t) v = old_tail[i];
      }
      st[(size_t)j * C] = v;
    }
  }
}

extern "C" int qe_short_conv(const void* x, long ldx, const float* w, float* state, const int* cu_q, const int* ctx_lens,
                             const int* slot_ids, float* y, int R, int max_q_len, int C, int taps, int write_state,
                             int silu, int dtype, cudaStream_t stream) {
  if (R <= 0 || C <= 0 || max_q_len <= 0) return 0;
  if (taps < 1 || taps > SC_MAX_TAPS) QE_REFUSE("short_conv: %d taps are outside 1..%d", taps, SC_MAX_TAPS);
  if (R > 65535) QE_REFUSE("short_conv: %d requests", R);
  dim3 grid((C + 127) / 128, R, (max_q_len + SC_TOKENS - 1) / SC_TOKENS);
  if (grid.z > 65535) QE_REFUSE("short_conv: a portion of %d tokens is too long", max_q_len);
#define SCL(TT) qe_launch(short_conv_kernel<TT>, grid, dim3(128), 0, stream, (const TT*)x, ldx, w, state, cu_q, ctx_lens, \
                          slot_ids, y, C, taps, write_state, silu)
  if (dtype == QE_DTYPE_F32) SCL(float);
  else if (dtype == QE_DTYPE_BF16) SCL(__nv_bfloat16);
  else QE_REFUSE("short_conv: unknown dtype %d", dtype);
#undef SCL
  QE_CHECK_LAUNCH("short_conv");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// x[t, h, :] <- x[t, h, :] / sqrt(sum x^2 + eps) * scale, float32 in place (rows of ld floats); a warp per (token, head)
// ---------------------------------------------------------------------------------------------------------
__global__ void unit_norm_kernel(float* __restrict__ x, long ld, long items, int H, int D, float eps, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * warps + warp;
  if (item >= items) return;
  const long t = item / H;
  float* r = x + (size_t)t * ld + (size_t)(item - t * H) * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) ss = fmaf(r[d], r[d], ss);
  ss = warp_sum(ss);
  const float f = rsqrtf(ss + eps) * scale;
  for (int d = lane; d < D; d += 32) r[d] *= f;
}

extern "C" int qe_unit_norm(float* x, long ld, int T, int H, int D, float eps, float scale, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  const long items = (long)T * H;
  qe_launch(unit_norm_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, stream, x, ld, items, H, D, eps, scale);
  QE_CHECK_LAUNCH("unit_norm");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// the scan
// ---------------------------------------------------------------------------------------------------------
#define DR_MAX_CHUNK 16        // tokens staged at a time (fewer where a head's rows are long)
#define DR_MAX_THREADS 128

struct DeltaArgs {
  const float* q; const float* k; const float* v; const float* g;   // g may be null
  long ldq, ldk, ldv, ldg;                                          // row strides in floats
  const void* beta; long ld_beta; int beta_dtype;                   // [T, H] before the sigmoid, compute type; null: beta = 1
  const float* head_decay;                                          // with g null: one decay per head, or null for none
  const void* hd_in; long ld_hd; const float* hd_rate; const float* hd_bias;   // a decay per token and head, formed here; null: none
  float* state; const int* cu_q; const int* ctx_lens; const int* slot_ids; float* out;
  int H, G, dk, dv, L, VT, write_state, delta, chunk;
};

__device__ __forceinline__ void dr_cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void dr_cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

template <int DC> __device__ __forceinline__ int dr_pad(int c) { return c + (c / DC) * 4; }

template <int DC, int L>
__global__ void __launch_bounds__(DR_MAX_THREADS)
delta_rule_scan_kernel(DeltaArgs A) {
  extern __shared__ float smem[];
  const int req = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * A.VT;
  const int dk = A.dk, dv = A.dv, VT = A.VT, H = A.H;
  const int grp = head / (H / A.G);
  const int padded = L * DC;
  const int row_w = dr_pad<DC>(padded);                 // floats of a staged row of q, k or g
  const int tok_w = 3 * row_w + ((VT + 3) & ~3) + 4;    // + v of the tile + beta (and padding to 16 bytes)
  float* buf[2] = {smem, smem + (size_t)A.chunk * tok_w};
  const int tid = threadIdx.x;
  const int j = j0 + tid / L, l = tid % L;
  const bool owns = tid < VT * L && j < dv;
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = A.cu_q[req];
  const int n = A.cu_q[req + 1] - row0;
  if (n <= 0) return;
  const int ctx = A.ctx_lens[req];
  float* st = A.state + (((size_t)A.slot_ids[req] * H + head) * dv + (owns ? j : 0)) * dk;
  float s[DC];
#pragma unroll
  for (int i = 0; i < DC; ++i) { const int c = l * DC + i; s[i] = (owns && ctx > 0 && c < dk) ? st[c] : 0.f; }

  const float* q = A.q + (size_t)grp * dk;
  const float* k = A.k + (size_t)grp * dk;
  const float* v = A.v + (size_t)head * dv + j0;
  const float* g = A.g ? A.g + (size_t)head * dk : nullptr;
  const size_t ld_q = A.ldq, ld_k = A.ldk, ld_v = A.ldv, ld_g = A.ldg;
  const float hd = A.head_decay ? A.head_decay[head] : 1.f;
  const bool vec = (dk % 4 == 0) && (dv % 4 == 0) && (VT % 4 == 0) &&
                   ((((uintptr_t)A.q | (uintptr_t)A.k | (uintptr_t)A.v | (uintptr_t)A.g) & 15) == 0) &&
                   ((A.ldq | A.ldk | A.ldv | A.ldg) % 4 == 0);
  const int n_chunks = (n + A.chunk - 1) / A.chunk;

  // channels beyond the head and a constant decay are set once, in both buffers; the copies never touch them
  for (int e = tid; e < 2 * A.chunk * padded; e += blockDim.x) {
    const int t = e / padded, c = e - t * padded;
    float* dst = smem + (size_t)t * tok_w + dr_pad<DC>(c);
    if (c >= dk) { dst[0] = 0.f; dst[row_w] = 0.f; dst[2 * row_w] = 1.f; }
    else if (!g) dst[2 * row_w] = hd;
  }
  // Pieces of 16 bytes sit at the same places in every chunk: a thread works out once which of them are its own (the
  // chunk's row, where from within the row, where to), and a chunk's copies are then a few instructions each.
  constexpr int NP = 16;
  const int pk_ = dk / 4, pv_ = VT / 4;
  const int per_tok_v = (g ? 3 : 2) * pk_ + pv_;
  const bool described = vec && A.chunk * per_tok_v <= NP * (int)blockDim.x;
  int p_meta[NP], p_off[NP];                 // meta: destination (floats from the buffer's start) | kind << 20 | row << 24; -1: none
  if (described) {
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int e = tid + i * blockDim.x;
      p_meta[i] = -1; p_off[i] = 0;
      if (e < A.chunk * per_tok_v) {
        const int t = e / per_tok_v;
        int x = e - t * per_tok_v, kind, dst;
        if (x < pk_) { kind = 0; dst = dr_pad<DC>(x * 4); }
        else if ((x -= pk_) < pk_) { kind = 1; dst = row_w + dr_pad<DC>(x * 4); }
        else if (g && (x -= pk_) < pk_) { kind = 2; dst = 2 * row_w + dr_pad<DC>(x * 4); }
        else { x -= pk_; kind = j0 + x * 4 < dv ? 3 : 4; dst = 3 * row_w + x * 4; }
        if (kind < 4) { p_meta[i] = (t * tok_w + dst) | (kind << 20) | (t << 24); p_off[i] = x * 4; }
      }
    }
  }
  auto stage = [&](int ch) {
    float* b = buf[ch & 1];
    const int t_first = ch * A.chunk;
    const int rows = min(A.chunk, n - t_first);
    if (described) {
      const size_t base_row = (size_t)(row0 + t_first);
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int m = p_meta[i];
        if (m < 0 || (m >> 24) >= rows) continue;
        const int kind = (m >> 20) & 7;
        const size_t row = base_row + (m >> 24);
        const float* src = kind == 0 ? q + row * ld_q : kind == 1 ? k + row * ld_k : kind == 2 ? g + row * ld_g : v + row * ld_v;
        dr_cp_async16(b + (m & 0xfffff), src + p_off[i]);
      }
    } else if (vec) {
      const int pk = dk / 4, pv = VT / 4;
      const int per_tok = (g ? 3 : 2) * pk + pv;
      for (int e = tid; e < rows * per_tok; e += blockDim.x) {
        const int t = e / per_tok;
        int x = e - t * per_tok;
        const size_t row = (size_t)(row0 + t_first + t);
        float* dst = b + (size_t)t * tok_w;
        if (x < pk) dr_cp_async16(dst + dr_pad<DC>(x * 4), q + row * ld_q + x * 4);
        else if ((x -= pk) < pk) dr_cp_async16(dst + row_w + dr_pad<DC>(x * 4), k + row * ld_k + x * 4);
        else if (g && (x -= pk) < pk) dr_cp_async16(dst + 2 * row_w + dr_pad<DC>(x * 4), g + row * ld_g + x * 4);
        else {
          x -= pk;
          const int jj = x * 4;
          if (j0 + jj < dv) dr_cp_async16(dst + 3 * row_w + jj, v + row * ld_v + jj);
        }
      }
    } else {
      const int per_tok = (g ? 3 : 2) * dk + VT;
      for (int e = tid; e < rows * per_tok; e += blockDim.x) {
        const int t = e / per_tok;
        int x = e - t * per_tok;
        const size_t row = (size_t)(row0 + t_first + t);
        float* dst = b + (size_t)t * tok_w;
        if (x < dk) dr_cp_async4(dst + dr_pad<DC>(x), q + row * ld_q + x);
        else if ((x -= dk) < dk) dr_cp_async4(dst + row_w + dr_pad<DC>(x), k + row * ld_k + x);
        else if (g && (x -= dk) < dk) dr_cp_async4(dst + 2 * row_w + dr_pad<DC>(x), g + row * ld_g + x);
        else {
          x -= dk;
          if (j0 + x < dv) dr_cp_async4(dst + 3 * row_w + x, v + row * ld_v + x);
        }
      }
    }
    // beta = sigmoid of the projection's output, in float32
    for (int t = tid; t < rows; t += blockDim.x) {
      float bt = 1.f;
      if (A.beta) {
        const size_t at = (size_t)(row0 + t_first + t) * A.ld_beta + head;
        const float z = A.beta_dtype == QE_DTYPE_F32 ? ((const float*)A.beta)[at] : __bfloat162float(((const __nv_bfloat16*)A.beta)[at]);
        bt = 1.f / (1.f + expf(-z));
      }
      b[(size_t)t * tok_w + 3 * row_w + ((VT + 3) & ~3)] = bt;
      // the token's decay of the whole head (one where the head has none)
      float gd = 1.f;
      if (A.hd_in) {
        const size_t at = (size_t)(row0 + t_first + t) * A.ld_hd + head;
        const float z = (A.beta_dtype == QE_DTYPE_F32 ? ((const float*)A.hd_in)[at] : __bfloat162float(((const __nv_bfloat16*)A.hd_in)[at]))
                        + A.hd_bias[head];
        gd = expf(-expf(A.hd_rate[head]) * (fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)))));
      }
      b[(size_t)t * tok_w + 3 * row_w + ((VT + 3) & ~3) + 1] = gd;
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  __syncthreads();                  // (the constants above are in place before copies land beside them)
  stage(0);
  const size_t o_ld = (size_t)H * dv;
  for (int ch = 0; ch < n_chunks; ++ch) {
    if (ch + 1 < n_chunks) { stage(ch + 1); asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }
    else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    {
      // every thread of the CTA walks the tokens, also those whose column lies beyond the head (they keep zeros and store
      // nothing): the exchanges below are then whole-warp ones, which a warp runs in one go; a column's L lanes are
      // neighbours, so an exchange over distances below L stays within the column
      const int rows = min(A.chunk, n - ch * A.chunk);
      const float* r = buf[ch & 1] + l * (DC + 4);
      const float* rv = buf[ch & 1] + 3 * row_w;
      float* o = A.out + (size_t)(row0 + ch * A.chunk) * o_ld + (size_t)head * dv + j;
      for (int t = 0; t < rows; ++t) {
        float ks0 = 0.f, ks1 = 0.f, qs0 = 0.f, qs1 = 0.f, qk0 = 0.f, qk1 = 0.f;
        const float gd = rv[((VT + 3) & ~3) + 1];          // (times one changes no bit)
#pragma unroll
        for (int i = 0; i < DC; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(r + i);
          const float4 k4 = *reinterpret_cast<const float4*>(r + row_w + i);
          const float4 g4 = *reinterpret_cast<const float4*>(r + 2 * row_w + i);
          s[i] *= g4.x * gd; s[i + 1] *= g4.y * gd; s[i + 2] *= g4.z * gd; s[i + 3] *= g4.w * gd;
          ks0 = fmaf(k4.x, s[i], ks0);     qs0 = fmaf(q4.x, s[i], qs0);     qk0 = fmaf(q4.x, k4.x, qk0);
          ks1 = fmaf(k4.y, s[i + 1], ks1); qs1 = fmaf(q4.y, s[i + 1], qs1); qk1 = fmaf(q4.y, k4.y, qk1);
          ks0 = fmaf(k4.z, s[i + 2], ks0); qs0 = fmaf(q4.z, s[i + 2], qs0); qk0 = fmaf(q4.z, k4.z, qk0);
          ks1 = fmaf(k4.w, s[i + 3], ks1); qs1 = fmaf(q4.w, s[i + 3], qs1); qk1 = fmaf(q4.w, k4.w, qk1);
        }
        float ks = ks0 + ks1, qs = qs0 + qs1, qk = qk0 + qk1;
#pragma unroll
        for (int off = 1; off < L; off <<= 1) {
          ks += __shfl_xor_sync(0xffffffffu, ks, off);
          qs += __shfl_xor_sync(0xffffffffu, qs, off);
          qk += __shfl_xor_sync(0xffffffffu, qk, off);
        }
        const float vj = rv[min(j - j0, VT - 1)];
        const float beta = rv[(VT + 3) & ~3];
        const float u = A.delta ? beta * (vj - ks) : vj;
#pragma unroll
        for (int i = 0; i < DC; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(r + row_w + i);
          s[i] = fmaf(k4.x, u, s[i]); s[i + 1] = fmaf(k4.y, u, s[i + 1]); s[i + 2] = fmaf(k4.z, u, s[i + 2]); s[i + 3] = fmaf(k4.w, u, s[i + 3]);
        }
        if (owns && l == 0) o[(size_t)t * o_ld] = fmaf(qk, u, qs);
        r += tok_w; rv += tok_w;
      }
    }
    __syncthreads();
  }
  if (owns && A.write_state) {
#pragma unroll
    for (int i = 0; i < DC; ++i) { const int c = l * DC + i; if (c < dk) st[c] = s[i]; }
  }
}

// How many threads share a column of the state (a power of two up to 32; 0: the library chooses).  Fewer threads mean
// more key channels a thread (more independent multiply-adds between the exchanges) and fewer exchanges a token.
static int g_dr_lanes = 0;
extern "C" void qe_delta_rule_lanes(int lanes) { g_dr_lanes = lanes; }

extern "C" int qe_delta_rule_scan(const float* q, long ldq, const float* k, long ldk, const float* v, long ldv,
                                  const float* g, long ldg, const void* beta,
                                  long ld_beta, int beta_dtype, const float* head_decay, float* state, const int* cu_q,
                                  const int* ctx_lens, const int* slot_ids, float* out, int R, int H, int G, int dk, int dv,
                                  int write_state, int delta, const void* hd_in, long ld_hd, const float* hd_rate,
                                  const float* hd_bias, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (hd_in && (!hd_rate || !hd_bias)) QE_REFUSE("delta_rule_scan: a decay per token and head needs its rate and bias");
  if (dk < 1 || dk > 1024 || dv < 1) QE_REFUSE("delta_rule_scan: key size %d must be 1..1024, value size %d positive", dk, dv);
  if (H < 1 || H > 65535 || G < 1 || H % G) QE_REFUSE("delta_rule_scan: %d heads over %d key heads", H, G);
  int DC = dk <= 16 ? 4 : dk <= 64 ? 8 : dk <= 128 ? 16 : 32;
  if (g_dr_lanes > 0) {
    const int want = (dk + g_dr_lanes - 1) / g_dr_lanes;
    DC = want <= 4 ? 4 : want <= 8 ? 8 : want <= 16 ? 16 : want <= 32 ? 32 : 64;
  }
  int L = 1;
  while (L * DC < dk) L <<= 1;
  if (L > 32) QE_REFUSE("delta_rule_scan: key size %d is too large", dk);
  DeltaArgs A;
  A.q = q; A.k = k; A.v = v; A.g = g; A.ldq = ldq; A.ldk = ldk; A.ldv = ldv; A.ldg = g ? ldg : 0; A.beta = beta; A.ld_beta = ld_beta; A.beta_dtype = beta_dtype; A.head_decay = head_decay;
  A.hd_in = hd_in; A.ld_hd = ld_hd; A.hd_rate = hd_rate; A.hd_bias = hd_bias;
  A.state = state; A.cu_q = cu_q; A.ctx_lens = ctx_lens; A.slot_ids = slot_ids; A.out = out;
  A.H = H; A.G = G; A.dk = dk; A.dv = dv; A.L = L; A.write_state = write_state; A.delta = delta;
  int VT = DR_MAX_THREADS / L;
  if (VT > dv) VT = dv;
  while (VT > 8 && (long)R * H * ((dv + VT - 1) / VT) < 296 && VT * L > 32) VT = (VT + 1) / 2;
  if (VT % 4) VT = dv % 4 == 0 && VT > 4 ? (VT / 4) * 4 : VT;
  A.VT = VT;
  const int row_w = L * DC + ((L * DC) / DC) * 4;
  const int tok_w = 3 * row_w + ((VT + 3) & ~3) + 4;
  int chunk = DR_MAX_CHUNK;
  while (chunk > 1 && (size_t)2 * chunk * tok_w * sizeof(float) > 200 * 1024) chunk >>= 1;
  A.chunk = chunk;
  const size_t smem = (size_t)2 * A.chunk * tok_w * sizeof(float);
  if (smem > 200 * 1024) QE_REFUSE("delta_rule_scan: key size %d needs %zu bytes of shared memory", dk, smem);
  const int threads = ((VT * L + 31) / 32) * 32;
#define DRL(DCC, LL) do { \
    static bool configured = false; \
    if (!configured) { \
      cudaError_t e = cudaFuncSetAttribute(delta_rule_scan_kernel<DCC, LL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      if (e != cudaSuccess) QE_REFUSE("delta_rule_scan: shared memory: %s", cudaGetErrorString(e)); \
      configured = true; \
    } \
    qe_launch(delta_rule_scan_kernel<DCC, LL>, dim3(R, H, (dv + VT - 1) / VT), dim3(threads), smem, stream, A); } while (0)
#define DRL_L(DCC) do { switch (L) { case 1: DRL(DCC, 1); break; case 2: DRL(DCC, 2); break; case 4: DRL(DCC, 4); break; \
    case 8: DRL(DCC, 8); break; case 16: DRL(DCC, 16); break; default: DRL(DCC, 32); break; } } while (0)
  switch (DC) { case 4: DRL_L(4); break; case 8: DRL_L(8); break; case 16: DRL_L(16); break; case 32: DRL_L(32); break; default: DRL_L(64); break; }
#undef DRL_L
#undef DRL
  QE_CHECK_LAUNCH("delta_rule_scan");
  return 0;
}
