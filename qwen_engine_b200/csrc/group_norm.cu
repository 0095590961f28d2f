// RMS norm in groups: a row of W channels is cut into `groups` equal consecutive parts, each part is divided by its own
// sqrt(mean(part^2) + eps), and the whole row is multiplied by a weight vector.  Float32 arithmetic throughout.
//
//   qe_group_rmsnorm    out[n] = norm(x[rows ? rows[n] : n]) * w; out float32 or the compute type
//   qe_group_norm_add   for arrangements that norm what a sublayer returns: dst[t] = src[t] + norm(branch[t]) * w on the
//                       float32 stream (src and dst may be the same rows), and, in the same pass, the norm of the new row
//                       for the sublayer that follows: next_out[t] = norm(dst[t]) * w_next (left out with a null pointer)
//
// One CTA per row, the row in shared memory.  A warp takes whole parts in turn (lane-strided sums, then the lanes' sums in
// a fixed order), so a row's bits depend on W and `groups` alone, never on what else is in the step.
#include "common.cuh"
#include <math.h>

#define GN_THREADS 256
#define GN_MAX_GROUPS 1024

template <typename T> struct GnVec4 { T v[4]; };

template <typename T>
__device__ __forceinline__ void gn_load4(const T* p, float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
  }
}
template <typename T>
__device__ __forceinline__ void gn_store4(T* p, const float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a); raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}

// 1 / sqrt(mean + eps) of every part of the row in `row` (shared memory) into `inv`; all threads meet before and after
__device__ __forceinline__ void gn_part_scales(const float* row, float* inv, int W, int groups, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int gs = W / groups;
  __syncthreads();
  for (int g = warp; g < groups; g += warps) {
    const float* part = row + (size_t)g * gs;
    float a0 = 0.f, a1 = 0.f;
    int d = lane;
    for (; d + 32 < gs; d += 64) { a0 = fmaf(part[d], part[d], a0); a1 = fmaf(part[d + 32], part[d + 32], a1); }
    if (d < gs) a0 = fmaf(part[d], part[d], a0);
    const float ss = warp_sum(a0 + a1);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
}

// TB: type of the rows that are normed first (x or branch); TO: type of the norm's output (out or next_out).
// ADD: the add form.  VEC: 16-byte (float32) or 8-byte (bfloat16) pieces when W is a multiple of 4.
template <typename TB, typename TO, bool ADD, bool VEC>
__global__ void __launch_bounds__(GN_THREADS)
group_norm_kernel(const float* __restrict__ src, const TB* __restrict__ x, const int* __restrict__ rows,
                  const float* __restrict__ w, float eps, int groups, int W, float* __restrict__ dst,
                  const float* __restrict__ w_next, TO* __restrict__ out) {
  extern __shared__ __align__(16) float gn_smem[];
  float* row = gn_smem;                          // [W]
  float* inv = gn_smem + ((W + 3) & ~3);         // [groups]
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const size_t at = (size_t)(rows ? rows[n] : n) * W;
  const size_t to = (size_t)n * W;
  const int gs = W / groups;
  if constexpr (VEC) {
    for (int d = threadIdx.x * 4; d < W; d += GN_THREADS * 4) {
      float f[4];
      gn_load4<TB>(x + at + d, f);
      *reinterpret_cast<float4*>(row + d) = make_float4(f[0], f[1], f[2], f[3]);
    }
  } else {
    for (int d = threadIdx.x; d < W; d += GN_THREADS) row[d] = to_f32(x[at + d]);
  }
  gn_part_scales(row, inv, W, groups, eps);
  if constexpr (!ADD) {
    if constexpr (VEC) {
      for (int d = threadIdx.x * 4; d < W; d += GN_THREADS * 4) {
        const float4 wv = *reinterpret_cast<const float4*>(w + d);
        float f[4] = {row[d] * inv[d / gs] * wv.x, row[d + 1] * inv[(d + 1) / gs] * wv.y,
                      row[d + 2] * inv[(d + 2) / gs] * wv.z, row[d + 3] * inv[(d + 3) / gs] * wv.w};
        gn_store4<TO>(out + to + d, f);
      }
    } else {
      for (int d = threadIdx.x; d < W; d += GN_THREADS) out[to + d] = from_f32<TO>(row[d] * inv[d / gs] * w[d]);
    }
    return;
  } else {
    // the add: every thread rewrites the channels it normed, so the row in shared memory becomes the new stream row
    if constexpr (VEC) {
      for (int d = threadIdx.x * 4; d < W; d += GN_THREADS * 4) {
        const float4 wv = *reinterpret_cast<const float4*>(w + d);
        const float4 sv = *reinterpret_cast<const float4*>(src + at + d);
        const float4 r = make_float4(sv.x + row[d] * inv[d / gs] * wv.x, sv.y + row[d + 1] * inv[(d + 1) / gs] * wv.y,
                                     sv.z + row[d + 2] * inv[(d + 2) / gs] * wv.z, sv.w + row[d + 3] * inv[(d + 3) / gs] * wv.w);
        *reinterpret_cast<float4*>(dst + at + d) = r;
        *reinterpret_cast<float4*>(row + d) = r;
      }
    } else {
      for (int d = threadIdx.x; d < W; d += GN_THREADS) {
        const float r = src[at + d] + row[d] * inv[d / gs] * w[d];
        dst[at + d] = r;
        row[d] = r;
      }
    }
    if (out == nullptr) return;
    gn_part_scales(row, inv, W, groups, eps);
    if constexpr (VEC) {
      for (int d = threadIdx.x * 4; d < W; d += GN_THREADS * 4) {
        const float4 wv = *reinterpret_cast<const float4*>(w_next + d);
        float f[4] = {row[d] * inv[d / gs] * wv.x, row[d + 1] * inv[(d + 1) / gs] * wv.y,
                      row[d + 2] * inv[(d + 2) / gs] * wv.z, row[d + 3] * inv[(d + 3) / gs] * wv.w};
        gn_store4<TO>(out + to + d, f);
      }
    } else {
      for (int d = threadIdx.x; d < W; d += GN_THREADS) out[to + d] = from_f32<TO>(row[d] * inv[d / gs] * w_next[d]);
    }
  }
}

// The same for rows whose parts are whole runs of 128 channels (a warp's 16-byte pieces of one turn lie in one part), up to
// 1024 ITER channels: the row stays in registers, every load of a thread is on its way before the first sum, a warp's sum
// of a turn is one partial sum, and a part's partial sums are added in their order.  Two meetings a norm.
template <typename TB, typename TO, bool ADD, int ITER>
__global__ void __launch_bounds__(GN_THREADS)
group_norm_regs_kernel(const float* __restrict__ src, const TB* __restrict__ x, const int* __restrict__ rows,
                       const float* __restrict__ w, float eps, int groups, int W, float* __restrict__ dst,
                       const float* __restrict__ w_next, TO* __restrict__ out) {
  __shared__ float part[ITER * (GN_THREADS / 32)];
  __shared__ float inv[64];                              // (parts of at least 128 of at most 8192 channels)
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t at = (size_t)(rows ? rows[n] : n) * W;
  const size_t to = (size_t)n * W;
  const int gs = W / groups, per = gs >> 7;              // 128-channel runs in a part
  float v[ITER][4];
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    const int d = (i * GN_THREADS + threadIdx.x) * 4;
    if (d < W) gn_load4<TB>(x + at + d, v[i]);
    else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
  }
  auto scales = [&]() {
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
      const float ss = warp_sum(fmaf(v[i][0], v[i][0], v[i][1] * v[i][1]) + fmaf(v[i][2], v[i][2], v[i][3] * v[i][3]));
      if (lane == 0) part[i * (GN_THREADS / 32) + warp] = ss;
    }
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += GN_THREADS) {
      float ss = 0.f;
      for (int p = 0; p < per; ++p) ss += part[g * per + p];
      inv[g] = 1.f / sqrtf(ss / (float)gs + eps);
    }
    __syncthreads();
  };
  scales();
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    const int d = (i * GN_THREADS + threadIdx.x) * 4;
    if (d >= W) continue;
    const float sc = inv[d / gs];
    const float4 wv = *reinterpret_cast<const float4*>(w + d);
    float y[4] = {v[i][0] * sc * wv.x, v[i][1] * sc * wv.y, v[i][2] * sc * wv.z, v[i][3] * sc * wv.w};
    if constexpr (ADD) {
      const float4 sv = *reinterpret_cast<const float4*>(src + at + d);
      v[i][0] = sv.x + y[0]; v[i][1] = sv.y + y[1]; v[i][2] = sv.z + y[2]; v[i][3] = sv.w + y[3];
      *reinterpret_cast<float4*>(dst + at + d) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
    } else {
      gn_store4<TO>(out + to + d, y);
    }
  }
  if constexpr (ADD) {
    if (out == nullptr) return;
    scales();                                             // (every thread has read the first norm's scales: it met the others since)
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
      const int d = (i * GN_THREADS + threadIdx.x) * 4;
      if (d >= W) continue;
      const float sc = inv[d / gs];
      const float4 wv = *reinterpret_cast<const float4*>(w_next + d);
      float y[4] = {v[i][0] * sc * wv.x, v[i][1] * sc * wv.y, v[i][2] * sc * wv.z, v[i][3] * sc * wv.w};
      gn_store4<TO>(out + to + d, y);
    }
  }
}

static int gn_check(const char* who, int W, int groups, size_t* smem) {
  if (groups < 1 || groups > GN_MAX_GROUPS || W < 1 || W % groups) QE_REFUSE("%s: %d channels do not split into %d equal parts", who, W, groups);
  *smem = ((size_t)((W + 3) & ~3) + (size_t)groups) * sizeof(float);
  if (*smem > 200 * 1024) QE_REFUSE("%s: a row of %d channels does not fit shared memory", who, W);
  return 0;
}

template <typename K>
static int gn_configure(K kernel, size_t smem) {
  if (smem <= 48 * 1024) return 0;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e != cudaSuccess) QE_REFUSE("group norm: shared memory: %s", cudaGetErrorString(e));
  return 0;
}

#define GN_REGS(TB, TO, ADD, ...) do { \
    if (W <= 1024) qe_launch(group_norm_regs_kernel<TB, TO, ADD, 1>, dim3(N), dim3(GN_THREADS), 0, stream, __VA_ARGS__); \
    else if (W <= 2048) qe_launch(group_norm_regs_kernel<TB, TO, ADD, 2>, dim3(N), dim3(GN_THREADS), 0, stream, __VA_ARGS__); \
    else if (W <= 4096) qe_launch(group_norm_regs_kernel<TB, TO, ADD, 4>, dim3(N), dim3(GN_THREADS), 0, stream, __VA_ARGS__); \
    else qe_launch(group_norm_regs_kernel<TB, TO, ADD, 8>, dim3(N), dim3(GN_THREADS), 0, stream, __VA_ARGS__); } while (0)
#define GN_LAUNCH(TB, TO, ADD, VEC, ...) do { auto kern_ = group_norm_kernel<TB, TO, ADD, VEC>; \
    if (int rc_ = gn_configure(kern_, smem)) return rc_; \
    qe_launch(kern_, dim3(N), dim3(GN_THREADS), smem, stream, __VA_ARGS__); } while (0)

extern "C" int qe_group_rmsnorm(const void* x, int x_dtype, const int* rows, const float* w, float eps, int groups, void* out,
                                int out_dtype, int N, int W, cudaStream_t stream) {
  if (N <= 0) return 0;
  size_t smem = 0;
  if (int rc = gn_check("group_rmsnorm", W, groups, &smem)) return rc;
  const bool vec = W % 4 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
  const bool regs = vec && W <= 8192 && (W / groups) % 128 == 0;
#define GN_ARGS (const float*)nullptr, (const TB_*)x, rows, w, eps, groups, W, (float*)nullptr, (const float*)nullptr, (TO_*)out
#define GN_PICK(TBT, TOT) do { using TB_ = TBT; using TO_ = TOT; if (regs) GN_REGS(TBT, TOT, false, GN_ARGS); \
    else if (vec) GN_LAUNCH(TBT, TOT, false, true, GN_ARGS); else GN_LAUNCH(TBT, TOT, false, false, GN_ARGS); } while (0)
  if (x_dtype == QE_DTYPE_F32 && out_dtype == QE_DTYPE_F32) GN_PICK(float, float);
  else if (x_dtype == QE_DTYPE_F32 && out_dtype == QE_DTYPE_BF16) GN_PICK(float, __nv_bfloat16);
  else if (x_dtype == QE_DTYPE_BF16 && out_dtype == QE_DTYPE_BF16) GN_PICK(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == QE_DTYPE_BF16 && out_dtype == QE_DTYPE_F32) GN_PICK(__nv_bfloat16, float);
  else QE_REFUSE("group_rmsnorm: unknown dtypes %d, %d", x_dtype, out_dtype);
#undef GN_PICK
#undef GN_ARGS
  QE_CHECK_LAUNCH("group_rmsnorm");
  return 0;
}

extern "C" int qe_group_norm_add(const float* src, const void* branch, int branch_dtype, const float* w, float eps, int groups,
                                 float* dst, const float* w_next, void* next_out, int next_dtype, int N, int W,
                                 cudaStream_t stream) {
  if (N <= 0) return 0;
  size_t smem = 0;
  if (int rc = gn_check("group_norm_add", W, groups, &smem)) return rc;
  if (next_out != nullptr && w_next == nullptr) QE_REFUSE("group_norm_add: the following norm needs its weights");
  if (next_out == nullptr) next_dtype = QE_DTYPE_F32;
  const bool vec = W % 4 == 0 && (((uintptr_t)src | (uintptr_t)branch | (uintptr_t)dst | (uintptr_t)next_out | (uintptr_t)w | (uintptr_t)w_next) & 15) == 0;
  const bool regs = vec && W <= 8192 && (W / groups) % 128 == 0;
#define GN_ARGS src, (const TB_*)branch, (const int*)nullptr, w, eps, groups, W, dst, w_next, (TO_*)next_out
#define GN_PICK(TBT, TOT) do { using TB_ = TBT; using TO_ = TOT; if (regs) GN_REGS(TBT, TOT, true, GN_ARGS); \
    else if (vec) GN_LAUNCH(TBT, TOT, true, true, GN_ARGS); else GN_LAUNCH(TBT, TOT, true, false, GN_ARGS); } while (0)
  if (branch_dtype == QE_DTYPE_F32 && next_dtype == QE_DTYPE_F32) GN_PICK(float, float);
  else if (branch_dtype == QE_DTYPE_F32 && next_dtype == QE_DTYPE_BF16) GN_PICK(float, __nv_bfloat16);
  else if (branch_dtype == QE_DTYPE_BF16 && next_dtype == QE_DTYPE_BF16) GN_PICK(__nv_bfloat16, __nv_bfloat16);
  else if (branch_dtype == QE_DTYPE_BF16 && next_dtype == QE_DTYPE_F32) GN_PICK(__nv_bfloat16, float);
  else QE_REFUSE("group_norm_add: unknown dtypes %d, %d", branch_dtype, next_dtype);
#undef GN_PICK
#undef GN_ARGS
  QE_CHECK_LAUNCH("group_norm_add");
  return 0;
}
