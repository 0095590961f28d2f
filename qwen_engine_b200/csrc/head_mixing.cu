// What happens to attention's heads between the weighted sums over the values and the output projection, where a design
// mixes the heads' attention weights or gates every head by one number.
//
// Mixing the weights.  With p_g(i, j) the weight head g puts on key j, a design may replace head h's weights by
// sum_g M[h, g] p_g(i, j) before they meet the values of h's own kv head c(h).  The sum over keys is linear, so
//     out_h(i) = sum_g M[h, g] * O[g, c(h)](i),      O[g, c](i) = sum_j p_g(i, j) v_c(j):
// the attention kernel runs once per shift s = 0 .. Hkv - 1 and gives, for every head g, its weights over the values of
// kv head (c(g) + s) mod Hkv; this kernel then forms the sums over g.  partial [S, T, H D] holds those outputs.
//
// The gate: out_h is multiplied by sigmoid(gate[t, h]), one number per token and head (columns of a wider row).
//
// qe_head_mix_gate: a thread per output element, float32 sums in the order of g, rounded once.  mix null: out = partial[0]
// (S = 1); gate null: no gate.
#include "common.cuh"
#include <math.h>

template <typename T>
__global__ void head_mix_gate_kernel(const T* __restrict__ partial, long shift_stride, const float* __restrict__ mix,
                                     const T* __restrict__ gate, long gate_stride, T* __restrict__ out, long out_stride,
                                     long total, int H, int Hkv, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int G = H / Hkv;
  const long HD = (long)H * D;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long t = e / HD;
    const int hd = (int)(e - t * HD);
    const int h = hd / D, d = hd - h * D;
    float acc;
    if (mix) {
      acc = 0.f;
      const int ch = h / G;
      for (int g = 0; g < H; ++g) {
        int s = ch - g / G;
        if (s < 0) s += Hkv;
        acc = fmaf(mix[h * H + g], to_f32(partial[(size_t)s * shift_stride + (size_t)t * HD + (size_t)g * D + d]), acc);
      }
    } else {
      acc = to_f32(partial[e]);
    }
    if (gate) acc *= 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));
    out[(size_t)t * out_stride + hd] = from_f32<T>(acc);
  }
}

// The same with 16 bytes a thread (8 bfloat16 or 4 float32 channels of one head): for heads whose size is a multiple of
// that, rows on 16-byte boundaries.  The sums over g are formed per channel in the same order as above.
template <typename T, int V>
__global__ void __launch_bounds__(256)
head_mix_gate_vec_kernel(const T* __restrict__ partial, long shift_stride, const float* __restrict__ mix,
                         const T* __restrict__ gate, long gate_stride, T* __restrict__ out, long out_stride,
                         long total_pieces, int H, int Hkv, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int G = H / Hkv;
  const int DP = D / V;                                // pieces in a head
  const long HP = (long)H * DP;
  const long HD = (long)H * D;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total_pieces; e += (long)gridDim.x * blockDim.x) {
    const long t = e / HP;
    const int hp = (int)(e - t * HP);
    const int h = hp / DP, d = (hp - h * DP) * V;
    float acc[V];
    auto load = [&](const T* p, float (&f)[V]) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p);
      if constexpr (sizeof(T) == 4) {
        f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
      } else {
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r[i]);
          f[2 * i] = __low2float(b); f[2 * i + 1] = __high2float(b);
        }
      }
    };
    if (mix) {
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      const int ch = h / G;
      const float* mrow = mix + (size_t)h * H;
#pragma unroll 4
      for (int g = 0; g < H; ++g) {
        int s = ch - g / G;
        if (s < 0) s += Hkv;
        float f[V];
        load(partial + (size_t)s * shift_stride + (size_t)t * HD + (size_t)g * D + d, f);
        const float m = mrow[g];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(m, f[i], acc[i]);
      }
    } else {
      load(partial + (size_t)t * HD + (size_t)h * D + d, acc);
    }
    if (gate) {
      const float gt = 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] *= gt;
    }
    uint4 o;
    if constexpr (sizeof(T) == 4) {
      o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
    } else {
      uint32_t r[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        r[i] = *reinterpret_cast<uint32_t*>(&b);
      }
      o = make_uint4(r[0], r[1], r[2], r[3]);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + (size_t)h * D + d) = o;
  }
}

extern "C" int qe_head_mix_gate(const void* partial, long shift_stride, int shifts, const float* mix, const void* gate,
                                long gate_stride, void* out, long out_stride, int T, int H, int Hkv, int D, int dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Hkv < 1 || H % Hkv) QE_REFUSE("head_mix_gate: %d heads do not group over %d kv heads", H, Hkv);
  if (mix != nullptr && shifts != Hkv) QE_REFUSE("head_mix_gate: mixing the heads needs one set of outputs per kv head (%d), got %d", Hkv, shifts);
  const int V = dtype == QE_DTYPE_BF16 ? 8 : 4;
  const size_t esz = dtype == QE_DTYPE_BF16 ? 2 : 4;
  if ((dtype == QE_DTYPE_BF16 || dtype == QE_DTYPE_F32) && D % V == 0 && (((uintptr_t)partial | (uintptr_t)out) & 15) == 0 &&
      (out_stride * esz) % 16 == 0 && (shift_stride * esz) % 16 == 0) {
    const long pieces = (long)T * H * (D / V);
    const unsigned vblocks = (unsigned)((pieces + 255) / 256 < 148 * 16 ? (pieces + 255) / 256 : 148 * 16);
#define HMV(TT, VV) qe_launch(head_mix_gate_vec_kernel<TT, VV>, dim3(vblocks), dim3(256), 0, stream, (const TT*)partial, shift_stride, mix, \
                              (const TT*)gate, gate_stride, (TT*)out, out_stride, pieces, H, Hkv, D)
    if (dtype == QE_DTYPE_BF16) HMV(__nv_bfloat16, 8); else HMV(float, 4);
#undef HMV
    QE_CHECK_LAUNCH("head_mix_gate");
    return 0;
  }
  const long total = (long)T * H * D;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define HM(TT) qe_launch(head_mix_gate_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)partial, shift_stride, mix, \
                         (const TT*)gate, gate_stride, (TT*)out, out_stride, total, H, Hkv, D)
  if (dtype == QE_DTYPE_F32) HM(float);
  else if (dtype == QE_DTYPE_BF16) HM(__nv_bfloat16);
  else QE_REFUSE("head_mix_gate: unknown dtype %d", dtype);
#undef HM
  QE_CHECK_LAUNCH("head_mix_gate");
  return 0;
}
