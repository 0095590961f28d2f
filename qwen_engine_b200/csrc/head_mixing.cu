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

extern "C" int qe_head_mix_gate(const void* partial, long shift_stride, int shifts, const float* mix, const void* gate,
                                long gate_stride, void* out, long out_stride, int T, int H, int Hkv, int D, int dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Hkv < 1 || H % Hkv) QE_REFUSE("head_mix_gate: %d heads do not group over %d kv heads", H, Hkv);
  if (mix != nullptr && shifts != Hkv) QE_REFUSE("head_mix_gate: mixing the heads needs one set of outputs per kv head (%d), got %d", Hkv, shifts);
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
