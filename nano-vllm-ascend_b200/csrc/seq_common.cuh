// seq_common.cuh -- helpers shared by the sequence-mixer kernels (seq_ops.cu, seq_mixers.cu).
//
// These kernels take three element types: bf16, fp16 and fp32 (B200_DTYPE_F32: every tensor in true
// 32-bit, the exact mode of the hybrid models). Small parameters (norm weights, convolution taps, decays,
// step-size biases) are always fp32.
#pragma once
#include "common.cuh"

namespace b200 {

template <>
__device__ __forceinline__ float to_f32<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
  return x;
}

// How the tokens of a step map to sequences. Two forms, as the runner publishes them:
//   varlen  (cu_q != nullptr): sequence s owns tokens [cu_q[s], cu_q[s+1]) of the packed batch and sees
//           cu_k[s+1] - cu_k[s] keys in all (the tokens of earlier steps come first);
//   decode  (cu_q == nullptr): sequence s owns token s and sees ctx_lens[s] keys; ctx_lens[s] == 0 marks a
//           padded row of a captured graph, which computes nothing and writes nothing.
struct SeqSpan {
  int q_start, q_len, k_len;
  __device__ __forceinline__ int first_pos() const { return k_len - q_len; }
};
__device__ __forceinline__ SeqSpan seq_span(const int* cu_q, const int* cu_k, const int* ctx_lens, int s) {
  SeqSpan r;
  if (cu_q != nullptr) {
    r.q_start = cu_q[s];
    r.q_len = cu_q[s + 1] - r.q_start;
    r.k_len = cu_k[s + 1] - cu_k[s];
  } else {
    r.k_len = ctx_lens[s];
    r.q_start = s;
    r.q_len = r.k_len > 0 ? 1 : 0;
  }
  return r;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
// log(1 + e^x) without overflow: the same function as the naive form wherever that one is finite
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

// sum over the CTA; `red` holds 32 floats. Every thread gets the total.
__device__ __forceinline__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (nw == 1) return v;
  __syncthreads();          // `red` may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

// 8 consecutive elements <-> fp32 registers (16 bytes of a 16-bit type, 32 bytes of fp32); p 16-byte aligned
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack2<T>(w[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack2<T>(f[0], f[1]), u.y = pack2<T>(f[2], f[3]), u.z = pack2<T>(f[4], f[5]), u.w = pack2<T>(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

#define B200_DISPATCH_3(dtype, T, ...)                    \
  do {                                                    \
    if ((dtype) == B200_DTYPE_BF16) {                     \
      using T = __nv_bfloat16;                            \
      __VA_ARGS__;                                        \
    } else if ((dtype) == B200_DTYPE_F16) {               \
      using T = __half;                                   \
      __VA_ARGS__;                                        \
    } else if ((dtype) == B200_DTYPE_F32) {               \
      using T = float;                                    \
      __VA_ARGS__;                                        \
    } else {                                              \
      return B200_ERR_BAD_DTYPE;                          \
    }                                                     \
  } while (0)

}  // namespace b200
