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
