// delta_rule.cu -- gated delta rule with one decay per head and key channel, state in fp32:
//
//   S <- diag(g_t) S;   w = beta_t (v_t - S^T k_t);   S <- S + k_t w^T;   o_t = S^T q_t          S [kdim x vdim] per head
//
// (the read-out sees the current token's write). q, k (unit vectors, per key/value group), g (per head and key
// channel) and beta arrive in fp32 from delta_prep; v in the model's element type. The state is carried between
// steps in a slot, exactly as the other recurrences: [slots, H, kdim, vdim] fp32; a span that starts at position 0
// ignores what the slot held.
//
// One CTA = 128 threads = one (sequence, head) and a band of value columns. A thread owns ONE value column and
// KPT <= 64 key rows of S in registers (NS = 1, 2 or 4 adjacent lanes share a column when kdim > 64). Per token it
// makes two passes over its rows -- decay + the projection S^T k, then the rank-one write + the read-out S^T q --
// with k, q, g read as float4 broadcasts from shared memory; the two dot products are finished with NS - 1
// shuffles. Tokens are staged kDeltaTok at a time; where the rows allow 16-byte copies (VEC) the next batch arrives by
// cp.async in a second set of buffers while the current one is consumed, otherwise batches are loaded in place.
#include "seq_common.cuh"

namespace b200 {

constexpr int kDeltaTok = 8;

struct DeltaParams {
  const float *q, *k;               // [tokens, groups * kdim]
  const float* g;                   // [tokens, H * kdim]
  const float* beta;                // [tokens, H]
  const void* v;                    // [tokens, H * vdim], element type
  int64_t q_stride, k_stride, v_stride;
  float* out;                       // [tokens, H * vdim] fp32
  float* state;                     // [slots, H, kdim, vdim] fp32 or nullptr
  const int *state_slots, *cu_q, *cu_k, *ctx_lens;
  int H, groups, kdim, vdim;
};

__device__ __forceinline__ void cp_async_4(uint32_t smem_addr, const void* gptr, bool pred) {
  const int bytes = pred ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_addr), "l"(gptr), "r"(bytes) : "memory");
}

template <typename TV, int KPT, int NS, bool VEC>
__global__ void __launch_bounds__(128)
delta_rule_kernel(const DeltaParams P) {
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  constexpr int KP = NS * KPT;                       // padded key rows
  constexpr int CC = 128 / NS;                       // value columns per CTA
  const int s = blockIdx.z, h = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  if (sp.q_len == 0) return;
  const int kdim = P.kdim, vdim = P.vdim;
  const int ksl = threadIdx.x % NS, cl = threadIdx.x / NS;
  const int c0 = blockIdx.x * CC, col = c0 + cl;
  const bool col_ok = col < vdim;
  const bool warp_live = c0 + (int)((threadIdx.x & ~31u) / NS) < vdim;
  const int grp = h / (P.H / P.groups);
  constexpr int NB = VEC ? 2 : 1;                    // sets of staging buffers
  constexpr int QK = kDeltaTok * KP;
  float* sq = smem;                                  // [NB][kDeltaTok][KP]
  float* sk = sq + NB * QK;
  float* sg = sk + NB * QK;
  float* sb = sg + NB * QK;                          // [NB][kDeltaTok]
  float* sx = sb + NB * kDeltaTok;                   // [kDeltaTok][CC] fp32 (in-place form)
  TV* sxr = reinterpret_cast<TV*>(sb + NB * kDeltaTok);   // [2][kDeltaTok][CC] as stored (cp.async form)

  float S[KPT];
  float* slot = P.state != nullptr
                    ? P.state + (((int64_t)P.state_slots[s] * P.H + h) * kdim) * (int64_t)vdim
                    : nullptr;
  const bool carried = slot != nullptr && sp.first_pos() > 0;
#pragma unroll
  for (int r = 0; r < KPT; ++r) {
    const int i = ksl * KPT + r;
    S[r] = (carried && col_ok && i < kdim) ? slot[(int64_t)i * vdim + col] : 0.f;
  }
  const float* q = P.q + (int64_t)grp * kdim;
  const float* k = P.k + (int64_t)grp * kdim;
  const float* g = P.g + (int64_t)h * kdim;
  const TV* v = (const TV*)P.v + (int64_t)h * vdim + c0;
  const int vcols = min(CC, vdim - c0);
  const int64_t g_stride = (int64_t)P.H * kdim;

  auto issue = [&](int t0, int b) {                  // cp.async form: batch t0 into buffer set b (zero-filled padding)
    const int nt = min(kDeltaTok, sp.q_len - t0);
    const int64_t tok0 = sp.q_start + t0;
    constexpr int K4 = KP / 4, VE = 16 / (int)sizeof(TV);
    for (int e = threadIdx.x; e < kDeltaTok * K4; e += 128) {
      const int tt = e / K4, i = (e % K4) * 4;
      const bool ok = tt < nt && i < kdim;
      const int64_t tok = tok0 + (tt < nt ? tt : 0);
      const int ii = ok ? i : 0;
      cp_async_16(smem_u32(sq + b * QK + tt * KP + i), q + tok * P.q_stride + ii, ok);
      cp_async_16(smem_u32(sk + b * QK + tt * KP + i), k + tok * P.k_stride + ii, ok);
      cp_async_16(smem_u32(sg + b * QK + tt * KP + i), g + tok * g_stride + ii, ok);
    }
    for (int e = threadIdx.x; e < kDeltaTok * CC / VE; e += 128) {
      const int tt = e / (CC / VE), c = (e % (CC / VE)) * VE;
      const bool ok = tt < nt && c < vcols;
      cp_async_16(smem_u32(sxr + (b * kDeltaTok + tt) * CC + c), v + (tok0 + (tt < nt ? tt : 0)) * P.v_stride + (ok ? c : 0), ok);
    }
    if (threadIdx.x < kDeltaTok) {
      const bool ok = (int)threadIdx.x < nt;
      cp_async_4(smem_u32(sb + b * kDeltaTok + threadIdx.x), P.beta + (tok0 + (ok ? threadIdx.x : 0)) * P.H + h, ok);
    }
    cp_async_commit();
  };
  if (VEC) issue(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < sp.q_len; t0 += kDeltaTok, b ^= (VEC ? 1 : 0)) {
    const int nt = min(kDeltaTok, sp.q_len - t0);
    const int64_t tok0 = sp.q_start + t0;
    if (VEC) {
      cp_async_wait<0>();
      __syncthreads();                               // batch b has landed everywhere; set b ^ 1 has been consumed
      if (t0 + kDeltaTok < sp.q_len) issue(t0 + kDeltaTok, b ^ 1);
    } else {
      __syncthreads();                               // the previous batch has been consumed
      for (int e = threadIdx.x; e < kDeltaTok * KP; e += 128) {
        const int tt = e / KP, i = e % KP;
        const bool ok = tt < nt && i < kdim;
        sq[e] = ok ? q[(tok0 + tt) * P.q_stride + i] : 0.f;
        sk[e] = ok ? k[(tok0 + tt) * P.k_stride + i] : 0.f;
        sg[e] = ok ? g[(tok0 + tt) * g_stride + i] : 0.f;
      }
      for (int e = threadIdx.x; e < kDeltaTok * CC; e += 128) {
        const int tt = e / CC, c = e % CC;
        sx[e] = (tt < nt && c < vcols) ? to_f32<TV>(v[(tok0 + tt) * P.v_stride + c]) : 0.f;
      }
      if (threadIdx.x < kDeltaTok) sb[threadIdx.x] = threadIdx.x < nt ? P.beta[(tok0 + threadIdx.x) * P.H + h] : 0.f;
      __syncthreads();
    }
    if (!warp_live) continue;
    float* outp = P.out + tok0 * ((int64_t)P.H * vdim) + (int64_t)h * vdim + col;
    for (int tt = 0; tt < nt; ++tt) {
      const float4* q4 = reinterpret_cast<const float4*>(sq + b * QK + tt * KP + ksl * KPT);
      const float4* k4 = reinterpret_cast<const float4*>(sk + b * QK + tt * KP + ksl * KPT);
      const float4* g4 = reinterpret_cast<const float4*>(sg + b * QK + tt * KP + ksl * KPT);
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < KPT / 4; ++r4) {
        const float4 gg = g4[r4], kk = k4[r4];
        S[r4 * 4 + 0] *= gg.x;
        d0 += S[r4 * 4 + 0] * kk.x;
        S[r4 * 4 + 1] *= gg.y;
        d1 += S[r4 * 4 + 1] * kk.y;
        S[r4 * 4 + 2] *= gg.z;
        d2 += S[r4 * 4 + 2] * kk.z;
        S[r4 * 4 + 3] *= gg.w;
        d3 += S[r4 * 4 + 3] * kk.w;
      }
      float d = (d0 + d1) + (d2 + d3);
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
      const float x = VEC ? to_f32<TV>(sxr[(b * kDeltaTok + tt) * CC + cl]) : sx[tt * CC + cl];
      const float w = sb[b * kDeltaTok + tt] * (x - d);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < KPT / 4; ++r4) {
        const float4 kk = k4[r4], qq = q4[r4];
        S[r4 * 4 + 0] += kk.x * w;
        o0 += S[r4 * 4 + 0] * qq.x;
        S[r4 * 4 + 1] += kk.y * w;
        o1 += S[r4 * 4 + 1] * qq.y;
        S[r4 * 4 + 2] += kk.z * w;
        o2 += S[r4 * 4 + 2] * qq.z;
        S[r4 * 4 + 3] += kk.w * w;
        o3 += S[r4 * 4 + 3] * qq.w;
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (ksl == 0 && col_ok) outp[(int64_t)tt * ((int64_t)P.H * vdim)] = o;
    }
  }
  if (slot != nullptr && col_ok) {
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
      const int i = ksl * KPT + r;
      if (i < kdim) slot[(int64_t)i * vdim + col] = S[r];
    }
  }
}

template <typename TV, int KPT, int NS>
static void delta_launch_as(const DeltaParams& P, int num_seqs, cudaStream_t stream) {
  constexpr int CC = 128 / NS;
  constexpr int VE = 16 / (int)sizeof(TV);
  const dim3 grid((P.vdim + CC - 1) / CC, P.H, num_seqs);
  const bool vec = P.kdim % 4 == 0 && P.q_stride % 4 == 0 && P.k_stride % 4 == 0 && aligned16(P.q) && aligned16(P.k) &&
                   aligned16(P.g) && P.vdim % VE == 0 && P.v_stride % VE == 0 && aligned16(P.v);
  if (vec) {
    const size_t smem = (size_t)2 * (3 * kDeltaTok * NS * KPT + kDeltaTok) * sizeof(float) +
                        (size_t)2 * kDeltaTok * CC * sizeof(TV);
    static bool configured = false;                   // one flag per instantiation
    if (!configured && smem > 48 * 1024) {
      cudaFuncSetAttribute(delta_rule_kernel<TV, KPT, NS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      configured = true;
    }
    launch_pdl(delta_rule_kernel<TV, KPT, NS, true>, grid, dim3(128), smem, stream, P);
  } else {
    const size_t smem = (size_t)(3 * kDeltaTok * NS * KPT + kDeltaTok + kDeltaTok * CC) * sizeof(float);
    launch_pdl(delta_rule_kernel<TV, KPT, NS, false>, grid, dim3(128), smem, stream, P);
  }
}

template <typename TV>
static int delta_launch(const DeltaParams& P, int num_seqs, cudaStream_t stream) {
  // 64 rows per thread wherever the key size allows: 32 rows on twice the lanes measured 3.6x slower at key size 128
  // (the lanes of a column then read four different slices of k, q, g per token instead of two)
  if (P.kdim <= 16) delta_launch_as<TV, 16, 1>(P, num_seqs, stream);
  else if (P.kdim <= 32) delta_launch_as<TV, 32, 1>(P, num_seqs, stream);
  else if (P.kdim <= 64) delta_launch_as<TV, 64, 1>(P, num_seqs, stream);
  else if (P.kdim <= 128) delta_launch_as<TV, 64, 2>(P, num_seqs, stream);
  else delta_launch_as<TV, 64, 4>(P, num_seqs, stream);
  return finish_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_delta_rule(float* out, const float* q, int64_t q_stride, const float* k, int64_t k_stride,
                               const void* v, int64_t v_stride, const float* g, const float* beta, float* state,
                               const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                               const int32_t* ctx_lens, int32_t num_seqs, int32_t num_heads, int32_t groups,
                               int32_t kdim, int32_t vdim, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || num_heads <= 0 || groups <= 0 || num_heads % groups != 0 || kdim <= 0 || vdim <= 0,
                 B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(kdim > 256, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || !v || !g || !beta || (cu_q == nullptr) == (ctx_lens == nullptr) ||
                     (cu_q && !cu_k) || (state && !state_slots), B200_ERR_NULL_POINTER);
  DeltaParams P;
  P.q = q, P.k = k, P.g = g, P.beta = beta, P.v = v, P.q_stride = q_stride, P.k_stride = k_stride;
  P.v_stride = v_stride, P.out = out, P.state = state, P.state_slots = state_slots, P.cu_q = cu_q, P.cu_k = cu_k;
  P.ctx_lens = ctx_lens, P.H = num_heads, P.groups = groups, P.kdim = kdim, P.vdim = vdim;
  B200_DISPATCH_3(dtype, TV, return delta_launch<TV>(P, num_seqs, (cudaStream_t)stream));
  return B200_OK;
}
