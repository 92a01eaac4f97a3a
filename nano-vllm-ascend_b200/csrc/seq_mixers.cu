// seq_mixers.cu -- the two sequence mixers that the tcgen05 attention kernels do not cover:
//
//   attn_generic       causal softmax attention for ANY head sizes (key size != value size, sizes that are
//                      not 64 or 128), any element type including fp32, packed or paged keys, and any mix of
//                      prompt portions and single tokens in one launch. fp32 scores, softmax and accumulation.
//   linear_recurrence  S_t = a_t S_(t-1) + k_t (b_t v_t)^T, o_t = S_t^T q_t (+ d v_t) per head with the state S
//                      [key size x value size] held in fp32 registers and carried between steps in a slot.
//                      Two forms: a constant decay per head (lightning attention), or a decay and a step size
//                      computed per token from a projected dt (the selective state-space form of Mamba-2).
#include "seq_common.cuh"

namespace b200 {

// ------------------------------------------------------------------ generic attention
// One CTA = 8 warps = 8 "rows" of one (sequence, kv head): row r is query token r / rep, query head
// g * rep + r % rep (rep = H / G), so that the CTA's rows share every key tile. Keys are staged 32 at a
// time in shared memory as fp32; lane j scores key j, then each lane owns value channels lane, lane+32, ...
constexpr int kAttnRows = 8;
constexpr int kAttnKeys = 32;
constexpr int kAttnMaxVChunks = 8;     // value size <= 256

template <typename T>
__global__ void __launch_bounds__(kAttnRows * 32)
attn_generic_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k,
                    int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
                    const int* __restrict__ block_tables, int bt_stride, int block_size,
                    const int* __restrict__ cu_q, const int* __restrict__ cu_k, const int* __restrict__ ctx_lens,
                    int H, int G, int dim, int vdim, float scale) {
  extern __shared__ float smem[];
  pdl_wait();
  const int s = blockIdx.z, g = blockIdx.y;
  const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
  const int rep = H / G;
  const int rows = sp.q_len * rep;
  const int r0 = blockIdx.x * kAttnRows;
  if (r0 >= rows) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = dim + 1;
  float* sq = smem;                                   // [8][dim]
  float* sk = sq + kAttnRows * dim;                   // [32][dim + 1]
  float* sv = sk + kAttnKeys * kpad;                  // [32][vdim]

  const int r = r0 + warp;
  const bool live = r < rows;
  const int tok = live ? r / rep : 0, head = g * rep + (live ? r % rep : 0);
  const int pos = sp.first_pos() + tok;               // this row sees keys 0 .. pos
  if (live) {
    const T* qr = q + (int64_t)(sp.q_start + tok) * q_stride + (int64_t)head * dim;
    for (int i = lane; i < dim; i += 32) sq[warp * dim + i] = to_f32<T>(qr[i]);
  }
  const int last_row = min(r0 + kAttnRows, rows) - 1;
  const int max_pos = sp.first_pos() + last_row / rep;
  const int64_t k_base = cu_k != nullptr && block_tables == nullptr ? cu_k[s] : 0;

  float m = -INFINITY, l = 0.f, acc[kAttnMaxVChunks];
#pragma unroll
  for (int c = 0; c < kAttnMaxVChunks; ++c) acc[c] = 0.f;

  for (int j0 = 0; j0 <= max_pos; j0 += kAttnKeys) {
    __syncthreads();                                  // previous tile fully consumed (and sq written)
    const int nk = min(kAttnKeys, max_pos + 1 - j0);
    for (int e = threadIdx.x; e < nk * dim; e += blockDim.x) {
      const int j = e / dim, i = e - j * dim;
      const int key = j0 + j;
      const int64_t row = block_tables != nullptr
                              ? (int64_t)block_tables[(int64_t)s * bt_stride + key / block_size] * block_size + key % block_size
                              : k_base + key;
      sk[j * kpad + i] = to_f32<T>(k[row * k_stride + (int64_t)g * dim + i]);
    }
    for (int e = threadIdx.x; e < nk * vdim; e += blockDim.x) {
      const int j = e / vdim, i = e - j * vdim;
      const int key = j0 + j;
      const int64_t row = block_tables != nullptr
                              ? (int64_t)block_tables[(int64_t)s * bt_stride + key / block_size] * block_size + key % block_size
                              : k_base + key;
      sv[j * vdim + i] = to_f32<T>(v[row * v_stride + (int64_t)g * vdim + i]);
    }
    __syncthreads();
    if (!live || j0 > pos) continue;
    float sc = -INFINITY;
    if (lane < nk && j0 + lane <= pos) {
      float d = 0.f;
      const float* kr = sk + lane * kpad;
      const float* qr = sq + warp * dim;
      for (int i = 0; i < dim; ++i) d += qr[i] * kr[i];
      sc = d * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float corr = expf(m - m_new);               // m = -inf on the first tile: exp(-inf) = 0
    const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < kAttnMaxVChunks; ++c) acc[c] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int c = 0; c < kAttnMaxVChunks; ++c) {
        const int i = lane + 32 * c;
        if (i < vdim) acc[c] += pj * sv[j * vdim + i];
      }
    }
  }
  if (!live) return;
  T* o = out + (int64_t)(sp.q_start + tok) * ((int64_t)H * vdim) + (int64_t)head * vdim;
  const float inv = 1.0f / l;
#pragma unroll
  for (int c = 0; c < kAttnMaxVChunks; ++c) {
    const int i = lane + 32 * c;
    if (i < vdim) o[i] = from_f32<T>(acc[c] * inv);
  }
}

// ------------------------------------------------------------------ linear recurrence with an fp32 state
// CTA = 128 threads = 32 value columns x 4 key slices of one (sequence, head). Thread (slice ks, column j)
// keeps S[ks + 4 r][j], r < KS, in registers; the 4 slices of a column sit in one warp (lanes l, l+8, l+16,
// l+24), so o_t[j] is two shuffles. Tokens are staged kRecTok at a time in shared memory.
constexpr int kRecTok = 8;
constexpr int kRecCols = 32;

struct RecParams {
  const void *q, *k, *v;            // element type T; q, k: [tokens, groups * kdim]; v: [tokens, H * vdim]
  int64_t q_stride, k_stride, v_stride;
  float* out;                       // [tokens, H * vdim] fp32
  float* state;                     // [slots, H, kdim, vdim] fp32 or nullptr (start from zero, keep nothing)
  const int *state_slots, *cu_q, *cu_k, *ctx_lens;
  int H, groups, kdim, vdim;
  int mode;                         // 0: constant decay per head; 1: selective (dt)
  int act_silu;                     // silu on q, k, v as they are read (mode 0)
  const float* decay;               // mode 0: [H]
  const void* dt;                   // mode 1: [tokens, H] element type T, before bias and softplus
  int64_t dt_stride;
  const float *dt_bias, *a_log, *d_skip;   // mode 1: [H] each
};

template <typename T, int KS>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const RecParams P) {
  extern __shared__ float smem[];
  pdl_wait();
  const int s = blockIdx.z, h = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  if (sp.q_len == 0) return;
  const int kdim = P.kdim, vdim = P.vdim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = lane >> 3, jl = warp * 8 + (lane & 7);
  const int j = blockIdx.x * kRecCols + jl;
  const bool col_ok = j < vdim;
  const int grp = h / (P.H / P.groups);
  float* sq = smem;                                  // [kRecTok][kdim]
  float* skk = sq + kRecTok * kdim;                  // [kRecTok][kdim]
  float* sx = skk + kRecTok * kdim;                  // [kRecTok][kRecCols] values of this CTA's columns
  float* sa = sx + kRecTok * kRecCols;               // [kRecTok] decay of the step
  float* sdt = sa + kRecTok;                         // [kRecTok] step size (1 for a constant decay)

  float S[KS];
  float* slot = P.state != nullptr
                    ? P.state + (((int64_t)P.state_slots[s] * P.H + h) * kdim) * (int64_t)vdim
                    : nullptr;
  const bool carried = slot != nullptr && sp.first_pos() > 0;
#pragma unroll
  for (int r = 0; r < KS; ++r) {
    const int i = ks + 4 * r;
    S[r] = (carried && col_ok && i < kdim) ? slot[(int64_t)i * vdim + j] : 0.f;
  }
  const T* q = (const T*)P.q;
  const T* k = (const T*)P.k;
  const T* v = (const T*)P.v;
  const T* dt = (const T*)P.dt;
  const float a_const = P.mode == 0 ? P.decay[h] : 0.f;
  const float rate = P.mode == 1 ? expf(P.a_log[h]) : 0.f;
  const float dt_b = P.mode == 1 ? P.dt_bias[h] : 0.f;
  const float d_skip = P.mode == 1 ? P.d_skip[h] : 0.f;

  for (int t0 = 0; t0 < sp.q_len; t0 += kRecTok) {
    const int nt = min(kRecTok, sp.q_len - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * kdim; e += blockDim.x) {
      const int tt = e / kdim, i = e - tt * kdim;
      const int64_t tok = sp.q_start + t0 + tt;
      float qv = to_f32<T>(q[tok * P.q_stride + (int64_t)grp * kdim + i]);
      float kv = to_f32<T>(k[tok * P.k_stride + (int64_t)grp * kdim + i]);
      if (P.act_silu) qv = silu_f(qv), kv = silu_f(kv);
      sq[tt * kdim + i] = qv;
      skk[tt * kdim + i] = kv;
    }
    if (threadIdx.x < nt) {
      float a = a_const, step = 1.f;
      if (P.mode == 1) {
        step = softplus_f(to_f32<T>(dt[(int64_t)(sp.q_start + t0 + threadIdx.x) * P.dt_stride + h]) + dt_b);
        a = expf(-rate * step);
      }
      sa[threadIdx.x] = a;
      sdt[threadIdx.x] = step;
    }
    for (int e = threadIdx.x; e < nt * kRecCols; e += blockDim.x) {
      const int tt = e / kRecCols, c = e - tt * kRecCols;
      const int col = blockIdx.x * kRecCols + c;
      float x = 0.f;
      if (col < vdim) x = to_f32<T>(v[(int64_t)(sp.q_start + t0 + tt) * P.v_stride + (int64_t)h * vdim + col]);
      if (P.act_silu) x = silu_f(x);
      sx[tt * kRecCols + c] = x;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float a = sa[tt], vj = sx[tt * kRecCols + jl] * sdt[tt];
      const float* qt = sq + tt * kdim;
      const float* kt = skk + tt * kdim;
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < KS; ++r) {
        const int i = ks + 4 * r;
        if (i < kdim) {
          S[r] = a * S[r] + kt[i] * vj;
          o += S[r] * qt[i];
        }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 8);
      o += __shfl_xor_sync(0xffffffffu, o, 16);
      if (ks == 0 && col_ok) {
        if (P.mode == 1) o += d_skip * sx[tt * kRecCols + jl];
        P.out[(int64_t)(sp.q_start + t0 + tt) * ((int64_t)P.H * vdim) + (int64_t)h * vdim + j] = o;
      }
    }
  }
  if (slot != nullptr && col_ok) {
#pragma unroll
    for (int r = 0; r < KS; ++r) {
      const int i = ks + 4 * r;
      if (i < kdim) slot[(int64_t)i * vdim + j] = S[r];
    }
  }
}

template <typename T>
static int recurrence_launch(const RecParams& P, int num_seqs, cudaStream_t stream) {
  const dim3 grid((P.vdim + kRecCols - 1) / kRecCols, P.H, num_seqs);
  const size_t smem = (size_t)(2 * kRecTok * P.kdim + kRecTok * kRecCols + 2 * kRecTok) * sizeof(float);
  if (P.kdim <= 32) launch_pdl(linear_recurrence_kernel<T, 8>, grid, dim3(128), smem, stream, P);
  else if (P.kdim <= 64) launch_pdl(linear_recurrence_kernel<T, 16>, grid, dim3(128), smem, stream, P);
  else if (P.kdim <= 128) launch_pdl(linear_recurrence_kernel<T, 32>, grid, dim3(128), smem, stream, P);
  else launch_pdl(linear_recurrence_kernel<T, 64>, grid, dim3(128), smem, stream, P);
  return finish_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_generic(void* out, const void* q, int64_t q_stride, const void* k, int64_t k_stride,
                                 const void* v, int64_t v_stride, const int32_t* block_tables,
                                 int32_t bt_stride, int32_t block_size, const int32_t* cu_q,
                                 const int32_t* cu_k, const int32_t* ctx_lens, int32_t num_seqs, int32_t max_q,
                                 int32_t num_heads, int32_t num_kv_heads, int32_t dim, int32_t vdim,
                                 float scale, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || max_q < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 ||
                     num_heads % num_kv_heads != 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(vdim > 32 * kAttnMaxVChunks, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0 || max_q == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || !v || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k),
                 B200_ERR_NULL_POINTER);
  B200_RETURN_IF(block_tables && block_size <= 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(!block_tables && !cu_q, B200_ERR_NULL_POINTER);       // decode rows read the paged cache
  const int rep = num_heads / num_kv_heads;
  const dim3 grid((max_q * rep + kAttnRows - 1) / kAttnRows, num_kv_heads, num_seqs);
  const size_t smem = (size_t)(kAttnRows * dim + kAttnKeys * (dim + 1) + kAttnKeys * vdim) * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  B200_DISPATCH_3(dtype, T, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(attn_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(attn_generic_kernel<T>, grid, dim3(kAttnRows * 32), smem, (cudaStream_t)stream, (T*)out,
               (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, block_tables, bt_stride,
               block_size, cu_q, cu_k, ctx_lens, num_heads, num_kv_heads, dim, vdim, scale);
  });
  return finish_launch();
}

extern "C" int b200_linear_recurrence(float* out, const void* q, int64_t q_stride, const void* k,
                                      int64_t k_stride, const void* v, int64_t v_stride, float* state,
                                      const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                                      const int32_t* ctx_lens, int32_t num_seqs, int32_t num_heads,
                                      int32_t groups, int32_t kdim, int32_t vdim, int32_t mode,
                                      int32_t act_silu, const float* decay, const void* dt, int64_t dt_stride,
                                      const float* dt_bias, const float* a_log, const float* d_skip,
                                      int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || num_heads <= 0 || groups <= 0 || num_heads % groups != 0 || kdim <= 0 ||
                     vdim <= 0 || (mode != 0 && mode != 1), B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(kdim > 256, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || !v || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k) ||
                     (state && !state_slots), B200_ERR_NULL_POINTER);
  B200_RETURN_IF(mode == 0 ? !decay : (!dt || !dt_bias || !a_log || !d_skip), B200_ERR_NULL_POINTER);
  RecParams P;
  P.q = q, P.k = k, P.v = v, P.q_stride = q_stride, P.k_stride = k_stride, P.v_stride = v_stride;
  P.out = out, P.state = state, P.state_slots = state_slots, P.cu_q = cu_q, P.cu_k = cu_k, P.ctx_lens = ctx_lens;
  P.H = num_heads, P.groups = groups, P.kdim = kdim, P.vdim = vdim, P.mode = mode, P.act_silu = act_silu;
  P.decay = decay, P.dt = dt, P.dt_stride = dt_stride, P.dt_bias = dt_bias, P.a_log = a_log, P.d_skip = d_skip;
  B200_DISPATCH_3(dtype, T, return recurrence_launch<T>(P, num_seqs, (cudaStream_t)stream));
  return B200_OK;
}
