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
// One CTA = 128 threads works on one (sequence, head) and a band of value columns. A thread owns ONE value column
// and KPT <= 64 key rows of the state in registers (all rows when kdim <= 64; 2 or 4 adjacent lanes share a column
// above that, one or two shuffles per token). Per token it reads k and q as float4 broadcasts from shared memory -- every lane of a warp reads the same
// address -- and its own value, and does KPT updates S <- a S + k v and KPT output terms: the loop is fp32-issue
// bound, and state rows are read and written as full 128-byte
// lines (lanes = consecutive columns). Key rows past kdim and columns past vdim are zero-padded in shared memory,
// so the inner loop has no bounds tests. Tokens are staged kRecTok at a time; the next batch is fetched into
// registers while the current one is consumed.
constexpr int kRecTok = 8;

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

template <typename T, int KPT, int NS>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const RecParams P) {
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  constexpr int KS = KPT;                            // slice stride (padding it against the 2-way bank conflict of
                                                     // the NS broadcasts cost more in index arithmetic than it saved)
  constexpr int KP = NS * KS;                        // row of padded keys
  constexpr int CC = 128 / NS;                       // value columns per CTA
  const int s = blockIdx.z, h = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  if (sp.q_len == 0) return;
  const int kdim = P.kdim, vdim = P.vdim;
  const int ksl = threadIdx.x % NS;                  // key slice: rows ksl*KPT .. ksl*KPT + KPT - 1
  const int cl = threadIdx.x / NS;                   // column within the CTA's band
  const int c0 = blockIdx.x * CC;                    // first column of the band
  const int col = c0 + cl;
  const bool col_ok = col < vdim;
  // a warp none of whose columns exist only helps with the staging (warp-uniform, so shuffles stay legal)
  const bool warp_live = c0 + (int)((threadIdx.x & ~31u) / NS) < vdim;
  const int grp = h / (P.H / P.groups);
  float* sq = smem;                                  // [kRecTok][KP]
  float* skk = sq + kRecTok * KP;                    // [kRecTok][KP]
  float* sx = skk + kRecTok * KP;                    // [kRecTok][CC]
  float* sa = sx + kRecTok * CC;                     // [kRecTok] decay of the step
  float* sdt = sa + kRecTok;                         // [kRecTok] step size (1 for a constant decay)

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
  const T* q = (const T*)P.q + (int64_t)grp * kdim;
  const T* k = (const T*)P.k + (int64_t)grp * kdim;
  const T* v = (const T*)P.v + (int64_t)h * vdim + c0;
  const T* dt = (const T*)P.dt;
  const float a_const = P.mode == 0 ? P.decay[h] : 0.f;
  const float rate = P.mode == 1 ? expf(P.a_log[h]) : 0.f;
  const float dt_b = P.mode == 1 ? P.dt_bias[h] : 0.f;
  const float d_skip = P.mode == 1 ? P.d_skip[h] : 0.f;
  const int vcols = min(CC, vdim - c0);

  constexpr int NQ = (kRecTok * KP + 127) / 128;     // q (and k) elements per thread per batch
  constexpr int NV = kRecTok * CC / 128;
  T pq[NQ], pk[NQ], pv[NV], pdt = from_f32<T>(0.f);
  auto fetch = [&](int t0) {
    const int nt = min(kRecTok, sp.q_len - t0);
    const int64_t tok0 = sp.q_start + t0;
#pragma unroll
    for (int n = 0; n < NQ; ++n) {
      const int e = threadIdx.x + n * 128;
      const int tt = e / KP, w = e % KP;
      const int i = (w / KS) * KPT + w % KS;              // key row of this shared-memory word (padding: none)
      const bool ok = tt < nt && w % KS < KPT && i < kdim;
      pq[n] = ok ? q[(tok0 + tt) * P.q_stride + i] : from_f32<T>(0.f);
      pk[n] = ok ? k[(tok0 + tt) * P.k_stride + i] : from_f32<T>(0.f);
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * 128;
      const int tt = e / CC, c = e % CC;
      pv[n] = (tt < nt && c < vcols) ? v[(tok0 + tt) * P.v_stride + c] : from_f32<T>(0.f);
    }
    if (P.mode == 1 && threadIdx.x < nt) pdt = dt[(tok0 + threadIdx.x) * P.dt_stride + h];
  };
  auto stage = [&](int t0) {                         // registers -> shared memory, activations applied once
    const int nt = min(kRecTok, sp.q_len - t0);
#pragma unroll
    for (int n = 0; n < NQ; ++n) {
      const int e = threadIdx.x + n * 128;
      float qv = to_f32<T>(pq[n]), kv = to_f32<T>(pk[n]);
      if (P.act_silu) qv = silu_f(qv), kv = silu_f(kv);           // silu(0) = 0: the padding stays zero
      if (e < kRecTok * KP) {
        sq[e] = qv;
        skk[e] = kv;
      }
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * 128;
      float x = to_f32<T>(pv[n]);
      if (P.act_silu) x = silu_f(x);
      sx[e] = x;
    }
    if (threadIdx.x < nt) {
      float a = a_const, step = 1.f;
      if (P.mode == 1) {
        step = softplus_f(to_f32<T>(pdt) + dt_b);
        a = expf(-rate * step);
      }
      sa[threadIdx.x] = a;
      sdt[threadIdx.x] = step;
    }
  };

  fetch(0);
  for (int t0 = 0; t0 < sp.q_len; t0 += kRecTok) {
    const int nt = min(kRecTok, sp.q_len - t0);
    __syncthreads();                                 // the previous batch has been consumed
    stage(t0);
    __syncthreads();
    if (t0 + kRecTok < sp.q_len) fetch(t0 + kRecTok);
    if (!warp_live) continue;
    float* outp = P.out + (int64_t)(sp.q_start + t0) * ((int64_t)P.H * vdim) + (int64_t)h * vdim + col;
    for (int tt = 0; tt < nt; ++tt) {
      const float a = sa[tt], x = sx[tt * CC + cl], vj = x * sdt[tt];
      const float4* q4 = reinterpret_cast<const float4*>(sq + tt * KP + ksl * KS);
      const float4* k4 = reinterpret_cast<const float4*>(skk + tt * KP + ksl * KS);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < KPT / 4; ++r4) {
        const float4 kq = k4[r4], qq = q4[r4];
        S[r4 * 4 + 0] = a * S[r4 * 4 + 0] + kq.x * vj;
        o0 += S[r4 * 4 + 0] * qq.x;
        S[r4 * 4 + 1] = a * S[r4 * 4 + 1] + kq.y * vj;
        o1 += S[r4 * 4 + 1] * qq.y;
        S[r4 * 4 + 2] = a * S[r4 * 4 + 2] + kq.z * vj;
        o2 += S[r4 * 4 + 2] * qq.z;
        S[r4 * 4 + 3] = a * S[r4 * 4 + 3] + kq.w * vj;
        o3 += S[r4 * 4 + 3] * qq.w;
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (ksl == 0 && col_ok) {
        if (P.mode == 1) o += d_skip * x;
        outp[(int64_t)tt * ((int64_t)P.H * vdim)] = o;
      }
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

template <typename T, int KPT, int NS>
static void recurrence_launch_as(const RecParams& P, int num_seqs, cudaStream_t stream) {
  constexpr int CC = 128 / NS;
  const dim3 grid((P.vdim + CC - 1) / CC, P.H, num_seqs);
  const size_t smem = (size_t)(2 * kRecTok * NS * KPT + kRecTok * CC + 2 * kRecTok) * sizeof(float);
  launch_pdl(linear_recurrence_kernel<T, KPT, NS>, grid, dim3(128), smem, stream, P);
}

template <typename T>
static int recurrence_launch(const RecParams& P, int num_seqs, cudaStream_t stream) {
  if (P.kdim <= 16) recurrence_launch_as<T, 16, 1>(P, num_seqs, stream);
  else if (P.kdim <= 32) recurrence_launch_as<T, 32, 1>(P, num_seqs, stream);
  else if (P.kdim <= 64) recurrence_launch_as<T, 64, 1>(P, num_seqs, stream);
  else if (P.kdim <= 128) recurrence_launch_as<T, 64, 2>(P, num_seqs, stream);
  else recurrence_launch_as<T, 64, 4>(P, num_seqs, stream);
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
