// Matrix memory with exponential gates and a running maximum (the mLSTM recurrence), token by token, in 32-bit.
// Per head, with log gates i_t and f_t:
//   m_t = max(f_t + m_(t-1), i_t)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T          (S: d x dv)
//   n_t = the same with k_t alone                                               (n: d)
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// S, n and m start at zero (m at 0, not at minus infinity) and are carried from token to token in the request's state
// slot, so a sequence may be cut into steps anywhere: the recurrence walks a request's tokens in order whatever the cut.
// The gates are made here from the projection's raw columns: i = cap tanh((x_i + b_i) / cap),
// f = logsigmoid(cap tanh((x_f + b_f) / cap)); cap <= 0 leaves the tanh out.
//
// One block per (tile of value columns, head, request). A column's d state values are spread over `parts` neighbouring
// lanes, R = 8, 16 or 32 rows each (parts = the power of two >= d / R), and the two dot products with q are finished by
// shuffles among those lanes. Every block keeps n and m for itself, so no block reads what another writes.
// Layout of a request's state, from `state_off` (in floats) inside its slot:
//   S as [heads][dv][d_pad]                         (d_pad = parts * R; rows >= d stay zero)
//   then [heads][col_tiles][d_pad + 4]: each block's n, and m behind it (three floats of padding keep 16-byte rows).
// Tokens are staged through shared memory 16 at a time (q scaled by q_scale, k, the tile's v columns, the two gates).
#include "common.cuh"

namespace tmk {

constexpr int kMemThreads = 256;
constexpr int kMemChunk = 16;

struct MemGeometry {
  int R, parts, cols, col_tiles, d_pad;
};

inline MemGeometry mem_geometry(int d, int dv) {
  MemGeometry g;
  g.R = d <= 256 ? 8 : (d <= 512 ? 16 : 32);
  int parts = 1;
  while (parts * g.R < d) parts *= 2;
  g.parts = parts;
  g.cols = kMemThreads / parts;
  g.col_tiles = (dv + g.cols - 1) / g.cols;
  g.d_pad = parts * g.R;
  return g;
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <int R>
__global__ void __launch_bounds__(kMemThreads) matrix_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
    const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int d, int dv, int parts, int cols,
    int col_tiles) {
  extern __shared__ __align__(16) float smem[];
  const int d_pad = parts * R;
  float* qs = smem;                         // [chunk][d_pad]
  float* ks = qs + kMemChunk * d_pad;       // [chunk][d_pad]
  float* vs = ks + kMemChunk * d_pad;       // [chunk][cols]
  float* gi = vs + kMemChunk * cols;        // [chunk]
  float* gf = gi + kMemChunk;               // [chunk]

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y, s = blockIdx.z;
  const int first = cu_q[s], n_tok = cu_q[s + 1] - first;
  if (n_tok <= 0) return;
  const int tid = threadIdx.x;
  const int part = tid % parts, col_local = tid / parts;
  const int col = tile * cols + col_local;
  const bool live = col < dv;
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off;
  float* S_g = slot + ((size_t)head * dv + (live ? col : 0)) * d_pad + part * R;
  float* aux = slot + (size_t)heads * dv * d_pad + ((size_t)head * col_tiles + tile) * (d_pad + 4);

  float S[R], n[R];
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    const float4 a = live ? *reinterpret_cast<const float4*>(S_g + r) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[r] = a.x; S[r + 1] = a.y; S[r + 2] = a.z; S[r + 3] = a.w;
    const float4 b = *reinterpret_cast<const float4*>(aux + part * R + r);
    n[r] = b.x; n[r + 1] = b.y; n[r + 2] = b.z; n[r + 3] = b.w;
  }
  float m = aux[d_pad];

  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  for (int c0 = 0; c0 < n_tok; c0 += kMemChunk) {
    const int cn = min(kMemChunk, n_tok - c0);
    __syncthreads();
    for (int idx = tid; idx < cn * d_pad; idx += kMemThreads) {
      const int tt = idx / d_pad, e = idx - tt * d_pad;
      const float* row = proj + (size_t)(first + c0 + tt) * ld;
      qs[idx] = e < d ? row[q_col + head * d + e] * q_scale : 0.f;
      ks[idx] = e < d ? row[k_col + head * d + e] : 0.f;
    }
    for (int idx = tid; idx < cn * cols; idx += kMemThreads) {
      const int tt = idx / cols, c = idx - tt * cols;
      const int cc = tile * cols + c;
      vs[idx] = cc < dv ? proj[(size_t)(first + c0 + tt) * ld + v_col + head * dv + cc] : 0.f;
    }
    if (tid < cn) {
      const float* row = proj + (size_t)(first + c0 + tid) * ld;
      float xi = row[i_col + head] + (i_bias ? i_bias[head] : 0.f);
      float xf = row[f_col + head] + (f_bias ? f_bias[head] : 0.f);
      if (cap > 0.f) {
        xi = cap * tanhf(xi * inv_cap);
        xf = cap * tanhf(xf * inv_cap);
      }
      gi[tid] = xi;
      gf[tid] = log_sigmoid(xf);
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float li = gi[tt], lf = gf[tt];
      const float m_new = fmaxf(lf + m, li);
      const float a = expf(lf + m - m_new), b = expf(li - m_new);
      m = m_new;
      const float bv = b * vs[tt * cols + col_local];
      const float* kr = ks + tt * d_pad + part * R;
      const float* qr = qs + tt * d_pad + part * R;
      float num = 0.f, dot = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + r);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + r);
        S[r] = fmaf(a, S[r], bv * k4.x);         n[r] = fmaf(a, n[r], b * k4.x);
        S[r + 1] = fmaf(a, S[r + 1], bv * k4.y); n[r + 1] = fmaf(a, n[r + 1], b * k4.y);
        S[r + 2] = fmaf(a, S[r + 2], bv * k4.z); n[r + 2] = fmaf(a, n[r + 2], b * k4.z);
        S[r + 3] = fmaf(a, S[r + 3], bv * k4.w); n[r + 3] = fmaf(a, n[r + 3], b * k4.w);
        num = fmaf(S[r], q4.x, num);     dot = fmaf(n[r], q4.x, dot);
        num = fmaf(S[r + 1], q4.y, num); dot = fmaf(n[r + 1], q4.y, dot);
        num = fmaf(S[r + 2], q4.z, num); dot = fmaf(n[r + 2], q4.z, dot);
        num = fmaf(S[r + 3], q4.w, num); dot = fmaf(n[r + 3], q4.w, dot);
      }
      for (int o = parts >> 1; o > 0; o >>= 1) {
        num += __shfl_xor_sync(0xffffffffu, num, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
      }
      if (part == 0 && live) {
        const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
        y[(size_t)(first + c0 + tt) * heads * dv + head * dv + col] = num / den;
      }
    }
  }

#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (live) *reinterpret_cast<float4*>(S_g + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
    if (col_local == 0) *reinterpret_cast<float4*>(aux + part * R + r) = make_float4(n[r], n[r + 1], n[r + 2], n[r + 3]);
  }
  if (tid == 0) aux[d_pad] = m;
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, with q at q_col (heads x d), k at k_col, v at v_col (heads x dv) and the
// gates' raw values at i_col, f_col (heads each); i_bias, f_bias [heads] float or null; state: float, a request's slot
// at state + slot * state_stride, its memory from state_off there (state_off a multiple of 4, as is state_stride);
// y [T, heads * dv] float.
extern "C" int tm_matrix_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                                const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                                long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                                float* y, int n_seqs, int heads, int d, int dv, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (d < 1 || d > 1024 || dv < 1 || (state_stride & 3) || (state_off & 3)) return TM_ERR_UNSUPPORTED_SHAPE;
  const tmk::MemGeometry g = tmk::mem_geometry(d, dv);
  const size_t smem = ((size_t)tmk::kMemChunk * (2 * g.d_pad + g.cols + 2)) * sizeof(float);
  const dim3 grid(g.col_tiles, heads, n_seqs);
#define TM_MEM_CASE(RR)                                                                                             \
  case RR: {                                                                                                        \
    auto kern = tmk::matrix_memory_kernel<RR>;                                                                      \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                                          \
    }                                                                                                               \
    return tmk::launch_pdl(kern, grid, dim3(tmk::kMemThreads), smem, stream, proj, ld, q_col, k_col, v_col, i_col, f_col, \
                           i_bias, f_bias, cap, q_scale, state, state_stride, state_off, cu_q, state_slots, y, heads, d, dv, \
                           g.parts, g.cols, g.col_tiles);                                                          \
  }
  switch (g.R) {
    TM_MEM_CASE(8) TM_MEM_CASE(16) TM_MEM_CASE(32)
    default: return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_MEM_CASE
}
