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
//
// Long portions run in three passes over time slices of `slice_len` tokens, so that a portion's slices work side by
// side. With F = the sum of a slice's f and mu = its own running maximum from an empty memory:
//   pass 1 (mode 1): every slice but a request's last, from S = 0, n = 0, m = -inf, no outputs; leaves (L, n_L, mu, F);
//   pass 2 (tm_matrix_memory_pass_states): per request, in order, from the slot's state A = (S_a, n_a, m_a): the slice's
//          record is replaced by A, its true start state, and A moves on:
//          m_b = max(F + m_a, mu),  S_b = exp(F + m_a - m_b) S_a + exp(mu - m_b) L   (n alike);
//   pass 3 (mode 2): every slice from its true start state, with outputs; a request's last slice leaves the slot's state.
// The result equals the walk in one piece up to rounding (m_b is the very maximum the walk would have reached).
// Slice records lie in a scratch laid out like a slot's memory, F behind m; request s owns records
// cu_q[s] / slice_len + s onwards (never more than its slices, and at most T / slice_len + requests in all).
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

// The block's request and slice: blockIdx.z counts slice records (request s owns cu_q[s] / slice_len + s onwards).
__device__ __forceinline__ bool mem_find_slice(const int* __restrict__ cu_q, int n_seqs, int slice_len, int z, int& s,
                                               int& c) {
  s = 0;
  for (int i = 1; i < n_seqs; ++i)
    if (cu_q[i] / slice_len + i <= z) s = i;
  c = z - (cu_q[s] / slice_len + s);
  return c * slice_len < cu_q[s + 1] - cu_q[s];
}

template <int R, int MODE>
__global__ void __launch_bounds__(kMemThreads) matrix_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
    const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int d, int dv, int parts, int cols,
    int col_tiles, int n_seqs, int slice_len, float* __restrict__ slices, long long slice_floats) {
  extern __shared__ __align__(16) float smem[];
  const int d_pad = parts * R;
  float* qs = smem;                         // [chunk][d_pad]
  float* ks = qs + kMemChunk * d_pad;       // [chunk][d_pad]
  float* vs = ks + kMemChunk * d_pad;       // [chunk][cols]
  float* gi = vs + kMemChunk * cols;        // [chunk]
  float* gf = gi + kMemChunk;               // [chunk]

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y;
  int s = blockIdx.z, c = 0;
  if (MODE != 0 && !mem_find_slice(cu_q, n_seqs, slice_len, blockIdx.z, s, c)) return;
  int first = cu_q[s], n_tok = cu_q[s + 1] - first;
  if (n_tok <= 0) return;
  bool last_slice = true;
  if (MODE != 0) {
    last_slice = (c + 1) * slice_len >= n_tok;
    if (MODE == 1 && last_slice) return;        // nobody needs the last slice's record
    first += c * slice_len;
    n_tok = min(slice_len, n_tok - c * slice_len);
  }
  const int tid = threadIdx.x;
  const int part = tid % parts, col_local = tid / parts;
  const int col = tile * cols + col_local;
  const bool live = col < dv;
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off;
  float* record = MODE == 0 ? slot : slices + (size_t)blockIdx.z * slice_floats;
  float* S_g = record + ((size_t)head * dv + (live ? col : 0)) * d_pad + part * R;
  float* aux = record + (size_t)heads * dv * d_pad + ((size_t)head * col_tiles + tile) * (d_pad + 4);

  float S[R], n[R];
  float m = -INFINITY, f_sum = 0.f;
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (MODE == 1) {
      S[r] = S[r + 1] = S[r + 2] = S[r + 3] = 0.f;
      n[r] = n[r + 1] = n[r + 2] = n[r + 3] = 0.f;
    } else {
      const float4 a = live ? *reinterpret_cast<const float4*>(S_g + r) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[r] = a.x; S[r + 1] = a.y; S[r + 2] = a.z; S[r + 3] = a.w;
      const float4 b = *reinterpret_cast<const float4*>(aux + part * R + r);
      n[r] = b.x; n[r + 1] = b.y; n[r + 2] = b.z; n[r + 3] = b.w;
    }
  }
  if (MODE != 1) m = aux[d_pad];

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
      if (MODE == 1) f_sum += lf;
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
        if (MODE != 1) {
          num = fmaf(S[r], q4.x, num);     dot = fmaf(n[r], q4.x, dot);
          num = fmaf(S[r + 1], q4.y, num); dot = fmaf(n[r + 1], q4.y, dot);
          num = fmaf(S[r + 2], q4.z, num); dot = fmaf(n[r + 2], q4.z, dot);
          num = fmaf(S[r + 3], q4.w, num); dot = fmaf(n[r + 3], q4.w, dot);
        }
      }
      if (MODE == 1) continue;
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

  if (MODE == 2) {                              // only a request's last slice leaves a state: the slot's
    if (!last_slice) return;
    S_g = slot + ((size_t)head * dv + (live ? col : 0)) * d_pad + part * R;
    aux = slot + (size_t)heads * dv * d_pad + ((size_t)head * col_tiles + tile) * (d_pad + 4);
  }
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (live) *reinterpret_cast<float4*>(S_g + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
    if (col_local == 0) *reinterpret_cast<float4*>(aux + part * R + r) = make_float4(n[r], n[r + 1], n[r + 2], n[r + 3]);
  }
  if (tid == 0) {
    aux[d_pad] = m;
    if (MODE == 1) aux[d_pad + 1] = f_sum;
  }
}

// Pass 2: one block per (tile of value columns, head, request), the thread layout of the kernel above. Walks the
// request's slices in order; each record (a slice's own sums from an empty memory) is replaced by the slice's true start
// state, and the running state takes the record in.
template <int R>
__global__ void __launch_bounds__(kMemThreads) matrix_memory_pass_kernel(
    const float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, int heads, int d, int dv, int parts, int cols, int col_tiles, int slice_len,
    float* __restrict__ slices, long long slice_floats) {
  const int d_pad = parts * R;
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y, s = blockIdx.z;
  const int n_tok = cu_q[s + 1] - cu_q[s];
  const int n_slices = (n_tok + slice_len - 1) / slice_len;
  if (n_slices <= 0) return;
  const int tid = threadIdx.x;
  const int part = tid % parts, col_local = tid / parts;
  const int col = tile * cols + col_local;
  const bool live = col < dv;
  const size_t s_off = ((size_t)head * dv + (live ? col : 0)) * d_pad + part * R;
  const size_t a_off = (size_t)heads * dv * d_pad + ((size_t)head * col_tiles + tile) * (d_pad + 4);
  const float* slot = state + (size_t)state_slots[s] * state_stride + state_off;
  float S[R], n[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    S[r] = live ? slot[s_off + r] : 0.f;
    n[r] = slot[a_off + part * R + r];
  }
  float m = slot[a_off + d_pad];
  float* rec = slices + (size_t)(cu_q[s] / slice_len + s) * slice_floats;
  for (int c = 0; c < n_slices; ++c, rec += slice_floats) {
    const bool has_record = c + 1 < n_slices;
    float mu = 0.f, F = 0.f, wa = 1.f, wl = 0.f, m_b = m;
    if (has_record) {
      mu = rec[a_off + d_pad];
      F = rec[a_off + d_pad + 1];
      m_b = fmaxf(F + m, mu);
      wa = expf(F + m - m_b);
      wl = expf(mu - m_b);
    }
    float Ls[R], Ln[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      Ls[r] = (has_record && live) ? rec[s_off + r] : 0.f;
      Ln[r] = has_record ? rec[a_off + part * R + r] : 0.f;
    }
    __syncthreads();                  // every thread has read the record (n, mu and F are shared) before it is replaced
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (live) rec[s_off + r] = S[r];
      if (col_local == 0) rec[a_off + part * R + r] = n[r];
      S[r] = wa * S[r] + wl * Ls[r];
      n[r] = wa * n[r] + wl * Ln[r];
    }
    if (tid == 0) rec[a_off + d_pad] = m;
    m = m_b;
  }
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, with q at q_col (heads x d), k at k_col, v at v_col (heads x dv) and the
// gates' raw values at i_col, f_col (heads each); i_bias, f_bias [heads] float or null; state: float, a request's slot
// at state + slot * state_stride, its memory from state_off there (state_off a multiple of 4, as is state_stride);
// y [T, heads * dv] float. mode 0: each request's tokens in one walk. modes 1 and 2 (passes 1 and 3 over time slices of
// slice_len tokens, tm_matrix_memory_pass_states between them): `slices` holds n_records records of slice_floats floats
// (a slot's memory layout; slice_floats a multiple of 4), n_records >= T / slice_len + n_seqs.
extern "C" int tm_matrix_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                                const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                                long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                                float* y, int n_seqs, int heads, int d, int dv, int mode, int slice_len, float* slices,
                                long long slice_floats, int n_records, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (d < 1 || d > 1024 || dv < 1 || (state_stride & 3) || (state_off & 3) || mode < 0 || mode > 2) return TM_ERR_UNSUPPORTED_SHAPE;
  const tmk::MemGeometry g = tmk::mem_geometry(d, dv);
  if (mode != 0 && (!slices || slice_len < 1 || (slice_floats & 3) || n_records < 1 ||
                    slice_floats < (long long)heads * dv * g.d_pad + (long long)heads * g.col_tiles * (g.d_pad + 4)))
    return TM_ERR_SCRATCH_TOO_SMALL;
  const size_t smem = ((size_t)tmk::kMemChunk * (2 * g.d_pad + g.cols + 2)) * sizeof(float);
  const dim3 grid(g.col_tiles, heads, mode == 0 ? n_seqs : n_records);
#define TM_MEM_LAUNCH(RR, MM)                                                                                       \
  {                                                                                                                 \
    auto kern = tmk::matrix_memory_kernel<RR, MM>;                                                                  \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                                          \
    }                                                                                                               \
    return tmk::launch_pdl(kern, grid, dim3(tmk::kMemThreads), smem, stream, proj, ld, q_col, k_col, v_col, i_col, f_col, \
                           i_bias, f_bias, cap, q_scale, state, state_stride, state_off, cu_q, state_slots, y, heads, d, dv, \
                           g.parts, g.cols, g.col_tiles, n_seqs, slice_len, slices, slice_floats);                 \
  }
#define TM_MEM_CASE(RR)                                                                                             \
  case RR:                                                                                                          \
    if (mode == 0) TM_MEM_LAUNCH(RR, 0)                                                                             \
    if (mode == 1) TM_MEM_LAUNCH(RR, 1)                                                                             \
    TM_MEM_LAUNCH(RR, 2)
  switch (g.R) {
    TM_MEM_CASE(8) TM_MEM_CASE(16) TM_MEM_CASE(32)
    default: return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_MEM_CASE
#undef TM_MEM_LAUNCH
}

// Pass 2 over the slice records (see the top of this file); the same state, cu_q, state_slots and slices as the passes
// around it.
extern "C" int tm_matrix_memory_pass_states(const float* state, long long state_stride, long long state_off,
                                            const int* cu_q, const int* state_slots, int n_seqs, int heads, int d, int dv,
                                            int slice_len, float* slices, long long slice_floats, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (d < 1 || d > 1024 || dv < 1 || !slices || slice_len < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  const tmk::MemGeometry g = tmk::mem_geometry(d, dv);
  const dim3 grid(g.col_tiles, heads, n_seqs);
#define TM_MEM_PASS(RR)                                                                                             \
  case RR:                                                                                                          \
    return tmk::launch_pdl(tmk::matrix_memory_pass_kernel<RR>, grid, dim3(tmk::kMemThreads), 0, stream, state, state_stride, \
                           state_off, cu_q, state_slots, heads, d, dv, g.parts, g.cols, g.col_tiles, slice_len, slices,   \
                           slice_floats);
  switch (g.R) {
    TM_MEM_PASS(8) TM_MEM_PASS(16) TM_MEM_PASS(32)
    default: return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_MEM_PASS
}
