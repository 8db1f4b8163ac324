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
// n is carried as one more column of S (the column whose v is 1), so the kernel walks dv + 1 columns alike and writes
// two things: y[t, head, c] = (S_t^T q_t)_c, not yet divided, and den[t, head] = max(|n_t . q_t|, exp(-m_t)) + 1e-6,
// which the column of n produces. The division is left to the kernel that norms the heads (it reads both anyway).
//
// One block per (tile of columns, head, request). A column's d state values are spread over `parts` neighbouring lanes,
// R = 8, 16 or 32 rows each (parts = the power of two >= d / R; lane p takes rows 4 p .. 4 p + 3 of every group of
// 4 * parts rows, so that neighbouring lanes read neighbouring 16 bytes of k and q in shared memory), and the dot product
// with q is finished by shuffles among those lanes. Every block keeps m for itself. Layout of a request's state, from `state_off` (in floats) inside its slot:
//   [heads][dv + 1][d_pad]                          (d_pad = parts * R; rows >= d stay zero; column dv is n)
//   then [heads][col_tiles][4]: m of each block; in a slice record also F and mu (below).
// Tokens are staged through shared memory 16 at a time (q, k, the tile's v columns, the factors made from the gates).
//
// Long portions run in three passes over time slices of `slice_len` tokens, so that a portion's slices work side by
// side. With F = the sum of a slice's f and mu = its own running maximum from an empty memory:
//   pass 1 (mode 1): every slice but a request's last, from S = 0, m = -inf, no outputs; leaves a record (L, mu, F);
//   pass 2 (tm_matrix_memory_pass_states): per request, in order, from the slot's state A = (S_a, m_a): the slice's
//          record is replaced by A, its true start state, and A moves on:
//          m_b = max(F + m_a, mu),  S_b = exp(F + m_a - m_b) S_a + exp(mu - m_b) L;
//   pass 3 (mode 2): every slice from its true start state, with outputs; a request's last slice leaves the slot's state.
// The result equals the walk in one piece up to rounding (m_b is the very maximum the walk would have reached).
// Slice records are laid out like a slot's memory; request s owns records cu_q[s] / slice_len + s onwards (never more
// than its slices, and at most T / slice_len + requests in all).
#include "common.cuh"

namespace tmk {

constexpr int kMemThreads = 256;
constexpr int kMemChunk = 16;

struct MemGeometry {
  int R, parts, cols, col_tiles, d_pad;
  long long floats;
};

inline MemGeometry mem_geometry(int heads, int d, int dv) {
  MemGeometry g;
  g.R = d <= 256 ? 8 : (d <= 512 ? 16 : 32);
  int parts = 1;
  while (parts * g.R < d) parts *= 2;
  g.parts = parts;
  g.cols = kMemThreads / parts;
  g.col_tiles = (dv + 1 + g.cols - 1) / g.cols;
  g.d_pad = parts * g.R;
  g.floats = (long long)heads * (dv + 1) * g.d_pad + (long long)heads * g.col_tiles * 4;
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

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Tokens pass through shared memory `chunk` at a time, in two buffers: while the block works on one chunk, the next
// one's q, k and v columns arrive by asynchronous copies, and warp 0 turns its gates into the per-token factors
// a = exp(f + m_prev - m), b = exp(i - m) and exp(-m) (the chain of maxima is short; the exponentials are taken a lane
// per token), so the walk itself takes no exponential. m lives in warp 0.
template <int R, int MODE>
__global__ void __launch_bounds__(kMemThreads) matrix_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
    const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, float* __restrict__ den, int heads, int d, int dv,
    int parts, int cols, int col_tiles, int n_seqs, int slice_len, float* __restrict__ slices, long long slice_floats,
    int chunk) {
  extern __shared__ __align__(16) float smem[];
  const int d_pad = parts * R;
  const int buf_floats = chunk * (2 * d_pad + cols + 4);
  // one buffer: q [chunk][d_pad], k [chunk][d_pad], v [chunk][cols], factors [chunk][4] = (a, b, exp(-m), -)

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
  const int tid = threadIdx.x, lane = tid & 31;
  const int part = tid % parts, col_local = tid / parts;
  const int col = tile * cols + col_local;
  const bool live = col <= dv;                  // column dv carries n
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off;
  float* record = MODE == 0 ? slot : slices + (size_t)blockIdx.z * slice_floats;
  const int gs = 4 * parts;                     // rows between a lane's groups of four
  float* S_g = record + ((size_t)head * (dv + 1) + (live ? col : 0)) * d_pad + part * 4;
  float* aux = record + (size_t)heads * (dv + 1) * d_pad + ((size_t)head * col_tiles + tile) * 4;

  float S[R];
  float m = -INFINITY, f_sum = 0.f;             // (used by warp 0)
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (MODE == 1 || !live) {
      S[r] = S[r + 1] = S[r + 2] = S[r + 3] = 0.f;
    } else {
      const float4 a = *reinterpret_cast<const float4*>(S_g + (r >> 2) * gs);
      S[r] = a.x; S[r + 1] = a.y; S[r + 2] = a.z; S[r + 3] = a.w;
    }
  }
  if (MODE != 1) m = aux[0];

  // what the copies never write: rows >= d of q and k (zero), the columns behind the values (1 for n, then zero)
  for (int idx = tid; idx < 2 * buf_floats; idx += kMemThreads) {
    const int in_buf = idx % buf_floats;
    float v = 0.f;
    if (in_buf >= 2 * chunk * d_pad && in_buf < chunk * (2 * d_pad + cols))
      v = tile * cols + (in_buf - 2 * chunk * d_pad) % cols == dv ? 1.f : 0.f;
    smem[idx] = v;
  }
  __syncthreads();

  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  const int n_chunks = (n_tok + chunk - 1) / chunk;
  const int v_live = max(0, min(cols, dv - tile * cols));      // value columns of this tile that come from proj

  auto stage = [&](int ci) {                    // asynchronous copies of chunk ci into its buffer
    float* buf = smem + (ci & 1) * buf_floats;
    const int cn = min(chunk, n_tok - ci * chunk);
    const float* base = proj + (size_t)(first + ci * chunk) * ld;
    for (int idx = tid; idx < cn * d; idx += kMemThreads) {
      const int tt = idx / d, e = idx - tt * d;
      const float* row = base + (size_t)tt * ld;
      if (MODE != 1) cp_async4(buf + tt * d_pad + e, row + q_col + head * d + e);
      cp_async4(buf + chunk * d_pad + tt * d_pad + e, row + k_col + head * d + e);
    }
    for (int idx = tid; idx < cn * v_live; idx += kMemThreads) {
      const int tt = idx / v_live, cc = idx - tt * v_live;
      cp_async4(buf + 2 * chunk * d_pad + tt * cols + cc, base + (size_t)tt * ld + v_col + head * dv + tile * cols + cc);
    }
  };
  auto load_gates = [&](int ci, float& xi, float& xf) {        // warp 0: lane t takes token t's raw gates
    xi = xf = 0.f;
    const int cn = min(chunk, n_tok - ci * chunk);
    if (tid < cn) {
      const float* row = proj + (size_t)(first + ci * chunk + tid) * ld;
      xi = row[i_col + head] + (i_bias ? i_bias[head] : 0.f);
      xf = row[f_col + head] + (f_bias ? f_bias[head] : 0.f);
    }
  };
  auto factors = [&](int ci, float xi, float xf) {             // warp 0: the chain of maxima, then a lane per token
    float* fac = smem + (ci & 1) * buf_floats + chunk * (2 * d_pad + cols);
    const int cn = min(chunk, n_tok - ci * chunk);
    if (cap > 0.f) {
      xi = cap * tanhf(xi * inv_cap);
      xf = cap * tanhf(xf * inv_cap);
    }
    const float li = xi, lf = log_sigmoid(xf);
    float m_prev = m, m_mine = m;
    for (int tt = 0; tt < cn; ++tt) {
      const float l_i = __shfl_sync(0xffffffffu, li, tt), l_f = __shfl_sync(0xffffffffu, lf, tt);
      const float m_new = fmaxf(l_f + m, l_i);
      if (lane == tt) {
        m_prev = m;
        m_mine = m_new;
      }
      m = m_new;
      if (MODE == 1) f_sum += l_f;
    }
    if (lane < cn) {
      fac[lane * 4] = expf(lf + m_prev - m_mine);
      fac[lane * 4 + 1] = expf(li - m_mine);
      fac[lane * 4 + 2] = expf(-m_mine);
    }
  };

  float xi = 0.f, xf = 0.f;
  stage(0);
  if (tid < 32) {
    load_gates(0, xi, xf);
    factors(0, xi, xf);
  }
  cp_async_wait_all();
  __syncthreads();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const bool more = ci + 1 < n_chunks;
    if (more) {
      stage(ci + 1);
      if (tid < 32) load_gates(ci + 1, xi, xf);
    }
    const float* buf = smem + (ci & 1) * buf_floats;
    const float* qs = buf;
    const float* ks = buf + chunk * d_pad;
    const float* vs = buf + 2 * chunk * d_pad;
    const float* fac = buf + chunk * (2 * d_pad + cols);
    const int cn = min(chunk, n_tok - ci * chunk);
#pragma unroll 4
    for (int tt = 0; tt < cn; ++tt) {
      const float4 f4 = *reinterpret_cast<const float4*>(fac + tt * 4);
      const float a = f4.x;
      const float bv = f4.y * vs[tt * cols + col_local];
      const float* kr = ks + tt * d_pad + part * 4;
      const float* qr = qs + tt * d_pad + part * 4;
      float num = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + (r >> 2) * gs);
        S[r] = fmaf(a, S[r], bv * k4.x);
        S[r + 1] = fmaf(a, S[r + 1], bv * k4.y);
        S[r + 2] = fmaf(a, S[r + 2], bv * k4.z);
        S[r + 3] = fmaf(a, S[r + 3], bv * k4.w);
        if (MODE != 1) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + (r >> 2) * gs);
          num = fmaf(S[r], q4.x, num);
          num = fmaf(S[r + 1], q4.y, num);
          num = fmaf(S[r + 2], q4.z, num);
          num = fmaf(S[r + 3], q4.w, num);
        }
      }
      if (MODE != 1) {
        for (int o = parts >> 1; o > 0; o >>= 1) num += __shfl_xor_sync(0xffffffffu, num, o);
        if (part == 0 && live) {
          const size_t t = (size_t)(first + ci * chunk + tt);
          num *= q_scale;
          if (col < dv) y[t * heads * dv + head * dv + col] = num;
          else den[t * heads + head] = fmaxf(fabsf(num), f4.z) + 1e-6f;
        }
      }
    }
    if (more && tid < 32) factors(ci + 1, xi, xf);
    cp_async_wait_all();
    __syncthreads();
  }

  if (MODE == 2) {                              // only a request's last slice leaves a state: the slot's
    if (!last_slice) return;
    S_g = slot + ((size_t)head * (dv + 1) + (live ? col : 0)) * d_pad + part * 4;
    aux = slot + (size_t)heads * (dv + 1) * d_pad + ((size_t)head * col_tiles + tile) * 4;
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; r += 4)
      *reinterpret_cast<float4*>(S_g + (r >> 2) * gs) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
  }
  if (tid == 0) {
    if (MODE == 1) {
      aux[1] = f_sum;
      aux[2] = m;
    } else {
      aux[0] = m;
    }
  }
}

// Pass 2: a thread per four neighbouring state values of a request, walking the request's slice records in order. Each
// record (a slice's own sums from an empty memory: L, and mu, F in its block's aux[2], aux[1]) is replaced by the slice's
// true start state (values in place, m in aux[0]), and the running state takes the record in. The next record's values
// are requested before the present one is worked on.
__global__ void __launch_bounds__(256) matrix_memory_pass_kernel(
    const float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, int heads, int dv, int d_pad, int cols, int col_tiles, int slice_len,
    float* __restrict__ slices, long long slice_floats) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int n_tok = cu_q[s + 1] - cu_q[s];
  const int n_slices = (n_tok + slice_len - 1) / slice_len;
  const long long quad = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long values = (long long)heads * (dv + 1) * d_pad;
  if (n_slices <= 0 || quad * 4 >= values) return;
  const long long off = quad * 4;
  const int head = (int)(off / ((long long)(dv + 1) * d_pad));
  const int col = (int)(off / d_pad) - head * (dv + 1);
  const long long a_off = values + ((long long)head * col_tiles + col / cols) * 4;
  const bool writes_m = col % cols == 0 && off % d_pad == 0;       // one thread per block of the walk
  const float* slot = state + (size_t)state_slots[s] * state_stride + state_off;
  float4 S = *reinterpret_cast<const float4*>(slot + off);
  float m = slot[a_off];
  float* rec = slices + (size_t)(cu_q[s] / slice_len + s) * slice_floats;
  float4 L = make_float4(0.f, 0.f, 0.f, 0.f);
  float F = 0.f, mu = 0.f;
  if (n_slices > 1) {
    L = *reinterpret_cast<const float4*>(rec + off);
    F = rec[a_off + 1];
    mu = rec[a_off + 2];
  }
  for (int c = 0; c < n_slices; ++c, rec += slice_floats) {
    const bool has_record = c + 1 < n_slices;
    float4 Ln = make_float4(0.f, 0.f, 0.f, 0.f);
    float Fn = 0.f, mun = 0.f;
    if (c + 2 < n_slices) {
      Ln = *reinterpret_cast<const float4*>(rec + slice_floats + off);
      Fn = rec[slice_floats + a_off + 1];
      mun = rec[slice_floats + a_off + 2];
    }
    *reinterpret_cast<float4*>(rec + off) = S;
    if (writes_m) rec[a_off] = m;
    if (has_record) {
      const float m_b = fmaxf(F + m, mu);
      const float wa = expf(F + m - m_b), wl = expf(mu - m_b);
      S.x = wa * S.x + wl * L.x;
      S.y = wa * S.y + wl * L.y;
      S.z = wa * S.z + wl * L.z;
      S.w = wa * S.w + wl * L.w;
      m = m_b;
    }
    L = Ln;
    F = Fn;
    mu = mun;
  }
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, with q at q_col (heads x d), k at k_col, v at v_col (heads x dv) and the
// gates' raw values at i_col, f_col (heads each); i_bias, f_bias [heads] float or null; state: float, a request's slot
// at state + slot * state_stride, its memory from state_off there (state_off a multiple of 4, as is state_stride);
// y [T, heads * dv] float (undivided), den [T, heads] float. mode 0: each request's tokens in one walk. modes 1 and 2
// (passes 1 and 3 over time slices of slice_len tokens, tm_matrix_memory_pass_states between them): `slices` holds
// n_records records of slice_floats floats (a slot's memory layout; slice_floats a multiple of 4),
// n_records >= T / slice_len + n_seqs.
extern "C" int tm_matrix_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                                const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                                long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                                float* y, float* den, int n_seqs, int heads, int d, int dv, int mode, int slice_len,
                                float* slices, long long slice_floats, int n_records, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (d < 1 || d > 1024 || dv < 1 || (state_stride & 3) || (state_off & 3) || mode < 0 || mode > 2) return TM_ERR_UNSUPPORTED_SHAPE;
  const tmk::MemGeometry g = tmk::mem_geometry(heads, d, dv);
  if (mode != 0 && (!slices || slice_len < 1 || (slice_floats & 3) || n_records < 1 || slice_floats < g.floats))
    return TM_ERR_SCRATCH_TOO_SMALL;
  int chunk = tmk::kMemChunk;                    // two buffers of `chunk` tokens; fewer where rows are long
  while (chunk > 2 && (size_t)2 * chunk * (2 * g.d_pad + g.cols + 4) * sizeof(float) > 96 * 1024) chunk /= 2;
  const size_t smem = (size_t)2 * chunk * (2 * g.d_pad + g.cols + 4) * sizeof(float);
  const dim3 grid(g.col_tiles, heads, mode == 0 ? n_seqs : n_records);
#define TM_MEM_LAUNCH(RR, MM)                                                                                       \
  {                                                                                                                 \
    auto kern = tmk::matrix_memory_kernel<RR, MM>;                                                                  \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                                          \
    }                                                                                                               \
    return tmk::launch_pdl(kern, grid, dim3(tmk::kMemThreads), smem, stream, proj, ld, q_col, k_col, v_col, i_col, f_col, \
                           i_bias, f_bias, cap, q_scale, state, state_stride, state_off, cu_q, state_slots, y, den, heads, d, \
                           dv, g.parts, g.cols, g.col_tiles, n_seqs, slice_len, slices, slice_floats, chunk);      \
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
  const tmk::MemGeometry g = tmk::mem_geometry(heads, d, dv);
  const long long quads = (long long)heads * (dv + 1) * g.d_pad / 4;
  return tmk::launch_pdl(tmk::matrix_memory_pass_kernel, dim3((unsigned)((quads + 255) / 256), n_seqs), dim3(256), 0, stream,
                         state, state_stride, state_off, cu_q, state_slots, heads, dv, g.d_pad, g.cols, g.col_tiles, slice_len,
                         slices, slice_floats);
}
