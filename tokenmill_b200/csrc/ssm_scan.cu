// A selective state-space mixer's two recurrent pieces: the short causal convolution with its carried inputs,
// and the state recurrence itself. Both read the mixer's fused input projection
//   proj[t] = [z (inner) | x (inner) | B (groups * N) | C (groups * N) | dt (heads)]
// and a per-request state slot [conv inputs ((taps - 1) * channels) | S (heads * vdim * N)] of 32-bit floats.
//
// tm_conv_silu_state: channels = inner + 2 * groups * N run a causal convolution over the request's tokens
// (weights [channels, taps], the LAST tap weighs the current token; what lies before the step's first token comes
// from the slot, zeros for a new request), plus bias, then silu; 32-bit arithmetic, one rounding to the activation
// dtype. Thread (token, channel). Only the thread of a request's first row touches the slot: it computes the up to
// taps - 1 outputs that need carried inputs, then writes the step's last taps - 1 inputs back.
//
// tm_ssm_scan: per head h (group g = h / (heads / groups)) and token t, all in 32-bit:
//   dt = softplus(dt_raw + dt_bias[h])        a = exp(-exp(A_log[h]) * dt)
//   S <- a * S + dt * B_t x_t^T               y_t = S^T C_t + D[h] * x_t
// One block per (head, request, slice of vdim); each group of 4 columns p is served by 8 lanes that hold N / 8
// state values of each of them in registers for the whole step (one load of B and of C serves the four). Tokens are taken in chunks through shared memory and
// walked strictly in order, so the result does not depend on how a request was cut into steps.
//
// A long prompt portion would leave one block per (head, request) walking thousands of tokens one after the other
// (about 0.4 us a token). Such steps run in three passes over time slices of `slice_len` tokens instead
// (tm_ssm_scan with mode 1, tm_ssm_pass_states, tm_ssm_scan with mode 2): every slice first runs the recurrence
// from a zero state (all slices at once) and leaves its end state and the product of its decays; a small kernel
// walks each request's slices in order, S_start[k+1] = a[k] S_start[k] + S_local[k], and writes the request's new
// state; then every slice runs again from its true start state and writes y. Twice the arithmetic, a slice's
// length of sequential steps instead of the portion's; the result differs from the token-by-token walk by 32-bit
// rounding only.
#include "common.cuh"

namespace tmk {

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(256) conv_silu_state_kernel(
    const T* __restrict__ proj, long long proj_stride, int col0, int channels, int taps,
    const float* __restrict__ weight, const float* __restrict__ bias, float* __restrict__ state,
    long long state_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_of_token,
    const int* __restrict__ state_slots, T* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = seq_of_token[t];
  const int first = cu_q[s];
  const int j = t - first;
  const int carried = taps - 1;
  if (j > 0 && j < carried) return;          // the first row's thread computes these
  float w[kMaxTaps];
  for (int k = 0; k < taps; ++k) w[k] = weight[(size_t)c * taps + k];
  const float bv = bias ? bias[c] : 0.f;
  const T* in = proj + col0 + c;
  if (j >= carried) {
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) acc = fmaf(w[k], to_float(in[(size_t)(t - carried + k) * proj_stride]), acc);
    acc += bv;
    out[(size_t)t * channels + c] = from_float<T>(acc / (1.0f + expf(-acc)));
    return;
  }
  // j == 0: this thread owns the request's carried inputs of channel c.
  const int q_len = cu_q[s + 1] - first;
  float* slot = state + (size_t)state_slots[s] * state_stride + c;       // carried input i at slot[i * channels]
  float old[kMaxTaps];
  for (int i = 0; i < carried; ++i) old[i] = slot[(size_t)i * channels];
  const int n_head = min(carried, q_len);
  for (int jj = 0; jj < n_head; ++jj) {
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
      const int src = jj - carried + k;        // offset inside the step; negative: carried input carried + src
      const float v = src >= 0 ? to_float(in[(size_t)(first + src) * proj_stride]) : old[carried + src];
      acc = fmaf(w[k], v, acc);
    }
    acc += bv;
    out[(size_t)(first + jj) * channels + c] = from_float<T>(acc / (1.0f + expf(-acc)));
  }
  for (int i = 0; i < carried; ++i) {
    const int src = q_len - carried + i;
    slot[(size_t)i * channels] = src >= 0 ? to_float(in[(size_t)(first + src) * proj_stride]) : old[i + q_len];
  }
}

// The same with VEC consecutive channels per thread (16 bytes per access; 2 to 4 taps) for the rows that need no carried input;
// a request's first row still owns the slot and walks its VEC channels one after the other.
template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(128) conv_silu_state_vec_kernel(
    const T* __restrict__ proj, long long proj_stride, int col0, int channels, int taps,
    const float* __restrict__ weight, const float* __restrict__ weight_t, const float* __restrict__ bias, float* __restrict__ state,
    long long state_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_of_token,
    const int* __restrict__ state_slots, T* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= channels) return;
  const int s = seq_of_token[t];
  const int first = cu_q[s];
  const int j = t - first;
  const int carried = taps - 1;
  if (j > 0 && j < carried) return;
  if (j >= carried) {
    // The weights come from the copy laid out [taps, channels]: a warp's loads of one tap are one contiguous
    // kilobyte (from [channels, taps] every lane would touch a line of its own, and the kernel was bound by that).
    float acc[VEC], wr[VEC * TAPS], bv[VEC];
#pragma unroll
    for (int k = 0; k < TAPS; ++k)
#pragma unroll
      for (int i = 0; i < VEC / 4; ++i) {
        const float4 w4 = *reinterpret_cast<const float4*>(weight_t + (size_t)k * channels + c0 + 4 * i);
        wr[(4 * i) * TAPS + k] = w4.x; wr[(4 * i + 1) * TAPS + k] = w4.y;
        wr[(4 * i + 2) * TAPS + k] = w4.z; wr[(4 * i + 3) * TAPS + k] = w4.w;
      }
#pragma unroll
    for (int i = 0; i < VEC / 4; ++i) {
      float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (bias) b4 = *reinterpret_cast<const float4*>(bias + c0 + 4 * i);
      bv[4 * i] = b4.x; bv[4 * i + 1] = b4.y; bv[4 * i + 2] = b4.z; bv[4 * i + 3] = b4.w;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < TAPS; ++k) {
      const uint4 raw = *reinterpret_cast<const uint4*>(proj + (size_t)(t - carried + k) * proj_stride + col0 + c0);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wr[e * TAPS + k], to_float(v[e]), acc[e]);
    }
    uint4 res;
    T* o = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float a = acc[e] + bv[e];
      o[e] = from_float<T>(a / (1.0f + expf(-a)));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * channels + c0) = res;
    return;
  }
  const int q_len = cu_q[s + 1] - first;
  for (int e = 0; e < VEC; ++e) {
    const int c = c0 + e;
    float w[kMaxTaps], old[kMaxTaps];
    for (int k = 0; k < taps; ++k) w[k] = weight[(size_t)c * taps + k];
    const float bv = bias ? bias[c] : 0.f;
    const T* in = proj + col0 + c;
    float* slot = state + (size_t)state_slots[s] * state_stride + c;
    for (int i = 0; i < carried; ++i) old[i] = slot[(size_t)i * channels];
    const int n_head = min(carried, q_len);
    for (int jj = 0; jj < n_head; ++jj) {
      float acc = 0.f;
      for (int k = 0; k < taps; ++k) {
        const int src = jj - carried + k;
        const float v = src >= 0 ? to_float(in[(size_t)(first + src) * proj_stride]) : old[carried + src];
        acc = fmaf(w[k], v, acc);
      }
      acc += bv;
      out[(size_t)(first + jj) * channels + c] = from_float<T>(acc / (1.0f + expf(-acc)));
    }
    for (int i = 0; i < carried; ++i) {
      const int src = q_len - carried + i;
      slot[(size_t)i * channels] = src >= 0 ? to_float(in[(size_t)(first + src) * proj_stride]) : old[i + q_len];
    }
  }
}

template <typename T>
int launch_conv_silu_state(const void* proj, long long proj_stride, int col0, int channels, int taps, const float* weight,
                           const float* weight_t, const float* bias, float* state, long long state_stride, const int* cu_q,
                           const int* seq_of_token, const int* state_slots, void* out, int T_, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned = channels % VEC == 0 && col0 % VEC == 0 && proj_stride % VEC == 0 &&
                       weight_t != nullptr &&
                       ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(out) |
                         reinterpret_cast<uintptr_t>(weight_t) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
#define TM_CONV_VEC(TAPS)                                                                                            \
  if (aligned && taps == TAPS)                                                                                       \
    return launch_pdl(conv_silu_state_vec_kernel<T, VEC, TAPS>, dim3(T_, (channels / VEC + 127) / 128), dim3(128), 0,  \
                      stream, (const T*)proj, proj_stride, col0, channels, taps, weight, weight_t, bias, state,      \
                      state_stride,                                                                                  \
                      cu_q, seq_of_token, state_slots, (T*)out);
  TM_CONV_VEC(2) TM_CONV_VEC(3) TM_CONV_VEC(4)
#undef TM_CONV_VEC
  return launch_pdl(conv_silu_state_kernel<T>, dim3(T_, (channels + 255) / 256), dim3(256), 0, stream, (const T*)proj,
                    proj_stride, col0, channels, taps, weight, bias, state, state_stride, cu_q, seq_of_token, state_slots,
                    (T*)out);
}

constexpr int kScanLanes = 8;        // lanes that share one column of the state

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

constexpr int kScanCols = 4;         // columns of the state a thread holds: they share every load of B and C

template <typename T, int NPL>       // NPL = ceil(N / 8) state values per lane and column
__global__ void __launch_bounds__(128) ssm_scan_kernel(
    const T* __restrict__ xbc, int channels, const T* __restrict__ proj, long long proj_stride, int dt_col,
    const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ Dskip,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int vdim, int N, int groups, int cols,
    int chunk, int mode, int slice_len, int max_slices, float* __restrict__ slice_S, float* __restrict__ slice_a,
    int vec) {
  extern __shared__ __align__(16) float sm[];
  float* Bs = sm;                               // [chunk][N]
  float* Cs = Bs + chunk * N;                   // [chunk][N]
  float* xs = Cs + chunk * N;                   // [chunk][cols]
  float* dts = xs + chunk * cols;               // [chunk]
  float* decs = dts + chunk;                    // [chunk]
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, p0 = blockIdx.z * cols;
  const int s = mode == 0 ? blockIdx.y : blockIdx.y / max_slices;
  const int slice = mode == 0 ? 0 : blockIdx.y % max_slices;
  const int g = h / (heads / groups);
  const int inner = heads * vdim;
  const int tid = threadIdx.x;
  const int r = tid & (kScanLanes - 1), pl = (tid / kScanLanes) * kScanCols;      // first of the thread's columns
  int first = cu_q[s], q_len = cu_q[s + 1] - first;
  if (mode != 0) {                               // this block's slice of the request's tokens
    if (slice * slice_len >= q_len) return;
    first += slice * slice_len;
    q_len = min(slice_len, q_len - slice * slice_len);
  }
  float* Sbase = mode == 0 ? state + (size_t)state_slots[s] * state_stride + state_off + (size_t)h * vdim * N
                           : slice_S + ((size_t)blockIdx.y * heads + h) * vdim * N;
  bool live[kScanCols];
  float st[kScanCols][NPL];
#pragma unroll
  for (int q = 0; q < kScanCols; ++q) {
    const int p = p0 + pl + q;
    live[q] = pl + q < cols && p < vdim;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = r + kScanLanes * i;
      st[q][i] = (live[q] && n < N && mode != 1) ? Sbase[(size_t)p * N + n] : 0.f;
    }
  }
  float dt_sum = 0.f;
  const float neg_a = -expf(A_log[h]), bias = dt_bias[h], dskip = Dskip[h];
  for (int c0 = 0; c0 < q_len; c0 += chunk) {
    const int nt = min(chunk, q_len - c0);
    __syncthreads();
    if (vec) {                                   // rows of B, C and x in 16-byte pieces (the host checked the alignment)
      constexpr int VEC = 16 / sizeof(T);
      const int per_row = N / VEC, per_x = cols / VEC;
      for (int idx = tid; idx < 2 * nt * per_row; idx += blockDim.x) {
        const int which = idx / (nt * per_row), rem = idx - which * nt * per_row;
        const int tt = rem / per_row, v = rem - tt * per_row;
        const uint4 raw = *reinterpret_cast<const uint4*>(xbc + (size_t)(first + c0 + tt) * channels + inner + g * N +
                                                          which * groups * N + v * VEC);
        const T* e = reinterpret_cast<const T*>(&raw);
        float* dst = (which ? Cs : Bs) + tt * N + v * VEC;
#pragma unroll
        for (int k = 0; k < VEC; ++k) dst[k] = to_float(e[k]);
      }
      for (int idx = tid; idx < nt * per_x; idx += blockDim.x) {
        const int tt = idx / per_x, v = idx - tt * per_x;
        const uint4 raw = *reinterpret_cast<const uint4*>(xbc + (size_t)(first + c0 + tt) * channels + h * vdim + p0 + v * VEC);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int k = 0; k < VEC; ++k) xs[tt * cols + v * VEC + k] = to_float(e[k]);
      }
    } else {
      for (int idx = tid; idx < nt * N; idx += blockDim.x) {
        const int tt = idx / N, n = idx - tt * N;
        const T* row = xbc + (size_t)(first + c0 + tt) * channels + inner + g * N + n;
        Bs[idx] = to_float(row[0]);
        Cs[idx] = to_float(row[groups * N]);
      }
      for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
        const int tt = idx / cols, pp = idx - tt * cols;
        xs[idx] = p0 + pp < vdim ? to_float(xbc[(size_t)(first + c0 + tt) * channels + h * vdim + p0 + pp]) : 0.f;
      }
    }
    for (int tt = tid; tt < nt; tt += blockDim.x) {
      const float dt = softplus_f(to_float(proj[(size_t)(first + c0 + tt) * proj_stride + dt_col + h]) + bias);
      dts[tt] = dt;
      decs[tt] = expf(neg_a * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {            // (every lane of a warp runs the loop: the shuffles want them all)
      const float dec = decs[tt], dt = dts[tt];
      const float* Bt = Bs + tt * N;
      const float* Ct = Cs + tt * N;
      float xv[kScanCols], dx[kScanCols], part[kScanCols];
#pragma unroll
      for (int q = 0; q < kScanCols; ++q) {
        xv[q] = pl + q < cols ? xs[tt * cols + pl + q] : 0.f;
        dx[q] = dt * xv[q];
        part[q] = 0.f;
      }
      dt_sum += dt;
      if (mode == 1) {                           // the state alone: nobody reads this pass's y
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int n = r + kScanLanes * i;
          if (n < N) {
            const float bv = Bt[n];
#pragma unroll
            for (int q = 0; q < kScanCols; ++q) st[q][i] = fmaf(dec, st[q][i], dx[q] * bv);
          }
        }
        continue;
      }
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int n = r + kScanLanes * i;
        if (n < N) {
          const float bv = Bt[n], cv = Ct[n];
#pragma unroll
          for (int q = 0; q < kScanCols; ++q) {
            st[q][i] = fmaf(dec, st[q][i], dx[q] * bv);
            part[q] = fmaf(st[q][i], cv, part[q]);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < kScanCols; ++q) {
        part[q] += __shfl_xor_sync(0xffffffffu, part[q], 1);
        part[q] += __shfl_xor_sync(0xffffffffu, part[q], 2);
        part[q] += __shfl_xor_sync(0xffffffffu, part[q], 4);
        if (r == 0 && live[q])
          y[(size_t)(first + c0 + tt) * inner + h * vdim + p0 + pl + q] = fmaf(dskip, xv[q], part[q]);
      }
    }
  }
  if (mode != 2) {
#pragma unroll
    for (int q = 0; q < kScanCols; ++q) {
      if (!live[q]) continue;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int n = r + kScanLanes * i;
        if (n < N) Sbase[(size_t)(p0 + pl + q) * N + n] = st[q][i];
      }
    }
  }
  if (mode == 1 && tid == 0 && blockIdx.z == 0) slice_a[(size_t)blockIdx.y * heads + h] = expf(neg_a * dt_sum);
}

// One thread per state value of a request: walk the request's slices in order. On entry slice_S[k] holds slice k's
// end state from a zero start and slice_a[k] its decay; on exit slice_S[k] holds slice k's start state and the
// request's slot its new state.
__global__ void __launch_bounds__(256) ssm_pass_states_kernel(
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ slice_S, const float* __restrict__ slice_a, int heads,
    int per_head, int slice_len, int max_slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)heads * per_head) return;
  const int h = (int)(e / per_head);
  const int q_len = cu_q[s + 1] - cu_q[s];
  const int n_slices = (q_len + slice_len - 1) / slice_len;
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off + e;
  float cur = *slot;
  for (int k = 0; k < n_slices; ++k) {
    const size_t at = (size_t)s * max_slices + k;
    float* p = slice_S + at * heads * per_head + e;
    const float local = *p;
    *p = cur;
    cur = fmaf(slice_a[at * heads + h], cur, local);
  }
  *slot = cur;
}

template <typename T>
int launch_ssm_scan(const void* xbc, int channels, const void* proj, long long proj_stride, int dt_col,
                    const float* A_log, const float* dt_bias, const float* Dskip, float* state, long long state_stride,
                    long long state_off, const int* cu_q, const int* state_slots, float* y, int n_seqs, int heads,
                    int vdim, int N, int groups, int max_q_len, int mode, int slice_len, int max_slices, float* slice_S,
                    float* slice_a, cudaStream_t stream) {
  if (N > 32 * kScanLanes || heads % groups) return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0 && (slice_len < 1 || max_slices < 1 || !slice_S || !slice_a)) return TM_ERR_SCRATCH_TOO_SMALL;
  const int cols = vdim < 64 ? ((vdim + 3) / 4) * 4 : 64;          // (a multiple of 4: whole warps)
  const int threads = ((cols / kScanCols * kScanLanes + 31) / 32) * 32;
  const dim3 grid(heads, mode == 0 ? n_seqs : n_seqs * max_slices, (vdim + cols - 1) / cols);
  if (grid.y > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0) max_q_len = slice_len;
  int chunk = max_q_len < 16 ? (max_q_len < 1 ? 1 : max_q_len) : 16;
  while (chunk > 1 && (size_t)chunk * (2 * N + cols + 2) * sizeof(float) > 40 * 1024) chunk /= 2;
  const size_t smem = (size_t)chunk * (2 * N + cols + 2) * sizeof(float);
  constexpr int VEC = 16 / sizeof(T);
  const int vec = N % VEC == 0 && channels % VEC == 0 && vdim % VEC == 0 && cols % VEC == 0 && vdim % cols == 0 &&
                  (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
  const int npl = (N + kScanLanes - 1) / kScanLanes;
#define TM_SCAN_CASE(NPL)                                                                                            \
  if (npl <= NPL)                                                                                                    \
    return launch_pdl(ssm_scan_kernel<T, NPL>, grid, dim3(threads), smem, stream, (const T*)xbc, channels,           \
                      (const T*)proj, proj_stride, dt_col, A_log, dt_bias, Dskip, state, state_stride, state_off, cu_q, \
                      state_slots, y, heads, vdim, N, groups, cols, chunk, mode, slice_len, max_slices, slice_S, slice_a, vec);
  TM_SCAN_CASE(1) TM_SCAN_CASE(2) TM_SCAN_CASE(4) TM_SCAN_CASE(8) TM_SCAN_CASE(16) TM_SCAN_CASE(32)
#undef TM_SCAN_CASE
  return TM_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace tmk

// proj [T, proj_stride] dtype, channels col0 .. col0 + channels - 1 are convolved; weight [channels, taps] (weight_t:
// the same as [taps, channels], or null), bias
// [channels] float; state [slots, state_stride] float, carried inputs first; out [T, channels] dtype.
extern "C" int tm_conv_silu_state(int dtype, const void* proj, long long proj_stride, int col0, int channels, int taps,
                                  const float* weight, const float* weight_t, const float* bias, float* state, long long state_stride,
                                  const int* cu_q, const int* seq_of_token, const int* state_slots, void* out, int T,
                                  cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || taps > tmk::kMaxTaps) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_conv_silu_state<float>(proj, proj_stride, col0, channels, taps, weight, weight_t, bias, state, state_stride,
                                              cu_q, seq_of_token, state_slots, out, T, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_conv_silu_state<__nv_bfloat16>(proj, proj_stride, col0, channels, taps, weight, weight_t, bias, state,
                                                      state_stride, cu_q, seq_of_token, state_slots, out, T, stream);
  return TM_ERR_BAD_DTYPE;
}

// xbc [T, channels] dtype = [x (heads * vdim) | B (groups * N) | C (groups * N)] after convolution and silu; dt_raw is
// column dt_col + h of proj; A_log, dt_bias, Dskip [heads] float; S of a request at state_off inside its slot,
// laid out [heads, vdim, N]; y [T, heads * vdim] float; max_q_len: the most tokens any request brings (sizes the chunks).
// mode 0: the whole step in order. mode 1 / 2: the first and last of the three passes over time slices (above);
// slice_S [n_seqs * max_slices, heads, vdim, N] and slice_a [n_seqs * max_slices, heads] float.
extern "C" int tm_ssm_scan(int dtype, const void* xbc, int channels, const void* proj, long long proj_stride, int dt_col,
                           const float* A_log, const float* dt_bias, const float* Dskip, float* state,
                           long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                           float* y, int n_seqs, int heads, int vdim, int N, int groups, int max_q_len, int mode,
                           int slice_len, int max_slices, float* slice_S, float* slice_a, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_ssm_scan<float>(xbc, channels, proj, proj_stride, dt_col, A_log, dt_bias, Dskip, state,
                                       state_stride, state_off, cu_q, state_slots, y, n_seqs, heads, vdim, N, groups,
                                       max_q_len, mode, slice_len, max_slices, slice_S, slice_a, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_ssm_scan<__nv_bfloat16>(xbc, channels, proj, proj_stride, dt_col, A_log, dt_bias, Dskip, state,
                                               state_stride, state_off, cu_q, state_slots, y, n_seqs, heads, vdim, N,
                                               groups, max_q_len, mode, slice_len, max_slices, slice_S, slice_a, stream);
  return TM_ERR_BAD_DTYPE;
}

extern "C" int tm_ssm_pass_states(float* state, long long state_stride, long long state_off, const int* cu_q,
                                  const int* state_slots, float* slice_S, const float* slice_a, int n_seqs, int heads,
                                  int vdim, int N, int slice_len, int max_slices, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (n_seqs > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  const long long total = (long long)heads * vdim * N;
  return tmk::launch_pdl(tmk::ssm_pass_states_kernel, dim3((unsigned)((total + 255) / 256), n_seqs), dim3(256), 0, stream,
                         state, state_stride, state_off, cu_q, state_slots, slice_S, slice_a, heads, vdim * N, slice_len,
                         max_slices);
}
