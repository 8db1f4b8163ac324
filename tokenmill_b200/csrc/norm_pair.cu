// RMSNorm computed wholly in 32-bit, for blocks whose two branches read the same stream, and the
// token shift that may follow it.
//
// tm_add_norm_pair, one block per row:
//   x = table[ids[row]]                          (the stream starts here), or
//   x = resid[row] + scale * (a[row] + b[row])   (either branch may be absent; sum taken and stored in 32-bit)
//   r = 1 / sqrt(mean(x^2) + eps)
//   out1[row] = x * r * w1        out2[row] = x * r * w2   (second output optional)
// Every product is 32-bit and each output is rounded once. The weights arrive ready to multiply (a norm whose
// checkpoint weight is stored around zero has had its 1 added when it was bound). out1 is either the activation
// dtype or float32 (`out1_f32`): the 32-bit form feeds the token shift below. With `rows`, only those rows are
// normed, written densely, and the stream is left as it is (the sums a and b are still added to the value read).
//
// tm_token_shift, one block per row: out[t] = h[t] + (h[t-1] - h[t]) * mu, where h[t-1] of a request's first row
// in this step is what the request's state slot holds (zero for a new request: slots are zeroed at admission).
// The block of a request's first row also moves the request's last h of this step into the slot, after it has
// read the old value: no other block touches that slot.
#include "common.cuh"

namespace tmk {

template <typename T, typename O1>
__global__ void __launch_bounds__(256) add_norm_pair_kernel(
    float* __restrict__ resid, const T* __restrict__ a, const T* __restrict__ b, float scale,
    const int* __restrict__ ids, const T* __restrict__ table, const int* __restrict__ rows,
    const float* __restrict__ w1, const float* __restrict__ w2, float eps, O1* __restrict__ out1,
    T* __restrict__ out2, int H) {
  extern __shared__ __align__(16) float xs[];  // H floats + 32 for the reduction
  float* red = xs + H;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const bool write_back = !rows && (ids || a || b);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float x;
    if (ids) {
      x = to_float(table[(size_t)ids[src] * H + i]);
    } else {
      x = resid[(size_t)src * H + i];
      if (a || b) {
        float add = 0.f;
        if (a) add += to_float(a[(size_t)src * H + i]);
        if (b) add += to_float(b[(size_t)src * H + i]);
        x = fmaf(scale, add, x);
      }
    }
    if (write_back) resid[(size_t)src * H + i] = x;
    xs[i] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float y = xs[i] * rstd;
    out1[(size_t)r * H + i] = from_float<O1>(y * w1[i]);
    if (out2) out2[(size_t)r * H + i] = from_float<T>(y * w2[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) token_shift_kernel(
    const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state, long long state_stride,
    const int* __restrict__ cu_q, const int* __restrict__ seq_of_token, const int* __restrict__ state_slots,
    T* __restrict__ out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int first = cu_q[s], last = cu_q[s + 1] - 1;
  float* slot = state + (size_t)state_slots[s] * state_stride;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float cur = h[(size_t)t * H + i];
    const float prev = t == first ? slot[i] : h[(size_t)(t - 1) * H + i];
    out[(size_t)t * H + i] = from_float<T>(cur + (prev - cur) * mu[i]);
    if (t == first) slot[i] = h[(size_t)last * H + i];
  }
}

// y [T, inner] float32 (a recurrent mixer's output) times silu(z) (z: columns z_col.. of a [T, z_stride] product in the
// activation dtype), then RMS-normed in `groups` equal parts, each by its own root mean square, times weight.
// One block per (row, part); 32-bit throughout, one rounding.
template <typename T>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(
    const float* __restrict__ y, const T* __restrict__ z, long long z_stride, const float* __restrict__ weight,
    float eps, T* __restrict__ out, int inner, int groups) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int width = inner / groups;
  const int c0 = g * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float zv = to_float(z[(size_t)t * z_stride + c0 + i]);
    const float v = y[(size_t)t * inner + c0 + i] * (zv / (1.0f + expf(-zv)));
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float zv = to_float(z[(size_t)t * z_stride + c0 + i]);
    const float v = y[(size_t)t * inner + c0 + i] * (zv / (1.0f + expf(-zv)));
    out[(size_t)t * inner + c0 + i] = from_float<T>(v * rstd * weight[c0 + i]);
  }
}

template <typename T>
int launch_add_norm_pair(float* resid, const void* a, const void* b, float scale, const int* ids, const void* table,
                         const int* rows, const float* w1, const float* w2, float eps, void* out1, int out1_f32,
                         void* out2, int n_rows, int H, cudaStream_t stream) {
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  if (out1_f32) {
    auto kern = add_norm_pair_kernel<T, float>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(kern, dim3(n_rows), dim3(256), smem, stream, resid, (const T*)a, (const T*)b, scale, ids,
                      (const T*)table, rows, w1, w2, eps, (float*)out1, (T*)out2, H);
  }
  auto kern = add_norm_pair_kernel<T, T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(kern, dim3(n_rows), dim3(256), smem, stream, resid, (const T*)a, (const T*)b, scale, ids,
                    (const T*)table, rows, w1, w2, eps, (T*)out1, (T*)out2, H);
}

}  // namespace tmk

// resid [n_tokens, H] float; a, b [n_tokens, H] dtype or null; ids/table: the stream starts as table[ids]; rows
// [n_rows] or null; w1, w2 [H] float (w2 and out2 may be null together); out1 [n_rows, H] float (out1_f32) or dtype.
extern "C" int tm_add_norm_pair(int dtype, float* resid, const void* a, const void* b, float scale, const int* ids,
                                const void* table, const int* rows, const float* w1, const float* w2, float eps,
                                void* out1, int out1_f32, void* out2, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if ((out2 == nullptr) != (w2 == nullptr)) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_add_norm_pair<float>(resid, a, b, scale, ids, table, rows, w1, w2, eps, out1, out1_f32, out2,
                                            n_rows, H, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_add_norm_pair<__nv_bfloat16>(resid, a, b, scale, ids, table, rows, w1, w2, eps, out1, out1_f32,
                                                    out2, n_rows, H, stream);
  return TM_ERR_BAD_DTYPE;
}

// h [T, H] float; mu [H] float; state [slots, state_stride] float (the first H of a slot hold the previous h);
// out [T, H] dtype.
extern "C" int tm_token_shift(int dtype, const float* h, const float* mu, float* state, long long state_stride,
                              const int* cu_q, const int* seq_of_token, const int* state_slots, void* out, int T,
                              int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::token_shift_kernel<float>, dim3(T), dim3(256), 0, stream, h, mu, state, state_stride,
                           cu_q, seq_of_token, state_slots, (float*)out, H);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, h, mu, state,
                           state_stride, cu_q, seq_of_token, state_slots, (__nv_bfloat16*)out, H);
  return TM_ERR_BAD_DTYPE;
}

// y [T, inner] float; z: column 0 of the gate inside a [T, z_stride] product; weight [inner] float; out [T, inner].
extern "C" int tm_gated_group_norm(int dtype, const float* y, const void* z, long long z_stride, const float* weight,
                                   float eps, void* out, int T, int inner, int groups, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (groups <= 0 || inner % groups) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid(T, groups);
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::gated_group_norm_kernel<float>, grid, dim3(128), 0, stream, y, (const float*)z,
                           z_stride, weight, eps, (float*)out, inner, groups);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, y,
                           (const __nv_bfloat16*)z, z_stride, weight, eps, (__nv_bfloat16*)out, inner, groups);
  return TM_ERR_BAD_DTYPE;
}
