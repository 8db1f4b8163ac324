// Attention over a cache of latents: every token keeps one row [c (rank) | k_rot (rot)] that all heads share, and
// keys and values are linear maps of c. The maps are applied to the query and to the result instead of to the cache:
//   score(i, j, h) = (q_lat[i, h] . c[j] + rope(q_rot[i, h]) . k_rot[j]) * scale,   q_lat[i, h] = W_uk[h]^T q_nope[i, h]
//   out_lat[i, h]  = sum_j softmax_j(score) c[j]                                    (values: W_uv[h] out_lat[i, h])
// so one cache row serves every head of a query (the two small per-head products run as batched matrix products
// around this kernel).
//
// tm_latent_prepare, one block per token, reads the fused down-projection [cq (q_rank) | c (rank) | k_rot (rot)]:
// cq and c are RMS-normed (32-bit, plain weights), k_rot is rotated by the token's position (rotate-half over its
// first rot_dims dimensions: i pairs with i + rot_dims/2, angle tables in 32-bit), and [c | k_rot] goes to the
// token's cache slot.
//
// tm_latent_attention: 32-bit arithmetic on CUDA cores for both dtypes. A tile is 32 consecutive (token, head) rows
// of one request; 8 warps x 4 rows. Keys are walked in tiles of 32 anchored at absolute positions 0, 32, 64, ..., so
// the order of every sum depends only on the query's own position, never on how the request was cut into steps or
// on what else is in the batch. A query at position p reads keys p - window + 1 .. p (window 0: all keys up to p).
// The query's rotated part is rotated while it is staged.
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const T* __restrict__ proj, int q_rank, int rank, int rot, int rot_dims, const float* __restrict__ wq,
    const float* __restrict__ wkv, float eps, const int* __restrict__ positions, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int n_positions, const int* __restrict__ slot_map, T* __restrict__ cq_out,
    T* __restrict__ cache, int* __restrict__ error) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int P = q_rank + rank + rot;
  const T* row = proj + (size_t)t * P;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_float(row[i]);
    ss += v * v;
  }
  float total = block_sum(ss, red);
  float rstd = 1.0f / sqrtf(total / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq_out[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * rstd * wq[i]);

  const int slot = slot_map[t];
  if (slot < 0) return;
  T* dst = cache + (size_t)slot * (rank + rot);
  ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(row[q_rank + i]);
    ss += v * v;
  }
  total = block_sum(ss, red);
  rstd = 1.0f / sqrtf(total / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = from_float<T>(to_float(row[q_rank + i]) * rstd * wkv[i]);

  const int pos = positions[t];
  if (pos < 0 || pos >= n_positions) {       // never read outside the tables: report instead
    if (threadIdx.x == 0) atomicExch(error, 31);
    return;
  }
  const int half = rot_dims >> 1;
  const T* kr = row + q_rank + rank;
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    float v = to_float(kr[i]);
    if (i < half) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      v = __fsub_rn(__fmul_rn(v, c), __fmul_rn(to_float(kr[i + half]), s));
    } else if (i < rot_dims) {
      const float c = cos_t[(size_t)pos * half + i - half], s = sin_t[(size_t)pos * half + i - half];
      v = __fadd_rn(__fmul_rn(v, c), __fmul_rn(to_float(kr[i - half]), s));
    }
    dst[rank + i] = from_float<T>(v);
  }
}

constexpr int kLatRowsPerWarp = 4;
constexpr int kLatWarps = 8;
constexpr int kLatTileRows = kLatRowsPerWarp * kLatWarps;  // 32
constexpr int kLatKeyTile = 32;

// QL: type of q_lat (float32 always here: the absorbed query keeps its 32-bit accumulator). NDV = ceil(rank / 32).
template <typename T, int NDV>
__global__ void __launch_bounds__(kLatWarps * 32) latent_attention_kernel(
    const float* __restrict__ q_lat, long long ql_stride_t, long long ql_stride_h,   // [.., rank]
    const T* __restrict__ q_rot, long long qr_stride_t, long long qr_stride_h,       // [.., rot], not yet rotated
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims, const T* __restrict__ cache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q,
    const int* __restrict__ kv_before, const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    T* __restrict__ out, long long out_stride_t, long long out_stride_h, int nh, int rank, int rot, int page_size,
    float scale, int window) {
  extern __shared__ __align__(16) float smem[];
  const int D = rank + rot;
  const int KS = D + 1;                       // padded key row: lanes read different rows, same column
  float* qs = smem;                           // [32][D]
  float* ks = qs + kLatTileRows * D;          // [32][D + 1]

  pdl_launch_dependents();
  pdl_wait();
  const int s = tile_seq[blockIdx.x];
  const int row0 = tile_row0[blockIdx.x];
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  const int n_rows = q_len * nh;
  if (row0 >= n_rows) return;
  const int row_end = min(row0 + kLatTileRows, n_rows);
  const int p_min = before + row0 / nh;
  const int p_max = before + (row_end - 1) / nh;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int j_hi = p_max;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_table + (size_t)s * bt_stride;
  const int half = rot_dims >> 1;

  for (int idx = tid; idx < kLatTileRows * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) {
      const int tok = q_start + row / nh, head = row % nh;
      if (d < rank) {
        v = q_lat[(size_t)tok * ql_stride_t + (size_t)head * ql_stride_h + d];
      } else {
        const int i = d - rank;
        const T* qr = q_rot + (size_t)tok * qr_stride_t + (size_t)head * qr_stride_h;
        v = to_float(qr[i]);
        const int pos = before + row / nh;
        if (i < half) {
          const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
          v = __fsub_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i + half]), sn));
        } else if (i < rot_dims) {
          const float c = cos_t[(size_t)pos * half + i - half], sn = sin_t[(size_t)pos * half + i - half];
          v = __fadd_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i - half]), sn));
        }
      }
    }
    qs[idx] = v;
  }

  float m[kLatRowsPerWarp], l[kLatRowsPerWarp], acc[kLatRowsPerWarp][NDV];
  int p_row[kLatRowsPerWarp], lo_row[kLatRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int dd = 0; dd < NDV; ++dd) acc[i][dd] = 0.f;
    const int row = row0 + warp * kLatRowsPerWarp + i;
    if (row < n_rows) {
      p_row[i] = before + row / nh;
      lo_row[i] = window > 0 ? max(0, p_row[i] - window + 1) : 0;
    } else {
      p_row[i] = -1;
      lo_row[i] = 0;
    }
  }

  for (int kt = (j_lo / kLatKeyTile) * kLatKeyTile; kt <= j_hi; kt += kLatKeyTile) {
    __syncthreads();
    for (int idx = tid; idx < kLatKeyTile * D; idx += blockDim.x) {
      const int jj = idx / D, d = idx - jj * D;
      const int j = kt + jj;
      float v = 0.f;
      if (j >= j_lo && j <= j_hi) {
        const int page = table[j / page_size];
        v = to_float(cache[((size_t)page * page_size + (j % page_size)) * D + d]);
      }
      ks[jj * KS + d] = v;
    }
    __syncthreads();

    float sc[kLatRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kLatRowsPerWarp; ++i) sc[i] = 0.f;
    const float* krow = ks + lane * KS;
    const float* qrow = qs + warp * kLatRowsPerWarp * D;
    for (int d = 0; d < D; ++d) {
      const float kk = krow[d];
#pragma unroll
      for (int i = 0; i < kLatRowsPerWarp; ++i) sc[i] = fmaf(qrow[i * D + d], kk, sc[i]);
    }
    const int j = kt + lane;
    float p[kLatRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kLatRowsPerWarp; ++i) {
      const bool ok = j >= j_lo && j <= j_hi && j <= p_row[i] && j >= lo_row[i];
      const float sv = ok ? sc[i] * scale : -INFINITY;
      const float tmax = warp_max(sv);
      const float m_new = fmaxf(m[i], tmax);
      float corr = 1.f, pv = 0.f;
      if (m_new != -INFINITY) {
        corr = expf(m[i] - m_new);
        pv = ok ? expf(sv - m_new) : 0.f;
      }
      const float tsum = warp_sum(pv);
      l[i] = l[i] * corr + tsum;
      m[i] = m_new;
      p[i] = pv;
#pragma unroll
      for (int dd = 0; dd < NDV; ++dd) acc[i][dd] *= corr;
    }
    // out_lat += P . c : the value of a key is the first `rank` numbers of its row; lane owns dims lane, lane + 32, ...
    for (int jj = 0; jj < kLatKeyTile; ++jj) {
      float vv[NDV];
#pragma unroll
      for (int dd = 0; dd < NDV; ++dd) {
        const int d = lane + 32 * dd;
        vv[dd] = d < rank ? ks[jj * KS + d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kLatRowsPerWarp; ++i) {
        const float pj = __shfl_sync(0xffffffffu, p[i], jj);
#pragma unroll
        for (int dd = 0; dd < NDV; ++dd) acc[i][dd] = fmaf(pj, vv[dd], acc[i][dd]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kLatRowsPerWarp; ++i) {
    const int row = row0 + warp * kLatRowsPerWarp + i;
    if (row >= n_rows) continue;
    const int tok = q_start + row / nh, head = row % nh;
    T* o = out + (size_t)tok * out_stride_t + (size_t)head * out_stride_h;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int dd = 0; dd < NDV; ++dd) {
      const int d = lane + 32 * dd;
      if (d < rank) o[d] = from_float<T>(acc[i][dd] * inv);
    }
  }
}

template <typename T>
int launch_latent_attention(const float* q_lat, long long ql_t, long long ql_h, const void* q_rot, long long qr_t,
                            long long qr_h, const float* cos_t, const float* sin_t, int rot_dims, const void* cache,
                            const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                            const int* tile_seq, const int* tile_row0, int n_tiles, void* out, long long o_t,
                            long long o_h, int nh, int rank, int rot, int page_size, float scale, int window,
                            cudaStream_t stream) {
  const int D = rank + rot;
  const size_t smem = ((size_t)kLatTileRows * D + (size_t)kLatKeyTile * (D + 1)) * sizeof(float);
  if (smem > 220 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  const int nd = (rank + 31) / 32;
#define TM_LAT_CASE(NDV)                                                                                          \
  case NDV: {                                                                                                     \
    auto kern = latent_attention_kernel<T, NDV>;                                                                  \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    return launch_pdl(kern, dim3(n_tiles), dim3(kLatWarps * 32), smem, stream, q_lat, ql_t, ql_h, (const T*)q_rot, \
                      qr_t, qr_h, cos_t, sin_t, rot_dims, (const T*)cache, block_table, bt_stride, cu_q, kv_before, \
                      tile_seq, tile_row0, (T*)out, o_t, o_h, nh, rank, rot, page_size, scale, window);           \
  }
  switch (nd) {
    TM_LAT_CASE(1) TM_LAT_CASE(2) TM_LAT_CASE(3) TM_LAT_CASE(4) TM_LAT_CASE(5) TM_LAT_CASE(6) TM_LAT_CASE(7) TM_LAT_CASE(8)
    TM_LAT_CASE(9) TM_LAT_CASE(10) TM_LAT_CASE(11) TM_LAT_CASE(12) TM_LAT_CASE(13) TM_LAT_CASE(14) TM_LAT_CASE(15)
    TM_LAT_CASE(16)
    default: return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_LAT_CASE
}

}  // namespace tmk

// proj [T, q_rank + rank + rot]; wq [q_rank], wkv [rank] float; cos/sin [n_positions, rot_dims / 2] float;
// slot_map [T] (negative: the token's row is not cached); cq_out [T, q_rank]; cache [slots, rank + rot].
extern "C" int tm_latent_prepare(int dtype, const void* proj, int q_rank, int rank, int rot, int rot_dims,
                                 const float* wq, const float* wkv, float eps, const int* positions,
                                 const float* cos_t, const float* sin_t, int n_positions, const int* slot_map,
                                 void* cq_out, void* cache, int T, int* error, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || q_rank <= 0 || rank <= 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::latent_prepare_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)proj, q_rank,
                           rank, rot, rot_dims, wq, wkv, eps, positions, cos_t, sin_t, n_positions, slot_map,
                           (float*)cq_out, (float*)cache, error);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream,
                           (const __nv_bfloat16*)proj, q_rank, rank, rot, rot_dims, wq, wkv, eps, positions, cos_t, sin_t,
                           n_positions, slot_map, (__nv_bfloat16*)cq_out, (__nv_bfloat16*)cache, error);
  return TM_ERR_BAD_DTYPE;
}

// q_lat: float, element (t, h, d) at t * ql_t + h * ql_h + d; q_rot, out: dtype, strided the same way; cache
// [pages, page_size, rank + rot] dtype; block_table [S, bt_stride]; tiles as for the shape-generic attention
// (32 rows of (token, head) per tile, heads fastest).
extern "C" int tm_latent_attention(int dtype, const float* q_lat, long long ql_t, long long ql_h, const void* q_rot,
                                   long long qr_t, long long qr_h, const float* cos_t, const float* sin_t, int rot_dims,
                                   const void* cache, const int* block_table, int bt_stride, const int* cu_q,
                                   const int* kv_before, const int* tile_seq, const int* tile_row0, int n_tiles,
                                   void* out, long long o_t, long long o_h, int nh, int rank, int rot, int page_size,
                                   float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_latent_attention<float>(q_lat, ql_t, ql_h, q_rot, qr_t, qr_h, cos_t, sin_t, rot_dims, cache,
                                               block_table, bt_stride, cu_q, kv_before, tile_seq, tile_row0, n_tiles, out,
                                               o_t, o_h, nh, rank, rot, page_size, scale, window, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_latent_attention<__nv_bfloat16>(q_lat, ql_t, ql_h, q_rot, qr_t, qr_h, cos_t, sin_t, rot_dims,
                                                       cache, block_table, bt_stride, cu_q, kv_before, tile_seq, tile_row0,
                                                       n_tiles, out, o_t, o_h, nh, rank, rot, page_size, scale, window,
                                                       stream);
  return TM_ERR_BAD_DTYPE;
}
