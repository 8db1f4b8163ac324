// Attention over a cache of latents on the tensor cores (bfloat16 operands, 32-bit accumulation), for prompt
// portions and decoded tokens alike. Same interface as tm_latent_attention (latent_attention.cu): every token's cache
// row is [c (rank) | k_rot (rot)], a query row is [q_lat (rank) | rope(q_rot) (rot)], the score is their dot product
// times scale over the last `window` positions, and the result is the softmax-weighted sum of the c rows.
//
// A block of four warps takes 64 consecutive (token, head) rows of one request (heads fastest, so a tile is a few
// tokens times all heads and reads each cache row once for all of them) and one slice of up to NV * 8 result
// columns; blocks with the same rows and another slice recompute the scores. Keys go in tiles of 32 anchored at
// absolute positions 0, 32, ..., through a two-stage cp.async ring (rows outside the tile's key range are
// zero-filled); S = Q K^T and O += P V are mma.sync.m16n8k16 with ldmatrix fragments (V is the first `rank`
// columns of the same shared-memory tile, read transposed). Scores, the running maximum and sum, and the
// rescaling are 32-bit; P is rounded to bfloat16 for the second product, q_lat for the first.
// With n_splits > 1 (steps of few rows, where row tiles alone would leave most multiprocessors idle) a tile's key
// tiles are dealt out in n_splits contiguous runs over blockIdx.z; each block writes its unnormalised sums with
// their maximum and weight to scratch, and tm_latent_attention_combine merges the runs in index order.
// Shapes: rank and rot multiples of 16.
#include "mma_util.cuh"

namespace tmk {

constexpr int kMlaRows = 64;
constexpr int kMlaKeys = 32;

template <int NV>   // result columns per block = NV * 8
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
    const float* __restrict__ q_lat, long long ql_stride_t, long long ql_stride_h,
    const __nv_bfloat16* __restrict__ q_rot, long long qr_stride_t, long long qr_stride_h,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_before, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_row0, __nv_bfloat16* __restrict__ out, long long out_stride_t,
    long long out_stride_h, int nh, int rank, int rot, int page_size, float scale, int window, int n_splits,
    float* __restrict__ part, int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = rank + rot;
  const int RS = D * 2 + 16;                                   // row stride in bytes: 8 rows fall into 8 different bank groups
  unsigned char* qs = smem_raw;                                // [64][RS]
  unsigned char* ks = qs + kMlaRows * RS;                      // 2 x [32][RS]

  pdl_launch_dependents();
  pdl_wait();
  const int s = tile_seq[blockIdx.x];
  const int row0 = tile_row0[blockIdx.x];
  const int c0 = blockIdx.y * NV * 8;
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  const int n_rows = q_len * nh;
  if (row0 >= n_rows) return;
  const int row_end = min(row0 + kMlaRows, n_rows);
  const int p_min = before + row0 / nh;
  const int p_max = before + (row_end - 1) / nh;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int j_hi = p_max;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_table + (size_t)s * bt_stride;
  const int half = rot_dims >> 1;
  const int segs = D / 8;                                      // 16-byte pieces of a cache row

  // A warp per key row (8 rows a warp): one page lookup per row, lanes over the row's 16-byte pieces.
  auto load_keys = [&](int kt, int stage) {
    unsigned char* dst = ks + stage * (kMlaKeys * RS);
    for (int jj = warp; jj < kMlaKeys; jj += 4) {
      const int j = kt + jj;
      const bool ok = j >= j_lo && j <= j_hi;
      const __nv_bfloat16* src = cache;
      if (ok) src = cache + ((size_t)table[j / page_size] * page_size + (j % page_size)) * D;
      for (int sg = lane; sg < segs; sg += 32) cp_async16(smem_u32(dst + jj * RS + sg * 16), ok ? src + sg * 8 : src, ok);
    }
    cp_async_commit();
  };

  int kt0 = (j_lo / kMlaKeys) * kMlaKeys;
  int kt_last = (j_hi / kMlaKeys) * kMlaKeys;
  if (n_splits > 1) {                                          // this block's run of the tile's key tiles (maybe empty)
    const int n_kt = (kt_last - kt0) / kMlaKeys + 1;
    const int per = (n_kt + n_splits - 1) / n_splits;
    kt0 += blockIdx.z * per * kMlaKeys;
    kt_last = min(kt_last, kt0 + (per - 1) * kMlaKeys);
  }
  if (kt0 <= kt_last) load_keys(kt0, 0);

  // Stage the queries, a warp per row: the latent part rounded to bfloat16, the rotated part rotated in 32-bit first.
  for (int r = warp; r < kMlaRows; r += 4) {
    const int row = row0 + r;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(qs + r * RS);
    if (row >= n_rows) {
      for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16_rn(0.f);
      continue;
    }
    const int tok = q_start + row / nh, head = row % nh;
    const float* ql = q_lat + (size_t)tok * ql_stride_t + (size_t)head * ql_stride_h;
    for (int d = lane; d < rank; d += 32) dst[d] = __float2bfloat16_rn(ql[d]);
    const __nv_bfloat16* qr = q_rot + (size_t)tok * qr_stride_t + (size_t)head * qr_stride_h;
    const int pos = before + row / nh;
    for (int i = lane; i < rot; i += 32) {
      float v = to_float(qr[i]);
      if (i < half) {
        const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
        v = __fsub_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i + half]), sn));
      } else if (i < rot_dims) {
        const float c = cos_t[(size_t)pos * half + i - half], sn = sin_t[(size_t)pos * half + i - half];
        v = __fadd_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i - half]), sn));
      }
      dst[rank + i] = __float2bfloat16_rn(v);
    }
  }

  // The two rows of this thread inside its warp's 16: g and g + 8.
  const int g = lane >> 2, qd = lane & 3;
  int p_row[2], lo_row[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + warp * 16 + g + 8 * i;
    if (row < n_rows) {
      p_row[i] = before + row / nh;
      lo_row[i] = window > 0 ? max(0, p_row[i] - window + 1) : 0;
    } else {
      p_row[i] = -1;
      lo_row[i] = 0;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NV][4];
#pragma unroll
  for (int n = 0; n < NV; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

  const uint32_t q_base = smem_u32(qs) + (warp * 16 + (lane & 15)) * RS + (lane >> 4) * 16;
  const int mi = lane >> 3, lr = lane & 7;
  const uint32_t k_off = ((mi >> 1) * 8 + lr) * RS + (mi & 1) * 16;        // S: matrices (keys 0-7 | 8-15) x (k 0-7 | 8-15)
  const uint32_t v_off = ((mi & 1) * 8 + lr) * RS + (mi >> 1) * 16;        // O: matrices (keys 0-7 | 8-15) x (dims 0-7 | 8-15), transposed
  const float sl2 = scale * 1.4426950408889634f;                           // scores kept in units of log2 e

  // stages == 2: the next tile's copy runs under this tile's arithmetic. stages == 1 (wide rows: two blocks fit a
  // multiprocessor only with one stage each): the copy for the next tile starts when this tile is done, and the
  // other block's arithmetic covers it.
  int stage = 0;
  for (int kt = kt0; kt <= kt_last; kt += kMlaKeys, stage ^= (stages - 1)) {
    if (stages == 2 && kt + kMlaKeys <= kt_last) {
      load_keys(kt + kMlaKeys, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_base = smem_u32(ks + stage * (kMlaKeys * RS));

    float sc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[n][e] = 0.f;
#pragma unroll 3
    for (int kk = 0; kk < D; kk += 16) {
      uint32_t a[4], b0, b1, b2, b3;
      ldmatrix_x4(q_base + kk * 2, a[0], a[1], a[2], a[3]);
      ldmatrix_x4(k_base + k_off + kk * 2, b0, b1, b2, b3);
      mma_bf16_16816(sc[0], a, b0, b1);
      mma_bf16_16816(sc[1], a, b2, b3);
      ldmatrix_x4(k_base + 16 * RS + k_off + kk * 2, b0, b1, b2, b3);
      mma_bf16_16816(sc[2], a, b0, b1);
      mma_bf16_16816(sc[3], a, b2, b3);
    }
    // mask, online softmax (rows g and g + 8; a row's 32 scores lie in the four lanes of a quad)
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = kt + n * 8 + qd * 2 + (e & 1);
        const bool ok = j >= j_lo && j <= j_hi && j <= p_row[i] && j >= lo_row[i];
        sc[n][e] = ok ? sc[n][e] * sl2 : -INFINITY;
        tmax[i] = fmaxf(tmax[i], sc[n][e]);
      }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
      const float m_new = fmaxf(m[i], tmax[i]);
      corr[i] = m_new == -INFINITY ? 1.f : exp2f(m[i] - m_new);
      m[i] = m_new;
    }
    float tsum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const float pv = m[i] == -INFINITY ? 0.f : exp2f(sc[n][e] - m[i]);
        sc[n][e] = pv;
        tsum[i] += pv;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tsum[i] += __shfl_xor_sync(0xffffffffu, tsum[i], 1);
      tsum[i] += __shfl_xor_sync(0xffffffffu, tsum[i], 2);
      l[i] = l[i] * corr[i] + tsum[i];
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    uint32_t pa[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      pa[kk][0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
      pa[kk][1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
      pa[kk][2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      pa[kk][3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
    }
#pragma unroll
    for (int dt = 0; dt < NV / 2; ++dt) {
      if (c0 + dt * 16 < rank) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(k_base + kk * 16 * RS + v_off + (c0 + dt * 16) * 2, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * dt], pa[kk], b0, b1);
          mma_bf16_16816(o[2 * dt + 1], pa[kk], b2, b3);
        }
      }
    }
    __syncthreads();               // the stage is free for the load after next
    if (stages == 1 && kt + kMlaKeys <= kt_last) load_keys(kt + kMlaKeys, 0);
  }

  if (n_splits > 1) {
    // scratch: [tile][split][64 rows][rank + 2] floats: unnormalised sums, then maximum (log2 units) and weight
    const int W = rank + 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = warp * 16 + g + 8 * i;
      float* dst = part + (((size_t)blockIdx.x * n_splits + blockIdx.z) * kMlaRows + r) * W;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        const int d = c0 + n * 8 + qd * 2;
        if (d < rank) *reinterpret_cast<float2*>(dst + d) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      }
      if (qd == 0 && blockIdx.y == 0) {
        dst[rank] = m[i];
        dst[rank + 1] = l[i];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + warp * 16 + g + 8 * i;
    if (row >= n_rows) continue;
    const int tok = q_start + row / nh, head = row % nh;
    __nv_bfloat16* dst = out + (size_t)tok * out_stride_t + (size_t)head * out_stride_h;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int d = c0 + n * 8 + qd * 2;
      if (d < rank) {
        const uint32_t v = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + d) = v;
      }
    }
  }
}

// The same work with warps in pairs (eight warps a block): warps w and w + 4 share 16 rows; each computes the scores
// of HALF the key tile (16 keys), they exchange the row maxima and their halves of P through shared memory, and each
// adds P V for half of the block's result columns. Per warp that is half the score arithmetic and half the
// accumulators of the kernel above, and a block covers up to 512 result columns, so the scores of a row tile are
// computed once whatever the rank.
constexpr int kPairPS = 48;                                   // bytes per row of an exchanged half of P (16 keys + padding)

__device__ __forceinline__ void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

template <int NVH, int MINB>   // result columns per warp = NVH * 8; per block 2 * NVH * 8
__global__ void __launch_bounds__(256, MINB) latent_attention_mma_pair_kernel(
    const float* __restrict__ q_lat, long long ql_stride_t, long long ql_stride_h,
    const __nv_bfloat16* __restrict__ q_rot, long long qr_stride_t, long long qr_stride_h,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_before, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_row0, __nv_bfloat16* __restrict__ out, long long out_stride_t,
    long long out_stride_h, int nh, int rank, int rot, int page_size, float scale, int window, int n_splits,
    float* __restrict__ part, int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = rank + rot;
  const int RS = D * 2 + 16;
  unsigned char* qs = smem_raw;                                // [64][RS]
  unsigned char* ks = qs + kMlaRows * RS;                      // stages x [32][RS]
  unsigned char* ps = ks + stages * kMlaKeys * RS;             // [2][64][kPairPS]: each half's P of the tile
  float* xm = reinterpret_cast<float*>(ps + 2 * kMlaRows * kPairPS);   // [2][64]: each half's row maxima (at the end: weights)

  pdl_launch_dependents();
  pdl_wait();
  const int s = tile_seq[blockIdx.x];
  const int row0 = tile_row0[blockIdx.x];
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  const int n_rows = q_len * nh;
  if (row0 >= n_rows) return;
  const int row_end = min(row0 + kMlaRows, n_rows);
  const int p_min = before + row0 / nh;
  const int p_max = before + (row_end - 1) / nh;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int j_hi = p_max;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wr = warp & 3, half_id = warp >> 2;
  const int c0 = blockIdx.y * (2 * NVH * 8) + half_id * NVH * 8;       // this warp's first result column
  const int* table = block_table + (size_t)s * bt_stride;
  const int half = rot_dims >> 1;
  const int segs = D / 8;

  auto load_keys = [&](int kt, int stage) {
    unsigned char* dst = ks + stage * (kMlaKeys * RS);
    for (int jj = warp; jj < kMlaKeys; jj += 8) {
      const int j = kt + jj;
      const bool ok = j >= j_lo && j <= j_hi;
      const __nv_bfloat16* src = cache;
      if (ok) src = cache + ((size_t)table[j / page_size] * page_size + (j % page_size)) * D;
      for (int sg = lane; sg < segs; sg += 32) cp_async16(smem_u32(dst + jj * RS + sg * 16), ok ? src + sg * 8 : src, ok);
    }
    cp_async_commit();
  };

  int kt0 = (j_lo / kMlaKeys) * kMlaKeys;
  int kt_last = (j_hi / kMlaKeys) * kMlaKeys;
  if (n_splits > 1) {
    const int n_kt = (kt_last - kt0) / kMlaKeys + 1;
    const int per = (n_kt + n_splits - 1) / n_splits;
    kt0 += blockIdx.z * per * kMlaKeys;
    kt_last = min(kt_last, kt0 + (per - 1) * kMlaKeys);
  }
  if (kt0 <= kt_last) load_keys(kt0, 0);

  for (int r = warp; r < kMlaRows; r += 8) {
    const int row = row0 + r;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(qs + r * RS);
    if (row >= n_rows) {
      for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16_rn(0.f);
      continue;
    }
    const int tok = q_start + row / nh, head = row % nh;
    const float* ql = q_lat + (size_t)tok * ql_stride_t + (size_t)head * ql_stride_h;
    for (int d = lane; d < rank; d += 32) dst[d] = __float2bfloat16_rn(ql[d]);
    const __nv_bfloat16* qr = q_rot + (size_t)tok * qr_stride_t + (size_t)head * qr_stride_h;
    const int pos = before + row / nh;
    for (int i = lane; i < rot; i += 32) {
      float v = to_float(qr[i]);
      if (i < half) {
        const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
        v = __fsub_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i + half]), sn));
      } else if (i < rot_dims) {
        const float c = cos_t[(size_t)pos * half + i - half], sn = sin_t[(size_t)pos * half + i - half];
        v = __fadd_rn(__fmul_rn(v, c), __fmul_rn(to_float(qr[i - half]), sn));
      }
      dst[rank + i] = __float2bfloat16_rn(v);
    }
  }

  const int g = lane >> 2, qd = lane & 3;
  int p_row[2], lo_row[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wr * 16 + g + 8 * i;
    if (row < n_rows) {
      p_row[i] = before + row / nh;
      lo_row[i] = window > 0 ? max(0, p_row[i] - window + 1) : 0;
    } else {
      p_row[i] = -1;
      lo_row[i] = 0;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // l: this warp's 16 keys of every tile only
  float o[NVH][4];
#pragma unroll
  for (int n = 0; n < NVH; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

  const uint32_t q_base = smem_u32(qs) + (wr * 16 + (lane & 15)) * RS + (lane >> 4) * 16;
  const int mi = lane >> 3, lr = lane & 7;
  const uint32_t k_off = (half_id * 16 + (mi >> 1) * 8 + lr) * RS + (mi & 1) * 16;   // this warp's 16 keys
  const uint32_t v_off = ((mi & 1) * 8 + lr) * RS + (mi >> 1) * 16;
  const float sl2 = scale * 1.4426950408889634f;
  unsigned char* ps_own = ps + half_id * (kMlaRows * kPairPS) + (wr * 16) * kPairPS;
  const uint32_t ps_other = smem_u32(ps + (half_id ^ 1) * (kMlaRows * kPairPS)) + (wr * 16 + (lane & 15)) * kPairPS +
                            (lane >> 4) * 16;
  float* xm_own = xm + half_id * kMlaRows + wr * 16;
  const float* xm_other = xm + (half_id ^ 1) * kMlaRows + wr * 16;
  const int bar = 1 + wr;

  int stage = 0;
  for (int kt = kt0; kt <= kt_last; kt += kMlaKeys, stage ^= (stages - 1)) {
    if (stages == 2 && kt + kMlaKeys <= kt_last) {
      load_keys(kt + kMlaKeys, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_base = smem_u32(ks + stage * (kMlaKeys * RS));

    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[n][e] = 0.f;
#pragma unroll 4
    for (int kk = 0; kk < D; kk += 16) {
      uint32_t a[4], b0, b1, b2, b3;
      ldmatrix_x4(q_base + kk * 2, a[0], a[1], a[2], a[3]);
      ldmatrix_x4(k_base + k_off + kk * 2, b0, b1, b2, b3);
      mma_bf16_16816(sc[0], a, b0, b1);
      mma_bf16_16816(sc[1], a, b2, b3);
    }
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = kt + half_id * 16 + n * 8 + qd * 2 + (e & 1);
        const bool ok = j >= j_lo && j <= j_hi && j <= p_row[i] && j >= lo_row[i];
        sc[n][e] = ok ? sc[n][e] * sl2 : -INFINITY;
        tmax[i] = fmaxf(tmax[i], sc[n][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
      if (qd == 0) xm_own[g + 8 * i] = tmax[i];
    }
    pair_barrier(bar);
    float corr[2], tsum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float m_new = fmaxf(m[i], fmaxf(tmax[i], xm_other[g + 8 * i]));
      corr[i] = m_new == -INFINITY ? 1.f : exp2f(m[i] - m_new);
      m[i] = m_new;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const float pv = m[i] == -INFINITY ? 0.f : exp2f(sc[n][e] - m[i]);
        sc[n][e] = pv;
        tsum[i] += pv;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tsum[i] += __shfl_xor_sync(0xffffffffu, tsum[i], 1);
      tsum[i] += __shfl_xor_sync(0xffffffffu, tsum[i], 2);
      l[i] = l[i] * corr[i] + tsum[i];
    }
    uint32_t pa_own[4], pa_other[4];
    pa_own[0] = pack_bf16(sc[0][0], sc[0][1]);
    pa_own[1] = pack_bf16(sc[0][2], sc[0][3]);
    pa_own[2] = pack_bf16(sc[1][0], sc[1][1]);
    pa_own[3] = pack_bf16(sc[1][2], sc[1][3]);
    *reinterpret_cast<uint32_t*>(ps_own + g * kPairPS + qd * 4) = pa_own[0];
    *reinterpret_cast<uint32_t*>(ps_own + (g + 8) * kPairPS + qd * 4) = pa_own[1];
    *reinterpret_cast<uint32_t*>(ps_own + g * kPairPS + 16 + qd * 4) = pa_own[2];
    *reinterpret_cast<uint32_t*>(ps_own + (g + 8) * kPairPS + 16 + qd * 4) = pa_own[3];
    pair_barrier(bar);
    ldmatrix_x4(ps_other, pa_other[0], pa_other[1], pa_other[2], pa_other[3]);
#pragma unroll
    for (int n = 0; n < NVH; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
#pragma unroll
    for (int dt = 0; dt < NVH / 2; ++dt) {
      if (c0 + dt * 16 < rank) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(k_base + kk * 16 * RS + v_off + (c0 + dt * 16) * 2, b0, b1, b2, b3);
          if (kk == half_id) {
            mma_bf16_16816(o[2 * dt], pa_own, b0, b1);
            mma_bf16_16816(o[2 * dt + 1], pa_own, b2, b3);
          } else {
            mma_bf16_16816(o[2 * dt], pa_other, b0, b1);
            mma_bf16_16816(o[2 * dt + 1], pa_other, b2, b3);
          }
        }
      }
    }
    __syncthreads();
    if (stages == 1 && kt + kMlaKeys <= kt_last) load_keys(kt + kMlaKeys, 0);
  }

  // A row's weight is the sum of the pair's two halves.
  if (qd == 0) {
    xm_own[g] = l[0];
    xm_own[g + 8] = l[1];
  }
  pair_barrier(bar);
  l[0] += xm_other[g];
  l[1] += xm_other[g + 8];

  if (n_splits > 1) {
    const int W = rank + 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = wr * 16 + g + 8 * i;
      float* dst = part + (((size_t)blockIdx.x * n_splits + blockIdx.z) * kMlaRows + r) * W;
#pragma unroll
      for (int n = 0; n < NVH; ++n) {
        const int d = c0 + n * 8 + qd * 2;
        if (d < rank) *reinterpret_cast<float2*>(dst + d) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      }
      if (qd == 0 && blockIdx.y == 0 && half_id == 0) {
        dst[rank] = m[i];
        dst[rank + 1] = l[i];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wr * 16 + g + 8 * i;
    if (row >= n_rows) continue;
    const int tok = q_start + row / nh, head = row % nh;
    __nv_bfloat16* dst = out + (size_t)tok * out_stride_t + (size_t)head * out_stride_h;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int n = 0; n < NVH; ++n) {
      const int d = c0 + n * 8 + qd * 2;
      if (d < rank) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
  }
}

// One block per row: merge the row's runs in index order (at most 32 runs; the first warp finds their weights).
__global__ void __launch_bounds__(128) latent_attention_combine_kernel(
    const float* __restrict__ part, int n_splits, const int* __restrict__ cu_q, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_row0, __nv_bfloat16* __restrict__ out, long long out_stride_t, long long out_stride_h,
    int nh, int rank) {
  __shared__ float wsh[33];
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x / kMlaRows, r = blockIdx.x % kMlaRows;
  const int s = tile_seq[tile], row0 = tile_row0[tile];
  const int q_start = cu_q[s], n_rows = (cu_q[s + 1] - q_start) * nh;
  const int row = row0 + r;
  if (row >= n_rows) return;
  const int W = rank + 2;
  const float* base = part + ((size_t)tile * n_splits * kMlaRows + r) * W;
  const size_t zs = (size_t)kMlaRows * W;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mz = -INFINITY, lz = 0.f;
    if (lane < n_splits) {
      mz = base[lane * zs + rank];
      lz = base[lane * zs + rank + 1];
    }
    const float mx = warp_max(mz);
    const float wz = mz == -INFINITY ? 0.f : exp2f(mz - mx);
    const float total = warp_sum(lz * wz);
    wsh[lane] = wz;
    if (lane == 0) wsh[32] = 1.0f / total;
  }
  __syncthreads();
  const float inv = wsh[32];
  const int tok = q_start + row / nh, head = row % nh;
  __nv_bfloat16* dst = out + (size_t)tok * out_stride_t + (size_t)head * out_stride_h;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      const float w = wsh[z];
      if (w != 0.f) a = fmaf(base[z * zs + d], w, a);
    }
    dst[d] = __float2bfloat16_rn(a * inv);
  }
}

template <int NV>
int launch_latent_mma(const float* q_lat, long long ql_t, long long ql_h, const void* q_rot, long long qr_t,
                      long long qr_h, const float* cos_t, const float* sin_t, int rot_dims, const void* cache,
                      const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                      const int* tile_seq, const int* tile_row0, int n_tiles, void* out, long long o_t, long long o_h,
                      int nh, int rank, int rot, int page_size, float scale, int window, int n_splits, float* part,
                      cudaStream_t stream) {
  const int D = rank + rot;
  // Two stages of keys where two blocks still fit a multiprocessor with them (or one stage would not bring a second in).
  const size_t row = (size_t)D * 2 + 16;
  const size_t two = (kMlaRows + 2 * kMlaKeys) * row, one = (kMlaRows + kMlaKeys) * row;
  const int stages = (two <= 113 * 1024 || one > 113 * 1024) ? 2 : 1;
  const size_t smem = stages == 2 ? two : one;
  if (smem > 220 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  auto kern = latent_attention_mma_kernel<NV>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid(n_tiles, (rank + NV * 8 - 1) / (NV * 8), n_splits);
  const int st = launch_pdl(kern, grid, dim3(128), smem, stream, q_lat, ql_t, ql_h, (const __nv_bfloat16*)q_rot, qr_t,
                            qr_h, cos_t, sin_t, rot_dims, (const __nv_bfloat16*)cache, block_table, bt_stride, cu_q,
                            kv_before, tile_seq, tile_row0, (__nv_bfloat16*)out, o_t, o_h, nh, rank, rot, page_size,
                            scale, window, n_splits, part, stages);
  if (st != 0 || n_splits <= 1) return st;
  return launch_pdl(latent_attention_combine_kernel, dim3(n_tiles * kMlaRows), dim3(128), 0, stream, (const float*)part, n_splits,
                    cu_q, tile_seq, tile_row0, (__nv_bfloat16*)out, o_t, o_h, nh, rank);
}

template <int NVH, int MINB>
int launch_latent_pair(const float* q_lat, long long ql_t, long long ql_h, const void* q_rot, long long qr_t,
                       long long qr_h, const float* cos_t, const float* sin_t, int rot_dims, const void* cache,
                       const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                       const int* tile_seq, const int* tile_row0, int n_tiles, void* out, long long o_t, long long o_h,
                       int nh, int rank, int rot, int page_size, float scale, int window, int n_splits, float* part,
                       cudaStream_t stream) {
  const int D = rank + rot;
  const size_t row = (size_t)D * 2 + 16, extra = 2 * kMlaRows * kPairPS + 2 * kMlaRows * sizeof(float);
  const size_t two = (kMlaRows + 2 * kMlaKeys) * row + extra, one = (kMlaRows + kMlaKeys) * row + extra;
  // Two key stages where as many blocks fit a multiprocessor with them as without.
  const size_t budget = MINB >= 2 ? 113 * 1024 : 220 * 1024;
  const int stages = (two <= budget || one > budget) ? 2 : 1;
  const size_t smem = stages == 2 ? two : one;
  if (smem > 220 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  auto kern = latent_attention_mma_pair_kernel<NVH, MINB>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid(n_tiles, (rank + 2 * NVH * 8 - 1) / (2 * NVH * 8), n_splits);
  const int st = launch_pdl(kern, grid, dim3(256), smem, stream, q_lat, ql_t, ql_h, (const __nv_bfloat16*)q_rot, qr_t,
                            qr_h, cos_t, sin_t, rot_dims, (const __nv_bfloat16*)cache, block_table, bt_stride, cu_q,
                            kv_before, tile_seq, tile_row0, (__nv_bfloat16*)out, o_t, o_h, nh, rank, rot, page_size,
                            scale, window, n_splits, part, stages);
  if (st != 0 || n_splits <= 1) return st;
  return launch_pdl(latent_attention_combine_kernel, dim3(n_tiles * kMlaRows), dim3(128), 0, stream, (const float*)part,
                    n_splits, cu_q, tile_seq, tile_row0, (__nv_bfloat16*)out, o_t, o_h, nh, rank);
}

}  // namespace tmk

// As tm_latent_attention, bfloat16 only, with tiles of 64 rows; rank and rot multiples of 16, even strides.
// n_splits > 1: part holds n_tiles * n_splits * 64 * (rank + 2) floats. paired: the kernel with warps in pairs.
extern "C" int tm_latent_attention_mma_bf16(const float* q_lat, long long ql_t, long long ql_h, const void* q_rot,
                                            long long qr_t, long long qr_h, const float* cos_t, const float* sin_t,
                                            int rot_dims, const void* cache, const int* block_table, int bt_stride,
                                            const int* cu_q, const int* kv_before, const int* tile_seq,
                                            const int* tile_row0, int n_tiles, void* out, long long o_t, long long o_h,
                                            int nh, int rank, int rot, int page_size, float scale, int window,
                                            int n_splits, float* part, int paired, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (n_splits < 1 || n_splits > 32 || (n_splits > 1 && part == nullptr)) return TM_ERR_SCRATCH_TOO_SMALL;
  if (rank % 16 || rot % 16 || (o_t & 1) || (o_h & 1) || (reinterpret_cast<uintptr_t>(out) & 3) ||
      (reinterpret_cast<uintptr_t>(cache) & 15))
    return TM_ERR_UNSUPPORTED_SHAPE;
#define TM_PAIR(NVH, MINB)                                                                                          \
  return tmk::launch_latent_pair<NVH, MINB>(q_lat, ql_t, ql_h, q_rot, qr_t, qr_h, cos_t, sin_t, rot_dims, cache,     \
                                            block_table, bt_stride, cu_q, kv_before, tile_seq, tile_row0, n_tiles, out, \
                                            o_t, o_h, nh, rank, rot, page_size, scale, window, n_splits, part, stream)
  if (paired) {                              // warps in pairs: up to 512 result columns a block
    if (rank <= 64) TM_PAIR(4, 2);
    if (rank <= 128) TM_PAIR(8, 2);
    if (rank <= 256) TM_PAIR(16, 2);
    TM_PAIR(32, 1);
  }
#undef TM_PAIR
#define TM_MLA(NV)                                                                                                   \
  return tmk::launch_latent_mma<NV>(q_lat, ql_t, ql_h, q_rot, qr_t, qr_h, cos_t, sin_t, rot_dims, cache, block_table, \
                                    bt_stride, cu_q, kv_before, tile_seq, tile_row0, n_tiles, out, o_t, o_h, nh, rank, \
                                    rot, page_size, scale, window, n_splits, part, stream)
  if (rank <= 64) TM_MLA(8);
  if (rank <= 128) TM_MLA(16);
  TM_MLA(32);
#undef TM_MLA
}
