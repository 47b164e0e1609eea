// Attention over a cache of latents: every token stores ONE row [c | r] (c: `rank` values,
// the normed low-rank latent; r: `rot` values, a rotated key part shared by all heads)
// instead of keys and values per head.  With the per-head up-projections folded into
// the query and the output (q_lat[h] = W_uk[h]^T q[h], o[h] = W_uv[h] o_lat[h]) every
// head attends the same rows:
//
//   score(t, h, j) = (q_lat[t, h] . c_j + q_rot[t, h] . r_j) * scale
//   o_lat[t, h]    = sum_j softmax_j(score) c_j
//
// Three kernels: `latent_prepare` (RMS norm of the latent, rotary on the shared key part
// and on the queries' rotated parts, cache write), `head_gemm` (the folded products, one
// small matrix per head) and `latent_attention` (one warp per (token, head), float32
// scores, softmax and sums, keys walked in runs of 32 from position 0 so that the order
// of every sum depends on the token's position alone).
#include "common.cuh"

// ---------------------------------------------------------------- prepare
// proj[t] = [q (heads x (nope + rot)) | latent (rank) | shared key part (rot)].
// Rotary pairs dimension 2i with 2i + 1 (interleaved) over the first `nrot` of the `rot`
// values; cos/sin tables are [T, nrot / 2] (any factor already in them).
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ proj, int ld, T* __restrict__ pages,
                      const float* __restrict__ norm_w, const float* __restrict__ cos_tab,
                      const float* __restrict__ sin_tab, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                      int bt_stride, int heads, int nope, int rot, int rank, int nrot,
                      int page_size, float eps, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * ld;
  T* lat = row + (size_t)heads * (nope + rot);
  const int half = nrot / 2;
  const float* ct = cos_tab + (size_t)t * half;
  const float* st = sin_tab + (size_t)t * half;
  const int pos = positions[t];
  T* dst = nullptr;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    dst = pages + ((size_t)page * page_size + pos % page_size) * (rank + rot);
  }
  // the latent, normed in float32
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float v = to_float(lat[c]); ss += v * v; }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
  if (dst)
    for (int c = threadIdx.x; c < rank; c += blockDim.x)
      dst[c] = from_float<T>(to_float(lat[c]) * rstd * norm_w[c]);
  // the shared key part: rotated pairs, the rest as it is
  if (dst) {
    const T* kr = lat + rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float u = to_float(kr[2 * i]), v = to_float(kr[2 * i + 1]);
      dst[rank + 2 * i] = from_float<T>(u * ct[i] - v * st[i]);
      dst[rank + 2 * i + 1] = from_float<T>(v * ct[i] + u * st[i]);
    }
    for (int c = nrot + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = kr[c];
  }
  // the queries' rotated parts, in place
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    T* qr = row + (size_t)h * (nope + rot) + nope;
    const float u = to_float(qr[2 * i]), v = to_float(qr[2 * i + 1]);
    qr[2 * i] = from_float<T>(u * ct[i] - v * st[i]);
    qr[2 * i + 1] = from_float<T>(v * ct[i] + u * st[i]);
  }
}

HB_EXPORT int hb_latent_prepare(void* proj, int ld, void* pages, const float* norm_w,
                                const float* cos_tab, const float* sin_tab, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride,
                                int T, int heads, int nope, int rot, int rank, int nrot,
                                int page_size, float eps, int write_cache, int act_dt,
                                cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || nope < 0 || rot < 0 || rank <= 0 || nrot < 0 || nrot > rot || nrot % 2 ||
      page_size <= 0 || ld < heads * (nope + rot) + rank + rot)
    return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(latent_prepare_kernel<TA>, dim3(T), dim3(128), 0, stream, (TA*)proj, ld, (TA*)pages,
              norm_w, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride, heads,
              nope, rot, rank, nrot, page_size, eps, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- one small matrix per head
// C[m, b, n] = sum_k A[m, b, k] * W[b, n, k] for b < batch: rows of A, W and C have strides,
// and so have the batches.  float32 sums, every element summed over k = 0..K-1 in that
// order in one thread, so a row's result does not depend on the other rows.
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_gemm_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, int M, int N,
                 int K, long lda, long ldw, long ldc, long a_batch, long w_batch, long c_batch) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[HG_BK][HG_BM + 4];
  __shared__ float Ws[HG_BK][HG_BN + 4];
  A += (size_t)blockIdx.z * a_batch;
  W += (size_t)blockIdx.z * w_batch;
  C += (size_t)blockIdx.z * c_batch;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += HG_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HG_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_float<T>(acc[i][j]);
    }
  }
}

HB_EXPORT int hb_head_gemm(void* C, const void* A, const void* W, int M, int N, int K, long lda,
                           long ldw, long ldc, int batch, long a_batch, long w_batch, long c_batch,
                           int act_dt, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return HB_OK;
  if (K <= 0 || batch > 65535) return HB_BAD_ARGUMENT;
  dim3 grid((N + HG_BN - 1) / HG_BN, (M + HG_BM - 1) / HG_BM, batch);
  if (grid.y > 65535) return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(head_gemm_kernel<TA>, grid, dim3(256), 0, stream, (TA*)C, (const TA*)A, (const TA*)W,
              M, N, K, lda, ldw, ldc, a_batch, w_batch, c_batch));
  return hb_check_launch();
}

// ---------------------------------------------------------------- attention
constexpr int LA_WARPS = 4;
constexpr int LA_MAX_RANK = 512;     // latent values a lane accumulates: 16 x 32
constexpr int LA_MAX_ROW = 1024;     // rank + rot

// q_lat[t, h] at q_lat + t * ql_t + h * ql_h (rank values); q_rot likewise (rot values).
// out [T, heads, rank], contiguous.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(T* __restrict__ out, const T* __restrict__ q_lat, long ql_t, long ql_h,
                        const T* __restrict__ q_rot, long qr_t, long qr_h,
                        const T* __restrict__ pages, const int* __restrict__ block_table,
                        int bt_stride, const int* __restrict__ seq_of_token,
                        const int* __restrict__ positions, int n_rows, int heads, int rank, int rot,
                        int page_size, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float q_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * LA_WARPS + warp;
  if (row >= n_rows) return;
  const int t = row / heads, h = row - t * heads;
  const int width = rank + rot;
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * bt_stride;

  float* qs = q_smem + (size_t)warp * width;
  const T* ql = q_lat + (size_t)t * ql_t + (size_t)h * ql_h;
  const T* qr = q_rot + (size_t)t * qr_t + (size_t)h * qr_h;
  for (int d = lane; d < rank; d += 32) qs[d] = to_float(ql[d]);
  for (int d = lane; d < rot; d += 32) qs[rank + d] = to_float(qr[d]);
  __syncwarp();

  constexpr int ND = LA_MAX_RANK / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = 0; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    int page = 0;
    float score = -INFINITY;
    if (valid) {
      page = table[key / page_size];
      const T* kr = pages + ((size_t)page * page_size + key % page_size) * width;
      float dot = 0.f;
      for (int d = 0; d < width; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
      score = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int n_valid = min(32, pos - base + 1);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int pagej = __shfl_sync(0xffffffffu, page, j);
      const T* vr = pages + ((size_t)pagej * page_size + (base + j) % page_size) * width;
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = out + ((size_t)t * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) orow[d] = from_float<T>(acc[i] * inv);
  }
}

HB_EXPORT int hb_latent_attention(void* out, const void* q_lat, long ql_t, long ql_h,
                                  const void* q_rot, long qr_t, long qr_h, const void* pages,
                                  const int* block_table, int bt_stride, const int* seq_of_token,
                                  const int* positions, int T, int heads, int rank, int rot,
                                  int page_size, float scale, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || rank <= 0 || rank > LA_MAX_RANK || rot < 0 || rank + rot > LA_MAX_ROW ||
      page_size <= 0)
    return HB_BAD_ARGUMENT;
  const int n_rows = T * heads;
  const int blocks = (n_rows + LA_WARPS - 1) / LA_WARPS;
  const size_t smem = (size_t)LA_WARPS * (rank + rot) * sizeof(float);
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(latent_attention_kernel<TA>, dim3(blocks), dim3(LA_WARPS * 32), smem, stream,
              (TA*)out, (const TA*)q_lat, ql_t, ql_h, (const TA*)q_rot, qr_t, qr_h,
              (const TA*)pages, block_table, bt_stride, seq_of_token, positions, n_rows, heads,
              rank, rot, page_size, scale));
  return hb_check_launch();
}
